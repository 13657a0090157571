// Paged attention over the cache, plain SIMT form, for any head size up to 256
// and both storage types.  It is the 32-bit path's attention and the reference
// that the tensor-core kernels are compared with.
//
// One warp per (query token, query head).  The query at position p of request r
// attends keys j of the same request with  j <= p  and, when window > 0,
// j > p - window;  key j lives in page block_table[r, j / page], slot j % page, its row in the
// layout of kv_pos (common.cuh).
// Scores, softmax and the output accumulation are float; softmax is computed
// online over chunks of 32 keys (one key per lane).
//
// Replaces paged_attention_kernel (src/attention/paged_attention.cu:7-93), which
// handles one query token per sequence, has no mask, walks the context twice and
// lets lane 0 accumulate the output alone.  Its "+1e-10" in the denominator is
// not kept: a row always has at least its own key.
#include "common.cuh"

#define ATT_MAX_D 256
#define ATT_WARPS 4

struct AttnArgs {
    const void* q;              // [n_tokens, nh * d]
    const void* cache;          // [pages][2][nkv][page][d]
    void* out;                  // [n_tokens, nh * d]
    const int* positions;
    const int* req_of_token;
    const int* block_table;
    int bt_stride, n_tokens, nh, nkv, d, page, window;
    float scale;
    int num_pages;              // a table entry outside [0, num_pages) is not read through: the key is left
    int* status;                // out and VCB_STATUS_BAD_PAGE is recorded here (may be null)
};

template <typename T>
__global__ void attention_simt_kernel(AttnArgs a) {
    extern __shared__ float qs_all[];
    pdl_start();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * ATT_WARPS + warp;
    if (item >= (long long)a.n_tokens * a.nh) return;
    const int t = (int)(item / a.nh), h = (int)(item % a.nh);
    const int g = h / (a.nh / a.nkv);                       // src/attention/paged_attention.cu:19
    const int pos = a.positions[t];
    const int* bt = a.block_table + (size_t)a.req_of_token[t] * a.bt_stride;
    float* qs = qs_all + warp * a.d;
    const T* qrow = (const T*)a.q + ((size_t)t * a.nh + h) * a.d;
    for (int i = lane; i < a.d; i += 32) qs[i] = to_f32<T>(qrow[i]) * a.scale;
    __syncwarp();

    const size_t page_elems = (size_t)2 * a.nkv * a.page * a.d;
    const size_t v_off = (size_t)a.nkv * a.page * a.d;
    const T* cache = (const T*)a.cache;

    float o[ATT_MAX_D / 32];
#pragma unroll
    for (int k = 0; k < ATT_MAX_D / 32; ++k) o[k] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    const int kstart = a.window > 0 ? max(0, pos - a.window + 1) : 0;

    for (int kb = kstart; kb <= pos; kb += 32) {
        const int j = kb + lane;
        bool valid = j <= pos;
        float s = -INFINITY;
        unsigned long long koff = 0;
        int pg = 0;
        if (valid) {
            const int lp = j / a.page;
            pg = lp < a.bt_stride ? bt[lp] : -1;
            if ((unsigned)pg >= (unsigned)a.num_pages) {
                if (a.status) atomicCAS(a.status, 0, VCB_STATUS_BAD_PAGE);
                valid = false;
            }
        }
        if (valid) {
            koff = (unsigned long long)pg * page_elems + (size_t)g * a.page * a.d;      // the head's block of the page
            const T* kr = cache + koff;
            const int slot = j % a.page;
            float acc = 0.0f;
            for (int i = 0; i < a.d; ++i) acc += qs[i] * to_f32<T>(kr[kv_pos(i, slot, a.d, a.page, (int)sizeof(T))]);
            s = acc;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);
        const float p = valid ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int k = 0; k < ATT_MAX_D / 32; ++k) o[k] *= corr;
        const int nvalid = min(32, pos - kb + 1);
        for (int jj = 0; jj < nvalid; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const unsigned long long off = __shfl_sync(0xffffffffu, koff, jj);
            const T* vr = cache + off + v_off;
            const int slot = (kb + jj) % a.page;
#pragma unroll
            for (int k = 0; k < ATT_MAX_D / 32; ++k) {
                const int dim = lane + 32 * k;
                if (dim < a.d) o[k] += pj * to_f32<T>(vr[kv_pos(dim, slot, a.d, a.page, (int)sizeof(T))]);
            }
        }
        m = m_new;
    }
    T* orow = (T*)a.out + ((size_t)t * a.nh + h) * a.d;
    const float inv = 1.0f / l;
#pragma unroll
    for (int k = 0; k < ATT_MAX_D / 32; ++k) {
        const int dim = lane + 32 * k;
        if (dim < a.d) orow[dim] = from_f32<T>(o[k] * inv);
    }
}

VCB_EXPORT int vcb_attention_simt(const void* q, const void* cache, void* out, const int* positions,
                                  const int* req_of_token, const int* block_table, int bt_stride,
                                  int n_tokens, int nh, int nkv, int d, int page, int window,
                                  float scale, int num_pages, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0 || d > ATT_MAX_D || nh <= 0 || nkv <= 0 || nh % nkv || page <= 0 || window < 0 || num_pages < 0)
        return VCB_ERR_BAD_ARG;
    AttnArgs a{q, cache, out, positions, req_of_token, block_table, bt_stride, n_tokens, nh, nkv, d,
               page, window, scale, num_pages, status};
    const long long items = (long long)n_tokens * nh;
    const int blocks = (int)((items + ATT_WARPS - 1) / ATT_WARPS);
    const size_t smem = (size_t)ATT_WARPS * d * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32) vcb_launch(attention_simt_kernel<float>, blocks, ATT_WARPS * 32, smem, s, a);
    else if (dtype == VCB_BF16) vcb_launch(attention_simt_kernel<__nv_bfloat16>, blocks, ATT_WARPS * 32, smem, s, a);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}
