// Memory-bound kernels of the decoder step: embedding gather, fused residual
// add + RMSNorm, gated activation, and the fused q/k/v bias + rotary position
// encoding + paged cache write.
//
// They replace, from the reference: embedding_lookup_kernel
// (src/kernels/embedding_kernel.cu:20-37), rms_norm_kernel + add_inplace_kernel
// (src/kernels/layernorm.cu:10-57, embedding_kernel.cu:73-87), swiglu_kernel
// (src/kernels/activation.cu:34-57), and add_bias_kernel + rope_kernel + the two
// per-token device copies into the cache (embedding_kernel.cu:55-67,
// src/kernels/rotary_embedding.cu:8-45, src/layers/attention.cpp:84-102).
#include "common.cuh"

int vcb_pdl_enabled = 0;
VCB_EXPORT void vcb_set_pdl(int on) { vcb_pdl_enabled = on ? 1 : 0; }

// ---------------------------------------------------------------- embedding
// residual[t, :] = float(table[ids[t], :]).  The residual stream is float in
// both precisions.  The host checks the ids it feeds; ids that stay on the device (a step launched
// before the step that samples them has been read) are checked here: an id outside [0, vocab)
// reads no row, leaves zeros and VCB_STATUS_BAD_TOKEN in the status word.
__device__ __forceinline__ bool token_ok(int id, int vocab, int* status) {
    if ((unsigned)id < (unsigned)vocab) return true;
    if (status && threadIdx.x == 0) atomicCAS(status, 0, VCB_STATUS_BAD_TOKEN);
    return false;
}

template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ residual, int hidden, int vocab, int* status) {
    pdl_start();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = token_ok(id, vocab, status);
    const T* row = table + (size_t)(ok ? id : 0) * hidden;
    float* out = residual + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = ok ? to_f32<T>(row[i]) : 0.0f;
}

// The same for bfloat16 rows of a multiple of 8 elements: 16-byte loads, all of a thread's in flight before the
// first is widened and stored (NV vectors a thread).
template <int NV>
__global__ void embedding_bf16x8_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids,
                                        float* __restrict__ residual, int hidden, int vocab, int* status) {
    pdl_start();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = token_ok(id, vocab, status);
    const uint4* row = reinterpret_cast<const uint4*>(table + (size_t)(ok ? id : 0) * hidden);
    float4* out = reinterpret_cast<float4*>(residual + (size_t)t * hidden);
    const int nvec = hidden >> 3;
    uint4 v[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        v[k] = (ok && i < nvec) ? row[i] : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i >= nvec) break;
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v[k]);
        const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]), c = __bfloat1622float2(p[2]),
                     d = __bfloat1622float2(p[3]);
        out[2 * i] = make_float4(a.x, a.y, b.x, b.y);
        out[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
    }
}

// vocab: rows of the table; status (may be null): the device's status word.
VCB_EXPORT int vcb_embedding(const void* table, const int* ids, float* residual, int n_tokens,
                             int hidden, int vocab, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (vocab <= 0) return VCB_ERR_BAD_ARG;
    const int threads = hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_BF16 && hidden % 8 == 0 && hidden / 8 <= 4 * 256 && !(((uintptr_t)table | (uintptr_t)residual) & 15)) {
        const int nvec = hidden / 8;
        if (nvec <= 2 * 256)
            vcb_launch(embedding_bf16x8_kernel<2>, n_tokens, nvec <= 2 * 128 ? 128 : 256, 0, s, (const __nv_bfloat16*)table, ids, residual,
                       hidden, vocab, status);
        else
            vcb_launch(embedding_bf16x8_kernel<4>, n_tokens, 256, 0, s, (const __nv_bfloat16*)table, ids, residual, hidden, vocab, status);
        return vcb_last_error();
    }
    if (dtype == VCB_F32)
        vcb_launch(embedding_kernel<float>, n_tokens, threads, 0, s, (const float*)table, ids, residual, hidden, vocab, status);
    else if (dtype == VCB_BF16)
        vcb_launch(embedding_kernel<__nv_bfloat16>, n_tokens, threads, 0, s, (const __nv_bfloat16*)table, ids, residual, hidden, vocab, status);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ---------------------------------------------------------- add + RMSNorm
// x = residual[row] (+ delta[row]);  r = 1/sqrt(mean(x^2) + eps);
// out[i] = (x * r) * gain      (multiply order of src/kernels/layernorm.cu:41,48)
// Without row_index: row = i and x is written back to residual (the residual sum,
// in float).  With row_index: row = row_index[i], nothing is written back (the
// final norm on the rows whose logits are wanted; an index may repeat).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const float* __restrict__ gain, T* __restrict__ out,
                                   const int* __restrict__ row_index, int hidden, float eps) {
    __shared__ float scratch[33];
    pdl_start();
    const int o = blockIdx.x;
    const int row = row_index ? row_index[o] : o;
    float* res = residual + (size_t)row * hidden;
    const T* dl = delta ? delta + (size_t)row * hidden : nullptr;
    T* dst = out + (size_t)o * hidden;
    const bool write_back = (row_index == nullptr) && (delta != nullptr);

    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float x = res[i];
        if (dl) x += to_f32<T>(dl[i]);
        if (write_back) res[i] = x;
        ss += x * x;
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float x = res[i];
        if (dl && !write_back) x += to_f32<T>(dl[i]);
        dst[i] = from_f32<T>((x * r) * gain[i]);
    }
}

// Same computation with 16-byte accesses and the row held in registers between the
// sum of squares and the scaling, so global memory is read once.  Needs hidden % 4 == 0
// and hidden <= 4 * NV * blockDim.x.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&a);
        u.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

template <typename T, int NV>
__global__ void __launch_bounds__(NV == 8 ? 512 : 256) add_rmsnorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                       const float* __restrict__ gain, T* __restrict__ out,
                                       const int* __restrict__ row_index, int hidden, float eps) {
    __shared__ float scratch[33];
    pdl_start();
    const int o = blockIdx.x;
    const int row = row_index ? row_index[o] : o;
    float* res = residual + (size_t)row * hidden;
    const T* dl = delta ? delta + (size_t)row * hidden : nullptr;
    T* dst = out + (size_t)o * hidden;
    const bool write_back = (row_index == nullptr) && (delta != nullptr);
    const int nvec = hidden >> 2;
    float4 x[NV], dv[NV];
    float ss = 0.0f;
    // every load of the row first: a store between two loads would order them
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        x[k] = i < nvec ? Vec4<float>::load(res + 4 * i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        dv[k] = (dl && i < nvec) ? Vec4<T>::load(dl + 4 * i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < nvec) {
            float4 v = x[k];
            if (dl) { v.x += dv[k].x; v.y += dv[k].y; v.z += dv[k].z; v.w += dv[k].w; }
            if (write_back) Vec4<float>::store(res + 4 * i, v);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            x[k] = v;
        }
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < nvec) {
            const float4 g = Vec4<float>::load(gain + 4 * i);
            float4 v = x[k];
            v.x = (v.x * r) * g.x; v.y = (v.y * r) * g.y; v.z = (v.z * r) * g.z; v.w = (v.w * r) * g.w;
            Vec4<T>::store(dst + 4 * i, v);
        }
    }
}

template <typename T>
static void launch_add_rmsnorm(float* residual, const T* delta, const float* gain, T* out, const int* row_index,
                               int n_rows, int hidden, float eps, cudaStream_t s) {
    const bool aligned = (hidden % 4 == 0) && ((((uintptr_t)residual | (uintptr_t)gain) & 15) == 0) &&
                         ((((uintptr_t)delta | (uintptr_t)out) & 7) == 0);
    const int nvec = hidden / 4;
    if (aligned && nvec <= 128 * 4)
        vcb_launch(add_rmsnorm_vec_kernel<T, 4>, n_rows, 128, 0, s, residual, delta, gain, out, row_index, hidden, eps);
    else if (aligned && nvec <= 256 * 4)
        vcb_launch(add_rmsnorm_vec_kernel<T, 4>, n_rows, 256, 0, s, residual, delta, gain, out, row_index, hidden, eps);
    else if (aligned && nvec <= 512 * 8)        // a row and its addend in registers: 64 of them a thread at eight vectors
        vcb_launch(add_rmsnorm_vec_kernel<T, 8>, n_rows, 512, 0, s, residual, delta, gain, out, row_index, hidden, eps);
    else {
        const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
        vcb_launch(add_rmsnorm_kernel<T>, n_rows, threads, 0, s, residual, delta, gain, out, row_index, hidden, eps);
    }
}

VCB_EXPORT int vcb_add_rmsnorm(float* residual, const void* delta, const float* gain, void* out,
                               const int* row_index, int n_rows, int hidden, float eps, int dtype,
                               void* stream) {
    if (n_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32)
        launch_add_rmsnorm<float>(residual, (const float*)delta, gain, (float*)out, row_index, n_rows, hidden, eps, s);
    else if (dtype == VCB_BF16)
        launch_add_rmsnorm<__nv_bfloat16>(residual, (const __nv_bfloat16*)delta, gain, (__nv_bfloat16*)out,
                                          row_index, n_rows, hidden, eps, s);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------------------- gated activation
// out[t, i] = silu(gu[t, i]) * gu[t, inter + i],  silu(z) = z / (1 + exp(-z))
// (src/kernels/activation.cu:8-10,34-39), evaluated in float with expf.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter) {
    pdl_start();
    const int t = blockIdx.y;
    const T* g = gu + (size_t)t * 2 * inter;
    const T* u = g + inter;
    T* o = out + (size_t)t * inter;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < inter; i += gridDim.x * blockDim.x) {
        const float z = to_f32<T>(g[i]);
        const float s = z / (1.0f + expf(-z));
        o[i] = from_f32<T>(s * to_f32<T>(u[i]));
    }
}

// Eight elements per vector with 16-byte accesses (bfloat16, inter % 8 == 0), four vectors per thread
// and round so that eight loads are in flight before the first is used.  The result is rounded to
// bfloat16, so the exponential and the division are the fast ones (a few units in the last place of a
// float); the 32-bit path above uses expf and a true division.
template <typename IDX>
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                       int inter, IDX n_vec) {
    pdl_start();
    constexpr int U = 4;
    const IDX vpr = (IDX)(inter >> 3);                // vectors per row
    const IDX stride = (IDX)gridDim.x * blockDim.x * U;
    for (IDX v0 = (IDX)blockIdx.x * blockDim.x * U + threadIdx.x; v0 < n_vec; v0 += stride) {
        uint4 g4[U], u4[U];
        size_t dst[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const IDX v = v0 + (IDX)k * blockDim.x;
            if (v >= n_vec) { dst[k] = ~(size_t)0; g4[k] = u4[k] = make_uint4(0, 0, 0, 0); continue; }
            const IDX t = v / vpr;
            const size_t i = (size_t)(v - t * vpr) << 3;
            const __nv_bfloat16* row = gu + (size_t)t * 2 * inter;
            g4[k] = *reinterpret_cast<const uint4*>(row + i);
            u4[k] = *reinterpret_cast<const uint4*>(row + inter + i);
            dst[k] = (size_t)t * inter + i;
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            if (dst[k] == ~(size_t)0) continue;
            const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4[k]);
            const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4[k]);
            uint4 o4;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
                const float a = __fdividef(g.x, 1.0f + __expf(-g.x)), b = __fdividef(g.y, 1.0f + __expf(-g.y));
                o2[e] = __floats2bfloat162_rn(a * u.x, b * u.y);
            }
            *reinterpret_cast<uint4*>(out + dst[k]) = o4;
        }
    }
}

VCB_EXPORT int vcb_silu_mul(const void* gu, void* out, int n_tokens, int inter, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_BF16 && inter % 8 == 0 && ((((uintptr_t)gu | (uintptr_t)out) & 15) == 0)) {
        const size_t n_vec = (size_t)n_tokens * (inter >> 3);
        size_t blocks = (n_vec + 1023) / 1024;
        if (blocks > vcb_sm_count() * 16) blocks = vcb_sm_count() * 16;
        if (n_vec < (1u << 30))
            vcb_launch(silu_mul_bf16x8_kernel<unsigned>, (int)blocks, 256, 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out,
                       inter, (unsigned)n_vec);
        else
            vcb_launch(silu_mul_bf16x8_kernel<size_t>, (int)blocks, 256, 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out,
                       inter, n_vec);
        return vcb_last_error();
    }
    const int threads = 256;
    int bx = (inter + threads - 1) / threads;
    if (bx > 64) bx = 64;
    dim3 grid(bx, n_tokens);
    if (dtype == VCB_F32)
        vcb_launch(silu_mul_kernel<float>, grid, threads, 0, s, (const float*)gu, (float*)out, inter);
    else if (dtype == VCB_BF16)
        vcb_launch(silu_mul_kernel<__nv_bfloat16>, grid, threads, 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------- q/k/v bias + rotary + cache write
// qkv: [n_tokens, (nh + 2*nkv) * d], heads laid out q..., k..., v...
// For token t at position p = positions[t] of request r = req_of_token[t]:
//   q, k, v get their bias (float); q and k heads are rotated over the first
//   `rot` elements of each head; q goes to q_out [n_tokens, nh*d]; k and v go to
//   page block_table[r, p / page] slot p % page of this layer's cache, laid out
//   [page][k|v][kv_head] blocks of page x d elements in the layout of kv_pos (common.cuh).
// Rotation (src/kernels/rotary_embedding.cu:18-33, table of src/model/qwen.cpp:119-128):
//   angle = p / denom[j],  denom[j] = theta^(2j/rot)  (computed on the host in float)
//   pairing 0 ("half"):        (a, b) = (x[j], x[j + rot/2])
//   pairing 1 ("interleaved"): (a, b) = (x[2j], x[2j+1])
//   a' = a cos - b sin,  b' = a sin + b cos.     rot = 0 disables the rotation.
struct RopeCacheArgs {
    const void* qkv;
    const float* bias;          // may be null
    const int* positions;
    const int* req_of_token;
    const int* block_table;     // [n_reqs, bt_stride]
    const float* denom;         // [rot/2]
    void* q_out;
    void* cache;                // this layer's pages
    int bt_stride, nh, nkv, d, rot, pairing, page, write_kv;
    int num_pages;              // pages of the cache: a table entry outside [0, num_pages) is not written through
    int* status;                // receives VCB_STATUS_BAD_PAGE then (may be null)
};

// The page a token's k and v rows go to, or -1 (and a note in the status word) if the request's table
// has no valid page there: a position beyond the table's width, an entry that was given back (-1) or one
// that is no page of this cache.  Nothing is written then; the step's results are wrong and
// ops.check_status() says why.
__device__ __forceinline__ int checked_page(const RopeCacheArgs& a, int r, int pos) {
    const int lp = pos / a.page;
    const int pg = lp < a.bt_stride ? a.block_table[(size_t)r * a.bt_stride + lp] : -1;
    if ((unsigned)pg >= (unsigned)a.num_pages) {
        if (a.status) atomicCAS(a.status, 0, VCB_STATUS_BAD_PAGE);
        return -1;
    }
    return pg;
}

template <typename T>
__global__ void rope_cache_kernel(RopeCacheArgs a, int heads_per_block) {
    pdl_start();
    const int t = blockIdx.x;
    const int nheads = a.nh + 2 * a.nkv;
    const int half = a.d / 2, rhalf = a.rot / 2;
    const int h = blockIdx.y * heads_per_block + threadIdx.x / half;
    const int j = threadIdx.x % half;
    if (h >= nheads || threadIdx.x >= heads_per_block * half) return;
    const int pos = a.positions[t];
    const T* src = (const T*)a.qkv + (size_t)t * nheads * a.d + (size_t)h * a.d;
    int ia, ib;
    if (j < rhalf) {                          // the pair that q and k rotate (v: the same slots, unrotated)
        if (a.pairing == 0) { ia = j; ib = j + rhalf; }
        else                { ia = 2 * j; ib = 2 * j + 1; }
    } else {                                  // beyond the rotary part: pass through
        ia = a.rot + 2 * (j - rhalf); ib = ia + 1;
    }
    float xa = to_f32<T>(src[ia]);
    float xb = to_f32<T>(src[ib]);
    if (a.bias) { xa += a.bias[h * a.d + ia]; xb += a.bias[h * a.d + ib]; }
    if (h < a.nh + a.nkv && j < rhalf) {
        const float ang = (float)pos / a.denom[j];
        float sn, cs;
        sincosf(ang, &sn, &cs);
        const float ra = xa * cs - xb * sn;
        const float rb = xa * sn + xb * cs;
        xa = ra; xb = rb;
    }
    if (h < a.nh) {
        T* dst = (T*)a.q_out + (size_t)t * a.nh * a.d + (size_t)h * a.d;
        dst[ia] = from_f32<T>(xa);
        dst[ib] = from_f32<T>(xb);
        return;
    }
    if (!a.write_kv) return;
    const int pg = checked_page(a, a.req_of_token[t], pos);
    if (pg < 0) return;
    const int slot = pos % a.page;
    // [page][2][nkv] blocks in the layout of kv_pos
    T* base = (T*)a.cache + (size_t)pg * 2 * a.nkv * a.page * a.d;
    const int kvh = h < a.nh + a.nkv ? h - a.nh : h - a.nh - a.nkv;
    const size_t which = h < a.nh + a.nkv ? 0 : (size_t)a.nkv * a.page * a.d;
    T* dst = base + which + (size_t)kvh * a.page * a.d;
    dst[kv_pos(ia, slot, a.d, a.page, (int)sizeof(T))] = from_f32<T>(xa);
    dst[kv_pos(ib, slot, a.d, a.page, (int)sizeof(T))] = from_f32<T>(xb);
}

// The same for the common case (bfloat16, rotate-half pairing over the whole head, head size a
// multiple of 16): 16-byte accesses, the angles' sines and cosines computed once per token and shared
// by all heads.  One CTA per (token, group of heads); a thread owns chunk c of the first half of a
// head and its partner chunk in the second half.
// The one-token variant is held to 40 registers: its CTAs then fit beside two CTAs of the product before it
// (150 registers x 192 threads each) and set themselves up while that one runs, also when a step has so many
// tokens that the product fills every SM twice; otherwise they start only when it has ended (6 against 3 us at
// 64 tokens).
template <int TOK>
__device__ __forceinline__ void rope_cache_vec_body(const RopeCacheArgs& a, int heads_per_block, int n_tokens) {
    extern __shared__ float2 trig[];                    // [TOK][d / 2] (cos, sin)
    // Positions, denominators and the block table belong to the step (copied in before its first
    // kernel), not to the kernel before this one: the table of sines and cosines is made while that
    // kernel still runs, and only qkv is read after griddepcontrol.wait.
    // A CTA takes TOK tokens (one for the few tokens of a decode step, several for a prompt's portion:
    // the biases are fetched once and the loads of all its tokens are in flight together).
    pdl_launch_dependents();
    const int t0 = blockIdx.x * TOK;
    const int nheads = a.nh + 2 * a.nkv;
    const int half = a.d / 2, chunks = half / 8;
    int pos[TOK];
#pragma unroll
    for (int k = 0; k < TOK; ++k) pos[k] = t0 + k < n_tokens ? a.positions[t0 + k] : 0;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float den = a.denom[j];
#pragma unroll
        for (int k = 0; k < TOK; ++k) {
            float sn, cs;
            sincosf((float)pos[k] / den, &sn, &cs);
            trig[k * half + j] = make_float2(cs, sn);
        }
    }
    const int h = blockIdx.y * heads_per_block + threadIdx.x / chunks;
    const int c = threadIdx.x % chunks;
    const bool mine = h < nheads && threadIdx.x < heads_per_block * chunks;
    const bool to_cache = mine && h >= a.nh;
    // where a k or v row goes
    __nv_bfloat16* row_dst[TOK];
    int slot[TOK];
#pragma unroll
    for (int k = 0; k < TOK; ++k) {
        row_dst[k] = nullptr;
        slot[k] = 0;
        if (to_cache && a.write_kv && t0 + k < n_tokens) {
            const int pg = checked_page(a, a.req_of_token[t0 + k], pos[k]);
            if (pg < 0) continue;
            slot[k] = pos[k] % a.page;
            __nv_bfloat16* base = (__nv_bfloat16*)a.cache + (size_t)pg * 2 * a.nkv * a.page * a.d;
            const int kvh = h < a.nh + a.nkv ? h - a.nh : h - a.nh - a.nkv;
            const size_t which = h < a.nh + a.nkv ? 0 : (size_t)a.nkv * a.page * a.d;
            row_dst[k] = base + which + (size_t)kvh * a.page * a.d;      // the head's block of the page
        }
    }
    float ba[8], bb[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) ba[e] = bb[e] = 0.0f;
    if (mine && a.bias) {
        const float* pa = a.bias + h * a.d + c * 8;
        if ((((uintptr_t)a.bias) & 15) == 0) {             // d is a multiple of 16 here: both runs of eight are 16-byte aligned
            const float4 a0 = *reinterpret_cast<const float4*>(pa), a1 = *reinterpret_cast<const float4*>(pa + 4);
            const float4 b0 = *reinterpret_cast<const float4*>(pa + half), b1 = *reinterpret_cast<const float4*>(pa + half + 4);
            ba[0] = a0.x; ba[1] = a0.y; ba[2] = a0.z; ba[3] = a0.w; ba[4] = a1.x; ba[5] = a1.y; ba[6] = a1.z; ba[7] = a1.w;
            bb[0] = b0.x; bb[1] = b0.y; bb[2] = b0.z; bb[3] = b0.w; bb[4] = b1.x; bb[5] = b1.y; bb[6] = b1.z; bb[7] = b1.w;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) { ba[e] = pa[e]; bb[e] = pa[half + e]; }
        }
    }
    __syncthreads();
    pdl_wait();
    if (!mine) return;
    uint4 va[TOK], vb[TOK];
#pragma unroll
    for (int k = 0; k < TOK; ++k) {
        if (t0 + k >= n_tokens) { va[k] = vb[k] = make_uint4(0, 0, 0, 0); continue; }
        const __nv_bfloat16* src = (const __nv_bfloat16*)a.qkv + ((size_t)(t0 + k) * nheads + h) * a.d;
        va[k] = *reinterpret_cast<const uint4*>(src + c * 8);
        vb[k] = *reinterpret_cast<const uint4*>(src + half + c * 8);
    }
    const bool rotate = h < a.nh + a.nkv;
#pragma unroll
    for (int k = 0; k < TOK; ++k) {
        if (t0 + k >= n_tokens) break;
        const __nv_bfloat16* pa = reinterpret_cast<const __nv_bfloat16*>(&va[k]);
        const __nv_bfloat16* pb = reinterpret_cast<const __nv_bfloat16*>(&vb[k]);
        __align__(16) __nv_bfloat16 oa[8], ob[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float xa = __bfloat162float(pa[e]) + ba[e], xb = __bfloat162float(pb[e]) + bb[e];
            if (rotate) {
                const float2 cs = trig[k * half + c * 8 + e];
                const float ra = xa * cs.x - xb * cs.y;
                const float rb = xa * cs.y + xb * cs.x;
                xa = ra; xb = rb;
            }
            oa[e] = __float2bfloat16_rn(xa);
            ob[e] = __float2bfloat16_rn(xb);
        }
        if (h < a.nh) {
            __nv_bfloat16* dst = (__nv_bfloat16*)a.q_out + ((size_t)(t0 + k) * a.nh + h) * a.d;
            *reinterpret_cast<uint4*>(dst + c * 8) = *reinterpret_cast<const uint4*>(oa);
            *reinterpret_cast<uint4*>(dst + half + c * 8) = *reinterpret_cast<const uint4*>(ob);
        } else if (row_dst[k]) {
            // whole 16-byte chunks move together in the block's layout (kv_pos)
            __nv_bfloat16* dst = row_dst[k];
            *reinterpret_cast<uint4*>(dst + kv_pos(c * 8, slot[k], a.d, a.page, 2)) = *reinterpret_cast<const uint4*>(oa);
            *reinterpret_cast<uint4*>(dst + kv_pos(half + c * 8, slot[k], a.d, a.page, 2)) = *reinterpret_cast<const uint4*>(ob);
        }
    }
}

template <int TOK>
__global__ void rope_cache_vec_kernel(RopeCacheArgs a, int heads_per_block, int n_tokens) {
    rope_cache_vec_body<TOK>(a, heads_per_block, n_tokens);
}

// one token a CTA, at most 40 registers a thread (see above)
__global__ void __launch_bounds__(256, 6) rope_cache_vec_one_kernel(RopeCacheArgs a, int heads_per_block, int n_tokens) {
    rope_cache_vec_body<1>(a, heads_per_block, n_tokens);
}

VCB_EXPORT int vcb_rope_cache_write(const void* qkv, const float* bias, const int* positions,
                                    const int* req_of_token, const int* block_table, int bt_stride,
                                    const float* denom, void* q_out, void* cache, int n_tokens,
                                    int nh, int nkv, int d, int rot, int pairing, int page,
                                    int write_kv, int num_pages, int* status, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0 || (d & 1) || rot < 0 || rot > d || (rot & 1) || page <= 0 || nh <= 0 || nkv < 0 || num_pages < 0)
        return VCB_ERR_BAD_ARG;
    RopeCacheArgs a{qkv, bias, positions, req_of_token, block_table, denom, q_out, cache,
                    bt_stride, nh, nkv, d, rot, pairing, page, write_kv, num_pages, status};
    const int half = d / 2, nheads = nh + 2 * nkv;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_BF16 && pairing == 0 && rot == d && d % 16 == 0 && denom &&
        !(((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)cache) & 15)) {
        const int chunks = half / 8;
        const int groups = (nheads * chunks + 255) / 256;
        const int per = (nheads + groups - 1) / groups;               // heads per CTA, at most 256 threads
        const int threads = ((per * chunks + 31) / 32) * 32;
        const dim3 grid_y((nheads + per - 1) / per);
        if (n_tokens >= 512)
            vcb_launch(rope_cache_vec_kernel<4>, dim3((n_tokens + 3) / 4, grid_y.x), threads, (size_t)4 * half * sizeof(float2),
                       s, a, per, n_tokens);
        else
            vcb_launch(rope_cache_vec_one_kernel, dim3(n_tokens, grid_y.x), threads, (size_t)half * sizeof(float2), s, a, per,
                       n_tokens);
        return vcb_last_error();
    }
    int hpb = 128 / half;                      // heads per CTA: about 128 threads
    if (hpb < 1) hpb = 1;
    if (hpb > nheads) hpb = nheads;
    const int threads = ((hpb * half + 31) / 32) * 32;
    dim3 grid(n_tokens, (nheads + hpb - 1) / hpb);
    if (dtype == VCB_F32) vcb_launch(rope_cache_kernel<float>, grid, threads, 0, s, a, hpb);
    else if (dtype == VCB_BF16) vcb_launch(rope_cache_kernel<__nv_bfloat16>, grid, threads, 0, s, a, hpb);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------------------------------- bias
// x[t, c] += bias[c] in float (src/kernels/embedding_kernel.cu:55-67).  Only the
// path of a position encoding that the fused kernel does not know uses it.
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, const float* __restrict__ bias, int cols) {
    pdl_start();
    T* row = x + (size_t)blockIdx.x * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) row[c] = from_f32<T>(to_f32<T>(row[c]) + bias[c]);
}

VCB_EXPORT int vcb_add_bias(void* x, const float* bias, int rows, int cols, int dtype, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32) vcb_launch(add_bias_kernel<float>, rows, 256, 0, s, (float*)x, bias, cols);
    else if (dtype == VCB_BF16) vcb_launch(add_bias_kernel<__nv_bfloat16>, rows, 256, 0, s, (__nv_bfloat16*)x, bias, cols);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}
