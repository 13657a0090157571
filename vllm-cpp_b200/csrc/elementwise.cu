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

// ---------------------------------------------------------------- embedding
// residual[t, :] = float(table[ids[t], :]).  The residual stream is float in
// both precisions.  Ids are validated on the host.
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ residual, int hidden) {
    const int t = blockIdx.x;
    const T* row = table + (size_t)ids[t] * hidden;
    float* out = residual + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_f32<T>(row[i]);
}

VCB_EXPORT int vcb_embedding(const void* table, const int* ids, float* residual, int n_tokens,
                             int hidden, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32)
        embedding_kernel<float><<<n_tokens, threads, 0, s>>>((const float*)table, ids, residual, hidden);
    else if (dtype == VCB_BF16)
        embedding_kernel<__nv_bfloat16><<<n_tokens, threads, 0, s>>>((const __nv_bfloat16*)table, ids, residual, hidden);
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

VCB_EXPORT int vcb_add_rmsnorm(float* residual, const void* delta, const float* gain, void* out,
                               const int* row_index, int n_rows, int hidden, float eps, int dtype,
                               void* stream) {
    if (n_rows <= 0) return 0;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32)
        add_rmsnorm_kernel<float><<<n_rows, threads, 0, s>>>(residual, (const float*)delta, gain,
                                                              (float*)out, row_index, hidden, eps);
    else if (dtype == VCB_BF16)
        add_rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, 0, s>>>(
            residual, (const __nv_bfloat16*)delta, gain, (__nv_bfloat16*)out, row_index, hidden, eps);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------------------- gated activation
// out[t, i] = silu(gu[t, i]) * gu[t, inter + i],  silu(z) = z / (1 + exp(-z))
// (src/kernels/activation.cu:8-10,34-39), evaluated in float with expf.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter) {
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

VCB_EXPORT int vcb_silu_mul(const void* gu, void* out, int n_tokens, int inter, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    const int threads = 256;
    int bx = (inter + threads - 1) / threads;
    if (bx > 64) bx = 64;
    dim3 grid(bx, n_tokens);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32)
        silu_mul_kernel<float><<<grid, threads, 0, s>>>((const float*)gu, (float*)out, inter);
    else if (dtype == VCB_BF16)
        silu_mul_kernel<__nv_bfloat16><<<grid, threads, 0, s>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter);
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
//   [page][k|v][kv_head][slot][d].
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
};

template <typename T>
__global__ void rope_cache_kernel(RopeCacheArgs a) {
    const int t = blockIdx.x;
    const int nheads = a.nh + 2 * a.nkv;
    const int half = a.d / 2, rhalf = a.rot / 2;
    const int pos = a.positions[t];
    const T* src = (const T*)a.qkv + (size_t)t * nheads * a.d;
    T* qdst = (T*)a.q_out + (size_t)t * a.nh * a.d;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (a.write_kv) {
        const int r = a.req_of_token[t];
        const int pg = a.block_table[(size_t)r * a.bt_stride + pos / a.page];
        const int slot = pos % a.page;
        // [page][2][nkv][slot][d]
        T* base = (T*)a.cache + (size_t)pg * 2 * a.nkv * a.page * a.d;
        kdst = base + (size_t)slot * a.d;
        vdst = base + (size_t)a.nkv * a.page * a.d + (size_t)slot * a.d;
    }
    const int items = nheads * half;
    for (int it = threadIdx.x; it < items; it += blockDim.x) {
        const int h = it / half, j = it % half;
        int ia, ib;
        bool rotate = false;
        if (h < a.nh + a.nkv && j < rhalf) {
            rotate = true;
            if (a.pairing == 0) { ia = j; ib = j + rhalf; }
            else                { ia = 2 * j; ib = 2 * j + 1; }
        } else if (j < rhalf) {               // v head, slots that q/k rotate: plain pair
            if (a.pairing == 0) { ia = j; ib = j + rhalf; }
            else                { ia = 2 * j; ib = 2 * j + 1; }
        } else {                              // beyond the rotary part: pass through
            ia = a.rot + 2 * (j - rhalf); ib = ia + 1;
        }
        float xa = to_f32<T>(src[h * a.d + ia]);
        float xb = to_f32<T>(src[h * a.d + ib]);
        if (a.bias) { xa += a.bias[h * a.d + ia]; xb += a.bias[h * a.d + ib]; }
        if (rotate) {
            const float ang = (float)pos / a.denom[j];
            float sn, cs;
            sincosf(ang, &sn, &cs);
            const float ra = xa * cs - xb * sn;
            const float rb = xa * sn + xb * cs;
            xa = ra; xb = rb;
        }
        if (h < a.nh) {
            qdst[h * a.d + ia] = from_f32<T>(xa);
            qdst[h * a.d + ib] = from_f32<T>(xb);
        } else if (a.write_kv) {
            if (h < a.nh + a.nkv) {
                T* p = kdst + (size_t)(h - a.nh) * a.page * a.d;
                p[ia] = from_f32<T>(xa); p[ib] = from_f32<T>(xb);
            } else {
                T* p = vdst + (size_t)(h - a.nh - a.nkv) * a.page * a.d;
                p[ia] = from_f32<T>(xa); p[ib] = from_f32<T>(xb);
            }
        }
    }
}

VCB_EXPORT int vcb_rope_cache_write(const void* qkv, const float* bias, const int* positions,
                                    const int* req_of_token, const int* block_table, int bt_stride,
                                    const float* denom, void* q_out, void* cache, int n_tokens,
                                    int nh, int nkv, int d, int rot, int pairing, int page,
                                    int write_kv, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0 || (d & 1) || rot < 0 || rot > d || (rot & 1) || page <= 0 || nh <= 0 || nkv < 0)
        return VCB_ERR_BAD_ARG;
    RopeCacheArgs a{qkv, bias, positions, req_of_token, block_table, denom, q_out, cache,
                    bt_stride, nh, nkv, d, rot, pairing, page, write_kv};
    const int items = (nh + 2 * nkv) * (d / 2);
    const int threads = items >= 1024 ? 256 : (items >= 256 ? 128 : 64);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32) rope_cache_kernel<float><<<n_tokens, threads, 0, s>>>(a);
    else if (dtype == VCB_BF16) rope_cache_kernel<__nv_bfloat16><<<n_tokens, threads, 0, s>>>(a);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}

// ------------------------------------------------------------------- bias
// x[t, c] += bias[c] in float (src/kernels/embedding_kernel.cu:55-67).  Only the
// path of a position encoding that the fused kernel does not know uses it.
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, const float* __restrict__ bias, int cols) {
    T* row = x + (size_t)blockIdx.x * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) row[c] = from_f32<T>(to_f32<T>(row[c]) + bias[c]);
}

VCB_EXPORT int vcb_add_bias(void* x, const float* bias, int rows, int cols, int dtype, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VCB_F32) add_bias_kernel<float><<<rows, 256, 0, s>>>((float*)x, bias, cols);
    else if (dtype == VCB_BF16) add_bias_kernel<__nv_bfloat16><<<rows, 256, 0, s>>>((__nv_bfloat16*)x, bias, cols);
    else return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}
