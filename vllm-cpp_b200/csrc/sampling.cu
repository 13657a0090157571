// Sampling on the device, one CTA per logits row, so that only token ids cross
// to the host.  The reference samples on the CPU after copying the whole row
// (src/core/engine.cpp:209-214, src/sampler/sampler.cpp:23-79).
//
// Per row, in the reference's order:
//   1. repetition penalty on the ids generated so far, each once:
//      l > 0 ? l / penalty : l * penalty            (sampler.cpp:81-92)
//   2. temperature <= 0: the largest logit, the lowest id on ties (sampler.cpp:11-21)
//   3. else l *= 1/temperature (sampler.cpp:94-99), softmax (topk_topp.cpp:37-47),
//      optional top-k and top-p in order of falling probability with ties by
//      lower id (topk_topp.cpp:8-35), and an inverse-CDF draw with the given
//      uniform number u: the first kept entry whose running sum exceeds u
//      (topk_topp.cpp:49-56).
// The uniform numbers come from the host (a counter-based generator keyed by the
// request's seed and the index of the token), which the reference does not do: its
// generator is seeded from random_device (sampler.cpp:68).
#include "common.cuh"

#define SAMPLE_THREADS 1024

// ------------------------------------------------------------ penalty
// ids: unique generated ids of all rows, CSR by row_start[n_rows + 1].
__global__ void repetition_penalty_kernel(float* logits, int ld, const int* ids, const int* row_start,
                                          const float* penalty, int vocab) {
    const int row = blockIdx.x;
    const float p = penalty[row];
    if (p == 1.0f) return;
    float* l = logits + (size_t)row * ld;
    for (int i = row_start[row] + threadIdx.x; i < row_start[row + 1]; i += blockDim.x) {
        const int id = ids[i];
        if (id < 0 || id >= vocab) continue;
        const float v = l[id];
        l[id] = v > 0.0f ? v / p : v * p;
    }
}

VCB_EXPORT int vcb_repetition_penalty(float* logits, int ld, const int* ids, const int* row_start,
                                      const float* penalty, int n_rows, int vocab, void* stream) {
    if (n_rows <= 0) return 0;
    repetition_penalty_kernel<<<n_rows, 256, 0, (cudaStream_t)stream>>>(logits, ld, ids, row_start, penalty, vocab);
    return vcb_last_error();
}

// ------------------------------------------------- greedy / temperature
__device__ __forceinline__ void argmax_combine(float& bv, int& bi, float ov, int oi) {
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}

// Inclusive scan of one float per thread over the CTA; returns this thread's
// inclusive value, *total gets the sum.  scratch: 33 floats.
__device__ __forceinline__ float block_inclusive_scan(float v, float* scratch, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    float x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = x;
    __syncthreads();
    if (warp == 0) {
        float w = lane < nwarps ? scratch[lane] : 0.0f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float y = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += y;
        }
        scratch[lane] = w;                 // inclusive sums of the warps
    }
    __syncthreads();
    const float before = warp > 0 ? scratch[warp - 1] : 0.0f;
    *total = scratch[nwarps - 1];
    return x + before;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temperature,
              const float* __restrict__ uniform, int* __restrict__ out) {
    __shared__ float scratch[33];
    __shared__ float sval[32];
    __shared__ int sidx[32];
    __shared__ int winner;
    const int row = blockIdx.x;
    const float* l = logits + (size_t)row * ld;
    const float temp = temperature[row];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;

    // The largest logit and its lowest id; the maximum is also softmax's shift.
    float bv = -INFINITY;
    int bi = vocab;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) argmax_combine(bv, bi, l[i], i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_combine(bv, bi, ov, oi);
    }
    if (lane == 0) { sval[warp] = bv; sidx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < nwarps ? sval[lane] : -INFINITY;
        bi = lane < nwarps ? sidx[lane] : vocab;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            argmax_combine(bv, bi, ov, oi);
        }
        if (lane == 0) { sval[0] = bv; sidx[0] = bi; }
    }
    __syncthreads();
    const float lmax = sval[0];
    const int imax = sidx[0] < vocab ? sidx[0] : 0;
    if (temp <= 0.0f) {
        if (threadIdx.x == 0) out[row] = imax;
        return;
    }

    // exp((l - max) / T) summed over a contiguous range of ids per thread, so
    // that the running sum follows the order of the ids.
    const float inv_t = 1.0f / temp;
    const float xmax = temp != 1.0f ? lmax * inv_t : lmax;
    const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
    const int lo = min(vocab, (int)threadIdx.x * chunk), hi = min(vocab, lo + chunk);
    float local = 0.0f;
    for (int i = lo; i < hi; ++i) {
        const float x = temp != 1.0f ? l[i] * inv_t : l[i];
        local += expf(x - xmax);
    }
    float total;
    const float incl = block_inclusive_scan(local, scratch, &total);
    const float target = uniform[row] * total;
    if (threadIdx.x == 0) winner = blockDim.x;
    __syncthreads();
    if (hi > lo && target < incl) atomicMin(&winner, (int)threadIdx.x);
    __syncthreads();
    if (winner == (int)blockDim.x) {             // u * total >= total after rounding: the last id
        if (threadIdx.x == 0) out[row] = vocab - 1;
        return;
    }
    if ((int)threadIdx.x == winner) {
        float c = incl - local;
        int tok = hi - 1;
        for (int i = lo; i < hi; ++i) {
            const float x = temp != 1.0f ? l[i] * inv_t : l[i];
            c += expf(x - xmax);
            if (target < c) { tok = i; break; }
        }
        out[row] = tok;
    }
}

VCB_EXPORT int vcb_sample(const float* logits, int ld, int vocab, const float* temperature,
                          const float* uniform, int* out, int n_rows, void* stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0 || ld < vocab) return VCB_ERR_BAD_ARG;
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, ld, vocab, temperature, uniform, out);
    return vcb_last_error();
}
