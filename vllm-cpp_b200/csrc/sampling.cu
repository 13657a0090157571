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
    if ((((uintptr_t)l) & 15) == 0) {
        const int nvec = vocab >> 2;
        const float4* l4 = reinterpret_cast<const float4*>(l);
        // four loads in flight per thread: one at a time is a round trip to the L2 cache per 16 bytes
        constexpr int U = 4;
        int i = threadIdx.x;
        for (; i + (U - 1) * (int)blockDim.x < nvec; i += U * blockDim.x) {
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = l4[i + u * blockDim.x];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int id = 4 * (i + u * (int)blockDim.x);
                argmax_combine(bv, bi, v[u].x, id); argmax_combine(bv, bi, v[u].y, id + 1);
                argmax_combine(bv, bi, v[u].z, id + 2); argmax_combine(bv, bi, v[u].w, id + 3);
            }
        }
        for (; i < nvec; i += blockDim.x) {
            const float4 v = l4[i];
            argmax_combine(bv, bi, v.x, 4 * i); argmax_combine(bv, bi, v.y, 4 * i + 1);
            argmax_combine(bv, bi, v.z, 4 * i + 2); argmax_combine(bv, bi, v.w, 4 * i + 3);
        }
        for (int i = (nvec << 2) + threadIdx.x; i < vocab; i += blockDim.x) argmax_combine(bv, bi, l[i], i);
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) argmax_combine(bv, bi, l[i], i);
    }
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

    // e_i = exp((l_i - max) / T).  Every warp owns a contiguous slab of ids, so the warps' sums, taken in the
    // order of the warps, follow the order of the ids; inside its slab a warp reads rows of 128 ids (a float4
    // a lane, four rows in flight), each lane adding up what it reads.  The slab that holds the draw is then
    // walked once more by its warp, row by row in the order of the ids.
    const float inv_t = 1.0f / temp;
    const float xmax = temp != 1.0f ? lmax * inv_t : lmax;
    const bool scaled = temp != 1.0f;
    auto weight = [&](float v) { return expf((scaled ? v * inv_t : v) - xmax); };
    const bool aligned = (((uintptr_t)l) & 15) == 0;
    const int slab = ((vocab + nwarps - 1) / nwarps + 127) & ~127;
    const int lo = min(vocab, warp * slab), hi = min(vocab, lo + slab);
    // the four weights of this lane in the row that starts at id `base` (zero beyond the slab)
    auto row_weights = [&](int base, float (&e)[4]) {
        const int i = base + lane * 4;
        if (aligned && i + 3 < hi) {
            const float4 v = *reinterpret_cast<const float4*>(l + i);
            e[0] = weight(v.x); e[1] = weight(v.y); e[2] = weight(v.z); e[3] = weight(v.w);
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) e[k] = i + k < hi ? weight(l[i + k]) : 0.0f;
        }
    };
    float local = 0.0f;
    {
        constexpr int U = 4;
        int base = lo;
        if (aligned) {
            for (; base + U * 128 <= hi; base += U * 128) {
                float4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) v[u] = *reinterpret_cast<const float4*>(l + base + u * 128 + lane * 4);
#pragma unroll
                for (int u = 0; u < U; ++u) local += (weight(v[u].x) + weight(v[u].y)) + (weight(v[u].z) + weight(v[u].w));
            }
        }
        for (; base < hi; base += 128) {
            float e[4];
            row_weights(base, e);
            local += (e[0] + e[1]) + (e[2] + e[3]);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);      // the slab's sum, in all lanes
    if (lane == 0) scratch[warp] = local;
    __syncthreads();
    if (warp == 0) {
        float w = lane < nwarps ? scratch[lane] : 0.0f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float y = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += y;
        }
        scratch[lane] = w;                 // inclusive sums of the slabs
    }
    if (threadIdx.x == 0) winner = nwarps;
    __syncthreads();
    const float total = scratch[nwarps - 1];
    const float incl = scratch[warp];
    const float target = uniform[row] * total;
    if (lane == 0 && hi > lo && target < incl) atomicMin(&winner, warp);
    __syncthreads();
    if (winner == nwarps) {                      // u * total >= total after rounding: the last id
        if (threadIdx.x == 0) out[row] = vocab - 1;
        return;
    }
    if (warp != winner) return;
    float c = incl - local;                      // the sum before this slab
    int tok = hi - 1;                            // if rounding keeps the walk's sums below the draw: the slab's last id
    for (int base = lo; base < hi; base += 128) {
        float e[4];
        row_weights(base, e);
        const float p1 = e[0], p2 = p1 + e[1], p3 = p2 + e[2], p4 = p3 + e[3];
        float upto = p4;                         // inclusive sum of the lanes' four
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float y = __shfl_up_sync(0xffffffffu, upto, o);
            if (lane >= o) upto += y;
        }
        const float before = c + (upto - p4);
        const int i = base + lane * 4;
        int hit = -1;
        if (i < hi) {
            if (target < before + p1) hit = i;
            else if (target < before + p2 && i + 1 < hi) hit = i + 1;
            else if (target < before + p3 && i + 2 < hi) hit = i + 2;
            else if (target < before + p4 && i + 3 < hi) hit = i + 3;
        }
        const unsigned found = __ballot_sync(0xffffffffu, hit >= 0);
        if (found) {
            tok = __shfl_sync(0xffffffffu, hit, __ffs(found) - 1);
            break;
        }
        c += __shfl_sync(0xffffffffu, upto, 31);
    }
    if (lane == 0) out[row] = tok;
}

VCB_EXPORT int vcb_sample(const float* logits, int ld, int vocab, const float* temperature,
                          const float* uniform, int* out, int n_rows, void* stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0 || ld < vocab) return VCB_ERR_BAD_ARG;
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, ld, vocab, temperature, uniform, out);
    return vcb_last_error();
}

// --------------------------------------------------------- top-k / top-p
// Rows with temperature > 0 and (top_p < 1 or top_k > 0) are drawn here, in order
// of falling probability with ties by lower id, as the reference does after its
// sort (src/sampler/sampler.cpp:52-71, src/sampler/topk_topp.cpp:8-35,49-56).
// Nothing is sorted.  Every id gets the 52-bit key  (bits of e_i) << 20 | (0xFFFFF - i)
// with e_i = exp((l_i - max) / T) >= 0, so a larger key means "earlier in the
// reference's order".  With count(T) and sum(T) taken over the ids whose key is >= T:
//   top-k keeps keys >= T_k, the largest T with count(T) >= k;
//   top-p keeps keys >= T_p, the largest T with sum(T) >= p * sum(T_k);
//   the draw returns the id of the largest T with sum(T) > u * sum(T_p).
// Each threshold is found four bits at a time (13 passes over the row): a pass
// bins the ids that agree with the bits found so far by their next four bits and
// picks the largest digit for which the condition still holds.  The sums are
// taken in a fixed order, so a row's result does not change from run to run.
// e is kept in scratch memory supplied by the caller: rows * vocab floats.
#define FILT_THREADS 1024
enum { COND_COUNT_GE = 0, COND_SUM_GE = 1, COND_SUM_GT = 2 };

__device__ __forceinline__ unsigned long long filt_key(float e, int id) {
    return ((unsigned long long)__float_as_uint(e) << 20) | (unsigned long long)(0xFFFFF - id);
}

struct FiltShared {
    float wsum[32][16];
    int wcnt[32][16];
    float tsum[16];
    int tcnt[16];
    int digit;
    float above_sum, ge_sum;
    int above_cnt, ge_cnt;
};

// The largest key T (52 bits) for which the condition holds, counting only ids with
// key >= floor_key.  On return sh.ge_sum / sh.ge_cnt hold sum(T) / count(T).
template <int COND>
__device__ unsigned long long filt_search(const float* __restrict__ e, int vocab,
                                          unsigned long long floor_key, float bound, FiltShared& sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    unsigned long long prefix = 0;
    if (threadIdx.x == 0) { sh.above_sum = 0.0f; sh.above_cnt = 0; }
    for (int shift = 48; shift >= 0; shift -= 4) {
        float bs[16];
        int bc[16];
#pragma unroll
        for (int v = 0; v < 16; ++v) { bs[v] = 0.0f; bc[v] = 0; }
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float ei = e[i];
            const unsigned long long key = filt_key(ei, i);
            if (key < floor_key) continue;
            if ((key >> (shift + 4)) != (prefix >> (shift + 4))) continue;
            const int d = (int)((key >> shift) & 15);
#pragma unroll
            for (int v = 0; v < 16; ++v)
                if (d == v) { bs[v] += ei; bc[v] += 1; }
        }
#pragma unroll
        for (int v = 0; v < 16; ++v) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                bs[v] += __shfl_xor_sync(0xffffffffu, bs[v], o);
                bc[v] += __shfl_xor_sync(0xffffffffu, bc[v], o);
            }
        }
        __syncthreads();
        if (lane == 0) {
#pragma unroll
            for (int v = 0; v < 16; ++v) { sh.wsum[warp][v] = bs[v]; sh.wcnt[warp][v] = bc[v]; }
        }
        __syncthreads();
        if (threadIdx.x < 16) {
            float s = 0.0f;
            int c = 0;
            for (int w = 0; w < nwarps; ++w) { s += sh.wsum[w][threadIdx.x]; c += sh.wcnt[w][threadIdx.x]; }
            sh.tsum[threadIdx.x] = s;
            sh.tcnt[threadIdx.x] = c;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float s = sh.above_sum;
            int c = sh.above_cnt;
            int chosen = 0;
            float chosen_above_s = s, chosen_s = s;
            int chosen_above_c = c, chosen_c = c;
            bool found = false;
            for (int v = 15; v >= 0; --v) {
                const float s_above = s;
                const int c_above = c;
                s += sh.tsum[v];
                c += sh.tcnt[v];
                bool ok;
                if (COND == COND_COUNT_GE) ok = (float)c >= bound;
                else if (COND == COND_SUM_GE) ok = s >= bound;
                else ok = s > bound;
                if (ok && !found) {
                    found = true; chosen = v;
                    chosen_above_s = s_above; chosen_above_c = c_above;
                    chosen_s = s; chosen_c = c;
                }
            }
            if (!found) {
                // The digits above were chosen because their running sum met the bound; here the same ids,
                // added up bin by bin, fall short of it by a rounding step of the sum (which is as large as a
                // single id's share once the row has 10^5 ids of similar weight).  The bound then lies at the
                // end of this prefix's range: take all of it, which is the lowest digit that has any id.
                // (Digit 0 regardless would lead to a key that no id has.)
                int lowest = 0;
                while (lowest < 15 && sh.tcnt[lowest] == 0) ++lowest;
                chosen = lowest;
                chosen_above_s = s - sh.tsum[lowest]; chosen_above_c = c - sh.tcnt[lowest];
                chosen_s = s; chosen_c = c;
            }
            sh.digit = chosen;
            sh.above_sum = chosen_above_s; sh.above_cnt = chosen_above_c;
            sh.ge_sum = chosen_s; sh.ge_cnt = chosen_c;
        }
        __syncthreads();
        prefix |= (unsigned long long)sh.digit << shift;
    }
    return prefix;
}

__global__ void __launch_bounds__(FILT_THREADS)
sample_filtered_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temperature,
                       const float* __restrict__ uniform, const float* __restrict__ top_p,
                       const int* __restrict__ top_k, float* __restrict__ scratch, int* __restrict__ out) {
    __shared__ FiltShared sh;
    __shared__ float red[33];
    const int row = blockIdx.x;
    const float temp = temperature[row], p = top_p[row];
    const int k = top_k[row];
    if (!(temp > 0.0f) || !(p < 1.0f || k > 0)) return;      // sample_kernel has drawn this row
    const float* l = logits + (size_t)row * ld;
    float* e = scratch + (size_t)row * vocab;
    const float inv_t = 1.0f / temp;

    float mx = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, temp != 1.0f ? l[i] * inv_t : l[i]);
    mx = block_max(mx, red);
    float part = 0.0f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = expf((temp != 1.0f ? l[i] * inv_t : l[i]) - mx);
        e[i] = v;
        part += v;
    }
    float kept_sum = block_sum(part, red);        // also orders the writes of e before the reads below

    unsigned long long floor_key = 0;
    if (k > 0 && k < vocab) {
        floor_key = filt_search<COND_COUNT_GE>(e, vocab, 0ull, (float)k, sh);
        kept_sum = sh.ge_sum;
    }
    if (p < 1.0f) {
        floor_key = filt_search<COND_SUM_GE>(e, vocab, floor_key, p * kept_sum, sh);
        kept_sum = sh.ge_sum;
    }
    const unsigned long long t = filt_search<COND_SUM_GT>(e, vocab, floor_key, uniform[row] * kept_sum, sh);
    if (threadIdx.x == 0) out[row] = 0xFFFFF - (int)(t & 0xFFFFFull);
}

VCB_EXPORT int vcb_sample_filtered(const float* logits, int ld, int vocab, const float* temperature,
                                   const float* uniform, const float* top_p, const int* top_k,
                                   float* scratch, int* out, int n_rows, void* stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0 || ld < vocab) return VCB_ERR_BAD_ARG;
    if (vocab > (1 << 20)) return VCB_ERR_UNSUPPORTED;      // ids take 20 bits of the key
    sample_filtered_kernel<<<n_rows, FILT_THREADS, 0, (cudaStream_t)stream>>>(
        logits, ld, vocab, temperature, uniform, top_p, top_k, scratch, out);
    return vcb_last_error();
}
