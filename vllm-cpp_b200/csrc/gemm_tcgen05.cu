// bfloat16 matrix product on the fifth-generation tensor cores of sm_100a:
//   D[i, j] = sum_k P[i, k] * Q[j, k],   P: [rows_p, K], Q: [rows_q, K], both row-major
// tcgen05.mma (kind::f16, bfloat16 in, float accumulate in tensor memory) fed by TMA
// (cp.async.bulk.tensor, 128-byte swizzle) through a ring of shared-memory stages
// guarded by mbarriers, one CTA per 128 x BN tile of D and per slice of K.
//
// Two uses with the same kernel.  Prefill: P = activations (tokens), Q = weights, the
// tile is stored as it is: C[token, feature].  Decode: P = weights, Q = the few tokens
// of the step ("swap A and B"): the 128 rows of the tensor-core tile are weight rows,
// so a step with 8 tokens streams every weight once at full tile efficiency, and the
// tile is stored transposed: C[token, feature].  K can be split over CTAs so that
// products with few output tiles still fill the GPU; partial tiles meet in global
// scratch memory and the CTA that takes a tile's last ticket adds them up.
//
// Warp roles (192 threads): warp 0 issues TMA loads, warp 1 allocates tensor memory and
// issues the MMAs (one elected lane each), warps 2-5 read the accumulator back
// (tcgen05.ld, each warp its own 32 lanes) and store.  No load uses cluster multicast.
// Every wait on an mbarrier is bounded; a wait that runs out records where in *status,
// the CTA stops issuing work, frees its tensor memory and returns.
//
// Replaces cublasGemmEx of the reference (src/layers/linear.cpp:70-77).
#include "common.cuh"

#include <cuda.h>

namespace {

constexpr int BM = 128;          // rows of P per tile = UMMA M
constexpr int BK = 64;           // k per stage: 64 bfloat16 = 128 bytes = one swizzle span
constexpr int UMMA_K = 16;
constexpr int P_BYTES = BM * BK * 2;
constexpr int GEMM_THREADS = 192;
constexpr uint32_t SPIN_LIMIT = 1u << 22;     // try_wait attempts before a wait gives up

struct GemmArgs {
    void* out;
    float* partial;              // [splits][out rows][ldc] floats when splits > 1
    int* tickets;                // one per output tile, zero between launches
    int* status;                 // 0, or the code of the first wait that ran out
    int ldc, out_f32, swapped, rows_p, rows_q, k_slabs, splits, out_rows;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity.  False: gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.b32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, swizzled
// in 128-byte spans as TMA wrote it: 8-row groups 1024 bytes apart.
//   bits 0-13 address >> 4, 16-29 leading offset >> 4 (unused here: 1), 32-45 stride between
//   8-row groups >> 4, 46-47 version 1, 61-63 layout 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: float accumulator (bits 4-5 = 1), A and B bfloat16 (bits 7-9, 10-12 = 1),
// both K-major (bits 15, 16 = 0), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}


template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, GemmArgs a) {
    constexpr int Q_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = P_BYTES + Q_BYTES;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;        // tensor memory comes in powers of two from 32 columns
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + STAGES), acc_bar = smem_addr(bars + 2 * STAGES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
    volatile int* flags = reinterpret_cast<volatile int*>(tmem_slot + 1);      // [0] abort, [1] ticket
    const uint32_t tiles0 = smem_addr(smem);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p0 = blockIdx.x * BM, q0 = blockIdx.y * BN, split = blockIdx.z;
    const int per = (a.k_slabs + a.splits - 1) / a.splits;
    const int slab0 = split * per;
    const int n_slabs = max(0, min(a.k_slabs, slab0 + per) - slab0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(acc_bar, 1);
        flags[0] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer
        if (lane == 0) {
            for (int it = 0; it < n_slabs; ++it) {
                const int s = it % STAGES;
                const uint32_t phase = (it / STAGES) & 1;
                if (flags[0] || !mbar_wait(empty0 + 8 * s, phase ^ 1)) {
                    if (!flags[0]) { flags[0] = 1; atomicCAS(a.status, 0, 1); }
                    break;
                }
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                const uint32_t dst = tiles0 + s * STAGE_BYTES;
                tma_load_2d(dst, &map_p, full0 + 8 * s, (slab0 + it) * BK, p0);
                tma_load_2d(dst + P_BYTES, &map_q, full0 + 8 * s, (slab0 + it) * BK, q0);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BN);
            int it = 0;
            for (; it < n_slabs; ++it) {
                const int s = it % STAGES;
                const uint32_t phase = (it / STAGES) & 1;
                if (flags[0] || !mbar_wait(full0 + 8 * s, phase)) {
                    if (!flags[0]) { flags[0] = 1; atomicCAS(a.status, 0, 2); }
                    break;
                }
                tc_fence_after();
                const uint32_t pa = tiles0 + s * STAGE_BYTES, qa = pa + P_BYTES;
#pragma unroll
                for (int j = 0; j < BK / UMMA_K; ++j)
                    tc_mma(tmem_d, smem_desc(pa + j * UMMA_K * 2), smem_desc(qa + j * UMMA_K * 2), idesc,
                           (it > 0 || j > 0) ? 1u : 0u);
                tc_commit(empty0 + 8 * s);          // the stage is free once these MMAs have read it
            }
            tc_commit(acc_bar);                     // the accumulator is complete once all MMAs are done
        }
    } else {
        // ---- epilogue: warps 2..5 own tensor-memory lanes 32 * (warp % 4) ..
        const int lg = warp & 3;
        const int i = p0 + lg * 32 + lane;          // row of P this thread holds
        bool ok = !flags[0] && mbar_wait(acc_bar, 0);
        if (!ok && !flags[0]) { flags[0] = 1; atomicCAS(a.status, 0, 3); }
        ok = ok && !flags[0];
        tc_fence_after();
        float* part = a.splits > 1 ? a.partial + (size_t)split * a.out_rows * a.ldc : nullptr;
        if (ok) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                uint32_t v[16];
                if (n_slabs > 0) {
                    tc_ld16(tmem_d + ((uint32_t)(lg * 32) << 16) + c, v);
                } else {
#pragma unroll
                    for (int e = 0; e < 16; ++e) v[e] = 0;
                }
                if (i >= a.rows_p) continue;
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const int j = q0 + c + e;
                    if (j >= a.rows_q) break;
                    const size_t idx = a.swapped ? (size_t)j * a.ldc + i : (size_t)i * a.ldc + j;
                    const float f = __uint_as_float(v[e]);
                    if (part) part[idx] = f;
                    else if (a.out_f32) reinterpret_cast<float*>(a.out)[idx] = f;
                    else reinterpret_cast<__nv_bfloat16*>(a.out)[idx] = __float2bfloat16_rn(f);
                }
            }
        }
        if (part) {
            // partial tiles of all splits meet here; the last CTA of this tile adds them up
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) flags[1] = atomicAdd(&a.tickets[blockIdx.y * gridDim.x + blockIdx.x], 1);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (flags[1] == a.splits - 1) {
                __threadfence();
                if (i < a.rows_p) {
                    for (int c = 0; c < BN; ++c) {
                        const int j = q0 + c;
                        if (j >= a.rows_q) break;
                        const size_t idx = a.swapped ? (size_t)j * a.ldc + i : (size_t)i * a.ldc + j;
                        float f = 0.0f;
                        for (int sp = 0; sp < a.splits; ++sp) f += __ldcg(a.partial + (size_t)sp * a.out_rows * a.ldc + idx);
                        if (a.out_f32) reinterpret_cast<float*>(a.out)[idx] = f;
                        else reinterpret_cast<__nv_bfloat16*>(a.out)[idx] = __float2bfloat16_rn(f);
                    }
                }
                if (threadIdx.x == 64) a.tickets[blockIdx.y * gridDim.x + blockIdx.x] = 0;
            }
        }
    }
    // An aborted CTA may still have copies in flight: give each armed stage a bounded chance to land.
    if (flags[0] && threadIdx.x == 0)
        for (int s = 0; s < STAGES; ++s) mbar_wait(full0 + 8 * s, 0);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// A [rows, k] bfloat16 matrix with row stride ld, read in boxes of 64 x box_rows with 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int rows, int k, int ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return VCB_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : VCB_ERR_BAD_ARG;
}

template <int BN, int STAGES>
int launch(const CUtensorMap& mp, const CUtensorMap& mq, const GemmArgs& a, cudaStream_t s) {
    constexpr size_t smem = (size_t)STAGES * (P_BYTES + BN * BK * 2) + 1024 + 256;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((a.rows_p + BM - 1) / BM, (a.rows_q + BN - 1) / BN, a.splits);
    gemm_tcgen05_kernel<BN, STAGES><<<grid, GEMM_THREADS, smem, s>>>(mp, mq, a);
    return vcb_last_error();
}

}  // namespace

// out[r, c] (row stride ldc, bfloat16 or float) = sum_k ...
//   swapped = 0: P = activations [rows_p = tokens], Q = weights [rows_q = features]: out[p, q]
//   swapped = 1: P = weights [rows_p = features], Q = activations [rows_q = tokens]:  out[q, p]
// bn: columns of the tensor-core tile (16, 32, 64, 128 or 256; rows_q is cut into tiles of bn).
// splits > 1 needs partial (splits * out_rows * ldc floats) and tickets (one zeroed int per tile).
VCB_EXPORT int vcb_gemm_bf16_tcgen05(const void* p, int rows_p, int ldp, const void* q, int rows_q, int ldq, int k,
                                     void* out, int ldc, int out_f32, int swapped, int bn, int splits,
                                     float* partial, int* tickets, int* status, void* stream) {
    if (rows_p <= 0 || rows_q <= 0) return 0;
    if (k <= 0 || splits < 1 || !status) return VCB_ERR_BAD_ARG;
    // TMA needs 16-byte aligned bases and row strides
    if ((k % 8) || (ldp % 8) || (ldq % 8) || (((uintptr_t)p | (uintptr_t)q) & 15)) return VCB_ERR_UNSUPPORTED;
    if (splits > 1 && (!partial || !tickets)) return VCB_ERR_BAD_ARG;
    const int k_slabs = (k + BK - 1) / BK;
    if (splits > k_slabs) splits = k_slabs;
    CUtensorMap mp, mq;
    int c = make_map(&mp, p, rows_p, k, ldp, BM);
    if (c) return c;
    c = make_map(&mq, q, rows_q, k, ldq, bn);
    if (c) return c;
    GemmArgs a{out, partial, tickets, status, ldc, out_f32, swapped, rows_p, rows_q, k_slabs, splits,
               swapped ? rows_q : rows_p};
    cudaStream_t s = (cudaStream_t)stream;
    switch (bn) {
        case 16: return launch<16, 10>(mp, mq, a, s);
        case 32: return launch<32, 9>(mp, mq, a, s);
        case 64: return launch<64, 8>(mp, mq, a, s);
        case 128: return launch<128, 6>(mp, mq, a, s);
        case 256: return launch<256, 4>(mp, mq, a, s);
        default: return VCB_ERR_BAD_ARG;
    }
}
