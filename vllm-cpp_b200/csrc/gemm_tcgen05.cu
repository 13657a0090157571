// bfloat16 matrix product on the fifth-generation tensor cores of sm_100a:
//   D[i, j] = sum_k P[i, k] * Q[j, k],   P: [rows_p, K], Q: [rows_q, K], both row-major
// tcgen05.mma (kind::f16, bfloat16 in, float accumulate in tensor memory) fed by TMA
// (cp.async.bulk.tensor, 128-byte swizzle) through a ring of shared-memory stages
// guarded by mbarriers.
//
// Two uses with the same kernel.  Prefill: P = activations (tokens), Q = weights, a
// 128 x BN tile is stored as it is: C[token, feature].  Decode: P = weights, Q = the few
// tokens of the step ("swap A and B"): the 128 rows of the tensor-core tile are weight
// rows, so a step with 8 tokens streams every weight once at full tile efficiency, and the
// tile is stored transposed: C[token, feature].
//
// Work is cut stream-K fashion: the (tile, 64-wide k slab) pairs of the whole product are
// numbered tile by tile and dealt out in equal contiguous runs to one persistent CTA per
// SM, so every SM streams the same number of bytes whatever the shape.  A CTA's run is a
// sequence of segments (a tile and a range of its slabs).  A segment that covers all of K
// is stored directly; the others leave float partial tiles in global scratch memory, take
// a ticket of their tile, and the CTA that draws the tile's last ticket adds them up: no CTA
// waits for another.  (Tiles of 32 columns and more share the merge among the tile's CTAs at the end
// of their runs instead, see the epilogue.)  The ring of stages runs on across segments, and two
// accumulators in tensor memory alternate, so loads and MMAs of the next segment overlap
// the read-back of the last.
//
// Weight layout for decode.  A TMA tensor copy pays for every 128-byte row piece of its box
// (about 7 cycles each on this part, measured: 35 GB/s per SM whatever the shape), which is
// below what a weight-bound product needs.  So the weights can also be given pre-tiled:
// the matrix cut into 128-row x 64-column tiles, each stored as the 16 KB image that the
// 128-byte-swizzled TMA copy would have produced in shared memory (vcb_tile_weights makes
// it once at load).  A stage is then filled by one plain bulk copy (cp.async.bulk) of 16 KB
// of contiguous memory, and only the few activation rows still go through a tensor map.
//
// Warp roles (192 threads): warp 0 issues TMA loads, warp 1 allocates tensor memory and
// issues the MMAs (one elected lane each), warps 2-5 read the accumulators back
// (tcgen05.ld, each warp its own 32 lanes) and store.  No load uses cluster multicast.
// Every wait on an mbarrier is bounded; a wait that runs out records where in *status,
// the CTA stops issuing work, frees its tensor memory and returns.
//
// Fused RMSNorm (decode).  norm(x) W^T = rsqrt(mean(x^2) + eps) * ((x * gain) W^T): the per-token factor
// can be applied after the product.  So the product that ends a residual branch (attention's output
// projection, the feed-forward's down projection) can, in its epilogue, add its tile into the float
// residual stream, store bfloat16(residual * gain of the next norm) as the next product's input and
// leave the sums of squares of the new residual, one partial per epilogue warp and token; and the
// next product sums those partials and multiplies its accumulators by the factor before storing.
// No norm kernel runs between the two.  The partials are summed in a fixed order: results do not
// depend on the order in which CTAs finish.
//
// Fused SwiGLU (decode).  For the gate and up projections of a gated feed-forward the tile image can be
// made so that every 128-row tile holds 64 gate rows and the 64 up rows of the same features
// (vcb_tile_weights with gated > 0).  The epilogue then exchanges the two halves through shared
// memory and stores silu(gate) * up: no activation kernel runs and the 2 x wider intermediate
// never reaches memory.
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
    float* partial;              // [ctas][2][BN][128] floats: a CTA's first and last segment
    int* tickets;                // one per tile, zero between launches
    int* status;                 // 0, or the code of the first wait that ran out
    const uint8_t* p_tiled;      // P as 16 KB tile images [tiles_p][k_slabs], or null: P comes through map_p
    int ldc, out_f32, swapped, rows_p, rows_q;
    int k_slabs, tiles_p, units_per_cta, total_units;
    // Fused norm, swapped products with one tile of tokens only (see the epilogue):
    const float* scale_sumsq;    // [scale_parts][scale_ld]: partial sums of squares per token, or null
    int scale_parts, scale_ld;
    float scale_inv_width, scale_eps;
    float* residual;             // [tokens][ldr] float: the product is added into it, or null
    const float* gain;           // [rows_p]: out = bfloat16(residual * gain)
    float* sumsq_out;            // [tiles_p * 4][sumsq_ld]: sums of squares of the new residual, per epilogue warp
    int ldr, sumsq_ld;
    // Gated feed-forward (swapped products on a gated tile image only): > 0 = the number of gate features.
    // Tile t holds gate rows 64 t .. and, in its upper half, the matching up rows;
    // out[token, 64 t + r] = silu(gate) * up.
    int gated;
};

// The segments of one CTA's run of (tile, slab) units.
struct Segments {
    int u, end, slabs;
    __device__ Segments(const GemmArgs& a, int cta)
        : u(cta * a.units_per_cta), end(min((cta + 1) * a.units_per_cta, a.total_units)), slabs(a.k_slabs) {}
    __device__ bool next(int& tile, int& s0, int& s1) {
        if (u >= end) return false;
        tile = u / slabs;
        s0 = u - tile * slabs;
        s1 = min(slabs, s0 + end - u);
        u += s1 - s0;
        return true;
    }
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
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
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

// Bounded wait until *p >= target (a count that other CTAs of this launch raise).  False: gave up.
__device__ __forceinline__ bool wait_count(const int* p, int target) {
    for (uint32_t spin = 0; spin < (1u << 21); ++spin) {
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
        if (v >= target) return true;
        __nanosleep(20);
    }
    return false;
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


__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// One (tile, slab) unit after the other of a CTA's run, for the producer.  What a stage's loads need
// is worked out once per segment, so that a step costs a few instructions: one thread issues every
// load of the CTA, and its instruction latency bounds the CTA's rate.
struct Units {
    Segments seg;
    const GemmArgs& a;
    int bn, slab, s1;
    int p_row, q_row;            // first row of the tile's P and Q boxes
    const uint8_t* p_image;      // the current slab's tile of a tiled P, or null
    bool ok;
    __device__ Units(const GemmArgs& a_, int cta, int bn_) : seg(a_, cta), a(a_), bn(bn_), slab(0), s1(0), p_row(0), q_row(0),
                                                             p_image(nullptr) { next_segment(); }
    __device__ void next_segment() {
        int tile, s0;
        ok = seg.next(tile, s0, s1);
        if (!ok) return;
        const int tp = tile % a.tiles_p;
        slab = s0;
        p_row = tp * BM;
        q_row = (tile / a.tiles_p) * bn;
        p_image = a.p_tiled ? a.p_tiled + ((size_t)tp * a.k_slabs + s0) * P_BYTES : nullptr;
    }
    __device__ __forceinline__ void advance() {
        ++slab;
        if (p_image) p_image += P_BYTES;
        if (slab >= s1) next_segment();
    }
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, GemmArgs a) {
    constexpr int Q_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = P_BYTES + Q_BYTES;
    constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;   // two accumulators; powers of two from 32 columns
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + STAGES);
    const uint32_t acc_full0 = smem_addr(bars + 2 * STAGES), acc_empty0 = smem_addr(bars + 2 * STAGES + 2);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* flags = reinterpret_cast<volatile int*>(tmem_slot + 1);      // [0] abort, [1] ticket
    const uint32_t tiles0 = smem_addr(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x;
    pdl_launch_dependents();            // the next kernel may set itself up while this one streams

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 4); }
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
        // ---- TMA producer.  With the weights on the P side (decode), P tiles of the first
        // stages are requested before the previous kernel has finished: weights depend on
        // nothing.  The activations (Q) follow once griddepcontrol.wait has returned.
        if (lane == 0) {
            Units ahead(a, cta, BN), units(a, cta, BN);
            int it_p = 0, it_q = 0;
            auto load_p = [&](const Units& u, uint32_t dst, uint32_t bar) {
                if (u.p_image) bulk_load(dst, u.p_image, P_BYTES, bar);
                else tma_load_2d(dst, &map_p, bar, u.slab * BK, u.p_row);
            };
            if (a.swapped) {
                for (; ahead.ok && it_p < STAGES; ++it_p, ahead.advance()) {
                    mbar_expect_tx(full0 + 8 * it_p, STAGE_BYTES);
                    load_p(ahead, tiles0 + it_p * STAGE_BYTES, full0 + 8 * it_p);
                }
            }
            pdl_wait();
            for (; it_q < it_p; ++it_q, units.advance())
                tma_load_2d(tiles0 + it_q * STAGE_BYTES + P_BYTES, &map_q, full0 + 8 * it_q, units.slab * BK, units.q_row);
            int s = it_q % STAGES;
            uint32_t parity = ((it_q / STAGES) & 1) ^ 1;
            for (; units.ok && !flags[0]; units.advance()) {
                if (!mbar_wait(empty0 + 8 * s, parity)) {
                    if (!flags[0]) { flags[0] = 1; atomicCAS(a.status, 0, 1); }
                    break;
                }
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                const uint32_t dst = tiles0 + s * STAGE_BYTES;
                load_p(units, dst, full0 + 8 * s);
                tma_load_2d(dst + P_BYTES, &map_q, full0 + 8 * s, units.slab * BK, units.q_row);
                if (++s == STAGES) { s = 0; parity ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BN);
            Segments seg(a, cta);
            int tile, s0, s1, it = 0, n = 0;
            while (!flags[0] && seg.next(tile, s0, s1)) {
                const int buf = n & 1;
                if (!mbar_wait(acc_empty0 + 8 * buf, ((n >> 1) & 1) ^ 1)) {
                    if (!flags[0]) { flags[0] = 1; atomicCAS(a.status, 0, 4); }
                    break;
                }
                tc_fence_after();
                const uint32_t acc = tmem_d + buf * BN;
                for (int slab = s0; slab < s1; ++slab, ++it) {
                    const int s = it % STAGES;
                    if (flags[0] || !mbar_wait(full0 + 8 * s, (it / STAGES) & 1)) {
                        if (!flags[0]) { flags[0] = 1; atomicCAS(a.status, 0, 2); }
                        break;
                    }
                    tc_fence_after();
                    const uint32_t pa = tiles0 + s * STAGE_BYTES, qa = pa + P_BYTES;
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j)
                        tc_mma(acc, smem_desc(pa + j * UMMA_K * 2), smem_desc(qa + j * UMMA_K * 2), idesc,
                               (slab > s0 || j > 0) ? 1u : 0u);
                    tc_commit(empty0 + 8 * s);      // the stage is free once these MMAs have read it
                }
                tc_commit(acc_full0 + 8 * buf);     // the accumulator is complete once all MMAs are done
                ++n;
            }
        }
    } else {
        // ---- epilogue: warps 2..5 own tensor-memory lanes 32 * (warp % 4) ..
        const int lg = warp & 3;
        const int r = lg * 32 + lane;               // row of the tile this thread holds
        const int U = a.units_per_cta, S = a.k_slabs;
        Segments seg(a, cta);
        int tile, s0, s1, n = 0;
        pdl_wait();                                 // nothing is written before the previous kernel is done
        float* rstd_s = reinterpret_cast<float*>(const_cast<int*>(flags + 2));      // [min(BN, 128)]
        float* xch = rstd_s + 128;                    // [64][8]: up halves; tiles of 32 columns and more: [2][16][64]
        if (a.scale_sumsq) {
            // The factor of every token: rsqrt(sum of the partials / width + eps), summed in a fixed order.
            // The 128 threads share the (token, partial) pairs: thread t takes token t % W (W: the power of
            // two that holds the tokens, so that neighbours read neighbours) and every (128 / W)-th partial,
            // and requests eight values before it adds the first.  A loop that adds as it loads, or a
            // shuffle between the loads, costs one trip to the L2 cache per value: 11 us for 64 tokens.
            // Threads of a warp that hold the same token meet by shuffles, the warps in shared memory (the
            // exchange area of the gated epilogue, which is used only after this).
            float* warp_sums = xch;                                                 // [4][32]
            const int n_tok = min(a.rows_q, BN);
            int W = 1;
            while (W < n_tok) W <<= 1;
            const int j = r & (W - 1), p0 = r / W, p_step = 128 / W;
            float sum = 0.0f;
            for (int part = p0; part < a.scale_parts; part += 8 * p_step) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int p = part + u * p_step;
                    v[u] = (p < a.scale_parts && j < n_tok) ? __ldcg(a.scale_sumsq + (size_t)p * a.scale_ld + j) : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) sum += v[u];
            }
            for (int o = 16; o >= W; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            warp_sums[lg * 32 + lane] = sum;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (r < n_tok) {
                float total = 0.0f;
#pragma unroll
                for (int w = 0; w < 4; ++w)
                    if (((w * 32 + (r & 31)) & (W - 1)) == r) total += warp_sums[w * 32 + (r & 31)];
                rstd_s[r] = rsqrtf(total * a.scale_inv_width + a.scale_eps);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        // Stores eight or sixteen finished columns c .. c + NE of row r (element (i, q0 + c + e)).
        constexpr int PRE = BN <= 32 ? BN : 1;
        auto emit = [&](const auto& v, int c, int i, int q0, int tile_p, const float* pre, float g) {
            constexpr int NE = (int)(sizeof(v) / sizeof(float));
            if (a.gated) {                          // swapped: rows 0-63 gate, 64-127 up of features 64 tile_p + ..
                const int feature = tile_p * 64 + (r & 63);
#pragma unroll
                for (int g8 = 0; g8 < NE; g8 += 8) {
                    if (q0 + c + g8 >= a.rows_q) break;             // the same for all 128 threads
                    if (r >= 64) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) xch[(r - 64) * 8 + e] = v[g8 + e];
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (r < 64 && feature < a.gated) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const int j = q0 + c + g8 + e;
                            if (j >= a.rows_q) break;
                            const float f = a.scale_sumsq ? rstd_s[j] : 1.0f;
                            const float z = v[g8 + e] * f, u = xch[r * 8 + e] * f;
                            reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)j * a.ldc + feature] =
                                __float2bfloat16_rn(z / (1.0f + expf(-z)) * u);
                        }
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");   // the halves are read before the next group overwrites them
                }
                return;
            }
            const bool row_ok = i < a.rows_p;
            if (a.residual) {                       // swapped, one tile of tokens: j = c + e is the token
                float x[NE];
#pragma unroll
                for (int e = 0; e < NE; ++e) {      // all loads first: the stores below would order them
                    const int j = q0 + c + e;
                    if (PRE > 1) x[e] = pre[c + e];
                    else x[e] = (row_ok && j < a.rows_q) ? __ldcg(a.residual + (size_t)j * a.ldr + i) : 0.0f;
                }
#pragma unroll
                for (int e = 0; e < NE; ++e) {
                    const int j = q0 + c + e;
                    if (j >= a.rows_q) break;       // the same for the whole warp
                    if (row_ok) {
                        x[e] += a.scale_sumsq ? v[e] * rstd_s[j] : v[e];
                        a.residual[(size_t)j * a.ldr + i] = x[e];
                        reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)j * a.ldc + i] = __float2bfloat16_rn(x[e] * g);
                    }
                    float sq = x[e] * x[e];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                    if (lane == 0) a.sumsq_out[(size_t)(tile_p * 4 + lg) * a.sumsq_ld + j] = sq;
                }
                return;
            }
            if (!row_ok) return;
#pragma unroll
            for (int e = 0; e < NE; ++e) {
                const int j = q0 + c + e;
                if (j >= a.rows_q) break;
                const size_t idx = a.swapped ? (size_t)j * a.ldc + i : (size_t)i * a.ldc + j;
                const float x = a.scale_sumsq ? v[e] * rstd_s[j] : v[e];
                if (a.out_f32) reinterpret_cast<float*>(a.out)[idx] = x;
                else reinterpret_cast<__nv_bfloat16*>(a.out)[idx] = __float2bfloat16_rn(x);
            }
        };
        [[maybe_unused]] int pending[2];       // wide tiles: this CTA's partial tiles, merged after the loop
        [[maybe_unused]] int n_pending = 0;
        while (seg.next(tile, s0, s1)) {
            const int buf = n & 1;
            const int tile_p = tile % a.tiles_p;
            const int p0 = tile_p * BM, q0 = (tile / a.tiles_p) * BN;
            const int i = p0 + r;
            // narrow tiles: the residual values this tile may be added to are fetched while the MMAs run
            [[maybe_unused]] float res_pre[PRE];
            const float gain_pre = (a.residual && i < a.rows_p) ? __ldg(a.gain + i) : 0.0f;
            if constexpr (PRE > 1) {
                if (a.residual) {
#pragma unroll
                    for (int e = 0; e < PRE; ++e)
                        res_pre[e] = (i < a.rows_p && q0 + e < a.rows_q) ? __ldcg(a.residual + (size_t)(q0 + e) * a.ldr + i) : 0.0f;
                }
            }
            if (flags[0] || !mbar_wait(acc_full0 + 8 * buf, (n >> 1) & 1)) {
                if (!flags[0]) { flags[0] = 1; atomicCAS(a.status, 0, 3); }
                break;
            }
            tc_fence_after();
            const bool whole = (s0 == 0 && s1 == S);
            // a CTA's run starts inside at most one tile and ends inside at most one: two scratch slots
            float* part = whole ? nullptr
                                : a.partial + ((size_t)cta * 2 + (cta * U >= tile * S ? 0 : 1)) * BN * BM;
            bool stored = false;
            if constexpr (BN >= 32) {
                // A whole gated tile of 32 or more columns: 32 columns a round, both halves of the CTA at work.
                // The gate rows' threads finish the round's first 16 columns, the up rows' threads the other
                // 16; each half hands the other the values it needs through shared memory, column-major so
                // that a warp's accesses fall into different banks.  (Eight columns a round with the up half
                // only writing, as emit does it, costs about 1 us per eight columns.)
                if (a.gated && !part) {
                    float* from_gate = xch;             // [16][64]: gate values of the round's last 16 columns
                    float* from_up = xch + 16 * 64;     // [16][64]: up values of its first 16
                    const int half_row = r & 63, feature = tile_p * 64 + half_row;
                    const bool is_gate = r < 64;
#pragma unroll 1
                    for (int c0 = 0; c0 < BN && q0 + c0 < a.rows_q; c0 += 32) {
                        uint32_t lo[16], hi[16];
                        tc_ld16(tmem_d + ((uint32_t)(lg * 32) << 16) + buf * BN + c0, lo);
                        tc_ld16(tmem_d + ((uint32_t)(lg * 32) << 16) + buf * BN + c0 + 16, hi);
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            if (is_gate) from_gate[e * 64 + half_row] = __uint_as_float(hi[e]);
                            else from_up[e * 64 + half_row] = __uint_as_float(lo[e]);
                        }
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (feature < a.gated) {
                            const int cb = q0 + c0 + (is_gate ? 0 : 16);
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                const int j = cb + e;
                                if (j >= a.rows_q) break;
                                const float f = a.scale_sumsq ? rstd_s[j] : 1.0f;
                                const float z = (is_gate ? __uint_as_float(lo[e]) : from_gate[e * 64 + half_row]) * f;
                                const float u = (is_gate ? from_up[e * 64 + half_row] : __uint_as_float(hi[e])) * f;
                                reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)j * a.ldc + feature] =
                                    __float2bfloat16_rn(z / (1.0f + expf(-z)) * u);
                            }
                        }
                        asm volatile("bar.sync 1, 128;" ::: "memory");   // read before the next round overwrites
                    }
                    stored = true;
                }
            }
#pragma unroll 1
            for (int c = 0; c < BN && !stored; c += 16) {
                uint32_t v[16];
                tc_ld16(tmem_d + ((uint32_t)(lg * 32) << 16) + buf * BN + c, v);
                if (part) {
#pragma unroll
                    for (int e = 0; e < 16; ++e) part[(c + e) * BM + r] = __uint_as_float(v[e]);
                } else {
                    float f[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) f[e] = __uint_as_float(v[e]);
                    emit(f, c, i, q0, tile_p, res_pre, gain_pre);
                }
            }
            // the accumulator has been read: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
            ++n;
            if (!part) continue;
            if constexpr (BN >= 32) {
                // wide tiles: count this segment in; the tile's CTAs share its merge at the end of their runs
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) atomicAdd(&a.tickets[tile], 1);
                pending[n_pending++] = tile;
                continue;
            }
            // partial tile: take a ticket; the last of the tile's segments to arrive adds them up
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) flags[1] = atomicAdd(&a.tickets[tile], 1);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int first_cta = (tile * S) / U;
            const int nseg = ((tile + 1) * S - 1) / U - first_cta + 1;
            const bool last = flags[1] == nseg - 1;
            asm volatile("bar.sync 1, 128;" ::: "memory");       // flags[1] is read before the next segment writes it
            if (!last) continue;
            __threadfence();
#pragma unroll 1
            for (int c = 0; c < BN; c += 8) {
                if (q0 + c >= a.rows_q) break;
                float acc[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
                // eight segments' values are requested before the first is added (in order: the sum does
                // not depend on which CTA finished when); a loop that adds as it loads would pay one trip
                // to the L2 cache per segment
                for (int sg0 = 0; sg0 < nseg; sg0 += 8) {
                    float v[8][8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const int x = first_cta + sg0 + k;
                        const float* src = a.partial + ((size_t)x * 2 + (x * U >= tile * S ? 0 : 1)) * BN * BM + r;
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[k][e] = sg0 + k < nseg ? __ldcg(src + (c + e) * BM) : 0.0f;
                    }
#pragma unroll
                    for (int k = 0; k < 8; ++k)
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[e] += v[k][e];
                }
                emit(acc, c, i, q0, tile_p, res_pre, gain_pre);
            }
            if (threadIdx.x == 64) a.tickets[tile] = 0;       // ready for the next launch
        }
        // Wide tiles (32 columns and more): adding a tile's partials up is too much for one CTA at the
        // end of the kernel, so every CTA that computed a segment of the tile merges a share of its
        // columns.  That needs all segments to be there: the CTAs wait for the tile's count, here, after
        // all their own segments are written (every CTA of the grid is resident by then: dependent
        // kernels start only after all of them have, and nobody waits before this point).  Bounded.
        if constexpr (BN >= 32) {
            for (int k = 0; k < n_pending; ++k) {
                const int tl = pending[k];
                const int first_cta = (tl * S) / U;
                const int nseg = ((tl + 1) * S - 1) / U - first_cta + 1;
                if (threadIdx.x == 64 && !flags[0] && !wait_count(a.tickets + tl, nseg)) {
                    flags[0] = 1;
                    atomicCAS(a.status, 0, 8);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (!flags[0]) {
                    __threadfence();
                    const int tile_p = tl % a.tiles_p;
                    const int q0 = (tl / a.tiles_p) * BN, i = tile_p * BM + r;
                    const int valid = min(BN, a.rows_q - q0);
                    const int share = (((valid + nseg - 1) / nseg) + 7) & ~7;          // whole groups of eight columns
                    const int c_begin = (cta - first_cta) * share, c_end = min(valid, c_begin + share);
                    [[maybe_unused]] float res_pre[PRE];
                    const float gain_pre = (a.residual && i < a.rows_p) ? __ldg(a.gain + i) : 0.0f;
                    if constexpr (PRE > 1) {
                        if (a.residual) {
#pragma unroll
                            for (int e = 0; e < PRE; ++e)
                                res_pre[e] = (i < a.rows_p && q0 + e < a.rows_q) ? __ldcg(a.residual + (size_t)(q0 + e) * a.ldr + i) : 0.0f;
                        }
                    }
#pragma unroll 1
                    for (int c = c_begin; c < c_end; c += 8) {
                        float acc[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
                        for (int sg0 = 0; sg0 < nseg; sg0 += 8) {
                            float v[8][8];
#pragma unroll
                            for (int kk = 0; kk < 8; ++kk) {
                                const int x = first_cta + sg0 + kk;
                                const float* src = a.partial + ((size_t)x * 2 + (x * U >= tl * S ? 0 : 1)) * BN * BM + r;
#pragma unroll
                                for (int e = 0; e < 8; ++e) v[kk][e] = sg0 + kk < nseg ? __ldcg(src + (c + e) * BM) : 0.0f;
                            }
#pragma unroll
                            for (int kk = 0; kk < 8; ++kk)
#pragma unroll
                                for (int e = 0; e < 8; ++e) acc[e] += v[kk][e];
                        }
                        emit(acc, c, i, q0, tile_p, res_pre, gain_pre);
                    }
                }
                // the last of the tile's CTAs to be done with it clears the count for the next launch
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64 && atomicAdd(&a.tickets[tl], 1) == 2 * nseg - 1) a.tickets[tl] = 0;
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
int launch(const CUtensorMap& mp, const CUtensorMap& mq, const GemmArgs& a, int ctas, cudaStream_t s) {
    // stages, 1 KB to align them, barriers with the epilogue's factor and exchange areas (2 KB, 8 KB for wide tiles)
    constexpr size_t smem = (size_t)STAGES * (P_BYTES + BN * BK * 2) + 1024 + (BN >= 32 ? 9216 : 3072);
    static unsigned long long configured = 0;
    if (int e = vcb_allow_dynamic_smem(gemm_tcgen05_kernel<BN, STAGES>, (int)smem, &configured)) return e;
    vcb_launch(gemm_tcgen05_kernel<BN, STAGES>, ctas, GEMM_THREADS, smem, s, mp, mq, a);
    return vcb_last_error();
}

}  // namespace

// One thread per 16-byte chunk of the tiled image: tile (tp, slab), row r, chunk c of the
// row-major matrix goes to chunk c ^ (r % 8) of row r of the tile, which is the 128-byte
// swizzle of the TMA copy.  Rows beyond the matrix and columns beyond K are zero.
__global__ void tile_weights_kernel(const __nv_bfloat16* __restrict__ w, int rows, int k, int ld, int k_slabs,
                                    uint4* __restrict__ out, size_t n_chunks, int gated) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n_chunks; idx += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(idx & 7), r = (int)((idx >> 3) & 127);
        const size_t tile = idx >> 10;
        const int slab = (int)(tile % k_slabs);
        const size_t tp = tile / k_slabs;
        // gated: tile tp = gate rows 64 tp .. 64 tp + 63, then the up rows (gated + the same) of a [2 gated, k] matrix
        const size_t row = gated ? (size_t)(r < 64 ? 0 : gated) + tp * 64 + (r & 63) : tp * BM + r;
        const bool row_ok = gated ? tp * 64 + (r & 63) < (size_t)gated : row < (size_t)rows;
        const int col = slab * BK + c * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row_ok) {
            if (col + 8 <= k && (ld % 8) == 0) {
                v = *reinterpret_cast<const uint4*>(w + row * ld + col);
            } else {
                __nv_bfloat16 tmp[8];
                for (int e = 0; e < 8; ++e) tmp[e] = col + e < k ? w[row * ld + col + e] : __float2bfloat16_rn(0.0f);
                v = *reinterpret_cast<uint4*>(tmp);
            }
        }
        out[(tile << 10) + ((size_t)r << 3) + (c ^ (r & 7))] = v;
    }
}

// Bytes of the tiled image of a [rows, k] matrix (gated > 0: of a [2 gated, k] gate-and-up matrix).
VCB_EXPORT long long vcb_tiled_weight_bytes(int rows, int k, int gated) {
    const int tiles = gated > 0 ? (gated + 63) / 64 : (rows + BM - 1) / BM;
    return (long long)tiles * ((k + BK - 1) / BK) * P_BYTES;
}

// out (vcb_tiled_weight_bytes bytes, 16-byte aligned) = the tiled image of w.  gated > 0: w is
// [2 gated, k], gate rows first; tile t of the image holds gate rows 64 t .. and the matching up rows.
VCB_EXPORT int vcb_tile_weights(const void* w, int rows, int k, int ld, int gated, void* out, void* stream) {
    if (rows <= 0 || k <= 0 || ld < k || ((uintptr_t)out & 15) || ((uintptr_t)w & 15)) return VCB_ERR_BAD_ARG;
    if (gated < 0 || (gated > 0 && rows != 2 * gated)) return VCB_ERR_BAD_ARG;
    const int k_slabs = (k + BK - 1) / BK;
    const int tiles = gated > 0 ? (gated + 63) / 64 : (rows + BM - 1) / BM;
    const size_t n_chunks = (size_t)tiles * k_slabs * 1024;
    size_t blocks = (n_chunks + 255) / 256;
    if (blocks > vcb_sm_count() * 32) blocks = vcb_sm_count() * 32;
    tile_weights_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)w, rows, k, ld, k_slabs,
                                                                       (uint4*)out, n_chunks, gated);
    return vcb_last_error();
}

// out[r, c] (row stride ldc, bfloat16 or float) = sum_k ...
//   swapped = 0: P = activations [rows_p = tokens], Q = weights [rows_q = features]: out[p, q]
//   swapped = 1: P = weights [rows_p = features], Q = activations [rows_q = tokens]:  out[q, p]
// bn: columns of the tensor-core tile (16, 32, 64, 128 or 256: with 128 rows the tensor core takes multiples of 16; rows_q is cut into tiles of bn).
// max_ctas: persistent CTAs (one per SM).  Scratch: partial holds max_ctas * 2 * bn * 128 floats,
// tickets one zeroed int per tile (the kernel leaves them zero).
// p_tiled: P as made by vcb_tile_weights (then p and ldp are not used), or null.
//
// Fused norm (both optional, swapped products with rows_q <= bn only):
//   scale_sumsq [scale_parts][scale_ld]: row j of the result is multiplied by
//       rsqrt(sum_part scale_sumsq[part][j] / scale_width + scale_eps);
//   residual [rows_q][ldr] float, gain [rows_p] float, sumsq_out [4 * ceil(rows_p / 128)][sumsq_ld]:
//       residual += result; out (bfloat16) = residual * gain; sumsq_out = partial sums over the features
//       of residual^2 for every token.
//   gated > 0: p_tiled is a gated image (vcb_tile_weights) of a [2 gated, k] matrix, rows_p = 2 gated;
//       out (bfloat16, [rows_q][>= gated]) = silu(gate) * up.
VCB_EXPORT int vcb_gemm_bf16_tcgen05_fused(const void* p, int rows_p, int ldp, const void* p_tiled, const void* q,
                                           int rows_q, int ldq, int k, void* out, int ldc, int out_f32, int swapped,
                                           int bn, int max_ctas, float* partial, int* tickets, int n_tickets,
                                           int* status, const float* scale_sumsq, int scale_parts, int scale_ld,
                                           int scale_width, float scale_eps, float* residual, int ldr,
                                           const float* gain, float* sumsq_out, int sumsq_ld, int gated, void* stream) {
    if (rows_p <= 0 || rows_q <= 0) return 0;
    if (k <= 0 || max_ctas < 1 || !status || !partial || !tickets) return VCB_ERR_BAD_ARG;
    // TMA needs 16-byte aligned bases and row strides
    if ((k % 8) || (ldq % 8) || (((uintptr_t)q | (uintptr_t)p_tiled) & 15)) return VCB_ERR_UNSUPPORTED;
    if (!p_tiled && ((ldp % 8) || ((uintptr_t)p & 15))) return VCB_ERR_UNSUPPORTED;
    if (bn != 16 && bn != 32 && bn != 64 && bn != 128 && bn != 256) return VCB_ERR_BAD_ARG;
    if (gated) {
        if (gated < 0 || rows_p != 2 * gated || !p_tiled || !swapped || rows_q > bn || bn > 128 || out_f32 || residual ||
            ldc < gated)
            return VCB_ERR_BAD_ARG;
        rows_p = 128 * ((gated + 63) / 64);       // rows of the image
    }
    if (scale_sumsq || residual) {
        if (!swapped || rows_q > bn || bn > 128) return VCB_ERR_UNSUPPORTED;
        if (scale_sumsq && (scale_parts < 1 || scale_ld < rows_q || scale_width < 1)) return VCB_ERR_BAD_ARG;
        if (residual && (!gain || !sumsq_out || out_f32 || ldr < rows_p || sumsq_ld < rows_q)) return VCB_ERR_BAD_ARG;
    }
    const int k_slabs = (k + BK - 1) / BK;
    const int tiles_p = (rows_p + BM - 1) / BM, tiles_q = (rows_q + bn - 1) / bn;
    const long long total = (long long)tiles_p * tiles_q * k_slabs;
    if (tiles_p * tiles_q > n_tickets || total > (1ll << 30)) return VCB_ERR_UNSUPPORTED;
    // equal runs of (tile, slab) units, at least four slabs each
    int ctas = (int)(total / 4 < 1 ? 1 : (total / 4 < max_ctas ? total / 4 : max_ctas));
    const int per = (int)((total + ctas - 1) / ctas);
    ctas = (int)((total + per - 1) / per);
    CUtensorMap mp, mq;
    int c = make_map(&mq, q, rows_q, k, ldq, bn);
    if (c) return c;
    if (p_tiled) mp = mq;                       // not used by the kernel
    else if ((c = make_map(&mp, p, rows_p, k, ldp, BM))) return c;
    GemmArgs a{out, partial, tickets, status, (const uint8_t*)p_tiled, ldc, out_f32, swapped, rows_p, rows_q,
               k_slabs, tiles_p, per, (int)total,
               scale_sumsq, scale_parts, scale_ld, scale_sumsq ? 1.0f / (float)scale_width : 0.0f, scale_eps,
               residual, gain, sumsq_out, ldr, sumsq_ld, gated};
    cudaStream_t s = (cudaStream_t)stream;
    switch (bn) {
        case 16: return launch<16, 6>(mp, mq, a, ctas, s);
        case 32: return launch<32, 5>(mp, mq, a, ctas, s);
        case 64: return max_ctas > vcb_sm_count() ? launch<64, 4>(mp, mq, a, ctas, s) : launch<64, 8>(mp, mq, a, ctas, s);
        case 128: return launch<128, 6>(mp, mq, a, ctas, s);
        default: return launch<256, 4>(mp, mq, a, ctas, s);
    }
}

VCB_EXPORT int vcb_gemm_bf16_tcgen05(const void* p, int rows_p, int ldp, const void* p_tiled, const void* q, int rows_q,
                                     int ldq, int k, void* out, int ldc, int out_f32, int swapped, int bn,
                                     int max_ctas, float* partial, int* tickets, int n_tickets, int* status,
                                     void* stream) {
    return vcb_gemm_bf16_tcgen05_fused(p, rows_p, ldp, p_tiled, q, rows_q, ldq, k, out, ldc, out_f32, swapped, bn,
                                       max_ctas, partial, tickets, n_tickets, status, nullptr, 0, 0, 1, 0.0f,
                                       nullptr, 0, nullptr, nullptr, 0, 0, stream);
}
