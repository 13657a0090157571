// Paged grouped-query attention on tensor cores for bfloat16, head sizes 64 and 128.
//
// Two kernels share the tile loader:
//   * attention_decode_kernel (mma.sync): one query token per request.  The query heads that share one kv
//     head are packed into the row dimension (row = head in group, G = heads / kv_heads), so one K/V
//     tile in shared memory serves all G heads; the G rows fill one 16-row fragment.  The context is
//     split over CTAs, and inside a CTA each warp takes 16 of every 64 keys.  Partial (max, sum, output)
//     triples are merged across warps in shared memory and across CTAs through scratch memory in global
//     memory: every CTA of a (request, kv head) takes a ticket when its partials are written, and the
//     one that draws the last ticket merges them.
//   * tc::attention_prefill_tc_kernel (tcgen05, further down, with its own description): portions of
//     prompts of any length and, in mixed batches, single tokens; row = token * G + head in group.
// Scores, softmax statistics and output accumulators are float; the probabilities
// are rounded to bfloat16 for the P*V product, as K and V are stored.  Exponentials
// are ex2.approx on scores pre-multiplied by log2(e) (this file is the bfloat16 path;
// the plain kernel of attention_simt.cu uses expf).
//
// Loading.  The cache stores every row already in the XOR-swizzled chunk order that
// ldmatrix wants (kv_pos in common.cuh), so a run of slots of a page is a ready-made
// piece of a shared-memory tile.  In the decode kernel a fifth warp is the producer: for every tile of
// 64 keys it issues one bulk copy (cp.async.bulk, the TMA unit, no tensor map, no multicast) per
// page piece of K and of V into a ring of stages, completing on the stage's mbarrier; the
// four consumer warps wait on that barrier and hand the stage back on another.  No thread
// that computes ever waits on a global load.  Pages wholly outside [lo, hi) may have been
// given back (window) or not exist yet: a page that does exist is copied in their place
// (their scores are masked, their finite values multiply a probability of zero).  Waits on
// mbarriers are bounded; one that runs out is recorded in *status.
//
// Replaces paged_attention_kernel (src/attention/paged_attention.cu:7-93) for the
// bfloat16 path; attention_simt.cu is its plain counterpart.
#include "common.cuh"

#define BN 64            // keys per tile
#define NTHREADS 128     // consumer threads (4 warps); warp 4 is the producer
#define BLOCK_THREADS 160

struct MmaAttnArgs {
    const __nv_bfloat16* q;        // [n_tokens, nh * d]
    const __nv_bfloat16* cache;    // [pages][2][nkv][page][d]
    __nv_bfloat16* out;            // [n_tokens, nh * d]
    const int* q_start;            // [n_reqs + 1]
    const int* ctx_lens;           // [n_reqs]
    const int* block_table;        // [n_reqs, bt_stride]
    const int* req_list;           // decode: requests to process (null: 0..n-1); prefill: tile -> request
    const int* tile_row0;          // prefill: tile -> first packed row
    float* part_o;                 // decode scratch: [n_list, nh, splits, d]
    float* part_ml;                // decode scratch: [n_list, nh, splits, 2]  (max in log2 units, sum)
    int* counters;                 // decode scratch: [n_list, nkv] tickets, zero between launches
    int* status;                   // nonzero after a bounded wait ran out (may be null)
    const int* split_tiles;        // decode: key tiles per split, on the device (null: every request in gridDim.x equal parts)
    int bt_stride, nh, nkv, page, window;
    float scale;
    int num_pages;                 // pages of the cache: a table entry outside [0, num_pages) is read as page 0
                                   // and VCB_STATUS_BAD_PAGE goes to the status word
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
#define LOG2E 1.4426950408889634f

// Byte offset of element (row, 16-byte chunk) in a tile of rows of D bfloat16 (the Q tile, which the
// kernels write themselves).
template <int D> __device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}
// The same for a K or V tile of TK keys, which arrives from the cache in planes of 128-byte row
// pieces (kv_pos in common.cuh): [plane][key][128 bytes], chunks swizzled inside a piece.
template <int D, int TK> __device__ __forceinline__ uint32_t swz_kv(int key, int chunk) {
    return (uint32_t)(((chunk >> 3) * TK + key) * 128 + (((chunk & 7) ^ (key & 7)) << 4));
}

// The request's block table as the producer warp sees it: a window of 64 consecutive entries in
// two registers per lane, refilled 32 entries at a time, so that no tile waits for a load of its
// page numbers (a dependent global load per tile is what would otherwise bound a CTA's rate).
// Entries for pages wholly outside [lo, hi) may have been given back (window) or not exist yet:
// the page of the last visible key, which always exists, is used in their place.
struct PageWindow {
    const int* bt;
    int base, n_pages, last_pg, cur, nxt, lane;
    int n_phys;                  // pages of the cache
    bool bad;                    // a page number outside [0, n_phys) was met (and replaced by page 0)
    __device__ __forceinline__ int fetch(int i) const { return i < n_pages ? __ldg(bt + i) : last_pg; }
    __device__ __forceinline__ int checked(int pg) {
        if ((unsigned)pg >= (unsigned)n_phys) { bad = true; return 0; }
        return pg;
    }
    __device__ __forceinline__ void init(const int* bt_, int first_page, int hi, int page, int lane_, int n_phys_) {
        bt = bt_; lane = lane_; n_phys = n_phys_; bad = false;
        n_pages = (hi - 1) / page + 1;
        last_pg = __ldg(bt + (hi - 1) / page);
        base = first_page;
        cur = fetch(base + lane);
        nxt = fetch(base + 32 + lane);
    }
    // entry of logical page lp >= base; the same call sequence in all 32 lanes
    __device__ __forceinline__ int get(int lp) {
        while (__any_sync(0xffffffffu, lp >= base + 64)) {   // not reached by tiles of at most 32 pages' span in order
            cur = nxt; base += 32; nxt = fetch(base + 32 + lane);
        }
        const int i = lp - base;
        const int a = __shfl_sync(0xffffffffu, cur, i & 31), b = __shfl_sync(0xffffffffu, nxt, i & 31);
        return i < 32 ? a : b;
    }
    // move on once every page below lp is done with
    __device__ __forceinline__ void advance(int lp) {
        if (lp >= base + 32) { cur = nxt; base += 32; nxt = fetch(base + 32 + lane); }
    }
};

// Division by the page size on the producer's path: a shift when the size is a power of two (the
// producer warp issues every copy of its CTA, so its instruction count bounds the CTA's rate).
struct PageDiv {
    int page, shift;             // shift < 0: not a power of two
    __device__ __forceinline__ explicit PageDiv(int page_) : page(page_), shift(-1) {
        if ((page_ & (page_ - 1)) == 0) { shift = 0; while ((1 << shift) < page_) ++shift; }
    }
    __device__ __forceinline__ int div(int x) const { return shift >= 0 ? x >> shift : x / page; }
    __device__ __forceinline__ int mul(int x) const { return shift >= 0 ? x << shift : x * page; }
};

// The producer warp's share of one tile of TK keys starting at key kb of kv head g.  A tile spans at
// most TK / 16 + 1 pages and D / 64 planes; lane = 16 * (K or V) + 8 * plane + page piece copies one run
// of 128-byte row pieces.  Lane 0 has armed the stage's barrier with the tile's byte count.
// head_base: the kv head's block inside a page's K half; page_stride, v_off: elements per page, K half to V half.
struct TilePiece {
    const __nv_bfloat16* src;    // K piece; the V piece lies v_off further
    uint32_t off, bytes;         // where in the tile, how much
    bool active;
};
// Where this lane's piece of the tile comes from: all the address arithmetic of a tile's copies, none of
// which depends on the stage being free, so a producer can do it for the next tile while it waits.
template <int D, int TK>
__device__ __forceinline__ TilePiece tile_piece(int kb, int lo, int hi, PageWindow& pw, const __nv_bfloat16* __restrict__ cache,
                                                size_t head_base, size_t page_stride, const PageDiv& pd, int lane) {
    constexpr int PLANES = D / 64;
    static_assert(PLANES == 1 || PLANES == 2, "head sizes 64 and 128");
    const int piece = lane & 7, plane = (lane >> 3) & 1;
    const int first_page = pd.div(kb);
    pw.advance(first_page);
    const int lp_piece = first_page + piece;
    const int start = piece == 0 ? kb : pd.mul(lp_piece);                   // first key of the piece
    TilePiece t;
    t.active = plane < PLANES && start < kb + TK;
    // the page itself if any of it is visible, else the page of the last visible key
    const int lp = t.active ? lp_piece : first_page;
    const int page_lo = pd.mul(lp);
    const bool visible = page_lo < hi && page_lo + pd.page > lo;
    const int got = pw.get(visible ? lp : first_page);                     // all lanes take part in the shuffles
    const int pg = pw.checked(visible ? got : pw.last_pg);
    const int end = min(page_lo + pd.page, kb + TK);
    // plane `plane` of the head's block: pd.page rows of 64 elements
    t.src = cache + (size_t)pg * page_stride + head_base + ((size_t)plane * pd.page + (start - page_lo)) * 64;
    t.off = (uint32_t)(plane * TK + (start - kb)) * 128;
    t.bytes = (uint32_t)(end - start) * 128;
    return t;
}
// which: 0 K and V, 1 K only, 2 V only (a kernel that fetches them at different times)
__device__ __forceinline__ void issue_piece(const TilePiece& t, uint32_t sk, uint32_t sv, uint32_t bar, size_t v_off, int lane,
                                            uint32_t bar_v = 0, int which = 0) {
    if (!t.active) return;
    if (lane < 16) { if (which != 2) cx_bulk_load(sk + t.off, t.src, t.bytes, bar); }
    else if (which != 1) cx_bulk_load(sv + t.off, t.src + v_off, t.bytes, bar_v ? bar_v : bar);
}
template <int D, int TK>
__device__ __forceinline__ void produce_tile(uint32_t sk, uint32_t sv, uint32_t bar, int kb, int lo, int hi,
                                             PageWindow& pw, const __nv_bfloat16* __restrict__ cache,
                                             size_t head_base, size_t page_stride, size_t v_off, const PageDiv& pd, int lane,
                                             uint32_t bar_v = 0, int which = 0) {
    issue_piece(tile_piece<D, TK>(kb, lo, hi, pw, cache, head_base, page_stride, pd, lane), sk, sv, bar, v_off, lane, bar_v, which);
}

// S[16 x 8*NB] += Q[16 x D] * K[keys key0 .. key0 + 8*NB)^T, K tile at sk.
template <int D, int TK, int NB>
__device__ __forceinline__ void qk_product(float (&s)[NB][4], const uint32_t (&qf)[D / 16][4], uint32_t sk, int key0) {
    const int lane = threadIdx.x & 31;
    const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int nb = 0; nb < NB; nb += 2) {
            uint32_t b[4];
            const int key = key0 + (nb + (mi >> 1)) * 8 + r8;
            ldmatrix_x4(b, sk + swz_kv<D, TK>(key, ks * 2 + (mi & 1)));
            mma_bf16(s[nb], qf[ks], b[0], b[1]);
            mma_bf16(s[nb + 1], qf[ks], b[2], b[3]);
        }
    }
}

// O[16 x D] += P[16 x 16*KK] * V[keys key0 .. key0 + 16*KK), V tile at sv.  pf[kk] is P's A fragment.
template <int D, int TK, int KK>
__device__ __forceinline__ void pv_product(float (&o)[D / 8][4], const uint32_t (&pf)[KK][4], uint32_t sv, int key0) {
    const int lane = threadIdx.x & 31;
    const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) {
#pragma unroll
        for (int nd = 0; nd < D / 8; nd += 2) {
            uint32_t b[4];
            const int key = key0 + kk * 16 + (mi & 1) * 8 + r8;
            ldmatrix_x4_trans(b, sv + swz_kv<D, TK>(key, nd + (mi >> 1)));
            mma_bf16(o[nd], pf[kk], b[0], b[1]);
            mma_bf16(o[nd + 1], pf[kk], b[2], b[3]);
        }
    }
}

// Q rows -> A fragments.  The tile at sq holds 16 rows per warp slot `wrow0`.
template <int D>
__device__ __forceinline__ void load_q_frags(uint32_t (&qf)[D / 16][4], uint32_t sq, int wrow0) {
    const int lane = threadIdx.x & 31;
    const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
        ldmatrix_x4(qf[ks], sq + swz<D>(wrow0 + (mi & 1) * 8 + r8, ks * 2 + (mi >> 1)));
}

// ------------------------------------------------------------------ decode
template <int D, int STAGES>
__global__ void __launch_bounds__(BLOCK_THREADS, 2)
attention_decode_kernel(MmaAttnArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    constexpr int TILE_BYTES = BN * D * 2;
    // The step's index arrays were copied in before its first kernel, and every cache row below the
    // request's newest position was written by an earlier step: both are read before
    // griddepcontrol.wait, while the kernel that rotates and stores this step's row still runs.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool producer = warp == 4;
    bool waited = false;                                 // producer: griddepcontrol.wait has been executed
    const int split = blockIdx.x, g = blockIdx.y, li = blockIdx.z;
    const int r = a.req_list ? a.req_list[li] : li;
    const int G = a.nh / a.nkv;
    const int t = a.q_start[r];
    const int pos = a.ctx_lens[r];                       // the single token's position
    const int hi = pos + 1;
    const int lo = a.window > 0 ? max(0, hi - a.window) : 0;
    const int* bt = a.block_table + (size_t)r * a.bt_stride;
    const float sl2 = a.scale * LOG2E;                   // scores in units of log2

    // The splits of a request.  With split_tiles no split of any request has more than that many tiles
    // (a request's tiles are dealt evenly to the splits it needs), so a request with a long context gets
    // more CTAs than one with a short context and the CTAs of a step with mixed contexts end together;
    // the CTAs beyond a request's splits leave at once.
    // (A number that would need more splits than the grid has falls back to equal parts.)
    const int tile0 = lo / BN, tile1 = (hi + BN - 1) / BN;
    const int grid_splits = gridDim.x;
    int per = (tile1 - tile0 + grid_splits - 1) / grid_splits, nsplit = grid_splits;
    if (a.split_tiles) {
        const int want = max(1, __ldg(a.split_tiles));
        const int needs = (tile1 - tile0 + want - 1) / want;
        if (needs <= grid_splits) { nsplit = max(1, needs); per = (tile1 - tile0 + nsplit - 1) / nsplit; }
    }
    if (split >= nsplit) return;
    const int my0 = tile0 + split * per, my1 = min(tile1, my0 + per);

    // [STAGES x (K, V) tiles][Q: 16 x D][barriers]; the merge buffers reuse the tiles
    const uint32_t s_tiles = smem_u32(smem);
    unsigned char* q_ptr = smem + (size_t)STAGES * 2 * TILE_BYTES;
    const uint32_t sq = smem_u32(q_ptr);
    uint64_t* bars = reinterpret_cast<uint64_t*>(q_ptr + 16 * D * 2);
    const uint32_t full0 = cx_smem(bars), empty0 = cx_smem(bars + STAGES);
    float* red_o = reinterpret_cast<float*>(smem);                          // [4][16][D]
    float* red_ml = reinterpret_cast<float*>(smem + 4 * 16 * D * 4);        // [4][16][2]
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { cx_mbar_init(full0 + 8 * s, 1); cx_mbar_init(empty0 + 8 * s, 4); }
        cx_mbar_init_fence();
    }
    int it = 0;                                          // tiles handled so far: stage and phase of the ring
    bool gave_up = false;

    for (int mt = 0; mt * 16 < G; ++mt) {
        __syncthreads();                                 // barriers initialised; the merge of the pass before has been read
        if (!producer) {
            // Q rows of this group: row i -> head g*G + mt*16 + i (written by the previous kernel)
            pdl_wait();
            for (int idx = threadIdx.x; idx < 16 * (D / 8); idx += NTHREADS) {
                const int row = idx / (D / 8), c = idx % (D / 8);
                const int hg = mt * 16 + row;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (hg < G) v = *reinterpret_cast<const uint4*>(a.q + ((size_t)t * a.nh + g * G + hg) * D + c * 8);
                *reinterpret_cast<uint4*>(q_ptr + swz<D>(row, c)) = v;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");   // the four consumer warps only
        }
        float o[D / 8][4];
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
        float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;   // rows lane/4 and lane/4 + 8

        if (producer) {
            PageWindow pw;
            const PageDiv pd(a.page);
            pw.init(bt, pd.div(my0 * BN), hi, a.page, lane, a.num_pages);
            const size_t page_stride = (size_t)2 * a.nkv * a.page * D, head_base = (size_t)g * a.page * D,
                         v_off = (size_t)a.nkv * a.page * D;
            for (int tile = my0; tile < my1; ++tile, ++it) {
                const int st = it % STAGES;
                if (!waited && (tile + 1) * BN > pos) { pdl_wait(); waited = true; }   // the tile with this step's row
                if (!cx_mbar_wait(empty0 + 8 * st, ((it / STAGES) & 1) ^ 1)) gave_up = true;
                if (lane == 0) cx_mbar_expect_tx(full0 + 8 * st, 2 * TILE_BYTES);
                __syncwarp();
                produce_tile<D, BN>(s_tiles + st * 2 * TILE_BYTES, s_tiles + st * 2 * TILE_BYTES + TILE_BYTES,
                                    full0 + 8 * st, tile * BN, lo, hi, pw, a.cache, head_base, page_stride, v_off, pd, lane);
            }
            if (pw.bad && a.status) atomicCAS(a.status, 0, VCB_STATUS_BAD_PAGE);
        } else {
            uint32_t qf[D / 16][4];
            load_q_frags<D>(qf, sq, 0);
            for (int tile = my0; tile < my1; ++tile, ++it) {
                const int st = it % STAGES;
                if (!cx_mbar_wait(full0 + 8 * st, (it / STAGES) & 1)) gave_up = true;
                const uint32_t sk = s_tiles + st * 2 * TILE_BYTES, sv = sk + TILE_BYTES;
                const int kb = tile * BN + warp * 16;    // this warp's 16 keys
                float s[2][4];
#pragma unroll
                for (int i = 0; i < 2; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; }
                qk_product<D, BN, 2>(s, qf, sk, warp * 16);
                // only a tile that crosses lo or hi has keys to mask (the same for the whole CTA)
                if (tile * BN < lo || tile * BN + BN > hi) {
#pragma unroll
                    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j = kb + nb * 8 + (lane & 3) * 2 + (e & 1);
                            if (j < lo || j >= hi) s[nb][e] = -INFINITY;
                        }
                }
                // raw scores from here on; 2^(s * sl2 - m * sl2) is one multiply-add and one ex2.
                // all rows of a decode tile share the position, but keep the two row sets apart
                float ta = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
                float tb = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
                ta = fmaxf(ta, __shfl_xor_sync(0xffffffffu, ta, 1)); ta = fmaxf(ta, __shfl_xor_sync(0xffffffffu, ta, 2));
                tb = fmaxf(tb, __shfl_xor_sync(0xffffffffu, tb, 1)); tb = fmaxf(tb, __shfl_xor_sync(0xffffffffu, tb, 2));
                const float na = fmaxf(m_a, ta), nb_ = fmaxf(m_b, tb);
                // the accumulators are rescaled only when some row's maximum rose (rare after the first tiles)
                if (__any_sync(0xffffffffu, na != m_a || nb_ != m_b)) {
                    const float ca = na == -INFINITY ? 1.0f : fast_exp2((m_a - na) * sl2);   // m = -inf: 2^-inf = 0, sums are 0 anyway
                    const float cb = nb_ == -INFINITY ? 1.0f : fast_exp2((m_b - nb_) * sl2);
                    m_a = na; m_b = nb_;
                    l_a *= ca; l_b *= cb;
#pragma unroll
                    for (int i = 0; i < D / 8; ++i) { o[i][0] *= ca; o[i][1] *= ca; o[i][2] *= cb; o[i][3] *= cb; }
                }
                const float sa = m_a == -INFINITY ? 0.0f : m_a * sl2, sb = m_b == -INFINITY ? 0.0f : m_b * sl2;
                uint32_t pf[1][4];
                float p[2][4];
#pragma unroll
                for (int nb = 0; nb < 2; ++nb) {
                    p[nb][0] = fast_exp2(fmaf(s[nb][0], sl2, -sa)); p[nb][1] = fast_exp2(fmaf(s[nb][1], sl2, -sa));
                    p[nb][2] = fast_exp2(fmaf(s[nb][2], sl2, -sb)); p[nb][3] = fast_exp2(fmaf(s[nb][3], sl2, -sb));
                }
                l_a += (p[0][0] + p[0][1] + p[1][0] + p[1][1]);
                l_b += (p[0][2] + p[0][3] + p[1][2] + p[1][3]);
                pf[0][0] = pack_bf16(p[0][0], p[0][1]); pf[0][1] = pack_bf16(p[0][2], p[0][3]);
                pf[0][2] = pack_bf16(p[1][0], p[1][1]); pf[0][3] = pack_bf16(p[1][2], p[1][3]);
                pv_product<D, BN, 1>(o, pf, sv, warp * 16);
                __syncwarp();
                if (lane == 0) cx_mbar_arrive(empty0 + 8 * st);      // this warp is done with the stage
            }
        }
        if (producer && !waited) { pdl_wait(); waited = true; }   // nothing is written before the previous kernel is done
        // Only now may the next kernel's CTAs come: if they came earlier they would take the place of
        // this kernel's own second CTA on the SM (they wait, holding shared memory), and the tiles
        // of this kernel would be read in two rounds.
        pdl_launch_dependents();
        __syncthreads();                                 // every copy has landed and been read: reuse the tiles
        const int Gm = min(16, G - mt * 16);             // rows of this pass that are heads
        if (!producer) {
            l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
            l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
            const int ra = lane >> 2, rb = ra + 8;
#pragma unroll
            for (int nd = 0; nd < D / 8; ++nd) {
                const int col = nd * 8 + (lane & 3) * 2;
                if (ra < Gm) *reinterpret_cast<float2*>(red_o + ((size_t)(warp * 16 + ra)) * D + col) = make_float2(o[nd][0], o[nd][1]);
                if (rb < Gm) *reinterpret_cast<float2*>(red_o + ((size_t)(warp * 16 + rb)) * D + col) = make_float2(o[nd][2], o[nd][3]);
            }
            if ((lane & 3) == 0) {
                // maxima leave the loop in units of log2
                red_ml[(warp * 16 + ra) * 2] = m_a * sl2; red_ml[(warp * 16 + ra) * 2 + 1] = l_a;
                red_ml[(warp * 16 + rb) * 2] = m_b * sl2; red_ml[(warp * 16 + rb) * 2 + 1] = l_b;
            }
        }
        __syncthreads();
        // the four warps' partials of a row: out = sum_w o_w 2^(m_w - m), four dimensions per thread
        for (int item = threadIdx.x; item < Gm * (D / 4); item += BLOCK_THREADS) {
            const int row = item / (D / 4), dim = (item % (D / 4)) * 4;
            float mw[4], f[4], mx = -INFINITY, l = 0.0f;
#pragma unroll
            for (int w = 0; w < 4; ++w) { mw[w] = red_ml[(w * 16 + row) * 2]; mx = fmaxf(mx, mw[w]); }
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                f[w] = mw[w] == -INFINITY ? 0.0f : fast_exp2(mw[w] - mx);
                l += red_ml[(w * 16 + row) * 2 + 1] * f[w];
                const float4 v = *reinterpret_cast<const float4*>(red_o + ((size_t)(w * 16 + row)) * D + dim);
                acc.x += v.x * f[w]; acc.y += v.y * f[w]; acc.z += v.z * f[w]; acc.w += v.w * f[w];
            }
            const int head = g * G + mt * 16 + row;
            if (nsplit == 1) {
                const float inv = 1.0f / l;
                uint2 packed = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
                *reinterpret_cast<uint2*>(a.out + ((size_t)t * a.nh + head) * D + dim) = packed;
            } else {
                const size_t pi = ((size_t)li * a.nh + head) * grid_splits + split;
                *reinterpret_cast<float4*>(a.part_o + pi * D + dim) = acc;
                if (dim == 0) { a.part_ml[pi * 2] = mx; a.part_ml[pi * 2 + 1] = l; }
            }
        }
    }
    if (gave_up && a.status) atomicCAS(a.status, 0, 5);
    if (nsplit == 1) return;

    // Merge of the splits.  This CTA's partials are in global memory; the CTA that takes
    // the last ticket of this (request, kv head) sees all of them and writes the output:
    // out[t, head, :] = sum_s part_o[s] * 2^(m_s - m) / sum_s l_s * 2^(m_s - m).
    __shared__ int s_ticket;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_ticket = atomicAdd(&a.counters[li * a.nkv + g], 1);
    __syncthreads();
    if (s_ticket != nsplit - 1) return;
    __threadfence();
    // (max, sum) of every (head, split) into shared memory with one round of loads; the tiles are dead
    float2* ml = reinterpret_cast<float2*>(smem);          // [G][nsplit]
    for (int i = threadIdx.x; i < G * nsplit; i += BLOCK_THREADS) {
        const int hg = i / nsplit, sp = i - hg * nsplit;
        ml[i] = __ldcg(reinterpret_cast<const float2*>(a.part_ml) + ((size_t)li * a.nh + g * G + hg) * grid_splits + sp);
    }
    __syncthreads();
    // four dimensions of one head per thread: all its loads of partial outputs are independent
    for (int item = threadIdx.x; item < G * (D / 4); item += BLOCK_THREADS) {
        const int hg = item / (D / 4), dim = (item % (D / 4)) * 4;
        const int head = g * G + hg;
        const float2* mlh = ml + hg * nsplit;
        float mx = -INFINITY, total = 0.0f;
        for (int sp = 0; sp < nsplit; ++sp) mx = fmaxf(mx, mlh[sp].x);
        const float* po = a.part_o + ((size_t)li * a.nh + head) * grid_splits * D + dim;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
        for (int sp = 0; sp < nsplit; ++sp) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(po + (size_t)sp * D));
            const float2 m_l = mlh[sp];
            const float f = m_l.x == -INFINITY ? 0.0f : fast_exp2(m_l.x - mx);
            total += m_l.y * f;
            acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
        }
        const float inv = 1.0f / total;
        uint2 packed = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
        *reinterpret_cast<uint2*>(a.out + ((size_t)t * a.nh + head) * D + dim) = packed;
    }
    if (threadIdx.x == 0) a.counters[li * a.nkv + g] = 0;       // ready for the next launch
}

// ---------------------------------------------------------------- launchers
template <int D>
static int launch_decode(const MmaAttnArgs& a, int n_list, int nsplit, cudaStream_t s) {
    constexpr int STAGES = 3;
    const size_t smem = (size_t)STAGES * 2 * BN * D * 2 + 16 * D * 2 + 2 * STAGES * 8 + 64;   // tiles, Q, barriers
    static unsigned long long configured = 0;
    if (int e = vcb_allow_dynamic_smem(attention_decode_kernel<D, STAGES>, (int)smem, &configured)) return e;
    dim3 grid(nsplit, a.nkv, n_list);
    vcb_launch(attention_decode_kernel<D, STAGES>, grid, BLOCK_THREADS, smem, s, a);
    return vcb_last_error();
}

// ------------------------------------------------- prefill on tcgen05
// Attention for prompt portions, head sizes 64 and 128, on the fifth-generation tensor cores.  A CTA owns 128 packed rows (token x head in group) of one kv head and walks the keys in tiles
// of 64:
//   S = Q K^T      tcgen05.mma, Q and K from shared memory (K-major, 128-byte swizzle: the cache's
//                  planes are that layout already), S (128 x 64 float) in tensor memory, two buffers;
//   softmax        four warps, one thread per row: tcgen05.ld of its row, mask, maximum, ex2.approx,
//                  sum; P rounded to bfloat16 and stored (tcgen05.st) over the first half of the
//                  row's own scores in tensor memory, two keys to a 32-bit column;
//   O += P V       tcgen05.mma with P from tensor memory and V from shared memory as it lies in the
//                  cache (MN-major operand), accumulated in tensor memory (128 x head size, float).
// The exponent's reference is not the running maximum but a value that follows it lazily: it moves
// only when the maximum has risen by more than 8 (in units of log2), and then the row's thread
// rescales its row of O in tensor memory and its sum.  Probabilities stay below 2^8, sums and O in
// float; the rescaling is rare after the first tiles.
// Warp 0 copies K tiles and warp 1 V tiles (bulk copies from the pages, two K stages and three V stages,
// separate barriers so a K stage is free as soon as S is done), warp 2 issues the MMAs, warps 3-6 do the
// rest.  The MMA of tile j + 1's scores is issued before tile j's P V, so the tensor cores work while
// tile j's softmax runs, and two CTAs share an SM (256 columns of tensor memory and, at head size 128,
// 112 KB of shared memory each), so one CTA's softmax runs under the other's MMAs and waits.  Every wait
// is bounded; one that runs out sets *status and the CTA drains and leaves.
namespace tc {
constexpr int BMT = 128, TKT = 64;
constexpr int THREADS = 224;
// stages of the K and of the V ring: what fits beside Q when two CTAs share an SM's shared memory
template <int D> __host__ __device__ constexpr int k_stages() { return D == 64 ? 4 : 2; }
template <int D> __host__ __device__ constexpr int v_stages() { return D == 64 ? 4 : 3; }
constexpr int TMEM_COLS = 256;                                               // S0, S1 (64 each), O (head size)
constexpr float RESCALE_STEP = 8.0f;
// Q, the K and V stages, barriers; no slack: the base must be 1024-aligned
template <int D> constexpr int smem_bytes() { return BMT * D * 2 + (k_stages<D>() + v_stages<D>()) * TKT * D * 2 + 256; }

__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// Two floats to a 64-bit register and packed arithmetic on them (one instruction for two elements), a
// maximum of three: the softmax warps are bound by the instructions they issue.
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// the same with A (128 x 16 bfloat16: row = lane, two elements of k to a column) in tensor memory
__device__ __forceinline__ void mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr),
                   "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                   "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                   "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                   "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
                   "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                   "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
                   "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
                   "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
                 : "memory");
}
__device__ __forceinline__ void st32u(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr),
                   "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                   "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
                   "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
                   "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
                 : "memory");
}
// K-major operand, rows of 128 bytes, 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand (V: the head dimension runs along a row), 128-byte swizzle: planes of 64 elements
// `plane_bytes` apart (leading offset), groups of 8 keys 1024 bytes apart (stride offset).
__device__ __forceinline__ uint64_t desc_mn(uint32_t addr, uint32_t plane_bytes) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((plane_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// float accumulator, bfloat16 A and B, M = 128, N = n; b_mn: B is MN-major
__host__ __device__ constexpr uint32_t idesc(int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

template <int D>
__global__ void __launch_bounds__(THREADS, 2)
attention_prefill_tc_kernel(MmaAttnArgs a) {
    static_assert(D == 64 || D == 128, "one or two planes of 64 elements; S, S and O fit 256 columns");
    constexpr int Q_BYTES = BMT * D * 2, KV_BYTES = TKT * D * 2, K_STAGES = k_stages<D>(), V_STAGES = v_stages<D>();
    extern __shared__ __align__(1024) unsigned char smem[];
    // No early release of the next kernel here: its CTAs would sit on this SM holding tensor memory
    // while CTAs of this kernel still wait to be placed.
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // CTAs start in the order of their index: tile-major, so that the work list's first tiles (those with
    // the most keys) start first for every kv head.  Head-major, a head's long tiles would start after the
    // heads before it had started all of theirs, short ones included, and the kernel would end with them.
    const int tile = blockIdx.x / a.nkv, g = blockIdx.x % a.nkv;
    const int r = a.req_list[tile];
    const int row0 = a.tile_row0[tile];
    const int G = a.nh / a.nkv;
    const int q0 = a.q_start[r], q_len = a.q_start[r + 1] - q0, ctx = a.ctx_lens[r];
    const int rows_total = q_len * G;
    const int* bt = a.block_table + (size_t)r * a.bt_stride;
    const float sl2 = a.scale * LOG2E;

    // [Q][K stages][V stages][barriers]
    const uint32_t sq = smem_u32(smem), sk0 = sq + Q_BYTES, sv0 = sk0 + K_STAGES * KV_BYTES;
    unsigned char* q_ptr = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Q_BYTES + (K_STAGES + V_STAGES) * KV_BYTES);
    // full and empty per K stage and per V stage, s_full and s_free per S buffer, p_full, pv_done, q_ready,
    // o_done (the last P V: a barrier of its own, because a parity tells one phase only and the softmax
    // warps do not follow every phase of pv_done)
    constexpr int FULL_K = 0, EMPTY_K = FULL_K + K_STAGES, FULL_V = EMPTY_K + K_STAGES, EMPTY_V = FULL_V + V_STAGES,
                  S_FULL = EMPTY_V + V_STAGES, S_FREE = S_FULL + 2, P_FULL = S_FREE + 2, PV_DONE = P_FULL + 1,
                  Q_READY = PV_DONE + 1, O_DONE = Q_READY + 1, N_BARS = O_DONE + 1;
    const uint32_t b0 = cx_smem(bars);
    auto B = [&](int i) { return b0 + 8 * i; };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (threadIdx.x == 0) {
        for (int i = 0; i < K_STAGES; ++i) { cx_mbar_init(B(FULL_K + i), 1); cx_mbar_init(B(EMPTY_K + i), 1); }
        for (int i = 0; i < V_STAGES; ++i) { cx_mbar_init(B(FULL_V + i), 1); cx_mbar_init(B(EMPTY_V + i), 1); }
        for (int i = 0; i < 2; ++i) { cx_mbar_init(B(S_FULL + i), 1); cx_mbar_init(B(S_FREE + i), 4); }
        cx_mbar_init(B(P_FULL), 4); cx_mbar_init(B(PV_DONE), 1); cx_mbar_init(B(Q_READY), 4); cx_mbar_init(B(O_DONE), 1);
        // the tiles' swizzle is computed from shared-memory addresses: the base must be a multiple of 1024
        *abort_flag = (sq & 1023) ? 1 : 0;
        if ((sq & 1023) && a.status) atomicCAS(a.status, 0, 10);
        cx_mbar_init_fence();
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tm_s0 = tmem, tm_o = tmem + 2 * TKT;          // S buffers at columns 0 and 64, O at 128

    // keys that any row of the tile can see
    const int last_row = min(row0 + BMT, rows_total) - 1;
    const int hi = ctx + last_row / G + 1;
    const int lo = a.window > 0 ? max(0, ctx + row0 / G + 1 - a.window) : 0;
    const int tile0 = lo / TKT, tile1 = (hi + TKT - 1) / TKT;
    const int n_tiles = *abort_flag ? 0 : tile1 - tile0;

    auto give_up = [&](int code) {
        if (!*abort_flag) { *abort_flag = 1; if (a.status) atomicCAS(a.status, 0, code); }
    };

    if (warp == 0 || warp == 1) {
        // ---- producers: warp 0 copies K tiles (three stages), warp 1 V tiles (two stages).  A tile's copies
        // cost a warp some 0.6 us of address arithmetic and issue, so one warp for both would take longer
        // than the softmax does for the tile.  K_j's stage is free once S_{j-3} is done, V_j's once the P V of
        // tile j - 2 is.
        PageWindow pw;
        const PageDiv pd(a.page);
        pw.init(bt, pd.div(tile0 * TKT), hi, a.page, lane, a.num_pages);
        const size_t page_stride = (size_t)2 * a.nkv * a.page * D, head_base = (size_t)g * a.page * D,
                     v_off = (size_t)a.nkv * a.page * D;
        // a tile's addresses are worked out before its stage is waited for
        TilePiece pc = tile_piece<D, TKT>(tile0 * TKT, lo, hi, pw, a.cache, head_base, page_stride, pd, lane);
        if (warp == 0) {
            int ks = 0, kphase = 1;             // K stage of tile j and the parity its empty barrier is waited with
            for (int j = 0; j < n_tiles && !*abort_flag; ++j) {
                if (!cx_mbar_wait(B(EMPTY_K + ks), kphase)) { give_up(9); break; }
                if (lane == 0) cx_mbar_expect_tx(B(FULL_K + ks), KV_BYTES);
                __syncwarp();
                issue_piece(pc, sk0 + ks * KV_BYTES, 0, B(FULL_K + ks), v_off, lane, 0, 1);
                if (++ks == K_STAGES) { ks = 0; kphase ^= 1; }
                if (j + 1 < n_tiles) pc = tile_piece<D, TKT>((tile0 + j + 1) * TKT, lo, hi, pw, a.cache, head_base, page_stride, pd, lane);
            }
        } else {
            int vs = 0, vphase = 1;
            for (int j = 0; j < n_tiles && !*abort_flag; ++j) {
                if (!cx_mbar_wait(B(EMPTY_V + vs), vphase)) { give_up(9); break; }
                if (lane == 0) cx_mbar_expect_tx(B(FULL_V + vs), KV_BYTES);
                __syncwarp();
                issue_piece(pc, 0, sv0 + vs * KV_BYTES, 0, v_off, lane, B(FULL_V + vs), 2);
                if (++vs == V_STAGES) { vs = 0; vphase ^= 1; }
                if (j + 1 < n_tiles) pc = tile_piece<D, TKT>((tile0 + j + 1) * TKT, lo, hi, pw, a.cache, head_base, page_stride, pd, lane);
            }
        }
        if (pw.bad && a.status) atomicCAS(a.status, 0, VCB_STATUS_BAD_PAGE);
    } else if (warp == 2) {
        // ---- MMA issuer.  The whole warp walks the loop and waits, one elected lane issues: addresses and
        // descriptors are then the same in all lanes, which lets the compiler keep them in uniform
        // registers, where tcgen05.mma wants them; a loop inside "if (lane == 0)" computes them in vector
        // registers and moves every operand of every instruction across.
        if (n_tiles > 0) {
            constexpr uint32_t id_s = idesc(TKT, false), id_pv = idesc(D, true);
            uint32_t leader;
            asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(leader));
            bool ok = cx_mbar_wait(B(Q_READY), 0);            // Q tile written
            fence_after();
            int vs = 0, vphase = 0;
            auto issue_pv = [&](int j) -> bool {                // O += P_j V_j, P_j in the first half of S buffer j & 1
                const int st = j & 1;
                if (!cx_mbar_wait(B(P_FULL), j & 1) || !cx_mbar_wait(B(FULL_V + vs), vphase)) return false;
                fence_after();
                const uint32_t v_base = sv0 + vs * KV_BYTES, tm_p = tm_s0 + st * TKT;
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < TKT / 16; ++kk)       // 16 keys a step: eight columns of P
                        mma_ts(tm_o, tm_p + kk * 8, desc_mn(v_base + kk * 16 * 128, TKT * 128), id_pv, (j > 0 || kk > 0) ? 1u : 0u);
                    commit(B(PV_DONE));         // P read, O updated
                    commit(B(EMPTY_V + vs));    // V stage free
                    if (j == n_tiles - 1) commit(B(O_DONE));
                }
                __syncwarp();
                if (++vs == V_STAGES) { vs = 0; vphase ^= 1; }
                return true;
            };
            int ks = 0, kphase = 0;
            for (int j = 0; j < n_tiles && ok && !*abort_flag; ++j) {
                const int st = j & 1;
                // S_j = Q K_j^T into S buffer j & 1 (free once the softmax of tile j - 2 has read it; the P V
                // of tile j - 2, which read P from the same columns, was issued before and runs before)
                if (!cx_mbar_wait(B(FULL_K + ks), kphase) || !cx_mbar_wait(B(S_FREE + st), ((j >> 1) & 1) ^ 1)) { ok = false; break; }
                fence_after();
                const uint32_t k_base = sk0 + ks * KV_BYTES;
                if (leader) {
#pragma unroll
                    for (int kd = 0; kd < D / 16; ++kd)         // 16 dims a step: plane kd / 4
                        mma(tm_s0 + st * TKT, desc_k(sq + (kd >> 2) * (BMT * 128) + (kd & 3) * 32),
                            desc_k(k_base + (kd >> 2) * (TKT * 128) + (kd & 3) * 32), id_s, kd > 0 ? 1u : 0u);
                    commit(B(S_FULL + st));         // S complete
                    commit(B(EMPTY_K + ks));        // K stage free
                }
                __syncwarp();
                if (++ks == K_STAGES) { ks = 0; kphase ^= 1; }
                if (j > 0 && !issue_pv(j - 1)) { ok = false; break; }
            }
            if (ok && !*abort_flag && !issue_pv(n_tiles - 1)) ok = false;
            if (!ok && lane == 0) give_up(9);
        }
    } else {
        // ---- softmax and output: thread i of warps 3..6 owns row 32 * (warp % 4) + lane (its tensor-memory lane)
        const int lg = warp & 3;
        const int row = lg * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(lg * 32) << 16;
        // Q tile: packed row -> (token, head in group); two planes of 128-byte pieces, chunks swizzled.
        // All of a thread's loads are issued before the first is stored: one at a time they cost a trip
        // to the L2 cache each, 5 us for the tile.
        {
            constexpr int PER_THREAD = BMT * (D / 8) / 128;
            uint4 v[PER_THREAD];
#pragma unroll
            for (int i = 0; i < PER_THREAD; ++i) {
                const int idx = (int)threadIdx.x - 96 + i * 128;
                const int rr = idx / (D / 8), c = idx % (D / 8);
                const int pr = row0 + rr;
                v[i] = make_uint4(0, 0, 0, 0);
                if (pr < rows_total) {
                    const int tt = pr / G, hg = pr % G;
                    v[i] = *reinterpret_cast<const uint4*>(a.q + ((size_t)(q0 + tt) * a.nh + g * G + hg) * D + c * 8);
                }
            }
#pragma unroll
            for (int i = 0; i < PER_THREAD; ++i) {
                const int idx = (int)threadIdx.x - 96 + i * 128;
                *reinterpret_cast<uint4*>(q_ptr + swz_kv<D, BMT>(idx / (D / 8), idx % (D / 8))) = v[i];
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) cx_mbar_arrive(B(Q_READY));

        const int pr = row0 + row;
        const bool row_ok = pr < rows_total;
        const int pos = ctx + min(pr, rows_total - 1) / G;                 // the row's position
        const int row_lo = a.window > 0 ? max(0, pos + 1 - a.window) : 0;
        float m_ref = -INFINITY, l = 0.0f;           // the exponent's reference (in raw score units) and the sum relative to it
        bool ok = true;
        for (int j = 0; j < n_tiles && !*abort_flag; ++j) {
            const int st = j & 1;
            const int kb = (tile0 + j) * TKT;
            if (!cx_mbar_wait(B(S_FULL + st), (j >> 1) & 1)) { ok = false; break; }
            fence_after();
            const uint32_t s_addr = tm_s0 + st * TKT + lane_addr;
            // does any row of the tile mask any key of this tile? (the first row sees the fewest late keys,
            // the last row the fewest early ones)
            const bool edge = kb + TKT - 1 > ctx + row0 / G || (a.window > 0 && kb < ctx + last_row / G + 1 - a.window);
            float s[TKT];
            {
                float t0[32], t1[32];
                ld32(s_addr, t0);
                ld32(s_addr + 32, t1);
#pragma unroll
                for (int i = 0; i < 32; ++i) { s[i] = t0[i]; s[32 + i] = t1[i]; }
            }
            // the S buffer has been read: the scores of tile j + 2 may overwrite it
            fence_before();
            __syncwarp();
            if (lane == 0) cx_mbar_arrive(B(S_FREE + st));
            float mt = -INFINITY;
            if (edge) {
#pragma unroll
                for (int i = 0; i < TKT; ++i) {
                    const int key = kb + i;
                    if (!(key >= row_lo && key <= pos)) s[i] = -INFINITY;
                }
            }
            {
                float m2 = -INFINITY;
#pragma unroll
                for (int i = 0; i < TKT; i += 4) { mt = max3(mt, s[i], s[i + 1]); m2 = max3(m2, s[i + 2], s[i + 3]); }
                mt = fmaxf(mt, m2);
            }
            // move the reference only when the maximum has left it far behind
            float factor = 1.0f;
            if (mt > m_ref && (m_ref == -INFINITY || (mt - m_ref) * sl2 > RESCALE_STEP)) {
                factor = m_ref == -INFINITY ? 0.0f : fast_exp2((m_ref - mt) * sl2);
                m_ref = mt;
            }
            const float base = m_ref == -INFINITY ? 0.0f : m_ref * sl2;
            uint32_t pk[TKT / 2];
            const uint64_t scale2 = pack2(sl2, sl2), minus_base2 = pack2(-base, -base);
            uint64_t sum2[2] = {pack2(0.0f, 0.0f), pack2(0.0f, 0.0f)};
#pragma unroll
            for (int i = 0; i < TKT; i += 2) {
                float e0, e1;
                unpack2(fma2(pack2(s[i], s[i + 1]), scale2, minus_base2), e0, e1);
                const float p0 = fast_exp2(e0), p1 = fast_exp2(e1);
                sum2[(i >> 1) & 1] = add2(sum2[(i >> 1) & 1], pack2(p0, p1));
                pk[i >> 1] = pack_bf16(p0, p1);
            }
            float lt;
            {
                float a0, a1, b0, b1;
                unpack2(sum2[0], a0, a1);
                unpack2(sum2[1], b0, b1);
                lt = (a0 + a1) + (b0 + b1);
            }
            if (j > 0 && __any_sync(0xffffffffu, factor != 1.0f)) {
                // somebody's reference moved: the warp rescales its rows of O (factor 1 where nothing moved),
                // once the P V of the tile before, which adds into them, is done.  (That of tile j - 2 is: the
                // scores of this tile were computed after it.  So the barrier is one or no phase behind and
                // its parity tells which.)
                if (!cx_mbar_wait(B(PV_DONE), (j & 1) ^ 1)) { ok = false; break; }
                fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    float t[32];
                    ld32(tm_o + lane_addr + c0, t);
#pragma unroll
                    for (int i = 0; i < 32; ++i) t[i] *= factor;
                    st32(tm_o + lane_addr + c0, t);
                }
            }
            l = l * factor + lt;
            // P over the row's own scores (this thread has read them; the tensor cores write these columns
            // again only with the scores of tile j + 2, after the P V that reads P)
            st32u(s_addr, pk);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            // the four warps arrive on one barrier per tile: a warp that runs ahead must not count towards
            // a tile that another warp has not finished
            if (j > 0 && !cx_mbar_wait(B(P_FULL), (j - 1) & 1)) { ok = false; break; }
            fence_before();
            __syncwarp();
            if (lane == 0) cx_mbar_arrive(B(P_FULL));
        }
        if (ok && n_tiles > 0 && !*abort_flag) {
            if (!cx_mbar_wait(B(O_DONE), 0)) ok = false;       // the last P V
            fence_after();
            if (ok) {
                const float inv = l > 0.0f ? 1.0f / l : 0.0f;
                const int prc = min(pr, rows_total - 1);
                __nv_bfloat16* dst = a.out + ((size_t)(q0 + prc / G) * a.nh + g * G + prc % G) * D;
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    float t[32];
                    ld32(tm_o + lane_addr + c0, t);
                    if (row_ok) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8)
                            *reinterpret_cast<uint4*>(dst + c0 + i) =
                                make_uint4(pack_bf16(t[i] * inv, t[i + 1] * inv), pack_bf16(t[i + 2] * inv, t[i + 3] * inv),
                                           pack_bf16(t[i + 4] * inv, t[i + 5] * inv), pack_bf16(t[i + 6] * inv, t[i + 7] * inv));
                    }
                }
            }
        }
        if (!ok) give_up(9);
    }
    fence_before();
    __syncthreads();
    if (warp == 2) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}
}  // namespace tc

template <int D>
static int launch_prefill_tc(const MmaAttnArgs& a, int n_tiles, cudaStream_t s) {
    static unsigned long long configured = 0;
    if (int e = vcb_allow_dynamic_smem(tc::attention_prefill_tc_kernel<D>, tc::smem_bytes<D>(), &configured)) return e;
    vcb_launch(tc::attention_prefill_tc_kernel<D>, dim3((unsigned)n_tiles * a.nkv), tc::THREADS, (size_t)tc::smem_bytes<D>(), s, a);
    return vcb_last_error();
}

// Both kernels copy a tile of 64 keys as at most eight runs of whole pages' rows (tile_piece: one lane
// per run), so a page holds a multiple of 8 slots; with smaller pages a tile's byte count would never
// arrive and every wait would run to its limit.
static int check_common(int nh, int nkv, int d, int page, int window, int num_pages) {
    if (nh <= 0 || nkv <= 0 || nh % nkv || page <= 0 || window < 0 || num_pages <= 0) return VCB_ERR_BAD_ARG;
    if (d != 64 && d != 128) return VCB_ERR_UNSUPPORTED;
    if (page % 8) return VCB_ERR_UNSUPPORTED;
    return 0;
}

// split_tiles (device, may be null): key tiles of 64 per split; a request then takes as many of the nsplit
// grid columns as its context needs (see the kernel).
// Scratch for the split-KV merge (nsplit > 1): part_o needs n_list*nh*nsplit*d floats, part_ml
// n_list*nh*nsplit*2 floats, counters n_list*nkv ints that are zero when the kernel starts (it
// leaves them zero).
VCB_EXPORT int vcb_attention_decode_mma(const void* q, const void* cache, void* out, const int* q_start,
                                        const int* ctx_lens, const int* block_table, int bt_stride,
                                        const int* req_list, int n_list, int nsplit, float* part_o,
                                        float* part_ml, int* counters, const int* split_tiles, int nh, int nkv,
                                        int d, int page, int window, float scale, int num_pages, int* status,
                                        void* stream) {
    if (n_list <= 0) return 0;
    int c = check_common(nh, nkv, d, page, window, num_pages);
    if (c) return c;
    if (nsplit < 1 || nsplit > 32 || (nsplit > 1 && (!part_o || !part_ml || !counters))) return VCB_ERR_BAD_ARG;
    MmaAttnArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, (__nv_bfloat16*)out, q_start, ctx_lens,
                  block_table, req_list, nullptr, part_o, part_ml, counters, status, split_tiles, bt_stride, nh, nkv,
                  page, window, scale, num_pages};
    cudaStream_t s = (cudaStream_t)stream;
    return d == 64 ? launch_decode<64>(a, n_list, nsplit, s) : launch_decode<128>(a, n_list, nsplit, s);
}

// Prompt portions (and, in mixed batches, single tokens) on tcgen05 tensor cores: head sizes 64 and 128,
// pages of a multiple of 8 tokens; tiles (tile_req, tile_row0) of 128 packed rows, row = token * G + head
// in group.
VCB_EXPORT int vcb_attention_prefill_tc(const void* q, const void* cache, void* out, const int* q_start,
                                        const int* ctx_lens, const int* block_table, int bt_stride,
                                        const int* tile_req, const int* tile_row0, int n_tiles, int nh,
                                        int nkv, int d, int page, int window, float scale, int num_pages,
                                        int* status, void* stream) {
    if (n_tiles <= 0) return 0;
    int c = check_common(nh, nkv, d, page, window, num_pages);
    if (c) return c;
    MmaAttnArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, (__nv_bfloat16*)out, q_start, ctx_lens,
                  block_table, tile_req, tile_row0, nullptr, nullptr, nullptr, status, nullptr, bt_stride, nh, nkv, page,
                  window, scale, num_pages};
    return d == 64 ? launch_prefill_tc<64>(a, n_tiles, (cudaStream_t)stream) : launch_prefill_tc<128>(a, n_tiles, (cudaStream_t)stream);
}

// ------------------------------------------------ no-allocation entry point
// See no_alloc.h for who this is for and its limits.
#include "no_alloc.h"

// Merge scratch of the static variant: rows of (d floats of partial output), then
// rows of (max, sum).  In host code this name is only a handle for the symbol; the
// device address is looked up below.
static __device__ __align__(256) float vcb_static_scratch[VCB_STATIC_SCRATCH_ROWS * (VCB_STATIC_SCRATCH_DIM + 2)];

// Tickets of the split merge, one per (request, kv head); cleared before every launch.
static __device__ __align__(256) int vcb_static_counters[VCB_STATIC_SCRATCH_ROWS];

// Where the kernel notes that it gave up on a bounded wait or met a page number outside the cache;
// vcb_attention_decode_mma_static_status reads and clears it.
static __device__ int vcb_static_status_word;

#define VCB_MAX_DEVICES 64
static float* vcb_static_scratch_addr[VCB_MAX_DEVICES];
static int* vcb_static_counters_addr[VCB_MAX_DEVICES];
static int* vcb_static_status_addr[VCB_MAX_DEVICES];

// The arrays' addresses on the current device, looked up once per device.
static int static_scratch_address(float** addr, int** counters, int** status) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= VCB_MAX_DEVICES) return VCB_ERR_BAD_ARG;
    if (vcb_static_scratch_addr[dev] == nullptr || vcb_static_counters_addr[dev] == nullptr ||
        vcb_static_status_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, vcb_static_scratch);
        if (e != cudaSuccess) return (int)e;
        void* pc = nullptr;
        e = cudaGetSymbolAddress(&pc, vcb_static_counters);
        if (e != cudaSuccess) return (int)e;
        void* ps = nullptr;
        e = cudaGetSymbolAddress(&ps, vcb_static_status_word);
        if (e != cudaSuccess) return (int)e;
        vcb_static_scratch_addr[dev] = static_cast<float*>(p);
        vcb_static_counters_addr[dev] = static_cast<int*>(pc);
        vcb_static_status_addr[dev] = static_cast<int*>(ps);
    }
    *addr = vcb_static_scratch_addr[dev];
    *counters = vcb_static_counters_addr[dev];
    *status = vcb_static_status_addr[dev];
    return 0;
}

VCB_EXPORT int vcb_attention_decode_mma_static(const void* q, const void* cache, void* out, const int* q_start,
                                               const int* ctx_lens, const int* block_table, int bt_stride,
                                               const int* req_list, int n_list, int nsplit, int nh, int nkv,
                                               int d, int page, int window, float scale, int num_pages,
                                               void* stream) {
    if (n_list <= 0) return 0;
    int c = check_common(nh, nkv, d, page, window, num_pages);
    if (c) return c;
    if (nsplit < 1 || nsplit > 32) return VCB_ERR_BAD_ARG;
    const long long rows = nsplit > 1 ? (long long)n_list * nh * nsplit : 0;
    if (rows > VCB_STATIC_SCRATCH_ROWS || d > VCB_STATIC_SCRATCH_DIM) return VCB_ERR_SCRATCH_TOO_SMALL;
    float* part_o = nullptr;
    float* part_ml = nullptr;
    float* base = nullptr;
    int* counters = nullptr;
    int* status = nullptr;
    cudaStream_t s = (cudaStream_t)stream;
    c = static_scratch_address(&base, &counters, &status);
    if (c) return c;
    if (nsplit > 1) {
        part_o = base;
        part_ml = base + (size_t)VCB_STATIC_SCRATCH_ROWS * VCB_STATIC_SCRATCH_DIM;
        // the tickets must start at zero whatever an earlier call left behind
        cudaError_t e = cudaMemsetAsync(counters, 0, sizeof(int) * (size_t)n_list * nkv, s);
        if (e != cudaSuccess) return (int)e;
    }
    MmaAttnArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, (__nv_bfloat16*)out, q_start, ctx_lens,
                  block_table, req_list, nullptr, nsplit > 1 ? part_o : nullptr, part_ml, nsplit > 1 ? counters : nullptr,
                  status, nullptr, bt_stride, nh, nkv, page, window, scale, num_pages};
    return d == 64 ? launch_decode<64>(a, n_list, nsplit, s) : launch_decode<128>(a, n_list, nsplit, s);
}

VCB_EXPORT int vcb_attention_decode_mma_static_status(int* code) {
    float* base = nullptr;
    int* counters = nullptr;
    int* status = nullptr;
    int c = static_scratch_address(&base, &counters, &status);
    if (c) return c;
    int seen = 0;
    cudaError_t e = cudaMemcpy(&seen, status, sizeof(int), cudaMemcpyDeviceToHost);     // waits for the device
    if (e != cudaSuccess) return (int)e;
    if (seen) {
        e = cudaMemset(status, 0, sizeof(int));
        if (e != cudaSuccess) return (int)e;
    }
    if (code) *code = seen;
    return 0;
}
