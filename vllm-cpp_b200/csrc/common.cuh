// Shared helpers for the sm_100a kernels of this engine.
//
// Every kernel is a template over the storage type T of activations, weights
// and cache (float for the true 32-bit path, __nv_bfloat16 for serving).  All
// arithmetic that decides a result's accuracy (softmax, norms, rotation angles,
// the residual sum, every accumulation) is done in float regardless of T.
// No translation unit is compiled with --use_fast_math.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define VCB_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side (csrc/ops.py)
enum { VCB_F32 = 0, VCB_BF16 = 1 };

// Return codes of the exported launchers beyond cudaError_t values.
enum { VCB_ERR_BAD_ARG = 10001, VCB_ERR_UNSUPPORTED = 10002 };

// Codes that kernels leave in the device status word (csrc/ops.py STATUS_MEANING names them all).
enum { VCB_STATUS_BAD_PAGE = 11, VCB_STATUS_BAD_TOKEN = 12 };

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a whole CTA (blockDim.x a multiple of 32, at most 1024); every thread
// gets the result.  `scratch` holds at least 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();                       // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

static inline int vcb_last_error() { return (int)cudaGetLastError(); }

// Streaming multiprocessors of the current device, asked once per device (a cap for grid-stride grids).
static inline int vcb_sm_count() {
    static int count[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 128;
    if (count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 128;
        count[dev] = n;
    }
    return count[dev];
}

// A kernel's cap on dynamic shared memory belongs to the (kernel, device) pair.  `done` is the calling
// launcher's own word, one bit per device: the attribute is set at the first launch on each device.
// (Two host threads that race here both set the same value.)
template <typename K>
static inline int vcb_allow_dynamic_smem(K kernel, int bytes, unsigned long long* done) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    const unsigned long long bit = 1ull << (dev & 63);
    if (dev < 64 && (__atomic_load_n(done, __ATOMIC_RELAXED) & bit)) return 0;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return (int)e;
    if (dev < 64) __atomic_fetch_or(done, bit, __ATOMIC_RELAXED);
    return 0;
}

// ---- layout of the cache
// A page holds [k|v][kv head] blocks of page * head_dim elements.  When a row (one slot of one head)
// is a multiple of 128 bytes, a block is stored in planes of 128-byte row pieces,
// [plane][slot][128 bytes], and inside a piece the 16-byte chunks are XOR-swizzled by the slot
// number: chunk c of slot s lives at chunk c ^ (s & 7).  A run of slots of one plane is then, byte for
// byte, a run of rows of the 128-byte-swizzled K-major (or MN-major) tile that the tensor cores read from
// shared memory -- tcgen05.mma through its shared-memory descriptor, mma.sync through conflict-free
// ldmatrix -- and one plain bulk copy brings it there.  Rows of other sizes are stored as they are,
// [slot][head_dim].  kv_pos: offset of element `elem` of slot `slot` inside its block.
__host__ __device__ __forceinline__ int kv_pos(int elem, int slot, int d, int page, int esize) {
    if ((d * esize) & 127) return slot * d + elem;
    const int per_plane = 128 / esize, per_chunk = 16 / esize;
    const int plane = elem / per_plane, w = elem - plane * per_plane;
    const int chunk = w / per_chunk, within = w - chunk * per_chunk;
    return plane * (page * per_plane) + slot * per_plane + ((chunk ^ (slot & 7)) * per_chunk) + within;
}

// ---- mbarriers and bulk copies (shared by the kernels that stage memory asynchronously)
#define CX_SPIN_LIMIT (1u << 22)
__device__ __forceinline__ uint32_t cx_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cx_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void cx_mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void cx_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cx_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait for the phase with the given parity.  False: gave up.
__device__ __forceinline__ bool cx_mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < CX_SPIN_LIMIT; ++spin) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.b32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// Contiguous global -> shared copy by the TMA unit; completes on the mbarrier.  No multicast.
__device__ __forceinline__ void cx_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// ---- programmatic dependent launch
// Kernels of a step are launched so that the next kernel in the stream may begin while the
// previous one still runs: its CTAs become resident, set themselves up (and, in the matrix
// products, start streaming weights, which depend on nothing) and then block in
// griddepcontrol.wait until the previous kernel has completed and its writes are visible.
// Every kernel launched this way executes pdl_start() (or its two halves) before it touches
// memory that another kernel writes or reads.  With the switch off, launches are ordinary.
extern int vcb_pdl_enabled;                 // defined in elementwise.cu; set by vcb_set_pdl

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_start() { pdl_launch_dependents(); pdl_wait(); }

template <typename... KArgs, typename... Args>
static inline void vcb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = vcb_pdl_enabled ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
