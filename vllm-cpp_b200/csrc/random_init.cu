// Random weights on the device: element i of a tensor is a function of (key, i) alone.
//
// The reference has no random-weights mode; this one exists so that a model of any size can be
// filled without a checkpoint and so that a host program can reproduce every value of it.
// weights/random_init.py holds the same arithmetic in numpy, step for step; the two agree to
// the bit because every floating-point step below is a single correctly rounded IEEE operation
// (add, multiply, divide, square root, written with the _rn intrinsics so that the compiler
// fuses none of them) and everything else is integer arithmetic.  No library logarithm, sine or
// cosine is used: theirs differ between libm and CUDA.
//
//   z      = splitmix64 finaliser of (key + (i + 1) * 0x9E3779B97F4A7C15)
//   a, b   = bits 63..40 and 39..16 of z (24 bits each)
//   u1     = (a + 1) / 2^24                         in (0, 1]
//   radius = sqrt(-2 ln u1)                         ln by argument reduction + an atanh series
//   angle  = 2 pi (b + 1/2) / 2^24                  cosine by quadrant + Taylor polynomials
//   normal = radius * cos(angle)                    (Box-Muller, one value per element)
//   value  = mean + std * normal, then rounded to the storage type
#include "common.cuh"

namespace {

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
// constants by bit pattern, the same words that weights/random_init.py uses
#define F32_BITS(x) __int_as_float((int)(x))

// ln(n / 2^24) for an integer n in [1, 2^24]
__device__ __forceinline__ float ln_u24(uint32_t n) {
    int e = 31 - __clz(n);                                   // n = m * 2^e, m in [1, 2)
    float m = mul(__uint2float_rn(n), __int_as_float((127 - e) << 23));   // exact: a power of two
    if (m > F32_BITS(0x3fb504f3u) /* sqrt 2 */) { m = mul(m, 0.5f); e += 1; }       // m in (0.707, 1.414]
    const float s = __fdiv_rn(add(m, -1.0f), add(m, 1.0f));
    const float s2 = mul(s, s);
    float p = F32_BITS(0x3de38e39u);                           // 1/9
    p = add(mul(p, s2), F32_BITS(0x3e124925u));                // 1/7
    p = add(mul(p, s2), F32_BITS(0x3e4ccccdu));                // 1/5
    p = add(mul(p, s2), F32_BITS(0x3eaaaaabu));                // 1/3
    p = add(mul(p, s2), 1.0f);
    const float ln_m = mul(mul(2.0f, s), p);
    return add(mul((float)(e - 24), F32_BITS(0x3f317218u) /* ln 2 */), ln_m);
}

// cos(2 pi (b + 1/2) / 2^24) for an integer b in [0, 2^24)
__device__ __forceinline__ float cos_u24(uint32_t b) {
    const uint32_t quadrant = b >> 22, f = b & 0x3FFFFFu;
    const float x = mul(add(__uint2float_rn(f), 0.5f), F32_BITS(0x34800000u));   // (f + 1/2) / 2^22, exact
    const bool upper = x > 0.5f;
    const float y = upper ? add(1.0f, -x) : x;               // in (0, 1/2]
    const float t = mul(y, F32_BITS(0x3fc90fdbu) /* pi/2 */);                     // angle in (0, pi/4]
    const float t2 = mul(t, t);
    float sp = F32_BITS(0x3638ef1du);                          // 1/9!
    sp = add(mul(sp, t2), F32_BITS(0xb9500d01u));               // -1/7!
    sp = add(mul(sp, t2), F32_BITS(0x3c088889u));               // 1/5!
    sp = add(mul(sp, t2), F32_BITS(0xbe2aaaabu));               // -1/3!
    sp = add(mul(sp, t2), 1.0f);
    const float sn = mul(t, sp);
    float cp = F32_BITS(0xb493f27eu);                          // -1/10!
    cp = add(mul(cp, t2), F32_BITS(0x37d00d01u));               // 1/8!
    cp = add(mul(cp, t2), F32_BITS(0xbab60b61u));               // -1/6!
    cp = add(mul(cp, t2), F32_BITS(0x3d2aaaabu));               // 1/4!
    cp = add(mul(cp, t2), -0.5f);
    cp = add(mul(cp, t2), 1.0f);
    const float c = upper ? sn : cp, s = upper ? cp : sn;    // cos and sin of x * pi/2
    return quadrant == 0 ? c : quadrant == 1 ? -s : quadrant == 2 ? -c : s;
}

template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, size_t n, uint64_t key, float mean, float std_) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint64_t z = mix64(key + (uint64_t)(i + 1) * 0x9E3779B97F4A7C15ull);
        const uint32_t a = (uint32_t)(z >> 40), b = (uint32_t)(z >> 16) & 0xFFFFFFu;
        const float radius = __fsqrt_rn(mul(-2.0f, ln_u24(a + 1)));
        const float normal = mul(radius, cos_u24(b));
        out[i] = from_f32<T>(add(mean, mul(std_, normal)));
    }
}

}  // namespace

// out[i] = mean + std * normal(key, first + i) for i < n, in the storage type; `first` lets a caller
// fill a slice of a tensor (rows of a matrix) with the values the whole tensor would have there.
VCB_EXPORT int vcb_random_normal(void* out, unsigned long long n, unsigned long long first, unsigned long long key,
                                 float mean, float std_, int dtype, void* stream) {
    if (n == 0) return 0;
    const int threads = 256;
    const unsigned long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 4096 ? want : 4096);          // a grid-stride loop covers the rest
    cudaStream_t s = (cudaStream_t)stream;
    const uint64_t k = key + first * 0x9E3779B97F4A7C15ull;      // the kernel adds (i + 1) times the same constant
    if (dtype == VCB_F32)
        random_normal_kernel<float><<<blocks, threads, 0, s>>>((float*)out, (size_t)n, k, mean, std_);
    else if (dtype == VCB_BF16)
        random_normal_kernel<__nv_bfloat16><<<blocks, threads, 0, s>>>((__nv_bfloat16*)out, (size_t)n, k, mean, std_);
    else
        return VCB_ERR_BAD_ARG;
    return vcb_last_error();
}
