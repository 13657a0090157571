// True 32-bit matrix product for the float path:  C[M,N] = A[M,K] * W[N,K]^T.
//
// Plain FMA on float operands with float accumulation: no TF32, no split
// operands, no tensor cores.  The reference has no such path; its products always
// round the operands to half precision (src/layers/linear.cpp:67-77).
// W is stored as the checkpoint stores it, [out_features, in_features] row-major.
//
// 64x64 output tile per CTA, 16-deep k slices staged in shared memory, a 4x4
// register tile per thread.  Every edge is guarded, so any M, N, K >= 1 works.
#include "common.cuh"

#define GT 64
#define GK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K, int lda, int ldw, int ldc) {
    __shared__ float As[GK][GT + 1];
    __shared__ float Ws[GK][GT + 1];
    pdl_start();
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += GK) {
        // 64 rows x 16 k per operand = 1024 elements, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = threadIdx.x + e * 256;
            const int r = idx / GK, kk = idx % GK;
            const int k = k0 + kk;
            As[kk][r] = (m0 + r < M && k < K) ? A[(size_t)(m0 + r) * lda + k] : 0.0f;
            Ws[kk][r] = (n0 + r < N && k < K) ? W[(size_t)(n0 + r) * ldw + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
        }
    }
}

VCB_EXPORT int vcb_gemm_f32(const float* A, const float* W, float* C, int M, int N, int K,
                            int lda, int ldw, int ldc, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return VCB_ERR_BAD_ARG;
    dim3 grid((N + GT - 1) / GT, (M + GT - 1) / GT);
    vcb_launch(gemm_f32_kernel, grid, 256, 0, (cudaStream_t)stream, A, W, C, M, N, K, lda, ldw, ldc);
    return vcb_last_error();
}
