// True 32-bit matrix product C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores: IEEE float32
// multiply-add, no TF32, no reduced-precision staging.  It serves the float32 path of the
// whole model, whose purpose is to show faults that bfloat16 rounding hides, so it favours a
// fixed summation order over speed: every output element adds its K products in the same
// order whatever M is, hence a token's logits do not depend on what else is in the batch.
// (The reference reaches float32 by running its library path with DTYPE=float32 on the CPU,
// tests/test_batching.py:57; it has no float32 GPU path.)
#include "common.cuh"

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256) gemm_f32_nt_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W,
                                                          float* __restrict__ C, int ldc, int M, int N, int K) {
    __shared__ float As[BK][BM + 4], Ws[BK][BN + 4];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += 256) {
            const int r = i / BK, c = i % BK;
            const int m = m0 + r, n = n0 + r, k = k0 + c;
            As[c][r] = (m < M && k < K) ? A[(size_t)m * lda + k] : 0.f;
            Ws[c][r] = (n < N && k < K) ? W[(size_t)n * K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[k][ty * 4 + i]; b[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
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

MI_EXPORT int mi_gemm_f32_nt(const float* A, int lda, const float* W, float* C, int ldc, int M, int N, int K,
                             cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_f32_nt_kernel<<<grid, 256, 0, stream>>>(A, lda, W, C, ldc, M, N, K);
    return (int)cudaGetLastError();
}
