// True 32-bit matrix product for the float32 path:  C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]).
//
// FFMA only: no tensor cores, no TF32, no split-K.  Every output element is the sum of its K
// products taken in ascending k by one thread, so a row's result does not depend on M, on the
// other rows of the batch or on where the row sits in it.  The reference calls cuBLAS for
// every contraction (gpu/cuda/matmul.cu:316-355) and has no float32 path.
#include "ng_common.cuh"

#define BM 64
#define BN 64
#define BK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                float* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    ng_pdl_trigger();
    ng_pdl_wait();
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tr = tid / 16, tc = tid % 16;          // thread's 4x4 sub-tile: rows tr*4.., cols tc*4..
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // loader mapping: 256 threads load 64 rows x 16 k, 4 elements each (one k-quad of one row)
    const int lrow = tid / 4, lk = (tid % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k = k0 + lk + q;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + q][lrow] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
            Ws[lk + q][lrow] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][tr * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tc * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tr * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tc * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = acc[i][j] + (bias ? bias[n] : 0.f);
        }
    }
}

NG_EXPORT int ng_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K,
                          int lda, int ldw, int ldc, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return NG_OK;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return NG_BAD_SIZE;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return NG_BAD_SIZE;
    NG_LAUNCH((gemm_f32_kernel), grid, 256, 0, stream, A, W, bias, C, M, N, K, lda, ldw, ldc);
    return ng_launch_status();
}
