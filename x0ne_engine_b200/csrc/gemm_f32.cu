// C[M,N] = A[M,K] * W[N,K]^T in true float32: FMA on the CUDA cores, no tensor-core mode.
//
// This is the matrix product of the 32-bit path.  Each output is ONE chain of fused
// multiply-adds over k = 0, 1, ..., K-1 in that order, whatever M is and wherever the output
// lies in its tile, so a row's result is bit-identical whether the row is computed alone, in a
// batch, in a prompt or in a decode step.  (The library engine calls cublasGemmEx for its
// products, x0ne-core/runtime/src/gpu.rs:1098-1149; a library picks its algorithm by shape, so
// the same row can round differently at different M, which this kernel exists to rule out.)
//
// Tile 128 x 64 x 16, 256 threads, 8 x 4 outputs per thread, operands staged through shared
// memory with the k index outermost.
#include "common.cuh"

#define BM 128
#define BN 64
#define BK 16
#define TM 8
#define TN 4

__global__ void __launch_bounds__(256) gemm_f32_nt_kernel(const float* __restrict__ A, const float* __restrict__ W,
                                                           float* __restrict__ C, int M, int N, int K, int lda,
                                                           int ldw, int ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_prologue();
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;  // tx: 16 column groups of 4, ty: 16 row groups of 8
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // A tile: 128 rows x 16 k = 2048 values, 8 per thread
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int idx = tid + it * 256;
            const int r = idx / BK, kk = idx % BK;
            const int gm = m0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? A[(int64_t)gm * lda + gk] : 0.f;
        }
        // W tile: 64 rows x 16 k = 1024 values, 4 per thread
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * 256;
            const int r = idx / BK, kk = idx % BK;
            const int gn = n0 + r, gk = k0 + kk;
            Ws[kk][r] = (gn < N && gk < K) ? W[(int64_t)gn * ldw + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) C[(int64_t)gm * ldc + gn] = acc[i][j];
        }
    }
}

X0NE_API int x0ne_gemm_f32_nt(const float* A, const float* W, float* C, int M, int N, int K, int lda, int ldw, int ldc,
                              cudaStream_t stream) {
    X0NE_REQUIRE(M >= 0 && N > 0 && K > 0 && lda >= K && ldw >= K && ldc >= N, "gemm_f32: M %d N %d K %d lda %d ldw %d ldc %d",
                 M, N, K, lda, ldw, ldc);
    if (M == 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    X0NE_REQUIRE(grid.y <= 65535, "gemm_f32: M %d needs more than 65535 row tiles", M);
    x0ne_launch(gemm_f32_nt_kernel, dim3(grid), dim3(256), 0, stream, A, W, C, M, N, K, lda, ldw, ldc);
    X0NE_LAUNCH_CHECK();
}
