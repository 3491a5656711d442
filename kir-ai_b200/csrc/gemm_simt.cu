// Plain matrix product on the CUDA cores: C[M, N] = A[M, K] * W[N, K]^T with
// 32-bit fused multiply-adds, k walked in order for every output element (no
// split along K), so an output row does not depend on which other rows are in
// the batch.  With float operands this is the true 32-bit path of every linear
// layer; with bf16 operands it is the plain reference beside the tensor-core
// kernel.  Any M, N, K >= 1; A and C may have row strides.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TIn* __restrict__ A, const TIn* __restrict__ W, TOut* __restrict__ C, int M, int N, int K,
                 long lda, long ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, each a 4 x 4 patch
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    // each thread loads 4 values of A and 4 of W per k-step: 64 rows x 16 k = 1024 values / 256 threads
    const int load_row = tid / 4;        // 0..63
    const int load_k = (tid % 4) * 4;    // 0,4,8,12
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + load_k + i;
            const int ar = row0 + load_row, wr = col0 + load_row;
            As[load_k + i][load_row] = (ar < M && k < K) ? to_f32<TIn>(A[(size_t)ar * lda + k]) : 0.0f;
            Ws[load_k + i][load_row] = (wr < N && k < K) ? to_f32<TIn>(W[(size_t)wr * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty * 4 + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = col0 + tx * 4 + j;
            if (c < N) C[(size_t)r * ldc + c] = from_f32<TOut>(acc[i][j]);
        }
    }
}

template <typename TIn, typename TOut>
static int gemm_simt_launch(const void* A, const void* W, void* C, int M, int N, int K, long lda, long ldc,
                            cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return KIRAI_ERR_BAD_SIZE;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return KIRAI_ERR_BAD_SIZE;
    gemm_simt_kernel<TIn, TOut><<<grid, 256, 0, stream>>>((const TIn*)A, (const TIn*)W, (TOut*)C, M, N, K, lda, ldc);
    return launch_status();
}

KIRAI_EXPORT int kirai_gemm_simt_f32(const void* A, const void* W, void* C, int M, int N, int K, long lda, long ldc,
                                     cudaStream_t stream) {
    return gemm_simt_launch<float, float>(A, W, C, M, N, K, lda, ldc, stream);
}
KIRAI_EXPORT int kirai_gemm_simt_bf16(const void* A, const void* W, void* C, int M, int N, int K, long lda, long ldc,
                                      cudaStream_t stream) {
    return gemm_simt_launch<bf16, bf16>(A, W, C, M, N, K, lda, ldc, stream);
}
KIRAI_EXPORT int kirai_gemm_simt_bf16_out_f32(const void* A, const void* W, void* C, int M, int N, int K, long lda,
                                              long ldc, cudaStream_t stream) {
    return gemm_simt_launch<bf16, float>(A, W, C, M, N, K, lda, ldc, stream);
}
