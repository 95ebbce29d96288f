// C[M, N] = A[M, K] * W[N, K]^T with float32 multiply-add on the CUDA cores: the matrix product of
// the true 32-bit path (no tensor cores, no TF32) and the fallback of the bfloat16 path for
// shapes the tensor-core kernels refuse.
//
// Every output element is the sum over k = 0..K-1 in ascending order inside one thread, so a
// row's result does not depend on M, on the tile it falls in or on what else is in the batch.
// Weight layout [out, in] row-major, no bias, as in the reference
// (src/module/linear.zig:48-82, src/backend/cpu/linear.zig:7-28); the reference's own CUDA path
// is a bfloat16 GEMV or cuBLAS (src/backend/cuda/linear/linear.cu:22-96) and has no float32
// product.
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

constexpr int BN = 64, BK = 16, THREADS = 256;

// Tile BM x BN per block, 16 x 16 threads, each thread TM x 4 outputs (BM = 16 * TM).
template <typename TA, typename TW, typename TC, int TM>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(TC* __restrict__ C, const TA* __restrict__ A, const TW* __restrict__ W, int M, int N, int K,
                 long long lda, long long ldw, long long ldc, int accumulate) {
    constexpr int BM = 16 * TM;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][4];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // A tile: BM x BK values, W tile: BN x BK values; consecutive threads walk along k.
        for (int idx = threadIdx.x; idx < BM * BK; idx += THREADS) {
            const int r = idx / BK, c = idx % BK;
            const int gm = m0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? to_float(A[(size_t)gm * lda + gk]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < BN * BK; idx += THREADS) {
            const int r = idx / BK, c = idx % BK;
            const int gn = n0 + r, gk = k0 + c;
            Ws[c][r] = (gn < N && gk < K) ? to_float(W[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[4];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            TC* c = C + (size_t)gm * ldc + gn;
            float v = acc[i][j];
            if (accumulate) v += to_float(*c);
            *c = from_float<TC>(v);
        }
    }
}

template <typename TA, typename TW, typename TC>
static void launch(void* C, const void* A, const void* W, int M, int N, int K, long long lda, long long ldw,
                   long long ldc, int accumulate, cudaStream_t s) {
    if (M <= 16) {
        dim3 grid(ceil_div(N, BN), ceil_div(M, 16));
        gemm_simt_kernel<TA, TW, TC, 1><<<grid, THREADS, 0, s>>>((TC*)C, (const TA*)A, (const TW*)W, M, N, K, lda,
                                                                  ldw, ldc, accumulate);
    } else {
        dim3 grid(ceil_div(N, BN), ceil_div(M, 64));
        gemm_simt_kernel<TA, TW, TC, 4><<<grid, THREADS, 0, s>>>((TC*)C, (const TA*)A, (const TW*)W, M, N, K, lda,
                                                                  ldw, ldc, accumulate);
    }
}

// dtype: storage of A and W; out_dtype: storage of C (float32 output of a bfloat16 product is
// what the logits use).  accumulate != 0 adds into C.
LLMK_EXPORT int llmk_gemm_simt(void* C, const void* A, const void* W, int M, int N, int K, long long lda,
                               long long ldw, long long ldc, int accumulate, int dtype, int out_dtype,
                               void* stream) {
    if (M <= 0 || N <= 0) return LLMK_OK;
    if (K <= 0) LLMK_FAIL("gemm_simt: K=%d", K);
    if (lda < K || ldw < K || ldc < N) LLMK_FAIL("gemm_simt: strides lda=%lld ldw=%lld ldc=%lld too small for K=%d N=%d", lda, ldw, ldc, K, N);
    if (ceil_div(M, 16) > 65535) LLMK_FAIL("gemm_simt: M=%d too large", M);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == LLMK_F32 && out_dtype == LLMK_F32)
        launch<float, float, float>(C, A, W, M, N, K, lda, ldw, ldc, accumulate, s);
    else if (dtype == LLMK_BF16 && out_dtype == LLMK_BF16)
        launch<bf16, bf16, bf16>(C, A, W, M, N, K, lda, ldw, ldc, accumulate, s);
    else if (dtype == LLMK_BF16 && out_dtype == LLMK_F32)
        launch<bf16, bf16, float>(C, A, W, M, N, K, lda, ldw, ldc, accumulate, s);
    else
        LLMK_FAIL("gemm_simt: unsupported dtypes in=%d out=%d", dtype, out_dtype);
    LLMK_CHECK_LAUNCH("gemm_simt");
    return LLMK_OK;
}
