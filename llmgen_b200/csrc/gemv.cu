// C[M, N] = A[M, K] * W[N, K]^T for a handful of rows (M <= 4) in bfloat16: the weight-streaming
// product of small decode batches.  One warp per output column n streams W[n, :] once with
// 16-byte loads and keeps M float32 accumulators; the few rows of A come from L1.
//
// Same role as the reference's `gemv_kernel<M, OUT_F32>` (src/backend/cuda/linear/linear.cu:22-61:
// one warp per output row, 16-byte weight loads, K % 8 == 0, M <= SV_GEMV_MAX_M = 2).  Here
// M <= 4, an optional float32 output (logits) and an optional accumulate into C.
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

constexpr int WARPS = 8;

template <int M, typename TC>
__global__ void __launch_bounds__(WARPS * 32)
gemv_bf16_kernel(TC* __restrict__ C, const bf16* __restrict__ A, const bf16* __restrict__ W, int N, int K,
                 long long lda, long long ldw, long long ldc, int accumulate) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * WARPS + (threadIdx.x >> 5);
    if (n >= N) return;
    const uint4* w = reinterpret_cast<const uint4*>(W + (size_t)n * ldw);
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    const int kv = K / 8;  // 16-byte vectors per row
    for (int v0 = lane; v0 < kv; v0 += 32 * 4) {
        uint4 wv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = v0 + 32 * u;
            wv[u] = v < kv ? __ldcs(w + v) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = v0 + 32 * u;
            if (v >= kv) continue;
            float wf[8];
            Vec16<bf16> t;
            t.raw = wv[u];
            t.unpack(wf);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                Vec16<bf16> a;
                a.raw = __ldg(reinterpret_cast<const uint4*>(A + (size_t)m * lda) + v);
                float af[8];
                a.unpack(af);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[m] = fmaf(af[i], wf[i], acc[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
        const float v = warp_sum(acc[m]);
        if (lane == 0) {
            TC* c = C + (size_t)m * ldc + n;
            *c = from_float<TC>(accumulate ? v + to_float(*c) : v);
        }
    }
}

template <typename TC>
static int launch_m(void* C, const void* A, const void* W, int M, int N, int K, long long lda, long long ldw,
                    long long ldc, int accumulate, cudaStream_t s) {
    const int grid = ceil_div(N, WARPS);
#define CASE(MM)                                                                                               \
    case MM:                                                                                                   \
        gemv_bf16_kernel<MM, TC><<<grid, WARPS * 32, 0, s>>>((TC*)C, (const bf16*)A, (const bf16*)W, N, K, lda, \
                                                              ldw, ldc, accumulate);                           \
        break;
    switch (M) {
        CASE(1) CASE(2) CASE(3) CASE(4)
        default: return LLMK_BAD_ARG;
    }
#undef CASE
    return LLMK_OK;
}

LLMK_EXPORT int llmk_gemv_max_rows() { return 4; }

// Usable iff M <= 4, K % 8 == 0, and A, W rows start on 16-byte boundaries.
LLMK_EXPORT int llmk_gemv_bf16(void* C, const void* A, const void* W, int M, int N, int K, long long lda,
                               long long ldw, long long ldc, int accumulate, int out_dtype, void* stream) {
    if (M <= 0 || N <= 0) return LLMK_OK;
    if (M > 4) LLMK_FAIL("gemv_bf16: M=%d above 4", M);
    if (K <= 0 || K % 8 != 0) LLMK_FAIL("gemv_bf16: K=%d must be a positive multiple of 8", K);
    if (lda % 8 != 0 || ldw % 8 != 0 || !host_aligned16(A) || !host_aligned16(W))
        LLMK_FAIL("gemv_bf16: rows of A and W must start on 16-byte boundaries");
    if (ldc < N) LLMK_FAIL("gemv_bf16: ldc=%lld below N=%d", ldc, N);
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    if (out_dtype == LLMK_BF16)
        rc = launch_m<bf16>(C, A, W, M, N, K, lda, ldw, ldc, accumulate, s);
    else if (out_dtype == LLMK_F32)
        rc = launch_m<float>(C, A, W, M, N, K, lda, ldw, ldc, accumulate, s);
    else
        LLMK_FAIL("gemv_bf16: unknown output dtype %d", out_dtype);
    if (rc != LLMK_OK) LLMK_FAIL("gemv_bf16: unsupported M=%d", M);
    LLMK_CHECK_LAUNCH("gemv_bf16");
    return LLMK_OK;
}
