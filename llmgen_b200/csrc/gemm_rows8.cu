// out[slices][M][N] (float32) = partial sums of x[M][K] * W[N][K]^T in bfloat16 for up to 8 rows of x (a decode step
// of up to 8 sequences): the weight-streaming product with the shortest way from global memory to the sum.
//
// A warp owns 16 rows of W and one slice of K.  It asks for all of its W (16 bytes a lane and row and 32-wide block
// of K, straight into registers: no shared memory, no barrier, no tensor memory) BEFORE the wait for the kernel that
// makes x, since W is a weight that no kernel writes; after the wait it loads its slice of x the same way and issues
// `mma.sync.m16n8k16` with W's rows as the MMA's rows and the rows of x as its 8 columns.  The 8 values a lane loads
// per row and block are 8 consecutive k; the MMA's fragment layout wants (2t, 2t+1, 2t+8, 2t+9) of a 16-wide k step,
// but a sum over k does not care which k meets which as long as A and B agree, and both are loaded alike.
// The slices of K are added up by the consumer (`ops.Partials`), as for the other products cut along K.
//
// Measured against the tcgen05 few-rows product (csrc/gemm_skinny.cu: TMA ring, mbarriers, tensor-memory accumulator)
// on the decode products of the 0.6B shape at 8 rows, graph of 40 launches of one product, weights streamed from HBM:
// qkv 3.57 -> 3.0 us, o_proj 3.02 -> 2.03, down_proj 3.55 -> 2.32.  Inside a decode step the gain is smaller, because
// there a product's time is mostly the wait for the kernel before: steps of 1 / 2 / 4 / 8 sequences take 0.780 / 0.773 /
// 0.898 / 0.918 ms with this kernel against 0.798 / 0.816 / 0.905 / 0.910 ms with the tcgen05 one, so the engine uses it
// up to 4 rows (`ops.ROWS8_BEST_ROWS`).  What the loads before the wait are worth shows when they are held back: with
// 6, 3 and 0 of a warp's 12 blocks of W asked for before the wait a step of 8 sequences takes 1.03, 1.11 and 1.22 ms.
//
// The reference streams weights with a GEMV kernel for one row and calls cublasGemmEx for more
// (src/backend/cuda/linear/linear.cu:22-96).
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

namespace {

constexpr int WARPS = 4;
constexpr int ROWS_PER_WARP = 16;
constexpr int KBLOCK = 32;          // k values a warp takes per pair of MMAs: 4 lanes x 8 values a row
constexpr int MAX_KB = 12;          // blocks of K per warp: 2 x 12 x 4 registers of W in flight

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 16 bytes of a weight through the read-only path.  A volatile statement: the compiler keeps it where it stands, in
// front of `griddepcontrol.wait` (an ordinary load it may move behind the wait, which is the one place it must not be).
__device__ __forceinline__ uint4 load_weight16(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// KB: 32-wide blocks of K per slice (the last slice may hold fewer values: what lies beyond K is zero)
template <int KB>
__global__ void __launch_bounds__(WARPS * 32)
gemm_rows8_kernel(float* __restrict__ out, const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ W,
                  long long ldw, int M, int N, int K, int pre) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;          // the MMA's row group and thread in the group
    const int n0 = (blockIdx.x * WARPS + warp) * ROWS_PER_WARP;
    const int k0 = blockIdx.y * KB * KBLOCK + t * 8;       // this lane's first k of the slice
    pdl_launch_dependents();
    const bool r0_live = n0 + g < N, r1_live = n0 + g + 8 < N;
    uint4 w0[KB], w1[KB];
    {
        const bf16* r0 = W + (size_t)(n0 + g) * ldw + k0;
        const bf16* r1 = r0 + (size_t)8 * ldw;
#pragma unroll
        for (int b = 0; b < KB; ++b) {
            const bool in_k = k0 + b * KBLOCK < K;          // K is a multiple of 8: a lane's 8 values are inside or outside
            w0[b] = make_uint4(0, 0, 0, 0);
            w1[b] = make_uint4(0, 0, 0, 0);
            if (b < pre) {
                if (r0_live && in_k) w0[b] = load_weight16(r0 + b * KBLOCK);
                if (r1_live && in_k) w1[b] = load_weight16(r1 + b * KBLOCK);
            }
        }
        pdl_wait();          // x comes from the kernel before
        // `pre` (a kernel argument, all blocks unless a measurement sets it otherwise) splits the loads into those
        // before and those after the wait; because the second loop might run, the first cannot be moved behind the
        // wait to save registers, which the assembler otherwise does
#pragma unroll
        for (int b = 0; b < KB; ++b) {
            const bool in_k = k0 + b * KBLOCK < K;
            if (b >= pre) {
                if (r0_live && in_k) w0[b] = load_weight16(r0 + b * KBLOCK);
                if (r1_live && in_k) w1[b] = load_weight16(r1 + b * KBLOCK);
            }
        }
    }
    if (n0 >= N) return;
    uint4 xv[KB];
    const bf16* xr = x + (size_t)g * ldx + k0;
#pragma unroll
    for (int b = 0; b < KB; ++b)
        xv[b] = (g < M && k0 + b * KBLOCK < K) ? __ldcg(reinterpret_cast<const uint4*>(xr + b * KBLOCK)) : make_uint4(0, 0, 0, 0);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int b = 0; b < KB; ++b) {
        const uint32_t a_lo[4] = {w0[b].x, w1[b].x, w0[b].y, w1[b].y};
        mma_16816(acc, a_lo, xv[b].x, xv[b].y);
        const uint32_t a_hi[4] = {w0[b].z, w1[b].z, w0[b].w, w1[b].w};
        mma_16816(acc, a_hi, xv[b].z, xv[b].w);
    }
    // acc[0], acc[1]: W row n0 + g against rows 2t, 2t + 1 of x; acc[2], acc[3]: W row n0 + g + 8
    float* o = out + (size_t)blockIdx.y * M * N;
    const int m0 = 2 * t, m1 = 2 * t + 1;
    if (m0 < M) {
        if (r0_live) o[(size_t)m0 * N + n0 + g] = acc[0];
        if (r1_live) o[(size_t)m0 * N + n0 + g + 8] = acc[2];
    }
    if (m1 < M) {
        if (r0_live) o[(size_t)m1 * N + n0 + g] = acc[1];
        if (r1_live) o[(size_t)m1 * N + n0 + g + 8] = acc[3];
    }
}

// the division as a reciprocal and a product, as in the other gated products (the exact one is a call with a slow path)
__device__ __forceinline__ float silu(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

// The gate/up product with its activation: W interleaves 16 gate rows and the 16 matching up rows.  A block owns one
// such group of 32 rows, its four warps a quarter of K each; the warps leave their sums in shared memory and the
// block writes out[m][j] = silu(gate) * up for its 16 columns.  Loads as above: all of W before the wait.  Inside a
// decode step it wins for one sequence only (0.780 -> 0.767 ms a step; with 2 and 4 sequences 0.773 -> 0.817 and
// 0.898 -> 1.015 ms: its 12.6 MB of requests, all at once as soon as the block is resident, hold up the kernels
// before it, whose own loads grow with the sequences), so the engine uses it there (`ops.ROWS8_GATED_BEST_ROWS`).
template <int KB>
__global__ void __launch_bounds__(WARPS * 32)
gemm_rows8_gated_kernel(bf16* __restrict__ out, long long ldo, const bf16* __restrict__ x, long long ldx,
                        const bf16* __restrict__ W, long long ldw, int M, int N, int K, int pre) {
    __shared__ float part[WARPS][2][16][8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 32;                        // first gate row of the group; its up rows start 16 further
    const int k0 = warp * KB * KBLOCK + t * 8;
    pdl_launch_dependents();
    uint4 wg0[KB], wg1[KB], wu0[KB], wu1[KB];
    {
        const bf16* r = W + (size_t)(n0 + g) * ldw + k0;
#pragma unroll
        for (int b = 0; b < KB; ++b) {
            const bool in_k = k0 + b * KBLOCK < K;
            const uint4 zero = make_uint4(0, 0, 0, 0);
            wg0[b] = wg1[b] = wu0[b] = wu1[b] = zero;
            if (b < pre) {
                if (in_k && n0 + g < N) wg0[b] = load_weight16(r + b * KBLOCK);
                if (in_k && n0 + g + 8 < N) wg1[b] = load_weight16(r + (size_t)8 * ldw + b * KBLOCK);
                if (in_k && n0 + g + 16 < N) wu0[b] = load_weight16(r + (size_t)16 * ldw + b * KBLOCK);
                if (in_k && n0 + g + 24 < N) wu1[b] = load_weight16(r + (size_t)24 * ldw + b * KBLOCK);
            }
        }
        pdl_wait();          // x comes from the kernel before
        // `pre` is the kernel's argument and always covers every block: the loads below never run, but because they
        // might, the ones above cannot be moved behind the wait to save registers (which the assembler otherwise does:
        // the kernel came out with 56 registers where its weights alone are 128 to 192)
#pragma unroll
        for (int b = 0; b < KB; ++b) {
            const bool in_k = k0 + b * KBLOCK < K;
            if (b >= pre) {
                if (in_k && n0 + g < N) wg0[b] = load_weight16(r + b * KBLOCK);
                if (in_k && n0 + g + 8 < N) wg1[b] = load_weight16(r + (size_t)8 * ldw + b * KBLOCK);
                if (in_k && n0 + g + 16 < N) wu0[b] = load_weight16(r + (size_t)16 * ldw + b * KBLOCK);
                if (in_k && n0 + g + 24 < N) wu1[b] = load_weight16(r + (size_t)24 * ldw + b * KBLOCK);
            }
        }
    }
    uint4 xv[KB];
    const bf16* xr = x + (size_t)g * ldx + k0;
#pragma unroll
    for (int b = 0; b < KB; ++b)
        xv[b] = (g < M && k0 + b * KBLOCK < K) ? __ldcg(reinterpret_cast<const uint4*>(xr + b * KBLOCK)) : make_uint4(0, 0, 0, 0);
    float ag[4] = {0.f, 0.f, 0.f, 0.f}, au[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int b = 0; b < KB; ++b) {
        const uint32_t g_lo[4] = {wg0[b].x, wg1[b].x, wg0[b].y, wg1[b].y}, g_hi[4] = {wg0[b].z, wg1[b].z, wg0[b].w, wg1[b].w};
        const uint32_t u_lo[4] = {wu0[b].x, wu1[b].x, wu0[b].y, wu1[b].y}, u_hi[4] = {wu0[b].z, wu1[b].z, wu0[b].w, wu1[b].w};
        mma_16816(ag, g_lo, xv[b].x, xv[b].y);
        mma_16816(au, u_lo, xv[b].x, xv[b].y);
        mma_16816(ag, g_hi, xv[b].z, xv[b].w);
        mma_16816(au, u_hi, xv[b].z, xv[b].w);
    }
    // a lane's sums: rows g and g + 8 of the group against rows 2t and 2t + 1 of x
    part[warp][0][g][2 * t] = ag[0]; part[warp][0][g][2 * t + 1] = ag[1]; part[warp][0][g + 8][2 * t] = ag[2]; part[warp][0][g + 8][2 * t + 1] = ag[3];
    part[warp][1][g][2 * t] = au[0]; part[warp][1][g][2 * t + 1] = au[1]; part[warp][1][g + 8][2 * t] = au[2]; part[warp][1][g + 8][2 * t + 1] = au[3];
    __syncthreads();
    const int r = threadIdx.x >> 3, m = threadIdx.x & 7;          // 16 rows x 8 rows of x: one value a thread
    const int col = blockIdx.x * 16 + r;
    if (m < M && n0 + 16 + r < N) {
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {          // in the order of K
            gate += part[w][0][r][m];
            up += part[w][1][r][m];
        }
        out[(size_t)m * ldo + col] = from_float<bf16>(silu(gate) * up);
    }
}

// 32-wide blocks of K per slice: the most (up to MAX_KB, in steps of 4) that still leave about 3.4 warps an SM, at
// most 8 slices (the consumer reads every slice).
int plan_blocks(int N, int K) {
    const int total_kb = ceil_div(K, KBLOCK);
    const long long want = (long long)device_sm_count() * 34 / 10;
    const long long row_groups = ceil_div(N, ROWS_PER_WARP);
    int kb = 4;
    for (int cand = MAX_KB; cand >= 4; cand -= 4) {
        if (row_groups * ceil_div(total_kb, cand) >= want) {
            kb = cand;
            break;
        }
    }
    while (kb < MAX_KB && ceil_div(total_kb, kb) > 8) kb += 4;
    return kb;
}

int g_pre_blocks = MAX_KB;      // blocks of K whose W is asked for before the wait (for measurements)

}  // namespace

LLMK_EXPORT void llmk_gemm_rows8_set_pre(int blocks) { g_pre_blocks = blocks; }

// 1 if the kernel takes this product: up to 8 rows, 16-byte aligned rows of x and W, a K of whole 16-byte pieces, and
// no more K than 8 slices of the largest size hold.
LLMK_EXPORT int llmk_gemm_rows8_usable(const void* x, const void* W, int M, int N, int K, long long ldx, long long ldw) {
    if (M <= 0 || M > 8 || N <= 0 || K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return 0;
    if (!host_aligned16(x) || !host_aligned16(W)) return 0;
    if (ceil_div(ceil_div(K, KBLOCK), MAX_KB) > 8) return 0;
    return 1;
}

// Into how many slices of K the product is cut (the first dimension of `out`).
LLMK_EXPORT int llmk_gemm_rows8_slices(int N, int K) {
    if (N <= 0 || K <= 0) return 1;
    return ceil_div(ceil_div(K, KBLOCK), plan_blocks(N, K));
}

// 1 if the gated form takes this product: as above, W's rows in groups of 16 gate and 16 up rows (N a multiple of 32),
// and a K that four warps hold in registers (at most 4 * 12 * 32).
LLMK_EXPORT int llmk_gemm_rows8_gated_usable(const void* x, const void* W, int M, int N, int K, long long ldx, long long ldw) {
    if (!llmk_gemm_rows8_usable(x, W, M, N, K, ldx, ldw)) return 0;
    return (N % 32 == 0 && ceil_div(K, KBLOCK) <= WARPS * MAX_KB) ? 1 : 0;
}

// out[M][N / 2] (bfloat16, row stride ldo) = silu(gate) * up of x W^T, W interleaving gate and up rows in groups of 16.
LLMK_EXPORT int llmk_gemm_rows8_gated(void* out, long long ldo, const void* x, const void* W, int M, int N, int K, long long ldx,
                                      long long ldw, void* stream) {
    if (!llmk_gemm_rows8_gated_usable(x, W, M, N, K, ldx, ldw))
        LLMK_FAIL("gemm_rows8_gated: not taken (M %d must be 1..8, N %d a multiple of 32, K %d a multiple of 8 and at most %d)", M, N, K,
                  WARPS * MAX_KB * KBLOCK);
    const int kb = ceil_div(ceil_div(K, KBLOCK), WARPS);
    const dim3 grid(N / 32);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
#define LAUNCH_GATED(KB_)                                                                                                       \
    e = llmk_launch(gemm_rows8_gated_kernel<KB_>, grid, dim3(WARPS * 32), 0, s, true, (bf16*)out, ldo, (const bf16*)x, ldx, \
                    (const bf16*)W, ldw, M, N, K, g_pre_blocks)
    if (kb <= 2) LAUNCH_GATED(2);
    else if (kb <= 4) LAUNCH_GATED(4);
    else if (kb <= 6) LAUNCH_GATED(6);
    else if (kb <= 8) LAUNCH_GATED(8);
    else if (kb <= 10) LAUNCH_GATED(10);
    else LAUNCH_GATED(12);
#undef LAUNCH_GATED
    LLMK_CHECK_LAUNCH_RC("gemm_rows8_gated", e);
    return LLMK_OK;
}

// out[llmk_gemm_rows8_slices(N, K)][M][N] (float32, contiguous) = the slices' partial sums.
LLMK_EXPORT int llmk_gemm_rows8(float* out, const void* x, const void* W, int M, int N, int K, long long ldx, long long ldw,
                                void* stream) {
    if (!llmk_gemm_rows8_usable(x, W, M, N, K, ldx, ldw))
        LLMK_FAIL("gemm_rows8: not taken (M %d must be 1..8, N %d, K %d a multiple of 8 and at most %d, rows 16-byte aligned)", M, N, K,
                  8 * MAX_KB * KBLOCK);
    const int kb = plan_blocks(N, K);
    const int slices = ceil_div(ceil_div(K, KBLOCK), kb);
    const dim3 grid(ceil_div(ceil_div(N, ROWS_PER_WARP), WARPS), slices);
    if (grid.x > 2147483647u / 2 || grid.y > 65535) LLMK_FAIL("gemm_rows8: grid too large");
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    switch (kb) {
        case 4: e = llmk_launch(gemm_rows8_kernel<4>, grid, dim3(WARPS * 32), 0, s, true, out, (const bf16*)x, ldx, (const bf16*)W, ldw, M, N, K, g_pre_blocks); break;
        case 8: e = llmk_launch(gemm_rows8_kernel<8>, grid, dim3(WARPS * 32), 0, s, true, out, (const bf16*)x, ldx, (const bf16*)W, ldw, M, N, K, g_pre_blocks); break;
        default: e = llmk_launch(gemm_rows8_kernel<12>, grid, dim3(WARPS * 32), 0, s, true, out, (const bf16*)x, ldx, (const bf16*)W, ldw, M, N, K, g_pre_blocks); break;
    }
    LLMK_CHECK_LAUNCH_RC("gemm_rows8", e);
    return LLMK_OK;
}
