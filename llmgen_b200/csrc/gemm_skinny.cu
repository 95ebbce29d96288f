// C[M, N] = X[M, K] * W[N, K]^T for few rows (M <= 256) in bfloat16: the weight-streaming product of
// decode steps, on the 5th-generation tensor cores with the operands swapped.
//
// With a handful of rows the product is bound by reading W once, so the kernel is shaped for
// bandwidth: a block owns 128 rows of W (they fill the 128 lanes of `tcgen05.mma`) and a slice of K;
// the rows of X, padded to MPAD in {16, 32, 64, 128, 256}, are the instruction's N.  The grid is
// (N / 128, splits): K is cut into `splits` slices so that about one block per SM streams its
// share of W through a ring of TMA stages.  A block's accumulator [128 weight rows x MPAD rows of X]
// sits in tensor memory; four warps read it back with `tcgen05.ld` and write
//   OUT_DIRECT         C[m, n]                      (splits == 1), bfloat16 or float32
//   OUT_GATED          C[m, j] = silu(gate) * up    (splits == 1), W interleaving gate and up rows in groups of 16
//   OUT_PARTIAL        P[split, m, n] float32       the consumer adds the `splits` slices in a fixed order
//   OUT_CLUSTER_GATED  C[m, j] = silu(gate) * up    the slices of K of a tile are a thread-block cluster (2 or 4
//                                                   blocks) and are added up through its shared memory
// Consumers of partial sums are the residual add + RMSNorm and the q/k-norm + rotary + cache-write
// kernels, so a split product costs no extra launch.
//
// Launched with programmatic dependent launch: barrier set-up, tensor-memory allocation and the
// first TMA loads of W (which no earlier kernel writes) run before `griddepcontrol.wait`; only the
// loads of X wait for the kernel before.
//
// Rows of W beyond N, rows of X beyond M and columns beyond K are zero-filled by TMA.  Every wait is
// bounded (tcgen05.cuh); a wait that gives up raises `*error_flag` and the block still frees its
// tensor memory.
//
// The reference uses a one-warp-per-output-row GEMV for M <= 2 and cuBLAS above
// (src/backend/cuda/linear/linear.cu:22-96); this kernel covers both ranges up to 256 rows.
#include <string.h>
#include "common.cuh"
#include "tcgen05.cuh"

LLMK_DEFINE_LAST_ERROR()

namespace {

constexpr int BW = 128;          // rows of W per block
constexpr int BK = 64;           // one 128-byte swizzle row of bfloat16
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
enum { OUT_DIRECT = 0, OUT_PARTIAL = 1, OUT_GATED = 2, OUT_CLUSTER_GATED = 5 };

// A ring stage holds a tile of W and one of X.
template <int MPAD, int STAGES>
struct Smem {
    static constexpr int W_BYTES = BW * BK * 2;
    static constexpr int X_BYTES = MPAD * BK * 2;
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 2) * 8 + 16 + 1024;  // + alignment slack
};

// the division as a reciprocal and a product: the exact one is a call with a slow path, which keeps the
// compiler from overlapping the elements of a row (measured: 9 us against 2 us for the epilogue of a tile)
__device__ __forceinline__ float silu(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

template <typename TC, int MPAD, int STAGES, int MODE>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   TC* __restrict__ C, int M, int N, int K, long long ldc, int kb_per_split, int* error_flag) {
    using L = Smem<MPAD, STAGES>;
    constexpr int TMEM_COLS = MPAD < 32 ? 32 : MPAD;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* acc_full = bars + 2 * STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BW;
    const int split = blockIdx.y;
    const int num_kb = (K + BK - 1) / BK;
    const int kb0 = split * kb_per_split;
    const int nkb = min(kb_per_split, num_kb - kb0);   // >= 1: the launcher leaves no slice empty

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(tc::smem_u32(&full[s]), 1);
            tc::mbar_init(tc::smem_u32(&empty[s]), 1);
        }
        tc::mbar_init(tc::smem_u32(acc_full), 1);
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&map_w);
        tc::prefetch_tensormap(&map_x);
    }
    if (warp == 1) {
        tc::tmem_alloc(tc::smem_u32(tmem_slot), TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            pdl_launch_dependents();   // at once: releasing the next kernel later (after the loads, after the products) was slower
            // W is written by no kernel of the step: its first loads go out before the wait.
            const int first = min(nkb, STAGES);
            for (int i = 0; i < first; ++i) {
                const uint32_t bar = tc::smem_u32(&full[i]);
                tc::mbar_expect_tx(bar, L::STAGE_BYTES);
                tc::tma_load_2d(tc::smem_u32(smem + i * L::STAGE_BYTES), &map_w, bar, (kb0 + i) * BK, n0);
            }
            pdl_wait();   // X was written by the kernel before this one
            for (int i = 0; i < first; ++i)
                tc::tma_load_2d(tc::smem_u32(smem + i * L::STAGE_BYTES + L::W_BYTES), &map_x, tc::smem_u32(&full[i]),
                                (kb0 + i) * BK, 0);
            int issued = first;
            for (int kb = first; kb < nkb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t round = kb / STAGES;
                if (!tc::mbar_wait(tc::smem_u32(&empty[s]), (round & 1) ^ 1, abort_flag)) break;
                const uint32_t bar = tc::smem_u32(&full[s]);
                tc::mbar_expect_tx(bar, L::STAGE_BYTES);
                const uint32_t dst = tc::smem_u32(smem + s * L::STAGE_BYTES);
                tc::tma_load_2d(dst, &map_w, bar, (kb0 + kb) * BK, n0);
                tc::tma_load_2d(dst + L::W_BYTES, &map_x, bar, (kb0 + kb) * BK, 0);
                issued = kb + 1;
            }
            if (*abort_flag) {
                // Let the copies that are in flight land before the block's memory is given up.
                for (int kb = max(0, issued - STAGES); kb < issued; ++kb) {
                    const unsigned long long t0 = tc::global_timer();
                    while (!tc::mbar_try_wait(tc::smem_u32(&full[kb % STAGES]), (kb / STAGES) & 1) &&
                           tc::global_timer() - t0 < tc::WAIT_LIMIT_NS) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::idesc_bf16_f32(BW, MPAD);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % STAGES;
                const uint32_t round = kb / STAGES;
                ok = tc::mbar_wait(tc::smem_u32(&full[s]), round & 1, abort_flag);
                if (!ok) break;
                tc::tc_fence_after_sync();
                const uint32_t w_addr = tc::smem_u32(smem + s * L::STAGE_BYTES);
                const uint32_t x_addr = w_addr + L::W_BYTES;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint64_t da = tc::smem_desc_sw128(w_addr + k * UMMA_K * 2);
                    const uint64_t db = tc::smem_desc_sw128(x_addr + k * UMMA_K * 2);
                    tc::mma_bf16_ss(tmem_base, da, db, idesc, (kb | k) != 0);
                }
                tc::mma_commit(tc::smem_u32(&empty[s]));
            }
            if (ok) tc::mma_commit(tc::smem_u32(acc_full));
        }
    } else {
        // Epilogue: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31; a lane is a row of W
        // (an output column), a column of tensor memory is a row of X.
        const int quarter = warp & 3;
        const int n = n0 + quarter * 32 + lane;
        const bool ok = __all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(acc_full), 0, abort_flag));
        tc::tc_fence_after_sync();
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < MPAD; c0 += 16) {
                if (c0 >= M) break;   // uniform over the block
                uint32_t r[16];
                __syncwarp();
                tc::tmem_ld_32x16_wait(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int m = c0 + i;
                    const float v = __uint_as_float(r[i]);
                    if constexpr (MODE == OUT_CLUSTER_GATED) {
                        // this block's slice of the sum, for the cluster to add up: [row of X][row of W]
                        if (m < M) reinterpret_cast<float*>(smem)[m * BW + quarter * 32 + lane] = v;
                    } else if constexpr (MODE == OUT_GATED) {
                        // lanes 0..15 hold 16 gate rows, lanes 16..31 the matching up rows
                        const float u = __shfl_down_sync(0xffffffffu, v, 16);
                        if (m < M && lane < 16 && n < N)
                            C[(size_t)m * ldc + (n0 + quarter * 32) / 2 + lane] = from_float<TC>(silu(v) * u);
                    } else if constexpr (MODE == OUT_PARTIAL) {
                        if (m < M && n < N) C[((size_t)split * M + m) * ldc + n] = from_float<TC>(v);
                    } else {
                        if (m < M && n < N) C[(size_t)m * ldc + n] = from_float<TC>(v);
                    }
                }
            }
        }
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && *abort_flag && error_flag) atomicExch(error_flag, 1);
    if constexpr (MODE == OUT_CLUSTER_GATED) {
        // The blocks of a cluster hold the slices of K of one tile.  Each left its float32 slice in its own
        // shared memory (over the TMA ring, which is idle by now).  W interleaves gate and up rows in groups of
        // 16: block r owns whole groups of 32 rows (S <= 4), adds up gate row j and up row j of each over the
        // blocks, in slice order, and writes silu(gate) * up, so the packed product never reaches memory and no
        // activation kernel follows.  Nobody leaves before all have read.
        cluster_sync_all();
        const uint32_t S = gridDim.y, rank = cluster_ctarank();
        const int pairs_per = BW / (int)S / 2;
        const uint32_t red = tc::smem_u32(smem);
        for (int idx = threadIdx.x; idx < pairs_per * M; idx += THREADS) {
            const int m = idx / pairs_per, jj = idx % pairs_per;
            const int gate_row = (int)rank * 2 * pairs_per + (jj / 16) * 32 + jj % 16;
            const uint32_t local = red + (uint32_t)(m * BW + gate_row) * 4u;
            float g = 0.f, u = 0.f;
            for (uint32_t q = 0; q < S; ++q) {
                const uint32_t remote = cluster_map_shared(local, q);
                g += cluster_ld_f32(remote);
                u += cluster_ld_f32(remote + 16u * 4u);
            }
            const int col = (n0 + gate_row) / 32 * 16 + jj % 16;
            if (n0 + gate_row + 16 < N) C[(size_t)m * ldc + col] = from_float<TC>(g / (1.0f + expf(-g)) * u);
        }
        cluster_sync_all();
    }
}

template <typename TC, int MPAD, int STAGES, int MODE>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, void* C, int M, int N, int K, long long ldc, int splits,
           int kb_per_split, int* error_flag, cudaStream_t s) {
    using L = Smem<MPAD, STAGES>;
    auto kernel = gemm_skinny_kernel<TC, MPAD, STAGES, MODE>;
    static bool configured = false;   // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) LLMK_FAIL("gemm_skinny: cannot raise shared memory to %d: %s", L::TOTAL, cudaGetErrorString(e));
        configured = true;
    }
    if constexpr (MODE == OUT_CLUSTER_GATED) {
        LLMK_CHECK_LAUNCH_RC("gemm_skinny", llmk_launch_cluster(kernel, dim3(ceil_div(N, BW), splits), dim3(THREADS), L::TOTAL, s,
                                                                true, (unsigned)splits, mw, mx, (TC*)C, M, N, K, ldc,
                                                                kb_per_split, error_flag));
    } else {
        LLMK_CHECK_LAUNCH_RC("gemm_skinny", llmk_launch(kernel, dim3(ceil_div(N, BW), splits), dim3(THREADS), L::TOTAL, s,
                                                        true, mw, mx, (TC*)C, M, N, K, ldc, kb_per_split, error_flag));
    }
    return LLMK_OK;
}

template <typename TC, int MODE>
int dispatch_rows(const CUtensorMap& mw, const void* X, void* C, int M, int N, int K, long long ldx, long long ldc,
                  int splits, int kb_per_split, int* error_flag, cudaStream_t s) {
    const int mpad = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    CUtensorMap mx;
    if (!tc_host::cached_map_bf16_2d(&mx, X, M, K, ldx, mpad))
        LLMK_FAIL("gemm_skinny: cuTensorMapEncodeTiled failed for X (M=%d K=%d ldx=%lld)", M, K, ldx);
    switch (mpad) {
        case 16: return launch<TC, 16, 6, MODE>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, s);
        case 32: return launch<TC, 32, 5, MODE>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, s);
        case 64: return launch<TC, 64, 4, MODE>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, s);
        default: break;
    }
    if constexpr (MODE == OUT_CLUSTER_GATED) {
        LLMK_FAIL("gemm_skinny: the sum over a cluster takes at most 64 rows, not %d", M);
    } else {
        if (mpad == 128) return launch<TC, 128, 6, MODE>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, s);
        return launch<TC, 256, 4, MODE>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, s);
    }
}

}  // namespace

LLMK_EXPORT int llmk_gemm_skinny_max_rows() { return 256; }

// How many slices of K suit this product: about one block per SM but at most 8 slices, at least two
// 64-wide slices of K per block, and partial sums (splits * M * N floats) no larger than W itself.
LLMK_EXPORT int llmk_gemm_skinny_splits(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 1;
    const int tiles = ceil_div(N, BW);
    const int num_kb = ceil_div(K, BK);
    int splits = (device_sm_count() + tiles / 2) / tiles;
    splits = min(splits, num_kb / 2);
    splits = min(splits, K / (2 * M));
    // at most 8: the kernel that adds the slices up pays for every one of them, and a decode step was
    // fastest with 8 (1.171 / 0.987 / 0.939 / 0.917 / 0.921 / 0.930 / 0.966 ms at batch 8 with at most
    // 2 / 4 / 6 / 8 / 10 / 12 / 16 slices), although the product alone likes 16
    splits = min(splits, 8);
    splits = max(splits, 1);
    const int per = ceil_div(num_kb, splits);
    return ceil_div(num_kb, per);
}

// Into how many slices of K a product whose slices are added up inside a thread-block cluster is
// cut: a power of two up to 16 (it is the cluster's size), about 200 blocks in all, at least two
// 64-wide slices of K per block.  1: use the plain product.
LLMK_EXPORT int llmk_gemm_skinny_cluster_splits(int M, int N, int K) {
    if (M <= 0 || M > 64 || N <= 0 || K <= 0) return 1;
    const int tiles = ceil_div(N, BW);
    const int num_kb = ceil_div(K, BK);
    int splits = 1;
    while (splits * 2 <= 16 && tiles * splits * 2 <= 200 && num_kb / (splits * 2) >= 2 && num_kb % (splits * 2) == 0) splits *= 2;
    return splits;
}

// mode 0: C[M, N] (out_dtype), splits must be 1.  mode 1: C is float32 [splits, M, ldc] partial sums.
// mode 2: gated, W interleaves gate and up rows in groups of 16, C is [M, N / 2] (out_dtype), splits 1.
// mode 5: gated as mode 2 from `splits` slices of K (2 or 4) added up inside a cluster, M <= 64.
LLMK_EXPORT int llmk_gemm_skinny(void* C, const void* X, const void* W, int M, int N, int K, long long ldx,
                                 long long ldw, long long ldc, int splits, int mode, int out_dtype, int* error_flag,
                                 void* stream) {
    if (M <= 0 || N <= 0) return LLMK_OK;
    if (M > 256) LLMK_FAIL("gemm_skinny: M=%d above 256", M);
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || !host_aligned16(X) || !host_aligned16(W))
        LLMK_FAIL("gemm_skinny: operands not usable (K=%d ldx=%lld ldw=%lld must be multiples of 8, bases 16-byte aligned)", K, ldx, ldw);
    const int num_kb = ceil_div(K, BK);
    if (splits < 1 || splits > num_kb || splits > 65535) LLMK_FAIL("gemm_skinny: %d slices for K=%d", splits, K);
    const int per = ceil_div(num_kb, splits);
    if ((splits - 1) * per >= num_kb) LLMK_FAIL("gemm_skinny: %d slices of K=%d would leave one empty", splits, K);
    if (mode != OUT_PARTIAL && mode != OUT_CLUSTER_GATED && splits != 1)
        LLMK_FAIL("gemm_skinny: a product written directly cannot be sliced (%d)", splits);
    if (mode == OUT_CLUSTER_GATED && (splits != 2 && splits != 4))
        LLMK_FAIL("gemm_skinny: the gated sum over a cluster takes 2 or 4 slices, not %d", splits);
    if (mode == OUT_CLUSTER_GATED && (N % 32 != 0 || out_dtype != LLMK_BF16 || M > 64))
        LLMK_FAIL("gemm_skinny: the gated sum over a cluster writes bfloat16, N=%d a multiple of 32, at most 64 rows", N);
    if (mode == OUT_GATED && N % 32 != 0) LLMK_FAIL("gemm_skinny: gated epilogue needs N=%d to be a multiple of 32", N);
    if (ldc < (mode == OUT_GATED || mode == OUT_CLUSTER_GATED ? N / 2 : N)) LLMK_FAIL("gemm_skinny: ldc=%lld too small", ldc);
    CUtensorMap mw;
    if (!tc_host::cached_map_bf16_2d(&mw, W, N, K, ldw, BW))
        LLMK_FAIL("gemm_skinny: cuTensorMapEncodeTiled failed for W (N=%d K=%d ldw=%lld)", N, K, ldw);
    cudaStream_t s = (cudaStream_t)stream;
    if (mode == OUT_PARTIAL) return dispatch_rows<float, OUT_PARTIAL>(mw, X, C, M, N, K, ldx, ldc, splits, per, error_flag, s);
    if (mode == OUT_GATED) {
        if (out_dtype != LLMK_BF16) LLMK_FAIL("gemm_skinny: the gated epilogue writes bfloat16");
        return dispatch_rows<bf16, OUT_GATED>(mw, X, C, M, N, K, ldx, ldc, 1, per, error_flag, s);
    }
    if (mode == OUT_CLUSTER_GATED) return dispatch_rows<bf16, OUT_CLUSTER_GATED>(mw, X, C, M, N, K, ldx, ldc, splits, per, error_flag, s);
    if (mode != OUT_DIRECT) LLMK_FAIL("gemm_skinny: unknown mode %d", mode);
    if (out_dtype == LLMK_BF16) return dispatch_rows<bf16, OUT_DIRECT>(mw, X, C, M, N, K, ldx, ldc, 1, per, error_flag, s);
    if (out_dtype == LLMK_F32) return dispatch_rows<float, OUT_DIRECT>(mw, X, C, M, N, K, ldx, ldc, 1, per, error_flag, s);
    LLMK_FAIL("gemm_skinny: unknown output dtype %d", out_dtype);
}
