// C[M, N] = X[M, K] * W[N, K]^T for few rows (M <= 256) in bfloat16: the weight-streaming product of
// decode steps, on the 5th-generation tensor cores with the operands swapped.
//
// With a handful of rows the product is bound by reading W once, so the kernel is shaped for
// bandwidth: a block owns 128 rows of W (they fill the 128 lanes of `tcgen05.mma`) and a slice of K;
// the rows of X, padded to MPAD in {16, 32, 64, 128, 256}, are the instruction's N.  The grid is
// (N / 128, splits): K is cut into `splits` slices so that about one block per SM streams its
// share of W through a ring of TMA stages.  A block's accumulator [128 weight rows x MPAD rows of X]
// sits in tensor memory; four warps read it back with `tcgen05.ld` and write
//   OUT_DIRECT   C[m, n]                      (splits == 1), bfloat16 or float32
//   OUT_GATED    C[m, j] = silu(gate) * up    (splits == 1), W interleaving gate and up rows in groups of 16
//   OUT_PARTIAL  P[split, m, n] float32       the consumer adds the `splits` slices in a fixed order
// Consumers of partial sums are the residual add + RMSNorm, the q/k-norm + rotary + cache-write
// kernel and the gated activation, so a split product costs no extra launch.
//
// Fused forms for the chain of a decoder layer at few rows (`llmk_gemm_skinny_fused`), which take
// the norm and the activation between two products out of the launch list:
//   X_NORM        the rows of X are built in shared memory by the block itself,
//                 x = resid * (1 / sqrt(sum of squares / K + eps)) * (gain + offset), the sums of squares
//                 coming in parts (one per 128 columns) from the product that wrote the residual;
//   X_GATED       x = silu(gate) * up from the partial sums of the product before;
//   X_ADDNORM     the residual add and the norm before the product, in the product: the slices of K
//                 of a tile are a thread-block cluster; each block adds the slices of the product
//                 before to the residual for its columns, the blocks exchange their shares of the
//                 rows' sums of squares through each other's shared memory, and each builds its
//                 slice of the normalised rows; the tile-0 cluster also writes the new residual (to
//                 another array than the one all read);
//   OUT_RESIDUAL  the slices are written as in OUT_PARTIAL, and the block that finishes a tile last
//                 (a ticket per tile) adds them in slice order to the float32 residual and leaves
//                 the tile's share of each row's sum of squares for the norm that follows.
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
constexpr int NUM_SMS = 148;
enum { OUT_DIRECT = 0, OUT_PARTIAL = 1, OUT_GATED = 2, OUT_CLUSTER = 3, OUT_RESIDUAL = 4, OUT_CLUSTER_GATED = 5 };
constexpr bool is_cluster_mode(int mode) { return mode == OUT_CLUSTER || mode == OUT_CLUSTER_GATED; }
enum { X_TMA = 0, X_NORM = 1, X_GATED = 2, X_ADDNORM = 3 };
constexpr int BUILDERS = 128;    // the four epilogue warps build X when it does not come through TMA
constexpr int MAX_SMEM = 227 * 1024;

// With X through TMA a ring stage holds a tile of W and one of X.  When the block builds X itself
// the ring holds W only and the block's whole slice of X, `nkb` tiles of [MPAD x 64] in the
// 128-byte swizzle, follows the barriers (two kilobytes are kept for them and the small arrays).
template <int MPAD, int STAGES, int XSRC = X_TMA, int TW = BW>
struct Smem {
    static constexpr int W_BYTES = TW * BK * 2;
    static constexpr int X_BYTES = MPAD * BK * 2;
    static constexpr int STAGE_BYTES = W_BYTES + (XSRC == X_TMA ? X_BYTES : 0);
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int XR_OFFSET = BAR_OFFSET + 2048;
    static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 2) * 8 + 16 + 1024;  // + alignment slack
    static constexpr int total(int nkb) { return XSRC == X_TMA ? TOTAL : XR_OFFSET + nkb * X_BYTES + 1024; }
};

// -DLLMK_SKINNY_TIMELINE: the blocks of tile 0 of a fused launch stamp the global timer at their
// phases (a profiling build; launches take turns over 8 records of [slices][16] stamps).
#ifdef LLMK_SKINNY_TIMELINE
__device__ unsigned long long g_skinny_tl[8 * 32 * 16];
#define TL_STAMP(slot)                                                                                  \
    do {                                                                                                \
        if (blockIdx.x == 0 && blockIdx.y < 32)                                                         \
            g_skinny_tl[(fa.tl_id * 32 + blockIdx.y) * 16 + (slot)] = tc::global_timer();                \
    } while (0)
#else
#define TL_STAMP(slot) do {} while (0)
#endif

// What the fused forms need beyond the plain product.
struct FusedArgs {
    int tl_id;                   // profiling builds: which timeline record this launch writes
    // X_NORM: x[m, k] = x_resid[m, k] * rinv[m] * (gain[k] + gain_offset), rinv from the parts of the sums of squares
    const float* x_resid;
    long long x_ld;
    const float* sq_parts;       // [n_sq_parts][M]
    int n_sq_parts;
    const float* gain;
    float eps, gain_offset;
    // X_GATED: x[m, j] = silu(g) * u, g and u the sums over `gu_splits` slices of the packed gate/up product
    const float* gu;             // [gu_splits][M][gu_ld], gate and up columns alternating in groups of `group`
    int gu_splits;
    long long gu_split_stride, gu_ld;
    int group;
    // X_ADDNORM: v = an_resid_in + the sum of `an_splits` slices of an_delta; x = v * rinv * (gain + gain_offset);
    // blocks with blockIdx.x == 0 write v to an_resid_out (not the array that is read)
    const float* an_resid_in;
    const float* an_delta;       // [an_splits][M][an_ld]
    float* an_resid_out;
    long long an_ld, an_split_stride;
    int an_splits;
    // OUT_RESIDUAL
    float* resid;                // [M][resid_ld] float32, += the product
    long long resid_ld;
    float* sq_out;               // [tiles][M]: this tile's share of sum(resid[m, :]^2)
    int* tickets;                // [tiles], zero between launches
};

// the division as a reciprocal and a product: the exact one is a call with a slow path, which keeps the
// compiler from overlapping the elements of a row (measured: 9 us against 2 us for the epilogue of a tile)
__device__ __forceinline__ float silu(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

__device__ __forceinline__ void builders_sync() { asm volatile("bar.sync 1, %0;" ::"n"(BUILDERS) : "memory"); }

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Address of the 16-byte chunk `chunk` (8 bfloat16) of row `m` in tile `kb` of the block's slice of
// X: rows of 128 bytes, the chunk index XORed with the row's index in its group of 8, which is
// where TMA's 128-byte swizzle would have put it.
template <int MPAD>
__device__ __forceinline__ uint32_t x_chunk_addr(uint32_t xr, int kb, int m, int chunk) {
    return xr + (uint32_t)kb * (MPAD * 128) + (uint32_t)m * 128 + (uint32_t)((chunk ^ (m & 7)) << 4);
}

// TW: rows of W per block, 128 or 64.  With 64 the accumulator lies in lanes 0..15 of each warp's 32
// lanes of tensor memory (row m of the tile in lane 32 * (m / 16) + m % 16), and a product of few
// tiles fills twice as many SMs; only the forms that store their accumulator directly take it.
template <typename TC, int MPAD, int STAGES, int MODE, int XSRC = X_TMA, int TW = BW>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   TC* __restrict__ C, int M, int N, int K, long long ldc, int kb_per_split, int* error_flag,
                   const FusedArgs fa) {
    using L = Smem<MPAD, STAGES, XSRC, TW>;
    static_assert(TW == BW || (TW == 64 && XSRC == X_TMA && (MODE == OUT_PARTIAL || MODE == OUT_DIRECT)),
                  "64-row tiles: plain operands, accumulator stored directly");
    constexpr int TMEM_COLS = MPAD < 32 ? 32 : MPAD;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* acc_full = bars + 2 * STAGES;
    uint64_t* x_ready = bars + 2 * STAGES + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* last_slot = reinterpret_cast<int*>(tmem_slot + 2);           // is this block the last of its tile?
    float* rinv_s = reinterpret_cast<float*>(tmem_slot + 4);          // [MPAD] for X_NORM (MPAD <= 64 there)
    // X_ADDNORM (MPAD = 16): this block's shares of the sums of squares per warp-wide segment, and the
    // shares of every block of the cluster, pushed there by their owners
    uint64_t* sq_ready = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET + 384);
    float* sq_seg = reinterpret_cast<float*>(smem + L::BAR_OFFSET + 400);          // [4 segments][16 rows] ... 256 bytes
    float* sq_all = reinterpret_cast<float*>(smem + L::BAR_OFFSET + 400 + 256);    // [8 blocks][16 rows] ... 512 bytes

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TW;
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
        tc::mbar_init(tc::smem_u32(x_ready), BUILDERS);
        if constexpr (XSRC == X_ADDNORM) tc::mbar_init(tc::smem_u32(sq_ready), gridDim.y);   // one arrival per block of the cluster
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&map_w);
        if constexpr (XSRC == X_TMA) tc::prefetch_tensormap(&map_x);
    }
    if (warp == 1) {
        tc::tmem_alloc(tc::smem_u32(tmem_slot), TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    if constexpr (XSRC == X_ADDNORM) {
        __syncwarp();
        cluster_sync_all();      // every block's barriers exist before another block arrives on them
    } else {
        __syncthreads();
    }
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            TL_STAMP(0);
            pdl_launch_dependents();   // at once: releasing the next kernel later (after the loads, after the products) was slower
            // W is written by no kernel of the step: its first loads go out before the wait.
            const int first = min(nkb, STAGES);
            for (int i = 0; i < first; ++i) {
                const uint32_t bar = tc::smem_u32(&full[i]);
                tc::mbar_expect_tx(bar, L::STAGE_BYTES);
                tc::tma_load_2d(tc::smem_u32(smem + i * L::STAGE_BYTES), &map_w, bar, (kb0 + i) * BK, n0);
            }
            if constexpr (XSRC == X_TMA) {
                pdl_wait();   // X was written by the kernel before this one
                for (int i = 0; i < first; ++i)
                    tc::tma_load_2d(tc::smem_u32(smem + i * L::STAGE_BYTES + L::W_BYTES), &map_x, tc::smem_u32(&full[i]),
                                    (kb0 + i) * BK, 0);
            }
            int issued = first;
            for (int kb = first; kb < nkb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t round = kb / STAGES;
                if (!tc::mbar_wait(tc::smem_u32(&empty[s]), (round & 1) ^ 1, abort_flag)) break;
                const uint32_t bar = tc::smem_u32(&full[s]);
                tc::mbar_expect_tx(bar, L::STAGE_BYTES);
                const uint32_t dst = tc::smem_u32(smem + s * L::STAGE_BYTES);
                tc::tma_load_2d(dst, &map_w, bar, (kb0 + kb) * BK, n0);
                if constexpr (XSRC == X_TMA) tc::tma_load_2d(dst + L::W_BYTES, &map_x, bar, (kb0 + kb) * BK, 0);
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
            constexpr uint32_t idesc = tc::idesc_bf16_f32(TW, MPAD);
            bool ok = true;
            if constexpr (XSRC != X_TMA) ok = tc::mbar_wait(tc::smem_u32(x_ready), 0, abort_flag);
            TL_STAMP(4);
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % STAGES;
                const uint32_t round = kb / STAGES;
                ok = tc::mbar_wait(tc::smem_u32(&full[s]), round & 1, abort_flag);
                if (!ok) break;
                tc::tc_fence_after_sync();
                const uint32_t w_addr = tc::smem_u32(smem + s * L::STAGE_BYTES);
                const uint32_t x_addr = XSRC == X_TMA ? w_addr + L::W_BYTES
                                                      : tc::smem_u32(smem + L::XR_OFFSET) + (uint32_t)kb * L::X_BYTES;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint64_t da = tc::smem_desc_sw128(w_addr + k * UMMA_K * 2);
                    const uint64_t db = tc::smem_desc_sw128(x_addr + k * UMMA_K * 2);
                    tc::mma_bf16_ss(tmem_base, da, db, idesc, (kb | k) != 0);
                }
                tc::mma_commit(tc::smem_u32(&empty[s]));
            }
            if (ok) tc::mma_commit(tc::smem_u32(acc_full));
            TL_STAMP(5);
        }
    } else {
        // Epilogue: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31; a lane is a row of W
        // (an output column), a column of tensor memory is a row of X.
        const int quarter = warp & 3;
        const int n = TW == BW || lane < TW / 4 ? n0 + quarter * (TW / 4) + lane : N;   // N: a lane without a row
        const int tid = threadIdx.x - 64;        // 0 .. BUILDERS - 1
        if constexpr (XSRC != X_TMA) {
            // Build this block's slice of X: columns [kb0 * 64, (kb0 + nkb) * 64) of rows 0 .. MPAD - 1.
            const uint32_t xr = tc::smem_u32(smem + L::XR_OFFSET);
            const int chunks = nkb * (BK / 8);                      // 16-byte chunks per row
            for (int c = tid; c < (MPAD - M) * chunks; c += BUILDERS)   // rows beyond M: zeros, before the wait
                st_shared_v4(x_chunk_addr<MPAD>(xr, (c % chunks) / 8, M + c / chunks, (c % chunks) % 8), 0u, 0u, 0u, 0u);
            pdl_wait();
            if (tid == 0) TL_STAMP(1);
            if constexpr (XSRC == X_ADDNORM) {
                // v = residual + slices for this block's columns (two 16-byte chunks of a row per thread and
                // round, so that a warp's 32 chunks lie in one row: `chunks` is a multiple of 32)
                constexpr int MAXR = 4;                              // rounds: M * chunks <= 4 * 2 * BUILDERS
                float v[MAXR][2][8];
                const int total = M * chunks;
                const uint32_t S = gridDim.y, rank = cluster_ctarank();
#pragma unroll
                for (int rd = 0; rd < MAXR; ++rd) {
                    if (rd * 2 * BUILDERS >= total) break;
                    float4 t[2][2];
                    const float* src[2];
                    bool live[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int c = rd * 2 * BUILDERS + h * BUILDERS + tid;
                        live[h] = c < total;
                        const int m = live[h] ? c / chunks : 0, k = (kb0 * (BK / 8) + (live[h] ? c % chunks : 0)) * 8;
                        src[h] = fa.an_delta + (size_t)m * fa.an_ld + k;
                        const float* rp = fa.an_resid_in + (size_t)m * fa.an_ld + k;
                        t[h][0] = live[h] ? __ldcg(reinterpret_cast<const float4*>(rp)) : make_float4(0.f, 0.f, 0.f, 0.f);
                        t[h][1] = live[h] ? __ldcg(reinterpret_cast<const float4*>(rp + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    float acc[2][8];
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[h][i] = 0.f;
                    for (int s0 = 0; s0 < fa.an_splits; s0 += 4) {
                        float4 d[2][4][2];
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const bool on = live[h] && s0 + u < fa.an_splits;
                                const float* q = src[h] + (size_t)(s0 + u) * fa.an_split_stride;
                                d[h][u][0] = on ? __ldcg(reinterpret_cast<const float4*>(q)) : make_float4(0.f, 0.f, 0.f, 0.f);
                                d[h][u][1] = on ? __ldcg(reinterpret_cast<const float4*>(q + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                acc[h][0] += d[h][u][0].x; acc[h][1] += d[h][u][0].y; acc[h][2] += d[h][u][0].z; acc[h][3] += d[h][u][0].w;
                                acc[h][4] += d[h][u][1].x; acc[h][5] += d[h][u][1].y; acc[h][6] += d[h][u][1].z; acc[h][7] += d[h][u][1].w;
                            }
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        v[rd][h][0] = t[h][0].x + acc[h][0]; v[rd][h][1] = t[h][0].y + acc[h][1];
                        v[rd][h][2] = t[h][0].z + acc[h][2]; v[rd][h][3] = t[h][0].w + acc[h][3];
                        v[rd][h][4] = t[h][1].x + acc[h][4]; v[rd][h][5] = t[h][1].y + acc[h][5];
                        v[rd][h][6] = t[h][1].z + acc[h][6]; v[rd][h][7] = t[h][1].w + acc[h][7];
                        float sq = 0.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) sq += v[rd][h][i] * v[rd][h][i];
                        sq = warp_sum(sq);                           // a warp's 32 chunks: one segment of one row
                        const int c0 = rd * 2 * BUILDERS + h * BUILDERS + (tid & ~31);
                        if (lane == 0 && c0 < total) sq_seg[((c0 % chunks) / 32) * 16 + c0 / chunks] = sq;
                    }
                }
                builders_sync();
                // one thread per row: the row's share of this block, pushed into every block of the cluster
                if (tid < M) {
                    float sq = 0.f;
                    for (int sg = 0; sg < chunks / 32; ++sg) sq += sq_seg[sg * 16 + tid];
                    const uint32_t mine = tc::smem_u32(sq_all + rank * 16 + tid);
                    for (uint32_t q = 0; q < S; ++q)
                        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_map_shared(mine, q)), "f"(sq) : "memory");
                    asm volatile("fence.acq_rel.cluster;" ::: "memory");
                }
                __syncwarp();
                if (tid == 0)
                    for (uint32_t q = 0; q < S; ++q) tc::mbar_arrive_cluster(cluster_map_shared(tc::smem_u32(sq_ready), q));
                const bool got = tc::mbar_wait(tc::smem_u32(sq_ready), 0, abort_flag);
                asm volatile("fence.acq_rel.cluster;" ::: "memory");
                if (tid < M) {
                    float ss = 0.f;
                    for (uint32_t q = 0; q < S; ++q) ss += sq_all[q * 16 + tid];
                    rinv_s[tid] = got ? 1.0f / sqrtf(ss / (float)K + fa.eps) : 0.f;
                }
                builders_sync();
#pragma unroll
                for (int rd = 0; rd < MAXR; ++rd) {
                    if (rd * 2 * BUILDERS >= total) break;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int c = rd * 2 * BUILDERS + h * BUILDERS + tid;
                        if (c >= total) continue;
                        const int m = c / chunks, j = c % chunks, k = (kb0 * (BK / 8) + j) * 8;
                        const float4 ga = *reinterpret_cast<const float4*>(fa.gain + k);
                        const float4 gb = *reinterpret_cast<const float4*>(fa.gain + k + 4);
                        const float r = rinv_s[m], o = fa.gain_offset;
                        const float* x = v[rd][h];
                        st_shared_v4(x_chunk_addr<MPAD>(xr, j / 8, m, j % 8),
                                     pack_bf16x2(x[0] * r * (ga.x + o), x[1] * r * (ga.y + o)),
                                     pack_bf16x2(x[2] * r * (ga.z + o), x[3] * r * (ga.w + o)),
                                     pack_bf16x2(x[4] * r * (gb.x + o), x[5] * r * (gb.y + o)),
                                     pack_bf16x2(x[6] * r * (gb.z + o), x[7] * r * (gb.w + o)));
                        if (blockIdx.x == 0) {
                            float* wp = fa.an_resid_out + (size_t)m * fa.an_ld + k;
                            *reinterpret_cast<float4*>(wp) = make_float4(x[0], x[1], x[2], x[3]);
                            *reinterpret_cast<float4*>(wp + 4) = make_float4(x[4], x[5], x[6], x[7]);
                        }
                    }
                }
            } else if constexpr (XSRC == X_NORM) {
                if (tid < M) {
                    float ss = 0.f;
                    for (int p0 = 0; p0 < fa.n_sq_parts; p0 += 8) {
                        float t[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) t[u] = p0 + u < fa.n_sq_parts ? __ldcg(fa.sq_parts + (size_t)(p0 + u) * M + tid) : 0.f;
#pragma unroll
                        for (int u = 0; u < 8; ++u) ss += t[u];
                    }
                    rinv_s[tid] = 1.0f / sqrtf(ss / (float)K + fa.eps);
                }
                // the loads of the first chunk go out before the barrier
                float4 a[2], b[2], ga[2], gb[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int c = tid + u * BUILDERS;
                    const int k = (kb0 * (BK / 8) + c % chunks) * 8;
                    const bool live = c < M * chunks && k < K;
                    const float* src = fa.x_resid + (size_t)(c / chunks) * fa.x_ld + k;
                    a[u] = live ? __ldcg(reinterpret_cast<const float4*>(src)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    b[u] = live ? __ldcg(reinterpret_cast<const float4*>(src + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    ga[u] = live ? *reinterpret_cast<const float4*>(fa.gain + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                    gb[u] = live ? *reinterpret_cast<const float4*>(fa.gain + k + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                builders_sync();
                for (int c0 = 0; c0 < M * chunks; c0 += 2 * BUILDERS) {
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int c = c0 + tid + u * BUILDERS;
                        if (c >= M * chunks) continue;
                        const int m = c / chunks, j = c % chunks;
                        if (c0 > 0) {
                            const int k = (kb0 * (BK / 8) + j) * 8;
                            const bool live = k < K;
                            const float* src = fa.x_resid + (size_t)m * fa.x_ld + k;
                            a[u] = live ? __ldcg(reinterpret_cast<const float4*>(src)) : make_float4(0.f, 0.f, 0.f, 0.f);
                            b[u] = live ? __ldcg(reinterpret_cast<const float4*>(src + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
                            ga[u] = live ? *reinterpret_cast<const float4*>(fa.gain + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                            gb[u] = live ? *reinterpret_cast<const float4*>(fa.gain + k + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                        const float r = rinv_s[m], o = fa.gain_offset;
                        st_shared_v4(x_chunk_addr<MPAD>(xr, j / 8, m, j % 8),
                                     pack_bf16x2(a[u].x * r * (ga[u].x + o), a[u].y * r * (ga[u].y + o)),
                                     pack_bf16x2(a[u].z * r * (ga[u].z + o), a[u].w * r * (ga[u].w + o)),
                                     pack_bf16x2(b[u].x * r * (gb[u].x + o), b[u].y * r * (gb[u].y + o)),
                                     pack_bf16x2(b[u].z * r * (gb[u].z + o), b[u].w * r * (gb[u].w + o)));
                    }
                }
            } else {
                // silu(gate) * up from the partial sums; the 8 columns of a chunk lie in one group.  Two
                // chunks and four slices at a time keep enough loads in flight: the block waits for this.
                for (int c0 = 0; c0 < M * chunks; c0 += 2 * BUILDERS) {
                    float g[2][8], up[2][8];
                    const float* base[2];
                    bool live[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int c = c0 + tid + h * BUILDERS;
                        const int col = (kb0 * (BK / 8) + c % chunks) * 8;
                        live[h] = c < M * chunks && col < K;
                        base[h] = fa.gu + (size_t)(live[h] ? c / chunks : 0) * fa.gu_ld +
                                  (live[h] ? 2 * fa.group * (col / fa.group) + col % fa.group : 0);
#pragma unroll
                        for (int i = 0; i < 8; ++i) g[h][i] = up[h][i] = 0.f;
                    }
                    for (int sp0 = 0; sp0 < fa.gu_splits; sp0 += 4) {
                        float4 t[2][4][4];
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const bool on = live[h] && sp0 + u < fa.gu_splits;
                                const float* q = base[h] + (size_t)(sp0 + u) * fa.gu_split_stride;
                                const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
                                t[h][u][0] = on ? __ldcg(reinterpret_cast<const float4*>(q)) : z;
                                t[h][u][1] = on ? __ldcg(reinterpret_cast<const float4*>(q + 4)) : z;
                                t[h][u][2] = on ? __ldcg(reinterpret_cast<const float4*>(q + fa.group)) : z;
                                t[h][u][3] = on ? __ldcg(reinterpret_cast<const float4*>(q + fa.group + 4)) : z;
                            }
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                g[h][0] += t[h][u][0].x; g[h][1] += t[h][u][0].y; g[h][2] += t[h][u][0].z; g[h][3] += t[h][u][0].w;
                                g[h][4] += t[h][u][1].x; g[h][5] += t[h][u][1].y; g[h][6] += t[h][u][1].z; g[h][7] += t[h][u][1].w;
                                up[h][0] += t[h][u][2].x; up[h][1] += t[h][u][2].y; up[h][2] += t[h][u][2].z; up[h][3] += t[h][u][2].w;
                                up[h][4] += t[h][u][3].x; up[h][5] += t[h][u][3].y; up[h][6] += t[h][u][3].z; up[h][7] += t[h][u][3].w;
                            }
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int c = c0 + tid + h * BUILDERS;
                        if (c >= M * chunks) continue;
                        float x[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) x[i] = g[h][i] / (1.0f + expf(-g[h][i])) * up[h][i];
                        st_shared_v4(x_chunk_addr<MPAD>(xr, (c % chunks) / 8, c / chunks, (c % chunks) % 8), pack_bf16x2(x[0], x[1]),
                                     pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
                    }
                }
            }
            if (tid == 0) TL_STAMP(2);
            tc::fence_proxy_async();          // the tensor core reads what these threads wrote
            tc::mbar_arrive(tc::smem_u32(x_ready));
            if (tid == 0) TL_STAMP(3);
        } else if constexpr (MODE == OUT_RESIDUAL) {
            pdl_wait();                       // the residual is written by kernels before this one
        }
        const bool ok = __all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(acc_full), 0, abort_flag));
        tc::tc_fence_after_sync();
        if (tid == 0) TL_STAMP(6);
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
                    if constexpr (is_cluster_mode(MODE)) {
                        // this block's slice of the sum, for the cluster to add up: [row of X][row of W]
                        if (m < M) reinterpret_cast<float*>(smem)[m * BW + quarter * 32 + lane] = v;
                    } else if constexpr (MODE == OUT_GATED) {
                        // lanes 0..15 hold 16 gate rows, lanes 16..31 the matching up rows
                        const float u = __shfl_down_sync(0xffffffffu, v, 16);
                        if (m < M && lane < 16 && n < N)
                            C[(size_t)m * ldc + (n0 + quarter * 32) / 2 + lane] = from_float<TC>(silu(v) * u);
                    } else if constexpr (MODE == OUT_PARTIAL || MODE == OUT_RESIDUAL) {
                        if (m < M && n < N) C[((size_t)split * M + m) * ldc + n] = from_float<TC>(v);
                    } else {
                        if (m < M && n < N) C[(size_t)m * ldc + n] = from_float<TC>(v);
                    }
                }
            }
        }
        if constexpr (MODE == OUT_RESIDUAL) {
            // The block that finishes its tile last adds the slices, in slice order, to the residual.
            if (tid == 0) TL_STAMP(7);
            __threadfence();
            builders_sync();
            if (tid == 0) TL_STAMP(8);
            if (tid == 0) *last_slot = ok && atomicAdd(fa.tickets + blockIdx.x, 1) == (int)gridDim.y - 1;
            builders_sync();
            if (tid == 0) TL_STAMP(9);
            if (*last_slot) {
                __threadfence();
                const int S = (int)gridDim.y;
                const float* P = reinterpret_cast<const float*>(C);
                // a warp takes a row: 32 lanes x 4 columns are the tile's 128 columns.  Two rows and
                // sixteen slices at a time: this block works alone now, so its loads must overlap.
                const int nn = n0 + lane * 4;
                const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int m0 = tid >> 5; m0 < M; m0 += 2 * (BUILDERS / 32)) {
                    float4 acc[2] = {z, z}, r[2];
                    bool live[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int m = m0 + h * (BUILDERS / 32);
                        live[h] = m < M && nn < N;
                        r[h] = live[h] ? __ldcg(reinterpret_cast<const float4*>(fa.resid + (size_t)m * fa.resid_ld + nn)) : z;
                    }
                    for (int s0 = 0; s0 < S; s0 += 16) {
                        float4 t[2][16];
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int u = 0; u < 16; ++u)
                                t[h][u] = live[h] && s0 + u < S
                                              ? __ldcg(reinterpret_cast<const float4*>(
                                                    P + ((size_t)(s0 + u) * M + m0 + h * (BUILDERS / 32)) * ldc + nn))
                                              : z;
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int u = 0; u < 16; ++u) {
                                acc[h].x += t[h][u].x; acc[h].y += t[h][u].y; acc[h].z += t[h][u].z; acc[h].w += t[h][u].w;
                            }
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int m = m0 + h * (BUILDERS / 32);
                        if (m >= M) continue;                       // uniform over the warp
                        float sq = 0.f;
                        if (live[h]) {
                            const float4 v = make_float4(acc[h].x + r[h].x, acc[h].y + r[h].y, acc[h].z + r[h].z, acc[h].w + r[h].w);
                            *reinterpret_cast<float4*>(fa.resid + (size_t)m * fa.resid_ld + nn) = v;
                            sq = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                        }
                        sq = warp_sum(sq);
                        if (lane == 0) fa.sq_out[(size_t)blockIdx.x * M + m] = sq;
                    }
                }
                if (tid == 0) TL_STAMP(10);
                if (tid == 0) fa.tickets[blockIdx.x] = 0;      // ready for the next launch
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
        // As below, and W interleaves gate and up rows in groups of 16: block r owns whole groups of 32
        // rows (S <= 4), adds up gate row j and up row j of each and writes silu(gate) * up, so the packed
        // product never reaches memory and no activation kernel follows.
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
    if constexpr (MODE == OUT_CLUSTER) {
        // The blocks of a cluster hold the slices of K of one tile.  Each left its float32 slice in its
        // own shared memory (over the TMA ring, which is idle by now); block r now adds up, in slice
        // order, rows [r, r + 1) * 128 / S of W for every row of X, reading the other blocks' shared
        // memory, and writes the finished values.  Nobody leaves before all have read.
        cluster_sync_all();
        const uint32_t S = gridDim.y, rank = cluster_ctarank();
        const int rows_per = BW / (int)S;
        const uint32_t red = tc::smem_u32(smem);
        for (int idx = threadIdx.x; idx < rows_per * M; idx += THREADS) {
            const int m = idx / rows_per, rr = (int)rank * rows_per + idx % rows_per;
            const uint32_t local = red + (uint32_t)(m * BW + rr) * 4u;
            float acc = 0.f;
            for (uint32_t q = 0; q < S; ++q) acc += cluster_ld_f32(cluster_map_shared(local, q));
            const int n = n0 + rr;
            if (n < N) C[(size_t)m * ldc + n] = from_float<TC>(acc);
        }
        cluster_sync_all();
    }
}

template <typename TC, int MPAD, int STAGES, int MODE, int TW = BW>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, void* C, int M, int N, int K, long long ldc, int splits,
           int kb_per_split, int* error_flag, cudaStream_t s) {
    using L = Smem<MPAD, STAGES, X_TMA, TW>;
    auto kernel = gemm_skinny_kernel<TC, MPAD, STAGES, MODE, X_TMA, TW>;
    static bool configured = false;   // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) LLMK_FAIL("gemm_skinny: cannot raise shared memory to %d: %s", L::TOTAL, cudaGetErrorString(e));
        configured = true;
    }
    if constexpr (is_cluster_mode(MODE)) {
        static bool wide_ok = false;
        if (splits > 8 && !wide_ok) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            if (e != cudaSuccess) LLMK_FAIL("gemm_skinny: clusters of %d blocks are not allowed: %s", splits, cudaGetErrorString(e));
            wide_ok = true;
        }
        LLMK_CHECK_LAUNCH_RC("gemm_skinny", llmk_launch_cluster(kernel, dim3(ceil_div(N, BW), splits), dim3(THREADS), L::TOTAL, s,
                                                                true, (unsigned)splits, mw, mx, (TC*)C, M, N, K, ldc,
                                                                kb_per_split, error_flag, FusedArgs{}));
    } else {
        LLMK_CHECK_LAUNCH_RC("gemm_skinny", llmk_launch(kernel, dim3(ceil_div(N, TW), splits), dim3(THREADS), L::TOTAL, s,
                                                        true, mw, mx, (TC*)C, M, N, K, ldc, kb_per_split, error_flag, FusedArgs{}));
    }
    return LLMK_OK;
}

template <int MPAD, int STAGES, int MODE, int XSRC, typename TC = float>
int launch_fused(const CUtensorMap& mw, const CUtensorMap& mx, TC* C, int M, int N, int K, long long ldc, int splits,
                 int kb_per_split, int* error_flag, const FusedArgs& fa, cudaStream_t s) {
    using L = Smem<MPAD, STAGES, XSRC>;
    auto kernel = gemm_skinny_kernel<TC, MPAD, STAGES, MODE, XSRC>;
    const int bytes = L::total(kb_per_split);
    if (bytes > MAX_SMEM)
        LLMK_FAIL("gemm_skinny_fused: %d rows x %d columns of X need %d bytes of shared memory (limit %d)", MPAD,
                  kb_per_split * BK, bytes, MAX_SMEM);
    static int configured = 0;   // per instantiation: the largest size asked for so far
    if (bytes > configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) LLMK_FAIL("gemm_skinny_fused: cannot raise shared memory to %d: %s", bytes, cudaGetErrorString(e));
        configured = bytes;
    }
    if constexpr (XSRC == X_ADDNORM || is_cluster_mode(MODE)) {
        // the slices of K of a tile are one thread-block cluster
        LLMK_CHECK_LAUNCH_RC("gemm_skinny_fused", llmk_launch_cluster(kernel, dim3(ceil_div(N, BW), splits), dim3(THREADS),
                                                                      (size_t)bytes, s, true, (unsigned)splits, mw, mx, C, M, N, K,
                                                                      ldc, kb_per_split, error_flag, fa));
    } else {
        LLMK_CHECK_LAUNCH_RC("gemm_skinny_fused", llmk_launch(kernel, dim3(ceil_div(N, BW), splits), dim3(THREADS), (size_t)bytes, s,
                                                              true, mw, mx, C, M, N, K, ldc, kb_per_split, error_flag, fa));
    }
    return LLMK_OK;
}

template <int MODE, int XSRC>
int dispatch_fused(const CUtensorMap& mw, const CUtensorMap& mx, float* C, int M, int N, int K, long long ldc, int splits,
                   int kb_per_split, int* error_flag, const FusedArgs& fa, cudaStream_t s) {
    if (M <= 16) return launch_fused<16, 6, MODE, XSRC>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, fa, s);
    if (M <= 32) return launch_fused<32, 5, MODE, XSRC>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, fa, s);
    return launch_fused<64, 4, MODE, XSRC>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, fa, s);
}

template <typename TC, int MODE>
int dispatch_rows(const CUtensorMap& mw, const void* X, void* C, int M, int N, int K, long long ldx, long long ldc,
                  int splits, int kb_per_split, int* error_flag, cudaStream_t s, bool half_tiles = false) {
    const int mpad = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    CUtensorMap mx;
    if (!tc_host::cached_map_bf16_2d(&mx, X, M, K, ldx, mpad))
        LLMK_FAIL("gemm_skinny: cuTensorMapEncodeTiled failed for X (M=%d K=%d ldx=%lld)", M, K, ldx);
    if constexpr (MODE == OUT_PARTIAL) {
        if (half_tiles) {            // `mw` then has boxes of 64 rows
            switch (mpad) {
                case 16: return launch<TC, 16, 6, MODE, 64>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, s);
                case 32: return launch<TC, 32, 5, MODE, 64>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, s);
                case 64: return launch<TC, 64, 4, MODE, 64>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, s);
                default: LLMK_FAIL("gemm_skinny: 64-row tiles take at most 64 rows of X, not %d", M);
            }
        }
    }
    switch (mpad) {
        case 16: return launch<TC, 16, 6, MODE>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, s);
        case 32: return launch<TC, 32, 5, MODE>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, s);
        case 64: return launch<TC, 64, 4, MODE>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, s);
        default: break;
    }
    if constexpr (is_cluster_mode(MODE)) {
        LLMK_FAIL("gemm_skinny: the sum over a cluster takes at most 64 rows, not %d", M);
    } else {
        if (mpad == 128) return launch<TC, 128, 6, MODE>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, s);
        return launch<TC, 256, 4, MODE>(mw, mx, C, M, N, K, ldc, splits, kb_per_split, error_flag, s);
    }
}

}  // namespace

LLMK_EXPORT int llmk_gemm_skinny_max_rows() { return 256; }

// Tiles of 64 rows of W for partial sums of products with few tiles: off unless LLMGEN_SKINNY_TILES=64
// is in the environment.  Twice the blocks (128 instead of 64 for a [1024, K] matrix in 8 slices), yet a
// decode step at batch 8 took 0.925 ms with them and 0.910 ms without: the blocks' fixed cost counts
// for more than the SMs left idle.
static bool g_half_tiles = [] { const char* v = getenv("LLMGEN_SKINNY_TILES"); return v && strcmp(v, "64") == 0; }();
// 0: tiles of 128 rows everywhere; 1: 64-row tiles where 128-row tiles leave half the SMs without a block.
LLMK_EXPORT void llmk_gemm_skinny_set_half_tiles(int on) { g_half_tiles = on != 0; }

// How many slices of K suit this product: about one block per SM but at most 8 slices, at least two
// 64-wide slices of K per block, and partial sums (splits * M * N floats) no larger than W itself.
LLMK_EXPORT int llmk_gemm_skinny_splits(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 1;
    const int tiles = ceil_div(N, BW);
    const int num_kb = ceil_div(K, BK);
    int splits = (NUM_SMS + tiles / 2) / tiles;
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
// mode 3: C[M, N] (out_dtype) from `splits` slices of K (2, 4, 8 or 16) added up inside a cluster, M <= 64.
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
    if (mode != OUT_PARTIAL && !is_cluster_mode(mode) && splits != 1)
        LLMK_FAIL("gemm_skinny: a product written directly cannot be sliced (%d)", splits);
    if (mode == OUT_CLUSTER_GATED && (splits != 2 && splits != 4))
        LLMK_FAIL("gemm_skinny: the gated sum over a cluster takes 2 or 4 slices, not %d", splits);
    if (mode == OUT_CLUSTER_GATED && (N % 32 != 0 || out_dtype != LLMK_BF16 || M > 64))
        LLMK_FAIL("gemm_skinny: the gated sum over a cluster writes bfloat16, N=%d a multiple of 32, at most 64 rows", N);
    if (mode == OUT_CLUSTER && (splits < 2 || splits > 16 || (splits & (splits - 1)) != 0 || M > 64))
        LLMK_FAIL("gemm_skinny: a cluster adds up 2, 4, 8 or 16 slices of at most 64 rows (%d slices, %d rows)", splits, M);
    if (mode == OUT_GATED && N % 32 != 0) LLMK_FAIL("gemm_skinny: gated epilogue needs N=%d to be a multiple of 32", N);
    if (ldc < (mode == OUT_GATED || mode == OUT_CLUSTER_GATED ? N / 2 : N)) LLMK_FAIL("gemm_skinny: ldc=%lld too small", ldc);
    // Partial sums of a product with so few tiles that half the SMs would idle: tiles of 64 rows of W.
    const bool half_tiles = mode == OUT_PARTIAL && g_half_tiles && M <= 64 && ceil_div(N, BW) * splits * 2 <= NUM_SMS;
    CUtensorMap mw;
    if (!tc_host::cached_map_bf16_2d(&mw, W, N, K, ldw, half_tiles ? 64 : BW))
        LLMK_FAIL("gemm_skinny: cuTensorMapEncodeTiled failed for W (N=%d K=%d ldw=%lld)", N, K, ldw);
    cudaStream_t s = (cudaStream_t)stream;
    if (mode == OUT_PARTIAL)
        return dispatch_rows<float, OUT_PARTIAL>(mw, X, C, M, N, K, ldx, ldc, splits, per, error_flag, s, half_tiles);
    if (mode == OUT_GATED) {
        if (out_dtype != LLMK_BF16) LLMK_FAIL("gemm_skinny: the gated epilogue writes bfloat16");
        return dispatch_rows<bf16, OUT_GATED>(mw, X, C, M, N, K, ldx, ldc, 1, per, error_flag, s);
    }
    if (mode == OUT_CLUSTER_GATED) return dispatch_rows<bf16, OUT_CLUSTER_GATED>(mw, X, C, M, N, K, ldx, ldc, splits, per, error_flag, s);
    if (mode == OUT_CLUSTER) {
        if (out_dtype == LLMK_BF16) return dispatch_rows<bf16, OUT_CLUSTER>(mw, X, C, M, N, K, ldx, ldc, splits, per, error_flag, s);
        if (out_dtype == LLMK_F32) return dispatch_rows<float, OUT_CLUSTER>(mw, X, C, M, N, K, ldx, ldc, splits, per, error_flag, s);
        LLMK_FAIL("gemm_skinny: unknown output dtype %d", out_dtype);
    }
    if (mode != OUT_DIRECT) LLMK_FAIL("gemm_skinny: unknown mode %d", mode);
    if (out_dtype == LLMK_BF16) return dispatch_rows<bf16, OUT_DIRECT>(mw, X, C, M, N, K, ldx, ldc, 1, per, error_flag, s);
    if (out_dtype == LLMK_F32) return dispatch_rows<float, OUT_DIRECT>(mw, X, C, M, N, K, ldx, ldc, 1, per, error_flag, s);
    LLMK_FAIL("gemm_skinny: unknown output dtype %d", out_dtype);
}

LLMK_EXPORT int llmk_gemm_skinny_fused_max_rows() { return 64; }

// Can the block-built X of the fused forms be held in shared memory?  `splits` slices of K for M rows.
LLMK_EXPORT int llmk_gemm_skinny_fused_fits(int M, int K, int splits) {
    if (M <= 0 || M > 64 || K <= 0 || splits < 1) return 0;
    const int mpad = M <= 16 ? 16 : M <= 32 ? 32 : 64;
    const int stages = mpad == 16 ? 6 : mpad == 32 ? 5 : 4;
    const int per = ceil_div(ceil_div(K, BK), splits);
    return stages * BW * BK * 2 + 2048 + per * mpad * BK * 2 + 1024 <= MAX_SMEM ? 1 : 0;
}

// The fused forms of the few-rows product (M <= 64, bfloat16 weights, float32 slices in C):
//   x_source 0   X is a bfloat16 array [M, K] (ldx), loaded by TMA
//            1   X is built from the float32 rows `x_resid` (x_ld): RMS-normalised with the row sums of
//                squares given in `n_sq_parts` parts `sq_parts[p * M + m]`, times (gain + gain_offset)
//            2   X is silu(gate) * up from `gu_splits` float32 slices `gu` of a packed gate/up product
//                ([M, gu_ld] each, `gu_split_stride` floats apart, columns alternating in groups of `group`)
//   resid != null: after the slices are written, the last block of each 128-column tile adds them to
//                resid[M, resid_ld] and writes the tile's share of every row's sum of squares to
//                sq_out[tile * M + m]; `tickets` holds one zeroed int per tile and is left zeroed.
//                Otherwise the slices in C are the result (as mode 1 of llmk_gemm_skinny).
LLMK_EXPORT int llmk_gemm_skinny_fused(float* C, const void* W, int M, int N, int K, long long ldw, long long ldc,
                                       int splits, int x_source, const void* X, long long ldx, const float* x_resid,
                                       long long x_ld, const float* sq_parts, int n_sq_parts, const float* gain,
                                       float eps, float gain_offset, const float* gu, int gu_splits,
                                       long long gu_split_stride, long long gu_ld, int group, float* resid,
                                       long long resid_ld, float* sq_out, int* tickets, int* error_flag, void* stream) {
    if (M <= 0 || N <= 0) return LLMK_OK;
    if (M > 64) LLMK_FAIL("gemm_skinny_fused: M=%d above 64", M);
    if (K <= 0 || K % 8 != 0 || ldw % 8 != 0 || !host_aligned16(W))
        LLMK_FAIL("gemm_skinny_fused: W not usable (K=%d ldw=%lld must be multiples of 8, base 16-byte aligned)", K, ldw);
    const int num_kb = ceil_div(K, BK);
    if (splits < 1 || splits > num_kb || splits > 65535) LLMK_FAIL("gemm_skinny_fused: %d slices for K=%d", splits, K);
    const int per = ceil_div(num_kb, splits);
    if ((splits - 1) * per >= num_kb) LLMK_FAIL("gemm_skinny_fused: %d slices of K=%d would leave one empty", splits, K);
    if (ldc < N || ldc % 4 != 0 || !host_aligned16(C)) LLMK_FAIL("gemm_skinny_fused: ldc=%lld not usable for N=%d", ldc, N);
    FusedArgs fa{};
#ifdef LLMK_SKINNY_TIMELINE
    static int tl_next = 0;
    fa.tl_id = tl_next++ % 8;
#endif
    CUtensorMap mw, mx{};
    if (!tc_host::cached_map_bf16_2d(&mw, W, N, K, ldw, BW))
        LLMK_FAIL("gemm_skinny_fused: cuTensorMapEncodeTiled failed for W (N=%d K=%d ldw=%lld)", N, K, ldw);
    if (x_source == X_TMA) {
        if (!X || ldx % 8 != 0 || !host_aligned16(X)) LLMK_FAIL("gemm_skinny_fused: X not usable (ldx=%lld)", ldx);
        const int mpad = M <= 16 ? 16 : M <= 32 ? 32 : 64;
        if (!tc_host::cached_map_bf16_2d(&mx, X, M, K, ldx, mpad))
            LLMK_FAIL("gemm_skinny_fused: cuTensorMapEncodeTiled failed for X (M=%d K=%d ldx=%lld)", M, K, ldx);
    } else if (x_source == X_NORM) {
        if (!x_resid || !sq_parts || !gain || n_sq_parts < 1 || x_ld < K || x_ld % 4 != 0 || !host_aligned16(x_resid) ||
            !host_aligned16(gain))
            LLMK_FAIL("gemm_skinny_fused: the rows to normalise are not usable (x_ld=%lld, %d parts)", x_ld, n_sq_parts);
        fa.x_resid = x_resid; fa.x_ld = x_ld; fa.sq_parts = sq_parts; fa.n_sq_parts = n_sq_parts;
        fa.gain = gain; fa.eps = eps; fa.gain_offset = gain_offset;
    } else if (x_source == X_GATED) {
        if (!gu || gu_splits < 1 || group < 8 || group % 8 != 0 || K % group != 0 || gu_ld < 2 * (long long)K || gu_ld % 4 != 0 ||
            gu_split_stride % 4 != 0 || !host_aligned16(gu))
            LLMK_FAIL("gemm_skinny_fused: the gate/up slices are not usable (group=%d gu_ld=%lld K=%d)", group, gu_ld, K);
        fa.gu = gu; fa.gu_splits = gu_splits; fa.gu_split_stride = gu_split_stride; fa.gu_ld = gu_ld; fa.group = group;
    } else {
        LLMK_FAIL("gemm_skinny_fused: unknown source of X %d", x_source);
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (resid) {
        if (!sq_out || !tickets || N % 4 != 0 || resid_ld < N || resid_ld % 4 != 0 || !host_aligned16(resid))
            LLMK_FAIL("gemm_skinny_fused: the residual is not usable (N=%d resid_ld=%lld)", N, resid_ld);
        fa.resid = resid; fa.resid_ld = resid_ld; fa.sq_out = sq_out; fa.tickets = tickets;
        if (x_source == X_TMA) return dispatch_fused<OUT_RESIDUAL, X_TMA>(mw, mx, C, M, N, K, ldc, splits, per, error_flag, fa, s);
        if (x_source == X_NORM) return dispatch_fused<OUT_RESIDUAL, X_NORM>(mw, mx, C, M, N, K, ldc, splits, per, error_flag, fa, s);
        return dispatch_fused<OUT_RESIDUAL, X_GATED>(mw, mx, C, M, N, K, ldc, splits, per, error_flag, fa, s);
    }
    if (x_source == X_TMA) return dispatch_fused<OUT_PARTIAL, X_TMA>(mw, mx, C, M, N, K, ldc, splits, per, error_flag, fa, s);
    if (x_source == X_NORM) return dispatch_fused<OUT_PARTIAL, X_NORM>(mw, mx, C, M, N, K, ldc, splits, per, error_flag, fa, s);
    return dispatch_fused<OUT_PARTIAL, X_GATED>(mw, mx, C, M, N, K, ldc, splits, per, error_flag, fa, s);
}

#ifdef LLMK_SKINNY_TIMELINE
LLMK_EXPORT int llmk_gemm_skinny_timeline(unsigned long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, g_skinny_tl, sizeof(g_skinny_tl)) == cudaSuccess ? LLMK_OK : 1;
}
#endif

// The residual add and the RMSNorm before a few-rows product, done by the product itself (M <= 16):
//   v = resid_in + the sum of `delta_splits` float32 slices of delta ([delta_splits][M][ld], `delta_split_stride`
//   floats apart); x = v / sqrt(mean(v^2) + eps) * (gain + gain_offset); C = x W^T; resid_out = v
// K (the width of the residual) is cut into `splits` slices (2, 4 or 8, each a multiple of 256 columns),
// the blocks of a tile's slices are a cluster and exchange their shares of the rows' sums of squares.
// gated == 0: C is float32 [splits][M][ldc], the slices of the product.  gated != 0: W interleaves gate
// and up rows in groups of 16, the slices are added up inside the cluster (splits 2 or 4) and C is
// bfloat16 [M][ldc] = silu(gate) * up.  resid_out must not be resid_in: other blocks still read it.
LLMK_EXPORT int llmk_gemm_skinny_addnorm(void* C, const void* W, int M, int N, int K, long long ldw, long long ldc,
                                         int splits, int gated, const float* resid_in, const float* delta,
                                         int delta_splits, long long delta_split_stride, long long ld,
                                         float* resid_out, const float* gain, float eps, float gain_offset,
                                         int* error_flag, void* stream) {
    if (M <= 0 || N <= 0) return LLMK_OK;
    if (M > 16) LLMK_FAIL("gemm_skinny_addnorm: M=%d above 16", M);
    if (K <= 0 || K % BK != 0 || ldw % 8 != 0 || !host_aligned16(W))
        LLMK_FAIL("gemm_skinny_addnorm: W not usable (K=%d a multiple of 64, ldw=%lld of 8, base 16-byte aligned)", K, ldw);
    const int num_kb = K / BK;
    if ((splits != 2 && splits != 4 && splits != 8) || num_kb % splits != 0 || (num_kb / splits) % 4 != 0 || num_kb / splits > 16)
        LLMK_FAIL("gemm_skinny_addnorm: %d slices of K=%d (2, 4 or 8 slices of 256, 512, 768 or 1024 columns each)", splits, K);
    if (M * (num_kb / splits) * 8 > 4 * 2 * BUILDERS) LLMK_FAIL("gemm_skinny_addnorm: %d rows of %d columns per block are too many", M, K / splits);
    if (gated && (splits > 4 || N % 32 != 0)) LLMK_FAIL("gemm_skinny_addnorm: the gated form takes 2 or 4 slices and N=%d a multiple of 32", N);
    if (!resid_in || !delta || !resid_out || !gain || resid_out == resid_in || delta_splits < 1 || ld < K || ld % 4 != 0 ||
        delta_split_stride % 4 != 0 || !host_aligned16(resid_in) || !host_aligned16(delta) || !host_aligned16(resid_out) ||
        !host_aligned16(gain))
        LLMK_FAIL("gemm_skinny_addnorm: the residual, the slices or the gain are not usable (ld=%lld)", ld);
    if (ldc < (gated ? N / 2 : N) || !host_aligned16(C)) LLMK_FAIL("gemm_skinny_addnorm: ldc=%lld not usable for N=%d", ldc, N);
    FusedArgs fa{};
    fa.an_resid_in = resid_in; fa.an_delta = delta; fa.an_resid_out = resid_out; fa.an_ld = ld;
    fa.an_split_stride = delta_split_stride; fa.an_splits = delta_splits;
    fa.gain = gain; fa.eps = eps; fa.gain_offset = gain_offset;
    CUtensorMap mw, mx{};
    if (!tc_host::cached_map_bf16_2d(&mw, W, N, K, ldw, BW))
        LLMK_FAIL("gemm_skinny_addnorm: cuTensorMapEncodeTiled failed for W (N=%d K=%d ldw=%lld)", N, K, ldw);
    cudaStream_t s = (cudaStream_t)stream;
    const int per = num_kb / splits;
    if (gated)
        return launch_fused<16, 6, OUT_CLUSTER_GATED, X_ADDNORM, bf16>(mw, mx, (bf16*)C, M, N, K, ldc, splits, per, error_flag, fa, s);
    return launch_fused<16, 6, OUT_PARTIAL, X_ADDNORM, float>(mw, mx, (float*)C, M, N, K, ldc, splits, per, error_flag, fa, s);
}
