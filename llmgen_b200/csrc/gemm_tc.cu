// C[M, N] = A[M, K] * W[N, K]^T in bfloat16 on the 5th-generation tensor cores of sm_100a:
// operand tiles arrive in shared memory through TMA (`cp.async.bulk.tensor`, 128-byte swizzle),
// one thread issues `tcgen05.mma` with the float32 accumulator in tensor memory, and four
// epilogue warps read it back with `tcgen05.ld`, round once and store.
//
// A block computes 128 x BN output tiles (BN = 64, 128 or 256) one after the other, 192 threads
// (from 4,096 rows on, two blocks of a cluster compute 256 x 256 tiles together, see PAIR below):
//   warp 0     TMA producer: for every 64-wide slice of K, one A box [128, 64] and one W box
//              [BN, 64] into a ring of STAGES buffers; `full[s]` counts the bytes.
//   warp 1     owns the tensor memory (two accumulators of BN columns) and issues the MMAs: 4
//              instructions of K = 16 per slice; `tcgen05.commit` releases the buffer (`empty[s]`) when
//              they have read it, and signals `acc_full[i]` after a tile's last slice; the next tile
//              goes to the other accumulator once the epilogue has released it (`acc_empty[i]`).
//   warps 2-5  epilogue: each reads the 32 accumulator lanes its warp id allows, 32 columns at a
//              time.  bfloat16 results are rounded into a slab of shared memory (32 rows x 64
//              columns, 128-byte swizzle) that one lane hands to a TMA store, two slabs per warp in
//              turn; float32 results, and results TMA cannot address, are stored by the threads,
//              64 or 128 contiguous bytes per row.
// Rows of A beyond M, rows of W beyond N and columns beyond K are zero-filled by TMA, so any M and
// N are taken; K must be a multiple of 8 and the bases 16-byte aligned (TMA's rules), otherwise
// the launcher refuses and the caller uses the CUDA-core product.
//
// Optionally the epilogue applies the gated activation to a W whose rows interleave gate and up in
// groups of 16 (`GATED`): out[m, j] = silu(c[m, gate j]) * c[m, up j], N/2 columns wide.
//
// Every wait is bounded (see tcgen05.cuh); a wait that gives up raises `*error_flag`, and the
// block still frees its tensor memory before it returns.
//
// The reference calls `cublasGemmEx` for this product (src/backend/cuda/linear/linear.cu:89-96).
#include "common.cuh"
#include "tcgen05.cuh"

#include <mutex>
#include <unordered_map>

LLMK_DEFINE_LAST_ERROR()

namespace {

constexpr int BM = 128;
constexpr int BK = 64;           // one 128-byte swizzle row of bfloat16
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;

template <int BN, int STAGES, int MB, bool PAIR = false, int KS = 1>
struct Smem {
    static constexpr int A_BYTES = BM * BK * 2;        // one block of 128 rows of A
    static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BK * 2;   // a pair's blocks hold half of the W rows each
    static constexpr int SUB_BYTES = MB * A_BYTES + B_BYTES;        // one step of 64 along K: A blocks, then W
    static constexpr int STAGE_BYTES = KS * SUB_BYTES;              // a stage of the ring holds KS such steps
    // the epilogue's staging: per epilogue warp two slabs of 32 rows x 64 bfloat16 columns (128-byte swizzle)
    static constexpr int SLAB_BYTES = 32 * 128;
    static constexpr int STAGING_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int STAGING_BYTES = 4 * 2 * SLAB_BYTES;
    static constexpr int BAR_OFFSET = STAGING_OFFSET + STAGING_BYTES;
    static constexpr int NUM_BARS = 2 * STAGES + 4;     // full, empty, acc_full[2], acc_empty[2]
    static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16 + 1024;  // + alignment slack
};

// the division as a reciprocal and a product: the exact one is a call with a slow path, which keeps the
// compiler from overlapping the elements of a row (measured: 9 us against 2 us for the epilogue of a tile)
__device__ __forceinline__ float silu(float g) { return __fdividef(g, 1.0f + __expf(-g)); }


// Persistent: block b computes tiles b, b + gridDim.x, ... (tile t = (t % m_tiles) rows, (t / m_tiles)
// columns, so blocks that run together share W tiles).  A tile is MB blocks of 128 rows by BN
// columns: with MB = 2 the two MMAs of a k-step share the W tile, which halves what the block pulls
// from L2 per flop (the wide products are bound by that, not by the tensor core).  When two
// accumulator sets fit into tensor memory (2 * MB * BN <= 512 columns) they are used in turn: while
// the epilogue warps read tile i out of one, the MMA warp fills the other with tile i + 1; the TMA
// ring runs on across tiles either way.
//
// PAIR: the kernel runs as clusters of two blocks (an SM pair) and a tile is 256 rows by BN columns,
// computed by `tcgen05.mma.cta_group::2`.  Each block loads its 128 rows of A and its half of the W
// rows (no multicast: every block loads what it holds), so a block pulls A + W/2 per k-step where a
// lone block pulls A + W: the wide products are bound by what the SMs pull from L2.  The bytes of
// both blocks are counted on the `full` barriers of the block of rank 0, which issues the MMAs; its
// commits arrive on the `empty` and `acc_full` barriers of both blocks; the epilogue warps of both
// release an accumulator set on rank 0's `acc_empty`.  Each block reads its own 128 rows of the
// accumulator out of its own tensor memory.
template <typename TC, int BN, int STAGES, bool GATED, int MB, bool PAIR = false, int KS = 1>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_c, int store_by_tma, int splits,
               TC* __restrict__ C, int M, int N, int K, long long ldc, int* error_flag) {
    static_assert(!PAIR || MB == 1, "a pair of blocks takes one block of rows each");
    using L = Smem<BN, STAGES, MB, PAIR, KS>;
    constexpr int ROWS = (PAIR ? 2 : MB) * BM;                     // rows of a tile
    constexpr int ACC_SETS = 2 * MB * BN <= 512 ? 2 : 1;
    constexpr uint32_t TMEM_COLS = ACC_SETS * MB * BN;             // 128, 256 or 512: a power of two
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* acc_full = bars + 2 * STAGES;         // 2
    uint64_t* acc_empty = bars + 2 * STAGES + 2;    // 2, four arrivals each (one per epilogue warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::NUM_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + BK - 1) / BK;
    const int m_tiles = (M + ROWS - 1) / ROWS;
    const int n_tiles = (N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    // K may be cut into `splits` slices (float32 results only): work item i is slice i / total_tiles of tile
    // i % total_tiles and leaves its sum in slice `split` of C ([splits][M][ldc]) for the consumer to add up
    const int total_items = total_tiles * splits;
    // a stage of the ring holds KS steps of 64 along K under one barrier (the hand-over of a stage costs about as
    // much as the copy of a narrow tile's step, so narrow tiles take two steps a stage); a slice begins on a stage
    const int kb_per_split = ((num_kb + splits - 1) / splits + KS - 1) / KS * KS;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;           // which block of the pair
    const int unit = PAIR ? (int)blockIdx.x / 2 : (int)blockIdx.x; // this block's (or pair's) place in the grid
    const int units = PAIR ? (int)gridDim.x / 2 : (int)gridDim.x;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(tc::smem_u32(&full[s]), 1);
            tc::mbar_init(tc::smem_u32(&empty[s]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            tc::mbar_init(tc::smem_u32(&acc_full[i]), 1);
            tc::mbar_init(tc::smem_u32(&acc_empty[i]), PAIR ? 8 : 4);
        }
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&map_a);
        tc::prefetch_tensormap(&map_w);
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            tc::tmem_alloc_pair(tc::smem_u32(tmem_slot), TMEM_COLS);
            tc::tmem_relinquish_pair();
        } else {
            tc::tmem_alloc(tc::smem_u32(tmem_slot), TMEM_COLS);
            tc::tmem_relinquish();
        }
    }
    tc::tc_fence_before_sync();
    if constexpr (PAIR) {
        __syncwarp();
        cluster_sync_all();     // both blocks' barriers and tensor memory are ready before either uses the other's
    } else {
        __syncthreads();
    }
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            pdl_launch_dependents();
            // W is a weight: no kernel of the stream writes it, so the first slices of it are asked for before the
            // wait for the kernel that makes A, and arrive while that kernel ends.
            uint32_t w_ahead = 0;
            if constexpr (!PAIR) {
                if (unit < total_items) {
                    const int tile = unit % total_tiles, kb0 = (unit / total_tiles) * kb_per_split;
                    const int sts = (min(num_kb, kb0 + kb_per_split) - kb0 + KS - 1) / KS;     // stages of the first item
                    w_ahead = (uint32_t)(sts < STAGES ? sts : STAGES);
                    const int n0 = (tile / m_tiles) * BN;
                    for (uint32_t i = 0; i < w_ahead; ++i) {
                        const uint32_t bar = tc::smem_u32(&full[i]);
                        tc::mbar_expect_tx(bar, L::STAGE_BYTES);
#pragma unroll
                        for (int h = 0; h < KS; ++h)      // a step beyond K is filled with zeros and counts its bytes all the same
                            tc::tma_load_2d(tc::smem_u32(smem + i * L::STAGE_BYTES + h * L::SUB_BYTES) + MB * L::A_BYTES, &map_w, bar,
                                            (kb0 + (int)i * KS + h) * BK, n0);
                    }
                }
            }
            pdl_wait();   // A was written by the kernel before this one
            uint32_t it = 0;        // k-slices loaded so far, over all tiles of this block
            bool ok = true;
            for (int item = unit; item < total_items && ok; item += units) {
                const int tile = item % total_tiles, split = item / total_tiles;
                const int m0 = (tile % m_tiles) * ROWS + (int)rank * BM;
                const int n0 = (tile / m_tiles) * BN + (PAIR ? (int)rank * (BN / 2) : 0);
                const int kb_end = min(num_kb, (split + 1) * kb_per_split);
                for (int kb = split * kb_per_split; kb < kb_end; kb += KS, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (!tc::mbar_wait(tc::smem_u32(&empty[s]), (round & 1) ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t bar = tc::smem_u32(&full[s]);
                    if constexpr (PAIR) {
                        // both blocks' bytes are counted on rank 0's barrier
                        if (rank == 0) tc::mbar_expect_tx(bar, 2 * L::STAGE_BYTES);
                        const uint32_t bar0 = cluster_map_shared(bar, 0);
#pragma unroll
                        for (int h = 0; h < KS; ++h) {
                            const uint32_t a_dst = tc::smem_u32(smem + s * L::STAGE_BYTES + h * L::SUB_BYTES);
                            tc::tma_load_2d_pair(a_dst, &map_a, bar0, (kb + h) * BK, m0);
                            tc::tma_load_2d_pair(a_dst + L::A_BYTES, &map_w, bar0, (kb + h) * BK, n0);
                        }
                    } else {
                        const bool w_here = it < w_ahead;       // its bytes are expected and W is on its way
                        if (!w_here) tc::mbar_expect_tx(bar, L::STAGE_BYTES);
#pragma unroll
                        for (int h = 0; h < KS; ++h) {
                            const uint32_t a_dst = tc::smem_u32(smem + s * L::STAGE_BYTES + h * L::SUB_BYTES);
#pragma unroll
                            for (int i = 0; i < MB; ++i) tc::tma_load_2d(a_dst + i * L::A_BYTES, &map_a, bar, (kb + h) * BK, m0 + i * BM);
                            if (!w_here) tc::tma_load_2d(a_dst + MB * L::A_BYTES, &map_w, bar, (kb + h) * BK, n0);
                        }
                    }
                }
            }
            if (*abort_flag && rank == 0) {
                // Let the copies that are in flight land before the block's memory is given up (rank 0's
                // barriers count the other block's copies too, and that block leaves only after rank 0).
                for (uint32_t k = it > (uint32_t)STAGES ? it - STAGES : 0; k < it; ++k) {
                    const long long t0 = clock64();
                    while (!tc::mbar_try_wait(tc::smem_u32(&full[k % STAGES]), (k / STAGES) & 1) &&
                           clock64() - t0 < tc::WAIT_LIMIT_CYCLES) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = tc::idesc_bf16_f32(PAIR ? 2 * BM : BM, BN);
            // The descriptor of the ring's first byte, built once: every operand tile's descriptor is this one plus
            // its byte offset in units of 16 (the start address is the descriptor's lowest field); built per
            // instruction they cost the one issuing thread a few per cent (11.1 -> 10.9 us, 15.2 -> 14.9 us on the
            // N = 1,024 products of a 2,048-token prompt).
            const uint64_t ring_desc = tc::smem_desc_sw128(tc::smem_u32(smem));
            uint32_t it = 0;
            bool ok = true;
            int tile_iter = 0;
            for (int item = unit; item < total_items && ok; item += units, ++tile_iter) {
                const int split = item / total_tiles;
                const int kb_begin = split * kb_per_split, kb_end = min(num_kb, (split + 1) * kb_per_split);
                const int buf = tile_iter % ACC_SETS;
                // the epilogue must have read this accumulator set before it is filled again
                ok = tc::mbar_wait(tc::smem_u32(&acc_empty[buf]), ((tile_iter / ACC_SETS) & 1) ^ 1, abort_flag);
                if (!ok) break;
                tc::tc_fence_after_sync();
                const uint32_t acc = tmem_base + (uint32_t)(buf * MB * BN);
                for (int kb = kb_begin; kb < kb_end; kb += KS, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    ok = tc::mbar_wait(tc::smem_u32(&full[s]), round & 1, abort_flag);
                    if (!ok) break;
                    tc::tc_fence_after_sync();
#pragma unroll
                    for (int h = 0; h < KS; ++h) {
                        if (kb + h >= kb_end) break;            // a step beyond K holds zeros: nothing to add
                        const uint64_t a_desc = ring_desc + (uint64_t)((s * L::STAGE_BYTES + h * L::SUB_BYTES) >> 4);
                        const uint64_t b_desc = a_desc + (uint64_t)((MB * L::A_BYTES) >> 4);
                        const bool first = kb + h == kb_begin;
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            const uint64_t db = b_desc + (uint64_t)((k * UMMA_K * 2) >> 4);
                            const bool add = !first || k != 0;
                            if constexpr (PAIR) {
                                tc::mma_bf16_ss_pair(acc, a_desc + (uint64_t)((k * UMMA_K * 2) >> 4), db, idesc, add);
                            } else {
#pragma unroll
                                for (int i = 0; i < MB; ++i)
                                    tc::mma_bf16_ss(acc + (uint32_t)(i * BN), a_desc + (uint64_t)((i * L::A_BYTES + k * UMMA_K * 2) >> 4),
                                                    db, idesc, add);
                            }
                        }
                    }
                    if constexpr (PAIR) tc::mma_commit_pair(tc::smem_u32(&empty[s]), (uint16_t)3);
                    else tc::mma_commit(tc::smem_u32(&empty[s]));
                }
                if (ok) {
                    if constexpr (PAIR) tc::mma_commit_pair(tc::smem_u32(&acc_full[buf]), (uint16_t)3);
                    else tc::mma_commit(tc::smem_u32(&acc_full[buf]));
                }
            }
        }
    } else {
        // Epilogue: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31.
        const int quarter = warp & 3;
        const int n_out = GATED ? N / 2 : N;
        const bool vec_ok = (ldc % (16 / (int)sizeof(TC)) == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
        bool ok = true;
        int tile_iter = 0;
        uint32_t box_iter = 0;          // boxes this warp has handed to TMA
        for (int item = unit; item < total_items && ok; item += units, ++tile_iter) {
            const int tile = item % total_tiles, split = item / total_tiles;
            const int buf = tile_iter % ACC_SETS;
            const int m0 = (tile % m_tiles) * ROWS + (int)rank * BM, n0 = (tile / m_tiles) * BN;
            ok = __all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(&acc_full[buf]), (tile_iter / ACC_SETS) & 1, abort_flag));
            if (!ok) break;
            tc::tc_fence_after_sync();
            if constexpr (sizeof(TC) == 2 && MB == 1) {
                if (store_by_tma) {
                    // Row-per-thread stores to global memory are slow and hold up the TMA loads of the next
                    // tile (measured: 4.3 us a tile against 1 us without them).  Each warp rounds its 32
                    // rows into a slab of shared memory, 64 output columns at a time, in the layout of a
                    // 128-byte-swizzled box (a lane's 16-byte pieces then fall into different banks), and
                    // one lane hands the slab to TMA, which writes whole rows and clips at M and N.
                    constexpr int ACC_COLS = GATED ? 128 : 64;          // accumulator columns per 64 output columns
                    const uint32_t slabs = tc::smem_u32(smem + L::STAGING_OFFSET) + (uint32_t)quarter * 2 * L::SLAB_BYTES;
                    const uint32_t acc0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN);
                    const bool rows_live = m0 + quarter * 32 < M;      // uniform over the warp
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += ACC_COLS) {
                        if (n0 + c0 >= N || !rows_live) break;
                        const uint32_t slab = slabs + (uint32_t)(box_iter & 1) * L::SLAB_BYTES;
                        if (lane == 0) tc::bulk_wait_read<1>();         // the store that read this slab two boxes ago
                        __syncwarp();
#pragma unroll
                        for (int h = 0; h < ACC_COLS / 32; ++h) {
                            uint32_t r[32];
                            tc::tmem_ld_32x32_wait(acc0 + (uint32_t)(c0 + 32 * h), r);
                            if constexpr (GATED) {
                                float o[16];
#pragma unroll
                                for (int i = 0; i < 16; ++i) o[i] = silu(__uint_as_float(r[i])) * __uint_as_float(r[16 + i]);
#pragma unroll
                                for (int q = 0; q < 2; ++q) {
                                    Vec16<bf16> v;
                                    v.pack(o + 8 * q);
                                    const int chunk = 2 * h + q;
                                    tc::st_shared_v4(slab + (uint32_t)lane * 128 + (uint32_t)((chunk ^ (lane & 7)) << 4), v.raw);
                                }
                            } else {
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    float f[8];
#pragma unroll
                                    for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[8 * q + j]);
                                    Vec16<bf16> v;
                                    v.pack(f);
                                    const int chunk = 4 * h + q;
                                    tc::st_shared_v4(slab + (uint32_t)lane * 128 + (uint32_t)((chunk ^ (lane & 7)) << 4), v.raw);
                                }
                            }
                        }
                        tc::fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) {
                            tc::tma_store_2d(&map_c, slab, GATED ? (n0 + c0) / 2 : n0 + c0, m0 + quarter * 32);
                            tc::bulk_commit();
                        }
                        ++box_iter;
                    }
                    tc::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (PAIR) tc::mbar_arrive_cluster(cluster_map_shared(tc::smem_u32(&acc_empty[buf]), 0));
                        else tc::mbar_arrive(tc::smem_u32(&acc_empty[buf]));
                    }
                    continue;
                }
            }
            if constexpr (sizeof(TC) == 4 && MB == 1 && !GATED) {
                if (store_by_tma) {
                    // float32 slices: slabs of 32 rows x 32 columns (128 bytes a row), handed to TMA the same way
                    const uint32_t slabs = tc::smem_u32(smem + L::STAGING_OFFSET) + (uint32_t)quarter * 2 * L::SLAB_BYTES;
                    const uint32_t acc0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN);
                    const bool rows_live = m0 + quarter * 32 < M;      // uniform over the warp
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 32) {
                        if (n0 + c0 >= N || !rows_live) break;
                        const uint32_t slab = slabs + (uint32_t)(box_iter & 1) * L::SLAB_BYTES;
                        if (lane == 0) tc::bulk_wait_read<1>();
                        __syncwarp();
                        uint32_t r[32];
                        tc::tmem_ld_32x32_wait(acc0 + (uint32_t)c0, r);
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            tc::st_shared_v4(slab + (uint32_t)lane * 128 + (uint32_t)((q ^ (lane & 7)) << 4),
                                             make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]));
                        tc::fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) {
                            tc::tma_store_3d(&map_c, slab, n0 + c0, m0 + quarter * 32, split);
                            tc::bulk_commit();
                        }
                        ++box_iter;
                    }
                    tc::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (PAIR) tc::mbar_arrive_cluster(cluster_map_shared(tc::smem_u32(&acc_empty[buf]), 0));
                        else tc::mbar_arrive(tc::smem_u32(&acc_empty[buf]));
                    }
                    continue;
                }
            }
#pragma unroll 1
            for (int cc = 0; cc < MB * BN; cc += 32) {
                const int mb = cc / BN, c0 = cc % BN;          // which block of rows, which columns of it
                const int row = m0 + mb * BM + quarter * 32 + lane;
                const uint32_t acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * MB * BN + mb * BN);
                if (n0 + c0 >= N || m0 + mb * BM >= M) continue;   // uniform over the warp
                uint32_t r[32];
                __syncwarp();
                tc::tmem_ld_32x32_wait(acc + (uint32_t)c0, r);
                if (row >= M) {
                    // nothing to store for this lane; it still takes part in the loads above
                } else if constexpr (GATED) {
                    // columns [c0, c0 + 16) are gates, [c0 + 16, c0 + 32) the matching ups
                    const int j0 = (n0 + c0) / 2;
                    float o[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = silu(__uint_as_float(r[i])) * __uint_as_float(r[16 + i]);
                    TC* dst = C + (size_t)row * ldc + j0;
                    if (vec_ok && j0 + 16 <= n_out) {
                        if constexpr (sizeof(TC) == 2) {
                            Vec16<bf16> v0, v1;
                            v0.pack(o);
                            v1.pack(o + 8);
                            reinterpret_cast<uint4*>(dst)[0] = v0.raw;
                            reinterpret_cast<uint4*>(dst)[1] = v1.raw;
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                reinterpret_cast<float4*>(dst)[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
                        }
                    } else {
                        for (int i = 0; i < 16; ++i)
                            if (j0 + i < n_out) dst[i] = from_float<TC>(o[i]);
                    }
                } else {
                    TC* dst = C + ((size_t)split * M + row) * ldc + n0 + c0;
                    if (vec_ok && n0 + c0 + 32 <= N) {
                        if constexpr (sizeof(TC) == 2) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                float f[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[8 * i + j]);
                                Vec16<bf16> v;
                                v.pack(f);
                                reinterpret_cast<uint4*>(dst)[i] = v.raw;
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                reinterpret_cast<float4*>(dst)[i] =
                                    make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                                __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                        }
                    } else {
                        for (int i = 0; i < 32; ++i)
                            if (n0 + c0 + i < N) dst[i] = from_float<TC>(__uint_as_float(r[i]));
                    }
                }
            }
            // this warp has read its lanes of the half: let the MMA warp fill it again
            tc::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR) tc::mbar_arrive_cluster(cluster_map_shared(tc::smem_u32(&acc_empty[buf]), 0));
                else tc::mbar_arrive(tc::smem_u32(&acc_empty[buf]));
            }
        }
        if (lane == 0) tc::bulk_wait_read<0>();     // the slabs are read before the block's memory is given up
    }
    tc::tc_fence_before_sync();
    if constexpr (PAIR) {
        __syncwarp();
        cluster_sync_all();     // neither block leaves, or frees tensor memory, while the other may still use it
    } else {
        __syncthreads();
    }
    if (warp == 1) {
        tc::tc_fence_after_sync();
        if constexpr (PAIR) tc::tmem_dealloc_pair(tmem_base, TMEM_COLS);
        else tc::tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && *abort_flag && error_flag) atomicExch(error_flag, 1);
}

// ------------------------------------------------------------------------ tensor-map cache
struct MapKey {
    const void* base;
    uint64_t rows, cols, ld;
    uint32_t box_rows;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.base);
        h = h * 1000003u ^ k.rows;
        h = h * 1000003u ^ k.cols;
        h = h * 1000003u ^ k.ld;
        return h * 1000003u ^ k.box_rows;
    }
};
std::mutex g_map_lock;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

bool get_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    MapKey key{base, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> guard(g_map_lock);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
        *out = it->second;
        return true;
    }
    if (!tc_host::make_map_bf16_2d(out, base, rows, cols, ld, box_rows)) return false;
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps.emplace(key, *out);
    return true;
}

int g_store_by_tma = 1;      // 0: the threads store their rows themselves (for measurements)

// float32 slices of C ([splits][M][ldc]) for TMA stores of [32 x 32] boxes
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_slice_maps;
bool get_slice_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t slices) {
    MapKey key{base, rows, cols, ld, slices};
    std::lock_guard<std::mutex> guard(g_map_lock);
    auto it = g_slice_maps.find(key);
    if (it != g_slice_maps.end()) {
        *out = it->second;
        return true;
    }
    if (!tc_host::make_map_f32_slices(out, base, rows, cols, ld, slices, 32)) return false;
    if (g_slice_maps.size() > 1024) g_slice_maps.clear();
    g_slice_maps.emplace(key, *out);
    return true;
}

template <typename TC, int BN, int STAGES, bool GATED, int MB, bool PAIR = false, int KS = 1>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int M, int N, int K, long long ldc,
           int* error_flag, int pdl, cudaStream_t s, int splits = 1) {
    using L = Smem<BN, STAGES, MB, PAIR, KS>;
    auto kernel = gemm_tc_kernel<TC, BN, STAGES, GATED, MB, PAIR, KS>;
    static bool configured = false;   // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) LLMK_FAIL("gemm_tc: cannot raise shared memory to %d: %s", L::TOTAL, cudaGetErrorString(e));
        configured = true;
    }
    // bfloat16 results leave through shared memory and TMA stores of [32 rows x 64 columns] boxes
    // where TMA can address C (16-byte aligned base and rows); otherwise the threads store their rows
    CUtensorMap mc{};
    int store_by_tma = 0;
    // (a TMA store clips at the tensor's last column in units of 16 bytes, measured: with a width that is no
    // multiple of 16 bytes it writes up to 7 bfloat16 columns beyond it, so such results are stored by the threads)
    if (sizeof(TC) == 2 && MB == 1 && g_store_by_tma && host_aligned16(C) && ldc % 8 == 0 && (GATED ? N / 2 : N) % 8 == 0)
        store_by_tma = get_map(&mc, C, M, GATED ? N / 2 : N, ldc, 32) ? 1 : 0;
    if (sizeof(TC) == 4 && MB == 1 && !GATED && g_store_by_tma && host_aligned16(C) && ldc % 4 == 0 && N % 4 == 0)
        store_by_tma = get_slice_map(&mc, C, M, N, ldc, splits) ? 1 : 0;
    const int NUM_SMS = device_sm_count();
    if constexpr (PAIR) {
        // clusters of two blocks, one pair of SMs each
        const int tiles = ceil_div(N, BN) * ceil_div(M, 2 * BM) * splits;
        const int pairs = tiles < NUM_SMS / 2 ? tiles : NUM_SMS / 2;
        LLMK_CHECK_LAUNCH_RC("gemm_tc", llmk_launch_clusters(kernel, dim3(2 * pairs), dim3(THREADS), L::TOTAL, s, pdl != 0,
                                                             dim3(2, 1, 1), ma, mw, mc, store_by_tma, splits, (TC*)C, M, N, K,
                                                             ldc, error_flag));
    } else {
        const int tiles = ceil_div(N, BN) * ceil_div(M, MB * BM) * splits;
        LLMK_CHECK_LAUNCH_RC("gemm_tc", llmk_launch(kernel, dim3(tiles < NUM_SMS ? tiles : NUM_SMS), dim3(THREADS), L::TOTAL, s,
                                                    pdl != 0, ma, mw, mc, store_by_tma, splits, (TC*)C, M, N, K, ldc,
                                                    error_flag));
    }
    return LLMK_OK;
}

// 0: lone blocks only.  1: pairs of blocks (`cta_group::2`) where the product has rows for them.
// 2, 3: pairs always, with tiles 256 or 128 columns wide (for measurements).
int g_pair_mode = 1;

// ring depth of the narrower tiles (3, 4 and 6 were measured on a prompt's products: no difference
// beyond 4, the MMA instructions set the pace)
constexpr int STAGES_128 = 3, KS_128 = 2, STAGES_64 = 4;      // 128-wide tiles: three stages of two steps along K

template <typename TC, bool GATED>
int dispatch_tile(const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldw,
                  long long ldc, int* error_flag, int pdl, cudaStream_t s) {
    // Tile width: the one whose tiles take the least time in rounds over the SMs.  The relative times
    // of a tile were measured on the products of a 2,048-token prompt.  (Tiles of two row blocks,
    // MB = 2, were measured too: 256 x 256 is no faster than 128 x 256 with its epilogue overlapped,
    // so they are not used.)
    const int NUM_SMS = device_sm_count();
    struct Shape { int bn; long long time; };
    const Shape shapes[] = {{256, 528}, {128, 348}, {64, 264}};
    int bn = GATED ? 128 : 64;
    long long best = -1;
    for (const Shape& sh : shapes) {
        if (GATED && sh.bn == 64) continue;          // the gated epilogue is built for the wider tiles only
        const long long tiles = (long long)ceil_div(M, BM) * ceil_div(N, sh.bn);
        const long long cost = ((tiles + NUM_SMS - 1) / NUM_SMS) * sh.time;
        if (best < 0 || cost < best) {
            best = cost;
            bn = sh.bn;
        }
    }
    int pair_bn = 0;
    if (g_pair_mode >= 2) pair_bn = g_pair_mode == 2 ? 256 : 128;
    else if (g_pair_mode == 1 && M >= 4096 && (long long)ceil_div(M, 2 * BM) * ceil_div(N, 256) >= 2 * (NUM_SMS / 2))
        pair_bn = 256;      // measured: pairs win from about 4,096 rows, with two rounds of 256 x 256 tiles for the 74 SM pairs
    if (pair_bn) {
        CUtensorMap pa, pw;
        if (!get_map(&pa, A, M, K, lda, BM) || !get_map(&pw, W, N, K, ldw, pair_bn / 2))
            LLMK_FAIL("gemm_tc: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d lda=%lld ldw=%lld)", M, N, K, lda, ldw);
        if (pair_bn == 256) return launch<TC, 256, 6, GATED, 1, true>(pa, pw, C, M, N, K, ldc, error_flag, pdl, s);
        return launch<TC, 128, 4, GATED, 1, true, 2>(pa, pw, C, M, N, K, ldc, error_flag, pdl, s);
    }
    CUtensorMap ma, mw;
    if (!get_map(&ma, A, M, K, lda, BM) || !get_map(&mw, W, N, K, ldw, bn))
        LLMK_FAIL("gemm_tc: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d lda=%lld ldw=%lld)", M, N, K, lda, ldw);
    switch (bn) {
        case 256: return launch<TC, 256, 4, GATED, 1>(ma, mw, C, M, N, K, ldc, error_flag, pdl, s);
        case 128: return launch<TC, 128, STAGES_128, GATED, 1, false, KS_128>(ma, mw, C, M, N, K, ldc, error_flag, pdl, s);
        default: return launch<TC, 64, STAGES_64, false, 1>(ma, mw, C, M, N, K, ldc, error_flag, pdl, s);
    }
}

}  // namespace

// 1 if the tensor-core kernel takes these operands (TMA needs 16-byte aligned bases and row strides).
LLMK_EXPORT int llmk_gemm_tc_usable(const void* A, const void* W, int M, int N, int K, long long lda, long long ldw) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0) return 0;
    if (!host_aligned16(A) || !host_aligned16(W)) return 0;
    return 1;
}

// Into how many slices of K a product is best cut when its tiles of 128 x 128 are too few for the SMs: about
// one work item per SM, at least 4 steps of 64 along K per item, at most 16 slices.  1: not cut.
LLMK_EXPORT int llmk_gemm_tc_splits(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 1;
    const int NUM_SMS = device_sm_count();
    const long long tiles = (long long)ceil_div(M, BM) * ceil_div(N, 128);
    if (tiles * 4 >= 3LL * NUM_SMS) return 1;           // the tiles alone keep three quarters of the SMs busy
    const int num_kb = ceil_div(K, BK);
    int splits = (int)(NUM_SMS / tiles);
    if (splits > num_kb / 4) splits = num_kb / 4;
    if (splits > 16) splits = 16;
    if (splits < 2) return 1;
    const int per = ceil_div(ceil_div(num_kb, splits), KS_128) * KS_128;      // a slice begins on a stage of the ring
    return ceil_div(num_kb, per);                        // no slice is left empty
}

// C (float32, [splits][M][ldc]) receives the sums over `splits` slices of K of A[M, K] * W[N, K]^T, in tiles of
// 128 x 128; the consumer adds the slices up in slice order.
LLMK_EXPORT int llmk_gemm_tc_sliced(float* C, const void* A, const void* W, int M, int N, int K, long long lda,
                                    long long ldw, long long ldc, int splits, int* error_flag, int pdl, void* stream) {
    if (M <= 0 || N <= 0) return LLMK_OK;
    if (K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || !host_aligned16(A) || !host_aligned16(W))
        LLMK_FAIL("gemm_tc: operands not usable (K=%d lda=%lld ldw=%lld must be multiples of 8, bases 16-byte aligned)", K, lda, ldw);
    const int num_kb = ceil_div(K, BK);
    if (splits < 1 || splits > num_kb) LLMK_FAIL("gemm_tc: %d slices for K=%d", splits, K);
    if ((splits - 1) * (ceil_div(ceil_div(num_kb, splits), KS_128) * KS_128) >= num_kb)
        LLMK_FAIL("gemm_tc: %d slices of K=%d would leave one empty (slices are multiples of %d columns)", splits, K, KS_128 * BK);
    if (ldc < N) LLMK_FAIL("gemm_tc: ldc=%lld too small", ldc);
    CUtensorMap ma, mw;
    if (!get_map(&ma, A, M, K, lda, BM) || !get_map(&mw, W, N, K, ldw, 128))
        LLMK_FAIL("gemm_tc: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d lda=%lld ldw=%lld)", M, N, K, lda, ldw);
    return launch<float, 128, STAGES_128, false, 1, false, KS_128>(ma, mw, C, M, N, K, ldc, error_flag, pdl, (cudaStream_t)stream, splits);
}

LLMK_EXPORT void llmk_gemm_tc_set_pair_mode(int mode) { g_pair_mode = mode; }
LLMK_EXPORT void llmk_gemm_tc_set_store_by_tma(int on) { g_store_by_tma = on; }

// out_dtype: storage of C (bfloat16, or float32 for logits).  gated != 0: W interleaves gate and up
// rows in groups of 16 and C is [M, N / 2].  error_flag (device int, may be null) is raised if a
// wait inside the kernel gave up.
LLMK_EXPORT int llmk_gemm_tc(void* C, const void* A, const void* W, int M, int N, int K, long long lda,
                             long long ldw, long long ldc, int gated, int out_dtype, int* error_flag, int pdl,
                             void* stream) {
    if (M <= 0 || N <= 0) return LLMK_OK;
    if (!llmk_gemm_tc_usable(A, W, M, N, K, lda, ldw))
        LLMK_FAIL("gemm_tc: operands not usable (K=%d lda=%lld ldw=%lld must be multiples of 8, bases 16-byte aligned)", K, lda, ldw);
    if (gated && N % 32 != 0) LLMK_FAIL("gemm_tc: gated epilogue needs N=%d to be a multiple of 32", N);
    if (ldc < (gated ? N / 2 : N)) LLMK_FAIL("gemm_tc: ldc=%lld too small", ldc);
    if (ceil_div(M, BM) > 65535) LLMK_FAIL("gemm_tc: M=%d too large", M);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == LLMK_BF16)
        return gated ? dispatch_tile<bf16, true>(A, W, C, M, N, K, lda, ldw, ldc, error_flag, pdl, s)
                     : dispatch_tile<bf16, false>(A, W, C, M, N, K, lda, ldw, ldc, error_flag, pdl, s);
    if (out_dtype == LLMK_F32)
        return gated ? dispatch_tile<float, true>(A, W, C, M, N, K, lda, ldw, ldc, error_flag, pdl, s)
                     : dispatch_tile<float, false>(A, W, C, M, N, K, lda, ldw, ldc, error_flag, pdl, s);
    LLMK_FAIL("gemm_tc: unknown output dtype %d", out_dtype);
}

