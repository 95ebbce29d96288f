// C[M, N] = A[M, K] * W[N, K]^T in bfloat16 on the 5th-generation tensor cores of sm_100a:
// operand tiles arrive in shared memory through TMA (`cp.async.bulk.tensor`, 128-byte swizzle),
// one thread issues `tcgen05.mma` with the float32 accumulator in tensor memory, and four
// epilogue warps read it back with `tcgen05.ld`, round once and store.
//
// A block computes 128 x BN output tiles (BN = 64, 128 or 256) one after the other, 192 threads:
//   warp 0     TMA producer: for every 64-wide slice of K, one A box [128, 64] and one W box
//              [BN, 64] into a ring of STAGES buffers; `full[s]` counts the bytes.
//   warp 1     owns the tensor memory (two accumulators of BN columns) and issues the MMAs: 4
//              instructions of K = 16 per slice; `tcgen05.commit` releases the buffer (`empty[s]`) when
//              they have read it, and signals `acc_full[i]` after a tile's last slice; the next tile
//              goes to the other accumulator once the epilogue has released it (`acc_empty[i]`).
//   warps 2-5  epilogue: each reads the 32 accumulator lanes its warp id allows, 32 columns at a
//              time, and writes 64 (bfloat16) or 128 (float32) contiguous bytes per row.
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
constexpr int NUM_SMS = 148;

template <int BN, int STAGES, int MB>
struct Smem {
    static constexpr int A_BYTES = BM * BK * 2;        // one block of 128 rows of A
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = MB * A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int NUM_BARS = 2 * STAGES + 4;     // full, empty, acc_full[2], acc_empty[2]
    static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16 + 1024;  // + alignment slack
};

__device__ __forceinline__ float silu(float g) { return g / (1.0f + __expf(-g)); }

// Persistent: block b computes tiles b, b + gridDim.x, ... (tile t = (t % m_tiles) rows, (t / m_tiles)
// columns, so blocks that run together share W tiles).  A tile is MB blocks of 128 rows by BN
// columns: with MB = 2 the two MMAs of a k-step share the W tile, which halves what the block pulls
// from L2 per flop (the wide products are bound by that, not by the tensor core).  When two
// accumulator sets fit into tensor memory (2 * MB * BN <= 512 columns) they are used in turn: while
// the epilogue warps read tile i out of one, the MMA warp fills the other with tile i + 1; the TMA
// ring runs on across tiles either way.
template <typename TC, int BN, int STAGES, bool GATED, int MB>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               TC* __restrict__ C, int M, int N, int K, long long ldc, int* error_flag) {
    using L = Smem<BN, STAGES, MB>;
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
    const int m_tiles = (M + MB * BM - 1) / (MB * BM);
    const int n_tiles = (N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(tc::smem_u32(&full[s]), 1);
            tc::mbar_init(tc::smem_u32(&empty[s]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            tc::mbar_init(tc::smem_u32(&acc_full[i]), 1);
            tc::mbar_init(tc::smem_u32(&acc_empty[i]), 4);
        }
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&map_a);
        tc::prefetch_tensormap(&map_w);
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
            pdl_launch_dependents();
            pdl_wait();   // A was written by the kernel before this one
            uint32_t it = 0;        // k-slices loaded so far, over all tiles of this block
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * (MB * BM), n0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (!tc::mbar_wait(tc::smem_u32(&empty[s]), (round & 1) ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t bar = tc::smem_u32(&full[s]);
                    tc::mbar_expect_tx(bar, L::STAGE_BYTES);
                    const uint32_t a_dst = tc::smem_u32(smem + s * L::STAGE_BYTES);
#pragma unroll
                    for (int i = 0; i < MB; ++i) tc::tma_load_2d(a_dst + i * L::A_BYTES, &map_a, bar, kb * BK, m0 + i * BM);
                    tc::tma_load_2d(a_dst + MB * L::A_BYTES, &map_w, bar, kb * BK, n0);
                }
            }
            if (*abort_flag) {
                // Let the copies that are in flight land before the block's memory is given up.
                for (uint32_t k = it > (uint32_t)STAGES ? it - STAGES : 0; k < it; ++k) {
                    const long long t0 = clock64();
                    while (!tc::mbar_try_wait(tc::smem_u32(&full[k % STAGES]), (k / STAGES) & 1) &&
                           clock64() - t0 < tc::WAIT_LIMIT_CYCLES) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::idesc_bf16_f32(BM, BN);
            uint32_t it = 0;
            bool ok = true;
            int tile_iter = 0;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tile_iter) {
                const int buf = tile_iter % ACC_SETS;
                // the epilogue must have read this accumulator set before it is filled again
                ok = tc::mbar_wait(tc::smem_u32(&acc_empty[buf]), ((tile_iter / ACC_SETS) & 1) ^ 1, abort_flag);
                if (!ok) break;
                tc::tc_fence_after_sync();
                const uint32_t acc = tmem_base + (uint32_t)(buf * MB * BN);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    ok = tc::mbar_wait(tc::smem_u32(&full[s]), round & 1, abort_flag);
                    if (!ok) break;
                    tc::tc_fence_after_sync();
                    const uint32_t a_addr = tc::smem_u32(smem + s * L::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + MB * L::A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t db = tc::smem_desc_sw128(b_addr + k * UMMA_K * 2);
#pragma unroll
                        for (int i = 0; i < MB; ++i)
                            tc::mma_bf16_ss(acc + (uint32_t)(i * BN), tc::smem_desc_sw128(a_addr + i * L::A_BYTES + k * UMMA_K * 2),
                                            db, idesc, (kb | k) != 0);
                    }
                    tc::mma_commit(tc::smem_u32(&empty[s]));
                }
                if (ok) tc::mma_commit(tc::smem_u32(&acc_full[buf]));
            }
        }
    } else {
        // Epilogue: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31.
        const int quarter = warp & 3;
        const int n_out = GATED ? N / 2 : N;
        const bool vec_ok = (ldc % (16 / (int)sizeof(TC)) == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
        bool ok = true;
        int tile_iter = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tile_iter) {
            const int buf = tile_iter % ACC_SETS;
            const int m0 = (tile % m_tiles) * (MB * BM), n0 = (tile / m_tiles) * BN;
            ok = __all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(&acc_full[buf]), (tile_iter / ACC_SETS) & 1, abort_flag));
            if (!ok) break;
            tc::tc_fence_after_sync();
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
                    TC* dst = C + (size_t)row * ldc + n0 + c0;
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
            if (lane == 0) tc::mbar_arrive(tc::smem_u32(&acc_empty[buf]));
        }
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(tmem_base, TMEM_COLS);
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

template <typename TC, int BN, int STAGES, bool GATED, int MB>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int M, int N, int K, long long ldc,
           int* error_flag, int pdl, cudaStream_t s) {
    using L = Smem<BN, STAGES, MB>;
    auto kernel = gemm_tc_kernel<TC, BN, STAGES, GATED, MB>;
    static bool configured = false;   // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) LLMK_FAIL("gemm_tc: cannot raise shared memory to %d: %s", L::TOTAL, cudaGetErrorString(e));
        configured = true;
    }
    const int tiles = ceil_div(N, BN) * ceil_div(M, MB * BM);
    LLMK_CHECK_LAUNCH_RC("gemm_tc", llmk_launch(kernel, dim3(tiles < NUM_SMS ? tiles : NUM_SMS), dim3(THREADS), L::TOTAL, s,
                                                pdl != 0, ma, mw, (TC*)C, M, N, K, ldc, error_flag));
    return LLMK_OK;
}

template <typename TC, bool GATED>
int dispatch_tile(const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldw,
                  long long ldc, int* error_flag, int pdl, cudaStream_t s) {
    // Tile width: the one whose tiles take the least time in rounds over the SMs.  The relative times
    // of a tile were measured on the products of a 2,048-token prompt.  (Tiles of two row blocks,
    // MB = 2, were measured too: 256 x 256 is no faster than 128 x 256 with its epilogue overlapped,
    // so they are not used.)
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
    CUtensorMap ma, mw;
    if (!get_map(&ma, A, M, K, lda, BM) || !get_map(&mw, W, N, K, ldw, bn))
        LLMK_FAIL("gemm_tc: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d lda=%lld ldw=%lld)", M, N, K, lda, ldw);
    switch (bn) {
        case 256: return launch<TC, 256, 4, GATED, 1>(ma, mw, C, M, N, K, ldc, error_flag, pdl, s);
        case 128: return launch<TC, 128, 4, GATED, 1>(ma, mw, C, M, N, K, ldc, error_flag, pdl, s);
        default: return launch<TC, 64, 4, false, 1>(ma, mw, C, M, N, K, ldc, error_flag, pdl, s);
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
