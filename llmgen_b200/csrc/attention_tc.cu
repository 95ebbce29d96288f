// Causal grouped-query attention over the paged cache for prompts and prompt portions in bfloat16,
// on the 5th-generation tensor cores of sm_100a: S = Q K^T and O = P V are `tcgen05.mma`
// instructions with their accumulators in tensor memory; K and V pages arrive through TMA.
//
// Block = one tile of 128 rows of one (sequence, kv head): 128 / gc queries x gc query heads of the
// kv head's group (gc = the largest power of two dividing the group size, at most 16), so a K/V
// tile is read once for gc heads.  352 threads:
//   warp 0     TMA producer: the Q tile once (a 3-D box [queries, gc heads, 64] per half of the head),
//              then per tile of 128 keys the K pages of the block table into a ring of two stages.
//   warp 10    TMA producer of the V pages, a ring of two stages of its own.
//   warp 1     owns tensor memory (S0 | S1 | O: 2 x 128 + head_dim columns) and issues the MMAs:
//              S[j] = Q K_j^T (K-major operands), O += P_j V_j (V read MN-major: keys are V's rows
//              in shared memory; O adds up in tensor memory over all tiles).  S is double-buffered so
//              that Q K_{j+1}^T runs under the softmax of tile j.
//   warps 2-9  softmax: two threads per row, each with half of the row's key columns and half of the
//              head.  Pass 1 reads S from tensor memory and finds the row maximum (causal and window
//              mask on the tiles that need it; the two halves exchange maxima through shared memory);
//              pass 2 writes P = exp2((s - m) * scale *
//              log2 e) as bfloat16 into shared memory in the swizzled K-major layout the second MMA
//              reads.  m is the row's reference maximum: it follows the true maximum only when that grew
//              by more than 8 in the exponent's scale, and only then is O rescaled (read from tensor
//              memory, multiplied by exp(m_old - m_new), written back) before the tile's P V is issued;
//              l and O are kept against the same reference, so the quotient is the softmax whatever the
//              reference.  O is read once, after the last tile.  Reductions run as four independent
//              chains: with so few warps per SM the latency of a dependent chain is what costs.
// Statistics (m, l), the accumulator and the final division are float32.
//
// Tiles follow the reference's prefill kernel in spirit (src/backend/cuda/attention/attention.cu:300-466:
// 64-query tiles, `mma.sync`, K/V through `cp.async`, group sizes 1 and 2 only); semantics follow its
// CPU attention (src/backend/cpu/attention.zig:64-118): query j of a portion sits at position
// ctx - q_len + j and sees keys 0..position (or the last `window` of them); a row with ctx < q_len
// gives zeros.
//
// Taken: head_dim 64 or 128, page sizes 16, 32, 64, 128, any group size.  Everything else is refused
// with an error and the caller uses the CUDA-core kernel (csrc/attention.cu).  The cache arrays must
// hold finite values everywhere (slots never written are zero): masked keys enter the second MMA
// with weight 0.  Every wait is bounded; a wait that gives up raises `*error_flag`.
#include "common.cuh"
#include "tcgen05.cuh"

LLMK_DEFINE_LAST_ERROR()

namespace {

constexpr int BM = 128;     // rows of a tile
constexpr int BN = 128;     // keys per tile
constexpr int THREADS = 352;    // K producer, MMA, eight softmax warps, V producer

struct Params {
    bf16* out;
    long long o_stride;
    const int* block_tables;
    const int* ctx_len;
    const int* cu_q;
    const int* tile_seq;
    const int* tile_q0;
    int* error_flag;
    int max_blocks, nq, nkv, page_size, window, gc, bq, chunks;
    float scale_log2;
    unsigned v_lbo, v_sbo;
};


template <int HD>
struct Smem {
    static constexpr int Q_BYTES = BM * HD * 2;
    static constexpr int KV_BYTES = BN * HD * 2;       // one K or V tile
    static constexpr int P_BYTES = BM * BN * 2;
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = Q_OFF + Q_BYTES;       // 2 stages
    static constexpr int V_OFF = K_OFF + 2 * KV_BYTES;  // 2 stages
    static constexpr int P_OFF = V_OFF + 2 * KV_BYTES;  // 2 buffers
    static constexpr int XCHG_OFF = P_OFF + 2 * P_BYTES;   // float [2][2][BM]: row maxima (and at the end sums) of the two halves
    static constexpr int BAR_OFF = XCHG_OFF + 2 * 2 * BM * 4;
    static constexpr int NUM_BARS = 14;
    // No slack for aligning the base: the kernel has no static shared memory, so the dynamic part
    // starts on a 1024-byte boundary; the kernel checks that and reports an error otherwise.
    static constexpr int TOTAL = BAR_OFF + NUM_BARS * 8 + 16;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The page ids of the tile of keys starting at `k0`, as the block table has them (pages past the sequence's last
// one are replaced by the last page: their keys are masked).  Only the loads are issued here: the caller asks for
// the next tile's ids before it waits for a free stage and issues the copies of this tile, so that the table's
// latency (1,300 to 1,900 cycles a tile when it was looked up in turn, half of a tile's time) is not waited for.
// PS (the page size) is a template parameter throughout: the producers are single threads whose instruction count
// per tile is what bounds them, and constant trip counts and strides halve it.
template <int PS>
__device__ __forceinline__ void page_ids(int (&ids)[BN / PS], const int* bt, int k0, int last_page) {
    const int page0 = k0 / PS;
#pragma unroll
    for (int pg = 0; pg < BN / PS; ++pg) ids[pg] = __ldg(bt + min(page0 + pg, last_page));
}

// One tile of BN keys, page by page: per page and 64-wide block of the head a box [PS, 64] whose first cache row
// is (page * nkv + kvh) * PS (a page already given back by a window, id -1, is replaced by the last page: its keys
// are masked).
template <int HB, int PS>
__device__ __forceinline__ void load_pages(uint32_t dst, const CUtensorMap* map, uint32_t bar, const int (&ids)[BN / PS],
                                           const int* bt, int last_page, int nkv, int kvh) {
    tc::mbar_expect_tx(bar, BN * HB * 128);
#pragma unroll
    for (int pg = 0; pg < BN / PS; ++pg) {
        int page = ids[pg];
        if (page < 0) page = __ldg(bt + last_page);
        const int row = (page * nkv + kvh) * PS;
#pragma unroll
        for (int h = 0; h < HB; ++h) tc::tma_load_2d(dst + h * BN * 128 + pg * PS * 128, map, bar, h * 64, row);
    }
}

template <int HD, int PS>
__global__ void __launch_bounds__(THREADS)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const Params p) {
    using L = Smem<HD>;
    constexpr int HB = HD / 64;                 // 64-wide blocks of the head
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t S_COL0 = 0, S_COL1 = BN, O_COL0 = 2 * BN;
    extern __shared__ __align__(1024) uint8_t smem[];
    // A tile whose sequence is -1 is padding of a list of fixed length (a launch shape kept for replay): the
    // block leaves before it sets anything up.  The list is read ahead of `griddepcontrol.wait`: it belongs
    // to the step's arrays, which a copy wrote before the step's first kernel started, never a kernel of the
    // step itself.
    if (p.tile_seq[blockIdx.y] < 0) {
        // the block still waits for the kernel before: were all tiles padding, this grid would otherwise count as
        // complete before that kernel is, and the kernel after this one could start too early
        pdl_wait();
        return;
    }
    if ((tc::smem_u32(smem) & 1023u) != 0) {      // uniform over the block: nothing has been set up yet
        if (threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 2);
        return;
    }
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
    uint64_t* q_full = bars;            // 1
    uint64_t* k_full = bars + 1;        // 2
    uint64_t* v_full = bars + 3;        // 2
    uint64_t* k_empty = bars + 5;       // 2
    uint64_t* v_empty = bars + 7;       // 2
    uint64_t* s_full = bars + 9;        // 2
    uint64_t* p_full = bars + 11;       // 1, 256 arrivals
    uint64_t* o_full = bars + 12;       // 2
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::NUM_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.nq / p.nkv;
    // heads vary fastest over the grid: the caller lists the tiles heaviest first, and the blocks of a
    // grid start in the order of their linear index, so the long tiles of every head start first
    const int kvh = blockIdx.x / p.chunks;
    const int chunk = blockIdx.x % p.chunks;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < L::NUM_BARS; ++i) tc::mbar_init(tc::smem_u32(&bars[i]), i == 11 ? 256 : 1);
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&map_q);
        tc::prefetch_tensormap(&map_k);
        tc::prefetch_tensormap(&map_v);
        pdl_launch_dependents();
    }
    if (warp == 1) {
        tc::tmem_alloc(tc::smem_u32(tmem_slot), TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();   // q, the cache and the step's arrays come from earlier work of the stream

    const int s = p.tile_seq[blockIdx.y];
    const int q0 = p.tile_q0[blockIdx.y];
    const int q_beg = p.cu_q[s];
    const int q_len = p.cu_q[s + 1] - q_beg;
    const int ctx = p.ctx_len[s];
    const int nq_tile = min(p.bq, q_len - q0);
    const bool padding = ctx < q_len || nq_tile <= 0;
    const int first_pos = ctx - q_len + q0;
    int kt0 = 0, n_tiles = 0;
    if (!padding) {
        const int k_end = first_pos + nq_tile;
        const int k_beg = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
        kt0 = (k_beg / BN) * BN;
        n_tiles = (k_end - kt0 + BN - 1) / BN;
    }
    const int head0 = kvh * G + chunk * p.gc;

    if (warp == 0) {
        if (lane == 0 && n_tiles > 0) {
            const uint32_t qbar = tc::smem_u32(q_full);
            tc::mbar_expect_tx(qbar, L::Q_BYTES);
#pragma unroll
            for (int h = 0; h < HB; ++h)
                tc::tma_load_3d(tc::smem_u32(smem + L::Q_OFF + h * BM * 128), &map_q, qbar, h * 64, head0, q_beg + q0);
            const int* bt = p.block_tables + (size_t)s * p.max_blocks;
            const int last_page = (ctx - 1) / PS;
            int ids[BN / PS], next_ids[BN / PS];
            page_ids<PS>(next_ids, bt, kt0, last_page);
            for (int j = 0; j < n_tiles; ++j) {
                const int st = j & 1;
                const uint32_t round = j >> 1;
#pragma unroll
                for (int pg = 0; pg < BN / PS; ++pg) ids[pg] = next_ids[pg];
                if (j + 1 < n_tiles) page_ids<PS>(next_ids, bt, kt0 + (j + 1) * BN, last_page);
                if (!tc::mbar_wait(tc::smem_u32(&k_empty[st]), (round & 1) ^ 1, abort_flag)) break;
                load_pages<HB, PS>(tc::smem_u32(smem + L::K_OFF + st * L::KV_BYTES), &map_k, tc::smem_u32(&k_full[st]), ids, bt,
                                   last_page, p.nkv, kvh);
            }
        }
    } else if (warp == 10) {
        // V producer: a ring of its own, so that K of the next tiles never waits for a V slot.
        if (lane == 0 && n_tiles > 0) {
            const int* bt = p.block_tables + (size_t)s * p.max_blocks;
            const int last_page = (ctx - 1) / PS;
            int ids[BN / PS], next_ids[BN / PS];
            page_ids<PS>(next_ids, bt, kt0, last_page);
            for (int j = 0; j < n_tiles; ++j) {
                const int st = j & 1;
                const uint32_t round = j >> 1;
#pragma unroll
                for (int pg = 0; pg < BN / PS; ++pg) ids[pg] = next_ids[pg];
                if (j + 1 < n_tiles) page_ids<PS>(next_ids, bt, kt0 + (j + 1) * BN, last_page);
                if (!tc::mbar_wait(tc::smem_u32(&v_empty[st]), (round & 1) ^ 1, abort_flag)) break;
                load_pages<HB, PS>(tc::smem_u32(smem + L::V_OFF + st * L::KV_BYTES), &map_v, tc::smem_u32(&v_full[st]), ids, bt,
                                   last_page, p.nkv, kvh);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_tiles > 0) {
            constexpr uint32_t idesc_s = tc::idesc_bf16_f32(BM, BN);
            constexpr uint32_t idesc_o = tc::idesc_bf16_f32_b_mn(BM, HD);
            // descriptors of the four operands, built once: a step along K (or along the keys) adds to the start
            // address, which is the descriptor's lowest field in units of 16 bytes
            const uint64_t q_desc = tc::smem_desc_sw128(tc::smem_u32(smem + L::Q_OFF));
            const uint64_t k_desc[2] = {tc::smem_desc_sw128(tc::smem_u32(smem + L::K_OFF)),
                                        tc::smem_desc_sw128(tc::smem_u32(smem + L::K_OFF + L::KV_BYTES))};
            const uint64_t p_desc[2] = {tc::smem_desc_sw128(tc::smem_u32(smem + L::P_OFF)),
                                        tc::smem_desc_sw128(tc::smem_u32(smem + L::P_OFF + L::P_BYTES))};
            const uint64_t v_desc[2] = {tc::smem_desc_sw128_mn(tc::smem_u32(smem + L::V_OFF), p.v_lbo, p.v_sbo),
                                        tc::smem_desc_sw128_mn(tc::smem_u32(smem + L::V_OFF + L::KV_BYTES), p.v_lbo, p.v_sbo)};
            auto issue_qk = [&](int j) -> bool {
                const int st = j & 1;
                if (!tc::mbar_wait(tc::smem_u32(&k_full[st]), (j >> 1) & 1, abort_flag)) return false;
                tc::tc_fence_after_sync();
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint64_t off = (uint64_t)(((k / 4) * (BM * 128) + (k % 4) * 32) >> 4);
                    tc::mma_bf16_ss(tmem_base + (st ? S_COL1 : S_COL0), q_desc + off, k_desc[st] + off, idesc_s, k != 0);
                }
                tc::mma_commit(tc::smem_u32(&s_full[st]));
                tc::mma_commit(tc::smem_u32(&k_empty[st]));
                return true;
            };
            bool ok = tc::mbar_wait(tc::smem_u32(q_full), 0, abort_flag);
            if (ok) tc::tc_fence_after_sync();
            ok = ok && issue_qk(0);
            if (ok && n_tiles > 1) ok = issue_qk(1);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int st = j & 1;
                ok = tc::mbar_wait(tc::smem_u32(p_full), j & 1, abort_flag) &&
                     tc::mbar_wait(tc::smem_u32(&v_full[st]), (j >> 1) & 1, abort_flag);
                if (!ok) break;
                tc::tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint64_t da = p_desc[st] + (uint64_t)(((kk / 4) * (BM * 128) + (kk % 4) * 32) >> 4);
                    const uint64_t db = v_desc[st] + (uint64_t)((kk * 16 * 128) >> 4);
                    tc::mma_bf16_ss(tmem_base + O_COL0, da, db, idesc_o, (j | kk) != 0);   // O adds up in tensor memory over the tiles
                }
                tc::mma_commit(tc::smem_u32(&o_full[st]));
                tc::mma_commit(tc::smem_u32(&v_empty[st]));
                if (j + 2 < n_tiles) ok = issue_qk(j + 2);
            }
        }
    } else {
        // Softmax and accumulation, eight warps.  Warp w may touch tensor-memory lanes
        // 32 * (w % 4) .. + 31, so a row of the tile belongs to two warps: `half` 0 takes key columns
        // 0..63 of S and the first half of the head in O, `half` 1 the rest.  The two exchange their
        // row maxima through shared memory once per tile; sums stay separate until the end.
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;
        const int qi = r / p.gc;
        const int head = head0 + r % p.gc;
        const bool row_valid = !padding && qi < nq_tile && (chunk * p.gc + r % p.gc) < G;
        const int qpos = first_pos + qi;
        const int lo = p.window > 0 ? qpos - p.window : -1;   // keys at positions > lo are visible
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const float sl2 = p.scale_log2;
        constexpr int OC = HD / 2;            // columns of O this thread accumulates
        constexpr int SC = BN / 2;            // columns of S this thread turns into P
        float m = -INFINITY, l = 0.f;
        uint8_t* p_row0 = smem + L::P_OFF + half * (BM * 128) + r * 128;
        float* xchg = reinterpret_cast<float*>(smem + L::XCHG_OFF);      // [2 tiles][2 halves][128 rows]
        bool ok = true;

        const uint32_t o_addr = tmem_base + lane_addr + O_COL0 + half * OC;     // this thread's columns of O

        // This thread's scores of a tile: read from tensor memory once and kept for both passes.  (Asking for the
        // next tile's scores in the middle of pass 2, into the registers just used up, was measured: 41.1 against
        // 35.4 us on a 2,048-token prompt.)
        uint32_t v[SC / 32][32];
        static_assert(SC == 64, "two loads of 32 columns");
        const uint32_t s_col = lane_addr + half * SC;
        const int pair_barrier = 1 + quarter;       // the two warps of a row exchange its maxima: a barrier of their own

        for (int j = 0; j < n_tiles; ++j) {
            const int st = j & 1;
            const int k0 = kt0 + j * BN + half * SC;      // first key of this thread's columns
            const bool need_mask = (k0 + SC - 1 > qpos) || (k0 <= lo);
            uint8_t* p_row = p_row0 + st * L::P_BYTES;       // P is double-buffered: P V of the tile before may still read the other
            // pass 1: the maximum of this thread's half of the row (four independent chains)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (ok) ok = __all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(&s_full[st]), (j >> 1) & 1, abort_flag));
            tc::tc_fence_after_sync();
            if (ok) {
                const uint32_t s_addr = tmem_base + s_col + (st ? S_COL1 : S_COL0);
                tc::tmem_ld_32x32_x2_wait(s_addr, s_addr + 32, v[0], v[1]);
#pragma unroll
                for (int c = 0; c < SC / 32; ++c) {
                    if (need_mask) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int kpos = k0 + c * 32 + i;
                            if (kpos <= qpos && kpos > lo) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[c][i]));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[c][i]));
                    }
                }
            }
            const float mx_own = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            xchg[(st * 2 + half) * BM + r] = mx_own;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");       // the row's two warps
            const float mx = fmaxf(mx_own, xchg[(st * 2 + (half ^ 1)) * BM + r]);
            // The row's reference maximum follows the true one lazily: only when that grew by more than 8 in
            // the exponent's scale (P then stays below 2^8, and the result is the same up to rounding, as
            // l and O are kept against the same reference).  O lives in tensor memory and is rescaled there
            // on the few tiles where a row of the warp moves its reference.
            const float m_new = fmaxf(m, mx);
            const bool move = m_new > m && (m == -INFINITY || (m_new - m) * sl2 > 8.f);
            const bool fix = move && m != -INFINITY && j > 0;      // O and l hold something to rescale
            const float alpha = fix ? fast_exp2((m - m_new) * sl2) : 1.f;
            if (move) m = m_new;
            if (ok && __any_sync(0xffffffffu, fix)) {
                ok = __all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(&o_full[(j - 1) & 1]), ((j - 1) >> 1) & 1, abort_flag));
                tc::tc_fence_after_sync();
                if (ok) {
#pragma unroll
                    for (int c = 0; c < OC / 32; ++c) {
                        uint32_t o[32];
                        tc::tmem_ld_32x32_wait(o_addr + c * 32, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tc::tmem_st_32x32(o_addr + c * 32, o);
                    }
                    tc::tmem_st_wait();
                }
            }
            // pass 2: P into shared memory, row sum
            if (ok) {
                const float mb = (m == -INFINITY) ? 0.f : m * sl2;
                float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c = 0; c < SC / 32; ++c) {
                    float pv[32];
                    if (need_mask) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int kpos = k0 + c * 32 + i;
                            const bool vis = kpos <= qpos && kpos > lo;
                            pv[i] = vis ? fast_exp2(fmaf(__uint_as_float(v[c][i]), sl2, -mb)) : 0.f;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) pv[i] = fast_exp2(fmaf(__uint_as_float(v[c][i]), sl2, -mb));
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i) sum4[i & 3] += pv[i];
#pragma unroll
                    for (int q8 = 0; q8 < 4; ++q8) {
                        Vec16<bf16> pk;
                        pk.pack(pv + q8 * 8);
                        const int chunk16 = c * 4 + q8;       // 16-byte chunk inside this half's 64 columns
                        *reinterpret_cast<uint4*>(p_row + ((chunk16 ^ (r & 7)) << 4)) = pk.raw;
                    }
                }
                l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
                tc::fence_proxy_async();
                tc::tc_fence_before_sync();
                tc::mbar_arrive(tc::smem_u32(p_full));
            }
        }
        if (ok && n_tiles > 0) {
            ok = __all_sync(0xffffffffu, tc::mbar_wait(tc::smem_u32(&o_full[(n_tiles - 1) & 1]), ((n_tiles - 1) >> 1) & 1, abort_flag));
            tc::tc_fence_after_sync();
        }
        // the row's sum is the two halves' sums (both were kept against the same maxima)
        const int pair_barrier_end = 1 + quarter;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier_end) : "memory");       // every read of the last tile's maxima is done
        xchg[half * BM + r] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier_end) : "memory");
        const float l_row = l + xchg[(half ^ 1) * BM + r];
        const bool writes = ok && qi < max(nq_tile, 0) && (chunk * p.gc + r % p.gc) < G;
        const float inv = (row_valid && l_row > 0.f) ? 1.0f / l_row : 0.f;
        bf16* o = p.out + (size_t)(q_beg + q0 + qi) * p.o_stride + (size_t)head * HD + half * OC;
#pragma unroll
        for (int c = 0; c < OC / 32; ++c) {
            uint32_t acc[32];
            if (ok && n_tiles > 0) {                     // uniform over the warp: the load is a warp's instruction
                tc::tmem_ld_32x32_wait(o_addr + c * 32, acc);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] = 0u;
            }
            if (writes) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    float f[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) f[e] = inv > 0.f ? __uint_as_float(acc[i + e]) * inv : 0.f;
                    Vec16<bf16> pk;
                    pk.pack(f);
                    *reinterpret_cast<uint4*>(o + c * 32 + i) = pk.raw;
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
    if (threadIdx.x == 0 && *abort_flag && p.error_flag) atomicExch(p.error_flag, 1);
}

int group_chunk(int G) {
    int gc = 1;
    while (gc < 16 && G % (gc * 2) == 0) gc *= 2;
    return gc;
}

template <int HD, int PS>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const Params& p, dim3 grid,
           cudaStream_t s) {
    using L = Smem<HD>;
    auto kernel = attention_tc_kernel<HD, PS>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) LLMK_FAIL("attention_tc: cannot raise shared memory to %d: %s", L::TOTAL, cudaGetErrorString(e));
        configured = true;
    }
    LLMK_CHECK_LAUNCH_RC("attention_tc", llmk_launch(kernel, grid, dim3(THREADS), L::TOTAL, s, true, mq, mk, mv, p));
    return LLMK_OK;
}

}  // namespace

// Queries per tile for this group size (0: the kernel does not take these sizes).
LLMK_EXPORT int llmk_attention_tc_tile_queries(int nq, int nkv, int hd, int page_size) {
    if (nkv <= 0 || nq <= 0 || nq % nkv != 0) return 0;
    if (hd != 64 && hd != 128) return 0;
    if (page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128) return 0;
    return BM / group_chunk(nq / nkv);
}

// out[t, nq*hd] = attention of q[t] (bfloat16, row stride q_stride) over the paged cache
// [num_pages, nkv, page_size, hd].  tile_seq / tile_q0 list tiles of `llmk_attention_tc_tile_queries`
// queries each; an entry with sequence -1 is skipped.  The two lists must not be written by a kernel of this
// library launched just before (they are read before the wait on the kernel before).  v_lbo / v_sbo: 0 for the defaults (descriptor strides of the V operand).
LLMK_EXPORT int llmk_attention_tc(void* out, long long o_stride, const void* q, long long q_stride, int n_tokens,
                                  const void* kcache, const void* vcache, long long num_pages,
                                  const int* block_tables, int max_blocks, const int* ctx_len, const int* cu_q,
                                  const int* tile_seq, const int* tile_q0, int n_tiles, int nq, int nkv, int hd,
                                  int page_size, int window, float scale, int* error_flag, unsigned v_lbo,
                                  unsigned v_sbo, void* stream
) {
    if (n_tiles <= 0 || n_tokens <= 0) return LLMK_OK;
    const int bq = llmk_attention_tc_tile_queries(nq, nkv, hd, page_size);
    if (bq == 0)
        LLMK_FAIL("attention_tc: not taken (heads %d/%d, head_dim %d must be 64 or 128, page size %d must be 16, 32, 64 or 128)",
                  nq, nkv, hd, page_size);
    if (q_stride % 8 != 0 || o_stride % 8 != 0 || !host_aligned16(q) || !host_aligned16(out) || !host_aligned16(kcache) ||
        !host_aligned16(vcache))
        LLMK_FAIL("attention_tc: q, out and the cache must start on 16-byte boundaries with row strides that are multiples of 8");
    if (nkv > 65535) LLMK_FAIL("attention_tc: grid too large");
    Params p;
    const int G = nq / nkv;
    p.gc = group_chunk(G);
    p.bq = bq;
    p.chunks = G / p.gc;
    p.out = (bf16*)out;
    p.o_stride = o_stride;
    p.block_tables = block_tables;
    p.ctx_len = ctx_len;
    p.cu_q = cu_q;
    p.tile_seq = tile_seq;
    p.tile_q0 = tile_q0;
    p.error_flag = error_flag;
    p.max_blocks = max_blocks;
    p.nq = nq;
    p.nkv = nkv;
    p.page_size = page_size;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.v_lbo = v_lbo ? v_lbo : (unsigned)(BN * 128);
    p.v_sbo = v_sbo ? v_sbo : 1024u;
    CUtensorMap mq, mk, mv;
    if (!tc_host::make_map_bf16_3d(&mq, q, hd, nq, n_tokens, hd, q_stride, p.gc, p.bq))
        LLMK_FAIL("attention_tc: cuTensorMapEncodeTiled failed for q");
    const uint64_t rows = (uint64_t)num_pages * nkv * page_size;
    if (!tc_host::cached_map_bf16_2d(&mk, kcache, rows, hd, hd, page_size) ||
        !tc_host::cached_map_bf16_2d(&mv, vcache, rows, hd, hd, page_size))
        LLMK_FAIL("attention_tc: cuTensorMapEncodeTiled failed for the cache");
    if (n_tiles > 65535) LLMK_FAIL("attention_tc: %d tiles of queries in one launch (limit 65535)", n_tiles);
    dim3 grid(nkv * p.chunks, n_tiles);
    cudaStream_t s = (cudaStream_t)stream;
    switch (page_size) {
        case 16: return hd == 128 ? launch<128, 16>(mq, mk, mv, p, grid, s) : launch<64, 16>(mq, mk, mv, p, grid, s);
        case 32: return hd == 128 ? launch<128, 32>(mq, mk, mv, p, grid, s) : launch<64, 32>(mq, mk, mv, p, grid, s);
        case 64: return hd == 128 ? launch<128, 64>(mq, mk, mv, p, grid, s) : launch<64, 64>(mq, mk, mv, p, grid, s);
        default: return hd == 128 ? launch<128, 128>(mq, mk, mv, p, grid, s) : launch<64, 128>(mq, mk, mv, p, grid, s);
    }
}
