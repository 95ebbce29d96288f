// Attention of single decoded tokens over the paged cache in bfloat16, shaped for memory bandwidth:
// flash-decoding with the merge of the key parts fused into the same kernel.
//
// Grid (parts, kv heads x head chunks, sequences), 128 threads.  A block owns one sequence, one kv
// head, up to GC query heads of its group (they share every K and V row that is read) and one part
// of the visible keys [lo, ctx), where lo = max(0, ctx - window) for a windowed layer: the visible
// range is cut evenly into `parts` pieces, so the launch shape does not depend on the context
// lengths (a CUDA graph replays it).
//   stream   every warp takes 16 of each 64 keys and brings their K and V rows into shared memory
//            through a cp.async ring of its own (3 stages; keys past the part's end are zero-filled),
//            so the loop has no block-wide barrier.  Both products of a step run on the tensor cores
//            (`mma.sync.m16n8k16`: the chunk's heads are the rows of Q, which sits in registers
//            pre-multiplied by scale; K through `ldmatrix`, V through `ldmatrix.trans`), with a running
//            (m, l, acc) per head in float32.  The four warps' states are merged at the end.
//   merge    with 2 to 8 parts the launch makes the parts of a (sequence, kv head) one thread-block
//            cluster: the blocks leave their sums in shared memory and, after the cluster's barrier,
//            each merges a share of the outputs reading the others' shared memory.  With more parts
//            (long contexts) the block writes its un-normalised sums and (m, l) to scratch and takes
//            a ticket from a per-(sequence, head chunk) counter; the block that draws the last ticket
//            merges all parts in part order, sum_p e^{m_p - M} o_p / sum_p e^{m_p - M} l_p, writes
//            the output row and resets the counter.  The result does not depend on which block
//            merges.  Counters must be zero before the first launch and are left zero.
// A sequence with ctx <= 0 (a padding row of a captured batch) gets zeros.
//
// Optionally the kernel starts from the packed q/k/v projection (bfloat16 rows or the float32 slices
// of a product cut along K) and does the per-head RMSNorm, the rotary encoding and the cache write
// itself: every block makes its q heads, and the block whose part holds the sequence's newest
// position makes that position's k and v, stores them in the cache and then reads them back with
// the rest of its keys.  That saves the launch of csrc/attn_prep.cu in a decode step.
//
// Same algorithm as the reference's `attn_decode_kernel<G>` + `attn_decode_reduce_kernel`
// (src/backend/cuda/attention/attention.cu:51-207): one block per (kv head, sequence, part), the
// group's heads share K/V reads, three phases, partial (m, l, o) merged afterwards; here the merge
// needs no second launch, any group size is taken (chunks of up to 8 heads), head_dim is 64 or
// 128, and a window is cut into parts too.  Other head sizes use csrc/attention.cu.
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

namespace {

constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;

struct DecodeParams {
    const bf16* q;
    const bf16* kcache;
    const bf16* vcache;
    bf16* out;
    const int* block_tables;
    const int* ctx_len;
    const int* cu_q;
    float* part_o;       // [tokens][nq][parts][hd]
    float* part_ml;      // [tokens][nq][parts][2]
    int* counters;       // [sequences][gridDim.y]
    long long q_stride, o_stride;
    int max_blocks, nq, nkv, log2_page, window, chunks, page_cap;
    int cluster_merge;   // the blocks of a sequence's parts are a thread-block cluster and merge through shared memory
    float scale;
    // With `packed` set, q is not read from `q`: the block makes it (and, in the block that owns the
    // sequence's newest key, k and v, which it also writes to the cache) from the packed projection
    // rows [q heads | k heads | v heads]: per-head RMSNorm of q and k, then rotary encoding.
    const void* packed;          // bfloat16 rows, or float32 partial sums (splits > 0)
    long long packed_stride, split_stride;
    int splits, nk, rot;         // nk: k (and v) heads present in the packed rows (0: q only)
    const int* positions;
    const int* slots;
    const float* cos_tab;
    const float* sin_tab;
    const float* q_gain;
    const float* k_gain;
    float eps, q_off, k_off;
    int* error_flag;             // raised (2) when a sequence is longer than the bound the launch was sized for
};

// One head's row of the packed projection: lane holds the values lane, lane + 32, ... of the head
// (slices added in order), optionally normalised (RMSNorm over the head, gain + offset) and rotated
// (half-split pairs (i, i + rot / 2), rot a multiple of 64, so that a pair sits in one lane).
// What a head's preparation needs besides the row itself and what no kernel of the step writes: this
// lane's gains (offset added) for q and k rows and its cos / sin values at the token's position.  Loaded
// before the wait for the kernel that makes the row.
template <int HD>
struct HeadConsts {
    float gq[HD / 32], gk[HD / 32], cs[HD / 64], sn[HD / 64];
};
template <int HD>
__device__ __forceinline__ void load_head_consts(const DecodeParams& p, int t, int lane, HeadConsts<HD>& hc) {
    constexpr int VPL = HD / 32;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        hc.gq[i] = p.q_gain ? p.q_gain[lane + 32 * i] + p.q_off : 1.f;
        hc.gk[i] = p.k_gain ? p.k_gain[lane + 32 * i] + p.k_off : 1.f;
    }
    const int half = p.rot / 2, hv = half / 32;
    const int pos = p.cos_tab ? p.positions[t] : 0;
#pragma unroll
    for (int i = 0; i < VPL / 2; ++i) {
        const bool on = p.cos_tab && i < hv;
        hc.cs[i] = on ? p.cos_tab[(size_t)pos * half + lane + 32 * i] : 1.f;
        hc.sn[i] = on ? p.sin_tab[(size_t)pos * half + lane + 32 * i] : 0.f;
    }
}

template <int HD>
__device__ __forceinline__ void prep_head(const DecodeParams& p, int t, int head_in_row, const float* gain,
                                          const float (&gvals)[HD / 32], const HeadConsts<HD>& hc,
                                          bool rotate, int lane, float (&vals)[HD / 32]) {
    constexpr int VPL = HD / 32;
    const size_t base = (size_t)t * p.packed_stride + (size_t)head_in_row * HD;
    if (p.splits == 0) {
        const bf16* x = static_cast<const bf16*>(p.packed) + base;
#pragma unroll
        for (int i = 0; i < VPL; ++i) vals[i] = to_float(x[lane + 32 * i]);
    } else {
        const float* x = static_cast<const float*>(p.packed) + base;
#pragma unroll
        for (int i = 0; i < VPL; ++i) vals[i] = 0.f;
#pragma unroll 4
        for (int sp = 0; sp < p.splits; ++sp)
#pragma unroll
            for (int i = 0; i < VPL; ++i) vals[i] += __ldcg(x + (size_t)sp * p.split_stride + lane + 32 * i);
    }
    if (gain) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) ss += vals[i] * vals[i];
        ss = warp_sum(ss);
        const float rinv = 1.0f / sqrtf(ss / (float)HD + p.eps);
#pragma unroll
        for (int i = 0; i < VPL; ++i) vals[i] = vals[i] * rinv * gvals[i];
    }
    if (rotate && p.cos_tab) {
        const int hv = p.rot / 64;              // values per lane in each half of the rotated part
#pragma unroll
        for (int i = 0; i < VPL / 2; ++i) {
            if (i < hv) {
                const float x0 = vals[i], x1 = vals[i + hv], cs = hc.cs[i], sv = hc.sn[i];
                vals[i] = x0 * cs - x1 * sv;
                vals[i + hv] = x1 * cs + x0 * sv;
            }
        }
    }
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;     // 0: the 16 bytes are zero-filled, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int HD, int GC>
struct DecodeSmem {
    static constexpr int KPW = 16;                            // keys a warp takes per step
    static constexpr int STAGES = 3;
    static constexpr int ROW = HD * 2;                        // bytes of one key's K or V row
    static constexpr int STAGE = 2 * KPW * ROW;               // one warp's stage: KPW rows of K, then of V
    static constexpr int KV_OFF = 0;                          // [WARPS][STAGES][STAGE]
    static constexpr int Q_OFF = KV_OFF + WARPS * STAGES * STAGE;   // float [GC][HD]
    static constexpr int MRG_OFF = Q_OFF + GC * HD * 4;       // float [WARPS][GC][HD + 2]
    static constexpr int PAGES_OFF = MRG_OFF + WARPS * GC * (HD + 2) * 4;
    static size_t bytes(int page_cap) { return (size_t)PAGES_OFF + (size_t)page_cap * 4; }
};

// Tensor-core helpers (warp-level `mma.sync`, enough for a kernel bound by memory).
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr) : "memory");
}
// d (16 x 8, float32) += a (16 x 16, bfloat16, row-major) * b (16 x 8, bfloat16, column-major)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// The two products of a step of 16 keys run on the tensor cores (`mma.sync.m16n8k16`, the chunk's heads
// are the rows of a 16-row tile): float32 arithmetic on the CUDA cores took about eight times the
// instructions per key and, with many heads per kv head, was bound by them and not by memory.
template <int HD, int GC>
__global__ void __launch_bounds__(THREADS) attention_decode_kernel(const DecodeParams p) {
    using L = DecodeSmem<HD, GC>;
    constexpr int KPW = L::KPW;         // keys a warp takes per step
    constexpr int STAGES = L::STAGES;   // depth of each warp's cp.async ring
    constexpr int DPL = HD / 32;        // values of a head per lane when a warp holds one row
    constexpr int CPR = HD / 8;         // 16-byte chunks per row
    constexpr int CPL = KPW * CPR / 32; // chunks of K (and of V) a lane copies per stage
    extern __shared__ __align__(16) unsigned char smem[];
    float* q_s = reinterpret_cast<float*>(smem + L::Q_OFF);
    float* mrg = reinterpret_cast<float*>(smem + L::MRG_OFF);
    int* pages_s = reinterpret_cast<int*>(smem + L::PAGES_OFF);
    __shared__ int is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int part = blockIdx.x, parts = gridDim.x;
    const int kvh = blockIdx.y / p.chunks, chunk = blockIdx.y % p.chunks;
    const int s = blockIdx.z;
    const int G = p.nq / p.nkv;
    const int g0 = chunk * GC;                      // first head of the chunk inside the group
    const int n_heads = min(GC, G - g0);
    pdl_launch_dependents();
    // What the step's arrays say (lengths, block tables) was uploaded before the step, and the cache holds
    // earlier steps' keys: with the fused preparation only the packed projection comes from the kernel
    // before this one, so the wait for it stands after the first copies of keys have been issued.
    const bool fused = p.packed != nullptr;
    if (!fused) pdl_wait();
    const int ctx = p.ctx_len[s];
    const int t = p.cu_q[s];
    if (ctx <= 0) {
        if (fused) pdl_wait();          // the output rows may still be read by a kernel before the one before
        if (part == 0)
            for (int i = tid; i < n_heads * HD; i += THREADS)
                p.out[(size_t)t * p.o_stride + (size_t)(kvh * G + g0) * HD + i] = from_float<bf16>(0.f);
        return;
    }
    const int lo = p.window > 0 ? max(0, ctx - p.window) : 0;
    const int part_len = ceil_div(ceil_div(ctx - lo, parts), KPW) * KPW;
    const int k_beg = lo + part * part_len;
    const int k_end = min(ctx, k_beg + part_len);
    const int n_keys = max(0, k_end - k_beg);
    const int lps = p.log2_page, ps_mask = (1 << p.log2_page) - 1;
    const int page_base = k_beg >> lps;
    const int n_pages = n_keys > 0 ? ((k_end - 1) >> lps) - page_base + 1 : 0;
    const int* bt = p.block_tables + (size_t)s * p.max_blocks;

    if (n_pages > p.page_cap) {
        // ctx_len[s] exceeds the `max_ctx` this launch was sized for: the part's page ids would not fit the
        // shared array.  Nothing is read or written for this block; the host sees the flag.
        if (tid == 0 && p.error_flag) atomicExch(p.error_flag, 2);
        if (p.cluster_merge) {           // the other blocks of the cluster wait at both barriers
            cluster_sync_all();
            cluster_sync_all();
        } else if (parts > 1 && tid == 0) {
            // still draw the ticket, so that the counter is back at zero after the launch
            int* counter = p.counters + (size_t)s * gridDim.y + blockIdx.y;
            if (atomicAdd(counter, 1) == parts - 1) *counter = 0;
        }
        return;
    }
    // The part's page ids first: the copies of keys need them.
    for (int i = tid; i < n_pages; i += THREADS) pages_s[i] = bt[page_base + i];
    __syncthreads();

    // Each warp streams the keys it is given (KPW of every WARPS * KPW) through a cp.async ring of
    // its own, so the loop needs no block-wide barrier.  K rows are stored with their 16-byte chunks
    // swizzled by the key's parity: the four lanes of two neighbouring keys then read eight different
    // bank groups.  Keys past the part's end are zero-filled.
    const int n_steps = ceil_div(n_keys, WARPS * KPW);
    unsigned char* ring = smem + L::KV_OFF + warp * STAGES * L::STAGE;
    // When a step's 8 keys always lie in one page (parts start on multiples of 8 and pages hold a
    // multiple of 8 keys) the page is looked up once per step and every copy's source is a constant
    // offset from the page's row: a handful of instructions per copy instead of a dozen.
    const bool one_page = ((k_beg & (KPW - 1)) == 0) && (((ps_mask + 1) & (KPW - 1)) == 0);
    const size_t lane_off = (size_t)(lane / CPR) * HD + (size_t)(lane % CPR) * 8;     // this lane's first copy inside the 8 rows
    // where a 16-byte chunk of a row goes: XORed with the key's low 3 bits, which is what `ldmatrix`
    // needs to read 8 rows without bank conflicts
    auto k_chunk = [](int key, int l) { return l ^ (key & 7); };
    auto v_chunk = [](int key, int l) { return l ^ (key & 7); };
    constexpr int KSTEP = 32 / CPR;       // keys between two copies of one lane
    auto issue = [&](int step, int stage) {
        unsigned char* dst = ring + stage * L::STAGE;
        const int kidx0 = step * (WARPS * KPW) + warp * KPW;
        if (one_page) {
            const int kpos0 = k_beg + min(kidx0, max(n_keys - 1, 0));
            const int page = pages_s[(kpos0 >> lps) - page_base];
            const size_t row0 = ((((size_t)page * p.nkv + kvh) << lps) + (kpos0 & ps_mask)) * HD + lane_off;
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                // copy i of this lane: key (lane / CPR) + i * KSTEP, the same 16-byte chunk of the row
                const int key = lane / CPR + i * KSTEP, l = lane % CPR;
                const bool valid = kidx0 + key < n_keys;
                const size_t off = row0 + (size_t)(i * KSTEP) * HD;
                cp_async_16(dst + key * L::ROW + (k_chunk(key, l) << 4), p.kcache + off, valid);
                cp_async_16(dst + KPW * L::ROW + key * L::ROW + (v_chunk(key, l) << 4), p.vcache + off, valid);
            }
        } else {
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                const int c = lane + 32 * i;
                const int key = c / CPR, l = c % CPR;
                const int kidx = kidx0 + key;
                const bool valid = kidx < n_keys;
                const int kpos = k_beg + (valid ? kidx : 0);
                const int page = pages_s[(kpos >> lps) - page_base];
                const size_t off = ((((size_t)page * p.nkv + kvh) << lps) + (kpos & ps_mask)) * HD + l * 8;
                cp_async_16(dst + key * L::ROW + (k_chunk(key, l) << 4), p.kcache + off, valid);
                cp_async_16(dst + KPW * L::ROW + key * L::ROW + (v_chunk(key, l) << 4), p.vcache + off, valid);
            }
        }
        cp_async_commit();
    };
    // In the block that will write the newest key to the cache, copies that would read that key must wait
    // for the write; they are among the first STAGES - 1 steps only when the part is that short.
    const bool newest_here = fused && p.nk > 0 && k_beg <= ctx - 1 && ctx - 1 < k_end;
    const bool early = fused && !(newest_here && n_steps <= STAGES - 1);
    auto first_copies = [&]() {
#pragma unroll
        for (int st = 0; st < STAGES - 1; ++st) {
            if (st < n_steps) issue(st, st); else cp_async_commit();
        }
    };
    if (early) first_copies();
    HeadConsts<HD> hc;
    if (fused) {
        load_head_consts<HD>(p, t, lane, hc);
        pdl_wait();
    }

    // The part's page ids and q (float32, pre-multiplied by scale; zeros for heads beyond the group).
    if (p.packed == nullptr) {
        for (int i = tid; i < GC * HD; i += THREADS) {
            const int g = i / HD;
            q_s[i] = g < n_heads ? to_float(p.q[(size_t)t * p.q_stride + (size_t)(kvh * G + g0 + g) * HD + i % HD]) * p.scale : 0.f;
        }
    } else {
        // A warp per row of the packed projection: the chunk's q heads, and in the block whose part
        // holds the newest position also this kv head's k and v, which go to the cache before the
        // block reads its keys (other blocks of the same kv head write the same values).
        const bool newest = p.nk > 0 && k_beg <= ctx - 1 && ctx - 1 < k_end;
        const int n_tasks = GC + (newest ? 2 : 0);
        for (int task = warp; task < n_tasks; task += WARPS) {
            float vals[DPL];
            if (task < GC) {
                if (task < n_heads) {
                    prep_head<HD>(p, t, kvh * G + g0 + task, p.q_gain, hc.gq, hc, true, lane, vals);
#pragma unroll
                    for (int i = 0; i < DPL; ++i) q_s[task * HD + lane + 32 * i] = vals[i] * p.scale;
                } else {
#pragma unroll
                    for (int i = 0; i < DPL; ++i) q_s[task * HD + lane + 32 * i] = 0.f;
                }
            } else {
                const bool is_v = task == GC + 1;
                prep_head<HD>(p, t, p.nq + (is_v ? p.nk : 0) + kvh, is_v ? nullptr : p.k_gain, hc.gk, hc, !is_v, lane, vals);
                const int slot = p.slots ? p.slots[t] : -1;
                if (slot >= 0) {
                    bf16* dst = const_cast<bf16*>(is_v ? p.vcache : p.kcache) +
                                ((((size_t)(slot >> lps)) * p.nkv + kvh) * (size_t)(ps_mask + 1) + (slot & ps_mask)) * HD;
#pragma unroll
                    for (int i = 0; i < DPL; ++i) dst[lane + 32 * i] = from_float<bf16>(vals[i]);
                }
            }
        }
    }
    __syncthreads();


    if (!early) first_copies();

    {
        // Lane (g = lane / 4, t = lane % 4) of a warp holds, of every
        // 16 x 8 accumulator tile, row g columns 2t, 2t + 1 (and row g + 8, which no head uses: a
        // chunk has at most 8 heads).  Q's rows are the chunk's heads.
        const int g = lane >> 2, t4 = lane & 3;
        uint32_t qa[HD / 16][4];
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            const float* qrow = q_s + (g < GC ? g : 0) * HD + kk * 16 + 2 * t4;
            qa[kk][0] = g < GC ? pack_bf16x2(qrow[0], qrow[1]) : 0u;
            qa[kk][1] = 0u;
            qa[kk][2] = g < GC ? pack_bf16x2(qrow[8], qrow[9]) : 0u;
            qa[kk][3] = 0u;
        }
        float m_run = -INFINITY, l_run = 0.f;
        float o[HD / 8][4];
#pragma unroll
        for (int nt = 0; nt < HD / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[nt][e] = 0.f;
        const uint32_t ring_addr = (uint32_t)__cvta_generic_to_shared(ring);
        // ldmatrix row addresses: lane i gives row i % 8 of matrix i / 8
        const int lm_row = lane & 7, lm_mat = lane >> 3;
        for (int step = 0; step < n_steps; ++step) {
            const int stage = step % STAGES;
            if (step + STAGES - 1 < n_steps) issue(step + STAGES - 1, (step + STAGES - 1) % STAGES); else cp_async_commit();
            cp_async_wait<STAGES - 1>();
            __syncwarp();
            const uint32_t Ks = ring_addr + stage * L::STAGE;
            const uint32_t Vs = Ks + KPW * L::ROW;
            const int kidx0 = step * (WARPS * KPW) + warp * KPW;
            // S = Q K^T for two tiles of 8 keys
            float sc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[nt][e] = 0.f;
#pragma unroll
                for (int kk = 0; kk < HD / 16; kk += 2) {
                    // four 8 x 8 matrices: keys nt*8.., head values [kk*16, +8), [kk*16+8, +8), [(kk+1)*16, +8), [(kk+1)*16+8, +8)
                    const int key = nt * 8 + lm_row, chunk = kk * 2 + lm_mat;
                    uint32_t b[4];
                    ldmatrix_x4(b, Ks + key * L::ROW + ((chunk ^ (key & 7)) << 4));
                    mma_16816(sc[nt], qa[kk], b[0], b[1]);
                    mma_16816(sc[nt], qa[kk + 1], b[2], b[3]);
                }
            }
            // online softmax of row g over the step's 16 keys: this lane has keys 2t, 2t+1, 8+2t, 8+2t+1
            float pv[4];
            float mx = -INFINITY;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = (e >> 1) * 8 + 2 * t4 + (e & 1);
                pv[e] = kidx0 + key < n_keys ? sc[e >> 1][e & 1] : -INFINITY;
                mx = fmaxf(mx, pv[e]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run, mx);
            const float alpha = (m_run == -INFINITY) ? 0.f : __expf(m_run - m_new);
            float sum = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                pv[e] = pv[e] == -INFINITY ? 0.f : __expf(pv[e] - m_new);
                sum += pv[e];
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l_run = l_run * alpha + sum;
            m_run = m_new;
#pragma unroll
            for (int nt = 0; nt < HD / 8; ++nt) {
                o[nt][0] *= alpha;
                o[nt][1] *= alpha;
            }
            // P (16 heads x 16 keys) as the A operand: the accumulator layout of the two key tiles is it
            uint32_t pa[4];
            pa[0] = pack_bf16x2(pv[0], pv[1]);
            pa[1] = 0u;
            pa[2] = pack_bf16x2(pv[2], pv[3]);
            pa[3] = 0u;
            // O += P V: V rows are keys; ldmatrix.trans hands out the column-major fragments
#pragma unroll
            for (int nt = 0; nt < HD / 8; nt += 2) {
                // matrices: (keys 0-7, values nt*8..), (keys 8-15, same), (keys 0-7, values (nt+1)*8..), (keys 8-15, same)
                const int key = (lm_mat & 1) * 8 + lm_row, chunk = nt + (lm_mat >> 1);
                uint32_t b[4];
                ldmatrix_x4_trans(b, Vs + key * L::ROW + ((chunk ^ (key & 7)) << 4));
                mma_16816(o[nt], pa, b[0], b[1]);
                mma_16816(o[nt + 1], pa, b[2], b[3]);
            }
            __syncwarp();    // every lane has read the stage before it is refilled
        }
        cp_async_wait<0>();
        if (g < GC) {
            float* row = mrg + (warp * GC + g) * (HD + 2);
#pragma unroll
            for (int nt = 0; nt < HD / 8; ++nt) {
                row[nt * 8 + 2 * t4] = o[nt][0];
                row[nt * 8 + 2 * t4 + 1] = o[nt][1];
            }
            if (t4 == 0) {
                row[HD] = m_run;
                row[HD + 1] = l_run;
            }
        }
    }
    __syncthreads();
    auto merged = [&](int g, int d, float& M, float& Lsum) -> float {
        M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, mrg[(w * GC + g) * (HD + 2) + HD]);
        float o = 0.f;
        Lsum = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float* row = mrg + (w * GC + g) * (HD + 2);
            const float e = row[HD] == -INFINITY ? 0.f : __expf(row[HD] - M);
            o += e * row[d];
            Lsum += e * row[HD + 1];
        }
        return o;
    };

    // ---- the block's result
    if (parts == 1) {
        for (int i = tid; i < n_heads * HD; i += THREADS) {
            float M, Ls;
            const float o = merged(i / HD, i % HD, M, Ls);
            p.out[(size_t)t * p.o_stride + (size_t)(kvh * G + g0) * HD + i] = from_float<bf16>(Ls > 0.f ? o / Ls : 0.f);
        }
        return;
    }
    if (p.cluster_merge) {
        // The parts of this (sequence, kv head) are the blocks of one cluster: each leaves its sums in its
        // own shared memory (over q, which is no longer read), and after the cluster's barrier block r
        // merges outputs r * THREADS + tid, ... reading the others' shared memory: no trip through global
        // memory, no ticket.  Nobody leaves before all have read.
        __shared__ float res_ml[2 * GC];
        __syncthreads();                 // every warp is done with q_s
        for (int i = tid; i < n_heads * HD; i += THREADS) {
            float M, Ls;
            q_s[i] = merged(i / HD, i % HD, M, Ls);
            if (i % HD == 0) {
                res_ml[2 * (i / HD)] = M;
                res_ml[2 * (i / HD) + 1] = Ls;
            }
        }
        cluster_sync_all();
        const uint32_t o_base = (uint32_t)__cvta_generic_to_shared(q_s), ml_base = (uint32_t)__cvta_generic_to_shared(res_ml);
        for (int i = part * THREADS + tid; i < n_heads * HD; i += parts * THREADS) {
            const int g = i / HD;
            float ms[8], ls[8], os[8];
#pragma unroll
            for (int pt = 0; pt < 8; ++pt) {
                const bool on = pt < parts;
                ms[pt] = on ? cluster_ld_f32(cluster_map_shared(ml_base + (uint32_t)(2 * g) * 4u, pt)) : -INFINITY;
                ls[pt] = on ? cluster_ld_f32(cluster_map_shared(ml_base + (uint32_t)(2 * g + 1) * 4u, pt)) : 0.f;
                os[pt] = on ? cluster_ld_f32(cluster_map_shared(o_base + (uint32_t)i * 4u, pt)) : 0.f;
            }
            float M = -INFINITY;
#pragma unroll
            for (int pt = 0; pt < 8; ++pt)
                if (ls[pt] > 0.f) M = fmaxf(M, ms[pt]);
            float denom = 0.f, v = 0.f;
#pragma unroll
            for (int pt = 0; pt < 8; ++pt) {
                if (ls[pt] > 0.f) {
                    const float e = __expf(ms[pt] - M);
                    denom += e * ls[pt];
                    v += e * os[pt];
                }
            }
            p.out[(size_t)t * p.o_stride + (size_t)(kvh * G + g0) * HD + i] = from_float<bf16>(denom > 0.f ? v / denom : 0.f);
        }
        cluster_sync_all();
        return;
    }
    for (int i = tid; i < n_heads * HD; i += THREADS) {
        const int g = i / HD, d = i % HD;
        float M, Ls;
        const float o = merged(g, d, M, Ls);
        const size_t row = ((size_t)t * p.nq + kvh * G + g0 + g) * parts + part;
        p.part_o[row * HD + d] = o;
        if (d == 0) {
            p.part_ml[row * 2] = M;
            p.part_ml[row * 2 + 1] = Ls;
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* counter = p.counters + (size_t)s * gridDim.y + blockIdx.y;
        const int ticket = atomicAdd(counter, 1);
        is_last = ticket == parts - 1;
        if (is_last) *counter = 0;     // every other block of this (sequence, chunk) has already drawn
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // (m, l) of every part of the chunk's heads into shared memory, then each thread merges one
    // output value with independent loads of the parts' sums, in part order.
    float* ml_s = mrg;      // [n_heads][parts][2], fits: parts <= 128
    for (int i = tid; i < n_heads * parts * 2; i += THREADS) {
        const int g = i / (parts * 2);
        ml_s[i] = __ldcg(p.part_ml + ((size_t)t * p.nq + kvh * G + g0 + g) * parts * 2 + i % (parts * 2));
    }
    __syncthreads();
    for (int i = tid; i < n_heads * HD; i += THREADS) {
        const int g = i / HD, d = i % HD;
        const float* ml = ml_s + g * parts * 2;
        const float* po = p.part_o + ((size_t)t * p.nq + kvh * G + g0 + g) * parts * HD + d;
        float M = -INFINITY;
        for (int pt = 0; pt < parts; ++pt)
            if (ml[2 * pt + 1] > 0.f) M = fmaxf(M, ml[2 * pt]);
        float denom = 0.f, v = 0.f;
        for (int pt0 = 0; pt0 < parts; pt0 += 8) {
            float o[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) o[u] = pt0 + u < parts ? __ldcg(po + (size_t)(pt0 + u) * HD) : 0.f;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (pt0 + u < parts) {
                    const float lp = ml[2 * (pt0 + u) + 1];
                    if (lp > 0.f) {
                        const float e = __expf(ml[2 * (pt0 + u)] - M);
                        denom += e * lp;
                        v += e * o[u];
                    }
                }
            }
        }
        p.out[(size_t)t * p.o_stride + (size_t)(kvh * G + g0) * HD + i] = from_float<bf16>(denom > 0.f ? v / denom : 0.f);
    }
}

int g_cluster_merge = 1;      // 0: always merge through global memory and a ticket (for measurements)

template <int HD, int GC>
int launch(const DecodeParams& p, dim3 grid, cudaStream_t s) {
    const size_t smem = DecodeSmem<HD, GC>::bytes(p.page_cap);
    auto kernel = attention_decode_kernel<HD, GC>;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LLMK_FAIL("attention_decode: cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
        configured = smem;
    }
    if (p.cluster_merge)
        LLMK_CHECK_LAUNCH_RC("attention_decode", llmk_launch_clusters(kernel, grid, dim3(THREADS), smem, s, true, dim3(grid.x, 1, 1), p));
    else
        LLMK_CHECK_LAUNCH_RC("attention_decode", llmk_launch(kernel, grid, dim3(THREADS), smem, s, true, p));
    return LLMK_OK;
}

template <int HD>
int dispatch_group(int gc, const DecodeParams& p, dim3 grid, cudaStream_t s) {
    switch (gc) {
        case 1: return launch<HD, 1>(p, grid, s);
        case 2: return launch<HD, 2>(p, grid, s);
        case 4: return launch<HD, 4>(p, grid, s);
        default: return launch<HD, 8>(p, grid, s);
    }
}

int chunk_heads(int G) { return G <= 1 ? 1 : G <= 2 ? 2 : G <= 4 ? 4 : 8; }

}  // namespace

// 1 if the kernel takes these sizes.
LLMK_EXPORT int llmk_attention_decode_usable(int nq, int nkv, int hd, int page_size) {
    if (nkv <= 0 || nq <= 0 || nq % nkv != 0 || page_size <= 0) return 0;
    if ((page_size & (page_size - 1)) != 0) return 0;       // page and offset of a key by shift and mask
    return (hd == 64 || hd == 128) ? 1 : 0;
}

// Floats of scratch for `n_seqs` sequences cut into `parts`: partial outputs, then (m, l) pairs.
LLMK_EXPORT long long llmk_attention_decode_scratch_floats(int n_seqs, int nq, int hd, int parts) {
    return parts <= 1 ? 0 : (long long)n_seqs * nq * parts * (hd + 2);
}

// Ints of counters for `n_seqs` sequences (zero them once; every launch leaves them zero).
LLMK_EXPORT long long llmk_attention_decode_counters(int n_seqs, int nq, int nkv) {
    if (nkv <= 0) return 0;
    const int G = nq / nkv;
    return (long long)n_seqs * nkv * ceil_div(G, chunk_heads(G));
}

// 1 if the kernel can make q, k and v from the packed projection rows itself for this rotary width.
LLMK_EXPORT int llmk_attention_decode_fuses_prep(int hd, int rot) { return (rot % 64 == 0 && rot <= hd) ? 1 : 0; }

// out[t, nq*hd] for the single token t = cu_q[s] of each of n_seqs sequences.  With `packed` the
// kernel also does what csrc/attn_prep.cu does (see DecodeParams); `q` is then not read.  `max_ctx` bounds every
// ctx_len[s] of this launch (it sizes the shared-memory copy of a part's page ids).
LLMK_EXPORT int llmk_attention_decode(void* out, long long o_stride, const void* q, long long q_stride,
                                      const void* kcache, const void* vcache, const int* block_tables,
                                      int max_blocks, const int* ctx_len, const int* cu_q, int n_seqs, int nq,
                                      int nkv, int hd, int page_size, int window, float scale, int parts,
                                      int max_ctx, float* scratch, int* counters, const void* packed,
                                      long long packed_stride, int splits, long long split_stride, int nk, int rot,
                                      const int* positions, const int* slots, const float* cos_tab,
                                      const float* sin_tab, const float* q_gain, const float* k_gain, float eps,
                                      float q_off, float k_off, int pairing, int head_norm, int* error_flag, void* stream) {
    if (n_seqs <= 0) return LLMK_OK;
    if (packed && pairing != LLMK_PAIR_HALF_SPLIT)
        LLMK_FAIL("attention_decode: rotary pairing %d is not built (0: half-split, pairs (i, i + rot / 2))", pairing);
    if (packed && head_norm != LLMK_HEAD_NORM_RMS) LLMK_FAIL("attention_decode: per-head norm kind %d is not built (0: RMSNorm)", head_norm);
    if (!llmk_attention_decode_usable(nq, nkv, hd, page_size))
        LLMK_FAIL("attention_decode: not taken (heads %d/%d, head_dim %d must be 64 or 128, page size %d must be a power of two)", nq, nkv, hd, page_size);
    if (parts < 1 || parts > 128 || (parts > 1 && (!scratch || !counters)))
        LLMK_FAIL("attention_decode: bad split (%d parts, scratch %p, counters %p)", parts, (void*)scratch, (void*)counters);
    if (n_seqs > 65535) LLMK_FAIL("attention_decode: %d sequences exceed the grid", n_seqs);
    if (!host_aligned16(kcache) || !host_aligned16(vcache))
        LLMK_FAIL("attention_decode: the cache must start on a 16-byte boundary");
    if (!packed && !q) LLMK_FAIL("attention_decode: neither q nor packed projection rows");
    if (packed) {
        if (splits < 0 || (splits > 0 && split_stride <= 0)) LLMK_FAIL("attention_decode: bad partial sums (%d slices)", splits);
        if (nk != 0 && nk != nkv) LLMK_FAIL("attention_decode: packed rows hold %d k heads, the cache %d", nk, nkv);
        if (!cos_tab) rot = 0;
        if (rot % 64 != 0 || rot > hd) LLMK_FAIL("attention_decode: rotary width %d must be a multiple of 64, at most head_dim", rot);
        if (cos_tab && (!sin_tab || !positions)) LLMK_FAIL("attention_decode: rotary tables need sin and positions");
        if (nk > 0 && !slots) LLMK_FAIL("attention_decode: packed k and v need slots");
    }
    DecodeParams p;
    p.packed = packed; p.packed_stride = packed_stride; p.splits = splits; p.split_stride = split_stride;
    p.nk = nk; p.rot = rot; p.positions = positions; p.slots = slots; p.cos_tab = cos_tab; p.sin_tab = sin_tab;
    p.q_gain = q_gain; p.k_gain = k_gain; p.eps = eps; p.q_off = q_off; p.k_off = k_off;
    p.error_flag = error_flag;
    const int G = nq / nkv;
    const int gc = chunk_heads(G);
    p.q = (const bf16*)q; p.kcache = (const bf16*)kcache; p.vcache = (const bf16*)vcache; p.out = (bf16*)out;
    p.block_tables = block_tables; p.ctx_len = ctx_len; p.cu_q = cu_q;
    p.part_o = scratch;
    p.part_ml = parts > 1 ? scratch + (size_t)n_seqs * nq * parts * hd : nullptr;
    p.counters = counters;
    // up to 8 parts (a portable cluster) merge through the cluster's shared memory
    p.cluster_merge = (g_cluster_merge && parts >= 2 && parts <= 8) ? 1 : 0;
    p.q_stride = q_stride; p.o_stride = o_stride; p.max_blocks = max_blocks;
    p.nq = nq; p.nkv = nkv; p.window = window;
    p.log2_page = 0;
    while ((1 << p.log2_page) < page_size) ++p.log2_page;
    p.chunks = ceil_div(G, gc);
    const int visible = window > 0 ? min(window, max_ctx) : max_ctx;
    const int part_cap = ceil_div(ceil_div(max(visible, 1), parts), 16) * 16;
    p.page_cap = part_cap / page_size + 2;       // page ids of one part, kept in shared memory
    p.scale = scale;
    if ((size_t)p.page_cap * 4 > 64 * 1024)
        LLMK_FAIL("attention_decode: %d keys per part in pages of %d need too much shared memory; use more parts", part_cap, page_size);
    dim3 grid(parts, nkv * p.chunks, n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    return hd == 128 ? dispatch_group<128>(gc, p, grid, s) : dispatch_group<64>(gc, p, grid, s);
}

LLMK_EXPORT void llmk_attention_decode_set_cluster_merge(int on) { g_cluster_merge = on; }
