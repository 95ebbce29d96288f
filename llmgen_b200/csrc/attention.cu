// Causal grouped-query attention over the paged key/value cache, float32 arithmetic on the CUDA
// cores, for float32 or bfloat16 storage: the attention of the true 32-bit path, and the general
// kernel of the bfloat16 path for every shape (prompt portions, single decoded tokens and both
// mixed in one batch, any group size, any head_dim that is a multiple of 8 up to 512, a window).
//
// Semantics follow the reference's CPU attention (src/backend/cpu/attention.zig:64-118):
// sequence s owns query rows [cu_q[s], cu_q[s+1]) and has ctx[s] keys after this step; query j
// of the portion sits at position ctx - q_len + j and sees keys 0..position (with a window W:
// the last W of them); score = (q.k) * scale; online softmax with running (m, l) in float32;
// a row with ctx < q_len (padding) gives zeros.  The step's own keys were written to the cache
// before this kernel runs, so everything is read through the block table.
//
// Work split: one block per (tile of queries of one sequence, kv head, head chunk, key part).
// The rows of a block are `bq` queries x `gc` heads of one kv group (<= 16 rows), two rows
// per warp, so each K/V tile of 32 keys is read from the cache once for all of them (the
// reference's decode kernel shares K/V over the group the same way,
// src/backend/cuda/attention/attention.cu:51-184).  With num_parts > 1 (flash-decoding) a block
// covers keys [part * part_size, (part + 1) * part_size) (part_size = 0: an even split of the
// sequence's own keys) and writes un-normalised partial sums
// and (m, l); `llmk_attention_reduce` merges them as
// sum_p e^{m_p - M} o_p / sum_p e^{m_p - M} l_p (attention.cu:186-207 in the reference).
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

constexpr int NWARPS = 8;
constexpr int MAX_ROWS = 16;
constexpr int KT = 32;  // keys per tile

struct AttnParams {
    const void* q;
    const void* kcache;
    const void* vcache;
    void* out;
    const int* block_tables;
    const int* ctx_len;
    const int* cu_q;
    const int* tile_seq;
    const int* tile_q0;
    float* part_o;
    float* part_ml;
    long long q_stride, o_stride;
    int max_blocks, nq, nkv, hd, page_size, window, num_parts, part_size, bq, gc, chunks;
    float scale;
};

template <typename T, int HDL>
__global__ void __launch_bounds__(NWARPS * 32) paged_attention_kernel(AttnParams p) {
    extern __shared__ float smem[];
    const int hd = p.hd;
    float* Qs = smem;                       // [MAX_ROWS][hd], pre-multiplied by scale
    float* Ks = Qs + MAX_ROWS * hd;         // [KT][hd + 1]
    float* Vs = Ks + KT * (hd + 1);         // [KT][hd]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int s = p.tile_seq[blockIdx.x];
    if (s < 0) return;                      // padding of a tile list of fixed length
    const int q0 = p.tile_q0[blockIdx.x];
    const int G = p.nq / p.nkv;
    const int kvh = blockIdx.y / p.chunks;
    const int chunk = blockIdx.y % p.chunks;
    const int part = blockIdx.z;
    const int q_beg = p.cu_q[s];
    const int q_len = p.cu_q[s + 1] - q_beg;
    const int ctx = p.ctx_len[s];
    const int nq_tile = min(p.bq, q_len - q0);
    const bool padding = ctx < q_len || nq_tile <= 0;
    const int first_pos = ctx - q_len + q0;
    int k_beg = 0, k_end = 0;
    if (!padding) {
        k_end = first_pos + nq_tile;
        k_beg = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
    }
    if (p.num_parts > 1) {
        // part_size <= 0: split this sequence's own keys evenly (whole key tiles per part), so the
        // launch shape does not depend on the context lengths.
        int part_size = p.part_size;
        if (part_size <= 0) part_size = ceil_div(ceil_div(max(ctx, 1), p.num_parts), KT) * KT;
        k_beg = max(k_beg, part * part_size);
        k_end = min(k_end, (part + 1) * part_size);
    }
    const T* qbase = static_cast<const T*>(p.q);
    const T* kc = static_cast<const T*>(p.kcache);
    const T* vc = static_cast<const T*>(p.vcache);
    const int* bt = p.block_tables + (size_t)s * p.max_blocks;

    // Rows of this block: r -> (query qi, head hh of the chunk).
    const int rows = p.bq * p.gc;
    for (int idx = threadIdx.x; idx < MAX_ROWS * hd; idx += blockDim.x) {
        const int r = idx / hd, d = idx % hd;
        const int qi = r / p.gc, hh = chunk * p.gc + r % p.gc;
        float v = 0.f;
        if (r < rows && qi < nq_tile && hh < G)
            v = to_float(qbase[(size_t)(q_beg + q0 + qi) * p.q_stride + (size_t)(kvh * G + hh) * hd + d]) * p.scale;
        Qs[idx] = v;
    }
    int r_of[2], qi_of[2], head_of[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        r_of[i] = warp + i * NWARPS;
        qi_of[i] = r_of[i] / p.gc;
        const int hh = chunk * p.gc + r_of[i] % p.gc;
        head_of[i] = kvh * G + hh;
        valid[i] = r_of[i] < rows && qi_of[i] < nq_tile && hh < G && !padding;
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float acc[2][HDL];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < HDL; ++j) acc[i][j] = 0.f;

    constexpr int VN = Vec16<T>::N;
    const int vecs = hd / VN;
    for (int t0 = k_beg; t0 < k_end; t0 += KT) {
        __syncthreads();  // previous tile consumed (and Qs written, first time)
        for (int idx = threadIdx.x; idx < KT * vecs; idx += blockDim.x) {
            const int key = idx / vecs, vec = idx % vecs;
            const int kpos = t0 + key;
            float kf[VN], vf[VN];
            if (kpos < k_end) {
                const int page = bt[kpos / p.page_size];
                const size_t off = (((size_t)page * p.nkv + kvh) * p.page_size + kpos % p.page_size) * hd + (size_t)vec * VN;
                Vec16<T> kv, vv;
                kv.raw = *reinterpret_cast<const decltype(kv.raw)*>(kc + off);
                vv.raw = *reinterpret_cast<const decltype(vv.raw)*>(vc + off);
                kv.unpack(kf);
                vv.unpack(vf);
            } else {
#pragma unroll
                for (int i = 0; i < VN; ++i) kf[i] = vf[i] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < VN; ++i) {
                Ks[key * (hd + 1) + vec * VN + i] = kf[i];
                Vs[key * hd + vec * VN + i] = vf[i];
            }
        }
        __syncthreads();
        if (!valid[0] && !valid[1]) continue;
        // scores of key `lane` for both rows
        float sc[2] = {0.f, 0.f};
        {
            const float* kr = Ks + lane * (hd + 1);
            const float4* qa = reinterpret_cast<const float4*>(Qs + r_of[0] * hd);
            const float4* qb = reinterpret_cast<const float4*>(Qs + (valid[1] ? r_of[1] : r_of[0]) * hd);
            for (int d4 = 0; d4 < hd / 4; ++d4) {
                const float4 a = qa[d4], b = qb[d4];
                const float k0 = kr[4 * d4], k1 = kr[4 * d4 + 1], k2 = kr[4 * d4 + 2], k3 = kr[4 * d4 + 3];
                sc[0] = fmaf(a.x, k0, sc[0]); sc[0] = fmaf(a.y, k1, sc[0]);
                sc[0] = fmaf(a.z, k2, sc[0]); sc[0] = fmaf(a.w, k3, sc[0]);
                sc[1] = fmaf(b.x, k0, sc[1]); sc[1] = fmaf(b.y, k1, sc[1]);
                sc[1] = fmaf(b.z, k2, sc[1]); sc[1] = fmaf(b.w, k3, sc[1]);
            }
        }
        const int kpos = t0 + lane;
        float pr[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int qpos = first_pos + qi_of[i];
            const bool ok = valid[i] && kpos < k_end && kpos <= qpos && (p.window <= 0 || kpos > qpos - p.window);
            const float sv = ok ? sc[i] : -INFINITY;
            const float tmax = warp_max(sv);
            const float m_new = fmaxf(m[i], tmax);
            float corr = 1.f;
            pr[i] = 0.f;
            if (m_new > -INFINITY) {
                corr = m[i] > -INFINITY ? expf(m[i] - m_new) : 0.f;
                pr[i] = ok ? expf(sv - m_new) : 0.f;
                m[i] = m_new;
            }
            l[i] = l[i] * corr + warp_sum(pr[i]);
#pragma unroll
            for (int j = 0; j < HDL; ++j) acc[i][j] *= corr;
        }
        const int kmax = min(KT, k_end - t0);
        for (int k = 0; k < kmax; ++k) {
            const float p0 = __shfl_sync(0xffffffffu, pr[0], k);
            const float p1 = __shfl_sync(0xffffffffu, pr[1], k);
            const float* vr = Vs + k * hd;
#pragma unroll
            for (int j = 0; j < HDL; ++j) {
                const int d = lane + 32 * j;
                if (d < hd) {
                    const float v = vr[d];
                    acc[0][j] = fmaf(p0, v, acc[0][j]);
                    acc[1][j] = fmaf(p1, v, acc[1][j]);
                }
            }
        }
    }

    // Write the rows this warp owns (also when no key was visible: zeros / empty partials).
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int hh = chunk * p.gc + r_of[i] % p.gc;
        const bool owned = r_of[i] < rows && qi_of[i] < max(nq_tile, 0) && hh < G;
        if (!owned) continue;
        const size_t tok = (size_t)(q_beg + q0 + qi_of[i]);
        if (p.num_parts > 1) {
            const size_t row = (tok * p.nq + head_of[i]) * p.num_parts + part;
#pragma unroll
            for (int j = 0; j < HDL; ++j) {
                const int d = lane + 32 * j;
                if (d < hd) p.part_o[row * hd + d] = acc[i][j];
            }
            if (lane == 0) {
                p.part_ml[row * 2] = m[i];
                p.part_ml[row * 2 + 1] = l[i];
            }
        } else {
            T* o = static_cast<T*>(p.out) + tok * p.o_stride + (size_t)head_of[i] * hd;
            const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
            for (int j = 0; j < HDL; ++j) {
                const int d = lane + 32 * j;
                if (d < hd) o[d] = from_float<T>(acc[i][j] * inv);
            }
        }
    }
}

// One warp per (token, head): merge the partial results of the key parts.
template <typename T>
__global__ void attention_reduce_kernel(T* __restrict__ out, long long o_stride, const float* __restrict__ part_o,
                                        const float* __restrict__ part_ml, int n_rows, int nq, int hd,
                                        int num_parts) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const float* ml = part_ml + (size_t)row * num_parts * 2;
    float M = -INFINITY;
    for (int pt = 0; pt < num_parts; ++pt)
        if (ml[2 * pt + 1] > 0.f) M = fmaxf(M, ml[2 * pt]);
    float denom = 0.f;
    for (int pt = 0; pt < num_parts; ++pt)
        if (ml[2 * pt + 1] > 0.f) denom += expf(ml[2 * pt] - M) * ml[2 * pt + 1];
    const float inv = denom > 0.f ? 1.0f / denom : 0.f;
    const size_t tok = (size_t)(row / nq), head = (size_t)(row % nq);
    T* o = out + tok * o_stride + head * hd;
    for (int d = lane; d < hd; d += 32) {
        float v = 0.f;
        for (int pt = 0; pt < num_parts; ++pt)
            if (ml[2 * pt + 1] > 0.f) v += expf(ml[2 * pt] - M) * part_o[((size_t)row * num_parts + pt) * hd + d];
        o[d] = from_float<T>(v * inv);
    }
}

static int hdl_of(int hd) { return hd <= 32 ? 1 : hd <= 64 ? 2 : hd <= 128 ? 4 : hd <= 256 ? 8 : 16; }

template <typename T, int HDL>
static int launch_attention(const AttnParams& p, dim3 grid, size_t smem, cudaStream_t s) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(paged_attention_kernel<T, HDL>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LLMK_FAIL("paged_attention: cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
    }
    paged_attention_kernel<T, HDL><<<grid, NWARPS * 32, smem, s>>>(p);
    return LLMK_OK;
}

template <typename T>
static int dispatch_attention(const AttnParams& p, dim3 grid, size_t smem, cudaStream_t s) {
    switch (hdl_of(p.hd)) {
        case 1: return launch_attention<T, 1>(p, grid, smem, s);
        case 2: return launch_attention<T, 2>(p, grid, smem, s);
        case 4: return launch_attention<T, 4>(p, grid, smem, s);
        case 8: return launch_attention<T, 8>(p, grid, smem, s);
        default: return launch_attention<T, 16>(p, grid, smem, s);
    }
}

// Queries per tile for a given group size: rows = bq * gc <= 16.
LLMK_EXPORT int llmk_attention_tile_queries(int nq, int nkv) {
    if (nkv <= 0 || nq <= 0 || nq % nkv != 0) return 0;
    const int G = nq / nkv;
    const int gc = G < MAX_ROWS ? G : MAX_ROWS;
    return MAX_ROWS / gc;
}

// Bytes of scratch for `n_tokens` rows split into `num_parts`: partial outputs then (m, l) pairs.
LLMK_EXPORT long long llmk_attention_scratch_bytes(int n_tokens, int nq, int hd, int num_parts) {
    if (num_parts <= 1) return 0;
    return (long long)n_tokens * nq * num_parts * (hd + 2) * (long long)sizeof(float);
}

LLMK_EXPORT int llmk_paged_attention(void* out, long long o_stride, const void* q, long long q_stride,
                                     const void* kcache, const void* vcache, const int* block_tables,
                                     int max_blocks, const int* ctx_len, const int* cu_q, const int* tile_seq,
                                     const int* tile_q0, int n_tiles, int n_tokens, int nq, int nkv, int hd,
                                     int page_size, int window, float scale, int num_parts, int part_size,
                                     void* scratch, int dtype, void* stream) {
    if (n_tiles <= 0 || n_tokens <= 0) return LLMK_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0) LLMK_FAIL("paged_attention: %d query heads are not a multiple of %d kv heads", nq, nkv);
    if (hd <= 0 || hd % 8 != 0 || hd > 512) LLMK_FAIL("paged_attention: head_dim %d must be a multiple of 8, at most 512", hd);
    if (page_size <= 0) LLMK_FAIL("paged_attention: page_size %d", page_size);
    if (num_parts < 1 || (num_parts > 1 && !scratch)) LLMK_FAIL("paged_attention: bad split (%d parts, scratch %p)", num_parts, scratch);
    if (num_parts > 65535 || nkv > 65535) LLMK_FAIL("paged_attention: grid too large");
    AttnParams p;
    const int G = nq / nkv;
    p.gc = G < MAX_ROWS ? G : MAX_ROWS;
    p.bq = MAX_ROWS / p.gc;
    p.chunks = ceil_div(G, p.gc);
    p.q = q; p.kcache = kcache; p.vcache = vcache; p.out = out;
    p.block_tables = block_tables; p.ctx_len = ctx_len; p.cu_q = cu_q; p.tile_seq = tile_seq; p.tile_q0 = tile_q0;
    p.q_stride = q_stride; p.o_stride = o_stride; p.max_blocks = max_blocks;
    p.nq = nq; p.nkv = nkv; p.hd = hd; p.page_size = page_size; p.window = window;
    p.num_parts = num_parts; p.part_size = part_size; p.scale = scale;
    p.part_o = (float*)scratch;
    p.part_ml = num_parts > 1 ? (float*)scratch + (size_t)n_tokens * nq * num_parts * hd : nullptr;
    const size_t smem = ((size_t)MAX_ROWS * hd + (size_t)KT * (hd + 1) + (size_t)KT * hd) * sizeof(float);
    dim3 grid(n_tiles, nkv * p.chunks, num_parts);
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    if (dtype == LLMK_F32)
        rc = dispatch_attention<float>(p, grid, smem, s);
    else if (dtype == LLMK_BF16)
        rc = dispatch_attention<bf16>(p, grid, smem, s);
    else
        LLMK_FAIL("paged_attention: unknown dtype %d", dtype);
    if (rc != LLMK_OK) return rc;
    LLMK_CHECK_LAUNCH("paged_attention");
    if (num_parts > 1) {
        const int n_rows = n_tokens * nq;
        const int warps = 4;
        const int blocks = ceil_div(n_rows, warps);
        if (dtype == LLMK_F32)
            attention_reduce_kernel<float><<<blocks, warps * 32, 0, s>>>((float*)out, o_stride, p.part_o, p.part_ml, n_rows, nq, hd, num_parts);
        else
            attention_reduce_kernel<bf16><<<blocks, warps * 32, 0, s>>>((bf16*)out, o_stride, p.part_o, p.part_ml, n_rows, nq, hd, num_parts);
        LLMK_CHECK_LAUNCH("attention_reduce");
    }
    return LLMK_OK;
}
