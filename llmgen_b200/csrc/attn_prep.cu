// Between the QKV projection and attention, in one pass over the packed rows:
// per-head RMSNorm of q and k, rotary position encoding of q and k, and the write of k and v
// into the paged cache at this step's slots.
//
// It replaces five launches of the reference: `rmsnorm_head_kernel` on q and on k
// (src/backend/cuda/norm/norm_final.cu:28-45), `rope_kernel` on q and on k
// (src/backend/cuda/rope/rope_v1.cu:11-45) and `store_kv_kernel`
// (src/backend/cuda/attention/attention.cu:18-33).  Those fix head_dim = 128 and at most 32
// heads; here any head_dim up to 512 that is a multiple of 2, any head counts, and a rotary
// width below the head width (src/module/rope.zig:86-88) are taken.
//
// Layouts: qkv[t] = [q heads | k heads | v heads], each head `hd` values, row stride given;
// q is normalised and rotated into `q_out` (which may be the packed rows themselves).  The packed
// rows are of the storage type T, or (splits > 0) `splits` float32 slices [splits][n][row_stride],
// `split_stride` floats apart, added in slice order: the partial sums of a projection cut along K.
// Cache arrays are [page][kv_head][page_size][hd]
// (src/memory/page_atten.zig:2) and slot = page * page_size + offset, slot < 0 = do not store.
// cos/sin tables are float32 [max_positions, rot/2], computed on the host in float64.
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

constexpr int MAX_PAIRS = 8;   // rot/2 <= 256 per lane-strided loop of 32
constexpr int MAX_TAIL = 16;   // hd - rot <= 512

template <typename T>
struct PackedRow {
    const T* x;
    const float* p;
    int splits;
    long long split_stride;
    __device__ __forceinline__ float operator[](int e) const {
        if (splits == 0) return to_float(x[e]);
        float acc = p[e];
        for (int sp = 1; sp < splits; ++sp) acc += p[(size_t)sp * split_stride + e];
        return acc;
    }
};

template <typename T>
__global__ void attn_prep_kernel(const void* __restrict__ qkv, long long row_stride, int splits, long long split_stride,
                                 T* __restrict__ q_out, long long q_stride, T* __restrict__ kcache,
                                 T* __restrict__ vcache, const int* __restrict__ positions,
                                 const int* __restrict__ slots, const float* __restrict__ cos_tab,
                                 const float* __restrict__ sin_tab, const float* __restrict__ q_gain,
                                 const float* __restrict__ k_gain, int n_tokens, int nq, int nk, int nkv_cache,
                                 int hd, int rot, int page_size, float eps, float q_off, float k_off) {
    const int lane = threadIdx.x & 31;
    const int warps_per_block = blockDim.x >> 5;
    const int heads = nq + 2 * nk;
    const long long item = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    if (item >= (long long)n_tokens * heads) return;
    const int t = (int)(item / heads);
    const int h = (int)(item % heads);
    pdl_launch_dependents();
    pdl_wait();
    PackedRow<T> x;
    x.x = static_cast<const T*>(qkv) + (size_t)t * row_stride + (size_t)h * hd;
    x.p = static_cast<const float*>(qkv) + (size_t)t * row_stride + (size_t)h * hd;
    x.splits = splits;
    x.split_stride = split_stride;
    const int slot = slots ? slots[t] : -1;

    if (h >= nq + nk) {  // a value head: copy into the cache
        if (slot < 0 || !vcache) return;
        const int kvh = h - nq - nk;
        T* dst = vcache + (((size_t)(slot / page_size) * nkv_cache + kvh) * page_size + slot % page_size) * hd;
        if (splits == 0) {
            for (int i = lane; i < hd; i += 32) dst[i] = x.x[i];
            return;
        }
        float vv[MAX_TAIL];
#pragma unroll
        for (int i = 0; i < MAX_TAIL; ++i) vv[i] = 0.f;
#pragma unroll 4
        for (int sp = 0; sp < splits; ++sp) {
            const float* ps = x.p + (size_t)sp * split_stride;
#pragma unroll
            for (int i = 0; i < MAX_TAIL; ++i)
                if (lane + 32 * i < hd) vv[i] += __ldcg(ps + lane + 32 * i);
        }
#pragma unroll
        for (int i = 0; i < MAX_TAIL; ++i)
            if (lane + 32 * i < hd) dst[lane + 32 * i] = from_float<T>(vv[i]);
        return;
    }
    const bool is_q = h < nq;
    const float* gain = is_q ? q_gain : k_gain;
    const float goff = is_q ? q_off : k_off;
    const int half = rot / 2;

    float a[MAX_PAIRS], b[MAX_PAIRS], tail[MAX_TAIL];
    float ss = 0.f;
    if (splits == 0) {
#pragma unroll
        for (int i = 0; i < MAX_PAIRS; ++i) {
            const int p = lane + 32 * i;
            if (p < half) {
                a[i] = to_float(x.x[p]);
                b[i] = to_float(x.x[p + half]);
            }
        }
#pragma unroll
        for (int i = 0; i < MAX_TAIL; ++i) {
            const int e = rot + lane + 32 * i;
            if (e < hd) tail[i] = to_float(x.x[e]);
        }
    } else {
        // partial sums: the loads of one slice are independent, slices are added in order
#pragma unroll
        for (int i = 0; i < MAX_PAIRS; ++i) a[i] = b[i] = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_TAIL; ++i) tail[i] = 0.f;
#pragma unroll 4
        for (int sp = 0; sp < splits; ++sp) {
            const float* ps = x.p + (size_t)sp * split_stride;
#pragma unroll
            for (int i = 0; i < MAX_PAIRS; ++i) {
                const int p = lane + 32 * i;
                if (p < half) {
                    a[i] += __ldcg(ps + p);
                    b[i] += __ldcg(ps + p + half);
                }
            }
#pragma unroll
            for (int i = 0; i < MAX_TAIL; ++i) {
                const int e = rot + lane + 32 * i;
                if (e < hd) tail[i] += __ldcg(ps + e);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_PAIRS; ++i)
        if (lane + 32 * i < half) ss += a[i] * a[i] + b[i] * b[i];
#pragma unroll
    for (int i = 0; i < MAX_TAIL; ++i)
        if (rot + lane + 32 * i < hd) ss += tail[i] * tail[i];
    if (gain) {
        ss = warp_sum(ss);
        const float rinv = 1.0f / sqrtf(ss / (float)hd + eps);
#pragma unroll
        for (int i = 0; i < MAX_PAIRS; ++i) {
            const int p = lane + 32 * i;
            if (p < half) {
                a[i] = a[i] * rinv * (gain[p] + goff);
                b[i] = b[i] * rinv * (gain[p + half] + goff);
            }
        }
#pragma unroll
        for (int i = 0; i < MAX_TAIL; ++i) {
            const int e = rot + lane + 32 * i;
            if (e < hd) tail[i] = tail[i] * rinv * (gain[e] + goff);
        }
    }
    if (cos_tab) {
        const int pos = positions[t];
        const float* c = cos_tab + (size_t)pos * half;
        const float* s = sin_tab + (size_t)pos * half;
#pragma unroll
        for (int i = 0; i < MAX_PAIRS; ++i) {
            const int p = lane + 32 * i;
            if (p < half) {
                const float x0 = a[i], x1 = b[i], cs = c[p], sn = s[p];
                a[i] = x0 * cs - x1 * sn;
                b[i] = x1 * cs + x0 * sn;
            }
        }
    }
    T* dst;
    if (is_q) {
        dst = q_out + (size_t)t * q_stride + (size_t)h * hd;
    } else {
        if (slot < 0 || !kcache) return;
        const int kvh = h - nq;
        dst = kcache + (((size_t)(slot / page_size) * nkv_cache + kvh) * page_size + slot % page_size) * hd;
    }
#pragma unroll
    for (int i = 0; i < MAX_PAIRS; ++i) {
        const int p = lane + 32 * i;
        if (p < half) {
            dst[p] = from_float<T>(a[i]);
            dst[p + half] = from_float<T>(b[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_TAIL; ++i) {
        const int e = rot + lane + 32 * i;
        if (e < hd) dst[e] = from_float<T>(tail[i]);
    }
}

// The same for whole prompts, with 16-byte accesses: `LPR` lanes share one (token, head) row, each
// holding one 16-byte vector of it, so a warp works on 32 / LPR rows at a time; the rotary partner of
// a value sits LPR / 2 lanes away.  Taken when the rotary width is the head width, the rows are not
// partial sums, and everything is 16-byte aligned.
template <typename T, int LPR>
__global__ void __launch_bounds__(256)
attn_prep_vec_kernel(const T* __restrict__ qkv, long long row_stride, T* __restrict__ q_out, long long q_stride,
                     T* __restrict__ kcache, T* __restrict__ vcache, const int* __restrict__ positions,
                     const int* __restrict__ slots, const float* __restrict__ cos_tab,
                     const float* __restrict__ sin_tab, const float* __restrict__ q_gain,
                     const float* __restrict__ k_gain, int n_tokens, int nq, int nk, int nkv_cache, int hd,
                     int page_size, float eps, float q_off, float k_off) {
    constexpr int EPL = Vec16<T>::N;            // elements per lane
    constexpr int RPW = 32 / LPR;               // rows per warp
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int sub = lane % LPR;                 // which vector of the row
    // 32-bit row numbers (the launcher refuses more rows): divisions of 64-bit numbers by `heads` were
    // a quarter of the kernel's instructions
    const unsigned heads = (unsigned)(nq + 2 * nk);
    const unsigned n_rows = (unsigned)n_tokens * heads;
    const unsigned warp_id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const unsigned n_warps = gridDim.x * (blockDim.x >> 5);
    const int half_lanes = LPR / 2;
    const float inv_hd = 1.0f / (float)hd;
    for (unsigned row0 = warp_id * RPW; row0 < n_rows; row0 += n_warps * RPW) {
        const unsigned row = row0 + lane / LPR;
        const bool live = row < n_rows;
        const int t = live ? (int)(row / heads) : 0;
        const int h = live ? (int)(row - (unsigned)t * heads) : 0;
        const int slot = slots ? slots[t] : -1;
        const int pos = cos_tab ? positions[t] : 0;        // asked for here, with the row: its cos and sin follow it
        Vec16<T> x;
        x.raw = *reinterpret_cast<const decltype(x.raw)*>(qkv + (size_t)t * row_stride + (size_t)h * hd + sub * EPL);
        float f[EPL];
        x.unpack(f);
        const bool is_v = h >= nq + nk;
        const bool is_q = h < nq;
        const float* gain = is_q ? q_gain : k_gain;
        const float goff = is_q ? q_off : k_off;
        // every lane takes part in the shuffles, whatever kind of row it holds
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) ss += f[i] * f[i];
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (!is_v && gain) {
            // bfloat16 rows: the reciprocal root of the special-function unit (2 ulp, far below the rounding
            // of the result); the exact root and division are calls with slow paths that a row would wait for
            float rinv;
            if constexpr (sizeof(T) == 2) rinv = rsqrtf(fmaf(ss, inv_hd, eps));
            else rinv = 1.0f / sqrtf(ss / (float)hd + eps);
            float g[EPL];
#pragma unroll
            for (int i = 0; i < EPL; i += 4) {
                const float4 gv = *reinterpret_cast<const float4*>(gain + sub * EPL + i);
                g[i] = gv.x; g[i + 1] = gv.y; g[i + 2] = gv.z; g[i + 3] = gv.w;
            }
#pragma unroll
            for (int i = 0; i < EPL; ++i) f[i] = f[i] * rinv * (g[i] + goff);
        }
        float partner[EPL];
#pragma unroll
        for (int i = 0; i < EPL; ++i) partner[i] = __shfl_xor_sync(0xffffffffu, f[i], half_lanes);
        if (!is_v && cos_tab) {
            const int p0 = (sub % half_lanes) * EPL;          // index of the pair inside the half
            const float* c = cos_tab + (size_t)pos * (hd / 2) + p0;
            const float* sn = sin_tab + (size_t)pos * (hd / 2) + p0;
            const float sign = sub < half_lanes ? -1.f : 1.f;  // low half: x cos - y sin; high half: x cos + y sin
#pragma unroll
            for (int i = 0; i < EPL; i += 4) {
                const float4 cv = *reinterpret_cast<const float4*>(c + i);
                const float4 sv = *reinterpret_cast<const float4*>(sn + i);
                f[i] = f[i] * cv.x + sign * partner[i] * sv.x;
                f[i + 1] = f[i + 1] * cv.y + sign * partner[i + 1] * sv.y;
                f[i + 2] = f[i + 2] * cv.z + sign * partner[i + 2] * sv.z;
                f[i + 3] = f[i + 3] * cv.w + sign * partner[i + 3] * sv.w;
            }
        }
        if (!live) continue;
        T* dst = nullptr;
        if (is_q) {
            dst = q_out + (size_t)t * q_stride + (size_t)h * hd;
        } else if (slot >= 0) {
            T* cache = is_v ? vcache : kcache;
            const int kvh = is_v ? h - nq - nk : h - nq;
            const int page = slot / page_size;
            if (cache) dst = cache + (((size_t)page * nkv_cache + kvh) * page_size + (slot - page * page_size)) * hd;
        }
        if (dst) {
            Vec16<T> y;
            y.pack(f);
            *reinterpret_cast<decltype(y.raw)*>(dst + sub * EPL) = is_v ? x.raw : y.raw;
        }
    }
}

// The same, a warp taking `U` rounds of rows of ONE token at a time: position, slot, the lane's cos and
// sin values and its gains are read once for U * 32 / LPR rows (16 heads of 128 in bfloat16) instead of
// once a row, and the U loads of the rows are in flight together.
template <typename T, int LPR, int U>
__global__ void __launch_bounds__(256)
attn_prep_token_kernel(const T* __restrict__ qkv, long long row_stride, T* __restrict__ q_out, long long q_stride,
                       T* __restrict__ kcache, T* __restrict__ vcache, const int* __restrict__ positions,
                       const int* __restrict__ slots, const float* __restrict__ cos_tab,
                       const float* __restrict__ sin_tab, const float* __restrict__ q_gain,
                       const float* __restrict__ k_gain, int n_tokens, int nq, int nk, int nkv_cache, int hd,
                       int page_size, float eps, float q_off, float k_off) {
    constexpr int EPL = Vec16<T>::N;            // elements per lane
    constexpr int RPW = 32 / LPR;               // rows per round
    constexpr int RC = U * RPW;                 // rows per item
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int sub = lane % LPR;                 // which vector of the row
    const int half_lanes = LPR / 2;
    const int heads = nq + 2 * nk;
    const int chunks = (heads + RC - 1) / RC;
    const unsigned n_items = (unsigned)n_tokens * (unsigned)chunks;
    const unsigned warp_id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const unsigned n_warps = gridDim.x * (blockDim.x >> 5);
    const float inv_hd = 1.0f / (float)hd;
    // the gains are weights: read before the wait
    float gq[EPL], gk[EPL];
#pragma unroll
    for (int i = 0; i < EPL; i += 4) {
        const float4 a = q_gain ? *reinterpret_cast<const float4*>(q_gain + sub * EPL + i) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 b = k_gain ? *reinterpret_cast<const float4*>(k_gain + sub * EPL + i) : make_float4(1.f, 1.f, 1.f, 1.f);
        gq[i] = a.x + q_off; gq[i + 1] = a.y + q_off; gq[i + 2] = a.z + q_off; gq[i + 3] = a.w + q_off;
        gk[i] = b.x + k_off; gk[i + 1] = b.y + k_off; gk[i + 2] = b.z + k_off; gk[i + 3] = b.w + k_off;
    }
    const float sign = sub < half_lanes ? -1.f : 1.f;      // low half: x cos - y sin; high half: x cos + y sin
    pdl_wait();
    for (unsigned item = warp_id; item < n_items; item += n_warps) {
        const int t = (int)(item / (unsigned)chunks);
        const int h0 = (int)(item - (unsigned)t * (unsigned)chunks) * RC + lane / LPR;
        const T* src = qkv + (size_t)t * row_stride + sub * EPL;
        Vec16<T> x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int h = h0 + u * RPW;
            if (h < heads) x[u].raw = *reinterpret_cast<const decltype(x[u].raw)*>(src + (size_t)h * hd);
            else x[u].raw = decltype(x[u].raw){};
        }
        const int slot = slots ? slots[t] : -1;
        float cv[EPL], sv[EPL];
        if (cos_tab) {
            const int pos = positions[t];
            const int p0 = (sub % half_lanes) * EPL;          // index of the pair inside the half
            const float* c = cos_tab + (size_t)pos * (hd / 2) + p0;
            const float* sn = sin_tab + (size_t)pos * (hd / 2) + p0;
#pragma unroll
            for (int i = 0; i < EPL; i += 4) {
                const float4 a = *reinterpret_cast<const float4*>(c + i);
                const float4 b = *reinterpret_cast<const float4*>(sn + i);
                cv[i] = a.x; cv[i + 1] = a.y; cv[i + 2] = a.z; cv[i + 3] = a.w;
                sv[i] = sign * b.x; sv[i + 1] = sign * b.y; sv[i + 2] = sign * b.z; sv[i + 3] = sign * b.w;
            }
        }
        const int page = slot >= 0 ? slot / page_size : 0;
        const int in_page = slot - page * page_size;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int h = h0 + u * RPW;
            const bool live = h < heads;
            const bool is_q = h < nq;
            const bool is_v = h >= nq + nk;
            float f[EPL];
            x[u].unpack(f);
            // every lane takes part in the shuffles, whatever kind of row it holds
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < EPL; ++i) ss += f[i] * f[i];
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (!is_v && (is_q ? q_gain != nullptr : k_gain != nullptr)) {
                float rinv;
                if constexpr (sizeof(T) == 2) rinv = rsqrtf(fmaf(ss, inv_hd, eps));
                else rinv = 1.0f / sqrtf(ss / (float)hd + eps);
#pragma unroll
                for (int i = 0; i < EPL; ++i) f[i] = f[i] * rinv * (is_q ? gq[i] : gk[i]);
            }
            float partner[EPL];
#pragma unroll
            for (int i = 0; i < EPL; ++i) partner[i] = __shfl_xor_sync(0xffffffffu, f[i], half_lanes);
            if (!is_v && cos_tab) {
#pragma unroll
                for (int i = 0; i < EPL; ++i) f[i] = f[i] * cv[i] + partner[i] * sv[i];
            }
            if (!live) continue;
            T* dst = nullptr;
            if (is_q) {
                dst = q_out + (size_t)t * q_stride + (size_t)h * hd;
            } else if (slot >= 0) {
                T* cache = is_v ? vcache : kcache;
                const int kvh = is_v ? h - nq - nk : h - nq;
                if (cache) dst = cache + (((size_t)page * nkv_cache + kvh) * page_size + in_page) * hd;
            }
            if (dst) {
                Vec16<T> y;
                y.pack(f);
                *reinterpret_cast<decltype(y.raw)*>(dst + sub * EPL) = is_v ? x[u].raw : y.raw;
            }
        }
    }
}

static bool g_prep_by_token = true;
LLMK_EXPORT void llmk_attn_prep_set_by_token(int on) { g_prep_by_token = on != 0; }

template <typename T>
static bool launch_vec(const void* qkv, long long row_stride, void* q_out, long long q_stride, void* kcache, void* vcache,
                       const int* positions, const int* slots, const float* cos_tab, const float* sin_tab,
                       const float* q_gain, const float* k_gain, int n_tokens, int nq, int nk, int nkv_cache, int hd,
                       int rot, int page_size, float eps, float q_off, float k_off, cudaStream_t s, cudaError_t* err) {
    constexpr int EPL = Vec16<T>::N;
    if (hd % EPL != 0 || (cos_tab && rot != hd)) return false;
    const int lpr = hd / EPL;
    if (lpr != 8 && lpr != 16 && lpr != 32) return false;
    if (row_stride % EPL != 0 || q_stride % EPL != 0 || !host_aligned16(qkv) || !host_aligned16(q_out) ||
        (kcache && !host_aligned16(kcache)) || (vcache && !host_aligned16(vcache)))
        return false;
    // gains and rotary tables are read four floats at a time
    if ((q_gain && !host_aligned16(q_gain)) || (k_gain && !host_aligned16(k_gain)) || (cos_tab && !host_aligned16(cos_tab)) ||
        (sin_tab && !host_aligned16(sin_tab)) || (hd / 2) % 4 != 0)
        return false;
    const long long rows = (long long)n_tokens * (nq + 2 * nk);
    if (rows >= (1LL << 31) - (1LL << 20)) return false;       // the kernel counts rows in 32 bits
    const int rpw = 32 / lpr;
    if (g_prep_by_token) {
#define LAUNCH_TOKEN(L, U)                                                                                                  \
    do {                                                                                                                    \
        const int chunks = (nq + 2 * nk + U * rpw - 1) / (U * rpw);                                                         \
        long long tblocks = ((long long)n_tokens * chunks + 7) / 8;                                                         \
        if (tblocks > device_sm_count() * 8) tblocks = device_sm_count() * 8;                                                                           \
        *err = llmk_launch(attn_prep_token_kernel<T, L, U>, dim3((unsigned)tblocks), dim3(256), 0, s, true, (const T*)qkv,  \
                           row_stride, (T*)q_out, q_stride, (T*)kcache, (T*)vcache, positions, slots, cos_tab, sin_tab,     \
                           q_gain, k_gain, n_tokens, nq, nk, nkv_cache, hd, page_size, eps, q_off, k_off);                  \
    } while (0)
        // eight rounds of rows in flight per warp: 13.3 us on 2,048 tokens of 32 heads of 128 in bfloat16,
        // 15.2 us with four, 14.5 us a row at a time
        if (lpr == 8) LAUNCH_TOKEN(8, 8);
        else if (lpr == 16) LAUNCH_TOKEN(16, 8);
        else LAUNCH_TOKEN(32, 8);
#undef LAUNCH_TOKEN
        return true;
    }
    long long blocks = (rows + 8 * rpw - 1) / (8 * rpw);
    if (blocks > device_sm_count() * 8) blocks = device_sm_count() * 8;
#define LAUNCH_VEC(L)                                                                                                   \
    *err = llmk_launch(attn_prep_vec_kernel<T, L>, dim3((unsigned)blocks), dim3(256), 0, s, true, (const T*)qkv, row_stride, \
                       (T*)q_out, q_stride, (T*)kcache, (T*)vcache, positions, slots, cos_tab, sin_tab, q_gain, k_gain,  \
                       n_tokens, nq, nk, nkv_cache, hd, page_size, eps, q_off, k_off)
    if (lpr == 8) LAUNCH_VEC(8);
    else if (lpr == 16) LAUNCH_VEC(16);
    else LAUNCH_VEC(32);
#undef LAUNCH_VEC
    return true;
}

// nk = number of k (and v) heads present in the packed rows: num_kv_heads for a layer that
// writes its cache, 0 for a layer that only reads another layer's cache.
LLMK_EXPORT int llmk_attn_prep(const void* qkv, long long row_stride, int splits, long long split_stride, void* q_out,
                               long long q_stride, void* kcache, void* vcache, const int* positions,
                               const int* slots, const float* cos_tab, const float* sin_tab, const float* q_gain,
                               const float* k_gain, int n_tokens, int nq, int nk, int nkv_cache, int hd, int rot,
                               int page_size, float eps, float q_off, float k_off, int pairing, int head_norm, int dtype,
                               void* stream) {
    if (n_tokens <= 0) return LLMK_OK;
    if (pairing != LLMK_PAIR_HALF_SPLIT)
        LLMK_FAIL("attn_prep: rotary pairing %d is not built (0: half-split, pairs (i, i + rot / 2))", pairing);
    if (head_norm != LLMK_HEAD_NORM_RMS) LLMK_FAIL("attn_prep: per-head norm kind %d is not built (0: RMSNorm)", head_norm);
    if (hd <= 0 || hd % 2 != 0 || hd > 512) LLMK_FAIL("attn_prep: head_dim %d must be even and at most 512", hd);
    if (rot < 0 || rot > hd || rot % 2 != 0) LLMK_FAIL("attn_prep: rotary width %d must be even and at most head_dim %d", rot, hd);
    if (rot / 2 > 32 * MAX_PAIRS || hd - rot > 32 * MAX_TAIL) LLMK_FAIL("attn_prep: head_dim %d / rotary width %d too large", hd, rot);
    if (nq < 0 || nk < 0 || nq + nk <= 0) LLMK_FAIL("attn_prep: bad head counts nq=%d nk=%d", nq, nk);
    if (nk > 0 && (page_size <= 0 || nkv_cache < nk)) LLMK_FAIL("attn_prep: bad cache geometry page_size=%d kv heads=%d", page_size, nkv_cache);
    if (splits < 0 || (splits > 0 && split_stride <= 0)) LLMK_FAIL("attn_prep: bad partial sums (%d slices)", splits);
    if (!q_out && nq > 0) LLMK_FAIL("attn_prep: no place for q");
    if (!cos_tab) rot = 0;
    if (cos_tab && (!sin_tab || !positions)) LLMK_FAIL("attn_prep: rotary tables need sin and positions");
    cudaStream_t s = (cudaStream_t)stream;
    const int warps = 4;
    const long long items = (long long)n_tokens * (nq + 2 * nk);
    const long long blocks = (items + warps - 1) / warps;
    if (blocks > 2147483647LL) LLMK_FAIL("attn_prep: too many rows");
    cudaError_t e;
    if (splits == 0 && n_tokens >= 32) {
        bool taken = false;
        if (dtype == LLMK_F32)
            taken = launch_vec<float>(qkv, row_stride, q_out, q_stride, kcache, vcache, positions, slots, cos_tab, sin_tab,
                                      q_gain, k_gain, n_tokens, nq, nk, nkv_cache, hd, rot, page_size, eps, q_off, k_off, s, &e);
        else if (dtype == LLMK_BF16)
            taken = launch_vec<bf16>(qkv, row_stride, q_out, q_stride, kcache, vcache, positions, slots, cos_tab, sin_tab,
                                     q_gain, k_gain, n_tokens, nq, nk, nkv_cache, hd, rot, page_size, eps, q_off, k_off, s, &e);
        if (taken) {
            LLMK_CHECK_LAUNCH_RC("attn_prep", e);
            return LLMK_OK;
        }
    }
    if (dtype == LLMK_F32)
        e = llmk_launch(attn_prep_kernel<float>, dim3((unsigned)blocks), dim3(warps * 32), 0, s, true, qkv, row_stride,
                        splits, split_stride, (float*)q_out, q_stride, (float*)kcache, (float*)vcache, positions, slots,
                        cos_tab, sin_tab, q_gain, k_gain, n_tokens, nq, nk, nkv_cache, hd, rot, page_size, eps, q_off,
                        k_off);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(attn_prep_kernel<bf16>, dim3((unsigned)blocks), dim3(warps * 32), 0, s, true, qkv, row_stride,
                        splits, split_stride, (bf16*)q_out, q_stride, (bf16*)kcache, (bf16*)vcache, positions, slots,
                        cos_tab, sin_tab, q_gain, k_gain, n_tokens, nq, nk, nkv_cache, hd, rot, page_size, eps, q_off,
                        k_off);
    else
        LLMK_FAIL("attn_prep: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("attn_prep", e);
    return LLMK_OK;
}
