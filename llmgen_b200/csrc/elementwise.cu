// Row-wise kernels around the matrix products: embedding gather, residual add fused with
// RMSNorm (optionally on gathered rows), and the gated activation of the feed-forward.
//
// What they replace in the reference: `embedding_kernel` (src/backend/cuda/embedding/embedding.cu:3-13),
// `add_kernel` + `rmsnorm_row_kernel` (src/backend/cuda/arithmetic/add_v1.cu:3-15,
// src/backend/cuda/norm/norm_final.cu:9-26), `gather_rows_kernel`
// (src/backend/cuda/memory/memcpy.cu:58-67) and `silu_kernel` + `mul_kernel`
// (src/backend/cuda/activation/silu_v1.cu:6-18, src/backend/cuda/arithmetic/mul_v1.cu:3-16).
// The residual stream is float32 here, so the sum x + delta is never rounded to bfloat16.
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

// ---------------------------------------------------------------- embedding gather
// out[t, :] = table[ids[t], :] widened to float32.  An id outside [0, V) gives a zero row and
// raises *bad (the host checks ids before the step, this is the device-side guard the
// reference's kernel lacks).  With `ids_from`, row t whose ids_from[t] >= 0 takes its id from
// sampled[ids_from[t]] instead: the token that the step before sampled for that row and that
// the host has not read yet.
template <typename T>
__global__ void embed_rows_kernel(float* __restrict__ out, const T* __restrict__ table,
                                  const int* __restrict__ ids, const int* __restrict__ ids_from,
                                  const int* __restrict__ sampled, int H, int V, int* bad, float scale) {
    const int t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int from = ids_from ? ids_from[t] : -1;
    const int id = from >= 0 ? sampled[from] : ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0 && bad) atomicAdd(bad, 1);
    const T* row = table + (size_t)(ok ? id : 0) * H;
    float* dst = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = ok ? to_float(row[i]) * scale : 0.f;
}

LLMK_EXPORT int llmk_embed_rows(float* out, const void* table, const int* ids, const int* ids_from, const int* sampled,
                                int n_tokens, int H, int V, int* bad_flag, int dtype, float scale, void* stream) {
    if (n_tokens <= 0) return LLMK_OK;
    if (H <= 0 || V <= 0) LLMK_FAIL("embed_rows: bad sizes H=%d V=%d", H, V);
    if ((ids_from != nullptr) != (sampled != nullptr)) LLMK_FAIL("embed_rows: ids_from and sampled come together");
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    cudaError_t e;
    if (dtype == LLMK_F32)
        e = llmk_launch(embed_rows_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, true, out, (const float*)table, ids, ids_from, sampled, H, V, bad_flag, scale);
    else if (dtype == LLMK_BF16)
        e = llmk_launch(embed_rows_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, true, out, (const bf16*)table, ids, ids_from, sampled, H, V, bad_flag, scale);
    else
        LLMK_FAIL("embed_rows: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH_RC("embed_rows", e);
    return LLMK_OK;
}

// x = cap * tanh(x / cap) on float32 logits, in place: an architecture's bound on its logits (none here has one;
// `ModelSpec.logit_cap` is the slot).
__global__ void logit_cap_kernel(float* __restrict__ x, long long n, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    const float inv = 1.0f / cap;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
}

LLMK_EXPORT int llmk_logit_cap(float* x, long long n, float cap, void* stream) {
    if (n <= 0) return LLMK_OK;
    if (!(cap > 0.f)) LLMK_FAIL("logit_cap: the cap must be positive, got %g", (double)cap);
    long long blocks = (n + 255) / 256;
    if (blocks > device_sm_count() * 8) blocks = device_sm_count() * 8;
    LLMK_CHECK_LAUNCH_RC("logit_cap", llmk_launch(logit_cap_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, true, x, n, cap));
    return LLMK_OK;
}

// ------------------------------------------------------- residual add + RMSNorm
// For output row r, source row s = rows ? rows[r] : r:
//   v    = resid[s, :] + (delta ? delta[s, :] : 0)          (float32)
//          where delta is a [n, H] array of T, or (splits > 0) `splits` float32 slices
//          [splits][n_src][H], `split_stride` floats apart, added in slice order: the partial sums
//          of a matrix product cut along K
//   resid[s, :] = v                    if write_resid
//   out[r, :]   = v * (1 / sqrt(mean(v^2) + eps)) * (w + w_offset)      rounded once to T
// The row is kept in shared memory between the two passes.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const void* __restrict__ delta,
                                   const float* __restrict__ w, T* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps, float w_offset,
                                   int write_resid, int splits, long long split_stride) {
    extern __shared__ float srow[];  // H floats + 33 scratch
    float* scratch = srow + H;
    const int r = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int s = rows ? rows[r] : r;
    float* x = resid + (size_t)s * H;
    const T* d = (delta && splits == 0) ? static_cast<const T*>(delta) + (size_t)s * H : nullptr;
    const float* dp = (delta && splits > 0) ? static_cast<const float*>(delta) + (size_t)s * H : nullptr;
    float ss = 0.f;
    if (dp && (H & 3) == 0 && (split_stride & 3) == 0 && aligned16(dp) && aligned16(x)) {
        // Partial sums: 16-byte loads, eight slices in flight at a time, added in slice order.
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(x + i);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int sp0 = 0; sp0 < splits; sp0 += 8) {
                float4 t[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    t[u] = sp0 + u < splits ? __ldcg(reinterpret_cast<const float4*>(dp + (size_t)(sp0 + u) * split_stride + i))
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    acc.x += t[u].x; acc.y += t[u].y; acc.z += t[u].z; acc.w += t[u].w;
                }
            }
            v.x += acc.x; v.y += acc.y; v.z += acc.z; v.w += acc.w;
            *reinterpret_cast<float4*>(srow + i) = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            if (write_resid) *reinterpret_cast<float4*>(x + i) = v;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = x[i];
            if (d) v += to_float(d[i]);
            if (dp) {
                float acc = dp[i];
                for (int sp = 1; sp < splits; ++sp) acc += dp[(size_t)sp * split_stride + i];
                v += acc;
            }
            srow[i] = v;
            ss += v * v;
            if (write_resid) x[i] = v;
        }
    }
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_float<T>(srow[i] * rinv * (w[i] + w_offset));
}

// The same with the row kept in registers and 16-byte accesses: thread t holds the float4 vectors
// t, t + blockDim, ... of the row (at most VPT of them).  Taken when H is a multiple of 4, at most
// 4 * VPT * blockDim, and the arrays are 16-byte aligned.
template <int N> struct Pack4;
template <> struct Pack4<4> { typedef float4 type; };     // four float32
template <> struct Pack4<2> { typedef uint2 type; };      // four bfloat16
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = raw;
}

template <typename T, int VPT>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const void* __restrict__ delta,
                                       const float* __restrict__ w, T* __restrict__ out,
                                       const int* __restrict__ rows, int H, float eps, float w_offset,
                                       int write_resid, int splits, long long split_stride) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    pdl_launch_dependents();
    // the gains are weights: a prefetch before the wait (loading them into registers here, or with the row
    // after the wait, made a decode step 15 % slower)
#pragma unroll
    for (int it = 0; it < VPT; ++it) {
        const int i = (it * blockDim.x + threadIdx.x) * 4;
        if (i < H) asm volatile("prefetch.global.L1 [%0];" ::"l"(w + i));
    }
    pdl_wait();
    const int s = rows ? rows[r] : r;
    float* x = resid + (size_t)s * H;
    const T* d = (delta && splits == 0) ? static_cast<const T*>(delta) + (size_t)s * H : nullptr;
    const float* dp = (delta && splits > 0) ? static_cast<const float*>(delta) + (size_t)s * H : nullptr;
    float4 v[VPT];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < VPT; ++it) {
        const int i = (it * blockDim.x + threadIdx.x) * 4;
        v[it] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < H) {
            v[it] = load4(x + i);
            if (d) {
                const float4 a = load4(d + i);
                v[it].x += a.x; v[it].y += a.y; v[it].z += a.z; v[it].w += a.w;
            }
            if (dp) {
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int sp0 = 0; sp0 < splits; sp0 += 8) {
                    float4 t[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        t[u] = sp0 + u < splits ? __ldcg(reinterpret_cast<const float4*>(dp + (size_t)(sp0 + u) * split_stride + i))
                                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        acc.x += t[u].x; acc.y += t[u].y; acc.z += t[u].z; acc.w += t[u].w;
                    }
                }
                v[it].x += acc.x; v[it].y += acc.y; v[it].z += acc.z; v[it].w += acc.w;
            }
            ss += v[it].x * v[it].x + v[it].y * v[it].y + v[it].z * v[it].z + v[it].w * v[it].w;
            if (write_resid) store4(x + i, v[it]);
        }
    }
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
#pragma unroll
    for (int it = 0; it < VPT; ++it) {
        const int i = (it * blockDim.x + threadIdx.x) * 4;
        if (i < H) {
            const float4 g = load4(w + i);
            store4(o + i, make_float4(v[it].x * rinv * (g.x + w_offset), v[it].y * rinv * (g.y + w_offset),
                                      v[it].z * rinv * (g.z + w_offset), v[it].w * rinv * (g.w + w_offset)));
        }
    }
}

// Many rows (a prompt): a warp per row, the row in registers as LPT float4 per lane, all loads of a
// row in flight at once and nothing but warp shuffles between the two passes.  Rows in order, delta
// in T or absent.  (A block per row with one float4 per thread ran at 2.5 TB/s on 2,048 rows of 1,024.)
template <typename T, int LPT>
__global__ void __launch_bounds__(128)
add_rmsnorm_warp_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ w,
                        T* __restrict__ out, int n_rows, int H, float eps, float w_offset, int write_resid) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const int lane = threadIdx.x & 31;
    float* x = resid + (size_t)r * H;
    float4 v[LPT];
#pragma unroll
    for (int it = 0; it < LPT; ++it) {
        const int i = (it * 32 + lane) * 4;
        v[it] = i < H ? load4(x + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (delta) {
        const T* d = delta + (size_t)r * H;
        float4 a[LPT];
#pragma unroll
        for (int it = 0; it < LPT; ++it) {
            const int i = (it * 32 + lane) * 4;
            a[it] = i < H ? load4(d + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int it = 0; it < LPT; ++it) {
            v[it].x += a[it].x; v[it].y += a[it].y; v[it].z += a[it].z; v[it].w += a[it].w;
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < LPT; ++it) {
        const int i = (it * 32 + lane) * 4;
        ss += v[it].x * v[it].x + v[it].y * v[it].y + v[it].z * v[it].z + v[it].w * v[it].w;
        if (write_resid && i < H) store4(x + i, v[it]);
    }
    ss = warp_sum(ss);
    const float rinv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
#pragma unroll
    for (int it = 0; it < LPT; ++it) {
        const int i = (it * 32 + lane) * 4;
        if (i < H) {
            const float4 g = load4(w + i);
            store4(o + i, make_float4(v[it].x * rinv * (g.x + w_offset), v[it].y * rinv * (g.y + w_offset),
                                      v[it].z * rinv * (g.z + w_offset), v[it].w * rinv * (g.w + w_offset)));
        }
    }
}

LLMK_EXPORT int llmk_add_rmsnorm(float* resid, const void* delta, const float* w, void* out, const int* rows,
                                 int n_rows, int H, float eps, float w_offset, int write_resid, int splits,
                                 long long split_stride, int dtype, void* stream) {
    if (n_rows <= 0) return LLMK_OK;
    if (H <= 0) LLMK_FAIL("add_rmsnorm: bad width H=%d", H);
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    if (smem > 200 * 1024) LLMK_FAIL("add_rmsnorm: width %d needs %zu bytes of shared memory (limit 204800)", H, smem);
    if (rows && write_resid) LLMK_FAIL("add_rmsnorm: gathered rows cannot be written back");
    if (splits < 0 || (splits > 0 && split_stride < H)) LLMK_FAIL("add_rmsnorm: bad partial sums (%d slices, stride %lld)", splits, split_stride);
    cudaStream_t s = (cudaStream_t)stream;
    int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const bool aligned = host_aligned16(resid) && host_aligned16(w) && host_aligned16(out) &&
                         (!delta || host_aligned16(delta)) && (splits == 0 || split_stride % 4 == 0);
    if (H % 4 == 0 && H <= 2048 && n_rows >= 512 && !rows && splits == 0 && aligned && (dtype == LLMK_F32 || dtype == LLMK_BF16)) {
        const int lpt = (H / 4 + 31) / 32;
        const dim3 grid((n_rows + 3) / 4), block(128);
        cudaError_t e;
#define LAUNCH_WARP(T, L)                                                                                          \
    e = llmk_launch(add_rmsnorm_warp_kernel<T, L>, grid, block, 0, s, true, resid, (const T*)delta, w, (T*)out, n_rows, H, \
                    eps, w_offset, write_resid)
        if (dtype == LLMK_F32) {
            if (lpt <= 4) LAUNCH_WARP(float, 4); else if (lpt <= 8) LAUNCH_WARP(float, 8); else LAUNCH_WARP(float, 16);
        } else {
            if (lpt <= 4) LAUNCH_WARP(bf16, 4); else if (lpt <= 8) LAUNCH_WARP(bf16, 8); else LAUNCH_WARP(bf16, 16);
        }
#undef LAUNCH_WARP
        LLMK_CHECK_LAUNCH_RC("add_rmsnorm", e);
        return LLMK_OK;
    }
    if (H % 4 == 0 && H <= 8192 && aligned && (dtype == LLMK_F32 || dtype == LLMK_BF16)) {
        int vthreads = (H / 4 + 31) / 32 * 32;
        if (vthreads > 512) vthreads = 512;
        const int vpt = (H / 4 + vthreads - 1) / vthreads;
        cudaError_t e;
#define LAUNCH_VEC(T, V)                                                                                               \
    e = llmk_launch(add_rmsnorm_vec_kernel<T, V>, dim3(n_rows), dim3(vthreads), 0, s, true, resid, delta, w, (T*)out, rows, H, \
                    eps, w_offset, write_resid, splits, split_stride)
        if (dtype == LLMK_F32) {
            if (vpt == 1) LAUNCH_VEC(float, 1); else if (vpt == 2) LAUNCH_VEC(float, 2); else LAUNCH_VEC(float, 4);
        } else {
            if (vpt == 1) LAUNCH_VEC(bf16, 1); else if (vpt == 2) LAUNCH_VEC(bf16, 2); else LAUNCH_VEC(bf16, 4);
        }
#undef LAUNCH_VEC
        LLMK_CHECK_LAUNCH_RC("add_rmsnorm", e);
        return LLMK_OK;
    }
#define LAUNCH(T)                                                                                            \
    do {                                                                                                     \
        if (smem > 48 * 1024) {                                                                              \
            cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<T>,                                      \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
            if (e != cudaSuccess) LLMK_FAIL("add_rmsnorm: cannot raise shared memory: %s", cudaGetErrorString(e)); \
        }                                                                                                    \
        launch_rc = llmk_launch(add_rmsnorm_kernel<T>, dim3(n_rows), dim3(threads), smem, s, true, resid, delta, w, \
                                (T*)out, rows, H, eps, w_offset, write_resid, splits, split_stride);         \
    } while (0)
    cudaError_t launch_rc = cudaSuccess;
    if (dtype == LLMK_F32)
        LAUNCH(float);
    else if (dtype == LLMK_BF16)
        LAUNCH(bf16);
    else
        LLMK_FAIL("add_rmsnorm: unknown dtype %d", dtype);
#undef LAUNCH
    LLMK_CHECK_LAUNCH_RC("add_rmsnorm", launch_rc);
    return LLMK_OK;
}

// ------------------------------------------------------------- gated activation
// in [n, 2F] alternates `group` gate columns and `group` up columns (group = F: gate in columns
// [0, F), up in [F, 2F)); out[n, F] = silu(gate) * up with silu(g) = g / (1 + exp(-g)) in float32,
// rounded once.  Output column j reads gate column 2 * group * (j / group) + j % group and the up
// column `group` further.
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ in, int n, int F, int ld_in, int group) {
    const size_t total = (size_t)n * F;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int row = (int)(idx / F), col = (int)(idx % F);
        const int gcol = 2 * group * (col / group) + col % group;
        const float g = to_float(in[(size_t)row * ld_in + gcol]);
        const float u = to_float(in[(size_t)row * ld_in + gcol + group]);
        out[idx] = from_float<T>(g / (1.0f + expf(-g)) * u);
    }
}

template <typename T>
__global__ void silu_mul_vec_kernel(T* __restrict__ out, const T* __restrict__ in, int n, int F, int ld_in, int group) {
    constexpr int N = Vec16<T>::N;
    const int fv = F / N;
    const size_t total = (size_t)n * fv;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int row = (int)(idx / fv), col = (int)(idx % fv) * N;
        const int gcol = 2 * group * (col / group) + col % group;
        const T* base = in + (size_t)row * ld_in + gcol;
        Vec16<T> g, u, o;
        g.raw = *reinterpret_cast<const decltype(g.raw)*>(base);
        u.raw = *reinterpret_cast<const decltype(u.raw)*>(base + group);
        float gf[N], uf[N], of[N];
        g.unpack(gf);
        u.unpack(uf);
#pragma unroll
        for (int i = 0; i < N; ++i) of[i] = gf[i] / (1.0f + expf(-gf[i])) * uf[i];
        o.pack(of);
        *reinterpret_cast<decltype(o.raw)*>(out + (size_t)row * F + col) = o.raw;
    }
}

// The same from the float32 partial sums of a product cut along K: in is [splits][n][ld_in] with
// slices `split_stride` floats apart, added in slice order before the activation.
template <typename T>
__global__ void silu_mul_partials_kernel(T* __restrict__ out, const float* __restrict__ in, int n, int F, int ld_in,
                                         int group, int splits, long long split_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)n * F;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int row = (int)(idx / F), col = (int)(idx % F);
        const int gcol = 2 * group * (col / group) + col % group;
        const float* base = in + (size_t)row * ld_in + gcol;
        float g = base[0], u = base[group];
        for (int sp = 1; sp < splits; ++sp) {
            g += base[(size_t)sp * split_stride];
            u += base[(size_t)sp * split_stride + group];
        }
        out[idx] = from_float<T>(g / (1.0f + expf(-g)) * u);
    }
}

template <typename T>
static int launch_silu_mul(void* out, const void* in, int n, int F, int ld_in, int group, cudaStream_t s) {
    constexpr int N = Vec16<T>::N;
    const bool vec = (F % N == 0) && (group % N == 0) && (ld_in % N == 0) && host_aligned16(out) && host_aligned16(in);
    const size_t work = vec ? (size_t)n * (F / N) : (size_t)n * F;
    const int threads = 256;
    size_t blocks = (work + threads - 1) / threads;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    if (blocks == 0) return LLMK_OK;
    if (vec)
        silu_mul_vec_kernel<T><<<(int)blocks, threads, 0, s>>>((T*)out, (const T*)in, n, F, ld_in, group);
    else
        silu_mul_kernel<T><<<(int)blocks, threads, 0, s>>>((T*)out, (const T*)in, n, F, ld_in, group);
    return LLMK_OK;
}

LLMK_EXPORT int llmk_silu_mul(void* out, const void* in, int n_rows, int F, int ld_in, int group, int splits,
                              long long split_stride, int dtype, void* stream) {
    if (n_rows <= 0) return LLMK_OK;
    if (F <= 0 || ld_in < 2 * F) LLMK_FAIL("silu_mul: bad sizes F=%d ld_in=%d", F, ld_in);
    if (group <= 0 || F % group != 0) LLMK_FAIL("silu_mul: group %d must divide F=%d", group, F);
    cudaStream_t s = (cudaStream_t)stream;
    if (splits > 0) {
        const size_t work = (size_t)n_rows * F;
        size_t blocks = (work + 255) / 256;
        if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
        cudaError_t e;
        if (dtype == LLMK_F32)
            e = llmk_launch(silu_mul_partials_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, true, (float*)out,
                            (const float*)in, n_rows, F, ld_in, group, splits, split_stride);
        else if (dtype == LLMK_BF16)
            e = llmk_launch(silu_mul_partials_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, s, true, (bf16*)out,
                            (const float*)in, n_rows, F, ld_in, group, splits, split_stride);
        else
            LLMK_FAIL("silu_mul: unknown dtype %d", dtype);
        LLMK_CHECK_LAUNCH_RC("silu_mul", e);
        return LLMK_OK;
    }
    if (dtype == LLMK_F32)
        launch_silu_mul<float>(out, in, n_rows, F, ld_in, group, s);
    else if (dtype == LLMK_BF16)
        launch_silu_mul<bf16>(out, in, n_rows, F, ld_in, group, s);
    else
        LLMK_FAIL("silu_mul: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH("silu_mul");
    return LLMK_OK;
}

// --------------------------------------------------------- convert rows to float32
// out[n, W] float32 = in[n, W] of type T (used to hand bfloat16 logits out as float32).
template <typename T>
__global__ void widen_kernel(float* __restrict__ out, const T* __restrict__ in, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x)
        out[idx] = to_float(in[idx]);
}

LLMK_EXPORT int llmk_widen(float* out, const void* in, long long total, int dtype, void* stream) {
    if (total <= 0) return LLMK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    long long blocks = (total + 255) / 256;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    if (dtype == LLMK_F32)
        widen_kernel<float><<<(int)blocks, 256, 0, s>>>(out, (const float*)in, (size_t)total);
    else if (dtype == LLMK_BF16)
        widen_kernel<bf16><<<(int)blocks, 256, 0, s>>>(out, (const bf16*)in, (size_t)total);
    else
        LLMK_FAIL("widen: unknown dtype %d", dtype);
    LLMK_CHECK_LAUNCH("widen");
    return LLMK_OK;
}
