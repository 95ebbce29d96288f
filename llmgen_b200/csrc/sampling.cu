// Sampling on the GPU, so that a step hands back one int32 per sequence instead of its logits.
//
// Same scheme as the reference (src/backend/cuda/sample/sample.cu:33-77,
// src/backend/cpu/sample.zig:16-45): temperature <= 0 is argmax with ties to the smaller id;
// temperature > 0 is Gumbel-max, argmax(logit / T - log(-log u)), with u from a stateless
// hash: u = ((r >> 40) + 0.5) / 2^24, r = splitmix64(row_seed + id),
// row_seed = splitmix64(step_seed ^ (row << 40)).  Two stages: each of SPLIT blocks per row scans
// a slice of the vocabulary, then one warp merges the candidates.  Logits are float32 here
// (bfloat16 in the reference), and log is the accurate `logf`, so that a host restatement
// picks the same ids.
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

constexpr int SPLIT = 32;
constexpr int THREADS = 256;

__host__ __device__ inline unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__device__ __forceinline__ void argmax_merge(float& best, int& best_i, float ov, int oi) {
    if (ov > best || (ov == best && oi < best_i)) {
        best = ov;
        best_i = oi;
    }
}
__device__ __forceinline__ void warp_argmax(float& best, int& best_i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        argmax_merge(best, best_i, ov, oi);
    }
}

__global__ void __launch_bounds__(THREADS)
sample_partial_kernel(float* __restrict__ pv, int* __restrict__ pi, const float* __restrict__ logits,
                      long long ld, const float* __restrict__ temps, const unsigned long long* seed_ptr, int V) {
    const int s = blockIdx.x, part = blockIdx.y;
    const int chunk = (V + SPLIT - 1) / SPLIT;
    const int beg = part * chunk, end = min(V, beg + chunk);
    const float* row = logits + (size_t)s * ld;
    const float temp = temps[s];
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    if (temp > 0.f) {
        const unsigned long long seed = splitmix64(*seed_ptr ^ ((unsigned long long)s << 40));
        const float inv_t = 1.f / temp;
        for (int i = beg + threadIdx.x; i < end; i += THREADS) {
            const unsigned long long r = splitmix64(seed + (unsigned long long)i);
            const float u = ((float)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);
            argmax_merge(best, best_i, row[i] * inv_t - logf(-logf(u)), i);
        }
    } else {
        for (int i = beg + threadIdx.x; i < end; i += THREADS) argmax_merge(best, best_i, row[i], i);
    }
    warp_argmax(best, best_i);
    __shared__ float sv[THREADS / 32];
    __shared__ int si[THREADS / 32];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) {
        sv[wid] = best;
        si[wid] = best_i;
    }
    __syncthreads();
    if (wid == 0) {
        best = lane < THREADS / 32 ? sv[lane] : -INFINITY;
        best_i = lane < THREADS / 32 ? si[lane] : 0x7fffffff;
        warp_argmax(best, best_i);
        if (lane == 0) {
            pv[s * SPLIT + part] = best;
            pi[s * SPLIT + part] = best_i;
        }
    }
}

__global__ void sample_final_kernel(int* __restrict__ out, const float* __restrict__ pv, const int* __restrict__ pi) {
    const int s = blockIdx.x, lane = threadIdx.x;
    float best = pv[s * SPLIT + lane];
    int best_i = pi[s * SPLIT + lane];
    warp_argmax(best, best_i);
    if (lane == 0) out[s] = best_i;
}

LLMK_EXPORT long long llmk_sample_scratch_bytes(int max_rows) { return (long long)max_rows * SPLIT * 8; }

// out[s] = sampled id of row s of logits [n_rows, V] (row stride ld); temps[s] <= 0 is greedy.
// `seed` points at the step's 64-bit seed on the device (so a replayed CUDA graph only needs
// the value refreshed).
LLMK_EXPORT int llmk_sample(int* out, const float* logits, long long ld, const float* temps,
                            const unsigned long long* seed, int n_rows, int V, void* scratch, void* stream) {
    if (n_rows <= 0) return LLMK_OK;
    if (V <= 0 || ld < V) LLMK_FAIL("sample: bad sizes V=%d ld=%lld", V, ld);
    if (!scratch || !seed || !temps) LLMK_FAIL("sample: scratch, seed and temperatures are required");
    cudaStream_t s = (cudaStream_t)stream;
    float* pv = (float*)scratch;
    int* pi = (int*)(pv + (size_t)n_rows * SPLIT);
    sample_partial_kernel<<<dim3(n_rows, SPLIT), THREADS, 0, s>>>(pv, pi, logits, ld, temps, seed, V);
    LLMK_CHECK_LAUNCH("sample_partial");
    sample_final_kernel<<<n_rows, 32, 0, s>>>(out, pv, pi);
    LLMK_CHECK_LAUNCH("sample_final");
    return LLMK_OK;
}

// ------------------------------------------------------------------ sampling without an allocator
// `llmk_sample_static` (declared in llmk_sample_static.h) is `llmk_sample` for callers that cannot
// hand over scratch memory because they cannot allocate any: code running where cudaMalloc is off
// limits, such as a host that embeds this library beside a runtime owning all device memory, or a
// callback that must not call into an allocator.  The candidates of the first stage go to a
// file-scope device array instead of a caller's buffer.  Every GPU that loads this library holds
// the array (LLMK_SAMPLE_STATIC_MAX_ROWS * 32 * 8 bytes = 64 KiB) until the process exits.
//
// In host code `g_sample_static_scratch` is only a handle for the runtime, not a device address;
// the address is asked for once per device with cudaGetSymbolAddress, with that device current,
// on the first call made on that device.  That first call should therefore come before any stream
// capture.  Both stages overwrite every slot they read, so nothing has to be cleared between calls;
// but all calls share the one array, so two calls that overlap on the GPU (different streams) race.
#include "llmk_sample_static.h"

#include <mutex>

static __device__ __align__(256) unsigned char g_sample_static_scratch[LLMK_SAMPLE_STATIC_MAX_ROWS * SPLIT * 8];

namespace {
constexpr int MAX_DEVICES = 64;
std::mutex g_static_lock;
void* g_static_ptr[MAX_DEVICES] = {};
}  // namespace

LLMK_EXPORT int llmk_sample_static_max_rows() { return LLMK_SAMPLE_STATIC_MAX_ROWS; }

LLMK_EXPORT int llmk_sample_static(int* out, const float* logits, long long ld, const float* temps,
                                   const unsigned long long* seed, int n_rows, int V, void* stream) {
    if (n_rows <= 0) return LLMK_OK;
    if (n_rows > LLMK_SAMPLE_STATIC_MAX_ROWS)
        LLMK_FAIL("sample_static: %d rows exceed the built-in scratch of %d rows; use llmk_sample with scratch of your own",
                  n_rows, LLMK_SAMPLE_STATIC_MAX_ROWS);
    if (V <= 0 || ld < V) LLMK_FAIL("sample_static: bad sizes V=%d ld=%lld", V, ld);
    if (!out || !logits || !seed || !temps) LLMK_FAIL("sample_static: out, logits, seed and temperatures are required");
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
        LLMK_FAIL("sample_static: no usable current device (%s, device %d)", cudaGetErrorString(e), dev);
    void* base = nullptr;
    {
        std::lock_guard<std::mutex> guard(g_static_lock);
        if (!g_static_ptr[dev]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_sample_static_scratch);
            if (e != cudaSuccess || !p) {
                snprintf(g_llmk_error, sizeof(g_llmk_error), "sample_static: cudaGetSymbolAddress failed on device %d: %s",
                         dev, cudaGetErrorString(e));
                return LLMK_CUDA_ERROR;
            }
            g_static_ptr[dev] = p;
        }
        base = g_static_ptr[dev];
    }
    cudaStream_t s = (cudaStream_t)stream;
    float* pv = (float*)base;
    int* pi = (int*)(pv + (size_t)n_rows * SPLIT);
    sample_partial_kernel<<<dim3(n_rows, SPLIT), THREADS, 0, s>>>(pv, pi, logits, ld, temps, seed, V);
    LLMK_CHECK_LAUNCH("sample_static (first stage)");
    sample_final_kernel<<<n_rows, 32, 0, s>>>(out, pv, pi);
    LLMK_CHECK_LAUNCH("sample_static (second stage)");
    return LLMK_OK;
}
