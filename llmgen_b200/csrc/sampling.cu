// Sampling on the GPU, so that a step hands back one int32 per sequence instead of its logits.
//
// The scheme is the reference's (src/backend/cpu/sample.zig:16-45, src/backend/cuda/sample/sample.cu):
// temperature <= 0 is argmax with ties to the smaller id; temperature > 0 is Gumbel-max,
// argmax(logit / T - log(-log u)), with u from a stateless hash: u = ((r >> 40) + 0.5) / 2^24,
// r = splitmix64(row_seed + id), row_seed = splitmix64(row_key), where row_key is step_seed ^ (row << 40)
// (the reference's rule) or, when the caller gives an array of keys, that row's own key (the engine passes
// keys made of the request and the position, so that a draw does not depend on the batch).  Logits are float32
// here (bfloat16 in the reference), the division by T is a division and log is the accurate `logf`,
// so that a host restatement in float32 picks the same ids.
//
// One launch.  A (score, id) pair is packed into one 64-bit key whose unsigned order is "higher score
// first, then smaller id": the score's bits made monotonic in the upper word, ~id in the lower.  Every
// reduction is then a plain maximum.  SPLIT blocks a row each scan a share of the vocabulary with 16-byte
// loads, reduce their keys by shuffles and leave one candidate in scratch; the block that draws the
// row's last ticket takes the maximum of the candidates, writes the id and puts the ticket counter back
// to zero.  Scratch: SPLIT keys a row, then one counter a row, which must be zero before the first
// launch and is zero after every launch.  A row without any comparable score (all NaN) gives id 0.
#include "common.cuh"

LLMK_DEFINE_LAST_ERROR()

constexpr int SPLIT = 32;          // candidates a row
constexpr int THREADS = 256;
constexpr int PER_LOAD = 4;        // logits per 16-byte load

__host__ __device__ inline unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// 0 is below every key of a real score.
__device__ __forceinline__ unsigned long long sample_key(float score, int id) {
    if (score != score) return 0ull;                    // not comparable: never chosen
    const unsigned bits = __float_as_uint(score + 0.0f);          // -0 becomes +0: equal scores, equal bits
    const unsigned ordered = bits ^ ((bits >> 31) ? 0xFFFFFFFFu : 0x80000000u);
    return ((unsigned long long)ordered << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)id);
}
__device__ __forceinline__ int key_id(unsigned long long key, int V) {
    const unsigned id = 0xFFFFFFFFu - (unsigned)(key & 0xFFFFFFFFull);
    return key != 0ull && id < (unsigned)V ? (int)id : 0;
}
__device__ __forceinline__ unsigned long long warp_max_key(unsigned long long k) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, k, o);
        k = other > k ? other : k;
    }
    return k;
}

__device__ __forceinline__ float gumbel_score(float logit, float temp, unsigned long long row_seed, int id) {
    const unsigned long long r = splitmix64(row_seed + (unsigned long long)id);
    const float u = ((float)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);      // in (0, 1)
    return logit / temp - logf(-logf(u));
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(int* __restrict__ out, unsigned long long* __restrict__ cand, unsigned* __restrict__ tickets,
              const float* __restrict__ logits, long long ld, const float* __restrict__ temps,
              const unsigned long long* seed_ptr, const unsigned long long* __restrict__ row_keys, int V) {
    const int share = blockIdx.x, row = blockIdx.y;
    const float* x = logits + (size_t)row * ld;
    const float temp = temps[row];
    const bool draw = temp > 0.f;
    const unsigned long long row_seed =
        draw ? splitmix64(row_keys ? row_keys[row] : (*seed_ptr ^ ((unsigned long long)row << 40))) : 0ull;
    // shares start on multiples of 4 ids, so that a row on a 16-byte boundary is read 16 bytes at a time
    const int per = (((V + SPLIT - 1) / SPLIT) + PER_LOAD - 1) / PER_LOAD * PER_LOAD;
    const int beg = share * per, end = min(V, beg + per);
    unsigned long long best = 0ull;
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        for (int i = beg + threadIdx.x * PER_LOAD; i < end; i += THREADS * PER_LOAD) {
            float v[PER_LOAD];
            if (i + PER_LOAD <= end) {
                const float4 q = __ldcs(reinterpret_cast<const float4*>(x + i));
                v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
            } else {
#pragma unroll
                for (int e = 0; e < PER_LOAD; ++e) v[e] = i + e < end ? x[i + e] : __int_as_float(0x7fc00000);   // NaN: skipped
            }
#pragma unroll
            for (int e = 0; e < PER_LOAD; ++e) {
                const unsigned long long k = sample_key(draw ? gumbel_score(v[e], temp, row_seed, i + e) : v[e], i + e);
                best = k > best ? k : best;
            }
        }
    } else {
        for (int i = beg + threadIdx.x; i < end; i += THREADS) {
            const unsigned long long k = sample_key(draw ? gumbel_score(x[i], temp, row_seed, i) : x[i], i);
            best = k > best ? k : best;
        }
    }
    __shared__ unsigned long long warp_best[THREADS / 32];
    __shared__ int merges;
    best = warp_max_key(best);
    if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 1; w < THREADS / 32; ++w) best = warp_best[w] > best ? warp_best[w] : best;
        cand[(size_t)row * SPLIT + share] = best;
        __threadfence();                                         // the candidate is visible before the ticket is
        merges = atomicAdd(&tickets[row], 1u) == (unsigned)(SPLIT - 1);
    }
    __syncthreads();
    if (!merges || threadIdx.x >= 32) return;
    __threadfence();
    unsigned long long k = __ldcg(&cand[(size_t)row * SPLIT + threadIdx.x]);     // SPLIT == 32: a candidate a lane
    k = warp_max_key(k);
    if (threadIdx.x == 0) {
        out[row] = key_id(k, V);
        tickets[row] = 0u;                                       // every block of the row has drawn: ready for the next launch
    }
}

// Bytes of scratch for up to `max_rows` rows; its last max_rows * 4 bytes (the ticket counters) must be zero
// before the first launch.
LLMK_EXPORT long long llmk_sample_scratch_bytes(int max_rows) { return (long long)max_rows * (SPLIT * 8 + 4); }

static int launch_sample(int* out, void* scratch, const float* logits, long long ld, const float* temps,
                         const unsigned long long* seed, const unsigned long long* row_keys, int n_rows, int V,
                         int scratch_rows, cudaStream_t s, const char* what) {
    unsigned long long* cand = static_cast<unsigned long long*>(scratch);
    unsigned* tickets = reinterpret_cast<unsigned*>(cand + (size_t)scratch_rows * SPLIT);
    sample_kernel<<<dim3(SPLIT, n_rows), THREADS, 0, s>>>(out, cand, tickets, logits, ld, temps, seed, row_keys, V);
    LLMK_CHECK_LAUNCH(what);
    return LLMK_OK;
}

// out[s] = sampled id of row s of logits [n_rows, V] (row stride ld); temps[s] <= 0 is greedy.
// `seed` points at the step's 64-bit seed on the device (so a replayed CUDA graph only needs
// the value refreshed); with `row_keys` (64 bits a row, device) it is not read and may be null.  `scratch` holds llmk_sample_scratch_bytes(scratch_rows) bytes, scratch_rows >= n_rows,
// 8-byte aligned, its ticket counters zero (they are left zero).
LLMK_EXPORT int llmk_sample(int* out, const float* logits, long long ld, const float* temps,
                            const unsigned long long* seed, const unsigned long long* row_keys, int n_rows, int V,
                            void* scratch, int scratch_rows, void* stream) {
    if (n_rows <= 0) return LLMK_OK;
    if (V <= 0 || ld < V) LLMK_FAIL("sample: bad sizes V=%d ld=%lld", V, ld);
    if (n_rows > 65535) LLMK_FAIL("sample: %d rows exceed the grid", n_rows);
    if (!scratch || (!seed && !row_keys) || !temps) LLMK_FAIL("sample: scratch, a seed or row keys, and temperatures are required");
    if (scratch_rows < n_rows || (reinterpret_cast<uintptr_t>(scratch) & 7) != 0)
        LLMK_FAIL("sample: scratch for %d rows (8-byte aligned) cannot serve %d", scratch_rows, n_rows);
    return launch_sample(out, scratch, logits, ld, temps, seed, row_keys, n_rows, V, scratch_rows, (cudaStream_t)stream, "sample");
}

// ------------------------------------------------------------------ sampling without an allocator
// `llmk_sample_static` (declared in llmk_sample_static.h) is `llmk_sample` for callers that cannot
// hand over scratch memory because they cannot allocate any: code running where cudaMalloc is off
// limits, such as a host that embeds this library beside a runtime owning all device memory, or a
// callback that must not call into an allocator.  The blocks' candidates and the rows' ticket counters
// go to a file-scope device array instead of a caller's buffer.  Every GPU that loads this library holds
// the array (LLMK_SAMPLE_STATIC_MAX_ROWS * (32 * 8 + 4) bytes = 65 KiB) until the process exits.
//
// In host code `g_sample_static_scratch` is only a handle for the runtime, not a device address;
// the address is asked for once per device with cudaGetSymbolAddress, with that device current,
// on the first call made on that device.  That first call should therefore come before any stream
// capture.  The candidates are overwritten before they are read, and the ticket counters, which must
// start at zero, do: the array is zero when the library is loaded, and the block that merges a row puts
// that row's counter back to zero, so nothing has to be cleared between calls.  But all calls share the
// one array, so two calls that overlap on the GPU (different streams) race.
#include "llmk_sample_static.h"

#include <mutex>

static __device__ __align__(256) unsigned char g_sample_static_scratch[LLMK_SAMPLE_STATIC_MAX_ROWS * (SPLIT * 8 + 4)];

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
    return launch_sample(out, base, logits, ld, temps, seed, nullptr, n_rows, V, LLMK_SAMPLE_STATIC_MAX_ROWS, (cudaStream_t)stream,
                         "sample_static");
}
