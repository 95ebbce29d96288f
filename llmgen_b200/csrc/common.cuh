// Shared device helpers and the C-ABI conventions of every kernel module.
//
// Conventions: each exported function is `extern "C" int llmk_<name>(..., int dtype, void* stream)`;
// it returns 0 on success and a non-zero code after writing a message that
// `llmk_last_error()` returns.  `dtype` is 0 for float32 and 1 for bfloat16 and selects the
// storage type of activations, matrices and the cache; reductions, softmax, norms, rotary
// angles and the residual stream are float32 in both.  Nothing here allocates or synchronises.
//
// The reference keeps the same split between `extern "C"` launchers and kernels and shares
// `bf16x8`, `warp_sum`, `block_sum` helpers (src/backend/cuda/utils.cuh:30-126); its errors are
// printed and swallowed (utils.cuh:79-90), here they are returned.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <utility>

#define LLMK_EXPORT extern "C" __attribute__((visibility("default")))

enum { LLMK_OK = 0, LLMK_BAD_ARG = 1, LLMK_CUDA_ERROR = 2 };
enum { LLMK_F32 = 0, LLMK_BF16 = 1 };
// How a rotary encoding pairs the values of a head, and which norm runs over a head of q and k before it:
// kernels take the codes and refuse the ones they do not implement.
enum { LLMK_PAIR_HALF_SPLIT = 0, LLMK_PAIR_INTERLEAVED = 1 };
enum { LLMK_HEAD_NORM_RMS = 0 };

typedef __nv_bfloat16 bf16;

static thread_local char g_llmk_error[1024] = "";

#define LLMK_FAIL(...)                                              \
    do {                                                            \
        snprintf(g_llmk_error, sizeof(g_llmk_error), __VA_ARGS__);  \
        return LLMK_BAD_ARG;                                        \
    } while (0)

#define LLMK_CHECK_LAUNCH(what)                                                                  \
    do {                                                                                         \
        cudaError_t e__ = cudaGetLastError();                                                    \
        if (e__ != cudaSuccess) {                                                                \
            snprintf(g_llmk_error, sizeof(g_llmk_error), "%s: %s", what, cudaGetErrorString(e__)); \
            return LLMK_CUDA_ERROR;                                                              \
        }                                                                                        \
    } while (0)

#define LLMK_DEFINE_LAST_ERROR() \
    LLMK_EXPORT const char* llmk_last_error() { return g_llmk_error; }

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float x) { return __float2bfloat16_rn(x); }

// A 16-byte vector of T: 4 floats or 8 bfloat16.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    float4 raw;
    __device__ __forceinline__ void unpack(float* f) const { f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w; }
    __device__ __forceinline__ void pack(const float* f) { raw = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec16<bf16> {
    static constexpr int N = 8;
    uint4 raw;
    __device__ __forceinline__ void unpack(float* f) const {
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 v = __bfloat1622float2(p[i]);
            f[2 * i] = v.x;
            f[2 * i + 1] = v.y;
        }
    }
    __device__ __forceinline__ void pack(const float* f) {
        __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    }
};

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline bool host_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Streaming multiprocessors of the current device, asked once per device; launch plans (how many
// slices, how many blocks) are made from it.  Without a device (a build check on a CPU box): a B200's 148.
inline int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return 148;
    }
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = 148;
        }
        cached[dev] = n;
    }
    return cached[dev];
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the block; every thread gets the result.  `scratch` holds 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// ------------------------------------------------------------- programmatic dependent launch
// A kernel launched with `llmk_launch(..., pdl = true)` may start while the kernel before it in
// the stream is still draining.  Such a kernel must call `pdl_wait()` before it reads anything an
// earlier kernel wrote or writes anything an earlier kernel may still read; what comes before the
// wait (barrier set-up, loads of weights) overlaps the predecessor's tail.  `pdl_launch_dependents()`
// lets the next kernel begin its own prologue.  Both are no-ops in a plain launch.  LLMGEN_PDL=0 in
// the environment turns the attribute off everywhere.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool llmk_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("LLMGEN_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on != 0;
}

template <typename... KArgs, typename... Args>
inline cudaError_t llmk_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               bool pdl, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl && llmk_pdl_enabled()) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// The same for a grid of thread-block clusters of `cluster` blocks.
template <typename... KArgs, typename... Args>
inline cudaError_t llmk_launch_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                        bool pdl, dim3 cluster, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x;
    attr[0].val.clusterDim.y = cluster.y;
    attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl && llmk_pdl_enabled()) ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
// ... of (1, cluster_y, 1) blocks
template <typename... KArgs, typename... Args>
inline cudaError_t llmk_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                       bool pdl, unsigned cluster_y, Args&&... args) {
    return llmk_launch_clusters(kernel, grid, block, smem, stream, pdl, dim3(1, cluster_y, 1), std::forward<Args>(args)...);
}

// Thread-block clusters: rank of this block, another block's view of a shared-memory address, a load
// through it, and the cluster-wide barrier (every thread of every block of the cluster executes it).
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_map_shared(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float cluster_ld_f32(uint32_t cluster_addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

#define LLMK_CHECK_LAUNCH_RC(what, rc__)                                                           \
    do {                                                                                           \
        cudaError_t e__ = (rc__);                                                                  \
        if (e__ != cudaSuccess) {                                                                  \
            snprintf(g_llmk_error, sizeof(g_llmk_error), "%s: %s", what, cudaGetErrorString(e__)); \
            return LLMK_CUDA_ERROR;                                                                \
        }                                                                                          \
    } while (0)
