// What the second pass of an attention softmax costs by itself on one SM: every thread holds 64 scores in registers
// and, per tile, turns them into exponentials (one fma and one `ex2.approx` each), sums them, packs them to bfloat16
// and stores them to shared memory in 16-byte pieces.  Printed: cycles a tile and cycles per value and thread, for
// 4, 8 and 16 warps a block (one block an SM), with the parts added one by one, and with every 4th or 2nd
// exponential computed by a cubic on the FMA pipe instead of the special-function unit.
//
// A 128 x 128 tile of scores is 16,384 exponentials: at 16 results a clock and SM the unit alone needs 1,024 cycles,
// as long as the tile's two products take on the tensor core.
#include <cstdint>
#include <cstdio>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

__device__ __forceinline__ float unit_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 2^x = 2^n * 2^r, n the nearest integer (left in the low mantissa bits of x + 1.5 * 2^23), r in [-0.5, 0.5], a cubic
// for 2^r (relative error 7.5e-5), n added to the exponent field
__device__ __forceinline__ float cubic_exp2(float x) {
    x = fmaxf(x, -125.f);
    const float t = x + 12582912.f;
    const float r = x - (t - 12582912.f);
    float p = fmaf(0.0551716648f, r, 0.2426111251f);
    p = fmaf(p, r, 0.6932609677f);
    p = fmaf(p, r, 0.9999280572f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}

// PARTS: 0 fma + ex2 (+ a max that keeps the result alive), 1 + the row sum, 2 + packing, 3 + the stores.
// CUBIC: every CUBIC-th value by the cubic (0: none, 1: all).
template <int PARTS, int CUBIC>
__global__ void __launch_bounds__(512) second_pass(float* out, long long* cycles, int tiles, float scale, float shift0) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int r = threadIdx.x & 127, half = (threadIdx.x >> 7) & 1;
    uint8_t* p_row = smem + half * (128 * 128) + r * 128 + (threadIdx.x >> 8) * 32768;
    float v[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = (float)((threadIdx.x * 7 + i * 13) % 97) * 0.01f;
    float l = 0.f, shift = shift0;
    __syncthreads();
    const long long t0 = clock64();
    for (int j = 0; j < tiles; ++j) {
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            float pv[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float x = fmaf(v[c * 32 + i], scale, -shift);
                constexpr int every = CUBIC > 0 ? CUBIC : 1;
                if (CUBIC > 0 && i % every == every - 1) pv[i] = cubic_exp2(x);
                else pv[i] = unit_exp2(x);
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                if (PARTS >= 1) sum4[i & 3] += pv[i];
                else sum4[i & 3] = fmaxf(sum4[i & 3], pv[i]);
            }
            if (PARTS >= 2) {
#pragma unroll
                for (int q8 = 0; q8 < 4; ++q8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat162 two = __floats2bfloat162_rn(pv[q8 * 8 + 2 * e], pv[q8 * 8 + 2 * e + 1]);
                        w[e] = *reinterpret_cast<const uint32_t*>(&two);
                    }
                    if (PARTS >= 3) {
                        const int piece = c * 4 + q8;
                        *reinterpret_cast<uint4*>(p_row + ((piece ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    } else {
                        sum4[q8] += __uint_as_float(w[0] ^ w[1] ^ w[2] ^ w[3]) * 1e-30f;
                    }
                }
            }
        }
        l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        shift += 1e-3f;            // the next tile's exponentials are new work
    }
    const long long t1 = clock64();
    out[blockIdx.x * blockDim.x + threadIdx.x] = l;
    if (threadIdx.x == 0 && blockIdx.x == 0) *cycles = t1 - t0;
}

template <int PARTS, int CUBIC>
static int run(const char* what, int warps, int sms) {
    float* out = nullptr;
    long long* cyc = nullptr;
    if (cudaMalloc(&out, (size_t)sms * 512 * 4) != cudaSuccess || cudaMalloc(&cyc, 8) != cudaSuccess) return 1;
    const int tiles = 64;
    cudaFuncSetAttribute(second_pass<PARTS, CUBIC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    for (int it = 0; it < 2; ++it) second_pass<PARTS, CUBIC><<<sms, warps * 32, 65536>>>(out, cyc, tiles, 0.1275f, 0.3f);
    const cudaError_t e = cudaDeviceSynchronize();
    long long h = 0;
    cudaMemcpy(&h, cyc, 8, cudaMemcpyDeviceToHost);
    printf("| %-52s | %2d | %7.0f | %5.1f |%s\n", what, warps, (double)h / tiles, (double)h / tiles / 64,
           e == cudaSuccess ? "" : cudaGetErrorString(e));
    cudaFree(out);
    cudaFree(cyc);
    return e == cudaSuccess ? 0 : 1;
}

int main() {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, 0) != cudaSuccess) return 1;
    const int sms = prop.multiProcessorCount;
    printf("\nexp_rate: the softmax's second pass alone, 64 values a thread and tile, one block on each of %d SMs\n\n", sms);
    printf("| what a value costs | warps | cycles a tile | cycles per value and thread |\n|---|---:|---:|---:|\n");
    int bad = 0;
    for (int warps : {4, 8, 16}) {
        bad += run<0, 0>("fma, ex2", warps, sms);
        bad += run<1, 0>("fma, ex2, row sum", warps, sms);
        bad += run<2, 0>("+ pack to bfloat16", warps, sms);
        bad += run<3, 0>("+ 16-byte stores to shared memory", warps, sms);
        bad += run<3, 4>("all of it, every 4th exponential by a cubic", warps, sms);
        bad += run<3, 2>("all of it, every 2nd exponential by a cubic", warps, sms);
        bad += run<1, 1>("fma, cubic, row sum (no ex2)", warps, sms);
    }
    return bad ? 1 : 0;
}
