// How long one tcgen05.mma (M = 128, N = 64 / 128 / 256, K = 16, bfloat16 operands in shared memory, float32
// accumulator in tensor memory) takes when one thread issues them back to back, on one SM and on all.  The only wait
// is bounded (tc::mbar_wait).  Build and run: baseline/device_rates.py.
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include "tcgen05.cuh"

template <int N, int NACC>
__global__ void __launch_bounds__(128) rate_kernel(long long* cycles, unsigned long long* ns, int iters, int* err) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < (16384 + N * 128) / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        tc::mbar_init(tc::smem_u32(&bar), 1);
        tc::fence_barrier_init();
    }
    tc::fence_proxy_async();
    if (warp == 1) {
        tc::tmem_alloc(tc::smem_u32(&tmem_slot), 512);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    if (threadIdx.x == 0) {
        const uint64_t adesc = tc::smem_desc_sw128(tc::smem_u32(smem));
        const uint64_t bdesc = tc::smem_desc_sw128(tc::smem_u32(smem + 16384));
        constexpr uint32_t idesc = tc::idesc_bf16_f32(128, N);
        const long long c0 = clock64();
        const unsigned long long t0 = tc::global_timer();
        for (int it = 0; it < iters; ++it) {
            const uint32_t d = tmem + (uint32_t)((it % NACC) * N);
#pragma unroll
            for (int k = 0; k < 4; ++k) tc::mma_bf16_ss(d, adesc + 2 * k, bdesc + 2 * k, idesc, true);
        }
        tc::mma_commit(tc::smem_u32(&bar));
        const bool ok = tc::mbar_wait(tc::smem_u32(&bar), 0, &abort_flag);
        const long long c1 = clock64();
        const unsigned long long t1 = tc::global_timer();
        if (!ok) atomicExch(err, 1);
        cycles[blockIdx.x] = c1 - c0;
        ns[blockIdx.x] = t1 - t0;
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, 512);
}

template <int N, int NACC>
void run(int blocks, int iters) {
    long long* cyc; unsigned long long* ns; int* err;
    cudaMalloc(&cyc, blocks * 8); cudaMalloc(&ns, blocks * 8); cudaMalloc(&err, 4); cudaMemset(err, 0, 4);
    const int smem = 16384 + N * 128 + 1024;
    cudaFuncSetAttribute(rate_kernel<N, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    for (int rep = 0; rep < 2; ++rep) rate_kernel<N, NACC><<<blocks, 128, smem>>>(cyc, ns, iters, err);
    cudaError_t e = cudaDeviceSynchronize();
    long long hc[148]; unsigned long long hn[148]; int herr;
    cudaMemcpy(hc, cyc, blocks * 8, cudaMemcpyDeviceToHost); cudaMemcpy(hn, ns, blocks * 8, cudaMemcpyDeviceToHost);
    cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost);
    double mc = 0, mn = 0;
    for (int i = 0; i < blocks; ++i) { mc += hc[i]; mn += hn[i]; }
    mc /= blocks; mn /= blocks;
    const double per = 4.0 * iters;
    printf("M=128 N=%3d acc=%d blocks=%3d: %7.1f cycles / mma, %6.1f ns / mma, %6.0f TFLOP/s all blocks (%s, err %d)\n", N, NACC, blocks,
           mc / per, mn / per, 2.0 * 128 * N * 16 * blocks / (mn / per) / 1e3, cudaGetErrorString(e), herr);
    cudaFree(cyc); cudaFree(ns); cudaFree(err);
}

int main() {
    const int iters = 2000;
    for (int blocks : {1, 148}) {
        run<64, 1>(blocks, iters);
        run<128, 1>(blocks, iters);
        run<128, 2>(blocks, iters);
        run<256, 1>(blocks, iters);
        run<256, 2>(blocks, iters);
    }
    return 0;
}
