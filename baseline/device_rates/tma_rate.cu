// L2 -> shared memory rate of TMA tile loads, per SM and over all SMs, with no compute: a ring of STAGES stages of
// BOXES boxes of [BOXROWS rows, 64 bfloat16] each (128-byte swizzle), one mbarrier per stage; one thread (or two)
// issues the copies, another frees a stage as soon as it is full.  The source (32 MB) stays in L2.  Every wait is
// bounded (tc::mbar_wait).  Build and run: baseline/device_rates.py.
#include <cstdio>
#include <cstdint>
#include <mutex>
#include <unordered_map>
#include <cuda.h>
#include <cuda_runtime.h>
#include "tcgen05.cuh"

template <int STAGES, int BOXES, int PRODUCERS, int BOXROWS>
__global__ void __launch_bounds__(96) tma_kernel(const __grid_constant__ CUtensorMap map, long long* cycles, int slices,
                                                 int rows_total, int k_slices, int* err) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ uint64_t full[STAGES], empty[STAGES];
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < STAGES; ++i) { tc::mbar_init(tc::smem_u32(&full[i]), 1); tc::mbar_init(tc::smem_u32(&empty[i]), 1); }
        tc::fence_barrier_init();
    }
    __syncthreads();
    const long long c0 = clock64();
    if (threadIdx.x == 0 || (PRODUCERS == 2 && threadIdx.x == 64)) {                      // producer(s)
        const int me = threadIdx.x == 0 ? 0 : 1;
        bool ok = true;
        int kb = 0, rowbase = (blockIdx.x * BOXES * BOXROWS) % rows_total, s = 0, ph = 1;
        for (int i = 0; i < slices && ok; ++i) {
            if (i >= STAGES) ok = tc::mbar_wait(tc::smem_u32(&empty[s]), ph, &abort_flag);
            if (!ok) break;
            if (me == 0) tc::mbar_expect_tx(tc::smem_u32(&full[s]), BOXES * BOXROWS * 128);
            for (int b = me; b < BOXES; b += PRODUCERS)
                tc::tma_load_2d(tc::smem_u32(smem + (s * BOXES + b) * BOXROWS * 128), &map, tc::smem_u32(&full[s]), kb * 64, rowbase + b * BOXROWS);
            if (++kb == k_slices) { kb = 0; rowbase += 37 * 128; if (rowbase + BOXES * BOXROWS > rows_total) rowbase -= rows_total - BOXES * BOXROWS; if (rowbase < 0) rowbase = 0; }
            if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) atomicExch(err, 1);
    } else if (threadIdx.x == 32) {              // consumer
        bool ok = true;
        int s = 0, ph = 0;
        for (int i = 0; i < slices && ok; ++i) {
            ok = tc::mbar_wait(tc::smem_u32(&full[s]), ph, &abort_flag);
            tc::mbar_arrive(tc::smem_u32(&empty[s]));
            if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) atomicExch(err, 2);
        cycles[blockIdx.x] = clock64() - c0;
    }
}

template <int STAGES, int BOXES, int PRODUCERS, int BOXROWS>
void run(int blocks, const CUtensorMap& map, int rows, int k_slices) {
    long long* cyc; int* err;
    cudaMalloc(&cyc, blocks * 8); cudaMalloc(&err, 4); cudaMemset(err, 0, 4);
    const int smem = STAGES * BOXES * BOXROWS * 128 + 1024;
    cudaFuncSetAttribute(tma_kernel<STAGES, BOXES, PRODUCERS, BOXROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    const int slices = 4000;
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    tma_kernel<STAGES, BOXES, PRODUCERS, BOXROWS><<<blocks, 96, smem>>>(map, cyc, slices, rows, k_slices, err);
    cudaEventRecord(e0);
    tma_kernel<STAGES, BOXES, PRODUCERS, BOXROWS><<<blocks, 96, smem>>>(map, cyc, slices, rows, k_slices, err);
    cudaEventRecord(e1);
    cudaError_t e = cudaDeviceSynchronize();
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    long long hc[148]; int herr;
    cudaMemcpy(hc, cyc, blocks * 8, cudaMemcpyDeviceToHost); cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost);
    double mc = 0; for (int i = 0; i < blocks; ++i) mc += hc[i]; mc /= blocks;
    const double bytes = (double)slices * BOXES * BOXROWS * 128;
    printf("stages %d x %d boxes of %3d rows, %d producers, blocks %3d: %6.1f B/clk/SM, %6.0f cycles / slice, %7.2f TB/s over all (%s, err %d)\n", STAGES, BOXES, BOXROWS, PRODUCERS, blocks,
           bytes / mc, mc / slices, bytes * blocks / (ms * 1e-3) / 1e12, cudaGetErrorString(e), herr);
    cudaFree(cyc); cudaFree(err);
}

int main() {
    const int rows = 8192, cols = 2048;         // 32 MB of bfloat16: stays in L2
    void* buf; cudaMalloc(&buf, (size_t)rows * cols * 2); cudaMemset(buf, 0, (size_t)rows * cols * 2);
    CUtensorMap map128, map64, map16;
    if (!tc_host::make_map_bf16_2d(&map128, buf, rows, cols, cols, 128) || !tc_host::make_map_bf16_2d(&map64, buf, rows, cols, cols, 64) ||
        !tc_host::make_map_bf16_2d(&map16, buf, rows, cols, cols, 16)) { printf("map failed\n"); return 1; }
    const int ks = cols / 64;
    for (int blocks : {1, 148}) {
        run<4, 1, 1, 128>(blocks, map128, rows, ks);     // 16 KB a stage
        run<4, 2, 1, 128>(blocks, map128, rows, ks);     // 32 KB: a 128 x 128 tile's step of 64 along K
        run<6, 2, 1, 128>(blocks, map128, rows, ks);     // the same with a deeper ring
        run<4, 2, 2, 128>(blocks, map128, rows, ks);     // the same with two issuing threads
        run<4, 3, 1, 128>(blocks, map128, rows, ks);     // 48 KB: a 128 x 256 tile's step
        run<3, 4, 1, 128>(blocks, map128, rows, ks);     // 64 KB: two steps of a 128 x 128 tile
        run<2, 6, 1, 128>(blocks, map128, rows, ks);     // 96 KB
        run<6, 2, 1, 64>(blocks, map64, rows, ks);       // 16 KB in two boxes
        run<4, 16, 1, 16>(blocks, map16, rows, ks);      // 32 KB in 16 boxes of 16 rows: a key tile of 8 pages of 16 keys
    }
    return 0;
}
