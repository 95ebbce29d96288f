// How long one tcgen05.mma (M = 128, N = 64 / 128 / 256, K = 16, bfloat16 operands in shared memory, float32
// accumulator in tensor memory) takes when one thread issues them back to back, on one SM and on all.  The only wait
// is bounded (tc::mbar_wait).  Build and run: baseline/device_rates.py.
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include "tcgen05.cuh"

// BMN: B is read MN-major (its rows contiguous, as a [K, N] tile: the V operand of attention's P V).
// NOISE: what the block's other three warps do meanwhile: 0 nothing, 1 load tensor memory, 2 store to shared memory,
// 3 one thread has TMA write boxes of [128, 64] (16 KB) from L2 into eight other buffers of the block's shared memory,
// two boxes per barrier, four barriers in flight, each pair asked for again as soon as it has landed: shared memory then
// serves the MMA's operand reads and TMA's writes.
// SETS: how many different operand sets (A and B tiles, 16 KB + N * 128 bytes each) the instructions walk through in
// turn, a set per four instructions (one step of 64 along K), as a kernel's ring of stages does; 1: the same tiles again.
template <int N, int NACC, bool BMN = false, int NOISE = 0, int SETS = 1>
__global__ void __launch_bounds__(128) rate_kernel(long long* cycles, unsigned long long* ns, int iters, int* err,
                                                   const __grid_constant__ CUtensorMap map, long long* tma_bytes) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ volatile int done;
    constexpr int TB = 4;                  // pairs of boxes in flight
    __shared__ uint64_t tma_bar[TB];
    const int warp = threadIdx.x >> 5;
    constexpr int SET_BYTES = 16384 + N * 128;
    for (int i = threadIdx.x; i < SETS * SET_BYTES / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        done = 0;
        tc::mbar_init(tc::smem_u32(&bar), 1);
        for (int b = 0; b < TB; ++b) tc::mbar_init(tc::smem_u32(&tma_bar[b]), 1);
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
        const uint64_t bdesc = BMN ? tc::smem_desc_sw128_mn(tc::smem_u32(smem + 16384), 128 * 128, 1024)
                                   : tc::smem_desc_sw128(tc::smem_u32(smem + 16384));
        constexpr uint32_t idesc = BMN ? tc::idesc_bf16_f32_b_mn(128, N) : tc::idesc_bf16_f32(128, N);
        const long long c0 = clock64();
        const unsigned long long t0 = tc::global_timer();
        for (int it = 0; it < iters; ++it) {
            const uint32_t d = tmem + (uint32_t)((it % NACC) * N);
            const uint64_t off = (uint64_t)(((it % SETS) * SET_BYTES) >> 4);      // the start address is the descriptor's lowest field, in units of 16 bytes
#pragma unroll
            for (int k = 0; k < 4; ++k) tc::mma_bf16_ss(d, adesc + off + 2 * k, bdesc + off + (BMN ? 128 * k : 2 * k), idesc, true);
        }
        tc::mma_commit(tc::smem_u32(&bar));
        const bool ok = tc::mbar_wait(tc::smem_u32(&bar), 0, &abort_flag);
        const long long c1 = clock64();
        const unsigned long long t1 = tc::global_timer();
        if (!ok) atomicExch(err, 1);
        cycles[blockIdx.x] = c1 - c0;
        ns[blockIdx.x] = t1 - t0;
        done = 1;
    } else if (NOISE == 3) {
        if (threadIdx.x == 32) {
            // a pair is asked for again as soon as it has landed.  Bounded by the issuing thread's end and by a count;
            // what is in flight at the end is waited for (bounded) before the block leaves.
            const uint32_t ring = tc::smem_u32(smem) + SETS * SET_BYTES + 1024;
            const int row0 = (blockIdx.x % 32) * 256;
            long long boxes = 0;
            uint32_t phase[TB];
            bool ok = true;
            for (int b = 0; b < TB; ++b) {
                phase[b] = 0;
                tc::mbar_expect_tx(tc::smem_u32(&tma_bar[b]), 32768);
                tc::tma_load_2d(ring + b * 32768, &map, tc::smem_u32(&tma_bar[b]), b * 64, row0);
                tc::tma_load_2d(ring + b * 32768 + 16384, &map, tc::smem_u32(&tma_bar[b]), b * 64, row0 + 128);
            }
            for (int it = 0; it < 400000 && ok; ++it) {
                const int b = it % TB;
                ok = tc::mbar_wait(tc::smem_u32(&tma_bar[b]), phase[b], &abort_flag);
                phase[b] ^= 1;
                boxes += 2;
                if (done || !ok) {          // the other pairs are still in flight
                    for (int o = 1; o < TB && ok; ++o) {
                        ok = tc::mbar_wait(tc::smem_u32(&tma_bar[(b + o) % TB]), phase[(b + o) % TB], &abort_flag);
                        boxes += 2;
                    }
                    break;
                }
                tc::mbar_expect_tx(tc::smem_u32(&tma_bar[b]), 32768);
                tc::tma_load_2d(ring + b * 32768, &map, tc::smem_u32(&tma_bar[b]), (it % 16) * 64, row0);
                tc::tma_load_2d(ring + b * 32768 + 16384, &map, tc::smem_u32(&tma_bar[b]), (it % 16) * 64, row0 + 128);
            }
            if (!ok) atomicExch(err, 3);
            tma_bytes[blockIdx.x] = boxes * 16384;
        }
    } else if (NOISE != 0 && warp >= 1 && warp < 4) {
        // bounded by the issuing thread's own end (its wait is bounded) and by a count of its own
        uint32_t r[32];
        for (int i = 0; i < 32; ++i) r[i] = threadIdx.x + i;
        for (int it = 0; it < 400000 && !done; ++it) {
            if (NOISE == 1) {
                tc::tmem_ld_32x32_wait(tmem + ((uint32_t)(warp * 32) << 16) + 256u + (uint32_t)((it & 3) * 32), r);
            } else {
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    tc::st_shared_v4(tc::smem_u32(smem) + SETS * SET_BYTES + 1024 + (uint32_t)(((threadIdx.x * 8 + q + it) & 1023) << 4),
                                     make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]));
            }
        }
        if (r[0] == 0xdeadbeefu) atomicExch(err, 7);     // keeps the loads alive
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, 512);
}

CUtensorMap g_map;        // [8192, 1024] bfloat16 in boxes of [128, 64], for the TMA writes of NOISE 3

template <int N, int NACC, bool BMN = false, int NOISE = 0, int SETS = 1>
void run(int blocks, int iters) {
    long long* cyc; unsigned long long* ns; int* err; long long* tb;
    cudaMalloc(&cyc, blocks * 8); cudaMalloc(&ns, blocks * 8); cudaMalloc(&err, 4); cudaMemset(err, 0, 4);
    cudaMalloc(&tb, blocks * 8); cudaMemset(tb, 0, blocks * 8);
    // A, B, alignment slack, and what the noise writes: 16 KB for the stores, 128 KB for the TMA boxes
    const int smem = SETS * (16384 + N * 128) + 1024 + 1024 + (NOISE == 3 ? 131072 : 16384);
    cudaFuncSetAttribute(rate_kernel<N, NACC, BMN, NOISE, SETS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    for (int rep = 0; rep < 2; ++rep) rate_kernel<N, NACC, BMN, NOISE, SETS><<<blocks, 128, smem>>>(cyc, ns, iters, err, g_map, tb);
    cudaError_t e = cudaDeviceSynchronize();
    long long hc[148], hb[148]; unsigned long long hn[148]; int herr;
    cudaMemcpy(hc, cyc, blocks * 8, cudaMemcpyDeviceToHost); cudaMemcpy(hn, ns, blocks * 8, cudaMemcpyDeviceToHost);
    cudaMemcpy(hb, tb, blocks * 8, cudaMemcpyDeviceToHost);
    cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost);
    double mc = 0, mn = 0, mb = 0;
    for (int i = 0; i < blocks; ++i) { mc += hc[i]; mn += hn[i]; mb += hb[i]; }
    mc /= blocks; mn /= blocks; mb /= blocks;
    const double per = 4.0 * iters;
    printf("M=128 N=%3d acc=%d %s %s blocks=%3d: %7.1f cycles / mma, %6.1f ns / mma, %6.0f TFLOP/s all blocks", N, NACC, BMN ? "B MN-major" : "B K-major ",
           NOISE == 0 ? (SETS > 1 ? "alone, 4 operand sets" : "alone            ") : NOISE == 1 ? "beside tmem loads" : NOISE == 2 ? "beside smem stores"
                      : (SETS > 1 ? "beside TMA writes, 2 operand sets" : "beside TMA writes "), blocks,
           mc / per, mn / per, 2.0 * 128 * N * 16 * blocks / (mn / per) / 1e3);
    if (NOISE == 3) printf(", TMA wrote %.1f B/clk, the MMAs read %.1f B/clk", mb / mc, (128 + N) * 32.0 / (mc / per));
    printf(" (%s, err %d)\n", cudaGetErrorString(e), herr);
    cudaFree(cyc); cudaFree(ns); cudaFree(err); cudaFree(tb);
}

int main() {
    const int iters = 2000;
    void* buf = nullptr;
    if (cudaMalloc(&buf, (size_t)8192 * 1024 * 2) != cudaSuccess) return 1;
    cudaMemset(buf, 0, (size_t)8192 * 1024 * 2);
    if (!tc_host::make_map_bf16_2d(&g_map, buf, 8192, 1024, 1024, 128)) { printf("map failed\n"); return 1; }
    for (int blocks : {1, 148}) {
        run<64, 1>(blocks, iters);
        run<128, 1>(blocks, iters);
        run<128, 2>(blocks, iters);
        run<256, 1>(blocks, iters);
        run<256, 2>(blocks, iters);
        run<128, 1, true>(blocks, iters);
        run<128, 1, false, 1>(blocks, iters);
        run<128, 1, false, 2>(blocks, iters);
        run<128, 1, true, 1>(blocks, iters);
        run<128, 1, false, 3>(blocks, iters);
        run<256, 1, false, 3>(blocks, iters);
        run<64, 1, false, 3>(blocks, iters);
        run<128, 1, false, 0, 4>(blocks, iters);
        run<256, 1, false, 0, 4>(blocks, iters);
        run<128, 1, false, 3, 2>(blocks, iters);
    }
    return 0;
}
