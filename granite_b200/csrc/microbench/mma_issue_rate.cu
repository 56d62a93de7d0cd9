// Micro-benchmark: how fast can tcgen05.mma instructions be issued and retired on one SM?
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_issue_rate mma_issue_rate.cu
//   ./mma_issue_rate
//
// One CTA per SM; one or two threads (in different warps) issue a stream of 128xNx16 fp16 MMAs
// with both operands in shared memory (SS) or A in TMEM (TS), accumulating into TMEM, and the
// clocks per instruction are printed.  It is the evidence behind two design choices of fa_tc.cu:
// N = 128 instructions cost ~93-118 clocks when a single thread issues them (about 64 would be the
// nominal math time), and a second issuing thread brings the pair to ~70-87 clocks per MMA.
#include <cstdio>
#include <cuda_runtime.h>
#include "../ptx.cuh"
using namespace gb200;
__global__ void __launch_bounds__(128,1) k(int mode, int iters, long long* out) {
    extern __shared__ uint8_t raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t bar, bar2; __shared__ uint32_t tbase; __shared__ int abortf;
    for (int i = threadIdx.x; i < 160*1024/4; i += 128) ((uint32_t*)smem)[i] = 0;
    if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_init(&bar2, 1); abortf = 0; mbar_fence_init(); }
    if (threadIdx.x < 32) { tmem_alloc(&tbase, 512); tmem_relinquish(); }
    fence_proxy_async_smem();
    tc_fence_before_sync(); __syncthreads(); tc_fence_after_sync();
    uint32_t tm = tbase;
    if (threadIdx.x == 0 || ((mode & 8) && threadIdx.x == 32)) {
        const int who = threadIdx.x >> 5;
        int N = (mode & 1) ? 256 : 128;
        bool ts = mode & 2;
        uint32_t idesc = umma_idesc_f16(128, N, false, ts ? true : false);
        uint32_t a_lo = desc_lo(smem_u32(smem), 16), b_lo = desc_lo(smem_u32(smem) + 32768, ts ? 16384 : 16);
        long long t0 = clock64();
        for (int i = 0; i < iters; i++) {
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                const uint32_t dd = (mode & 8) ? tm + who * 256 : ((mode & 4) ? tm + (ks & 1) * 128 : tm);
                if (ts) umma_ts_words(dd, tm + 128 + ks * 8, b_lo + ks * 128, kDescHiSw128, idesc, 1u);
                else umma_ss_words(dd, a_lo + (ks&3)*2 + (ks>>2)*1024, b_lo + (ks&3)*2 + (ks>>2)*1024, kDescHiSw128, idesc, 1u);
            }
        }
        tc_commit(who ? &bar2 : &bar);
        mbar_wait(who ? &bar2 : &bar, 0, &abortf);
        long long t1 = clock64();
        if (!who) out[blockIdx.x] = t1 - t0;
    }
    tc_fence_before_sync(); __syncthreads();
    if (threadIdx.x < 32) { tc_fence_after_sync(); tmem_dealloc(tm, 512); }
}
int main() {
    long long* out; cudaMallocManaged(&out, 148 * 8);
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const char* names[4] = {"SS N=128", "SS N=256", "TS N=128", "TS N=256"};
    for (int grid : {148}) for (int mode : {0, 2, 8, 10, 1, 3, 9, 11}) {
        int iters = 200;
        k<<<grid, 128, 200 * 1024>>>(mode, iters, out);
        cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { printf("err %s\n", cudaGetErrorString(e)); return 1; }
        double clk = (double)out[0] / (iters * 8);
        int N = (mode & 1) ? 256 : 128;
        printf("grid %3d issuers=%d %s: %.1f clk per MMA (128x%dx16) -> %.0f flop/clk/SM\n", grid, 1 + ((mode>>3)&1), names[mode&3], clk, N, 2.0 * 128 * N * 16 / clk);
    }
    return 0;
}
