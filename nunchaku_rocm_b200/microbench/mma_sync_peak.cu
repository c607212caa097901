// Peak rate of the legacy warp-level integer tensor path on the current GPU: mma.sync.m16n8k64.s4 and m16n8k32.s8 with
// operands resident in registers, 8 independent accumulator chains per warp, 16 warps per SM on every SM.  Answers
// whether feeding the int4 codes to mma.sync directly could compete with the tcgen05 kernels.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o mma_sync_peak mma_sync_peak.cu && ./mma_sync_peak
#include <cstdio>
#include <cuda_runtime.h>
template <int MODE>
__global__ void __launch_bounds__(512) k(int iters, int* sink, long long* clocks) {
    int acc[8][4];
    for (int i = 0; i < 8; ++i) for (int j = 0; j < 4; ++j) acc[i][j] = 0;
    unsigned a0 = threadIdx.x * 2654435761u, a1 = a0 ^ 0x9e3779b9u, a2 = a0 + 77u, a3 = a1 + 13u, b0 = a0 * 3u, b1 = a1 * 5u;
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (MODE == 0)
                asm volatile("mma.sync.aligned.m16n8k64.row.col.s32.s4.s4.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+r"(acc[i][0]), "+r"(acc[i][1]), "+r"(acc[i][2]), "+r"(acc[i][3])
                             : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
            else
                asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+r"(acc[i][0]), "+r"(acc[i][1]), "+r"(acc[i][2]), "+r"(acc[i][3])
                             : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
        }
    }
    long long t1 = clock64();
    int s = 0;
    for (int i = 0; i < 8; ++i) for (int j = 0; j < 4; ++j) s += acc[i][j];
    if (s == 0x12345678) sink[0] = s;
    if (threadIdx.x == 0 && blockIdx.x == 0) clocks[0] = t1 - t0;
}
template <int MODE>
void run(const char* name, int kdim) {
    int dev = 0, sms = 0, khz = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
    int* sink; long long* clk;
    cudaMalloc(&sink, 4); cudaMalloc(&clk, 8);
    const int iters = 20000;
    k<MODE><<<sms, 512>>>(100, sink, clk);
    cudaDeviceSynchronize();
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaEventRecord(e0);
    k<MODE><<<sms, 512>>>(iters, sink, clk);
    cudaEventRecord(e1);
    cudaDeviceSynchronize();
    float ms = 0; cudaEventElapsedTime(&ms, e0, e1);
    long long c = 0; cudaMemcpy(&c, clk, 8, cudaMemcpyDeviceToHost);
    const double ops = 2.0 * 16 * 8 * kdim * 8.0 * iters * 16 * sms;  // per warp-instruction 16 x 8 x k MACs
    printf("%s: %.3f ms, %.1f TOPS, %.1f MAC/clk/SM (clock64 %lld for %d iterations), err=%s\n", name, ms, ops / ms / 1e9,
           16.0 * 8 * kdim * 8.0 * iters * 16 / (double)c, c, iters, cudaGetErrorString(cudaGetLastError()));
}
int main() {
    run<0>("mma.sync.m16n8k64.s4", 64);
    run<1>("mma.sync.m16n8k32.s8", 32);
    return 0;
}
