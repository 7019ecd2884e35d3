// Measures the 32-bit logic-op (LOP3) issue rate of the device: the denominator of the
// integer-pipe roofline the SC accumulation kernel is reported against.
#include "sc_common.h"

namespace geo {

constexpr int kChains = 16;
constexpr int kUnroll = 8;

__global__ void __launch_bounds__(256) lop3_peak_kernel(uint32_t *sink, int iters, uint32_t seed) {
    uint32_t x[kChains];
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
#pragma unroll
    for (int i = 0; i < kChains; i++) x[i] = tid * 2654435761u + i * 40503u + seed;
    const uint32_t b = tid | 0x0f0f0f0fu, c = seed ^ 0x33333333u;
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
#pragma unroll
            for (int i = 0; i < kChains; i++)
                asm volatile("lop3.b32 %0, %0, %1, %2, 0x6A;" : "+r"(x[i]) : "r"(b), "r"(c));  // x ^ (b & c)
        }
    }
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < kChains; i++) r ^= x[i];
    if (r == 0x12345678u) sink[0] = r;  // practically never true; keeps the chains alive
}

}  // namespace geo

extern "C" int geo_sc_measure_lop3_peak(double *lop3_per_second, double *milliseconds) {
    using namespace geo;
    if (!lop3_per_second) return fail(GEO_SC_ERR_NULL, "lop3_per_second is NULL");
    int dev = 0, sms = 0;
    GEO_CUDA_CHECK(cudaGetDevice(&dev));
    GEO_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    uint32_t *sink = nullptr;
    GEO_CUDA_CHECK(cudaMalloc(&sink, 256));
    cudaEvent_t e0, e1;
    GEO_CUDA_CHECK(cudaEventCreate(&e0));
    GEO_CUDA_CHECK(cudaEventCreate(&e1));
    const int blocks = sms * 8, threads = 256, iters = 4096;
    float best = 1e30f;
    for (int rep = 0; rep < 5; rep++) {
        cudaEventRecord(e0);
        lop3_peak_kernel<<<blocks, threads>>>(sink, iters, (uint32_t)rep);
        cudaEventRecord(e1);
        cudaError_t e = cudaEventSynchronize(e1);
        if (e != cudaSuccess) {
            cudaFree(sink);
            return fail(GEO_SC_ERR_CUDA, "lop3 peak kernel: %s", cudaGetErrorString(e));
        }
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        if (rep > 0 && ms < best) best = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(sink);
    const double ops = (double)blocks * threads * (double)iters * kChains * kUnroll;
    *lop3_per_second = ops / (best * 1e-3);
    if (milliseconds) *milliseconds = best;
    return GEO_SC_OK;
}
