// Measured fp32 FMA throughput of the device: the denominator of the roofline of the CUDA-core (fp32)
// convolution path.  Every thread runs eight independent multiply-add chains from registers; nothing touches
// memory in the timed loop.  Timed with CUDA events on the given stream.
#include "apr_device.cuh"

namespace {

__global__ void __launch_bounds__(256) fma_chain_kernel(float* out, int iters, float a, float b) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (float) (threadIdx.x + i) * 1e-3f;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int r = 0; r < 16; ++r) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = fmaf(v[i], a, b);
        }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += v[i];
    if (s == 123.456f) out[0] = s;          // keeps the chains alive; practically never true
}

} // namespace

// tflops_out[0] = best of `repeats` runs, in TFLOP/s (2 flops per FMA)
extern "C" int aprnet_measure_fp32_fma_tflops(int repeats, double* tflops_out, void* stream) {
    APRNET_ARG_CHECK(tflops_out && repeats > 0 && repeats <= 100, "bad argument");
    cudaStream_t st = (cudaStream_t) stream;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    float* sink = nullptr;
    APRNET_CUDA_CHECK(cudaMalloc((void**) &sink, sizeof(float)));
    cudaEvent_t e0, e1;
    APRNET_CUDA_CHECK(cudaEventCreate(&e0));
    APRNET_CUDA_CHECK(cudaEventCreate(&e1));
    const int iters = 4096, blocks = sms * 8, threads = 256;
    const double flops = 2.0 * 8 * 16 * (double) iters * blocks * threads;
    double best = 0.0;
    for (int r = 0; r <= repeats; ++r) {           // run 0 warms up
        cudaEventRecord(e0, st);
        fma_chain_kernel<<<blocks, threads, 0, st>>>(sink, iters, 1.0000001f, 1e-7f);
        cudaEventRecord(e1, st);
        if (cudaEventSynchronize(e1) != cudaSuccess) break;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (r > 0 && ms > 0.f) best = std::max(best, flops / (ms * 1e-3) / 1e12);
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    cudaFree(sink);
    APRNET_LAUNCH_CHECK();
    *tflops_out = best;
    return APRNET_OK;
}
