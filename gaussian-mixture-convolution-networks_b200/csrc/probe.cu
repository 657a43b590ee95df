// FP32 throughput probe: independent scalar FFMA chains in registers, nothing else. The benchmark times it with CUDA
// events to get the FP32 peak of the GPU it runs on (the denominator of the roofline of the FP32-bound kernels), at
// the clocks of that moment.
#include "common.cuh"

namespace gmc {
namespace {

constexpr int kProbeThreads = 128;
constexpr int kProbeChains = 8;
constexpr int kProbeUnroll = 8;

__global__ void __launch_bounds__(kProbeThreads) fp32_fma_probe_kernel(float* sink, int iterations, float a, float b) {
    float acc[kProbeChains];
#pragma unroll
    for (int i = 0; i < kProbeChains; ++i) acc[i] = float(threadIdx.x) * 0.001f + float(i);
    for (int it = 0; it < iterations; ++it) {
#pragma unroll
        for (int r = 0; r < kProbeUnroll; ++r)
#pragma unroll
            for (int i = 0; i < kProbeChains; ++i) acc[i] = fmaf(acc[i], a, b);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kProbeChains; ++i) s += acc[i];
    if (s == 12345.678f) sink[0] = s;      // never true for the arguments used; keeps the chains alive
}

}  // namespace
}  // namespace gmc

extern "C" int gmc_fp32_fma_probe(float* sink, int iterations, double* flop_out, void* stream) {
    using namespace gmc;
    if (!sink || !flop_out) return GMC_ERR_NULL_POINTER;
    if (iterations <= 0) return GMC_ERR_BAD_DIMS;
    int device = 0, sms = 0;
    GMC_CUDA_TRY(cudaGetDevice(&device));
    GMC_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const int blocks = sms * 8;            // 32 warps per SM
    fp32_fma_probe_kernel<<<blocks, kProbeThreads, 0, as_stream(stream)>>>(sink, iterations, 1.0001f, 0.0001f);
    GMC_LAUNCH_CHECK();
    *flop_out = 2.0 * double(blocks) * kProbeThreads * double(iterations) * kProbeUnroll * kProbeChains;
    return GMC_OK;
}
