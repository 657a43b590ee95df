// Benchmark helper, not part of the product library: FP32 throughput probe (independent scalar FFMA chains in
// registers, nothing else). bench.py builds this file into bench_probe.so, times the launch with CUDA events and uses the
// result as the FP32 peak of the GPU it runs on (the denominator of the roofline of the FP32-bound kernels), at the
// clocks of that moment.
#include <cuda_runtime.h>

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

// Returns 0 and the flop count of the launch in *flop_out; non-zero on a bad argument or a CUDA error.
extern "C" int gmc_bench_fp32_fma_probe(float* sink, int iterations, double* flop_out, void* stream) {
    if (!sink || !flop_out || iterations <= 0) return 1;
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 2;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 2;
    const int blocks = sms * 8;            // 32 warps per SM
    fp32_fma_probe_kernel<<<blocks, kProbeThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(sink, iterations, 1.0001f,
                                                                                                0.0001f);
    if (cudaGetLastError() != cudaSuccess) return 2;
    *flop_out = 2.0 * double(blocks) * kProbeThreads * double(iterations) * kProbeUnroll * kProbeChains;
    return 0;
}
