// Small per-element operators: batched 2x2 / 3x3 matrix inverse and the mixture integral.
// Both are streaming kernels bounded by HBM bandwidth.
#include "common.cuh"

namespace gmc {
namespace {

constexpr int kThreads = 256;

// One matrix per thread. A CTA first moves its kThreads * D * D contiguous floats through shared memory
// with coalesced accesses, so global traffic is full-width although each thread owns 4 or 9 floats.
template <int D>
__global__ void __launch_bounds__(kThreads) matrix_inverse_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                  long long n) {
    constexpr int E = D * D;
    __shared__ float tile[kThreads * E];
    const long long first = (long long)blockIdx.x * kThreads;
    const int here = int(min((long long)kThreads, n - first));
    const float* src = in + first * E;
    float* dst = out + first * E;
    for (int i = threadIdx.x; i < here * E; i += kThreads) tile[i] = __ldg(src + i);
    __syncthreads();
    if (threadIdx.x < here) {
        float* m = tile + threadIdx.x * E;   // stride 4 or 9 floats: 9 is conflict free, 4 is 4-way (tiny kernel)
        if constexpr (D == 2) {
            const float a = m[0], b = m[1], c = m[2], d = m[3];
            const float r = 1.f / (a * d - b * c);
            m[0] = d * r; m[1] = -b * r; m[2] = -c * r; m[3] = a * r;
        } else {
            const float a = m[0], b = m[1], c = m[2], d = m[3], e = m[4], f = m[5], g = m[6], h = m[7], k = m[8];
            const float A = e * k - f * h, B = -(d * k - f * g), C = d * h - e * g;
            const float r = 1.f / (a * A + b * B + c * C);
            m[0] = A * r; m[1] = -(b * k - c * h) * r; m[2] = (b * f - c * e) * r;
            m[3] = B * r; m[4] = (a * k - c * g) * r;  m[5] = -(a * f - c * d) * r;
            m[6] = C * r; m[7] = -(a * h - b * g) * r; m[8] = (a * e - b * d) * r;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < here * E; i += kThreads) dst[i] = tile[i];
}

// One warp per mixture: sum of the weight column.
__global__ void __launch_bounds__(kThreads) integrate_kernel(const float* __restrict__ mixture, float* __restrict__ out,
                                                             long long n_mixtures, int n_components, int record) {
    const long long warp = ((long long)blockIdx.x * kThreads + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n_mixtures) return;
    const float* m = mixture + warp * (long long)n_components * record;
    float s = 0.f;
    for (int g = lane; g < n_components; g += 32) s += __ldg(m + (size_t)g * record);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[warp] = s;
}

}  // namespace
}  // namespace gmc

GMC_DEFINE_TU_CHECK_READER(small_ops)

extern "C" int gmc_matrix_inverse(const float* matrices, float* inverses, long long n_matrices, int n_dims,
                                  void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_matrices < 0) return GMC_ERR_BAD_DIMS;
    if (n_matrices == 0) return GMC_OK;
    if (!matrices || !inverses) return GMC_ERR_NULL_POINTER;
    const long long blocks = (n_matrices + kThreads - 1) / kThreads;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    if (n_dims == 2) matrix_inverse_kernel<2><<<unsigned(blocks), kThreads, 0, as_stream(stream)>>>(matrices, inverses, n_matrices);
    else matrix_inverse_kernel<3><<<unsigned(blocks), kThreads, 0, as_stream(stream)>>>(matrices, inverses, n_matrices);
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

extern "C" int gmc_integrate(const float* mixture, float* integrals, long long n_mixtures, int n_components,
                             int n_dims, void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_mixtures < 0 || n_components <= 0) return GMC_ERR_BAD_DIMS;
    if (n_mixtures == 0) return GMC_OK;
    if (!mixture || !integrals) return GMC_ERR_NULL_POINTER;
    const long long blocks = (n_mixtures * 32 + kThreads - 1) / kThreads;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    integrate_kernel<<<unsigned(blocks), kThreads, 0, as_stream(stream)>>>(mixture, integrals, n_mixtures, n_components,
                                                                          1 + n_dims + n_dims * n_dims);
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}
