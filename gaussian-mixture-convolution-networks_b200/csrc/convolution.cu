// Exact convolution of Gaussian mixtures: every (input component, input channel, kernel component) triple gives one
// output Gaussian (w_d w_k, mu_d + mu_k, C_d + C_k), output index t = comp_in + G * (ch_in + Cin * comp_k).
// Replaces convolution::forward_impl_t / backward_impl_t
// (src/gmc/cpp/extensions/convolution/implementation_forward.h:27-103, implementation_backward.h:27-121).
// Forward is a pure streaming kernel (HBM bound, 4 * V bytes written per product). The backward replaces the
// reference's per-element atomics by two gather kernels whose threads walk contiguous runs of the gradient tensor.
#include "common.cuh"

namespace gmc {
namespace {

constexpr int kTile = 256;   // products per CTA in the forward

template <int D>
__global__ void __launch_bounds__(kTile)
convolution_forward_kernel(const float* __restrict__ data, const float* __restrict__ kernels, float* __restrict__ out,
                           int n_channels_in, int n_components, int n_channels_out, int n_kernel_components,
                           int tiles_per_mixture) {
    constexpr int RF = 1 + D + D * D;
    __shared__ float tile[kTile * RF];
    const int T = n_channels_in * n_components * n_kernel_components;
    const int mix = blockIdx.x / tiles_per_mixture;
    const int t0 = (blockIdx.x - mix * tiles_per_mixture) * kTile;
    const int b = mix / n_channels_out, o = mix - b * n_channels_out;
    const int t = t0 + threadIdx.x;
    if (t < T) {
        const int comp_k = t / (n_components * n_channels_in);
        const int rem = t - comp_k * n_components * n_channels_in;
        const int ch_in = rem / n_components;
        const int comp_in = rem - ch_in * n_components;
        const float* dg = data + ((size_t(b) * n_channels_in + ch_in) * n_components + comp_in) * RF;
        const float* kg = kernels + ((size_t(o) * n_channels_in + ch_in) * n_kernel_components + comp_k) * RF;
        float* dst = tile + threadIdx.x * RF;     // RF is odd: conflict-free
        dst[0] = __ldg(dg) * __ldg(kg);
#pragma unroll
        for (int f = 1; f < RF; ++f) dst[f] = __ldg(dg + f) + __ldg(kg + f);
    }
    __syncthreads();
    const int n_here = min(kTile, T - t0);
    float* dst = out + (size_t(mix) * T + t0) * RF;
    for (int i = threadIdx.x; i < n_here * RF; i += kTile) dst[i] = tile[i];
}

// grad_data[b, ci, g, :] = sum over (o, k) of grad[b, o, t(g, ci, k), :] (weight field times the kernel weight).
// A warp owns 32 consecutive input components of one (b, ci): for fixed (o, k) their gradients are one contiguous run
// of 32 * V floats, which the lanes read with stride 32; lane l accumulates flat positions l, l + 32, ...
template <int D>
__global__ void __launch_bounds__(128)
convolution_backward_data_kernel(const float* __restrict__ grad, const float* __restrict__ kernels,
                                 float* __restrict__ grad_data, int n_batch, int n_channels_in, int n_components,
                                 int n_channels_out, int n_kernel_components) {
    constexpr int RF = 1 + D + D * D;
    const int lane = threadIdx.x & 31;
    const int chunks = (n_components + 31) / 32;
    const long long warp = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (warp >= (long long)n_batch * n_channels_in * chunks) return;
    const int chunk = int(warp % chunks);
    const int ci = int((warp / chunks) % n_channels_in);
    const int b = int(warp / chunks / n_channels_in);
    const int g0 = chunk * 32;
    const int n_floats = min(32, n_components - g0) * RF;
    const size_t T = size_t(n_channels_in) * n_components * n_kernel_components;
    float acc[RF];
    bool is_weight[RF];
#pragma unroll
    for (int i = 0; i < RF; ++i) { acc[i] = 0.f; is_weight[i] = ((lane + 32 * i) % RF) == 0; }
    for (int o = 0; o < n_channels_out; ++o) {
        for (int k = 0; k < n_kernel_components; ++k) {
            const float wk = __ldg(kernels + ((size_t(o) * n_channels_in + ci) * n_kernel_components + k) * RF);
            const float* src = grad + ((size_t(b) * n_channels_out + o) * T +
                                       (size_t(k) * n_channels_in + ci) * n_components + g0) * RF;
#pragma unroll
            for (int i = 0; i < RF; ++i) {
                const int j = lane + 32 * i;
                if (j < n_floats) acc[i] += __ldg(src + j) * (is_weight[i] ? wk : 1.f);
            }
        }
    }
    float* dst = grad_data + ((size_t(b) * n_channels_in + ci) * n_components + g0) * RF;
#pragma unroll
    for (int i = 0; i < RF; ++i) {
        const int j = lane + 32 * i;
        if (j < n_floats) dst[j] = acc[i];
    }
}

// grad_kernels[o, ci, k, :] = sum over (b, g) of grad[b, o, t(g, ci, k), :] (weight field times the data weight).
// One CTA of 32 * V threads per kernel Gaussian; thread j always sees field j % V.
template <int D>
__global__ void convolution_backward_kernels_kernel(const float* __restrict__ grad, const float* __restrict__ data,
                                                    float* __restrict__ grad_kernels, int n_batch, int n_channels_in,
                                                    int n_components, int n_channels_out, int n_kernel_components) {
    constexpr int RF = 1 + D + D * D;
    constexpr int THREADS = 32 * RF;
    __shared__ float red[THREADS];
    const int k = blockIdx.x % n_kernel_components;
    const int ci = (blockIdx.x / n_kernel_components) % n_channels_in;
    const int o = blockIdx.x / n_kernel_components / n_channels_in;
    const int f = threadIdx.x % RF;
    const size_t T = size_t(n_channels_in) * n_components * n_kernel_components;
    const int run = n_components * RF;
    float acc = 0.f;
    for (int b = 0; b < n_batch; ++b) {
        const float* src = grad + ((size_t(b) * n_channels_out + o) * T + (size_t(k) * n_channels_in + ci) * n_components) * RF;
        const float* dw = data + (size_t(b) * n_channels_in + ci) * n_components * RF;
        for (int j = threadIdx.x; j < run; j += THREADS) {
            const float g = __ldg(src + j);
            acc += f == 0 ? g * __ldg(dw + j) : g;     // j is a multiple of V when f == 0: dw[j] is the data weight
        }
    }
    red[threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.x < RF) {
        float s = 0.f;
        for (int i = threadIdx.x; i < THREADS; i += RF) s += red[i];
        grad_kernels[size_t(blockIdx.x) * RF + threadIdx.x] = s;
    }
}

int check_conv_args(int n_batch, int n_channels_in, int n_components, int n_channels_out, int n_kernel_components,
                    int n_dims) {
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_batch <= 0 || n_channels_in <= 0 || n_components <= 0 || n_channels_out <= 0 || n_kernel_components <= 0)
        return GMC_ERR_BAD_DIMS;
    const long long T = (long long)n_channels_in * n_components * n_kernel_components;
    if (T > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    return GMC_OK;
}

}  // namespace
}  // namespace gmc

GMC_DEFINE_TU_CHECK_READER(convolution)

extern "C" int gmc_convolution_forward(const float* data, const float* kernels, float* out, int n_batch,
                                       int n_channels_in, int n_components, int n_channels_out,
                                       int n_kernel_components, int n_dims, void* stream) {
    using namespace gmc;
    if (int s = check_conv_args(n_batch, n_channels_in, n_components, n_channels_out, n_kernel_components, n_dims)) return s;
    if (!data || !kernels || !out) return GMC_ERR_NULL_POINTER;
    const long long T = (long long)n_channels_in * n_components * n_kernel_components;
    const long long tiles = (T + kTile - 1) / kTile;
    const long long blocks = tiles * n_batch * n_channels_out;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    if (n_dims == 2)
        convolution_forward_kernel<2><<<unsigned(blocks), kTile, 0, as_stream(stream)>>>(
            data, kernels, out, n_channels_in, n_components, n_channels_out, n_kernel_components, int(tiles));
    else
        convolution_forward_kernel<3><<<unsigned(blocks), kTile, 0, as_stream(stream)>>>(
            data, kernels, out, n_channels_in, n_components, n_channels_out, n_kernel_components, int(tiles));
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

extern "C" int gmc_convolution_backward(const float* grad, const float* data, const float* kernels, float* grad_data,
                                        float* grad_kernels, int n_batch, int n_channels_in, int n_components,
                                        int n_channels_out, int n_kernel_components, int n_dims, void* stream) {
    using namespace gmc;
    if (int s = check_conv_args(n_batch, n_channels_in, n_components, n_channels_out, n_kernel_components, n_dims)) return s;
    if (!grad || !data || !kernels) return GMC_ERR_NULL_POINTER;
    cudaStream_t st = as_stream(stream);
    if (grad_data) {
        const long long warps = (long long)n_batch * n_channels_in * ((n_components + 31) / 32);
        const long long blocks = (warps + 3) / 4;
        if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
        if (n_dims == 2)
            convolution_backward_data_kernel<2><<<unsigned(blocks), 128, 0, st>>>(grad, kernels, grad_data, n_batch, n_channels_in, n_components, n_channels_out, n_kernel_components);
        else
            convolution_backward_data_kernel<3><<<unsigned(blocks), 128, 0, st>>>(grad, kernels, grad_data, n_batch, n_channels_in, n_components, n_channels_out, n_kernel_components);
        GMC_LAUNCH_CHECK();
    }
    if (grad_kernels) {
        const long long blocks = (long long)n_channels_out * n_channels_in * n_kernel_components;
        if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
        if (n_dims == 2)
            convolution_backward_kernels_kernel<2><<<unsigned(blocks), 32 * 7, 0, st>>>(grad, data, grad_kernels, n_batch, n_channels_in, n_components, n_channels_out, n_kernel_components);
        else
            convolution_backward_kernels_kernel<3><<<unsigned(blocks), 32 * 13, 0, st>>>(grad, data, grad_kernels, n_batch, n_channels_in, n_components, n_channels_out, n_kernel_components);
        GMC_LAUNCH_CHECK();
    }
    return GMC_OK;
}
