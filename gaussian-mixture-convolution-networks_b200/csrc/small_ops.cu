// Small per-element operators: batched 2x2 / 3x3 matrix inverse and the mixture integral.
// Both are streaming kernels bounded by HBM bandwidth.
#include "common.cuh"
#include "symeig_device.cuh"

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

// Gradient of the inverse: out = -inv * grad * inv per matrix (the reference's formula, transposes dropped), one matrix
// per thread, through shared memory like the forward.
template <int D>
__global__ void __launch_bounds__(kThreads) matrix_inverse_backward_kernel(const float* __restrict__ inverses,
                                                                           const float* __restrict__ grad,
                                                                           float* __restrict__ out, long long n) {
    constexpr int E = D * D;
    __shared__ float tile_inv[kThreads * E];
    __shared__ float tile_grad[kThreads * E];
    const long long first = (long long)blockIdx.x * kThreads;
    const int here = int(min((long long)kThreads, n - first));
    for (int i = threadIdx.x; i < here * E; i += kThreads) {
        tile_inv[i] = __ldg(inverses + first * E + i);
        tile_grad[i] = __ldg(grad + first * E + i);
    }
    __syncthreads();
    if (threadIdx.x < here) {
        const float* a = tile_inv + threadIdx.x * E;
        float* g = tile_grad + threadIdx.x * E;
        float ag[E], r[E];
#pragma unroll
        for (int i = 0; i < D; ++i)
#pragma unroll
            for (int j = 0; j < D; ++j) {
                float acc = 0.f;
#pragma unroll
                for (int k = 0; k < D; ++k) acc += a[i * D + k] * g[k * D + j];
                ag[i * D + j] = acc;
            }
#pragma unroll
        for (int i = 0; i < D; ++i)
#pragma unroll
            for (int j = 0; j < D; ++j) {
                float acc = 0.f;
#pragma unroll
                for (int k = 0; k < D; ++k) acc += ag[i * D + k] * a[k * D + j];
                r[i * D + j] = -acc;
            }
#pragma unroll
        for (int e = 0; e < E; ++e) g[e] = r[e];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < here * E; i += kThreads) out[first * E + i] = tile_grad[i];
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

// One warp per mixture: scale = mean trace of the matrix slot / D; writes 1 / sqrt(scale) and sqrt(scale).
__global__ void __launch_bounds__(kThreads) trace_scale_kernel(const float* __restrict__ mixture, float* __restrict__ forth,
                                                               float* __restrict__ back, long long n_mixtures,
                                                               int n_components, int n_dims) {
    const long long warp = ((long long)blockIdx.x * kThreads + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n_mixtures) return;
    const int record = 1 + n_dims + n_dims * n_dims;
    const float* m = mixture + warp * (long long)n_components * record + 1 + n_dims;
    float s = 0.f;
    for (int g = lane; g < n_components; g += 32) {
        float t = 0.f;
        for (int d = 0; d < n_dims; ++d) t += __ldg(m + (size_t)g * record + d * n_dims + d);
        s += t;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
        const float scale = s / float(n_components) / float(n_dims);
        const float root = sqrtf(scale);
        back[warp] = root;
        forth[warp] = 1.f / root;
    }
}

// Positions times f, matrices times f * f, weights unchanged; f per mixture. One thread per float of the output.
__global__ void __launch_bounds__(kThreads) spatial_scale_kernel(const float* __restrict__ mixture,
                                                                 const float* __restrict__ factors, float* __restrict__ out,
                                                                 long long n_floats, int n_components, int n_dims) {
    const long long i = (long long)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n_floats) return;
    const int record = 1 + n_dims + n_dims * n_dims;
    const long long gaussian = i / record;
    const int field = int(i - gaussian * record);
    const float f = __ldg(factors + gaussian / n_components);
    const float v = __ldg(mixture + i);
    out[i] = field == 0 ? v : (field <= n_dims ? v * f : (f * f) * v);
}


// ---------------------------------------------------------------------------------------------------------------
// Input normalisation of a one-channel mixture per sample, the two per-sample normalisations the network applies to its
// input in one kernel (the reference's CovScaleNorm(batch_norm=False) followed by BatchNorm(batch_norm=False),
// src/gmc/modules.py:313-351 and 354-420):
//   f  = sqrt(D / mean_g trace(C_g));  positions *= f, covariances *= f * f
//   values of the scaled mixture at n_samples uniform points of the box of its centres (2D: the box widened by 15 %),
//   weights *= scaling / max(sd, 0.001) with the unbiased standard deviation sd of those values, constant = -mean.
// One CTA per sample. The uniform numbers come from `uniforms` ([n_batch, n_samples, D], for tests) or from a
// counter-based hash of *seed (drawn by the caller from its own generator, so a seeded run repeats).
// ---------------------------------------------------------------------------------------------------------------
constexpr int kNormThreads = 256;

__device__ __forceinline__ float uniform_from_counter(unsigned long long seed, unsigned long long counter) {
    unsigned long long z = seed + (counter + 1ull) * 0x9E3779B97F4A7C15ull;      // splitmix64
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return float(unsigned(z >> 40)) * (1.0f / 16777216.0f);                       // 24 bits -> [0, 1)
}

template <int D>
__global__ void __launch_bounds__(kNormThreads)
input_normalise_kernel(const float* __restrict__ mixture, const long long* __restrict__ seed, const float* __restrict__ uniforms,
                       const float* __restrict__ scaling, int n_components, int n_samples, float* __restrict__ out,
                       float* __restrict__ out_constants) {
    constexpr int RF = 1 + D + D * D;
    constexpr int RD = D + D * D + 1;                  // centre, inverse covariance, weight * norm
    extern __shared__ __align__(16) float smem[];
    float* ready = smem;                               // [G][RD]
    float* values = smem + size_t(n_components) * RD;  // [n_samples]
    __shared__ float red[kNormThreads / 32][2 * D + 1];
    __shared__ float s_f, s_lo[D], s_hi[D], s_mean, s_factor;
    const int G = n_components;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* src = mixture + size_t(blockIdx.x) * G * RF;

    // ---- mean trace, box of the centres ----
    float tr = 0.f, lo[D], hi[D];
#pragma unroll
    for (int d = 0; d < D; ++d) { lo[d] = INFINITY; hi[d] = -INFINITY; }
    for (int g = tid; g < G; g += kNormThreads) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            tr += __ldg(src + size_t(g) * RF + 1 + D + d * D + d);
            const float p = __ldg(src + size_t(g) * RF + 1 + d);
            lo[d] = fminf(lo[d], p);
            hi[d] = fmaxf(hi[d], p);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        tr += __shfl_xor_sync(0xffffffffu, tr, o);
#pragma unroll
        for (int d = 0; d < D; ++d) {
            lo[d] = fminf(lo[d], __shfl_xor_sync(0xffffffffu, lo[d], o));
            hi[d] = fmaxf(hi[d], __shfl_xor_sync(0xffffffffu, hi[d], o));
        }
    }
    if (lane == 0) {
        red[warp][0] = tr;
#pragma unroll
        for (int d = 0; d < D; ++d) { red[warp][1 + d] = lo[d]; red[warp][1 + D + d] = hi[d]; }
    }
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (int w = 0; w < kNormThreads / 32; ++w) t += red[w][0];
        const float f = sqrtf(float(D) / (t / float(G)));
        s_f = f;
#pragma unroll
        for (int d = 0; d < D; ++d) {
            float l = red[0][1 + d], h = red[0][1 + D + d];
            for (int w = 1; w < kNormThreads / 32; ++w) { l = fminf(l, red[w][1 + d]); h = fmaxf(h, red[w][1 + D + d]); }
            // the box of the SCALED centres, with the ordering a negative-free factor keeps
            s_lo[d] = l * f;
            s_hi[d] = h * f;
        }
    }
    __syncthreads();
    const float f = s_f;

    // ---- scaled Gaussians in evaluation form ----
    for (int g = tid; g < G; g += kNormThreads) {
        float C[D * D], inv[D * D];
#pragma unroll
        for (int k = 0; k < D * D; ++k) C[k] = (f * f) * __ldg(src + size_t(g) * RF + 1 + D + k);
        float det;
        if constexpr (D == 2) {
            det = C[0] * C[3] - C[1] * C[2];
            const float r = 1.f / det;
            inv[0] = C[3] * r; inv[1] = -C[1] * r; inv[2] = -C[2] * r; inv[3] = C[0] * r;
        } else {
            const float c0 = C[4] * C[8] - C[5] * C[7], c1 = C[3] * C[8] - C[5] * C[6], c2 = C[3] * C[7] - C[4] * C[6];
            det = C[0] * c0 - C[1] * c1 + C[2] * c2;
            const float r = 1.f / det;
            inv[0] = c0 * r; inv[1] = -(C[1] * C[8] - C[2] * C[7]) * r; inv[2] = (C[1] * C[5] - C[2] * C[4]) * r;
            inv[3] = -c1 * r; inv[4] = (C[0] * C[8] - C[2] * C[6]) * r; inv[5] = -(C[0] * C[5] - C[2] * C[3]) * r;
            inv[6] = c2 * r; inv[7] = -(C[0] * C[7] - C[1] * C[6]) * r; inv[8] = (C[0] * C[4] - C[1] * C[3]) * r;
        }
        float* r = ready + size_t(g) * RD;
#pragma unroll
        for (int d = 0; d < D; ++d) r[d] = f * __ldg(src + size_t(g) * RF + 1 + d);
#pragma unroll
        for (int k = 0; k < D * D; ++k) r[D + k] = inv[k];
        // weight * (2 pi)^(-D/2) / sqrt(det C)
        r[D + D * D] = __ldg(src + size_t(g) * RF) * (D == 2 ? 0.15915494309189535f : 0.06349363593424097f) * rsqrtf(det);
    }
    __syncthreads();

    // ---- values at the sample points ----
    const unsigned long long sd_bits = seed != nullptr ? (unsigned long long)(*seed) : 0ull;
    float sum = 0.f;
    for (int i = tid; i < n_samples; i += kNormThreads) {
        float x[D];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            float u = uniforms != nullptr ? __ldg(uniforms + (size_t(blockIdx.x) * n_samples + i) * D + d)
                                          : uniform_from_counter(sd_bits, (size_t(blockIdx.x) * n_samples + i) * D + d);
            if constexpr (D == 2) u = u * 1.3f - 0.15f;
            x[d] = u * (s_hi[d] - s_lo[d]) + s_lo[d];
        }
        float v = 0.f;
        for (int g = 0; g < G; ++g) {
            const float* r = ready + size_t(g) * RD;
            float t[D];
#pragma unroll
            for (int d = 0; d < D; ++d) t[d] = x[d] - r[d];
            float q = 0.f;
#pragma unroll
            for (int a = 0; a < D; ++a) {
                float acc = 0.f;
#pragma unroll
                for (int c = 0; c < D; ++c) acc = fmaf(r[D + a * D + c], t[c], acc);
                q = fmaf(t[a], acc, q);
            }
            v = fmaf(r[D + D * D], __expf(-0.5f * q), v);
        }
        values[i] = v;
        sum += v;
    }
    // ---- mean and unbiased standard deviation (two passes over the stored values) ----
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncthreads();
    if (lane == 0) red[warp][0] = sum;
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (int w = 0; w < kNormThreads / 32; ++w) t += red[w][0];
        s_mean = t / float(n_samples);
    }
    __syncthreads();
    const float mean = s_mean;
    float sq = 0.f;
    for (int i = tid; i < n_samples; i += kNormThreads) { const float dv = values[i] - mean; sq = fmaf(dv, dv, sq); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    __syncthreads();
    if (lane == 0) red[warp][0] = sq;
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (int w = 0; w < kNormThreads / 32; ++w) t += red[w][0];
        const float sd = sqrtf(t / float(n_samples - 1));
        s_factor = (scaling != nullptr ? __ldg(scaling) : 1.f) / fmaxf(sd, 0.001f);
        out_constants[blockIdx.x] = -mean;
    }
    __syncthreads();
    const float wf = s_factor;
    float* dst = out + size_t(blockIdx.x) * G * RF;
    for (int i = tid; i < G * RF; i += kNormThreads) {
        const int field = i % RF;
        const float v = __ldg(src + i);
        dst[i] = field == 0 ? v * wf : (field <= D ? v * f : (f * f) * v);
    }
}

// One matrix per thread; the decomposition itself is symeig_device (symeig_device.cuh).
template <int D>
__global__ void __launch_bounds__(kThreads) symeig_kernel(const float* __restrict__ in, float* __restrict__ values,
                                                          float* __restrict__ vectors, long long n) {
    const long long i = (long long)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n) return;
    symeig_device<D>(in + i * D * D, values + i * D, vectors + i * D * D);
}

}  // namespace
}  // namespace gmc

namespace gmc {
namespace {
#ifdef GMC_BOUNDS_CHECK
__global__ void index_check_probe_kernel(const float* one, long long index, long long n, float* out) {
    *out = one[GMC_IDX(index, n)];      // an index outside [0, n) is reported and replaced by 0
}
#endif
}  // namespace
}  // namespace gmc

GMC_DEFINE_TU_CHECK_READER(small_ops)

extern "C" int gmc_symeig(const float* matrices, float* eigenvalues, float* eigenvectors, long long n_matrices,
                          int n_dims, void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_matrices < 0) return GMC_ERR_BAD_DIMS;
    if (n_matrices == 0) return GMC_OK;
    if (!matrices || !eigenvalues || !eigenvectors) return GMC_ERR_NULL_POINTER;
    const long long blocks = (n_matrices + kThreads - 1) / kThreads;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    if (n_dims == 2) symeig_kernel<2><<<unsigned(blocks), kThreads, 0, as_stream(stream)>>>(matrices, eigenvalues, eigenvectors, n_matrices);
    else symeig_kernel<3><<<unsigned(blocks), kThreads, 0, as_stream(stream)>>>(matrices, eigenvalues, eigenvectors, n_matrices);
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

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

extern "C" int gmc_matrix_inverse_backward(const float* inverses, const float* grad, float* grad_matrices,
                                           long long n_matrices, int n_dims, void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_matrices < 0) return GMC_ERR_BAD_DIMS;
    if (n_matrices == 0) return GMC_OK;
    if (!inverses || !grad || !grad_matrices) return GMC_ERR_NULL_POINTER;
    const long long blocks = (n_matrices + kThreads - 1) / kThreads;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    if (n_dims == 2)
        matrix_inverse_backward_kernel<2><<<unsigned(blocks), kThreads, 0, as_stream(stream)>>>(inverses, grad, grad_matrices, n_matrices);
    else
        matrix_inverse_backward_kernel<3><<<unsigned(blocks), kThreads, 0, as_stream(stream)>>>(inverses, grad, grad_matrices, n_matrices);
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

extern "C" int gmc_trace_scale(const float* mixture, float* forth, float* back, long long n_mixtures, int n_components,
                               int n_dims, void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_mixtures < 0 || n_components <= 0) return GMC_ERR_BAD_DIMS;
    if (n_mixtures == 0) return GMC_OK;
    if (!mixture || !forth || !back) return GMC_ERR_NULL_POINTER;
    const long long blocks = (n_mixtures * 32 + kThreads - 1) / kThreads;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    trace_scale_kernel<<<unsigned(blocks), kThreads, 0, as_stream(stream)>>>(mixture, forth, back, n_mixtures, n_components, n_dims);
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

extern "C" int gmc_spatial_scale(const float* mixture, const float* factors, float* out, long long n_mixtures,
                                 int n_components, int n_dims, void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_mixtures < 0 || n_components <= 0) return GMC_ERR_BAD_DIMS;
    if (n_mixtures == 0) return GMC_OK;
    if (!mixture || !factors || !out) return GMC_ERR_NULL_POINTER;
    const long long n_floats = n_mixtures * n_components * (1 + n_dims + n_dims * n_dims);
    const long long blocks = (n_floats + kThreads - 1) / kThreads;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    spatial_scale_kernel<<<unsigned(blocks), kThreads, 0, as_stream(stream)>>>(mixture, factors, out, n_floats, n_components, n_dims);
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

extern "C" int gmc_input_normalise(const float* mixture, const long long* seed, const float* uniforms, const float* scaling,
                                   long long n_batch, int n_components, int n_dims, int n_samples, float* out_mixture,
                                   float* out_constants, void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_batch < 0 || n_components <= 0 || n_samples < 2) return GMC_ERR_BAD_DIMS;
    if (n_batch == 0) return GMC_OK;
    if (n_batch > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    if (!mixture || !out_mixture || !out_constants || (!seed && !uniforms)) return GMC_ERR_NULL_POINTER;
    const size_t smem = sizeof(float) * (size_t(n_components) * (n_dims + n_dims * n_dims + 1) + size_t(n_samples));
    if (smem > 200 * 1024) return GMC_ERR_BAD_DIMS;
    cudaStream_t st = as_stream(stream);
    if (n_dims == 2) {
        if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(input_normalise_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        input_normalise_kernel<2><<<unsigned(n_batch), kNormThreads, smem, st>>>(mixture, seed, uniforms, scaling, n_components, n_samples, out_mixture, out_constants);
    } else {
        if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(input_normalise_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        input_normalise_kernel<3><<<unsigned(n_batch), kNormThreads, smem, st>>>(mixture, seed, uniforms, scaling, n_components, n_samples, out_mixture, out_constants);
    }
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

extern "C" int gmc_debug_index_check(const float* one_float, float* out, long long index, long long n, void* stream) {
    using namespace gmc;
    if (!one_float || !out) return GMC_ERR_NULL_POINTER;
#ifdef GMC_BOUNDS_CHECK
    if (index < 0 || n <= 0) return GMC_ERR_BAD_DIMS;
    if (index < n && index != 0) return GMC_ERR_BAD_DIMS;   // the buffer holds one float: in-range means index 0
    index_check_probe_kernel<<<1, 1, 0, as_stream(stream)>>>(one_float, index, n, out);
    GMC_LAUNCH_CHECK();
    return GMC_OK;
#else
    (void)index; (void)n; (void)stream;
    return GMC_ERR_UNSUPPORTED;                              // this build carries no index checks
#endif
}
