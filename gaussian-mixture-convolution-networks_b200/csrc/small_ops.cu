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

// Closed-form eigen-decomposition of symmetric 2x2 / 3x3 matrices, one matrix per thread. Eigenvalues ascending,
// eigenvectors in the columns of the output matrix (torch.linalg.eigh convention).
// 2x2: lambda = T/2 -+ sqrt(|T^2/4 - det|), vectors from the numerically larger of (b, lambda - a) / (lambda - d, b).
// 3x3: trigonometric solution of the characteristic polynomial; the vector of an eigenvalue is the longest column of
// the product of (A - other eigenvalue I) over the two other eigenvalues, the third is the cross product.
// Same formulas and branch rules as the reference's src/gmc/cpp/extensions/math/symeig_detail.h:17-138 (including its
// shortcut "off-diagonal exactly zero -> identity eigenvectors" in 2D).
__device__ __forceinline__ void longest_column_normalised(const float* m, float* v) {
    float best = 0.f;
    int idx = 0;
#pragma unroll
    for (int c = 0; c < 3; ++c) {
        const float len = m[c] * m[c] + m[3 + c] * m[3 + c] + m[6 + c] * m[6 + c];
        if (len > best) { best = len; idx = c; }
    }
    const float inv = 1.f / sqrtf(best);
    v[0] = m[idx] * inv; v[1] = m[3 + idx] * inv; v[2] = m[6 + idx] * inv;
}

template <int D>
__global__ void __launch_bounds__(kThreads) symeig_kernel(const float* __restrict__ in, float* __restrict__ values,
                                                          float* __restrict__ vectors, long long n) {
    const long long i = (long long)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n) return;
    const float* A = in + i * D * D;
    float* val = values + i * D;
    float* vec = vectors + i * D * D;
    if constexpr (D == 2) {
        const float a = A[0], b = A[2], d = A[3];
        const float T = a + d, det = a * d - A[1] * A[2];
        const float f1 = T * 0.5f, f2 = sqrtf(fabsf(T * T * 0.25f - det));
        const float l0 = f1 - f2, l1 = f1 + f2;
        val[0] = l0; val[1] = l1;
        if (b == 0.f) { vec[0] = 1.f; vec[1] = 0.f; vec[2] = 0.f; vec[3] = 1.f; return; }
        float e0x, e0y, e1x, e1y;
        if (a < d) { e0x = b; e0y = l0 - a; e1x = b; e1y = l1 - a; }
        else { e0x = l0 - d; e0y = b; e1x = l1 - d; e1y = b; }
        const float n0 = 1.f / sqrtf(e0x * e0x + e0y * e0y), n1 = 1.f / sqrtf(e1x * e1x + e1y * e1y);
        vec[0] = e0x * n0; vec[1] = e1x * n1; vec[2] = e0y * n0; vec[3] = e1y * n1;
    } else {
        float m[9];
#pragma unroll
        for (int k = 0; k < 9; ++k) m[k] = A[k];
        float eig0, eig1, eig2;   // eig2 <= eig1 <= eig0
        const float p1 = m[1] * m[1] + m[2] * m[2] + m[5] * m[5];
        if (p1 <= 0.0000001f) { eig0 = m[0]; eig1 = m[4]; eig2 = m[8]; }
        else {
            const float q = (m[0] + m[4] + m[8]) / 3.f;
            const float p2 = (m[0] - q) * (m[0] - q) + (m[4] - q) * (m[4] - q) + (m[8] - q) * (m[8] - q) + 2.f * p1;
            const float p = sqrtf(p2 / 6.f);
            float B[9];
#pragma unroll
            for (int k = 0; k < 9; ++k) B[k] = (m[k] - ((k % 4 == 0) ? q : 0.f)) / p;
            const float r = 0.5f * (B[0] * (B[4] * B[8] - B[5] * B[7]) - B[1] * (B[3] * B[8] - B[5] * B[6]) + B[2] * (B[3] * B[7] - B[4] * B[6]));
            const float pi = 3.14159265358979323846f;
            float phi;
            if (r <= -1.f) phi = pi / 3.f;
            else if (r >= 1.f) phi = 0.f;
            else phi = acosf(r) / 3.f;
            eig0 = q + 2.f * p * cosf(phi);
            eig2 = q + 2.f * p * cosf(phi + 2.f * pi / 3.f);
            eig1 = 3.f * q - eig0 - eig2;
        }
        auto shifted_product = [&](float s, float t, float* out) {   // (A - s I)(A - t I)
            float X[9], Y[9];
#pragma unroll
            for (int k = 0; k < 9; ++k) { X[k] = m[k] - ((k % 4 == 0) ? s : 0.f); Y[k] = m[k] - ((k % 4 == 0) ? t : 0.f); }
#pragma unroll
            for (int r2 = 0; r2 < 3; ++r2)
#pragma unroll
                for (int c = 0; c < 3; ++c) out[r2 * 3 + c] = X[r2 * 3] * Y[c] + X[r2 * 3 + 1] * Y[3 + c] + X[r2 * 3 + 2] * Y[6 + c];
        };
        float P[9], v0[3], v1[3], v2[3];
        shifted_product(eig1, eig2, P);
        longest_column_normalised(P, v0);
        shifted_product(eig0, eig2, P);
        longest_column_normalised(P, v1);
        v2[0] = v0[1] * v1[2] - v0[2] * v1[1];
        v2[1] = v0[2] * v1[0] - v0[0] * v1[2];
        v2[2] = v0[0] * v1[1] - v0[1] * v1[0];
        val[0] = eig2; val[1] = eig1; val[2] = eig0;
#pragma unroll
        for (int r2 = 0; r2 < 3; ++r2) { vec[r2 * 3 + 0] = v2[r2]; vec[r2 * 3 + 1] = v1[r2]; vec[r2 * 3 + 2] = v0[r2]; }
    }
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
