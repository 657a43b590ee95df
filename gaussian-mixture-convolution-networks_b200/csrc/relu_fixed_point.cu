// ReLU approximation of a mixture by one fixed-point step, fused into one kernel (inference path).
//
// For a mixture (w_j, mu_j, C_j) with constant c the reference (src/gmc/fitting.py:279-312 with n_iter = 1) computes
//   initial weights  w'_j = w_j                 if w_j + c > 0
//                          -max(c, 0)           otherwise
//   start            x0_j = |w'_j| + 0.1
//   target           b_i  = max(sum_j w_j  E_ij + c, 0) - max(c, 0)
//   step             x_i  = x0_i (b_i + 0.05) / (sum_j x0_j E_ij + 0.05)
// with E_ij = (2 pi)^(-D/2) sqrt(det S_j) exp(-1/2 (mu_i - mu_j)^T S_j (mu_i - mu_j)), S_j = C_j^-1: both mixtures are
// evaluated at the component centres and share centres and covariances, so one exponential per (i, j) serves both
// sums, and the inverse covariances never leave the chip. Output: (x, mu, C) and the constant max(c, 0).
//
// Layout of the work: thread = one centre i of one mixture; the Gaussians of a mixture are staged in shared memory in
// "ready" form (negated centre, A = -1/2 log2(e) sym(S), norm, w, x0) in chunks of kChunk. A CTA of 128 threads serves
// 128 / G whole mixtures when G <= 128 and one mixture otherwise.
#include "common.cuh"

namespace gmc {
namespace {

constexpr int kThreads = 128;
constexpr int kChunk = 1024;
constexpr float kExpScale = -0.5f * kLog2e;

// Optional transforms of the layer the fit sits in, applied on load / on store (none: {1.f, nullptr, 1}):
//   input weights are divided by weight_divisor (the network divides a convolution's output by its input channels);
//   output centres are multiplied by f and output covariances by f * f, f = spatial_scale[mixture % n_channels]
//   (the covariance-scale normalisation that follows the fit in evaluation mode).
struct LayerTransform {
    float weight_divisor;
    const float* spatial_scale;
    int n_channels;
};

template <int D>
__device__ __forceinline__ void store_geometry(float* dst, const float* __restrict__ src, float f) {
    constexpr int RF = 1 + D + D * D;
    const float ff = f * f;
#pragma unroll
    for (int k = 1; k <= D; ++k) dst[k] = __ldg(src + k) * f;
#pragma unroll
    for (int k = 1 + D; k < RF; ++k) dst[k] = ff * __ldg(src + k);
}

template <int D>
struct Ready {
    static constexpr int kFloats = D + D * (D + 1) / 2 + 3;    // -mu | A | norm, w, x0: 8 (2D) or 12 (3D) floats
};

// Floats between the staged mixtures of one CTA: a multiple of 4 (float4 reads) whose quarter is odd, so that the
// records read by the mixtures of one warp fall into different banks.
__host__ __device__ inline int stage_stride_floats(int floats) {
    int quads = (floats + 3) / 4;
    if ((quads & 1) == 0) ++quads;
    return quads * 4;
}

template <int D>
__device__ __forceinline__ void make_ready(const float* r, float constant, float relu_constant, float weight_divisor,
                                           float* out) {
    constexpr int NS = D * (D + 1) / 2;
    const float w = r[0] / weight_divisor;
#pragma unroll
    for (int d = 0; d < D; ++d) out[d] = -r[1 + d];
    const float* C = r + 1 + D;
    float det;
    if constexpr (D == 2) {
        det = C[0] * C[3] - C[1] * C[2];
        const float inv = 1.f / det;
        out[D + 0] = kExpScale * C[3] * inv;
        out[D + 1] = kExpScale * -0.5f * (C[1] + C[2]) * inv;
        out[D + 2] = kExpScale * C[0] * inv;
    } else {
        const float a = C[0], b = C[1], c = C[2], d = C[3], e = C[4], f = C[5], g = C[6], h = C[7], k = C[8];
        const float A = e * k - f * h, B = -(d * k - f * g), Cc = d * h - e * g;
        det = a * A + b * B + c * Cc;
        const float inv = 1.f / det;
        const float s01 = -(b * k - c * h) * inv, s02 = (b * f - c * e) * inv, s10 = B * inv, s12 = -(a * f - c * d) * inv;
        const float s20 = Cc * inv, s21 = -(a * h - b * g) * inv;
        out[D + 0] = kExpScale * A * inv;
        out[D + 1] = kExpScale * 0.5f * (s01 + s10);
        out[D + 2] = kExpScale * 0.5f * (s02 + s20);
        out[D + 3] = kExpScale * (a * k - c * g) * inv;
        out[D + 4] = kExpScale * 0.5f * (s12 + s21);
        out[D + 5] = kExpScale * (a * e - b * d) * inv;
    }
    out[D + NS + 0] = gauss_norm_factor<D>() * rsqrtf(det);         // sqrt(det S) = 1 / sqrt(det C)
    out[D + NS + 1] = w;
    const float initial = (w + constant > 0.f) ? w : -relu_constant;
    out[D + NS + 2] = fabsf(initial) + 0.1f;
}

template <int D>
__global__ void __launch_bounds__(kThreads)
relu_fixed_point_kernel(const float* __restrict__ mixtures, const float* __restrict__ constants,
                        float* __restrict__ out_mixtures, float* __restrict__ out_constants,
                        float* __restrict__ out_initial, long long n_mixtures, int G, int mixtures_per_cta,
                        LayerTransform tf) {
    constexpr int RF = 1 + D + D * D;
    constexpr int NS = D * (D + 1) / 2;
    constexpr int RD = Ready<D>::kFloats;
    extern __shared__ __align__(16) float ready[];     // [mixtures_per_cta][min(G, kChunk)][RD]
    const int tid = threadIdx.x;
    const long long first = (long long)blockIdx.x * mixtures_per_cta;
    const int local = mixtures_per_cta > 1 ? tid / G : 0;            // which of the CTA's mixtures
    const long long mix = first + local;
    const bool mixture_ok = local < mixtures_per_cta && mix < n_mixtures;
    const float constant = (mixture_ok && constants != nullptr) ? __ldg(constants + mix) : 0.f;
    const float relu_constant = fmaxf(constant, 0.f);
    const float out_scale = (mixture_ok && tf.spatial_scale != nullptr) ? __ldg(tf.spatial_scale + mix % tf.n_channels) : 1.f;
    const float* src = mixtures + mix * (long long)G * RF;
    const int stage_stride = stage_stride_floats(min(G, kChunk) * RD);
    const bool single_chunk = G <= kChunk;

    // rows of this thread: i = row0, row0 + kThreads, ... (one row when G <= kThreads)
    const int row0 = mixtures_per_cta > 1 ? tid - local * G : tid;
    for (int base = 0; base < G; base += (mixtures_per_cta > 1 ? G : kThreads)) {
        const int i = base + row0;
        const bool row_ok = mixture_ok && i < G;
        float p[D], sum_w = 0.f, sum_x = 0.f;
#pragma unroll
        for (int d = 0; d < D; ++d) p[d] = row_ok ? __ldg(src + (size_t)i * RF + 1 + d) : 0.f;
        for (int j0 = 0; j0 < G; j0 += kChunk) {
            const int jc = min(kChunk, G - j0);
            __syncthreads();                                          // previous chunk fully consumed
            if (single_chunk && base > 0) {
                // the only chunk is already staged
            } else if (mixtures_per_cta > 1) {
                if (mixture_ok && row0 < jc) {                        // thread (mixture, j) stages Gaussian j
                    float r[RF];
#pragma unroll
                    for (int f = 0; f < RF; ++f) r[f] = __ldg(src + (size_t)(j0 + row0) * RF + f);
                    make_ready<D>(r, constant, relu_constant, tf.weight_divisor, ready + local * stage_stride + row0 * RD);
                }
            } else {
                for (int j = tid; j < jc; j += kThreads) {
                    float r[RF];
#pragma unroll
                    for (int f = 0; f < RF; ++f) r[f] = __ldg(src + (size_t)(j0 + j) * RF + f);
                    make_ready<D>(r, constant, relu_constant, tf.weight_divisor, ready + j * RD);
                }
            }
            __syncthreads();
            if (row_ok) {
                const float4* g4 = reinterpret_cast<const float4*>(ready + local * stage_stride);
#pragma unroll 4
                for (int j = 0; j < jc; ++j) {
                    float g[RD];
#pragma unroll
                    for (int v = 0; v < RD / 4; ++v) {
                        const float4 t = g4[j * (RD / 4) + v];
                        g[4 * v] = t.x; g[4 * v + 1] = t.y; g[4 * v + 2] = t.z; g[4 * v + 3] = t.w;
                    }
                    float q;
                    if constexpr (D == 2) {
                        const float t0 = p[0] + g[0], t1 = p[1] + g[1];
                        q = t0 * (g[2] * t0 + 2.f * g[3] * t1) + t1 * (g[4] * t1);
                    } else {
                        const float t0 = p[0] + g[0], t1 = p[1] + g[1], t2 = p[2] + g[2];
                        q = t0 * (g[3] * t0 + 2.f * (g[4] * t1 + g[5] * t2)) + t1 * (g[6] * t1 + 2.f * g[7] * t2) +
                            t2 * (g[8] * t2);
                    }
                    const float e = g[D + NS] * ex2_approx(q);
                    sum_w = fmaf(g[D + NS + 1], e, sum_w);
                    sum_x = fmaf(g[D + NS + 2], e, sum_x);
                }
            }
        }
        if (row_ok) {
            const float w = __ldg(src + (size_t)i * RF) / tf.weight_divisor;
            const float initial = (w + constant > 0.f) ? w : -relu_constant;
            const float x0 = fabsf(initial) + 0.1f;
            const float b = fmaxf(sum_w + constant, 0.f) - relu_constant;
            const float x = x0 * (b + 0.05f) / (sum_x + 0.05f);
            float* dst = out_mixtures + (mix * (long long)G + i) * RF;
            dst[0] = x;
            if (tf.spatial_scale != nullptr) {
                store_geometry<D>(dst, src + (size_t)i * RF, out_scale);
            } else {
#pragma unroll
                for (int f = 1; f < RF; ++f) dst[f] = __ldg(src + (size_t)i * RF + f);
            }
            if (out_initial) {
                float* ini = out_initial + (mix * (long long)G + i) * RF;
                ini[0] = initial;
#pragma unroll
                for (int f = 1; f < RF; ++f) ini[f] = __ldg(src + (size_t)i * RF + f);
            }
            if (i == 0) out_constants[mix] = relu_constant;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Large mixtures (one CTA per mixture, G >= kLargeMin): the pair loop in packed fp32x2 arithmetic. Two Gaussians share
// one instruction (their ready values are interleaved in shared memory, so one broadcast float4 load delivers two
// packed operands), a thread owns P centres, and the normalisation is folded into the two weights, which leaves
// 9 (2D) / 14 (3D) packed operations and two ex2 per (centre, Gaussian pair) for BOTH sums.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kLargeMin = 256;
constexpr int kLargePoints = 4;

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }
__device__ __forceinline__ float2 ex2_2(float2 q) { return make_float2(ex2_approx(q.x), ex2_approx(q.y)); }

// 2^(-|y|^2) with the sign flipped by two scalar FFMAs (the packed instructions have no operand negation).
__device__ __forceinline__ float2 ex2_of_minus_square(float2 y0, float2 y1) {
    const float2 w = __fmul2_rn(y0, y0);
    return make_float2(ex2_approx(fmaf(-y1.x, y1.x, -w.x)), ex2_approx(fmaf(-y1.y, y1.y, -w.y)));
}
__device__ __forceinline__ float2 ex2_of_minus_square(float2 y0, float2 y1, float2 y2) {
    const float2 w = __ffma2_rn(y1, y1, __fmul2_rn(y0, y0));
    return make_float2(ex2_approx(fmaf(-y2.x, y2.x, -w.x)), ex2_approx(fmaf(-y2.y, y2.y, -w.y)));
}

// Triangular form of a Gaussian from its ready form (make_ready: -mu | A = -1/2 log2(e) sym(S) | ...): with
// -A = L L^T (Cholesky) the exponent is -|L^T (x - mu)|^2, and y = L^T x' + nb with x' = x - origin and
// nb = -L^T (mu - origin) needs no subtraction per pair (the evaluation kernels use the same form; see their note on its
// rounding). tri: nb[D] | L (l00 l10 [l20] l11 [l21 l22]). Returns the largest absolute row sum of L^T, +inf if the
// matrix is not positive definite.
template <int D>
__device__ __forceinline__ float triangular_from_ready(const float* rdy, const float* origin, float* tri) {
    if constexpr (D == 2) {
        const float a00 = -rdy[2], a01 = -rdy[3], a11 = -rdy[4];
        const float l00 = sqrtf(a00), l10 = a01 / l00;
        const float d1 = a11 - l10 * l10;
        const float l11 = sqrtf(d1);
        const float m0 = -rdy[0] - origin[0], m1 = -rdy[1] - origin[1];
        tri[0] = -(l00 * m0 + l10 * m1);
        tri[1] = -(l11 * m1);
        tri[2] = l00; tri[3] = l10; tri[4] = l11;
        return (a00 > 0.f && d1 > 0.f) ? fmaxf(fabsf(l00) + fabsf(l10), fabsf(l11)) : INFINITY;
    } else {
        const float a00 = -rdy[3], a01 = -rdy[4], a02 = -rdy[5], a11 = -rdy[6], a12 = -rdy[7], a22 = -rdy[8];
        const float l00 = sqrtf(a00), l10 = a01 / l00, l20 = a02 / l00;
        const float d1 = a11 - l10 * l10;
        const float l11 = sqrtf(d1), l21 = (a12 - l20 * l10) / l11;
        const float d2 = a22 - l20 * l20 - l21 * l21;
        const float l22 = sqrtf(d2);
        const float m0 = -rdy[0] - origin[0], m1 = -rdy[1] - origin[1], m2 = -rdy[2] - origin[2];
        tri[0] = -(l00 * m0 + l10 * m1 + l20 * m2);
        tri[1] = -(l11 * m1 + l21 * m2);
        tri[2] = -(l22 * m2);
        tri[3] = l00; tri[4] = l10; tri[5] = l20; tri[6] = l11; tri[7] = l21; tri[8] = l22;
        const float bound = fmaxf(fabsf(l00) + fabsf(l10) + fabsf(l20), fmaxf(fabsf(l11) + fabsf(l21), fabsf(l22)));
        return (a00 > 0.f && d1 > 0.f && d2 > 0.f) ? bound : INFINITY;
    }
}

// (row-sum bound) x (half extent of the mixture's centres) up to which the triangular loop is used: the error of a
// pair's value stays below 3e-5 of the Gaussian's peak (the forward evaluation kernel uses the same limit).
constexpr float kTriangularLimit = 350.f;

template <int D>
struct ReadyLarge {
    // per Gaussian: -mu | A (off-diagonals doubled) | norm w, norm x0 | pad = 8 (2D) or 12 (3D) floats, whole float4
    static constexpr int kPairFloats = 2 * (D == 2 ? 8 : 12);
};

template <int D, int P>
__global__ void __launch_bounds__(kThreads)
relu_fixed_point_large_kernel(const float* __restrict__ mixtures, const float* __restrict__ constants,
                              float* __restrict__ out_mixtures, float* __restrict__ out_constants,
                              float* __restrict__ out_initial, int G, LayerTransform tf) {
    constexpr int RF = 1 + D + D * D;
    constexpr int NS = D * (D + 1) / 2;
    constexpr int RD = Ready<D>::kFloats;
    constexpr int PF = ReadyLarge<D>::kPairFloats;
    constexpr int PV = PF / 4;                        // float4 per Gaussian pair
    extern __shared__ __align__(16) float ready[];    // [kChunk / 2][PF]
    const int tid = threadIdx.x;
    const long long mix = blockIdx.x;
    const float constant = constants != nullptr ? __ldg(constants + mix) : 0.f;
    const float relu_constant = fmaxf(constant, 0.f);
    const float out_scale = tf.spatial_scale != nullptr ? __ldg(tf.spatial_scale + mix % tf.n_channels) : 1.f;
    const float* src = mixtures + mix * (long long)G * RF;
    const bool single_chunk = G <= kChunk;

    // ---- box of the centres and the largest row-sum bound of the mixture: which pair loop ----
    __shared__ float s_red[kThreads / 32][2 * D + 1];
    __shared__ float s_origin[D];
    __shared__ int s_triangular;
    {
        float lo[D], hi[D], bound = 0.f;
        float zero[D];
#pragma unroll
        for (int d = 0; d < D; ++d) { lo[d] = INFINITY; hi[d] = -INFINITY; zero[d] = 0.f; }
        for (int j = tid; j < G; j += kThreads) {
            float r[RF], rdy[RD], tri[D + NS];
#pragma unroll
            for (int f = 0; f < RF; ++f) r[f] = __ldg(src + (size_t)j * RF + f);
            make_ready<D>(r, constant, relu_constant, tf.weight_divisor, rdy);
            const float b = triangular_from_ready<D>(rdy, zero, tri);
            bound = (b >= bound) ? b : (b == b ? bound : INFINITY);
#pragma unroll
            for (int d = 0; d < D; ++d) { lo[d] = fminf(lo[d], r[1 + d]); hi[d] = fmaxf(hi[d], r[1 + d]); }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            bound = fmaxf(bound, __shfl_xor_sync(0xffffffffu, bound, o));
#pragma unroll
            for (int d = 0; d < D; ++d) {
                lo[d] = fminf(lo[d], __shfl_xor_sync(0xffffffffu, lo[d], o));
                hi[d] = fmaxf(hi[d], __shfl_xor_sync(0xffffffffu, hi[d], o));
            }
        }
        if ((tid & 31) == 0) {
            s_red[tid >> 5][0] = bound;
#pragma unroll
            for (int d = 0; d < D; ++d) { s_red[tid >> 5][1 + d] = lo[d]; s_red[tid >> 5][1 + D + d] = hi[d]; }
        }
        __syncthreads();
        if (tid == 0) {
            float bmax = 0.f, half = 0.f;
            for (int w = 0; w < kThreads / 32; ++w) bmax = fmaxf(bmax, s_red[w][0]);     // fmaxf keeps +inf; NaN became +inf above
#pragma unroll
            for (int d = 0; d < D; ++d) {
                float l = s_red[0][1 + d], h = s_red[0][1 + D + d];
                for (int w = 1; w < kThreads / 32; ++w) { l = fminf(l, s_red[w][1 + d]); h = fmaxf(h, s_red[w][1 + D + d]); }
                const float centre = 0.5f * l + 0.5f * h;
                s_origin[d] = centre;
                half = fmaxf(half, fmaxf(h - centre, centre - l));
            }
            s_triangular = (bmax * half <= kTriangularLimit) ? 1 : 0;
        }
        __syncthreads();
    }
    const bool triangular = s_triangular != 0;
    float origin[D];
#pragma unroll
    for (int d = 0; d < D; ++d) origin[d] = s_origin[d];

    for (int base = 0; base < G; base += kThreads * P) {
        float2 x[P][D], sum_w[P], sum_x[P];
#pragma unroll
        for (int p = 0; p < P; ++p) {
            const int i = base + tid + p * kThreads;
#pragma unroll
            for (int d = 0; d < D; ++d) {
                const float v = i < G ? __ldg(src + (size_t)i * RF + 1 + d) - origin[d] : 0.f;
                x[p][d] = f2(v, v);
            }
            sum_w[p] = f2(0.f, 0.f);
            sum_x[p] = f2(0.f, 0.f);
        }
        for (int j0 = 0; j0 < G; j0 += kChunk) {
            const int jc = min(kChunk, G - j0);
            const int jc_even = (jc + 1) & ~1;
            __syncthreads();
            if (!(single_chunk && base > 0)) {
                for (int j = tid; j < jc_even; j += kThreads) {
                    float rdy[RD];
                    float* dst = ready + (j >> 1) * PF + (j & 1);
                    if (j < jc) {
                        float r[RF];
#pragma unroll
                        for (int f = 0; f < RF; ++f) r[f] = __ldg(src + (size_t)(j0 + j) * RF + f);
                        make_ready<D>(r, constant, relu_constant, tf.weight_divisor, rdy);
                    } else {
#pragma unroll
                        for (int f = 0; f < RD; ++f) rdy[f] = 0.f;      // padding Gaussian: both weights 0
                    }
                    if (triangular) {
                        float tri[D + NS];
                        if (j < jc) {
                            triangular_from_ready<D>(rdy, origin, tri);
                        } else {
#pragma unroll
                            for (int f = 0; f < D + NS; ++f) tri[f] = 0.f;
                        }
#pragma unroll
                        for (int f = 0; f < D + NS; ++f) dst[2 * f] = tri[f];
                    } else {
#pragma unroll
                        for (int f = 0; f < D; ++f) dst[2 * f] = rdy[f] + origin[f];        // origin - mu
                        if constexpr (D == 2) {
                            dst[2 * 2] = rdy[2]; dst[2 * 3] = 2.f * rdy[3]; dst[2 * 4] = rdy[4];
                        } else {
                            dst[2 * 3] = rdy[3]; dst[2 * 4] = 2.f * rdy[4]; dst[2 * 5] = 2.f * rdy[5];
                            dst[2 * 6] = rdy[6]; dst[2 * 7] = 2.f * rdy[7]; dst[2 * 8] = rdy[8];
                        }
                    }
                    dst[2 * (D + NS)] = rdy[D + NS] * rdy[D + NS + 1];          // norm * w
                    dst[2 * (D + NS + 1)] = rdy[D + NS] * rdy[D + NS + 2];      // norm * x0
                    dst[2 * (D + NS + 2)] = 0.f;                                // pad
                }
            }
            __syncthreads();
            const float4* rp = reinterpret_cast<const float4*>(ready);
            const int n_pairs = jc_even >> 1;
            if (triangular) {
#pragma unroll 2
                for (int j = 0; j < n_pairs; ++j) {
                    float4 v[PV];
#pragma unroll
                    for (int k = 0; k < PV; ++k) v[k] = rp[j * PV + k];
                    if constexpr (D == 2) {
                        const float2 nb0 = f2(v[0].x, v[0].y), nb1 = f2(v[0].z, v[0].w), l00 = f2(v[1].x, v[1].y),
                                     l10 = f2(v[1].z, v[1].w), l11 = f2(v[2].x, v[2].y), cw = f2(v[2].z, v[2].w),
                                     cx = f2(v[3].x, v[3].y);
#pragma unroll
                        for (int p = 0; p < P; ++p) {
                            const float2 y1 = __ffma2_rn(l11, x[p][1], nb1);
                            const float2 y0 = __ffma2_rn(l00, x[p][0], __ffma2_rn(l10, x[p][1], nb0));
                            const float2 e = ex2_of_minus_square(y0, y1);
                            sum_w[p] = __ffma2_rn(cw, e, sum_w[p]);
                            sum_x[p] = __ffma2_rn(cx, e, sum_x[p]);
                        }
                    } else {
                        const float2 nb0 = f2(v[0].x, v[0].y), nb1 = f2(v[0].z, v[0].w), nb2 = f2(v[1].x, v[1].y),
                                     l00 = f2(v[1].z, v[1].w), l10 = f2(v[2].x, v[2].y), l20 = f2(v[2].z, v[2].w),
                                     l11 = f2(v[3].x, v[3].y), l21 = f2(v[3].z, v[3].w), l22 = f2(v[4].x, v[4].y),
                                     cw = f2(v[4].z, v[4].w), cx = f2(v[5].x, v[5].y);
#pragma unroll
                        for (int p = 0; p < P; ++p) {
                            const float2 y2 = __ffma2_rn(l22, x[p][2], nb2);
                            const float2 y1 = __ffma2_rn(l11, x[p][1], __ffma2_rn(l21, x[p][2], nb1));
                            const float2 y0 = __ffma2_rn(l00, x[p][0], __ffma2_rn(l10, x[p][1], __ffma2_rn(l20, x[p][2], nb0)));
                            const float2 e = ex2_of_minus_square(y0, y1, y2);
                            sum_w[p] = __ffma2_rn(cw, e, sum_w[p]);
                            sum_x[p] = __ffma2_rn(cx, e, sum_x[p]);
                        }
                    }
                }
            } else {
#pragma unroll 2
                for (int j = 0; j < n_pairs; ++j) {
                    float4 v[PV];
#pragma unroll
                    for (int k = 0; k < PV; ++k) v[k] = rp[j * PV + k];
                    if constexpr (D == 2) {
                        const float2 nm0 = f2(v[0].x, v[0].y), nm1 = f2(v[0].z, v[0].w), a00 = f2(v[1].x, v[1].y),
                                     a01 = f2(v[1].z, v[1].w), a11 = f2(v[2].x, v[2].y), cw = f2(v[2].z, v[2].w),
                                     cx = f2(v[3].x, v[3].y);
#pragma unroll
                        for (int p = 0; p < P; ++p) {
                            const float2 t0 = __fadd2_rn(x[p][0], nm0), t1 = __fadd2_rn(x[p][1], nm1);
                            const float2 r0 = __ffma2_rn(a01, t1, __fmul2_rn(a00, t0));
                            const float2 r1 = __fmul2_rn(a11, t1);
                            const float2 e = ex2_2(__ffma2_rn(t1, r1, __fmul2_rn(t0, r0)));
                            sum_w[p] = __ffma2_rn(cw, e, sum_w[p]);
                            sum_x[p] = __ffma2_rn(cx, e, sum_x[p]);
                        }
                    } else {
                        const float2 nm0 = f2(v[0].x, v[0].y), nm1 = f2(v[0].z, v[0].w), nm2 = f2(v[1].x, v[1].y),
                                     a00 = f2(v[1].z, v[1].w), a01 = f2(v[2].x, v[2].y), a02 = f2(v[2].z, v[2].w),
                                     a11 = f2(v[3].x, v[3].y), a12 = f2(v[3].z, v[3].w), a22 = f2(v[4].x, v[4].y),
                                     cw = f2(v[4].z, v[4].w), cx = f2(v[5].x, v[5].y);
#pragma unroll
                        for (int p = 0; p < P; ++p) {
                            const float2 t0 = __fadd2_rn(x[p][0], nm0), t1 = __fadd2_rn(x[p][1], nm1),
                                         t2 = __fadd2_rn(x[p][2], nm2);
                            const float2 r0 = __ffma2_rn(a02, t2, __ffma2_rn(a01, t1, __fmul2_rn(a00, t0)));
                            const float2 r1 = __ffma2_rn(a12, t2, __fmul2_rn(a11, t1));
                            const float2 r2 = __fmul2_rn(a22, t2);
                            const float2 e = ex2_2(__ffma2_rn(t2, r2, __ffma2_rn(t1, r1, __fmul2_rn(t0, r0))));
                            sum_w[p] = __ffma2_rn(cw, e, sum_w[p]);
                            sum_x[p] = __ffma2_rn(cx, e, sum_x[p]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int p = 0; p < P; ++p) {
            const int i = base + tid + p * kThreads;
            if (i >= G) continue;
            const float w = __ldg(src + (size_t)i * RF) / tf.weight_divisor;
            const float initial = (w + constant > 0.f) ? w : -relu_constant;
            const float x0 = fabsf(initial) + 0.1f;
            const float b = fmaxf(sum_w[p].x + sum_w[p].y + constant, 0.f) - relu_constant;
            float* dst = out_mixtures + (mix * (long long)G + i) * RF;
            dst[0] = x0 * (b + 0.05f) / (sum_x[p].x + sum_x[p].y + 0.05f);
            if (tf.spatial_scale != nullptr) {
                store_geometry<D>(dst, src + (size_t)i * RF, out_scale);
            } else {
#pragma unroll
                for (int f = 1; f < RF; ++f) dst[f] = __ldg(src + (size_t)i * RF + f);
            }
            if (out_initial) {
                float* ini = out_initial + (mix * (long long)G + i) * RF;
                ini[0] = initial;
#pragma unroll
                for (int f = 1; f < RF; ++f) ini[f] = __ldg(src + (size_t)i * RF + f);
            }
        }
        if (base == 0 && tid == 0) out_constants[mix] = relu_constant;
    }
}

template <int D>
int launch_relu_fixed_point(const float* mixtures, const float* constants, float* out_mixtures, float* out_constants,
                            float* out_initial, long long n_mixtures, int G, LayerTransform tf, cudaStream_t st) {
    if (G >= kLargeMin) {
        if (n_mixtures > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
        const int staged_pairs = (min(G, kChunk) + 1) / 2;
        const size_t smem = sizeof(float) * size_t(staged_pairs) * ReadyLarge<D>::kPairFloats;
        auto kernel = relu_fixed_point_large_kernel<D, kLargePoints>;
        if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        kernel<<<unsigned(n_mixtures), kThreads, smem, st>>>(mixtures, constants, out_mixtures, out_constants, out_initial, G, tf);
        GMC_LAUNCH_CHECK();
        return GMC_OK;
    }
    const int per_cta = G <= kThreads ? kThreads / G : 1;
    const long long blocks = (n_mixtures + per_cta - 1) / per_cta;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    const size_t smem = sizeof(float) * size_t(per_cta) * stage_stride_floats(min(G, kChunk) * Ready<D>::kFloats);
    auto kernel = relu_fixed_point_kernel<D>;
    if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    kernel<<<unsigned(blocks), kThreads, smem, st>>>(mixtures, constants, out_mixtures, out_constants, out_initial,
                                                    n_mixtures, G, per_cta, tf);
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

}  // namespace
}  // namespace gmc

GMC_DEFINE_TU_CHECK_READER(relu_fixed_point)

extern "C" int gmc_relu_fixed_point_layer(const float* mixtures, const float* constants, float* out_mixtures,
                                          float* out_constants, float* out_initial, long long n_mixtures,
                                          int n_components, int n_dims, float weight_divisor,
                                          const float* spatial_scale, int n_channels, void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_mixtures < 0 || n_components <= 0) return GMC_ERR_BAD_DIMS;
    if (!(weight_divisor != 0.f)) return GMC_ERR_UNSUPPORTED;
    if (spatial_scale != nullptr && n_channels <= 0) return GMC_ERR_BAD_DIMS;
    if (n_mixtures == 0) return GMC_OK;
    if (!mixtures || !out_mixtures || !out_constants) return GMC_ERR_NULL_POINTER;
    cudaStream_t st = as_stream(stream);
    const LayerTransform tf{weight_divisor, spatial_scale, spatial_scale ? n_channels : 1};
    return n_dims == 2 ? launch_relu_fixed_point<2>(mixtures, constants, out_mixtures, out_constants, out_initial,
                                                    n_mixtures, n_components, tf, st)
                       : launch_relu_fixed_point<3>(mixtures, constants, out_mixtures, out_constants, out_initial,
                                                    n_mixtures, n_components, tf, st);
}

extern "C" int gmc_relu_fixed_point(const float* mixtures, const float* constants, float* out_mixtures,
                                    float* out_constants, float* out_initial, long long n_mixtures, int n_components,
                                    int n_dims, void* stream) {
    if (n_mixtures > 0 && !constants) return GMC_ERR_NULL_POINTER;
    return gmc_relu_fixed_point_layer(mixtures, constants, out_mixtures, out_constants, out_initial, n_mixtures,
                                      n_components, n_dims, 1.f, nullptr, 1, stream);
}
