// Mixture evaluation (inverse-covariance form), forward and backward, for sm_100a.
//
//   out[b,l,n] = sum_g w_g * (2 pi)^(-D/2) * sqrt(det S_g) * exp(-1/2 (x_n - mu_g)^T S_g (x_n - mu_g))
//
// Same arithmetic as the reference's gpe::evaluate_inversed / gpe::grad::evaluate_inversed
// (src/gmc/cpp/extensions/util/gaussian.h:82-95, util/grad/gaussian.h:19-66), organised differently:
//
//  forward : a CTA owns one (batch, layer) mixture and a tile of query points. Gaussians are staged
//            chunk-wise in shared memory (raw records arrive by one non-multicast bulk copy when the
//            chunk is 16-byte aligned) and rewritten once per CTA into "ready" form
//                c = w (2 pi)^(-D/2) sqrt(det S),  mu,  A = -1/2 log2(e) S  (off-diagonals folded)
//            so the pair loop is   t = x - mu;  q = t^T A t;  acc += c * ex2(q)   (FMA pipe + one MUFU),
//            or, where its rounding allows (decided per chunk, see make_triangular), into "triangular" form
//                c,  L with 1/2 log2(e) S = L L^T,  nb = -L^T mu
//            with the shorter loop   y = L^T x + nb;  acc += c * ex2(-|y|^2)   (no subtraction per pair).
//            Both loops work on coordinates relative to the centre of the tile's points.
//            Every thread keeps P query points in registers and reads Gaussians as broadcast float4.
//  backward: a CTA owns one (batch, layer), a tile of query points and a chunk of Gaussians. Every thread
//            keeps GQ Gaussians and their 1 + D + D(D+1)/2 gradient sums in registers and streams the
//            tile's points (x, grad_out) from shared memory, so the per-Gaussian sums need no cross-lane
//            traffic in the pair loop. The per-point position gradient is what crosses lanes: each lane
//            writes its D partial sums into its warp's own padded shared rows and the warp folds them once
//            per 16 points (no CTA barrier in the loop). Totals go to global memory with one atomic per value.
#include <cstddef>
#include <type_traits>

#include "common.cuh"

namespace gmc {
namespace {

// Tuning constants (overridable at compile time for experiments).
#ifndef GMC_FWD_CHUNK
#define GMC_FWD_CHUNK 256
#endif
#ifndef GMC_FWD_P
#define GMC_FWD_P 4
#endif
#ifndef GMC_FWD_MINB
#define GMC_FWD_MINB 6
#endif
#ifndef GMC_BWD_PPI
#define GMC_BWD_PPI 2
#endif
#ifndef GMC_BWD_UNROLL
#define GMC_BWD_UNROLL 2            // iterations of the point loop unrolled (1, 4, 8 measured within 1 %)
#endif
#ifndef GMC_BWD_MINB
#define GMC_BWD_MINB 4
#endif
#ifndef GMC_BWD_GP_LARGE
#define GMC_BWD_GP_LARGE 2          // packed Gaussian pairs per thread for mixtures of 384 components and more
#endif
#ifndef GMC_BWD_THREADS_LARGE
#define GMC_BWD_THREADS_LARGE 128   // CTA size of that variant (all threads along the Gaussian axis)
#endif
constexpr int kFwdThreads = 128;
constexpr int kFwdChunk = GMC_FWD_CHUNK;   // Gaussians staged per shared-memory chunk
constexpr int kFwdPoints = GMC_FWD_P;      // query points per thread in the large-problem variant

template <int D>
struct Raw {
    static constexpr int kFloats = 1 + D + D * D;
};

// ---------------------------------------------------------------------------------------------
// Packed fp32x2 arithmetic. sm_100 executes one packed instruction on two fp32 lanes of a 64-bit register
// pair, so a pair loop written on float2 needs half the issue slots of the scalar form; the two halves
// always belong to two different Gaussians evaluated at the same query point.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 ex2_2(float2 q) { return make_float2(ex2_approx(q.x), ex2_approx(q.y)); }

constexpr float kExpScale = -0.5f * kLog2e;

// 2^(-|y|^2) for the packed pair (y0, y1[, y2]). The packed instructions have no operand negation, the scalar FFMA has:
// the last term is added by two scalar FFMAs that flip both signs on the way (a packed FFMA plus two negations, or a
// packed multiply by -1, measured 4 % slower in the forward kernel).
__device__ __forceinline__ float2 ex2_of_minus_square(float2 y0, float2 y1) {
    const float2 w = mul2(y0, y0);
    return make_float2(ex2_approx(fmaf(-y1.x, y1.x, -w.x)), ex2_approx(fmaf(-y1.y, y1.y, -w.y)));
}
__device__ __forceinline__ float2 ex2_of_minus_square(float2 y0, float2 y1, float2 y2) {
    const float2 w = fma2(y1, y1, mul2(y0, y0));
    return make_float2(ex2_approx(fmaf(-y2.x, y2.x, -w.x)), ex2_approx(fmaf(-y2.y, y2.y, -w.y)));
}

__device__ __forceinline__ float det2(const float* S) { return S[0] * S[3] - S[1] * S[2]; }
__device__ __forceinline__ float det3(const float* S) {
    return S[0] * (S[4] * S[8] - S[5] * S[7]) - S[1] * (S[3] * S[8] - S[5] * S[6]) +
           S[2] * (S[3] * S[7] - S[4] * S[6]);
}

// "ready" form of one Gaussian for the forward pair loop:
//   nm = -mu, c = w (2 pi)^(-D/2) sqrt(det S), a_ii = k S_ii, a_ij = k (S_ij + S_ji) (i < j), k = -1/2 log2(e)
// 2D: nm0 nm1 c a00 a01 a11 (6 values); 3D: nm0 nm1 nm2 c a00 a01 a02 a11 a12 a22 (10 values).
template <int D>
struct ReadyCount {
    static constexpr int value = D == 2 ? 6 : 10;
};

template <int D>
__device__ __forceinline__ void make_ready(const float* r, const float* origin, float* out) {
    if constexpr (D == 2) {
        const float* S = r + 3;
        out[0] = origin[0] - r[1]; out[1] = origin[1] - r[2];
        out[2] = r[0] * kInv2Pi * sqrtf(det2(S));
        out[3] = kExpScale * S[0]; out[4] = kExpScale * (S[1] + S[2]); out[5] = kExpScale * S[3];
    } else {
        const float* S = r + 4;
        out[0] = origin[0] - r[1]; out[1] = origin[1] - r[2]; out[2] = origin[2] - r[3];
        out[3] = r[0] * kInv2Pi15 * sqrtf(det3(S));
        out[4] = kExpScale * S[0]; out[5] = kExpScale * (S[1] + S[3]); out[6] = kExpScale * (S[2] + S[6]);
        out[7] = kExpScale * S[4]; out[8] = kExpScale * (S[5] + S[7]); out[9] = kExpScale * S[8];
    }
}

// "triangular" form of one Gaussian for the short pair loop: with A = 1/2 log2(e) sym(S) = L L^T (Cholesky, L lower
// triangular) the exponent is -|L^T (x - mu)|^2 in base 2, and y = L^T x' + nb with x' = x - origin,
// nb = -L^T (mu - origin) needs no separate subtraction per pair: 9 multiply-adds for y and |y|^2 in 3D instead of 12.
// 2D: nb0 nb1 c l00 l10 l11; 3D: nb0 nb1 nb2 c l00 l10 l20 l11 l21 l22 (the same record sizes as the ready form).
// The price is rounding: y is a difference of terms of size |L| |x'|, so the form is only used where that size, bounded
// by the largest absolute row sum of L^T (returned here; +inf if S is not positive definite) times the half extent of
// the tile's points, keeps the error of the exponent far below the tolerance (see kTriangularLimit).
template <int D>
__device__ __forceinline__ float make_triangular(const float* r, const float* origin, float* out) {
    constexpr float k = 0.5f * kLog2e;
    if constexpr (D == 2) {
        const float* S = r + 3;
        const float a00 = k * S[0], a01 = 0.5f * k * (S[1] + S[2]), a11 = k * S[3];
        const float l00 = sqrtf(a00), l10 = a01 / l00;
        const float d1 = a11 - l10 * l10;
        const float l11 = sqrtf(d1);
        const float m0 = r[1] - origin[0], m1 = r[2] - origin[1];
        out[0] = -(l00 * m0 + l10 * m1);
        out[1] = -(l11 * m1);
        out[2] = r[0] * kInv2Pi * sqrtf(det2(S));
        out[3] = l00; out[4] = l10; out[5] = l11;
        const float bound = fmaxf(fabsf(l00) + fabsf(l10), fabsf(l11));
        return (a00 > 0.f && d1 > 0.f) ? bound : INFINITY;
    } else {
        const float* S = r + 4;
        const float a00 = k * S[0], a01 = 0.5f * k * (S[1] + S[3]), a02 = 0.5f * k * (S[2] + S[6]);
        const float a11 = k * S[4], a12 = 0.5f * k * (S[5] + S[7]), a22 = k * S[8];
        const float l00 = sqrtf(a00), l10 = a01 / l00, l20 = a02 / l00;
        const float d1 = a11 - l10 * l10;
        const float l11 = sqrtf(d1), l21 = (a12 - l20 * l10) / l11;
        const float d2 = a22 - l20 * l20 - l21 * l21;
        const float l22 = sqrtf(d2);
        const float m0 = r[1] - origin[0], m1 = r[2] - origin[1], m2 = r[3] - origin[2];
        out[0] = -(l00 * m0 + l10 * m1 + l20 * m2);
        out[1] = -(l11 * m1 + l21 * m2);
        out[2] = -(l22 * m2);
        out[3] = r[0] * kInv2Pi15 * sqrtf(det3(S));
        out[4] = l00; out[5] = l10; out[6] = l20; out[7] = l11; out[8] = l21; out[9] = l22;
        const float bound = fmaxf(fabsf(l00) + fabsf(l10) + fabsf(l20), fmaxf(fabsf(l11) + fabsf(l21), fabsf(l22)));
        return (a00 > 0.f && d1 > 0.f && d2 > 0.f) ? bound : INFINITY;
    }
}

// Largest (row sum of |L^T|) x (half extent of the tile's points) for which a chunk of Gaussians takes the triangular
// loop. The rounding error of y is at most 2 eps x that product for a pair that matters (a Gaussian within reach of
// the tile), which changes the pair's value by at most 0.71 x that much of the Gaussian's peak: 350 -> 3e-5 of the peak.
constexpr float kTriangularLimit = 350.f;
// The backward pass sums gradients, which feel an error of y more than the value does (a term's relative error is about
// (2 ln 2 |y| + 2 / |y|) times it): a tighter limit, still twice what the 3D benchmark configuration needs.
constexpr float kTriangularLimitBackward = 120.f;

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
// Shared layout of the ready records: Gaussians 2j and 2j+1 are interleaved value by value,
//   pair j = [v0(2j) v0(2j+1) v1(2j) v1(2j+1) ...], 2 * ReadyCount floats = 3 (2D) or 5 (3D) float4,
// so one broadcast float4 load delivers two packed operands.
template <int D, int P>
struct FwdSmem {
    static constexpr int kTile = kFwdThreads * P;
    static constexpr int kPairFloats = 2 * ReadyCount<D>::value;
    alignas(16) float raw[kFwdChunk * Raw<D>::kFloats];
    alignas(16) float ready[(kFwdChunk / 2) * kPairFloats];
    alignas(16) float xs[kTile * D];
    alignas(8) uint64_t bar;
    float box_lo[D][kFwdThreads / 32], box_hi[D][kFwdThreads / 32];
    float origin[D];
    float half_extent;
    int row_sum_bits;      // largest row-sum bound of the chunk, as the bit pattern of a non-negative float
};

template <int D, int P>
__global__ void __launch_bounds__(kFwdThreads, GMC_FWD_MINB)
eval_forward_kernel(const float* __restrict__ mixture, const float* __restrict__ xes, float* __restrict__ out,
                    int n_layers, int n_components, int n_batch_xes, int n_layers_xes, int n_xes,
                    int tiles_per_mixture, int lose_copy) {
    constexpr int RF = Raw<D>::kFloats;
    constexpr int RC = ReadyCount<D>::value;
    constexpr int PF = 2 * RC;
    constexpr int TILE = kFwdThreads * P;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    FwdSmem<D, P>& sm = *reinterpret_cast<FwdSmem<D, P>*>(smem_bytes);

    const int tid = threadIdx.x;
    const int bl = blockIdx.x / tiles_per_mixture;
    const int tile = blockIdx.x - bl * tiles_per_mixture;
    const int b = bl / n_layers;
    const int l = bl - b * n_layers;
    const int bx = n_batch_xes == 1 ? 0 : b;
    const int lx = n_layers_xes == 1 ? 0 : l;
    const int n0 = tile * TILE;
    const int n_here = min(TILE, n_xes - n0);

    // ---- stage the tile's query points (flat float stream; float4 when aligned) ----
    {
        const float* src = xes + (size_t(bx) * n_layers_xes + lx) * size_t(n_xes) * D + size_t(n0) * D;
        const int n_floats = n_here * D;
        if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
            const int n4 = n_floats >> 2;
            const float4* src4 = reinterpret_cast<const float4*>(src);
            float4* dst4 = reinterpret_cast<float4*>(sm.xs);
            for (int i = tid; i < n4; i += kFwdThreads) dst4[i] = __ldg(src4 + i);
            for (int i = (n4 << 2) + tid; i < n_floats; i += kFwdThreads) sm.xs[i] = __ldg(src + i);
        } else {
            for (int i = tid; i < n_floats; i += kFwdThreads) sm.xs[i] = __ldg(src + i);
        }
        for (int i = n_floats + tid; i < TILE * D; i += kFwdThreads) sm.xs[i] = 0.f;
    }
    if (tid == 0) {
        mbar_init(&sm.bar, 1);
        fence_mbar_init();
    }
    __syncthreads();

    // ---- origin = centre of the box of the tile's points; the pair loops work on x' = x - origin ----
    {
        float lo[D], hi[D];
#pragma unroll
        for (int d = 0; d < D; ++d) { lo[d] = INFINITY; hi[d] = -INFINITY; }
#pragma unroll
        for (int p = 0; p < P; ++p) {
            const int i = tid + p * kFwdThreads;
            if (i < n_here) {
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const float v = sm.xs[i * D + d];
                    lo[d] = fminf(lo[d], v);
                    hi[d] = fmaxf(hi[d], v);
                }
            }
        }
#pragma unroll
        for (int d = 0; d < D; ++d) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                lo[d] = fminf(lo[d], __shfl_xor_sync(0xffffffffu, lo[d], o));
                hi[d] = fmaxf(hi[d], __shfl_xor_sync(0xffffffffu, hi[d], o));
            }
            if ((tid & 31) == 0) { sm.box_lo[d][tid >> 5] = lo[d]; sm.box_hi[d][tid >> 5] = hi[d]; }
        }
        __syncthreads();
        if (tid == 0) {
            float half = 0.f;
#pragma unroll
            for (int d = 0; d < D; ++d) {
                float l = sm.box_lo[d][0], h = sm.box_hi[d][0];
                for (int w = 1; w < kFwdThreads / 32; ++w) { l = fminf(l, sm.box_lo[d][w]); h = fmaxf(h, sm.box_hi[d][w]); }
                const float centre = 0.5f * l + 0.5f * h;
                sm.origin[d] = centre;
                half = fmaxf(half, fmaxf(h - centre, centre - l));
            }
            sm.half_extent = half;
            sm.row_sum_bits = 0;
        }
        __syncthreads();
    }
    float origin[D];
#pragma unroll
    for (int d = 0; d < D; ++d) origin[d] = sm.origin[d];
    const float half_extent = sm.half_extent;

    float2 x[P][D];    // x - origin, every coordinate duplicated into both halves
    float2 acc[P];
#pragma unroll
    for (int p = 0; p < P; ++p) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const float v = sm.xs[(tid + p * kFwdThreads) * D + d] - origin[d];
            x[p][d] = f2(v, v);
        }
        acc[p] = f2(0.f, 0.f);
    }

    const float* mix = mixture + size_t(bl) * n_components * RF;
    unsigned phase = 0;
    for (int g0 = 0; g0 < n_components; g0 += kFwdChunk) {
        const int gc = min(kFwdChunk, n_components - g0);
        const int gc_even = (gc + 1) & ~1;
        const float* chunk = mix + size_t(g0) * RF;
        const unsigned bytes = unsigned(gc) * RF * 4u;
        const bool bulk = ((reinterpret_cast<uintptr_t>(chunk) & 15u) == 0) && ((bytes & 15u) == 0);
        if (g0 > 0) __syncthreads();   // everyone is done reading the previous chunk
        if (bulk) {
            if (tid == 0) {
                fence_proxy_async();
                mbar_arrive_expect_tx(&sm.bar, bytes);
                // lose_copy (error-path test only): the copy is never issued, so nothing is in flight and the wait
                // below must run out
                if (!lose_copy) bulk_copy_g2s(sm.raw, chunk, bytes, &sm.bar);
            }
            const bool ok = mbar_wait_bounded(&sm.bar, phase, lose_copy ? (1 << 10) : (1 << 22));
            phase ^= 1u;
            if (__syncthreads_or(!ok)) {
                // CTA-wide decision. The wait only runs out when the copy never arrives; the check word is set, and the
                // tile's outputs become NaN so that the failure cannot pass for a result.
                float* o_bad = out + size_t(bl) * n_xes + n0;
                for (int i = tid; i < n_here; i += kFwdThreads) o_bad[i] = __int_as_float(0x7fc00000);
                return;
            }
        }
        auto raw_record = [&](int g, float* r) {
            if (bulk) {
#pragma unroll
                for (int i = 0; i < RF; ++i) r[i] = sm.raw[g * RF + i];
            } else {
#pragma unroll
                for (int i = 0; i < RF; ++i) r[i] = __ldg(chunk + g * RF + i);
            }
        };
        // ---- which loop for this chunk: the largest row-sum bound of its Gaussians against the tile's extent ----
        {
            float bound = 0.f;
            for (int g = tid; g < gc; g += kFwdThreads) {
                float r[RF], tri[RC];
                raw_record(g, r);
                const float b = make_triangular<D>(r, origin, tri);
                bound = (b >= bound) ? b : (b == b ? bound : INFINITY);      // NaN counts as "not usable"
            }
            atomicMax(&sm.row_sum_bits, __float_as_int(bound));
        }
        __syncthreads();
        const bool triangular = __int_as_float(sm.row_sum_bits) * half_extent <= kTriangularLimit;
        for (int g = tid; g < gc_even; g += kFwdThreads) {
            float rdy[RC];
            if (g < gc) {
                float r[RF];
                raw_record(g, r);
                if (triangular) make_triangular<D>(r, origin, rdy);
                else make_ready<D>(r, origin, rdy);
            } else {
#pragma unroll
                for (int i = 0; i < RC; ++i) rdy[i] = 0.f;   // padding Gaussian: c = 0
            }
            float* dst = sm.ready + (g >> 1) * PF + (g & 1);
#pragma unroll
            for (int i = 0; i < RC; ++i) dst[2 * i] = rdy[i];
        }
        __syncthreads();
        if (tid == 0) sm.row_sum_bits = 0;          // for the next chunk (read again only after two more barriers)

        const float4* rp = reinterpret_cast<const float4*>(sm.ready);
        const int n_pairs = gc_even >> 1;
        if constexpr (D == 3) {
            if (triangular) {
#pragma unroll 2
                for (int j = 0; j < n_pairs; ++j) {
                    const float4 v0 = rp[j * 5 + 0], v1 = rp[j * 5 + 1], v2 = rp[j * 5 + 2], v3 = rp[j * 5 + 3],
                                 v4 = rp[j * 5 + 4];
                    const float2 nb0 = f2(v0.x, v0.y), nb1 = f2(v0.z, v0.w), nb2 = f2(v1.x, v1.y), c = f2(v1.z, v1.w);
                    const float2 l00 = f2(v2.x, v2.y), l10 = f2(v2.z, v2.w), l20 = f2(v3.x, v3.y), l11 = f2(v3.z, v3.w);
                    const float2 l21 = f2(v4.x, v4.y), l22 = f2(v4.z, v4.w);
#pragma unroll
                    for (int p = 0; p < P; ++p) {
                        const float2 y2 = fma2(l22, x[p][2], nb2);
                        const float2 y1 = fma2(l11, x[p][1], fma2(l21, x[p][2], nb1));
                        const float2 y0 = fma2(l00, x[p][0], fma2(l10, x[p][1], fma2(l20, x[p][2], nb0)));
                        acc[p] = fma2(c, ex2_of_minus_square(y0, y1, y2), acc[p]);
                    }
                }
            } else {
#pragma unroll 2
                for (int j = 0; j < n_pairs; ++j) {
                    const float4 v0 = rp[j * 5 + 0], v1 = rp[j * 5 + 1], v2 = rp[j * 5 + 2], v3 = rp[j * 5 + 3],
                                 v4 = rp[j * 5 + 4];
                    const float2 nm0 = f2(v0.x, v0.y), nm1 = f2(v0.z, v0.w), nm2 = f2(v1.x, v1.y), c = f2(v1.z, v1.w);
                    const float2 a00 = f2(v2.x, v2.y), a01 = f2(v2.z, v2.w), a02 = f2(v3.x, v3.y), a11 = f2(v3.z, v3.w);
                    const float2 a12 = f2(v4.x, v4.y), a22 = f2(v4.z, v4.w);
#pragma unroll
                    for (int p = 0; p < P; ++p) {
                        const float2 t0 = add2(x[p][0], nm0), t1 = add2(x[p][1], nm1), t2 = add2(x[p][2], nm2);
                        const float2 r0 = fma2(a02, t2, fma2(a01, t1, mul2(a00, t0)));
                        const float2 r1 = fma2(a12, t2, mul2(a11, t1));
                        const float2 r2 = mul2(a22, t2);
                        const float2 q = fma2(t2, r2, fma2(t1, r1, mul2(t0, r0)));
                        acc[p] = fma2(c, ex2_2(q), acc[p]);
                    }
                }
            }
        } else {
            if (triangular) {
#pragma unroll 2
                for (int j = 0; j < n_pairs; ++j) {
                    const float4 v0 = rp[j * 3 + 0], v1 = rp[j * 3 + 1], v2 = rp[j * 3 + 2];
                    const float2 nb0 = f2(v0.x, v0.y), nb1 = f2(v0.z, v0.w), c = f2(v1.x, v1.y), l00 = f2(v1.z, v1.w);
                    const float2 l10 = f2(v2.x, v2.y), l11 = f2(v2.z, v2.w);
#pragma unroll
                    for (int p = 0; p < P; ++p) {
                        const float2 y1 = fma2(l11, x[p][1], nb1);
                        const float2 y0 = fma2(l00, x[p][0], fma2(l10, x[p][1], nb0));
                        acc[p] = fma2(c, ex2_of_minus_square(y0, y1), acc[p]);
                    }
                }
            } else {
#pragma unroll 2
                for (int j = 0; j < n_pairs; ++j) {
                    const float4 v0 = rp[j * 3 + 0], v1 = rp[j * 3 + 1], v2 = rp[j * 3 + 2];
                    const float2 nm0 = f2(v0.x, v0.y), nm1 = f2(v0.z, v0.w), c = f2(v1.x, v1.y), a00 = f2(v1.z, v1.w);
                    const float2 a01 = f2(v2.x, v2.y), a11 = f2(v2.z, v2.w);
#pragma unroll
                    for (int p = 0; p < P; ++p) {
                        const float2 t0 = add2(x[p][0], nm0), t1 = add2(x[p][1], nm1);
                        const float2 r0 = fma2(a01, t1, mul2(a00, t0));
                        const float2 r1 = mul2(a11, t1);
                        const float2 q = fma2(t1, r1, mul2(t0, r0));
                        acc[p] = fma2(c, ex2_2(q), acc[p]);
                    }
                }
            }
        }
    }

    float* o = out + size_t(bl) * n_xes + n0;
#pragma unroll
    for (int p = 0; p < P; ++p) {
        const int i = tid + p * kFwdThreads;
        if (i < n_here) o[i] = acc[p].x + acc[p].y;
    }
}

// ---------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------
constexpr int kBwdUnroll = GMC_BWD_UNROLL;
constexpr int kBwdPointChunk = 16;     // points between two folds of the position-gradient partial sums
constexpr int kBwdTilePoints = 512;    // points per CTA
constexpr int kBwdRowStride = 36;      // floats per row of a warp's partial array: 32 lanes + 4 (rows stay 16-byte aligned,
                                       // float4 reads of consecutive rows fall on distinct banks)

template <int D>
struct BwdSmem {
    alignas(16) float4 pts[kBwdTilePoints * 2];                            // (x,x,y,y) (z,z,g,g) per point, x - origin
    float box_lo[D][8], box_hi[D][8];                                      // per-warp box of the tile's points
    float origin[D];                                                       // centre of that box
    float half_extent;
    int bound_bits;                                                        // largest row-sum bound of the CTA's Gaussians
    alignas(16) float partial[1];                                          // [warp][point * D + dim][kBwdRowStride]
    static constexpr size_t bytes(int n_warps) {
        return offsetof(BwdSmem, partial) + sizeof(float) * size_t(n_warps) * kBwdPointChunk * D * kBwdRowStride;
    }
};

// The Gaussians a thread owns (2 * GP of them, two per packed register pair) in the form the pair loop reads, and
// their gradient sums. Two forms (see make_ready / make_triangular of the forward pass):
//   general:     nmu = origin - mu, A = k S (symmetrised, k = -1/2 log2 e), sums over t = x - mu
//   triangular:  nmu = nb = -L^T (mu - origin), A = L (l00 l10 l20 l11 l21 l22; -k S = L L^T), sums over y = L^T t
template <int D, int GP>
struct BwdOwned {
    static constexpr int NS = D * (D + 1) / 2;
    float2 nmu[GP][D], A[GP][NS], cw2[GP];      // see above;  cw2 = w norm 2 ln 2
    float2 sa[GP], U[GP][D], M[GP][NS];         // sum a;  sum c2 t (or y);  sum c2 t t^T (or y y^T), upper triangle
};

// Largest row-sum bound (make_triangular) of the Gaussians this thread owns.
template <int D, int GP>
__device__ __forceinline__ float bwd_owned_bound(const float* __restrict__ mix, int n_components, int gbase, int tg, int TG,
                                                 const float* origin) {
    constexpr int RF = Raw<D>::kFloats;
    float bound = 0.f;
#pragma unroll
    for (int i = 0; i < 2 * GP; ++i) {
        const int g = gbase + tg + i * TG;
        if (g < n_components) {
            float r[RF], tri[ReadyCount<D>::value];
#pragma unroll
            for (int f = 0; f < RF; ++f) r[f] = __ldg(mix + size_t(g) * RF + f);
            const float b = make_triangular<D>(r, origin, tri);
            bound = (b >= bound) ? b : (b == b ? bound : INFINITY);
        }
    }
    return bound;
}

template <int D, int GP, bool TRI>
__device__ __forceinline__ void bwd_load_owned(BwdOwned<D, GP>& o, const float* __restrict__ mix, int n_components,
                                               int gbase, int tg, int TG, const float* origin) {
    constexpr int RF = Raw<D>::kFloats;
    constexpr int NS = D * (D + 1) / 2;
#pragma unroll
    for (int q = 0; q < GP; ++q) {
        float v[2][D + NS + 1];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int i = 0; i < D + NS + 1; ++i) v[h][i] = 0.f;
            const int g = gbase + tg + (2 * q + h) * TG;
            if (g < n_components) {
                float r[RF];
#pragma unroll
                for (int f = 0; f < RF; ++f) r[f] = __ldg(mix + size_t(g) * RF + f);
                if constexpr (TRI) {
                    float tri[ReadyCount<D>::value];            // nb[D], w norm, L[NS]
                    make_triangular<D>(r, origin, tri);
#pragma unroll
                    for (int d = 0; d < D; ++d) v[h][d] = tri[d];
#pragma unroll
                    for (int e = 0; e < NS; ++e) v[h][D + e] = tri[D + 1 + e];
                    v[h][D + NS] = tri[D] * (2.f * kLn2);
                } else {
                    const float w = r[0];
#pragma unroll
                    for (int d = 0; d < D; ++d) v[h][d] = origin[d] - r[1 + d];
                    const float* S = r + 1 + D;
                    float det;
                    if constexpr (D == 2) {
                        det = det2(S);
                        v[h][D + 0] = kExpScale * S[0];
                        v[h][D + 1] = kExpScale * 0.5f * (S[1] + S[2]);
                        v[h][D + 2] = kExpScale * S[3];
                    } else {
                        det = det3(S);
                        v[h][D + 0] = kExpScale * S[0];
                        v[h][D + 1] = kExpScale * 0.5f * (S[1] + S[3]);
                        v[h][D + 2] = kExpScale * 0.5f * (S[2] + S[6]);
                        v[h][D + 3] = kExpScale * S[4];
                        v[h][D + 4] = kExpScale * 0.5f * (S[5] + S[7]);
                        v[h][D + 5] = kExpScale * S[8];
                    }
                    // c2 = w * norm * (2 ln 2): folds the 1/k of "S t = (A t) / k" and the sign of d/dx
                    v[h][D + NS] = w * gauss_norm_factor<D>() * sqrtf(det) * (2.f * kLn2);
                }
            }
        }
#pragma unroll
        for (int d = 0; d < D; ++d) { o.nmu[q][d] = f2(v[0][d], v[1][d]); o.U[q][d] = f2(0.f, 0.f); }
#pragma unroll
        for (int s = 0; s < NS; ++s) { o.A[q][s] = f2(v[0][D + s], v[1][D + s]); o.M[q][s] = f2(0.f, 0.f); }
        o.cw2[q] = f2(v[0][D + NS], v[1][D + NS]);
        o.sa[q] = f2(0.f, 0.f);
    }
}

// One query point against packed pair q of the owned Gaussians.
// General form: 33 packed operations + 2 ex2 in 3D (21 + 2 in 2D); dx accumulates c2 (A t) = the position gradient.
// Triangular form: 29 packed + 2 scalar operations + 2 ex2 in 3D (18 + 2 + 2 in 2D): y = L^T x' + nb without a
// subtraction, sums over y, and dx accumulates L (c2 y) = MINUS the position gradient (the caller flips the sign).
template <int D, int GP, bool TRI>
__device__ __forceinline__ void bwd_pair(BwdOwned<D, GP>& o, int q, const float2 (&X)[3], float2 GO, float2 (&dx)[D]) {
    if constexpr (TRI && D == 3) {
        const float2 (&L)[6] = o.A[q];
        const float2 y2 = fma2(L[5], X[2], o.nmu[q][2]);
        const float2 y1 = fma2(L[3], X[1], fma2(L[4], X[2], o.nmu[q][1]));
        const float2 y0 = fma2(L[0], X[0], fma2(L[1], X[1], fma2(L[2], X[2], o.nmu[q][0])));
        const float2 a = mul2(ex2_of_minus_square(y0, y1, y2), GO);
        o.sa[q] = add2(o.sa[q], a);
        const float2 c2 = mul2(a, o.cw2[q]);
        const float2 u0 = mul2(c2, y0), u1 = mul2(c2, y1), u2 = mul2(c2, y2);
        dx[0] = fma2(L[0], u0, dx[0]);
        dx[1] = fma2(L[3], u1, fma2(L[1], u0, dx[1]));
        dx[2] = fma2(L[5], u2, fma2(L[4], u1, fma2(L[2], u0, dx[2])));
        o.U[q][0] = add2(o.U[q][0], u0);
        o.U[q][1] = add2(o.U[q][1], u1);
        o.U[q][2] = add2(o.U[q][2], u2);
        o.M[q][0] = fma2(u0, y0, o.M[q][0]);
        o.M[q][1] = fma2(u0, y1, o.M[q][1]);
        o.M[q][2] = fma2(u0, y2, o.M[q][2]);
        o.M[q][3] = fma2(u1, y1, o.M[q][3]);
        o.M[q][4] = fma2(u1, y2, o.M[q][4]);
        o.M[q][5] = fma2(u2, y2, o.M[q][5]);
    } else if constexpr (TRI) {
        const float2 (&L)[3] = o.A[q];                   // l00 l10 l11
        const float2 y1 = fma2(L[2], X[1], o.nmu[q][1]);
        const float2 y0 = fma2(L[0], X[0], fma2(L[1], X[1], o.nmu[q][0]));
        const float2 a = mul2(ex2_of_minus_square(y0, y1), GO);
        o.sa[q] = add2(o.sa[q], a);
        const float2 c2 = mul2(a, o.cw2[q]);
        const float2 u0 = mul2(c2, y0), u1 = mul2(c2, y1);
        dx[0] = fma2(L[0], u0, dx[0]);
        dx[1] = fma2(L[2], u1, fma2(L[1], u0, dx[1]));
        o.U[q][0] = add2(o.U[q][0], u0);
        o.U[q][1] = add2(o.U[q][1], u1);
        o.M[q][0] = fma2(u0, y0, o.M[q][0]);
        o.M[q][1] = fma2(u0, y1, o.M[q][1]);
        o.M[q][2] = fma2(u1, y1, o.M[q][2]);
    } else if constexpr (D == 3) {
        const float2 t0 = add2(X[0], o.nmu[q][0]), t1 = add2(X[1], o.nmu[q][1]), t2 = add2(X[2], o.nmu[q][2]);
        const float2 r0 = fma2(o.A[q][2], t2, fma2(o.A[q][1], t1, mul2(o.A[q][0], t0)));
        const float2 r1 = fma2(o.A[q][4], t2, fma2(o.A[q][3], t1, mul2(o.A[q][1], t0)));
        const float2 r2 = fma2(o.A[q][5], t2, fma2(o.A[q][4], t1, mul2(o.A[q][2], t0)));
        const float2 qq = fma2(t2, r2, fma2(t1, r1, mul2(t0, r0)));
        const float2 a = mul2(ex2_2(qq), GO);
        o.sa[q] = add2(o.sa[q], a);
        const float2 c2 = mul2(a, o.cw2[q]);
        dx[0] = fma2(c2, r0, dx[0]);
        dx[1] = fma2(c2, r1, dx[1]);
        dx[2] = fma2(c2, r2, dx[2]);
        const float2 u0 = mul2(c2, t0), u1 = mul2(c2, t1), u2 = mul2(c2, t2);
        o.U[q][0] = add2(o.U[q][0], u0);
        o.U[q][1] = add2(o.U[q][1], u1);
        o.U[q][2] = add2(o.U[q][2], u2);
        o.M[q][0] = fma2(u0, t0, o.M[q][0]);
        o.M[q][1] = fma2(u0, t1, o.M[q][1]);
        o.M[q][2] = fma2(u0, t2, o.M[q][2]);
        o.M[q][3] = fma2(u1, t1, o.M[q][3]);
        o.M[q][4] = fma2(u1, t2, o.M[q][4]);
        o.M[q][5] = fma2(u2, t2, o.M[q][5]);
    } else {
        const float2 t0 = add2(X[0], o.nmu[q][0]), t1 = add2(X[1], o.nmu[q][1]);
        const float2 r0 = fma2(o.A[q][1], t1, mul2(o.A[q][0], t0));
        const float2 r1 = fma2(o.A[q][2], t1, mul2(o.A[q][1], t0));
        const float2 qq = fma2(t1, r1, mul2(t0, r0));
        const float2 a = mul2(ex2_2(qq), GO);
        o.sa[q] = add2(o.sa[q], a);
        const float2 c2 = mul2(a, o.cw2[q]);
        dx[0] = fma2(c2, r0, dx[0]);
        dx[1] = fma2(c2, r1, dx[1]);
        const float2 u0 = mul2(c2, t0), u1 = mul2(c2, t1);
        o.U[q][0] = add2(o.U[q][0], u0);
        o.U[q][1] = add2(o.U[q][1], u1);
        o.M[q][0] = fma2(u0, t0, o.M[q][0]);
        o.M[q][1] = fma2(u0, t1, o.M[q][1]);
        o.M[q][2] = fma2(u1, t1, o.M[q][2]);
    }
}

// Finishes the per-Gaussian gradient from the sums, one atomic per value (other CTAs and point slices add theirs).
// Triangular form: with Z = L^-1 the sums over y turn into the sums over t: sum c2 t = Z^T U, sum c2 t t^T = Z^T M Z,
// and d/d mu = S sum(c t) = L U.
template <int D, int GP, bool TRI>
__device__ __forceinline__ void bwd_store_owned(const BwdOwned<D, GP>& o, const float* __restrict__ mix,
                                                float* __restrict__ grad_mix, int n_components, int gbase, int tg,
                                                int TG) {
    constexpr int RF = Raw<D>::kFloats;
    constexpr int NS = D * (D + 1) / 2;
#pragma unroll
    for (int q = 0; q < GP; ++q) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int g = gbase + tg + (2 * q + h) * TG;
            if (g >= n_components) continue;
            const float sa_h = h ? o.sa[q].y : o.sa[q].x;
            float Uh[D], Mh[NS];
#pragma unroll
            for (int d = 0; d < D; ++d) Uh[d] = h ? o.U[q][d].y : o.U[q][d].x;
#pragma unroll
            for (int s = 0; s < NS; ++s) Mh[s] = h ? o.M[q][s].y : o.M[q][s].x;
            const float* r = mix + size_t(g) * RF;
            const float w = __ldg(r);
            float S[D * D];
#pragma unroll
            for (int i = 0; i < D * D; ++i) S[i] = __ldg(r + 1 + D + i);
            float* go = grad_mix + size_t(g) * RF;
            constexpr float inv2ln2 = 1.f / (2.f * kLn2);
            float det, cof[D * D];
            if constexpr (D == 2) {
                det = det2(S);
                cof[0] = S[3]; cof[1] = -S[2]; cof[2] = -S[1]; cof[3] = S[0];
            } else {
                det = det3(S);
                cof[0] = S[4] * S[8] - S[5] * S[7];
                cof[1] = -(S[3] * S[8] - S[5] * S[6]);
                cof[2] = S[3] * S[7] - S[4] * S[6];
                cof[3] = -(S[1] * S[8] - S[2] * S[7]);
                cof[4] = S[0] * S[8] - S[2] * S[6];
                cof[5] = -(S[0] * S[7] - S[1] * S[6]);
                cof[6] = S[1] * S[5] - S[2] * S[4];
                cof[7] = -(S[0] * S[5] - S[2] * S[3]);
                cof[8] = S[0] * S[4] - S[1] * S[3];
            }
            const float root = sqrtf(det);
            const float norm = gauss_norm_factor<D>() * root;
            atomicAdd(go, norm * sa_h);
            float Mfull[D * D];                      // sum c2 t t^T
            if constexpr (TRI) {
                float Lh[NS];
#pragma unroll
                for (int s = 0; s < NS; ++s) Lh[s] = h ? o.A[q][s].y : o.A[q][s].x;
                float Lm[D][D], Z[D][D], My[D][D];   // L (lower), its inverse, the symmetric sum over y
#pragma unroll
                for (int i = 0; i < D; ++i)
#pragma unroll
                    for (int j = 0; j < D; ++j) { Lm[i][j] = 0.f; Z[i][j] = 0.f; }
                if constexpr (D == 2) {
                    Lm[0][0] = Lh[0]; Lm[1][0] = Lh[1]; Lm[1][1] = Lh[2];
                    Z[0][0] = 1.f / Lh[0]; Z[1][1] = 1.f / Lh[2];
                    Z[1][0] = -Lh[1] * Z[0][0] * Z[1][1];
                } else {
                    Lm[0][0] = Lh[0]; Lm[1][0] = Lh[1]; Lm[2][0] = Lh[2]; Lm[1][1] = Lh[3]; Lm[2][1] = Lh[4]; Lm[2][2] = Lh[5];
                    Z[0][0] = 1.f / Lh[0]; Z[1][1] = 1.f / Lh[3]; Z[2][2] = 1.f / Lh[5];
                    Z[1][0] = -Lh[1] * Z[0][0] * Z[1][1];
                    Z[2][1] = -Lh[4] * Z[1][1] * Z[2][2];
                    Z[2][0] = (Lh[1] * Lh[4] - Lh[2] * Lh[3]) * Z[0][0] * Z[1][1] * Z[2][2];
                }
                int s_idx = 0;
#pragma unroll
                for (int i = 0; i < D; ++i)
#pragma unroll
                    for (int j = i; j < D; ++j) { My[i][j] = Mh[s_idx]; My[j][i] = Mh[s_idx]; ++s_idx; }
                // d/d mu = L U
#pragma unroll
                for (int i = 0; i < D; ++i) {
                    float acc = 0.f;
#pragma unroll
                    for (int j = 0; j <= i; ++j) acc = fmaf(Lm[i][j], Uh[j], acc);
                    atomicAdd(go + 1 + i, acc);
                }
                float B[D][D];                        // My Z
#pragma unroll
                for (int i = 0; i < D; ++i)
#pragma unroll
                    for (int j = 0; j < D; ++j) {
                        float acc = 0.f;
#pragma unroll
                        for (int m = j; m < D; ++m) acc = fmaf(My[i][m], Z[m][j], acc);
                        B[i][j] = acc;
                    }
#pragma unroll
                for (int i = 0; i < D; ++i)
#pragma unroll
                    for (int j = 0; j < D; ++j) {
                        float acc = 0.f;
#pragma unroll
                        for (int m = i; m < D; ++m) acc = fmaf(Z[m][i], B[m][j], acc);
                        Mfull[i * D + j] = acc;
                    }
            } else {
                // d/d mu = S * sum(c t);  U holds sum(c2 t) with c2 = c * 2 ln 2
#pragma unroll
                for (int i = 0; i < D; ++i) {
                    float s = 0.f;
#pragma unroll
                    for (int j = 0; j < D; ++j) s = fmaf(0.5f * (S[i * D + j] + S[j * D + i]), Uh[j] * inv2ln2, s);
                    atomicAdd(go + 1 + i, s);
                }
                int s_idx = 0;
#pragma unroll
                for (int i = 0; i < D; ++i)
#pragma unroll
                    for (int j = i; j < D; ++j) {
                        Mfull[i * D + j] = Mh[s_idx];
                        Mfull[j * D + i] = Mh[s_idx];
                        ++s_idx;
                    }
            }
            // d/d S = -1/2 sum(c t t^T) + (w sum(a) factor / (2 sqrt(det))) cof(S)
            const float gdet = w * sa_h * gauss_norm_factor<D>() / (2.f * root);
#pragma unroll
            for (int i = 0; i < D * D; ++i)
                atomicAdd(go + 1 + D + i, fmaf(-0.5f * inv2ln2, Mfull[i], gdet * cof[i]));
        }
    }
}

// GP = packed Gaussian pairs per thread (a thread owns 2 * GP Gaussians: g = base + tg + (2 q + h) * TG).
// THREADS = CTA size. TG threads lie along the Gaussian axis (a multiple of 32, so a warp never straddles two point
// slices); the THREADS / TG slices take contiguous blocks of the tile's points.
// A warp is self-contained after the staging barrier: it walks its points in chunks of 16, every lane writes its D
// partial position-gradient sums per point into the warp's own shared rows, the warp folds the rows (one lane per
// (point, dim) row, float4 reads) and adds the results to global memory. No CTA barrier in the loop.
template <int D, int GP, int THREADS>
__global__ void __launch_bounds__(THREADS, GMC_BWD_MINB)
eval_backward_kernel(const float* __restrict__ grad_out, const float* __restrict__ mixture,
                     const float* __restrict__ xes, float* __restrict__ grad_mixture,
                     float* __restrict__ grad_xes, int n_layers, int n_components, int n_batch_xes,
                     int n_layers_xes, int n_xes, int tg_threads, int n_point_tiles, int n_gauss_chunks) {
    constexpr int RF = Raw<D>::kFloats;
    constexpr int ROWS = kBwdPointChunk * D;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    BwdSmem<D>& sm = *reinterpret_cast<BwdSmem<D>*>(smem_bytes);

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    int bid = blockIdx.x;
    const int gchunk = bid % n_gauss_chunks;
    bid /= n_gauss_chunks;
    const int ptile = bid % n_point_tiles;
    const int bl = bid / n_point_tiles;
    const int b = bl / n_layers;
    const int l = bl - b * n_layers;
    const int bx = n_batch_xes == 1 ? 0 : b;
    const int lx = n_layers_xes == 1 ? 0 : l;

    const int TG = tg_threads;                 // threads along the Gaussian axis (32, 64 or 128)
    const int TP = THREADS / TG;               // point slices
    const int tg = tid % TG;
    const int slice = tid / TG;

    const int n0 = ptile * kBwdTilePoints;
    const int n_here = min(kBwdTilePoints, n_xes - n0);
    const size_t xes_row = (size_t(bx) * n_layers_xes + lx) * size_t(n_xes);

    // ---- stage points: (x - origin, grad_out), every value duplicated for the packed pair loop; origin = centre of the
    //      box of the tile's points ----
    {
        constexpr int PER = (kBwdTilePoints + THREADS - 1) / THREADS;
        float px[PER], py[PER], pz[PER], go[PER];
        float lo[D], hi[D];
#pragma unroll
        for (int d = 0; d < D; ++d) { lo[d] = INFINITY; hi[d] = -INFINITY; }
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = tid + k * THREADS;
            px[k] = py[k] = pz[k] = go[k] = 0.f;
            if (i < n_here) {
                const float* xp = xes + (xes_row + n0 + i) * D;
                go[k] = __ldg(grad_out + size_t(bl) * n_xes + n0 + i);
                px[k] = __ldg(xp);
                py[k] = __ldg(xp + 1);
                if constexpr (D == 3) pz[k] = __ldg(xp + 2);
                lo[0] = fminf(lo[0], px[k]); hi[0] = fmaxf(hi[0], px[k]);
                lo[1] = fminf(lo[1], py[k]); hi[1] = fmaxf(hi[1], py[k]);
                if constexpr (D == 3) { lo[2] = fminf(lo[2], pz[k]); hi[2] = fmaxf(hi[2], pz[k]); }
            }
        }
#pragma unroll
        for (int d = 0; d < D; ++d) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                lo[d] = fminf(lo[d], __shfl_xor_sync(0xffffffffu, lo[d], o));
                hi[d] = fmaxf(hi[d], __shfl_xor_sync(0xffffffffu, hi[d], o));
            }
            if (lane == 0) { sm.box_lo[d][tid >> 5] = lo[d]; sm.box_hi[d][tid >> 5] = hi[d]; }
        }
        __syncthreads();
        if (tid == 0) {
            float half = 0.f;
#pragma unroll
            for (int d = 0; d < D; ++d) {
                float l = sm.box_lo[d][0], h = sm.box_hi[d][0];
                for (int w = 1; w < THREADS / 32; ++w) { l = fminf(l, sm.box_lo[d][w]); h = fmaxf(h, sm.box_hi[d][w]); }
                const float centre = 0.5f * l + 0.5f * h;
                sm.origin[d] = centre;
                half = fmaxf(half, fmaxf(h - centre, centre - l));
            }
            sm.half_extent = half;
            sm.bound_bits = 0;
        }
        __syncthreads();
        const float ox = sm.origin[0], oy = sm.origin[1], oz = D == 3 ? sm.origin[D - 1] : 0.f;
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = tid + k * THREADS;
            if (i < kBwdTilePoints) {
                const bool live = i < n_here;
                const float x0 = live ? px[k] - ox : 0.f, x1 = live ? py[k] - oy : 0.f, x2 = live ? pz[k] - oz : 0.f;
                sm.pts[2 * i] = make_float4(x0, x0, x1, x1);
                sm.pts[2 * i + 1] = make_float4(x2, x2, go[k], go[k]);
            }
        }
    }
    float origin[D];
#pragma unroll
    for (int d = 0; d < D; ++d) origin[d] = sm.origin[d];

    const float* mix = mixture + size_t(bl) * n_components * RF;
    const int gbase = gchunk * TG * GP * 2;
    // ---- which pair loop: the largest row-sum bound of the CTA's Gaussians against the extent of its points ----
    atomicMax(&sm.bound_bits, __float_as_int(bwd_owned_bound<D, GP>(mix, n_components, gbase, tg, TG, origin)));
    __syncthreads();
    const bool triangular = __int_as_float(sm.bound_bits) * sm.half_extent <= kTriangularLimitBackward;

    const bool need_gx = grad_xes != nullptr;
    const int part = (tid >> 5) * ROWS * kBwdRowStride;     // first float of this warp's rows in sm.partial
    constexpr int PPI = GMC_BWD_PPI;   // points in flight per loop iteration (independent dependency chains)
    const int per_slice = kBwdTilePoints / TP;
    const int p_end = min(n_here, (slice + 1) * per_slice);

    auto run = [&](auto form) {
        constexpr bool TRI = decltype(form)::value;
        BwdOwned<D, GP> own;
        bwd_load_owned<D, GP, TRI>(own, mix, n_components, gbase, tg, TG, origin);
        for (int c0 = slice * per_slice; c0 < p_end; c0 += kBwdPointChunk) {
#pragma unroll kBwdUnroll
            for (int pp0 = 0; pp0 < kBwdPointChunk; pp0 += PPI) {
                float2 X[PPI][3], GO[PPI], dx[PPI][D];
#pragma unroll
                for (int k = 0; k < PPI; ++k) {
                    const float4 pa = sm.pts[2 * (c0 + pp0 + k)];
                    const float4 pb = sm.pts[2 * (c0 + pp0 + k) + 1];
                    X[k][0] = f2(pa.x, pa.y); X[k][1] = f2(pa.z, pa.w); X[k][2] = f2(pb.x, pb.y);
                    GO[k] = f2(pb.z, pb.w);
#pragma unroll
                    for (int d = 0; d < D; ++d) dx[k][d] = f2(0.f, 0.f);
                }
#pragma unroll
                for (int q = 0; q < GP; ++q) {
#pragma unroll
                    for (int k = 0; k < PPI; ++k) bwd_pair<D, GP, TRI>(own, q, X[k], GO[k], dx[k]);
                }
                if (need_gx) {
#pragma unroll
                    for (int k = 0; k < PPI; ++k)
#pragma unroll
                        for (int d = 0; d < D; ++d) {
                            // the triangular loop accumulates minus the gradient
                            const float v = TRI ? (-dx[k][d].x) - dx[k][d].y : dx[k][d].x + dx[k][d].y;
                            sm.partial[part + ((pp0 + k) * D + d) * kBwdRowStride + lane] = v;
                        }
                }
            }
            if (need_gx) {
                __syncwarp();
                // rows 0..31: one lane per row, 32 values each
                float* gx = grad_xes + (xes_row + n0 + c0) * D;
                {
                    const float4* src = reinterpret_cast<const float4*>(sm.partial + part + lane * kBwdRowStride);
                    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float4 v = src[i];
                        s0 += v.x; s1 += v.y; s2 += v.z; s3 += v.w;
                    }
                    if (c0 + lane / D < n_here) atomicAdd(gx + lane, (s0 + s1) + (s2 + s3));
                }
                if constexpr (ROWS > 32) {
                    // rows 32..47: two lanes per row, 16 values each
                    const int row = 32 + (lane & 15);
                    const float4* src = reinterpret_cast<const float4*>(sm.partial + part + row * kBwdRowStride + (lane >> 4) * 16);
                    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float4 v = src[i];
                        s0 += v.x; s1 += v.y; s2 += v.z; s3 += v.w;
                    }
                    float s = (s0 + s1) + (s2 + s3);
                    s += __shfl_xor_sync(0xffffffffu, s, 16);
                    if (lane < 16 && c0 + row / D < n_here) atomicAdd(gx + row, s);
                }
                __syncwarp();
            }
        }
        if (grad_mixture != nullptr)
            bwd_store_owned<D, GP, TRI>(own, mix, grad_mixture + size_t(bl) * n_components * RF, n_components, gbase, tg, TG);
    };
    if (triangular) run(std::true_type{});
    else run(std::false_type{});
}

template <typename K>
int set_smem(K kernel, size_t bytes) {
    if (bytes > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)));
    return GMC_OK;
}

int check_eval_args(int n_batch, int n_layers, int n_components, int n_dims, int n_batch_xes, int n_layers_xes,
                    int n_xes) {
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_batch <= 0 || n_layers <= 0 || n_components <= 0 || n_xes <= 0) return GMC_ERR_BAD_DIMS;
    if (n_batch_xes != 1 && n_batch_xes != n_batch) return GMC_ERR_BAD_BROADCAST;
    if (n_layers_xes != 1 && n_layers_xes != n_layers) return GMC_ERR_BAD_BROADCAST;
    return GMC_OK;
}

template <int D, int P>
int launch_forward(const float* mixture, const float* xes, float* out, int n_batch, int n_layers, int n_components,
                   int n_batch_xes, int n_layers_xes, int n_xes, cudaStream_t stream, int lose_copy = 0) {
    constexpr int TILE = kFwdThreads * P;
    const long long tiles = (n_xes + TILE - 1) / TILE;
    const long long blocks = tiles * n_batch * n_layers;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    auto kernel = eval_forward_kernel<D, P>;
    const size_t smem = sizeof(FwdSmem<D, P>);
    if (int s = set_smem(kernel, smem)) return s;
    kernel<<<unsigned(blocks), kFwdThreads, smem, stream>>>(mixture, xes, out, n_layers, n_components, n_batch_xes,
                                                            n_layers_xes, n_xes, int(tiles), lose_copy);
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

template <int D, int GP, int THREADS>
int launch_backward(const float* grad_out, const float* mixture, const float* xes, float* grad_mixture,
                    float* grad_xes, int n_batch, int n_layers, int n_components, int n_batch_xes, int n_layers_xes,
                    int n_xes, int tg, cudaStream_t stream) {
    const long long ptiles = (n_xes + kBwdTilePoints - 1) / kBwdTilePoints;
    const long long gchunks = (n_components + tg * GP * 2 - 1) / (tg * GP * 2);
    const long long blocks = ptiles * gchunks * n_batch * n_layers;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    auto kernel = eval_backward_kernel<D, GP, THREADS>;
    const size_t smem = BwdSmem<D>::bytes(THREADS / 32);
    if (int s = set_smem(kernel, smem)) return s;
    kernel<<<unsigned(blocks), THREADS, smem, stream>>>(grad_out, mixture, xes, grad_mixture, grad_xes, n_layers,
                                                        n_components, n_batch_xes, n_layers_xes, n_xes, tg,
                                                        int(ptiles), int(gchunks));
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

}  // namespace
}  // namespace gmc

GMC_DEFINE_TU_CHECK_READER(eval_inversed)

extern "C" int gmc_eval_inversed_forward(const float* mixture, const float* xes, float* out, int n_batch, int n_layers,
                                         int n_components, int n_dims, int n_batch_xes, int n_layers_xes, int n_xes,
                                         void* stream) {
    using namespace gmc;
    if (int s = check_eval_args(n_batch, n_layers, n_components, n_dims, n_batch_xes, n_layers_xes, n_xes)) return s;
    if (!mixture || !xes || !out) return GMC_ERR_NULL_POINTER;
    cudaStream_t st = as_stream(stream);
    // points per thread: keep enough CTAs in flight for small problems
    const long long pairs_rows = (long long)n_batch * n_layers * n_xes;
    const bool small = pairs_rows < 148LL * 4 * kFwdThreads * kFwdPoints;
    if (n_dims == 2) {
        return small ? launch_forward<2, 1>(mixture, xes, out, n_batch, n_layers, n_components, n_batch_xes, n_layers_xes, n_xes, st)
                     : launch_forward<2, kFwdPoints>(mixture, xes, out, n_batch, n_layers, n_components, n_batch_xes, n_layers_xes, n_xes, st);
    }
    return small ? launch_forward<3, 1>(mixture, xes, out, n_batch, n_layers, n_components, n_batch_xes, n_layers_xes, n_xes, st)
                 : launch_forward<3, kFwdPoints>(mixture, xes, out, n_batch, n_layers, n_components, n_batch_xes, n_layers_xes, n_xes, st);
}

extern "C" int gmc_debug_eval_forward_lost_copy(const float* mixture, const float* xes, float* out, int n_batch,
                                                int n_layers, int n_components, int n_dims, int n_batch_xes,
                                                int n_layers_xes, int n_xes, void* stream) {
    using namespace gmc;
    if (int s = check_eval_args(n_batch, n_layers, n_components, n_dims, n_batch_xes, n_layers_xes, n_xes)) return s;
    if (!mixture || !xes || !out) return GMC_ERR_NULL_POINTER;
    cudaStream_t st = as_stream(stream);
    if (n_dims == 2)
        return launch_forward<2, 1>(mixture, xes, out, n_batch, n_layers, n_components, n_batch_xes, n_layers_xes, n_xes, st, 1);
    return launch_forward<3, 1>(mixture, xes, out, n_batch, n_layers, n_components, n_batch_xes, n_layers_xes, n_xes, st, 1);
}

extern "C" int gmc_eval_inversed_backward(const float* grad_out, const float* mixture, const float* xes,
                                          float* grad_mixture, float* grad_xes, int n_batch, int n_layers,
                                          int n_components, int n_dims, int n_batch_xes, int n_layers_xes, int n_xes,
                                          void* stream) {
    using namespace gmc;
    if (int s = check_eval_args(n_batch, n_layers, n_components, n_dims, n_batch_xes, n_layers_xes, n_xes)) return s;
    if (!grad_out || !mixture || !xes) return GMC_ERR_NULL_POINTER;
    cudaStream_t st = as_stream(stream);
    const size_t rf = size_t(1 + n_dims + n_dims * n_dims);
    if (grad_mixture)
        GMC_CUDA_TRY(cudaMemsetAsync(grad_mixture, 0, sizeof(float) * rf * n_batch * n_layers * n_components, st));
    if (grad_xes)
        GMC_CUDA_TRY(cudaMemsetAsync(grad_xes, 0, sizeof(float) * size_t(n_batch_xes) * n_layers_xes * n_xes * n_dims, st));
    if (!grad_mixture && !grad_xes) return GMC_OK;

    // packed Gaussian pairs per thread (2, 4 or 8 Gaussians), CTA size and threads along the Gaussian axis
    int gp, tg;
    if (n_components >= 384) { gp = GMC_BWD_GP_LARGE; tg = GMC_BWD_THREADS_LARGE; }
    else if (n_components > 128) { gp = 1; tg = 128; }
    else if (n_components > 64) { gp = 1; tg = 64; }
    else { gp = 1; tg = 32; }
#define GMC_BWD(D_, GP_, T_) launch_backward<D_, GP_, T_>(grad_out, mixture, xes, grad_mixture, grad_xes, n_batch, \
                                                          n_layers, n_components, n_batch_xes, n_layers_xes, n_xes, tg, st)
    if (n_dims == 2) return gp > 1 ? GMC_BWD(2, GMC_BWD_GP_LARGE, GMC_BWD_THREADS_LARGE) : GMC_BWD(2, 1, 128);
    return gp > 1 ? GMC_BWD(3, GMC_BWD_GP_LARGE, GMC_BWD_THREADS_LARGE) : GMC_BWD(3, 1, 128);
#undef GMC_BWD
}
