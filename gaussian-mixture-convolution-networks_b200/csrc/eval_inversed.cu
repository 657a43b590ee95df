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
//            so the pair loop is   t = x - mu;  q = t^T A t;  acc += c * ex2(q)   (FMA pipe + one MUFU).
//            Every thread keeps P query points in registers and reads Gaussians as broadcast float4.
//  backward: a CTA owns one (batch, layer), a tile of query points and a chunk of Gaussians. Every thread
//            keeps GQ Gaussians and their 1 + D + D(D+1)/2 gradient sums in registers and streams the
//            tile's points (x, grad_out) from shared memory, so the per-Gaussian sums need no cross-lane
//            traffic in the pair loop. The per-point position gradient is what crosses lanes: each thread
//            writes its D partial sums to a padded shared array and the CTA folds them once per 16 points.
//            CTA totals go to global memory with one atomic per value.
#include "common.cuh"

namespace gmc {
namespace {

constexpr int kFwdThreads = 128;
constexpr int kFwdChunk = 256;   // Gaussians staged per shared-memory chunk

template <int D>
struct Raw {
    static constexpr int kFloats = 1 + D + D * D;
};

// ---------------------------------------------------------------------------------------------
// "ready" records: 2D = float4 (mx, my, c, a00) + float2 (a01, a11);
//                  3D = float4 (mx, my, mz, c) + float4 (a00, a01, a02, a11) + float2 (a12, a22),
// with a_ij = k (S_ij + S_ji) for i != j, a_ii = k S_ii, k = -1/2 log2(e).
// ---------------------------------------------------------------------------------------------
constexpr float kExpScale = -0.5f * kLog2e;

__device__ __forceinline__ float det2(const float* S) { return S[0] * S[3] - S[1] * S[2]; }
__device__ __forceinline__ float det3(const float* S) {
    return S[0] * (S[4] * S[8] - S[5] * S[7]) - S[1] * (S[3] * S[8] - S[5] * S[6]) +
           S[2] * (S[3] * S[7] - S[4] * S[6]);
}

__device__ __forceinline__ void make_ready(const float* r, float4& a, float2& b) {
    const float* S = r + 3;
    const float c = r[0] * kInv2Pi * sqrtf(det2(S));
    a = make_float4(r[1], r[2], c, kExpScale * S[0]);
    b = make_float2(kExpScale * (S[1] + S[2]), kExpScale * S[3]);
}
__device__ __forceinline__ void make_ready(const float* r, float4& a, float4& b, float2& c2) {
    const float* S = r + 4;
    const float c = r[0] * kInv2Pi15 * sqrtf(det3(S));
    a = make_float4(r[1], r[2], r[3], c);
    b = make_float4(kExpScale * S[0], kExpScale * (S[1] + S[3]), kExpScale * (S[2] + S[6]), kExpScale * S[4]);
    c2 = make_float2(kExpScale * (S[5] + S[7]), kExpScale * S[8]);
}

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
template <int D, int P>
struct FwdSmem {
    static constexpr int kTile = kFwdThreads * P;
    alignas(16) float raw[kFwdChunk * Raw<D>::kFloats];
    alignas(16) float4 ra[kFwdChunk];
    alignas(16) float4 rb[D == 3 ? kFwdChunk : 1];
    alignas(16) float2 rc[kFwdChunk];
    alignas(16) float xs[kTile * D];
    alignas(8) uint64_t bar;
};

template <int D, int P>
__global__ void __launch_bounds__(kFwdThreads)
eval_forward_kernel(const float* __restrict__ mixture, const float* __restrict__ xes, float* __restrict__ out,
                    int n_layers, int n_components, int n_batch_xes, int n_layers_xes, int n_xes,
                    int tiles_per_mixture) {
    constexpr int RF = Raw<D>::kFloats;
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

    float x[P][D];
    float acc[P];
#pragma unroll
    for (int p = 0; p < P; ++p) {
#pragma unroll
        for (int d = 0; d < D; ++d) x[p][d] = sm.xs[(tid + p * kFwdThreads) * D + d];
        acc[p] = 0.f;
    }

    const float* mix = mixture + size_t(bl) * n_components * RF;
    unsigned phase = 0;
    bool ok = true;
    for (int g0 = 0; g0 < n_components; g0 += kFwdChunk) {
        const int gc = min(kFwdChunk, n_components - g0);
        const float* chunk = mix + size_t(g0) * RF;
        const unsigned bytes = unsigned(gc) * RF * 4u;
        const bool bulk = ((reinterpret_cast<uintptr_t>(chunk) & 15u) == 0) && ((bytes & 15u) == 0);
        if (g0 > 0) __syncthreads();   // everyone is done reading the previous chunk
        if (bulk) {
            if (tid == 0) {
                fence_proxy_async();
                mbar_arrive_expect_tx(&sm.bar, bytes);
                bulk_copy_g2s(sm.raw, chunk, bytes, &sm.bar);
            }
            ok = mbar_wait_bounded(&sm.bar, phase);
            phase ^= 1u;
            // a CTA-wide decision keeps the barriers below convergent
            if (__syncthreads_or(!ok)) return;
            for (int g = tid; g < gc; g += kFwdThreads) {
                if constexpr (D == 2) make_ready(sm.raw + g * RF, sm.ra[g], sm.rc[g]);
                else make_ready(sm.raw + g * RF, sm.ra[g], sm.rb[g], sm.rc[g]);
            }
        } else {
            for (int g = tid; g < gc; g += kFwdThreads) {
                float r[RF];
#pragma unroll
                for (int i = 0; i < RF; ++i) r[i] = __ldg(chunk + g * RF + i);
                if constexpr (D == 2) make_ready(r, sm.ra[g], sm.rc[g]);
                else make_ready(r, sm.ra[g], sm.rb[g], sm.rc[g]);
            }
        }
        __syncthreads();

        if constexpr (D == 3) {
#pragma unroll 2
            for (int g = 0; g < gc; ++g) {
                const float4 ga = sm.ra[g];
                const float4 gb = sm.rb[g];
                const float2 gcv = sm.rc[g];
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    const float t0 = x[p][0] - ga.x;
                    const float t1 = x[p][1] - ga.y;
                    const float t2 = x[p][2] - ga.z;
                    const float r0 = fmaf(gb.z, t2, fmaf(gb.y, t1, gb.x * t0));
                    const float r1 = fmaf(gcv.x, t2, gb.w * t1);
                    const float r2 = gcv.y * t2;
                    const float q = fmaf(t2, r2, fmaf(t1, r1, t0 * r0));
                    acc[p] = fmaf(ga.w, ex2_approx(q), acc[p]);
                }
            }
        } else {
#pragma unroll 2
            for (int g = 0; g < gc; ++g) {
                const float4 ga = sm.ra[g];
                const float2 gb = sm.rc[g];
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    const float t0 = x[p][0] - ga.x;
                    const float t1 = x[p][1] - ga.y;
                    const float r0 = fmaf(gb.x, t1, ga.w * t0);
                    const float r1 = gb.y * t1;
                    const float q = fmaf(t1, r1, t0 * r0);
                    acc[p] = fmaf(ga.z, ex2_approx(q), acc[p]);
                }
            }
        }
    }

    float* o = out + size_t(bl) * n_xes + n0;
#pragma unroll
    for (int p = 0; p < P; ++p) {
        const int i = tid + p * kFwdThreads;
        if (i < n_here) o[i] = acc[p];
    }
}

// ---------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------
constexpr int kBwdThreads = 128;
constexpr int kBwdPointChunk = 16;     // points folded per shared-memory round
constexpr int kBwdTilePoints = 512;    // points per CTA

template <int D>
struct BwdSmem {
    alignas(16) float4 pts[kBwdTilePoints];                                // x, y, (z), grad_out
    alignas(16) float partial[kBwdPointChunk * D * (kBwdThreads + 4)];      // [point][dim][thread] (+pad)
};

template <int D, int GQ>
__global__ void __launch_bounds__(kBwdThreads)
eval_backward_kernel(const float* __restrict__ grad_out, const float* __restrict__ mixture,
                     const float* __restrict__ xes, float* __restrict__ grad_mixture,
                     float* __restrict__ grad_xes, int n_layers, int n_components, int n_batch_xes,
                     int n_layers_xes, int n_xes, int tg_threads, int n_point_tiles, int n_gauss_chunks) {
    constexpr int RF = Raw<D>::kFloats;
    constexpr int NS = D * (D + 1) / 2;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    BwdSmem<D>& sm = *reinterpret_cast<BwdSmem<D>*>(smem_bytes);

    const int tid = threadIdx.x;
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
    const int TP = kBwdThreads / TG;           // point slices
    const int tg = tid % TG;
    const int slice = tid / TG;
    const int TGP = TG + 4;                    // padded row length of the partial array

    const int n0 = ptile * kBwdTilePoints;
    const int n_here = min(kBwdTilePoints, n_xes - n0);
    const size_t xes_row = (size_t(bx) * n_layers_xes + lx) * size_t(n_xes);

    // ---- stage points: (x, grad_out) ----
    for (int i = tid; i < kBwdTilePoints; i += kBwdThreads) {
        float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n_here) {
            const float* xp = xes + (xes_row + n0 + i) * D;
            const float go = __ldg(grad_out + size_t(bl) * n_xes + n0 + i);
            if constexpr (D == 3) p = make_float4(__ldg(xp), __ldg(xp + 1), __ldg(xp + 2), go);
            else p = make_float4(__ldg(xp), __ldg(xp + 1), 0.f, go);
        }
        sm.pts[i] = p;
    }

    // ---- my Gaussians, in ready form for the backward pair loop ----
    float mu[GQ][D], A[GQ][NS], cw2[GQ];
    float sa[GQ], U[GQ][D], M[GQ][NS];
    const float* mix = mixture + size_t(bl) * n_components * RF;
    const int gbase = gchunk * TG * GQ;
#pragma unroll
    for (int q = 0; q < GQ; ++q) {
        const int g = gbase + tg + q * TG;
        sa[q] = 0.f;
#pragma unroll
        for (int d = 0; d < D; ++d) { U[q][d] = 0.f; mu[q][d] = 0.f; }
#pragma unroll
        for (int s = 0; s < NS; ++s) { M[q][s] = 0.f; A[q][s] = 0.f; }
        cw2[q] = 0.f;
        if (g < n_components) {
            const float* r = mix + size_t(g) * RF;
            const float w = __ldg(r);
#pragma unroll
            for (int d = 0; d < D; ++d) mu[q][d] = __ldg(r + 1 + d);
            float S[D * D];
#pragma unroll
            for (int i = 0; i < D * D; ++i) S[i] = __ldg(r + 1 + D + i);
            float det;
            if constexpr (D == 2) {
                det = det2(S);
                A[q][0] = kExpScale * S[0];
                A[q][1] = kExpScale * 0.5f * (S[1] + S[2]);
                A[q][2] = kExpScale * S[3];
            } else {
                det = det3(S);
                A[q][0] = kExpScale * S[0];
                A[q][1] = kExpScale * 0.5f * (S[1] + S[3]);
                A[q][2] = kExpScale * 0.5f * (S[2] + S[6]);
                A[q][3] = kExpScale * S[4];
                A[q][4] = kExpScale * 0.5f * (S[5] + S[7]);
                A[q][5] = kExpScale * S[8];
            }
            // c2 = w * norm * (2 ln 2): folds the 1/k of "S t = (A t) / k" and the sign of d/dx
            cw2[q] = w * gauss_norm_factor<D>() * sqrtf(det) * (2.f * kLn2);
        }
    }
    __syncthreads();

    const bool need_gx = grad_xes != nullptr;
    for (int c0 = 0; c0 < n_here; c0 += kBwdPointChunk) {
        for (int pp = slice; pp < kBwdPointChunk; pp += TP) {
            const float4 pt = sm.pts[c0 + pp];
            float dx[D];
#pragma unroll
            for (int d = 0; d < D; ++d) dx[d] = 0.f;
#pragma unroll
            for (int q = 0; q < GQ; ++q) {
                if constexpr (D == 3) {
                    const float t0 = pt.x - mu[q][0], t1 = pt.y - mu[q][1], t2 = pt.z - mu[q][2];
                    const float r0 = fmaf(A[q][2], t2, fmaf(A[q][1], t1, A[q][0] * t0));
                    const float r1 = fmaf(A[q][4], t2, fmaf(A[q][3], t1, A[q][1] * t0));
                    const float r2 = fmaf(A[q][5], t2, fmaf(A[q][4], t1, A[q][2] * t0));
                    const float qq = fmaf(t2, r2, fmaf(t1, r1, t0 * r0));
                    const float a = ex2_approx(qq) * pt.w;
                    sa[q] += a;
                    const float c2 = a * cw2[q];
                    dx[0] = fmaf(c2, r0, dx[0]);
                    dx[1] = fmaf(c2, r1, dx[1]);
                    dx[2] = fmaf(c2, r2, dx[2]);
                    const float u0 = c2 * t0, u1 = c2 * t1, u2 = c2 * t2;
                    U[q][0] += u0; U[q][1] += u1; U[q][2] += u2;
                    M[q][0] = fmaf(u0, t0, M[q][0]);
                    M[q][1] = fmaf(u0, t1, M[q][1]);
                    M[q][2] = fmaf(u0, t2, M[q][2]);
                    M[q][3] = fmaf(u1, t1, M[q][3]);
                    M[q][4] = fmaf(u1, t2, M[q][4]);
                    M[q][5] = fmaf(u2, t2, M[q][5]);
                } else {
                    const float t0 = pt.x - mu[q][0], t1 = pt.y - mu[q][1];
                    const float r0 = fmaf(A[q][1], t1, A[q][0] * t0);
                    const float r1 = fmaf(A[q][2], t1, A[q][1] * t0);
                    const float qq = fmaf(t1, r1, t0 * r0);
                    const float a = ex2_approx(qq) * pt.w;
                    sa[q] += a;
                    const float c2 = a * cw2[q];
                    dx[0] = fmaf(c2, r0, dx[0]);
                    dx[1] = fmaf(c2, r1, dx[1]);
                    const float u0 = c2 * t0, u1 = c2 * t1;
                    U[q][0] += u0; U[q][1] += u1;
                    M[q][0] = fmaf(u0, t0, M[q][0]);
                    M[q][1] = fmaf(u0, t1, M[q][1]);
                    M[q][2] = fmaf(u1, t1, M[q][2]);
                }
            }
            if (need_gx) {
#pragma unroll
                for (int d = 0; d < D; ++d) sm.partial[(pp * D + d) * TGP + tg] = dx[d];
            }
        }
        if (need_gx) {
            __syncthreads();
            // fold: row = (point, dim); SPLIT threads share a row, each sums TG / SPLIT entries
            constexpr int ROWS = kBwdPointChunk * D;
            constexpr int SPLIT = (kBwdThreads / ROWS) >= 4 ? 4 : ((kBwdThreads / ROWS) >= 2 ? 2 : 1);
            const int row = tid / SPLIT;
            const int part = tid - row * SPLIT;
            if (row < ROWS) {
                const int per = TG / SPLIT;    // multiple of 4 because TG >= 32 and SPLIT <= 4
                const float4* src = reinterpret_cast<const float4*>(sm.partial + row * TGP + part * per);
                float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
                for (int i = 0; i < per / 4; ++i) {
                    const float4 v = src[i];
                    s0 += v.x; s1 += v.y; s2 += v.z; s3 += v.w;
                }
                const int pp = row / D;
                const int d = row - pp * D;
                if (c0 + pp < n_here) atomicAdd(grad_xes + (xes_row + n0 + c0 + pp) * D + d, (s0 + s1) + (s2 + s3));
            }
            __syncthreads();
        }
    }

    if (grad_mixture == nullptr) return;

    // ---- fold point slices, finish the per-Gaussian gradient, one atomic per value ----
    // (slices > 1 only when the mixture is small; their partial sums simply issue separate atomics.)
#pragma unroll
    for (int q = 0; q < GQ; ++q) {
        const int g = gbase + tg + q * TG;
        if (g >= n_components) continue;
        const float* r = mix + size_t(g) * RF;
        const float w = __ldg(r);
        float S[D * D];
#pragma unroll
        for (int i = 0; i < D * D; ++i) S[i] = __ldg(r + 1 + D + i);
        float* go = grad_mixture + (size_t(bl) * n_components + g) * RF;
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
        atomicAdd(go, norm * sa[q]);
        // d/d mu = S * sum(c t);  U holds sum(c2 t) with c2 = c * 2 ln 2
        float Uc[D];
#pragma unroll
        for (int d = 0; d < D; ++d) Uc[d] = U[q][d] * inv2ln2;
#pragma unroll
        for (int i = 0; i < D; ++i) {
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < D; ++j) s = fmaf(0.5f * (S[i * D + j] + S[j * D + i]), Uc[j], s);
            atomicAdd(go + 1 + i, s);
        }
        // d/d S = -1/2 sum(c t t^T) + (w sum(a) factor / (2 sqrt(det))) cof(S)
        const float gdet = w * sa[q] * gauss_norm_factor<D>() / (2.f * root);
        int s_idx = 0;
        float Mfull[D * D];
#pragma unroll
        for (int i = 0; i < D; ++i)
#pragma unroll
            for (int j = i; j < D; ++j) {
                Mfull[i * D + j] = M[q][s_idx];
                Mfull[j * D + i] = M[q][s_idx];
                ++s_idx;
            }
#pragma unroll
        for (int i = 0; i < D * D; ++i) atomicAdd(go + 1 + D + i, fmaf(-0.5f * inv2ln2, Mfull[i], gdet * cof[i]));
    }
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
                   int n_batch_xes, int n_layers_xes, int n_xes, cudaStream_t stream) {
    constexpr int TILE = kFwdThreads * P;
    const long long tiles = (n_xes + TILE - 1) / TILE;
    const long long blocks = tiles * n_batch * n_layers;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    auto kernel = eval_forward_kernel<D, P>;
    const size_t smem = sizeof(FwdSmem<D, P>);
    if (int s = set_smem(kernel, smem)) return s;
    kernel<<<unsigned(blocks), kFwdThreads, smem, stream>>>(mixture, xes, out, n_layers, n_components, n_batch_xes,
                                                            n_layers_xes, n_xes, int(tiles));
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

template <int D, int GQ>
int launch_backward(const float* grad_out, const float* mixture, const float* xes, float* grad_mixture,
                    float* grad_xes, int n_batch, int n_layers, int n_components, int n_batch_xes, int n_layers_xes,
                    int n_xes, int tg, cudaStream_t stream) {
    const long long ptiles = (n_xes + kBwdTilePoints - 1) / kBwdTilePoints;
    const long long gchunks = (n_components + tg * GQ - 1) / (tg * GQ);
    const long long blocks = ptiles * gchunks * n_batch * n_layers;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    auto kernel = eval_backward_kernel<D, GQ>;
    const size_t smem = sizeof(BwdSmem<D>);
    if (int s = set_smem(kernel, smem)) return s;
    kernel<<<unsigned(blocks), kBwdThreads, smem, stream>>>(grad_out, mixture, xes, grad_mixture, grad_xes, n_layers,
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
    const bool small = pairs_rows < 148LL * 4 * kFwdThreads * 4;
    if (n_dims == 2) {
        return small ? launch_forward<2, 1>(mixture, xes, out, n_batch, n_layers, n_components, n_batch_xes, n_layers_xes, n_xes, st)
                     : launch_forward<2, 4>(mixture, xes, out, n_batch, n_layers, n_components, n_batch_xes, n_layers_xes, n_xes, st);
    }
    return small ? launch_forward<3, 1>(mixture, xes, out, n_batch, n_layers, n_components, n_batch_xes, n_layers_xes, n_xes, st)
                 : launch_forward<3, 4>(mixture, xes, out, n_batch, n_layers, n_components, n_batch_xes, n_layers_xes, n_xes, st);
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

    // Gaussians per thread and threads along the Gaussian axis
    int gq, tg;
    if (n_components >= 512) { gq = 4; tg = 128; }
    else if (n_components >= 256) { gq = 2; tg = 128; }
    else if (n_components > 64) { gq = 1; tg = 128; }
    else if (n_components > 32) { gq = 1; tg = 64; }
    else { gq = 1; tg = 32; }
#define GMC_BWD(D_, GQ_) launch_backward<D_, GQ_>(grad_out, mixture, xes, grad_mixture, grad_xes, n_batch, n_layers, \
                                                  n_components, n_batch_xes, n_layers_xes, n_xes, tg, st)
    if (n_dims == 2) return gq == 4 ? GMC_BWD(2, 4) : (gq == 2 ? GMC_BWD(2, 2) : GMC_BWD(2, 1));
    return gq == 4 ? GMC_BWD(3, 4) : (gq == 2 ? GMC_BWD(3, 2) : GMC_BWD(3, 1));
#undef GMC_BWD
}
