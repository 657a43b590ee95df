// BVH-MHEM reduction of a mixture of G Gaussians to K Gaussians (forward).
//
// Algorithm (same decisions as the reference's bvh_mhem_fit/implementation_forward.h:35-484): over the LBVH of the
// component means, every internal node gathers the Gaussians of its two children (left first, |w| < 1e-7 dropped) and,
// if there are more than R, replaces them by R Gaussians with one hierarchical-EM step (initial representatives by
// single-linkage clustering of the centres, KL-gated responsibilities, moment matching); afterwards nodes are selected
// greedily from the root by |integral| until about K Gaussians are collected.
//
// Organisation on the GPU: one CTA per mixture. Tree levels (height above the leaves) are computed in shared memory
// with the "second arriver continues" pass; levels are then processed in order, one warp per node, with the 2R x R
// likelihood / KL / responsibility matrices spread one entry per lane. The single-linkage clustering of fit_initial:
// when all finite centre distances of a node differ, the heap's pop order is the rank of the distance, so the warp ranks
// the pairs with shuffles and every lane merges the sub-graphs in registers; with equal distances the order among equal
// keys is the heap's own, and lane 0 runs the restated heap. Node results live in a global attribute array that is also
// what the backward pass reads: per internal node R Gaussians, the integral, the Gaussian count, the R initial indices.
#include <mutex>

#include "common.cuh"
#include "lbvh_device.cuh"

namespace gmc {

int lbvh_build_launch(const float* mixture, long long n_mixtures, int n_components, int n_dims, int layout, uint64_t* sorted_keys,
                      uint16_t* nodes, cudaStream_t stream);

namespace {

// Child and object indices read from the node array (checked in GMC_BOUNDS_CHECK builds, see common.cuh)
#define GMC_NODE(i, n_internal) GMC_IDX(int(i), 2 * (n_internal) + 1)
#define GMC_OBJ(i, n_internal) GMC_IDX(int(i), (n_internal) + 1)

#ifndef GMC_FIT_THREADS
#define GMC_FIT_THREADS 384
#endif
constexpr int kThreads = GMC_FIT_THREADS;      // largest CTA; the launch picks the size by the mixture's size
constexpr int kWarps = kThreads / 32;
// One warp fits one node: mixtures of 512 components and more keep twelve warps busy (1.41 -> 1.37 ms at 1024 components,
// 1024 mixtures), small ones are faster with eight (more mixtures resident per SM).
inline int fit_threads(int n_components) { return n_components >= 512 ? kThreads : (kThreads < 256 ? kThreads : 256); }
constexpr int kMaxLevels = 72;
constexpr int kSharedBookkeepingMax = 8192;   // above this many components the per-node arrays go to global scratch
// bytes of global bookkeeping per mixture: level [2G-1 -> 16] + arrive / order [4 (G-1)] + has_grad [G], at most 8 G
__host__ __device__ inline size_t big_scratch_bytes(int G) {
    return ((size_t(2 * G - 1) + 15) & ~size_t(15)) + 4 * size_t(G - 1) + ((size_t(G) + 15) & ~size_t(15));
}
constexpr float kEpsSmall = 0.0000000000001f;
constexpr float kEpsLarge = 0.0000001f;
constexpr float kKlThreshold = 0.5f;

// The EM step is written once on a value type T: float in the forward pass (its decisions and values are the
// reference's fp32 ones) and double in the backward pass, where differences of nearly equal terms are scaled by squared
// inverse covariances (fp32 there loses three to four digits on mixtures with small covariances).
__device__ __forceinline__ float clip(float v) { return fmaxf(v, kEpsSmall); }
__device__ __forceinline__ double clip(double v) { return fmax(v, double(kEpsSmall)); }
template <typename T> __device__ __forceinline__ int sign_of(T v) { return v >= T(0) ? 1 : -1; }
__device__ __forceinline__ float g_exp(float v) { return expf(v); }
__device__ __forceinline__ double g_exp(double v) { return exp(v); }
__device__ __forceinline__ float g_log(float v) { return logf(v); }
__device__ __forceinline__ double g_log(double v) { return log(v); }
__device__ __forceinline__ float g_pow(float a, float b) { return powf(a, b); }
__device__ __forceinline__ double g_pow(double a, double b) { return pow(a, b); }
__device__ __forceinline__ float g_sqrt(float v) { return sqrtf(v); }
__device__ __forceinline__ double g_sqrt(double v) { return sqrt(v); }
template <int D, typename T> __device__ __forceinline__ T norm_factor_t() {
    if constexpr (sizeof(T) == 4) return T(gauss_norm_factor<D>());
    else return D == 2 ? T(0.15915494309189535) : T(0.06349363593424097);     // (2 pi)^(-D/2)
}

template <int D, typename T> __device__ __forceinline__ T det(const T* m) {
    if constexpr (D == 2) return m[0] * m[3] - m[1] * m[2];
    else return m[0] * (m[4] * m[8] - m[5] * m[7]) - m[1] * (m[3] * m[8] - m[5] * m[6]) + m[2] * (m[3] * m[7] - m[4] * m[6]);
}
template <int D, typename T> __device__ __forceinline__ void inverse(const T* m, T* o) {
    const T r = T(1) / det<D, T>(m);
    if constexpr (D == 2) {
        o[0] = m[3] * r; o[1] = -m[1] * r; o[2] = -m[2] * r; o[3] = m[0] * r;
    } else {
        o[0] = (m[4] * m[8] - m[5] * m[7]) * r; o[1] = -(m[1] * m[8] - m[2] * m[7]) * r; o[2] = (m[1] * m[5] - m[2] * m[4]) * r;
        o[3] = -(m[3] * m[8] - m[5] * m[6]) * r; o[4] = (m[0] * m[8] - m[2] * m[6]) * r; o[5] = -(m[0] * m[5] - m[2] * m[3]) * r;
        o[6] = (m[3] * m[7] - m[4] * m[6]) * r; o[7] = -(m[0] * m[7] - m[1] * m[6]) * r; o[8] = (m[0] * m[4] - m[1] * m[3]) * r;
    }
}

// Attribute record of an internal node: [R * RF floats | integral | count | initial indices (4 x uint8) | reserved]
template <int D, int R>
struct Attr {
    static constexpr int RF = 1 + D + D * D;
    static constexpr int kFloats = R * RF + 4;
};

// Per-warp scratch in shared memory.
template <int D, int R>
struct WarpScratch {
    static constexpr int RF = 1 + D + D * D;
    static constexpr int NT = 2 * R;
    static constexpr int NH = (NT * NT - NT) / 2;
    float tgt[NT][RF];        // gathered child Gaussians, padded with (0, 0, I)
    float heap_d[NH];
    unsigned char heap_a[NH], heap_b[NH];
    unsigned char order[32];  // pair (lane) with the k-th smallest distance
    int idx[R];               // initial representatives
    float r3[NT][R];
    float fw[R];
    float outp[R][D];
    float outc[R][D * D];
    float gin[R][RF];         // backward: gradient of the node's Gaussians
    float tgrad[NT][RF];      // backward: gradient of the gathered child Gaussians
};

// Sub-graphs of the single-linkage clustering (valid Gaussians are 0 .. n_valid-1, sub-graph i starts as {i}). Merging
// appends the higher sub-graph's member list to the lower one's, which keeps the member order that the first-max rule
// of select() depends on. All state is packed into 64-bit words (8 bits per Gaussian), so it lives in registers:
//   labels: sub-graph of Gaussian g;  nexts: successor of g in its member list (0xFF = end);  tails: last member.
template <int NT>
struct SubGraphs {
    uint64_t labels = 0ull, tails = 0ull, nexts = ~0ull;
    __device__ __forceinline__ SubGraphs() {
#pragma unroll
        for (int i = 0; i < NT; ++i) { labels |= uint64_t(i) << (8 * i); tails |= uint64_t(i) << (8 * i); }
    }
    static __device__ __forceinline__ int get(uint64_t v, int i) { return int((v >> (8 * i)) & 0xFFull); }
    static __device__ __forceinline__ void set(uint64_t& v, int i, int x) {
        v = (v & ~(0xFFull << (8 * i))) | (uint64_t(x) << (8 * i));
    }
    // joins the sub-graphs of Gaussians a and b; false if they already were one
    __device__ __forceinline__ bool merge(int a, int b) {
        const int sa = get(labels, a), sb = get(labels, b);
        if (sa == sb) return false;
        const int lo = min(sa, sb), hi = max(sa, sb);
        // every label byte equal to hi becomes lo (byte-wise compare on the two halves of the packed word)
        const unsigned hi4 = unsigned(hi) * 0x01010101u, lo4 = unsigned(lo) * 0x01010101u;
        unsigned l0 = unsigned(labels), l1 = unsigned(labels >> 32);
        const unsigned m0 = __vcmpeq4(l0, hi4), m1 = __vcmpeq4(l1, hi4);      // 0xFF in the matching bytes
        l0 = (l0 & ~m0) | (lo4 & m0);
        l1 = (l1 & ~m1) | (lo4 & m1);
        labels = uint64_t(l0) | (uint64_t(l1) << 32);
        set(nexts, get(tails, lo), hi);       // the head of sub-graph hi is Gaussian hi
        set(tails, lo, get(tails, hi));
        return true;
    }
    // representative of each of the first R live sub-graphs: its member with the largest |weight| (first of equals)
    template <int D, int R, typename Scratch>
    __device__ __forceinline__ void select(Scratch& ws, int n_valid, bool write) const {
        int sg = -1;
        for (int i = 0; i < R; ++i) {
            do { ++sg; } while (sg < n_valid && get(labels, sg) != sg);   // alive while its head labels itself
            int selected = 255;
            float max_abs = 0.f;
            if (sg < n_valid) {
                for (int gid = sg; gid != 0xFF; gid = get(nexts, gid)) {
                    const float aw = fabsf(ws.tgt[gid][0]);
                    if (aw > max_abs) { max_abs = aw; selected = gid; }
                }
            }
            if (write) ws.idx[i] = selected;
        }
    }
};

// ---- the sequential part of fit_initial, run by one lane ----
template <int D, int R>
__device__ void cluster_and_select(WarpScratch<D, R>& ws, int n_valid) {
    constexpr int NT = 2 * R;
    constexpr int NH = (NT * NT - NT) / 2;
    // heap primitives (min-heap on the disparity, ties resolved as in the reference's ArrayHeap)
    auto two_children = [](unsigned i) { return i < unsigned((NH - 1) / 2); };
    auto is_leaf = [](unsigned i) { return i >= unsigned(NH / 2); };
    auto replace_element = [&](float vd, unsigned char va, unsigned char vb, unsigned index, float& rd, unsigned char& ra,
                               unsigned char& rb) {
        rd = ws.heap_d[index]; ra = ws.heap_a[index]; rb = ws.heap_b[index];
        unsigned cur = index;
        while (two_children(cur)) {
            const unsigned l = cur * 2 + 1, r = cur * 2 + 2;
            const float ld = ws.heap_d[l], rdv = ws.heap_d[r];
            if (vd <= ld && vd <= rdv) break;
            if (ld <= rdv) { ws.heap_d[cur] = ld; ws.heap_a[cur] = ws.heap_a[l]; ws.heap_b[cur] = ws.heap_b[l]; cur = l; }
            else { ws.heap_d[cur] = rdv; ws.heap_a[cur] = ws.heap_a[r]; ws.heap_b[cur] = ws.heap_b[r]; cur = r; }
        }
        if (!is_leaf(cur)) {
            const unsigned l = cur * 2 + 1;
            const float ld = ws.heap_d[l];
            if (ld <= vd) { ws.heap_d[cur] = ld; ws.heap_a[cur] = ws.heap_a[l]; ws.heap_b[cur] = ws.heap_b[l]; cur = l; }
        }
        ws.heap_d[cur] = vd; ws.heap_a[cur] = va; ws.heap_b[cur] = vb;
    };
    float rd; unsigned char ra, rb;
    for (unsigned i = (NH - 2) / 2; i < unsigned(NH); --i) {
        const float vd = ws.heap_d[i];
        const unsigned char va = ws.heap_a[i], vb = ws.heap_b[i];
        replace_element(vd, va, vb, i, rd, ra, rb);
    }
    SubGraphs<NT> graphs;
    int n_subgraphs = n_valid;
    while (n_subgraphs > R) {
        replace_element(INFINITY, 255, 255, 0, rd, ra, rb);
        if (!(rd < INFINITY)) break;
        if (graphs.merge(ra, rb)) --n_subgraphs;
    }
    graphs.template select<D, R>(ws, n_valid, true);
}

// The same clustering when all finite distances differ (the usual case): a min-heap then pops the pairs in ascending
// order of distance, so the pop order is the rank of a pair's distance. Lane e < NH holds pair e = (a, b) with
// distance d (+inf = no edge); the ranks come from NH shuffles, the merges run on registers, uniformly in all lanes.
// Returns false (and does nothing) if two finite distances are equal or one is NaN: the caller then runs the heap,
// whose order among equal keys is part of the reference's result.
template <int D, int R>
__device__ __forceinline__ bool cluster_and_select_ranked(WarpScratch<D, R>& ws, int n_valid, float d, int a, int b) {
    constexpr int NT = 2 * R;
    constexpr int NH = (NT * NT - NT) / 2;
    const int lane = threadIdx.x & 31;
    const bool finite = lane < NH && d < INFINITY;
    bool unusable = lane < NH && d != d;
    int rank = 0;
#pragma unroll
    for (int k = 0; k < NH; ++k) {
        const float dk = __shfl_sync(0xffffffffu, d, k);
        if (k != lane) {
            if (dk < d || (dk == d && k < lane)) ++rank;
            if (finite && dk == d) unusable = true;
        }
    }
    if (__any_sync(0xffffffffu, unusable)) return false;
    if (lane < NH) ws.order[rank] = (unsigned char)lane;
    __syncwarp();
    const int ab = a | (b << 8);
    SubGraphs<NT> graphs;
    int n_subgraphs = n_valid;
    for (int k = 0; k < NH && n_subgraphs > R; ++k) {
        const int e = ws.order[k];
        const float dk = __shfl_sync(0xffffffffu, d, e);
        const int abk = __shfl_sync(0xffffffffu, ab, e);
        if (!(dk < INFINITY)) break;
        if (graphs.merge(abk & 0xFF, abk >> 8)) --n_subgraphs;
    }
    graphs.template select<D, R>(ws, n_valid, lane == 0);
    return true;
}

// Reductions over the lanes of one matrix row (fixed target t, lanes t*R .. t*R+R-1) or one matrix column (fixed s,
// lanes s, s+R, ...); every lane of the row / column ends up with the total.
template <int R, typename T>
__device__ __forceinline__ T row_sum(T v) {
#pragma unroll
    for (int off = 1; off < R; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}
template <int R, typename T>
__device__ __forceinline__ T col_sum(T v) {
#pragma unroll
    for (int off = R; off < 2 * R * R; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Values of matrix entry (t, s) of the EM step, one entry per lane (lanes beyond the matrix repeat the last entry).
template <int D, typename T = float>
struct Entry {
    int t, s, fi;
    T W, Wc, V, Vc;       // target / initial integral and their clipped versions
    T a, b;               // weights scaled to integral one: a_t = w_t / Wc, b_s = v_s / Vc
    T inv[D * D];         // inverse covariance of initial Gaussian s
    T diff[D];            // mu_t - mu_initial(s)
    T val_a, val_b, ab;   // N(mu_t; initial s), exp(-1/2 tr(inv Sigma_t)), their product
    T lik, gate, u, x, X, r1, r2, fw, fwc, r3;
};

// Needs ws.tgt (padded targets) and ws.idx. Sums that feed decisions run in a fixed order (as on the CPU checker).
// gate_in == nullptr: the KL gate is decided here (forward pass, T = float). Otherwise *gate_in is this entry's gate as
// the forward pass decided it, and the values are recomputed in T around that decision (backward pass, T = double).
template <int D, int R, typename T = float>
__device__ __forceinline__ Entry<D, T> em_entry(const WarpScratch<D, R>& ws, int lane, const float* gate_in = nullptr) {
    constexpr int NT = 2 * R;
    constexpr int NE = NT * R;
    Entry<D, T> e;
    T W = T(0);
#pragma unroll
    for (int i = 0; i < NT; ++i) W += T(ws.tgt[i][0]);
    e.W = W; e.Wc = clip(W);
    T V = T(0);
#pragma unroll
    for (int s = 0; s < R; ++s) V += T(ws.tgt[ws.idx[s] < NT ? ws.idx[s] : 0][0]);
    e.V = V; e.Vc = clip(V);
    const int ent = lane < NE ? lane : NE - 1;
    e.t = ent / R; e.s = ent - e.t * R;
    e.fi = ws.idx[e.s] < NT ? ws.idx[e.s] : 0;
    e.a = T(ws.tgt[e.t][0]) / e.Wc;
    e.b = T(ws.tgt[e.fi][0]) / e.Vc;
    T icov[D * D], tcov[D * D];
#pragma unroll
    for (int k = 0; k < D * D; ++k) { icov[k] = T(ws.tgt[e.fi][1 + D + k]); tcov[k] = T(ws.tgt[e.t][1 + D + k]); }
    inverse<D, T>(icov, e.inv);
#pragma unroll
    for (int k = 0; k < D; ++k) e.diff[k] = T(ws.tgt[e.t][1 + k]) - T(ws.tgt[e.fi][1 + k]);
    T maha = T(0);
#pragma unroll
    for (int i = 0; i < D; ++i) {
        T acc = T(0);
#pragma unroll
        for (int j = 0; j < D; ++j) acc += e.inv[i * D + j] * e.diff[j];
        maha += e.diff[i] * acc;
    }
    T tr = T(0);
#pragma unroll
    for (int i = 0; i < D; ++i)
#pragma unroll
        for (int j = 0; j < D; ++j) tr += e.inv[i * D + j] * tcov[j * D + i];
    e.val_a = g_sqrt(det<D, T>(e.inv)) * norm_factor_t<D, T>() * g_exp(T(-0.5) * maha);
    e.val_b = g_exp(T(-0.5) * tr);
    e.ab = e.val_a * e.val_b;
    e.lik = g_pow(clip(e.ab), T(4) * e.a);
    const int row_base = e.t * R;
    if (gate_in == nullptr) {
        const T lg = g_log(det<D, T>(tcov) / det<D, T>(icov));
        const T kl = sign_of(e.b) == sign_of(e.a) ? T(0.5) * (maha + tr - T(D) - lg) : T(0);
        e.gate = kl < T(kKlThreshold) ? T(1) : T(0);
        // per target: the component with the smallest KL is always gated in (first strict minimum)
        int best = -1;
        T smallest = T(INFINITY);
#pragma unroll
        for (int s2 = 0; s2 < R; ++s2) {
            const T v = __shfl_sync(0xffffffffu, kl, row_base + s2);
            if (v < smallest) { smallest = v; best = s2; }
        }
        if (best == e.s) e.gate = T(1);
    } else {
        e.gate = T(*gate_in);
    }
    e.u = e.b * e.lik;
    e.x = clip(e.u) * e.gate;
    T X = T(0);
#pragma unroll
    for (int s2 = 0; s2 < R; ++s2) X += __shfl_sync(0xffffffffu, e.x, row_base + s2);
    e.X = X;
    e.r1 = e.x / X;
    e.r2 = e.r1 * e.a;
    T fw = T(0);
#pragma unroll
    for (int t2 = 0; t2 < NT; ++t2) fw += __shfl_sync(0xffffffffu, e.r2, t2 * R + e.s);
    e.fw = fw; e.fwc = clip(fw);
    e.r3 = e.r2 / e.fwc;
    return e;
}

// Fitted positions from ws.r3 (needs a __syncwarp before and after).
template <int D, int R>
__device__ __forceinline__ void em_positions(WarpScratch<D, R>& ws, int lane) {
    constexpr int NT = 2 * R;
    for (int o = lane; o < R * D; o += 32) {
        const int so = o / D, d = o - so * D;
        float acc = 0.f;
#pragma unroll
        for (int t2 = 0; t2 < NT; ++t2) acc += ws.r3[t2][so] * ws.tgt[t2][1 + d];
        ws.outp[so][d] = acc;
    }
}

// ---- one hierarchical-EM step on the padded targets in ws.tgt; result goes to `out` (R * RF floats) ----
template <int D, int R>
__device__ void fit_em_warp(WarpScratch<D, R>& ws, int n_target, float* __restrict__ out, int* initial_packed) {
    constexpr int RF = 1 + D + D * D;
    constexpr int NT = 2 * R;
    constexpr int NH = (NT * NT - NT) / 2;
    constexpr int NE = NT * R;   // matrix entries: 32 (R = 4) or 8 (R = 2)
    const int lane = threadIdx.x & 31;

    // pairwise centre distances in the reference's heap fill order: all pairs i < j of the n_target valid
    // Gaussians (they are compacted in front), row major; the rest of the heap array is +inf padding
    {
        int i = 0, rem = lane < NH ? lane : 0;
        while (rem >= NT - 1 - i) { rem -= NT - 1 - i; ++i; }
        const int j = i + 1 + rem;
        const bool real_pair = lane < NH && j < n_target;
        float d = INFINITY;
        if (real_pair) {
            const float wa = ws.tgt[i][0], wb = ws.tgt[j][0];
            d = 0.f;
#pragma unroll
            for (int k = 0; k < D; ++k) { const float tt = ws.tgt[i][1 + k] - ws.tgt[j][1 + k]; d += tt * tt; }
            if (sign_of(wa) != sign_of(wb) || fabsf(wa) < kEpsLarge || fabsf(wb) < kEpsLarge) d = INFINITY;
        }
        if (!cluster_and_select_ranked<D, R>(ws, n_target, d, i, j)) {
            // equal distances: the heap decides their order
            if (lane < NH) { ws.heap_d[lane] = INFINITY; ws.heap_a[lane] = 255; ws.heap_b[lane] = 255; }
            __syncwarp();
            if (real_pair) {
                const int pos = i * n_target - (i * (i + 1)) / 2 + (j - i - 1);
                ws.heap_d[pos] = d; ws.heap_a[pos] = (unsigned char)i; ws.heap_b[pos] = (unsigned char)j;
            }
            __syncwarp();
            if (lane == 0) cluster_and_select<D, R>(ws, n_target);
        }
    }
    __syncwarp();

    const Entry<D> e = em_entry<D, R>(ws, lane);
    if (lane < NE) {
        ws.r3[e.t][e.s] = e.r3;
        if (e.t == 0) ws.fw[e.s] = e.fw;
    }
    __syncwarp();
    em_positions<D, R>(ws, lane);
    __syncwarp();
    for (int o = lane; o < R * D * D; o += 32) {
        const int so = o / (D * D), ij = o - so * D * D, i = ij / D, j = ij - i * D;
        float acc = 0.f;
#pragma unroll
        for (int t2 = 0; t2 < NT; ++t2) {
            const float di = ws.tgt[t2][1 + i] - ws.outp[so][i], dj = ws.tgt[t2][1 + j] - ws.outp[so][j];
            acc += ws.r3[t2][so] * (di * dj + ws.tgt[t2][1 + D + ij]);
        }
        if (ws.fw[so] < kEpsLarge) acc = (i == j) ? 1.f : 0.f;
        ws.outc[so][ij] = acc;
    }
    __syncwarp();
    for (int o = lane; o < R * RF; o += 32) {
        const int so = o / RF, f = o - so * RF;
        float v;
        if (f == 0) v = ws.fw[so] * e.Wc;
        else if (f <= D) v = ws.outp[so][f - 1];
        else v = ws.outc[so][f - 1 - D];
        out[o] = v;
    }
    if (lane == 0) {
        int packed = 0;
#pragma unroll
        for (int s2 = 0; s2 < R; ++s2) packed |= (ws.idx[s2] & 0xFF) << (8 * s2);
        *initial_packed = packed;
    }
    __syncwarp();
}

// ---- reverse of fit_em_warp: ws.tgt (padded targets), ws.idx and ws.gin (gradient of the R fitted Gaussians) in,
//      ws.tgrad (gradient of the targets) out. The KL gate, the initial indices and every threshold decision (clip,
//      covariance replaced by the identity) are the forward pass's fp32 ones; the values around them are recomputed
//      and differentiated in double. ----
template <int D, int R>
__device__ void grad_em_warp(WarpScratch<D, R>& ws) {
    using T = double;
    constexpr int RF = 1 + D + D * D;
    constexpr int NT = 2 * R;
    constexpr int NE = NT * R;
    const int lane = threadIdx.x & 31;

    const Entry<D, float> f = em_entry<D, R, float>(ws, lane);          // decisions as the forward pass took them
    const float gate = f.gate;
    const Entry<D, T> e = em_entry<D, R, T>(ws, lane, &gate);

    T tg[RF];
#pragma unroll
    for (int k = 0; k < RF; ++k) tg[k] = T(ws.tgt[e.t][k]);
    const T gw = T(ws.gin[e.s][0]);
    T gP[D], gC[D * D];
#pragma unroll
    for (int i = 0; i < D; ++i) gP[i] = T(ws.gin[e.s][1 + i]);
#pragma unroll
    for (int ij = 0; ij < D * D; ++ij) gC[ij] = f.fw < kEpsLarge ? T(0) : T(ws.gin[e.s][1 + D + ij]);

    // ---- moment matching ----
    T d[D];
#pragma unroll
    for (int i = 0; i < D; ++i) d[i] = tg[1 + i] - col_sum<R, T>(e.r3 * tg[1 + i]);      // mu_t - fitted centre s
    T g_r3 = T(0);
#pragma unroll
    for (int i = 0; i < D; ++i)
#pragma unroll
        for (int j = 0; j < D; ++j) g_r3 += gC[i * D + j] * (d[i] * d[j] + tg[1 + D + i * D + j]);
    T t_mu[D], t_cov[D * D];     // this entry's share of the target gradient
    T gPt[D];
#pragma unroll
    for (int i = 0; i < D; ++i) {
        T acc = T(0);
#pragma unroll
        for (int j = 0; j < D; ++j) acc += (gC[i * D + j] + gC[j * D + i]) * d[j];
        const T gd = e.r3 * acc;
        gPt[i] = gP[i] - col_sum<R, T>(gd);
        t_mu[i] = gd + e.r3 * gPt[i];
    }
#pragma unroll
    for (int i = 0; i < D; ++i) g_r3 += gPt[i] * tg[1 + i];
#pragma unroll
    for (int ij = 0; ij < D * D; ++ij) t_cov[ij] = e.r3 * gC[ij];

    // ---- responsibilities ----
    T gWc = T(0);
#pragma unroll
    for (int s2 = 0; s2 < R; ++s2) gWc += T(ws.gin[s2][0]) * __shfl_sync(0xffffffffu, e.fw, s2);   // lane s2 = entry (0, s2)
    T gF = gw * e.Wc;
    const T gFc = col_sum<R, T>(-g_r3 * e.r2 / (e.fwc * e.fwc));
    if (f.fw > kEpsSmall) gF += gFc;
    const T g_r2 = g_r3 / e.fwc + gF;
    const T g_r1 = g_r2 * e.a;
    T g_a = g_r2 * e.r1;
    T g_x = g_r1 / e.X;
    g_x += row_sum<R, T>(-g_r1 * e.x / (e.X * e.X));
    const T g_u = f.u > kEpsSmall ? g_x * e.gate : T(0);
    const T g_b = col_sum<R, T>(g_u * e.lik);
    const T g_L = g_u * e.b;

    // ---- likelihood: L = clip(a b)^(4 a_t) ----
    const T abc = clip(e.ab), wbar = T(4) * e.a;
    const T g_abc = g_L * wbar * g_pow(abc, wbar - T(1));
    g_a += T(4) * (g_L * e.lik * g_log(abc));
    const T g_ab = f.ab > kEpsSmall ? g_abc : T(0);
    const T c1 = e.val_a * (g_ab * e.val_b);             // val_a * dL/dval_a
    const T gh = (g_ab * e.val_a) * e.val_b;             // dL/dh, val_b = exp(h), h = -1/2 tr(inv Sigma_t)
    T i_mu[D], gS[D * D];                                // gradient of the initial centre / of inv
#pragma unroll
    for (int i = 0; i < D; ++i) {
        T st = T(0);
#pragma unroll
        for (int j = 0; j < D; ++j) st += e.inv[i * D + j] * e.diff[j];
        t_mu[i] -= c1 * st;
        i_mu[i] = c1 * st;
    }
    T ic[D * D];
#pragma unroll
    for (int k = 0; k < D * D; ++k) ic[k] = T(ws.tgt[e.fi][1 + D + k]);
#pragma unroll
    for (int i = 0; i < D; ++i)
#pragma unroll
        for (int j = 0; j < D; ++j) {
            t_cov[i * D + j] += T(-0.5) * gh * e.inv[j * D + i];
            gS[i * D + j] = c1 * (T(0.5) * ic[j * D + i] - T(0.5) * e.diff[i] * e.diff[j]) - T(0.5) * gh * tg[1 + D + j * D + i];
        }
    T i_cov[D * D];                                      // d/d Sigma_initial = -inv^T gS inv^T
#pragma unroll
    for (int i = 0; i < D; ++i)
#pragma unroll
        for (int j = 0; j < D; ++j) {
            T acc = T(0);
#pragma unroll
            for (int k = 0; k < D; ++k)
#pragma unroll
                for (int l = 0; l < D; ++l) acc += e.inv[k * D + i] * gS[k * D + l] * e.inv[j * D + l];
            i_cov[i * D + j] = -acc;
        }

    // ---- fold over rows (targets) and columns (initial Gaussians) ----
    g_a = row_sum<R, T>(g_a);
#pragma unroll
    for (int i = 0; i < D; ++i) { t_mu[i] = row_sum<R, T>(t_mu[i]); i_mu[i] = col_sum<R, T>(i_mu[i]); }
#pragma unroll
    for (int ij = 0; ij < D * D; ++ij) { t_cov[ij] = row_sum<R, T>(t_cov[ij]); i_cov[ij] = col_sum<R, T>(i_cov[ij]); }
    // integrals: a_t = w_t / Wc, b_s = v_s / Vc
    gWc += col_sum<R, T>(-g_a * tg[0] / (e.Wc * e.Wc));
    const T gW = f.W > kEpsSmall ? gWc : T(0);
    const T gVc = row_sum<R, T>(-g_b * T(ws.tgt[e.fi][0]) / (e.Vc * e.Vc));
    const T g_v = g_b / e.Vc + (f.V > kEpsSmall ? gVc : T(0));
    if (lane < NE && e.s == 0) {
        ws.tgrad[e.t][0] = float(g_a / e.Wc + gW);
#pragma unroll
        for (int i = 0; i < D; ++i) ws.tgrad[e.t][1 + i] = float(t_mu[i]);
#pragma unroll
        for (int ij = 0; ij < D * D; ++ij) ws.tgrad[e.t][1 + D + ij] = float(t_cov[ij]);
    }
    __syncwarp();
    if (lane < NE && e.t == 0) {      // the initial Gaussians are targets e.fi (distinct per s)
        ws.tgrad[e.fi][0] += float(g_v);
#pragma unroll
        for (int i = 0; i < D; ++i) ws.tgrad[e.fi][1 + i] += float(i_mu[i]);
#pragma unroll
        for (int ij = 0; ij < D * D; ++ij) ws.tgrad[e.fi][1 + D + ij] += float(i_cov[ij]);
    }
    __syncwarp();
}

template <int D, int R>
struct FitSmem {
    WarpScratch<D, R> warp[kWarps];
};

// Levels above the leaves (leaves 0, internal node = 1 + max of its children) by the second-arriver climb.
// `arrive` and `level` live in shared memory; returns after a CTA-wide barrier with *max_level set.
__device__ __forceinline__ void compute_levels(const uint16_t* __restrict__ nodes, int G, unsigned char* level, int* arrive,
                                               int* max_level) {
    const int n_internal = G - 1, n_nodes = 2 * G - 1;
    for (int i = threadIdx.x; i < n_internal; i += int(blockDim.x)) arrive[i] = 0;
    for (int i = threadIdx.x; i < n_nodes; i += int(blockDim.x)) level[i] = 0;
    if (threadIdx.x == 0) *max_level = 0;
    __syncthreads();
    for (int leaf = threadIdx.x; leaf < G; leaf += int(blockDim.x)) {
        int parent = nodes[size_t(n_internal + leaf) * 4];
        for (int guard = 0; guard < kMaxLevels && parent != 0xFFFF; ++guard) {
            __threadfence_block();
            if (atomicAdd(&arrive[parent], 1) == 0) break;
            __threadfence_block();
            const int l = GMC_NODE(nodes[size_t(parent) * 4 + 1], n_internal), r = GMC_NODE(nodes[size_t(parent) * 4 + 2], n_internal);
            const int lv = 1 + max(int(((volatile unsigned char*)level)[l]), int(((volatile unsigned char*)level)[r]));
            ((volatile unsigned char*)level)[parent] = (unsigned char)lv;
            atomicMax(max_level, lv);
            parent = nodes[size_t(parent) * 4];
        }
    }
    __syncthreads();
}

// Node ids grouped by level (counting sort): nodes of level lv are order[level_start[lv] .. level_start[lv + 1]), in no
// particular order inside a level. With it the warps of a CTA share the nodes of a level evenly whatever their ids are.
// level_start and level_cursor hold 258 ints each; ends with a CTA-wide barrier.
__device__ __forceinline__ void group_by_level(const unsigned char* level, int n_internal, int max_level, uint16_t* order,
                                               int* level_start, int* level_cursor) {
    const int tid = threadIdx.x;
    for (int i = tid; i < 258; i += int(blockDim.x)) level_start[i] = 0;
    __syncthreads();
    for (int i = tid; i < n_internal; i += int(blockDim.x)) atomicAdd(&level_start[level[i]], 1);
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int lv = 0; lv <= max_level + 1; ++lv) {
            const int c = level_start[lv];
            level_start[lv] = run;
            level_cursor[lv] = run;
            run += c;
        }
    }
    __syncthreads();
    for (int i = tid; i < n_internal; i += int(blockDim.x)) order[atomicAdd(&level_cursor[level[i]], 1)] = uint16_t(i);
    __syncthreads();
}

// Gathers the Gaussians of the two children of `id` into ws.tgt (left first, |w| < 1e-7 dropped, padded with (0,0,I)).
// Lane j < R stands for the left child's j-th Gaussian, lane R + j for the right child's. Returns the number gathered;
// `in_range` / `valid` / `pos` describe this lane's Gaussian.
template <int D, int R>
__device__ __forceinline__ int gather_children(WarpScratch<D, R>& ws, const float* __restrict__ mix, const uint16_t* __restrict__ nodes,
                                               const float* attrs, int n_internal, int id, int lane, int& child,
                                               int& child_slot, bool& in_range, bool& valid, int& pos) {
    constexpr int RF = 1 + D + D * D;
    constexpr int AF = Attr<D, R>::kFloats;
    const int l = GMC_NODE(nodes[size_t(id) * 4 + 1], n_internal), r = GMC_NODE(nodes[size_t(id) * 4 + 2], n_internal);
    auto count_of = [&](int n) -> int { return n >= n_internal ? 1 : __float_as_int(attrs[size_t(n) * AF + R * RF + 1]); };
    const int cl = count_of(l), cr = count_of(r);
    child = lane < R ? l : r;
    child_slot = lane < R ? lane : lane - R;
    in_range = lane < 2 * R && child_slot < (lane < R ? cl : cr);
    const float* src = nullptr;
    if (in_range) src = child >= n_internal ? mix + size_t(GMC_OBJ(nodes[size_t(child) * 4 + 3], n_internal)) * RF
                                            : attrs + size_t(child) * AF + size_t(child_slot) * RF;
    valid = in_range && fabsf(src[0]) >= kEpsLarge;
    const unsigned vmask = __ballot_sync(0xffffffffu, valid);
    const int n_target = __popc(vmask);
    pos = __popc(vmask & ((1u << lane) - 1u));
    if (valid) {
#pragma unroll
        for (int f = 0; f < RF; ++f) ws.tgt[pos][f] = src[f];
    }
    if (lane >= n_target && lane < 2 * R) {
        ws.tgt[lane][0] = 0.f;
#pragma unroll
        for (int f = 0; f < D; ++f) ws.tgt[lane][1 + f] = 0.f;
#pragma unroll
        for (int f = 0; f < D * D; ++f) ws.tgt[lane][1 + D + f] = (f / D == f % D) ? 1.f : 0.f;
    }
    __syncwarp();
    return n_target;
}

// Greedy selection from the root (one warp): list of selected nodes in sel_node, their first output slot in
// sel_offset; returns the list length, *written = number of Gaussians they hold.
template <int D, int R>
__device__ __forceinline__ int select_nodes(const float* __restrict__ mix, const uint16_t* __restrict__ nodes, const float* attrs,
                                            int n_internal, int K, int sel_cap, int* sel_node, float* sel_rating,
                                            int* sel_offset, int lane, int* written) {
    constexpr int RF = 1 + D + D * D;
    constexpr int AF = Attr<D, R>::kFloats;
    auto count_of = [&](int n) -> int { return n >= n_internal ? 1 : __float_as_int(attrs[size_t(n) * AF + R * RF + 1]); };
    auto integral_of = [&](int n) -> float {
        return n >= n_internal ? mix[size_t(GMC_OBJ(nodes[size_t(n) * 4 + 3], n_internal)) * RF] : attrs[size_t(n) * AF + R * RF];
    };
    auto rating_of = [&](int n) -> float { return count_of(n) < R ? -2.f : fabsf(integral_of(n)); };
    if (lane == 0) { sel_node[0] = 0; sel_rating[0] = rating_of(0); }
    __syncwarp();
    int n_list = 1;
    int n_selected = count_of(0);
    while (n_selected < K - R && n_list < sel_cap) {
        float best_rating = -1.f;
        int best = 0x7fffffff;
        for (int i = lane; i < n_list; i += 32)
            if (sel_rating[i] > best_rating) { best_rating = sel_rating[i]; best = i; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float orat = __shfl_xor_sync(0xffffffffu, best_rating, o);
            const int oidx = __shfl_xor_sync(0xffffffffu, best, o);
            if (orat > best_rating || (orat == best_rating && oidx < best)) { best_rating = orat; best = oidx; }
        }
        if (best == 0x7fffffff) break;   // no full node left
        const int id = sel_node[best];
        const int l = GMC_NODE(nodes[size_t(id) * 4 + 1], n_internal), r = GMC_NODE(nodes[size_t(id) * 4 + 2], n_internal);
        __syncwarp();
        if (lane == 0) {
            sel_node[best] = l; sel_rating[best] = rating_of(l);
            sel_node[n_list] = r; sel_rating[n_list] = rating_of(r);
        }
        n_selected = n_selected - R + count_of(l) + count_of(r);
        ++n_list;
        __syncwarp();
    }
    if (lane == 0) {
        int w = 0;
        for (int i = 0; i < n_list; ++i) { sel_offset[i] = w; w += count_of(sel_node[i]); }
        *written = w;
    }
    __syncwarp();
    return n_list;
}

// Shared layout: [FitSmem][level bytes: 2G-1 rounded up][arrive: G-1 ints][selection: 3 x sel_cap words][has_grad bytes]
template <int D, int R>
__global__ void __launch_bounds__(kThreads)
mhem_fit_forward_kernel(const float* __restrict__ mixture, const uint16_t* __restrict__ nodes_all, float* __restrict__ attrs_all,
                        float* __restrict__ out_all, int n_components, int n_fitting, unsigned char* big_scratch) {
    constexpr int RF = 1 + D + D * D;
    constexpr int AF = Attr<D, R>::kFloats;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    FitSmem<D, R>& sm = *reinterpret_cast<FitSmem<D, R>*>(smem_bytes);
    const int G = n_components, K = n_fitting;
    const int n_internal = G - 1, n_nodes = 2 * G - 1;
    // per-node bookkeeping: in shared memory, or (mixtures too large for that) in this mixture's slice of big_scratch
    unsigned char* small = smem_bytes + sizeof(WarpScratch<D, R>) * (blockDim.x >> 5);
    unsigned char* level = big_scratch ? big_scratch + size_t(blockIdx.x) * big_scratch_bytes(G) : small;
    int* arrive = reinterpret_cast<int*>(level + ((n_nodes + 15) & ~15));
    const int sel_cap = K > 1024 ? K : 1024;   // capacity of the selection list (the reference holds 1024 entries)
    int* sel_node = big_scratch ? reinterpret_cast<int*>(small) : arrive + n_internal;
    float* sel_rating = reinterpret_cast<float*>(sel_node + sel_cap);
    int* sel_offset = reinterpret_cast<int*>(sel_rating + sel_cap);
    __shared__ int s_max_level, s_n_selected_nodes, s_written;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* mix = mixture + size_t(blockIdx.x) * G * RF;
    const uint16_t* nodes = nodes_all + size_t(blockIdx.x) * n_nodes * 4;
    float* attrs = attrs_all + size_t(blockIdx.x) * n_internal * AF;
    float* out = out_all + size_t(blockIdx.x) * K * RF;

    compute_levels(nodes, G, level, arrive, &s_max_level);
    const int max_level = s_max_level;

    auto child_count = [&](int id) -> int { return id >= n_internal ? 1 : __float_as_int(attrs[size_t(id) * AF + R * RF + 1]); };
    auto child_integral = [&](int id) -> float {
        return id >= n_internal ? mix[size_t(GMC_OBJ(nodes[size_t(id) * 4 + 3], n_internal)) * RF] : attrs[size_t(id) * AF + R * RF];
    };

    // ---- node ids grouped by level (arrive[] is dead after compute_levels and holds the list) ----
    __shared__ int level_start[258], level_cursor[258];
    uint16_t* order = reinterpret_cast<uint16_t*>(arrive);
    group_by_level(level, n_internal, max_level, order, level_start, level_cursor);

    // ---- bottom-up, level by level, one warp per node ----
    WarpScratch<D, R>& ws = sm.warp[warp];
    for (int lv = 1; lv <= max_level; ++lv) {
        {
            const int level_end = level_start[lv + 1];
            for (int at = level_start[lv] + warp; at < level_end; at += int(blockDim.x >> 5)) {
                const int id = order[at];
                int child, child_slot, pos;
                bool in_range, valid;
                const int n_target = gather_children<D, R>(ws, mix, nodes, attrs, n_internal, id, lane, child, child_slot, in_range, valid, pos);
                float* rec = attrs + size_t(id) * AF;
                if (lane == 0) {
                    rec[R * RF] = child_integral(GMC_NODE(nodes[size_t(id) * 4 + 1], n_internal)) + child_integral(GMC_NODE(nodes[size_t(id) * 4 + 2], n_internal));
                    rec[R * RF + 1] = __int_as_float(n_target > R ? R : n_target);
                    rec[R * RF + 3] = 0.f;
                }
                if (n_target > R) {
                    fit_em_warp<D, R>(ws, n_target, rec, reinterpret_cast<int*>(rec + R * RF + 2));
                } else {
                    for (int o = lane; o < R * RF; o += 32) {
                        const int so = o / RF, f = o - so * RF;
                        rec[o] = so < n_target ? ws.tgt[so][f] : 0.f;
                    }
                    if (lane == 0) rec[R * RF + 2] = __int_as_float(-1);
                    __syncwarp();
                }
            }
        }
        __threadfence_block();
        __syncthreads();
    }

    // ---- greedy selection from the root (warp 0), then copy-out ----
    if (warp == 0) {
        const int n_list = select_nodes<D, R>(mix, nodes, attrs, n_internal, K, sel_cap, sel_node, sel_rating, sel_offset, lane, &s_written);
        if (lane == 0) s_n_selected_nodes = n_list;
    }
    __syncthreads();
    const int n_list = s_n_selected_nodes;
    const int written = min(s_written, K);
    for (int i = warp; i < n_list; i += int(blockDim.x >> 5)) {
        const int id = sel_node[i];
        const int cnt = child_count(id);
        const float* src = id >= n_internal ? mix + size_t(GMC_OBJ(nodes[size_t(id) * 4 + 3], n_internal)) * RF : attrs + size_t(id) * AF;
        for (int o = lane; o < cnt * RF; o += 32) {
            const int slot = sel_offset[i] + o / RF;
            if (slot < K) out[size_t(sel_offset[i]) * RF + o] = src[o];
        }
    }
    for (int o = written * RF + tid; o < K * RF; o += int(blockDim.x)) {
        const int f = o % RF;
        float v = 0.f;
        if (f > D && ((f - 1 - D) / D == (f - 1 - D) % D)) v = 1.f;
        out[o] = v;
    }
}

// Backward: the selection is replayed to put the incoming gradient on the selected nodes, then levels are processed
// from the top; a node that holds a gradient passes it to the Gaussians of its children (through grad_em_warp if the
// node was fitted, unchanged otherwise). node_grad [n_internal, R * RF] is scratch; grad_target starts zeroed.
template <int D, int R>
__global__ void __launch_bounds__(kThreads < 256 ? kThreads : 256)
mhem_fit_backward_kernel(const float* __restrict__ grad_all, const float* __restrict__ mixture,
                         const uint16_t* __restrict__ nodes_all, const float* __restrict__ attrs_all,
                         float* __restrict__ node_grad_all, float* __restrict__ grad_target_all, int n_components,
                         int n_fitting, unsigned char* big_scratch) {
    constexpr int RF = 1 + D + D * D;
    constexpr int AF = Attr<D, R>::kFloats;
    constexpr int NT = 2 * R;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    FitSmem<D, R>& sm = *reinterpret_cast<FitSmem<D, R>*>(smem_bytes);
    const int G = n_components, K = n_fitting;
    const int n_internal = G - 1, n_nodes = 2 * G - 1;
    unsigned char* small = smem_bytes + sizeof(WarpScratch<D, R>) * (blockDim.x >> 5);
    unsigned char* level = big_scratch ? big_scratch + size_t(blockIdx.x) * big_scratch_bytes(G) : small;
    int* arrive = reinterpret_cast<int*>(level + ((n_nodes + 15) & ~15));
    const int sel_cap = K > 1024 ? K : 1024;
    int* sel_node = big_scratch ? reinterpret_cast<int*>(small) : arrive + n_internal;
    float* sel_rating = reinterpret_cast<float*>(sel_node + sel_cap);
    int* sel_offset = reinterpret_cast<int*>(sel_rating + sel_cap);
    unsigned char* has_grad = big_scratch ? reinterpret_cast<unsigned char*>(arrive + n_internal)
                                          : reinterpret_cast<unsigned char*>(sel_offset + sel_cap);
    __shared__ int s_max_level, s_n_selected_nodes, s_written;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* mix = mixture + size_t(blockIdx.x) * G * RF;
    const uint16_t* nodes = nodes_all + size_t(blockIdx.x) * n_nodes * 4;
    const float* attrs = attrs_all + size_t(blockIdx.x) * n_internal * AF;
    const float* grad = grad_all + size_t(blockIdx.x) * K * RF;
    float* node_grad = node_grad_all + size_t(blockIdx.x) * n_internal * R * RF;
    float* grad_target = grad_target_all + size_t(blockIdx.x) * G * RF;

    for (int i = tid; i < n_internal; i += int(blockDim.x)) has_grad[i] = 0;
    compute_levels(nodes, G, level, arrive, &s_max_level);
    const int max_level = s_max_level;
    auto count_of = [&](int n) -> int { return n >= n_internal ? 1 : __float_as_int(attrs[size_t(n) * AF + R * RF + 1]); };

    if (warp == 0) {
        const int n_list = select_nodes<D, R>(mix, nodes, attrs, n_internal, K, sel_cap, sel_node, sel_rating, sel_offset, lane, &s_written);
        if (lane == 0) s_n_selected_nodes = n_list;
    }
    __syncthreads();
    const int n_list = s_n_selected_nodes;
    for (int i = warp; i < n_list; i += int(blockDim.x >> 5)) {
        const int id = sel_node[i];
        const int cnt = count_of(id);
        if (id >= n_internal) {      // a selected leaf hands its gradient straight to its Gaussian
            const int obj = GMC_OBJ(nodes[size_t(id) * 4 + 3], n_internal);
            if (sel_offset[i] < K && fabsf(mix[size_t(obj) * RF]) >= kEpsLarge)
                for (int f = lane; f < RF; f += 32) grad_target[size_t(obj) * RF + f] = grad[size_t(sel_offset[i]) * RF + f];
        } else {
            for (int o = lane; o < R * RF; o += 32) {
                const int slot = sel_offset[i] + o / RF;
                node_grad[size_t(id) * R * RF + o] = (o < cnt * RF && slot < K) ? grad[size_t(sel_offset[i]) * RF + o] : 0.f;
            }
            if (lane == 0) has_grad[id] = 1;
        }
    }
    __threadfence_block();
    __syncthreads();

    __shared__ int level_start[258], level_cursor[258];
    uint16_t* order = reinterpret_cast<uint16_t*>(arrive);     // arrive[] is dead after compute_levels
    group_by_level(level, n_internal, max_level, order, level_start, level_cursor);

    WarpScratch<D, R>& ws = sm.warp[warp];
    for (int lv = max_level; lv >= 1; --lv) {
        {
            const int level_end = level_start[lv + 1];
            for (int at = level_start[lv] + warp; at < level_end; at += int(blockDim.x >> 5)) {
                const int id = order[at];
                if (!has_grad[id]) continue;
                int child, child_slot, pos;
                bool in_range, valid;
                const int n_target = gather_children<D, R>(ws, mix, nodes, attrs, n_internal, id, lane, child, child_slot, in_range, valid, pos);
                if (n_target > R) {
                    for (int o = lane; o < R * RF; o += 32) ws.gin[o / RF][o % RF] = node_grad[size_t(id) * R * RF + o];
                    if (lane < R) ws.idx[lane] = (__float_as_int(attrs[size_t(id) * AF + R * RF + 2]) >> (8 * lane)) & 0xFF;
                    __syncwarp();
                    grad_em_warp<D, R>(ws);
                } else {
                    for (int o = lane; o < NT * RF; o += 32) {
                        const int so = o / RF;
                        ws.tgrad[so][o % RF] = so < n_target ? node_grad[size_t(id) * R * RF + o] : 0.f;
                    }
                    __syncwarp();
                }
                // hand the gradients to the children's Gaussians (dropped ones get zero)
                if (in_range) {
                    if (child >= n_internal) {
                        if (valid) {
                            float* dst = grad_target + size_t(GMC_OBJ(nodes[size_t(child) * 4 + 3], n_internal)) * RF;
#pragma unroll
                            for (int f = 0; f < RF; ++f) dst[f] = ws.tgrad[pos][f];
                        }
                    } else {
                        float* dst = node_grad + size_t(child) * R * RF + size_t(child_slot) * RF;
#pragma unroll
                        for (int f = 0; f < RF; ++f) dst[f] = valid ? ws.tgrad[pos][f] : 0.f;
                        has_grad[child] = 1;
                    }
                }
                __syncwarp();
            }
        }
        __threadfence_block();
        __syncthreads();
    }
}

template <int D, int R>
size_t fit_smem_bytes(int G, int K, int threads) {
    const int n_nodes = 2 * G - 1;
    const size_t fixed = sizeof(WarpScratch<D, R>) * size_t(threads / 32) + size_t(K > 1024 ? K : 1024) * 12;
    if (G > kSharedBookkeepingMax) return fixed;                  // per-node arrays live in global scratch
    return fixed + size_t((n_nodes + 15) & ~15) + sizeof(int) * size_t(G - 1) + size_t((G + 15) & ~15);
}

template <int D, int R>
int launch_fit(const float* mixture, long long n_mixtures, int G, int K, const uint16_t* nodes, float* attrs, float* out,
               cudaStream_t stream, unsigned char* big_scratch = nullptr) {
    auto kernel = mhem_fit_forward_kernel<D, R>;
    const size_t smem = fit_smem_bytes<D, R>(G, K, fit_threads(G));
    if (smem > 200 * 1024) return GMC_ERR_BAD_DIMS;
    if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    if (G > kSharedBookkeepingMax && big_scratch == nullptr) return GMC_ERR_NULL_POINTER;
    kernel<<<unsigned(n_mixtures), fit_threads(G), smem, stream>>>(mixture, nodes, attrs, out, G, K,
                                                            G > kSharedBookkeepingMax ? big_scratch : nullptr);
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

template <int D, int R>
int launch_fit_backward(const float* grad, const float* mixture, long long n_mixtures, int G, int K, const uint16_t* nodes,
                        const float* attrs, float* node_grad, float* grad_target, cudaStream_t stream) {
    auto kernel = mhem_fit_backward_kernel<D, R>;
    constexpr int kBackwardThreads = kThreads < 256 ? kThreads : 256;     // 128 registers: two CTAs of 256 per SM
    const size_t smem = fit_smem_bytes<D, R>(G, K, kBackwardThreads);
    if (smem > 200 * 1024) return GMC_ERR_BAD_DIMS;
    if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    // large mixtures: the per-node bookkeeping follows the node gradients in the caller's scratch
    unsigned char* big = G > kSharedBookkeepingMax
                             ? reinterpret_cast<unsigned char*>(node_grad + size_t(n_mixtures) * size_t(G - 1) * R * (1 + D + D * D))
                             : nullptr;
    kernel<<<unsigned(n_mixtures), kBackwardThreads, smem, stream>>>(grad, mixture, nodes, attrs, node_grad, grad_target, G, K, big);
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

}  // namespace
}  // namespace gmc

GMC_DEFINE_TU_CHECK_READER(mhem_fit)

extern "C" size_t gmc_mhem_fit_attribute_floats(int n_components, int n_dims, int reduction_n) {
    if (n_components < 2 || (n_dims != 2 && n_dims != 3) || (reduction_n != 2 && reduction_n != 4)) return 0;
    return size_t(n_components - 1) * size_t(reduction_n * (1 + n_dims + n_dims * n_dims) + 4);
}

extern "C" int gmc_mhem_fit_forward(const float* mixture, long long n_mixtures, int n_components, int n_dims,
                                    int n_components_fitting, int reduction_n, float* fitting, int16_t* bvh_nodes,
                                    float* bvh_attributes, uint64_t* scratch_keys, void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (reduction_n != 2 && reduction_n != 4) return GMC_ERR_UNSUPPORTED;
    if (n_components_fitting <= 0 || n_components_fitting % reduction_n != 0 || n_components_fitting > 4096) return GMC_ERR_BAD_DIMS;
    if (n_mixtures < 0 || n_components < 2) return GMC_ERR_BAD_DIMS;
    if (n_mixtures == 0) return GMC_OK;
    if (!mixture || !fitting || !bvh_nodes || !bvh_attributes || !scratch_keys) return GMC_ERR_NULL_POINTER;
    cudaStream_t st = as_stream(stream);
    uint16_t* nodes = reinterpret_cast<uint16_t*>(bvh_nodes);
    if (int s = lbvh_build_launch(mixture, n_mixtures, n_components, n_dims, 0, scratch_keys, nodes, st)) return s;
    // the Morton keys are dead once the nodes exist: for large mixtures their buffer (8 bytes per component) takes the
    // per-node bookkeeping of the fit kernel (at most 8 bytes per component, see big_scratch_bytes)
    unsigned char* big = reinterpret_cast<unsigned char*>(scratch_keys);
#define GMC_FIT(D_, R_) launch_fit<D_, R_>(mixture, n_mixtures, n_components, n_components_fitting, nodes, bvh_attributes, fitting, st, big)
    if (n_dims == 2) return reduction_n == 2 ? GMC_FIT(2, 2) : GMC_FIT(2, 4);
    return reduction_n == 2 ? GMC_FIT(3, 2) : GMC_FIT(3, 4);
#undef GMC_FIT
}

extern "C" int gmc_mhem_fit_backward(const float* grad, const float* mixture, long long n_mixtures, int n_components,
                                     int n_dims, int n_components_fitting, int reduction_n, const int16_t* bvh_nodes,
                                     const float* bvh_attributes, float* scratch_node_grad, float* grad_mixture,
                                     void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (reduction_n != 2 && reduction_n != 4) return GMC_ERR_UNSUPPORTED;
    if (n_components_fitting <= 0 || n_components_fitting % reduction_n != 0 || n_components_fitting > 4096) return GMC_ERR_BAD_DIMS;
    if (n_mixtures < 0 || n_components < 2) return GMC_ERR_BAD_DIMS;
    if (n_mixtures == 0) return GMC_OK;
    if (!grad || !mixture || !bvh_nodes || !bvh_attributes || !scratch_node_grad || !grad_mixture) return GMC_ERR_NULL_POINTER;
    cudaStream_t st = as_stream(stream);
    const size_t rf = size_t(1 + n_dims + n_dims * n_dims);
    GMC_CUDA_TRY(cudaMemsetAsync(grad_mixture, 0, sizeof(float) * rf * size_t(n_mixtures) * n_components, st));
    const uint16_t* nodes = reinterpret_cast<const uint16_t*>(bvh_nodes);
#define GMC_FITB(D_, R_) launch_fit_backward<D_, R_>(grad, mixture, n_mixtures, n_components, n_components_fitting, nodes, bvh_attributes, scratch_node_grad, grad_mixture, st)
    if (n_dims == 2) return reduction_n == 2 ? GMC_FITB(2, 2) : GMC_FITB(2, 4);
    return reduction_n == 2 ? GMC_FITB(3, 2) : GMC_FITB(3, 4);
#undef GMC_FITB
}

// ---------------------------------------------------------------------------------------------------------------
// Forward fit for callers that cannot hand over scratch memory.
//
// Some hosts of this library have no allocator to turn to when a call needs working memory: a serving process that
// reserved the whole device for its own pools at start-up (a cudaMalloc made later simply fails), a plug-in that
// is only ever given its input and output buffers, or a control loop that must not take the implicit device-wide
// synchronisation an allocation or free can bring. For them the Morton-key scratch of the fit lives inside the
// library image: a fixed array in device memory that every GPU loading the library carries until the process exits.
// ---------------------------------------------------------------------------------------------------------------
namespace gmc {
namespace {

constexpr long long kBuiltinKeyCapacity = 1ll << 20;   // keys: n_mixtures * n_components may not exceed this (8 MiB)

// In host code this name is only a handle for the symbol, not a device address; the address a kernel can use is
// looked up once per device with cudaGetSymbolAddress (below). Device code may use the name directly.
static __device__ __align__(256) unsigned long long g_builtin_fit_keys[kBuiltinKeyCapacity];

constexpr int kMaxDevices = 64;
std::mutex g_builtin_mutex;
uint64_t* g_builtin_keys_address[kMaxDevices] = {};

// Device address of the built-in array on the device that is current for the calling thread.
int builtin_keys_for_current_device(uint64_t** address) {
    int device = -1;
    GMC_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return GMC_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_builtin_mutex);
    if (g_builtin_keys_address[device] == nullptr) {
        void* p = nullptr;
        GMC_CUDA_TRY(cudaGetSymbolAddress(&p, g_builtin_fit_keys));
        if (p == nullptr) return GMC_ERR_CUDA;
        g_builtin_keys_address[device] = static_cast<uint64_t*>(p);
    }
    *address = g_builtin_keys_address[device];
    return GMC_OK;
}

}  // namespace
}  // namespace gmc

extern "C" long long gmc_mhem_fit_forward_noalloc_capacity(void) { return gmc::kBuiltinKeyCapacity; }

extern "C" int gmc_mhem_fit_forward_noalloc(const float* mixture, long long n_mixtures, int n_components, int n_dims,
                                            int n_components_fitting, int reduction_n, float* fitting,
                                            int16_t* bvh_nodes, float* bvh_attributes, void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (reduction_n != 2 && reduction_n != 4) return GMC_ERR_UNSUPPORTED;
    if (n_components_fitting <= 0 || n_components_fitting % reduction_n != 0 || n_components_fitting > 4096) return GMC_ERR_BAD_DIMS;
    if (n_mixtures < 0 || n_components < 2) return GMC_ERR_BAD_DIMS;
    // the one limit that the caller-scratch entry point does not have
    if (n_mixtures * (long long)n_components > kBuiltinKeyCapacity) return GMC_ERR_BUILTIN_SCRATCH;
    if (n_mixtures == 0) return GMC_OK;
    if (!mixture || !fitting || !bvh_nodes || !bvh_attributes) return GMC_ERR_NULL_POINTER;
    uint64_t* keys = nullptr;
    if (int s = builtin_keys_for_current_device(&keys)) return s;
    cudaStream_t st = as_stream(stream);
    uint16_t* nodes = reinterpret_cast<uint16_t*>(bvh_nodes);
    // every key slot that is read is written first by the build kernel, so the array needs no clearing between calls
    if (int s = lbvh_build_launch(mixture, n_mixtures, n_components, n_dims, 0, keys, nodes, st)) return s;
    unsigned char* big = reinterpret_cast<unsigned char*>(keys);     // dead keys = bookkeeping of large mixtures
    if (n_dims == 2) {
        return reduction_n == 2
                   ? launch_fit<2, 2>(mixture, n_mixtures, n_components, n_components_fitting, nodes, bvh_attributes, fitting, st, big)
                   : launch_fit<2, 4>(mixture, n_mixtures, n_components, n_components_fitting, nodes, bvh_attributes, fitting, st, big);
    }
    return reduction_n == 2
               ? launch_fit<3, 2>(mixture, n_mixtures, n_components, n_components_fitting, nodes, bvh_attributes, fitting, st, big)
               : launch_fit<3, 4>(mixture, n_mixtures, n_components, n_components_fitting, nodes, bvh_attributes, fitting, st, big);
}
