// Fused convolution + reduction to K Gaussians per (batch, output channel), forward.
//
// The T = Cin * G * Gk product Gaussians (w_d w_k, mu_d + mu_k, C_d + C_k) of an output channel are never
// materialised. Two kernels: the tree kernel (one CTA per (batch, output channel) tree, everything but the inputs
// and the saved outputs in shared memory) does keys .. selection; the aggregation kernel (one warp per output
// Gaussian) does the last step:
//   keys        (w_d w_k > 0) << 62 | 30-bit Morton code of mu_d + mu_k in the tree's bounding box << 32 | product index
//   sort        ascending, stable 8-bit LSD radix sort in shared memory
//   tree+mass   the binary radix tree over (key high word + sorted position) -- the same hierarchy as the reference's
//               Karras construction -- is built bottom-up: every leaf climbs; a child swaps a 64-bit message (its id,
//               its end of the leaf range, its mass) into the parent's slot with one atomic exchange, the second
//               child to arrive gets the sibling's message back, completes the node (range, children,
//               mass = mass(left) + mass(right)) and queues it; the queue of one round is the dense work list of the
//               next, so construction and the mass pass are one sweep without binary searches and without idle lanes
//   selection   K - 1 greedy splits of the selected internal node with the largest |mass|
//   aggregation per selected subtree the weighted mean / scatter of the product centres and the weighted mean of
//               the product covariances; one warp per output Gaussian, lanes hold partial aggregates that are
//               merged pairwise (the reference walks the leaves sequentially in one thread)
// Same decisions as the reference's convolution_fitting/Tree.cu:63-408 and implementation_forward.h:19-124.
#include "common.cuh"
#include "lbvh_device.cuh"

namespace gmc {
namespace {

#ifndef GMC_CONVFIT_THREADS
#define GMC_CONVFIT_THREADS 512
#endif
constexpr int kThreads = GMC_CONVFIT_THREADS;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxProducts = 8192;
constexpr int kMaxLevels = 72;
#ifndef GMC_CONVFIT_MINB
#define GMC_CONVFIT_MINB 4
#endif

struct Dims {
    int n_batch, n_channels_in, n_components, n_channels_out, n_kernel_components, n_fitting;
};

template <int D>
struct Agg {            // weighted mean / scatter of positions, weighted mean of covariances
    float w;            // sum of weights
    float m[D];         // mean position
    float C[D * D];     // sum w (p - m)(p - m)^T
    float cm[D * D];    // weighted mean covariance
};

template <int D>
__device__ __forceinline__ void agg_add(Agg<D>& a, float w, const float* p, const float* cov) {
    a.w += w;
    if (w == 0.f) return;
    const float f = w / a.w;
    float d1[D], d2[D];
#pragma unroll
    for (int i = 0; i < D; ++i) { d1[i] = p[i] - a.m[i]; a.m[i] += f * d1[i]; d2[i] = p[i] - a.m[i]; }
#pragma unroll
    for (int i = 0; i < D; ++i)
#pragma unroll
        for (int j = 0; j < D; ++j) a.C[i * D + j] += w * (d1[j] * d2[i]);
#pragma unroll
    for (int e = 0; e < D * D; ++e) a.cm[e] += f * (cov[e] - a.cm[e]);
}

// merges b into a (b comes later in leaf order)
template <int D>
__device__ __forceinline__ void agg_merge(Agg<D>& a, const Agg<D>& b) {
    const float w = a.w + b.w;
    if (b.w == 0.f && a.w != 0.f) return;   // nothing to add (keeps a's moments untouched)
    if (w == 0.f) {                         // both empty, or weights that cancel exactly: no defined mean
        if (a.w == 0.f && b.w == 0.f) return;
    }
    const float f = (w != 0.f) ? b.w / w : 0.f;
    float delta[D];
#pragma unroll
    for (int i = 0; i < D; ++i) delta[i] = b.m[i] - a.m[i];
    const float cross = a.w * f;
#pragma unroll
    for (int i = 0; i < D; ++i)
#pragma unroll
        for (int j = 0; j < D; ++j) a.C[i * D + j] += b.C[i * D + j] + cross * delta[i] * delta[j];
#pragma unroll
    for (int i = 0; i < D; ++i) a.m[i] += f * delta[i];
#pragma unroll
    for (int e = 0; e < D * D; ++e) a.cm[e] += f * (b.cm[e] - a.cm[e]);
    a.w = w;
}

template <int D>
__device__ __forceinline__ Agg<D> agg_shfl_down(const Agg<D>& a, int offset) {
    Agg<D> r;
    r.w = __shfl_down_sync(0xffffffffu, a.w, offset);
#pragma unroll
    for (int i = 0; i < D; ++i) r.m[i] = __shfl_down_sync(0xffffffffu, a.m[i], offset);
#pragma unroll
    for (int e = 0; e < D * D; ++e) {
        r.C[e] = __shfl_down_sync(0xffffffffu, a.C[e], offset);
        r.cm[e] = __shfl_down_sync(0xffffffffu, a.cm[e], offset);
    }
    return r;
}

template <int D>
__global__ void __launch_bounds__(kThreads, GMC_CONVFIT_MINB)
convolution_fitting_tree_kernel(const float* __restrict__ data, const float* __restrict__ kernels, Dims n,
                                int* __restrict__ nodesobjs_all, int* __restrict__ subtrees_all) {
    constexpr int RF = 1 + D + D * D;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    const int Cin = n.n_channels_in, G = n.n_components, Gk = n.n_kernel_components, K = n.n_fitting;
    const int T = Cin * G * Gk;
    const int n_internal = T - 1;
    // shared layout: [keys A: T x 8][keys B: T x 8][radix scratch | cpl, selection]
    // after the sort the buffer without the sorted keys holds one 64-bit slot per internal node (hand-over message of
    // the first child, then {mass(left), mass(right)}); once the keys are dead their buffer holds the node arrays
    uint64_t* keys_a = reinterpret_cast<uint64_t*>(smem_bytes);
    uint64_t* keys_b = keys_a + T;
    void* radix_scratch = keys_b + T;
    unsigned char* cpl = reinterpret_cast<unsigned char*>(keys_b + T);            // common prefix of leaf i, i+1
    int* sel_node = reinterpret_cast<int*>(cpl + ((n_internal + 15) & ~15));      // K
    unsigned* sel_rating = reinterpret_cast<unsigned*>(sel_node + K);             // K
    uint16_t* queues = reinterpret_cast<uint16_t*>(sel_rating + K);               // 2 x queue_stride: completed nodes
    const int queue_stride = (T / 2 + 8) & ~7;                                    // of a round (ping-pong)
    __shared__ int queue_count[kMaxLevels + 1];
    __shared__ float s_hi[kWarps][D], s_lo[kWarps][D], box_hi[D], box_lo[D];
    __shared__ int s_root;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x / n.n_channels_out, o = blockIdx.x - b * n.n_channels_out;
    const float* data_b = data + size_t(b) * Cin * G * RF;
    const float* kernels_o = kernels + size_t(o) * Cin * Gk * RF;
    int* nodesobjs = nodesobjs_all + size_t(blockIdx.x) * T;
    int* subtrees = subtrees_all + size_t(blockIdx.x) * 2 * K;

    // ---- bounding box: max over channels of (data max + kernel max), min likewise ----
    {
        float hi[D], lo[D];
#pragma unroll
        for (int d = 0; d < D; ++d) { hi[d] = -INFINITY; lo[d] = INFINITY; }
        for (int ci = warp; ci < Cin; ci += kWarps) {
            float dh[D], dl[D], kh[D], kl[D];
#pragma unroll
            for (int d = 0; d < D; ++d) { dh[d] = kh[d] = -INFINITY; dl[d] = kl[d] = INFINITY; }
            for (int g = lane; g < G; g += 32)
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const float v = __ldg(data_b + (size_t(ci) * G + g) * RF + 1 + d);
                    dh[d] = fmaxf(dh[d], v); dl[d] = fminf(dl[d], v);
                }
            for (int g = lane; g < Gk; g += 32)
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const float v = __ldg(kernels_o + (size_t(ci) * Gk + g) * RF + 1 + d);
                    kh[d] = fmaxf(kh[d], v); kl[d] = fminf(kl[d], v);
                }
#pragma unroll
            for (int d = 0; d < D; ++d) {
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    dh[d] = fmaxf(dh[d], __shfl_xor_sync(0xffffffffu, dh[d], off));
                    dl[d] = fminf(dl[d], __shfl_xor_sync(0xffffffffu, dl[d], off));
                    kh[d] = fmaxf(kh[d], __shfl_xor_sync(0xffffffffu, kh[d], off));
                    kl[d] = fminf(kl[d], __shfl_xor_sync(0xffffffffu, kl[d], off));
                }
                hi[d] = fmaxf(hi[d], __fadd_rn(dh[d], kh[d]));
                lo[d] = fminf(lo[d], __fadd_rn(dl[d], kl[d]));
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int d = 0; d < D; ++d) { s_hi[warp][d] = hi[d]; s_lo[warp][d] = lo[d]; }
        }
        __syncthreads();
        if (tid < D) {
            float h = s_hi[0][tid], l = s_lo[0][tid];
            for (int w = 1; w < kWarps; ++w) { h = fmaxf(h, s_hi[w][tid]); l = fminf(l, s_lo[w][tid]); }
            box_hi[tid] = h; box_lo[tid] = l;
        }
        __syncthreads();
    }

    auto product_parts = [&](int t, int& comp_in, int& ch_in, int& comp_k) {
        comp_k = t / (G * Cin);
        const int rem = t - comp_k * G * Cin;
        ch_in = rem / G;
        comp_in = rem - ch_in * G;
    };

    // ---- keys, sort (stable on bits 32..63 = sign | Morton code; equal codes keep ascending product index) ----
    for (int t = tid; t < T; t += kThreads) {
        int gi, ci, ki;
        product_parts(t, gi, ci, ki);
        const float* dg = data_b + (size_t(ci) * G + gi) * RF;
        const float* kg = kernels_o + (size_t(ci) * Gk + ki) * RF;
        uint32_t q[3] = {0u, 0u, 0u};
#pragma unroll
        for (int d = 0; d < D; ++d) q[d] = lbvh::quantise(__fadd_rn(__ldg(dg + 1 + d), __ldg(kg + 1 + d)), box_lo[d], box_hi[d]);
        const uint64_t sign = __fmul_rn(__ldg(dg), __ldg(kg)) > 0.f ? 1ull : 0ull;
        keys_a[t] = (sign << 62) | (uint64_t(lbvh::morton30(q[0], q[1], q[2])) << 32) | uint64_t(uint32_t(t));
    }
    __syncthreads();
    const uint64_t* keys = lbvh::radix_sort_shared(keys_a, keys_b, T, 32, 4, radix_scratch);   // 4 passes: back in A

    // ---- leaves; common prefix lengths of neighbouring codes; empty slots ----
    uint64_t* slots = keys == keys_a ? keys_b : keys_a;
    uint32_t* children = reinterpret_cast<uint32_t*>(const_cast<uint64_t*>(keys));   // left | right << 16
    uint32_t* ranges = children + n_internal;                                        // first | last << 16 (leaf range)
    for (int j = tid; j < T; j += kThreads) nodesobjs[j] = int(uint32_t(keys[j]));
    for (int i = tid; i < n_internal; i += kThreads) slots[i] = 0ull;
    for (int i = tid; i <= kMaxLevels; i += kThreads) queue_count[i] = 0;
    {
        const lbvh::PositionTieBreakCode code{keys};
        for (int i = tid; i < n_internal; i += kThreads) cpl[i] = (unsigned char)lbvh::common_upper_bits(code(i), code(i + 1));
    }
    __syncthreads();   // keys are dead from here on: their buffer becomes the node arrays

    // ---- bottom-up construction with the mass pass folded in ----
    // Internal node p is the split between leaves p and p + 1. A node with leaf range [l, r] hangs below node r (as its
    // left child) if the codes differ less across r | r+1 than across l-1 | l, else below node l - 1 (as right child).
    // message: bit 63 valid | node id << 45 | own end of the leaf range << 32 | mass bits
    // Round 0 sends every leaf to its parent; round k sends the nodes completed in round k - 1 (read back from the
    // node arrays). Nobody waits: the first child to arrive just leaves its message.
    const unsigned lt_mask = (1u << lane) - 1u;
    auto arrive = [&](bool active, uint32_t node, int l, int r, float m, uint16_t* queue_out, int* count_out) {
        bool completed = false;
        int p = 0;
        if (active) {
            const bool up_right = (l == 0) || (r != T - 1 && cpl[r] > cpl[l - 1]);
            p = up_right ? r : l - 1;
            const uint32_t hi = 0x80000000u | (node << 13) | uint32_t(up_right ? l : r);
            const unsigned long long old = atomicExch(reinterpret_cast<unsigned long long*>(slots + p),
                                                      (uint64_t(hi) << 32) | __float_as_uint(m));
            if (old != 0ull) {                       // second child: complete node p
                const uint32_t sib_hi = uint32_t(old >> 32);
                const uint32_t sib_node = (sib_hi >> 13) & 0x3fffu, sib_end = sib_hi & 0x1fffu;
                const float sib_mass = __uint_as_float(uint32_t(old));
                if (up_right) {                      // this child is the left one
                    children[p] = node | (sib_node << 16);
                    r = int(sib_end);
                    *reinterpret_cast<float2*>(slots + p) = make_float2(m, sib_mass);
                } else {
                    children[p] = sib_node | (node << 16);
                    l = int(sib_end);
                    *reinterpret_cast<float2*>(slots + p) = make_float2(sib_mass, m);
                }
                ranges[p] = uint32_t(l) | (uint32_t(r) << 16);
                if (l == 0 && r == T - 1) s_root = p;
                else completed = true;
            }
        }
        const unsigned done = __ballot_sync(0xffffffffu, completed);
        if (done != 0u) {
            int at = 0;
            if (lane == 0) at = atomicAdd(count_out, __popc(done));
            at = __shfl_sync(0xffffffffu, at, 0);
            if (completed) queue_out[at + __popc(done & lt_mask)] = uint16_t(p);
        }
    };
    for (int leaf0 = 0; leaf0 < T; leaf0 += kThreads) {
        const int leaf = leaf0 + tid;
        float m = 0.f;
        if (leaf < T) {
            int gi, ci, ki;
            product_parts(nodesobjs[leaf], gi, ci, ki);
            m = __fmul_rn(__ldg(data_b + (size_t(ci) * G + gi) * RF), __ldg(kernels_o + (size_t(ci) * Gk + ki) * RF));
        }
        arrive(leaf < T, uint32_t(n_internal + leaf), leaf, leaf, m, queues, &queue_count[1]);
    }
    __syncthreads();
    for (int round = 1; round < kMaxLevels; ++round) {
        const int n_in = queue_count[round];
        if (n_in == 0) break;
        const uint16_t* queue_in = queues + ((round - 1) & 1) * queue_stride;
        for (int i0 = 0; i0 < n_in; i0 += kThreads) {
            const int i = i0 + tid;
            uint32_t node = 0u, lr = 0u;
            float m = 0.f;
            if (i < n_in) {
                node = queue_in[i];
                lr = ranges[node];
                const float2 masses = *reinterpret_cast<const float2*>(slots + node);
                m = __fadd_rn(masses.x, masses.y);
            }
            arrive(i < n_in, node, int(lr & 0xffffu), int(lr >> 16), m, queues + (round & 1) * queue_stride,
                   &queue_count[round + 1]);
        }
        __syncthreads();
    }

    // ---- greedy selection of K subtree roots (warp 0) ----
    // rating as an order-preserving integer: internal node -> bits(|mass|) + 1, leaf -> 0 (never selected)
    if (warp == 0) {
        auto rating_of = [&](int id, float mass) -> unsigned {
            return id >= n_internal ? 0u : __float_as_uint(fabsf(mass)) + 1u;
        };
        // the root is expanded first whatever its mass: any non-zero rating does
        if (lane == 0) { sel_node[0] = s_root; sel_rating[0] = s_root >= n_internal ? 0u : 1u; }
        __syncwarp();
        int n_sel = 1;
        while (n_sel < K) {
            unsigned best_rating = 0u;
            int best = 0x7fffffff;
            for (int i = lane; i < n_sel; i += 32)
                if (sel_rating[i] > best_rating) { best_rating = sel_rating[i]; best = i; }
            const unsigned top = __reduce_max_sync(0xffffffffu, best_rating);
            if (top == 0u) break;                                        // only leaves left
            best = __reduce_min_sync(0xffffffffu, best_rating == top ? best : 0x7fffffff);   // first of the maxima
            if (lane == 0) {
                const int id = sel_node[best];
                const int l = int(children[id] & 0xffffu), r = int(children[id] >> 16);
                const float2 masses = *reinterpret_cast<const float2*>(slots + id);
                sel_node[best] = l; sel_rating[best] = rating_of(l, masses.x);
                sel_node[n_sel] = r; sel_rating[n_sel] = rating_of(r, masses.y);
            }
            ++n_sel;
            __syncwarp();
        }
        // leaf ranges [start, end) of the selected roots
        for (int k = lane; k < K; k += 32) {
            int start = -1, end = -1;
            if (k < n_sel) {
                const int id = sel_node[k];
                start = id >= n_internal ? id : n_internal + int(ranges[id] & 0xffffu);
                end = id >= n_internal ? id + 1 : n_internal + int(ranges[id] >> 16) + 1;
            }
            subtrees[2 * k] = start;
            subtrees[2 * k + 1] = end;
        }
    }
}

// Aggregation kernel: one warp per output Gaussian (batch, output channel, k), reading the leaf order and the
// subtree ranges that the tree kernel wrote. Lanes take contiguous slices of the leaf range and keep partial weighted
// mean / scatter aggregates that are merged pairwise in leaf order.
template <int D>
__global__ void __launch_bounds__(256)
convolution_fitting_aggregate_kernel(const float* __restrict__ data, const float* __restrict__ kernels, Dims n,
                                     const int* __restrict__ nodesobjs_all, const int* __restrict__ subtrees_all,
                                     float* __restrict__ fitting, float* __restrict__ cached_pos_covs,
                                     long long n_outputs) {
    constexpr int RF = 1 + D + D * D;
    const int Cin = n.n_channels_in, G = n.n_components, Gk = n.n_kernel_components, K = n.n_fitting;
    const int T = Cin * G * Gk;
    const int n_internal = T - 1;
    const int lane = threadIdx.x & 31;
    const long long out_id = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (out_id >= n_outputs) return;
    const long long tree = out_id / K;
    const int k = int(out_id - tree * K);
    const int b = int(tree / n.n_channels_out), o = int(tree - (long long)b * n.n_channels_out);
    const float* data_b = data + size_t(b) * Cin * G * RF;
    const float* kernels_o = kernels + size_t(o) * Cin * Gk * RF;
    const int* nodesobjs = nodesobjs_all + size_t(tree) * T;
    const int start = subtrees_all[size_t(tree) * 2 * K + 2 * k], end = subtrees_all[size_t(tree) * 2 * K + 2 * k + 1];
    float* o_k = fitting + size_t(out_id) * RF;
    float* c_k = cached_pos_covs + size_t(out_id) * D * D;
    if (start < 0) {
        for (int f = lane; f < RF; f += 32) {
            float v = 0.f;
            if (f > D && ((f - 1 - D) / D == (f - 1 - D) % D)) v = 1.f;
            o_k[f] = v;
        }
        for (int e = lane; e < D * D; e += 32) c_k[e] = 0.f;
        return;
    }
    Agg<D> a;
    a.w = 0.f;
#pragma unroll
    for (int i = 0; i < D; ++i) a.m[i] = 0.f;
#pragma unroll
    for (int e = 0; e < D * D; ++e) { a.C[e] = 0.f; a.cm[e] = 0.f; }
    // lane l takes a contiguous slice of the range so that merging neighbours keeps the leaf order
    const int len = end - start;
    const int per = (len + 31) / 32;
    const int s0 = start + lane * per, s1 = min(end, s0 + per);
    for (int i = s0; i < s1; ++i) {
        const int t = nodesobjs[i - n_internal];
        const int ki = t / (G * Cin);
        const int rem = t - ki * G * Cin;
        const int ci = rem / G;
        const int gi = rem - ci * G;
        const float* dg = data_b + (size_t(ci) * G + gi) * RF;
        const float* kg = kernels_o + (size_t(ci) * Gk + ki) * RF;
        float p[D], cov[D * D];
#pragma unroll
        for (int d = 0; d < D; ++d) p[d] = __ldg(dg + 1 + d) + __ldg(kg + 1 + d);
#pragma unroll
        for (int e = 0; e < D * D; ++e) cov[e] = __ldg(dg + 1 + D + e) + __ldg(kg + 1 + D + e);
        agg_add<D>(a, __ldg(dg) * __ldg(kg), p, cov);
    }
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const Agg<D> other = agg_shfl_down<D>(a, off);
        if ((lane & (2 * off - 1)) == 0) agg_merge<D>(a, other);
    }
    if (lane == 0) {
        o_k[0] = a.w;
#pragma unroll
        for (int d = 0; d < D; ++d) o_k[1 + d] = a.m[d];
#pragma unroll
        for (int e = 0; e < D * D; ++e) {
            const float pc = (a.w == 0.f) ? ((e / D == e % D) ? 1.f : 0.f) : a.C[e] / a.w;
            c_k[e] = pc;
            o_k[1 + D + e] = a.cm[e] + pc;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------------------------
// With the tree frozen, output k is (W, S1 / W, S3 / W + S2 / W - m m^T) with the leaf sums W = sum w, S1 = sum w p,
// S2 = sum w p p^T, S3 = sum w C over its leaves (p = mu_d + mu_k, C = C_d + C_k, w = w_d w_k). The gradient of every
// sum depends on the output only, so each output gets one coefficient record
//     a1 = dL/dS1, A2 = dL/dS2 = dL/dS3, c0 = dL/dW (all paths)
// and a product's gradient is dw = [a1.p + <A2, p p^T + C>] (w != 0) + c0, dp = w (a1 + (A2 + A2^T) p), dC = w A2
// (the derivative the reference spells out in util/grad/welford.h:14-97). Products are visited from the side of the
// tensor they contribute to -- by data Gaussian, then by kernel Gaussian -- so all sums stay in registers and global
// memory sees one atomic per value and CTA.
template <int D>
struct SlotCoef {
    float a1[D];
    float A2[D * D];
    float c0;
};

template <int D>
__device__ __forceinline__ void product_gradient(const SlotCoef<D>& c, float w, const float* p, const float* cov,
                                                 float& dw, float* dp, float* dC) {
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < D; ++i) q += c.a1[i] * p[i];
#pragma unroll
    for (int i = 0; i < D; ++i)
#pragma unroll
        for (int j = 0; j < D; ++j) q += c.A2[i * D + j] * (p[i] * p[j] + cov[i * D + j]);
    dw = (w != 0.f ? q : 0.f) + c.c0;
#pragma unroll
    for (int i = 0; i < D; ++i) {
        float acc = c.a1[i];
#pragma unroll
        for (int j = 0; j < D; ++j) acc += (c.A2[i * D + j] + c.A2[j * D + i]) * p[j];
        dp[i] = w * acc;
    }
#pragma unroll
    for (int e = 0; e < D * D; ++e) dC[e] = w * c.A2[e];
}

template <int D>
__global__ void __launch_bounds__(kThreads)
convolution_fitting_backward_kernel(const float* __restrict__ grad, const float* __restrict__ data,
                                    const float* __restrict__ kernels, Dims n, const float* __restrict__ fitting,
                                    const float* __restrict__ cached_pos_covs, const int* __restrict__ nodesobjs_all,
                                    const int* __restrict__ subtrees_all, float* __restrict__ grad_data,
                                    float* __restrict__ grad_kernels) {
    constexpr int RF = 1 + D + D * D;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    const int Cin = n.n_channels_in, G = n.n_components, Gk = n.n_kernel_components, K = n.n_fitting;
    const int T = Cin * G * Gk;
    const int n_internal = T - 1;
    SlotCoef<D>* coef = reinterpret_cast<SlotCoef<D>*>(smem_bytes);                              // K records
    uint16_t* slot_of = reinterpret_cast<uint16_t*>(smem_bytes + ((sizeof(SlotCoef<D>) * K + 15) & ~size_t(15)));   // T

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x / n.n_channels_out, o = blockIdx.x - b * n.n_channels_out;
    const float* data_b = data + size_t(b) * Cin * G * RF;
    const float* kernels_o = kernels + size_t(o) * Cin * Gk * RF;
    const int* nodesobjs = nodesobjs_all + size_t(blockIdx.x) * T;
    const int* subtrees = subtrees_all + size_t(blockIdx.x) * 2 * K;

    for (int t = tid; t < T; t += kThreads) slot_of[t] = 0xFFFFu;
    for (int k = tid; k < K; k += kThreads) {
        SlotCoef<D> c;
#pragma unroll
        for (int i = 0; i < D; ++i) c.a1[i] = 0.f;
#pragma unroll
        for (int e = 0; e < D * D; ++e) c.A2[e] = 0.f;
        c.c0 = 0.f;
        const float* f = fitting + (size_t(blockIdx.x) * K + k) * RF;
        const float* g = grad + (size_t(blockIdx.x) * K + k) * RF;
        const float* pc = cached_pos_covs + (size_t(blockIdx.x) * K + k) * D * D;
        const float W = f[0];
        if (subtrees[2 * k] >= 0 && W != 0.f) {
            const float inv_w = 1.f / W;
            float m[D], gC[D * D], vmg[D];
#pragma unroll
            for (int i = 0; i < D; ++i) m[i] = f[1 + i];
#pragma unroll
            for (int e = 0; e < D * D; ++e) gC[e] = g[1 + D + e];
            float dot_gc_s2 = 0.f, dot_gc_cm = 0.f, dot_vmg_m = 0.f;
#pragma unroll
            for (int i = 0; i < D; ++i) {
                float acc = g[1 + i];
#pragma unroll
                for (int j = 0; j < D; ++j) acc -= (gC[i * D + j] + gC[j * D + i]) * m[j];
                vmg[i] = acc;
                dot_vmg_m += acc * m[i];
            }
#pragma unroll
            for (int i = 0; i < D; ++i)
#pragma unroll
                for (int j = 0; j < D; ++j) {
                    const int e = i * D + j;
                    dot_gc_s2 += gC[e] * (pc[e] + m[i] * m[j]);
                    dot_gc_cm += gC[e] * (f[1 + D + e] - pc[e]);
                }
#pragma unroll
            for (int i = 0; i < D; ++i) c.a1[i] = vmg[i] * inv_w;
#pragma unroll
            for (int e = 0; e < D * D; ++e) c.A2[e] = gC[e] * inv_w;
            c.c0 = g[0] - (dot_gc_s2 + dot_vmg_m + dot_gc_cm) * inv_w;
        }
        coef[k] = c;
    }
    __syncthreads();
    for (int k = warp; k < K; k += kWarps) {
        const int start = subtrees[2 * k], end = subtrees[2 * k + 1];
        if (start < 0) continue;
        for (int j = start - n_internal + lane; j < end - n_internal; j += 32) slot_of[nodesobjs[j]] = uint16_t(k);
    }
    __syncthreads();

    auto load_product = [&](int gi, int ci, int ki, float& w, float& wd, float& wk, float* p, float* cov) {
        const float* dg = data_b + (size_t(ci) * G + gi) * RF;
        const float* kg = kernels_o + (size_t(ci) * Gk + ki) * RF;
        wd = __ldg(dg); wk = __ldg(kg);
        w = wd * wk;
#pragma unroll
        for (int d = 0; d < D; ++d) p[d] = __ldg(dg + 1 + d) + __ldg(kg + 1 + d);
#pragma unroll
        for (int e = 0; e < D * D; ++e) cov[e] = __ldg(dg + 1 + D + e) + __ldg(kg + 1 + D + e);
    };

    // ---- by data Gaussian: thread r = (ci, g) sums over the kernel components ----
    if (grad_data != nullptr) {
        for (int r = tid; r < Cin * G; r += kThreads) {
            const int ci = r / G, gi = r - ci * G;
            float acc[RF];
#pragma unroll
            for (int f = 0; f < RF; ++f) acc[f] = 0.f;
            for (int ki = 0; ki < Gk; ++ki) {
                const int slot = slot_of[gi + G * (ci + Cin * ki)];
                if (slot == 0xFFFF) continue;
                float w, wd, wk, p[D], cov[D * D], dw, dp[D], dC[D * D];
                load_product(gi, ci, ki, w, wd, wk, p, cov);
                product_gradient<D>(coef[slot], w, p, cov, dw, dp, dC);
                acc[0] += dw * wk;
#pragma unroll
                for (int d = 0; d < D; ++d) acc[1 + d] += dp[d];
#pragma unroll
                for (int e = 0; e < D * D; ++e) acc[1 + D + e] += dC[e];
            }
            float* dst = grad_data + ((size_t(b) * Cin + ci) * G + gi) * RF;
#pragma unroll
            for (int f = 0; f < RF; ++f) atomicAdd(dst + f, acc[f]);
        }
    }
    // ---- by kernel Gaussian: warp per (ci, k), lanes stride over the data components ----
    if (grad_kernels != nullptr) {
        for (int r = warp; r < Cin * Gk; r += kWarps) {
            const int ci = r / Gk, ki = r - ci * Gk;
            float acc[RF];
#pragma unroll
            for (int f = 0; f < RF; ++f) acc[f] = 0.f;
            for (int gi = lane; gi < G; gi += 32) {
                const int slot = slot_of[gi + G * (ci + Cin * ki)];
                if (slot == 0xFFFF) continue;
                float w, wd, wk, p[D], cov[D * D], dw, dp[D], dC[D * D];
                load_product(gi, ci, ki, w, wd, wk, p, cov);
                product_gradient<D>(coef[slot], w, p, cov, dw, dp, dC);
                acc[0] += dw * wd;
#pragma unroll
                for (int d = 0; d < D; ++d) acc[1 + d] += dp[d];
#pragma unroll
                for (int e = 0; e < D * D; ++e) acc[1 + D + e] += dC[e];
            }
#pragma unroll
            for (int f = 0; f < RF; ++f) {
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) acc[f] += __shfl_xor_sync(0xffffffffu, acc[f], off);
            }
            if (lane == 0) {
                float* dst = grad_kernels + ((size_t(o) * Cin + ci) * Gk + ki) * RF;
#pragma unroll
                for (int f = 0; f < RF; ++f) atomicAdd(dst + f, acc[f]);
            }
        }
    }
}

size_t convfit_smem_bytes(int T, int K) {
    const int n_internal = T - 1;
    size_t bytes = 2 * size_t(T) * 8;
    const size_t after_sort = size_t((n_internal + 15) & ~15) + 8 * size_t(K)    // cpl, selection,
                              + 2 * 2 * size_t((T / 2 + 8) & ~7);                 // two node queues
    const size_t radix = 2 * size_t(kWarps + 1) * 256 + 32;                      // dead once the keys are sorted
    bytes += after_sort > radix ? after_sort : radix;
    return bytes;
}

}  // namespace
}  // namespace gmc

GMC_DEFINE_TU_CHECK_READER(convolution_fitting)

extern "C" int gmc_convolution_fitting_forward(const float* data, const float* kernels, int n_batch, int n_channels_in,
                                               int n_components, int n_channels_out, int n_kernel_components,
                                               int n_dims, int n_components_fitting, float* fitting,
                                               float* cached_pos_covs, int32_t* nodesobjs, int32_t* fitting_subtrees,
                                               void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_batch <= 0 || n_channels_in <= 0 || n_components <= 0 || n_channels_out <= 0 || n_kernel_components <= 0)
        return GMC_ERR_BAD_DIMS;
    const long long T = (long long)n_channels_in * n_components * n_kernel_components;
    if (T < 2 || T > kMaxProducts) return GMC_ERR_BAD_DIMS;
    if (n_components_fitting <= 0 || n_components_fitting > 8192) return GMC_ERR_BAD_DIMS;
    if (!data || !kernels || !fitting || !cached_pos_covs || !nodesobjs || !fitting_subtrees) return GMC_ERR_NULL_POINTER;
    const long long blocks = (long long)n_batch * n_channels_out;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    const size_t smem = convfit_smem_bytes(int(T), n_components_fitting);
    if (smem > 220 * 1024) return GMC_ERR_BAD_DIMS;
    const Dims n{n_batch, n_channels_in, n_components, n_channels_out, n_kernel_components, n_components_fitting};
    cudaStream_t st = as_stream(stream);
    const long long n_outputs = blocks * n_components_fitting;
    const long long agg_blocks = (n_outputs + 7) / 8;
    if (agg_blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    if (n_dims == 2) {
        if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(convolution_fitting_tree_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        convolution_fitting_tree_kernel<2><<<unsigned(blocks), kThreads, smem, st>>>(data, kernels, n, nodesobjs, fitting_subtrees);
        GMC_LAUNCH_CHECK();
        convolution_fitting_aggregate_kernel<2><<<unsigned(agg_blocks), 256, 0, st>>>(data, kernels, n, nodesobjs, fitting_subtrees, fitting, cached_pos_covs, n_outputs);
    } else {
        if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(convolution_fitting_tree_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        convolution_fitting_tree_kernel<3><<<unsigned(blocks), kThreads, smem, st>>>(data, kernels, n, nodesobjs, fitting_subtrees);
        GMC_LAUNCH_CHECK();
        convolution_fitting_aggregate_kernel<3><<<unsigned(agg_blocks), 256, 0, st>>>(data, kernels, n, nodesobjs, fitting_subtrees, fitting, cached_pos_covs, n_outputs);
    }
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

extern "C" int gmc_convolution_fitting_backward(const float* grad, const float* data, const float* kernels, int n_batch,
                                                int n_channels_in, int n_components, int n_channels_out,
                                                int n_kernel_components, int n_dims, int n_components_fitting,
                                                const float* fitting, const float* cached_pos_covs,
                                                const int32_t* nodesobjs, const int32_t* fitting_subtrees,
                                                float* grad_data, float* grad_kernels, void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_batch <= 0 || n_channels_in <= 0 || n_components <= 0 || n_channels_out <= 0 || n_kernel_components <= 0)
        return GMC_ERR_BAD_DIMS;
    const long long T = (long long)n_channels_in * n_components * n_kernel_components;
    if (T < 2 || T > 65534) return GMC_ERR_BAD_DIMS;
    if (n_components_fitting <= 0 || n_components_fitting > 8192) return GMC_ERR_BAD_DIMS;
    if (!grad || !data || !kernels || !fitting || !cached_pos_covs || !nodesobjs || !fitting_subtrees) return GMC_ERR_NULL_POINTER;
    const long long blocks = (long long)n_batch * n_channels_out;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    cudaStream_t st = as_stream(stream);
    const size_t rf = size_t(1 + n_dims + n_dims * n_dims);
    if (grad_data) GMC_CUDA_TRY(cudaMemsetAsync(grad_data, 0, sizeof(float) * rf * n_batch * n_channels_in * n_components, st));
    if (grad_kernels) GMC_CUDA_TRY(cudaMemsetAsync(grad_kernels, 0, sizeof(float) * rf * n_channels_out * n_channels_in * n_kernel_components, st));
    if (!grad_data && !grad_kernels) return GMC_OK;
    const Dims n{n_batch, n_channels_in, n_components, n_channels_out, n_kernel_components, n_components_fitting};
    const size_t coef_bytes = (n_dims == 2 ? sizeof(SlotCoef<2>) : sizeof(SlotCoef<3>)) * size_t(n_components_fitting);
    const size_t smem = ((coef_bytes + 15) & ~size_t(15)) + 2 * size_t(T);
    if (smem > 220 * 1024) return GMC_ERR_BAD_DIMS;
    if (n_dims == 2) {
        if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(convolution_fitting_backward_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        convolution_fitting_backward_kernel<2><<<unsigned(blocks), kThreads, smem, st>>>(grad, data, kernels, n, fitting, cached_pos_covs, nodesobjs, fitting_subtrees, grad_data, grad_kernels);
    } else {
        if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(convolution_fitting_backward_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        convolution_fitting_backward_kernel<3><<<unsigned(blocks), kThreads, smem, st>>>(grad, data, kernels, n, fitting, cached_pos_covs, nodesobjs, fitting_subtrees, grad_data, grad_kernels);
    }
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}
