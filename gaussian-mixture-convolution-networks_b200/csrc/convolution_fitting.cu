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
//               the product covariances; one warp per output Gaussian, lanes sum a strided share of the leaves in
//               cluster-local coordinates (the reference walks the leaves sequentially in one thread)
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

// Warp-wide maximum / minimum of floats (no NaN) with one integer reduction instruction each: the bit pattern with
// the magnitude bits of negative numbers flipped orders like the float.
__device__ __forceinline__ int ordered_bits(float v) {
    const int i = __float_as_int(v);
    return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float from_ordered_bits(int i) { return __int_as_float(i ^ ((i >> 31) & 0x7fffffff)); }
__device__ __forceinline__ float warp_max(float v) { return from_ordered_bits(__reduce_max_sync(0xffffffffu, ordered_bits(v))); }
__device__ __forceinline__ float warp_min(float v) { return from_ordered_bits(__reduce_min_sync(0xffffffffu, ordered_bits(v))); }

// Quotient and remainder of small non-negative integers (below 2^23) by a fixed divisor without the integer
// division sequence: the float estimate is off by at most one.
struct FastDivisor {
    int d;
    float inv;
    __device__ __forceinline__ explicit FastDivisor(int divisor) : d(divisor), inv(1.0f / float(divisor)) {}
    __device__ __forceinline__ void split(int x, int& q, int& r) const {
        q = __float2int_rz(__fmul_rn(float(x), inv));
        r = x - q * d;
        if (r < 0) { r += d; --q; }
        else if (r >= d) { r -= d; ++q; }
    }
};

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

    // ---- (weight, centre) of the tree's input Gaussians: data records [Cin * G], then kernel records [Cin * Gk], one
    //      float4 each, in key buffer B (free until the sort) when they fit; else every use gathers from global ----
    const int n_data = Cin * G;
    const bool staged = size_t(n_data + Cin * Gk) * sizeof(float4) <= size_t(T) * sizeof(uint64_t);
    const float4* records = reinterpret_cast<const float4*>(keys_b);
    if (staged) {
        float4* dst = reinterpret_cast<float4*>(keys_b);
        for (int i = tid; i < n_data + Cin * Gk; i += kThreads) {
            const float* r = i < n_data ? data_b + size_t(i) * RF : kernels_o + size_t(i - n_data) * RF;
            dst[i] = make_float4(__ldg(r), __ldg(r + 1), __ldg(r + 2), D == 3 ? __ldg(r + 3) : 0.f);
        }
        __syncthreads();
    }
    auto record = [&](bool kernel_side, int idx) -> float4 {
        if (staged) return records[kernel_side ? n_data + idx : idx];
        const float* r = kernel_side ? kernels_o + size_t(idx) * RF : data_b + size_t(idx) * RF;
        return make_float4(__ldg(r), __ldg(r + 1), __ldg(r + 2), D == 3 ? __ldg(r + 3) : 0.f);
    };
    auto coordinate = [](const float4& v, int d) -> float { return d == 0 ? v.y : (d == 1 ? v.z : v.w); };

    // ---- bounding box: max over channels of (data max + kernel max), min likewise ----
    {
        float hi[D], lo[D];
#pragma unroll
        for (int d = 0; d < D; ++d) { hi[d] = -INFINITY; lo[d] = INFINITY; }
        if (staged && G <= 32 && (G & (G - 1)) == 0 && Cin <= 256) {
            // the channels' data records are segments of G lanes: one record per thread, a shuffle reduction inside the
            // segment, the segment's first lane keeps the channel's extremes (in the radix scratch, free until the sort)
            float* chan = reinterpret_cast<float*>(radix_scratch);          // [Cin][max D | min D]
            for (int i0 = 0; i0 < n_data; i0 += kThreads) {
                const int i = i0 + tid;
                float vh[D], vl[D];
#pragma unroll
                for (int d = 0; d < D; ++d) { vh[d] = -INFINITY; vl[d] = INFINITY; }
                if (i < n_data) {
                    const float4 v = records[i];
#pragma unroll
                    for (int d = 0; d < D; ++d) vh[d] = vl[d] = coordinate(v, d);
                }
                for (int o = G >> 1; o > 0; o >>= 1) {
#pragma unroll
                    for (int d = 0; d < D; ++d) {
                        vh[d] = fmaxf(vh[d], __shfl_xor_sync(0xffffffffu, vh[d], o));
                        vl[d] = fminf(vl[d], __shfl_xor_sync(0xffffffffu, vl[d], o));
                    }
                }
                if (i < n_data && (i & (G - 1)) == 0) {
                    float* c = chan + (i / G) * 2 * D;
#pragma unroll
                    for (int d = 0; d < D; ++d) { c[d] = vh[d]; c[D + d] = vl[d]; }
                }
            }
            __syncthreads();
            for (int ci = tid; ci < Cin; ci += kThreads) {
                float kh[D], kl[D];
#pragma unroll
                for (int d = 0; d < D; ++d) { kh[d] = -INFINITY; kl[d] = INFINITY; }
                for (int g = 0; g < Gk; ++g) {
                    const float4 v = records[n_data + ci * Gk + g];
#pragma unroll
                    for (int d = 0; d < D; ++d) { kh[d] = fmaxf(kh[d], coordinate(v, d)); kl[d] = fminf(kl[d], coordinate(v, d)); }
                }
                const float* c = chan + ci * 2 * D;
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    hi[d] = fmaxf(hi[d], __fadd_rn(c[d], kh[d]));
                    lo[d] = fminf(lo[d], __fadd_rn(c[D + d], kl[d]));
                }
            }
#pragma unroll
            for (int d = 0; d < D; ++d) { hi[d] = warp_max(hi[d]); lo[d] = warp_min(lo[d]); }
            __syncthreads();             // the scratch is handed back before the sort uses it
        } else
        for (int ci = warp; ci < Cin; ci += kWarps) {
            float dh[D], dl[D], kh[D], kl[D];
#pragma unroll
            for (int d = 0; d < D; ++d) { dh[d] = kh[d] = -INFINITY; dl[d] = kl[d] = INFINITY; }
            for (int g = lane; g < G; g += 32) {
                const float4 v = record(false, ci * G + g);
#pragma unroll
                for (int d = 0; d < D; ++d) { dh[d] = fmaxf(dh[d], coordinate(v, d)); dl[d] = fminf(dl[d], coordinate(v, d)); }
            }
            for (int g = lane; g < Gk; g += 32) {
                const float4 v = record(true, ci * Gk + g);
#pragma unroll
                for (int d = 0; d < D; ++d) { kh[d] = fmaxf(kh[d], coordinate(v, d)); kl[d] = fminf(kl[d], coordinate(v, d)); }
            }
#pragma unroll
            for (int d = 0; d < D; ++d) {
                hi[d] = fmaxf(hi[d], __fadd_rn(warp_max(dh[d]), warp_max(kh[d])));
                lo[d] = fminf(lo[d], __fadd_rn(warp_min(dl[d]), warp_min(kl[d])));
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

    const FastDivisor by_gc(G * Cin), by_g(G);
    auto product_parts = [&](int t, int& comp_in, int& ch_in, int& comp_k) {
        int rem;
        by_gc.split(t, comp_k, rem);
        by_g.split(rem, ch_in, comp_in);
    };

    // ---- keys, sort (stable on bits 32..63 = sign | Morton code; equal codes keep ascending product index) ----
    for (int t = tid; t < T; t += kThreads) {
        int gi, ci, ki;
        product_parts(t, gi, ci, ki);
        const float4 dg = record(false, ci * G + gi), kg = record(true, ci * Gk + ki);
        uint32_t q[3] = {0u, 0u, 0u};
#pragma unroll
        for (int d = 0; d < D; ++d) q[d] = lbvh::quantise(__fadd_rn(coordinate(dg, d), coordinate(kg, d)), box_lo[d], box_hi[d]);
        const uint64_t sign = __fmul_rn(dg.x, kg.x) > 0.f ? 1ull : 0ull;
        keys_a[t] = (sign << 62) | (uint64_t(lbvh::morton30(q[0], q[1], q[2])) << 32) | uint64_t(uint32_t(t));
    }
    __syncthreads();
    // (sorting on the top 16 or 24 code bits first and ordering the runs of equal top bits afterwards was measured: the
    // products of the deeper network layers crowd into few Morton cells, runs of 128 equal top-16 prefixes per tree, and
    // with 24 bits the run pass costs what the saved radix pass did)
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
            product_parts(GMC_IDX(nodesobjs[leaf], T), gi, ci, ki);
            m = __fmul_rn(__ldg(data_b + (size_t(ci) * G + gi) * RF), __ldg(kernels_o + (size_t(ci) * Gk + ki) * RF));
        }
        arrive(leaf < T, uint32_t(n_internal + leaf), leaf, leaf, m, queues, &queue_count[1]);
    }
    __syncthreads();
    for (int round = 1; round < kMaxLevels; ++round) {
        const int n_in = queue_count[round];
        if (n_in == 0) break;
        if (n_in <= 32) {
            // the number of completed nodes never grows from round to round (every arrival completes at most one node):
            // warp 0, which also runs the selection, finishes the narrow top of the tree without CTA barriers
            if (warp == 0) {
                for (int tail = round; tail < kMaxLevels; ++tail) {
                    const int n_tail = queue_count[tail];
                    if (n_tail == 0) break;
                    const uint16_t* queue_in = queues + ((tail - 1) & 1) * queue_stride;
                    uint32_t node = 0u, lr = 0u;
                    float m = 0.f;
                    if (lane < n_tail) {
                        node = queue_in[lane];
                        lr = ranges[node];
                        const float2 masses = *reinterpret_cast<const float2*>(slots + node);
                        m = __fadd_rn(masses.x, masses.y);
                    }
                    arrive(lane < n_tail, node, int(lr & 0xffffu), int(lr >> 16), m, queues + (tail & 1) * queue_stride,
                           &queue_count[tail + 1]);
                    __syncwarp();
                }
            }
            break;
        }
        const uint16_t* queue_in = queues + ((round - 1) & 1) * queue_stride;
        for (int i0 = 0; i0 < n_in; i0 += kThreads) {
            if (i0 + warp * 32 >= n_in) break;               // nothing queued for this warp (warp-uniform)
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

// ---------------------------------------------------------------------------------------------------------------
// Trees of more than kMaxProducts products (up to 65535): the same construction with every array in global scratch
// instead of shared memory, one CTA of 1024 threads per tree. Per tree the scratch holds (T = number of products):
//   keys A, keys B [T] uint64 | left, right, first, last [T-1] int32 | parent [2T-1] int32 | mass [2T-1] fp32 |
//   arrivals [T-1] int32                                      (convfit_large_scratch_bytes(T) bytes, 16-byte aligned)
// Steps: bounding box and keys as in the shared-memory kernel; stable radix sort of the keys in global memory; Karras
// range / split search per internal node on (sign | Morton code, sorted position); masses bottom-up, the second child to
// arrive adds mass(left) + mass(right); greedy selection by warp 0.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kLargeTreeThreads = 1024;
constexpr int kMaxProductsLarge = 65535;      // ranks and digit offsets of the sort are 16 bit

__host__ __device__ inline size_t convfit_large_scratch_bytes(long long T) {
    const size_t t = size_t(T);
    return ((16 * t + 4 * 4 * (t - 1) + 4 * (2 * t - 1) + 4 * (2 * t - 1) + 4 * (t - 1)) + 15) & ~size_t(15);
}

template <int D>
__global__ void __launch_bounds__(kLargeTreeThreads)
convolution_fitting_tree_large_kernel(const float* __restrict__ data, const float* __restrict__ kernels, Dims n,
                                      int* __restrict__ nodesobjs_all, int* __restrict__ subtrees_all,
                                      unsigned char* __restrict__ scratch_all) {
    constexpr int RF = 1 + D + D * D;
    constexpr int NW = kLargeTreeThreads / 32;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    const int Cin = n.n_channels_in, G = n.n_components, Gk = n.n_kernel_components, K = n.n_fitting;
    const int T = Cin * G * Gk;
    const int n_internal = T - 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x / n.n_channels_out, o = blockIdx.x - b * n.n_channels_out;
    const float* data_b = data + size_t(b) * Cin * G * RF;
    const float* kernels_o = kernels + size_t(o) * Cin * Gk * RF;
    int* nodesobjs = nodesobjs_all + size_t(blockIdx.x) * T;
    int* subtrees = subtrees_all + size_t(blockIdx.x) * 2 * K;
    unsigned char* scratch = scratch_all + size_t(blockIdx.x) * convfit_large_scratch_bytes(T);
    uint64_t* keys_a = reinterpret_cast<uint64_t*>(scratch);
    uint64_t* keys_b = keys_a + T;
    int* left = reinterpret_cast<int*>(keys_b + T);
    int* right = left + n_internal;
    int* first = right + n_internal;
    int* last = first + n_internal;
    int* parent = last + n_internal;                     // [2T-1]
    float* mass = reinterpret_cast<float*>(parent + (2 * T - 1));   // [2T-1]
    int* arrivals = reinterpret_cast<int*>(mass + (2 * T - 1));     // [T-1]
    // shared: ranks of the sort [T] uint16 (later the selection list), then the sort's histograms
    uint16_t* ranks = reinterpret_cast<uint16_t*>(smem_bytes);
    const size_t list_bytes = size_t(K) * 8 > size_t(T) * 2 ? size_t(K) * 8 : size_t(T) * 2;
    void* sort_scratch = smem_bytes + ((list_bytes + 15) & ~size_t(15));
    int* sel_node = reinterpret_cast<int*>(smem_bytes);
    unsigned* sel_rating = reinterpret_cast<unsigned*>(sel_node + K);
    __shared__ float s_hi[NW][D], s_lo[NW][D], box_hi[D], box_lo[D];

    // ---- bounding box: max over channels of (data max + kernel max), min likewise ----
    {
        float hi[D], lo[D];
#pragma unroll
        for (int d = 0; d < D; ++d) { hi[d] = -INFINITY; lo[d] = INFINITY; }
        for (int ci = warp; ci < Cin; ci += NW) {
            float dh[D], dl[D], kh[D], kl[D];
#pragma unroll
            for (int d = 0; d < D; ++d) { dh[d] = kh[d] = -INFINITY; dl[d] = kl[d] = INFINITY; }
            for (int g = lane; g < G; g += 32) {
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const float v = __ldg(data_b + (size_t(ci) * G + g) * RF + 1 + d);
                    dh[d] = fmaxf(dh[d], v); dl[d] = fminf(dl[d], v);
                }
            }
            for (int g = lane; g < Gk; g += 32) {
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const float v = __ldg(kernels_o + (size_t(ci) * Gk + g) * RF + 1 + d);
                    kh[d] = fmaxf(kh[d], v); kl[d] = fminf(kl[d], v);
                }
            }
#pragma unroll
            for (int d = 0; d < D; ++d) {
                hi[d] = fmaxf(hi[d], __fadd_rn(warp_max(dh[d]), warp_max(kh[d])));
                lo[d] = fminf(lo[d], __fadd_rn(warp_min(dl[d]), warp_min(kl[d])));
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int d = 0; d < D; ++d) { s_hi[warp][d] = hi[d]; s_lo[warp][d] = lo[d]; }
        }
        __syncthreads();
        if (tid < D) {
            float h = s_hi[0][tid], l = s_lo[0][tid];
            for (int w = 1; w < NW; ++w) { h = fmaxf(h, s_hi[w][tid]); l = fminf(l, s_lo[w][tid]); }
            box_hi[tid] = h; box_lo[tid] = l;
        }
        __syncthreads();
    }
    auto product_parts = [&](int t, int& comp_in, int& ch_in, int& comp_k) {
        comp_k = t / (G * Cin);
        const int rem = t - comp_k * (G * Cin);
        ch_in = rem / G;
        comp_in = rem - ch_in * G;
    };
    // ---- keys; leaf masses ----
    for (int t = tid; t < T; t += kLargeTreeThreads) {
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
    for (int i = tid; i < n_internal; i += kLargeTreeThreads) arrivals[i] = 0;
    __threadfence_block();
    __syncthreads();
    const uint64_t* keys = lbvh::radix_sort_global(keys_a, keys_b, T, 32, 4, ranks, sort_scratch);   // back in A
    for (int j = tid; j < T; j += kLargeTreeThreads) {
        const int t = int(uint32_t(keys[j]));
        nodesobjs[j] = t;
        int gi, ci, ki;
        product_parts(t, gi, ci, ki);
        mass[n_internal + j] = __fmul_rn(__ldg(data_b + (size_t(ci) * G + gi) * RF), __ldg(kernels_o + (size_t(ci) * Gk + ki) * RF));
    }
    // ---- internal nodes ----
    {
        const lbvh::PositionTieBreakCode code{keys};
        for (int i = tid; i < n_internal; i += kLargeTreeThreads) {
            const int2 r = lbvh::determine_range(code, T, i);
            const int gamma = lbvh::find_split(code, r.x, r.y);
            int l = gamma, rr = gamma + 1;
            if (min(r.x, r.y) == gamma) l += n_internal;
            if (max(r.x, r.y) == gamma + 1) rr += n_internal;
            left[i] = l; right[i] = rr; first[i] = r.x; last[i] = r.y;
            parent[l] = i; parent[rr] = i;
            if (i == 0) parent[0] = -1;
        }
    }
    __threadfence_block();
    __syncthreads();
    // ---- masses, bottom-up: the second child to arrive at a node completes it and climbs on ----
    for (int leaf = tid; leaf < T; leaf += kLargeTreeThreads) {
        int node = parent[n_internal + leaf];
        for (int guard = 0; guard < 4 * kMaxLevels && node >= 0; ++guard) {
            __threadfence_block();
            if (atomicAdd(&arrivals[node], 1) == 0) break;
            __threadfence_block();
            const float ml = ((volatile float*)mass)[left[node]], mr = ((volatile float*)mass)[right[node]];
            ((volatile float*)mass)[node] = __fadd_rn(ml, mr);
            node = parent[node];
        }
    }
    __threadfence_block();
    __syncthreads();
    // ---- greedy selection of K subtree roots (warp 0); the list replaces the sort's ranks ----
    if (warp == 0) {
        auto rating_of = [&](int id) -> unsigned { return id >= n_internal ? 0u : __float_as_uint(fabsf(mass[id])) + 1u; };
        if (lane == 0) { sel_node[0] = 0; sel_rating[0] = 1u; }       // the root is expanded first whatever its mass
        __syncwarp();
        int n_sel = 1;
        while (n_sel < K) {
            unsigned best_rating = 0u;
            int best = 0x7fffffff;
            for (int i = lane; i < n_sel; i += 32)
                if (sel_rating[i] > best_rating) { best_rating = sel_rating[i]; best = i; }
            const unsigned top = __reduce_max_sync(0xffffffffu, best_rating);
            if (top == 0u) break;
            best = __reduce_min_sync(0xffffffffu, best_rating == top ? best : 0x7fffffff);
            if (lane == 0) {
                const int id = sel_node[best];
                const int l = left[id], r = right[id];
                sel_node[best] = l; sel_rating[best] = rating_of(l);
                sel_node[n_sel] = r; sel_rating[n_sel] = rating_of(r);
            }
            ++n_sel;
            __syncwarp();
        }
        for (int k = lane; k < K; k += 32) {
            int start = -1, end = -1;
            if (k < n_sel) {
                const int id = sel_node[k];
                start = id >= n_internal ? id : n_internal + first[id];
                end = id >= n_internal ? id + 1 : n_internal + last[id] + 1;
            }
            subtrees[2 * k] = start;
            subtrees[2 * k + 1] = end;
        }
    }
}

// Staged input record. 3D: the 13 floats of a Gaussian are read as 4 float4; records are 20 floats apart, an odd
// number of float4, so that arbitrary records spread evenly over the 8 groups of 4 banks (a stride of 16 floats would
// put all records on two of them). 2D: the 7 floats are read one by one at their natural (odd) stride, which measured
// faster than 2 float4 at a stride of 12.
template <int D>
struct StagedRecord {
    static constexpr int kFloats = D == 2 ? 7 : 16;
    static constexpr int kStride = D == 2 ? 7 : 20;
};

// All floats of input Gaussian `index`: from the padded shared-memory copy (float4 reads: a quarter of the
// shared-memory wavefronts of scalar reads at arbitrary records) or from global memory.
template <int D, bool STAGED>
__device__ __forceinline__ void load_gaussian(const float* base, int index, float* out) {
    constexpr int RF = 1 + D + D * D;
    if constexpr (STAGED && D == 2) {
        const float* src = base + size_t(index) * RF;
#pragma unroll
        for (int f = 0; f < RF; ++f) out[f] = src[f];
    } else if constexpr (STAGED) {
        constexpr int RP = StagedRecord<D>::kFloats;
        const float4* src = reinterpret_cast<const float4*>(base + size_t(index) * StagedRecord<D>::kStride);
        float padded[RP];
#pragma unroll
        for (int v = 0; v < RP / 4; ++v) {
            const float4 t = src[v];
            padded[4 * v] = t.x; padded[4 * v + 1] = t.y; padded[4 * v + 2] = t.z; padded[4 * v + 3] = t.w;
        }
#pragma unroll
        for (int f = 0; f < RF; ++f) out[f] = padded[f];
    } else {
        const float* src = base + size_t(index) * RF;
#pragma unroll
        for (int f = 0; f < RF; ++f) out[f] = __ldg(src + f);
    }
}

// One warp, one output Gaussian: sums over the leaves [start, end) of its subtree (see the kernel below).
template <int D, bool STAGED>
__device__ __forceinline__ void aggregate_output(const float* data_b, const float* kernels_o, const int* nodesobjs,
                                                 const int* subtree, float* o_k, float* c_k, const FastDivisor& by_gc,
                                                 const FastDivisor& by_g, int G, int Gk, int lane) {
    constexpr int RF = 1 + D + D * D;
    constexpr int NS = D * (D + 1) / 2;
    const int start = subtree[0], end = subtree[1];
    if (start < 0) {
        for (int f = lane; f < RF; f += 32) {
            float v = 0.f;
            if (f > D && ((f - 1 - D) / D == (f - 1 - D) % D)) v = 1.f;
            o_k[f] = v;
        }
        for (int e = lane; e < D * D; e += 32) c_k[e] = 0.f;
        return;
    }
    auto records = [&](int t, float* dg, float* kg) {
        int ki, rem, ci, gi;
        t = GMC_IDX(t, by_gc.d * Gk);              // product index below Cin * G * Gk
        by_gc.split(t, ki, rem);
        by_g.split(rem, ci, gi);
        load_gaussian<D, STAGED>(data_b, ci * G + gi, dg);
        load_gaussian<D, STAGED>(kernels_o, ci * Gk + ki, kg);
    };
    float p0[D];
    {
        float dg[RF], kg[RF];
        records(__ldg(nodesobjs + start), dg, kg);
#pragma unroll
        for (int d = 0; d < D; ++d) p0[d] = dg[1 + d] + kg[1 + d];
    }
    float W = 0.f, S1[D], S2[NS], S3[D * D];
#pragma unroll
    for (int d = 0; d < D; ++d) S1[d] = 0.f;
#pragma unroll
    for (int e = 0; e < NS; ++e) S2[e] = 0.f;
#pragma unroll
    for (int e = 0; e < D * D; ++e) S3[e] = 0.f;
    int t_next = start + lane < end ? __ldg(nodesobjs + start + lane) : 0;
    for (int i = start + lane; i < end; i += 32) {
        float dg[RF], kg[RF];
        const int t = t_next;
        if (i + 32 < end) t_next = __ldg(nodesobjs + i + 32);     // the next leaf's index is on its way while this one is summed
        records(t, dg, kg);
        const float w = dg[0] * kg[0];
        float q[D], wq[D];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            q[d] = (dg[1 + d] + kg[1 + d]) - p0[d];
            wq[d] = w * q[d];
            S1[d] += wq[d];
        }
        W += w;
        int e2 = 0;
#pragma unroll
        for (int a = 0; a < D; ++a)
#pragma unroll
            for (int c = a; c < D; ++c) { S2[e2] = fmaf(wq[a], q[c], S2[e2]); ++e2; }
#pragma unroll
        for (int e = 0; e < D * D; ++e) S3[e] = fmaf(w, dg[1 + D + e] + kg[1 + D + e], S3[e]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        W += __shfl_xor_sync(0xffffffffu, W, off);
#pragma unroll
        for (int d = 0; d < D; ++d) S1[d] += __shfl_xor_sync(0xffffffffu, S1[d], off);
#pragma unroll
        for (int e = 0; e < NS; ++e) S2[e] += __shfl_xor_sync(0xffffffffu, S2[e], off);
#pragma unroll
        for (int e = 0; e < D * D; ++e) S3[e] += __shfl_xor_sync(0xffffffffu, S3[e], off);
    }
    if (lane == 0) {
        o_k[0] = W;
        if (W == 0.f) {
#pragma unroll
            for (int d = 0; d < D; ++d) o_k[1 + d] = 0.f;
#pragma unroll
            for (int e = 0; e < D * D; ++e) {
                const float pc = (e / D == e % D) ? 1.f : 0.f;
                c_k[e] = pc;
                o_k[1 + D + e] = pc;
            }
            return;
        }
        const float inv = 1.f / W;
        float mq[D];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            mq[d] = S1[d] * inv;
            o_k[1 + d] = p0[d] + mq[d];
        }
        int e2 = 0;
        float pc[D * D];
#pragma unroll
        for (int a = 0; a < D; ++a)
#pragma unroll
            for (int c = a; c < D; ++c) {
                const float v = S2[e2++] * inv - mq[a] * mq[c];
                pc[a * D + c] = v;
                pc[c * D + a] = v;
            }
#pragma unroll
        for (int e = 0; e < D * D; ++e) {
            c_k[e] = pc[e];
            o_k[1 + D + e] = S3[e] * inv + pc[e];
        }
    }
}


// Aggregation kernel: one warp per output Gaussian (batch, output channel, k), reading the leaf order and the
// subtree ranges that the tree kernel wrote. With q = p - p0 (p0 = centre of the first leaf of the range, so the sums
// stay in cluster-local coordinates) the lanes accumulate
//     W = sum w, S1 = sum w q, S2 = sum w q q^T, S3 = sum w C
// over a strided share of the leaves and a butterfly adds the 32 partial sums. Output: weight W, position
// p0 + S1 / W, covariance S3 / W + [S2 / W - (S1 / W)(S1 / W)^T]; the bracket (the scatter of the centres) is saved in
// cached_pos_covs for the backward pass. W == 0 gives (0, 0, identity) like the sequential weighted update of the
// reference (implementation_forward.h:60-124), which never leaves its initial state in that case.
//
// A CTA (8 warps) serves up to kAggOutputsPerCta outputs of ONE tree. When the tree's input records (Cin * (G + Gk)
// Gaussians) fit, they are staged in shared memory first (STAGED): the leaves of a subtree name arbitrary records,
// and gathering 26 floats per leaf from global memory is bound by L1 wavefronts.
#ifndef GMC_AGG_OUTPUTS_PER_CTA
#define GMC_AGG_OUTPUTS_PER_CTA 128
#endif
constexpr int kAggOutputsPerCta = GMC_AGG_OUTPUTS_PER_CTA;
constexpr size_t kAggMaxStagedBytes = 96 * 1024;

template <int D, bool STAGED>
__global__ void __launch_bounds__(256)
convolution_fitting_aggregate_kernel(const float* __restrict__ data, const float* __restrict__ kernels, Dims n,
                                     const int* __restrict__ nodesobjs_all, const int* __restrict__ subtrees_all,
                                     float* __restrict__ fitting, float* __restrict__ cached_pos_covs,
                                     int groups_per_tree) {
    constexpr int RF = 1 + D + D * D;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    const int Cin = n.n_channels_in, G = n.n_components, Gk = n.n_kernel_components, K = n.n_fitting;
    const int T = Cin * G * Gk;
    const int n_internal = T - 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long tree = blockIdx.x / groups_per_tree;
    const int group = blockIdx.x - int(tree) * groups_per_tree;
    const int b = int(tree / n.n_channels_out), o = int(tree - (long long)b * n.n_channels_out);
    const float* data_b = data + size_t(b) * Cin * G * RF;
    const float* kernels_o = kernels + size_t(o) * Cin * Gk * RF;
    if constexpr (STAGED) {
        constexpr int RP = StagedRecord<D>::kStride;
        float* staged = reinterpret_cast<float*>(smem_bytes);
        const int n_data = Cin * G * RF, n_kernel = Cin * Gk * RF;
        // eight loads in flight per thread: the copy is bound by the latency of the global loads
        for (int i0 = threadIdx.x; i0 < n_data + n_kernel; i0 += 256 * 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + u * 256;
                v[u] = i < n_data ? __ldg(data_b + i) : (i < n_data + n_kernel ? __ldg(kernels_o + (i - n_data)) : 0.f);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + u * 256;
                const int record = i / RF;                   // kernel records follow the data records
                if (i < n_data + n_kernel) staged[record * RP + (i - record * RF)] = v[u];
            }
        }
        __syncthreads();
        data_b = staged;
        kernels_o = staged + size_t(Cin) * G * RP;
    }
    const int* nodesobjs = nodesobjs_all + size_t(tree) * T - n_internal;     // indexed by node id of the leaf
    const FastDivisor by_gc(G * Cin), by_g(G);
    const int k_end = min(K, (group + 1) * kAggOutputsPerCta);
    for (int k = group * kAggOutputsPerCta + warp; k < k_end; k += 8)
        aggregate_output<D, STAGED>(data_b, kernels_o, nodesobjs, subtrees_all + (size_t(tree) * K + k) * 2,
                                    fitting + (size_t(tree) * K + k) * RF, cached_pos_covs + (size_t(tree) * K + k) * D * D,
                                    by_gc, by_g, G, Gk, lane);
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
        for (int j = start - n_internal + lane; j < end - n_internal; j += 32) slot_of[GMC_IDX(nodesobjs[GMC_IDX(j, T)], T)] = uint16_t(k);
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

template <int D>
int launch_convfit_forward(const float* data, const float* kernels, const Dims& n, int32_t* nodesobjs,
                           int32_t* fitting_subtrees, float* fitting, float* cached_pos_covs, long long blocks,
                           size_t smem, long long agg_blocks, int groups_per_tree, bool staged, size_t staged_bytes,
                           cudaStream_t st) {
    if (smem > 48 * 1024)
        GMC_CUDA_TRY(cudaFuncSetAttribute(convolution_fitting_tree_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    convolution_fitting_tree_kernel<D><<<unsigned(blocks), kThreads, smem, st>>>(data, kernels, n, nodesobjs, fitting_subtrees);
    GMC_LAUNCH_CHECK();
    if (staged) {
        if (staged_bytes > 48 * 1024)
            GMC_CUDA_TRY(cudaFuncSetAttribute(convolution_fitting_aggregate_kernel<D, true>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, int(staged_bytes)));
        convolution_fitting_aggregate_kernel<D, true><<<unsigned(agg_blocks), 256, staged_bytes, st>>>(
            data, kernels, n, nodesobjs, fitting_subtrees, fitting, cached_pos_covs, groups_per_tree);
    } else {
        convolution_fitting_aggregate_kernel<D, false><<<unsigned(agg_blocks), 256, 0, st>>>(
            data, kernels, n, nodesobjs, fitting_subtrees, fitting, cached_pos_covs, groups_per_tree);
    }
    GMC_LAUNCH_CHECK();
    return GMC_OK;
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
    const int groups_per_tree = (n_components_fitting + kAggOutputsPerCta - 1) / kAggOutputsPerCta;
    const long long agg_blocks = blocks * groups_per_tree;
    if (agg_blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    const size_t staged_bytes = sizeof(float) * size_t(n_channels_in) * (n_components + n_kernel_components) *
                                size_t(n_dims == 2 ? StagedRecord<2>::kStride : StagedRecord<3>::kStride);
    const bool staged = staged_bytes <= kAggMaxStagedBytes;
    if (n_dims == 2) {
        if (int s = launch_convfit_forward<2>(data, kernels, n, nodesobjs, fitting_subtrees, fitting, cached_pos_covs,
                                              blocks, smem, agg_blocks, groups_per_tree, staged, staged_bytes, st))
            return s;
    } else {
        if (int s = launch_convfit_forward<3>(data, kernels, n, nodesobjs, fitting_subtrees, fitting, cached_pos_covs,
                                              blocks, smem, agg_blocks, groups_per_tree, staged, staged_bytes, st))
            return s;
    }
    return GMC_OK;
}

extern "C" size_t gmc_convolution_fitting_large_scratch_bytes(int n_batch, int n_channels_in, int n_components,
                                                              int n_channels_out, int n_kernel_components) {
    const long long T = (long long)n_channels_in * n_components * n_kernel_components;
    if (n_batch <= 0 || n_channels_out <= 0 || T < 2 || T > gmc::kMaxProductsLarge) return 0;
    return size_t(n_batch) * size_t(n_channels_out) * gmc::convfit_large_scratch_bytes(T);
}

extern "C" int gmc_convolution_fitting_forward_large(const float* data, const float* kernels, int n_batch,
                                                     int n_channels_in, int n_components, int n_channels_out,
                                                     int n_kernel_components, int n_dims, int n_components_fitting,
                                                     float* fitting, float* cached_pos_covs, int32_t* nodesobjs,
                                                     int32_t* fitting_subtrees, void* scratch, size_t scratch_bytes,
                                                     void* stream) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_batch <= 0 || n_channels_in <= 0 || n_components <= 0 || n_channels_out <= 0 || n_kernel_components <= 0)
        return GMC_ERR_BAD_DIMS;
    const long long T = (long long)n_channels_in * n_components * n_kernel_components;
    if (T < 2 || T > kMaxProductsLarge) return GMC_ERR_BAD_DIMS;
    if (n_components_fitting <= 0 || n_components_fitting > 8192) return GMC_ERR_BAD_DIMS;
    if (!data || !kernels || !fitting || !cached_pos_covs || !nodesobjs || !fitting_subtrees || !scratch) return GMC_ERR_NULL_POINTER;
    const long long blocks = (long long)n_batch * n_channels_out;
    if (blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    if (scratch_bytes < size_t(blocks) * convfit_large_scratch_bytes(T)) return GMC_ERR_BAD_DIMS;
    if ((reinterpret_cast<uintptr_t>(scratch) & 15u) != 0) return GMC_ERR_BAD_DIMS;
    const Dims n{n_batch, n_channels_in, n_components, n_channels_out, n_kernel_components, n_components_fitting};
    cudaStream_t st = as_stream(stream);
    const size_t list = size_t(n_components_fitting) * 8 > size_t(T) * 2 ? size_t(n_components_fitting) * 8 : size_t(T) * 2;
    const size_t smem = ((list + 15) & ~size_t(15)) + 2 * size_t((kLargeTreeThreads / 32) + 1) * 256 + 32;
    if (smem > 220 * 1024) return GMC_ERR_BAD_DIMS;
    unsigned char* sc = static_cast<unsigned char*>(scratch);
    if (n_dims == 2) {
        GMC_CUDA_TRY(cudaFuncSetAttribute(convolution_fitting_tree_large_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        convolution_fitting_tree_large_kernel<2><<<unsigned(blocks), kLargeTreeThreads, smem, st>>>(data, kernels, n, nodesobjs, fitting_subtrees, sc);
    } else {
        GMC_CUDA_TRY(cudaFuncSetAttribute(convolution_fitting_tree_large_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        convolution_fitting_tree_large_kernel<3><<<unsigned(blocks), kLargeTreeThreads, smem, st>>>(data, kernels, n, nodesobjs, fitting_subtrees, sc);
    }
    GMC_LAUNCH_CHECK();
    // aggregation: the kernel of the regular path, reading the sorted products and the subtree ranges from global memory
    const int groups_per_tree = (n_components_fitting + kAggOutputsPerCta - 1) / kAggOutputsPerCta;
    const long long agg_blocks = blocks * groups_per_tree;
    if (agg_blocks > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    const size_t staged_bytes = sizeof(float) * size_t(n_channels_in) * (n_components + n_kernel_components) *
                                size_t(n_dims == 2 ? StagedRecord<2>::kStride : StagedRecord<3>::kStride);
    const bool staged = staged_bytes <= kAggMaxStagedBytes;
#define GMC_AGG(D_)                                                                                                        \
    if (staged) {                                                                                                          \
        if (staged_bytes > 48 * 1024)                                                                                      \
            GMC_CUDA_TRY(cudaFuncSetAttribute(convolution_fitting_aggregate_kernel<D_, true>,                              \
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, int(staged_bytes)));            \
        convolution_fitting_aggregate_kernel<D_, true><<<unsigned(agg_blocks), 256, staged_bytes, st>>>(                   \
            data, kernels, n, nodesobjs, fitting_subtrees, fitting, cached_pos_covs, groups_per_tree);                     \
    } else {                                                                                                               \
        convolution_fitting_aggregate_kernel<D_, false><<<unsigned(agg_blocks), 256, 0, st>>>(                             \
            data, kernels, n, nodesobjs, fitting_subtrees, fitting, cached_pos_covs, groups_per_tree);                     \
    }
    if (n_dims == 2) { GMC_AGG(2) } else { GMC_AGG(3) }
#undef GMC_AGG
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
