// Linear BVH over the means of each mixture: whole AABB, 30-bit Morton keys (<< 16 | component id; or one of the
// covariance-aware key layouts of lbvh::Config::MortonCodeAlgorithm), ascending sort, Karras internal nodes. One CTA per mixture keeps the keys in shared memory from the Morton stage to the
// last node, so global traffic is the means in, the sorted keys and the node array out. Mixtures of more than 8192
// components (up to the 32768 that 16-bit node indices allow) take lbvh_build_large_kernel: same steps, keys in global
// memory, radix-sorted between the key output buffer and the (not yet written) node buffer.
// Replaces lbvh::Bvh::construct (src/gmc/cpp/extensions/lbvh/bvh.cu:23-144, 241-299, 373-458); with make_aabbs a
// second kernel adds the ellipsoid boxes of the leaves and merges them bottom-up (lbvh/bvh.cu:164-231, 460-510).
#include "common.cuh"
#include "lbvh_device.cuh"
#include "symeig_device.cuh"

namespace gmc {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxComponents = 8192;          // keys of one mixture fit in shared memory (64 KB) up to here
constexpr int kMaxComponentsLarge = 32768;    // node indices are 16 bit with 0xFFFF = none: 2G - 2 <= 65534 (the reference
                                              // accepts up to 65534 components, implementation_forward.h:498-500, but its
                                              // uint16 node indices, lbvh/bvh.h:16-24, wrap beyond this size)


// Per-mixture extent of the means (and, for the covariance-aware key layouts, the maxima of the matrix diagonal).
template <int D>
struct Extent {
    float lo[D], hi[D], diag_max[D];
    float red[3][D][32];
};

template <int D, int THREADS>
__device__ __forceinline__ void mixture_extent(const float* __restrict__ mix, int G, int layout, Extent<D>& ext) {
    constexpr int RF = 1 + D + D * D;
    const int tid = threadIdx.x;
    float lo[D], hi[D], dm[D];
#pragma unroll
    for (int d = 0; d < D; ++d) { lo[d] = INFINITY; hi[d] = -INFINITY; dm[d] = -INFINITY; }
    for (int g = tid; g < G; g += THREADS) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const float v = __ldg(mix + size_t(g) * RF + 1 + d);
            lo[d] = fminf(lo[d], v);
            hi[d] = fmaxf(hi[d], v);
            if (layout != 0) dm[d] = fmaxf(dm[d], __ldg(mix + size_t(g) * RF + 1 + D + d * D + d));
        }
    }
#pragma unroll
    for (int d = 0; d < D; ++d) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo[d] = fminf(lo[d], __shfl_xor_sync(0xffffffffu, lo[d], o));
            hi[d] = fmaxf(hi[d], __shfl_xor_sync(0xffffffffu, hi[d], o));
            dm[d] = fmaxf(dm[d], __shfl_xor_sync(0xffffffffu, dm[d], o));
        }
        if ((tid & 31) == 0) { ext.red[0][d][tid >> 5] = lo[d]; ext.red[1][d][tid >> 5] = hi[d]; ext.red[2][d][tid >> 5] = dm[d]; }
    }
    __syncthreads();
    if (tid < D) {
        float l = ext.red[0][tid][0], h = ext.red[1][tid][0], m = ext.red[2][tid][0];
        for (int w = 1; w < THREADS / 32; ++w) {
            l = fminf(l, ext.red[0][tid][w]);
            h = fmaxf(h, ext.red[1][tid][w]);
            m = fmaxf(m, ext.red[2][tid][w]);
        }
        ext.lo[tid] = l;
        ext.hi[tid] = h;
        ext.diag_max[tid] = m;
    }
    __syncthreads();
}

template <int D>
__device__ __forceinline__ uint64_t key_of_component(const float* __restrict__ mix, int g, int layout, const Extent<D>& ext) {
    constexpr int RF = 1 + D + D * D;
    uint32_t q[3] = {0u, 0u, 0u}, c[3] = {0u, 0u, 0u};
#pragma unroll
    for (int d = 0; d < D; ++d) {
        q[d] = lbvh::quantise(__ldg(mix + size_t(g) * RF + 1 + d), ext.lo[d], ext.hi[d]);
        if (layout != 0) c[d] = lbvh::quantise_unit(__fdiv_rn(__ldg(mix + size_t(g) * RF + 1 + D + d * D + d), ext.diag_max[d]));
    }
    return lbvh::component_key(layout, lbvh::morton30(q[0], q[1], q[2]), lbvh::morton30(c[0], c[1], c[2]), uint32_t(g));
}

template <int D>
__global__ void __launch_bounds__(kThreads)
lbvh_build_kernel(const float* __restrict__ mixture, int n_components, int layout, uint64_t* __restrict__ sorted_keys,
                  uint16_t* __restrict__ nodes) {
    constexpr int RF = 1 + D + D * D;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    uint64_t* keys = reinterpret_cast<uint64_t*>(smem_bytes);
    __shared__ Extent<D> ext;
    __shared__ int s_sort_fallback;

    const int G = n_components;
    const int tid = threadIdx.x;
    const float* mix = mixture + size_t(blockIdx.x) * G * RF;

    mixture_extent<D, kThreads>(mix, G, layout, ext);

    // ---- Morton keys, ascending ----
    if (layout == 0) {
        // sorted as (Morton code << 32 | id) by the radix sort that the convolution fit uses (its rank bits 16..31 must
        // be free), then shifted back to the output format (code << 16 | id)
        uint64_t* keys_b = keys + G;
        for (int g = tid; g < G; g += kThreads) {
            const uint64_t k = key_of_component<D>(mix, g, 0, ext);
            keys[g] = ((k >> 16) << 32) | (k & 0xFFFFull);
        }
        __syncthreads();
        const uint64_t* sorted = lbvh::sort_codes_shared<3>(keys, keys_b, G, keys_b + G, &s_sort_fallback);
        for (int g = tid; g < G; g += kThreads) {             // element-wise, so in place or across the buffers alike
            const uint64_t k = sorted[g];
            keys[g] = ((k >> 32) << 16) | (k & 0xFFFFull);
        }
        __syncthreads();
    } else {
        const int P = lbvh::next_pow2(G);
        for (int g = tid; g < P; g += kThreads) keys[g] = g < G ? key_of_component<D>(mix, g, layout, ext) : ~0ull;
        __syncthreads();
        lbvh::bitonic_sort_shared(keys, P);
    }

    // ---- leaves and internal nodes ----
    uint64_t* out_keys = sorted_keys + size_t(blockIdx.x) * G;
    uint16_t* nd = nodes + size_t(blockIdx.x) * (2 * size_t(G) - 1) * 4;
    for (int j = tid; j < G; j += kThreads) {
        const uint64_t k = keys[j];
        out_keys[j] = k;
        uint16_t* leaf = nd + size_t(G - 1 + j) * 4;
        leaf[1] = 0xFFFFu;
        leaf[2] = 0xFFFFu;
        leaf[3] = uint16_t(k);
    }
    const lbvh::PlainCode code{keys};
    for (int i = tid; i < G - 1; i += kThreads) {
        const int2 r = lbvh::determine_range(code, G, i);
        const int gamma = lbvh::find_split(code, r.x, r.y);
        int left = gamma, right = gamma + 1;
        if (min(r.x, r.y) == gamma) left += G - 1;
        if (max(r.x, r.y) == gamma + 1) right += G - 1;
        uint16_t* node = nd + size_t(i) * 4;
        node[1] = uint16_t(left);
        node[2] = uint16_t(right);
        node[3] = uint16_t(i);
        nd[size_t(left) * 4] = uint16_t(i);
        nd[size_t(right) * 4] = uint16_t(i);
        if (i == 0) node[0] = 0xFFFFu;
    }
}


// ---- more than kMaxComponents components: keys in global memory ----
constexpr int kLargeThreads = 1024;

template <int D>
__global__ void __launch_bounds__(kLargeThreads)
lbvh_build_large_kernel(const float* __restrict__ mixture, int n_components, int layout,
                        uint64_t* __restrict__ sorted_keys, uint16_t* __restrict__ nodes) {
    constexpr int RF = 1 + D + D * D;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    __shared__ Extent<D> ext;
    const int G = n_components;
    const int tid = threadIdx.x;
    const float* mix = mixture + size_t(blockIdx.x) * G * RF;
    uint64_t* keys = sorted_keys + size_t(blockIdx.x) * G;
    uint16_t* nd = nodes + size_t(blockIdx.x) * (2 * size_t(G) - 1) * 4;
    uint16_t* ranks = reinterpret_cast<uint16_t*>(smem_bytes);                              // [G]
    void* sort_scratch = smem_bytes + ((size_t(G) * 2 + 15) & ~size_t(15));

    mixture_extent<D, kLargeThreads>(mix, G, layout, ext);
    for (int g = tid; g < G; g += kLargeThreads) keys[g] = key_of_component<D>(mix, g, layout, ext);
    __threadfence_block();
    __syncthreads();
    // layout 0: keys are unique through the component id in bits 0..15 and arrive in id order, so a stable sort on the
    // Morton bits 16..47 (four 8-bit passes, back in `keys`) is the full ascending order; the other layouts use all 64 bits
    if (layout == 0) lbvh::radix_sort_global(keys, reinterpret_cast<uint64_t*>(nd), G, 16, 4, ranks, sort_scratch);
    else lbvh::radix_sort_global(keys, reinterpret_cast<uint64_t*>(nd), G, 0, 8, ranks, sort_scratch);

    for (int j = tid; j < G; j += kLargeThreads) {
        uint16_t* leaf = nd + size_t(G - 1 + j) * 4;
        leaf[1] = 0xFFFFu;
        leaf[2] = 0xFFFFu;
        leaf[3] = uint16_t(keys[j]);
    }
    const lbvh::PlainCode code{keys};
    for (int i = tid; i < G - 1; i += kLargeThreads) {
        const int2 r = lbvh::determine_range(code, G, i);
        const int gamma = lbvh::find_split(code, r.x, r.y);
        int left = gamma, right = gamma + 1;
        if (min(r.x, r.y) == gamma) left += G - 1;
        if (max(r.x, r.y) == gamma + 1) right += G - 1;
        uint16_t* node = nd + size_t(i) * 4;
        node[1] = uint16_t(left);
        node[2] = uint16_t(right);
        node[3] = uint16_t(i);
        nd[size_t(left) * 4] = uint16_t(i);
        nd[size_t(right) * 4] = uint16_t(i);
        if (i == 0) node[0] = 0xFFFFu;
    }
}

// ---- make_aabbs: boxes of all nodes, [2G-1][upper.xyzw, lower.xyzw] per mixture ----
// Leaf: the box of the ellipsoid on which the component's density falls to `threshold` (at least the 95 % ellipsoid):
// mean -+ delta with delta[r] = factor * sqrt(sum_k lambda_k * v_r[k]^2) over the eigen-pairs (lambda, v) of the
// covariance, eigenvalues ascending -- the pairing of eigenvector r with coordinate r is the reference's
// (lbvh/bvh.cu:180-200) and is kept as it is. The matrix slot holds INVERSE covariances (lbvh/bvh.cu:204).
// Internal nodes: union of the children, bottom-up; the second thread to arrive at a node does the merge. The arrival
// flag is the unused w lane of the node's upper corner, zero again at the end.
template <int D>
__global__ void __launch_bounds__(kThreads)
lbvh_aabb_kernel(const float* __restrict__ mixture, int n_components, float threshold, const uint16_t* __restrict__ nodes,
                 float* __restrict__ aabbs) {
    constexpr int RF = 1 + D + D * D;
    const int G = n_components;
    const int tid = threadIdx.x;
    const float* mix = mixture + size_t(blockIdx.x) * G * RF;
    const uint16_t* nd = nodes + size_t(blockIdx.x) * (2 * size_t(G) - 1) * 4;
    float* bx = aabbs + size_t(blockIdx.x) * (2 * size_t(G) - 1) * 8;

    for (int i = tid; i < (G - 1) * 8; i += kThreads) bx[i] = 0.f;
    for (int j = tid; j < G; j += kThreads) {
        const float* g = mix + size_t(nd[size_t(G - 1 + j) * 4 + 3]) * RF;
        float inv[D * D], cov[D * D], val[D], vec[D * D];
#pragma unroll
        for (int k = 0; k < D * D; ++k) inv[k] = __ldg(g + 1 + D + k);
        if constexpr (D == 2) {
            const float r = 1.f / (inv[0] * inv[3] - inv[1] * inv[2]);
            cov[0] = inv[3] * r; cov[1] = -inv[1] * r; cov[2] = -inv[2] * r; cov[3] = inv[0] * r;
        } else {
            const float c0 = inv[4] * inv[8] - inv[5] * inv[7], c1 = inv[3] * inv[8] - inv[5] * inv[6], c2 = inv[3] * inv[7] - inv[4] * inv[6];
            const float r = 1.f / (inv[0] * c0 - inv[1] * c1 + inv[2] * c2);
            cov[0] = c0 * r; cov[1] = -(inv[1] * inv[8] - inv[2] * inv[7]) * r; cov[2] = (inv[1] * inv[5] - inv[2] * inv[4]) * r;
            cov[3] = -c1 * r; cov[4] = (inv[0] * inv[8] - inv[2] * inv[6]) * r; cov[5] = -(inv[0] * inv[5] - inv[2] * inv[3]) * r;
            cov[6] = c2 * r; cov[7] = -(inv[0] * inv[7] - inv[1] * inv[6]) * r; cov[8] = (inv[0] * inv[4] - inv[1] * inv[3]) * r;
        }
        symeig_device<D>(cov, val, vec);
        const float weight = __ldg(g);
        const float factor = sqrtf(fmaxf(-2.f * logf(threshold / fabsf(weight)), 5.991464547107982f));
        float* b = bx + size_t(G - 1 + j) * 8;
#pragma unroll
        for (int r = 0; r < D; ++r) {
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < D; ++k) acc += val[k] * vec[k * D + r] * vec[k * D + r];
            const float delta = factor * sqrtf(acc);
            const float mean = __ldg(g + 1 + r);
            b[r] = mean + delta;
            b[4 + r] = mean - delta;
        }
#pragma unroll
        for (int r = D; r < 4; ++r) { b[r] = 0.f; b[4 + r] = 0.f; }
    }
    __threadfence_block();
    __syncthreads();

    volatile float* vbx = bx;
    for (int j = tid; j < G; j += kThreads) {
        int cur = G - 1 + j;
        for (int level = 0; level < 2 * G; ++level) {            // a path to the root has fewer than G nodes
            const unsigned parent = nd[size_t(cur) * 4];
            if (parent == 0xFFFFu) break;
            __threadfence_block();                               // own box before the flag
            if (atomicExch(reinterpret_cast<int*>(bx + size_t(parent) * 8 + 3), 1) == 0) break;   // first to arrive leaves
            __threadfence_block();
            const size_t l = size_t(nd[size_t(parent) * 4 + 1]) * 8, r = size_t(nd[size_t(parent) * 4 + 2]) * 8;
#pragma unroll
            for (int d = 0; d < 3; ++d) {
                vbx[size_t(parent) * 8 + d] = fmaxf(vbx[l + d], vbx[r + d]);
                vbx[size_t(parent) * 8 + 4 + d] = fminf(vbx[l + 4 + d], vbx[r + 4 + d]);
            }
            cur = int(parent);
        }
    }
    __syncthreads();
    for (int i = tid; i < G - 1; i += kThreads) bx[size_t(i) * 8 + 3] = 0.f;
}

}  // namespace

int lbvh_build_launch(const float* mixture, long long n_mixtures, int n_components, int n_dims, int layout, uint64_t* sorted_keys,
                      uint16_t* nodes, cudaStream_t stream) {
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (layout < 0 || layout > 4) return GMC_ERR_UNSUPPORTED;
    if (n_mixtures < 0 || n_components < 2 || n_components > kMaxComponentsLarge) return GMC_ERR_BAD_DIMS;
    if (n_mixtures == 0) return GMC_OK;
    if (n_mixtures > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    if (!mixture || !sorted_keys || !nodes) return GMC_ERR_NULL_POINTER;
    if (n_components > kMaxComponents) {
        const size_t smem_large = ((size_t(n_components) * 2 + 15) & ~size_t(15)) + 2 * ((kLargeThreads / 32) * 256 + 256) + 32;
        if (n_dims == 2) {
            GMC_CUDA_TRY(cudaFuncSetAttribute(lbvh_build_large_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_large)));
            lbvh_build_large_kernel<2><<<unsigned(n_mixtures), kLargeThreads, smem_large, stream>>>(mixture, n_components, layout, sorted_keys, nodes);
        } else {
            GMC_CUDA_TRY(cudaFuncSetAttribute(lbvh_build_large_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_large)));
            lbvh_build_large_kernel<3><<<unsigned(n_mixtures), kLargeThreads, smem_large, stream>>>(mixture, n_components, layout, sorted_keys, nodes);
        }
        GMC_LAUNCH_CHECK();
        return GMC_OK;
    }
    // layout 0: two key buffers + the radix scratch; other layouts: one power-of-two buffer for the bitonic network
    const size_t smem = layout == 0 ? sizeof(uint64_t) * 2 * size_t(n_components) + 2 * ((kThreads / 32) * 256 + 256) + 32
                                    : sizeof(uint64_t) * size_t(lbvh::next_pow2(n_components));
    if (n_dims == 2) {
        if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(lbvh_build_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        lbvh_build_kernel<2><<<unsigned(n_mixtures), kThreads, smem, stream>>>(mixture, n_components, layout, sorted_keys, nodes);
    } else {
        if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(lbvh_build_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        lbvh_build_kernel<3><<<unsigned(n_mixtures), kThreads, smem, stream>>>(mixture, n_components, layout, sorted_keys, nodes);
    }
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

int lbvh_aabbs_launch(const float* mixture, long long n_mixtures, int n_components, int n_dims, float threshold,
                      const uint16_t* nodes, float* aabbs, cudaStream_t stream) {
    if (n_mixtures == 0) return GMC_OK;
    if (!aabbs) return GMC_ERR_NULL_POINTER;
    if (!(threshold > 0.f)) return GMC_ERR_BAD_DIMS;
    if (n_dims == 2) lbvh_aabb_kernel<2><<<unsigned(n_mixtures), kThreads, 0, stream>>>(mixture, n_components, threshold, nodes, aabbs);
    else lbvh_aabb_kernel<3><<<unsigned(n_mixtures), kThreads, 0, stream>>>(mixture, n_components, threshold, nodes, aabbs);
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

}  // namespace gmc

GMC_DEFINE_TU_CHECK_READER(lbvh)

extern "C" int gmc_lbvh_build(const float* mixture, long long n_mixtures, int n_components, int n_dims,
                              uint64_t* sorted_keys, int16_t* nodes, void* stream) {
    return gmc::lbvh_build_launch(mixture, n_mixtures, n_components, n_dims, 0, sorted_keys,
                                  reinterpret_cast<uint16_t*>(nodes), gmc::as_stream(stream));
}

extern "C" int gmc_lbvh_build_ex(const float* mixture, long long n_mixtures, int n_components, int n_dims,
                                 int morton_code_algorithm, int make_aabbs, float aabb_threshold, uint64_t* sorted_keys,
                                 int16_t* nodes, float* aabbs, void* stream) {
    // the leaf of a key is its low 16 bits; only layouts 0 and 1 keep the component index there, so only they can
    // look up the component of a leaf for its box
    if (make_aabbs && (morton_code_algorithm < 0 || morton_code_algorithm > 1)) return GMC_ERR_UNSUPPORTED;
    const int rc = gmc::lbvh_build_launch(mixture, n_mixtures, n_components, n_dims, morton_code_algorithm, sorted_keys,
                                          reinterpret_cast<uint16_t*>(nodes), gmc::as_stream(stream));
    if (rc != GMC_OK || !make_aabbs) return rc;
    return gmc::lbvh_aabbs_launch(mixture, n_mixtures, n_components, n_dims, aabb_threshold,
                                  reinterpret_cast<const uint16_t*>(nodes), aabbs, gmc::as_stream(stream));
}
