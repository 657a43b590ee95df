// Linear BVH over the means of each mixture: whole AABB, 30-bit Morton keys (<< 16 | component id), ascending
// sort, Karras internal nodes. One CTA per mixture keeps the keys in shared memory from the Morton stage to the
// last node, so global traffic is the means in, the sorted keys and the node array out. Mixtures of more than 8192
// components (up to the 32768 that 16-bit node indices allow) take lbvh_build_large_kernel: same steps, keys in global
// memory, radix-sorted between the key output buffer and the (not yet written) node buffer.
// Replaces lbvh::Bvh::construct with make_aabbs = false (src/gmc/cpp/extensions/lbvh/bvh.cu:23-144, 241-299, 373-458).
#include "common.cuh"
#include "lbvh_device.cuh"

namespace gmc {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxComponents = 8192;          // keys of one mixture fit in shared memory (64 KB) up to here
constexpr int kMaxComponentsLarge = 32768;    // node indices are 16 bit with 0xFFFF = none: 2G - 2 <= 65534 (the reference
                                              // accepts up to 65534 components, implementation_forward.h:498-500, but its
                                              // uint16 node indices, lbvh/bvh.h:16-24, wrap beyond this size)

template <int D>
__global__ void __launch_bounds__(kThreads)
lbvh_build_kernel(const float* __restrict__ mixture, int n_components, uint64_t* __restrict__ sorted_keys,
                  uint16_t* __restrict__ nodes) {
    constexpr int RF = 1 + D + D * D;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    uint64_t* keys = reinterpret_cast<uint64_t*>(smem_bytes);
    __shared__ float red_lo[D][kThreads / 32], red_hi[D][kThreads / 32];
    __shared__ float box_lo[D], box_hi[D];

    const int G = n_components;
    const int tid = threadIdx.x;
    const float* mix = mixture + size_t(blockIdx.x) * G * RF;

    // ---- whole AABB of the means ----
    float lo[D], hi[D];
#pragma unroll
    for (int d = 0; d < D; ++d) { lo[d] = INFINITY; hi[d] = -INFINITY; }
    for (int g = tid; g < G; g += kThreads) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const float v = __ldg(mix + size_t(g) * RF + 1 + d);
            lo[d] = fminf(lo[d], v);
            hi[d] = fmaxf(hi[d], v);
        }
    }
#pragma unroll
    for (int d = 0; d < D; ++d) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo[d] = fminf(lo[d], __shfl_xor_sync(0xffffffffu, lo[d], o));
            hi[d] = fmaxf(hi[d], __shfl_xor_sync(0xffffffffu, hi[d], o));
        }
        if ((tid & 31) == 0) { red_lo[d][tid >> 5] = lo[d]; red_hi[d][tid >> 5] = hi[d]; }
    }
    __syncthreads();
    if (tid < D) {
        float l = red_lo[tid][0], h = red_hi[tid][0];
        for (int w = 1; w < kThreads / 32; ++w) { l = fminf(l, red_lo[tid][w]); h = fmaxf(h, red_hi[tid][w]); }
        box_lo[tid] = l;
        box_hi[tid] = h;
    }
    __syncthreads();

    // ---- Morton keys ----
    const int P = lbvh::next_pow2(G);
    for (int g = tid; g < P; g += kThreads) {
        uint64_t key = ~0ull;
        if (g < G) {
            uint32_t q[3] = {0u, 0u, 0u};
#pragma unroll
            for (int d = 0; d < D; ++d) q[d] = lbvh::quantise(__ldg(mix + size_t(g) * RF + 1 + d), box_lo[d], box_hi[d]);
            key = (uint64_t(lbvh::morton30(q[0], q[1], q[2])) << 16) | uint64_t(g);
        }
        keys[g] = key;
    }
    __syncthreads();
    lbvh::bitonic_sort_shared(keys, P);

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
lbvh_build_large_kernel(const float* __restrict__ mixture, int n_components, uint64_t* __restrict__ sorted_keys,
                        uint16_t* __restrict__ nodes) {
    constexpr int RF = 1 + D + D * D;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    __shared__ float red_lo[D][kLargeThreads / 32], red_hi[D][kLargeThreads / 32];
    __shared__ float box_lo[D], box_hi[D];
    const int G = n_components;
    const int tid = threadIdx.x;
    const float* mix = mixture + size_t(blockIdx.x) * G * RF;
    uint64_t* keys = sorted_keys + size_t(blockIdx.x) * G;
    uint16_t* nd = nodes + size_t(blockIdx.x) * (2 * size_t(G) - 1) * 4;
    uint16_t* ranks = reinterpret_cast<uint16_t*>(smem_bytes);                              // [G]
    void* sort_scratch = smem_bytes + ((size_t(G) * 2 + 15) & ~size_t(15));

    float lo[D], hi[D];
#pragma unroll
    for (int d = 0; d < D; ++d) { lo[d] = INFINITY; hi[d] = -INFINITY; }
    for (int g = tid; g < G; g += kLargeThreads) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const float v = __ldg(mix + size_t(g) * RF + 1 + d);
            lo[d] = fminf(lo[d], v);
            hi[d] = fmaxf(hi[d], v);
        }
    }
#pragma unroll
    for (int d = 0; d < D; ++d) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo[d] = fminf(lo[d], __shfl_xor_sync(0xffffffffu, lo[d], o));
            hi[d] = fmaxf(hi[d], __shfl_xor_sync(0xffffffffu, hi[d], o));
        }
        if ((tid & 31) == 0) { red_lo[d][tid >> 5] = lo[d]; red_hi[d][tid >> 5] = hi[d]; }
    }
    __syncthreads();
    if (tid < D) {
        float l = red_lo[tid][0], h = red_hi[tid][0];
        for (int w = 1; w < kLargeThreads / 32; ++w) { l = fminf(l, red_lo[tid][w]); h = fmaxf(h, red_hi[tid][w]); }
        box_lo[tid] = l;
        box_hi[tid] = h;
    }
    __syncthreads();
    for (int g = tid; g < G; g += kLargeThreads) {
        uint32_t q[3] = {0u, 0u, 0u};
#pragma unroll
        for (int d = 0; d < D; ++d) q[d] = lbvh::quantise(__ldg(mix + size_t(g) * RF + 1 + d), box_lo[d], box_hi[d]);
        keys[g] = (uint64_t(lbvh::morton30(q[0], q[1], q[2])) << 16) | uint64_t(g);
    }
    __threadfence_block();
    __syncthreads();
    // keys are unique through the component id in bits 0..15 and arrive in id order, so a stable sort on the Morton
    // bits 16..47 (four 8-bit passes, back in `keys`) is the full ascending order
    lbvh::radix_sort_global(keys, reinterpret_cast<uint64_t*>(nd), G, 16, 4, ranks, sort_scratch);

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

}  // namespace

int lbvh_build_launch(const float* mixture, long long n_mixtures, int n_components, int n_dims, uint64_t* sorted_keys,
                      uint16_t* nodes, cudaStream_t stream) {
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_mixtures < 0 || n_components < 2 || n_components > kMaxComponentsLarge) return GMC_ERR_BAD_DIMS;
    if (n_mixtures == 0) return GMC_OK;
    if (n_mixtures > 0x7fffffffLL) return GMC_ERR_BAD_DIMS;
    if (!mixture || !sorted_keys || !nodes) return GMC_ERR_NULL_POINTER;
    if (n_components > kMaxComponents) {
        const size_t smem_large = ((size_t(n_components) * 2 + 15) & ~size_t(15)) + 2 * ((kLargeThreads / 32) * 256 + 256) + 32;
        if (n_dims == 2) {
            GMC_CUDA_TRY(cudaFuncSetAttribute(lbvh_build_large_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_large)));
            lbvh_build_large_kernel<2><<<unsigned(n_mixtures), kLargeThreads, smem_large, stream>>>(mixture, n_components, sorted_keys, nodes);
        } else {
            GMC_CUDA_TRY(cudaFuncSetAttribute(lbvh_build_large_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_large)));
            lbvh_build_large_kernel<3><<<unsigned(n_mixtures), kLargeThreads, smem_large, stream>>>(mixture, n_components, sorted_keys, nodes);
        }
        GMC_LAUNCH_CHECK();
        return GMC_OK;
    }
    const size_t smem = sizeof(uint64_t) * size_t(lbvh::next_pow2(n_components));
    if (n_dims == 2) {
        if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(lbvh_build_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        lbvh_build_kernel<2><<<unsigned(n_mixtures), kThreads, smem, stream>>>(mixture, n_components, sorted_keys, nodes);
    } else {
        if (smem > 48 * 1024) GMC_CUDA_TRY(cudaFuncSetAttribute(lbvh_build_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        lbvh_build_kernel<3><<<unsigned(n_mixtures), kThreads, smem, stream>>>(mixture, n_components, sorted_keys, nodes);
    }
    GMC_LAUNCH_CHECK();
    return GMC_OK;
}

}  // namespace gmc

GMC_DEFINE_TU_CHECK_READER(lbvh)

extern "C" int gmc_lbvh_build(const float* mixture, long long n_mixtures, int n_components, int n_dims,
                              uint64_t* sorted_keys, int16_t* nodes, void* stream) {
    return gmc::lbvh_build_launch(mixture, n_mixtures, n_components, n_dims, sorted_keys,
                                  reinterpret_cast<uint16_t*>(nodes), gmc::as_stream(stream));
}
