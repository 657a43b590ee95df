// Device-side building blocks of the linear BVH (Karras 2012) shared by the BVH-MHEM fit and the convolution fit:
// Morton quantisation, a CTA-wide bitonic sort of 64-bit keys in shared memory, and the range / split search.
// Semantics follow the reference's lbvh/morton_code.h:77-85, 145-156 and lbvh/building.h:11-103 (and the
// convolution_fitting/building.h variant that replaces the low 32 key bits by the sorted position).
// Everything that feeds integer results is written with explicit IEEE intrinsics so that fast-math or FMA
// contraction of the surrounding file cannot change a Morton code.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace gmc {
namespace lbvh {

__device__ __forceinline__ uint32_t expand_bits3(uint32_t v) {
    v = (v * 0x00010001u) & 0xFF0000FFu;
    v = (v * 0x00000101u) & 0x0F00F00Fu;
    v = (v * 0x00000011u) & 0xC30C30C3u;
    v = (v * 0x00000005u) & 0x49249249u;
    return v;
}

// 10-bit cell of `pos` inside [lower, upper]; an empty extent (0/0 in the reference) gives cell 0.
__device__ __forceinline__ uint32_t quantise(float pos, float lower, float upper) {
    const float extent = __fsub_rn(upper, lower);
    if (!(extent > 0.0f)) return 0u;
    const float p = __fdiv_rn(__fsub_rn(pos, lower), extent);
    const float scaled = __fmul_rn(p, 1024.0f);
    const uint32_t q = scaled > 0.0f ? __float2uint_rz(scaled) : 0u;
    return min(q, 1023u);
}

__device__ __forceinline__ uint32_t morton30(uint32_t qx, uint32_t qy, uint32_t qz) {
    return (expand_bits3(qx) << 2) + (expand_bits3(qy) << 1) + expand_bits3(qz);
}

// Spreads the low 32 bits of v over the even bit positions of a 64-bit word.
__device__ __forceinline__ uint64_t expand_bits2(uint32_t v) {
    uint64_t t = v;
    t = ((t << 16) | t) & 0x0000FFFF0000FFFFull;
    t = ((t << 8) | t) & 0x00FF00FF00FF00FFull;
    t = ((t << 4) | t) & 0x0F0F0F0F0F0F0F0Full;
    t = ((t << 2) | t) & 0x3333333333333333ull;
    t = ((t << 1) | t) & 0x5555555555555555ull;
    return t;
}

// 10-bit cell of a value in [0, 1] (diagonal entry of the matrix slot over its per-mixture maximum).
__device__ __forceinline__ uint32_t quantise_unit(float v) {
    const float scaled = __fmul_rn(v, 1024.0f);
    const uint32_t q = scaled > 0.0f ? __float2uint_rz(scaled) : 0u;
    return min(q, 1023u);
}

// Sort key of one component from the 30-bit Morton codes of its position and of its matrix diagonal and its index:
// layout 0 = position << 16 | id; 1 = 12 position bits, 36 bits position / diagonal interleaved, 16 bits id;
// 2 = 54 interleaved bits, 10 bits id; 3 = 27 position, 27 diagonal, 10 id; 4 = 27 diagonal, 27 position, 10 id
// (the reference's lbvh/morton_code.h:170-252; only layouts 0 and 1 keep the whole id in the low 16 bits).
__device__ __forceinline__ uint64_t component_key(int layout, uint32_t pos, uint32_t cov, uint32_t id) {
    switch (layout) {
        case 0: return (uint64_t(pos) << 16) | uint64_t(id & 0xFFFFu);
        case 1: {
            uint64_t result = pos >> 18;
            const uint64_t poscov = (expand_bits2(pos & 0x3FFFFu) << 1) | expand_bits2(cov >> 12);
            result = (result << 36) | poscov;
            return (result << 16) | uint64_t(id & 0xFFFFu);
        }
        case 2: return ((((expand_bits2(pos) << 1) | expand_bits2(cov)) << 4) & 0xFFFFFFFFFFFFFC00ull) | uint64_t(id & 0xFFFFu);
        case 3: return (uint64_t(pos & ~0x7u) << 34) | (uint64_t(cov & ~0x7u) << 7) | uint64_t(id & 0x3FFu);
        default: return (uint64_t(cov & ~0x7u) << 34) | (uint64_t(pos & ~0x7u) << 7) | uint64_t(id & 0x3FFu);
    }
}

// Sorts keys[0 .. n_pow2) ascending; n_pow2 is a power of two, entries beyond the real count hold ~0ull.
// All threads of the CTA must call it.
__device__ __forceinline__ void bitonic_sort_shared(uint64_t* keys, int n_pow2) {
    for (int k = 2; k <= n_pow2; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = threadIdx.x; t < (n_pow2 >> 1); t += blockDim.x) {
                // t-th pair of this stage: insert a zero bit at position log2(j)
                const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                const int p = i | j;
                const uint64_t a = keys[i], b = keys[p];
                const bool ascending = (i & k) == 0;
                if ((a > b) == ascending) {
                    keys[i] = b;
                    keys[p] = a;
                }
            }
            __syncthreads();
        }
    }
}

// Stable LSD radix sort of n 64-bit keys on the bit range [first_bit, first_bit + 8 * n_passes), CTA-wide, in shared
// memory. `a` holds the input and `b` is a second buffer of n keys; the sorted keys end up in `a` if n_passes is even
// and in `b` otherwise (the function returns the pointer). `scratch` needs 2 * ((number of warps) * 256 + 256) + 32 bytes, 4-byte aligned; n must stay below 65536.
// Bits 16..31 of every key must be zero and outside the sorted bit range: they carry the rank between the two loops of
// a pass (n / number of warps, rounded up to 32, must stay below 65536) and are zero again on return.
//
// Every warp owns a contiguous slice of the keys. Counting loop: per 32-key step __match_any_sync groups equal digits,
// the first lane of a group bumps the warp's digit counter and hands the old value to its group, and every key stores
// its rank among the warp's keys of that digit. The CTA then turns the (digit, warp) counts into offsets, and the
// scatter loop is one independent read-modify-write per key, so equal digits keep their input order.
__device__ __forceinline__ uint64_t* radix_sort_shared(uint64_t* a, uint64_t* b, int n, int first_bit, int n_passes,
                                                       void* scratch) {
    const int n_warps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunk = (((n + n_warps - 1) / n_warps) + 31) & ~31;
    const int begin = min(n, warp * chunk), end = min(n, begin + chunk);
    uint16_t* hist = reinterpret_cast<uint16_t*>(scratch);      // [warp][digit]: counts, then offsets below 65536
    uint16_t* my_hist = hist + warp * 256;
    uint16_t* totals = hist + n_warps * 256;
    unsigned* warp_sums = reinterpret_cast<unsigned*>(totals + 256);
    const unsigned lt_mask = (1u << lane) - 1u;
    for (int pass = 0; pass < n_passes; ++pass) {
        const int shift = first_bit + 8 * pass;
#pragma unroll
        for (int k = 0; k < 4; ++k) reinterpret_cast<unsigned*>(my_hist)[lane + 32 * k] = 0u;
        __syncwarp();
        for (int i0 = begin; i0 < end; i0 += 32) {
            const int i = i0 + lane;
            const bool active = i < end;
            const unsigned act = __ballot_sync(0xffffffffu, active);
            if (active) {
                const unsigned digit = unsigned(a[i] >> shift) & 0xFFu;
                const unsigned peers = __match_any_sync(act, digit);
                const int leader = __ffs(peers) - 1;
                unsigned before = 0u;
                if (lane == leader) {
                    before = my_hist[digit];
                    my_hist[digit] = uint16_t(before + __popc(peers));
                }
                before = __shfl_sync(act, before, leader);
                reinterpret_cast<uint16_t*>(a + i)[1] = uint16_t(before + __popc(peers & lt_mask));
            }
            __syncwarp();
        }
        __syncthreads();
        // (digit, warp) counts -> exclusive offsets: over the warps of a digit, then over the digits
        if (threadIdx.x < 256) {
            unsigned run = 0u;
            for (int w = 0; w < n_warps; ++w) {
                const unsigned c = hist[w * 256 + threadIdx.x];
                hist[w * 256 + threadIdx.x] = uint16_t(run);
                run += c;
            }
            unsigned incl = run;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const unsigned o = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += o;
            }
            totals[threadIdx.x] = uint16_t(incl - run);        // exclusive inside this group of 32 digits
            if (lane == 31) warp_sums[warp] = incl;
        }
        __syncthreads();
        unsigned group_base = 0u;                    // lane k < 8: number of keys with a digit below 32 * k
#pragma unroll
        for (int k = 0; k < 7; ++k) group_base += k < lane ? warp_sums[k] : 0u;
        for (int i0 = begin; i0 < end; i0 += 32) {
            const int i = i0 + lane;
            const bool active = i < end;
            const uint64_t key = active ? a[i] : 0ull;
            const unsigned digit = unsigned(key >> shift) & 0xFFu;
            const unsigned base = __shfl_sync(0xffffffffu, group_base, int(digit >> 5));
            if (active)
                b[base + unsigned(totals[digit]) + unsigned(my_hist[digit]) + (unsigned(key >> 16) & 0xFFFFu)] =
                    key & ~0xFFFF0000ull;
        }
        __syncthreads();
        uint64_t* t = a; a = b; b = t;
    }
    return a;
}

// Ascending order of n unique keys whose bits 32..62 hold a code and whose low bits hold the input position (bit 63 and
// bits 16..31 zero, n <= 8192; the input must already be in ascending position order among equal codes, which key
// generation by position gives): the result equals a stable sort on the code bits.
// TOP_PASSES stable 8-bit passes order the keys on their top 8 * TOP_PASSES code bits; a run of keys that share those
// bits is then in input order, and each of its members finds its place by counting the smaller keys of the run (runs
// are short when the codes spread over the top bits: Morton codes of scattered positions). A run longer than
// kMaxRun makes the whole CTA fall back to the plain four passes over all 32 code bits, from the partially sorted
// state (still in position order among equal codes). `flag` is one shared int. Returns the buffer with the result.
constexpr int kMaxRun = 64;

template <int TOP_PASSES>
__device__ __forceinline__ uint64_t* sort_codes_shared(uint64_t* a, uint64_t* b, int n, void* scratch, int* flag) {
    constexpr int kFirstBit = 63 - 8 * TOP_PASSES;
    if (threadIdx.x == 0) *flag = 0;
    uint64_t* cur = radix_sort_shared(a, b, n, kFirstBit, TOP_PASSES, scratch);      // ends with a CTA barrier
    uint64_t* other = cur == a ? b : a;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const uint64_t key = cur[i];
        const uint64_t top = key >> kFirstBit;
        const bool left_same = i > 0 && (cur[i - 1] >> kFirstBit) == top;
        const bool right_same = i + 1 < n && (cur[i + 1] >> kFirstBit) == top;
        if (!left_same && !right_same) { other[i] = key; continue; }
        int s = i, e = i + 1;
        while (s > 0 && i - s <= kMaxRun && (cur[s - 1] >> kFirstBit) == top) --s;
        while (e < n && e - i <= kMaxRun && (cur[e] >> kFirstBit) == top) ++e;
        if (e - s > kMaxRun) { *flag = 1; continue; }
        int rank = 0;
        for (int j = s; j < e; ++j) rank += cur[j] < key ? 1 : 0;
        other[s + rank] = key;
    }
    __syncthreads();
    if (*flag == 0) return other;
    return radix_sort_shared(cur, other, n, 32, 4, scratch);
}

// The same stable LSD radix sort for keys that live in GLOBAL memory (trees too large for shared memory): `a` and `b`
// are global buffers of n keys, the rank that a key carries between the counting and the scatter loop sits in the
// shared array `ranks` (n uint16) instead of in key bits, `scratch` as above. n < 65536. Sorted keys end up in `a` for an
// even number of passes. One CTA sorts one segment; all its threads must call.
__device__ __forceinline__ uint64_t* radix_sort_global(uint64_t* a, uint64_t* b, int n, int first_bit, int n_passes,
                                                       uint16_t* ranks, void* scratch) {
    const int n_warps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunk = (((n + n_warps - 1) / n_warps) + 31) & ~31;
    const int begin = min(n, warp * chunk), end = min(n, begin + chunk);
    uint16_t* hist = reinterpret_cast<uint16_t*>(scratch);
    uint16_t* my_hist = hist + warp * 256;
    uint16_t* totals = hist + n_warps * 256;
    unsigned* warp_sums = reinterpret_cast<unsigned*>(totals + 256);
    const unsigned lt_mask = (1u << lane) - 1u;
    for (int pass = 0; pass < n_passes; ++pass) {
        const int shift = first_bit + 8 * pass;
#pragma unroll
        for (int k = 0; k < 4; ++k) reinterpret_cast<unsigned*>(my_hist)[lane + 32 * k] = 0u;
        __syncwarp();
        for (int i0 = begin; i0 < end; i0 += 32) {
            const int i = i0 + lane;
            const bool active = i < end;
            const unsigned act = __ballot_sync(0xffffffffu, active);
            if (active) {
                const unsigned digit = unsigned(a[i] >> shift) & 0xFFu;
                const unsigned peers = __match_any_sync(act, digit);
                const int leader = __ffs(peers) - 1;
                unsigned before = 0u;
                if (lane == leader) {
                    before = my_hist[digit];
                    my_hist[digit] = uint16_t(before + __popc(peers));
                }
                before = __shfl_sync(act, before, leader);
                ranks[i] = uint16_t(before + __popc(peers & lt_mask));
            }
            __syncwarp();
        }
        __syncthreads();
        if (threadIdx.x < 256) {
            unsigned run = 0u;
            for (int w = 0; w < n_warps; ++w) {
                const unsigned c = hist[w * 256 + threadIdx.x];
                hist[w * 256 + threadIdx.x] = uint16_t(run);
                run += c;
            }
            unsigned incl = run;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const unsigned o = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += o;
            }
            totals[threadIdx.x] = uint16_t(incl - run);
            if (lane == 31) warp_sums[warp] = incl;
        }
        __syncthreads();
        unsigned group_base = 0u;
#pragma unroll
        for (int k = 0; k < 7; ++k) group_base += k < lane ? warp_sums[k] : 0u;
        for (int i0 = begin; i0 < end; i0 += 32) {
            const int i = i0 + lane;
            const bool active = i < end;
            const uint64_t key = active ? a[i] : 0ull;
            const unsigned digit = unsigned(key >> shift) & 0xFFu;
            const unsigned base = __shfl_sync(0xffffffffu, group_base, int(digit >> 5));
            if (active) b[base + unsigned(totals[digit]) + unsigned(my_hist[digit]) + unsigned(ranks[i])] = key;
        }
        __threadfence_block();
        __syncthreads();
        uint64_t* t = a; a = b; b = t;
    }
    return a;
}

__device__ __forceinline__ int common_upper_bits(uint64_t a, uint64_t b) { return __clzll(int64_t(a ^ b)); }

// Code functor: plain key (BVH fit) or (key & high 32 bits) + sorted position (convolution fit).
struct PlainCode {
    const uint64_t* keys;
    __device__ __forceinline__ uint64_t operator()(int idx) const { return keys[idx]; }
};
struct PositionTieBreakCode {
    const uint64_t* keys;
    __device__ __forceinline__ uint64_t operator()(int idx) const {
        return (keys[idx] & 0xFFFFFFFF00000000ull) + uint64_t(uint32_t(idx));
    }
};

template <typename Code>
__device__ __forceinline__ int2 determine_range(const Code& code, int num_leaves, int idx) {
    if (idx == 0) return make_int2(0, num_leaves - 1);
    const uint64_t self = code(idx);
    const int l_delta = common_upper_bits(self, code(idx - 1));
    const int r_delta = common_upper_bits(self, code(idx + 1));
    const int d = (r_delta > l_delta) ? 1 : -1;
    const int delta_min = min(l_delta, r_delta);
    auto delta_at = [&](long long i) -> int {
        return (i >= 0 && i < num_leaves) ? common_upper_bits(self, code(int(i))) : -1;
    };
    int l_max = 2;
    while (delta_at((long long)idx + (long long)d * l_max) > delta_min) l_max <<= 1;
    int l = 0;
    for (int t = l_max >> 1; t > 0; t >>= 1) {
        if (delta_at((long long)idx + (long long)(l + t) * d) > delta_min) l += t;
    }
    const int jdx = idx + l * d;
    return d < 0 ? make_int2(jdx, idx) : make_int2(idx, jdx);
}

template <typename Code>
__device__ __forceinline__ int find_split(const Code& code, int first, int last) {
    const uint64_t first_code = code(first), last_code = code(last);
    if (first_code == last_code) return (first + last) >> 1;
    const int delta_node = common_upper_bits(first_code, last_code);
    int split = first;
    int stride = last - first;
    do {
        stride = (stride + 1) >> 1;
        const int middle = split + stride;
        if (middle < last && common_upper_bits(first_code, code(middle)) > delta_node) split = middle;
    } while (stride > 1);
    return split;
}

__host__ __device__ __forceinline__ int next_pow2(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

}  // namespace lbvh
}  // namespace gmc
