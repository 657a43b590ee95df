// TEST INFRASTRUCTURE, NOT PRODUCT CODE. CPU restatement of the reference's linear BVH build over the means of
// each mixture (the make_aabbs = false path that the BVH-MHEM fit uses). Compiled with IEEE fp32 arithmetic
// (no fast-math, no FMA contraction) so that the integer results can be compared bit for bit.
//
// Follows:
//   whole AABB            src/gmc/cpp/extensions/util/mixture.h:129-135 (per-mixture max / min of the means)
//   Morton key            lbvh/bvh.cu:241-299 (normalise into the AABB), lbvh/morton_code.h:145-156 (10 bits per
//                         axis, interleave (xx<<2)+(yy<<1)+zz), :254-263 (key = morton << 16 | component id)
//   sort                  lbvh/morton_code.h:20-75 (ascending per mixture; keys are unique)
//   leaf / internal nodes lbvh/bvh.cu:373-458, lbvh/building.h:11-103 (Karras range + split on clz(a ^ b)),
//                         node layout lbvh/bvh.h:16-24: {parent, left, right, object} as uint16, internal nodes
//                         0..G-2 (root 0), leaves G-1..2G-2 in sorted order, untouched fields stay 0xFFFF.
// Pinned where the reference is undefined: a coordinate whose AABB extent is zero (always the z axis in 2D, 0/0 =
// NaN in the reference) contributes the quantised value 0.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

inline uint32_t expand_bits3(uint32_t v) {
    v = (v * 0x00010001u) & 0xFF0000FFu;
    v = (v * 0x00000101u) & 0x0F00F00Fu;
    v = (v * 0x00000011u) & 0xC30C30C3u;
    v = (v * 0x00000005u) & 0x49249249u;
    return v;
}

inline uint32_t quantise(float pos, float lower, float upper) {
    const float extent = upper - lower;
    if (!(extent > 0.0f)) return 0u;               // pinned: 0/0 in the reference
    float p = pos - lower;
    p = p / extent;
    const float scaled = p * 1024.0f;
    uint32_t q = scaled > 0.0f ? static_cast<uint32_t>(scaled) : 0u;
    return std::min(q, 1023u);
}

inline int common_upper_bits(uint64_t a, uint64_t b) { return a == b ? 64 : __builtin_clzll(a ^ b); }

struct Range { unsigned first, last; };

Range determine_range(const uint64_t* code, unsigned num_leaves, unsigned idx) {
    if (idx == 0) return {0, num_leaves - 1};
    const uint64_t self = code[idx];
    const int L_delta = common_upper_bits(self, code[idx - 1]);
    const int R_delta = common_upper_bits(self, code[idx + 1]);
    const int d = (R_delta > L_delta) ? 1 : -1;
    const int delta_min = std::min(L_delta, R_delta);
    int l_max = 2;
    auto delta_at = [&](long long i) -> int {
        return (0 <= i && i < (long long)num_leaves) ? common_upper_bits(self, code[i]) : -1;
    };
    int delta = delta_at((long long)idx + (long long)d * l_max);
    while (delta > delta_min) {
        l_max <<= 1;
        delta = delta_at((long long)idx + (long long)d * l_max);
    }
    int l = 0;
    for (int t = l_max >> 1; t > 0; t >>= 1) {
        if (delta_at((long long)idx + (long long)(l + t) * d) > delta_min) l += t;
    }
    unsigned jdx = idx + l * d;
    if (d < 0) std::swap(idx, jdx);
    return {idx, jdx};
}

unsigned find_split(const uint64_t* code, unsigned first, unsigned last) {
    const uint64_t first_code = code[first], last_code = code[last];
    if (first_code == last_code) return (first + last) >> 1;
    const int delta_node = common_upper_bits(first_code, last_code);
    int split = first;
    int stride = last - first;
    do {
        stride = (stride + 1) >> 1;
        const int middle = split + stride;
        if (middle < (int)last && common_upper_bits(first_code, code[middle]) > delta_node) split = middle;
    } while (stride > 1);
    return split;
}

}  // namespace

extern "C" {

// mixture: [n_mixtures, G, 1+D+D*D] fp32 (only the means are read). sorted_keys: [n_mixtures, G] uint64.
// nodes: [n_mixtures, 2G-1, 4] uint16 {parent, left, right, object}.
void oracle_lbvh_build(const float* mixture, int n_mixtures, int G, int D, uint64_t* sorted_keys, uint16_t* nodes) {
    const int RF = 1 + D + D * D;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < n_mixtures; ++m) {
        const float* mix = mixture + (size_t)m * G * RF;
        float lower[3] = {0, 0, 0}, upper[3] = {0, 0, 0};
        for (int d = 0; d < D; ++d) {
            lower[d] = upper[d] = mix[1 + d];
            for (int g = 1; g < G; ++g) {
                lower[d] = std::min(lower[d], mix[(size_t)g * RF + 1 + d]);
                upper[d] = std::max(upper[d], mix[(size_t)g * RF + 1 + d]);
            }
        }
        uint64_t* keys = sorted_keys + (size_t)m * G;
        for (int g = 0; g < G; ++g) {
            uint32_t q[3] = {0, 0, 0};
            for (int d = 0; d < D; ++d) q[d] = quantise(mix[(size_t)g * RF + 1 + d], lower[d], upper[d]);
            const uint32_t morton = (expand_bits3(q[0]) << 2) + (expand_bits3(q[1]) << 1) + expand_bits3(q[2]);
            keys[g] = ((uint64_t)morton << 16) | (uint64_t)(uint16_t)g;
        }
        std::sort(keys, keys + G);
        uint16_t* nd = nodes + (size_t)m * (2 * G - 1) * 4;
        std::memset(nd, 0xFF, sizeof(uint16_t) * (size_t)(2 * G - 1) * 4);
        for (int j = 0; j < G; ++j) nd[(size_t)(G - 1 + j) * 4 + 3] = (uint16_t)keys[j];
        for (int i = 0; i < G - 1; ++i) {
            const Range r = determine_range(keys, G, i);
            const unsigned gamma = find_split(keys, r.first, r.last);
            unsigned left = gamma, right = gamma + 1;
            if (std::min(r.first, r.last) == gamma) left += G - 1;
            if (std::max(r.first, r.last) == gamma + 1) right += G - 1;
            nd[(size_t)i * 4 + 1] = (uint16_t)left;
            nd[(size_t)i * 4 + 2] = (uint16_t)right;
            nd[(size_t)i * 4 + 3] = (uint16_t)i;
            nd[(size_t)left * 4 + 0] = (uint16_t)i;
            nd[(size_t)right * 4 + 0] = (uint16_t)i;
        }
    }
}

}  // extern "C"
