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
#include <cmath>
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


// ---------------------------------------------------------------------------------------------------------------
// Options of lbvh::Config (lbvh/Config.h): the covariance-aware key layouts (lbvh/morton_code.h:170-252, cov_diag =
// diagonal of the matrix slot divided by its per-mixture maximum, lbvh/bvh.cu:254-276) and make_aabbs
// (ellipsoid boxes of the leaves lbvh/bvh.cu:164-231, bottom-up merge :460-510).
// ---------------------------------------------------------------------------------------------------------------
}  // extern "C"

namespace {

inline uint64_t expand_bits2(uint32_t v) {
    uint64_t t = v;
    t = ((t << 16) | t) & 0x0000FFFF0000FFFFull;
    t = ((t << 8) | t) & 0x00FF00FF00FF00FFull;
    t = ((t << 4) | t) & 0x0F0F0F0F0F0F0F0Full;
    t = ((t << 2) | t) & 0x3333333333333333ull;
    t = ((t << 1) | t) & 0x5555555555555555ull;
    return t;
}

inline uint64_t mix_key(int algorithm, uint32_t pos, uint32_t cov, uint16_t id) {
    switch (algorithm) {
        case 0: return ((uint64_t)pos << 16) | id;
        case 1: {   // 12 bits position, 18 + 18 bits position / covariance interleaved, 16 bits id
            uint64_t result = pos >> 18;
            const uint64_t poscov = (expand_bits2(pos & 0x3FFFFu) << 1) | expand_bits2(cov >> 12);
            result = (result << 36) | poscov;
            return (result << 16) | id;
        }
        case 2: return (((((expand_bits2(pos) << 1) | expand_bits2(cov)) << 4) & 0xFFFFFFFFFFFFFC00ull) | id);
        case 3: return ((uint64_t)(pos & ~0x7u) << 34) | ((uint64_t)(cov & ~0x7u) << 7) | (uint64_t)(id & 0x3FF);
        default: return ((uint64_t)(cov & ~0x7u) << 34) | ((uint64_t)(pos & ~0x7u) << 7) | (uint64_t)(id & 0x3FF);
    }
}

inline uint32_t quantise_unit(float v) {            // lbvh/morton_code.h:145-168: min(max(uint32(v * 1024), 0), 1023)
    const float scaled = v * 1024.0f;
    const uint32_t q = scaled > 0.0f ? static_cast<uint32_t>(scaled) : 0u;
    return std::min(q, 1023u);
}

void inverse_small(const float* m, int D, float* o) {
    if (D == 2) {
        const float r = 1.f / (m[0] * m[3] - m[1] * m[2]);
        o[0] = m[3] * r; o[1] = -m[1] * r; o[2] = -m[2] * r; o[3] = m[0] * r;
        return;
    }
    const float det = m[0] * (m[4] * m[8] - m[5] * m[7]) - m[1] * (m[3] * m[8] - m[5] * m[6]) + m[2] * (m[3] * m[7] - m[4] * m[6]);
    const float r = 1.f / det;
    o[0] = (m[4] * m[8] - m[5] * m[7]) * r; o[1] = -(m[1] * m[8] - m[2] * m[7]) * r; o[2] = (m[1] * m[5] - m[2] * m[4]) * r;
    o[3] = -(m[3] * m[8] - m[5] * m[6]) * r; o[4] = (m[0] * m[8] - m[2] * m[6]) * r; o[5] = -(m[0] * m[5] - m[2] * m[3]) * r;
    o[6] = (m[3] * m[7] - m[4] * m[6]) * r; o[7] = -(m[0] * m[7] - m[1] * m[6]) * r; o[8] = (m[0] * m[4] - m[1] * m[3]) * r;
}

using real = float;

// Closed form of math/symeig_detail.h:17-138, in fp32 like the reference: with two close eigenvalues the eigenvectors, and
// through them the boxes, depend on the rounding, so the arithmetic type is part of the definition.
// val ascending, vec[k * D + r] = component k of eigenvector r.
void symeig_small(const float* Af, int D, real* val, real* vec) {
    real A[9];
    for (int i = 0; i < D * D; ++i) A[i] = Af[i];
    if (D == 2) {
        const real a = A[0], b = A[2], d = A[3];
        const real T = a + d, det = a * d - A[1] * A[2];
        const real f1 = T * real(0.5), f2 = std::sqrt(std::fabs(T * T * real(0.25) - det));
        val[0] = f1 - f2; val[1] = f1 + f2;
        if (b == real(0.0)) { vec[0] = 1; vec[1] = 0; vec[2] = 0; vec[3] = 1; return; }
        real e0x, e0y, e1x, e1y;
        if (a < d) { e0x = b; e0y = val[0] - a; e1x = b; e1y = val[1] - a; }
        else { e0x = val[0] - d; e0y = b; e1x = val[1] - d; e1y = b; }
        const real n0 = real(1.0) / std::sqrt(e0x * e0x + e0y * e0y), n1 = real(1.0) / std::sqrt(e1x * e1x + e1y * e1y);
        vec[0] = e0x * n0; vec[1] = e1x * n1; vec[2] = e0y * n0; vec[3] = e1y * n1;
        return;
    }
    const real* m = A;
    real eig0, eig1, eig2;
    const real p1 = m[1] * m[1] + m[2] * m[2] + m[5] * m[5];
    if (p1 <= real(0.0000001)) { eig0 = m[0]; eig1 = m[4]; eig2 = m[8]; }
    else {
        const real q = (m[0] + m[4] + m[8]) / real(3.0);
        const real p2 = (m[0] - q) * (m[0] - q) + (m[4] - q) * (m[4] - q) + (m[8] - q) * (m[8] - q) + real(2.0) * p1;
        const real pp = std::sqrt(p2 / real(6.0));
        real B[9];
        for (int k = 0; k < 9; ++k) B[k] = (m[k] - ((k % 4 == 0) ? q : real(0.0))) / pp;
        const real r = real(0.5) * (B[0] * (B[4] * B[8] - B[5] * B[7]) - B[1] * (B[3] * B[8] - B[5] * B[6]) + B[2] * (B[3] * B[7] - B[4] * B[6]));
        const real pi = real(3.14159265358979323846);
        real phi;
        if (r <= -real(1.0)) phi = pi / real(3.0);
        else if (r >= real(1.0)) phi = real(0.0);
        else phi = std::acos(r) / real(3.0);
        eig0 = q + real(2.0) * pp * std::cos(phi);
        eig2 = q + real(2.0) * pp * std::cos(phi + real(2.0) * pi / real(3.0));
        eig1 = real(3.0) * q - eig0 - eig2;
    }
    auto longest = [&](real s, real t, real* v) {     // longest column of (A - s I)(A - t I), normalised
        real X[9], Y[9], P[9];
        for (int k = 0; k < 9; ++k) { X[k] = m[k] - ((k % 4 == 0) ? s : real(0.0)); Y[k] = m[k] - ((k % 4 == 0) ? t : real(0.0)); }
        for (int r2 = 0; r2 < 3; ++r2)
            for (int c = 0; c < 3; ++c) P[r2 * 3 + c] = X[r2 * 3] * Y[c] + X[r2 * 3 + 1] * Y[3 + c] + X[r2 * 3 + 2] * Y[6 + c];
        real best = 0; int idx = 0;
        for (int c = 0; c < 3; ++c) {
            const real len = P[c] * P[c] + P[3 + c] * P[3 + c] + P[6 + c] * P[6 + c];
            if (len > best) { best = len; idx = c; }
        }
        const real inv = real(1.0) / std::sqrt(best);
        v[0] = P[idx] * inv; v[1] = P[3 + idx] * inv; v[2] = P[6 + idx] * inv;
    };
    real v0[3], v1[3], v2[3];
    longest(eig1, eig2, v0);
    longest(eig0, eig2, v1);
    v2[0] = v0[1] * v1[2] - v0[2] * v1[1];
    v2[1] = v0[2] * v1[0] - v0[0] * v1[2];
    v2[2] = v0[0] * v1[1] - v0[1] * v1[0];
    val[0] = eig2; val[1] = eig1; val[2] = eig0;
    for (int r2 = 0; r2 < 3; ++r2) { vec[r2 * 3 + 0] = v2[r2]; vec[r2 * 3 + 1] = v1[r2]; vec[r2 * 3 + 2] = v0[r2]; }
}

}  // namespace

extern "C" {

// As oracle_lbvh_build with the options of lbvh::Config. aabbs (may be NULL unless make_aabbs): [n_mixtures, 2G-1, 8]
// = upper.xyzw, lower.xyzw. With make_aabbs the matrix slot of the mixture holds INVERSE covariances (lbvh/bvh.cu:204).
// Returns 1 for make_aabbs with a key layout whose low 16 bits are not the component id (layouts 2..4).
int oracle_lbvh_build_ex(const float* mixture, int n_mixtures, int G, int D, int algorithm, int make_aabbs, float threshold,
                         uint64_t* sorted_keys, uint16_t* nodes, float* aabbs) {
    if (make_aabbs && algorithm > 1) return 1;
    const int RF = 1 + D + D * D;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < n_mixtures; ++m) {
        const float* mix = mixture + (size_t)m * G * RF;
        float lower[3] = {0, 0, 0}, upper[3] = {0, 0, 0}, cov_max[3] = {0, 0, 0};
        for (int d = 0; d < D; ++d) {
            lower[d] = upper[d] = mix[1 + d];
            cov_max[d] = mix[1 + D + d * D + d];
            for (int g = 1; g < G; ++g) {
                lower[d] = std::min(lower[d], mix[(size_t)g * RF + 1 + d]);
                upper[d] = std::max(upper[d], mix[(size_t)g * RF + 1 + d]);
                cov_max[d] = std::max(cov_max[d], mix[(size_t)g * RF + 1 + D + d * D + d]);
            }
        }
        uint64_t* keys = sorted_keys + (size_t)m * G;
        for (int g = 0; g < G; ++g) {
            uint32_t q[3] = {0, 0, 0}, c[3] = {0, 0, 0};
            for (int d = 0; d < D; ++d) {
                q[d] = quantise(mix[(size_t)g * RF + 1 + d], lower[d], upper[d]);
                c[d] = quantise_unit(mix[(size_t)g * RF + 1 + D + d * D + d] / cov_max[d]);
            }
            const uint32_t pos = (expand_bits3(q[0]) << 2) + (expand_bits3(q[1]) << 1) + expand_bits3(q[2]);
            const uint32_t cov = (expand_bits3(c[0]) << 2) + (expand_bits3(c[1]) << 1) + expand_bits3(c[2]);
            keys[g] = mix_key(algorithm, pos, cov, (uint16_t)g);
        }
        std::sort(keys, keys + G);
        uint16_t* nd = nodes + (size_t)m * (2 * G - 1) * 4;
        std::memset(nd, 0xFF, sizeof(uint16_t) * (size_t)(2 * G - 1) * 4);
        for (int j = 0; j < G; ++j) nd[(size_t)(G - 1 + j) * 4 + 3] = (uint16_t)keys[j];
        std::vector<unsigned> first(G - 1), last(G - 1);
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
            first[i] = r.first; last[i] = r.last;
        }
        if (!make_aabbs) continue;
        float* bx = aabbs + (size_t)m * (2 * G - 1) * 8;
        std::memset(bx, 0, sizeof(float) * (size_t)(2 * G - 1) * 8);
        for (int j = 0; j < G; ++j) {
            const float* g = mix + (size_t)nd[(size_t)(G - 1 + j) * 4 + 3] * RF;
            float factor = -2.f * std::log(threshold / std::fabs(g[0]));
            factor = std::sqrt(std::max(factor, float(-2 * -2.995732273553991)));
            float cov[9];
            inverse_small(g + 1 + D, D, cov);
            real val[3], vec[9];
            symeig_small(cov, D, val, vec);
            float* b = bx + (size_t)(G - 1 + j) * 8;
            for (int r = 0; r < D; ++r) {
                // the reference pairs eigenvector r with coordinate r and weights its components with ALL eigenvalues:
                // length of column r of transpose(factor * E diag(sqrt lambda)), E holding the eigenvectors in its rows
                real acc = 0;
                for (int k = 0; k < D; ++k) acc += val[k] * vec[k * D + r] * vec[k * D + r];
                const float delta = factor * (float)std::sqrt(acc);
                b[r] = g[1 + r] + delta;
                b[4 + r] = g[1 + r] - delta;
            }
        }
        // internal boxes: children before parents (shorter leaf ranges first)
        std::vector<int> order(G - 1);
        for (int i = 0; i < G - 1; ++i) order[i] = i;
        std::sort(order.begin(), order.end(), [&](int a, int b2) { return (last[a] - first[a]) < (last[b2] - first[b2]); });
        for (int i : order) {
            const float* l = bx + (size_t)nd[(size_t)i * 4 + 1] * 8;
            const float* r = bx + (size_t)nd[(size_t)i * 4 + 2] * 8;
            float* o = bx + (size_t)i * 8;
            for (int d = 0; d < 3; ++d) { o[d] = std::fmax(l[d], r[d]); o[4 + d] = std::fmin(l[4 + d], r[4 + d]); }
        }
    }
    return 0;
}
}  // extern "C"
