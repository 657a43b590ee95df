// TEST INFRASTRUCTURE, NOT PRODUCT CODE. CPU restatement (fp32, IEEE) of the reference's fused convolution + fit:
// data [B, Cin, G, V] (*) kernels [Cout, Cin, Gk, V] -> K Gaussians per (batch, out channel) without materialising the
// T = Cin*G*Gk product Gaussians.
//
// Follows src/gmc/cpp/extensions/convolution_fitting/:
//   product index split      util/helper.h:9-24 (component_in fastest, then channel_in, then kernel component)
//   bounding box             Tree.cu:63-77   (max/min over channels of data extreme + kernel extreme)
//   keys                     Tree.cu:79-137  ((w_d w_k > 0) << 62 | morton30 << 32 | product index)
//   sort                     morton_code.h (stable on bits 32..62 == full-key sort, because bit 63 is clear and the
//                            low word ascends with the input order)
//   leaves / internal nodes  Tree.cu:139-227, building.h (Karras on (key & high word) + sorted position)
//   mass                     Tree.cu:229-297 -- pinned to mass(node) = mass(left) + mass(right): the reference adds
//                            with two independent atomics, which gives this value in the race-free interleaving
//   selection                Tree.cu:299-408 (greedy split of the internal node with the largest |mass|)
//   aggregation              implementation_forward.h:19-124 with util/welford.h:11-69 (sequential, sorted order)
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
inline uint32_t quantise_sum(float a, float b, float lower, float upper) {
    const float extent = upper - lower;
    if (!(extent > 0.0f)) return 0u;
    float p = (a + b) - lower;
    p = p / extent;
    const float scaled = p * 1024.0f;
    uint32_t q = scaled > 0.0f ? static_cast<uint32_t>(scaled) : 0u;
    return std::min(q, 1023u);
}
inline int common_upper_bits(uint64_t a, uint64_t b) { return a == b ? 64 : __builtin_clzll(a ^ b); }

struct Codes {
    const uint64_t* keys;
    uint64_t operator()(long long i) const { return (keys[i] & 0xFFFFFFFF00000000ull) + (uint64_t)(uint32_t)i; }
};

void karras(const uint64_t* keys, int n_leaves, std::vector<int>& parent, std::vector<int>& left, std::vector<int>& right,
            std::vector<int>& first, std::vector<int>& last) {
    Codes code{keys};
    const int n_internal = n_leaves - 1;
    parent.assign(2 * n_leaves - 1, -1);
    left.assign(n_internal, -1);
    right.assign(n_internal, -1);
    first.assign(n_internal, 0);
    last.assign(n_internal, 0);
    for (int idx = 0; idx < n_internal; ++idx) {
        int lo = 0, hi = n_leaves - 1;
        if (idx != 0) {
            const uint64_t self = code(idx);
            const int L = common_upper_bits(self, code(idx - 1)), R = common_upper_bits(self, code(idx + 1));
            const int d = R > L ? 1 : -1;
            const int delta_min = std::min(L, R);
            auto delta_at = [&](long long i) { return (i >= 0 && i < n_leaves) ? common_upper_bits(self, code(i)) : -1; };
            int l_max = 2;
            while (delta_at((long long)idx + (long long)d * l_max) > delta_min) l_max <<= 1;
            int l = 0;
            for (int t = l_max >> 1; t > 0; t >>= 1)
                if (delta_at((long long)idx + (long long)(l + t) * d) > delta_min) l += t;
            const int j = idx + l * d;
            lo = std::min(idx, j);
            hi = std::max(idx, j);
        }
        int split;
        const uint64_t fc = code(lo), lc = code(hi);
        if (fc == lc) split = (lo + hi) >> 1;
        else {
            const int delta_node = common_upper_bits(fc, lc);
            split = lo;
            int stride = hi - lo;
            do {
                stride = (stride + 1) >> 1;
                const int middle = split + stride;
                if (middle < hi && common_upper_bits(fc, code(middle)) > delta_node) split = middle;
            } while (stride > 1);
        }
        int l = split, r = split + 1;
        if (lo == split) l += n_leaves - 1;
        if (hi == split + 1) r += n_leaves - 1;
        left[idx] = l; right[idx] = r; first[idx] = lo; last[idx] = hi;
        parent[l] = idx; parent[r] = idx;
    }
}

template <int D>
void fit_tree(const float* data_b, const float* kernels_o, int Cin, int G, int Gk, int K, float* out, float* cached,
              int32_t* nodesobjs, int32_t* subtrees, uint64_t* keys_out) {
    constexpr int RF = 1 + D + D * D;
    const int T = Cin * G * Gk;
    const int n_internal = T - 1;
    // bounding box: max over channels of (data max + kernel max), min likewise
    float upper[D], lower[D];
    for (int c = 0; c < Cin; ++c) {
        float du[D], dl[D], ku[D], kl[D];
        for (int d = 0; d < D; ++d) {
            du[d] = dl[d] = data_b[((size_t)c * G) * RF + 1 + d];
            for (int g = 1; g < G; ++g) {
                const float v = data_b[((size_t)c * G + g) * RF + 1 + d];
                du[d] = std::max(du[d], v); dl[d] = std::min(dl[d], v);
            }
            ku[d] = kl[d] = kernels_o[((size_t)c * Gk) * RF + 1 + d];
            for (int g = 1; g < Gk; ++g) {
                const float v = kernels_o[((size_t)c * Gk + g) * RF + 1 + d];
                ku[d] = std::max(ku[d], v); kl[d] = std::min(kl[d], v);
            }
            const float u = du[d] + ku[d], l = dl[d] + kl[d];
            if (c == 0) { upper[d] = u; lower[d] = l; }
            else { upper[d] = std::max(upper[d], u); lower[d] = std::min(lower[d], l); }
        }
    }
    auto split = [&](uint32_t t, int& comp_in, int& ch_in, int& comp_k) {
        comp_k = t / (G * Cin);
        t -= comp_k * (G * Cin);
        ch_in = t / G;
        comp_in = t - ch_in * G;
    };
    std::vector<uint64_t> keys(T);
    for (int t = 0; t < T; ++t) {
        int gi, ci, ki;
        split(t, gi, ci, ki);
        const float* dg = data_b + ((size_t)ci * G + gi) * RF;
        const float* kg = kernels_o + ((size_t)ci * Gk + ki) * RF;
        uint32_t q[3] = {0, 0, 0};
        for (int d = 0; d < D; ++d) q[d] = quantise_sum(dg[1 + d], kg[1 + d], lower[d], upper[d]);
        const uint64_t morton = (expand_bits3(q[0]) << 2) + (expand_bits3(q[1]) << 1) + expand_bits3(q[2]);
        const uint64_t sign = (dg[0] * kg[0]) > 0 ? 1 : 0;
        keys[t] = (sign << 62) | (morton << 32) | (uint64_t)t;
    }
    std::sort(keys.begin(), keys.end());
    if (keys_out) std::memcpy(keys_out, keys.data(), sizeof(uint64_t) * T);
    for (int j = 0; j < T; ++j) nodesobjs[j] = (int32_t)(uint32_t)keys[j];

    std::vector<int> parent, left, right, first, last;
    karras(keys.data(), T, parent, left, right, first, last);

    auto leaf_weight = [&](int j) {
        int gi, ci, ki;
        split((uint32_t)nodesobjs[j], gi, ci, ki);
        return data_b[((size_t)ci * G + gi) * RF] * kernels_o[((size_t)ci * Gk + ki) * RF];
    };
    // mass in tree order (children before parents: process by increasing range length)
    std::vector<float> mass(2 * T - 1);
    for (int j = 0; j < T; ++j) mass[n_internal + j] = leaf_weight(j);
    std::vector<int> order(n_internal);
    for (int i = 0; i < n_internal; ++i) order[i] = i;
    std::sort(order.begin(), order.end(), [&](int a, int b) { return (last[a] - first[a]) < (last[b] - first[b]); });
    for (int i : order) mass[i] = mass[left[i]] + mass[right[i]];

    // greedy selection
    std::vector<int> sel;
    std::vector<float> rating;
    auto rate = [&](int id) { return id >= n_internal ? -2.f : std::fabs(mass[id]); };
    sel.push_back(0); rating.push_back(rate(0));
    while ((int)sel.size() < K) {
        float best_rating = -1; int best = -1;
        for (size_t i = 0; i < sel.size(); ++i)
            if (rating[i] > best_rating) { best_rating = rating[i]; best = (int)i; }
        if (best < 0) break;
        const int id = sel[best];
        sel[best] = left[id]; rating[best] = rate(left[id]);
        sel.push_back(right[id]); rating.push_back(rate(right[id]));
    }
    for (int k = 0; k < 2 * K; ++k) subtrees[k] = -1;
    for (size_t k = 0; k < sel.size(); ++k) {
        const int id = sel[k];
        subtrees[2 * k] = id >= n_internal ? id : n_internal + first[id];
        subtrees[2 * k + 1] = id >= n_internal ? id + 1 : n_internal + last[id] + 1;
    }

    // aggregation (sequential weighted Welford in sorted order)
    for (int k = 0; k < K; ++k) {
        float* o = out + (size_t)k * RF;
        float* cp = cached + (size_t)k * D * D;
        const uint32_t start = (uint32_t)subtrees[2 * k];
        if (start >= (uint32_t)(2 * T - 1)) {
            o[0] = 0;
            for (int d = 0; d < D; ++d) o[1 + d] = 0;
            for (int i = 0; i < D * D; ++i) o[1 + D + i] = (i / D == i % D) ? 1.f : 0.f;
            for (int i = 0; i < D * D; ++i) cp[i] = 0.f;   // the reference leaves this slot unwritten
            continue;
        }
        const uint32_t end = (uint32_t)subtrees[2 * k + 1];
        float w_sum = 0, mean[D] = {}, C[D * D] = {};
        float cw_sum = 0, cmean[D * D] = {};
        for (uint32_t i = start; i < end; ++i) {
            int gi, ci, ki;
            split((uint32_t)nodesobjs[i - n_internal], gi, ci, ki);
            const float* dg = data_b + ((size_t)ci * G + gi) * RF;
            const float* kg = kernels_o + ((size_t)ci * Gk + ki) * RF;
            const float w = dg[0] * kg[0];
            float p[D], cov[D * D];
            for (int d = 0; d < D; ++d) p[d] = dg[1 + d] + kg[1 + d];
            for (int e = 0; e < D * D; ++e) cov[e] = dg[1 + D + e] + kg[1 + D + e];
            w_sum += w;
            cw_sum += w;
            if (w == 0.f) continue;
            float d1[D], d2[D];
            const float f = w / w_sum;
            for (int d = 0; d < D; ++d) { d1[d] = p[d] - mean[d]; mean[d] += f * d1[d]; d2[d] = p[d] - mean[d]; }
            // glm::outerProduct(delta1, delta2)[col][row] = delta1[row] * delta2[col]; stored column-major = read back
            // row-major as element (i, j) = delta1[j] * delta2[i]
            for (int i = 0; i < D; ++i)
                for (int j = 0; j < D; ++j) C[i * D + j] += w * (d1[j] * d2[i]);
            const float fc = w / cw_sum;
            for (int e = 0; e < D * D; ++e) cmean[e] += fc * (cov[e] - cmean[e]);
        }
        o[0] = w_sum;
        for (int d = 0; d < D; ++d) o[1 + d] = mean[d];
        for (int e = 0; e < D * D; ++e) {
            const float pc = (w_sum == 0.f) ? ((e / D == e % D) ? 1.f : 0.f) : C[e] / w_sum;
            cp[e] = pc;
            o[1 + D + e] = cmean[e] + pc;
        }
    }
}

}  // namespace

extern "C" {

// data [B, Cin, G, V], kernels [Cout, Cin, Gk, V] -> out [B, Cout, K, V], cached_pos_covs [B, Cout, K, D*D],
// nodesobjs [B, Cout, T] int32, subtrees [B, Cout, 2K] int32 (-1 = unused), optional sorted keys [B, Cout, T].
int oracle_convolution_fitting_forward(const float* data, const float* kernels, int B, int Cin, int G, int Cout, int Gk,
                                       int D, int K, float* out, float* cached_pos_covs, int32_t* nodesobjs,
                                       int32_t* subtrees, uint64_t* keys) {
    if (D != 2 && D != 3) return 1;
    const int RF = 1 + D + D * D;
    const size_t T = (size_t)Cin * G * Gk;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int b = 0; b < B; ++b)
        for (int o = 0; o < Cout; ++o) {
            const size_t m = (size_t)b * Cout + o;
            const float* db = data + (size_t)b * Cin * G * RF;
            const float* ko = kernels + (size_t)o * Cin * Gk * RF;
            if (D == 2) fit_tree<2>(db, ko, Cin, G, Gk, K, out + m * K * RF, cached_pos_covs + m * K * D * D, nodesobjs + m * T, subtrees + m * 2 * K, keys ? keys + m * T : nullptr);
            else fit_tree<3>(db, ko, Cin, G, Gk, K, out + m * K * RF, cached_pos_covs + m * K * D * D, nodesobjs + m * T, subtrees + m * 2 * K, keys ? keys + m * T : nullptr);
        }
    return 0;
}

}  // extern "C"
