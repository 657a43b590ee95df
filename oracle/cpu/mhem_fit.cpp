// TEST INFRASTRUCTURE, NOT PRODUCT CODE. CPU restatement (fp32) of the reference's BVH-MHEM reduction of a mixture
// of G Gaussians to K Gaussians: bottom-up pass over the LBVH in which every internal node fits at most R Gaussians
// to the (at most 2R) Gaussians of its children with one hierarchical-EM step, then a greedy top-down selection of
// nodes by |integral|.
//
// Follows src/gmc/cpp/extensions/bvh_mhem_fit/implementation_forward.h:
//   cluster_centroid_distance :35-42      clusterise_using_heap :45-140 (min-heap util/containers.h:84-177)
//   cluster_select_maxWeight  :143-162    fit_initial           :165-186
//   fit_em                    :188-323    iterate_over_nodes    :325-393
//   collect_result            :395-484
// and implementation_common.h:98-106 (collect_child_gaussians), util/gaussian.h:97-129 (likelihood with 4 virtual
// points, kl_divergence), util/epsilon.h:9-15 (small = 1e-13, large = 1e-7), bvh_mhem_fit/Config.h:10
// (em_kl_div_threshold = 0.5).
// Pinned where the reference is undefined: if the disparity heap runs out of finite entries before R clusters are
// reached (only possible with mixed-sign inputs, which the reference does not support), merging stops and the first R
// non-empty clusters are used.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

namespace {

constexpr float kEpsSmall = 0.0000000000001f;
constexpr float kEpsLarge = 0.0000001f;
constexpr float kKlThreshold = 0.5f;
inline float clip(float v) { return std::max(v, kEpsSmall); }
inline int sign_of(float v) { return v >= 0 ? 1 : -1; }

template <int D>
struct Gaussian {
    float w;
    float p[D];
    float c[D * D];
};

template <int D>
Gaussian<D> zero_identity() {
    Gaussian<D> g;
    g.w = 0;
    for (int i = 0; i < D; ++i) g.p[i] = 0;
    for (int i = 0; i < D * D; ++i) g.c[i] = (i / D == i % D) ? 1.f : 0.f;
    return g;
}

template <int D> float det(const float* m);
template <> float det<2>(const float* m) { return m[0] * m[3] - m[1] * m[2]; }
template <> float det<3>(const float* m) {
    return m[0] * (m[4] * m[8] - m[5] * m[7]) - m[1] * (m[3] * m[8] - m[5] * m[6]) + m[2] * (m[3] * m[7] - m[4] * m[6]);
}
template <int D> void inverse(const float* m, float* o);
template <> void inverse<2>(const float* m, float* o) {
    const float r = 1.f / det<2>(m);
    o[0] = m[3] * r; o[1] = -m[1] * r; o[2] = -m[2] * r; o[3] = m[0] * r;
}
template <> void inverse<3>(const float* m, float* o) {
    const float r = 1.f / det<3>(m);
    o[0] = (m[4] * m[8] - m[5] * m[7]) * r; o[1] = -(m[1] * m[8] - m[2] * m[7]) * r; o[2] = (m[1] * m[5] - m[2] * m[4]) * r;
    o[3] = -(m[3] * m[8] - m[5] * m[6]) * r; o[4] = (m[0] * m[8] - m[2] * m[6]) * r; o[5] = -(m[0] * m[5] - m[2] * m[3]) * r;
    o[6] = (m[3] * m[7] - m[4] * m[6]) * r; o[7] = -(m[0] * m[7] - m[1] * m[6]) * r; o[8] = (m[0] * m[4] - m[1] * m[3]) * r;
}

template <int D>
float quad_form(const float* S, const float* t) {
    float v = 0;
    for (int i = 0; i < D; ++i) {
        float s = 0;
        for (int j = 0; j < D; ++j) s += S[i * D + j] * t[j];
        v += t[i] * s;
    }
    return v;
}

template <int D>
float trace_of_product(const float* a, const float* b) {   // trace(a * b)
    float t = 0;
    for (int i = 0; i < D; ++i)
        for (int j = 0; j < D; ++j) t += a[i * D + j] * b[j * D + i];
    return t;
}

// util/gaussian.h:104-113
template <int D>
float likelihood(const Gaussian<D>& target, const Gaussian<D>& fitting) {
    const float factor = float(std::pow(2.0 * M_PI, -0.5 * D));
    float inv[D * D];
    inverse<D>(fitting.c, inv);
    float t[D];
    for (int i = 0; i < D; ++i) t[i] = target.p[i] - fitting.p[i];
    const float a = std::sqrt(det<D>(inv)) * factor * std::exp(-0.5f * quad_form<D>(inv, t));
    const float b = std::exp(-0.5f * trace_of_product<D>(inv, target.c));
    const float wi_bar = 4.f * target.w;
    return std::pow(clip(a * b), wi_bar);
}

// util/gaussian.h:115-129
template <int D>
float kl_divergence(const Gaussian<D>& target, const Gaussian<D>& fitting) {
    float inv[D * D];
    inverse<D>(fitting.c, inv);
    float t[D];
    for (int i = 0; i < D; ++i) t[i] = target.p[i] - fitting.p[i];
    const float maha = quad_form<D>(inv, t);
    const float tr = trace_of_product<D>(inv, target.c);
    const float lg = std::log(det<D>(target.c) / det<D>(fitting.c));
    return 0.5f * (maha + tr - float(D) - lg);
}

// min-heap of util/containers.h:84-177 on (disparity, a, b) compared by disparity with <=
struct Disparity {
    float d;
    uint8_t a, b;
};
template <int N>
struct Heap {
    Disparity data[N];
    static bool two_children(unsigned i) { return i < (N - 1) / 2; }
    static bool is_leaf(unsigned i) { return i >= N / 2; }
    Disparity replace_element(Disparity value, unsigned index) {
        const Disparity ret = data[index];
        unsigned cur = index;
        while (two_children(cur)) {
            const unsigned l = cur * 2 + 1, r = cur * 2 + 2;
            const Disparity lv = data[l], rv = data[r];
            if (value.d <= lv.d && value.d <= rv.d) break;
            if (lv.d <= rv.d) { data[cur] = lv; cur = l; }
            else { data[cur] = rv; cur = r; }
        }
        if (!is_leaf(cur)) {
            const unsigned l = cur * 2 + 1;
            const Disparity lv = data[l];
            if (lv.d <= value.d) { data[cur] = lv; cur = l; }
        }
        data[cur] = value;
        return ret;
    }
    void build() {
        for (unsigned i = (N - 1 - 1) / 2; i < unsigned(N); --i) {
            const Disparity copy = data[i];
            replace_element(copy, i);
        }
    }
};

// fit_initial (:165-186): indices (into the padded target array) of the R initial representatives
template <int D, int R>
void fit_initial(const Gaussian<D>* target, uint8_t* result) {
    constexpr int NT = 2 * R;
    constexpr int NH = (NT * NT - NT) / 2;
    const float inf = std::numeric_limits<float>::infinity();
    uint8_t valid[NT];
    int n_valid = 0;
    for (int i = 0; i < NT; ++i)
        if (std::fabs(target[i].w) >= kEpsLarge) valid[n_valid++] = uint8_t(i);

    auto disparity = [&](int i, int j) -> float {
        const Gaussian<D>& a = target[i];
        const Gaussian<D>& b = target[j];
        if (sign_of(a.w) != sign_of(b.w)) return inf;
        if (std::fabs(a.w) < kEpsLarge || std::fabs(b.w) < kEpsLarge) return inf;
        float s = 0;
        for (int d = 0; d < D; ++d) s += (a.p[d] - b.p[d]) * (a.p[d] - b.p[d]);
        return s;
    };

    // sub-graphs, indexed by position in the valid list
    uint8_t members[NT][NT];
    int n_members[NT];
    for (int i = 0; i < n_valid; ++i) { members[i][0] = valid[i]; n_members[i] = 1; }
    int n_subgraphs = n_valid;

    Heap<NH> heap;
    int n_disp = 0;
    for (int i = 0; i < n_valid; ++i)
        for (int j = i + 1; j < n_valid; ++j) heap.data[n_disp++] = Disparity{disparity(valid[i], valid[j]), valid[i], valid[j]};
    const Disparity invalid{inf, 255, 255};
    for (int i = n_disp; i < NH; ++i) heap.data[i] = invalid;
    heap.build();

    auto subgraph_of = [&](uint8_t id) -> int {
        for (int i = 0; i < n_valid; ++i)
            for (int j = 0; j < n_members[i]; ++j)
                if (members[i][j] == id) return i;
        return -1;
    };
    while (n_subgraphs > R) {
        const Disparity cur = heap.replace_element(invalid, 0);
        if (!(cur.d < inf)) break;   // pinned: no finite disparity left
        const int sa = subgraph_of(cur.a), sb = subgraph_of(cur.b);
        if (sa != sb) {
            const int lo = std::min(sa, sb), hi = std::max(sa, sb);
            for (int j = 0; j < n_members[hi]; ++j) members[lo][n_members[lo]++] = members[hi][j];
            n_members[hi] = 0;
            --n_subgraphs;
        }
    }
    int sg = -1;
    for (int i = 0; i < R; ++i) {
        do { ++sg; } while (sg < n_valid && n_members[sg] == 0);
        // cluster_select_maxWeight (:143-162)
        uint8_t selected = 255;
        float max_abs = 0;
        if (sg < n_valid) {
            for (int j = 0; j < n_members[sg]; ++j) {
                const uint8_t gid = members[sg][j];
                if (std::fabs(target[gid].w) > max_abs) { max_abs = std::fabs(target[gid].w); selected = gid; }
            }
        }
        result[i] = selected;
    }
}

// fit_em (:188-323). target: n_target (> R, <= 2R) Gaussians; result: R Gaussians; initial_out: the cached indices.
template <int D, int R>
void fit_em(const Gaussian<D>* target_in, int n_target, Gaussian<D>* result, uint8_t* initial_out) {
    constexpr int NT = 2 * R;
    Gaussian<D> target[NT];
    for (int i = 0; i < NT; ++i) target[i] = i < n_target ? target_in[i] : zero_identity<D>();

    float target_integral = 0;
    for (int i = 0; i < NT; ++i) target_integral += target[i].w;
    const float target_clipped_integral = clip(target_integral);
    float int1_w[NT];
    for (int i = 0; i < NT; ++i) int1_w[i] = target[i].w / target_clipped_integral;

    uint8_t idx[R];
    fit_initial<D, R>(target, idx);
    for (int s = 0; s < R; ++s) initial_out[s] = idx[s];

    float initial_integral = 0;
    for (int s = 0; s < R; ++s) initial_integral += target[idx[s]].w;
    const float initial_clipped_integral = clip(initial_integral);
    Gaussian<D> initial_int1[R];
    for (int s = 0; s < R; ++s) {
        initial_int1[s] = target[idx[s]];
        initial_int1[s].w = target[idx[s]].w / initial_clipped_integral;
    }
    Gaussian<D> target_int1[NT];
    for (int t = 0; t < NT; ++t) { target_int1[t] = target[t]; target_int1[t].w = int1_w[t]; }

    float lik[NT][R], kl[NT][R], clamp[NT][R];
    for (int t = 0; t < NT; ++t)
        for (int s = 0; s < R; ++s) {
            lik[t][s] = likelihood<D>(target_int1[t], initial_int1[s]);
            kl[t][s] = sign_of(initial_int1[s].w) == sign_of(target_int1[t].w) ? kl_divergence<D>(target_int1[t], initial_int1[s]) : 0.f;
            clamp[t][s] = kl[t][s] < kKlThreshold ? 1.f : 0.f;
        }
    for (int t = 0; t < NT; ++t) {
        int best = -1;
        float smallest = std::numeric_limits<float>::infinity();
        for (int s = 0; s < R; ++s)
            if (kl[t][s] < smallest) { smallest = kl[t][s]; best = s; }
        if (best >= 0) clamp[t][best] = 1.f;
    }

    float r2[NT][R];
    for (int t = 0; t < NT; ++t) {
        float wl[R], sum = 0;
        for (int s = 0; s < R; ++s) {
            wl[s] = clip(initial_int1[s].w * lik[t][s]) * clamp[t][s];
            sum += wl[s];
        }
        for (int s = 0; s < R; ++s) r2[t][s] = (wl[s] / sum) * int1_w[t];
    }
    float fw[R];
    for (int s = 0; s < R; ++s) fw[s] = 0;
    for (int t = 0; t < NT; ++t)
        for (int s = 0; s < R; ++s) fw[s] += r2[t][s];

    for (int s = 0; s < R; ++s) {
        const float cfw = clip(fw[s]);
        float r3[NT];
        for (int t = 0; t < NT; ++t) r3[t] = r2[t][s] / cfw;
        Gaussian<D>& out = result[s];
        for (int d = 0; d < D; ++d) {
            float acc = 0;
            for (int t = 0; t < NT; ++t) acc += r3[t] * target[t].p[d];
            out.p[d] = acc;
        }
        for (int i = 0; i < D; ++i)
            for (int j = 0; j < D; ++j) {
                float acc = 0;
                for (int t = 0; t < NT; ++t) {
                    const float di = target[t].p[i] - out.p[i], dj = target[t].p[j] - out.p[j];
                    acc += r3[t] * (di * dj + target[t].c[i * D + j]);
                }
                out.c[i * D + j] = acc;
            }
        if (fw[s] < kEpsLarge)
            for (int i = 0; i < D * D; ++i) out.c[i] = (i / D == i % D) ? 1.f : 0.f;
        out.w = fw[s] * target_clipped_integral;
    }
}

template <int D, int R>
void fit_one(const float* mixture, int G, const uint16_t* nodes, int K, float* out, float* node_gaussians,
             int32_t* node_counts, float* node_integrals, uint8_t* node_initial) {
    constexpr int RF = 1 + D + D * D;
    const int n_internal = G - 1, n_nodes = 2 * G - 1;
    std::vector<Gaussian<D>> attr((size_t)n_nodes * R);
    std::vector<int> count(n_nodes, 0);
    std::vector<float> integral(n_nodes, 0.f);
    std::vector<uint8_t> initial((size_t)n_nodes * R, 255);
    std::vector<int> pending(n_internal, 0);

    auto process_internal = [&](int id) {
        const int l = nodes[(size_t)id * 4 + 1], r = nodes[(size_t)id * 4 + 2];
        integral[id] = integral[l] + integral[r];
        Gaussian<D> child[2 * R];
        int n = 0;
        for (int c : {l, r})
            for (int i = 0; i < count[c]; ++i)
                if (std::fabs(attr[(size_t)c * R + i].w) >= kEpsLarge) child[n++] = attr[(size_t)c * R + i];
        if (n > R) {
            fit_em<D, R>(child, n, &attr[(size_t)id * R], &initial[(size_t)id * R]);
            count[id] = R;
        } else {
            for (int i = 0; i < n; ++i) attr[(size_t)id * R + i] = child[i];
            count[id] = n;
        }
    };
    // bottom-up: a node is processed when its second child arrives (iterate_over_nodes :325-393)
    for (int leaf = 0; leaf < G; ++leaf) {
        int id = n_internal + leaf;
        const int obj = nodes[(size_t)id * 4 + 3];
        Gaussian<D> g;
        std::memcpy(&g, mixture + (size_t)obj * RF, sizeof(g));
        attr[(size_t)id * R] = g;
        count[id] = 1;
        integral[id] = g.w;
        int parent = nodes[(size_t)id * 4 + 0];
        while (parent != 0xFFFF) {
            if (++pending[parent] < 2) break;
            process_internal(parent);
            parent = nodes[(size_t)parent * 4 + 0];
        }
    }

    // collect_result (:395-484)
    std::vector<int> selected;
    std::vector<float> rating;
    auto compute_rating = [&](int id) -> float { return count[id] < R ? -2.f : std::fabs(integral[id]); };
    selected.push_back(0);
    rating.push_back(compute_rating(0));
    int n_selected = count[0];
    while (n_selected < K - R) {
        float best_rating = -1;
        int best = -1;
        for (size_t i = 0; i < selected.size(); ++i)
            if (rating[i] > best_rating) { best_rating = rating[i]; best = int(i); }
        if (best < 0) break;
        const int id = selected[best];
        const int l = nodes[(size_t)id * 4 + 1], r = nodes[(size_t)id * 4 + 2];
        selected[best] = l;
        rating[best] = compute_rating(l);
        selected.push_back(r);
        rating.push_back(compute_rating(r));
        n_selected = n_selected - R + count[l] + count[r];
    }
    int write = 0;
    for (int id : selected)
        for (int j = 0; j < count[id]; ++j) std::memcpy(out + (size_t)(write++) * RF, &attr[(size_t)id * R + j], sizeof(Gaussian<D>));
    const Gaussian<D> pad = zero_identity<D>();
    for (int i = write; i < K; ++i) std::memcpy(out + (size_t)i * RF, &pad, sizeof(pad));

    if (node_gaussians) {
        std::memset(node_gaussians, 0, sizeof(float) * (size_t)n_nodes * R * RF);
        for (int id = 0; id < n_nodes; ++id)
            for (int j = 0; j < count[id]; ++j)
                std::memcpy(node_gaussians + ((size_t)id * R + j) * RF, &attr[(size_t)id * R + j], sizeof(Gaussian<D>));
    }
    if (node_counts) for (int id = 0; id < n_nodes; ++id) node_counts[id] = count[id];
    if (node_integrals) for (int id = 0; id < n_nodes; ++id) node_integrals[id] = integral[id];
    if (node_initial) std::memcpy(node_initial, initial.data(), (size_t)n_nodes * R);
}

}  // namespace

extern "C" {

// mixture [n_mixtures, G, RF] (covariance form), nodes [n_mixtures, 2G-1, 4] uint16 from the LBVH build,
// out [n_mixtures, K, RF]. Optional per-node dumps (may be NULL): node_gaussians [n_mixtures, 2G-1, R, RF],
// node_counts [n_mixtures, 2G-1] int32, node_integrals [n_mixtures, 2G-1], node_initial [n_mixtures, 2G-1, R] uint8.
int oracle_mhem_fit_forward(const float* mixture, int n_mixtures, int G, int D, const uint16_t* nodes, int K, int R,
                            float* out, float* node_gaussians, int32_t* node_counts, float* node_integrals,
                            uint8_t* node_initial) {
    if (!((D == 2 || D == 3) && (R == 2 || R == 4))) return 1;
    const int RF = 1 + D + D * D;
    const size_t n_nodes = 2 * (size_t)G - 1;
#pragma omp parallel for schedule(dynamic)
    for (int m = 0; m < n_mixtures; ++m) {
        const float* mix = mixture + (size_t)m * G * RF;
        const uint16_t* nd = nodes + (size_t)m * n_nodes * 4;
        float* o = out + (size_t)m * K * RF;
        float* ng = node_gaussians ? node_gaussians + (size_t)m * n_nodes * R * RF : nullptr;
        int32_t* nc = node_counts ? node_counts + (size_t)m * n_nodes : nullptr;
        float* ni = node_integrals ? node_integrals + (size_t)m * n_nodes : nullptr;
        uint8_t* nn = node_initial ? node_initial + (size_t)m * n_nodes * R : nullptr;
        if (D == 2 && R == 2) fit_one<2, 2>(mix, G, nd, K, o, ng, nc, ni, nn);
        else if (D == 2 && R == 4) fit_one<2, 4>(mix, G, nd, K, o, ng, nc, ni, nn);
        else if (D == 3 && R == 2) fit_one<3, 2>(mix, G, nd, K, o, ng, nc, ni, nn);
        else fit_one<3, 4>(mix, G, nd, K, o, ng, nc, ni, nn);
    }
    return 0;
}

}  // extern "C"
