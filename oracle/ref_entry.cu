// TEST INFRASTRUCTURE: C entry points around the REFERENCE's own native sources (CPU path), built into
// oracle/_ref/libgmc_ref_fit.so and libgmc_ref_convfit.so by oracle/build_ref.py.  The reference sources are compiled where they lie (they are not
// copied); this file only converts between raw host pointers and the torch::Tensor arguments the reference functions
// take.  Used to pin oracle/cpu/* (and through it the CUDA kernels) to the reference itself, and as the timed CPU
// baseline.  One source, several translation units: the build compiles it once per REF_PART_* macro because the
// reference headers hold their template bodies and each part is slow to compile.
//
// Everything runs on CPU tensors, i.e. through gpe::start_parallel's OpenMP branch
// (src/gmc/cpp/extensions/parallel_start.h:92-111).
#include <cstdint>
#include <cstring>
#include <exception>
#include <string>

#include <omp.h>
#include <torch/types.h>

std::string& gmc_ref_error_slot();  // defined in the REF_PART_COMMON unit
bool& gmc_ref_serial_flag();        // defined in the REF_PART_COMMON unit

namespace {
// Serial mode: the reference's CPU launcher opens an OpenMP team of as many threads as a CUDA block has
// (parallel_start.h:92-111). Called from inside an active parallel region of our own, with nested parallelism off, that
// team has one thread and the "CUDA threads" run one after the other: race-free and reproducible. Needed because the
// reference's convolution_fitting mass pass adds a node's mass and its count with two independent atomics
// (convolution_fitting/Tree.cu:289-294), and the interleaving changes the masses, hence the selected subtrees.
// Not usable for code that waits on a CPU barrier across its threads (bvh_mhem_fit backward, ParallelStack.h:20).
template <typename Fn> int guarded(Fn&& fn) {
    try {
        if (gmc_ref_serial_flag()) {
            std::exception_ptr err;
            omp_set_max_active_levels(1);
#pragma omp parallel num_threads(2)
            {
                if (omp_get_thread_num() == 0) {
                    try {
                        fn();
                    } catch (...) {
                        err = std::current_exception();
                    }
                }
            }
            if (err) std::rethrow_exception(err);
        } else {
            fn();
        }
        return 0;
    } catch (const std::exception& e) {
        gmc_ref_error_slot() = e.what();
        return 1;
    }
}

template <typename T> torch::Tensor wrap(const T* p, std::initializer_list<int64_t> shape, torch::ScalarType dtype) {
    return torch::from_blob(const_cast<T*>(p), torch::IntArrayRef(shape), torch::TensorOptions().dtype(dtype)).clone();
}

template <typename T> void copy_out(const torch::Tensor& t, T* dst) {
    if (dst == nullptr) return;
    const auto c = t.contiguous();
    std::memcpy(dst, c.data_ptr(), size_t(c.numel()) * size_t(c.element_size()));
}
inline int64_t vlen(int D) { return 1 + D + D * D; }
}  // namespace

#if defined(REF_PART_COMMON)
std::string& gmc_ref_error_slot() {
    static thread_local std::string slot;
    return slot;
}
bool& gmc_ref_serial_flag() {
    static bool serial = false;
    return serial;
}
extern "C" const char* gmc_ref_last_error() { return gmc_ref_error_slot().c_str(); }
// 1: run the reference's CPU "threads" one after the other (see guarded()); 0: as the reference runs them.
extern "C" void gmc_ref_set_serial(int serial) { gmc_ref_serial_flag() = serial != 0; }
#endif

// ---------------------------------------------------------------------------------------------------------------
#if defined(REF_PART_LBVH)
#include "lbvh/bvh.h"
#include "lbvh/morton_code.h"

namespace {
template <int D>
void lbvh_build(const float* mixture, int B, int L, int G, int algorithm, int make_aabbs, float aabb_threshold,
                int64_t* sorted_keys, int16_t* nodes, float* aabbs) {
    using Bvh = lbvh::Bvh<D, float>;
    const auto m = wrap(mixture, {B, L, G, vlen(D)}, torch::kFloat);
    lbvh::Config config;
    config.morton_code_algorithm = static_cast<lbvh::Config::MortonCodeAlgorithm>(algorithm);
    config.make_aabbs = make_aabbs != 0;
    config.aabb_threshold = aabb_threshold;
    const Bvh bvh(m, config);  // lbvh/bvh.h:122-129 -> construct() (lbvh/bvh.cu:23-144)
    copy_out(bvh.m_nodes, nodes);
    if (make_aabbs) copy_out(bvh.m_aabbs, aabbs);
    if (sorted_keys != nullptr) {
        // construct() keeps the keys private; the same two public steps it runs give them (lbvh/bvh.cu:70-116).
        Bvh shell(m, torch::Tensor(), torch::Tensor());
        const auto whole = gpe::aabb_from_positions(gpe::positions(m));
        torch::Tensor codes;
        switch (algorithm) {
            case 0: codes = shell.template compute_morton_codes<0>(whole); break;
            case 1: codes = shell.template compute_morton_codes<1>(whole); break;
            case 2: codes = shell.template compute_morton_codes<2>(whole); break;
            case 3: codes = shell.template compute_morton_codes<3>(whole); break;
            default: codes = shell.template compute_morton_codes<4>(whole); break;
        }
        if (make_aabbs) {
            const auto object_aabbs = shell.compute_aabbs();
            codes = std::get<0>(shell.sort_morton_codes(codes, object_aabbs));
        } else {
            codes = lbvh::sort_morton_codes<typename Bvh::morton_cuda_t, typename Bvh::morton_torch_t>(codes);
        }
        copy_out(codes, sorted_keys);
    }
}
}  // namespace

// mixture [B, L, G, 1+D+D*D] fp32 -> sorted keys int64 [B*L, G] (nullable), nodes int16 [B, L, 2G-1, 4],
// aabbs fp32 [B, L, 2G-1, 8] (only written with make_aabbs).  With make_aabbs the mixture must hold INVERSE
// covariances (lbvh/bvh.cu:204 inverts them again).
extern "C" int gmc_ref_lbvh_build(const float* mixture, int B, int L, int G, int D, int algorithm, int make_aabbs,
                                  float aabb_threshold, int64_t* sorted_keys, int16_t* nodes, float* aabbs) {
    return guarded([&] {
        if (D == 2)
            lbvh_build<2>(mixture, B, L, G, algorithm, make_aabbs, aabb_threshold, sorted_keys, nodes, aabbs);
        else
            lbvh_build<3>(mixture, B, L, G, algorithm, make_aabbs, aabb_threshold, sorted_keys, nodes, aabbs);
    });
}
#endif

// ---------------------------------------------------------------------------------------------------------------
#if defined(REF_PART_MHEM_FWD) || defined(REF_PART_MHEM_BWD)
#include "bvh_mhem_fit/implementation_forward.h"
#if defined(REF_PART_MHEM_BWD)
#include "bvh_mhem_fit/implementation_backward.h"
#endif

namespace {
template <int R, int D>
bvh_mhem_fit::ForwardOutput mhem_forward(const float* mixture, int B, int L, int G, int K, float kl_threshold) {
    bvh_mhem_fit::Config config;
    config.reduction_n = R;
    config.n_components_fitting = unsigned(K);
    config.em_kl_div_threshold = kl_threshold;
    const auto m = wrap(mixture, {B, L, G, vlen(D)}, torch::kFloat);
    return bvh_mhem_fit::forward_impl_t<R, float, D>(m, config);  // bvh_mhem_fit/implementation_forward.h:490-560
}

#if defined(REF_PART_MHEM_FWD)
template <int R, int D>
void mhem_forward_dump(const float* mixture, int B, int L, int G, int K, float kl_threshold, float* fitting,
                       int16_t* nodes, float* node_gaussians, int32_t* node_counts, float* node_integrals,
                       uint8_t* node_initial, int32_t* node_child_leaves) {
    using Attr = typename bvh_mhem_fit::AugmentedBvh<float, D, R>::NodeAttributes;
    const auto out = mhem_forward<R, D>(mixture, B, L, G, K, kl_threshold);
    copy_out(out.fitting, fitting);
    copy_out(out.bvh_nodes, nodes);
    if (node_gaussians == nullptr) return;
    const int64_t n_nodes = 2 * int64_t(G) - 1, n_mix = int64_t(B) * L, V = vlen(D);
    const auto attrs = out.bvh_attributes.contiguous();
    const auto* a = reinterpret_cast<const Attr*>(attrs.data_ptr());
    for (int64_t i = 0; i < n_mix * n_nodes; ++i) {
        const Attr& at = a[i];
        const unsigned count = unsigned(at.gaussians.size());
        node_counts[i] = int32_t(count);
        node_integrals[i] = at.gm_integral;
        node_child_leaves[i] = int32_t(at.n_child_leaves);
        for (int r = 0; r < R; ++r) {
            node_initial[i * R + r] = at.gradient_cache_data.initial_indices[r];
            float* dst = node_gaussians + (i * R + r) * V;
            if (unsigned(r) < count)
                std::memcpy(dst, &at.gaussians[r], size_t(V) * sizeof(float));
            else
                std::memset(dst, 0, size_t(V) * sizeof(float));
        }
    }
}
#endif
}  // namespace

#if defined(REF_PART_MHEM_FWD)
// mixture [B, L, G, V] fp32 (covariance form) -> fitting [B, L, K, V], nodes int16 [B, L, 2G-1, 4] and, when
// node_gaussians != NULL, the per-node state of the bottom-up pass: node_gaussians [B*L, 2G-1, R, V] (zeros beyond
// the node's count), node_counts, node_integrals, node_child_leaves [B*L, 2G-1], node_initial uint8 [B*L, 2G-1, R].
extern "C" int gmc_ref_mhem_fit_forward(const float* mixture, int B, int L, int G, int D, int K, int R,
                                        float kl_threshold, float* fitting, int16_t* nodes, float* node_gaussians,
                                        int32_t* node_counts, float* node_integrals, uint8_t* node_initial,
                                        int32_t* node_child_leaves) {
    return guarded([&] {
#define GMC_REF_CALL(RR, DD)                                                                                           \
    mhem_forward_dump<RR, DD>(mixture, B, L, G, K, kl_threshold, fitting, nodes, node_gaussians, node_counts,         \
                              node_integrals, node_initial, node_child_leaves)
        if (R == 2 && D == 2) GMC_REF_CALL(2, 2);
        else if (R == 2 && D == 3) GMC_REF_CALL(2, 3);
        else if (R == 4 && D == 2) GMC_REF_CALL(4, 2);
        else if (R == 4 && D == 3) GMC_REF_CALL(4, 3);
        else throw std::runtime_error("unsupported R / D");
#undef GMC_REF_CALL
    });
}
#endif

#if defined(REF_PART_MHEM_BWD)
namespace {
template <int R, int D>
void mhem_backward(const float* grad, const float* mixture, int B, int L, int G, int K, float kl_threshold,
                   float* grad_target) {
    bvh_mhem_fit::Config config;
    config.reduction_n = R;
    config.n_components_fitting = unsigned(K);
    config.em_kl_div_threshold = kl_threshold;
    auto forward_out = mhem_forward<R, D>(mixture, B, L, G, K, kl_threshold);
    const auto g = wrap(grad, {B, L, K, vlen(D)}, torch::kFloat);
    // bvh_mhem_fit/implementation_backward.h:525-594 (overwrites forward_out.bvh_attributes, which is ours)
    const auto gt = bvh_mhem_fit::backward_impl_t<R, float, D>(g, forward_out, config);
    copy_out(gt, grad_target);
}
}  // namespace

// Runs the reference forward, then its backward on the result: grad [B, L, K, V] -> grad_target [B, L, G, V].
extern "C" int gmc_ref_mhem_fit_backward(const float* grad, const float* mixture, int B, int L, int G, int D, int K,
                                         int R, float kl_threshold, float* grad_target) {
    return guarded([&] {
        if (R == 2 && D == 2) mhem_backward<2, 2>(grad, mixture, B, L, G, K, kl_threshold, grad_target);
        else if (R == 2 && D == 3) mhem_backward<2, 3>(grad, mixture, B, L, G, K, kl_threshold, grad_target);
        else if (R == 4 && D == 2) mhem_backward<4, 2>(grad, mixture, B, L, G, K, kl_threshold, grad_target);
        else if (R == 4 && D == 3) mhem_backward<4, 3>(grad, mixture, B, L, G, K, kl_threshold, grad_target);
        else throw std::runtime_error("unsupported R / D");
    });
}
#endif
#endif

// ---------------------------------------------------------------------------------------------------------------
#if defined(REF_PART_CONVFIT_FWD) || defined(REF_PART_CONVFIT_BWD)
#include "convolution_fitting/implementation_forward.h"
#if defined(REF_PART_CONVFIT_BWD)
#include "convolution_fitting/implementation_backward.h"
#endif

namespace {
#if defined(REF_PART_CONVFIT_FWD)
template <int D>
void convfit_forward(const float* data, const float* kernels, int B, int Cin, int G, int Cout, int Gk, int K,
                     float* fitting, float* cached_pos_covs, int32_t* nodesobjs, int32_t* fitting_subtrees,
                     int32_t* nodes, float* node_mass, int32_t* node_count, int64_t* sorted_keys) {
    using Tree = convolution_fitting::Tree<float, unsigned(D)>;
    const auto d = wrap(data, {B, Cin, G, vlen(D)}, torch::kFloat);
    const auto k = wrap(kernels, {Cout, Cin, Gk, vlen(D)}, torch::kFloat);
    convolution_fitting::Config config;
    config.n_components_fitting = unsigned(K);
    // the four steps of forward_impl_t (convolution_fitting/implementation_forward.h:126-137), spelled out so that the
    // intermediate tree can be read
    typename Tree::Data storage;
    Tree tree(d, k, &storage, config);
    tree.create_tree_nodes();
    tree.create_attributes();
    tree.select_fitting_subtrees();
    const auto out = convolution_fitting::forward_with_given_tree(config, tree);
    copy_out(out.fitting, fitting);
    copy_out(out.cached_pos_covs, cached_pos_covs);
    copy_out(out.nodesobjs, nodesobjs);
    copy_out(out.fitting_subtrees, fitting_subtrees);
    copy_out(storage.nodes, nodes);
    if (node_mass != nullptr) {
        const auto attrs = storage.node_attributes.contiguous();
        const auto* a = reinterpret_cast<const typename Tree::NodeAttributes*>(attrs.data_ptr());
        const int64_t n = int64_t(B) * Cout * (int64_t(Cin) * G * Gk - 1);
        for (int64_t i = 0; i < n; ++i) {
            node_mass[i] = a[i].mass;
            node_count[i] = int32_t(a[i].n_gaussians);
        }
    }
    if (sorted_keys != nullptr) copy_out(tree.compute_morton_codes(), sorted_keys);
}
#endif
}  // namespace

#if defined(REF_PART_CONVFIT_FWD)
// data [B, Cin, G, V], kernels [Cout, Cin, Gk, V] -> fitting [B, Cout, K, V], cached_pos_covs [B, Cout, K, D*D],
// nodesobjs int32 [B, Cout, T], fitting_subtrees int32 [B, Cout, 2K]; optional tree read-outs: nodes int32
// [B, Cout, 2T-1, 3], node_mass / node_count [B, Cout, T-1], sorted_keys int64 [B, Cout, T].
extern "C" int gmc_ref_convolution_fitting_forward(const float* data, const float* kernels, int B, int Cin, int G,
                                                   int Cout, int Gk, int D, int K, float* fitting,
                                                   float* cached_pos_covs, int32_t* nodesobjs,
                                                   int32_t* fitting_subtrees, int32_t* nodes, float* node_mass,
                                                   int32_t* node_count, int64_t* sorted_keys) {
    return guarded([&] {
        if (D == 2)
            convfit_forward<2>(data, kernels, B, Cin, G, Cout, Gk, K, fitting, cached_pos_covs, nodesobjs,
                               fitting_subtrees, nodes, node_mass, node_count, sorted_keys);
        else
            convfit_forward<3>(data, kernels, B, Cin, G, Cout, Gk, K, fitting, cached_pos_covs, nodesobjs,
                               fitting_subtrees, nodes, node_mass, node_count, sorted_keys);
    });
}
#endif

#if defined(REF_PART_CONVFIT_BWD)
namespace {
template <int D>
void convfit_backward(const float* grad, const float* data, const float* kernels, int B, int Cin, int G, int Cout,
                      int Gk, int K, float* grad_data, float* grad_kernels) {
    const auto d = wrap(data, {B, Cin, G, vlen(D)}, torch::kFloat);
    const auto k = wrap(kernels, {Cout, Cin, Gk, vlen(D)}, torch::kFloat);
    const auto g = wrap(grad, {B, Cout, K, vlen(D)}, torch::kFloat);
    convolution_fitting::Config config;
    config.n_components_fitting = unsigned(K);
    const auto forward_out = convolution_fitting::forward_impl_t<4, float, unsigned(D)>(d, k, config);
    // convolution_fitting/implementation_backward.h:22-159
    const auto grads = convolution_fitting::backward_impl_t<4, float, unsigned(D)>(g, d, k, forward_out, config);
    copy_out(grads.first, grad_data);
    copy_out(grads.second, grad_kernels);
}
}  // namespace

// Runs the reference forward, then its backward: grad [B, Cout, K, V] -> grad_data [B, Cin, G, V],
// grad_kernels [Cout, Cin, Gk, V].
extern "C" int gmc_ref_convolution_fitting_backward(const float* grad, const float* data, const float* kernels, int B,
                                                    int Cin, int G, int Cout, int Gk, int D, int K, float* grad_data,
                                                    float* grad_kernels) {
    return guarded([&] {
        if (D == 2) convfit_backward<2>(grad, data, kernels, B, Cin, G, Cout, Gk, K, grad_data, grad_kernels);
        else convfit_backward<3>(grad, data, kernels, B, Cin, G, Cout, Gk, K, grad_data, grad_kernels);
    });
}
#endif
#endif

// ---------------------------------------------------------------------------------------------------------------
#if defined(REF_PART_EVAL)
#include "evaluate_inversed/implementations.h"

// The reference's CPU evaluation (evaluate_inversed/parallel_implementation.cu:23-195): the path its Python wrapper
// takes for CPU tensors (evaluate_inversed/evaluate_inversed.cpp:11-35).  xes [Bx, Lx, N, D] with Bx in {1, B}.
extern "C" int gmc_ref_eval_forward(const float* mixture, const float* xes, float* out, int B, int L, int G, int D,
                                    int Bx, int Lx, int N) {
    return guarded([&] {
        const auto m = wrap(mixture, {B, L, G, vlen(D)}, torch::kFloat);
        const auto x = wrap(xes, {Bx, Lx, N, D}, torch::kFloat);
        copy_out(parallel_forward_impl(m, x), out);
    });
}

extern "C" int gmc_ref_eval_backward(const float* grad_out, const float* mixture, const float* xes,
                                     float* grad_mixture, float* grad_xes, int B, int L, int G, int D, int Bx, int Lx,
                                     int N) {
    return guarded([&] {
        const auto m = wrap(mixture, {B, L, G, vlen(D)}, torch::kFloat);
        const auto x = wrap(xes, {Bx, Lx, N, D}, torch::kFloat);
        const auto g = wrap(grad_out, {B, L, N}, torch::kFloat);
        const auto grads = parallel_backward_impl(g, m, x, grad_mixture != nullptr, grad_xes != nullptr);
        if (grad_mixture != nullptr) copy_out(std::get<0>(grads), grad_mixture);
        if (grad_xes != nullptr) copy_out(std::get<1>(grads), grad_xes);
    });
}

// Same entry points in fp64 (the reference dispatches float and double: parallel_implementation.cu:75).
extern "C" int gmc_ref_eval_forward_f64(const double* mixture, const double* xes, double* out, int B, int L, int G,
                                        int D, int Bx, int Lx, int N) {
    return guarded([&] {
        const auto m = wrap(mixture, {B, L, G, vlen(D)}, torch::kDouble);
        const auto x = wrap(xes, {Bx, Lx, N, D}, torch::kDouble);
        copy_out(parallel_forward_impl(m, x), out);
    });
}
#endif
