/*
 * gmc_b200.h -- C ABI of the B200 (sm_100a) Gaussian-mixture operator library.
 *
 * Every entry point takes plain pointers, sizes and a CUDA stream (passed as void*, nullptr = the
 * legacy default stream) and returns an int status (GMC_OK == 0). There is no CPU code path: a
 * call on a machine without a CUDA device returns GMC_ERR_CUDA.
 *
 * Allocation, state and synchronisation, exactly:
 *  - The device-pointer entry points (everything except the three named below) allocate nothing and keep
 *    no state: outputs and scratch are owned by the caller, all kernels are enqueued on the given stream
 *    and the call returns without synchronising. They may set function attributes (dynamic shared memory
 *    size) on first use and can be captured in a CUDA graph.
 *  - gmc_eval_inversed_host (HOST buffers) owns per-device state: four device slots (cudaMalloc on first
 *    use, re-allocated when a larger problem arrives), six streams and twelve events, kept until
 *    gmc_host_pipeline_release(). It blocks until the host outputs are complete; one mutex serialises the
 *    calls of a process.
 *  - gmc_device_check_word synchronises the whole device, gmc_sync_and_check the given stream; both read
 *    and clear a per-device __device__ word that kernels set instead of hanging or trapping.
 *  - gmc_mhem_fit_forward_noalloc uses an 8 MiB __device__ array inside the library as its scratch.
 *
 * Data layout (identical to the reference's packed mixtures, src/gmc/mixture.py:37-67 and
 * src/gmc/cpp/extensions/util/gaussian.h:14-46): a mixture is a contiguous fp32 array
 * [n_batch, n_layers, n_components, 1 + D + D*D] = [weight | position(D) | matrix(DxD, row major)],
 * D in {2, 3}. "layers" are feature channels.
 *
 * The reference binds each operator through pybind11 functions that take torch::Tensor; the
 * comment above each declaration names the reference function it replaces.
 */
#ifndef GMC_B200_H
#define GMC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum gmc_status {
    GMC_OK = 0,
    GMC_ERR_BAD_DIMS = 1,        /* D not in {2,3} or a size is <= 0 / exceeds a documented limit     */
    GMC_ERR_BAD_BROADCAST = 2,   /* xes batch/layer extent is neither 1 nor the mixture's             */
    GMC_ERR_NULL_POINTER = 3,    /* a required pointer is NULL                                        */
    GMC_ERR_UNSUPPORTED = 4,     /* e.g. reduction_n not in {2,4}                                     */
    GMC_ERR_CUDA = 6,            /* a CUDA runtime call failed (see gmc_last_cuda_error)              */
    GMC_ERR_DEVICE_CHECK = 7,    /* a kernel-side bounded wait or self check gave up                  */
    GMC_ERR_BUILTIN_SCRATCH = 9  /* problem larger than the built-in scratch of a *_noalloc entry point */
};

/* Human-readable text for a status code (static storage, never NULL). */
const char* gmc_status_string(int status);
/* cudaGetErrorString of the last CUDA error this library saw on the calling thread ("" if none). */
const char* gmc_last_cuda_error(void);
/* Library version, "major.minor". */
const char* gmc_version(void);
/* Reads and clears the device-side check word of the current device (synchronises the WHOLE device).
 * 0 = no kernel reported a problem since the last call. Bit 1: a bounded wait for a bulk copy ran out (the kernel
 * wrote NaN to the outputs it could not compute); bit 4: an index check of a bounds-checked build failed. */
int gmc_device_check_word(int* word_out);
/* Waits for `stream` and returns GMC_ERR_DEVICE_CHECK if any kernel of this library reported a problem since the last
 * check (the word is cleared), GMC_OK otherwise. Call it wherever the host synchronises anyway: device-side give-ups
 * never hang and never abort, this is how they become visible. Not for use during stream capture. */
int gmc_sync_and_check(void* stream);
/* Test aid of the bounds-checked build (libgmc_b200_checked.so, compiled with -DGMC_BOUNDS_CHECK: every index that a
 * kernel reads from data -- tree children, object ids, sorted product indices -- is range-checked; a bad one sets bit 4
 * of the check word and is replaced by 0, so the access stays inside its array). Runs the check itself once on a
 * one-float buffer: index >= n must set the word and read element 0. Regular builds return GMC_ERR_UNSUPPORTED. */
int gmc_debug_index_check(const float* one_float, float* out, long long index, long long n, void* stream);
/* Error-path test aid: the forward evaluation with its bulk copy deliberately left out, so that the bounded wait runs
 * out after about a thousand polls: every output becomes NaN and the check word gets bit 1. Nothing is in flight when
 * the kernel gives up; the context stays usable. No reference counterpart. */
int gmc_debug_eval_forward_lost_copy(const float* mixture, const float* xes, float* out, int n_batch, int n_layers,
                                     int n_components, int n_dims, int n_batch_xes, int n_layers_xes, int n_xes,
                                     void* stream);

/* ------------------------------------------------------------------------------------------------
 * Mixture evaluation with the matrix slot holding the INVERSE covariance S:
 *   out[b,l,n] = sum_g w * (2 pi)^(-D/2) * sqrt(det S_g) * exp(-1/2 (x - mu_g)^T S_g (x - mu_g))
 * xes is [n_batch_xes, n_layers_xes, n_xes, D] with n_batch_xes in {1, n_batch} and n_layers_xes in
 * {1, n_layers} (broadcast). out is [n_batch, n_layers, n_xes] and is fully overwritten.
 *
 * Replaces evaluate_inversed::parallel_forward
 *   (src/gmc/cpp/extensions/evaluate_inversed/evaluate_inversed.cpp:11-20,
 *    parallel_implementation_optimised_forward.cu:59-98; math util/gaussian.h:82-95).
 * ---------------------------------------------------------------------------------------------- */
int gmc_eval_inversed_forward(const float* mixture, const float* xes, float* out,
                              int n_batch, int n_layers, int n_components, int n_dims,
                              int n_batch_xes, int n_layers_xes, int n_xes, void* stream);

/* Gradients of the evaluation above for an incoming grad_out [n_batch, n_layers, n_xes].
 * grad_mixture ([n_batch, n_layers, n_components, 1+D+D*D], full DxD matrix gradient) and grad_xes
 * (same shape as xes; summed over the broadcast axes) may each be NULL, which skips that gradient.
 * Non-NULL outputs are fully overwritten (the library zeroes them before accumulating).
 *
 * Replaces evaluate_inversed::parallel_backward
 *   (evaluate_inversed.cpp:22-34, parallel_implementation_optimised_backward.cu:111-169;
 *    math util/grad/gaussian.h:19-66).
 * ---------------------------------------------------------------------------------------------- */
int gmc_eval_inversed_backward(const float* grad_out, const float* mixture, const float* xes,
                               float* grad_mixture, float* grad_xes,
                               int n_batch, int n_layers, int n_components, int n_dims,
                               int n_batch_xes, int n_layers_xes, int n_xes, void* stream);

/* The evaluation above (and, when grad_out is not NULL, its gradients) for tensors that live in HOST memory:
 * every pointer is a host pointer, the work is done on the current CUDA device. The batch is cut into n_slices equal
 * slices (0 = default plan: about eight slices with short ones at both ends) that move through a copy-in / kernels /
 * copy-out pipeline on internal streams, so with page-locked buffers the copies of both directions overlap the kernels. The call returns when the host outputs are
 * complete. out may be NULL when only gradients are wanted; grad_mixture / grad_xes may each be NULL. When xes is
 * shared by the whole batch (n_batch_xes == 1 < n_batch) the batch is processed as one slice.
 * The device workspace and the streams are created on first use and kept per device; gmc_host_pipeline_release()
 * frees those of the current device.
 *
 * Serves the callers that hand CPU tensors to evaluate_inversed::parallel_forward / parallel_backward, which the
 * reference sends to its host implementation (evaluate_inversed.cpp:19 and :34); here they run on the GPU.
 * ---------------------------------------------------------------------------------------------- */
int gmc_eval_inversed_host(const float* mixture, const float* xes, const float* grad_out, float* out,
                           float* grad_mixture, float* grad_xes, int n_batch, int n_layers, int n_components,
                           int n_dims, int n_batch_xes, int n_layers_xes, int n_xes, int n_slices);
int gmc_host_pipeline_release(void);

/* ------------------------------------------------------------------------------------------------
 * ReLU approximation of mixtures (covariance form, [n_mixtures, n_components, 1+D+D*D]) with per-mixture constants by
 * one fixed-point step, fused (inference path, no gradient):
 *   out_mixtures  = fixed_point_iteration_to_relu(mixture, constant, initial_approx_to_relu(mixture, constant))
 *   out_constants = max(constant, 0)
 *   out_initial   = initial_approx_to_relu(mixture, constant)          (may be NULL)
 * Replaces the chain of the reference's src/gmc/fitting.py:279-312 (initial_approx_to_relu,
 * fixed_point_iteration_to_relu with n_iter = 1: two mixture evaluations at the component centres, two covariance
 * inversions and the element-wise updates around them).
 * ---------------------------------------------------------------------------------------------- */
int gmc_relu_fixed_point(const float* mixtures, const float* constants, float* out_mixtures, float* out_constants,
                         float* out_initial, long long n_mixtures, int n_components, int n_dims, void* stream);
/* The same step with the two element-wise stages that surround it in a network layer folded in (evaluation mode):
 *   input weights are divided by weight_divisor first
 *       (src/gmc/model.py:189-190: a convolution's output is divided by its number of input channels);
 *   output centres are multiplied by f and output covariances by f * f, f = spatial_scale[mixture % n_channels]
 *       (src/gmc/modules.py:313-351, CovScaleNorm in evaluation mode: f = sqrt(D / averaged_cov_trace) per channel).
 * constants == NULL means all zero; spatial_scale == NULL means no scaling. weight_divisor must not be 0. */
int gmc_relu_fixed_point_layer(const float* mixtures, const float* constants, float* out_mixtures, float* out_constants,
                               float* out_initial, long long n_mixtures, int n_components, int n_dims,
                               float weight_divisor, const float* spatial_scale, int n_channels, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Batched inverse of n_matrices contiguous row-major DxD matrices (D in {2,3}); `inverses` holds the
 * mathematical inverse in the same layout. In-place (inverses == matrices) is allowed.
 *
 * Replaces matrix_inverse_cuda.forward (src/gmc/cpp/extensions/math/matrix_inverse_cuda.cu:18-63,
 * Python wrapper math/matrix_inverse.py:14-36) and pieces_bindings.matrix_inverse
 * (src/gmc/cpp/extensions/pieces/matrix_inverse.cu:23-73).
 * ---------------------------------------------------------------------------------------------- */
int gmc_matrix_inverse(const float* matrices, float* inverses, long long n_matrices, int n_dims, void* stream);
/* Gradient of the inverse for an incoming gradient of the same shape: grad_matrices = -inverse * grad * inverse per
 * matrix, with the inverses that gmc_matrix_inverse returned.
 * Replaces MatrixInverse.backward (src/gmc/cpp/extensions/math/matrix_inverse.py:31-33). */
int gmc_matrix_inverse_backward(const float* inverses, const float* grad, float* grad_matrices,
                                long long n_matrices, int n_dims, void* stream);

/* Eigen-decomposition of n_matrices symmetric row-major DxD matrices: eigenvalues [n, D] ascending, eigenvectors
 * [n, D, D] with the vectors in the columns. Closed form; accuracy about 1e-3 relative in fp32 for nearly degenerate
 * spectra (the reference states the same for its implementation).
 * Replaces pieces_bindings.symeig (src/gmc/cpp/extensions/pieces/symeig.cu, math/symeig_detail.h:17-138).
 * ---------------------------------------------------------------------------------------------- */
int gmc_symeig(const float* matrices, float* eigenvalues, float* eigenvectors, long long n_matrices, int n_dims,
               void* stream);

/* Integral of each mixture = sum of its weights (weights are integrals, not amplitudes).
 * mixture is [n_mixtures, n_components, 1+D+D*D], integrals is [n_mixtures].
 * Replaces gm.integrate (src/gmc/mixture.py:87-91), which the reference computes with a torch reduction.
 * ---------------------------------------------------------------------------------------------- */
int gmc_integrate(const float* mixture, float* integrals, long long n_mixtures, int n_components, int n_dims,
                  void* stream);

/* ------------------------------------------------------------------------------------------------
 * The scaling around the BVH-MHEM fit (src/gmc/fitting.py:342-358: the mixture is scaled per (batch, layer) so that the
 * mean trace of its covariances is D, fitted, and scaled back) as two small kernels instead of a chain of tensor ops.
 * gmc_trace_scale: per mixture scale = mean over components of trace(matrix) / D;
 *                  forth[m] = 1 / sqrt(scale), back[m] = sqrt(scale)                     (forth, back: [n_mixtures])
 * gmc_spatial_scale: out = (weight, position * f, matrix * f * f) with f = factors[m]     (gm.spatial_scale,
 *                  src/gmc/mixture.py:281-292, isotropic factor); out may be the input buffer.
 * ---------------------------------------------------------------------------------------------- */
int gmc_trace_scale(const float* mixture, float* forth, float* back, long long n_mixtures, int n_components,
                    int n_dims, void* stream);
int gmc_spatial_scale(const float* mixture, const float* factors, float* out, long long n_mixtures, int n_components,
                      int n_dims, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Per-sample normalisation of a one-channel input mixture [n_batch, 1, n_components, 1+D+D*D] (covariance form), the
 * two steps the network applies to its input in evaluation mode in one kernel: CovScaleNorm(batch_norm=False) followed
 * by BatchNorm(batch_norm=False) of the reference (src/gmc/modules.py:313-351, 354-420):
 *   f = sqrt(D / mean trace);  positions *= f, covariances *= f*f;
 *   the scaled mixture is evaluated at n_samples (>= 2) uniform points of the box of its centres (2D: widened by 15 %);
 *   weights *= scaling / max(sd, 0.001) (unbiased sd of the values; scaling = device pointer to the channel's learnable
 *   factor, NULL = 1), out_constants[b] = -mean.
 * The uniform numbers are `uniforms` [n_batch, n_samples, D] in [0, 1) if given (tests), else a counter-based hash of
 * *seed (device pointer to one int64 that the caller draws from its own generator).
 * n_components * (D + D*D + 1) + n_samples floats must fit in 200 KB of shared memory.
 * ---------------------------------------------------------------------------------------------- */
int gmc_input_normalise(const float* mixture, const long long* seed, const float* uniforms, const float* scaling,
                        long long n_batch, int n_components, int n_dims, int n_samples, float* out_mixture,
                        float* out_constants, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Linear BVH over the component means of each mixture (the tree of the BVH-MHEM fit).
 *   key      = (30-bit Morton code of the mean inside the mixture's own min/max box) << 16 | component id
 *   sorted_keys [n_mixtures, n_components] uint64, ascending per mixture
 *   nodes    [n_mixtures, 2*n_components-1, 4] uint16 {parent, left, right, object}: internal nodes first
 *            (root = 0, object = own id), leaves at n_components-1 .. in sorted order (object = component id);
 *            fields without a value hold 0xFFFF.
 * 2 <= n_components <= 32768 (node indices are 16 bit with 0xFFFF = none; the reference lets up to 65534 through, but
 * its uint16 node indices wrap beyond 32768). Up to 8192 components the tree is built in shared memory, above that in
 * global memory (the node buffer doubles as sort scratch before it is written). Integer results are bit-identical to an
 * IEEE fp32 evaluation of the reference formulas; a box axis with zero extent (always z in 2D) contributes Morton cell 0.
 *
 * Replaces lbvh::Bvh<D,float>::construct with make_aabbs=false
 * (src/gmc/cpp/extensions/lbvh/bvh.cu:23-144, 241-299, 373-458; lbvh/morton_code.h; lbvh/building.h).
 * ---------------------------------------------------------------------------------------------- */
int gmc_lbvh_build(const float* mixture, long long n_mixtures, int n_components, int n_dims,
                   uint64_t* sorted_keys, int16_t* nodes, void* stream);

/* The same build with the options of lbvh::Config (src/gmc/cpp/extensions/lbvh/Config.h).
 *   morton_code_algorithm  0 Old (gmc_lbvh_build), 1 Cov1_12p36pc16i, 2 Cov2_54pc10i, 3 Cov3_27p27c10i, 4 Cov4_27c27p10i:
 *                          key layouts that mix the 30-bit Morton code of the diagonal of the matrix slot (each axis
 *                          divided by its maximum over the mixture) into the key (lbvh/morton_code.h:170-252,
 *                          lbvh/bvh.cu:254-276). The object of a leaf is the low 16 bits of its key, as in the reference;
 *                          layouts 2..4 keep only 10 index bits there.
 *   make_aabbs != 0        also writes aabbs [n_mixtures, 2*n_components-1, 8] fp32 = {upper.x,y,z,0, lower.x,y,z,0}
 *                          (z = 0 in 2D): leaves = box of the ellipsoid where the component's density falls to
 *                          aabb_threshold (> 0), at least the 95 % ellipsoid; internal nodes = union of their children
 *                          (lbvh/bvh.cu:164-231, 460-510). The matrix slot must then hold INVERSE covariances
 *                          (lbvh/bvh.cu:204). Only with algorithms 0 and 1 (the leaf must name its component);
 *                          others return GMC_ERR_UNSUPPORTED. aabbs may be NULL when make_aabbs == 0.
 * Keys and nodes are bit-identical to the reference's; boxes agree to fp32 rounding of the closed-form
 * eigen-decomposition (math/symeig_detail.h). */
int gmc_lbvh_build_ex(const float* mixture, long long n_mixtures, int n_components, int n_dims,
                      int morton_code_algorithm, int make_aabbs, float aabb_threshold, uint64_t* sorted_keys,
                      int16_t* nodes, float* aabbs, void* stream);

/* ------------------------------------------------------------------------------------------------
 * BVH-MHEM reduction: fits n_components_fitting (K, a multiple of reduction_n) Gaussians to each covariance-form
 * mixture of n_components Gaussians (2 <= n_components <= 32768, reduction_n R in {2,4}).
 *   fitting        [n_mixtures, K, 1+D+D*D]            out; unused slots are (0, 0, identity)
 *   bvh_nodes      [n_mixtures, 2*n_components-1, 4]   out; as gmc_lbvh_build
 *   bvh_attributes [n_mixtures, gmc_mhem_fit_attribute_floats(...)] fp32, out; per internal node
 *                  [R Gaussians | integral | count | R initial indices (uint8) | reserved]; input of the backward
 *   scratch_keys   [n_mixtures, n_components] uint64   scratch (sorted Morton keys on return for n_components <= 8192;
 *                  larger mixtures reuse it for the fit's per-node bookkeeping, so its content is undefined then)
 * Weights are expected non-negative (the network applies the fit after the ReLU fixed-point step).
 *
 * Replaces bvh_mhem_fit_forward (src/gmc/cpp/extensions/bvh_mhem_fit/bindings.cpp:11-22,
 * implementation_forward.h:490-560).
 * ---------------------------------------------------------------------------------------------- */
size_t gmc_mhem_fit_attribute_floats(int n_components, int n_dims, int reduction_n);
int gmc_mhem_fit_forward(const float* mixture, long long n_mixtures, int n_components, int n_dims,
                         int n_components_fitting, int reduction_n, float* fitting, int16_t* bvh_nodes,
                         float* bvh_attributes, uint64_t* scratch_keys, void* stream);

/* Gradient of gmc_mhem_fit_forward with the tree, the node selection, the initial representatives and the KL gate
 * held fixed. grad is [n_mixtures, K, V]; mixture, bvh_nodes and bvh_attributes are the forward's input / outputs (not
 * modified); scratch_node_grad is [n_mixtures, (n_components-1) * reduction_n * V] floats of scratch, followed for
 * n_components > 8192 by 2 * n_components more floats per mixture (per-node bookkeeping that no longer fits in shared
 * memory); grad_mixture [n_mixtures, n_components, V] is fully overwritten.
 *
 * Replaces bvh_mhem_fit_backward (src/gmc/cpp/extensions/bvh_mhem_fit/bindings.cpp:24-40,
 * implementation_backward.h:41-594). Unlike the reference, the saved attributes are not overwritten, so the same
 * forward result can be differentiated more than once. */
int gmc_mhem_fit_backward(const float* grad, const float* mixture, long long n_mixtures, int n_components, int n_dims,
                          int n_components_fitting, int reduction_n, const int16_t* bvh_nodes,
                          const float* bvh_attributes, float* scratch_node_grad, float* grad_mixture, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Exact convolution of mixtures: data [n_batch, n_channels_in, n_components, V] (*) kernels
 * [n_channels_out, n_channels_in, n_kernel_components, V] -> out [n_batch, n_channels_out, T, V] with
 * T = n_channels_in * n_components * n_kernel_components; product t = comp_in + n_components * (ch_in +
 * n_channels_in * comp_k) is (w_d w_k, mu_d + mu_k, C_d + C_k).
 * Backward: grad [n_batch, n_channels_out, T, V] -> grad_data (like data) and grad_kernels (like kernels); either
 * may be NULL. Outputs are fully overwritten; no atomics, results are deterministic.
 *
 * Replaces convolution::forward_impl / backward_impl (src/gmc/cpp/extensions/convolution/bindings.cpp:10-27,
 * implementation_forward.h:27-103, implementation_backward.h:27-121).
 * ---------------------------------------------------------------------------------------------- */
int gmc_convolution_forward(const float* data, const float* kernels, float* out, int n_batch, int n_channels_in,
                            int n_components, int n_channels_out, int n_kernel_components, int n_dims, void* stream);
int gmc_convolution_backward(const float* grad, const float* data, const float* kernels, float* grad_data,
                             float* grad_kernels, int n_batch, int n_channels_in, int n_components,
                             int n_channels_out, int n_kernel_components, int n_dims, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Fused convolution + fit: the T product Gaussians of every (batch, output channel) are reduced to
 * n_components_fitting (K) Gaussians without being materialised (2 <= T <= 8192).
 *   fitting          [n_batch, n_channels_out, K, V]      out; unused slots are (0, 0, identity)
 *   cached_pos_covs  [n_batch, n_channels_out, K, D*D]    out; scatter of the product centres per output (backward)
 *   nodesobjs        [n_batch, n_channels_out, T] int32   out; product index of every leaf in sorted-key order
 *   fitting_subtrees [n_batch, n_channels_out, 2K] int32  out; [start, end) leaf-node ids (leaves are numbered from
 *                    T-1) of every output, -1 for unused slots
 *
 * Replaces convolution_fitting_forward (src/gmc/cpp/extensions/convolution_fitting/bindings.cpp:11-21,
 * Tree.cu:21-408, implementation_forward.h:19-137).
 * ---------------------------------------------------------------------------------------------- */
int gmc_convolution_fitting_forward(const float* data, const float* kernels, int n_batch, int n_channels_in,
                                    int n_components, int n_channels_out, int n_kernel_components, int n_dims,
                                    int n_components_fitting, float* fitting, float* cached_pos_covs,
                                    int32_t* nodesobjs, int32_t* fitting_subtrees, void* stream);
/* The same operator for trees of more than 8192 products (up to 65535; the reference indexes products with 32 bits,
 * src/gmc/cpp/extensions/convolution_fitting/Tree.cu:29-30): the tree is built in caller-provided global scratch instead
 * of shared memory (one CTA per tree; slower per product). scratch must be 16-byte aligned and hold
 * gmc_convolution_fitting_large_scratch_bytes(...) bytes (0 = sizes out of range); its content is undefined afterwards.
 * Results obey the same rules as gmc_convolution_fitting_forward, whose outputs it fills. */
size_t gmc_convolution_fitting_large_scratch_bytes(int n_batch, int n_channels_in, int n_components, int n_channels_out,
                                                   int n_kernel_components);
int gmc_convolution_fitting_forward_large(const float* data, const float* kernels, int n_batch, int n_channels_in,
                                          int n_components, int n_channels_out, int n_kernel_components, int n_dims,
                                          int n_components_fitting, float* fitting, float* cached_pos_covs,
                                          int32_t* nodesobjs, int32_t* fitting_subtrees, void* scratch,
                                          size_t scratch_bytes, void* stream);


/* Gradient of gmc_convolution_fitting_forward with the tree frozen. grad is [n_batch, n_channels_out, K, V]; fitting,
 * cached_pos_covs, nodesobjs and fitting_subtrees are the forward's outputs (not modified). grad_data (like data) and
 * grad_kernels (like kernels) may each be NULL; non-NULL outputs are fully overwritten.
 *
 * Replaces convolution_fitting_backward (src/gmc/cpp/extensions/convolution_fitting/bindings.cpp:23-35,
 * implementation_backward.h:22-159; util/grad/welford.h:14-97). */
int gmc_convolution_fitting_backward(const float* grad, const float* data, const float* kernels, int n_batch,
                                     int n_channels_in, int n_components, int n_channels_out, int n_kernel_components,
                                     int n_dims, int n_components_fitting, const float* fitting,
                                     const float* cached_pos_covs, const int32_t* nodesobjs,
                                     const int32_t* fitting_subtrees, float* grad_data, float* grad_kernels,
                                     void* stream);

/* ------------------------------------------------------------------------------------------------
 * gmc_mhem_fit_forward for callers that have no scratch memory to give. (No counterpart in the reference, which
 * allocates its temporaries itself.)
 *
 * Who needs it: hosts that cannot allocate device memory at the time of the call -- a server that handed the whole
 * GPU to its own pools when it started, a plug-in that only ever sees its input and output buffers, a loop that must
 * not risk the device-wide synchronisation an allocation can cause. The call takes the same inputs and outputs as
 * gmc_mhem_fit_forward, minus scratch_keys: the Morton-key scratch is a fixed 8 MiB array that is part of the
 * library image, so every GPU that loads the library holds those 8 MiB until the process ends. The entry point
 * itself never allocates or frees memory, on the host or on the device.
 *
 * Limit: n_mixtures * n_components <= gmc_mhem_fit_forward_noalloc_capacity() (2^20 keys); larger problems are
 * refused with GMC_ERR_BUILTIN_SCRATCH before any GPU work is issued -- use gmc_mhem_fit_forward for those.
 * Set-up: the first call on each device looks up the device address of the built-in array (once per device, with
 * that device current); make that first call before starting any stream capture. The address is remembered per
 * device ordinal for the life of the process: after a cudaDeviceReset() in the same process it is stale and the
 * library must be reloaded. Pointers and stream must belong to the device that is current when the call is made.
 * Sharing: all calls on a device use the same array and it keeps whatever the previous call left in it. Nothing in
 * it has to start at zero (every slot read is written first), but two calls that run concurrently on the GPU -- on
 * different streams or from different threads -- would overwrite each other's keys: order such calls yourself.
 * Results are identical to gmc_mhem_fit_forward.
 * ---------------------------------------------------------------------------------------------- */
long long gmc_mhem_fit_forward_noalloc_capacity(void);
int gmc_mhem_fit_forward_noalloc(const float* mixture, long long n_mixtures, int n_components, int n_dims,
                                 int n_components_fitting, int reduction_n, float* fitting, int16_t* bvh_nodes,
                                 float* bvh_attributes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GMC_B200_H */
