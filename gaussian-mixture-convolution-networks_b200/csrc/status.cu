// Status strings, the per-thread CUDA error message and the device check word reader.
#include "common.cuh"

namespace gmc {
namespace {
thread_local cudaError_t t_last_error = cudaSuccess;
}
void set_last_cuda_error(cudaError_t e) { t_last_error = e; }
}  // namespace gmc

// one reader per translation unit that owns kernels
int gmc_tu_check_eval_inversed(int* word);
int gmc_tu_check_small_ops(int* word);
int gmc_tu_check_lbvh(int* word);
int gmc_tu_check_mhem_fit(int* word);
int gmc_tu_check_convolution(int* word);
int gmc_tu_check_convolution_fitting(int* word);
int gmc_tu_check_relu_fixed_point(int* word);

extern "C" const char* gmc_status_string(int status) {
    switch (status) {
        case GMC_OK: return "ok";
        case GMC_ERR_BAD_DIMS: return "bad dimensions: D must be 2 or 3 and every extent positive and within its limit";
        case GMC_ERR_BAD_BROADCAST: return "xes must have a batch and layer extent of one or equal to the mixture's";
        case GMC_ERR_NULL_POINTER: return "a required pointer is NULL";
        case GMC_ERR_UNSUPPORTED: return "unsupported parameter value";
        case GMC_ERR_CUDA: return "CUDA runtime error";
        case GMC_ERR_DEVICE_CHECK: return "a device-side check failed";
        case GMC_ERR_BUILTIN_SCRATCH:
            return "problem exceeds the built-in scratch of the no-allocation entry point (n_mixtures * n_components > "
                   "2^20); use the entry point that takes caller scratch";
        default: return "unknown status";
    }
}

extern "C" const char* gmc_last_cuda_error(void) {
    return gmc::t_last_error == cudaSuccess ? "" : cudaGetErrorString(gmc::t_last_error);
}

extern "C" const char* gmc_version(void) { return "0.1"; }

static int read_all_check_words(int* word_out);

extern "C" int gmc_sync_and_check(void* stream) {
    GMC_CUDA_TRY(cudaStreamSynchronize(gmc::as_stream(stream)));
    int word = 0;
    if (int s = read_all_check_words(&word)) return s;
    return word != 0 ? GMC_ERR_DEVICE_CHECK : GMC_OK;
}

extern "C" int gmc_device_check_word(int* word_out) {
    if (!word_out) return GMC_ERR_NULL_POINTER;
    *word_out = 0;
    GMC_CUDA_TRY(cudaDeviceSynchronize());
    return read_all_check_words(word_out);
}

static int read_all_check_words(int* word_out) {
    if (int s = gmc_tu_check_eval_inversed(word_out)) return s;
    if (int s = gmc_tu_check_small_ops(word_out)) return s;
    if (int s = gmc_tu_check_lbvh(word_out)) return s;
    if (int s = gmc_tu_check_mhem_fit(word_out)) return s;
    if (int s = gmc_tu_check_convolution(word_out)) return s;
    if (int s = gmc_tu_check_convolution_fitting(word_out)) return s;
    if (int s = gmc_tu_check_relu_fixed_point(word_out)) return s;
    return GMC_OK;
}
