// Shared helpers of the sm_100a kernels: status plumbing, the device-side check word,
// bounded mbarrier waits and non-multicast bulk (TMA) copies from this GPU's own memory.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "gmc_b200.h"

namespace gmc {

// Last CUDA error seen by this thread (message only; the status code carries the category).
void set_last_cuda_error(cudaError_t e);

#define GMC_CUDA_TRY(expr)                                  \
    do {                                                    \
        cudaError_t gmc_e_ = (expr);                        \
        if (gmc_e_ != cudaSuccess) {                        \
            ::gmc::set_last_cuda_error(gmc_e_);             \
            return GMC_ERR_CUDA;                            \
        }                                                   \
    } while (0)

#define GMC_LAUNCH_CHECK() GMC_CUDA_TRY(cudaGetLastError())

// One word per translation unit (the library is built without relocatable device code). Kernels OR
// a code into it when a bounded wait gives up or a self check fails; gmc_device_check_word() reads
// and clears the word of every unit through the reader that GMC_DEFINE_TU_CHECK_READER defines.
static __device__ int g_device_check_word;

#define GMC_DEFINE_TU_CHECK_READER(name)                                                          \
    int gmc_tu_check_##name(int* word) {                                                          \
        int w = 0;                                                                                \
        const int zero = 0;                                                                       \
        GMC_CUDA_TRY(cudaMemcpyFromSymbol(&w, ::gmc::g_device_check_word, sizeof(int)));          \
        if (w != 0) GMC_CUDA_TRY(cudaMemcpyToSymbol(::gmc::g_device_check_word, &zero, sizeof(int))); \
        *word |= w;                                                                               \
        return GMC_OK;                                                                            \
    }

enum DeviceCheck : int {
    CHECK_MBARRIER_TIMEOUT = 1,     // a bounded wait for a bulk copy ran out
    CHECK_INDEX_RANGE = 4,          // GMC_BOUNDS_CHECK builds only: a data-dependent index left its array
};

__device__ __forceinline__ void report_check(int code) { atomicOr(&g_device_check_word, code); }

// Data-dependent indices (tree children, sorted object ids, subtree ranges) are checked in builds compiled with
// -DGMC_BOUNDS_CHECK: an index outside [0, n) sets CHECK_INDEX_RANGE in the check word and is replaced by 0, so the
// access that follows stays inside the array. Regular builds compile the macro to the index itself.
#ifdef GMC_BOUNDS_CHECK
template <typename I, typename N>
__device__ __forceinline__ I checked_index(I i, N n) {
    if (static_cast<unsigned long long>(i) >= static_cast<unsigned long long>(n)) {
        report_check(CHECK_INDEX_RANGE);
        return I(0);
    }
    return i;
}
#define GMC_IDX(i, n) ::gmc::checked_index((i), (n))
#else
#define GMC_IDX(i, n) (i)
#endif

static inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kInv2Pi = 0.15915494309189535f;       // (2 pi)^-1
constexpr float kInv2Pi15 = 0.06349363593424097f;     // (2 pi)^-1.5

template <int D>
__host__ __device__ constexpr float gauss_norm_factor() {
    return D == 2 ? kInv2Pi : kInv2Pi15;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---------------------------------------------------------------------------------------------
// mbarrier + bulk async copy (TMA, untiled form), CTA-local, never multicast.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

// Bulk copy global -> shared of `bytes` (multiple of 16; both addresses 16-byte aligned),
// completion signalled on `bar`. The source must be memory of the GPU running the kernel.
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src_gmem, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Waits for the phase with the given parity, giving up after `max_polls` polls. Returns false
// (after recording CHECK_MBARRIER_TIMEOUT) if the phase never completed.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity, int max_polls = (1 << 22)) {
    const uint32_t addr = smem_u32(bar);
    for (int it = 0; it < max_polls; ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    report_check(CHECK_MBARRIER_TIMEOUT);
    return false;
}

}  // namespace gmc
