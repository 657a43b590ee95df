// Mixture evaluation (forward, optionally with its backward) on HOST buffers.
//
// The batch is cut into slices. Streams run a software pipeline over kSlots device slots:
//   copy-in  : host -> device of slice i+1 (mixture, xes, grad_out)
//   compute  : forward + backward kernels of slice i (one stream per slot, so that the first CTAs of a slice fill the
//              SMs that the last wave of the previous slice leaves idle)
//   copy-out : device -> host of slice i-1 (out, grad_mixture, grad_xes)
// PCIe is full duplex, so with page-locked host buffers both copy directions hide behind the kernels and the
// call costs about one slice of copy-in, the kernels, and one slice of copy-out.
//
// The device workspace (cudaMalloc, grown with cudaFree + cudaMalloc when a larger problem arrives), six streams and
// twelve events are created once per device and kept until gmc_host_pipeline_release(). One mutex serialises the calls
// of a process: the slots are shared. The call blocks until the host buffers are complete.
#include <mutex>

#include "common.cuh"

namespace gmc {
namespace {

constexpr int kSlots = 4;
constexpr int kMaxDevices = 64;

struct DevicePipe {
    bool ready = false;
    cudaStream_t s_in = nullptr, s_comp[kSlots] = {}, s_out = nullptr;
    cudaEvent_t in_done[kSlots] = {}, comp_done[kSlots] = {}, out_done[kSlots] = {};
    float* slot[kSlots] = {};
    size_t slot_floats = 0;
};

std::mutex g_pipe_mutex;
DevicePipe g_pipes[kMaxDevices];

int pipe_prepare(DevicePipe& p, size_t need_floats) {
    if (!p.ready) {
        GMC_CUDA_TRY(cudaStreamCreateWithFlags(&p.s_in, cudaStreamNonBlocking));
        for (int k = 0; k < kSlots; ++k) GMC_CUDA_TRY(cudaStreamCreateWithFlags(&p.s_comp[k], cudaStreamNonBlocking));
        GMC_CUDA_TRY(cudaStreamCreateWithFlags(&p.s_out, cudaStreamNonBlocking));
        for (int k = 0; k < kSlots; ++k) {
            GMC_CUDA_TRY(cudaEventCreateWithFlags(&p.in_done[k], cudaEventDisableTiming));
            GMC_CUDA_TRY(cudaEventCreateWithFlags(&p.comp_done[k], cudaEventDisableTiming));
            GMC_CUDA_TRY(cudaEventCreateWithFlags(&p.out_done[k], cudaEventDisableTiming));
        }
        p.ready = true;
    }
    if (need_floats > p.slot_floats) {
        for (int k = 0; k < kSlots; ++k) {
            if (p.slot[k]) GMC_CUDA_TRY(cudaFree(p.slot[k]));
            p.slot[k] = nullptr;
        }
        p.slot_floats = 0;
        for (int k = 0; k < kSlots; ++k) GMC_CUDA_TRY(cudaMalloc(&p.slot[k], need_floats * sizeof(float)));
        p.slot_floats = need_floats;
    }
    return GMC_OK;
}

int pipe_release(DevicePipe& p) {
    if (!p.ready) return GMC_OK;
    for (int k = 0; k < kSlots; ++k) {
        if (p.slot[k]) GMC_CUDA_TRY(cudaFree(p.slot[k]));
        p.slot[k] = nullptr;
        GMC_CUDA_TRY(cudaEventDestroy(p.in_done[k]));
        GMC_CUDA_TRY(cudaEventDestroy(p.comp_done[k]));
        GMC_CUDA_TRY(cudaEventDestroy(p.out_done[k]));
    }
    GMC_CUDA_TRY(cudaStreamDestroy(p.s_in));
    for (int k = 0; k < kSlots; ++k) GMC_CUDA_TRY(cudaStreamDestroy(p.s_comp[k]));
    GMC_CUDA_TRY(cudaStreamDestroy(p.s_out));
    p = DevicePipe();
    return GMC_OK;
}

inline size_t round64(size_t n) { return (n + 63) & ~size_t(63); }   // keeps every sub-buffer 256-byte aligned

}  // namespace
}  // namespace gmc

int gmc_tu_check_eval_inversed(int* word);   // reads and clears the check word of the evaluation kernels (eval_inversed.cu)

extern "C" int gmc_eval_inversed_host(const float* mixture, const float* xes, const float* grad_out, float* out,
                                      float* grad_mixture, float* grad_xes, int n_batch, int n_layers,
                                      int n_components, int n_dims, int n_batch_xes, int n_layers_xes, int n_xes,
                                      int n_slices) {
    using namespace gmc;
    if (n_dims != 2 && n_dims != 3) return GMC_ERR_BAD_DIMS;
    if (n_batch <= 0 || n_layers <= 0 || n_components <= 0 || n_xes <= 0) return GMC_ERR_BAD_DIMS;
    if (n_batch_xes != 1 && n_batch_xes != n_batch) return GMC_ERR_BAD_BROADCAST;
    if (n_layers_xes != 1 && n_layers_xes != n_layers) return GMC_ERR_BAD_BROADCAST;
    if (!mixture || !xes) return GMC_ERR_NULL_POINTER;
    if (!out && !grad_out) return GMC_ERR_NULL_POINTER;
    if (!grad_out && (grad_mixture || grad_xes)) return GMC_ERR_NULL_POINTER;
    const bool backward = grad_out != nullptr && (grad_mixture != nullptr || grad_xes != nullptr);

    int device = 0;
    GMC_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return GMC_ERR_BAD_DIMS;

    // xes shared by the whole batch: its gradient sums over the batch inside one launch, so the batch stays whole
    const bool shared_xes = n_batch_xes == 1 && n_batch > 1;
    // Slice plan. n_slices > 0: equal slices. n_slices == 0: slices of about n_batch / 8 with short slices at both
    // ends (1, 2, ... entries), because the copy-in of the first slice and the copy-out of the last one are the only
    // copies that nothing overlaps.
    constexpr int kMaxSlices = 256;
    int starts[kMaxSlices + 1];
    int per;                                                       // largest slice
    if (shared_xes || n_slices == 1) {
        starts[0] = 0; starts[1] = n_batch; n_slices = 1; per = n_batch;
    } else if (n_slices > 0) {
        if (n_slices > n_batch) n_slices = n_batch;
        if (n_slices > kMaxSlices) n_slices = kMaxSlices;
        per = (n_batch + n_slices - 1) / n_slices;
        n_slices = (n_batch + per - 1) / per;
        for (int i = 0; i <= n_slices; ++i) starts[i] = i * per < n_batch ? i * per : n_batch;
    } else {
        per = n_batch >= 8 ? n_batch / 8 : 1;
        int sizes[kMaxSlices];
        int n = 0, head = 0, tail = n_batch;
        // ramp up from the front and mirror it at the back while at least two full slices remain in the middle
        int ramp[8], n_ramp = 0;
        for (int r = 1; r < per && n_ramp < 8 && tail - head - 2 * r >= 2 * per; r *= 2) {
            ramp[n_ramp++] = r; head += r; tail -= r;
        }
        for (int i = 0; i < n_ramp; ++i) sizes[n++] = ramp[i];
        for (int b0 = head; b0 < tail && n < kMaxSlices - 8; b0 += per) sizes[n++] = (b0 + per <= tail) ? per : tail - b0;
        for (int i = n_ramp - 1; i >= 0; --i) sizes[n++] = ramp[i];
        n_slices = n;
        starts[0] = 0;
        for (int i = 0; i < n; ++i) starts[i + 1] = starts[i] + sizes[i];
        if (starts[n_slices] != n_batch) {                         // plan did not fit the table: one slice per entry group
            n_slices = 1; starts[1] = n_batch; per = n_batch;
        }
    }

    const size_t rf = size_t(1 + n_dims + n_dims * n_dims);
    const size_t m_row = size_t(n_layers) * n_components * rf;     // floats per batch entry
    const size_t x_row = size_t(n_layers_xes) * n_xes * n_dims;
    const size_t o_row = size_t(n_layers) * n_xes;
    const int per_x = n_batch_xes == 1 ? 1 : per;
    // slot layout: mixture | xes | grad_out | out | grad_mixture | grad_xes
    const size_t off_m = 0;
    const size_t off_x = off_m + round64(m_row * per);
    const size_t off_g = off_x + round64(x_row * per_x);
    const size_t off_o = off_g + round64(o_row * per);
    const size_t off_gm = off_o + round64(o_row * per);
    const size_t off_gx = off_gm + round64(m_row * per);
    const size_t need = off_gx + round64(x_row * per_x);

    std::lock_guard<std::mutex> lock(g_pipe_mutex);
    DevicePipe& p = g_pipes[device];
    if (int s = pipe_prepare(p, need)) return s;

    // Inside the loop an error is recorded and the loop left; the streams are drained below in every case, because copies
    // already queued keep reading and writing the caller's buffers until they finish.
    int status = GMC_OK;
#define GMC_PIPE_TRY(expr)                                    \
    {                                                         \
        const cudaError_t pipe_e_ = (expr);                   \
        if (pipe_e_ != cudaSuccess) {                         \
            set_last_cuda_error(pipe_e_);                     \
            status = GMC_ERR_CUDA;                            \
            break;                                            \
        }                                                     \
    }
    for (int i = 0; i < n_slices && status == GMC_OK; ++i) {
        const int k = i % kSlots;
        const int b0 = starts[i];
        const int nb = starts[i + 1] - b0;
        const int nbx = n_batch_xes == 1 ? 1 : nb;
        const int bx0 = n_batch_xes == 1 ? 0 : b0;
        float* d = p.slot[k];

        // copy-in: the slot's inputs are free once the kernels of the slice that used it before (i - kSlots) are done
        if (i >= kSlots) GMC_PIPE_TRY(cudaStreamWaitEvent(p.s_in, p.comp_done[k], 0));
        GMC_PIPE_TRY(cudaMemcpyAsync(d + off_m, mixture + m_row * b0, m_row * nb * sizeof(float),
                                     cudaMemcpyHostToDevice, p.s_in));
        GMC_PIPE_TRY(cudaMemcpyAsync(d + off_x, xes + x_row * bx0, x_row * nbx * sizeof(float), cudaMemcpyHostToDevice,
                                     p.s_in));
        if (grad_out)
            GMC_PIPE_TRY(cudaMemcpyAsync(d + off_g, grad_out + o_row * b0, o_row * nb * sizeof(float),
                                         cudaMemcpyHostToDevice, p.s_in));
        GMC_PIPE_TRY(cudaEventRecord(p.in_done[k], p.s_in));

        // compute: the slot's outputs are free once slice i - kSlots has been copied out
        GMC_PIPE_TRY(cudaStreamWaitEvent(p.s_comp[k], p.in_done[k], 0));
        if (i >= kSlots) GMC_PIPE_TRY(cudaStreamWaitEvent(p.s_comp[k], p.out_done[k], 0));
        if (out)
            status = gmc_eval_inversed_forward(d + off_m, d + off_x, d + off_o, nb, n_layers, n_components, n_dims, nbx,
                                               n_layers_xes, n_xes, p.s_comp[k]);
        if (status == GMC_OK && backward)
            status = gmc_eval_inversed_backward(d + off_g, d + off_m, d + off_x, grad_mixture ? d + off_gm : nullptr,
                                                grad_xes ? d + off_gx : nullptr, nb, n_layers, n_components, n_dims,
                                                nbx, n_layers_xes, n_xes, p.s_comp[k]);
        if (status != GMC_OK) break;
        GMC_PIPE_TRY(cudaEventRecord(p.comp_done[k], p.s_comp[k]));

        // copy-out
        GMC_PIPE_TRY(cudaStreamWaitEvent(p.s_out, p.comp_done[k], 0));
        if (out)
            GMC_PIPE_TRY(cudaMemcpyAsync(out + o_row * b0, d + off_o, o_row * nb * sizeof(float), cudaMemcpyDeviceToHost,
                                         p.s_out));
        if (backward && grad_mixture)
            GMC_PIPE_TRY(cudaMemcpyAsync(grad_mixture + m_row * b0, d + off_gm, m_row * nb * sizeof(float),
                                         cudaMemcpyDeviceToHost, p.s_out));
        if (backward && grad_xes)
            GMC_PIPE_TRY(cudaMemcpyAsync(grad_xes + x_row * bx0, d + off_gx, x_row * nbx * sizeof(float),
                                         cudaMemcpyDeviceToHost, p.s_out));
        GMC_PIPE_TRY(cudaEventRecord(p.out_done[k], p.s_out));
    }
#undef GMC_PIPE_TRY
    // the host buffers are valid when the call returns; drain every stream even after an error
    cudaError_t e1 = cudaStreamSynchronize(p.s_in);
    cudaError_t e2 = cudaSuccess;
    for (int k = 0; k < kSlots; ++k) {
        const cudaError_t e = cudaStreamSynchronize(p.s_comp[k]);
        if (e2 == cudaSuccess) e2 = e;
    }
    cudaError_t e3 = cudaStreamSynchronize(p.s_out);
    if (status != GMC_OK) return status;
    GMC_CUDA_TRY(e1);
    GMC_CUDA_TRY(e2);
    GMC_CUDA_TRY(e3);
    // everything is synchronised here anyway: a kernel that gave up (bounded wait) turns into an error status
    int word = 0;
    if (int s = gmc_tu_check_eval_inversed(&word)) return s;
    return word != 0 ? GMC_ERR_DEVICE_CHECK : GMC_OK;
}

extern "C" int gmc_host_pipeline_release(void) {
    using namespace gmc;
    int device = 0;
    GMC_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return GMC_ERR_BAD_DIMS;
    std::lock_guard<std::mutex> lock(g_pipe_mutex);
    return pipe_release(g_pipes[device]);
}
