// Internal launch interface between the C-ABI layer (api.cu) and the kernel translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flashmhf.h"

namespace fmhf {

// Per-device control words and facts, resolved once per device (with that device current).
//   status    : 0, or the code of the first bounded wait that ran out since the host last read it
//   abort_seq : sequence number of the launch whose wait ran out; the other CTAs of THAT launch see it at
//               their start and return at once, later launches (other numbers) run normally
struct DeviceCtl {
    int *status = nullptr;
    unsigned *abort_seq = nullptr;
    int num_sms = 0;
    int device = -1;
};
const DeviceCtl *device_ctl();  // nullptr if the device query failed
unsigned next_launch_seq();     // process-wide, never 0
// SM count of the current device (the B200's 148 when no device can be queried, e.g. sizing a workspace on a CPU-only host).
inline int num_sms() {
    const DeviceCtl *c = device_ctl();
    return c ? c->num_sms : 148;
}

// What every tensor-core kernel needs for its bounded waits.
struct WaitArgs {
    int *status;
    unsigned *abort_seq;
    unsigned seq;
    long long limit_cycles;
};
constexpr long long kDefaultWaitLimitCycles = 3LL << 30;  // ~1.5 s at 1.4-1.9 GHz; a healthy kernel waits microseconds
inline WaitArgs wait_args(const DeviceCtl *c) {
    return WaitArgs{c->status, c->abort_seq, next_launch_seq(), kDefaultWaitLimitCycles};
}

// ---- fp32 check kernels (CUDA cores) -------------------------------------------------------
cudaError_t simt_forward(const flashmhf_fwd_params &p, cudaStream_t st, int *n_launch);
cudaError_t simt_backward(const flashmhf_bwd_params &p, cudaStream_t st, int *n_launch);

// ---- bf16 tensor-core kernels (tcgen05 / TMEM / TMA) ---------------------------------------
// Each returns a flashmhf_status (tensor-map encoding can fail with BAD_STRIDE / CUDA).
// `chained`: launched so that it may overlap the end of the kernel before it on the stream (see flashmhf_forward_chained)
int tc_forward(const flashmhf_fwd_params &p, cudaStream_t st, int *n_launch, bool chained);
size_t tc_forward_workspace_bytes(const flashmhf_dims &d);
int tc_backward(const flashmhf_bwd_params &p, cudaStream_t st, int *n_launch);
size_t tc_backward_workspace_bytes(const flashmhf_dims &d);
int tc_backward_static_scratch(const flashmhf_bwd_params &p, cudaStream_t st, int *n_launch);

// ---- fused layer prologue (per-head RMSNorm + router weights), HBM-bound CUDA-core kernels --
int prologue_forward(const flashmhf_prologue_params &p, cudaStream_t st, int *n_launch);
size_t prologue_backward_workspace_bytes(const flashmhf_prologue_params &p);
int prologue_backward(const flashmhf_prologue_bwd_params &p, cudaStream_t st, int *n_launch);

// ---- helpers for the measurement LM: rotary embedding and hidden-size RMSNorm (lm_aux.cu) ----
int lm_rope(const void *x, void *y, const float *cos_t, const float *sin_t, long long tokens, int S, int heads, int hd,
            long long x_tok, long long y_tok, int transpose, cudaStream_t st, int *n_launch);
int lm_rmsnorm_forward(const void *x, const float *w, void *y, long long rows, int n, float eps, cudaStream_t st, int *n_launch);
size_t lm_rmsnorm_backward_workspace_bytes(long long rows, int n);
int lm_rmsnorm_backward(const void *x, const float *w, const void *g, void *dx, float *dw, void *workspace,
                        size_t workspace_bytes, long long rows, int n, float eps, cudaStream_t st, int *n_launch);

void set_cuda_error(cudaError_t e, const char *where);
int selftest_bounded_wait(long long limit_cycles, cudaStream_t st, int *n_launch);

// Kernel-boundary marks for the profiling aid (flashmhf_profile_begin/end): records an event on
// `st` tagged `tag` when profiling is on, does nothing otherwise.
enum { kMarkStart = 0, kMarkFwd = 1, kMarkBwdDq = 2, kMarkBwdDw = 3, kMarkBwdReduce = 4, kMarkFwdReduce = 5,
       kMarkPrologueFwd = 6, kMarkPrologueBwd = 7, kMarkPrologueReduce = 8 };
void prof_mark(cudaStream_t st, int tag);

}  // namespace fmhf
