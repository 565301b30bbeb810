// Self-test of the bounded-wait path shared by the tensor-core kernels: a one-CTA kernel waits on an
// mbarrier that nothing arrives at, with a caller-given cycle limit, through the same mbar_wait /
// WaitCtl code the operator kernels use.  When the limit runs out the wait records its code in the
// device status word and returns false, and the kernel ends normally.  No trap, no fault, no endless loop.
#include "kernels.h"
#include "tc_common.cuh"

namespace fmhf {
namespace {

__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(const WaitArgs wait) {
    __shared__ __align__(8) unsigned long long barrier_word;
    __shared__ int abort_word;
    const uint32_t bar = smem_u32(&barrier_word);
    if (threadIdx.x == 0) {
        abort_word = launch_aborted(wait);
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncwarp();
    const WaitCtl ctl{&abort_word, wait};
    // Every lane waits, as the element-wise warps of the operator kernels do; one of them records the code.
    const bool arrived = mbar_wait(bar, 0, ctl, kKernelSelfTest * 100 + 1);
    (void)arrived;  // always false here: nothing arrives at the barrier
    __syncwarp();
}

}  // namespace

int selftest_bounded_wait(long long limit_cycles, cudaStream_t st, int *n_launch) {
    const DeviceCtl *dc = device_ctl();
    if (!dc) return FLASHMHF_ERR_CUDA;
    WaitArgs w = wait_args(dc);
    w.limit_cycles = limit_cycles;
    bounded_wait_selftest_kernel<<<1, 32, 0, st>>>(w);
    *n_launch += 1;
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_cuda_error(e, "bounded_wait_selftest_kernel launch"); return FLASHMHF_ERR_CUDA; }
    return FLASHMHF_OK;
}

}  // namespace fmhf
