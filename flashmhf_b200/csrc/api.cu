// C-ABI layer: argument validation, dispatch to the kernel families, status word, error text.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "kernels.h"

namespace fmhf {

// Per device: the status word (first failure wins) and the sequence number of the launch that failed.
static __device__ int g_status_word;
static __device__ unsigned g_abort_seq;

namespace {
std::atomic<uint64_t> g_launches{0};
std::atomic<unsigned> g_seq{0};
thread_local char tl_cuda_error[256] = "";
constexpr int kMaxDevices = 64;
std::mutex g_mu;
DeviceCtl g_ctl[kMaxDevices];
std::atomic<bool> g_ctl_ready[kMaxDevices];
}  // namespace

namespace {
struct Profile {
    std::atomic<bool> on{false};
    std::vector<cudaEvent_t> ev;
    std::vector<int> tag;
    size_t n = 0;
};
Profile g_prof;
}  // namespace

void prof_mark(cudaStream_t st, int tag) {
    if (!g_prof.on) return;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_prof.on || g_prof.n >= g_prof.ev.size()) return;
    if (cudaEventRecord(g_prof.ev[g_prof.n], st) == cudaSuccess) g_prof.tag[g_prof.n++] = tag;
}

void set_cuda_error(cudaError_t e, const char *where) {
    snprintf(tl_cuda_error, sizeof(tl_cuda_error), "%s: %s", where, cudaGetErrorString(e));
}

unsigned next_launch_seq() {
    unsigned s = ++g_seq;
    return s ? s : ++g_seq;
}

const DeviceCtl *device_ctl() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_cuda_error(e, "cudaGetDevice");
        return nullptr;
    }
    if (g_ctl_ready[dev].load(std::memory_order_acquire)) return &g_ctl[dev];
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_ctl_ready[dev].load(std::memory_order_relaxed)) {
        void *ps = nullptr, *pa = nullptr;
        int sms = 0;
        e = cudaGetSymbolAddress(&ps, g_status_word);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&pa, g_abort_seq);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || sms < 1) {
            set_cuda_error(e, "device set-up (status word, SM count)");
            return nullptr;
        }
        g_ctl[dev].status = static_cast<int *>(ps);
        g_ctl[dev].abort_seq = static_cast<unsigned *>(pa);
        g_ctl[dev].num_sms = sms;
        g_ctl[dev].device = dev;
        g_ctl_ready[dev].store(true, std::memory_order_release);
    }
    return &g_ctl[dev];
}

namespace {

int check_scaling(const flashmhf_scaling &s) {
    for (float v : {s.head_scaling, s.up_scaling, s.final_scaling})
        if (!(v == v) || v == 0.f || v - v != 0.f) return FLASHMHF_ERR_BAD_SHAPE;  // NaN, zero or infinite
    return FLASHMHF_OK;
}

int check_dims(const flashmhf_dims &d) {
    if (d.dtype != FLASHMHF_BF16 && d.dtype != FLASHMHF_F32_CHECK) return FLASHMHF_ERR_BAD_DTYPE;
    if (d.B < 1 || d.H < 1 || d.S < 1 || d.Hkuv < 1 || d.E < 1 || d.De < 1) return FLASHMHF_ERR_BAD_SHAPE;
    if (d.H % d.Hkuv != 0) return FLASHMHF_ERR_BAD_SHAPE;
    if (d.De % 64 != 0) return FLASHMHF_ERR_BAD_SHAPE;
    if (d.Dh != 64 && d.Dh != 96 && d.Dh != 128) return FLASHMHF_ERR_BAD_SHAPE;
    if ((long long)d.E * d.De > (1LL << 30) || d.B > 65535 || d.H > 65535) return FLASHMHF_ERR_BAD_SHAPE;
    return FLASHMHF_OK;
}

// `align`: 16 bytes for the bf16 tensors (TMA), 4 for the routing weights and their gradient, which the
// kernels read and write one fp32 element at a time.
int check_tensor(const flashmhf_tensor &t, unsigned align = 16) {
    if (!t.ptr) return FLASHMHF_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(t.ptr) & (align - 1u)) != 0) return FLASHMHF_ERR_MISALIGNED;
    for (int i = 0; i < 3; ++i)
        if (t.stride[i] < 0) return FLASHMHF_ERR_BAD_STRIDE;
    return FLASHMHF_OK;
}

int check_arch() {
    static std::atomic<int> major_of[kMaxDevices];   // 0 = not asked yet
    int dev = 0, major = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess && dev >= 0 && dev < kMaxDevices && (major = major_of[dev].load(std::memory_order_relaxed)) != 0)
        return major == 10 ? FLASHMHF_OK : FLASHMHF_ERR_ARCH;
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) {
        set_cuda_error(e, "device query");
        return FLASHMHF_ERR_CUDA;
    }
    if (dev >= 0 && dev < kMaxDevices) major_of[dev].store(major, std::memory_order_relaxed);
    return major == 10 ? FLASHMHF_OK : FLASHMHF_ERR_ARCH;
}

}  // namespace
}  // namespace fmhf

using namespace fmhf;

extern "C" {

int flashmhf_abi_version(void) { return FLASHMHF_ABI_VERSION; }

const char *flashmhf_strerror(int status) {
    switch (status) {
        case FLASHMHF_OK: return "ok";
        case FLASHMHF_ERR_NULL: return "a required pointer is NULL";
        case FLASHMHF_ERR_BAD_SHAPE:
            return "unsupported shape (need d_h in {64,96,128}, d_e % 64 == 0, H % H_kuv == 0, all dims >= 1)";
        case FLASHMHF_ERR_BAD_DTYPE: return "unsupported dtype (FLASHMHF_BF16 or FLASHMHF_F32_CHECK)";
        case FLASHMHF_ERR_BAD_STRIDE:
            return "stride not expressible (negative, not a multiple of 16 bytes, or E and d_e do not collapse)";
        case FLASHMHF_ERR_MISALIGNED: return "base pointer not 16-byte aligned";
        case FLASHMHF_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case FLASHMHF_ERR_ARCH: return "current device is not compute capability 10.x (B200)";
        case FLASHMHF_ERR_CUDA: return "CUDA call failed (see flashmhf_last_cuda_error)";
        case FLASHMHF_ERR_DEVICE_TIMEOUT: return "a kernel gave up on a bounded wait";
        case FLASHMHF_ERR_SCRATCH_LIMIT:
            return "these dims need more scratch than the library's built-in 72 MiB array; use flashmhf_backward with a workspace";
        default: return "unknown status";
    }
}

const char *flashmhf_last_cuda_error(void) { return tl_cuda_error; }

uint64_t flashmhf_launch_count(void) { return g_launches.load(); }

static int forward_entry(const flashmhf_fwd_params *p, void *stream, bool chained) {
    if (!p) return FLASHMHF_ERR_NULL;
    int rc = check_dims(p->d);
    if (rc) return rc;
    if ((rc = check_scaling(p->scale)) != 0) return rc;
    const flashmhf_tensor *ts[] = {&p->Q, &p->K, &p->U, &p->V, &p->O};
    for (const flashmhf_tensor *t : ts)
        if ((rc = check_tensor(*t)) != 0) return rc;
    if ((rc = check_tensor(p->R, 4)) != 0) return rc;
    if ((rc = check_arch()) != 0) return rc;
    if (!device_ctl()) return FLASHMHF_ERR_CUDA;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int n = 0;
    if (p->d.dtype == FLASHMHF_F32_CHECK) {
        if (chained) return FLASHMHF_ERR_BAD_DTYPE;
        cudaError_t e = simt_forward(*p, st, &n);
        if (e != cudaSuccess) {
            set_cuda_error(e, "check forward launch");
            rc = FLASHMHF_ERR_CUDA;
        }
    } else {
        rc = tc_forward(*p, st, &n, chained);
    }
    g_launches += (uint64_t)n;
    return rc;
}

int flashmhf_forward(const flashmhf_fwd_params *p, void *stream) { return forward_entry(p, stream, false); }

int flashmhf_forward_chained(const flashmhf_fwd_params *p, void *stream) { return forward_entry(p, stream, true); }

size_t flashmhf_forward_workspace_bytes(const flashmhf_dims *d) {
    if (!d || check_dims(*d) != 0) return 0;
    if (d->dtype == FLASHMHF_F32_CHECK) return 0;
    return tc_forward_workspace_bytes(*d);
}

size_t flashmhf_backward_workspace_bytes(const flashmhf_dims *d) {
    if (!d || check_dims(*d) != 0) return 0;
    if (d->dtype == FLASHMHF_F32_CHECK) return 0;
    return tc_backward_workspace_bytes(*d);
}

// Shared argument checks of the two backward entry points.  Tensors of a part that is not asked for are not looked at.
static int check_bwd(const flashmhf_bwd_params *p, unsigned *parts_out) {
    if (!p) return FLASHMHF_ERR_NULL;
    int rc = check_dims(p->d);
    if (rc) return rc;
    if ((rc = check_scaling(p->scale)) != 0) return rc;
    if (p->parts & ~(FLASHMHF_BWD_INPUTS | FLASHMHF_BWD_WEIGHTS)) return FLASHMHF_ERR_BAD_SHAPE;
    const unsigned parts = p->parts ? p->parts : (FLASHMHF_BWD_INPUTS | FLASHMHF_BWD_WEIGHTS);
    for (const flashmhf_tensor *t : {&p->Q, &p->K, &p->U, &p->V, &p->dO})
        if ((rc = check_tensor(*t)) != 0) return rc;
    if ((rc = check_tensor(p->R, 4)) != 0) return rc;
    if (parts & FLASHMHF_BWD_INPUTS) {
        if ((rc = check_tensor(p->dQ)) != 0) return rc;
        if ((rc = check_tensor(p->dR, 4)) != 0) return rc;
    }
    if (parts & FLASHMHF_BWD_WEIGHTS)
        for (const flashmhf_tensor *t : {&p->dK, &p->dU, &p->dV})
            if ((rc = check_tensor(*t)) != 0) return rc;
    *parts_out = parts;
    return FLASHMHF_OK;
}

int flashmhf_backward(const flashmhf_bwd_params *p, void *stream) {
    unsigned parts = 0;
    int rc = check_bwd(p, &parts);
    if (rc) return rc;
    if (parts & FLASHMHF_BWD_WEIGHTS) {
        const size_t need = flashmhf_backward_workspace_bytes(&p->d);
        if (need > 0 && (!p->workspace || p->workspace_bytes < need || (reinterpret_cast<uintptr_t>(p->workspace) & 255u)))
            return FLASHMHF_ERR_WORKSPACE;
    }
    if ((rc = check_arch()) != 0) return rc;
    if (!device_ctl()) return FLASHMHF_ERR_CUDA;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int n = 0;
    flashmhf_bwd_params q = *p;
    q.parts = parts;
    if (p->d.dtype == FLASHMHF_F32_CHECK) {
        cudaError_t e = simt_backward(q, st, &n);
        if (e != cudaSuccess) {
            set_cuda_error(e, "check backward launch");
            rc = FLASHMHF_ERR_CUDA;
        }
    } else {
        rc = tc_backward(q, st, &n);
    }
    g_launches += (uint64_t)n;
    return rc;
}

int flashmhf_backward_static_scratch(const flashmhf_bwd_params *p, void *stream) {
    unsigned parts = 0;
    int rc = check_bwd(p, &parts);
    if (rc) return rc;
    if (p->d.dtype != FLASHMHF_BF16) return FLASHMHF_ERR_BAD_DTYPE;
    if ((rc = check_arch()) != 0) return rc;
    if (!device_ctl()) return FLASHMHF_ERR_CUDA;
    int n = 0;
    flashmhf_bwd_params q = *p;
    q.parts = parts;
    rc = tc_backward_static_scratch(q, static_cast<cudaStream_t>(stream), &n);
    g_launches += (uint64_t)n;
    return rc;
}

int flashmhf_selftest_bounded_wait(long long limit_cycles, void *stream) {
    if (limit_cycles < 1 || limit_cycles > kDefaultWaitLimitCycles) return FLASHMHF_ERR_BAD_SHAPE;
    int rc = check_arch();
    if (rc) return rc;
    if (!device_ctl()) return FLASHMHF_ERR_CUDA;
    int n = 0;
    rc = selftest_bounded_wait(limit_cycles, static_cast<cudaStream_t>(stream), &n);
    g_launches += (uint64_t)n;
    return rc;
}

int flashmhf_prologue_forward(const flashmhf_prologue_params *p, void *stream) {
    if (!p) return FLASHMHF_ERR_NULL;
    int rc = check_arch();
    if (rc) return rc;
    int n = 0;
    rc = prologue_forward(*p, static_cast<cudaStream_t>(stream), &n);
    g_launches += (uint64_t)n;
    return rc;
}

size_t flashmhf_prologue_backward_workspace_bytes(const flashmhf_prologue_params *p) {
    if (!p || p->B < 1 || p->S < 1 || p->H < 1 || p->E < 1 || p->Dh < 1) return 0;
    return prologue_backward_workspace_bytes(*p);
}

int flashmhf_prologue_backward(const flashmhf_prologue_bwd_params *p, void *stream) {
    if (!p) return FLASHMHF_ERR_NULL;
    int rc = check_arch();
    if (rc) return rc;
    int n = 0;
    rc = prologue_backward(*p, static_cast<cudaStream_t>(stream), &n);
    g_launches += (uint64_t)n;
    return rc;
}

int flashmhf_lm_rope(const void *x, void *y, const float *cos_t, const float *sin_t, int64_t tokens, int32_t S,
                     int32_t heads, int32_t head_dim, int64_t x_token_stride, int64_t y_token_stride, int32_t transpose,
                     void *stream) {
    int rc = check_arch();
    if (rc) return rc;
    int n = 0;
    rc = lm_rope(x, y, cos_t, sin_t, tokens, S, heads, head_dim, x_token_stride, y_token_stride, transpose,
                 static_cast<cudaStream_t>(stream), &n);
    g_launches += (uint64_t)n;
    return rc;
}

int flashmhf_lm_rmsnorm_forward(const void *x, const float *w, void *y, int64_t rows, int32_t n, float eps, void *stream) {
    int rc = check_arch();
    if (rc) return rc;
    int nl = 0;
    rc = lm_rmsnorm_forward(x, w, y, rows, n, eps, static_cast<cudaStream_t>(stream), &nl);
    g_launches += (uint64_t)nl;
    return rc;
}

size_t flashmhf_lm_rmsnorm_backward_workspace_bytes(int64_t rows, int32_t n) {
    return lm_rmsnorm_backward_workspace_bytes(rows, n);
}

int flashmhf_lm_rmsnorm_backward(const void *x, const float *w, const void *g, void *dx, float *dw, void *workspace,
                                 size_t workspace_bytes, int64_t rows, int32_t n, float eps, void *stream) {
    int rc = check_arch();
    if (rc) return rc;
    int nl = 0;
    rc = lm_rmsnorm_backward(x, w, g, dx, dw, workspace, workspace_bytes, rows, n, eps, static_cast<cudaStream_t>(stream), &nl);
    g_launches += (uint64_t)nl;
    return rc;
}

int flashmhf_profile_begin(int max_marks) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_prof.on || max_marks < 2) return FLASHMHF_ERR_BAD_SHAPE;
    g_prof.ev.resize((size_t)max_marks);
    g_prof.tag.assign((size_t)max_marks, 0);
    for (int i = 0; i < max_marks; ++i) {
        cudaError_t e = cudaEventCreate(&g_prof.ev[i]);
        if (e != cudaSuccess) {
            for (int j = 0; j < i; ++j) cudaEventDestroy(g_prof.ev[j]);
            g_prof.ev.clear();
            set_cuda_error(e, "cudaEventCreate");
            return FLASHMHF_ERR_CUDA;
        }
    }
    g_prof.n = 0;
    g_prof.on = true;
    return FLASHMHF_OK;
}

int flashmhf_profile_end(float *ms, int *tags, int capacity, int *n_out) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_prof.on) return FLASHMHF_ERR_BAD_SHAPE;
    g_prof.on = false;
    int n = 0, rc = FLASHMHF_OK;
    cudaError_t e = cudaDeviceSynchronize();
    for (size_t i = 1; e == cudaSuccess && i < g_prof.n; ++i) {
        if (g_prof.tag[i] == kMarkStart) continue;  // interval between two calls, not a kernel
        float t = 0.f;
        e = cudaEventElapsedTime(&t, g_prof.ev[i - 1], g_prof.ev[i]);
        if (e == cudaSuccess && ms && tags && n < capacity) {
            ms[n] = t;
            tags[n] = g_prof.tag[i];
            ++n;
        }
    }
    if (e != cudaSuccess) {
        set_cuda_error(e, "flashmhf_profile_end");
        rc = FLASHMHF_ERR_CUDA;
    }
    for (cudaEvent_t ev : g_prof.ev) cudaEventDestroy(ev);
    g_prof.ev.clear();
    g_prof.n = 0;
    if (n_out) *n_out = n;
    return rc;
}

int flashmhf_device_status(int *code) {
    if (code) *code = 0;
    const DeviceCtl *ctl = device_ctl();
    if (!ctl) return FLASHMHF_ERR_CUDA;
    int *addr = ctl->status;
    cudaError_t e = cudaDeviceSynchronize();
    int v = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&v, addr, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && v != 0) e = cudaMemset(addr, 0, sizeof(int));
    if (e != cudaSuccess) {
        set_cuda_error(e, "flashmhf_device_status");
        return FLASHMHF_ERR_CUDA;
    }
    if (code) *code = v;
    return v == 0 ? FLASHMHF_OK : FLASHMHF_ERR_DEVICE_TIMEOUT;
}

}  // extern "C"
