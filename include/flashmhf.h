/*
 * flashmhf.h -- C ABI of the B200 (sm_100a) FlashMHF multi-head FFN operator
 *
 *     O = sum_e R_e * ((SiLU(Q K_e^T) * (Q U_e^T)) V_e)          forward and backward
 *
 * Plain pointers and sizes only; no framework types.  Every entry point returns 0 or a negative
 * flashmhf_status code, never throws, never aborts, never blocks on the stream (except where a
 * comment says "synchronous").  The caller owns every buffer, including the workspace.
 *
 * The entry points stand where the reference's native extension has its two pybind functions,
 *   flashffn_moe_forward(Q,K,U,V,R,O)                         kernels/thunderkittens/flash_ffn_moe.cu:938-1007
 *   flashffn_moe_backward(Q,K,U,V,R,dQ,dK,dU,dV,dR,dO)        kernels/thunderkittens/flash_ffn_moe.cu:1012-1133
 * and where its Triton wrapper launches its three kernels (kernels/triton/flash_mlp_moe.py:777-790,
 * 832-866).  Shapes follow that wrapper's docstring (flash_mlp_moe.py:745-753):
 *
 *   Q, O, dO, dQ : [B, H, S, d_h]        K, U, V, dK, dU, dV : [H_kuv, E, d_e, d_h]
 *   R, dR        : [B, H, S, E] fp32     H % H_kuv == 0, d_e % 64 == 0, d_h in {64, 96, 128}
 *
 * Unlike the reference's R-transposing wrapper (kernels/thunderkittens/flash_ffn_moe_torch.py:9)
 * R is taken as the model produces it, [B,H,S,E].
 */
#ifndef FLASHMHF_H_
#define FLASHMHF_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLASHMHF_ABI_VERSION 3

typedef enum flashmhf_status {
    FLASHMHF_OK = 0,
    FLASHMHF_ERR_NULL = -1,          /* a required pointer is NULL */
    FLASHMHF_ERR_BAD_SHAPE = -2,     /* unsupported d_h, d_e % 64 != 0, H % H_kuv != 0, a dim < 1 ... */
    FLASHMHF_ERR_BAD_DTYPE = -3,     /* dtype is neither FLASHMHF_BF16 nor FLASHMHF_F32_CHECK */
    FLASHMHF_ERR_BAD_STRIDE = -4,    /* stride not expressible (negative, not a multiple of 16 bytes, E and d_e do not collapse) */
    FLASHMHF_ERR_MISALIGNED = -5,    /* base pointer not 16-byte aligned */
    FLASHMHF_ERR_WORKSPACE = -6,     /* workspace NULL or smaller than flashmhf_backward_workspace_bytes() */
    FLASHMHF_ERR_ARCH = -7,          /* current device is not compute capability 10.x */
    FLASHMHF_ERR_CUDA = -8,          /* a CUDA runtime/driver call failed (see flashmhf_last_cuda_error) */
    FLASHMHF_ERR_DEVICE_TIMEOUT = -9, /* a kernel gave up on a bounded wait and returned early (flashmhf_device_status) */
    FLASHMHF_ERR_SCRATCH_LIMIT = -10  /* flashmhf_backward_static_scratch: these dims need more than FLASHMHF_STATIC_SCRATCH_BYTES */
} flashmhf_status;

typedef enum flashmhf_dtype {
    FLASHMHF_BF16 = 0,      /* Q,K,U,V,O,dO,dQ,dK,dU,dV bfloat16; tensor-core (tcgen05) kernels, fp32 accumulation */
    FLASHMHF_F32_CHECK = 1  /* the same tensors float32; CUDA-core check kernels, fp32 throughout (test mode) */
} flashmhf_dtype;

/* A 4-D tensor whose innermost dimension is contiguous.  stride[i] is the ELEMENT stride of outer
 * dimension i (for Q: B, H, S; for K: H_kuv, E, d_e; for R: B, H, S).  For the bf16 path every
 * stride must be a multiple of 8 elements (16 bytes) and the pointer 16-byte aligned; for K/U/V
 * (and dK/dU/dV) stride[1] must equal d_e * stride[2] so that (E, d_e) is one row index. */
typedef struct flashmhf_tensor {
    void *ptr;
    int64_t stride[3];
} flashmhf_tensor;

typedef struct flashmhf_dims {
    int32_t B, H, S, Dh;      /* batch, FFN heads, sequence length, head dim */
    int32_t Hkuv, E, De;      /* K/U/V heads, sub-networks per head, rows per sub-network */
    int32_t dtype;            /* flashmhf_dtype */
} flashmhf_dims;

/* The three constants of the reference's eager loop (models/flashmhf/modeling_mhffnmoe.py:270-279, 420-425):
 *   O = sum_e R_e * final_scaling * ((SiLU(head_scaling * Q K_e^T) * (up_scaling * Q U_e^T)) V_e).
 * Each must be finite and non-zero (else FLASHMHF_ERR_BAD_SHAPE); the layer uses head_scaling = up_scaling in
 * {1, sqrt(H), H} and final_scaling in {1, sqrt(3/8)}. */
typedef struct flashmhf_scaling {
    float head_scaling, up_scaling, final_scaling;
} flashmhf_scaling;

/* flashmhf_bwd_params.parts: which gradients a backward call produces.  Data-parallel training calls the
 * weights part first, starts the all-reduce of dK, dU, dV, and runs the inputs part under it. */
#define FLASHMHF_BWD_INPUTS 1u   /* dQ and dR (dK, dU, dV, workspace may then be left unset) */
#define FLASHMHF_BWD_WEIGHTS 2u  /* dK, dU and dV (dQ, dR may then be left unset) */

typedef struct flashmhf_fwd_params {
    flashmhf_dims d;
    flashmhf_tensor Q, K, U, V, R; /* inputs */
    flashmhf_tensor O;             /* output, every element written; no pre-zeroing needed */
    void *workspace;               /* device scratch, 256-byte aligned; needed only when                 */
    size_t workspace_bytes;        /* flashmhf_forward_workspace_bytes() > 0 (short token counts), else NULL/0 */
    flashmhf_scaling scale;        /* the eager layer's three constants; {1,1,1} for every shipped configuration */
} flashmhf_fwd_params;

typedef struct flashmhf_bwd_params {
    flashmhf_dims d;
    flashmhf_tensor Q, K, U, V, R, dO; /* inputs (dO may be a transposed view, like any other tensor here) */
    flashmhf_tensor dQ, dK, dU, dV, dR; /* outputs, every element written; dR is fp32 */
    void *workspace;                    /* device scratch, 256-byte aligned, contents undefined on entry and exit */
    size_t workspace_bytes;
    flashmhf_scaling scale;             /* as in the forward call */
    uint32_t parts;                     /* 0 = everything; else a mask of FLASHMHF_BWD_INPUTS | FLASHMHF_BWD_WEIGHTS */
} flashmhf_bwd_params;

/* ABI version of the loaded library (== FLASHMHF_ABI_VERSION of the header it was built from).
 * Reference counterpart: none (pybind modules carry no version). */
int flashmhf_abi_version(void);

/* Static, NUL-terminated description of a status code.
 * Reference counterpart: the TORCH_CHECK / CHECK_CUDA_ERROR messages, flash_ffn_moe.cu:940-960, 1006. */
const char *flashmhf_strerror(int status);

/* Text of the last CUDA error this thread's calls met (valid until the next failing call). */
const char *flashmhf_last_cuda_error(void);

/* Forward.  Enqueues on `stream` (a cudaStream_t; NULL = legacy default stream) of the CURRENT
 * device and returns.  Replaces flashffn_moe_forward, flash_ffn_moe.cu:938-1007, and the launch at
 * kernels/triton/flash_mlp_moe.py:777-790. */
int flashmhf_forward(const flashmhf_fwd_params *p, void *stream);

/* Forward for back-to-back calls over constant weights (a decode loop: the O of one layer's call becomes, a few small
 * kernels later, the Q of the next).  Same arguments, same results (bit for bit) as flashmhf_forward; bf16 only.  Its
 * kernels are launched with programmatic stream serialization: they may become resident while the operation before
 * them on the stream is still running, and the forward kernel streams K, U, V tiles in meanwhile; Q and R are read, and
 * O and the workspace written, only after that operation has completed.  Between two such calls the GPU therefore
 * never waits for a launch, and the second call's first weight tiles are in shared memory when its Q arrives.
 * The caller promises that K, U and V are not written by the operation directly before this call on the stream.
 * Capturable in a CUDA graph.  Reference counterpart: the same launches as flashmhf_forward
 * (flash_ffn_moe.cu:938-1007), which the reference issues in plain stream order. */
int flashmhf_forward_chained(const flashmhf_fwd_params *p, void *stream);

/* Bytes of scratch flashmhf_forward needs for these dims.  0 unless there are fewer token tiles
 * (ceil(S/128) * H * B) than about half the SMs -- the decode-shaped case (reference: batched decode
 * through the same call, models/flashmhf/modeling_mhffnmoe.py:406-408) -- where the intermediate
 * dimension is split over CTAs and fp32 partial outputs are summed in a fixed order.  Pure host
 * arithmetic.  Reference counterpart: none. */
size_t flashmhf_forward_workspace_bytes(const flashmhf_dims *d);

/* Bytes of scratch flashmhf_backward needs for these dims (0 is possible).  Pure host arithmetic. */
size_t flashmhf_backward_workspace_bytes(const flashmhf_dims *d);

/* Backward: dQ, dK, dU, dV, dR from dO, recomputing the intermediate.  Enqueues on `stream` and
 * returns.  Deterministic (no floating-point atomics).  Replaces flashffn_moe_backward,
 * flash_ffn_moe.cu:1012-1133, and the two launches at kernels/triton/flash_mlp_moe.py:832-866. */
int flashmhf_backward(const flashmhf_bwd_params *p, void *stream);

/* Size of the scratch array built into the library for flashmhf_backward_static_scratch: 72 MiB
 * (enough for the 370M layer shape, H_kuv=8, E*d_e=2816, d_h=128, with its two-way token split). */
#define FLASHMHF_STATIC_SCRATCH_BYTES (72u << 20)

/* Backward for callers that cannot hand over a workspace and must not trigger an allocation: a host
 * runtime that gave all device memory to its own planner at start-up (so a cudaMalloc would fail or
 * stall -- cudaMalloc and cudaFree synchronise the whole device), or one that binds this ABI over
 * an FFI and has no device allocator to offer.  Same kernels, same results and same argument rules
 * as flashmhf_backward, but `workspace` / `workspace_bytes` are ignored: the partial sums of dK, dU
 * and dV go to a static array inside the library (FLASHMHF_STATIC_SCRATCH_BYTES per GPU that loads
 * the library, held until the process exits).  The caller still passes every input and output.
 *   - bf16 only.  Dims whose flashmhf_backward_workspace_bytes() exceeds the array are refused
 *     with FLASHMHF_ERR_SCRATCH_LIMIT; nothing is launched.
 *   - The call makes no cudaMalloc, cudaFree or other allocating call.  Its FIRST call on a device
 *     looks up the array's device address (once per device, with that device current).
 *   - All calls on a device share the one array and it keeps the previous call's contents.  The
 *     kernels overwrite everything they later read, so stale contents are harmless, but two calls
 *     whose kernels overlap on the GPU (different streams, no ordering between them) race on it:
 *     order them, or use flashmhf_backward with separate workspaces.
 *   - Make the first call on each device outside any stream capture (the address look-up is not a
 *     stream operation).  The address is cached per device ordinal for the life of the process and is
 *     not refreshed after a cudaDeviceReset(): do not reset a device this library has been used on.
 * This entry point has no counterpart in the reference. */
int flashmhf_backward_static_scratch(const flashmhf_bwd_params *p, void *stream);

/* ---- Fused layer prologue (optional companion of the operator) ------------------------------
 * What the reference layer does between its first projection and the operator, in one kernel
 * (models/flashmhf/modeling_mhffnmoe.py:362-386; per-head RMSNorm :116-135):
 *   X [B,S,H,d_h] bf16 (token stride x_token_stride >= H*d_h elements)
 *     -> Q = bf16(RMSNorm_h(X) * norm_weight[h,:])  written at the same offsets as X, i.e. in [B,S,H,d_h]
 *        layout (skipped when norm_weight is NULL: then Q is X itself); the operator reads it in place
 *        through flashmhf_tensor strides (B: S*x_token_stride, H: d_h, S: x_token_stride), no transposing copy
 *     -> R [B,H,S,E] fp32 = sigmoid(float(Q) . router[h]) normalised over E (denominator clamped at 1e-20)
 * d_h in {64, 96, 128}, E <= 32.  norm_weight [H,d_h] and router [H,d_h,E] are fp32. */
typedef struct flashmhf_prologue_params {
    int32_t B, S, H, Dh, E;
    float eps;
    const void *X;
    int64_t x_token_stride;
    const float *norm_weight; /* NULL = no RMSNorm */
    const float *router;
    void *Q;                  /* bf16, same layout as X; ignored when norm_weight is NULL */
    float *R;
} flashmhf_prologue_params;

typedef struct flashmhf_prologue_bwd_params {
    flashmhf_prologue_params fwd; /* X, norm_weight, router as in the forward call (Q, R unused) */
    const void *dQ;               /* bf16 gradient w.r.t. Q, logical [B,H,S,d_h] with element strides dq_stride (B,H,S) */
    int64_t dq_stride[3];
    const float *dR;              /* [B,H,S,E] contiguous */
    void *dX;                     /* out, bf16, same layout as X */
    float *d_router;              /* out, [H,d_h,E] */
    float *d_norm_weight;         /* out, [H,d_h]; ignored when norm_weight is NULL */
    void *workspace;              /* flashmhf_prologue_backward_workspace_bytes(), 256-byte aligned */
    size_t workspace_bytes;
} flashmhf_prologue_bwd_params;

/* Replaces modeling_mhffnmoe.py:362-386 (forward) and its autograd (backward).  Enqueue and return. */
int flashmhf_prologue_forward(const flashmhf_prologue_params *p, void *stream);
size_t flashmhf_prologue_backward_workspace_bytes(const flashmhf_prologue_params *p);
int flashmhf_prologue_backward(const flashmhf_prologue_bwd_params *p, void *stream);

/* ---- Helpers for the measurement LM (flashmhf_b200/lm.py), outside the operator -------------------
 * Rotary position embedding on [tokens, heads, head_dim] bf16 (token strides in elements, multiples of 8):
 *   y[..., :h] = x[..., :h] cos - x[..., h:] sin ;  y[..., h:] = x[..., h:] cos + x[..., :h] sin,  h = head_dim/2,
 * with cos_t, sin_t fp32 [S, h] and the position of token t being t % S; transpose != 0 applies the transposed
 * rotation (the backward).  Replaces modeling_mhffnmoe.py:178-206 (apply_rotary_pos_emb).  x == y is allowed. */
int flashmhf_lm_rope(const void *x, void *y, const float *cos_t, const float *sin_t, int64_t tokens, int32_t S,
                     int32_t heads, int32_t head_dim, int64_t x_token_stride, int64_t y_token_stride, int32_t transpose,
                     void *stream);

/* RMSNorm over contiguous rows of n in {768, 1024, 2048} bf16 elements with an fp32 weight [n]:
 * y = x * rsqrt(mean(x^2) + eps) * w (fp32 arithmetic, one rounding).  Replaces modeling_mhffnmoe.py:82-87.
 * Backward: dx (bf16) and dw (fp32 [n]) from x, w and the gradient g; workspace of
 * flashmhf_lm_rmsnorm_backward_workspace_bytes(rows, n) bytes, 16-byte aligned; deterministic. */
int flashmhf_lm_rmsnorm_forward(const void *x, const float *w, void *y, int64_t rows, int32_t n, float eps, void *stream);
size_t flashmhf_lm_rmsnorm_backward_workspace_bytes(int64_t rows, int32_t n);
int flashmhf_lm_rmsnorm_backward(const void *x, const float *w, const void *g, void *dx, float *dw, void *workspace,
                                 size_t workspace_bytes, int64_t rows, int32_t n, float eps, void *stream);

/* SYNCHRONOUS.  Waits for the current device, then reads and clears the status word the kernels
 * write when a bounded wait runs out.  *code = 0 if none did; otherwise a kernel/role identifier
 * (kernel * 100 + wait), and the call returns FLASHMHF_ERR_DEVICE_TIMEOUT.
 * Semantics of a run-out wait: every mbarrier wait in the kernels is bounded (about 1.5 s); the launch
 * whose wait ran out returns early through its normal teardown and leaves its outputs UNWRITTEN, its
 * remaining CTAs drain at once, and the first code is kept in the word until this call reads it.  Later
 * launches are not affected: they run normally whether or not the word has been read.  Because the
 * entry points only enqueue work they cannot report the condition themselves; call this wherever the
 * host already synchronises (after reading back a loss, at the end of a step).
 * Reference counterpart: none. */
int flashmhf_device_status(int *code);

/* Self-test of the bounded-wait path: one small kernel waits, for at most `limit_cycles` SM clock
 * cycles, on a barrier that nothing ever arrives at, records code 9901 in the status word and returns
 * through the same teardown the operator kernels use.  Nothing faults or hangs; the next
 * flashmhf_device_status() reports FLASHMHF_ERR_DEVICE_TIMEOUT with that code.  Reference counterpart: none. */
int flashmhf_selftest_bounded_wait(long long limit_cycles, void *stream);

/* Profiling aid.  Between flashmhf_profile_begin and flashmhf_profile_end every forward/backward
 * call records a CUDA event on its stream before its first kernel and after each kernel (no
 * synchronisation, up to `max_marks` events in total).  flashmhf_profile_end is SYNCHRONOUS: it
 * waits for the device and returns, for each kernel launched in between, its duration in
 * milliseconds and a tag (1 forward, 2 backward dQ/dR, 3 backward dK/dU/dV, 4 backward split
 * reductions, 5 forward split reduction, 6 prologue forward, 7 prologue backward, 8 its reductions).
 * One profiling session at a time, calls from one stream.  Reference counterpart: none. */
int flashmhf_profile_begin(int max_marks);
int flashmhf_profile_end(float *ms, int *tags, int capacity, int *n_out);

/* Number of kernel launches this library has enqueued since it was loaded (all threads). */
uint64_t flashmhf_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* FLASHMHF_H_ */
