"""Host side of the operator: torch tensors in, C-ABI calls out.

``flash_mhf(Q, K, U, V, R)`` has the call signature of the reference's
``FlashMLPFunction.apply`` (kernels/triton/flash_mlp_moe.py:739-868) and of its ThunderKittens
twin (kernels/thunderkittens/flash_ffn_moe_torch.py:5-24): it saves the five inputs, keeps no
intermediate, and recomputes in backward.  PyTorch supplies device memory and the current stream;
all arithmetic runs in the CUDA library."""
import ctypes as C
import threading

import torch

from . import _lib

_DT = {torch.bfloat16: _lib.BF16, torch.float32: _lib.F32_CHECK}


def _tensor(t):
    s = t.stride()
    return _lib.Tensor(t.data_ptr(), (s[0], s[1], s[2]))


class _on_device:
    """`with torch.cuda.device(dev)` only when `dev` is not the current device already (the context manager costs
    several microseconds a call, which matters for decode-shaped calls)."""

    def __init__(self, dev):
        self.ctx = None if dev.index is None or dev.index == torch.cuda.current_device() else torch.cuda.device(dev)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *a):
        if self.ctx is not None:
            self.ctx.__exit__(*a)


def _strided_ok(t, is_weight, de):
    """Can the library address this tensor in place? (unit inner stride, 16-byte aligned outer strides, E/d_e collapse)"""
    if t.stride(-1) != 1 and t.size(-1) != 1:
        return False
    if t.data_ptr() % 16:
        return False
    if t.dtype == torch.bfloat16:
        for i in range(3):
            if t.size(i) > 1 and (t.stride(i) % 8 or t.stride(i) <= 0):
                return False
    if is_weight and t.size(1) > 1 and t.stride(1) != de * t.stride(2):
        return False
    return True


def _prep(t, is_weight=False, de=0):
    return t if _strided_ok(t, is_weight, de) else t.contiguous()


def _validate(Q, K, U, V, R):
    if Q.dim() != 4 or K.dim() != 4 or R.dim() != 4:
        raise ValueError("expected Q [B,H,S,d_h], K/U/V [H_kuv,E,d_e,d_h], R [B,H,S,E]")
    B, H, S, dh = Q.shape
    hk, E, de, dh2 = K.shape
    if de % 64 != 0:
        raise ValueError(f"Expert dimension {de} must be divisible by 64")
    if U.shape != K.shape or V.shape != K.shape or dh2 != dh:
        raise ValueError(f"K/U/V shapes must agree and end in d_h={dh}: {tuple(K.shape)}, {tuple(U.shape)}, {tuple(V.shape)}")
    if hk < 1 or H % hk != 0:
        raise ValueError(f"num_heads {H} must be a multiple of num_kuv_heads {hk}")
    if tuple(R.shape) != (B, H, S, E):
        raise ValueError(f"R must be {(B, H, S, E)}, got {tuple(R.shape)}")
    if dh not in (64, 96, 128):
        raise ValueError(f"head_dim {dh} not supported (64, 96 or 128)")
    if Q.dtype not in _DT or any(t.dtype != Q.dtype for t in (K, U, V)):
        raise TypeError("flash_mhf expects Q, K, U, V all in torch.bfloat16 (or all float32 for the check mode), got"
                        f" Q={Q.dtype}, K={K.dtype}, V={V.dtype}, U={U.dtype}")
    if not Q.is_cuda or any(t.device != Q.device for t in (K, U, V, R)):
        raise ValueError("flash_mhf runs on CUDA tensors of one device; there is no CPU path")
    return B, H, S, dh, hk, E, de


def _dims(B, H, S, dh, hk, E, de, dtype):
    return _lib.Dims(B, H, S, dh, hk, E, de, _DT[dtype])


def _scaling(scaling):
    """(head_scaling, up_scaling, final_scaling) of the eager layer (modeling_mhffnmoe.py:270-279) -> C struct."""
    hs, us, fs = (float(v) for v in scaling)
    for v in (hs, us, fs):
        if v == 0.0 or v != v or v in (float("inf"), float("-inf")):
            raise ValueError(f"scaling constants must be finite and non-zero, got {tuple(scaling)}")
    return _lib.Scaling(hs, us, fs)


def _routing(R):
    """R as the kernels read it: fp32, unit inner stride, 4-byte aligned (any outer strides)."""
    R = R.to(torch.float32)
    return R if R.stride(-1) == 1 or R.size(-1) == 1 else R.contiguous()


def _tokens_as_sequence(*ts):
    """Decode-shaped call (S == 1, B > 1): view [B,H,1,X] tensors as [1,H,B,X] -- a pure permutation, no copy --
    so that the B token rows share tiles instead of occupying one 128-row tile each."""
    return [t.permute(2, 1, 0, 3) for t in ts]


class _FwdPlan:
    """What a forward call over tensors of given shapes, strides, dtypes and alignment needs, worked out once: the
    parameter struct (strides, dims, scaling filled in; the five data pointers are set per call), the scratch size, and
    whether a decode-shaped call is passed as one sequence."""
    __slots__ = ("params", "ref", "ws_bytes", "call")


class _PlanCache(threading.local):
    """Per thread (a plan's parameter struct is written into on every call)."""

    def __init__(self):
        self.plans = {}


_fwd_plans = _PlanCache()
_MAX_PLANS = 256


def _fwd_key(Q, K, U, V, R, out, scaling, chained):
    return (Q.shape, Q.stride(), Q.dtype, Q.device, Q.data_ptr() & 15,
            K.shape, K.stride(), K.dtype, K.device, K.data_ptr() & 15,
            U.shape, U.stride(), U.dtype, U.device, U.data_ptr() & 15,
            V.shape, V.stride(), V.dtype, V.device, V.data_ptr() & 15,
            R.shape, R.stride(), R.dtype, R.device, R.data_ptr() & 3,
            None if out is None else (out.shape, out.stride(), out.dtype, out.device, out.data_ptr() & 15),
            scaling if type(scaling) is tuple else tuple(scaling), chained)


def forward_raw(Q, K, U, V, R, out=None, scaling=_lib.NO_SCALING, chained=False, workspace=None):
    """O = flashmhf_forward(...) on the current stream; no autograd.

    ``chained``: use ``flashmhf_forward_chained`` -- for back-to-back calls over constant weights (a decode loop,
    usually replayed from a CUDA graph): the call may start, and stream in its first weight tiles, while the kernel
    before it on the stream still runs.  The caller promises that K, U, V are not written by the operation directly
    before the call.  Same result, bit for bit.
    ``workspace``: optional uint8 tensor to use as the call's scratch (at least ``flashmhf_forward_workspace_bytes``).

    The checks and the layout decisions depend only on shapes, strides, dtypes, devices and pointer alignment; they are
    made once per such combination and remembered (per thread), so that a repeated call costs little more than filling
    in five pointers -- a decode-shaped call lasts some twenty microseconds on the GPU."""
    key = _fwd_key(Q, K, U, V, R, out, scaling, chained)
    plan = _fwd_plans.plans.get(key)
    if plan is None:
        return _forward_first(key, Q, K, U, V, R, out, scaling, chained, workspace)
    O = torch.empty_like(Q) if out is None else out
    p = plan.params
    p.Q.ptr, p.K.ptr, p.U.ptr, p.V.ptr, p.R.ptr, p.O.ptr = (Q.data_ptr(), K.data_ptr(), U.data_ptr(), V.data_ptr(),
                                                            R.data_ptr(), O.data_ptr())
    ws = None
    if plan.ws_bytes:
        ws = _scratch(workspace, plan.ws_bytes, Q.device)
        p.workspace = ws.data_ptr()
    with _on_device(Q.device):
        _lib.check(plan.call(plan.ref, torch.cuda.current_stream().cuda_stream))
    return O


def _scratch(workspace, nbytes, device):
    if workspace is None:
        return torch.empty(nbytes, dtype=torch.uint8, device=device)
    if workspace.device != device or workspace.dtype != torch.uint8 or workspace.numel() < nbytes or \
            workspace.data_ptr() % 256:
        raise ValueError(f"workspace must be a 256-byte aligned uint8 tensor of at least {nbytes} bytes on {device}")
    return workspace


def _forward_first(key, Q0, K0, U0, V0, R0, out, scaling, chained, workspace):
    """The full path: validate, copy what the library cannot address in place, call; remember the plan when the call
    needed no copy (then the same key always leads to the same parameter struct)."""
    B, H, S, dh, hk, E, de = _validate(Q0, K0, U0, V0, R0)
    lib = _lib.load()
    sc = _scaling(scaling)
    Q, K, U, V = _prep(Q0), _prep(K0, True, de), _prep(U0, True, de), _prep(V0, True, de)
    R = _routing(R0)
    O = torch.empty_like(Q) if out is None else out  # keeps Q's memory layout ([B,H,S,d] or [B,S,H,d])
    Qk, Rk, Ok = Q, R, O
    if S == 1 and B > 1:
        Qk, Rk, Ok = _tokens_as_sequence(Q, R, O)
        if all(_strided_ok(t, False, 0) for t in (Qk, Ok)):
            B, S = 1, B
        else:
            Qk, Rk, Ok = Q, R, O
    d = _dims(B, H, S, dh, hk, E, de, Q.dtype)
    nbytes = int(lib.flashmhf_forward_workspace_bytes(C.byref(d)))
    ws = _scratch(workspace, nbytes, Q.device) if nbytes else None
    p = _lib.FwdParams(d, _tensor(Qk), _tensor(K), _tensor(U), _tensor(V), _tensor(Rk), _tensor(Ok),
                       ws.data_ptr() if nbytes else None, nbytes, sc)
    call = lib.flashmhf_forward_chained if chained else lib.flashmhf_forward
    ref = C.byref(p)
    with _on_device(Q.device):
        _lib.check(call(ref, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    in_place = all(a is b for a, b in ((Q, Q0), (K, K0), (U, U0), (V, V0), (R, R0)))
    if in_place and len(_fwd_plans.plans) < _MAX_PLANS:
        plan = _FwdPlan()
        plan.params, plan.ref, plan.ws_bytes, plan.call = p, ref, nbytes, call
        _fwd_plans.plans[key] = plan
    return O


def backward_raw(Q, K, U, V, R, dO, scaling=_lib.NO_SCALING, parts="all", weight_grads=None):
    """(dQ, dK, dU, dV, dR) = flashmhf_backward(...) on the current stream; no autograd.

    ``parts``: "all", or "weights" (dK, dU, dV only; dQ and dR come back as None) or "inputs" (the reverse) --
    data-parallel training runs the weights part first and overlaps its all-reduce with the inputs part.
    ``weight_grads``: optional (dK, dU, dV) tensors to write into (e.g. three views of one all-reduce bucket)."""
    B, H, S, dh, hk, E, de = _validate(Q, K, U, V, R)
    if dO.shape != Q.shape:
        raise AssertionError("grad_output shape should be the same as Q")
    if parts not in ("all", "weights", "inputs"):
        raise ValueError(f"parts must be 'all', 'weights' or 'inputs', got {parts!r}")
    lib = _lib.load()
    sc = _scaling(scaling)
    Q, K, U, V = _prep(Q), _prep(K, True, de), _prep(U, True, de), _prep(V, True, de)
    dO = _prep(dO.to(Q.dtype))
    R = _routing(R)
    none = _lib.Tensor(None, (0, 0, 0))
    dQ = dR = dK = dU = dV = None
    tQ = tR = tK = tU = tV = none
    ws_ptr, nbytes = None, 0
    d = _dims(B, H, S, dh, hk, E, de, Q.dtype)
    if parts != "weights":
        dQ = torch.empty_like(Q)  # keeps Q's memory layout
        dR = torch.empty((B, H, S, E), dtype=torch.float32, device=Q.device)
        tQ, tR = _tensor(dQ), _tensor(dR)
    if parts != "inputs":
        if weight_grads is not None:
            dK, dU, dV = weight_grads
            for g, w in ((dK, K), (dU, U), (dV, V)):
                if g.shape != w.shape or g.dtype != w.dtype or g.device != w.device:
                    raise ValueError("weight_grads must match K, U, V in shape, dtype and device")
        else:
            # in the weights' own memory layout (the layer passes strided views of [I, H_kuv*d_h] parameters: their
            # gradients then need no re-layout copy); the fp32 check kernels write contiguous outputs
            fmt = torch.preserve_format if Q.dtype == torch.bfloat16 else torch.contiguous_format
            dK, dU, dV = (torch.empty_like(t, memory_format=fmt) for t in (K, U, V))
        tK, tU, tV = _tensor(dK), _tensor(dU), _tensor(dV)
        nbytes = int(lib.flashmhf_backward_workspace_bytes(C.byref(d)))
        ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=Q.device)
        ws_ptr = ws.data_ptr()
    mask = {"all": 0, "inputs": _lib.BWD_INPUTS, "weights": _lib.BWD_WEIGHTS}[parts]
    p = _lib.BwdParams(d, _tensor(Q), _tensor(K), _tensor(U), _tensor(V), _tensor(R), _tensor(dO), tQ, tK, tU, tV, tR,
                       ws_ptr, nbytes, sc, mask)
    with _on_device(Q.device):
        _lib.check(lib.flashmhf_backward(C.byref(p), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return dQ, dK, dU, dV, dR


class FlashMHFFunction(torch.autograd.Function):
    """forward(ctx, Q, K, U, V, R[, head_scaling, up_scaling, final_scaling]) -> O ;
    backward(ctx, dO) -> dQ, dK, dU, dV, dR (and None for the three constants).

    The constants are those of the reference's eager loop (models/flashmhf/modeling_mhffnmoe.py:270-279, 420-425);
    its own flash path has none (kernels/triton/flash_mlp_moe.py:741), which is the default of 1."""

    @staticmethod
    def forward(ctx, Q, K, U, V, R, head_scaling=1.0, up_scaling=1.0, final_scaling=1.0):
        ctx.scaling = (float(head_scaling), float(up_scaling), float(final_scaling))
        O = forward_raw(Q, K, U, V, R, scaling=ctx.scaling)
        ctx.save_for_backward(Q, K, U, V, R)
        return O

    @staticmethod
    def backward(ctx, grad_output):
        Q, K, U, V, R = ctx.saved_tensors
        dQ, dK, dU, dV, dR = backward_raw(Q, K, U, V, R, grad_output, scaling=ctx.scaling)
        return dQ, dK, dU, dV, dR.to(R.dtype), None, None, None


def flash_mhf(Q, K, U, V, R, head_scaling=1.0, up_scaling=1.0, final_scaling=1.0):
    return FlashMHFFunction.apply(Q, K, U, V, R, head_scaling, up_scaling, final_scaling)


def check_device_status():
    """Synchronise and raise FlashMHFError if a kernel of this library gave up on a bounded wait (its outputs are then
    unwritten).  The entry points only enqueue work, so this is the place a host loop learns of it: call it where the
    loop synchronises anyway (after the loss is read back, at the end of a step)."""
    _lib.device_status()
