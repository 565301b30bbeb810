"""The FFN layer around the operator, with the fused prologue.

``fused_prologue`` replaces what the reference layer does between its first projection and the
operator (models/flashmhf/modeling_mhffnmoe.py:362-386): head split, per-head RMSNorm, the
transposing copy of Q, and the router weights.  One CUDA kernel reads the projected activations
in their own [B,S,H,d_h] layout and writes the normalised Q in the same layout plus R; the operator
then reads Q in place through strides and writes O in that layout too, so the two
``transpose(1,2).contiguous()`` copies of the reference (modeling:374, 408) vanish.

``mhffn_layer`` is the whole layer (modeling:352-431) built from it; parameter names and shapes are the
reference's (w_self, w_self_2 [hid,hid]; gate/up/down_weight [I, H_kuv*d_h]; router [H,d_h,E];
q_norm [H,d_h]) so its state dicts load."""
import ctypes as C

import torch
import torch.nn.functional as F

from . import _lib
from .functional import flash_mhf


class FusedPrologueFunction(torch.autograd.Function):
    """(x_proj [B,S,H*d_h] bf16, q_norm [H,d_h] or None, router [H,d_h,E]) -> (Q [B,H,S,d_h] view, R [B,H,S,E] fp32)."""

    @staticmethod
    def forward(ctx, x_proj, q_norm, router, eps):
        if x_proj.dtype != torch.bfloat16 or not x_proj.is_cuda:
            raise TypeError("fused_prologue expects a CUDA bfloat16 activation tensor")
        H, dh, E = router.shape
        B, S, hid = x_proj.shape
        if hid != H * dh:
            raise ValueError(f"hidden size {hid} != H*d_h = {H}*{dh}")
        if dh not in (64, 96, 128) or E > 32:
            raise ValueError("fused_prologue supports d_h in {64, 96, 128} and at most 32 sub-networks")
        lib = _lib.load()
        x = x_proj.contiguous()
        w = None if q_norm is None else q_norm.detach().to(torch.float32).contiguous()
        r = router.detach().to(torch.float32).contiguous()
        q = torch.empty_like(x) if w is not None else x
        R = torch.empty(B, H, S, E, dtype=torch.float32, device=x.device)
        p = _lib.PrologueParams(B, S, H, dh, E, float(eps), x.data_ptr(), H * dh, None if w is None else w.data_ptr(),
                                r.data_ptr(), q.data_ptr(), R.data_ptr())
        with torch.cuda.device(x.device):
            _lib.check(lib.flashmhf_prologue_forward(C.byref(p), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        ctx.save_for_backward(x, w if w is not None else x.new_empty(0), r)
        ctx.has_norm, ctx.eps, ctx.dims = w is not None, float(eps), (B, S, H, dh, E)
        ctx.norm_dtype = None if q_norm is None else q_norm.dtype
        ctx.router_dtype = router.dtype
        return q.view(B, S, H, dh).transpose(1, 2), R

    @staticmethod
    def backward(ctx, dQ, dR):
        x, w, r = ctx.saved_tensors
        B, S, H, dh, E = ctx.dims
        lib = _lib.load()
        if dQ is None:
            dQ = torch.zeros(B, H, S, dh, dtype=torch.bfloat16, device=x.device)
        if dR is None:
            dR = torch.zeros(B, H, S, E, dtype=torch.float32, device=x.device)
        dQ = dQ.to(torch.bfloat16)
        if dQ.stride(-1) != 1:
            dQ = dQ.contiguous()
        dR = dR.to(torch.float32).contiguous()
        dX = torch.empty_like(x)
        d_router = torch.empty_like(r)
        d_norm = torch.empty_like(w) if ctx.has_norm else None
        fwd = _lib.PrologueParams(B, S, H, dh, E, ctx.eps, x.data_ptr(), H * dh, w.data_ptr() if ctx.has_norm else None,
                                  r.data_ptr(), None, None)
        nbytes = int(lib.flashmhf_prologue_backward_workspace_bytes(C.byref(fwd)))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        p = _lib.PrologueBwdParams(fwd, dQ.data_ptr(), (C.c_int64 * 3)(*dQ.stride()[:3]), dR.data_ptr(), dX.data_ptr(),
                                   d_router.data_ptr(), d_norm.data_ptr() if ctx.has_norm else None, ws.data_ptr(), nbytes)
        with torch.cuda.device(x.device):
            _lib.check(lib.flashmhf_prologue_backward(C.byref(p), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return (dX, d_norm.to(ctx.norm_dtype) if ctx.has_norm else None, d_router.to(ctx.router_dtype), None)


def fused_prologue(x_proj, q_norm, router, eps=1e-5):
    return FusedPrologueFunction.apply(x_proj, q_norm, router, eps)


def torch_prologue(x_proj, q_norm, router, eps=1e-5):
    """The same two results from library element-wise kernels, for router shapes the fused kernels do not take (more
    than 32 sub-networks per head): per-head RMSNorm in fp32, Q as a [B,H,S,d_h] view, R = normalised sigmoid."""
    H, dh, _ = router.shape
    B, S, _ = x_proj.shape
    q = x_proj.view(B, S, H, dh)
    if q_norm is not None:
        qf = q.float()
        q = (qf * torch.rsqrt(qf.pow(2).mean(-1, keepdim=True) + eps) * q_norm.float()[None, None]).to(x_proj.dtype)
    Q = q.transpose(1, 2)
    R = (Q.float() @ router.float()).sigmoid()
    return Q, R / R.sum(dim=-1, keepdim=True).clamp(min=1e-20)


def expert_views(gate_weight, up_weight, down_weight, Hkuv, E):
    """[I, H_kuv*d_h] parameters -> [H_kuv, E, d_e, d_h] strided views the operator reads in place (no copy)."""
    I = gate_weight.shape[0]
    dh = gate_weight.shape[1] // Hkuv
    f = lambda w: w.view(E, I // E, Hkuv, dh).permute(2, 0, 1, 3)
    return f(gate_weight), f(up_weight), f(down_weight)


def mhffn_layer(x, p, *, H, Hkuv, E, apply_rmsnorm, eps=1e-5, head_scaling=1.0, up_scaling=1.0, final_scaling=1.0):
    """y = w_self_2(op(prologue(w_self(x)))) for bf16 CUDA tensors; p holds the reference's parameter names
    (optionally ``w_self_bias`` / ``w_self_2_bias``, the biases the reference creates with config.mlp_bias).
    The three constants are the eager layer's (models/flashmhf/modeling_mhffnmoe.py:270-279); every shipped
    configuration leaves them at 1."""
    B, S, hid = x.shape
    q_lin = F.linear(x, p["w_self"], p.get("w_self_bias")) if p.get("w_self") is not None else x
    prologue = fused_prologue if E <= 32 else torch_prologue
    Q, R = prologue(q_lin, p["q_norm"] if apply_rmsnorm else None, p["router"], eps)
    K, U, V = expert_views(p["gate_weight"], p["up_weight"], p["down_weight"], Hkuv, E)
    O = flash_mhf(Q, K, U, V, R, head_scaling, up_scaling, final_scaling)  # [B,H,S,d_h] view of [B,S,H,d_h] memory
    O = O.transpose(1, 2).reshape(B, S, hid)          # no copy when O kept Q's layout
    return F.linear(O, p["w_self_2"], p.get("w_self_2_bias")) if p.get("w_self_2") is not None else O
