"""CPU oracle for the FlashMHF multi-head FFN operator.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the arithmetic of the reference's eager
("naive MH-FFN") path and of its documented backward.  It is the checker the CUDA path is
compared with; nothing in the product package imports it.  Only the tests, the smoke entry and
the benchmark's CPU-baseline leg may call it.

Parity pin: the restatement is checked against outputs of the reference's own
``MHFFNMoEMultiHeadFFNFlash(cfg, use_flash=False)`` layer, captured on seeded inputs by
``tests/golden/make_golden.py`` and committed as fixtures under ``tests/golden/``.  The reference
holds no golden vectors of its own for this path, so those fixtures are the pin.

What each function follows (paths inside the reference project):

* ``mhffn_forward``      models/flashmhf/modeling_mhffnmoe.py:412-427 (eager expert loop) and
                         kernels/thunderkittens/run_from_python.py:19-24 (inline ground truth)
* ``repeat_kuv``         models/flashmhf/modeling_mhffnmoe.py:224-253
* ``mhffn_backward``     kernels/triton/flash_mlp_moe.py:384-414 (backward derivation) with the
                         routing weight folded in as in flash_mlp_moe.py:527-540
* ``router_weights``     models/flashmhf/modeling_mhffnmoe.py:384-386
* ``multihead_rmsnorm``  models/flashmhf/modeling_mhffnmoe.py:116-135
* ``mhffn_layer_forward`` models/flashmhf/modeling_mhffnmoe.py:352-431
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def repeat_kuv(w: torch.Tensor, n_rep: int) -> torch.Tensor:
    """[H_kuv, E, d_e, d_h] -> [H_kuv * n_rep, E, d_e, d_h], each K/U/V head repeated n_rep times in place."""
    if n_rep == 1:
        return w
    hk, e, de, dh = w.shape
    return w[:, None].expand(hk, n_rep, e, de, dh).reshape(hk * n_rep, e, de, dh)


def mhffn_forward(Q, K, U, V, R, *, out_dtype=None, head_scaling=1.0, up_scaling=1.0, final_scaling=1.0):
    """O = sum_e R_e * ((silu(Q K_e^T) * (Q U_e^T)) V_e), evaluated the way the eager layer does, including its
    three constants (modeling_mhffnmoe.py:270-279; applied at :420, :422, :425; 1 in every shipped configuration).

    Q [B,H,S,d_h]; K,U,V [H_kuv,E,d_e,d_h]; R [B,H,S,E].  Every matmul runs in the dtype of Q
    (so bf16 inputs round every intermediate to bf16, as the eager path does); the sum over
    experts is kept in fp32 (fp64 for fp64 inputs) and the routing weight is applied to the
    fp32 copy of each expert's output; the result is cast to ``out_dtype`` (default: Q's dtype).
    """
    B, H, S, dh = Q.shape
    hk, E, de, _ = K.shape
    g = H // hk
    K, U, V = repeat_kuv(K, g), repeat_kuv(U, g), repeat_kuv(V, g)
    acc_dtype = torch.float64 if Q.dtype == torch.float64 else torch.float32
    out = torch.zeros(Q.shape, dtype=acc_dtype, device=Q.device)
    for e in range(E):
        w = F.silu(Q @ K[:, e].transpose(1, 2) * head_scaling)
        w = w * (Q @ U[:, e].transpose(1, 2) * up_scaling)
        out += (w @ V[:, e] * final_scaling).to(acc_dtype) * R[..., e:e + 1].to(acc_dtype)
    return out.to(out_dtype if out_dtype is not None else Q.dtype)


def mhffn_backward(Q, K, U, V, R, dO, *, head_scaling=1.0, up_scaling=1.0, final_scaling=1.0):
    """Explicit gradients of ``mhffn_forward`` for upstream gradient dO; returns (dQ,dK,dU,dV,dR).
    With the constants s0, s1, s2 (head, up, final): M = s0 Q K^T, N = s1 Q U^T, dA = s2 dO V^T, and the
    chain rule hands s0 to dM, s1 to dN and s2 to the A that multiplies dO in dV.

    Per expert e with r = R[..., e]:  M = Q K_e^T, N = Q U_e^T, sg = sigmoid(M), s = M*sg,
    dA = dO V_e^T, dR_e = rowsum(dA*s*N), dM = dA*(r*N)*(sg + s*(1-sg)), dN = dA*s*r,
    dQ += dM K_e + dN U_e, dK_e = sum_t dM^T Q, dU_e = sum_t dN^T Q, dV_e = sum_t (s*N*r)^T dO.
    With grouped K/U/V heads (H_kuv < H) the weight gradients sum over the G query heads that
    share a weight head.  All arithmetic in the dtype of the inputs (use fp64/fp32 inputs).
    """
    B, H, S, dh = Q.shape
    hk, E, de, _ = K.shape
    g = H // hk
    Kr, Ur, Vr = repeat_kuv(K, g), repeat_kuv(U, g), repeat_kuv(V, g)
    dQ = torch.zeros_like(Q)
    dKr, dUr, dVr = torch.zeros_like(Kr), torch.zeros_like(Ur), torch.zeros_like(Vr)
    dR = torch.zeros(R.shape, dtype=Q.dtype, device=Q.device)
    for e in range(E):
        r = R[..., e:e + 1].to(Q.dtype)
        M = Q @ Kr[:, e].transpose(1, 2) * head_scaling
        N = Q @ Ur[:, e].transpose(1, 2) * up_scaling
        sg = torch.sigmoid(M)
        s = M * sg
        dA = dO @ Vr[:, e].transpose(1, 2) * final_scaling
        dR[..., e] = (dA * s * N).sum(-1)
        dM = dA * (r * N) * (sg + s * (1 - sg)) * head_scaling
        dN = dA * s * r * up_scaling
        dQ += dM @ Kr[:, e] + dN @ Ur[:, e]
        dKr[:, e] = (dM.transpose(2, 3) @ Q).sum(0)
        dUr[:, e] = (dN.transpose(2, 3) @ Q).sum(0)
        dVr[:, e] = ((s * N * r * final_scaling).transpose(2, 3) @ dO).sum(0)
    if g > 1:
        fold = lambda t: t.view(hk, g, E, de, dh).sum(1)
        dKr, dUr, dVr = fold(dKr), fold(dUr), fold(dVr)
    return dQ, dKr, dUr, dVr, dR


class _OracleOp(torch.autograd.Function):
    """Forward = mhffn_forward, backward = the explicit formulas (not autograd of the forward),
    so a layer-level gradient comparison with the reference exercises ``mhffn_backward``."""

    @staticmethod
    def forward(ctx, Q, K, U, V, R, hs, us, fs):
        ctx.save_for_backward(Q, K, U, V, R)
        ctx.kw = dict(head_scaling=hs, up_scaling=us, final_scaling=fs)
        return mhffn_forward(Q, K, U, V, R, **ctx.kw)

    @staticmethod
    def backward(ctx, dO):
        Q, K, U, V, R = ctx.saved_tensors
        dQ, dK, dU, dV, dR = mhffn_backward(Q, K, U, V, R, dO.to(Q.dtype), **ctx.kw)
        return dQ, dK, dU, dV, dR.to(R.dtype), None, None, None


def oracle_op(Q, K, U, V, R, head_scaling=1.0, up_scaling=1.0, final_scaling=1.0):
    return _OracleOp.apply(Q, K, U, V, R, head_scaling, up_scaling, final_scaling)


def router_weights(Q, router):
    """R = sigmoid(Q_f32 @ router_f32) normalised over experts with the denominator clamped at 1e-20.

    Q [B,H,S,d_h], router [H,d_h,E] -> R [B,H,S,E] fp32."""
    R = (Q.to(torch.float32) @ router.to(torch.float32)).sigmoid()
    return R / R.sum(dim=-1, keepdim=True).clamp(min=1e-20)


def multihead_rmsnorm(x, weight, eps):
    """Per-head RMSNorm over the last dim of x [B,S,H,d_h] in fp32 with weight [H,d_h]; cast back."""
    dt = x.dtype
    x = x.to(torch.float32)
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return (x * weight[None, None]).to(dt)


def split_heads(x_proj, gate_w, up_w, down_w, H, Hkuv, E):
    """Turn the layer's flat tensors into the operator's operands.

    x_proj [B,S,H*d_h] -> Q [B,H,S,d_h] (contiguous); gate/up/down [I, Hkuv*d_h] -> [Hkuv,E,d_e,d_h]."""
    B, S, hid = x_proj.shape
    dh = hid // H
    I = gate_w.shape[0]
    Q = x_proj.view(B, S, H, dh).transpose(1, 2).contiguous()
    f = lambda w: w.view(I, Hkuv, dh).transpose(0, 1).reshape(Hkuv, E, I // E, dh).contiguous()
    return Q, f(gate_w), f(up_w), f(down_w)


def mhffn_layer_forward(x, p, *, H, Hkuv, E, apply_rmsnorm, eps, op=None, scaling=(1.0, 1.0, 1.0)):
    """The whole FFN layer around the operator.

    p: dict with w_self [hid,hid], w_self_2 [hid,hid], gate_weight/up_weight/down_weight
    [I, Hkuv*d_h], router [H,d_h,E], q_norm [H,d_h].  ``op`` is the core operator
    (default: the oracle); tests pass the CUDA operator here to check the drop-in site."""
    op = op or oracle_op
    B, S, hid = x.shape
    dh = hid // H
    I = p["gate_weight"].shape[0]
    q = F.linear(x, p["w_self"], p.get("w_self_bias")).view(B, S, H, dh)
    if apply_rmsnorm:
        q = multihead_rmsnorm(q, p["q_norm"], eps)
    Q = q.transpose(1, 2).contiguous()
    f = lambda w: w.view(I, Hkuv, dh).transpose(0, 1).reshape(Hkuv, E, I // E, dh).contiguous()
    K, U, V = f(p["gate_weight"]), f(p["up_weight"]), f(p["down_weight"])
    R = router_weights(Q, p["router"])
    O = op(Q, K, U, V, R.contiguous(), *scaling) if tuple(scaling) != (1.0, 1.0, 1.0) else op(Q, K, U, V, R.contiguous())
    O = O.transpose(1, 2).contiguous().view(B, S, hid)
    return F.linear(O, p["w_self_2"], p.get("w_self_2_bias"))


def rel_l2(a, b):
    """||a-b|| / ||b|| in fp64 (b is the reference side)."""
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def make_op_inputs(B, H, S, dh, E, de, *, Hkuv=None, seed=0, dtype=torch.float32, w_std=0.02, with_dO=True):
    """Seeded operator inputs: Q~N(0,1); K,U,V~N(0,w_std); routing logits~N(0,1) -> sigmoid ->
    normalised over E; dO~N(0,1).  Generated in fp32 on the CPU generator then cast, so the
    same seed gives the same values for every dtype."""
    Hkuv = Hkuv or H
    g = torch.Generator().manual_seed(seed)
    Q = torch.randn(B, H, S, dh, generator=g)
    K = torch.randn(Hkuv, E, de, dh, generator=g) * w_std
    U = torch.randn(Hkuv, E, de, dh, generator=g) * w_std
    V = torch.randn(Hkuv, E, de, dh, generator=g) * w_std
    R = torch.randn(B, H, S, E, generator=g).sigmoid()
    R = R / R.sum(-1, keepdim=True)
    out = [Q.to(dtype), K.to(dtype), U.to(dtype), V.to(dtype), R]
    if with_dO:
        out.append(torch.randn(B, H, S, dh, generator=g).to(dtype))
    return out
