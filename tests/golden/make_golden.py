"""Generate the golden fixtures in this folder from the UNMODIFIED reference layer.

Run where a checkout of the reference is available:

    python tests/golden/make_golden.py /path/to/reference

It imports ``models/flashmhf/modeling_mhffnmoe.py`` without touching it (a stub package
``transformers.models.mhffnmoe`` satisfies its relative imports; ``transformers.utils.LossKwargs``
is the one name newer transformers releases dropped), builds
``MHFFNMoEMultiHeadFFNFlash(cfg, use_flash=False)`` -- the reference's eager path -- overwrites
every parameter from a seeded generator, and records inputs, outputs and gradients.  The operator
operands (Q, K, U, V, R) are captured at the reference's own call site by running the same layer a
second time through its flash branch with a recording stand-in for ``flash_mlp``
(modeling_mhffnmoe.py:394-408).

The fixtures are small .npz files; the tests read only those, never the reference.
"""
import importlib.util
import os
import sys
import types
from typing import TypedDict

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(ref_root):
    import transformers
    import transformers.models
    import transformers.utils

    if not hasattr(transformers.utils, "LossKwargs"):
        class LossKwargs(TypedDict, total=False):
            ...
        transformers.utils.LossKwargs = LossKwargs
    ref = os.path.join(ref_root, "models", "flashmhf")
    pkg = types.ModuleType("transformers.models.mhffnmoe")
    pkg.__path__ = [ref]
    sys.modules[pkg.__name__] = pkg

    def load(name):
        spec = importlib.util.spec_from_file_location(f"{pkg.__name__}.{name}", os.path.join(ref, name + ".py"))
        m = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = m
        spec.loader.exec_module(m)
        return m

    return load("configuration_mhffnmoe"), load("modeling_mhffnmoe")


def seeded_params(layer, seed, std=0.02):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in sorted(layer.named_parameters()):
            if name == "q_norm.weight":
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=g))
            else:
                p.copy_(torch.randn(p.shape, generator=g) * std)


class Recorder(torch.nn.Module):
    """Stand-in for flash_mlp that records the operands the reference passes and returns zeros."""

    def __init__(self):
        super().__init__()
        self.args = None

    def forward(self, Q, K, U, V, R):
        self.args = [t.detach().clone() for t in (Q, K, U, V, R)]
        return torch.zeros_like(Q)


def run_case(C, M, name, *, hidden, inter, H, Hkuv, E, B, S, rmsnorm, seed, full, skip_linear=False, scaled=False,
             big=False):
    """full: store every parameter and gradient (else only two moments of each gradient; parameters come from the seed).
    scaled: turn on the layer's dot scaling (head/up = sqrt(H)) and final scaling (sqrt(3/8)).
    big: a full-size case -- x and the loss weights are not stored (they come from the seed), dx is stored for every
    fourth token only."""
    cfg = C.MHFFNMoEConfig(hidden_size=hidden, intermediate_size=inter, num_attention_heads=max(1, hidden // 64),
                           mhffnmoe_num_heads=H, mhffnmoe_num_kuv_heads=Hkuv, mhffnmoe_num_experts=E,
                           mhffnmoe_use_flash=False, mhffnmoe_custom_init=True, mhffnmoe_apply_rmsnorm=rmsnorm,
                           mhffnmoe_skip_linear=skip_linear, mhffnmoe_apply_dot_scaling=scaled,
                           mhffnmoe_apply_final_scaling=scaled,
                           rms_norm_eps=1e-5)
    layer = M.MHFFNMoEMultiHeadFFNFlash(cfg, use_flash=False)
    seeded_params(layer, seed)
    g = torch.Generator().manual_seed(seed + 1000)
    x = torch.randn(B, S, hidden, generator=g, requires_grad=True)
    wloss = torch.randn(B, S, hidden, generator=g)
    y = layer(x)
    (y * wloss).sum().backward()
    out = {"x": x.detach(), "wloss": wloss, "y": y.detach(), "dx": x.grad}
    if big:
        out = {"y": y.detach(), "dx_every4": x.grad[:, ::4].contiguous()}
    hs, us, fs = float(layer.head_scaling), float(layer.up_scaling), float(layer.final_scaling)
    out["scaling"] = np.array([hs, us, fs], dtype=np.float64)
    for n, p in layer.named_parameters():
        key = n.replace(".weight", "").replace(".", "_")
        if p.grad is None:  # q_norm when the per-head RMSNorm is off
            continue
        if full:
            out["p_" + key] = p.detach()
            out["g_" + key] = p.grad
        else:  # parameters are reproducible from the seed; keep only two moments of each gradient
            out["gsum_" + key] = p.grad.double().sum().reshape(1)
            out["gabs_" + key] = p.grad.double().abs().sum().reshape(1)
    # operator operands as the reference hands them to its flash back-end, and the eager O for them
    rec = Recorder()
    layer.flash, layer.flash_mlp = True, rec
    with torch.no_grad():
        layer(x.detach())
    layer.flash, layer.flash_mlp = False, None
    Q, K, U, V, R = rec.args
    Kr, Ur, Vr = (M.repeat_kuv(t, H // Hkuv) for t in (K, U, V))
    O = torch.zeros(Q.shape, dtype=torch.float32)
    for i in range(E):  # the eager expression, evaluated with the reference's own helper for the head repeat
        w = torch.nn.functional.silu(Q @ Kr[:, i].transpose(1, 2) * hs) * (Q @ Ur[:, i].transpose(1, 2) * us)
        O += (w @ Vr[:, i] * fs).float() * R[..., i:i + 1]
    if full:
        out.update(op_Q=Q, op_K=K, op_U=U, op_V=V, op_R=R, op_O=O)
    else:
        out.update(op_R=R, op_O=O)
    out["meta"] = np.array([hidden, inter, H, Hkuv, E, B, S, int(rmsnorm), seed, int(skip_linear)], dtype=np.int64)
    np.savez(os.path.join(HERE, name + ".npz"), **{k: (v.numpy() if torch.is_tensor(v) else v) for k, v in out.items()})
    print(name, "y rms", float(y.pow(2).mean().sqrt()))


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python %s /path/to/reference" % os.path.basename(__file__))
    ref_root = sys.argv[1]
    torch.manual_seed(0)
    C, M = load_reference(ref_root)
    # tiny layer, every tensor stored
    run_case(C, M, "layer_tiny_dh64", hidden=128, inter=128, H=2, Hkuv=2, E=2, B=2, S=24, rmsnorm=True, seed=1, full=True)
    # shared K/U/V heads (G = 2)
    run_case(C, M, "layer_tiny_gqa", hidden=256, inter=128, H=4, Hkuv=2, E=2, B=1, S=20, rmsnorm=False, seed=2, full=True,
             skip_linear=True)
    # the 128M model's layer dims (hidden 768, 8 heads of 96, 8 x 256), short sequence; params from the seed
    run_case(C, M, "layer_128m_dims", hidden=768, inter=2048, H=8, Hkuv=8, E=8, B=1, S=8, rmsnorm=False, seed=3, full=False)
    # the 370M model's layer dims (hidden 1024, 8 heads of 128, 11 x 256), per-head RMSNorm on
    run_case(C, M, "layer_370m_dims", hidden=1024, inter=2816, H=8, Hkuv=8, E=11, B=1, S=8, rmsnorm=True, seed=4, full=False)
    # dot scaling and final scaling on (head/up = sqrt(H), final = sqrt(3/8)), every tensor stored
    run_case(C, M, "layer_tiny_scaled", hidden=128, inter=128, H=2, Hkuv=2, E=2, B=2, S=20, rmsnorm=True, seed=5, full=True,
             scaled=True)
    # the single-layer fp32 configuration in full: batch 2 x 512 tokens, hidden 768, 8 heads of 96, 8 x 256
    run_case(C, M, "layer_128m_full", hidden=768, inter=2048, H=8, Hkuv=8, E=8, B=2, S=512, rmsnorm=False, seed=6,
             full=False, big=True)


if __name__ == "__main__":
    main()
