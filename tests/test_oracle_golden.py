"""CPU: the oracle restatement reproduces the reference layer's recorded outputs and gradients."""
import pytest
import torch

from oracle import mhffn_oracle as orc
from tests.golden_util import layer_params, load_golden

CASES = ["layer_tiny_dh64", "layer_tiny_gqa", "layer_128m_dims", "layer_370m_dims", "layer_tiny_scaled",
         "layer_128m_full"]   # the last: batch 2 x 512 tokens, hidden 768, 8 heads of 96, 8 x 256, fp32


def _run_layer(d, op=None):
    cfg = d["cfg"]
    p = {k: v.clone().requires_grad_(True) for k, v in layer_params(d).items()}
    x = d["x"].clone().requires_grad_(True)
    y = orc.mhffn_layer_forward(x, p, H=cfg["H"], Hkuv=cfg["Hkuv"], E=cfg["E"], apply_rmsnorm=cfg["rmsnorm"],
                                eps=1e-5, op=op, scaling=cfg["scaling"])
    (y * d["wloss"]).sum().backward()
    return x, p, y


@pytest.mark.parametrize("name", CASES)
def test_layer_forward_matches_reference(name):
    d = load_golden(name)
    _, _, y = _run_layer(d)
    assert orc.rel_l2(y.detach(), d["y"]) < 2e-6


@pytest.mark.parametrize("name", CASES)
def test_layer_gradients_match_reference(name):
    """Gradients flow through the oracle's explicit backward formulas, not autograd of its forward."""
    d = load_golden(name)
    x, p, _ = _run_layer(d)
    if "dx" in d:
        assert orc.rel_l2(x.grad, d["dx"]) < 2e-5
    else:
        assert orc.rel_l2(x.grad[:, ::4], d["dx_every4"]) < 2e-5
    for k, v in p.items():
        if d["cfg"]["skip_linear"] and k in ("w_self", "w_self_2"):
            continue
        if "g_" + k in d:
            assert orc.rel_l2(v.grad, d["g_" + k]) < 2e-5, k
        elif "gabs_" + k in d:
            ref_abs = float(d["gabs_" + k])
            assert abs(float(v.grad.double().abs().sum()) - ref_abs) < 1e-4 * ref_abs, k
            assert abs(float(v.grad.double().sum()) - float(d["gsum_" + k])) < 1e-4 * ref_abs, k


@pytest.mark.parametrize("name", CASES)
def test_operator_output_matches_reference_call_site(name):
    """Operands split the oracle's way equal what the reference passes to flash_mlp, and O matches."""
    d = load_golden(name)
    cfg = d["cfg"]
    p = layer_params(d)
    q = torch.nn.functional.linear(d["x"], p["w_self"])
    if cfg["rmsnorm"]:
        q = orc.multihead_rmsnorm(q.view(cfg["B"], cfg["S"], cfg["H"], cfg["dh"]), p["q_norm"], 1e-5).reshape(q.shape)
    Q, K, U, V = orc.split_heads(q, p["gate_weight"], p["up_weight"], p["down_weight"], cfg["H"], cfg["Hkuv"], cfg["E"])
    R = orc.router_weights(Q, p["router"])
    assert orc.rel_l2(R, d["op_R"]) < 1e-6
    if "op_Q" in d:
        assert orc.rel_l2(Q, d["op_Q"]) < 1e-6
        assert torch.equal(K, d["op_K"]) and torch.equal(U, d["op_U"]) and torch.equal(V, d["op_V"])
        Q, R = d["op_Q"], d["op_R"]
    hs, us, fs = cfg["scaling"]
    O = orc.mhffn_forward(Q, K, U, V, R, head_scaling=hs, up_scaling=us, final_scaling=fs)
    assert orc.rel_l2(O, d["op_O"]) < 2e-6
    if name == "layer_128m_full":   # "compare O elementwise against the reference output"
        assert float((O - d["op_O"]).abs().max()) < 1e-5 * float(d["op_O"].abs().max())


@pytest.mark.parametrize("dt", [torch.float64])
def test_explicit_backward_equals_autograd(dt):
    Q, K, U, V, R, dO = orc.make_op_inputs(2, 4, 33, 32, 3, 16, Hkuv=2, seed=5, dtype=dt)
    R = R.to(dt)
    ins = [t.clone().requires_grad_(True) for t in (Q, K, U, V, R)]
    O = orc.mhffn_forward(*ins)
    grads = torch.autograd.grad(O, ins, dO)
    mine = orc.mhffn_backward(Q, K, U, V, R, dO)
    for a, b in zip(mine, grads):
        assert orc.rel_l2(a, b) < 1e-13


def test_bf16_eager_vs_fp32_oracle_headroom():
    """The eager path in bf16 sits well inside the 1e-2 tolerance of the fp32 evaluation of the same inputs."""
    Q, K, U, V, R = orc.make_op_inputs(1, 2, 64, 64, 2, 64, seed=7, dtype=torch.bfloat16, with_dO=False)
    o16 = orc.mhffn_forward(Q, K, U, V, R)
    o32 = orc.mhffn_forward(Q.float(), K.float(), U.float(), V.float(), R)
    assert orc.rel_l2(o16.float(), o32) < 1e-2
