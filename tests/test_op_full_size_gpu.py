"""GPU parity at the sizes the measurements are quoted on, against the CPU oracle on the same seeded inputs.

* the benchmark workload in full (B=16 x S=2048 tokens, H=8, d_h=128, E=11, d_e=256): O and all five gradients;
* the single-layer fp32 configuration in full (batch 2 x 512, hidden 768, 8 heads of 96, 8 x 256), from the fixture
  captured from the unmodified reference layer: fp32 check mode element-wise, and bf16;
* corners of the operator sweep at T = 4096 (d_h in {64, 128}, H in {8, 16}, E in {16, 32}) and the 1.3B layer's
  backward (H=16, E=22).

Tolerances: bf16 rel-L2 <= 1e-2 against the oracle evaluated in fp32 on the same bf16-rounded inputs; fp32 check
mode <= 1e-5.  The oracle runs in fp32 here (fp64 at these sizes would take tens of GB of host memory)."""
import pytest
import torch

from oracle import mhffn_oracle as orc
from tests.golden_util import layer_params, load_golden

pytestmark = pytest.mark.gpu
TOL_BF16, TOL_F32 = 1e-2, 1e-5


@pytest.fixture(autouse=True)
def _status_clean():
    from flashmhf_b200 import _lib
    yield
    _lib.device_status()


def _compare_all(shape, seed):
    import flashmhf_b200 as fm
    B, H, Hk, S, dh, E, de = shape
    Q, K, U, V, R, dO = orc.make_op_inputs(B, H, S, dh, E, de, Hkuv=Hk, seed=seed, dtype=torch.bfloat16)
    dev = [t.cuda() for t in (Q, K, U, V, R, dO)]
    O = fm.forward_raw(*dev[:5]).cpu().float()
    got = [g.cpu().float() for g in fm.backward_raw(*dev)]
    del dev
    torch.cuda.empty_cache()
    f = [t.float() for t in (Q, K, U, V)]
    assert orc.rel_l2(O, orc.mhffn_forward(*f, R)) < TOL_BF16, ("O", shape)
    ref = orc.mhffn_backward(*f, R, dO.float())
    for name, a, b in zip("dQ dK dU dV dR".split(), got, ref):
        assert orc.rel_l2(a, b) < TOL_BF16, (name, shape)


def test_benchmark_workload_in_full_against_oracle():
    """2048 token tiles; in the dK/dU/dV kernel 256 token tiles per head, split over CTAs, 44 weight blocks per head."""
    _compare_all((16, 8, 8, 2048, 128, 11, 256), seed=101)


@pytest.mark.parametrize("shape", [
    (1, 16, 16, 4096, 128, 32, 320),   # d_h=128, H=16, E=32, d_e=(8/3)*128 rounded to 320
    (1, 16, 16, 4096, 64, 32, 192),    # d_h=64,  H=16, E=32, d_e=192
    (1, 8, 8, 4096, 128, 16, 256),     # d_h=128, H=8,  E=16, the shipped d_e
    (1, 16, 16, 256, 128, 22, 256),    # the 1.3B layer (backward with one token split: 16 x 88 weight blocks)
])
def test_operator_sweep_corners_against_oracle(shape):
    _compare_all(shape, seed=102)


def _fixture_operands(d):
    cfg = d["cfg"]
    p = layer_params(d)
    q = torch.nn.functional.linear(d["x"], p["w_self"])
    if cfg["rmsnorm"]:
        q = orc.multihead_rmsnorm(q.view(cfg["B"], cfg["S"], cfg["H"], cfg["dh"]), p["q_norm"], 1e-5).reshape(q.shape)
    Q, K, U, V = orc.split_heads(q, p["gate_weight"], p["up_weight"], p["down_weight"], cfg["H"], cfg["Hkuv"], cfg["E"])
    return Q, K, U, V, d["op_R"]


def test_single_layer_fp32_configuration_elementwise():
    """Batch 2 x seq 512, hidden 768 -> 8 heads of 96, 8 sub-networks of 256: O of the fp32 check mode against the O the
    reference's eager path produced for the same operands, element by element."""
    import flashmhf_b200 as fm
    d = load_golden("layer_128m_full")
    ops = _fixture_operands(d)
    O = fm.forward_raw(*[t.cuda() for t in ops]).cpu()
    ref = d["op_O"]
    assert orc.rel_l2(O, ref) < TOL_F32
    assert float((O - ref).abs().max()) < TOL_F32 * float(ref.abs().max())
    O16 = fm.forward_raw(*[t.cuda().to(torch.bfloat16) for t in ops[:4]], ops[4].cuda()).cpu().float()
    assert orc.rel_l2(O16, ref) < TOL_BF16


def test_single_layer_fp32_configuration_whole_layer():
    """The same configuration through the whole layer (projections, router, operator) in check mode and in bf16, against
    the reference layer's y and dx."""
    import flashmhf_b200 as fm
    d = load_golden("layer_128m_full")
    cfg = d["cfg"]
    for dtype, tol_y, tol_dx in ((torch.float32, 1e-5, 5e-5), (torch.bfloat16, 2e-2, 3e-2)):
        p = {k: v.cuda().to(dtype).requires_grad_(True) for k, v in layer_params(d).items()}
        x = d["x"].cuda().to(dtype).requires_grad_(True)
        y = orc.mhffn_layer_forward(x, p, H=cfg["H"], Hkuv=cfg["Hkuv"], E=cfg["E"], apply_rmsnorm=cfg["rmsnorm"],
                                    eps=1e-5, op=fm.flash_mhf)
        (y.float() * d["wloss"].cuda()).sum().backward()
        assert orc.rel_l2(y.detach().float().cpu(), d["y"]) < tol_y, dtype
        assert orc.rel_l2(x.grad.float().cpu()[:, ::4], d["dx_every4"]) < tol_dx, dtype
