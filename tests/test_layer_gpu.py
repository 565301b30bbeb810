"""GPU: the drop-in site.  The whole FFN layer (projection -> heads -> per-head RMSNorm -> router ->
operator -> merge -> projection, models/flashmhf/modeling_mhffnmoe.py:352-431) with the CUDA operator
in the place of `flash_mlp`, against what the UNMODIFIED reference layer produced (committed fixtures)."""
import pytest
import torch

from oracle import mhffn_oracle as orc
from tests.golden_util import layer_params, load_golden

pytestmark = pytest.mark.gpu
CASES = ["layer_tiny_dh64", "layer_tiny_gqa", "layer_128m_dims", "layer_370m_dims"]


def _run(d, dtype):
    import flashmhf_b200 as fm
    cfg = d["cfg"]
    p = {k: v.cuda().to(dtype).requires_grad_(True) for k, v in layer_params(d).items()}
    x = d["x"].cuda().to(dtype).requires_grad_(True)
    y = orc.mhffn_layer_forward(x, p, H=cfg["H"], Hkuv=cfg["Hkuv"], E=cfg["E"], apply_rmsnorm=cfg["rmsnorm"],
                                eps=1e-5, op=fm.flash_mhf)
    (y.float() * d["wloss"].cuda()).sum().backward()
    torch.cuda.synchronize()
    return x, p, y


@pytest.mark.parametrize("name", CASES)
def test_layer_fp32_check_mode_matches_reference(name):
    d = load_golden(name)
    x, p, y = _run(d, torch.float32)
    assert orc.rel_l2(y.detach().cpu(), d["y"]) < 1e-5
    assert orc.rel_l2(x.grad.cpu(), d["dx"]) < 5e-5
    for k, v in p.items():
        if "g_" + k in d and not (d["cfg"]["skip_linear"] and k.startswith("w_self")):
            assert orc.rel_l2(v.grad.cpu(), d["g_" + k]) < 5e-5, k


@pytest.mark.parametrize("name", CASES)
def test_layer_bf16_matches_reference_within_tolerance(name):
    """bf16 weights and activations through the tensor-core kernels vs the reference layer run in fp32."""
    d = load_golden(name)
    x, p, y = _run(d, torch.bfloat16)
    assert orc.rel_l2(y.detach().float().cpu(), d["y"]) < 2e-2   # includes bf16 rounding of the two projections
    assert orc.rel_l2(x.grad.float().cpu(), d["dx"]) < 3e-2


def test_reference_import_seam_modules_run_on_gpu():
    import flashmhf_b200
    flashmhf_b200.install_reference_seam()
    from ops.flash_mlp_moe import FlashMLPMoE
    from ops.flash_mlp import FlashMLP
    from flash_ffn_moe_torch import FlashFFNMoE
    Q, K, U, V, R = (t.cuda() for t in orc.make_op_inputs(1, 2, 100, 64, 2, 64, seed=31, dtype=torch.bfloat16, with_dO=False))
    a = FlashMLPMoE()(Q, K, U, V, R)
    b = FlashFFNMoE()(Q, K, U, V, R)
    assert torch.equal(a, b)
    ref = orc.mhffn_forward(Q.cpu().float(), K.cpu().float(), U.cpu().float(), V.cpu().float(), R.cpu())
    assert orc.rel_l2(a.cpu().float(), ref) < 1e-2
    # legacy module: one sub-network, no routing weight (== E = 1, R = 1)
    o = FlashMLP()(Q, K[:, 0], U[:, 0], V[:, 0], False, 1.0, 1.0, "silu")
    ref1 = orc.mhffn_forward(Q.cpu().float(), K[:, :1].cpu().float(), U[:, :1].cpu().float(), V[:, :1].cpu().float(),
                             torch.ones(1, 2, 100, 1))
    assert orc.rel_l2(o.cpu().float(), ref1) < 1e-2


def test_unmodified_reference_layer_runs_the_cuda_operator_through_its_import_seam():
    """Where a checkout of the reference is at hand (never on a bare GPU box: then skipped), build its own
    MHFFNMoEMultiHeadFFNFlash(cfg, use_flash=True) after install_reference_seam(): its constructor import
    (modeling_mhffnmoe.py:318-329) must pick up this package's FlashMLPMoE, and its flash branch (:394-408) must give
    what its eager branch gives."""
    import os
    import flashmhf_b200
    from tests.golden.make_golden import load_reference, seeded_params
    from tests.golden_util import find_reference_checkout
    ref_root = find_reference_checkout()
    if ref_root is None:
        pytest.skip("no reference checkout on this machine")
    flashmhf_b200.install_reference_seam()
    C_, M = load_reference(ref_root)
    cfg = C_.MHFFNMoEConfig(hidden_size=256, intermediate_size=256, num_attention_heads=4, mhffnmoe_num_heads=2,
                            mhffnmoe_num_kuv_heads=2, mhffnmoe_num_experts=2, mhffnmoe_use_flash=True,
                            mhffnmoe_custom_init=True, mhffnmoe_apply_rmsnorm=True, rms_norm_eps=1e-5)
    layer = M.MHFFNMoEMultiHeadFFNFlash(cfg, use_flash=True)
    assert layer.flash and type(layer.flash_mlp).__module__ == "ops.flash_mlp_moe"
    seeded_params(layer, 7)
    layer = layer.cuda().to(torch.bfloat16)
    x = torch.randn(2, 150, 256, generator=torch.Generator().manual_seed(8)).cuda().to(torch.bfloat16)
    y_flash = layer(x)
    layer.flash = False
    y_eager = layer(x)
    assert orc.rel_l2(y_flash.float().cpu(), y_eager.float().cpu()) < 2e-2
