"""GPU: the fused layer prologue (head split + per-head RMSNorm + router weights, forward and backward)
and the whole layer built on it, against the CPU restatement of the reference's element-wise path
(models/flashmhf/modeling_mhffnmoe.py:362-386, :116-135) and against the reference layer's fixtures.

Tolerances: Q is bf16, so a last-bit difference of rsqrt between CPU and GPU can flip a rounding
on a few elements (rel-L2 <= 2e-3 allows that); R is compared in fp32 (1e-5) on the Q the kernel wrote."""
import pytest
import torch

from oracle import mhffn_oracle as orc
from tests.golden_util import layer_params, load_golden

pytestmark = pytest.mark.gpu

# (B, S, H, d_h, E, rmsnorm)
CASES = [(2, 100, 3, 64, 4, True), (1, 257, 2, 96, 1, True), (3, 128, 4, 128, 11, True),
         (2, 77, 2, 128, 32, True), (2, 130, 3, 64, 5, False), (1, 1, 2, 128, 7, True), (4, 512, 8, 128, 11, True),
         (2, 150, 4, 128, 22, True), (1, 90, 2, 96, 17, True), (2, 40, 2, 64, 24, False), (1, 70, 2, 128, 25, True)]


def _inputs(B, S, H, dh, E, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, S, H * dh, generator=g).to(torch.bfloat16)
    w = 1.0 + 0.1 * torch.randn(H, dh, generator=g)
    router = torch.randn(H, dh, E, generator=g) * 0.2
    dQ = torch.randn(B, H, S, dh, generator=g).to(torch.bfloat16)
    dR = torch.randn(B, H, S, E, generator=g)
    return x, w, router, dQ, dR


def _oracle(x, w, router, H, norm, eps=1e-5):
    B, S, hid = x.shape
    q = x.view(B, S, H, hid // H)
    if norm:
        q = orc.multihead_rmsnorm(q, w, eps)
    Q = q.transpose(1, 2)
    return Q, orc.router_weights(Q, router)


@pytest.mark.parametrize("B,S,H,dh,E,norm", CASES)
def test_prologue_forward_matches_oracle(B, S, H, dh, E, norm):
    from flashmhf_b200 import fused_prologue
    x, w, router, _, _ = _inputs(B, S, H, dh, E, seed=B * 1000 + S)
    Q, R = fused_prologue(x.cuda(), w.cuda() if norm else None, router.cuda())
    torch.cuda.synchronize()
    Qo, Ro = _oracle(x, w, router, H, norm)
    assert Q.shape == (B, H, S, dh) and R.shape == (B, H, S, E) and R.dtype == torch.float32
    assert Q.stride() == (S * H * dh, dh, H * dh, 1)            # the projection's own layout, no transposing copy
    if norm:
        assert orc.rel_l2(Q.float().cpu(), Qo.float()) < 2e-3
        assert (Q.cpu() != Qo).float().mean() < 0.02             # only isolated last-bit flips
    else:
        assert torch.equal(Q.cpu(), Qo)
    assert orc.rel_l2(R.cpu(), orc.router_weights(Q.cpu(), router)) < 1e-5
    assert orc.rel_l2(R.cpu(), Ro) < 1e-3
    assert torch.allclose(R.sum(-1).cpu(), torch.ones(B, H, S), atol=1e-5)


@pytest.mark.parametrize("B,S,H,dh,E,norm", CASES)
@pytest.mark.parametrize("dq_layout", ["bshd", "bhsd"])
def test_prologue_backward_matches_oracle_autograd(B, S, H, dh, E, norm, dq_layout):
    from flashmhf_b200 import fused_prologue
    x, w, router, dQ, dR = _inputs(B, S, H, dh, E, seed=B * 1000 + S + 1)
    # oracle: autograd through the restatement, fp32 parameters, bf16 activations
    xo, wo, ro = x.clone().requires_grad_(True), w.clone().requires_grad_(True), router.clone().requires_grad_(True)
    Qo, Ro = _oracle(xo, wo, ro, H, norm)
    ((Qo.float() * dQ.float()).sum() + (Ro * dR).sum()).backward()
    # CUDA
    xg, rg = x.cuda().requires_grad_(True), router.cuda().requires_grad_(True)
    wg = w.cuda().requires_grad_(True) if norm else None
    Q, R = fused_prologue(xg, wg, rg)
    g = dQ.cuda() if dq_layout == "bhsd" else dQ.cuda().transpose(1, 2).contiguous().transpose(1, 2)
    torch.autograd.backward([Q, R], [g, dR.cuda()])
    torch.cuda.synchronize()
    assert orc.rel_l2(xg.grad.float().cpu(), xo.grad.float()) < 1e-2      # bf16 output
    if E == 1:   # R == 1 identically: the exact router gradient is zero, the oracle's is rounding noise
        assert rg.grad.abs().max() < 1e-5 and ro.grad.abs().max() < 1e-5
    else:
        assert orc.rel_l2(rg.grad.cpu(), ro.grad) < 2e-3
    if norm:
        assert orc.rel_l2(wg.grad.cpu(), wo.grad) < 2e-3


def test_prologue_backward_is_deterministic_and_ignores_stale_workspace():
    from flashmhf_b200 import fused_prologue
    x, w, router, dQ, dR = _inputs(4, 300, 4, 128, 11, seed=5)
    outs = []
    for _ in range(2):
        xg, wg, rg = (t.cuda().requires_grad_(True) for t in (x, w, router))
        Q, R = fused_prologue(xg, wg, rg)
        torch.autograd.backward([Q, R], [dQ.cuda(), dR.cuda()])
        outs.append((xg.grad.clone(), wg.grad.clone(), rg.grad.clone()))
        torch.empty(64 << 20, dtype=torch.uint8, device="cuda").fill_(0xFF)   # dirty the allocator's free blocks
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_prologue_argument_errors():
    from flashmhf_b200 import fused_prologue
    x, w, router, _, _ = _inputs(1, 8, 2, 64, 3, seed=1)
    with pytest.raises(TypeError):
        fused_prologue(x.cuda().float(), w.cuda(), router.cuda())
    with pytest.raises(ValueError):
        fused_prologue(x.cuda()[..., :96], w.cuda(), router.cuda())
    with pytest.raises(ValueError):
        fused_prologue(torch.zeros(1, 8, 2 * 32, dtype=torch.bfloat16, device="cuda"), None, torch.zeros(2, 32, 3, device="cuda"))
    with pytest.raises(ValueError):
        fused_prologue(torch.zeros(1, 8, 2 * 64, dtype=torch.bfloat16, device="cuda"), None, torch.zeros(2, 64, 33, device="cuda"))


LAYER_CASES = ["layer_tiny_dh64", "layer_tiny_gqa", "layer_128m_dims", "layer_370m_dims"]


@pytest.mark.parametrize("name", LAYER_CASES)
def test_fused_layer_matches_reference_fixtures(name):
    """The layer with the fused prologue and the in-place (strided) operands, bf16, against what the
    unmodified reference layer produced in fp32."""
    import flashmhf_b200 as fm
    d = load_golden(name)
    cfg = d["cfg"]
    p = {k: v.cuda().to(torch.bfloat16).requires_grad_(True) for k, v in layer_params(d).items()}
    if cfg["skip_linear"]:
        p["w_self"] = p["w_self_2"] = None
    x = d["x"].cuda().to(torch.bfloat16).requires_grad_(True)
    y = fm.mhffn_layer(x, p, H=cfg["H"], Hkuv=cfg["Hkuv"], E=cfg["E"], apply_rmsnorm=cfg["rmsnorm"], eps=1e-5)
    (y.float() * d["wloss"].cuda()).sum().backward()
    torch.cuda.synchronize()
    assert orc.rel_l2(y.detach().float().cpu(), d["y"]) < 2e-2
    assert orc.rel_l2(x.grad.float().cpu(), d["dx"]) < 3e-2
    for k in ("gate_weight", "up_weight", "down_weight", "router") + (("q_norm",) if cfg["rmsnorm"] else ()):
        if "g_" + k in d:
            assert orc.rel_l2(p[k].grad.float().cpu(), d["g_" + k]) < 3e-2, k


def test_fused_layer_equals_unfused_layer_on_gpu():
    """Same bf16 inputs through the oracle-shaped layer with the CUDA operator (copies, torch element-wise
    prologue) and through the fused layer: outputs agree to bf16 rounding of Q."""
    import flashmhf_b200 as fm
    d = load_golden("layer_128m_dims")
    cfg = d["cfg"]
    p = {k: v.cuda().to(torch.bfloat16) for k, v in layer_params(d).items()}
    x = d["x"].cuda().to(torch.bfloat16)
    kw = dict(H=cfg["H"], Hkuv=cfg["Hkuv"], E=cfg["E"], apply_rmsnorm=cfg["rmsnorm"], eps=1e-5)
    pf = {k: (v.float() if k in ("router", "q_norm") else v) for k, v in p.items()}
    a = orc.mhffn_layer_forward(x, pf, op=fm.flash_mhf, **kw)
    b = fm.mhffn_layer(x, p, **kw)
    assert orc.rel_l2(b.float().cpu(), a.float().cpu()) < 5e-3


def test_layer_with_more_sub_networks_than_the_fused_prologue_takes():
    """E = 40 > 32: the layer keeps working through torch's element-wise kernels for the prologue; the operator itself
    has no limit on E."""
    import flashmhf_b200 as fm
    g = torch.Generator().manual_seed(9)
    hid, H, E, de = 128, 2, 40, 64
    p = {"w_self": torch.randn(hid, hid, generator=g) * 0.05, "w_self_2": torch.randn(hid, hid, generator=g) * 0.05,
         "gate_weight": torch.randn(E * de, hid, generator=g) * 0.05, "up_weight": torch.randn(E * de, hid, generator=g) * 0.05,
         "down_weight": torch.randn(E * de, hid, generator=g) * 0.05, "router": torch.randn(H, hid // H, E, generator=g) * 0.2,
         "q_norm": 1.0 + 0.1 * torch.randn(H, hid // H, generator=g)}
    x = torch.randn(2, 50, hid, generator=g)
    kw = dict(H=H, Hkuv=H, E=E, apply_rmsnorm=True, eps=1e-5)
    pc = {k: v.cuda().bfloat16().requires_grad_(True) for k, v in p.items()}
    xc = x.cuda().bfloat16().requires_grad_(True)
    y = fm.mhffn_layer(xc, pc, **kw)
    y.float().sum().backward()
    po = {k: v.clone().requires_grad_(True) for k, v in p.items()}
    xo = x.clone().requires_grad_(True)
    yo = orc.mhffn_layer_forward(xo, po, **kw)
    yo.sum().backward()
    assert orc.rel_l2(y.float().cpu(), yo) < 2e-2
    assert orc.rel_l2(xc.grad.float().cpu(), xo.grad) < 3e-2
    assert orc.rel_l2(pc["router"].grad.float().cpu(), po["router"].grad) < 5e-2
