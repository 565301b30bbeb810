"""GPU: the operator's optional arguments and its failure reporting, through the C ABI.

* the eager layer's three constants (head, up and final scaling; models/flashmhf/modeling_mhffnmoe.py:270-279,
  420-425) in check mode and in bf16, forward and backward, and through the layer fixture recorded with them on;
* the legacy module (one sub-network, no routing weight) with dot scaling, which the reference's own legacy kernel
  rejects and its eager branch applies;
* backward in two parts (weights, then inputs) equals the one-call backward bit for bit;
* routing weights at an address that is only 4-byte aligned are read in place;
* the bounded-wait path: a self-test kernel lets a wait run out; the status call reports it once, and the next
  operator call is unaffected."""
import ctypes as C

import pytest
import torch

from oracle import mhffn_oracle as orc
from tests.golden_util import layer_params, load_golden

pytestmark = pytest.mark.gpu
SCALING = dict(head_scaling=2.0, up_scaling=1.5, final_scaling=0.6123724)


def _dev(ts):
    return [t.cuda() for t in ts]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("shape", [(2, 2, 2, 200, 128, 2, 128), (1, 4, 2, 130, 96, 3, 64), (1, 2, 2, 70, 64, 2, 64)])
def test_scaling_constants_forward_backward(shape, dtype, tol):
    import flashmhf_b200 as fm
    B, H, Hk, S, dh, E, de = shape
    Q, K, U, V, R, dO = orc.make_op_inputs(B, H, S, dh, E, de, Hkuv=Hk, seed=51, dtype=dtype)
    sc = tuple(SCALING.values())
    O = fm.forward_raw(*_dev([Q, K, U, V, R]), scaling=sc).cpu().double()
    d64 = [t.double() for t in (Q, K, U, V, R)]
    assert orc.rel_l2(O, orc.mhffn_forward(*d64, **SCALING)) < tol
    got = [g.cpu().double() for g in fm.backward_raw(*_dev([Q, K, U, V, R, dO]), scaling=sc)]
    for name, a, b in zip("dQ dK dU dV dR".split(), got, orc.mhffn_backward(*d64, dO.double(), **SCALING)):
        assert orc.rel_l2(a, b) < tol, name


def test_scaling_constants_through_autograd():
    import flashmhf_b200 as fm
    Q, K, U, V, R, dO = orc.make_op_inputs(1, 2, 150, 128, 2, 64, seed=52, dtype=torch.bfloat16)
    ins = [t.cuda().requires_grad_(True) for t in (Q, K, U, V, R)]
    fm.flash_mhf(*ins, *SCALING.values()).backward(dO.cuda())
    ref = orc.mhffn_backward(*(t.double() for t in (Q, K, U, V, R, dO)), **SCALING)
    for name, t, b in zip("dQ dK dU dV dR".split(), ins, ref):
        assert orc.rel_l2(t.grad.cpu().double(), b) < 1e-2, name


@pytest.mark.parametrize("dtype,tol_y,tol_g", [(torch.float32, 1e-5, 5e-5), (torch.bfloat16, 2e-2, 3e-2)])
def test_layer_fixture_with_dot_and_final_scaling(dtype, tol_y, tol_g):
    """The unmodified reference layer with apply_dot_scaling and apply_final_scaling on, against the CUDA operator."""
    import flashmhf_b200 as fm
    d = load_golden("layer_tiny_scaled")
    cfg = d["cfg"]
    assert cfg["scaling"] != (1.0, 1.0, 1.0)
    p = {k: v.cuda().to(dtype).requires_grad_(True) for k, v in layer_params(d).items()}
    x = d["x"].cuda().to(dtype).requires_grad_(True)
    y = orc.mhffn_layer_forward(x, p, H=cfg["H"], Hkuv=cfg["Hkuv"], E=cfg["E"], apply_rmsnorm=cfg["rmsnorm"], eps=1e-5,
                                op=fm.flash_mhf, scaling=cfg["scaling"])
    (y.float() * d["wloss"].cuda()).sum().backward()
    assert orc.rel_l2(y.detach().float().cpu(), d["y"]) < tol_y
    assert orc.rel_l2(x.grad.float().cpu(), d["dx"]) < tol_g
    if dtype == torch.float32:
        for k, v in p.items():
            if "g_" + k in d:
                assert orc.rel_l2(v.grad.cpu(), d["g_" + k]) < tol_g, k


def test_legacy_module_with_dot_scaling():
    """modeling_mhffnmoe.py:395-404: per sub-network calls with (apply_dot_scaling, head_scaling, up_scaling)."""
    import flashmhf_b200
    flashmhf_b200.install_reference_seam()
    from ops.flash_mlp import FlashMLP
    Q, K, U, V, R = orc.make_op_inputs(1, 2, 100, 64, 1, 128, seed=53, dtype=torch.bfloat16, with_dO=False)
    o = FlashMLP()(Q.cuda(), K[:, 0].cuda(), U[:, 0].cuda(), V[:, 0].cuda(), True, 2.0, 2.0, "silu")
    ref = orc.mhffn_forward(Q.float(), K.float(), U.float(), V.float(), torch.ones(1, 2, 100, 1), head_scaling=2.0,
                            up_scaling=2.0)
    assert orc.rel_l2(o.cpu().float(), ref) < 1e-2
    with pytest.raises(ValueError):
        FlashMLP()(Q.cuda(), K[:, 0].cuda(), U[:, 0].cuda(), V[:, 0].cuda(), False, 1.0, 1.0, "gelu")


def test_zero_or_nan_scaling_is_rejected():
    import flashmhf_b200 as fm
    ins = _dev(orc.make_op_inputs(1, 1, 64, 64, 1, 64, seed=54, dtype=torch.bfloat16, with_dO=False))
    for bad in ((0.0, 1.0, 1.0), (1.0, float("nan"), 1.0), (1.0, 1.0, float("inf"))):
        with pytest.raises(ValueError):
            fm.forward_raw(*ins, scaling=bad)


def test_backward_in_two_parts_equals_one_call():
    import flashmhf_b200 as fm
    ins = _dev(orc.make_op_inputs(2, 4, 300, 128, 3, 128, Hkuv=2, seed=55, dtype=torch.bfloat16))
    dQ, dK, dU, dV, dR = fm.backward_raw(*ins)
    bucket = torch.full((3 * dK.numel(),), float("nan"), dtype=torch.bfloat16, device="cuda")
    views = [bucket[i * dK.numel():(i + 1) * dK.numel()].view_as(dK) for i in range(3)]   # one all-reduce bucket
    q0, k1, u1, v1, r0 = fm.backward_raw(*ins, parts="weights", weight_grads=views)
    assert q0 is None and r0 is None and k1 is views[0]
    q2, k0, u0, v0, r2 = fm.backward_raw(*ins, parts="inputs")
    assert k0 is None and u0 is None and v0 is None
    for a, b in ((dQ, q2), (dR, r2), (dK, k1), (dU, u1), (dV, v1)):
        assert torch.equal(a, b)


def test_routing_weights_at_a_4_byte_aligned_address():
    """R[:, :, 1:] of an E = 11 tensor starts 44 bytes into the allocation; the kernels read R one float at a time."""
    import flashmhf_b200 as fm
    B, H, S, dh, E, de = 1, 2, 140, 128, 11, 64
    Q, K, U, V, R, dO = orc.make_op_inputs(B, H, S + 1, dh, E, de, seed=56, dtype=torch.bfloat16)
    Rv = R.cuda()[:, :, 1:]
    assert Rv.data_ptr() % 16 != 0 and Rv.stride(-1) == 1
    Qd, dOd = Q[:, :, 1:].contiguous().cuda(), dO[:, :, 1:].contiguous().cuda()
    O = fm.forward_raw(Qd, K.cuda(), U.cuda(), V.cuda(), Rv).cpu().float()
    f = [t.float() for t in (Q[:, :, 1:], K, U, V)]
    assert orc.rel_l2(O, orc.mhffn_forward(*f, R[:, :, 1:])) < 1e-2
    got = [g.cpu().float() for g in fm.backward_raw(Qd, K.cuda(), U.cuda(), V.cuda(), Rv, dOd)]
    for name, a, b in zip("dQ dK dU dV dR".split(), got, orc.mhffn_backward(*f, R[:, :, 1:], dO[:, :, 1:].float())):
        assert orc.rel_l2(a, b) < 1e-2, name


def test_bounded_wait_runs_out_is_reported_once_and_later_calls_are_unaffected():
    """No fault, no trap, no hang: a small kernel waits about a millisecond on a barrier nothing arrives at, gives up,
    records its code and returns.  The host learns of it from the status call, which clears the word; operator calls
    enqueued after the failed launch -- before or after the word is read -- produce correct results."""
    import flashmhf_b200 as fm
    from flashmhf_b200 import _lib
    lib = _lib.load()
    _lib.device_status()                                   # clean before
    ins = _dev(orc.make_op_inputs(1, 2, 200, 128, 2, 64, seed=57, dtype=torch.bfloat16))
    want = [fm.forward_raw(*ins[:5])] + list(fm.backward_raw(*ins))
    torch.cuda.synchronize()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.flashmhf_selftest_bounded_wait(2_000_000, stream) == 0      # ~1 ms of SM clock cycles
    got_before_read = [fm.forward_raw(*ins[:5])] + list(fm.backward_raw(*ins))   # enqueued behind the failed launch
    with pytest.raises(_lib.FlashMHFError) as err:
        _lib.device_status()
    assert err.value.status == -9 and err.value.code == _lib.SELFTEST_CODE
    _lib.device_status()                                   # reading cleared it
    got_after_read = [fm.forward_raw(*ins[:5])] + list(fm.backward_raw(*ins))
    fm.check_device_status()
    for got in (got_before_read, got_after_read):
        for a, b in zip(got, want):
            assert torch.equal(a, b)
    assert lib.flashmhf_selftest_bounded_wait(0, stream) == -2             # limit out of range
