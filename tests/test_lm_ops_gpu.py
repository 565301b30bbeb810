"""GPU: the rotary and RMSNorm helper kernels against the reference's expressions evaluated by torch
(models/flashmhf/modeling_mhffnmoe.py:82-87, :178-206) in fp32 on the same bf16 inputs."""
import pytest
import torch

from oracle import mhffn_oracle as orc

pytestmark = pytest.mark.gpu


def _rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


@pytest.mark.parametrize("B,S,nh,hd", [(2, 37, 3, 64), (1, 300, 4, 128), (3, 5, 2, 32), (2, 64, 12, 64)])
def test_rotary_forward_and_backward(B, S, nh, hd):
    from flashmhf_b200 import lm, lm_ops
    g = torch.Generator().manual_seed(S)
    x = torch.randn(B, S, nh, hd, generator=g).bfloat16().cuda().requires_grad_(True)
    go = torch.randn(B, S, nh, hd, generator=g).bfloat16().cuda()
    cos, sin = lm.rotary_tables(S, hd, 10000.0, x.device, torch.bfloat16)
    ct, st = lm_ops.rotary_tables_f32(cos, sin)
    y = lm_ops.RotaryFunction.apply(x, ct, st)
    y.backward(go)
    xr = x.detach().float().requires_grad_(True)
    c, s = cos.float()[None, :, None, :], sin.float()[None, :, None, :]
    yr = xr * c + _rotate_half(xr) * s
    yr.backward(go.float())
    assert orc.rel_l2(y.float(), yr) < 4e-3          # one bf16 rounding
    assert orc.rel_l2(x.grad.float(), xr.grad) < 4e-3


@pytest.mark.parametrize("rows,n", [(5, 768), (1000, 1024), (77, 2048), (4096, 1024)])
def test_rmsnorm_forward_and_backward(rows, n):
    from flashmhf_b200 import lm_ops
    g = torch.Generator().manual_seed(rows)
    x = (torch.randn(rows, n, generator=g) * 1.7).bfloat16().cuda().requires_grad_(True)
    w = (1.0 + 0.1 * torch.randn(n, generator=g)).cuda().requires_grad_(True)
    go = torch.randn(rows, n, generator=g).bfloat16().cuda()
    y = lm_ops.RMSNormFunction.apply(x, w, 1e-5)
    y.backward(go)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().clone().requires_grad_(True)
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    yr.backward(go.float())
    assert orc.rel_l2(y.float(), yr) < 4e-3
    assert orc.rel_l2(x.grad.float(), xr.grad) < 4e-3
    assert orc.rel_l2(w.grad, wr.grad) < 1e-4
    # deterministic
    x2, w2 = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    lm_ops.RMSNormFunction.apply(x2, w2, 1e-5).backward(go)
    assert torch.equal(x2.grad, x.grad) and torch.equal(w2.grad, w.grad)


def test_helper_argument_errors():
    from flashmhf_b200 import _lib, lm_ops
    x = torch.zeros(4, 512, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.FlashMHFError):
        lm_ops.RMSNormFunction.apply(x, torch.ones(512, device="cuda"), 1e-5)     # unsupported row length
    with pytest.raises(_lib.FlashMHFError):
        lm_ops.RotaryFunction.apply(torch.zeros(1, 4, 2, 24, dtype=torch.bfloat16, device="cuda"),
                                    torch.zeros(4, 12, device="cuda"), torch.zeros(4, 12, device="cuda"))
