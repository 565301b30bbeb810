"""Autograd wrappers of the two LM helper kernels (rotary embedding, hidden-size RMSNorm) in csrc/lm_aux.cu.

They serve flashmhf_b200/lm.py on CUDA bf16 tensors; the module keeps plain torch expressions for
everything else.  Both follow the reference's arithmetic (models/flashmhf/modeling_mhffnmoe.py:82-87,
:178-206) in fp32 with one rounding to bf16."""
import ctypes as C

import torch

from . import _lib

NORM_SIZES = (768, 1024, 2048)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class RotaryFunction(torch.autograd.Function):
    """x [B,S,heads,head_dim] bf16 contiguous, cos/sin fp32 [S, head_dim/2] -> rotated tensor of the same layout."""

    @staticmethod
    def _run(x, cos_t, sin_t, transpose):
        B, S, nh, hd = x.shape
        y = torch.empty_like(x)
        with torch.cuda.device(x.device):
            _lib.check(_lib.load().flashmhf_lm_rope(x.data_ptr(), y.data_ptr(), cos_t.data_ptr(), sin_t.data_ptr(), B * S, S, nh, hd,
                                                    nh * hd, nh * hd, int(transpose), _stream()))
        return y

    @staticmethod
    def forward(ctx, x, cos_t, sin_t):
        ctx.save_for_backward(cos_t, sin_t)
        return RotaryFunction._run(x.contiguous(), cos_t, sin_t, False)

    @staticmethod
    def backward(ctx, g):
        cos_t, sin_t = ctx.saved_tensors
        return RotaryFunction._run(g.contiguous(), cos_t, sin_t, True), None, None


class RMSNormFunction(torch.autograd.Function):
    """x [..., n] bf16, weight [n] (any float dtype) -> y; n in NORM_SIZES."""

    @staticmethod
    def forward(ctx, x, weight, eps):
        x = x.contiguous()
        w = weight.detach().float().contiguous()
        y = torch.empty_like(x)
        n = x.shape[-1]
        with torch.cuda.device(x.device):
            _lib.check(_lib.load().flashmhf_lm_rmsnorm_forward(x.data_ptr(), w.data_ptr(), y.data_ptr(), x.numel() // n, n,
                                                               float(eps), _stream()))
        ctx.save_for_backward(x, w)
        ctx.eps, ctx.wdtype = float(eps), weight.dtype
        return y

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        g = g.contiguous()
        n = x.shape[-1]
        rows = x.numel() // n
        lib = _lib.load()
        dx, dw = torch.empty_like(x), torch.empty_like(w)
        nbytes = int(lib.flashmhf_lm_rmsnorm_backward_workspace_bytes(rows, n))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        with torch.cuda.device(x.device):
            _lib.check(lib.flashmhf_lm_rmsnorm_backward(x.data_ptr(), w.data_ptr(), g.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                                                        ws.data_ptr(), nbytes, rows, n, ctx.eps, _stream()))
        return dx, dw.to(ctx.wdtype), None


def rotary_tables_f32(cos, sin):
    """The first half of the reference's (duplicated) cos/sin tables, as the fp32 values of their bf16 roundings."""
    h = cos.shape[-1] // 2
    return cos[:, :h].float().contiguous(), sin[:, :h].float().contiguous()
