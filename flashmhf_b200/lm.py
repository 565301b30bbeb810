"""A minimal decoder LM around the FFN layer, for whole-model measurements and layer-in-context tests.

The architecture and every parameter name follow the reference model
(models/flashmhf/modeling_mhffnmoe.py: decoder layer :601-652, attention :523-598, RMSNorm :73-90,
rotary tables :164-175, FFN layer :256-431, model :784-921, LM head :1055-1090), so a reference
state dict loads with ``load_state_dict``.  The FFN layer is this package's code (the fused prologue + the
CUDA operator), and on CUDA bf16 tensors the rotary embedding and the hidden-size RMSNorm run through two small
kernels of the same library (lm_ops.py); attention, projections, embeddings and the loss are plain PyTorch
calls: they are the surroundings the operator is measured in, not part of it.

``ffn`` lets a caller substitute the FFN layer function; the default is the CUDA layer and there is
no CPU stand-in for it in this package.
"""
import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class LMConfig:
    """Field meanings as in the reference's configuration files (configs/mhffnmoe/*.json)."""
    vocab_size: int = 50280
    hidden_size: int = 1024
    num_hidden_layers: int = 20
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    intermediate_size: int = 2816          # per-head intermediate width I = E * d_e
    mhffnmoe_num_heads: int = 8
    mhffnmoe_num_kuv_heads: int = 8
    mhffnmoe_num_experts: int = 11
    mhffnmoe_apply_rmsnorm: bool = True
    mhffnmoe_skip_linear: bool = False
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    mlp_bias: bool = False                  # bias of w_self / w_self_2 (modeling_mhffnmoe.py:337-338); off in every shipped config

    @staticmethod
    def lm_370m():
        """configs/mhffnmoe/configure-2-mhffnmoe-TriDao-350M.json with the 50280-entry vocabulary."""
        return LMConfig()

    @staticmethod
    def lm_128m():
        """configs/mhffnmoe/configure-1-tinymhffnmoe.json: hidden 768, 10 layers, 8 FFN heads of 96, 8 x 256."""
        return LMConfig(hidden_size=768, num_hidden_layers=10, num_attention_heads=12, num_key_value_heads=12,
                        intermediate_size=2048, mhffnmoe_num_heads=8, mhffnmoe_num_kuv_heads=8, mhffnmoe_num_experts=8,
                        mhffnmoe_apply_rmsnorm=False, tie_word_embeddings=True)

    @staticmethod
    def lm_1p3b():
        """configs/mhffnmoe/configure-3-mhffnmoe-TriDao-1.3B.json."""
        return LMConfig(hidden_size=2048, num_hidden_layers=20, num_attention_heads=32, num_key_value_heads=32,
                        intermediate_size=5632, mhffnmoe_num_heads=16, mhffnmoe_num_kuv_heads=16, mhffnmoe_num_experts=22)


class RMSNorm(nn.Module):
    """fp32 statistics, weight applied after the cast back (modeling_mhffnmoe.py:82-87)."""

    def __init__(self, n, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(n))
        self.eps = eps

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.bfloat16:
            # one kernel each way; differs from the expression below only in where the result is rounded to
            # bf16 (after the weight instead of before it)
            from . import lm_ops
            if x.shape[-1] in lm_ops.NORM_SIZES:
                return lm_ops.RMSNormFunction.apply(x, self.weight, self.eps)
            return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)
        dt = x.dtype
        x = x.float()
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps)
        return self.weight * x.to(dt)


def rotary_tables(S, head_dim, theta, device, dtype, first=0):
    """cos/sin [S, head_dim] of positions first .. first+S-1 as the reference builds them (fp32 angles, duplicated
    halves, cast to the activations' dtype)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64, device=device).float() / head_dim))
    ang = torch.arange(first, first + S, device=device).float()[:, None] * inv_freq[None, :]
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


class _Rotary(torch.autograd.Function):
    """x*cos + rotate_half(x)*sin (modeling_mhffnmoe.py:178-206) written on the two halves of the head
    dimension, four element-wise kernels each way and nothing saved but the tables:
    y1 = x1 c1 - x2 s1,  y2 = x2 c2 + x1 s2;   dx1 = g1 c1 + g2 s2,  dx2 = g2 c2 - g1 s1."""

    @staticmethod
    def forward(ctx, x, cos, sin):
        ctx.save_for_backward(cos, sin)
        h = x.shape[-1] // 2
        x1, x2, y = x[..., :h], x[..., h:], torch.empty_like(x)
        torch.mul(x1, cos[..., :h], out=y[..., :h]).addcmul_(x2, sin[..., :h], value=-1)
        torch.mul(x2, cos[..., h:], out=y[..., h:]).addcmul_(x1, sin[..., h:])
        return y

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        h = g.shape[-1] // 2
        g1, g2, dx = g[..., :h], g[..., h:], torch.empty_like(g)
        torch.mul(g1, cos[..., :h], out=dx[..., :h]).addcmul_(g2, sin[..., h:])
        torch.mul(g2, cos[..., h:], out=dx[..., h:]).addcmul_(g1, sin[..., :h], value=-1)
        return dx, None, None


def _attend_with_prefix(q, kp, vp, k, v, gqa):
    """Attention of S queries over P earlier positions (kp, vp: all visible) followed by their own S positions (k, v:
    causal).  On a GPU, as two calls of the library attention that return their log-sum-exp, merged exactly
    (o = o1 e^(l1-l) + o2 e^(l2-l), l = log(e^l1 + e^l2)): its causal kernel on the square part is several times faster
    than a masked call over the rectangle.  Elsewhere (CPU, grouped K/V heads) one call with a causal mask aligned to the
    lower right corner."""
    if q.is_cuda and not gqa and q.dtype in (torch.bfloat16, torch.float16):
        try:
            op = torch.ops.aten._scaled_dot_product_cudnn_attention
            o1, l1 = op(q, kp, vp, None, True, 0.0, False, False)[:2]
            o2, l2 = op(q, k, v, None, True, 0.0, True, False)[:2]
            l = torch.logaddexp(l1, l2)
            return (o1.float() * (l1 - l).exp() + o2.float() * (l2 - l).exp()).to(q.dtype)
        except (RuntimeError, AttributeError, TypeError):
            pass   # this build of torch has no such kernel for these shapes: the masked call below
    from torch.nn.attention.bias import causal_lower_right
    kk, vv = torch.cat((kp, k), dim=2), torch.cat((vp, v), dim=2)
    return F.scaled_dot_product_attention(q, kk, vv, attn_mask=causal_lower_right(q.shape[2], kk.shape[2]), enable_gqa=gqa)


class Attention(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.nh, self.nkv = cfg.num_attention_heads, cfg.num_key_value_heads
        self.hd = cfg.hidden_size // cfg.num_attention_heads
        self.q_proj = nn.Linear(cfg.hidden_size, self.nh * self.hd, bias=False)
        self.k_proj = nn.Linear(cfg.hidden_size, self.nkv * self.hd, bias=False)
        self.v_proj = nn.Linear(cfg.hidden_size, self.nkv * self.hd, bias=False)
        self.o_proj = nn.Linear(self.nh * self.hd, cfg.hidden_size, bias=False)

    def forward(self, x, cos, sin, kv_out=None, link=None):
        """``kv_out``: optional (k_cache, v_cache) of one layer, [B, n_kv, T_max, hd]; the keys (rotated) and values of
        the S positions are stored at [0, S) for later ``decode`` calls.
        ``link``: optional SequenceLink when a sequence is split over two ranks: the rank with the earlier part sends
        its keys and values on, the rank with the later part receives them and attends over both parts."""
        B, S, _ = x.shape
        q = self.q_proj(x).view(B, S, self.nh, self.hd)
        k = self.k_proj(x).view(B, S, self.nkv, self.hd)
        v = self.v_proj(x).view(B, S, self.nkv, self.hd).transpose(1, 2)
        if x.is_cuda and x.dtype == torch.bfloat16 and self.hd % 16 == 0:
            from . import lm_ops
            ct, st = lm_ops.rotary_tables_f32(cos, sin)
            q = lm_ops.RotaryFunction.apply(q, ct, st).transpose(1, 2)
            k = lm_ops.RotaryFunction.apply(k, ct, st).transpose(1, 2)
        else:
            q, k = _Rotary.apply(q.transpose(1, 2), cos, sin), _Rotary.apply(k.transpose(1, 2), cos, sin)
        if kv_out is not None:
            kv_out[0][:, :, :S].copy_(k)
            kv_out[1][:, :, :S].copy_(v)
        if link is not None and link.recv_from is not None:
            kp, vp = link.receive()
            if link.send_to is not None:
                link.send(torch.cat((kp, k), dim=2), torch.cat((vp, v), dim=2))
            o = _attend_with_prefix(q, kp, vp, k, v, self.nkv != self.nh)
        else:
            if link is not None and link.send_to is not None:
                link.send(k, v)
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.nkv != self.nh)
        return self.o_proj(o.transpose(1, 2).reshape(B, S, self.nh * self.hd))

    def decode(self, x, cos_p, sin_p, k_cache, v_cache, pos):
        """One new token per sequence: x [B,1,hidden] at position ``pos`` (a Python int: the same for every sequence),
        rotary tables of that position [1, hd]; appends this token's key and value to the layer's cache at ``pos`` and
        attends over positions [0, pos] (the cache update of modeling_mhffnmoe.py:568-571, as generation uses it)."""
        B = x.shape[0]
        q = self.q_proj(x).view(B, 1, self.nh, self.hd).transpose(1, 2)
        k = self.k_proj(x).view(B, 1, self.nkv, self.hd).transpose(1, 2)
        v = self.v_proj(x).view(B, 1, self.nkv, self.hd).transpose(1, 2)
        q, k = _Rotary.apply(q, cos_p, sin_p), _Rotary.apply(k, cos_p, sin_p)
        k_cache[:, :, pos:pos + 1].copy_(k)
        v_cache[:, :, pos:pos + 1].copy_(v)
        o = F.scaled_dot_product_attention(q, k_cache[:, :, :pos + 1], v_cache[:, :, :pos + 1], is_causal=False,
                                           enable_gqa=self.nkv != self.nh)
        return self.o_proj(o.transpose(1, 2).reshape(B, 1, self.nh * self.hd))


class _HeadNorm(nn.Module):
    def __init__(self, H, dh):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(H, dh))


class MHFFN(nn.Module):
    """The reference's FFN layer (modeling_mhffnmoe.py:256-431) with its parameter names; the arithmetic is ``ffn``."""

    def __init__(self, cfg, ffn):
        super().__init__()
        self.cfg, self.ffn = cfg, ffn
        H, Hk, hid, I = cfg.mhffnmoe_num_heads, cfg.mhffnmoe_num_kuv_heads, cfg.hidden_size, cfg.intermediate_size
        dh = hid // H
        if not cfg.mhffnmoe_skip_linear:
            self.w_self = nn.Linear(hid, hid, bias=cfg.mlp_bias)
            self.w_self_2 = nn.Linear(hid, hid, bias=cfg.mlp_bias)
        else:
            self.w_self = self.w_self_2 = None
        self.gate_weight = nn.Parameter(torch.empty(I, dh * Hk))
        self.up_weight = nn.Parameter(torch.empty(I, dh * Hk))
        self.down_weight = nn.Parameter(torch.empty(I, dh * Hk))
        self.router = nn.Parameter(torch.empty(H, dh, cfg.mhffnmoe_num_experts))
        self.q_norm = _HeadNorm(H, dh)

    def forward(self, x):
        c = self.cfg
        p = {"w_self": None if self.w_self is None else self.w_self.weight,
             "w_self_2": None if self.w_self_2 is None else self.w_self_2.weight,
             "gate_weight": self.gate_weight, "up_weight": self.up_weight, "down_weight": self.down_weight,
             "router": self.router, "q_norm": self.q_norm.weight}
        if self.w_self is not None and self.w_self.bias is not None:
            p["w_self_bias"], p["w_self_2_bias"] = self.w_self.bias, self.w_self_2.bias
        return self.ffn(x, p, H=c.mhffnmoe_num_heads, Hkuv=c.mhffnmoe_num_kuv_heads, E=c.mhffnmoe_num_experts,
                        apply_rmsnorm=c.mhffnmoe_apply_rmsnorm, eps=c.rms_norm_eps)


class DecoderLayer(nn.Module):
    def __init__(self, cfg, ffn):
        super().__init__()
        self.self_attn = Attention(cfg)
        self.mlp = MHFFN(cfg, ffn)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)

    def forward(self, h, cos, sin, kv_out=None, link=None):
        h = h + self.self_attn(self.input_layernorm(h), cos, sin, kv_out, link)
        return h + self.mlp(self.post_attention_layernorm(h))

    def decode(self, h, cos_p, sin_p, k_cache, v_cache, pos):
        h = h + self.self_attn.decode(self.input_layernorm(h), cos_p, sin_p, k_cache, v_cache, pos)
        return h + self.mlp(self.post_attention_layernorm(h))


class _Body(nn.Module):
    def __init__(self, cfg, ffn):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList(DecoderLayer(cfg, ffn) for _ in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)


class SequenceLink:
    """One rank's place in a sequence that is split into consecutive parts over ranks (a prefill on more GPUs than
    there are sequences).  Per layer, the rank of part p receives the keys and values of positions [0, first) from the
    rank of part p-1 and, unless it holds the last part, sends those of [0, first + S) on to the rank of part p+1 --
    point-to-point messages (NCCL send/recv on GPUs), the one exchange this split needs: the FFN, the projections and
    the norms are position-wise, and attention needs the earlier positions' keys and values only.  All receives of a
    forward pass are posted when it starts and the sends are not waited for until it ends, so the messages of later
    layers travel while earlier layers compute."""

    def __init__(self, first, recv_from=None, send_to=None, group=None):
        self.first, self.recv_from, self.send_to, self.group = first, recv_from, send_to, group
        self._recv, self._sent, self._layer = [], [], 0

    def start(self, cfg, batch, device, dtype):
        """Called by DecoderLM.hidden before the first layer."""
        import torch.distributed as dist
        self._recv, self._sent, self._layer = [], [], 0
        if self.recv_from is None:
            return
        hd = cfg.hidden_size // cfg.num_attention_heads
        for _ in range(cfg.num_hidden_layers):
            kp = torch.empty((batch, cfg.num_key_value_heads, self.first, hd), device=device, dtype=dtype)
            vp = torch.empty_like(kp)
            self._recv.append((kp, vp, dist.irecv(kp, self.recv_from, group=self.group),
                               dist.irecv(vp, self.recv_from, group=self.group)))

    def send(self, k, v):
        import torch.distributed as dist
        k, v = k.contiguous(), v.contiguous()
        self._sent.append((k, v, dist.isend(k, self.send_to, group=self.group), dist.isend(v, self.send_to, group=self.group)))

    def receive(self):
        """Keys and values of the earlier positions for the layer now running (layers call in order)."""
        kp, vp, wk, wv = self._recv[self._layer]
        self._layer += 1
        wk.wait()
        wv.wait()
        return kp, vp

    def finish(self):
        """Called by DecoderLM.hidden after the last layer: the sent tensors may be released once their sends are done."""
        for _, _, wk, wv in self._sent:
            wk.wait()
            wv.wait()
        self._recv, self._sent = [], []


class KVCache:
    """Keys (rotated) and values of every layer: two tensors [layers, B, n_kv, T_max, head_dim]."""

    def __init__(self, cfg, batch, max_len, device, dtype=torch.bfloat16):
        hd = cfg.hidden_size // cfg.num_attention_heads
        shape = (cfg.num_hidden_layers, batch, cfg.num_key_value_heads, max_len, hd)
        self.k = torch.zeros(shape, device=device, dtype=dtype)
        self.v = torch.zeros(shape, device=device, dtype=dtype)

    def nbytes(self, length):
        """Bytes of keys and values a step that attends over ``length`` positions reads."""
        L, B, n, _, hd = self.k.shape
        return 2 * L * B * n * length * hd * self.k.element_size()


class DecoderLM(nn.Module):
    """ids [B,S] -> logits [B,S,vocab]; ``loss`` is the next-token cross entropy the reference trains with
    (labels = ids shifted by one, mean over B*(S-1) positions, computed in fp32)."""

    def __init__(self, cfg, ffn=None):
        super().__init__()
        if ffn is None:
            from .layer import mhffn_layer as ffn  # the CUDA layer; raises at call time without the library or a GPU
        self.cfg = cfg
        self.model = _Body(cfg, ffn)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight

    @torch.no_grad()
    def init_weights(self, seed=0, std=0.02):
        """Every matrix ~ N(0, std) from one seeded generator in sorted-name order; norm weights stay 1.  Parameters on
        the CPU are drawn from the CPU generator (what the fixtures use); a model built on a GPU (``with torch.device``)
        is drawn there with that device's generator -- the same seed gives the same weights on every rank, and a
        billion-parameter model is ready in milliseconds instead of a minute of host time per rank."""
        gens = {}
        for name, p in sorted(self.named_parameters()):
            if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
                p.fill_(1.0)
                continue
            g = gens.get(p.device)
            if g is None:
                g = gens[p.device] = torch.Generator(device=p.device).manual_seed(seed)
            if p.is_cuda:
                p.normal_(0.0, std, generator=g)
            else:
                p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
        return self

    def hidden(self, ids, cache=None, link=None):
        """``cache``: optional KVCache to fill with the keys and values of these positions (a prefill before decoding).
        ``link``: optional SequenceLink: ``ids`` are then the positions [link.first, link.first + S) of longer sequences
        whose other parts other ranks hold (everything but attention is position-wise)."""
        B, S = ids.shape
        h = self.model.embed_tokens(ids)
        hd = self.cfg.hidden_size // self.cfg.num_attention_heads
        cos, sin = rotary_tables(S, hd, self.cfg.rope_theta, ids.device, h.dtype, first=0 if link is None else link.first)
        if link is not None:
            link.start(self.cfg, B, ids.device, h.dtype)
        for i, layer in enumerate(self.model.layers):
            h = layer(h, cos, sin, None if cache is None else (cache.k[i], cache.v[i]), link)
        if link is not None:
            link.finish()
        return self.model.norm(h)

    def decode_step(self, ids, cache, pos):
        """ids [B,1], the token at position ``pos`` of every sequence; the cache holds positions [0, pos).  Returns the
        logits [B, vocab] for position pos + 1 and leaves this token's keys and values in the cache."""
        h = self.model.embed_tokens(ids)
        hd = self.cfg.hidden_size // self.cfg.num_attention_heads
        cos_p, sin_p = rotary_tables(1, hd, self.cfg.rope_theta, ids.device, h.dtype, first=pos)
        for i, layer in enumerate(self.model.layers):
            h = layer.decode(h, cos_p, sin_p, cache.k[i], cache.v[i], pos)
        return self.lm_head(self.model.norm(h)[:, 0])

    def forward(self, ids):
        return self.lm_head(self.hidden(ids))

    def loss(self, ids):
        logits = self.lm_head(self.hidden(ids)[:, :-1])          # the last position has no label
        V = logits.shape[-1]
        return F.cross_entropy(logits.float().reshape(-1, V), ids[:, 1:].reshape(-1))


def train_step(model, opt, ids, reducer=None):
    """One full training step: forward, backward, gradient exchange (``reducer``: dp.GradReducer or None), AdamW."""
    opt.zero_grad(set_to_none=True)
    loss = model.loss(ids)
    loss.backward()
    if reducer is not None:
        reducer.finish()
    opt.step()
    return loss.detach()


def param_count(model):
    return sum(p.numel() for p in model.parameters())


def train_flops_per_token(cfg, S):
    """6 x (matrix parameters touched per token) + causal attention (12 * L * hidden * S / 2), for MFU lines."""
    hid, L, V = cfg.hidden_size, cfg.num_hidden_layers, cfg.vocab_size
    hd = hid // cfg.num_attention_heads
    attn = hid * hd * (2 * cfg.num_attention_heads + 2 * cfg.num_key_value_heads)
    dh = hid // cfg.mhffnmoe_num_heads
    ffn = (0 if cfg.mhffnmoe_skip_linear else 2 * hid * hid) + 3 * cfg.mhffnmoe_num_heads * cfg.intermediate_size * dh
    return 6 * (L * (attn + ffn) + V * hid) + 6 * L * hid * S
