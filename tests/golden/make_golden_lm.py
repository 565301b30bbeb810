"""Generate ``lm_tiny.npz``: a two-layer decoder LM composed from the UNMODIFIED reference modules.

    python tests/golden/make_golden_lm.py /path/to/reference

The reference's ``MHFFNMoEForCausalLM`` does not construct under the transformers release in this
image, so the model is assembled from the reference's own building blocks -- ``nn.Embedding``,
``MHFFNMoEDecoderLayer`` (attention + the eager FFN layer), ``MHFFNMoERMSNorm``, a bias-free head --
with rotary tables and the additive causal mask built as modeling_mhffnmoe.py:164-175 and its eager
attention (:505-520) expect them.  Parameters are drawn from a seeded generator in sorted-name order
under the names the reference's state dict uses, so the test can regenerate them; the file stores the
token ids, the logits, the loss and gradients of a few parameters.
"""
import os
import sys

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from make_golden import HERE, load_reference  # noqa: E402

CFG = dict(vocab_size=97, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
           intermediate_size=128, mhffnmoe_num_heads=2, mhffnmoe_num_kuv_heads=2, mhffnmoe_num_experts=2,
           mhffnmoe_apply_rmsnorm=True, rms_norm_eps=1e-5, rope_theta=10000.0)
B, S, SEED = 2, 24, 11


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python %s /path/to/reference" % os.path.basename(__file__))
    ref_root = sys.argv[1]
    C, M = load_reference(ref_root)
    cfg = C.MHFFNMoEConfig(mhffnmoe_use_flash=False, mhffnmoe_custom_init=True, max_position_embeddings=64, **CFG)
    cfg._attn_implementation = "eager"

    class LM(nn.Module):
        def __init__(self):
            super().__init__()
            self.model = nn.Module()
            self.model.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
            self.model.layers = nn.ModuleList(M.MHFFNMoEDecoderLayer(cfg, i) for i in range(cfg.num_hidden_layers))
            self.model.norm = M.MHFFNMoERMSNorm(cfg.hidden_size, eps=cfg.rms_norm_eps)
            self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)

        def forward(self, ids):
            h = self.model.embed_tokens(ids)
            hd = cfg.hidden_size // cfg.num_attention_heads
            inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, dtype=torch.int64).float() / hd))
            ang = torch.arange(S).float()[:, None] * inv_freq[None, :]
            emb = torch.cat((ang, ang), dim=-1)[None]
            pos = (emb.cos().to(h.dtype), emb.sin().to(h.dtype))
            mask = torch.full((S, S), torch.finfo(h.dtype).min).triu(1)[None, None]
            for layer in self.model.layers:
                h = layer(h, attention_mask=mask, position_embeddings=pos)[0]
            return self.lm_head(self.model.norm(h))

    lm = LM()
    g = torch.Generator().manual_seed(SEED)
    with torch.no_grad():
        for name, p in sorted(lm.named_parameters()):
            if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=g))
            else:
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
    ids = torch.randint(0, cfg.vocab_size, (B, S), generator=g)
    logits = lm(ids)
    loss = F.cross_entropy(logits[:, :-1].float().reshape(-1, cfg.vocab_size), ids[:, 1:].reshape(-1))
    loss.backward()
    out = {"ids": ids.numpy(), "logits": logits.detach().numpy(), "loss": loss.detach().numpy().reshape(1),
           "names": np.array(sorted(n for n, _ in lm.named_parameters()))}
    keep = ["model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.k_proj.weight",
            "model.layers.0.mlp.router", "model.layers.0.mlp.q_norm.weight", "model.layers.1.mlp.gate_weight",
            "model.layers.1.mlp.down_weight", "model.layers.1.mlp.w_self.weight", "model.layers.1.post_attention_layernorm.weight",
            "model.norm.weight", "lm_head.weight"]
    grads = dict(lm.named_parameters())
    for n in keep:
        out["g:" + n] = grads[n].grad.numpy()
    np.savez(os.path.join(HERE, "lm_tiny.npz"), **out)
    print("lm_tiny loss", float(loss), "params", sum(p.numel() for p in lm.parameters()))


if __name__ == "__main__":
    main()
