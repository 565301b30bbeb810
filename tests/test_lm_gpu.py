"""GPU: the decoder LM with the CUDA FFN layer (fused prologue + operator) in bf16, against the fixture made
from the unmodified reference modules in fp32, and against the same LM with the oracle as its FFN layer."""
import os

import numpy as np
import pytest
import torch

from flashmhf_b200 import lm
from oracle import mhffn_oracle as orc
from tests.golden_util import GOLDEN_DIR
from tests.test_lm_cpu import TINY, tiny_model

pytestmark = pytest.mark.gpu


def _cuda_copy(m, ffn=None):
    c = lm.DecoderLM(m.cfg, ffn=ffn)
    c.load_state_dict(m.state_dict())
    return c.cuda().to(torch.bfloat16)


def test_tiny_lm_bf16_cuda_ffn_matches_reference_fixture():
    z = np.load(os.path.join(GOLDEN_DIR, "lm_tiny.npz"))
    m, ids = tiny_model()
    c = _cuda_copy(m)
    logits = c(ids.cuda())
    assert orc.rel_l2(logits.float().cpu(), torch.from_numpy(z["logits"])) < 4e-2       # a whole bf16 model vs fp32
    loss = c.loss(ids.cuda())
    assert abs(float(loss.detach()) - float(z["loss"][0])) < 3e-2
    loss.backward()
    g = dict(c.named_parameters())
    for k in ("model.layers.1.mlp.gate_weight", "model.layers.1.mlp.down_weight", "model.layers.0.mlp.router", "lm_head.weight"):
        assert orc.rel_l2(g[k].grad.float().cpu(), torch.from_numpy(z["g:" + k])) < 8e-2, k


def test_tiny_lm_cuda_ffn_vs_oracle_ffn_same_precision():
    """Both models bf16 on the GPU; only the FFN layer differs (CUDA kernels vs torch restatement)."""
    m, ids = tiny_model()
    a, b = _cuda_copy(m), _cuda_copy(m, ffn=orc.mhffn_layer_forward)
    la, lb = a.loss(ids.cuda()), b.loss(ids.cuda())
    la.backward(); lb.backward()
    assert abs(float(la.detach()) - float(lb.detach())) < 2e-2
    ga, gb = dict(a.named_parameters()), dict(b.named_parameters())
    for k in ("model.layers.0.mlp.gate_weight", "model.layers.0.mlp.up_weight", "model.layers.1.mlp.down_weight",
              "model.layers.0.self_attn.q_proj.weight", "model.embed_tokens.weight"):
        assert orc.rel_l2(ga[k].grad.float(), gb[k].grad.float()) < 5e-2, k


def test_training_steps_reduce_the_loss_at_370m_layer_dims():
    """Two layers with the 370M model's widths, AdamW, a fixed batch: the loss must fall (the gradients point downhill)."""
    cfg = lm.LMConfig.lm_370m()
    cfg.num_hidden_layers, cfg.vocab_size = 2, 1024
    m = lm.DecoderLM(cfg).init_weights(seed=3).cuda().to(torch.bfloat16)
    opt = torch.optim.AdamW(m.parameters(), lr=1e-3, fused=True)
    ids = torch.randint(0, cfg.vocab_size, (2, 512), generator=torch.Generator().manual_seed(5)).cuda()
    losses = [float(lm.train_step(m, opt, ids)) for _ in range(8)]
    assert losses[-1] < losses[0] - 0.5, losses
    assert all(np.isfinite(losses))



def test_decode_steps_with_a_kv_cache_on_the_gpu():
    """bf16 on the GPU with the CUDA FFN layer (its decode-shaped, split forward): a prefill into the cache followed by
    single-token steps gives the full forward's logits at those positions, eagerly and replayed from a CUDA graph."""
    m, ids = tiny_model()
    c = _cuda_copy(m)
    ids = ids.cuda()
    with torch.no_grad():
        full = c(ids).float()
        cache = lm.KVCache(c.cfg, ids.shape[0], 32, "cuda")
        c.hidden(ids[:, :20], cache)
        for pos in range(20, 24):
            logits = c.decode_step(ids[:, pos:pos + 1], cache, pos).float()
            assert orc.rel_l2(logits, full[:, pos]) < 3e-2, pos
        # the last step once more from a graph (a fixed position per captured step, as the bench replays it)
        tok = ids[:, 23:24].clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            c.decode_step(tok, cache, 23)
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = c.decode_step(tok, cache, 23)
        g.replay()
        torch.cuda.synchronize()
        assert orc.rel_l2(out.float(), full[:, 23]) < 3e-2
