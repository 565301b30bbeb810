"""CPU: the minimal decoder LM (flashmhf_b200/lm.py) against a two-layer LM assembled from the unmodified
reference modules (fixture lm_tiny.npz, made by tests/golden/make_golden_lm.py).  The FFN layer function is
the CPU oracle here (the package has no CPU operator), so what this pins is everything AROUND the
operator: embeddings, rotary tables, grouped-query causal attention, norms, residuals, head, loss,
parameter names -- in fp32 to 1e-5.  A world_size-2 gloo run covers the overlapped gradient exchange."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashmhf_b200 import dp, lm
from oracle import mhffn_oracle as orc
from tests.golden_util import GOLDEN_DIR

TINY = dict(vocab_size=97, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
            intermediate_size=128, mhffnmoe_num_heads=2, mhffnmoe_num_kuv_heads=2, mhffnmoe_num_experts=2,
            mhffnmoe_apply_rmsnorm=True, rms_norm_eps=1e-5, rope_theta=10000.0)


def tiny_model(seed=11):
    """Same draw order as the fixture generator: sorted parameter names, then the token ids."""
    m = lm.DecoderLM(lm.LMConfig(**TINY), ffn=orc.mhffn_layer_forward)
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in sorted(m.named_parameters()):
            if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=g))
            else:
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
    ids = torch.randint(0, TINY["vocab_size"], (2, 24), generator=g)
    return m, ids


def test_parameter_names_are_the_reference_state_dict_names():
    z = np.load(os.path.join(GOLDEN_DIR, "lm_tiny.npz"))
    m, _ = tiny_model()
    assert sorted(n for n, _ in m.named_parameters()) == [str(n) for n in z["names"]]


def test_lm_matches_reference_modules_fp32():
    z = np.load(os.path.join(GOLDEN_DIR, "lm_tiny.npz"))
    m, ids = tiny_model()
    assert np.array_equal(ids.numpy(), z["ids"])
    logits = m(ids)
    assert orc.rel_l2(logits.detach(), torch.from_numpy(z["logits"])) < 1e-5
    loss = m.loss(ids)
    assert abs(float(loss) - float(z["loss"][0])) < 1e-5
    loss.backward()
    grads = dict(m.named_parameters())
    for k in z.files:
        if k.startswith("g:"):
            assert orc.rel_l2(grads[k[2:]].grad, torch.from_numpy(z[k])) < 2e-5, k


def test_decode_steps_with_a_kv_cache_equal_the_full_forward():
    """Prefill of the first 20 positions into a cache, then four single-token steps: each step's logits are the full
    forward's logits at that position (fp32, oracle FFN), and the cache ends up holding what a longer prefill stores."""
    m, ids = tiny_model()
    with torch.no_grad():
        full = m(ids)
        cache = lm.KVCache(m.cfg, ids.shape[0], 32, "cpu", torch.float32)
        m.hidden(ids[:, :20], cache)
        for pos in range(20, 24):
            logits = m.decode_step(ids[:, pos:pos + 1], cache, pos)
            assert (logits - full[:, pos]).abs().max() < 2e-5
        ref = lm.KVCache(m.cfg, ids.shape[0], 32, "cpu", torch.float32)
        m.hidden(ids, ref)
    assert (cache.k - ref.k).abs().max() < 1e-5 and (cache.v - ref.v).abs().max() < 1e-5
    assert cache.nbytes(24) == 2 * m.cfg.num_hidden_layers * 2 * m.cfg.num_key_value_heads * 24 * \
        (m.cfg.hidden_size // m.cfg.num_attention_heads) * 4


def test_flops_and_param_count_of_the_370m_config():
    cfg = lm.LMConfig.lm_370m()
    with torch.device("meta"):
        m = lm.DecoderLM(cfg, ffn=orc.mhffn_layer_forward)
    n = lm.param_count(m)
    assert 3.6e8 < n < 4.2e8
    # 6 * matrix parameters (embedding excluded, head included) + attention
    body = n - cfg.vocab_size * cfg.hidden_size - sum(p.numel() for k, p in m.named_parameters() if "norm" in k or "router" in k)
    assert lm.train_flops_per_token(cfg, 2048) == 6 * body + 6 * cfg.num_hidden_layers * cfg.hidden_size * 2048


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        m, ids = tiny_model()
        red = dp.GradReducer(buckets=dp.lm_buckets(m))
        opt = torch.optim.SGD(m.parameters(), lr=0.0)
        a, b = dp.shard_range(ids.shape[0], rank, world)
        for _ in range(2):                                   # two steps: the reducer re-arms itself
            loss = lm.train_step(m, opt, ids[a:b], red)
        ref, _ = tiny_model()
        ref.loss(ids).backward()                             # full batch on one process
        errs = {n: orc.rel_l2(p.grad, dict(ref.named_parameters())[n].grad) for n, p in m.named_parameters()}
        out.put((rank, float(loss), max(errs.values())))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_overlapped_gradient_exchange_world2_equals_full_batch():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [out.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, loss, err in res:
        assert err < 1e-5, (rank, err)


def test_grad_reducer_single_process_is_a_no_op():
    m, ids = tiny_model()
    red = dp.GradReducer(params=list(m.parameters()))
    assert red.world == 1 and not red._hooks
    lm.train_step(m, torch.optim.SGD(m.parameters(), lr=0.0), ids, red)
    assert all(p.grad is not None for p in m.parameters())


def _split_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        m, ids = tiny_model()
        S = ids.shape[1]
        a, b = dp.shard_range(S, rank, world)               # consecutive parts of every sequence
        link = lm.SequenceLink(first=a, recv_from=rank - 1 if rank > 0 else None,
                               send_to=rank + 1 if rank + 1 < world else None)
        with torch.no_grad():
            mine = m.hidden(ids[:, a:b], link=link)
            full = m.hidden(ids)
        out.put((rank, float((mine - full[:, a:b]).abs().max())))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_sequence_split_prefill_world3_equals_the_full_forward():
    """Every sequence cut into three consecutive parts, one per gloo rank: keys and values travel from part to part,
    each rank's hidden states are the full forward's at its positions (fp32, oracle FFN)."""
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_split_worker, args=(r, 3, port, out)) for r in range(3)]
    for p in procs:
        p.start()
    res = [out.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, err in res:
        assert err < 2e-5, (rank, err)
