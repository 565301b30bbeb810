"""CPU, world_size 2 over gloo: the token-sharding and gradient-exchange plumbing around the operator.

The CUDA operator cannot run here, so each rank uses the CPU oracle as its local operator; what is
under test is the host logic of flashmhf_b200/dp.py: shards cover the batch exactly once, sharded
forward equals the full forward, and one bucketed all-reduce of dK, dU, dV reproduces the
full-batch weight gradients."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashmhf_b200 import dp
from oracle import mhffn_oracle as orc


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
        B, H, S, dh, E, de = 5, 2, 24, 32, 2, 16      # B = 5: uneven split over 2 ranks
        Q, K, U, V, R, dO = orc.make_op_inputs(B, H, S, dh, E, de, seed=21, dtype=torch.float64)
        R = R.double()
        a, b = dp.shard_range(B, rank, world)
        Qs, Rs = dp.shard_tokens(Q, R, rank, world)
        O_local = orc.mhffn_forward(Qs, K, U, V, Rs)
        dQ, dK, dU, dV, dR = orc.mhffn_backward(Qs, K, U, V, Rs, dO[a:b])
        dp.allreduce_weight_grads([dK, dU, dV])
        full = orc.mhffn_backward(Q, K, U, V, R, dO)
        errs = [orc.rel_l2(x, y) for x, y in zip((dK, dU, dV), full[1:4])]
        errs.append(orc.rel_l2(O_local, orc.mhffn_forward(Q, K, U, V, R)[a:b]))
        errs.append(orc.rel_l2(dQ, full[0][a:b]))
        # the same exchange with the weight gradients written into one bucket first and reduced under the dQ/dR half
        bucket = dp.WeightGradBucket(K)

        def weights_fn(views):
            for v, g in zip(views, orc.mhffn_backward(Qs, K, U, V, Rs, dO[a:b])[1:4]):
                v.copy_(g)

        dQ2, dR2 = dp.exchange_under_inputs(weights_fn, lambda: (dQ.clone(), dR.clone()), bucket)
        errs += [orc.rel_l2(x, y) for x, y in zip(bucket.views, full[1:4])]
        errs.append(orc.rel_l2(dQ2, full[0][a:b]))
        assert bucket.views[0].data_ptr() == bucket.flat.data_ptr() and bucket.flat.numel() == 3 * K.numel()
        t = dp.max_over_ranks(10.0 + rank, torch.device("cpu"))
        out.put((rank, (a, b), errs, t))
    finally:
        dist.destroy_process_group()


def test_shard_range_partitions_exactly():
    for n in (1, 5, 16, 17):
        for world in (1, 2, 3, 8):
            spans = [dp.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        dp.shard_range(4, 2, 2)


def test_single_process_allreduce_is_identity():
    g = [torch.arange(6.0).view(2, 3), torch.ones(4)]
    ref = [t.clone() for t in g]
    dp.allreduce_weight_grads(g)
    assert all(torch.equal(a, b) for a, b in zip(g, ref))


@pytest.mark.timeout(180)
def test_two_ranks_gloo_token_sharding_and_grad_exchange():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=150) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert [r[1] for r in res] == [(0, 3), (3, 5)]
    for _, _, errs, t in res:
        assert max(errs) < 1e-12
        assert t == 11.0
