"""Two GPUs (skipped on a box with one): a sequence cut into two consecutive parts, one per rank, with the earlier
part's keys and values sent on by NCCL point-to-point messages -- bf16, CUDA FFN layer -- against the full forward."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashmhf_b200 import dp, lm
from oracle import mhffn_oracle as orc
from tests.test_lm_cpu import tiny_model

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        m, ids = tiny_model()
        c = lm.DecoderLM(m.cfg)
        c.load_state_dict(m.state_dict())
        c = c.cuda().to(torch.bfloat16)
        ids = ids.cuda()
        a, b = dp.shard_range(ids.shape[1], rank, world)
        link = lm.SequenceLink(first=a, recv_from=rank - 1 if rank > 0 else None, send_to=rank + 1 if rank + 1 < world else None)
        with torch.no_grad():
            for _ in range(2):
                mine = c.hidden(ids[:, a:b], link=link)
            full = c.hidden(ids)
        torch.cuda.synchronize()
        out.put((rank, float(orc.rel_l2(mine.float(), full[:, a:b].float()))))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_sequence_split_over_two_gpus_equals_the_full_forward():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [out.get(timeout=480) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, err in res:
        assert err < 3e-2, (rank, err)
