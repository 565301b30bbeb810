"""Host-side multi-GPU plumbing for the operator: one process per GPU, tokens sharded, weights replicated.

The operator has no cross-token dependence, so inference shards batch rows with no communication
and data-parallel training needs exactly one exchange per step: the sum of the weight gradients
dK, dU, dV over ranks.  The reference has no distributed code; this is the plumbing a one-process-
per-GPU job needs around the drop-in layer.  Works with any torch.distributed backend (NCCL on
GPUs, gloo in the CPU tests)."""
import torch
import torch.distributed as dist


def shard_range(n, rank, world):
    """Contiguous, balanced [start, stop) of n items for `rank` of `world` (first n % world ranks get one more)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_tokens(Q, R, rank, world):
    """Batch-row shard of the token-carrying operands: Q [B,H,S,d_h], R [B,H,S,E] -> views for this rank."""
    a, b = shard_range(Q.shape[0], rank, world)
    return Q[a:b], R[a:b]


def allreduce_weight_grads(grads, group=None, average=False):
    """Sum (or mean) dK, dU, dV (any list of same-dtype, same-device tensors) over ranks with ONE collective.

    The tensors are packed into one flat bucket, reduced, and copied back in place, so each step
    costs a single all-reduce launch whatever the number of tensors.  Returns the list."""
    grads = list(grads)
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return grads
    flat = torch.cat([g.reshape(-1) for g in grads])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    if average:
        flat /= dist.get_world_size(group)
    off = 0
    for g in grads:
        n = g.numel()
        g.copy_(flat[off:off + n].view_as(g))
        off += n
    return grads


def max_over_ranks(value, device, group=None):
    """Largest value of a Python float across ranks (used for device-timed durations)."""
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
