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


class WeightGradBucket:
    """dK, dU and dV as three views of ONE contiguous buffer, so that their exchange is one all-reduce with no packing
    copy before it and no copy back after it: the backward kernels write straight into the views."""

    def __init__(self, like):
        """`like`: a K-shaped tensor ([H_kuv, E, d_e, d_h]); the views are contiguous tensors of that shape."""
        n = like.numel()
        self.flat = torch.empty(3 * n, dtype=like.dtype, device=like.device)
        self.views = tuple(self.flat[i * n:(i + 1) * n].view(like.shape) for i in range(3))


def exchange_under_inputs(weights_fn, inputs_fn, bucket, group=None, average=False):
    """Backward of one layer with the gradient exchange hidden under half of it.

    ``weights_fn(views)`` computes dK, dU, dV into ``bucket.views`` (first, although autograd order would put dQ first);
    the all-reduce of the bucket starts as soon as that work is enqueued and runs while ``inputs_fn()`` computes dQ and
    dR, which no other rank needs.  Returns what ``inputs_fn`` returns; on return the current stream has been made to wait
    for the reduced bucket.  With one rank it just calls the two functions."""
    weights_fn(bucket.views)
    work = None
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        work = dist.all_reduce(bucket.flat, op=dist.ReduceOp.SUM, group=group, async_op=True)
    out = inputs_fn()
    if work is not None:
        work.wait()
        if average:
            bucket.flat /= dist.get_world_size(group)
    return out


def max_over_ranks(value, device, group=None):
    """Largest value of a Python float across ranks (used for device-timed durations)."""
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


class GradReducer:
    """Data-parallel gradient exchange overlapped with the backward pass.

    Parameters are grouped into buckets (one per decoder layer for the LM in flashmhf_b200/lm.py: pass
    ``buckets`` as lists of parameters, else one bucket per ``bucket_bytes`` in reverse order).  When the
    last gradient of a bucket has been accumulated, its gradients are packed into one flat tensor,
    pre-divided by the world size and all-reduced asynchronously, so the exchange of layer l runs
    while the backward of layer l-1 computes.  ``finish()`` waits for all buckets and copies the means
    back into ``p.grad``; call it before the optimizer step.  With one rank it does nothing."""

    def __init__(self, params=None, buckets=None, bucket_bytes=64 << 20, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self._pending, self._hooks = [], []
        if buckets is None:
            buckets, cur, size = [], [], 0
            for p in reversed([p for p in params if p.requires_grad]):
                cur.append(p)
                size += p.numel() * p.element_size()
                if size >= bucket_bytes:
                    buckets.append(cur)
                    cur, size = [], 0
            if cur:
                buckets.append(cur)
        self.buckets = [[p for p in b if p.requires_grad] for b in buckets]
        self.buckets = [b for b in self.buckets if b]
        self._left = [len(b) for b in self.buckets]
        if self.world > 1:
            for i, b in enumerate(self.buckets):
                for p in b:
                    self._hooks.append(p.register_post_accumulate_grad_hook(lambda _p, i=i: self._ready(i)))

    def _ready(self, i):
        self._left[i] -= 1
        if self._left[i] == 0:
            self._launch(i)

    def _launch(self, i):
        ps = self.buckets[i]
        flat = torch.cat([p.grad.reshape(-1) for p in ps])
        flat /= self.world
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self._pending.append((work, flat, ps))

    def finish(self):
        if self.world == 1:
            return
        for i, n in enumerate(self._left):       # buckets whose parameters did not all receive a gradient this step
            if n != 0 and n != len(self.buckets[i]):
                raise RuntimeError("a gradient bucket was only partly filled; pass buckets that match the graph")
        for work, flat, ps in self._pending:
            work.wait()
            off = 0
            for p in ps:
                n = p.numel()
                p.grad.copy_(flat[off:off + n].view_as(p.grad))
                off += n
        self._pending.clear()
        self._left = [len(b) for b in self.buckets]

    def remove(self):
        for h in self._hooks:
            h.remove()
        self._hooks.clear()


def lm_buckets(model):
    """One bucket per decoder layer (in backward order), one for the head and final norm, one for the embedding."""
    layers = [list(l.parameters()) for l in model.model.layers]
    seen, out = set(), []
    head = [model.lm_head.weight] + list(model.model.norm.parameters())
    for group in [head] + layers[::-1] + [[model.model.embed_tokens.weight]]:
        g = [p for p in group if id(p) not in seen]
        seen.update(id(p) for p in g)
        if g:
            out.append(g)
    return out
