"""Data-parallel training of the SC CNN: one process per GPU, batch sharded across ranks.

The SC forward shards with no data-path exchange at all: activation generators restart for every
image and weight generators do not depend on the batch, so a rank's outputs are bit-identical to
the same images inside any larger batch.  The only exchange of a training step is the sum of the
parameter gradients, done here as one flat all-reduce (NCCL over NVLink on GPUs, gloo in the CPU
tests).  The reference has no distributed code; this is the part added around its training loop.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class GradientAllReduce:
    """Callable for :class:`geo_b200.train.TrainStep` (``grad_hook``): averages ``p.grad`` over the
    process group.  All gradients travel in one flat fp32 buffer that is allocated once and
    reused; parameters without a gradient contribute zeros so that every rank reduces the same
    layout.  The three phases are also available separately -- :meth:`pack` (gradients into the
    flat buffer), :meth:`reduce` (the collective) and :meth:`unpack` (average back into the
    gradients) -- so that a caller replaying CUDA graphs can keep ``pack`` and ``unpack`` inside
    its graphs and issue only the collective between them."""

    def __init__(self, world_size=None, group=None, check=True):
        self.group = group
        self.world = world_size if world_size is not None else dist.get_world_size(group)
        self.flat = None
        self.views = None
        self.bytes_per_step = 0
        self._check = check     # first use: all ranks compare buffer sizes (ValueError on a mismatch)

    def _ensure(self, params):
        n = sum(p.numel() for p in params)
        ref = params[0]
        if self.flat is None or self.flat.numel() != n or self.flat.device != ref.device:
            self.flat = torch.zeros(n, dtype=torch.float32, device=ref.device)
            self.bytes_per_step = 4 * n
            self.views, off = [], 0
            for p in params:
                self.views.append(self.flat[off:off + p.numel()].view(p.shape))
                off += p.numel()
            if self._check and self.world > 1 and dist.is_initialized():
                verify_layout([n], self.group)

    def pack(self, params):
        params = list(params)
        self._ensure(params)
        have = [(v, p.grad) for v, p in zip(self.views, params) if p.grad is not None]
        for v, p in zip(self.views, params):
            if p.grad is None:
                v.zero_()
        if have:
            torch._foreach_copy_([v for v, _ in have], [g for _, g in have])

    def reduce(self):
        dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group)

    def unpack(self, params):
        self.flat.div_(self.world)
        have = [(p.grad, v) for v, p in zip(self.views, list(params)) if p.grad is not None]
        if have:
            torch._foreach_copy_([g for g, _ in have], [v for _, v in have])

    def __call__(self, params):
        if self.world <= 1:
            return
        params = list(params)
        self.pack(params)
        self.reduce()
        self.unpack(params)


def shard_batch(inputs, targets, rank, world):
    """Contiguous equal shard of a global batch for ``rank`` (the global batch must divide)."""
    n = inputs.shape[0]
    if n % world:
        raise ValueError(f"global batch {n} does not divide over {world} ranks")
    k = n // world
    return inputs[rank * k:(rank + 1) * k], targets[rank * k:(rank + 1) * k]


def verify_layout(sizes, group=None):
    """Every rank must reduce buffers of the same sizes; a rank whose model differs would otherwise corrupt the
    sum or stall the collective.  Exchanges the size list once and raises ``ValueError`` on every rank if they
    disagree."""
    world = dist.get_world_size(group)
    got = [None] * world
    dist.all_gather_object(got, [int(s) for s in sizes], group=group)
    if any(g != got[0] for g in got):
        raise ValueError(f"gradient buffers differ between ranks: {got}")


class BucketedGradientAllReduce:
    """Gradient averaging that overlaps the backward pass (eager launches only).

    The parameters are cut into buckets of about ``bucket_bytes`` in reverse order -- the order in which
    the backward pass produces their gradients.  A hook on every parameter notices when the last gradient
    of a bucket has been accumulated, copies the bucket's gradients into its flat buffer and starts an
    asynchronous all-reduce of that buffer while autograd carries on with the earlier layers.  Calling the
    object after ``backward()`` (it has the ``grad_hook`` signature of
    :class:`geo_b200.train.TrainStep`) waits for the collectives on the current stream, starts the buckets
    that never filled (parameters without a gradient contribute zeros) and writes the averages back into
    ``p.grad``.  In the VGG-11-style network nine tenths of the gradient bytes belong to the last layers,
    whose gradients are ready first, so their exchange hides behind the backward pass of the wide early
    layers.

    ``collective=False`` keeps the packing and unpacking but skips the all-reduce: the difference between
    two timed runs is the exposed communication time."""

    def __init__(self, params, world_size=None, group=None, bucket_bytes=8 << 20, collective=True, check=True):
        self.params = list(params)
        self.group = group
        self.world = world_size if world_size is not None else dist.get_world_size(group)
        self.collective = collective and self.world > 1
        self.buckets = []      # each: dict(params=[...], flat=None, views=None, ready=0, work=None, launched=False)
        cur, cur_bytes = [], 0
        for p in reversed(self.params):
            cur.append(p)
            cur_bytes += p.numel() * 4
            if cur_bytes >= bucket_bytes:
                self.buckets.append(self._make_bucket(cur))
                cur, cur_bytes = [], 0
        if cur:
            self.buckets.append(self._make_bucket(cur))
        self.bytes_per_step = 4 * sum(p.numel() for p in self.params)
        if check and self.collective:   # before any hook exists: a refused layout must leave nothing behind
            verify_layout([b["flat"].numel() for b in self.buckets], group)
        self._bucket_of = {}
        self._handles = []
        for b in self.buckets:
            for p in b["params"]:
                self._bucket_of[id(p)] = b
                self._handles.append(p.register_post_accumulate_grad_hook(self._on_grad))

    @staticmethod
    def _make_bucket(params):
        n = sum(p.numel() for p in params)
        flat = torch.zeros(n, dtype=torch.float32, device=params[0].device)
        views, off = [], 0
        for p in params:
            views.append(flat[off:off + p.numel()].view(p.shape))
            off += p.numel()
        return {"params": list(params), "flat": flat, "views": views, "ready": 0, "work": None, "launched": False}

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles = []

    def _on_grad(self, p):
        b = self._bucket_of[id(p)]
        b["ready"] += 1
        if b["ready"] == len(b["params"]) and not b["launched"]:
            self._launch(b)

    def _launch(self, b):
        if b["flat"].is_cuda and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("BucketedGradientAllReduce launches collectives during backward; it cannot run "
                               "inside a CUDA graph capture (use GradientAllReduce with graph replay)")
        have = [(v, p.grad) for v, p in zip(b["views"], b["params"]) if p.grad is not None]
        for v, p in zip(b["views"], b["params"]):
            if p.grad is None:
                v.zero_()
        if have:
            torch._foreach_copy_([v for v, _ in have], [g for _, g in have])
        if self.collective:
            b["work"] = dist.all_reduce(b["flat"], op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        b["launched"] = True

    def __call__(self, params=None):
        for b in self.buckets:
            if not b["launched"]:
                self._launch(b)
        for b in self.buckets:
            if b["work"] is not None:
                b["work"].wait()     # the current stream waits; the host does not (NCCL)
                b["work"] = None
            if self.world > 1:
                b["flat"].div_(self.world)
            have = [(p.grad, v) for v, p in zip(b["views"], b["params"]) if p.grad is not None]
            if have:
                torch._foreach_copy_([g for g, _ in have], [v for _, v in have])
            b["ready"], b["launched"] = 0, False
