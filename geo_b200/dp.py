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

    def __init__(self, world_size=None, group=None):
        self.group = group
        self.world = world_size if world_size is not None else dist.get_world_size(group)
        self.flat = None
        self.views = None
        self.bytes_per_step = 0

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
