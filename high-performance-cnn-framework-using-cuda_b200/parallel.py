"""Data-parallel host logic: one process per GPU, ``torch.distributed`` for the plumbing.

The reference is single-GPU (no collective anywhere in layer.cu / main.cu).  Two things shard:

* inference -- images are independent, so each rank takes a contiguous index range and there is
  no communication at all (``shard_range``);
* minibatch training -- each rank computes the summed gradient of its slice of the global batch
  (``Net.grad_batch``), the 2,368-float vectors are sum-all-reduced, and every rank applies the
  identical update ``params += (dt / global_batch) * G`` so parameters stay bit-identical across
  ranks (``DataParallelTrainer``).

Per-sample SGD does not shard: each step needs the previous step's parameters.

Two exchange mechanisms exist for the training path.  The default on GPUs is the library's own
(``DataParallel`` in the package: the exchange is fused into the update kernel as peer stores over
NVLink, see ``csrc/dp_exchange.cu``); ``DataParallelTrainer`` below is the portable fallback that
calls an injected all-reduce (NCCL on GPUs, gloo in the CPU tests).

The gradient function and the update function are injected, so the same driver runs on GPUs
(``Net`` methods + NCCL) and, in the CPU tests, on ``gloo`` ranks.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple


def shard_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous slice [lo, hi) of n items owned by ``rank``; sizes differ by at most one and the
    slices tile [0, n) in rank order."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank/world: %r/%r" % (rank, world))
    if n < 0:
        raise ValueError("negative item count")
    return (n * rank) // world, (n * (rank + 1)) // world


def batch_plan(n: int, global_batch: int):
    """[(first, size)] of the global batches of one epoch over n images in index order; the last
    batch may be smaller."""
    if global_batch <= 0:
        raise ValueError("global_batch must be positive")
    return [(first, min(global_batch, n - first)) for first in range(0, n, global_batch)]


def handle_exchange(dist):
    """An ``exchange`` callable for ``DataParallel``: all-gathers one bytes object per rank through
    ``torch.distributed`` (any backend) and returns them in rank order."""
    def exchange(handle: bytes):
        out = [None] * dist.get_world_size()
        dist.all_gather_object(out, handle)
        return out
    return exchange


class DataParallelTrainer:
    """Minibatch SGD over ``world`` ranks.

    grad_fn(lo, hi, out_grad)  fills ``out_grad`` (a tensor of ``grad_len`` floats on the rank's
                               device) with the summed gradient of images [lo, hi) at the current
                               parameters (zeros when lo == hi);
    update_fn(grad, scale)     applies ``params += scale * grad``;
    all_reduce(tensor)         in-place sum over ranks (``torch.distributed.all_reduce``); None
                               for a single rank.
    """

    def __init__(self, rank: int, world: int, grad_fn: Callable, update_fn: Callable,
                 all_reduce: Optional[Callable], grad_buffer, dt: float = 0.1):
        self.rank, self.world = rank, world
        self.grad_fn, self.update_fn, self.all_reduce = grad_fn, update_fn, all_reduce
        self.grad = grad_buffer
        self.dt = dt
        if world > 1 and all_reduce is None:
            raise ValueError("all_reduce is required when world > 1")

    def step(self, first: int, size: int) -> None:
        """One global batch: images [first, first+size) split over the ranks."""
        lo, hi = shard_range(size, self.rank, self.world)
        self.grad_fn(first + lo, first + hi, self.grad)
        if self.world > 1:
            self.all_reduce(self.grad)
        self.update_fn(self.grad, self.dt / float(size))

    def epoch(self, n: int, global_batch: int) -> int:
        steps = 0
        for first, size in batch_plan(n, global_batch):
            self.step(first, size)
            steps += 1
        return steps
