"""Data parallelism for the LeanFFN path: tokens are partitioned across ranks (they are independent through
LayerNorm, both GEMMs, the activation, dropout and the residual), parameters are replicated, and the only
exchange is the sum of parameter gradients (one process per GPU, torch.distributed / NCCL over NVLink).

The reference has no distributed code at all; this module is the token-partition counterpart of running its
LeanFFN under a data-parallel trainer.  ``GradSync`` starts each gradient's all-reduce the moment the backward
has produced it, so the output projection's reduction overlaps the input projection's GEMMs.
"""
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_tokens(total_tokens: int, world_size: int, rank: int) -> Tuple[int, int]:
    """(start, count) of this rank's contiguous token shard; the first ``total % world`` ranks get one extra."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of {world_size}")
    base, extra = divmod(total_tokens, world_size)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


class GradSync:
    """Sums gradients across the ranks of ``group`` with asynchronous all-reduces.

    ``reduce(name, grad)`` starts an in-place all-reduce (optionally through a lower-precision wire copy) and
    returns immediately; ``finish()`` blocks the current stream until every started reduction has landed and
    returns how many tensors were reduced.  Usable as the callback of ``ffn.set_grad_ready_hook``.
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None, wire_dtype: Optional[torch.dtype] = None,
                 average: bool = False):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.wire_dtype = wire_dtype
        self.average = average
        self._pending: List[tuple] = []
        self.reduced_names: List[str] = []

    def reduce(self, name: str, grad: torch.Tensor):
        if self.world_size == 1:
            self.reduced_names.append(name)
            return
        wire = grad
        if self.wire_dtype is not None and grad.dtype != self.wire_dtype:
            wire = grad.to(self.wire_dtype)
        if not wire.is_contiguous():
            wire = wire.contiguous()
        work = dist.all_reduce(wire, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self._pending.append((name, grad, wire, work))

    __call__ = reduce

    def finish(self) -> int:
        done = 0
        for name, grad, wire, work in self._pending:
            work.wait()
            if wire is not grad:
                grad.copy_(wire)
            if self.average:
                grad.div_(self.world_size)
            self.reduced_names.append(name)
            done += 1
        self._pending.clear()
        return done


def all_reduce_module_gradients(module: torch.nn.Module, group=None, wire_dtype=None) -> int:
    """Blocking fallback: all-reduce every ``.grad`` of ``module`` after the backward (no overlap)."""
    sync = GradSync(group, wire_dtype)
    for name, p in module.named_parameters():
        if p.grad is not None:
            sync.reduce(name, p.grad)
    return sync.finish()
