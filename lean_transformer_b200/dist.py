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

    ``comm_sms``: the tensor-core GEMMs are persistent kernels holding one CTA on every SM until they end, so a
    collective started meanwhile would find no SM to run on.  With ``comm_sms`` set, the GEMM grid is capped at
    ``SMs - comm_sms`` CTAs from the first started reduction until ``finish()``; GEMMs that run while nothing is in
    flight (the whole forward, the first gradient GEMMs) keep every SM.

    ``measure_tail``: record CUDA events around the waits of ``finish()``; ``tail_ms()`` then returns, per call, how
    long the compute stream stood still for the reductions (the part of the exchange that did not overlap).
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None, wire_dtype: Optional[torch.dtype] = None,
                 average: bool = False, comm_sms: Optional[int] = None, measure_tail: bool = False):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.wire_dtype = wire_dtype
        self.average = average
        self.comm_sms = comm_sms
        self.measure_tail = measure_tail
        self._tail_events: List[tuple] = []
        self._pending: List[tuple] = []
        self.reduced_names: List[str] = []

    def _cap_gemm_grid(self, on: bool):
        if self.comm_sms is None:
            return
        from . import ops
        if on:
            sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
            ops.set_max_ctas(max(1, sms - int(self.comm_sms)))
        else:
            ops.set_max_ctas(0)

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
        if not self._pending and grad.is_cuda:
            self._cap_gemm_grid(True)
        self._pending.append((name, grad, wire, work))

    __call__ = reduce

    def finish(self) -> int:
        done = 0
        timed = self.measure_tail and self._pending and self._pending[0][1].is_cuda
        if timed:
            before, after = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            before.record()
        for name, grad, wire, work in self._pending:
            work.wait()
            if wire is not grad:
                grad.copy_(wire)
            if self.average:
                grad.div_(self.world_size)
            self.reduced_names.append(name)
            done += 1
        if timed:
            after.record()
            self._tail_events.append((before, after))
        if self._pending and self._pending[0][1].is_cuda:
            self._cap_gemm_grid(False)
        self._pending.clear()
        return done

    def tail_ms(self) -> List[float]:
        """Milliseconds the compute stream waited in each ``finish()`` so far (after a device synchronisation);
        clears the record."""
        out = [a.elapsed_time(b) for a, b in self._tail_events]
        self._tail_events.clear()
        return out


def all_reduce_module_gradients(module: torch.nn.Module, group=None, wire_dtype=None) -> int:
    """Blocking fallback: all-reduce every ``.grad`` of ``module`` after the backward (no overlap)."""
    sync = GradSync(group, wire_dtype)
    for name, p in module.named_parameters():
        if p.grad is not None:
            sync.reduce(name, p.grad)
    return sync.finish()
