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
    returns how many tensors were reduced.

    As the callback of ``ffn.set_grad_ready_hook`` it is called as ``reduce(name, grad, param)`` from inside the
    backward.  Autograd would cast or copy the returned gradient on the compute stream while the reduction is still
    in flight on NCCL's stream, so in this mode the synchroniser TAKES the gradient (returns True, the backward
    hands None to autograd) and ``finish()`` stores the reduced tensor into ``.grad`` of the parameter, which it
    finds among ``params`` by storage address.  Gradients of tensors that are not in ``params`` (e.g. the
    concatenation of a shared low-rank factor and an adapter) are left to autograd, unreduced, and their names are
    collected in ``unclaimed``; reduce those after the backward (``all_reduce_module_gradients``).

    ``bucket_elems``: taken gradients with at most this many elements (biases, LayerNorm parameters) are not reduced
    one by one: ``finish()`` sums them all in ONE fp32 all-reduce of their concatenation, which costs one collective
    latency instead of one per tensor.

    ``comm_sms``: the tensor-core GEMMs are persistent kernels holding one CTA on every SM until they end, so a
    collective started meanwhile would find no SM to run on.  With ``comm_sms`` set, the GEMM grid is capped at
    ``SMs - comm_sms`` CTAs from the first started reduction until ``finish()``; GEMMs that run while nothing is in
    flight (the whole forward, the first gradient GEMMs) keep every SM.

    ``measure_tail``: record CUDA events around the waits of ``finish()``; ``tail_ms()`` then returns, per call, how
    long the compute stream stood still for the reductions (the part of the exchange that did not overlap).
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None, wire_dtype: Optional[torch.dtype] = None,
                 average: bool = False, comm_sms: Optional[int] = None, measure_tail: bool = False, params=None,
                 bucket_elems: int = 1 << 18):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.wire_dtype = wire_dtype
        self.average = average
        self.comm_sms = comm_sms
        self.measure_tail = measure_tail
        self._owners = {p.data_ptr(): p for p in params} if params is not None else {}
        self.bucket_elems = int(bucket_elems)
        self._small: List[tuple] = []
        self.unclaimed: List[str] = []
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

    def reduce(self, name: str, grad: torch.Tensor, param: Optional[torch.Tensor] = None) -> bool:
        owner = None
        if param is not None:  # called from inside a backward
            owner = self._owners.get(param.data_ptr())
            if owner is None or owner.shape != grad.shape:
                self.unclaimed.append(name)
                return False
        if self.world_size == 1:
            self.reduced_names.append(name)
            return False
        if owner is not None and grad.numel() <= self.bucket_elems:
            self._small.append((name, grad, owner))
            return True
        wire = grad
        if self.wire_dtype is not None and grad.dtype != self.wire_dtype:
            wire = grad.to(self.wire_dtype)
        if not wire.is_contiguous():
            wire = wire.contiguous()
        work = dist.all_reduce(wire, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        if not self._pending and grad.is_cuda:
            self._cap_gemm_grid(True)
        self._pending.append((name, grad, wire, work, owner))
        return owner is not None

    __call__ = reduce

    def finish(self) -> int:
        done = 0
        if self._small:
            flat = torch.cat([g.reshape(-1).to(torch.float32) for _, g, _ in self._small])
            small_work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        timed = bool(self.measure_tail and ((self._pending and self._pending[0][1].is_cuda) or
                                            (self._small and self._small[0][1].is_cuda)))
        if timed:
            before, after = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            before.record()
        for name, grad, wire, work, owner in self._pending:
            work.wait()
            if owner is None:
                if wire is not grad:
                    grad.copy_(wire)
                if self.average:
                    grad.div_(self.world_size)
            else:
                result = wire if wire.dtype == owner.dtype else wire.to(owner.dtype)
                if self.average:
                    result = result.div_(self.world_size)
                if owner.grad is None:
                    owner.grad = result
                else:
                    owner.grad.add_(result)
            self.reduced_names.append(name)
            done += 1
        if self._small:
            small_work.wait()
            if self.average:
                flat.div_(self.world_size)
            offset = 0
            for name, grad, owner in self._small:
                piece = flat[offset:offset + grad.numel()].view(grad.shape)
                piece = piece.clone() if owner.dtype == torch.float32 else piece.to(owner.dtype)  # own storage
                offset += grad.numel()
                if owner.grad is None:
                    owner.grad = piece
                else:
                    owner.grad.add_(piece)
                self.reduced_names.append(name)
                done += 1
            self._small.clear()
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


def owned_row_blocks(rows: int, world_size: int, rank: int, block_shift: int) -> range:
    """Indices of the ``2**block_shift``-row blocks of a ``rows``-row matrix that ``rank`` owns when the blocks are
    dealt round-robin (the ownership rule of ``leanffn_gemm``'s ``scatter_world`` mode)."""
    blocks = (rows + (1 << block_shift) - 1) >> block_shift
    return range(rank, blocks, world_size)


def handout_plan(rows: int, cols: int, itemsize: int, world_size: int, rank: int, block_shift: int):
    """Strided copy that covers exactly the row blocks ``rank`` owns in a row-major ``[rows, cols]`` matrix:
    ``(start_byte, pitch_bytes, width_bytes, height)`` for ``leanffn_copy_2d`` (same layout at source and
    destination).  ``rows`` must be a multiple of the block height."""
    block_rows = 1 << block_shift
    if rows % block_rows != 0:
        raise ValueError(f"{rows} rows are not a multiple of {block_rows}")
    block_bytes = block_rows * cols * itemsize
    return rank * block_bytes, world_size * block_bytes, block_bytes, len(owned_row_blocks(rows, world_size, rank, block_shift))


class ScatteredGradReducer:
    """Sum of dense weight gradients over the ranks, with the reduce-scatter half fused into the GEMM that
    produces the gradient.

    Every registered weight gets a slice of one symmetric (peer-mapped) buffer.  The weight-gradient GEMM does not
    store its tiles: its epilogue adds each tile straight into the replica of the rank that owns the tile's row
    block (``red.add`` over NVLink, 256-row blocks dealt round-robin so that all links carry traffic at any
    moment).  When a GEMM has finished on every rank, each rank holds the complete sum of its own blocks and hands
    them to the other ranks with copy-engine copies, which occupy no SM and run underneath the next GEMMs.
    Per step::

        reducer.begin_step()          # zero the owned blocks, synchronise the ranks
        out = ffn(x); out.backward(g) # weight gradients of registered weights come back as None
        reducer.finish()              # waits for the exchange; sets param.grad to the summed gradient

    Summation order across ranks is not fixed, so results are not bit-reproducible (bf16 gradients are also
    accumulated in bf16 at the owner).  Micro-batch accumulation: call ``begin_step`` once, run several
    backwards, then ``finish`` — every backward adds into the same blocks.

    ``finish`` makes ``param.grad`` a VIEW of the exchange buffer: the next ``begin_step`` zeroes part of that
    storage, so consume the gradient (optimizer step, or a copy) before it.  A gradient that some other path left
    in ``param.grad`` since ``begin_step`` (a shared matrix also used outside LeanFFN, whose contribution came
    through autograd) is added into the view on every rank's own replica only, i.e. it is NOT summed over ranks;
    reduce such contributions separately.  Registered weights must be bf16 or fp32 weights of bf16 products: the
    scattering epilogue exists in the tensor-core kernel only, so a model computing in fp32 keeps ``GradSync``.
    """

    BLOCK_SHIFT = 8  # 256 rows: the tile height of the weight-gradient GEMM

    def __init__(self, weights: Dict[str, torch.Tensor], group: Optional[dist.ProcessGroup] = None,
                 spare_sms: int = 2, barrier_limit_cycles: int = 0):
        import torch.distributed._symmetric_memory as symm

        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group if group is not None else dist.group.WORLD
        self.world_size, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world_size > 8:
            raise ValueError("the fused reduce-scatter addresses at most 8 replicas (one NVLink domain)")
        block_rows = 1 << self.BLOCK_SHIFT
        self._slices: Dict[str, tuple] = {}
        self._by_storage: Dict[int, str] = {}
        self._params: Dict[str, torch.Tensor] = {}
        offset = 0
        device = None
        for name, w in weights.items():
            if w.dim() != 2 or not w.is_cuda or not w.is_contiguous():
                raise ValueError(f"{name}: dense, contiguous 2-D CUDA weights only")
            if w.shape[0] % block_rows != 0:
                raise ValueError(f"{name}: {w.shape[0]} rows are not a multiple of {block_rows}")
            if w.dtype not in (torch.bfloat16, torch.float32):
                raise ValueError(f"{name}: {w.dtype} weights are not supported (bf16, or fp32 masters of bf16 products)")
            device = w.device
            nbytes = w.numel() * w.element_size()
            self._slices[name] = (offset, tuple(w.shape), w.dtype)
            self._by_storage[w.data_ptr()] = name
            self._params[name] = w
            offset += (nbytes + 255) // 256 * 256
        # flag words of the rank barrier (4 channels x 8 ranks x uint32) live behind the gradients in the same buffer
        self._flag_offset = offset
        offset += 256
        self._buffer = symm.empty(offset, dtype=torch.uint8, device=device)
        self._handle = symm.rendezvous(self._buffer, self.group.group_name)
        self._peer_bases = [int(p) for p in self._handle.buffer_ptrs]
        self._views = {name: self._buffer[off:off + torch.Size(shape).numel() * dt.itemsize]
                       .view(dt).view(shape) for name, (off, shape, dt) in self._slices.items()}
        self._side = torch.cuda.Stream(device)
        self._done: List[torch.cuda.Event] = []
        self._capped = False
        self._sms = torch.cuda.get_device_properties(device).multi_processor_count
        self._spare_sms = max(1, int(spare_sms))
        self._buffer.zero_()
        import ctypes
        self._flags = (ctypes.c_void_p * 8)(*[base + self._flag_offset for base in self._peer_bases])
        self._epochs = [0, 0, 0, 0]
        self._barrier_limit = int(barrier_limit_cycles)
        # every rank's flags (and gradients) are zero before any rank can signal: host-level rendezvous, once
        torch.cuda.synchronize(device)
        dist.barrier(self.group)

    def _barrier(self, channel: int, stream: Optional[torch.cuda.Stream] = None):
        """Rank barrier on ``stream`` through ``leanffn_peer_barrier``: the wait is bounded (``barrier_limit_cycles`` SM
        clocks, 0 = about 20 s) and a rank that never arrives makes the kernel record a status code and return; it
        neither hangs nor traps.  ``ops.check_device_status`` raises on that code at the caller's next check.
        (torch's own symmetric-memory ``barrier`` spins without limit when called with ``timeout_ms=0`` and traps the
        context when a non-zero timeout expires; neither is wanted underneath a training step.)"""
        from . import _native as N
        from . import ops
        self._epochs[channel] += 1
        stream = stream if stream is not None else torch.cuda.current_stream()
        N.check(N.lib.leanffn_peer_barrier(self._flags, self.rank, self.world_size, channel,
                                           self._epochs[channel] & 0xFFFFFFFF, self._barrier_limit,
                                           ops.status_word(self._buffer.device).data_ptr(), stream.cuda_stream),
                "leanffn_peer_barrier")

    def gradient(self, name: str) -> torch.Tensor:
        """This rank's replica of the summed gradient (valid after ``finish``)."""
        return self._views[name]

    def begin_step(self):
        """Zero the row blocks this rank owns and synchronise: no contribution may arrive before that."""
        block_rows = 1 << self.BLOCK_SHIFT
        for name, view in self._views.items():
            rows, cols = view.shape
            if rows % (block_rows * self.world_size) == 0:
                view.view(rows // (block_rows * self.world_size), self.world_size, block_rows * cols)[:, self.rank].zero_()
            else:
                view.zero_()
        self._barrier(0)

    def target(self, weight: torch.Tensor):
        """``(out, scatter)`` arguments of ``ops.gemm`` for the gradient of ``weight``, or None if not registered."""
        name = self._by_storage.get(weight.data_ptr())
        if name is None:
            return None
        offset = self._slices[name][0]
        return self._views[name], ([base + offset for base in self._peer_bases], self.BLOCK_SHIFT)

    def gradient_launched(self, weight: torch.Tensor):
        """Called right after the scattering GEMM of ``weight`` was enqueued on the current stream: queues, on a side
        stream, rank synchronisation -> copy-engine hand-out of the owned blocks -> rank synchronisation."""
        from . import ops

        name = self._by_storage[weight.data_ptr()]
        offset, (rows, cols), dtype = self._slices[name]
        if not self._capped:
            # the synchronisation kernels of the side stream (and NCCL's for the small tensors) need an SM while
            # persistent GEMMs hold the others
            ops.set_max_ctas(self._sms - self._spare_sms)
            self._capped = True
        ready = torch.cuda.Event()
        ready.record()
        self._side.wait_event(ready)
        first, pitch, width, height = handout_plan(rows, cols, dtype.itemsize, self.world_size, self.rank, self.BLOCK_SHIFT)
        with torch.cuda.stream(self._side):
            self._barrier(1, self._side)  # every rank's contributions have landed
            if height > 0:
                start = offset + first
                for shift in range(1, self.world_size):
                    peer = (self.rank + shift) % self.world_size
                    ops.copy_2d(self._peer_bases[peer] + start, pitch, self._peer_bases[self.rank] + start, pitch,
                                width, height, self._side)
            self._barrier(1, self._side)  # every rank's blocks have arrived here
            done = torch.cuda.Event()
            done.record()
        self._done.append(done)

    def finish(self) -> int:
        """Make the current stream wait for the exchanges started since ``begin_step``; point ``param.grad`` of
        every registered parameter at its summed gradient.  Returns the number of exchanges waited for."""
        from . import ops

        current = torch.cuda.current_stream()
        for event in self._done:
            current.wait_event(event)
        count = len(self._done)
        self._done.clear()
        if self._capped:
            ops.set_max_ctas(0)
            self._capped = False
        for name, w in self._params.items():
            if isinstance(w, torch.nn.Parameter) or w.requires_grad:
                view = self._views[name]
                stray = w.grad
                if stray is not None and stray.data_ptr() != view.data_ptr():
                    view.add_(stray.to(view.dtype))  # delivered by another path since begin_step: keep it
                w.grad = view
        return count


def all_reduce_module_gradients(module: torch.nn.Module, group=None, wire_dtype=None) -> int:
    """Blocking fallback: all-reduce every ``.grad`` of ``module`` after the backward (no overlap)."""
    sync = GradSync(group, wire_dtype)
    for name, p in module.named_parameters():
        if p.grad is not None:
            sync.reduce(name, p.grad)
    return sync.finish()
