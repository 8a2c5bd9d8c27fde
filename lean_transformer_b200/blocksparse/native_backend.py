"""Block-sparse matmul over the reference's native weight layout, computed by the CUDA kernels.

Same call signatures as lean_transformer/blocksparse/native_backend.py:9-76: the weight is
[in_features, blocks_per_input, block]; input block j and slot a hold a [block(out) x block(in)] matrix
that feeds output block backward_indices[j, a].  Where the reference materialises every active output
block ([nnz * block, tokens]) and gathers with embedding_bag, the kernels here walk only the nonzero
blocks of each output tile.
"""
import weakref
from typing import Dict, Optional, Tuple

import torch

from .. import ops
from .layout import tables_from_native_indices

_TABLE_CACHE: Dict[tuple, tuple] = {}


def backward_indices_from_forward(forward_indices: torch.Tensor, blocks_per_input: int) -> torch.Tensor:
    """Invert forward_indices: entry f = j * blocks_per_input + a listed under output block i means
    backward_indices[j, a] = i."""
    out_blocks, per_row = forward_indices.shape
    flat = forward_indices.to(torch.int64).flatten()
    owner = torch.arange(out_blocks, device=forward_indices.device).repeat_interleave(per_row)
    backward = torch.empty(flat.numel(), dtype=torch.int64, device=forward_indices.device)
    backward[flat] = owner
    return backward.view(-1, blocks_per_input)


def _validate_indices(forward_indices: Optional[torch.Tensor], backward_indices: Optional[torch.Tensor],
                      blocks_per_input: int):
    """Index buffers come from a state dict or straight from the caller, and the kernels use their entries as
    addresses without looking at them again: check them once, on the host, when their tables are first built."""
    if forward_indices is not None:
        if forward_indices.dim() != 2 or forward_indices.numel() == 0 or forward_indices.numel() % blocks_per_input:
            raise ValueError(f"forward_indices of shape {tuple(forward_indices.shape)} do not describe weight blocks "
                             f"with {blocks_per_input} blocks per input block")
        flat = forward_indices.to(torch.int64).flatten()
        if not bool(torch.equal(torch.sort(flat).values, torch.arange(flat.numel(), device=flat.device))):
            raise ValueError("forward_indices must list every weight block id 0 .. in_blocks * blocks_per_input - 1 "
                             "exactly once")
    if backward_indices is not None:
        if backward_indices.dim() != 2 or backward_indices.shape[1] != blocks_per_input:
            raise ValueError(f"backward_indices of shape {tuple(backward_indices.shape)} do not match a weight with "
                             f"{blocks_per_input} blocks per input block")
        low, high = int(backward_indices.min().item()), int(backward_indices.max().item())
        out_blocks = forward_indices.shape[0] if forward_indices is not None else high + 1
        if low < 0 or high >= out_blocks:
            raise ValueError(f"backward_indices entries must lie in [0, {out_blocks}); found [{low}, {high}]")
        if forward_indices is None:
            counts = torch.bincount(backward_indices.flatten().to(torch.int64), minlength=out_blocks)
            if not bool((counts == counts[0]).all()):
                raise ValueError("backward_indices describe an unbalanced layout (output blocks with different numbers "
                                 "of weight blocks); the native order needs a balanced one")
        elif forward_indices.shape[0] * forward_indices.shape[1] != backward_indices.numel():
            raise ValueError("forward_indices and backward_indices describe different numbers of weight blocks")
        else:
            owner = backward_indices.to(torch.int64).flatten()[forward_indices.to(torch.int64).flatten()]
            expect = torch.arange(forward_indices.shape[0], device=owner.device).repeat_interleave(forward_indices.shape[1])
            if not bool(torch.equal(owner, expect)):
                raise ValueError("forward_indices and backward_indices contradict each other")


def native_tables(forward_indices: Optional[torch.Tensor], backward_indices: Optional[torch.Tensor],
                  blocks_per_input: int):
    """(forward, dgrad, wgrad) pair tables on the indices' device.  Cached per index-tensor OBJECT (module
    buffers live as long as their module); the entry is dropped when the tensor is collected and ignored if
    the tensor was modified in place or re-pointed."""
    anchor = forward_indices if forward_indices is not None else backward_indices
    other = backward_indices if forward_indices is not None else None
    key = (id(anchor), id(other) if other is not None else 0, blocks_per_input)
    stamp = (anchor._version, anchor.data_ptr(), other._version if other is not None else 0,
             other.data_ptr() if other is not None else 0)
    hit = _TABLE_CACHE.get(key)
    if hit is not None and hit[0]() is anchor and (other is None or hit[1]() is other) and hit[2] == stamp:
        return hit[3]
    _validate_indices(forward_indices, backward_indices, blocks_per_input)
    if backward_indices is None:
        backward_indices = backward_indices_from_forward(forward_indices, blocks_per_input)
    if forward_indices is None:
        in_blocks, per_col = backward_indices.shape
        out_blocks = int(backward_indices.max().item()) + 1
        order = torch.argsort(backward_indices.flatten(), stable=True)  # flat ids grouped by owning output block
        forward_indices = order.view(out_blocks, -1).to(torch.int32)
    tables = tables_from_native_indices(forward_indices, backward_indices)
    drop = lambda _r, _k=key: _TABLE_CACHE.pop(_k, None)  # noqa: E731
    _TABLE_CACHE[key] = (weakref.ref(anchor, drop), weakref.ref(other, drop) if other is not None else None, stamp,
                         tables)
    return tables


def _bs_forward(x2d: torch.Tensor, weight: torch.Tensor, fwd_table: torch.Tensor, out_features: int,
                out: Optional[torch.Tensor] = None, bias=None, a2=None, b2=None,
                out_dtype: Optional[torch.dtype] = None, count: Optional[torch.Tensor] = None, **epilogue) -> torch.Tensor:
    """Y = X . W^T over the nonzero blocks; ``epilogue`` forwards fused-epilogue arguments of ``ops.gemm``."""
    block = weight.shape[-1]
    num_blocks = weight.numel() // (block * block)
    return ops.gemm(x2d, weight, M=x2d.shape[0], N_=out_features, K=x2d.shape[1], out=out, bias=bias, a2=a2, b2=b2,
                    out_dtype=out_dtype, bs_mode=1, bs_block=block, bs_nnz=fwd_table.shape[1],
                    bs_num_blocks=num_blocks, bs_index=fwd_table, bs_count=count, **epilogue)


def gate_and_linear_blocks_pair_up(fwd_table: torch.Tensor, count: Optional[torch.Tensor] = None) -> bool:
    """True if output blocks i and i + half (a gate block and its linear partner of a gated projection) read the
    same input blocks in the same order: the condition under which the gated activation can be fused into the
    block-sparse forward product.  The answer is remembered on the (cached, immutable) table tensor."""
    cached = getattr(fwd_table, "_leanffn_pairs_up", None)
    if cached is None:
        rows = fwd_table.shape[0]
        cached = rows % 2 == 0 and bool(torch.equal(fwd_table[:rows // 2, :, 1], fwd_table[rows // 2:, :, 1]))
        if cached and count is not None:
            cached = bool(torch.equal(count[:rows // 2], count[rows // 2:]))
        fwd_table._leanffn_pairs_up = cached
    return cached


def _bs_dgrad(dy2d: torch.Tensor, weight: torch.Tensor, dgrad_table: torch.Tensor, in_features: int,
              a2=None, b2=None, count: Optional[torch.Tensor] = None, **epilogue) -> torch.Tensor:
    """dX = dY . W over the nonzero blocks; ``epilogue`` = the activation-backward arguments of ``ops.gemm``
    (epilogue, act, aux, out, out2) when the product feeds an activation's backward directly."""
    block = weight.shape[-1]
    num_blocks = weight.numel() // (block * block)
    return ops.gemm(dy2d, weight, M=dy2d.shape[0], N_=in_features, K=dy2d.shape[1], b_mn_major=True, a2=a2, b2=b2,
                    bs_mode=2, bs_block=block, bs_nnz=dgrad_table.shape[1], bs_num_blocks=num_blocks,
                    bs_index=dgrad_table, bs_count=count, **epilogue)


def weight_blocks_pair_up(wgrad_table: torch.Tensor) -> bool:
    """True if weight blocks 2i and 2i+1 always read the same input block (native order with an even number of
    blocks per input block): one CTA can then produce both gradients from one tile of x.  Remembered on the
    (cached, immutable) table tensor."""
    cached = getattr(wgrad_table, "_leanffn_pairs_up", None)
    if cached is None:
        flat = wgrad_table.reshape(-1, 2)
        cached = flat.shape[0] % 2 == 0 and bool(torch.equal(flat[0::2, 1], flat[1::2, 1]))
        wgrad_table._leanffn_pairs_up = cached
    return cached


def _bs_wgrad(dy2d: torch.Tensor, x2d: torch.Tensor, weight_like: torch.Tensor, wgrad_table: torch.Tensor,
              out_dtype: torch.dtype) -> torch.Tensor:
    block = weight_like.shape[-1]
    num_blocks = weight_like.numel() // (block * block)
    out = torch.empty((num_blocks * block, block), dtype=out_dtype, device=dy2d.device)
    pairs = block == 128 and dy2d.dtype == torch.bfloat16 and weight_blocks_pair_up(wgrad_table)
    ops.gemm(dy2d, x2d, a_mn_major=True, b_mn_major=True, M=num_blocks * block, N_=block, K=dy2d.shape[0], out=out,
             bs_mode=3, bs_block=block, bs_nnz=1, bs_num_blocks=num_blocks, bs_index=wgrad_table, bs_wgrad_pairs=pairs)
    return out.view(weight_like.shape)


class _BlocksparseMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, forward_indices):
        in_features, blocks_per_input, block = weight.shape
        fwd, dgrad, wgrad = native_tables(forward_indices, None, blocks_per_input)
        x2d = input.reshape(-1, in_features).contiguous()
        out_features = forward_indices.shape[0] * block
        out = _bs_forward(x2d, weight.contiguous(), fwd, out_features)
        ctx.save_for_backward(input, weight)
        ctx.tables = (dgrad, wgrad)
        return out.view(*input.shape[:-1], out_features)

    @staticmethod
    def backward(ctx, grad_output):
        input, weight = ctx.saved_tensors
        dgrad, wgrad = ctx.tables
        dy = ops.cast(grad_output.reshape(-1, grad_output.shape[-1]).contiguous(), input.dtype)
        x2d = input.reshape(-1, input.shape[-1]).contiguous()
        grad_input = grad_weight = None
        if ctx.needs_input_grad[0]:
            grad_input = _bs_dgrad(dy, weight.contiguous(), dgrad, input.shape[-1]).view(input.shape)
        if ctx.needs_input_grad[1]:
            grad_weight = _bs_wgrad(dy, x2d, weight, wgrad, weight.dtype)
        return grad_input, grad_weight, None


def blocksparse_matmul(input: torch.Tensor, weight: torch.Tensor, forward_indices: torch.Tensor) -> torch.Tensor:
    """
    :param input: tensor [*batch_dims, in_features]
    :param weight: tensor [in_features, active_blocks_per_input, block_size]
    :param forward_indices: the first output of get_indices_from_layout(...)
    :returns: tensor [*batch_dims, out_features]
    """
    assert input.shape[-1] == weight.shape[0]
    return _BlocksparseMatmul.apply(input, weight, forward_indices)


def blocksparse_matmul_backward(grad_output: torch.Tensor, input: torch.Tensor, weight: torch.Tensor,
                                backward_indices: torch.Tensor, input_requires_grad: bool = True,
                                weight_requires_grad: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gradients of blocksparse_matmul w.r.t. input and / or weight without autograd."""
    assert input_requires_grad or weight_requires_grad, "computing backward but none of the inputs requires grad"
    in_features, blocks_per_input, block = weight.shape
    _, dgrad, wgrad = native_tables(None, backward_indices, blocks_per_input)
    dy = grad_output.reshape(-1, grad_output.shape[-1]).contiguous()
    x2d = input.reshape(-1, input.shape[-1]).contiguous()
    grad_input = grad_weight = torch.empty(0, device=grad_output.device)
    if input_requires_grad:
        grad_input = _bs_dgrad(dy, weight.contiguous(), dgrad, in_features).view(
            grad_output.shape[:-1] + input.shape[-1:])
    if weight_requires_grad:
        grad_weight = _bs_wgrad(dy, x2d, weight, wgrad, weight.dtype)
    return grad_input, grad_weight
