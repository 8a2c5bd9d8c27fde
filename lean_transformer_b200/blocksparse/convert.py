"""Converters between the two block-sparse weight storage orders of the reference.

The reference keeps two layouts of the same block-sparse matrix and states that they are not interchangeable
(lean_transformer/blocksparse/__init__.py:5-7):

* native (lean_transformer/blocksparse/linear.py:49): ``[in_features, blocks_per_input, block]``; flat block
  ``f = j * blocks_per_input + a`` is a ``[block(out), block(in)]`` matrix that multiplies input block ``j`` and
  adds into output block ``backward_indices[j, a]`` (lean_transformer/blocksparse/native_backend.py:9-76);
* Triton (lean_transformer/blocksparse/linear.py:51): ``[1, nnz, block, block]`` with the blocks in
  ``layout.nonzero()`` order (row-major over (out_block, in_block)), each again ``[block(out), block(in)]``.

Both are permutations of the same set of blocks, so a checkpoint written with one backend can be loaded into a
module built with the other.  Everything here is index work on the host or device of the given tensors.
"""
from typing import Tuple

import torch


def _native_block_coordinates(backward_indices: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(out_block, in_block) of every native flat block id, as two int64 vectors."""
    in_blocks, per_input = backward_indices.shape
    out_block = backward_indices.reshape(-1).to(torch.int64)
    in_block = torch.arange(in_blocks, device=backward_indices.device).repeat_interleave(per_input)
    return out_block, in_block


def native_to_triton_permutation(backward_indices: torch.Tensor, layout: torch.Tensor) -> torch.Tensor:
    """``perm`` with ``triton_blocks[k] = native_blocks[perm[k]]``.  Raises if the native index tensor does not
    describe exactly the nonzero blocks of ``layout`` (``layout`` is ``[out_blocks, in_blocks]`` boolean)."""
    out_block, in_block = _native_block_coordinates(backward_indices)
    in_blocks = layout.shape[1]
    key = out_block * in_blocks + in_block  # position in row-major (out, in) order
    nz = layout.to(torch.bool).reshape(-1).nonzero().reshape(-1).to(key.device)
    order = torch.argsort(key, stable=True)
    if key.numel() != nz.numel() or not torch.equal(key[order], nz):
        raise ValueError("backward_indices and layout describe different sets of blocks")
    return order


def native_to_triton_weight(weight: torch.Tensor, backward_indices: torch.Tensor, layout: torch.Tensor) -> torch.Tensor:
    """``[in_features, blocks_per_input, block]`` -> ``[1, nnz, block, block]``."""
    block = weight.shape[-1]
    perm = native_to_triton_permutation(backward_indices, layout).to(weight.device)
    return weight.reshape(-1, block, block)[perm].reshape(1, -1, block, block).contiguous()


def triton_to_native_weight(weight: torch.Tensor, backward_indices: torch.Tensor, layout: torch.Tensor) -> torch.Tensor:
    """``[1, nnz, block, block]`` -> ``[in_features, blocks_per_input, block]`` for the given native index tensor."""
    block = weight.shape[-1]
    in_blocks, per_input = backward_indices.shape
    perm = native_to_triton_permutation(backward_indices, layout).to(weight.device)
    native = torch.empty_like(weight.reshape(-1, block, block))
    native[perm] = weight.reshape(-1, block, block)
    return native.reshape(in_blocks * block, per_input, block).contiguous()


def native_weight_to_dense(weight: torch.Tensor, backward_indices: torch.Tensor, out_features: int) -> torch.Tensor:
    """The ``[out_features, in_features]`` matrix a native block-sparse weight stands for (zeros elsewhere)."""
    block = weight.shape[-1]
    in_blocks, per_input = backward_indices.shape
    out_block, in_block = _native_block_coordinates(backward_indices)
    dense = torch.zeros(out_features // block, in_blocks, block, block, dtype=weight.dtype, device=weight.device)
    dense[out_block.to(weight.device), in_block.to(weight.device)] = weight.reshape(-1, block, block)
    return dense.permute(0, 2, 1, 3).reshape(out_features, in_blocks * block).contiguous()


def triton_weight_to_dense(weight: torch.Tensor, layout: torch.Tensor) -> torch.Tensor:
    """The ``[out_features, in_features]`` matrix a Triton-ordered weight stands for."""
    block = weight.shape[-1]
    out_blocks, in_blocks = layout.shape
    coords = layout.to(torch.bool).nonzero().to(weight.device)
    dense = torch.zeros(out_blocks, in_blocks, block, block, dtype=weight.dtype, device=weight.device)
    dense[coords[:, 0], coords[:, 1]] = weight.reshape(-1, block, block)
    return dense.permute(0, 2, 1, 3).reshape(out_blocks * block, in_blocks * block).contiguous()


def dense_to_native_weight(dense: torch.Tensor, backward_indices: torch.Tensor, block: int) -> torch.Tensor:
    """Gather the blocks a native index tensor lists out of a dense ``[out_features, in_features]`` matrix."""
    out_features, in_features = dense.shape
    in_blocks, per_input = backward_indices.shape
    out_block, in_block = _native_block_coordinates(backward_indices)
    blocks = dense.reshape(out_features // block, block, in_features // block, block).permute(0, 2, 1, 3)
    picked = blocks[out_block.to(dense.device), in_block.to(dense.device)]
    return picked.reshape(in_blocks * block, per_input, block).contiguous()
