"""The ``blocksparse_backend='triton'`` operator, re-implemented on the CUDA kernels of this package.

It keeps the interface of lean_transformer/blocksparse/triton_backend.py:18-79 (a callable object with
``forward_functional`` / ``backward_functional`` and weights of shape [1, nnz, block, block] ordered like
``layout.nonzero()``), but no Triton is involved: the same tensor-core block-sparse kernels run with
index tables built for that block order.  Unlike the Triton operator it accepts any block size and needs
no token padding; ``TRITON_PAD_TO`` is kept so callers that pad keep working.
"""
import os
from typing import Sequence, Tuple

import torch

from .. import ops
from ..utils import pad_to_multiple
from .layout import tables_from_layout_row_major
from .native_backend import _bs_dgrad, _bs_forward, _bs_wgrad

TRITON_PAD_TO = int(os.environ.get("TRITON_PAD_TO", "128"))


class TritonMatmulForLinearLayer:
    """Block-sparse ``input @ W.T`` with W given by its nonzero blocks in row-major layout order."""

    def __init__(self, layout: torch.BoolTensor, block_size: int):
        self.layout = layout.cpu().bool()
        self.block = int(block_size)
        self.mode, self.trans_a, self.trans_b = "dds", False, True
        self.out_features = self.layout.shape[0] * self.block
        self.in_features = self.layout.shape[1] * self.block
        self._host_tables = tables_from_layout_row_major(self.layout)
        self._device_tables = {}

    def _tables(self, device):
        key = str(device)
        if key not in self._device_tables:
            self._device_tables[key] = tuple(t.to(device).contiguous() for t in self._host_tables)
        return self._device_tables[key]

    def _check_weight(self, weight: torch.Tensor):
        nnz = int(self.layout.sum())
        if weight.ndim != 4 or tuple(weight.shape) != (1, nnz, self.block, self.block):
            raise ValueError(f"weights are not in triton format: expected {(1, nnz, self.block, self.block)}, "
                             f"got {tuple(weight.shape)}")

    def __call__(self, input: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """
        :param input: tensor [*batch_dims, in_features]
        :param weight: tensor [1, nnz_blocks, block_size, block_size]
        :returns: output tensor [*batch_dims, out_features]
        """
        return _TritonOrderMatmul.apply(input, weight, self)

    def forward_functional(self, input: torch.Tensor, weight: torch.Tensor
                           ) -> Tuple[torch.Tensor, Tuple[torch.Tensor, ...]]:
        """:returns: output tensor, tensors_to_save"""
        self._check_weight(weight)
        fwd, fwd_count, _, _, _ = self._tables(input.device)
        x2d = input.reshape(-1, input.shape[-1])
        assert x2d.data_ptr() == input.data_ptr(), "input must be contiguous"
        out = _bs_forward(x2d, weight.contiguous(), fwd, self.out_features, count=fwd_count)
        return out.view(*input.shape[:-1], self.out_features), (input, weight)

    def backward_functional(self, grad_output: torch.Tensor, saved_tensors: Sequence[torch.Tensor],
                            needs_input_grad: Tuple[bool, ...]):
        grad_input = grad_weight = None
        input_padded, weight = saved_tensors
        _, _, dgrad, dgrad_count, wgrad = self._tables(grad_output.device)
        x2d = input_padded.reshape(-1, input_padded.shape[-1]).contiguous()
        dy = grad_output.reshape(-1, grad_output.shape[-1]).contiguous()
        dy = ops.cast(dy, x2d.dtype)
        if needs_input_grad[0]:
            grad_input = _bs_dgrad(dy, weight.contiguous(), dgrad, self.in_features, count=dgrad_count)
            grad_input = grad_input.view(*grad_output.shape[:-1], self.in_features)
        if needs_input_grad[1]:
            # rows of padding in input_padded carry no gradient: only the first len(dy) tokens are read
            grad_weight = _bs_wgrad(dy, x2d[: dy.shape[0]], weight, wgrad, weight.dtype)
        return grad_input, grad_weight


class _TritonOrderMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, op: TritonMatmulForLinearLayer):
        flat = input.reshape(-1, input.shape[-1]).contiguous()
        out, saved = op.forward_functional(flat, weight)
        ctx.save_for_backward(*saved)
        ctx.op, ctx.input_shape = op, input.shape
        return out.view(*input.shape[:-1], out.shape[-1])

    @staticmethod
    def backward(ctx, grad_output):
        grad_input, grad_weight = ctx.op.backward_functional(
            grad_output.reshape(-1, grad_output.shape[-1]), ctx.saved_tensors, ctx.needs_input_grad[:2])
        if grad_input is not None:
            grad_input = grad_input.view(ctx.input_shape)
        return grad_input, grad_weight, None


__all__ = ["TritonMatmulForLinearLayer", "TRITON_PAD_TO", "pad_to_multiple"]
