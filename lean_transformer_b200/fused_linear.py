"""Linear layer with dropout and the residual add in the GEMM's epilogue.

This is the tail of the reference's attention block (lean_transformer/attn.py:74-78):
``outputs = out_proj(x); outputs = dropout(outputs); outputs = outputs + residual.to(float32)``, computed as ONE
product whose epilogue adds the bias, rounds to the compute dtype (what ``out_proj`` returns under autocast), applies
the Philox dropout mask and adds the residual in the residual's own dtype (an fp32 residual stream gives an fp32
result, as in the reference).  The backward regenerates the mask from (seed, offset), like ``_LeanFFN`` does.
Works for ``nn.Linear`` and for ``GeneralizedLinear`` (dense, block-sparse, with low-rank terms).
"""
from typing import Optional

import torch
import torch.nn as nn

from . import _native as N
from . import ops
from .blocksparse.linear import (GeneralizedLinear, linear_backward_core, linear_forward_core, resolve_compute_dtype)
from .ffn import _projection_args, next_dropout_stream


class _LinearDropoutResidual(torch.autograd.Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, input, residual, weight, bias, lowrank_first, lowrank_second, forward_indices, backward_indices,
                matmul_op, p: float, training: bool):
        cdt = resolve_compute_dtype(input)
        x2d = ops.cast(input.reshape(-1, input.shape[-1]).contiguous(), cdt)
        tokens = x2d.shape[0]
        out_features = bias.shape[0] if bias is not None else (
            matmul_op.out_features if matmul_op is not None else
            forward_indices.shape[0] * weight.shape[-1] if forward_indices is not None else weight.shape[0])
        res2d = None
        if residual is not None:
            assert residual.shape[:-1] == input.shape[:-1] and residual.shape[-1] == out_features
            res2d = residual.reshape(-1, out_features).contiguous()
        use_dropout = bool(training and p)
        seed = offset = 0
        ctx._stream = None
        if use_dropout:
            seed, offset = next_dropout_stream(input.device, tokens * out_features, out_features)
            ctx._stream = (seed, offset)
        out_dtype = res2d.dtype if res2d is not None else cdt
        out2d, lowrank_hid = linear_forward_core(
            x2d, weight, bias, lowrank_first, lowrank_second, forward_indices, backward_indices, matmul_op, cdt,
            epilogue=N.EPI_DROPOUT_RESIDUAL, aux=res2d, dropout_p=p if use_dropout else 0.0, seed=seed,
            elem_offset=offset, out_dtype=out_dtype)
        ctx.save_for_backward(input, lowrank_hid, weight, lowrank_first, lowrank_second, forward_indices,
                              backward_indices)
        ctx._matmul_op, ctx._p, ctx._cdt = matmul_op, p, cdt
        ctx._residual_dtype = residual.dtype if residual is not None else None
        return out2d.view(*input.shape[:-1], out_features)

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        input, lowrank_hid, weight, lowrank_first, lowrank_second, forward_indices, backward_indices = ctx.saved_tensors
        needs = ctx.needs_input_grad
        cdt = ctx._cdt
        grad2d = grad_output.reshape(-1, grad_output.shape[-1]).contiguous()
        if ctx._stream is not None:
            seed, offset = ctx._stream
            dy2d = ops.dropout(grad2d, ctx._p, seed, offset, out_dtype=cdt)  # the forward's mask, regenerated
        else:
            dy2d = ops.cast(grad2d, cdt)
        x2d = ops.cast(input.reshape(-1, input.shape[-1]).contiguous(), cdt)
        g_in, g_w, g_b, g_l1, g_l2 = linear_backward_core(
            dy2d, x2d, lowrank_hid, weight, lowrank_first, lowrank_second, forward_indices, backward_indices,
            ctx._matmul_op, [needs[0], needs[2], needs[3], needs[4], needs[5]], cdt)
        if g_in is not None:
            g_in = ops.cast(g_in, input.dtype).view(input.shape)
        g_res = None
        if needs[1]:
            g_res = grad_output if grad_output.dtype == ctx._residual_dtype else grad_output.to(ctx._residual_dtype)
        return g_in, g_res, g_w, g_b, g_l1, g_l2, None, None, None, None, None


def linear_dropout_residual(input: torch.Tensor, linear: nn.Linear, residual: Optional[torch.Tensor] = None,
                            p: float = 0.0, training: bool = True) -> torch.Tensor:
    """``dropout(linear(input), p) + residual`` as one product with a fused epilogue.

    :param input: ``[..., in_features]`` CUDA tensor (fp32 or bf16; bf16 compute under ``torch.autocast``)
    :param linear: ``nn.Linear`` or ``GeneralizedLinear``
    :param residual: ``[..., out_features]`` or None; the result takes its dtype (fp32 residual stream -> fp32)
    :param p: dropout probability, applied only if ``training``
    """
    if not input.is_cuda:
        raise RuntimeError("linear_dropout_residual runs on CUDA tensors only (there is no CPU path)")
    if not isinstance(linear, (nn.Linear, GeneralizedLinear)):
        raise TypeError(f"expected nn.Linear or GeneralizedLinear, got {type(linear).__name__}")
    return _LinearDropoutResidual.apply(input, residual, linear.weight, linear.bias, *_projection_args(linear),
                                        float(p), bool(training))
