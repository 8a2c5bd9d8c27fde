"""LeanFFN on sm_100a kernels: same module API and the same memory-lean contract as the reference's
``lean_transformer/ffn.py`` (LeanFFN :14-132, _LeanFFN :135-321).

Forward: pre-LayerNorm -> input Linear (gated variants double the width) -> activation -> output Linear ->
[post-LayerNorm] -> dropout -> + residual.  Only ``input`` and ``pre_activation`` (plus the small low-rank
hiddens and the post-LN input when used) are kept for backward; the LayerNorm output and the activation
are rematerialised there.  The kernel schedule in bf16 is

  forward   LN kernel | GEMM1 (epilogue: bias + gated activation, writes pre_activation and hid)
            | GEMM2 (epilogue: bias + dropout + residual)
  backward  dropout(dY) | column sums | dgrad2 (epilogue: activation backward, writes dPre and rematerialised
            hid) | wgrad2 | LN kernel (remat) | wgrad1 | dgrad1 | LN backward (+ residual gradient)

Dropout masks are a pure function of (seed, offset, element index), so backward regenerates the forward's
mask from two integers instead of restoring RNG state (reference: ffn.py:243-245, :308-321).
"""
import os
from typing import Optional

import torch
import torch.nn as nn

from . import _native as N
from . import ops
from .blocksparse.linear import (GeneralizedLinear, TritonMatmulForLinearLayer, _GeneralizedLinear, _kind,
                                 can_fuse_gated_forward, cast_cached, input_grad, linear_backward_core, linear_forward_core,
                                 weight_grad,
                                 resolve_compute_dtype)
from .utils import ACT2FN, resolve_activation


# Optional callback ``fn(name, grad, param) -> bool`` invoked inside the backward as soon as a parameter gradient
# exists (names: "h2o_weight", "h2o_bias", "i2h_weight", ...; ``param`` is the tensor the gradient belongs to).  A
# data-parallel trainer uses it to start the all-reduce of the output projection's gradients while the input
# projection's are still being computed (see lean_transformer_b200.dist.GradSync); autograd hooks would only fire
# after the whole backward.  A callback that returns True has TAKEN the gradient: the backward then returns None
# for that parameter and the callback's owner delivers ``param.grad`` itself.  This matters because autograd may
# cast or copy a returned gradient on the compute stream while an asynchronous reduction is still writing it.
_grad_ready_hook = None


def set_grad_ready_hook(fn):
    """Install (or clear, with None) the gradient-ready callback; returns the previous one."""
    global _grad_ready_hook
    previous, _grad_ready_hook = _grad_ready_hook, fn
    return previous


def _offer(name, grad, param):
    """Hand a finished gradient to the callback; returns what the backward passes on to autograd."""
    if grad is None or _grad_ready_hook is None:
        return grad
    return None if _grad_ready_hook(name, grad, param) is True else grad


_token_window = None


def set_token_window(first_token: Optional[int], total_tokens: Optional[int] = None):
    """Token-partitioned data parallelism: declare that the rows this process feeds to LeanFFN are tokens
    ``[first_token, first_token + rows)`` of a global batch of ``total_tokens``.  Dropout masks are then drawn at
    the GLOBAL element index and the generator advances by the global size, so with equal seeds the union of the
    ranks' masks equals the single-process mask of the whole batch (partition-invariant training).  ``None``
    clears the window.  Returns the previous window."""
    global _token_window
    previous = _token_window
    _token_window = None if first_token is None else (int(first_token), int(total_tokens))
    return previous


def next_dropout_stream(device: torch.device, numel: int, row_elems: Optional[int] = None):
    """(seed, element offset) for a dropout mask of ``numel`` elements (rows of ``row_elems``), taken from (and
    advancing) torch's CUDA generator of ``device`` so torch.manual_seed and torch.utils.checkpoint's RNG stashing
    govern it."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    gen = torch.cuda.default_generators[index]
    seed, offset = gen.initial_seed(), gen.get_offset()
    shift = 0
    if _token_window is not None and row_elems:
        first, total = _token_window
        if first * row_elems + numel > total * row_elems:
            raise ValueError(f"token window [{first}, +{numel // row_elems}) exceeds the declared {total} tokens")
        shift, numel = first * row_elems, total * row_elems
    gen.set_offset(offset + 4 * ((numel + 15) // 16))  # offsets move in multiples of 4, one unit per 4 elements
    return seed & 0xFFFFFFFFFFFFFFFF, 4 * offset + shift


class LeanFFN(nn.Module):
    """
    A transformer FFN module that doesn't hog your GPU memory, computed by hand-written CUDA kernels.

    :param hidden_size: base hidden size of the transformer
    :param intermediate_size: a (typically larger) hidden dimension where activation is applied
    :param activation: a nonlinearity from ``ACT2FN`` (or an equivalent torch / transformers callable)
    :param gated: use gated activations (https://arxiv.org/abs/2002.05202); the input projection is 2x wide
    :param layer_norm_eps: see torch.nn.functional.layer_norm
    :param post_layer_norm: additional layer norm on the projected outputs before dropout and the residual
    :param dropout: hidden dropout probability, applied to the output projection (before adding residual)
    :param residual: if True, adds the original layer input to the final layer output
    :param ffn_custom_grad: if True (default), use the memory-lean hand-written backward
    :param i2h_proj: custom *first* linear layer (hidden_size -> intermediate_size or 2x intermediate_size)
    :param h2o_proj: custom *second* linear layer (intermediate_size -> hidden_size)
    """

    def __init__(self, hidden_size: int, intermediate_size: int, activation=ACT2FN["gelu_fused"],
                 gated: bool = False, layer_norm_eps: float = 1e-12, dropout: float = 0.0,
                 post_layer_norm: bool = False, i2h_proj: Optional[nn.Linear] = None,
                 h2o_proj: Optional[nn.Linear] = None, residual: bool = True, ffn_custom_grad: bool = True):
        super().__init__()
        i2h_out_features = intermediate_size * 2 if gated else intermediate_size
        self.i2h_proj = nn.Linear(hidden_size, i2h_out_features) if i2h_proj is None else i2h_proj
        self.h2o_proj = nn.Linear(intermediate_size, hidden_size) if h2o_proj is None else h2o_proj
        if ffn_custom_grad:
            assert type(self.i2h_proj) in (nn.Linear, GeneralizedLinear), \
                "custom grad supports only nn.Linear and GeneralizedLinear"
            assert type(self.h2o_proj) in (nn.Linear, GeneralizedLinear), \
                "custom grad supports only nn.Linear and GeneralizedLinear"
        assert self.i2h_proj.in_features == self.h2o_proj.out_features == hidden_size
        assert self.i2h_proj.out_features == i2h_out_features and self.h2o_proj.in_features == intermediate_size
        self.pre_layer_norm = nn.LayerNorm(hidden_size, eps=layer_norm_eps)
        self.post_layer_norm = nn.LayerNorm(hidden_size, eps=layer_norm_eps) if post_layer_norm else None
        self.activation = activation
        self.gated = gated
        self.dropout = dropout
        self.residual = residual
        self.ffn_custom_grad = ffn_custom_grad
        resolve_activation(activation)  # fail at construction for activations without a kernel

    def forward(self, input):
        return self._forward_custom(input) if self.ffn_custom_grad else self._forward_pytorch(input)

    def _forward_pytorch(self, input):
        """Plain-autograd twin (``ffn_custom_grad=False``): every stage is its own differentiable op and
        keeps its own activations, like the reference's ffn.py:69-85."""
        input_2d = input.reshape(-1, input.shape[-1])
        ln = self.pre_layer_norm
        input_ln = _LayerNormFunction.apply(input_2d, ln.weight, ln.bias, ln.eps)
        pre_activation = self._apply_proj(self.i2h_proj, input_ln)
        hid_act = _ActivationStage.apply(pre_activation, resolve_activation(self.activation), self.gated)
        out = self._apply_proj(self.h2o_proj, hid_act)
        if self.post_layer_norm is not None:
            pln = self.post_layer_norm
            out = _LayerNormFunction.apply(out, pln.weight, pln.bias, pln.eps)
        if self.dropout and self.training:
            out = _DropoutFunction.apply(out, self.dropout)
        if self.residual:
            out = out + input_2d.to(out.dtype)
        return out.view(*input.shape)

    @staticmethod
    def _apply_proj(proj, x):
        if isinstance(proj, GeneralizedLinear):
            return proj(x)
        return _GeneralizedLinear.apply(x, proj.weight, proj.bias, None, None, None, None, None)

    def _forward_custom(self, input):
        post_ln_weight = post_ln_bias = None
        if self.post_layer_norm is not None:
            post_ln_weight, post_ln_bias = self.post_layer_norm.weight, self.post_layer_norm.bias
        i2h = _projection_args(self.i2h_proj)
        h2o = _projection_args(self.h2o_proj)
        return _LeanFFN.apply(
            input, self.pre_layer_norm.weight, self.pre_layer_norm.bias,
            self.i2h_proj.weight, self.i2h_proj.bias, *i2h,
            self.h2o_proj.weight, self.h2o_proj.bias, *h2o,
            post_ln_weight, post_ln_bias, self.activation, self.gated, self.dropout, self.training,
            self.pre_layer_norm.eps, self.residual,
        )


def _projection_args(proj):
    """(lowrank_first, lowrank_second, forward_indices, backward_indices, matmul_op) of a projection."""
    if isinstance(proj, GeneralizedLinear):
        first, second = proj.get_combined_lowrank_components()
        return first, second, proj.matrix.forward_indices, proj.matrix.backward_indices, proj.matrix.matmul_op
    return None, None, None, None, None


# ---- the whole block through one C call ------------------------------------------------------------------------------
# ``leanffn_ffn_forward`` / ``leanffn_ffn_backward`` run the schedule below inside the library (one ctypes call per
# direction instead of one per kernel).  They cover the bf16 compute path without post-LayerNorm; everything else, and
# any step that must interleave Python between the kernels (gradient-ready callbacks, scattered gradient exchange),
# takes the piecewise schedule, which launches the same kernels.
_BLOCK_CALLS = os.environ.get("LEANFFN_BLOCK_CALLS", "1") != "0"
_EXPERIMENT_UNFUSED_ACT_BWD = os.environ.get("LEANFFN_UNFUSED_ACT_BWD", "0") == "1"  # piecewise schedule only


def set_block_calls(enabled: bool) -> bool:
    """Switch between the one-call-per-direction schedule (default) and the piecewise one; returns the previous value."""
    global _BLOCK_CALLS
    previous, _BLOCK_CALLS = _BLOCK_CALLS, bool(enabled)
    return previous


def _fill_linear(field, weight, bias, first, second, forward_indices, backward_indices, matmul_op, cdt, gated_input,
                 keep):
    """Describe one projection for the C call; returns False if it cannot be described."""
    from .blocksparse.native_backend import native_tables, weight_blocks_pair_up
    kind = _kind(weight, forward_indices, backward_indices, matmul_op)
    w = cast_cached(weight, cdt)
    keep.append(w)
    field.weight = w.data_ptr()
    if bias is not None:
        if bias.dtype not in (torch.float32, torch.bfloat16) or not bias.is_contiguous():
            return False
        field.bias, field.bias_dtype = bias.data_ptr(), ops._dt(bias)
    if first is not None and second is not None:
        if first.shape[0] % 8 != 0:
            return False
        l1, l2 = cast_cached(first, cdt), cast_cached(second, cdt)
        keep.extend((l1, l2))
        field.rank, field.lowrank_first, field.lowrank_second = first.shape[0], l1.data_ptr(), l2.data_ptr()
    if kind == "dense":
        return weight.dim() == 2
    block = weight.shape[-1]
    if kind == "native":
        fwd, dgrad, wgrad = native_tables(forward_indices, backward_indices, weight.shape[1])
        fwd_count = dgrad_count = None
    else:
        fwd, fwd_count, dgrad, dgrad_count, wgrad = matmul_op._tables(weight.device)
    keep.extend((fwd, dgrad, wgrad, fwd_count, dgrad_count))
    field.bs_block, field.bs_num_blocks = block, weight.numel() // (block * block)
    field.fwd_index, field.fwd_nnz = fwd.data_ptr(), fwd.shape[1]
    field.dgrad_index, field.dgrad_nnz = dgrad.data_ptr(), dgrad.shape[1]
    field.wgrad_index = wgrad.data_ptr()
    if fwd_count is not None:
        field.fwd_count, field.dgrad_count = fwd_count.data_ptr(), dgrad_count.data_ptr()
    field.wgrad_pairs = int(block == 128 and weight_blocks_pair_up(wgrad))
    field.fuse_gated_forward = int(gated_input and can_fuse_gated_forward(weight, forward_indices, backward_indices,
                                                                         matmul_op, cdt))
    return True


def _block_descriptor(input_2d, grad_dtype, ln_weight, ln_bias, i2h, h2o, act, gated, residual, ln_eps, cdt, inter):
    """(FfnDesc, keep-alive list) for the C call, or None when the configuration needs the piecewise schedule.
    ``i2h`` / ``h2o`` = (weight, bias, lowrank_first, lowrank_second, forward_indices, backward_indices, matmul_op)."""
    from .blocksparse import linear as _linear
    if not _BLOCK_CALLS or cdt != torch.bfloat16 or _grad_ready_hook is not None or _linear._weight_grad_reducer is not None:
        return None
    hidden = input_2d.shape[1]
    if hidden % 8 or inter % 8 or input_2d.dtype not in (torch.float32, torch.bfloat16):
        return None
    params = [t for t in (ln_weight, ln_bias, i2h[0], i2h[2], i2h[3], h2o[0], h2o[2], h2o[3]) if t is not None]
    param_dtype = i2h[0].dtype
    if param_dtype not in (torch.float32, torch.bfloat16) or any(t.dtype != param_dtype for t in params):
        return None
    if input_2d.dtype == torch.float32 and param_dtype == torch.bfloat16:
        return None
    if ln_weight is None or ln_bias is None or not ln_weight.is_contiguous() or not ln_bias.is_contiguous():
        return None
    d = N.FfnDesc()
    d.tokens, d.hidden, d.intermediate = input_2d.shape[0], hidden, inter
    d.gated, d.act, d.residual = int(gated), act, int(residual)
    d.compute_dtype, d.io_dtype, d.param_dtype = N.BF16, ops._dt(input_2d), N.BF16 if param_dtype == torch.bfloat16 else N.F32
    d.grad_out_dtype = N.BF16 if grad_dtype == torch.bfloat16 else N.F32
    d.eps = float(ln_eps)  # dropout_p / seed / elem_offset: set by the caller once it has drawn the stream position
    d.ln_weight, d.ln_bias = ln_weight.data_ptr(), ln_bias.data_ptr()
    keep = [ln_weight, ln_bias]
    if not _fill_linear(d.i2h, *i2h, cdt, gated, keep) or not _fill_linear(d.h2o, *h2o, cdt, False, keep):
        return None
    return d, keep


class _LeanFFN(torch.autograd.Function):
    """Autograd function for the transformer FFN with the reference's 25-argument signature."""

    @staticmethod
    def _apply_activation(pre_activation: torch.Tensor, activation, gated: bool):
        flat = pre_activation.reshape(-1, pre_activation.shape[-1]).contiguous()
        hid = ops.activation_forward(flat, gated, resolve_activation(activation))
        return hid.view(*pre_activation.shape[:-1], hid.shape[-1])

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, input, ln_weight, ln_bias,
                i2h_weight, i2h_bias, i2h_lowrank_first, i2h_lowrank_second, i2h_forward_indices,
                i2h_backward_indices, i2h_matmul_op,
                h2o_weight, h2o_bias, h2o_lowrank_first, h2o_lowrank_second, h2o_forward_indices,
                h2o_backward_indices, h2o_matmul_op,
                post_ln_weight, post_ln_bias, activation, gated: bool, dropout: float, training: bool,
                ln_eps: float, residual: bool):
        if not input.is_cuda:
            raise RuntimeError("LeanFFN (lean_transformer_b200) needs CUDA tensors: its only implementation is "
                               "the sm_100a kernel library; there is no CPU path")
        act = resolve_activation(activation)
        cdt = resolve_compute_dtype(input)
        ctx._dropout, ctx._training, ctx._ln_eps = dropout, training, ln_eps
        ctx._act, ctx._gated, ctx._residual, ctx._cdt = act, gated, residual, cdt
        ctx._i2h_matmul_op, ctx._h2o_matmul_op = i2h_matmul_op, h2o_matmul_op
        ctx._use_post_ln = post_ln_weight is not None
        ctx._dropout_stream = None

        hidden = input.shape[-1]
        input_2d = input.reshape(-1, hidden)
        if not input_2d.is_contiguous():
            input_2d = input_2d.contiguous()
        tokens = input_2d.shape[0]
        i2h_dense = _kind(i2h_weight, i2h_forward_indices, i2h_backward_indices, i2h_matmul_op) == "dense"
        out_features1 = i2h_bias.shape[0] if i2h_bias is not None else _out_features(
            i2h_weight, i2h_forward_indices, i2h_matmul_op)
        inter = out_features1 // 2 if gated else out_features1

        use_dropout = bool(training and dropout)
        ctx._block = None
        if not ctx._use_post_ln and tokens > 0:
            block = _block_descriptor(
                input_2d, cdt, ln_weight, ln_bias,
                (i2h_weight, i2h_bias, i2h_lowrank_first, i2h_lowrank_second, i2h_forward_indices, i2h_backward_indices,
                 i2h_matmul_op),
                (h2o_weight, h2o_bias, h2o_lowrank_first, h2o_lowrank_second, h2o_forward_indices, h2o_backward_indices,
                 h2o_matmul_op), act, gated, residual, ln_eps, cdt, inter)
            if block is not None:
                desc, keep = block
                seed = offset = 0
                if use_dropout:
                    seed, offset = next_dropout_stream(input.device, tokens * hidden, hidden)
                    desc.dropout_p, desc.seed, desc.elem_offset = float(dropout), seed, offset
                new = lambda *shape: torch.empty(shape, dtype=cdt, device=input.device)  # noqa: E731
                out, pre_activation = new(tokens, hidden), new(tokens, out_features1)
                i2h_lowrank_hid = new(tokens, desc.i2h.rank) if desc.i2h.rank else None
                h2o_lowrank_hid = new(tokens, desc.h2o.rank) if desc.h2o.rank else None
                fused = desc.i2h.bs_block == 0 or desc.i2h.fuse_gated_forward
                ops.ffn_forward(desc, input_2d, out, pre_activation, i2h_lowrank_hid, h2o_lowrank_hid,
                                launches=3 + (not fused) + bool(desc.i2h.rank) + bool(desc.h2o.rank))
                ctx._block = True
                ctx._dropout_stream = (seed, offset) if use_dropout else None
                ctx.save_for_backward(
                    input, pre_activation, ln_weight, ln_bias, None, post_ln_weight, post_ln_bias,
                    i2h_lowrank_hid, i2h_weight, i2h_lowrank_first, i2h_lowrank_second, i2h_forward_indices,
                    i2h_backward_indices,
                    h2o_lowrank_hid, h2o_weight, h2o_lowrank_first, h2o_lowrank_second, h2o_forward_indices,
                    h2o_backward_indices, i2h_bias, h2o_bias)
                return out.view(*input.shape)

        input_ln = ops.layer_norm_forward(input_2d, ln_weight, ln_bias, ln_eps, cdt)

        pre_activation = torch.empty((tokens, out_features1), dtype=cdt, device=input.device)
        i2h_fused = i2h_dense or (gated and can_fuse_gated_forward(i2h_weight, i2h_forward_indices,
                                                                   i2h_backward_indices, i2h_matmul_op, cdt))
        if i2h_fused:
            hid_act = torch.empty((tokens, inter), dtype=cdt, device=input.device)
            _, i2h_lowrank_hid = linear_forward_core(
                input_ln, i2h_weight, i2h_bias, i2h_lowrank_first, i2h_lowrank_second, i2h_forward_indices,
                i2h_backward_indices, i2h_matmul_op, cdt,
                epilogue=N.EPI_GLU_FWD if gated else N.EPI_ACT_FWD, act=act, out=pre_activation, out2=hid_act)
        else:
            _, i2h_lowrank_hid = linear_forward_core(
                input_ln, i2h_weight, i2h_bias, i2h_lowrank_first, i2h_lowrank_second, i2h_forward_indices,
                i2h_backward_indices, i2h_matmul_op, cdt, out=pre_activation)
            hid_act = ops.activation_forward(pre_activation, gated, act)
        del input_ln

        seed = offset = 0
        if use_dropout:
            seed, offset = next_dropout_stream(input.device, tokens * hidden, hidden)
            ctx._dropout_stream = (seed, offset)
        post_ln_input = None
        if ctx._use_post_ln:
            post_ln_input, h2o_lowrank_hid = linear_forward_core(
                hid_act, h2o_weight, h2o_bias, h2o_lowrank_first, h2o_lowrank_second, h2o_forward_indices,
                h2o_backward_indices, h2o_matmul_op, cdt)
            out = ops.layer_norm_forward(post_ln_input, post_ln_weight, post_ln_bias, ln_eps, cdt,
                                         dropout_p=dropout if use_dropout else 0.0, seed=seed,
                                         elem_offset=offset, residual=input_2d if residual else None)
        else:
            # dense or block-sparse: bias, dropout and the residual add ride in the product's epilogue
            out, h2o_lowrank_hid = linear_forward_core(
                hid_act, h2o_weight, h2o_bias, h2o_lowrank_first, h2o_lowrank_second, h2o_forward_indices,
                h2o_backward_indices, h2o_matmul_op, cdt,
                epilogue=N.EPI_DROPOUT_RESIDUAL, aux=input_2d if residual else None,
                dropout_p=dropout if use_dropout else 0.0, seed=seed, elem_offset=offset)
        del hid_act

        ctx.save_for_backward(
            input, pre_activation, ln_weight, ln_bias, post_ln_input, post_ln_weight, post_ln_bias,
            i2h_lowrank_hid, i2h_weight, i2h_lowrank_first, i2h_lowrank_second, i2h_forward_indices,
            i2h_backward_indices,
            h2o_lowrank_hid, h2o_weight, h2o_lowrank_first, h2o_lowrank_second, h2o_forward_indices,
            h2o_backward_indices, i2h_bias, h2o_bias)
        return out.view(*input.shape)

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        (input, pre_activation, ln_weight, ln_bias, post_ln_input, post_ln_weight, post_ln_bias,
         i2h_lowrank_hid, i2h_weight, i2h_lowrank_first, i2h_lowrank_second, i2h_forward_indices,
         i2h_backward_indices,
         h2o_lowrank_hid, h2o_weight, h2o_lowrank_first, h2o_lowrank_second, h2o_forward_indices,
         h2o_backward_indices, i2h_bias, h2o_bias) = ctx.saved_tensors
        cdt, act, gated = ctx._cdt, ctx._act, ctx._gated
        needs = ctx.needs_input_grad
        hidden = input.shape[-1]
        input_2d = input.reshape(-1, hidden)
        if not input_2d.is_contiguous():
            input_2d = input_2d.contiguous()
        grad_output_2d = grad_output.reshape(-1, hidden)
        if not grad_output_2d.is_contiguous():
            grad_output_2d = grad_output_2d.contiguous()
        grad_post_ln_weight = grad_post_ln_bias = None

        if getattr(ctx, "_block", None) and grad_output_2d.dtype in (torch.float32, torch.bfloat16):
            block = _block_descriptor(
                input_2d, grad_output_2d.dtype, ln_weight, ln_bias,
                (i2h_weight, i2h_bias, i2h_lowrank_first, i2h_lowrank_second, i2h_forward_indices, i2h_backward_indices,
                 ctx._i2h_matmul_op),
                (h2o_weight, h2o_bias, h2o_lowrank_first, h2o_lowrank_second, h2o_forward_indices, h2o_backward_indices,
                 ctx._h2o_matmul_op), act, gated, ctx._residual, ctx._ln_eps, cdt,
                pre_activation.shape[1] // 2 if gated else pre_activation.shape[1])
            if block is not None:
                return _LeanFFN._backward_block(ctx, block, needs, input, input_2d, grad_output_2d, pre_activation,
                                                i2h_lowrank_hid, h2o_lowrank_hid, ln_weight, i2h_weight, i2h_bias,
                                                i2h_lowrank_first, i2h_lowrank_second, h2o_weight, h2o_bias,
                                                h2o_lowrank_first, h2o_lowrank_second)

        # backward(... -> post_norm -> dropout -> residual)
        grad_residual_2d = ops.cast(grad_output_2d, cdt) if ctx._residual else None
        grad_h2o_bias = None
        seed, offset = ctx._dropout_stream if ctx._dropout_stream is not None else (0, 0)
        p_drop = ctx._dropout if ctx._dropout_stream is not None else 0.0
        if needs[11] and not ctx._use_post_ln and (p_drop or grad_output_2d.dtype != cdt):
            # mask + cast + column sums (the output projection's bias gradient) in one pass over the incoming gradient
            grad_h2o_out, grad_h2o_bias = ops.dropout_colsum(grad_output_2d, p_drop, seed, offset, out_dtype=cdt)
        elif p_drop:
            grad_h2o_out = ops.dropout(grad_output_2d, p_drop, seed, offset, out_dtype=cdt)
        else:
            grad_h2o_out = ops.cast(grad_output_2d, cdt)
        if ctx._use_post_ln:
            need_post = bool(needs[17] or needs[18])
            grad_h2o_out, grad_post_ln_weight, grad_post_ln_bias = ops.layer_norm_backward(
                grad_h2o_out, post_ln_input, post_ln_weight, ctx._ln_eps, None, cdt, need_param_grads=need_post)

        # backward(... -> nonlinearity -> linear_h2o -> ...): dgrad2 rematerialises the activation
        h2o_kind = _kind(h2o_weight, h2o_forward_indices, h2o_backward_indices, ctx._h2o_matmul_op)
        tokens = input_2d.shape[0]
        inter = pre_activation.shape[1] // 2 if gated else pre_activation.shape[1]
        need_hid = bool(needs[10] or needs[12])  # hid_act feeds the weight and first-low-rank gradients
        grad_pre = torch.empty_like(pre_activation)
        hid_act = torch.empty((tokens, inter), dtype=cdt, device=input.device) if need_hid else None
        if needs[11] and grad_h2o_bias is None:
            grad_h2o_bias = ops.column_sum(grad_h2o_out)
        # the input projection's bias gradient (column sums of grad_pre) rides in the epilogue that produces grad_pre
        bias1_partial = None
        if needs[4] and cdt == torch.bfloat16 and tokens > 0:
            bias1_partial = torch.empty(((tokens + 31) // 32, pre_activation.shape[1]), dtype=torch.float32,
                                        device=input.device)
        grad_lowrank_hid = a2 = b2 = None
        if h2o_lowrank_first is not None:
            grad_lowrank_hid = ops.gemm(grad_h2o_out, cast_cached(h2o_lowrank_second, cdt), b_mn_major=True)
            a2, b2 = grad_lowrank_hid, cast_cached(h2o_lowrank_first, cdt)
        # the input-gradient epilogue (dense or block-sparse weight alike) applies the activation backward and
        # rematerialises hid_act, which the weight gradients below then consume
        if _EXPERIMENT_UNFUSED_ACT_BWD and h2o_kind != "dense":
            # measurement switch: plain input-gradient product, then the activation backward as its own pass
            grad_hid = input_grad(h2o_kind, grad_h2o_out, h2o_weight, h2o_forward_indices, h2o_backward_indices,
                                  ctx._h2o_matmul_op, cdt, a2=a2, b2=b2)
            ops.activation_backward(grad_hid, pre_activation, gated, act, out=grad_pre, hid_out=hid_act)
            del grad_hid
            bias1_partial = None
        else:
            input_grad(h2o_kind, grad_h2o_out, h2o_weight, h2o_forward_indices, h2o_backward_indices,
                       ctx._h2o_matmul_op, cdt, a2=a2, b2=b2, epilogue=N.EPI_GLU_BWD if gated else N.EPI_ACT_BWD,
                       act=act, aux=pre_activation, out=grad_pre, out2=hid_act, colsum=bias1_partial)
        grad_i2h_bias_ready = ops.column_sum(bias1_partial) if bias1_partial is not None else None
        del bias1_partial
        grad_h2o_weight = grad_h2o_lowrank_first = grad_h2o_lowrank_second = None
        if needs[10]:
            grad_h2o_weight = weight_grad(h2o_kind, grad_h2o_out, hid_act, h2o_weight, h2o_forward_indices,
                                          h2o_backward_indices, ctx._h2o_matmul_op)
        if h2o_lowrank_first is not None and needs[13]:
            grad_h2o_lowrank_second = ops.gemm(grad_h2o_out, h2o_lowrank_hid, a_mn_major=True, b_mn_major=True,
                                               out_dtype=h2o_lowrank_second.dtype)
        if h2o_lowrank_first is not None and needs[12]:
            grad_h2o_lowrank_first = ops.gemm(grad_lowrank_hid, hid_act, a_mn_major=True, b_mn_major=True,
                                              out_dtype=h2o_lowrank_first.dtype)
        del hid_act, grad_h2o_out
        grad_h2o_weight = _offer("h2o_weight", only_if(needs[10], grad_h2o_weight), h2o_weight)
        grad_h2o_bias = _offer("h2o_bias", only_if(needs[11], grad_h2o_bias), h2o_bias)
        grad_h2o_lowrank_first = _offer("h2o_lowrank_first", only_if(needs[12], grad_h2o_lowrank_first),
                                        h2o_lowrank_first)
        grad_h2o_lowrank_second = _offer("h2o_lowrank_second", only_if(needs[13], grad_h2o_lowrank_second),
                                         h2o_lowrank_second)
        grad_post_ln_weight = _offer("post_ln_weight", grad_post_ln_weight, post_ln_weight)
        grad_post_ln_bias = _offer("post_ln_bias", grad_post_ln_bias, post_ln_bias)

        # backward(... -> input_layernorm -> linear_i2h -> ...)
        need_input_side = bool(needs[0] or needs[1] or needs[2])
        i2h_needs = [need_input_side, needs[3], needs[4], needs[5], needs[6]]
        input_ln = None
        if needs[3] or needs[5]:
            input_ln = ops.layer_norm_forward(input_2d, ln_weight, ln_bias, ctx._ln_eps, cdt)  # rematerialise
        (grad_input_ln, grad_i2h_weight, grad_i2h_bias, grad_i2h_lowrank_first,
         grad_i2h_lowrank_second) = linear_backward_core(
            grad_pre, input_ln, i2h_lowrank_hid, i2h_weight, i2h_lowrank_first, i2h_lowrank_second,
            i2h_forward_indices, i2h_backward_indices, ctx._i2h_matmul_op, i2h_needs, cdt,
            grad_bias=grad_i2h_bias_ready, on_param_grads=lambda w, b, l1, l2: (_offer("i2h_weight", w, i2h_weight), _offer("i2h_bias", b, i2h_bias),
                                                 _offer("i2h_lowrank_first", l1, i2h_lowrank_first),
                                                 _offer("i2h_lowrank_second", l2, i2h_lowrank_second)))
        del grad_pre, input_ln

        grad_input = grad_ln_weight = grad_ln_bias = None
        if need_input_side:
            grad_input, grad_ln_weight, grad_ln_bias = ops.layer_norm_backward(
                grad_input_ln, input_2d, ln_weight, ctx._ln_eps, grad_residual_2d, input.dtype,
                need_dx=bool(needs[0]), need_param_grads=bool(needs[1] or needs[2]))
            if grad_input is not None:
                grad_input = grad_input.view(*input.shape)
            grad_ln_weight = _offer("ln_weight", grad_ln_weight, ln_weight)
            grad_ln_bias = _offer("ln_bias", grad_ln_bias, ln_bias)
        only = only_if

        return (only(needs[0], grad_input), only(needs[1], grad_ln_weight), only(needs[2], grad_ln_bias),
                only(needs[3], grad_i2h_weight), only(needs[4], grad_i2h_bias),
                only(needs[5], grad_i2h_lowrank_first), only(needs[6], grad_i2h_lowrank_second), None, None, None,
                only(needs[10], grad_h2o_weight), only(needs[11], grad_h2o_bias),
                only(needs[12], grad_h2o_lowrank_first), only(needs[13], grad_h2o_lowrank_second), None, None, None,
                only(needs[17], grad_post_ln_weight), only(needs[18], grad_post_ln_bias),
                None, None, None, None, None, None)


def only_if(flag, value):
    return value if flag else None


def _backward_block(ctx, block, needs, input, input_2d, grad_output_2d, pre_activation, i2h_lowrank_hid, h2o_lowrank_hid,
                    ln_weight, i2h_weight, i2h_bias, i2h_lowrank_first, i2h_lowrank_second, h2o_weight, h2o_bias,
                    h2o_lowrank_first, h2o_lowrank_second):
    """The backward through ``leanffn_ffn_backward``: allocate the gradients autograd asked for, one C call."""
    desc, keep = block
    if ctx._dropout_stream is not None:
        desc.dropout_p = float(ctx._dropout)
        desc.seed, desc.elem_offset = ctx._dropout_stream
    device = input.device
    grads = N.FfnGrads()
    out = {}

    def want(flag, name, like=None, shape=None, dtype=None):
        if not flag:
            return None
        t = torch.empty_like(like) if like is not None else torch.empty(shape, dtype=dtype, device=device)
        setattr(grads, name, t.data_ptr())
        out[name] = t
        return t

    grad_input = want(needs[0], "grad_input", shape=input_2d.shape, dtype=input.dtype)
    grad_ln = None
    if needs[1] or needs[2]:
        grad_ln = torch.empty((2, input_2d.shape[1]), dtype=torch.float32, device=device)
        grads.grad_ln_weight, grads.grad_ln_bias = grad_ln[0].data_ptr(), grad_ln[1].data_ptr()
    g_w1 = want(needs[3], "grad_i2h_weight", like=i2h_weight)
    g_b1 = want(needs[4] and i2h_bias is not None, "grad_i2h_bias", shape=(pre_activation.shape[1],), dtype=torch.float32)
    g_l11 = want(needs[5] and i2h_lowrank_first is not None, "grad_i2h_lowrank_first", like=i2h_lowrank_first)
    g_l12 = want(needs[6] and i2h_lowrank_second is not None, "grad_i2h_lowrank_second", like=i2h_lowrank_second)
    g_w2 = want(needs[10], "grad_h2o_weight", like=h2o_weight)
    g_b2 = want(needs[11] and h2o_bias is not None, "grad_h2o_bias", shape=(input_2d.shape[1],), dtype=torch.float32)
    g_l21 = want(needs[12] and h2o_lowrank_first is not None, "grad_h2o_lowrank_first", like=h2o_lowrank_first)
    g_l22 = want(needs[13] and h2o_lowrank_second is not None, "grad_h2o_lowrank_second", like=h2o_lowrank_second)
    launches = 6 + 3 * bool(desc.i2h.rank) + 3 * bool(desc.h2o.rank) + 3 * (grad_ln is not None) + 4
    ops.ffn_backward(desc, grad_output_2d, input_2d, pre_activation, i2h_lowrank_hid, h2o_lowrank_hid, grads, launches)
    del keep
    return (grad_input.view(*input.shape) if grad_input is not None else None,
            grad_ln[0] if (grad_ln is not None and needs[1]) else None,
            grad_ln[1] if (grad_ln is not None and needs[2]) else None,
            g_w1, g_b1, g_l11, g_l12, None, None, None, g_w2, g_b2, g_l21, g_l22, None, None, None,
            None, None, None, None, None, None, None, None)


_LeanFFN._backward_block = staticmethod(_backward_block)


def _out_features(weight, forward_indices, matmul_op):
    if matmul_op is not None:
        return matmul_op.out_features
    if forward_indices is not None:
        return forward_indices.shape[0] * weight.shape[-1]
    return weight.shape[0]


# ---- stages of the plain-autograd twin ---------------------------------------------------------------
class _LayerNormFunction(torch.autograd.Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, x, weight, bias, eps):
        cdt = resolve_compute_dtype(x)
        ctx.save_for_backward(x, weight)
        ctx.eps, ctx.cdt = eps, cdt
        return ops.layer_norm_forward(x.contiguous(), weight, bias, eps, cdt)

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad):
        x, weight = ctx.saved_tensors
        need_params = bool(ctx.needs_input_grad[1] or ctx.needs_input_grad[2])
        dx, dg, db = ops.layer_norm_backward(ops.cast(grad.contiguous(), ctx.cdt), x.contiguous(), weight, ctx.eps,
                                             None, x.dtype, need_dx=ctx.needs_input_grad[0],
                                             need_param_grads=need_params)
        return dx, dg, db, None


class _ActivationStage(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pre, act: int, gated: bool):
        ctx.save_for_backward(pre)
        ctx.act, ctx.gated = act, gated
        return ops.activation_forward(pre.contiguous(), gated, act)

    @staticmethod
    def backward(ctx, grad):
        (pre,) = ctx.saved_tensors
        dpre, _ = ops.activation_backward(ops.cast(grad.contiguous(), pre.dtype), pre.contiguous(), ctx.gated, ctx.act)
        return dpre, None, None


class _DropoutFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p: float):
        ctx.p = p
        ctx.stream = next_dropout_stream(x.device, x.numel(), x.shape[-1])
        return ops.dropout(x.contiguous(), p, *ctx.stream)

    @staticmethod
    def backward(ctx, grad):
        return ops.dropout(grad.contiguous(), ctx.p, *ctx.stream), None
