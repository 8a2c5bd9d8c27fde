"""Linear layers with a shared (dense or block-sparse) matrix and low-rank adapters, on CUDA kernels.

Module and functional API follow lean_transformer/blocksparse/linear.py: ``GeneralizedMatrix`` (:19-103),
``GeneralizedLinear`` (:106-149) and ``_GeneralizedLinear.forward_functional`` / ``backward_functional``
(:161-193, :237-258) with the same argument order, saved-tensor order and parameter / buffer names, so
state dicts are interchangeable.  The arithmetic is one GEMM launch per product: the low-rank term
rides in the main kernel's k-loop as a continuation and the bias in its epilogue.
"""
import math
import weakref
from itertools import zip_longest
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .. import _native as N
from .. import ops
from ..utils import pad_to_multiple
from .layout import get_blocksparse_layout, get_indices_from_layout
from .native_backend import _bs_dgrad, _bs_forward, _bs_wgrad, gate_and_linear_blocks_pair_up, native_tables
from .triton_backend import TRITON_PAD_TO, TritonMatmulForLinearLayer


# ---- compute dtype and cached parameter casts -------------------------------------------------------
def resolve_compute_dtype(input: torch.Tensor) -> torch.dtype:
    """bf16 under CUDA autocast(bf16) or for bf16 inputs, fp32 for fp32 inputs outside autocast."""
    if torch.is_autocast_enabled("cuda"):
        dtype = torch.get_autocast_dtype("cuda")
        if dtype != torch.bfloat16:
            raise NotImplementedError(f"autocast dtype {dtype} is not supported: the tensor-core path is bf16")
        return dtype
    if input.dtype in (torch.float32, torch.bfloat16):
        return input.dtype
    raise TypeError(f"unsupported input dtype {input.dtype}")


_CAST_CACHE: Dict[int, tuple] = {}


def cast_cached(t: Optional[torch.Tensor], dtype: torch.dtype) -> Optional[torch.Tensor]:
    """``t`` as a contiguous tensor of ``dtype``; conversions are remembered per tensor OBJECT until it is
    modified in place (version counter), re-pointed at other storage, or garbage collected, so a weight is
    converted once per optimizer step, not once per use."""
    if t is None:
        return None
    if t.dtype == dtype and t.is_contiguous():
        return t.detach()
    key = id(t)
    hit = _CAST_CACHE.get(key)
    if hit is not None:
        ref, version, data_ptr, target, converted = hit
        if ref() is t and version == t._version and data_ptr == t.data_ptr() and target == dtype:
            return converted
    converted = ops.cast(t.detach().contiguous(), dtype)
    try:
        ref = weakref.ref(t, lambda _r, _k=key: _CAST_CACHE.pop(_k, None))
    except TypeError:
        return converted
    _CAST_CACHE[key] = (ref, t._version, t.data_ptr(), dtype, converted)
    return converted


def clear_cast_cache():
    _CAST_CACHE.clear()


# ---- one linear layer = one GEMM launch per product ---------------------------------------------------
def _kind(weight: torch.Tensor, forward_indices, backward_indices, matmul_op) -> str:
    if matmul_op is not None:
        return "rowmajor"  # blocks ordered like layout.nonzero() (the Triton operator's order)
    if forward_indices is not None or backward_indices is not None:
        return "native"
    return "dense"


def linear_forward_core(x2d, weight, bias, lowrank_first, lowrank_second, forward_indices, backward_indices,
                        matmul_op, cdt, *, epilogue=N.EPI_STORE, act=0, out=None, out2=None, aux=None,
                        dropout_p=0.0, seed=0, elem_offset=0, out_dtype=None):
    """output = x @ W^T (+ low rank) (+ bias) with an optional fused epilogue (block-sparse weights: dropout +
    residual always, the gated activation if ``can_fuse_gated_forward`` says so).  Returns (output, lowrank_hid)."""
    kind = _kind(weight, forward_indices, backward_indices, matmul_op)
    w = cast_cached(weight, cdt)
    lowrank_hid = a2 = b2 = None
    if lowrank_first is not None and lowrank_second is not None:
        lowrank_hid = ops.gemm(x2d, cast_cached(lowrank_first, cdt))
        a2, b2 = lowrank_hid, cast_cached(lowrank_second, cdt)
    if kind == "dense":
        out = ops.gemm(x2d, w, bias=bias, a2=a2, b2=b2, epilogue=epilogue, act=act, out=out, out2=out2, aux=aux,
                       dropout_p=dropout_p, seed=seed, elem_offset=elem_offset, out_dtype=out_dtype)
    else:
        assert epilogue in (N.EPI_STORE, N.EPI_GLU_FWD, N.EPI_DROPOUT_RESIDUAL)
        fused = {}
        if epilogue != N.EPI_STORE:
            fused = dict(epilogue=epilogue, act=act, out2=out2, aux=aux, dropout_p=dropout_p, seed=seed,
                         elem_offset=elem_offset)
        if kind == "native":
            fwd, _, _ = native_tables(forward_indices, backward_indices, weight.shape[1])
            out_features = fwd.shape[0] * weight.shape[-1]
            out = _bs_forward(x2d, w, fwd, out_features, out=out, bias=bias, a2=a2, b2=b2, out_dtype=out_dtype, **fused)
        else:
            fwd, fwd_count, _, _, _ = matmul_op._tables(x2d.device)
            out = _bs_forward(x2d, w, fwd, matmul_op.out_features, out=out, bias=bias, a2=a2, b2=b2,
                              out_dtype=out_dtype, count=fwd_count, **fused)
    return out, lowrank_hid


def can_fuse_gated_forward(weight, forward_indices, backward_indices, matmul_op, cdt) -> bool:
    """Whether the block-sparse forward product of a gated input projection can carry the activation in its
    epilogue: bf16 tensor-core path, 128-wide blocks, gate and linear blocks reading the same input blocks."""
    kind = _kind(weight, forward_indices, backward_indices, matmul_op)
    if kind == "dense" or cdt != torch.bfloat16 or weight.shape[-1] != 128:
        return False
    if kind == "native":
        fwd, _, _ = native_tables(forward_indices, backward_indices, weight.shape[1])
        return fwd.shape[0] % 2 == 0 and gate_and_linear_blocks_pair_up(fwd)
    fwd, fwd_count, _, _, _ = matmul_op._tables(weight.device)
    return fwd.shape[0] % 2 == 0 and gate_and_linear_blocks_pair_up(fwd, fwd_count)


_weight_grad_reducer = None


def set_weight_grad_reducer(reducer):
    """Install (or remove, with None) a ``dist.ScatteredGradReducer``: dense weight-gradient GEMMs of weights it
    has registered add their tiles into the owning rank's replica instead of storing them, and the gradient
    returned to autograd for such a weight is None (the reducer delivers the sum)."""
    global _weight_grad_reducer
    previous, _weight_grad_reducer = _weight_grad_reducer, reducer
    return previous


def dense_weight_grad(dy2d, x2d, weight):
    """dW = dyT . x for a dense weight (linear.py:304-305 of the reference), through the installed reducer if any."""
    reducer = _weight_grad_reducer
    # the scattering epilogue exists in the bf16 tensor-core kernel only: fp32 products keep the plain gradient,
    # which the caller's gradient hook (dist.GradSync) then reduces like any other
    target = reducer.target(weight) if (reducer is not None and dy2d.dtype == torch.bfloat16) else None
    if target is None:
        return ops.gemm(dy2d, x2d, a_mn_major=True, b_mn_major=True, out_dtype=weight.dtype)
    out, scatter = target
    ops.gemm(dy2d, x2d, a_mn_major=True, b_mn_major=True, out=out, scatter=scatter)
    reducer.gradient_launched(weight)
    return None


def weight_grad(kind, dy2d, x2d, weight, forward_indices, backward_indices, matmul_op):
    """dW in the weight's own storage format for a dense, native block-sparse or triton-ordered weight."""
    if kind == "dense":
        return dense_weight_grad(dy2d, x2d, weight)
    if kind == "native":
        tables = native_tables(forward_indices, backward_indices, weight.shape[1])
        return _bs_wgrad(dy2d, x2d, weight, tables[2], weight.dtype)
    return _bs_wgrad(dy2d, x2d, weight, matmul_op._tables(dy2d.device)[4], weight.dtype)


def input_grad(kind, dy2d, weight, forward_indices, backward_indices, matmul_op, cdt, a2=None, b2=None, **epilogue):
    """dX = dY . W (+ low-rank continuation a2 . b2) for any weight kind; ``epilogue`` forwards the fused
    activation-backward arguments of ``ops.gemm`` (epilogue, act, aux, out, out2)."""
    w = cast_cached(weight, cdt)
    if kind == "dense":
        return ops.gemm(dy2d, w, b_mn_major=True, a2=a2, b2=b2, **epilogue)
    if kind == "native":
        tables = native_tables(forward_indices, backward_indices, weight.shape[1])
        return _bs_dgrad(dy2d, w, tables[1], weight.shape[0], a2=a2, b2=b2, **epilogue)
    t = matmul_op._tables(dy2d.device)
    return _bs_dgrad(dy2d, w, t[2], matmul_op.in_features, a2=a2, b2=b2, count=t[3], **epilogue)


def linear_backward_core(dy2d, x2d, lowrank_hid, weight, lowrank_first, lowrank_second, forward_indices,
                         backward_indices, matmul_op, needs_input_grad, cdt, *, dgrad_epilogue=N.EPI_STORE, act=0,
                         dgrad_aux=None, dgrad_out=None, dgrad_out2=None, bias_dtype=None, on_param_grads=None,
                         grad_bias=None):
    """Gradients of linear_forward_core in the reference's order
    (input, weight, bias, lowrank_first, lowrank_second); ``x2d`` / ``dy2d`` are in the compute dtype.
    Weight-like gradients come back in their parameter's dtype.  The input gradient may carry a fused
    activation-backward epilogue.  ``on_param_grads(weight, bias, lowrank_first, lowrank_second)``
    is called once the parameter gradients are launched and before the input gradient is, so a data-parallel
    caller can start their reduction underneath the input-gradient product; it returns the four values to hand
    back (None for a gradient it has taken over).  ``grad_bias``: the bias gradient if the caller already has it
    (the kernel that produced ``dy2d`` can emit its column sums)."""
    kind = _kind(weight, forward_indices, backward_indices, matmul_op)
    need_x, need_w, need_b, need_l1, need_l2 = (list(needs_input_grad) + [False] * 5)[:5]
    grad_input = grad_weight = grad_l1 = grad_l2 = None
    has_lowrank = lowrank_first is not None and lowrank_second is not None
    l1 = cast_cached(lowrank_first, cdt) if has_lowrank else None
    l2 = cast_cached(lowrank_second, cdt) if has_lowrank else None
    grad_lowrank_hid = None
    if has_lowrank and (need_x or need_l1):
        grad_lowrank_hid = ops.gemm(dy2d, l2, b_mn_major=True)  # [tokens, rank] = dy @ L2
    if has_lowrank and need_l2:
        grad_l2 = ops.gemm(dy2d, lowrank_hid, a_mn_major=True, b_mn_major=True, out_dtype=lowrank_second.dtype)
    if has_lowrank and need_l1:
        grad_l1 = ops.gemm(grad_lowrank_hid, x2d, a_mn_major=True, b_mn_major=True, out_dtype=lowrank_first.dtype)
    if not need_b:
        grad_bias = None
    elif grad_bias is None:
        grad_bias = ops.column_sum(dy2d)
    if need_b:
        if bias_dtype is not None and bias_dtype != torch.float32:
            grad_bias = ops.cast(grad_bias, bias_dtype)
    if need_w:
        grad_weight = weight_grad(kind, dy2d, x2d, weight, forward_indices, backward_indices, matmul_op)
    if on_param_grads is not None:
        grad_weight, grad_bias, grad_l1, grad_l2 = on_param_grads(grad_weight, grad_bias, grad_l1, grad_l2)
    if need_x:
        a2, b2 = (grad_lowrank_hid, l1) if has_lowrank else (None, None)
        epilogue = {}
        if dgrad_epilogue != N.EPI_STORE:
            epilogue = dict(epilogue=dgrad_epilogue, act=act, aux=dgrad_aux, out=dgrad_out, out2=dgrad_out2)
        grad_input = input_grad(kind, dy2d, weight, forward_indices, backward_indices, matmul_op, cdt, a2=a2, b2=b2,
                                **epilogue)
    return grad_input, grad_weight, grad_bias, grad_l1, grad_l2


class GeneralizedMatrix(nn.Module):
    """A module that stores a shared weight tensor for use in GeneralizedLinear layers."""

    def __init__(self, in_features: int, out_features: int, blocksparse_layout: Optional[str] = None,
                 lowrank_dim: int = 0, blocksparse_backend: str = "native"):
        super().__init__()
        self.out_features, self.in_features = out_features, in_features
        self.blocksparse_backend = blocksparse_backend
        self._matmul_op = None
        scale = math.sqrt(2.0 / (5 * min(out_features, in_features)))

        if blocksparse_layout is None:
            assert blocksparse_backend == "native", "triton is only used for block-sparse matrices"
            self.weight = nn.Parameter(torch.empty(out_features, in_features))
            nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
            self.layout = self.forward_indices = self.backward_indices = None
        else:
            layout = get_blocksparse_layout(out_features, in_features, blocksparse_layout)
            assert out_features / layout.shape[0] == in_features / layout.shape[1] == in_features // layout.shape[1]
            block_size = in_features // layout.shape[1]
            self.register_buffer("layout", layout, persistent=True)
            if blocksparse_backend == "native":
                forward_indices, backward_indices = get_indices_from_layout(layout)
                self.register_buffer("forward_indices", forward_indices, persistent=True)
                self.register_buffer("backward_indices", backward_indices, persistent=True)
                blocks_per_input = self.forward_indices.numel() // (in_features // block_size)
                self.weight = nn.Parameter(torch.empty(in_features, blocks_per_input, block_size))
            elif blocksparse_backend == "triton":
                self.weight = nn.Parameter(torch.empty(1, int(self.layout.sum().item()), block_size, block_size))
                self.forward_indices = self.backward_indices = None
            else:
                raise NotImplementedError(f"Unrecognized sparsity backend: {blocksparse_backend}")
            nn.init.normal_(self.weight, std=scale)

        if lowrank_dim:
            self.lowrank_first = nn.Parameter(torch.zeros(lowrank_dim, self.in_features))
            self.lowrank_second = nn.Parameter(torch.zeros(self.out_features, lowrank_dim))
            nn.init.normal_(self.lowrank_first, std=scale)
            nn.init.normal_(self.lowrank_second, std=scale)
        else:
            self.lowrank_first = self.lowrank_second = None

    @property
    def shape(self):
        return self.out_features, self.in_features

    def __repr__(self):
        return f"{self.__class__.__name__}{tuple(self.shape)}"

    def forward(self, input: torch.Tensor, *, ignore_lowrank: bool = False):
        """Multiply by this matrix like torch.nn.Linear(..., bias=False).

        :param ignore_lowrank: if True, the low-rank components (lowrank_dim) are left out
        """
        use_lowrank = self.lowrank_first is not None and not ignore_lowrank
        return _GeneralizedLinear.apply(
            input, self.weight, None, self.lowrank_first if use_lowrank else None,
            self.lowrank_second if use_lowrank else None, self.forward_indices, self.backward_indices, self.matmul_op)

    @property
    def matmul_op(self) -> Optional[TritonMatmulForLinearLayer]:
        if self.blocksparse_backend == "native":
            return None
        if self._matmul_op is None:
            if self.weight.ndim != 4 or self.weight.shape[0] != 1 or self.weight.shape[-1] != self.weight.shape[-2]:
                raise ValueError("weights are not in triton format")
            self._matmul_op = TritonMatmulForLinearLayer(self.layout, self.weight.shape[-1])
        return self._matmul_op


class GeneralizedLinear(nn.Linear):
    """A linear layer with a shared full-rank matrix and an individual low-rank adapter."""

    def __init__(self, matrix: GeneralizedMatrix, adapter_dim: int = 0, bias: bool = True):
        nn.Module.__init__(self)
        self.matrix = matrix
        self.out_features, self.in_features = self.matrix.shape
        self.bias = nn.Parameter(torch.zeros(self.out_features)) if bias else None
        if adapter_dim != 0:
            self.adapter_first = nn.Parameter(torch.zeros(adapter_dim, self.in_features))
            self.adapter_second = nn.Parameter(torch.zeros(self.out_features, adapter_dim))
            nn.init.xavier_normal_(self.adapter_first)  # LoRA-style: first random, second zero
            nn.init.zeros_(self.adapter_second)
        else:
            self.adapter_first = self.adapter_second = None

    def get_combined_lowrank_components(self) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        """The matrix's shared low-rank pair and this layer's adapter, concatenated along the rank dim."""
        firsts = [t for t in (self.matrix.lowrank_first, self.adapter_first) if t is not None]
        seconds = [t for t in (self.matrix.lowrank_second, self.adapter_second) if t is not None]
        assert len(firsts) == len(seconds)
        if not firsts:
            return None, None
        if len(firsts) == 1:
            return firsts[0], seconds[0]
        return torch.cat(firsts, dim=0), torch.cat(seconds, dim=1)

    @property
    def weight(self):
        return self.matrix.weight

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return _GeneralizedLinear.apply(
            input, self.weight, self.bias, *self.get_combined_lowrank_components(),
            self.matrix.forward_indices, self.matrix.backward_indices, self.matrix.matmul_op)


class _GeneralizedLinear(torch.autograd.Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, *args):
        output, tensors_to_save = _GeneralizedLinear.forward_functional(*args)
        ctx.save_for_backward(*tensors_to_save)
        ctx._matmul_op = args[-1] if len(args) >= 8 else None
        return output

    @staticmethod
    def forward_functional(input: torch.Tensor, main_weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                           lowrank_first: Optional[torch.Tensor] = None,
                           lowrank_second: Optional[torch.Tensor] = None,
                           forward_indices: Optional[torch.Tensor] = None,
                           backward_indices: Optional[torch.Tensor] = None,
                           matmul_op: Optional[TritonMatmulForLinearLayer] = None):
        """Pure functional interface for use in other autograd functions: returns (output, tensors_to_save)
        with tensors_to_save = [input, lowrank_hid, main_weight, lowrank_first, lowrank_second,
        backward_indices]."""
        cdt = resolve_compute_dtype(input)
        x2d = ops.cast(input.reshape(-1, input.shape[-1]).contiguous(), cdt)
        out, lowrank_hid = linear_forward_core(x2d, main_weight, bias, lowrank_first, lowrank_second,
                                               forward_indices, backward_indices, matmul_op, cdt)
        output = out.view(*input.shape[:-1], out.shape[-1])
        return output, [input, lowrank_hid, main_weight, lowrank_first, lowrank_second, backward_indices]

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_output: torch.Tensor):
        grads = _GeneralizedLinear.backward_functional(grad_output, ctx.saved_tensors, ctx.needs_input_grad,
                                                       ctx._matmul_op)
        return tuple(grads) + (None,) * (len(ctx.needs_input_grad) - len(grads))

    @staticmethod
    def backward_functional(grad_output: torch.Tensor, saved_tensors: Sequence[torch.Tensor],
                            needs_input_grad: List[bool], matmul_op: Optional[TritonMatmulForLinearLayer] = None
                            ) -> Sequence[Optional[torch.Tensor]]:
        """Pure functional interface: gradients for (input, main_weight, bias, lowrank_first, lowrank_second,
        forward_indices, backward_indices), ``None`` where not needed."""
        input, lowrank_hid, main_weight, lowrank_first, lowrank_second, backward_indices = saved_tensors
        needs = list(needs_input_grad)[:7] + [False] * max(0, 7 - len(needs_input_grad))
        cdt = lowrank_hid.dtype if lowrank_hid is not None else resolve_compute_dtype(input)
        x2d = ops.cast(input.reshape(-1, input.shape[-1]).contiguous(), cdt)
        dy2d = ops.cast(grad_output.reshape(-1, grad_output.shape[-1]).contiguous(), cdt)
        sparse_native = matmul_op is None and main_weight.ndim == 3
        g_in, g_w, g_b, g_l1, g_l2 = linear_backward_core(
            dy2d, x2d, lowrank_hid, main_weight, lowrank_first, lowrank_second, None,
            backward_indices if sparse_native else None, matmul_op, needs[:5], cdt, bias_dtype=None)
        if g_in is not None:
            g_in = ops.cast(g_in, input.dtype).view(input.shape)
        grads = (g_in, g_w, g_b, g_l1, g_l2, None, None)
        return tuple(g if needed else None for g, needed in zip_longest(grads, needs[:7]))


__all__ = ["GeneralizedMatrix", "GeneralizedLinear", "_GeneralizedLinear", "TritonMatmulForLinearLayer",
           "TRITON_PAD_TO", "pad_to_multiple"]
