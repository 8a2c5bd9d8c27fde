"""Activation registry, padding helper and logger: the host-side counterparts of the reference's
``lean_transformer/utils.py`` (ACT2FN :80, GELU :41-50, pad_to_multiple :53-77, get_logger :9-12).

Activations are named objects carrying the id of a device function fused into the GEMM epilogues;
calling one on a CUDA tensor runs the stand-alone activation kernel (with autograd support).
"""
import logging
from typing import List, Union

import torch
import torch.nn.functional as F

from . import _native as N


def get_logger(name: str) -> logging.Logger:
    return logging.getLogger(name)


class _ActivationFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, act_id: int):
        from . import ops

        ctx.act_id = act_id
        ctx.save_for_backward(x)
        flat = x.contiguous().view(-1, x.shape[-1])
        return ops.activation_forward(flat, False, act_id).view(x.shape)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        from . import ops

        (x,) = ctx.saved_tensors
        flat = x.contiguous().view(-1, x.shape[-1])
        g = ops.cast(grad_output.contiguous().view(-1, x.shape[-1]), x.dtype)
        dpre, _ = ops.activation_backward(g, flat, False, ctx.act_id)
        return dpre.view(x.shape), None


class Activation:
    """An elementwise nonlinearity the CUDA kernels implement (``act_id`` = LEANFFN_ACT_* value)."""

    def __init__(self, name: str, act_id: int):
        self.name, self.act_id = name, act_id

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return _ActivationFunction.apply(x, self.act_id)

    def __repr__(self):
        return f"Activation({self.name})"


_GELU_TANH = Activation("gelu_fused", N.ACT_GELU_TANH)
_GELU_ERF = Activation("gelu", N.ACT_GELU_ERF)
_RELU = Activation("relu", N.ACT_RELU)
_SILU = Activation("silu", N.ACT_SILU)
_TANH = Activation("tanh", N.ACT_TANH)
_SIGMOID = Activation("sigmoid", N.ACT_SIGMOID)
_IDENTITY = Activation("linear", N.ACT_IDENTITY)

# Same keys as transformers' ACT2FN for every activation the kernels implement, plus "gelu_fused".
ACT2FN = {
    "gelu_fused": _GELU_TANH,
    "gelu_new": _GELU_TANH,
    "gelu_fast": _GELU_TANH,
    "gelu_pytorch_tanh": _GELU_TANH,
    "gelu": _GELU_ERF,
    "gelu_python": _GELU_ERF,
    "relu": _RELU,
    "silu": _SILU,
    "swish": _SILU,
    "tanh": _TANH,
    "sigmoid": _SIGMOID,
    "linear": _IDENTITY,
}

# Foreign callables (transformers activation modules, torch functions) recognised by type / identity.
_BY_CLASS_NAME = {
    "GELUActivation": N.ACT_GELU_ERF,
    "GELU": N.ACT_GELU_ERF,
    "NewGELUActivation": N.ACT_GELU_TANH,
    "FastGELUActivation": N.ACT_GELU_TANH,
    "PytorchGELUTanh": N.ACT_GELU_TANH,
    "GELUTanh": N.ACT_GELU_TANH,
    "ReLU": N.ACT_RELU,
    "SiLU": N.ACT_SILU,
    "SiLUActivation": N.ACT_SILU,
    "Tanh": N.ACT_TANH,
    "Sigmoid": N.ACT_SIGMOID,
    "LinearActivation": N.ACT_IDENTITY,
    "Identity": N.ACT_IDENTITY,
}
_BY_FUNCTION = {
    F.relu: N.ACT_RELU, torch.relu: N.ACT_RELU, F.silu: N.ACT_SILU, torch.tanh: N.ACT_TANH, F.tanh: N.ACT_TANH,
    torch.sigmoid: N.ACT_SIGMOID, F.sigmoid: N.ACT_SIGMOID, F.gelu: N.ACT_GELU_ERF,
}


def resolve_activation(activation) -> int:
    """Map an activation callable to the id of its device implementation; unknown callables are an error
    (no Python fallback is attempted)."""
    if isinstance(activation, Activation):
        return activation.act_id
    if isinstance(activation, str) and activation in ACT2FN:
        return ACT2FN[activation].act_id
    if isinstance(activation, torch.nn.GELU):
        return N.ACT_GELU_TANH if getattr(activation, "approximate", "none") == "tanh" else N.ACT_GELU_ERF
    # the reference's own GELU.apply (lean_transformer/utils.py:41-50) when a reference model is patched
    qualname = getattr(activation, "__qualname__", "")
    owner = getattr(activation, "__self__", None)
    if qualname.endswith("apply") and getattr(owner, "__name__", "") == "GELU":
        return N.ACT_GELU_TANH
    try:
        if activation in _BY_FUNCTION:
            return _BY_FUNCTION[activation]
    except TypeError:
        pass
    name = type(activation).__name__
    if name in _BY_CLASS_NAME:
        return _BY_CLASS_NAME[name]
    raise NotImplementedError(
        f"activation {activation!r} has no CUDA implementation in lean_transformer_b200; supported: "
        f"{sorted(ACT2FN)}"
    )


def pad_to_multiple(tensor: torch.Tensor, multiple: int, dims: Union[int, List[int]] = -1, value: float = 0):
    """Pad the given dims with ``value`` up to the next multiple; returns the same tensor object when
    nothing needs padding (lean_transformer/utils.py:53-77)."""
    dims = [dims] if isinstance(dims, int) else list(dims)
    pads = [0] * (2 * tensor.ndim)
    changed = False
    for d in dims:
        d = int(d) % tensor.ndim
        extra = -tensor.size(d) % multiple
        if extra:
            pads[2 * (tensor.ndim - d - 1) + 1] = extra
            changed = True
    return F.pad(tensor, pads, value=value) if changed else tensor
