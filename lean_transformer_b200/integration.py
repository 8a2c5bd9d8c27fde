"""Swapping the CUDA path into models built from the reference package.

``convert_model(model)`` walks any ``nn.Module`` built with the reference's classes (``lean_transformer.ffn.LeanFFN``,
``lean_transformer.blocksparse.linear.GeneralizedLinear`` / ``GeneralizedMatrix``) and replaces them, in place, with
this package's drop-ins.  Parameters and buffers are re-used (the very same ``nn.Parameter`` objects), so optimizer
state, weight sharing between layers (``share_large_matrices``) and checkpoints keep working.  Classes are recognised
by name, so the reference does not have to be importable here.
"""
from typing import Dict

import torch.nn as nn

from .blocksparse.linear import GeneralizedLinear, GeneralizedMatrix
from .ffn import LeanFFN


def _convert_matrix(ref, memo: Dict[int, nn.Module]) -> GeneralizedMatrix:
    if id(ref) in memo:
        return memo[id(ref)]
    new = GeneralizedMatrix.__new__(GeneralizedMatrix)
    nn.Module.__init__(new)
    new.out_features, new.in_features = ref.out_features, ref.in_features
    new.blocksparse_backend = getattr(ref, "blocksparse_backend", "native")
    new._matmul_op = None
    new.weight = ref.weight
    for name in ("layout", "forward_indices", "backward_indices"):
        value = getattr(ref, name, None)
        if value is not None:
            new.register_buffer(name, value, persistent=True)
        else:
            setattr(new, name, None)
    new.lowrank_first, new.lowrank_second = ref.lowrank_first, ref.lowrank_second
    memo[id(ref)] = new
    return new


def _convert_linear(ref, memo: Dict[int, nn.Module]) -> nn.Module:
    if type(ref).__name__ != "GeneralizedLinear" or isinstance(ref, GeneralizedLinear):
        return ref
    if id(ref) in memo:
        return memo[id(ref)]
    new = GeneralizedLinear.__new__(GeneralizedLinear)
    nn.Module.__init__(new)
    new.matrix = _convert_matrix(ref.matrix, memo)
    new.out_features, new.in_features = ref.out_features, ref.in_features
    new.bias = ref.bias
    new.adapter_first, new.adapter_second = ref.adapter_first, ref.adapter_second
    memo[id(ref)] = new
    return new


def _convert_ffn(ref, memo: Dict[int, nn.Module]) -> LeanFFN:
    new = LeanFFN.__new__(LeanFFN)
    nn.Module.__init__(new)
    new.i2h_proj = _convert_linear(ref.i2h_proj, memo)
    new.h2o_proj = _convert_linear(ref.h2o_proj, memo)
    new.pre_layer_norm = ref.pre_layer_norm
    new.post_layer_norm = ref.post_layer_norm
    new.activation = ref.activation
    new.gated, new.dropout, new.residual = ref.gated, ref.dropout, ref.residual
    new.ffn_custom_grad = ref.ffn_custom_grad
    new.train(ref.training)
    return new


def convert_model(model: nn.Module, convert_linears: bool = True) -> nn.Module:
    """Replace every reference ``LeanFFN`` (and, optionally, stand-alone ``GeneralizedLinear``) inside ``model``
    by the CUDA drop-in.  Returns ``model``."""
    memo: Dict[int, nn.Module] = {}

    def visit(parent: nn.Module):
        for name, child in list(parent.named_children()):
            kind = type(child).__name__
            if kind == "LeanFFN" and not isinstance(child, LeanFFN):
                setattr(parent, name, _convert_ffn(child, memo))
            elif convert_linears and kind == "GeneralizedLinear" and not isinstance(child, GeneralizedLinear):
                setattr(parent, name, _convert_linear(child, memo))
            else:
                visit(child)

    visit(model)
    return model
