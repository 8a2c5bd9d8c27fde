"""Swapping the CUDA path into models built from the reference package.

``convert_model(model)`` walks any ``nn.Module`` built with the reference's classes (``lean_transformer.ffn.LeanFFN``,
``lean_transformer.blocksparse.linear.GeneralizedLinear`` / ``GeneralizedMatrix``) and replaces them, in place, with
this package's drop-ins.  Parameters and buffers are re-used (the very same ``nn.Parameter`` objects), so optimizer
state, weight sharing between layers (``share_large_matrices``) and checkpoints keep working.  Classes are recognised
by name, so the reference does not have to be importable here.

``LeanSelfAttention`` blocks are converted too: LayerNorm, qkv projection, the attention core (the reference's
``SimpleAttentionCore`` / ``RotaryAttentionCore``; any other core module is kept and called as is) and output
projection + dropout + residual run on this package's kernels.

Every drop-in is an instance of a class derived from BOTH this package's class and the class it replaces (this
package's first in the method resolution order, so all behaviour is this package's).  The model's own code keeps
recognising its modules that way: ``LeanTransformer.set_optimizations`` finds its FFNs with ``isinstance(module,
LeanFFN)`` (lean_transformer/transformer.py:139-147, which otherwise asserts on any other module that has an
``ffn_custom_grad`` attribute) and re-generates block-sparse operators with ``isinstance(module, GeneralizedMatrix)``
(:149-152).
"""
from typing import Dict, Tuple

import torch.nn as nn

from .attn import LeanSelfAttention, RotaryAttentionCore, SimpleAttentionCore
from .blocksparse.linear import GeneralizedLinear, GeneralizedMatrix
from .ffn import LeanFFN

_DROPIN_CLASSES: Dict[Tuple[type, type], type] = {}


def _dropin_class(ours: type, theirs: type) -> type:
    """``ours`` if ``theirs`` already derives from it, else a class derived from (ours, theirs)."""
    if issubclass(theirs, ours):
        return theirs
    key = (ours, theirs)
    cls = _DROPIN_CLASSES.get(key)
    if cls is None:
        cls = type(ours.__name__, (ours, theirs), {"__module__": ours.__module__, "__doc__": ours.__doc__})
        _DROPIN_CLASSES[key] = cls
    return cls


def _convert_matrix(ref, memo: Dict[int, nn.Module]) -> GeneralizedMatrix:
    if isinstance(ref, GeneralizedMatrix):
        return ref
    if id(ref) in memo:
        return memo[id(ref)]
    cls = _dropin_class(GeneralizedMatrix, type(ref))
    new = cls.__new__(cls)
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
    cls = _dropin_class(GeneralizedLinear, type(ref))
    new = cls.__new__(cls)
    nn.Module.__init__(new)
    new.matrix = _convert_matrix(ref.matrix, memo)
    new.out_features, new.in_features = ref.out_features, ref.in_features
    new.bias = ref.bias
    new.adapter_first, new.adapter_second = ref.adapter_first, ref.adapter_second
    memo[id(ref)] = new
    return new


def _convert_ffn(ref, memo: Dict[int, nn.Module]) -> LeanFFN:
    if id(ref) in memo:
        return memo[id(ref)]
    cls = _dropin_class(LeanFFN, type(ref))
    new = cls.__new__(cls)
    nn.Module.__init__(new)
    new.i2h_proj = _convert_linear(ref.i2h_proj, memo)
    new.h2o_proj = _convert_linear(ref.h2o_proj, memo)
    new.pre_layer_norm = ref.pre_layer_norm
    new.post_layer_norm = ref.post_layer_norm
    new.activation = ref.activation
    new.gated, new.dropout, new.residual = ref.gated, ref.dropout, ref.residual
    new.ffn_custom_grad = ref.ffn_custom_grad
    new.train(ref.training)
    memo[id(ref)] = new
    return new


def _convert_core(ref, memo: Dict[int, nn.Module]) -> nn.Module:
    """The reference's SimpleAttentionCore / RotaryAttentionCore (lean_transformer/attn.py:85-171) become this
    package's kernel-backed cores; the rotary table module is kept (same buffers).  Any other core is passed through."""
    name = type(ref).__name__
    if name not in ("SimpleAttentionCore", "RotaryAttentionCore") or isinstance(ref, SimpleAttentionCore):
        return ref
    if id(ref) in memo:
        return memo[id(ref)]
    ours = RotaryAttentionCore if name == "RotaryAttentionCore" else SimpleAttentionCore
    cls = _dropin_class(ours, type(ref))
    new = cls.__new__(cls)
    nn.Module.__init__(new)
    new.attention_dropout = ref.attention_dropout
    new.hidden_size, new.num_attention_heads = ref.hidden_size, ref.num_attention_heads
    new.attention_head_size = ref.attention_head_size
    if name == "RotaryAttentionCore":
        new.rotary_emb = ref.rotary_emb
    new.train(ref.training)
    memo[id(ref)] = new
    return new


def _convert_attention(ref, memo: Dict[int, nn.Module], convert_core: bool = True) -> LeanSelfAttention:
    """The attention block (lean_transformer/attn.py:11-82): LayerNorm, both projections and the reference's own
    attention cores move to this package's kernels; a custom core module is passed through untouched."""
    if id(ref) in memo:
        return memo[id(ref)]
    cls = _dropin_class(LeanSelfAttention, type(ref))
    new = cls.__new__(cls)
    nn.Module.__init__(new)
    new.hidden_size = ref.hidden_size
    new.attention_core = _convert_core(ref.attention_core, memo) if convert_core else ref.attention_core
    new.qkv_proj = _convert_linear(ref.qkv_proj, memo)
    new.out_proj = _convert_linear(ref.out_proj, memo)
    new.pre_layer_norm, new.post_layer_norm = ref.pre_layer_norm, ref.post_layer_norm
    new.output_dropout = ref.output_dropout
    new.residual, new.checkpoint_attention_core = ref.residual, ref.checkpoint_attention_core
    new.train(ref.training)
    memo[id(ref)] = new
    return new


def _is_reference(module: nn.Module, name: str, ours: type) -> bool:
    return type(module).__name__ == name and not isinstance(module, ours)


def convert_model(model: nn.Module, convert_linears: bool = True, convert_attention: bool = True,
                  convert_attention_core: bool = True) -> nn.Module:
    """Replace every reference ``LeanFFN`` (and, optionally, ``LeanSelfAttention`` block and stand-alone
    ``GeneralizedLinear``) inside ``model`` by the CUDA drop-in.  Returns the converted model: ``model`` itself,
    modified in place, unless ``model`` IS one of those modules, in which case its drop-in is returned.

    ``convert_attention_core=False`` keeps the attention blocks' own core modules.  The kernel-backed cores compute in
    bfloat16 (under ``torch.autocast`` or on bfloat16 tensors) and raise on float32 tensors outside autocast, so a
    model that is to run in plain float32 keeps its cores."""
    memo: Dict[int, nn.Module] = {}
    if _is_reference(model, "LeanFFN", LeanFFN):
        return _convert_ffn(model, memo)
    if convert_attention and _is_reference(model, "LeanSelfAttention", LeanSelfAttention):
        return _convert_attention(model, memo, convert_attention_core)
    if convert_linears and _is_reference(model, "GeneralizedLinear", GeneralizedLinear):
        return _convert_linear(model, memo)

    def visit(parent: nn.Module):
        for name, child in list(parent.named_children()):
            if _is_reference(child, "LeanFFN", LeanFFN):
                setattr(parent, name, _convert_ffn(child, memo))
            elif convert_attention and _is_reference(child, "LeanSelfAttention", LeanSelfAttention):
                setattr(parent, name, _convert_attention(child, memo, convert_attention_core))
            elif convert_linears and _is_reference(child, "GeneralizedLinear", GeneralizedLinear):
                setattr(parent, name, _convert_linear(child, memo))
            else:
                if convert_attention_core and isinstance(child, LeanSelfAttention):
                    child.attention_core = _convert_core(child.attention_core, memo)  # block converted earlier
                visit(child)

    visit(model)
    # LeanTransformer keeps the layer sequence it runs in a plain tuple outside its module tree
    # (lean_transformer/transformer.py:33-45); its wrappers still hold the replaced modules.  The memo maps each old
    # module to the drop-in it already got, and the sequence keeps its checkpointing settings.
    for module in list(model.modules()):
        cached = getattr(module, "_sequential", None)
        if isinstance(cached, tuple):
            for sequence in cached:
                if isinstance(sequence, nn.Module):
                    visit(sequence)
    return model
