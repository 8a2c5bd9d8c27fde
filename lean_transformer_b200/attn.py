"""Attention block shell with its projections on the sm_100a kernels (lean_transformer/attn.py:11-82).

``LeanSelfAttention`` keeps the reference's constructor, attributes (``qkv_proj``, ``out_proj``, ``pre_layer_norm``,
``post_layer_norm``, ``output_dropout``, ``attention_core``, ``residual``, ``checkpoint_attention_core``) and
``forward(hidden_states, attention_mask=None, output_attentions=False)``.  What runs on this library's kernels:

  pre-LayerNorm                       ``leanffn_layer_norm_forward / backward``  (attn.py:67)
  qkv projection                      one GEMM (+ bias, low rank, block sparsity)  (attn.py:68)
  output projection -> dropout -> + residual.to(float32)
                                      ONE GEMM with the fused epilogue  (attn.py:73-78)

The attention core itself (attn.py:85-149: rotary, Q.K^T, softmax, P.V) is NOT a kernel of this library: the block
calls whatever ``attention_core`` module it is given, which for converted models is the model's own core.  The
default core below restates the reference's simple core with stock tensor operators so that the block is usable on
its own; it is a convenience, not part of the accelerated path.
"""
import math
from typing import Optional

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .blocksparse.linear import GeneralizedLinear, _GeneralizedLinear
from .ffn import _LayerNormFunction
from .fused_linear import linear_dropout_residual


class SimpleAttentionCore(nn.Module):
    """softmax(Q K^T / sqrt(d) + mask) V with stock tensor operators (lean_transformer/attn.py:85-149).
    Returns (outputs [batch, query_len, hidden], probs [batch, heads, query_len, kv_len])."""

    def __init__(self, hidden_size: int, num_attention_heads: int, attention_probs_dropout: float = 0.0):
        super().__init__()
        assert hidden_size % num_attention_heads == 0
        self.attention_dropout = nn.Dropout(attention_probs_dropout)
        self.hidden_size, self.num_attention_heads = hidden_size, num_attention_heads
        self.attention_head_size = hidden_size // num_attention_heads

    def forward(self, query, key, value, attention_mask):
        if attention_mask is not None:
            assert torch.is_floating_point(attention_mask), "expected float mask with negative values for masked items"
        heads = self.num_attention_heads
        split = lambda t: t.view(*t.shape[:-1], heads, -1).permute(0, 2, 1, 3)  # noqa: E731
        q, k, v = split(query), split(key), split(value)
        scores = torch.matmul(q, k.transpose(-1, -2) / math.sqrt(q.shape[-1]))
        if attention_mask is not None:
            scores = scores + attention_mask
        probs = self.attention_dropout(torch.softmax(scores, dim=-1))
        out = torch.matmul(probs, v).transpose(2, 1).flatten(2)
        return out, probs


class LeanSelfAttention(nn.Module):
    """Attention layer whose LayerNorm and projections run on the sm_100a kernels; same interface as the
    reference's ``LeanSelfAttention``.

    :param hidden_size: base hidden size of the transformer, before q/k/v projections
    :param num_attention_heads: number of heads
    :param dropout: hidden dropout probability, applied to the output projection (before adding the residual)
    :param layer_norm_eps: see torch.nn.functional.layer_norm
    :param post_layer_norm: additional layer norm on the projected attention outputs before the residual
    :param residual: if True, adds the original layer input to the final layer output
    :param attention_core: module ``(query, key, value, attention_mask) -> (outputs, probs)``
    :param checkpoint_attention_core: re-compute attention weights during backward instead of storing them
    :param qkv_proj: custom QKV projection layer (hidden_size -> 3 * hidden_size)
    :param out_proj: custom output projection layer (hidden_size -> hidden_size)
    :param kwargs: passed to the default attention core
    """

    def __init__(self, hidden_size: int, num_attention_heads: int, dropout: float = 0, layer_norm_eps: float = 1e-12,
                 post_layer_norm: bool = False, qkv_proj: Optional[nn.Linear] = None,
                 out_proj: Optional[nn.Linear] = None, residual: bool = True,
                 attention_core: Optional[nn.Module] = None, checkpoint_attention_core: bool = True, **kwargs):
        super().__init__()
        if attention_core is None:
            attention_core = SimpleAttentionCore(hidden_size, num_attention_heads, **kwargs)
        else:
            assert len(kwargs) == 0, f"Unexpected parameters: {kwargs}"
        self.hidden_size = hidden_size
        self.attention_core = attention_core
        self.qkv_proj = nn.Linear(hidden_size, hidden_size * 3) if qkv_proj is None else qkv_proj
        self.out_proj = nn.Linear(hidden_size, hidden_size) if out_proj is None else out_proj
        assert self.qkv_proj.in_features == self.out_proj.in_features == self.out_proj.out_features == hidden_size
        assert self.qkv_proj.out_features == hidden_size * 3
        self.pre_layer_norm = nn.LayerNorm(hidden_size, eps=layer_norm_eps)
        self.post_layer_norm = nn.LayerNorm(hidden_size, eps=layer_norm_eps) if post_layer_norm else None
        self.output_dropout = nn.Dropout(dropout, inplace=False)
        self.residual, self.checkpoint_attention_core = residual, checkpoint_attention_core

    @staticmethod
    def _project(proj: nn.Linear, x: torch.Tensor) -> torch.Tensor:
        if isinstance(proj, GeneralizedLinear):
            return proj(x)
        return _GeneralizedLinear.apply(x, proj.weight, proj.bias, None, None, None, None, None)

    def forward(self, hidden_states, attention_mask=None, output_attentions=False):
        if not hidden_states.is_cuda:
            raise RuntimeError("LeanSelfAttention (lean_transformer_b200) needs CUDA tensors: its LayerNorm and "
                               "projections exist only as sm_100a kernels")
        ln = self.pre_layer_norm
        flat = hidden_states.reshape(-1, hidden_states.shape[-1])
        hidden_states_ln = _LayerNormFunction.apply(flat, ln.weight, ln.bias, ln.eps).view(*hidden_states.shape)
        qkv_output = self._project(self.qkv_proj, hidden_states_ln)
        query, key, value = qkv_output.split(self.hidden_size, dim=qkv_output.ndim - 1)
        attention_output, attention_probs = self._maybe_checkpoint(self.attention_core, query, key, value,
                                                                   attention_mask)
        p, training = self.output_dropout.p, self.training
        residual = hidden_states.to(torch.float32, copy=False) if self.residual else None
        if self.post_layer_norm is None:
            # out_proj -> dropout -> + residual as one product with a fused epilogue
            outputs = linear_dropout_residual(attention_output, self.out_proj, residual, p, training)
        else:
            outputs = self._project(self.out_proj, attention_output)
            pln = self.post_layer_norm
            outputs = _LayerNormFunction.apply(outputs.reshape(-1, outputs.shape[-1]), pln.weight, pln.bias,
                                               pln.eps).view(*outputs.shape)
            outputs = self.output_dropout(outputs)
            if residual is not None:
                outputs = outputs + residual
        return (outputs, attention_probs) if output_attentions else (outputs,)

    def _maybe_checkpoint(self, func, *args):
        if torch.is_grad_enabled() and self.checkpoint_attention_core:
            return checkpoint(func, *args, use_reentrant=True)
        return func(*args)
