"""CPU oracle for the LeanFFN hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU and without autograd, the algorithm of the reference
(learning-at-home/lean_transformer) for LeanFFN forward / backward and the block-sparse ("pixelfly")
linear layer.  Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import it; the
product package never does.  Tensors are CPU torch tensors (torch is the reference's own array library;
nothing here touches CUDA); the Philox mask is plain numpy integer arithmetic.

Parity status: pinned.  tests/test_oracle_golden.py checks every function below against vectors produced
by the reference itself (tests/golden/make_golden.py imports it from its source tree) for dense, gated,
post-LN, block-sparse, low-rank and dropout configurations.

Each function cites the reference lines it follows (paths relative to the reference project root).
"""
import math
from typing import Dict, Optional, Tuple

import numpy as np
import torch

# ---------------------------------------------------------------------------------------------------
# activations: lean_transformer/utils.py:24-38 (gelu_fused, gelu_fused_grad); others follow torch's definitions
# ---------------------------------------------------------------------------------------------------
ACT_NAMES = ("gelu_tanh", "gelu_erf", "relu", "silu", "tanh", "sigmoid", "identity")


def act_forward(name: str, x: torch.Tensor) -> torch.Tensor:
    if name == "gelu_tanh":  # utils.py:30: x * 0.5 * (1 + tanh(0.79788456 * x * (1 + 0.044715 * x * x)))
        t = (x * x).mul_(0.044715).add_(1.0).mul_(x).mul_(0.79788456).tanh_()  # in place: one temporary
        return t.add_(1.0).mul_(x).mul_(0.5)
    if name == "gelu_erf":
        return x * 0.5 * (1.0 + torch.erf(x / math.sqrt(2.0)))
    if name == "relu":
        return torch.clamp_min(x, 0)
    if name == "silu":
        return x * torch.sigmoid(x)
    if name == "tanh":
        return torch.tanh(x)
    if name == "sigmoid":
        return torch.sigmoid(x)
    if name == "identity":
        return x
    raise ValueError(name)


def act_grad(name: str, x: torch.Tensor) -> torch.Tensor:
    """d act(x) / dx"""
    if name == "gelu_tanh":  # utils.py:33-38
        # jac = 0.5 x (1 - t^2)(0.79788456 + 0.1070322243 x^2) + 0.5 (1 + t),  t = tanh(0.79788456 x (1 + 0.044715 x^2))
        xx = x * x
        t = (xx * 0.044715).add_(1.0).mul_(x).mul_(0.79788456).tanh_()
        poly = xx.mul_(0.1070322243).add_(0.79788456)
        jac = (t * t).neg_().add_(1.0).mul_(poly).mul_(x).mul_(0.5)
        return jac.add_(t.add_(1.0).mul_(0.5))
    if name == "gelu_erf":
        return 0.5 * (1.0 + torch.erf(x / math.sqrt(2.0))) + x * torch.exp(-0.5 * x * x) / math.sqrt(2.0 * math.pi)
    if name == "relu":
        return (x > 0).to(x.dtype)
    if name == "silu":
        s = torch.sigmoid(x)
        return s * (1 + x * (1 - s))
    if name == "tanh":
        return 1 - torch.tanh(x) ** 2
    if name == "sigmoid":
        s = torch.sigmoid(x)
        return s * (1 - s)
    if name == "identity":
        return torch.ones_like(x)
    raise ValueError(name)


def apply_activation(pre: torch.Tensor, name: str, gated: bool) -> torch.Tensor:
    """_LeanFFN._apply_activation, lean_transformer/ffn.py:138-144: the FIRST half of the last dim is the gate."""
    if not gated:
        return act_forward(name, pre)
    gate, lin = (t.contiguous() for t in pre.split(pre.shape[-1] // 2, dim=-1))  # contiguous halves vectorise
    return act_forward(name, gate).mul_(lin)


def apply_activation_backward(dhid: torch.Tensor, pre: torch.Tensor, name: str, gated: bool) -> torch.Tensor:
    """Gradient of apply_activation w.r.t. pre (what autograd.grad computes at lean_transformer/ffn.py:275)."""
    if not gated:
        return dhid * act_grad(name, pre)
    gate, lin = (t.contiguous() for t in pre.split(pre.shape[-1] // 2, dim=-1))
    out = torch.empty_like(pre)
    half = pre.shape[-1] // 2
    out[..., :half] = act_grad(name, gate).mul_(lin).mul_(dhid)
    out[..., half:] = act_forward(name, gate).mul_(dhid)
    return out


# ---------------------------------------------------------------------------------------------------
# LayerNorm: F.layer_norm at lean_transformer/ffn.py:184 / :200 / :283 and its autograd at :290-293
# ---------------------------------------------------------------------------------------------------
def layer_norm_forward(x, gamma, beta, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)  # biased variance
    y = (x - mean) / torch.sqrt(var + eps)
    if gamma is not None:
        y = y * gamma
    if beta is not None:
        y = y + beta
    return y


def layer_norm_backward(dy, x, gamma, eps):
    """Returns (dx, dgamma, dbeta)."""
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    rstd = 1.0 / torch.sqrt(var + eps)
    xn = (x - mean) * rstd
    g = dy * gamma if gamma is not None else dy
    dx = rstd * (g - g.mean(-1, keepdim=True) - xn * (g * xn).mean(-1, keepdim=True))
    flat_dy, flat_xn = dy.reshape(-1, dy.shape[-1]), xn.reshape(-1, xn.shape[-1])
    return dx, (flat_dy * flat_xn).sum(0), flat_dy.sum(0)


# ---------------------------------------------------------------------------------------------------
# block-sparse matmul: lean_transformer/blocksparse/native_backend.py:9-76
# ---------------------------------------------------------------------------------------------------
def blocksparse_to_dense(weight: torch.Tensor, backward_indices: torch.Tensor, out_features: int) -> torch.Tensor:
    """Dense [out_features, in_features] matrix equal to the native block-sparse weight
    [in_features, blocks_per_input, block]: viewed as [in_blocks, blocks_per_input, block(out), block(in)],
    block (j, a) sits at output block backward_indices[j, a], input block j (native_backend.py:22-30)."""
    in_features, per_input, block = weight.shape
    in_blocks = in_features // block
    blocks = weight.reshape(in_blocks, per_input, block, block)
    dense = torch.zeros(out_features, in_features, dtype=weight.dtype)
    for j in range(in_blocks):
        for a in range(per_input):
            o = int(backward_indices[j, a])
            dense[o * block:(o + 1) * block, j * block:(j + 1) * block] += blocks[j, a]
    return dense


def blocksparse_matmul(x: torch.Tensor, weight: torch.Tensor, forward_indices: torch.Tensor) -> torch.Tensor:
    """native_backend.py:9-35 restated block by block: output block i sums, over its listed flat ids
    f = j * blocks_per_input + a, input block j times block f transposed."""
    in_features, per_input, block = weight.shape
    out_blocks = forward_indices.shape[0]
    blocks = weight.reshape(-1, block, block)
    flat = x.reshape(-1, in_features)
    out = torch.zeros(flat.shape[0], out_blocks * block, dtype=x.dtype)
    for i in range(out_blocks):
        for f in forward_indices[i].tolist():
            j = f // per_input
            out[:, i * block:(i + 1) * block] += flat[:, j * block:(j + 1) * block] @ blocks[f].t()
    return out.reshape(*x.shape[:-1], out_blocks * block)


def blocksparse_matmul_backward(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                                backward_indices: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """native_backend.py:38-76 restated block by block: (grad_input, grad_weight)."""
    in_features, per_input, block = weight.shape
    in_blocks = in_features // block
    blocks = weight.reshape(in_blocks, per_input, block, block)
    flat_dy, flat_x = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, in_features)
    dx = torch.zeros_like(flat_x)
    dw = torch.zeros_like(blocks)
    for j in range(in_blocks):
        xj = flat_x[:, j * block:(j + 1) * block]
        for a in range(per_input):
            o = int(backward_indices[j, a])
            dyo = flat_dy[:, o * block:(o + 1) * block]
            dx[:, j * block:(j + 1) * block] += dyo @ blocks[j, a]
            dw[j, a] = dyo.t() @ xj
    return dx.reshape(x.shape), dw.reshape(weight.shape)


# ---------------------------------------------------------------------------------------------------
# generalized linear: lean_transformer/blocksparse/linear.py:195-230 (forward), :260-328 (backward)
# ---------------------------------------------------------------------------------------------------
def linear_forward(x, weight, bias=None, lowrank_first=None, lowrank_second=None, forward_indices=None):
    """Returns (output, lowrank_hid)."""
    flat = x.reshape(-1, x.shape[-1])
    if forward_indices is not None:
        out = blocksparse_matmul(flat, weight, forward_indices)  # linear.py:212-216
    else:
        out = flat @ weight.t()  # linear.py:219
    if bias is not None:
        out = out + bias
    lowrank_hid = None
    if lowrank_first is not None and lowrank_second is not None:  # linear.py:221-226
        lowrank_hid = flat @ lowrank_first.t()
        out = out + lowrank_hid @ lowrank_second.t()
    return out.reshape(*x.shape[:-1], out.shape[-1]), lowrank_hid


def linear_backward(dy, x, lowrank_hid, weight, lowrank_first=None, lowrank_second=None, backward_indices=None):
    """Returns dict(input, weight, bias, lowrank_first, lowrank_second) (linear.py:260-328)."""
    flat_dy, flat_x = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
    grads: Dict[str, Optional[torch.Tensor]] = dict(lowrank_first=None, lowrank_second=None)
    grads["bias"] = flat_dy.sum(0)  # :293-294
    if backward_indices is None:
        grads["weight"] = flat_dy.t() @ flat_x  # :304-305
        dx = flat_dy @ weight  # :307-308
    else:
        dx, grads["weight"] = blocksparse_matmul_backward(flat_dy, flat_x, weight, backward_indices)  # :311-314
    if lowrank_first is not None and lowrank_second is not None:
        d_hid = flat_dy @ lowrank_second  # :281-282
        grads["lowrank_second"] = flat_dy.t() @ lowrank_hid  # :286-288
        grads["lowrank_first"] = d_hid.t() @ flat_x  # :289-292
        dx = dx + d_hid @ lowrank_first  # :317-325
    grads["input"] = dx.reshape(x.shape)
    return grads


# ---------------------------------------------------------------------------------------------------
# dropout mask: the CUDA kernels' counter-based definition (the reference delegates to torch.dropout,
# lean_transformer/ffn.py:204 / :245, whose mask is not reproducible by contract)
# ---------------------------------------------------------------------------------------------------
_PHILOX_M0, _PHILOX_M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85
_MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(group: np.ndarray, seed: int) -> np.ndarray:
    """Philox4x32-10 (Salmon et al., SC'11) with counter (group lo, group hi, 0, 0) and key
    (seed lo, seed hi).  ``group``: uint64 array [n]; returns uint32 array [n, 4]."""
    group = group.astype(np.uint64)
    c0, c1 = group & _MASK32, group >> np.uint64(32)
    c2, c3 = np.zeros_like(c0), np.zeros_like(c0)
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = _PHILOX_M0 * c0, _PHILOX_M1 * c2  # 32x32 -> 64 bit products
        hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK32
        hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK32
        c0, c1, c2, c3 = hi1 ^ c1 ^ np.uint64(k0), lo1, hi0 ^ c3 ^ np.uint64(k1), lo0
        k0, k1 = (k0 + _PHILOX_W0) & 0xFFFFFFFF, (k1 + _PHILOX_W1) & 0xFFFFFFFF
    return np.stack([c0, c1, c2, c3], axis=-1).astype(np.uint32)


def dropout_threshold(p: float) -> int:
    return min(int(np.float64(np.float32(p)) * 4294967296.0), 0xFFFFFFFF)


def dropout_keep_mask(numel: int, p: float, seed: int, elem_offset: int = 0) -> np.ndarray:
    """keep[i] for element index e = elem_offset + i: word (e & 3) of philox(e >> 2) >= floor(p * 2^32)."""
    if numel == 0:
        return np.zeros(0, dtype=bool)
    first, last = elem_offset >> 2, (elem_offset + numel - 1) >> 2
    groups = np.arange(first, last + 1, dtype=np.uint64)
    words = philox4x32_10(groups, seed).reshape(-1)  # element e sits at index e - 4 * first
    start = elem_offset - 4 * first
    return words[start:start + numel] >= np.uint32(dropout_threshold(p))


# ---------------------------------------------------------------------------------------------------
# LeanFFN: lean_transformer/ffn.py:146-217 (forward) and :233-306 (backward)
# ---------------------------------------------------------------------------------------------------
def leanffn_forward(x, params: Dict[str, Optional[torch.Tensor]], *, activation="gelu_tanh", gated=False, eps=1e-12,
                    residual=True, dropout_p=0.0, keep_mask: Optional[torch.Tensor] = None):
    """``params`` keys: ln_weight, ln_bias, i2h_weight, i2h_bias, i2h_lowrank_first, i2h_lowrank_second,
    i2h_forward_indices, i2h_backward_indices, h2o_* (same), post_ln_weight, post_ln_bias (missing = None).
    Returns (out, saved) where ``saved`` carries what backward needs."""
    P = lambda k: params.get(k)  # noqa: E731
    x2d = x.reshape(-1, x.shape[-1])
    x_ln = layer_norm_forward(x2d, P("ln_weight"), P("ln_bias"), eps)  # ffn.py:184
    pre, i2h_hid = linear_forward(x_ln, P("i2h_weight"), P("i2h_bias"), P("i2h_lowrank_first"),
                                  P("i2h_lowrank_second"), P("i2h_forward_indices"))  # :186-189
    hid = apply_activation(pre, activation, gated)  # :191
    out, h2o_hid = linear_forward(hid, P("h2o_weight"), P("h2o_bias"), P("h2o_lowrank_first"),
                                  P("h2o_lowrank_second"), P("h2o_forward_indices"))  # :193-196
    post_ln_input = None
    if P("post_ln_weight") is not None:  # :198-200
        post_ln_input = out
        out = layer_norm_forward(out, P("post_ln_weight"), P("post_ln_bias"), eps)
    if dropout_p and keep_mask is not None:  # :202-204
        out = out * keep_mask.reshape(out.shape).to(out.dtype) / (1.0 - dropout_p)
    if residual:  # :206-207
        out = out + x2d
    saved = dict(pre=pre, i2h_lowrank_hid=i2h_hid, h2o_lowrank_hid=h2o_hid, post_ln_input=post_ln_input)
    return out.reshape(x.shape), saved


def leanffn_backward(dout, x, params, saved, *, activation="gelu_tanh", gated=False, eps=1e-12, residual=True,
                     dropout_p=0.0, keep_mask: Optional[torch.Tensor] = None) -> Dict[str, Optional[torch.Tensor]]:
    """Gradients for input and every parameter, following the order of lean_transformer/ffn.py:233-306."""
    P = lambda k: params.get(k)  # noqa: E731
    grads: Dict[str, Optional[torch.Tensor]] = {}
    x2d = x.reshape(-1, x.shape[-1])
    dy = dout.reshape(-1, dout.shape[-1])
    d_residual = dy if residual else None  # :242
    if dropout_p and keep_mask is not None:  # :243-245 (same mask as forward)
        dy = dy * keep_mask.reshape(dy.shape).to(dy.dtype) / (1.0 - dropout_p)
    if P("post_ln_weight") is not None:  # :247-259
        dy, grads["post_ln_weight"], grads["post_ln_bias"] = layer_norm_backward(
            dy, saved["post_ln_input"], P("post_ln_weight"), eps)
    hid = apply_activation(saved["pre"], activation, gated)  # :265-268 (rematerialised)
    g = linear_backward(dy, hid, saved["h2o_lowrank_hid"], P("h2o_weight"), P("h2o_lowrank_first"),
                        P("h2o_lowrank_second"), P("h2o_backward_indices"))  # :270-273
    for k in ("weight", "bias", "lowrank_first", "lowrank_second"):
        grads["h2o_" + k] = g[k]
    d_pre = apply_activation_backward(g["input"], saved["pre"], activation, gated)  # :275
    x_ln = layer_norm_forward(x2d, P("ln_weight"), P("ln_bias"), eps)  # :280-283 (rematerialised)
    g = linear_backward(d_pre, x_ln, saved["i2h_lowrank_hid"], P("i2h_weight"), P("i2h_lowrank_first"),
                        P("i2h_lowrank_second"), P("i2h_backward_indices"))  # :285-288
    for k in ("weight", "bias", "lowrank_first", "lowrank_second"):
        grads["i2h_" + k] = g[k]
    dx, grads["ln_weight"], grads["ln_bias"] = layer_norm_backward(g["input"], x2d, P("ln_weight"), eps)  # :290-293
    if residual:  # :297-300
        dx = dx + d_residual
    grads["input"] = dx.reshape(x.shape)
    return grads


def leanffn_step(x, g, params, **kw):
    """One forward + backward with loss sum(out * g): returns (out, grads)."""
    out, saved = leanffn_forward(x, params, **kw)
    return out, leanffn_backward(g, x, params, saved, **kw)


# ---------------------------------------------------------------------------------------------------
# attention core: lean_transformer/attn.py:85-171, rotary tables and rotation: lean_transformer/rotary.py:43-68
# ---------------------------------------------------------------------------------------------------
def rotary_tables(length: int, dim: int, base: int = 10_000, dtype=torch.float64) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos / sin [length, dim] (rotary.py:48-60: the exponents and the position products are computed in float32)."""
    buf = torch.linspace(0, -1 + 2 / dim, dim // 2, dtype=torch.float32)
    inv_freq = torch.pow(base, buf).repeat(2)
    freqs = torch.arange(length, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(freqs).to(dtype), torch.sin(freqs).to(dtype)


def rotary_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [batch, len, heads, dim] -> x * cos + cat(-x_right, x_left) * sin (rotary.py:63-68)."""
    half = x.shape[-1] // 2
    rotated = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos[None, : x.shape[1], None, :] + rotated * sin[None, : x.shape[1], None, :]


def rotary_apply_transposed(g: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Gradient of rotary_apply with respect to x for an incoming gradient g."""
    half = g.shape[-1] // 2
    gs = g * sin[None, : g.shape[1], None, :]
    return g * cos[None, : g.shape[1], None, :] + torch.cat([gs[..., half:], -gs[..., :half]], dim=-1)


def attention_core_step(query, key, value, mask, heads: int, grad_out=None, rotary: bool = False, base: int = 10_000,
                        dropout_p: float = 0.0, keep_mask: Optional[torch.Tensor] = None):
    """Forward of the attention core and, given grad_out, the gradients for query / key / value, without autograd.
    query [batch, q_len, hidden], key / value [batch, kv_len, hidden], mask additive, broadcastable to
    [batch, heads, q_len, kv_len].  Follows attn.py:117-147: head split, keys divided by sqrt(head size), scores + mask,
    softmax over keys, probabilities times values, heads merged; with rotary=True queries and keys are rotated first
    (attn.py:163-171); with dropout_p > 0 the probabilities are multiplied by keep_mask / (1 - dropout_p) (attn.py:141-144,
    keep_mask [batch, heads, q_len, kv_len]).  Returns (out, dict(query=, key=, value=) or None)."""
    batch, q_len, hidden = query.shape
    kv_len, d = key.shape[1], hidden // heads
    q4, k4, v4 = (t.reshape(batch, -1, heads, d) for t in (query, key, value))
    if rotary:
        cos, sin = rotary_tables(max(q_len, kv_len), d, base, query.dtype)
        q4, k4 = rotary_apply(q4, cos, sin), rotary_apply(k4, cos, sin)
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q4, k4, v4))  # [batch, heads, len, d]
    inv = 1.0 / math.sqrt(d)
    scores = qh @ (kh * inv).transpose(-1, -2)
    if mask is not None:
        scores = scores + mask
    probs = torch.softmax(scores, dim=-1)
    drop = None
    if dropout_p and keep_mask is not None:
        drop = keep_mask.reshape(probs.shape).to(probs.dtype) / (1.0 - dropout_p)
    kept = probs if drop is None else probs * drop
    out = (kept @ vh).transpose(1, 2).reshape(batch, q_len, hidden)
    if grad_out is None:
        return out, None
    go = grad_out.reshape(batch, q_len, heads, d).permute(0, 2, 1, 3)
    d_v = kept.transpose(-1, -2) @ go
    d_probs = go @ vh.transpose(-1, -2)
    if drop is not None:
        d_probs = d_probs * drop
    d_scores = probs * (d_probs - (d_probs * probs).sum(-1, keepdim=True))
    d_q = (d_scores @ kh) * inv
    d_k = (d_scores.transpose(-1, -2) @ qh) * inv
    d_q4, d_k4, d_v4 = (t.permute(0, 2, 1, 3) for t in (d_q, d_k, d_v))
    if rotary:
        d_q4, d_k4 = rotary_apply_transposed(d_q4, cos, sin), rotary_apply_transposed(d_k4, cos, sin)
    grads = dict(query=d_q4.reshape(batch, q_len, hidden), key=d_k4.reshape(batch, kv_len, hidden),
                 value=d_v4.reshape(batch, kv_len, hidden))
    return out, grads
