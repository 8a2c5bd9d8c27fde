"""Shared helpers of the GPU parity tests: build a LeanFFN from the oracle's flat parameter dictionary,
run one forward + backward through the public module API, and name the gradients like the oracle does."""
from typing import Dict, Optional

import torch
import torch.nn as nn

import lean_transformer_b200 as L
from lean_transformer_b200.blocksparse.linear import GeneralizedLinear, GeneralizedMatrix


def _projection(prefix: str, params: Dict[str, torch.Tensor], in_features: int, out_features: int):
    weight = params[f"{prefix}_weight"]
    first = params.get(f"{prefix}_lowrank_first")
    if weight.ndim == 2 and first is None:
        proj = nn.Linear(in_features, out_features)
    else:
        layout = None
        if weight.ndim == 3:
            layout = f"pixelfly(block_size={weight.shape[-1]})"
        proj = GeneralizedLinear(GeneralizedMatrix(in_features, out_features, layout,
                                                   0 if first is None else first.shape[0]))
        if weight.ndim == 3:
            assert torch.equal(proj.matrix.forward_indices.cpu(), params[f"{prefix}_forward_indices"].cpu().int())
    return proj


def make_ffn(params: Dict[str, torch.Tensor], *, gated: bool, residual: bool = True, dropout: float = 0.0,
             activation="gelu_fused", eps: float = 1e-12, device="cuda", dtype=torch.float32,
             custom_grad: bool = True) -> L.LeanFFN:
    hidden = params["ln_weight"].shape[0]
    h2o_w = params["h2o_weight"]
    inter = h2o_w.shape[1] if h2o_w.ndim == 2 else h2o_w.shape[0]
    i2h_out = 2 * inter if gated else inter
    act = L.ACT2FN[activation] if isinstance(activation, str) else activation
    ffn = L.LeanFFN(hidden, inter, activation=act, gated=gated, layer_norm_eps=eps, dropout=dropout,
                    post_layer_norm="post_ln_weight" in params, i2h_proj=_projection("i2h", params, hidden, i2h_out),
                    h2o_proj=_projection("h2o", params, inter, hidden), residual=residual,
                    ffn_custom_grad=custom_grad)
    with torch.no_grad():
        ffn.pre_layer_norm.weight.copy_(params["ln_weight"])
        ffn.pre_layer_norm.bias.copy_(params["ln_bias"])
        if "post_ln_weight" in params:
            ffn.post_layer_norm.weight.copy_(params["post_ln_weight"])
            ffn.post_layer_norm.bias.copy_(params["post_ln_bias"])
        for prefix, proj in (("i2h", ffn.i2h_proj), ("h2o", ffn.h2o_proj)):
            proj.weight.copy_(params[f"{prefix}_weight"])
            proj.bias.copy_(params[f"{prefix}_bias"])
            if params.get(f"{prefix}_lowrank_first") is not None:
                proj.matrix.lowrank_first.copy_(params[f"{prefix}_lowrank_first"])
                proj.matrix.lowrank_second.copy_(params[f"{prefix}_lowrank_second"])
    return ffn.to(device=device, dtype=dtype)


def named_grads(ffn: L.LeanFFN) -> Dict[str, Optional[torch.Tensor]]:
    out = {"ln_weight": ffn.pre_layer_norm.weight.grad, "ln_bias": ffn.pre_layer_norm.bias.grad}
    if ffn.post_layer_norm is not None:
        out["post_ln_weight"], out["post_ln_bias"] = ffn.post_layer_norm.weight.grad, ffn.post_layer_norm.bias.grad
    for prefix, proj in (("i2h", ffn.i2h_proj), ("h2o", ffn.h2o_proj)):
        out[f"{prefix}_weight"], out[f"{prefix}_bias"] = proj.weight.grad, proj.bias.grad
        if isinstance(proj, GeneralizedLinear) and proj.matrix.lowrank_first is not None:
            out[f"{prefix}_lowrank_first"] = proj.matrix.lowrank_first.grad
            out[f"{prefix}_lowrank_second"] = proj.matrix.lowrank_second.grad
    return out


def run_step(ffn: L.LeanFFN, x: torch.Tensor, g: torch.Tensor, autocast: bool = False):
    """out, grads (oracle names, incl. 'input') of loss = sum(out * g)."""
    ffn.zero_grad(set_to_none=True)
    x = x.detach().clone().requires_grad_(True)
    if autocast:
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = ffn(x)
    else:
        out = ffn(x)
    (out.float() * g.float()).sum().backward()
    grads = named_grads(ffn)
    grads["input"] = x.grad
    L.check_device_status(x.device)
    return out.detach(), grads


def random_params(hidden: int, inter: int, gated: bool, *, seed: int = 0, std: float = 0.02, post_ln: bool = False,
                  bias_std: float = 0.0, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=gen, dtype=dtype)  # noqa: E731
    width = 2 * inter if gated else inter
    p = dict(ln_weight=1 + 0.1 * rn(hidden), ln_bias=0.1 * rn(hidden), i2h_weight=std * rn(width, hidden),
             i2h_bias=bias_std * rn(width), h2o_weight=std * rn(hidden, inter), h2o_bias=bias_std * rn(hidden))
    if post_ln:
        p.update(post_ln_weight=1 + 0.1 * rn(hidden), post_ln_bias=0.1 * rn(hidden))
    return p


# ---- noise-floor twin: the same step with stock PyTorch operators ---------------------------------------------------
def torch_twin_step(params: Dict[str, torch.Tensor], x: torch.Tensor, g: torch.Tensor, *, gated: bool,
                    residual: bool = True, dropout_p: float = 0.0, keep_mask: Optional[torch.Tensor] = None,
                    autocast: bool = True, eps: float = 1e-12, device="cuda"):
    """out, grads (oracle names) of loss = sum(out * g) computed by stock torch operators and autograd on the GPU,
    under ``torch.autocast(bfloat16)`` when ``autocast``: the arithmetic the reference's own mixed-precision run
    performs (cuBLAS bf16 products with fp32 accumulation, fp32 LayerNorm, every elementwise result rounded to bf16).
    TEST-ONLY code: its distance from the fp32 oracle is the noise floor of bf16 arithmetic for these shapes, which
    is what the kernels' distance is compared with.  Block-sparse weights are expanded to dense masked matrices."""
    import torch.nn.functional as F

    from lean_transformer_b200.blocksparse.convert import native_weight_to_dense

    leaves = {k: v.to(device).clone().requires_grad_(True) for k, v in params.items() if v.is_floating_point()}
    x = x.to(device).clone().requires_grad_(True)
    g = g.to(device)
    hidden = x.shape[-1]

    def project(prefix, inp, out_features):
        weight = leaves[f"{prefix}_weight"]
        if weight.ndim == 3:
            weight = native_weight_to_dense(weight, params[f"{prefix}_backward_indices"].to(device), out_features)
        out = F.linear(inp, weight, leaves.get(f"{prefix}_bias"))
        if f"{prefix}_lowrank_first" in leaves:
            out = out + F.linear(F.linear(inp, leaves[f"{prefix}_lowrank_first"]), leaves[f"{prefix}_lowrank_second"])
        return out

    def gelu_tanh(t):  # lean_transformer/utils.py:30, one rounding per elementwise operator under autocast
        return t * 0.5 * (1.0 + torch.tanh(0.79788456 * t * (1 + 0.044715 * t * t)))

    inter = leaves["h2o_weight"].shape[1] if leaves["h2o_weight"].ndim == 2 else leaves["h2o_weight"].shape[0]
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast):
        ln = F.layer_norm(x, (hidden,), leaves["ln_weight"], leaves["ln_bias"], eps)
        pre = project("i2h", ln, 2 * inter if gated else inter)
        if gated:
            gate, lin = pre.split(inter, dim=-1)
            hid = gelu_tanh(gate) * lin
        else:
            hid = gelu_tanh(pre)
        out = project("h2o", hid, hidden)
        if "post_ln_weight" in leaves:
            out = F.layer_norm(out, (hidden,), leaves["post_ln_weight"], leaves["post_ln_bias"], eps)
        if dropout_p:
            out = out * (keep_mask.to(device).to(out.dtype) / (1.0 - dropout_p))
        if residual:
            out = out + x
    (out.float() * g.float()).sum().backward()
    grads = {k: v.grad for k, v in leaves.items()}  # block-sparse weights: gradient in the leaf's own block format
    grads["input"] = x.grad
    return out.detach(), grads
