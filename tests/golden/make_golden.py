"""Generates the golden vectors in this folder by running the REFERENCE implementation
(learning-at-home/lean_transformer) on the CPU in float64.

Usage (only where the reference source tree is available; the GPU box never runs this):

    python tests/golden/make_golden.py /path/to/reference

The reference imports ``revlib`` (not installed here) for a module outside the LeanFFN path; a two-class
stand-in is registered before the import.  The dropout case injects the mask defined by the oracle's Philox
function into the reference by replacing ``torch.dropout_`` / ``torch.dropout`` for the duration of the call,
because the reference's own mask comes from torch's RNG and is not reproducible by contract.
"""
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch
import torch.nn as nn

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))


def import_reference(ref_root: str):
    stub = types.ModuleType("revlib")

    class ReversibleModule(nn.Module):
        pass

    class ReversibleSequential(nn.Sequential):
        pass

    stub.ReversibleModule, stub.ReversibleSequential = ReversibleModule, ReversibleSequential
    sys.modules.setdefault("revlib", stub)
    sys.path.insert(0, ref_root)
    import lean_transformer  # noqa: F401
    from lean_transformer import ffn as ref_ffn
    from lean_transformer.blocksparse import layout as ref_layout
    from lean_transformer.blocksparse import linear as ref_linear
    from lean_transformer.blocksparse import native_backend as ref_native
    from lean_transformer import utils as ref_utils
    return ref_ffn, ref_linear, ref_native, ref_layout, ref_utils


def to_np(t):
    return None if t is None else t.detach().cpu().numpy()


def ffn_params(ffn) -> dict:
    """Reference module -> the oracle's flat parameter dictionary."""
    out = dict(ln_weight=ffn.pre_layer_norm.weight, ln_bias=ffn.pre_layer_norm.bias)
    if ffn.post_layer_norm is not None:
        out.update(post_ln_weight=ffn.post_layer_norm.weight, post_ln_bias=ffn.post_layer_norm.bias)
    for name, proj in (("i2h", ffn.i2h_proj), ("h2o", ffn.h2o_proj)):
        out[f"{name}_weight"], out[f"{name}_bias"] = proj.weight, proj.bias
        if hasattr(proj, "get_combined_lowrank_components"):
            first, second = proj.get_combined_lowrank_components()
            out[f"{name}_lowrank_first"], out[f"{name}_lowrank_second"] = first, second
            out[f"{name}_forward_indices"] = proj.matrix.forward_indices
            out[f"{name}_backward_indices"] = proj.matrix.backward_indices
    return {k: v for k, v in out.items() if v is not None}


def combined_lowrank_grads(proj, grad_of):
    """Gradients w.r.t. the concatenated (shared low-rank, adapter) pair, assembled from the leaf gradients."""
    firsts = [t for t in (proj.matrix.lowrank_first, proj.adapter_first) if t is not None]
    seconds = [t for t in (proj.matrix.lowrank_second, proj.adapter_second) if t is not None]
    if not firsts:
        return None, None
    return torch.cat([grad_of[id(t)] for t in firsts], dim=0), torch.cat([grad_of[id(t)] for t in seconds], dim=1)


def run_ffn_case(name, ffn, x, g, extra=None):
    """Forward + backward of a reference LeanFFN with loss sum(out * g); stores inputs, params, out, grads."""
    ffn = ffn.double()
    x = x.double().requires_grad_(True)
    leaves = list(ffn.parameters())
    out = ffn(x)
    grads = torch.autograd.grad((out * g.double()).sum(), [x] + leaves)
    grad_of = {id(p): gv for p, gv in zip(leaves, grads[1:])}
    blob = {"x": to_np(x), "g": to_np(g.double()), "out": to_np(out), "grad_input": to_np(grads[0])}
    for k, v in ffn_params(ffn).items():
        blob["param_" + k] = to_np(v)
    blob["grad_ln_weight"] = to_np(grad_of[id(ffn.pre_layer_norm.weight)])
    blob["grad_ln_bias"] = to_np(grad_of[id(ffn.pre_layer_norm.bias)])
    if ffn.post_layer_norm is not None:
        blob["grad_post_ln_weight"] = to_np(grad_of[id(ffn.post_layer_norm.weight)])
        blob["grad_post_ln_bias"] = to_np(grad_of[id(ffn.post_layer_norm.bias)])
    for prefix, proj in (("i2h", ffn.i2h_proj), ("h2o", ffn.h2o_proj)):
        blob[f"grad_{prefix}_weight"] = to_np(grad_of[id(proj.weight)])
        blob[f"grad_{prefix}_bias"] = to_np(grad_of[id(proj.bias)])
        if hasattr(proj, "matrix"):
            first, second = combined_lowrank_grads(proj, grad_of)
            if first is not None:
                blob[f"grad_{prefix}_lowrank_first"], blob[f"grad_{prefix}_lowrank_second"] = to_np(first), to_np(second)
    if extra:
        blob.update(extra)
    np.savez_compressed(HERE / f"{name}.npz", **blob)
    print(f"wrote {name}.npz ({len(blob)} arrays)")


def main(ref_root: str):
    ref_ffn, ref_linear, ref_native, ref_layout, ref_utils = import_reference(ref_root)
    from oracle.leanffn_oracle import dropout_keep_mask

    LeanFFN = ref_ffn.LeanFFN
    GL, GM = ref_linear.GeneralizedLinear, ref_linear.GeneralizedMatrix

    def randomize(module, seed):
        gen = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for p in module.parameters():
                p.copy_(torch.randn(p.shape, generator=gen) * (0.3 if p.ndim > 1 else 0.5) + (1.0 if p.ndim == 1 else 0))

    torch.manual_seed(0)
    H, I = 32, 64
    x = torch.randn(2, 12, H)
    g = torch.randn(2, 12, H)

    ffn = LeanFFN(H, I)
    randomize(ffn, 1)
    run_ffn_case("ffn_dense_plain", ffn, x, g, dict(meta_gated=0, meta_residual=1))

    ffn = LeanFFN(H, I, gated=True, post_layer_norm=True, residual=False)
    randomize(ffn, 2)
    run_ffn_case("ffn_gated_postln", ffn, x, g, dict(meta_gated=1, meta_residual=0))

    layout = "pixelfly(16)"
    ffn = LeanFFN(H, I, gated=True, post_layer_norm=True,
                  i2h_proj=GL(GM(H, 2 * I, layout, 6), 2), h2o_proj=GL(GM(I, H, layout, 6), 2), residual=True)
    randomize(ffn, 3)
    run_ffn_case("ffn_pixelfly_lowrank", ffn, x, g, dict(meta_gated=1, meta_residual=1))

    # dropout with an injected mask
    p, seed, offset = 0.5, 1234, 64
    keep = torch.from_numpy(dropout_keep_mask(x.numel(), p, seed, offset)).view(-1, H)
    ffn = LeanFFN(H, I, gated=True, dropout=p)
    randomize(ffn, 4)
    ffn.train()
    orig_inplace, orig = torch.dropout_, torch.dropout
    torch.dropout_ = lambda t, prob, train: t.mul_(keep.to(t.dtype) / (1 - prob))
    torch.dropout = lambda t, prob, train: t * (keep.to(t.dtype) / (1 - prob))
    try:
        run_ffn_case("ffn_dropout_mask", ffn, x, g,
                     dict(meta_gated=1, meta_residual=1, meta_dropout=p, meta_seed=seed, meta_offset=offset,
                          keep_mask=keep.numpy()))
    finally:
        torch.dropout_, torch.dropout = orig_inplace, orig

    # generalized linear: block-sparse + shared low rank + adapter
    torch.manual_seed(5)
    lin = GL(GM(64, 64, "pixelfly(block_size=8)", 12), 4).double()
    randomize(lin, 5)
    xl = torch.randn(3, 5, 64, dtype=torch.float64, requires_grad=True)
    gl = torch.randn(3, 5, 64, dtype=torch.float64)
    out = lin(xl)
    leaves = list(lin.parameters())
    leaf_grads = torch.autograd.grad((out * gl).sum(), [xl] + leaves)
    grad_of = {id(p): gv for p, gv in zip(leaves, leaf_grads[1:])}
    first, second = lin.get_combined_lowrank_components()
    grads = (leaf_grads[0], grad_of[id(lin.matrix.weight)], grad_of[id(lin.bias)], *combined_lowrank_grads(lin, grad_of))
    np.savez_compressed(
        HERE / "linear_pixelfly_lowrank.npz", x=to_np(xl), g=to_np(gl), out=to_np(out), weight=to_np(lin.matrix.weight),
        bias=to_np(lin.bias), lowrank_first=to_np(first), lowrank_second=to_np(second),
        forward_indices=to_np(lin.matrix.forward_indices), backward_indices=to_np(lin.matrix.backward_indices),
        grad_input=to_np(grads[0]), grad_weight=to_np(grads[1]), grad_bias=to_np(grads[2]),
        grad_lowrank_first=to_np(grads[3]), grad_lowrank_second=to_np(grads[4]))
    print("wrote linear_pixelfly_lowrank.npz")

    # raw block-sparse matmul, rectangular, non power-of-two block
    torch.manual_seed(6)
    out_f, in_f, bs = 192, 48, 12
    lay = ref_layout.get_blocksparse_layout(out_f, in_f, f"pixelfly(block_size={bs})")
    fi, bi = ref_layout.get_indices_from_layout(lay)
    w = torch.randn(in_f, fi.numel() // (in_f // bs), bs, dtype=torch.float64, requires_grad=True)
    xb = torch.randn(2, 7, in_f, dtype=torch.float64, requires_grad=True)
    gb = torch.randn(2, 7, out_f, dtype=torch.float64)
    ob = ref_native.blocksparse_matmul(xb, w, fi)
    gx, gw = ref_native.blocksparse_matmul_backward(gb, xb, w, bi)
    np.savez_compressed(HERE / "blocksparse_matmul.npz", x=to_np(xb), g=to_np(gb), weight=to_np(w), layout=to_np(lay),
                        forward_indices=to_np(fi), backward_indices=to_np(bi), out=to_np(ob), grad_input=to_np(gx),
                        grad_weight=to_np(gw))
    print("wrote blocksparse_matmul.npz")

    # layouts and index tensors
    blob = {}
    specs = [
        (512, 128, "pixelfly(block_size=16)"), (128, 512, "pixelfly(block_size=16)"),
        (256, 256, "pixelfly(block_size=32)"), (1024, 256, "pixelfly(block_size=32, stretch=True)"),
        (512, 512, "pixelfly(16, 8, 2)"), (4096, 1024, "pixelfly(block_size=128)"), (32768, 4096, "pixelfly(block_size=128)"),
        (4096, 16384, "pixelfly(block_size=128)"),
        (512, 128, "hypercube(16)"), (128, 512, "hypercube(16, folded=True)"),
        (256, 256, "hypercube(32, stretch=True, folded=True)"),
    ]
    for n, (o, i, desc) in enumerate(specs):
        lay = ref_layout.get_blocksparse_layout(o, i, desc)
        blob[f"layout_{n}"] = to_np(lay)
        try:
            fi, bi = ref_layout.get_indices_from_layout(lay)
            blob[f"forward_{n}"], blob[f"backward_{n}"] = to_np(fi), to_np(bi)
        except AssertionError:
            pass
    blob["specs"] = np.array([f"{o}|{i}|{d}" for o, i, d in specs])
    np.savez_compressed(HERE / "layouts.npz", **blob)
    print("wrote layouts.npz")

    # activation
    xs = torch.linspace(-6, 6, 241, dtype=torch.float64)
    np.savez_compressed(HERE / "gelu_fused.npz", x=to_np(xs), y=to_np(ref_utils.gelu_fused(xs)),
                        dy=to_np(ref_utils.gelu_fused_grad(torch.ones_like(xs), xs)))
    print("wrote gelu_fused.npz")

    # attention cores (lean_transformer/attn.py:85-171): outputs and input gradients in float64
    from lean_transformer import attn as ref_attn
    torch.manual_seed(11)
    B, S, HID, HEADS = 2, 40, 96, 3
    for kind, cls in (("simple", ref_attn.SimpleAttentionCore), ("rotary", ref_attn.RotaryAttentionCore)):
        core = cls(HID, HEADS).double()
        q, k, v = (torch.randn(B, S, HID, dtype=torch.float64, requires_grad=True) for _ in range(3))
        g = torch.randn(B, S, HID, dtype=torch.float64)
        causal = (1.0 - torch.ones(S, S, dtype=torch.float64).tril()).view(1, 1, S, S) * -10000.0
        padding = torch.zeros(B, 1, 1, S, dtype=torch.float64)
        padding[1, :, :, S - 7:] = -10000.0
        mask = causal + padding
        out, probs = core(q, k, v, mask)
        out.backward(g)
        np.savez_compressed(HERE / f"attention_core_{kind}.npz", query=to_np(q), key=to_np(k), value=to_np(v),
                            mask=to_np(mask), grad_out=to_np(g), out=to_np(out), probs=to_np(probs),
                            grad_query=to_np(q.grad), grad_key=to_np(k.grad), grad_value=to_np(v.grad),
                            heads=np.array(HEADS))
        print(f"wrote attention_core_{kind}.npz")

    # attention core with dropout on the probabilities: the oracle's Philox mask injected into the reference
    torch.manual_seed(12)
    p_attn, seed_attn, offset_attn = 0.25, 77, 4096
    keep_attn = torch.from_numpy(dropout_keep_mask(B * HEADS * S * S, p_attn, seed_attn, offset_attn)).view(B, HEADS, S, S)
    core = ref_attn.SimpleAttentionCore(HID, HEADS, attention_probs_dropout=p_attn).double().train()
    q, k, v = (torch.randn(B, S, HID, dtype=torch.float64, requires_grad=True) for _ in range(3))
    g = torch.randn(B, S, HID, dtype=torch.float64)
    orig_inplace = torch.dropout_
    # out of place: softmax's backward needs its own output unchanged (same values and gradients as the in-place form)
    torch.dropout_ = lambda t, prob, train: t * (keep_attn.to(t.dtype) / (1 - prob))
    try:
        out, probs = core(q, k, v, causal)
        out.backward(g)
    finally:
        torch.dropout_ = orig_inplace
    np.savez_compressed(HERE / "attention_core_dropout.npz", query=to_np(q), key=to_np(k), value=to_np(v),
                        mask=to_np(causal), grad_out=to_np(g), out=to_np(out), grad_query=to_np(q.grad),
                        grad_key=to_np(k.grad), grad_value=to_np(v.grad), heads=np.array(HEADS),
                        dropout=np.array(p_attn), seed=np.array(seed_attn), offset=np.array(offset_attn))
    print("wrote attention_core_dropout.npz")

    # state-dict key names the drop-in modules must reproduce
    ffn = LeanFFN(H, I, gated=True, post_layer_norm=True,
                  i2h_proj=GL(GM(H, 2 * I, layout, 6), 2), h2o_proj=GL(GM(I, H, layout, 0, ), 0))
    with open(HERE / "state_dict_keys.txt", "w") as f:
        f.write("\n".join(f"{k} {tuple(v.shape)} {v.dtype}" for k, v in ffn.state_dict().items()) + "\n")
    print("wrote state_dict_keys.txt")


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LEAN_REFERENCE_ROOT")
    if not root:
        sys.exit("usage: make_golden.py <checkout of learning-at-home/lean_transformer>  (or set LEAN_REFERENCE_ROOT)")
    main(root)
