"""Attention-core kernels (leanffn_attention_forward / backward, leanffn_rotary) against the CPU oracle and the
golden vectors the reference produced (needs a B200).

Inputs are rounded to bfloat16 first and the oracle runs in float64 on exactly those values, so what is measured is
the kernels' own arithmetic: bf16 tensor-core products with fp32 accumulation, fp32 softmax, probabilities and score
gradients rounded to bf16 before the second products.  Tolerance: rtol 2e-2, atol 1e-2 (the bf16 bar), applied
literally to every element (torch.allclose's rule)."""
import math

import pytest
import torch

from conftest import BF16_ATOL, BF16_RTOL, assert_close, load_golden
from oracle import leanffn_oracle as O

pytestmark = pytest.mark.gpu


def _bf16(t):
    return t.to(torch.bfloat16)


def _check(got, want, what, scaled=False):
    # the literal rule |got - ref| <= atol + rtol * |ref| for every element, no outlier budget; ``scaled`` (dropout
    # cases, and gradients of sharply peaked rows): errors are checked at the rms size of the tensor, see test_attention_dropout_golden_and_oracle
    assert_close(got.float().cpu(), want.float(), BF16_RTOL, BF16_ATOL, what, scale_atol=scaled)


def _run_case(device, batch, heads, q_len, kv_len, head_dim, mask_kind, rotary, seed=0):
    import lean_transformer_b200 as L

    torch.manual_seed(seed)
    hidden = heads * head_dim
    if q_len == kv_len:  # the three slices of one fused projection output, read in place
        qkv = _bf16(torch.randn(batch, q_len, 3 * hidden)).to(device).requires_grad_(True)
        q, k, v = qkv.split(hidden, dim=-1)
    else:
        q = _bf16(torch.randn(batch, q_len, hidden)).to(device).requires_grad_(True)
        k = _bf16(torch.randn(batch, kv_len, hidden)).to(device).requires_grad_(True)
        v = _bf16(torch.randn(batch, kv_len, hidden)).to(device).requires_grad_(True)
    g = _bf16(torch.randn(batch, q_len, hidden)).to(device)
    mask = None
    if mask_kind == "causal":
        mask = (1.0 - torch.ones(q_len, kv_len).tril(kv_len - q_len)).view(1, 1, q_len, kv_len) * -10000.0
    elif mask_kind == "causal+padding":
        mask = (1.0 - torch.ones(q_len, kv_len).tril(kv_len - q_len)).view(1, 1, q_len, kv_len) * -10000.0
        pad = torch.zeros(batch, 1, 1, kv_len)
        pad[-1, :, :, kv_len - kv_len // 5:] = -10000.0
        mask = mask + pad
    elif mask_kind == "keys":
        mask = (torch.rand(batch, 1, 1, kv_len) < 0.3).float() * -10000.0
        mask[..., 0] = 0.0
    elif mask_kind == "per_head":
        mask = torch.randn(batch, heads, q_len, kv_len)
    core = (L.RotaryAttentionCore if rotary else L.SimpleAttentionCore)(hidden, heads).to(device).train()
    dmask = None if mask is None else mask.to(device)
    out, probs = core(q, k, v, dmask)
    assert probs is None and out.dtype == torch.bfloat16 and out.shape == (batch, q_len, hidden)
    out.backward(g)
    leaves = (qkv,) if q_len == kv_len else (q, k, v)
    got_grads = torch.cat([t.grad for t in leaves], dim=-1) if q_len == kv_len else None
    want, grads = O.attention_core_step(q.detach().double().cpu(), k.detach().double().cpu(), v.detach().double().cpu(),
                                        None if mask is None else mask.double(), heads, grad_out=g.double().cpu(),
                                        rotary=rotary)
    tag = f"attention b{batch} h{heads} q{q_len} kv{kv_len} d{head_dim} {mask_kind} rotary={rotary}"
    _check(out, want, f"{tag}:out")
    if q_len == kv_len:
        gq, gk, gv = got_grads.split(hidden, dim=-1)
    else:
        gq, gk, gv = q.grad, k.grad, v.grad
    _check(gq, grads["query"], f"{tag}:grad_query")
    _check(gk, grads["key"], f"{tag}:grad_key")
    _check(gv, grads["value"], f"{tag}:grad_value")
    L.check_device_status(device)
    return core


@pytest.mark.parametrize("kind", ["simple", "rotary"])
def test_attention_core_golden(cuda_device, kind):
    """The reference's own cores (float64 run, tests/golden/make_golden.py): causal + padding mask, 3 heads of 32."""
    import lean_transformer_b200 as L

    blob = {k: torch.from_numpy(v) for k, v in load_golden(f"attention_core_{kind}").items()}
    heads = int(blob["heads"])
    hidden = blob["query"].shape[-1]
    core = (L.RotaryAttentionCore if kind == "rotary" else L.SimpleAttentionCore)(hidden, heads).to(cuda_device)
    q, k, v = (_bf16(blob[n]).to(cuda_device).requires_grad_(True) for n in ("query", "key", "value"))
    out, _ = core(q, k, v, blob["mask"].float().to(cuda_device))
    out.backward(_bf16(blob["grad_out"]).to(cuda_device))
    # the golden run used the unrounded inputs: the input rounding (2^-9 relative per element) is part of the distance
    _check(out, blob["out"], f"attention golden {kind}:out")
    for n, t in (("query", q), ("key", k), ("value", v)):
        _check(t.grad, blob[f"grad_{n}"], f"attention golden {kind}:grad_{n}")


@pytest.mark.parametrize("batch,heads,q_len,kv_len,head_dim,mask_kind,rotary", [
    (1, 1, 128, 128, 64, None, False),
    (2, 3, 256, 256, 64, "causal", False),          # detected: mask never read, empty tiles skipped
    (2, 3, 256, 256, 48, "causal+padding", True),   # config 4's head size, general mask path
    (2, 2, 200, 200, 64, "per_head", False),        # ragged tiles, one mask per head
    (1, 2, 384, 384, 128, "keys", True),            # two 64-wide boxes per tile
    (1, 2, 100, 333, 32, "causal", False),          # cross lengths, offset causal rule
    (1, 2, 300, 300, 96, "causal", True),
    (2, 4, 77, 77, 16, None, True),                 # smallest head size, less than one tile
    (1, 1, 513, 513, 80, "causal+padding", False),
])
def test_attention_core_vs_oracle(cuda_device, batch, heads, q_len, kv_len, head_dim, mask_kind, rotary):
    _run_case(cuda_device, batch, heads, q_len, kv_len, head_dim, mask_kind, rotary)


def test_attention_core_config4_shape(cuda_device):
    """One batch row of config 4: 2048 tokens, 16 heads of 48, rotary, the causal mask the GPT model builds."""
    _run_case(cuda_device, 1, 16, 2048, 2048, 48, "causal", True, seed=4)


def test_attention_scores_growing_along_keys(cuda_device):
    """Scores that rise steadily with the key position: the forward kernel takes later key tiles against the reference
    maximum of earlier ones and has to notice when that stops being safe.  Head 0 rises by ~4 (base 2) per 128 keys:
    two tiles stay within the headroom, the third must rescale; head 1 by ~13: every tile must."""
    import lean_transformer_b200 as L

    torch.manual_seed(11)
    batch, heads, length, head_dim = 2, 2, 640, 48
    hidden = heads * head_dim
    direction = torch.nn.functional.normalize(torch.randn(heads, head_dim), dim=-1)
    slope = torch.tensor([0.34, 1.1]).view(1, 1, heads, 1)  # natural-log units per key before the 1/sqrt(d) scale
    pos = torch.arange(length).view(1, length, 1, 1) / 16.0
    q = (direction.view(1, 1, heads, head_dim) * 7.0 + 0.1 * torch.randn(batch, length, heads, head_dim))
    k = (direction.view(1, 1, heads, head_dim) * slope * pos + 0.1 * torch.randn(batch, length, heads, head_dim))
    v = torch.randn(batch, length, heads, head_dim)
    for mask_kind in ("none", "causal"):
        qkv = _bf16(torch.cat([t.reshape(batch, length, hidden) for t in (q, k, v)], dim=-1)).to(cuda_device)
        qkv.requires_grad_(True)
        g = _bf16(torch.randn(batch, length, hidden)).to(cuda_device)
        mask = None
        if mask_kind == "causal":
            mask = (1.0 - torch.ones(length, length).tril()).view(1, 1, length, length) * -10000.0
        core = L.SimpleAttentionCore(hidden, heads).to(cuda_device).train()
        qs, ks, vs = qkv.split(hidden, dim=-1)
        out, _ = core(qs, ks, vs, None if mask is None else mask.to(cuda_device))
        out.backward(g)
        want, grads = O.attention_core_step(qs.detach().double().cpu(), ks.detach().double().cpu(),
                                            vs.detach().double().cpu(), None if mask is None else mask.double(), heads,
                                            grad_out=g.double().cpu())
        _check(out, want, f"growing scores {mask_kind}:out")
        gq, gk, gv = qkv.grad.split(hidden, dim=-1)
        # dV = P^T dO re-creates P from the row statistics the forward pass wrote
        _check(gv, grads["value"], f"growing scores {mask_kind}:grad_value", scaled=True)
        # dQ and dK are not checked here: the keys are of size 40 along a direction in which the score gradients of a row
        # cancel, so that their bf16 rounding alone is ~10 % of the result; the other cases cover those products
        L.check_device_status(cuda_device)


def test_attention_edge_shapes(cuda_device):
    """One query against a long key sequence (a decoding step); more queries than keys under a finite causal mask
    (rows that see no key attend the shifted raw scores, as in the reference: the mask is read, not replaced by the
    in-kernel rule); a mask with -inf entries next to finite ones; a batch of three with one mask per batch row."""
    import lean_transformer_b200 as L
    from lean_transformer_b200.attn import mask_is_causal

    def one(batch, heads, q_len, kv_len, d, mask, tag):
        torch.manual_seed(13)
        q = _bf16(torch.randn(batch, q_len, heads * d)).to(cuda_device).requires_grad_(True)
        k = _bf16(torch.randn(batch, kv_len, heads * d)).to(cuda_device).requires_grad_(True)
        v = _bf16(torch.randn(batch, kv_len, heads * d)).to(cuda_device).requires_grad_(True)
        g = _bf16(torch.randn(batch, q_len, heads * d)).to(cuda_device)
        core = L.SimpleAttentionCore(heads * d, heads).to(cuda_device)
        out, _ = core(q, k, v, None if mask is None else mask.to(cuda_device))
        out.backward(g)
        want, grads = O.attention_core_step(q.detach().double().cpu(), k.detach().double().cpu(),
                                            v.detach().double().cpu(), None if mask is None else mask.double(), heads,
                                            grad_out=g.double().cpu())
        _check(out, want, f"attention edge {tag}:out")
        for name, t in (("query", q), ("key", k), ("value", v)):
            _check(t.grad, grads[name], f"attention edge {tag}:grad_{name}")

    one(2, 4, 1, 300, 64, None, "decode step")
    more_q = (1.0 - torch.ones(300, 100).tril(100 - 300)).view(1, 1, 300, 100) * -10000.0
    assert not mask_is_causal(more_q.to(cuda_device), 300, 100)
    one(1, 2, 300, 100, 32, more_q, "more queries than keys")
    partial = torch.zeros(2, 1, 130, 130)
    partial[:, :, :, 100:] = float("-inf")
    partial[1, :, :, :7] = -10000.0
    one(2, 2, 130, 130, 48, partial, "-inf and finite mask values")
    per_row = torch.randn(3, 1, 1, 257)
    one(3, 2, 257, 257, 112, per_row, "batch of three, key mask, head size 112")
    L.check_device_status(cuda_device)


def test_causal_mask_is_detected_and_equivalent(cuda_device):
    """The causal fast path (rule applied in the kernel, tiles skipped) and the general path (mask read) agree, and
    the detection keys on the tensor object, not on its address."""
    import lean_transformer_b200 as L
    from lean_transformer_b200.attn import mask_is_causal

    torch.manual_seed(2)
    S, heads, d = 320, 2, 64
    q, k, v = (_bf16(torch.randn(2, S, heads * d)).to(cuda_device) for _ in range(3))
    causal = ((1.0 - torch.ones(S, S).tril()).view(1, 1, S, S) * -10000.0).to(cuda_device)
    assert mask_is_causal(causal, S, S) and mask_is_causal(causal.expand(2, 1, S, S).contiguous(), S, S)
    padded = causal.expand(2, 1, S, S).clone()
    padded[1, :, :, 300:] = -10000.0
    assert not mask_is_causal(padded, S, S)
    causal[0, 0, 5, 3] = -10000.0  # in-place edit of a tensor already seen: the version counter invalidates the cache
    assert not mask_is_causal(causal, S, S)
    causal[0, 0, 5, 3] = 0.0
    scale = 1.0 / math.sqrt(d)
    fast, lse_fast = L.ops.attention_forward(q, k, v, heads, scale, None, True)
    slow, lse_slow = L.ops.attention_forward(q, k, v, heads, scale, causal, False)
    torch.testing.assert_close(fast.float(), slow.float(), rtol=0, atol=1e-2)
    torch.testing.assert_close(lse_fast, lse_slow, rtol=1e-5, atol=1e-5)
    # causal + padding at the end of a row: the rule in the kernel plus one mask row per batch entry
    from lean_transformer_b200.attn import analyze_mask
    is_causal, key_mask = analyze_mask(padded, S, S)
    assert is_causal and key_mask is not None and key_mask.shape == (2, 1, 1, S)
    split, lse_split = L.ops.attention_forward(q, k, v, heads, scale, key_mask, True)
    whole, lse_whole = L.ops.attention_forward(q, k, v, heads, scale, padded, False)
    torch.testing.assert_close(split.float(), whole.float(), rtol=0, atol=1e-2)
    torch.testing.assert_close(lse_split, lse_whole, rtol=1e-5, atol=1e-5)
    g = _bf16(torch.randn(2, S, heads * d)).to(cuda_device)
    grads_split = L.ops.attention_backward(g, q, k, v, split, lse_split, heads, scale, key_mask, True)
    grads_whole = L.ops.attention_backward(g, q, k, v, whole, lse_whole, heads, scale, padded, False)
    for a, b in zip(grads_split, grads_whole):
        torch.testing.assert_close(a.float(), b.float(), rtol=0, atol=2e-2)
    # padding at the START of a row leaves early queries without an unpadded visible key: read as it is
    left = causal.expand(2, 1, S, S).clone()
    left[1, :, :, :9] += -10000.0
    assert analyze_mask(left, S, S) == (False, left) or analyze_mask(left, S, S)[0] is False


def test_attention_dropout_golden_and_oracle(cuda_device):
    """Dropout on the probabilities: the kernels' mask is the Philox function of (seed, offset, element index over
    [batch, heads, q_len, kv_len]); with that mask injected, the reference's core (golden vector) and the oracle agree
    with the kernels, forward and backward."""
    import lean_transformer_b200 as L

    blob = load_golden("attention_core_dropout")
    p, seed, offset, heads = float(blob["dropout"]), int(blob["seed"]), int(blob["offset"]), int(blob["heads"])
    t = {k: torch.from_numpy(v) for k, v in blob.items() if v.ndim > 0}
    q, k, v = (_bf16(t[n]).to(cuda_device) for n in ("query", "key", "value"))
    g = _bf16(t["grad_out"]).to(cuda_device)
    mask = t["mask"].float().to(cuda_device)
    d = q.shape[-1] // heads
    out, lse = L.ops.attention_forward(q, k, v, heads, d ** -0.5, mask, False, p, seed, offset)
    dq, dk, dv = L.ops.attention_backward(g, q, k, v, out, lse, heads, d ** -0.5, mask, False, p, seed, offset)
    _check(out, t["out"], "attention dropout golden:out")
    for name, got in (("query", dq), ("key", dk), ("value", dv)):
        _check(got, t[f"grad_{name}"], f"attention dropout golden:grad_{name}", scaled=True)
    # a key length that is not a multiple of four (mask groups straddle the chunks), ragged tiles, 2 heads of 48
    torch.manual_seed(9)
    batch, heads, q_len, kv_len, d = 2, 2, 150, 203, 48
    q = _bf16(torch.randn(batch, q_len, heads * d)).to(cuda_device)
    k, v = (_bf16(torch.randn(batch, kv_len, heads * d)).to(cuda_device) for _ in range(2))
    g = _bf16(torch.randn(batch, q_len, heads * d)).to(cuda_device)
    p, seed, offset = 0.1, 1234567, 8
    keep = torch.from_numpy(O.dropout_keep_mask(batch * heads * q_len * kv_len, p, seed, offset)).view(batch, heads, q_len, kv_len)
    out, lse = L.ops.attention_forward(q, k, v, heads, d ** -0.5, None, True, p, seed, offset)
    dq, dk, dv = L.ops.attention_backward(g, q, k, v, out, lse, heads, d ** -0.5, None, True, p, seed, offset)
    causal = (1.0 - torch.ones(q_len, kv_len).tril(kv_len - q_len)).view(1, 1, q_len, kv_len).double() * -10000.0
    want, grads = O.attention_core_step(q.double().cpu(), k.double().cpu(), v.double().cpu(), causal, heads,
                                        grad_out=g.double().cpu(), dropout_p=p, keep_mask=keep)
    _check(out, want, "attention dropout ragged:out")
    for name, got in (("query", dq), ("key", dk), ("value", dv)):
        _check(got, grads[name], f"attention dropout ragged:grad_{name}", scaled=True)
    L.check_device_status(cuda_device)


def test_attention_dropout_module_behaviour(cuda_device):
    """Module level: the mask follows torch's CUDA generator (same seed, same result; another seed, another result),
    forward and backward use the same mask (gradient check against a finite difference is not needed: the golden test
    pins both), and evaluation mode drops nothing."""
    import lean_transformer_b200 as L

    core = L.SimpleAttentionCore(128, 2, attention_probs_dropout=0.3).to(cuda_device).train()
    x = _bf16(torch.randn(2, 96, 128)).to(cuda_device)

    def run(seed):
        torch.manual_seed(seed)
        leaf = x.clone().requires_grad_(True)
        out, _ = core(leaf, leaf, leaf, None)
        out.float().sum().backward()
        return out.detach().clone(), leaf.grad.clone()

    a, ga = run(1)
    b, gb = run(1)
    c, _ = run(2)
    assert torch.equal(a, b) and torch.equal(ga, gb), "same generator state must give the same mask"
    assert not torch.equal(a, c), "the mask ignored the generator"
    core.eval()
    e1, _ = core(x, x, x, None)
    plain, _ = L.SimpleAttentionCore(128, 2).to(cuda_device)(x, x, x, None)
    assert torch.equal(e1, plain), "dropout must be off in evaluation mode"


@pytest.mark.parametrize("rotary", [False, True])
def test_fused_qkv_entry_equals_the_three_slice_call(cuda_device, rotary):
    """forward_qkv (what this package's LeanSelfAttention calls) against forward on the three slices: same kernels,
    same bits, and the gradient arrives as one [batch, len, 3 * hidden] tensor."""
    import lean_transformer_b200 as L

    torch.manual_seed(5)
    heads, d, length = 4, 48, 200
    hidden = heads * d
    core = (L.RotaryAttentionCore if rotary else L.SimpleAttentionCore)(hidden, heads).to(cuda_device).train()
    base = _bf16(torch.randn(2, length, 3 * hidden)).to(cuda_device)
    g = _bf16(torch.randn(2, length, hidden)).to(cuda_device)
    mask = ((1.0 - torch.ones(length, length).tril()).view(1, 1, length, length) * -10000.0).to(cuda_device)
    mask = mask + torch.zeros(2, 1, 1, length, device=cuda_device)
    mask[1, :, :, length - 20:] = -10000.0
    a = base.clone().requires_grad_(True)
    out_a, _ = core(*a.split(hidden, dim=-1), mask)
    out_a.backward(g)
    b = base.clone().requires_grad_(True)
    out_b, probs = core.forward_qkv(b, mask)
    out_b.backward(g)
    assert probs is None and torch.equal(out_a, out_b)
    assert b.grad.shape == base.shape and torch.equal(a.grad, b.grad)


def test_rotary_kernel_matches_oracle(cuda_device):
    import lean_transformer_b200 as L

    torch.manual_seed(1)
    batch, length, heads, d = 2, 70, 3, 48
    x = torch.randn(batch, length, heads * d)
    emb = L.RotaryEmbeddings(d).to(cuda_device)
    cos, sin = emb.tables(length, cuda_device)
    ocos, osin = O.rotary_tables(length, d, dtype=torch.float32)
    torch.testing.assert_close(cos.cpu(), ocos, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(sin.cpu(), osin, rtol=1e-6, atol=1e-6)
    want = O.rotary_apply(x.view(batch, length, heads, d).double(), ocos.double(), osin.double())
    got = L.ops.rotary(x.to(cuda_device), cos, sin, heads, out_dtype=torch.float32)
    torch.testing.assert_close(got.cpu().view_as(want).double(), want, rtol=1e-5, atol=1e-5)
    back = L.ops.rotary(x.to(cuda_device), cos, sin, heads, inverse=True, out_dtype=torch.float32)
    want_back = O.rotary_apply_transposed(x.view(batch, length, heads, d).double(), ocos.double(), osin.double())
    torch.testing.assert_close(back.cpu().view_as(want_back).double(), want_back, rtol=1e-5, atol=1e-5)
    via_module = emb(x.to(cuda_device).view(batch, length, heads, d))
    torch.testing.assert_close(via_module.cpu().double(), want, rtol=1e-5, atol=1e-5)
    # a head size whose halves are not a multiple of eight takes the one-pair-per-thread kernel
    d2 = 20
    x2 = torch.randn(batch, length, heads * d2)
    cos2, sin2 = O.rotary_tables(length, d2, dtype=torch.float32)
    want2 = O.rotary_apply(x2.view(batch, length, heads, d2).double(), cos2.double(), sin2.double())
    got2 = L.ops.rotary(x2.to(cuda_device), cos2.to(cuda_device), sin2.to(cuda_device), heads, out_dtype=torch.float32)
    torch.testing.assert_close(got2.cpu().view_as(want2).double(), want2, rtol=1e-5, atol=1e-5)
    # bf16 in and out: one rounding of the fp32 result
    got_bf16 = L.ops.rotary(x.to(cuda_device).bfloat16(), cos, sin, heads)
    want_bf16 = O.rotary_apply(x.bfloat16().view(batch, length, heads, d).double(), ocos.double(), osin.double())
    torch.testing.assert_close(got_bf16.cpu().view_as(want_bf16).double(), want_bf16, rtol=2 ** -8, atol=1e-3)


def test_attention_rejections(cuda_device):
    """What the kernels do not cover fails loudly instead of running something else."""
    import lean_transformer_b200 as L

    x = torch.randn(1, 64, 128, device=cuda_device)
    core = L.SimpleAttentionCore(128, 2).to(cuda_device)
    with pytest.raises(NotImplementedError, match="bfloat16"):
        core(x, x, x, None)  # float32 outside autocast
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out, _ = core(x, x, x, None)  # same tensors under autocast: computed in bf16
    assert out.dtype == torch.bfloat16
    xb = x.bfloat16()
    with pytest.raises(NotImplementedError, match="head sizes"):
        L.SimpleAttentionCore(120, 5).to(cuda_device)(xb[..., :120], xb[..., :120], xb[..., :120], None)  # head size 24
    with pytest.raises(AssertionError, match="float mask"):
        core(xb, xb, xb, torch.ones(1, 1, 64, 64, dtype=torch.bool, device=cuda_device))
    block = L.LeanSelfAttention(128, 2).to(cuda_device)
    with torch.autocast("cuda", dtype=torch.bfloat16), pytest.raises(NotImplementedError, match="output_attentions"):
        block(x, None, output_attentions=True)
    with pytest.raises(RuntimeError, match="CUDA"):
        core(xb.cpu(), xb.cpu(), xb.cpu(), None)
