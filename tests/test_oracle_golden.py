"""Pins the CPU oracle to vectors produced by the reference implementation (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from conftest import assert_close, golden_ffn_case, load_golden
from oracle import leanffn_oracle as O

TIGHT = dict(rtol=1e-9, atol=1e-10)


@pytest.mark.parametrize("name", ["ffn_dense_plain", "ffn_gated_postln", "ffn_pixelfly_lowrank", "ffn_dropout_mask"])
def test_leanffn_matches_reference(name):
    x, g, params, expected, meta = golden_ffn_case(name)
    kw = dict(gated=bool(meta["gated"]), residual=bool(meta["residual"]), dropout_p=meta.get("dropout", 0.0),
              keep_mask=meta.get("keep_mask"))
    out, grads = O.leanffn_step(x, g, params, **kw)
    assert_close(out, expected["out"], what="out", **TIGHT)
    assert_close(grads["input"], expected["input"], what="grad_input", **TIGHT)
    checked = 0
    for key, ref in expected.items():
        if key in ("out", "input"):
            continue
        assert grads.get(key) is not None, f"oracle produced no gradient for {key}"
        assert_close(grads[key], ref, what=f"grad_{key}", **TIGHT)
        checked += 1
    assert checked >= 6


def test_dropout_mask_definition():
    """The mask stored with the golden dropout case is the oracle's Philox mask for the stored (seed, offset)."""
    _, _, _, _, meta = golden_ffn_case("ffn_dropout_mask")
    keep = O.dropout_keep_mask(meta["keep_mask"].numel(), meta["dropout"], meta["seed"], meta["offset"])
    assert np.array_equal(keep, meta["keep_mask"].numpy().reshape(-1))
    # offsets only shift the stream; rate is 1 - p
    a = O.dropout_keep_mask(4096, 0.25, 99, 0)
    b = O.dropout_keep_mask(2048, 0.25, 99, 2048)
    assert np.array_equal(a[2048:], b)
    assert abs(a.mean() - 0.75) < 0.03


def test_philox_known_answer():
    """Known-answer vectors of Philox4x32-10 from the Random123 distribution (kat_vectors):
    counter 0 / key 0, all ones, and the 'pi' vector restricted to what our counter layout can express."""
    out = O.philox4x32_10(np.array([0], dtype=np.uint64), 0)[0]
    assert [hex(v) for v in out] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]


def test_linear_matches_reference():
    b = {k: torch.from_numpy(v) for k, v in load_golden("linear_pixelfly_lowrank").items()}
    out, hid = O.linear_forward(b["x"], b["weight"], b["bias"], b["lowrank_first"], b["lowrank_second"],
                                b["forward_indices"])
    assert_close(out, b["out"], what="out", **TIGHT)
    grads = O.linear_backward(b["g"], b["x"], hid, b["weight"], b["lowrank_first"], b["lowrank_second"],
                              b["backward_indices"])
    for key in ("input", "weight", "bias", "lowrank_first", "lowrank_second"):
        assert_close(grads[key], b["grad_" + key], what=key, **TIGHT)


def test_blocksparse_matches_reference():
    b = {k: torch.from_numpy(v) for k, v in load_golden("blocksparse_matmul").items()}
    out = O.blocksparse_matmul(b["x"], b["weight"], b["forward_indices"])
    assert_close(out, b["out"], what="out", **TIGHT)
    dx, dw = O.blocksparse_matmul_backward(b["g"], b["x"], b["weight"], b["backward_indices"])
    assert_close(dx, b["grad_input"], what="dx", **TIGHT)
    assert_close(dw, b["grad_weight"], what="dw", **TIGHT)
    # the dense restatement has exactly the layout's support
    dense = O.blocksparse_to_dense(b["weight"], b["backward_indices"], b["out"].shape[-1])
    assert_close(b["x"] @ dense.t(), b["out"], what="dense equivalent", **TIGHT)
    bs = b["weight"].shape[-1]
    support = dense.reshape(dense.shape[0] // bs, bs, dense.shape[1] // bs, bs).abs().amax(dim=(1, 3)) > 0
    assert torch.equal(support, b["layout"].bool())


def test_gelu_matches_reference():
    b = {k: torch.from_numpy(v) for k, v in load_golden("gelu_fused").items()}
    assert_close(O.act_forward("gelu_tanh", b["x"]), b["y"], what="gelu", **TIGHT)
    assert_close(O.act_grad("gelu_tanh", b["x"]), b["dy"], what="gelu grad", **TIGHT)
    # reference test tests/test_utils.py: within 5e-4 of the exact GELU
    x = torch.linspace(-5, 5, 1000, dtype=torch.float64)
    assert (O.act_forward("gelu_tanh", x) - O.act_forward("gelu_erf", x)).abs().max() <= 5e-4


@pytest.mark.parametrize("name", O.ACT_NAMES)
def test_activation_grads_are_derivatives(name):
    x = torch.linspace(-4, 4, 401, dtype=torch.float64)
    x = x[x.abs() > 1e-3] if name == "relu" else x
    h = 1e-6
    numeric = (O.act_forward(name, x + h) - O.act_forward(name, x - h)) / (2 * h)
    assert_close(O.act_grad(name, x), numeric, rtol=1e-6, atol=1e-7, what=name)


def test_layer_norm_edge_cases():
    # constant rows with eps = 1e-12 must give exactly beta (zero variance), as F.layer_norm does
    x = torch.full((3, 16), 2.5, dtype=torch.float64)
    y = O.layer_norm_forward(x, torch.ones(16, dtype=torch.float64), torch.full((16,), 0.5, dtype=torch.float64), 1e-12)
    assert torch.equal(y, torch.full_like(y, 0.5))
    # backward against autograd
    x = torch.randn(5, 7, 24, dtype=torch.float64, requires_grad=True)
    gam = torch.randn(24, dtype=torch.float64, requires_grad=True)
    bet = torch.randn(24, dtype=torch.float64, requires_grad=True)
    dy = torch.randn(5, 7, 24, dtype=torch.float64)
    torch.nn.functional.layer_norm(x, (24,), gam, bet, 1e-5).backward(dy)
    dx, dg, db = O.layer_norm_backward(dy, x.detach(), gam.detach(), 1e-5)
    assert_close(dx, x.grad, what="dx", **TIGHT)
    assert_close(dg, gam.grad, what="dgamma", **TIGHT)
    assert_close(db, bet.grad, what="dbeta", **TIGHT)


@pytest.mark.parametrize("kind", ["simple", "rotary"])
def test_attention_core_matches_reference(kind):
    """The attention-core restatement (forward and hand-derived backward) against the reference's
    SimpleAttentionCore / RotaryAttentionCore run in float64 (tests/golden/make_golden.py)."""
    blob = {k: torch.from_numpy(v) for k, v in load_golden(f"attention_core_{kind}").items()}
    out, grads = O.attention_core_step(blob["query"], blob["key"], blob["value"], blob["mask"], int(blob["heads"]),
                                       grad_out=blob["grad_out"], rotary=kind == "rotary")
    torch.testing.assert_close(out, blob["out"], rtol=1e-9, atol=1e-11)
    for name in ("query", "key", "value"):
        torch.testing.assert_close(grads[name], blob[f"grad_{name}"], rtol=1e-9, atol=1e-11)


def test_rotary_transposed_is_the_gradient():
    torch.manual_seed(0)
    x = torch.randn(2, 9, 3, 8, dtype=torch.float64, requires_grad=True)
    g = torch.randn_like(x)
    cos, sin = O.rotary_tables(9, 8)
    O.rotary_apply(x, cos, sin).backward(g)
    torch.testing.assert_close(O.rotary_apply_transposed(g, cos, sin), x.grad, rtol=1e-12, atol=1e-12)


def test_attention_core_dropout_matches_reference():
    """Dropout on the probabilities: the reference's SimpleAttentionCore with the oracle's Philox mask injected in
    place of torch's (tests/golden/make_golden.py), against the restatement given the same mask."""
    blob = load_golden("attention_core_dropout")
    p, seed, offset, heads = float(blob["dropout"]), int(blob["seed"]), int(blob["offset"]), int(blob["heads"])
    t = {k: torch.from_numpy(v) for k, v in blob.items() if v.ndim > 0}
    batch, length = t["query"].shape[:2]
    keep = torch.from_numpy(O.dropout_keep_mask(batch * heads * length * length, p, seed, offset)).view(batch, heads, length, length)
    out, grads = O.attention_core_step(t["query"], t["key"], t["value"], t["mask"], heads, grad_out=t["grad_out"],
                                       dropout_p=p, keep_mask=keep)
    torch.testing.assert_close(out, t["out"], rtol=1e-9, atol=1e-11)
    for name in ("query", "key", "value"):
        torch.testing.assert_close(grads[name], t[f"grad_{name}"], rtol=1e-9, atol=1e-11)
