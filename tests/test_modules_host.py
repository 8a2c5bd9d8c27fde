"""Host-side behaviour of the drop-in modules: constructor contracts, parameter / buffer names, activation
registry, padding helper (no GPU involved)."""
from pathlib import Path

import pytest
import torch
import torch.nn as nn

import lean_transformer_b200 as L
from lean_transformer_b200 import _native as N
from lean_transformer_b200.blocksparse.linear import GeneralizedLinear, GeneralizedMatrix

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_state_dict_layout_matches_reference():
    layout = "pixelfly(16)"
    ffn = L.LeanFFN(32, 64, gated=True, post_layer_norm=True,
                    i2h_proj=GeneralizedLinear(GeneralizedMatrix(32, 128, layout, 6), 2),
                    h2o_proj=GeneralizedLinear(GeneralizedMatrix(64, 32, layout, 0), 0))
    ours = [f"{k} {tuple(v.shape)} {v.dtype}" for k, v in ffn.state_dict().items()]
    ref = (GOLDEN / "state_dict_keys.txt").read_text().strip().splitlines()
    assert ours == ref


def test_constructor_contracts():
    with pytest.raises(AssertionError):
        L.LeanFFN(32, 64, i2h_proj=nn.Linear(32, 100))  # wrong width
    with pytest.raises(AssertionError):
        L.LeanFFN(32, 64, i2h_proj=nn.Sequential(nn.Linear(32, 64)))  # custom grad needs Linear / GeneralizedLinear

    class Odd(nn.Linear):
        pass

    L.LeanFFN(32, 64, i2h_proj=Odd(32, 64), ffn_custom_grad=False)  # allowed without custom grad
    with pytest.raises(NotImplementedError):
        L.LeanFFN(32, 64, activation=lambda x: x * 2)  # no kernel for arbitrary callables
    with pytest.raises(NotImplementedError):
        GeneralizedMatrix(32, 32, "pixelfly(8)", blocksparse_backend="cusparse")
    with pytest.raises(AssertionError):
        GeneralizedMatrix(32, 32, None, blocksparse_backend="triton")
    m = GeneralizedMatrix(64, 128, "pixelfly(16)", blocksparse_backend="triton")
    assert tuple(m.weight.shape) == (1, int(m.layout.sum()), 16, 16) and m.forward_indices is None
    assert m.matmul_op.out_features == 128 and m.matmul_op is m.matmul_op
    assert repr(m) == "GeneralizedMatrix(128, 64)"


def test_combined_lowrank_components():
    lin = GeneralizedLinear(GeneralizedMatrix(32, 64, None, 6), 2)
    first, second = lin.get_combined_lowrank_components()
    assert first.shape == (8, 32) and second.shape == (64, 8)
    assert torch.equal(first[:6], lin.matrix.lowrank_first) and torch.equal(second[:, 6:], lin.adapter_second)
    assert GeneralizedLinear(GeneralizedMatrix(32, 64)).get_combined_lowrank_components() == (None, None)
    only_adapter = GeneralizedLinear(GeneralizedMatrix(32, 64), 3)
    assert only_adapter.get_combined_lowrank_components()[0] is only_adapter.adapter_first
    assert lin.weight is lin.matrix.weight


def test_activation_registry():
    assert L.resolve_activation(L.ACT2FN["gelu_fused"]) == N.ACT_GELU_TANH
    assert L.resolve_activation(nn.GELU()) == N.ACT_GELU_ERF
    assert L.resolve_activation(nn.GELU(approximate="tanh")) == N.ACT_GELU_TANH
    assert L.resolve_activation(torch.nn.functional.silu) == N.ACT_SILU
    assert L.resolve_activation(nn.ReLU()) == N.ACT_RELU
    assert L.resolve_activation("swish") == N.ACT_SILU
    for key in ("gelu", "gelu_new", "relu", "silu", "tanh", "sigmoid", "linear"):
        assert key in L.ACT2FN


def test_pad_to_multiple():
    x = torch.randn(3, 3)
    assert L.pad_to_multiple(x, multiple=3, dims=0) is x
    assert L.pad_to_multiple(x, multiple=3, dims=[0, 1]) is x
    assert L.pad_to_multiple(x, multiple=2, dims=1) is not x
    assert L.pad_to_multiple(x, multiple=2, dims=0).shape == (4, 3)
    assert L.pad_to_multiple(x, multiple=4, dims=1).shape == (3, 4)
    assert L.pad_to_multiple(x, multiple=2, dims=[0, 1]).shape == (4, 4)
    assert torch.allclose(L.pad_to_multiple(x, multiple=4, dims=1).sum(), x.sum())
    assert L.pad_to_multiple(x, multiple=10, dims=0)[3:].norm() == 0
    assert torch.equal(L.pad_to_multiple(x, multiple=2, dims=-1)[:, :3], x)


def test_attention_mask_analysis():
    """Host-side recognition of the causal pattern and of causal + per-key padding (no device needed)."""
    import torch
    from lean_transformer_b200.attn import analyze_mask, mask_is_causal

    S = 12
    causal = (1.0 - torch.ones(S, S).tril()).view(1, 1, S, S) * -10000.0
    assert analyze_mask(None, S, S) == (False, None)
    assert analyze_mask(causal, S, S) == (True, None) and mask_is_causal(causal, S, S)
    right = torch.zeros(3, 1, 1, S)
    right[1, 0, 0, 8:] = -10000.0
    is_causal, key_mask = analyze_mask(right + causal, S, S)
    assert is_causal and key_mask.shape == (3, 1, 1, S) and torch.equal(key_mask, right)
    assert not mask_is_causal(right + causal, S, S)
    left = torch.zeros(3, 1, 1, S)
    left[2, 0, 0, :4] = -10000.0  # the first query rows of that batch entry see padded keys only
    is_causal, to_read = analyze_mask(left + causal, S, S)
    assert not is_causal and to_read.shape == (3, 1, S, S)
    assert analyze_mask(torch.randn(2, 1, S, S), S, S)[0] is False
    assert analyze_mask(torch.zeros(1, 1, S, S), S, S)[0] is False  # no mask at all is not the causal pattern
    wide = (1.0 - torch.ones(S, S + 5).tril(5)).view(1, 1, S, S + 5) * -10000.0  # keys of a cache before the queries
    assert analyze_mask(wide, S, S + 5) == (True, None)
    tall = (1.0 - torch.ones(S + 5, S).tril(-5)).view(1, 1, S + 5, S) * -10000.0  # more queries than keys: read as it is
    assert analyze_mask(tall, S + 5, S)[0] is False
    edited = causal.clone()
    assert analyze_mask(edited, S, S) == (True, None)
    edited[0, 0, 3, 1] = -5.0  # an in-place edit of a tensor already analysed: the version counter invalidates the answer
    assert analyze_mask(edited, S, S)[0] is False
