"""convert_model swaps reference-named modules for the CUDA drop-ins while re-using parameters (host logic only)."""
import torch
import torch.nn as nn

import lean_transformer_b200 as L
from lean_transformer_b200.integration import convert_model


def _make_reference_like():
    """Stand-ins that carry the reference's class names and attributes (the reference is not importable here)."""
    class GeneralizedMatrix(nn.Module):
        def __init__(self, i, o):
            super().__init__()
            self.in_features, self.out_features, self.blocksparse_backend = i, o, "native"
            self.weight = nn.Parameter(torch.randn(o, i))
            self.layout = self.forward_indices = self.backward_indices = None
            self.lowrank_first, self.lowrank_second = nn.Parameter(torch.randn(4, i)), nn.Parameter(torch.randn(o, 4))

    class GeneralizedLinear(nn.Linear):
        def __init__(self, matrix):
            nn.Module.__init__(self)
            self.matrix, self.in_features, self.out_features = matrix, matrix.in_features, matrix.out_features
            self.bias = nn.Parameter(torch.zeros(matrix.out_features))
            self.adapter_first = self.adapter_second = None

    class LeanFFN(nn.Module):
        def __init__(self, shared_i2h, shared_h2o):
            super().__init__()
            self.i2h_proj, self.h2o_proj = GeneralizedLinear(shared_i2h), GeneralizedLinear(shared_h2o)
            self.pre_layer_norm, self.post_layer_norm = nn.LayerNorm(32), None
            self.activation, self.gated, self.dropout, self.residual = nn.GELU(), True, 0.1, True
            self.ffn_custom_grad = True

    m1, m2 = GeneralizedMatrix(32, 128), GeneralizedMatrix(64, 32)
    model = nn.Sequential(nn.Sequential(LeanFFN(m1, m2)), LeanFFN(m1, m2), GeneralizedLinear(m1))
    return model, m1, m2


def test_convert_model_reuses_parameters_and_sharing():
    model, m1, m2 = _make_reference_like()
    before = {k: v.data_ptr() for k, v in model.state_dict().items()}
    convert_model(model)
    first, second, lone = model[0][0], model[1], model[2]
    assert isinstance(first, L.LeanFFN) and isinstance(second, L.LeanFFN)
    assert isinstance(lone, L.GeneralizedLinear) and isinstance(first.i2h_proj, L.GeneralizedLinear)
    # shared matrices stay shared, parameters are the same objects
    assert first.i2h_proj.matrix is second.i2h_proj.matrix is lone.matrix
    assert first.i2h_proj.matrix.weight is m1.weight and first.h2o_proj.matrix.weight is m2.weight
    assert first.i2h_proj is not second.i2h_proj and first.i2h_proj.bias is not second.i2h_proj.bias
    after = {k: v.data_ptr() for k, v in model.state_dict().items()}
    assert before == after
    assert first.gated and first.dropout == 0.1 and L.resolve_activation(first.activation) == 1
    assert first.i2h_proj.get_combined_lowrank_components()[0] is m1.lowrank_first
    convert_model(model)  # idempotent
    assert model[1] is second


# ---- against the reference's real classes (needs the mirror made by oracle/build_ref.py) --------------------------
def _reference():
    import pytest
    from oracle import ref_harness
    ref = ref_harness.import_reference()
    if ref is None:
        pytest.skip("oracle/_ref has not been built (python oracle/build_ref.py)")
    return ref


def _tiny_gpt(ref, **overrides):
    kw = dict(vocab_size=100, hidden_size=64, embedding_size=64, num_hidden_layers=4, num_hidden_groups=2,
              num_attention_heads=4, position_embedding_type="rotary", hidden_act_gated=True, tie_word_embeddings=True,
              share_large_matrices=True, adapter_dim=4, hidden_dropout_prob=0.1)
    kw.update(overrides)
    return ref.gpt.LeanGPTModel(ref.gpt.LeanGPTConfig(**kw))


def test_converted_reference_model_keeps_its_own_api():
    """lean_transformer/transformer.py:89-152: set_optimizations must keep finding (and only finding) its FFNs and
    matrices after the swap, before and after the model has built its cached layer sequence."""
    ref = _reference()
    for build_sequence_first in (False, True):
        torch.manual_seed(0)
        model = _tiny_gpt(ref)
        keys = list(model.state_dict().keys())
        pointers = {k: v.data_ptr() for k, v in model.state_dict().items()}
        if build_sequence_first:
            model.transformer._get_sequential()
            model.set_optimizations(gradient_checkpointing=2)
        convert_model(model)
        assert list(model.state_dict().keys()) == keys
        assert {k: v.data_ptr() for k, v in model.state_dict().items()} == pointers
        ffns = [m for m in model.modules() if isinstance(m, L.LeanFFN)]
        assert len(ffns) == 2 and all(isinstance(m, ref.ffn.LeanFFN) for m in ffns)  # 2 groups of shared layers
        assert not any(type(m) is ref.ffn.LeanFFN for m in model.modules())
        # the layer sequence the model actually runs holds the drop-ins and kept its settings
        sequence = model.transformer._get_sequential()
        run = [w.module for w in sequence if type(w.module).__name__ == "LeanFFN"]
        assert len(run) == 4 and all(isinstance(m, L.LeanFFN) for m in run) and {id(m) for m in run} == {id(m) for m in ffns}
        if build_sequence_first:
            assert sequence.gradient_checkpointing == 2
        for flag in (False, True):
            model.set_optimizations(ffn_custom_grad=flag, checkpoint_attention_core=flag)
            assert all(m.ffn_custom_grad is flag for m in ffns)
        # shared matrices stay shared between the FFN layers of the two groups, adapters stay per layer
        assert ffns[0].i2h_proj.matrix is ffns[1].i2h_proj.matrix and ffns[0].i2h_proj is not ffns[1].i2h_proj
        assert ffns[0].i2h_proj.adapter_first is not ffns[1].i2h_proj.adapter_first
        matrices = [m for m in model.modules() if isinstance(m, L.GeneralizedMatrix)]
        assert matrices and all(isinstance(m, ref.linear.GeneralizedMatrix) for m in matrices)
        for m in matrices:
            m._matmul_op = "stale"
        model.set_optimizations(update_triton_blocksparse_ops=True)
        assert all(m._matmul_op is None for m in matrices)


def test_convert_model_on_a_root_ffn():
    ref = _reference()
    ffn = ref.ffn.LeanFFN(32, 64, gated=True, dropout=0.1)
    new = convert_model(ffn)
    assert isinstance(new, L.LeanFFN) and isinstance(new, ref.ffn.LeanFFN) and new is not ffn
    assert new.i2h_proj is ffn.i2h_proj and new.pre_layer_norm is ffn.pre_layer_norm and new.dropout == 0.1
    assert convert_model(new) is new
