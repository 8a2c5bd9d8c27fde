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
