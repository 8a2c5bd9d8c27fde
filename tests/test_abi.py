"""The C-ABI library loads and exports every symbol include/leanffn_b200.h declares (no compute calls)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "leanffn_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(leanffn_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from lean_transformer_b200 import _native

    names = declared_symbols()
    assert len(names) >= 14
    lib = ctypes.CDLL(str(_native.LIB_PATH))
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(_native.EXPORTED_SYMBOLS) == names, "ctypes bindings and header disagree"
    assert _native.lib.leanffn_abi_version() == 2
    assert _native.status_string(0) == "ok"
    assert "shape" in _native.status_string(-2)


def test_descriptor_layout_matches_header():
    """Field order of the ctypes mirror equals the field order of the C struct."""
    from lean_transformer_b200 import _native

    text = (ROOT / "include" / "leanffn_b200.h").read_text()
    body = text[text.index("typedef struct leanffn_gemm_desc {"):text.index("} leanffn_gemm_desc;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split("{", 1)[1].split(";"):
        decl = decl.strip()
        if not decl:
            continue
        names = decl.split(",")
        first = names[0].split()[-1].lstrip("*")
        fields.append(first)
        fields.extend(n.strip().lstrip("*") for n in names[1:])
    fields = [re.sub(r"\[\d+\]$", "", f) for f in fields]  # array members: name[8] -> name
    assert fields == [f[0] for f in _native.GemmDesc._fields_]


def test_argument_validation_without_gpu():
    """Rejected arguments return negative codes before anything is launched."""
    from lean_transformer_b200 import _native as N

    assert N.lib.leanffn_gemm(None, None) == -1
    d = N.GemmDesc()
    assert N.lib.leanffn_gemm(ctypes.byref(d), None) == -2  # empty shape
    d.M = d.N = d.K = 8
    assert N.lib.leanffn_gemm(ctypes.byref(d), None) == -1  # null operands
    assert N.lib.leanffn_layer_norm_forward(None, 0, None, None, 0, None, 0, 4, 4, 1e-5, 0.0, 0, 0, None, 0, None) == -1
    assert N.lib.leanffn_dropout(1, 0, 1, 0, 16, 1.5, 0, 0, None, 0, None) == -5  # p out of range
    assert N.lib.leanffn_activation_forward(1, 1, 0, 4, 6, 0, 0, None) == -2  # width not a multiple of 4
    assert N.lib.leanffn_activation_forward(1, 1, 0, 4, 8, 0, 99, None) == -5  # unknown activation
    assert N.lib.leanffn_layer_norm_backward_scratch_bytes(0, 16) == 0


def test_cpu_tensors_are_rejected_loudly():
    import lean_transformer_b200 as L

    ffn = L.LeanFFN(32, 64)
    with pytest.raises(RuntimeError, match="CUDA"):
        ffn(torch.randn(2, 3, 32))
    with pytest.raises(RuntimeError, match="CUDA"):
        L.blocksparse.linear.GeneralizedLinear(L.GeneralizedMatrix(32, 32))(torch.randn(2, 32))
