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
    assert _native.lib.leanffn_abi_version() == _native.ABI_VERSION == 4
    assert _native.status_string(0) == "ok"
    assert "shape" in _native.status_string(-2)


def _struct_fields(name: str):
    text = (ROOT / "include" / "leanffn_b200.h").read_text()
    body = text[text.index(f"typedef struct {name} {{"):text.index(f"}} {name};")]
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
    return [re.sub(r"\[\d+\]$", "", f) for f in fields]  # array members: name[8] -> name


def test_descriptor_layout_matches_header():
    """Field order of every ctypes mirror equals the field order of its C struct."""
    from lean_transformer_b200 import _native

    for c_name, mirror in (("leanffn_gemm_desc", _native.GemmDesc), ("leanffn_linear_desc", _native.LinearDesc),
                           ("leanffn_ffn_desc", _native.FfnDesc), ("leanffn_ffn_grads", _native.FfnGrads)):
        assert _struct_fields(c_name) == [f[0] for f in mirror._fields_], c_name


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


def test_struct_sizes_and_offsets_match_a_c_compiler(tmp_path):
    """The ctypes mirrors have the size and the member offsets a C compiler gives the header's structs."""
    import shutil
    import subprocess
    from lean_transformer_b200 import _native

    gcc = shutil.which("gcc") or shutil.which("cc")
    if gcc is None:
        pytest.skip("no C compiler")
    structs = {"leanffn_gemm_desc": _native.GemmDesc, "leanffn_linear_desc": _native.LinearDesc,
               "leanffn_ffn_desc": _native.FfnDesc, "leanffn_ffn_grads": _native.FfnGrads,
               "leanffn_attention_desc": _native.AttentionDesc}
    lines = ['#include <stddef.h>', '#include <stdio.h>', '#include "leanffn_b200.h"', 'int main(void) {']
    for c_name, mirror in structs.items():
        lines.append(f'  printf("{c_name} %zu\\n", sizeof({c_name}));')
        for field, _ in mirror._fields_:
            lines.append(f'  printf("{c_name}.{field} %zu\\n", offsetof({c_name}, {field}));')
    lines += ['  return 0;', '}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([gcc, "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    got = dict(line.split() for line in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.splitlines())
    for c_name, mirror in structs.items():
        assert int(got[c_name]) == ctypes.sizeof(mirror), c_name
        for field, _ in mirror._fields_:
            assert int(got[f"{c_name}.{field}"]) == getattr(mirror, field).offset, f"{c_name}.{field}"
