"""The C ABI from a host that is not Python: the header must be valid C and C++, and a plain-C program linked against
libleanffn_b200.so and the CUDA runtime must get correct results from the kernels."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "leanffn_b200.h"
CUDA = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))


@pytest.mark.parametrize("compiler,flags", [("gcc", ["-x", "c", "-std=c99"]), ("g++", ["-x", "c++", "-std=c++11"])])
def test_header_is_valid_c_and_cxx(compiler, flags):
    if shutil.which(compiler) is None:
        pytest.skip(f"{compiler} not installed")
    res = subprocess.run([compiler, "-fsyntax-only", "-Wall", "-Werror", *flags, str(HEADER)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr


def _build_c_host(out_dir: Path) -> Path:
    from lean_transformer_b200 import build
    lib = build.build()
    exe = out_dir / "leanffn_c_host"
    cmd = ["gcc", "-std=c99", "-O1", "-Wall", "-I", str(ROOT / "include"), "-I", str(CUDA / "include"),
           str(ROOT / "tests" / "c_host" / "leanffn_c_host.c"), "-o", str(exe), str(lib),
           "-L", str(CUDA / "lib64"), "-lcudart", "-lm", f"-Wl,-rpath,{lib.parent}", f"-Wl,-rpath,{CUDA / 'lib64'}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def test_c_host_compiles_and_links(tmp_path):
    if shutil.which("gcc") is None or not (CUDA / "include" / "cuda_runtime_api.h").exists():
        pytest.skip("gcc or the CUDA toolkit headers are not installed")
    assert _build_c_host(tmp_path).exists()


def _write_block_case(path: Path, name: str = "ffn_dropout_mask"):
    """A golden vector of the reference (gated, residual, dropout with the Philox mask) as the flat file the C host
    reads: int64 header, then float32 inputs, parameters and expected results."""
    import numpy as np
    blob = np.load(ROOT / "tests" / "golden" / f"{name}.npz")
    x = blob["x"].reshape(-1, blob["x"].shape[-1])
    tokens, hidden = x.shape
    inter = blob["param_h2o_weight"].shape[1]
    head = np.array([0x4C45414E, tokens, hidden, inter, int(blob["meta_gated"]), int(blob["meta_residual"]),
                     int(blob["meta_seed"]), int(blob["meta_offset"]), round(float(blob["meta_dropout"]) * 1e6), 0],
                    dtype=np.int64)
    order = ["x", "g", "param_ln_weight", "param_ln_bias", "param_i2h_weight", "param_i2h_bias", "param_h2o_weight",
             "param_h2o_bias", "out", "grad_input", "grad_ln_weight", "grad_ln_bias", "grad_i2h_weight", "grad_i2h_bias",
             "grad_h2o_weight", "grad_h2o_bias"]
    with open(path, "wb") as f:
        f.write(head.tobytes())
        for key in order:
            f.write(np.ascontiguousarray(blob[key], dtype=np.float32).tobytes())


def _write_attention_case(path: Path, name: str = "attention_core_simple"):
    """A golden vector of the reference's SimpleAttentionCore (causal + padding mask) as the flat file the C host reads."""
    import numpy as np
    blob = np.load(ROOT / "tests" / "golden" / f"{name}.npz")
    batch, length, hidden = blob["query"].shape
    heads = int(blob["heads"])
    head = np.array([0x4154544E, batch, length, heads, hidden // heads, 0], dtype=np.int64)
    mask = np.broadcast_to(blob["mask"], (batch, 1, length, length)).reshape(batch, length, length)
    with open(path, "wb") as f:
        f.write(head.tobytes())
        for arr in (blob["query"], blob["key"], blob["value"], blob["grad_out"], mask, blob["out"], blob["grad_query"],
                    blob["grad_key"], blob["grad_value"]):
            f.write(np.ascontiguousarray(arr, dtype=np.float32).tobytes())


@pytest.mark.gpu
def test_c_host_runs_the_kernels(tmp_path):
    exe = _build_c_host(tmp_path)
    case, attention = tmp_path / "block_case.bin", tmp_path / "attention_case.bin"
    _write_block_case(case)
    _write_attention_case(attention)
    res = subprocess.run([str(exe), str(case), str(attention)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "C HOST OK" in res.stdout and "block: grad W2" in res.stdout \
        and "attention: grad q" in res.stdout, res.stdout + res.stderr
