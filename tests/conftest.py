import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
GOLDEN = ROOT / "tests" / "golden"

# Parity tolerances against the fp32/fp64 oracle.
BF16_RTOL, BF16_ATOL = 2e-2, 1e-2   # bf16 tensor-core path
FP32_RTOL, FP32_ATOL = 1e-4, 1e-4   # fp32 mode


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_golden(name: str) -> dict:
    with np.load(GOLDEN / f"{name}.npz", allow_pickle=False) as f:
        return {k: f[k] for k in f.files}


def golden_ffn_case(name: str, dtype=torch.float64):
    """(x, g, params, expected, meta) of an LeanFFN golden file as torch tensors."""
    blob = load_golden(name)
    conv = lambda a: torch.from_numpy(a).to(dtype) if a.dtype.kind == "f" else torch.from_numpy(a)  # noqa: E731
    params = {k[len("param_"):]: conv(v) for k, v in blob.items() if k.startswith("param_")}
    expected = {k[len("grad_"):]: conv(v) for k, v in blob.items() if k.startswith("grad_")}
    expected["out"] = conv(blob["out"])
    meta = {k[len("meta_"):]: v.item() for k, v in blob.items() if k.startswith("meta_")}
    if "keep_mask" in blob:
        meta["keep_mask"] = torch.from_numpy(blob["keep_mask"])
    return conv(blob["x"]), conv(blob["g"]), params, expected, meta


def assert_close(got: torch.Tensor, ref: torch.Tensor, rtol: float, atol: float, what: str = "", scale_atol=False):
    """|got - ref| <= atol' + rtol * |ref| elementwise.  With ``scale_atol`` (used for gradients that sum
    over thousands of tokens) atol' = atol * max(1, rms(ref)): the absolute floor follows the size of the
    sums, whose rounding noise grows with the number and magnitude of the terms, not with the individual
    element that happens to be near zero."""
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    floor = atol * max(1.0, float(ref.pow(2).mean().sqrt())) if scale_atol else atol
    err = (got - ref).abs()
    bound = floor + rtol * ref.abs()
    bad = err > bound
    if bad.any():
        worst = int((err - bound).argmax())
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.numel()} elements out of tolerance (rtol {rtol}, atol {floor:.3g}); "
            f"worst |err| {float(err.flatten()[worst]):.4g} at ref {float(ref.flatten()[worst]):.4g}; "
            f"max |err| {float(err.max()):.4g}, max |ref| {float(ref.abs().max()):.4g}")


@pytest.fixture
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)
