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


def assert_close(got: torch.Tensor, ref: torch.Tensor, rtol: float, atol: float, what: str = "", scale_atol=False,
                 branch: torch.Tensor = None, outlier_frac: float = 0.0):
    """|got - ref| <= atol * max(1, S) + rtol * max(|ref|, |branch|, S), elementwise.

    With S = 0 and no branch this is torch.allclose's rule.  The two extensions judge an element at the scale
    of the computation that produced it rather than at the size it happens to end up with:

    ``scale_atol``: S = rms of the GEMM-produced tensor (``branch`` if given, else ``ref``).  A matrix product
    accumulates hundreds to tens of thousands of products; its rounding noise is proportional to the rms of
    the accumulated sums, also for the elements whose terms cancel to ~0.

    ``branch``: where a residual is added exactly (out = x + branch, dx = g + branch'), the reference value of
    the computed branch; an output that cancels against the residual is judged at the branch's size.

    ``outlier_frac`` (bf16 only): rounding noise is random, so among millions of elements a few land beyond any
    fixed multiple of its standard deviation.  Up to this fraction may exceed the bound; none may exceed 4x."""
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    mag = ref.abs()
    produced = ref
    if branch is not None:
        produced = branch.detach().double().cpu().reshape(ref.shape)
        mag = torch.maximum(mag, produced.abs())
    S = float(produced.pow(2).mean().sqrt()) if scale_atol and produced.numel() else 0.0
    err = (got - ref).abs()
    bound = atol * max(1.0, S) + rtol * mag.clamp_min(S)
    bad = err > bound
    if outlier_frac > 0 and int(bad.sum()) <= outlier_frac * bad.numel() and not (err > 4 * bound).any():
        return
    if bad.any():
        worst = int((err - bound).argmax())
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.numel()} elements out of tolerance (rtol {rtol}, atol {atol}, S {S:.3g}); "
            f"worst |err| {float(err.flatten()[worst]):.4g} at ref {float(ref.flatten()[worst]):.4g} "
            f"(bound {float(bound.flatten()[worst]):.4g}); max |err| {float(err.max()):.4g}, "
            f"max |ref| {float(ref.abs().max()):.4g}")


@pytest.fixture
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)
