import json
import os
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


# Every comparison made through assert_close / record_closeness leaves a row here; a GPU session writes them to
# parity_report.json (in the folder GPU runs hand back) so the distance of each tensor from the LITERAL rule
# |got - ref| <= atol + rtol * |ref| is on record next to the rule the tests enforce.
PARITY_REPORT = []


def closeness(got: torch.Tensor, ref: torch.Tensor, rtol: float, atol: float, branch: torch.Tensor = None,
              scale_atol: bool = False):
    """Error statistics of ``got`` against ``ref`` under two rules:
    literal  |got - ref| <= atol + rtol * |ref|                                   (torch.allclose)
    scaled   |got - ref| <= atol * max(1, S) + rtol * max(|ref|, |branch|, S),   S = rms of the produced tensor.
    Returns (stats dict, err, scaled bound)."""
    assert got.shape == ref.shape, f"shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    # small tensors: float64 on the host; very large ones (weight gradients of the widest configurations, 10^8.7
    # elements) stay on the GPU in float32, which resolves errors 10^4 times smaller than the tolerances
    if got.is_cuda and got.numel() > (1 << 24):
        where, prec = got.device, torch.float32
    else:
        where, prec = "cpu", torch.float64
    conv = lambda t: t.detach().to(device=where, dtype=prec)  # noqa: E731
    got, ref = conv(got), conv(ref)
    mag = ref.abs()
    produced = ref
    if branch is not None:
        produced = conv(branch).reshape(ref.shape)
        mag = torch.maximum(mag, produced.abs())
    S = float(produced.pow(2).mean().sqrt()) if scale_atol and produced.numel() else 0.0
    err = (got - ref).abs()
    bound = atol * max(1.0, S) + rtol * mag.clamp_min(S)
    literal = atol + rtol * ref.abs()
    n = max(1, err.numel())
    stats = dict(numel=err.numel(), rtol=rtol, atol=atol, S=S,
                 rms_ref=float(ref.pow(2).mean().sqrt()) if err.numel() else 0.0,
                 max_err=float(err.max()) if err.numel() else 0.0,
                 literal_frac_outside=float((err > literal).sum()) / n,
                 literal_worst=float((err / literal).max()) if err.numel() else 0.0,
                 scaled_frac_outside=float((err > bound).sum()) / n,
                 scaled_worst=float((err / bound).max()) if err.numel() else 0.0)
    return stats, err, bound


def _record(what: str, stats: dict):
    test = os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0]
    PARITY_REPORT.append(dict(test=test, what=what, **stats))


def record_closeness(got, ref, rtol, atol, what, branch=None, scale_atol=True):
    """Statistics only, no assertion (used for the stock-PyTorch noise-floor twin)."""
    stats, _, _ = closeness(got, ref, rtol, atol, branch=branch, scale_atol=scale_atol)
    _record(what, stats)
    return stats


def assert_close(got: torch.Tensor, ref: torch.Tensor, rtol: float, atol: float, what: str = "", scale_atol=False,
                 branch: torch.Tensor = None, outlier_frac: float = 0.0, outlier_cap: float = 4.0):
    """|got - ref| <= atol * max(1, S) + rtol * max(|ref|, |branch|, S), elementwise.

    With S = 0 and no branch this is torch.allclose's rule.  The two extensions check an element at the scale
    of the computation that produced it rather than at the size it happens to end up with:

    ``scale_atol``: S = rms of the GEMM-produced tensor (``branch`` if given, else ``ref``).  A matrix product
    accumulates hundreds to tens of thousands of products; its rounding noise is proportional to the rms of
    the accumulated sums, also for the elements whose terms cancel to ~0.

    ``branch``: where a residual is added exactly (out = x + branch, dx = g + branch'), the reference value of
    the computed branch; an output that cancels against the residual is checked at the branch's size.

    ``outlier_frac``: up to this fraction of the elements may exceed the bound, none by more than ``outlier_cap``
    times.  Used only where the recorded noise floor of stock PyTorch arithmetic shows the same tails."""
    stats, err, bound = closeness(got, ref, rtol, atol, branch=branch, scale_atol=scale_atol)
    _record(what, stats)
    ref = ref.detach().to(device=err.device, dtype=err.dtype)
    bad = err > bound
    if outlier_frac > 0 and int(bad.sum()) <= outlier_frac * bad.numel() and not (err > outlier_cap * bound).any():
        return stats
    if bad.any():
        worst = int((err - bound).argmax())
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.numel()} elements out of tolerance (rtol {rtol}, atol {atol}, "
            f"S {stats['S']:.3g}); worst |err| {float(err.flatten()[worst]):.4g} at ref {float(ref.flatten()[worst]):.4g} "
            f"(bound {float(bound.flatten()[worst]):.4g}); max |err| {float(err.max()):.4g}, "
            f"max |ref| {float(ref.abs().max()):.4g}")
    return stats


def pytest_sessionfinish(session, exitstatus):
    if not PARITY_REPORT or not torch.cuda.is_available():
        return
    out_dir = ROOT / "gpurun_out"
    try:
        out_dir.mkdir(exist_ok=True)
        with open(out_dir / "parity_report.json", "w") as f:
            json.dump(PARITY_REPORT, f, indent=0)
    except OSError:
        pass


@pytest.fixture
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)
