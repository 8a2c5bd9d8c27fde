"""Gradient exchange across GPUs (needs at least two): NCCL all-reduce and the reduce-scatter fused into the
weight-gradient GEMMs against the single-GPU whole-batch gradients."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]

# Gradients are sums over tokens of bf16 products; the exchanged sum adds one more bf16 rounding per rank.
# Bound on max |difference| relative to the rms of the gradient tensor.
REL_TO_RMS = 0.08


@pytest.mark.gpu
@pytest.mark.timeout(600)
def test_fused_reduce_scatter_matches_all_reduce_and_whole_batch():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                           "--master-addr", "127.0.0.1", "--master-port", "29741", str(ROOT / "tests" / "multi_gpu_worker.py")],
                          capture_output=True, text=True, env=env, timeout=540)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("MULTI_GPU_REPORT ")][-1]
    reports = json.loads(line[len("MULTI_GPU_REPORT "):])
    assert len(reports) == world
    for report in reports:
        for name, r in report.items():
            assert r["nccl_vs_full"] < REL_TO_RMS, (name, r)
            assert r["fused_vs_full"] < REL_TO_RMS, (name, r)
            assert r["fused_vs_nccl"] < REL_TO_RMS, (name, r)
