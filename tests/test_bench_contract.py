"""Host-side checks of bench.py: algorithmic work per token and the shape of the JSON line of the CPU arm."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_algorithmic_flops_per_token():
    sys.path.insert(0, str(ROOT))
    import bench
    # dense gated FFN: 18 * H * I (6 forward, 12 backward)
    assert bench.flops_per_token(8192, 32768) == 18 * 8192 * 32768
    assert bench.flops_per_token(768, 3072) == 18 * 768 * 3072
    # pixelfly 128-blocks + rank-128 low rank: 6 * (nonzero weights of both projections + low-rank factors)
    wl = bench.WORKLOADS["pixelfly_bf16_h4096"]
    assert bench.flops_per_token(wl["hidden"], wl["inter"], wl) == 6 * (25165824 + 12582912 + 4718592 + 2621440)


def test_reference_arm_prints_one_json_line():
    """`bench.py --impl reference` (the CPU arm): one JSON line with the contract's keys, no GPU needed."""
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "dense_fp32_h768",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["value"] > 0
    # the reference's own LeanFFN where its mirror (oracle/_ref) exists, the CPU port otherwise
    mirror = (ROOT / "oracle" / "_ref" / "lean_transformer" / "ffn.py").is_file()
    assert line["cpu_baseline"]["kind"] == ("reference" if mirror else "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
