"""Worker of tests/test_gpu_multi.py: one process per GPU (launched with torch.distributed.run).  Every rank runs a
LeanFFN step on its token shard and exchanges gradients twice: with NCCL all-reduces (``GradSync``) and with the
reduce-scatter fused into the weight-gradient GEMMs (``ScatteredGradReducer``).  Both must agree with each other and
with the gradients of the whole batch computed on one GPU."""
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from lean_transformer_b200 import LeanFFN, dist as ldist, ffn as lffn, ops  # noqa: E402
from lean_transformer_b200.blocksparse.linear import set_weight_grad_reducer  # noqa: E402


def scenario(device, rank, world, mixed):
    """``mixed``: fp32 parameters and residual stream with bf16 compute (fp32 gradients, fp32 atomics in the fused
    exchange); otherwise bf16 everywhere."""
    hidden, inter, tokens = 512, 1024, 1024 * world
    torch.manual_seed(0)
    ffn = LeanFFN(hidden, inter, gated=True).to(device)  # same seed: same weights on every rank
    if not mixed:
        ffn = ffn.to(torch.bfloat16)
    _forward = ffn.forward

    def forward(x):
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=mixed):
            return _forward(x)

    in_dtype = torch.float32 if mixed else torch.bfloat16
    gen = torch.Generator(device=device).manual_seed(1)
    x_all = torch.randn(tokens, hidden, device=device, generator=gen).to(in_dtype)
    g_all = torch.randn(tokens, hidden, device=device, generator=gen).bfloat16()
    start, count = ldist.shard_tokens(tokens, world, rank)
    x, g = x_all[start:start + count], g_all[start:start + count]
    names = dict(ffn.named_parameters())
    big = {"i2h": ffn.i2h_proj.weight, "h2o": ffn.h2o_proj.weight}

    def grads():
        return {k: p.grad.detach().float().clone() for k, p in names.items()}

    def clear():
        for p in names.values():
            p.grad = None

    # whole batch on this GPU
    clear()
    forward(x_all.clone().requires_grad_(True)).backward(g_all)
    full = grads()

    # NCCL exchange
    clear()
    sync = ldist.GradSync(params=list(ffn.parameters()))
    lffn.set_grad_ready_hook(sync.reduce)
    forward(x.clone().requires_grad_(True)).backward(g)
    sync.finish()
    nccl = grads()
    lffn.set_grad_ready_hook(None)

    # fused reduce-scatter for the two weights, NCCL for the small tensors; two steps in a row
    reducer = ldist.ScatteredGradReducer(big)
    set_weight_grad_reducer(reducer)
    sync = ldist.GradSync(params=list(ffn.parameters()))
    lffn.set_grad_ready_hook(sync.reduce)
    fused = None
    for _ in range(2):
        clear()
        reducer.begin_step()
        forward(x.clone().requires_grad_(True)).backward(g)
        sync.finish()
        assert reducer.finish() == 2
        fused = grads()
    set_weight_grad_reducer(None)
    lffn.set_grad_ready_hook(None)
    torch.cuda.synchronize()
    ops.check_device_status(device)

    if os.environ.get("LEANFFN_TEST_VERBOSE"):
        for k in full:
            print(rank, k, "full", full[k].flatten()[:4].tolist(), "nccl", nccl[k].flatten()[:4].tolist(), "fused",
                  fused[k].flatten()[:4].tolist(), flush=True)
    report = {}
    for k in full:
        scale = full[k].pow(2).mean().sqrt().item()
        report[k] = dict(rms=scale,
                         nccl_vs_full=(nccl[k] - full[k]).abs().max().item() / scale,
                         fused_vs_full=(fused[k] - full[k]).abs().max().item() / scale,
                         fused_vs_nccl=(fused[k] - nccl[k]).abs().max().item() / scale)
    return report


def main():
    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    report = {}
    for mixed in (False, True):
        for key, value in scenario(device, rank, world, mixed).items():
            report[("mixed." if mixed else "bf16.") + key] = value
    gathered = [None] * world
    dist.all_gather_object(gathered, report)
    if rank == 0:
        print("MULTI_GPU_REPORT " + json.dumps(gathered), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
