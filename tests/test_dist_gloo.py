"""Token partition + gradient all-reduce on 2 CPU ranks (gloo): the multi-GPU host logic without GPUs.

Each rank computes the gradients of its token shard with the CPU oracle (a stand-in for the CUDA backward, which
produces the same quantities), hands them to GradSync in the order the backward produces them, and the reduced
result must equal the full-batch gradients.  Failure handling is exercised on the host: a rank that raises
before the collective must surface as an error on the other rank instead of a hang.
"""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem():
    from helpers import random_params
    params = random_params(32, 64, True, seed=0, std=0.2, bias_std=0.1, dtype=torch.float64)
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(50, 32, generator=gen, dtype=torch.float64)  # 50 tokens: uneven over 4 ranks, even over 2
    g = torch.randn(50, 32, generator=gen, dtype=torch.float64)
    return params, x, g


def _worker(rank, world, port, mode, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=__import__("datetime").timedelta(seconds=20))
    try:
        from lean_transformer_b200 import dist as ldist
        from oracle import leanffn_oracle as O
        params, x, g = _problem()
        start, count = ldist.shard_tokens(x.shape[0], world, rank)
        if mode == "raise" and rank == 1:
            raise RuntimeError("injected failure before the collective")
        _, grads = O.leanffn_step(x[start:start + count], g[start:start + count], params, gated=True)
        sync = ldist.GradSync(wire_dtype=torch.float32 if mode == "wire" else None)
        order = ["h2o_weight", "h2o_bias", "i2h_weight", "i2h_bias", "ln_weight", "ln_bias"]  # backward's order
        for name in order:
            sync.reduce(name, grads[name])
        assert sync.finish() == len(order) and sync.reduced_names == order
        torch.save({k: grads[k] for k in order}, os.path.join(result_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["plain", "wire"])
def test_token_partition_and_gradient_allreduce(tmp_path, mode):
    from lean_transformer_b200 import dist as ldist
    from oracle import leanffn_oracle as O
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), mode, str(tmp_path)), nprocs=world, join=True)
    params, x, g = _problem()
    _, full = O.leanffn_step(x, g, params, gated=True)
    for rank in range(world):
        got = torch.load(tmp_path / f"rank{rank}.pt")
        for name, value in got.items():
            tol = 1e-5 if mode == "wire" else 1e-12  # fp32 wire format rounds once
            assert torch.allclose(value, full[name], rtol=tol, atol=tol), (rank, name)


def test_shard_tokens_covers_everything():
    from lean_transformer_b200 import dist as ldist
    for total, world in [(65536, 8), (50, 4), (7, 8), (0, 2)]:
        spans = [ldist.shard_tokens(total, world, r) for r in range(world)]
        assert spans[0][0] == 0 and sum(c for _, c in spans) == total
        assert all(spans[i][0] + spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        ldist.shard_tokens(8, 2, 2)


def _owner_worker(rank, world, port, result_dir, bucket_elems):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=__import__("datetime").timedelta(seconds=20))
    try:
        from lean_transformer_b200 import dist as ldist
        weight = torch.nn.Parameter(torch.zeros(6, 4))
        bias = torch.nn.Parameter(torch.zeros(6, dtype=torch.float64))  # gradient arrives in another dtype
        stranger = torch.zeros(3, 4)                                    # not among the registered parameters
        sync = ldist.GradSync(params=[weight, bias], wire_dtype=torch.float32, bucket_elems=bucket_elems)
        g_w = torch.full((6, 4), float(rank + 1))
        g_b = torch.full((6,), float(10 * (rank + 1)))
        g_s = torch.ones(3, 4)
        # the calling convention of the backward: (name, gradient, parameter) -> taken?
        assert sync.reduce("i2h_weight", g_w, weight.detach()) is True     # found by storage, not by object
        assert sync.reduce("i2h_bias", g_b, bias) is True
        assert sync.reduce("i2h_lowrank_first", g_s, stranger) is False   # left to autograd, unreduced
        assert weight.grad is None and bias.grad is None                  # nothing is delivered before finish()
        assert sync.finish() == 2 and sync.unclaimed == ["i2h_lowrank_first"]
        total = sum(range(1, world + 1))
        assert torch.equal(weight.grad, torch.full((6, 4), float(total)))
        assert bias.grad.dtype == torch.float64 and torch.equal(bias.grad, torch.full((6,), 10.0 * total, dtype=torch.float64))
        assert torch.equal(g_s, torch.ones(3, 4))
        # a second backward before the optimizer step accumulates
        assert sync.reduce("i2h_weight", torch.ones(6, 4), weight) is True
        sync.finish()
        assert torch.equal(weight.grad, torch.full((6, 4), float(total + world)))
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("bucket_elems", [0, 1 << 18])  # one all-reduce per tensor / one for all small tensors
def test_grad_sync_takes_ownership_of_hooked_gradients(tmp_path, bucket_elems):
    """GradSync as the gradient-ready callback: it keeps the gradient, reduces it and delivers ``param.grad`` in
    ``finish()`` (autograd never touches a tensor that a collective is still writing)."""
    mp.spawn(_owner_worker, args=(2, _free_port(), str(tmp_path), bucket_elems), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_failed_rank_surfaces_as_error_not_hang(tmp_path):
    """A rank that dies before the collective: the job ends with an exception within the group timeout."""
    with pytest.raises(Exception):
        mp.spawn(_worker, args=(2, _free_port(), "raise", str(tmp_path)), nprocs=2, join=True)


def test_dropout_mask_is_partition_invariant():
    """With elem_offset = first_row * hidden, a rank's mask equals the matching rows of the global mask."""
    from lean_transformer_b200 import dist as ldist
    from oracle import leanffn_oracle as O
    tokens, hidden, p, seed = 37, 24, 0.3, 11
    full = O.dropout_keep_mask(tokens * hidden, p, seed, 0).reshape(tokens, hidden)
    for rank in range(4):
        start, count = ldist.shard_tokens(tokens, 4, rank)
        part = O.dropout_keep_mask(count * hidden, p, seed, start * hidden).reshape(count, hidden)
        assert (part == full[start:start + count]).all()


@pytest.mark.parametrize("world,rows,cols", [(2, 512, 24), (4, 1024, 8), (8, 2048, 16), (8, 768, 8), (3, 1280, 4)])
def test_scattered_reduction_plan_sums_every_row_once(world, rows, cols):
    """Host logic of the fused reduce-scatter: emulate, with numpy, the epilogue's ownership rule (row blocks dealt
    round-robin), then the strided hand-out copies; every replica must end up holding the sum over ranks."""
    import numpy as np
    from lean_transformer_b200 import dist as ldist
    shift = ldist.ScatteredGradReducer.BLOCK_SHIFT
    rng = np.random.default_rng(0)
    contributions = rng.integers(-8, 8, size=(world, rows, cols)).astype(np.float32)
    replicas = np.full((world, rows, cols), np.nan, dtype=np.float32)
    for rank in range(world):  # begin_step: owned blocks are zeroed
        for b in ldist.owned_row_blocks(rows, world, rank, shift):
            replicas[rank, b << shift:(b + 1) << shift] = 0
    for rank in range(world):  # the GEMM epilogue of every rank: add each row into its owner's replica
        for r in range(rows):
            owner = (r >> shift) % world
            replicas[owner, r] += contributions[rank, r]
    flat = replicas.reshape(world, -1).view(np.uint8)
    for rank in range(world):  # hand-out: strided copy of the owned blocks to every other replica
        start, pitch, width, height = ldist.handout_plan(rows, cols, 4, world, rank, shift)
        for peer in range(world):
            if peer == rank:
                continue
            for h in range(height):
                lo = start + h * pitch
                flat[peer, lo:lo + width] = flat[rank, lo:lo + width]
    total = contributions.sum(0)
    for rank in range(world):
        assert np.array_equal(replicas[rank], total), rank
