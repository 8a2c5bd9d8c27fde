"""LeanFFN forward+backward throughput (tokens/s) on 1/2/4/8 B200s.

    python bench.py --gpus 1 --steps K --warmup W                  # this repository's CUDA path
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...                            # CPU baseline arm (host cores)

One JSON line is printed by rank 0.  Workloads (synthetic data, random-init weights of the named shape):
  dense_bf16_h8192   hidden 8192, intermediate 32768, GeGLU, bf16, 65536 tokens in total, no dropout; tokens are
                     partitioned across the N ranks and weight gradients are all-reduced (default: it is the
                     configuration the 1/2/4/8-GPU metric is quoted on and it fits one GPU)
  mixed_bf16_h1024   hidden 1024, intermediate 4096, GeGLU, 16 x 1024 tokens per rank, fp32 parameters and
                     residual stream with bf16 compute, dropout 0.1
  pixelfly_bf16_h4096  hidden 4096, intermediate 16384, both projections pixelfly block-sparse (128-blocks) plus a
                     rank-128 low-rank term, bf16, 65536 tokens per rank
  dense_fp32_h768    hidden 768, intermediate 3072, 8 x 512 tokens, fp32 end to end (the reference's CPU-runnable
                     case): products run as three TF32 tensor-core products with fp32 accuracy
  attention_bf16_h768  (other_workloads only, or --attention-only) the attention core of that model alone: rotary +
                     causal attention, 32 x 2048 tokens, 16 heads of 48, forward + backward
  leangpt_bf16_h768  (other_workloads only) the reference's 12-layer LeanGPT, 32 x 2048 tokens, autocast bf16, with the
                     reference's modules, with its FFN / linear modules swapped for this package's, and with its
                     attention cores swapped too
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    "dense_bf16_h8192": dict(hidden=8192, inter=32768, total_tokens=65536, scaling="strong", dropout=0.0, mixed=False),
    "mixed_bf16_h1024": dict(hidden=1024, inter=4096, tokens_per_rank=16384, scaling="weak", dropout=0.1, mixed=True),
    "dense_fp32_h768": dict(hidden=768, inter=3072, tokens_per_rank=4096, scaling="weak", dropout=0.0, mixed=False,
                            fp32=True),
    "pixelfly_bf16_h4096": dict(hidden=4096, inter=16384, tokens_per_rank=65536, scaling="weak", dropout=0.0, mixed=False,
                                layout="pixelfly(block_size=128)", lowrank=128),
}


def flops_per_token(hidden, inter, wl=None):
    if wl is not None and wl.get("layout"):
        # block-sparse + low rank: 6 * (nonzero weights of both projections + rank * (in + out) of both)
        import math
        block, rank = 128, wl["lowrank"]
        m1, m2 = min(2 * inter, hidden) // block, min(inter, hidden) // block
        per_row1, per_row2 = (int(math.log2(m1)) + 1) * (hidden // block) // m1, (int(math.log2(m2)) + 1) * (inter // block) // m2
        nnz1, nnz2 = per_row1 * (2 * inter // block), per_row2 * (hidden // block)
        return 6.0 * ((nnz1 + nnz2) * block * block + rank * (hidden + 2 * inter) + rank * (inter + hidden))
    return 18.0 * hidden * inter  # gated FFN: forward 6*H*I, backward 12*H*I


def captured_traffic(name, tokens):
    """DRAM bytes (read + written) per GEMM launch for `tokens` tokens on this GPU, from the ncu counter captures
    recorded per workload in profiles/dram_traffic.json (captured at a smaller token count under the capture-size
    rule and scaled by tokens: operand re-reads and activation traffic both grow with the token count).  None for a
    workload without a capture."""
    path = ROOT / "profiles" / "dram_traffic.json"
    if not path.exists():
        return None, None
    entry = json.loads(path.read_text()).get(name)
    if not entry:
        return None, None
    per_launch = entry["dram_bytes_total"] / entry["gemm_launches"] * tokens / entry["tokens_captured"]
    note = (f"ncu dram__bytes_read.sum + dram__bytes_write.sum over {entry['gemm_launches']} GEMM launches at "
            f"{entry['tokens_captured']} tokens ({entry['source']}), scaled by tokens to {tokens}; bytes per launch")
    return per_launch, note


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return dict(bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"], hbm=d["hbm_gbs"], source="measured")
    return dict(bf16=1590.0, bf16_sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, max_clock, reasons = [], None, set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6 or not parts[0].isdigit():
                continue
            clocks.append(int(parts[0]))
            max_clock = int(parts[1]) if parts[1].isdigit() else max_clock
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return dict(sm_mhz=clocks[len(clocks) // 2] if clocks else None, sm_max_mhz=max_clock, reasons=sorted(reasons),
                    samples=len(clocks))


# ------------------------------------------------------------------------------------------------------
# CPU baseline / reference arm: the oracle (a CPU restatement of the reference's algorithm) on host cores
# ------------------------------------------------------------------------------------------------------
def reference_step_time(hidden, inter, sample_tokens, steps, warmup, threads, wl=None):
    """Median fwd+bwd seconds of the REFERENCE's own LeanFFN (lean_transformer/ffn.py, ffn_custom_grad=True, fp32) on
    the host cores, or None where its mirror (oracle/_ref, made by oracle/build_ref.py) is absent."""
    from oracle import ref_harness

    ref = ref_harness.import_reference()
    if ref is None:
        return None
    torch.set_num_threads(threads)
    torch.manual_seed(0)
    i2h = h2o = None
    if wl is not None and wl.get("layout"):
        GM, GL = ref.linear.GeneralizedMatrix, ref.linear.GeneralizedLinear
        i2h = GL(GM(hidden, 2 * inter, wl["layout"], wl["lowrank"]))
        h2o = GL(GM(inter, hidden, wl["layout"], wl["lowrank"]))
    ffn = ref.ffn.LeanFFN(hidden, inter, gated=True, dropout=0.0, i2h_proj=i2h, h2o_proj=h2o, ffn_custom_grad=True)
    with torch.no_grad():
        for proj in (ffn.i2h_proj, ffn.h2o_proj):
            proj.weight.normal_(0.0, 0.02)
            proj.bias.zero_()
    x = torch.randn(1, sample_tokens, hidden)
    g = torch.randn(1, sample_tokens, hidden)
    times = []
    for i in range(warmup + steps):
        for p in ffn.parameters():
            p.grad = None
        xi = x.clone().requires_grad_(True)
        t0 = time.perf_counter()
        ffn(xi).backward(g)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    times.sort()
    return times[len(times) // 2]


def cpu_baseline_time(hidden, inter, sample_tokens, steps, warmup, threads, wl=None):
    """(seconds per step, kind): the reference's own LeanFFN where it can be imported, else the CPU port."""
    try:
        t = reference_step_time(hidden, inter, sample_tokens, steps, warmup, threads, wl)
    except Exception as e:  # an import or API problem of the mirrored package must not take the bench down
        print(f"reference LeanFFN unavailable ({type(e).__name__}: {e}); timing the CPU port", file=sys.stderr)
        t = None
    if t is not None:
        return t, "reference"
    return cpu_step_time(hidden, inter, sample_tokens, steps, warmup, threads, wl), "port"


def cpu_step_time(hidden, inter, sample_tokens, steps, warmup, threads, wl=None):
    from oracle import leanffn_oracle as O

    torch.set_num_threads(threads)
    gen = torch.Generator().manual_seed(0)
    rn = lambda *s: torch.randn(*s, generator=gen)  # noqa: E731
    params = dict(ln_weight=torch.ones(hidden), ln_bias=torch.zeros(hidden), i2h_bias=torch.zeros(2 * inter),
                  h2o_bias=torch.zeros(hidden))
    if wl is not None and wl.get("layout"):
        from lean_transformer_b200.blocksparse import layout as LY
        for prefix, fin, fout in (("i2h", hidden, 2 * inter), ("h2o", inter, hidden)):
            fwd, bwd = LY.get_indices_from_layout(LY.get_blocksparse_layout(fout, fin, wl["layout"]))
            block = fin // bwd.shape[0]
            params.update({f"{prefix}_weight": 0.02 * rn(fin, bwd.shape[1], block),
                           f"{prefix}_lowrank_first": 0.02 * rn(wl["lowrank"], fin),
                           f"{prefix}_lowrank_second": 0.02 * rn(fout, wl["lowrank"]),
                           f"{prefix}_forward_indices": fwd, f"{prefix}_backward_indices": bwd})
    else:
        params.update(i2h_weight=0.02 * rn(2 * inter, hidden), h2o_weight=0.02 * rn(hidden, inter))
    x, g = rn(sample_tokens, hidden), rn(sample_tokens, hidden)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.leanffn_step(x, g, params, gated=True)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    times.sort()
    return times[len(times) // 2]


def host_threads():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference_arm(args, wl, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    hidden, inter = wl["hidden"], wl["inter"]
    threads = host_threads()
    sample = 512 if hidden >= 4096 else 4096
    step_s, kind = cpu_baseline_time(hidden, inter, sample, args.steps, args.warmup, threads, wl)
    value = sample / step_s
    what = ("the reference's own LeanFFN (lean_transformer/ffn.py, ffn_custom_grad=True)" if kind == "reference"
            else "CPU restatement of the reference's LeanFFN")
    sample_desc = (f"{sample} tokens of the {name} workload per step (fp32, GeGLU, hidden {hidden}, intermediate {inter}), "
                   f"{what}, median of {args.steps} steps after {args.warmup} warm-up")
    line = dict(impl="reference", metric="LeanFFN fwd+bwd tokens/sec", value=value, unit="tokens/s", n_gpus=args.gpus,
                steps=args.steps, warmup=args.warmup, ms_per_step=step_s * 1e3, higher_is_better=True,
                scaling=wl["scaling"], vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=name, hidden=hidden, intermediate=inter, gated=True, sample_tokens=sample,
                            parallelism="host cores only"),
                cpu_baseline=dict(value=value, unit="tokens/s", cores=threads, kind=kind, sample=sample_desc),
                e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gflops=value * flops_per_token(hidden, inter, wl) / 1e9)
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------
# this repository's arm
# ------------------------------------------------------------------------------------------------------
def build_module(wl, device):
    import lean_transformer_b200 as L

    torch.manual_seed(0)
    i2h = h2o = None
    if wl.get("layout"):
        from lean_transformer_b200.blocksparse.linear import GeneralizedLinear, GeneralizedMatrix
        i2h = GeneralizedLinear(GeneralizedMatrix(wl["hidden"], 2 * wl["inter"], wl["layout"], wl["lowrank"]))
        h2o = GeneralizedLinear(GeneralizedMatrix(wl["inter"], wl["hidden"], wl["layout"], wl["lowrank"]))
    ffn = L.LeanFFN(wl["hidden"], wl["inter"], gated=True, dropout=wl["dropout"], i2h_proj=i2h, h2o_proj=h2o)
    with torch.no_grad():
        for proj in (ffn.i2h_proj, ffn.h2o_proj):
            proj.bias.zero_()
    ffn = ffn.to(device)
    with torch.no_grad():  # weights ~ N(0, 0.02), generated on the device (identical on every rank: same seed)
        gen = torch.Generator(device=device).manual_seed(0)
        for proj in (ffn.i2h_proj, ffn.h2o_proj):
            proj.weight.normal_(0.0, 0.02, generator=gen)
            if wl.get("layout"):
                proj.matrix.lowrank_first.normal_(0.0, 0.02, generator=gen)
                proj.matrix.lowrank_second.normal_(0.0, 0.02, generator=gen)
    if not wl["mixed"] and not wl.get("fp32"):
        ffn = ffn.bfloat16()
    return ffn.train()


def run_ours(args, wl, name):
    import torch.distributed as dist

    import lean_transformer_b200 as L
    from lean_transformer_b200 import dist as ldist
    from lean_transformer_b200 import ffn as lffn
    from lean_transformer_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    hidden, inter = wl["hidden"], wl["inter"]
    start = 0
    if wl["scaling"] == "strong":
        start, tokens = ldist.shard_tokens(wl["total_tokens"], world, rank)
        total_tokens = wl["total_tokens"]
    else:
        tokens = wl["tokens_per_rank"]
        total_tokens = tokens * world
    in_dtype = torch.float32 if (wl["mixed"] or wl.get("fp32")) else torch.bfloat16
    ffn = build_module(wl, device)
    params = [p for p in ffn.parameters()]
    # Inputs are a function of the GLOBAL token index: chunk c of the batch (1/8 of the strong-scaling batch, one
    # rank's shard otherwise) is drawn from a generator seeded with 1000 + c, and every rank draws the chunks of its
    # own shard.  The strong-scaling batch is therefore the same tensor at every N, and so are its gradients.
    first_token = start if wl["scaling"] == "strong" else rank * tokens
    chunk = max(1, wl["total_tokens"] // 8) if wl["scaling"] == "strong" else tokens
    if first_token % chunk or tokens % chunk:
        chunk = tokens  # shards that do not line up with the chunks (odd --tokens overrides): one chunk per rank
    g_dtype = torch.float32 if wl.get("fp32") else torch.bfloat16
    x_parts, g_parts = [], []
    for c in range(first_token // chunk, (first_token + tokens) // chunk):
        gen = torch.Generator(device=device).manual_seed(1000 + c)
        x_parts.append(torch.randn(chunk, hidden, device=device, generator=gen).to(in_dtype))
        g_parts.append(torch.randn(chunk, hidden, device=device, generator=gen).to(g_dtype))
    x_dev, g_dev = torch.cat(x_parts), torch.cat(g_parts)
    del x_parts, g_parts
    sync = (ldist.GradSync(wire_dtype=torch.bfloat16, comm_sms=args.comm_sms if args.grad_exchange == "nccl" else None,
                           measure_tail=True, params=params) if world > 1 else None)
    reducer = None
    exchange_note = args.grad_exchange
    if world > 1:
        lffn.set_grad_ready_hook(sync.reduce)
        if args.grad_exchange == "fused" and not wl.get("layout"):
            # the two dense weight gradients are reduce-scattered inside their GEMMs; NCCL keeps the small tensors
            from lean_transformer_b200.blocksparse.linear import set_weight_grad_reducer
            try:
                reducer = ldist.ScatteredGradReducer({"i2h_weight": ffn.i2h_proj.weight, "h2o_weight": ffn.h2o_proj.weight})
                set_weight_grad_reducer(reducer)
            except Exception as e:  # no peer-mapped memory on this machine: every gradient goes through NCCL
                exchange_note = f"nccl (peer-mapped buffer unavailable: {type(e).__name__})"
                sync.comm_sms = args.comm_sms
        elif args.grad_exchange == "fused":
            exchange_note = "nccl (block-sparse weights)"
            sync.comm_sms = args.comm_sms

    from lean_transformer_b200.blocksparse.linear import clear_cast_cache

    def step(x, g):
        if wl["mixed"]:
            clear_cast_cache()  # a real step updates the fp32 masters, so their bf16 copies are rebuilt every step
        for p in params:
            p.grad = None
        if reducer is not None:
            reducer.begin_step()
        x = x.requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=wl["mixed"]):
            out = ffn(x)
        out.backward(g)
        if sync is not None:
            sync.finish()
        if reducer is not None:
            reducer.finish()
        return out, x.grad

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing (value) ---------------------------------------------------------------
    for _ in range(args.warmup):
        step(x_dev.detach(), g_dev)
    L.check_device_status(device)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    launches0 = ops.launch_count
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sync is not None:
        torch.cuda.synchronize()
        sync.tail_ms()  # drop the warm-up records
    with ops.GemmTimer() as timer:
        t_start.record()
        for _ in range(args.steps):
            step(x_dev.detach(), g_dev)
        t_end.record()
        barrier()
    elapsed = torch.tensor([t_start.elapsed_time(t_end) * 1e-3], device=device, dtype=torch.float64)
    clocks = sampler.stop() if rank == 0 else None
    launches = ops.launch_count - launches0
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    seconds = float(elapsed.item())
    gemm_flops, gemm_seconds, gemm_launches = timer.summary()
    tails = sync.tail_ms() if sync is not None else []
    exposed_ms = sum(tails) / len(tails) if tails else 0.0
    L.check_device_status(device)

    if args.skip_e2e:
        if rank == 0:
            print(json.dumps(dict(profiling_run=True, workload=name, tokens=total_tokens, ms_per_step=seconds / args.steps * 1e3,
                                  exposed_allreduce_ms=exposed_ms, comm_sms=args.comm_sms, grad_exchange=exchange_note,
                                  gemm_tflops=gemm_flops / gemm_seconds / 1e12 if gemm_seconds else None)), flush=True)
        if world > 1:
            lffn.set_grad_ready_hook(None)
            if reducer is not None:
                set_weight_grad_reducer(None)
            dist.destroy_process_group()
        return

    # ---- end-to-end through the module API with host buffers (e2e) --------------------------------------
    # ---- N-invariant checksums of one more (untimed) step on the resident inputs --------------------------------
    out, dx = step(x_dev.detach(), g_dev)
    sums = torch.stack([(out.double().reshape(-1) * g_dev.double().reshape(-1)).sum(), dx.double().abs().sum()])
    if world > 1:
        dist.all_reduce(sums)  # partial sums over this rank's tokens -> whole batch
    sums = sums.detach()
    checksum = dict(sum_out_dot_g=float(sums[0]), sum_abs_grad_input=float(sums[1]),
                    sum_abs_grad_i2h_weight=float(ffn.i2h_proj.weight.grad.double().abs().sum()),
                    sum_abs_grad_h2o_weight=float(ffn.h2o_proj.weight.grad.double().abs().sum()),
                    sum_abs_grad_i2h_bias=float(ffn.i2h_proj.bias.grad.double().abs().sum()),
                    note=("computed on rank 0 after the gradient exchange; inputs are a function of the global token "
                          "index, so with strong scaling every value is the same at every N up to bf16 summation "
                          "order"))
    out_dtype, dx_dtype, out_shape = out.dtype, dx.dtype, tuple(out.shape)
    del out, dx, sums

    x_host = x_dev.detach().cpu().pin_memory()
    g_host = g_dev.cpu().pin_memory()
    copy_stream = torch.cuda.Stream(device)
    bufs = [(torch.empty_like(x_dev), torch.empty_like(g_dev)) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    # the step's results (output and input gradient) return to pinned host buffers, double-buffered like the uploads
    out_host = [torch.empty(out_shape, dtype=out_dtype).pin_memory() for _ in range(2)]
    dx_host = [torch.empty(out_shape, dtype=dx_dtype).pin_memory() for _ in range(2)]
    produced = [torch.cuda.Event() for _ in range(2)]
    drained = [torch.cuda.Event() for _ in range(2)]

    def upload(i):
        slot = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            bufs[slot][0].copy_(x_host, non_blocking=True)
            bufs[slot][1].copy_(g_host, non_blocking=True)
            ready[slot].record(copy_stream)

    def e2e_loop(n):
        losses = []
        main = torch.cuda.current_stream(device)
        for slot in range(2):
            consumed[slot].record(main)
            drained[slot].record(copy_stream)
        upload(0)
        for i in range(n):
            slot = i % 2
            if i + 1 < n:
                upload(i + 1)  # the next step's inputs cross PCIe while this step computes
            main.wait_event(ready[slot])
            xb, gb = bufs[slot]
            out, dx = step(xb.detach(), gb)
            loss = torch.dot(out.detach().reshape(-1), gb.reshape(-1).to(out.dtype))  # loss = sum(out * g)
            consumed[slot].record(main)
            produced[slot].record(main)
            with torch.cuda.stream(copy_stream):  # results cross PCIe underneath the next step
                copy_stream.wait_event(produced[slot])
                out_host[slot].copy_(out.detach(), non_blocking=True)
                dx_host[slot].copy_(dx, non_blocking=True)
                drained[slot].record(copy_stream)
            out.record_stream(copy_stream)
            dx.record_stream(copy_stream)
            losses.append(float(loss.item()))  # device -> host read of the step's loss
        for slot in range(2):
            main.wait_event(drained[slot])  # the timed region ends when the last results are on the host
        return losses

    e2e_loop(min(2, args.warmup))
    barrier()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    losses = e2e_loop(args.steps)
    e_end.record()
    barrier()
    e_elapsed = torch.tensor([e_start.elapsed_time(e_end) * 1e-3], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e_elapsed, op=dist.ReduceOp.MAX)
    e_seconds = float(e_elapsed.item())
    L.check_device_status(device)

    out_host_bytes = sum(t.numel() * t.element_size() for t in (out_host[0], dx_host[0]))
    extra = {}
    if rank == 0 and world == 1 and args.extra_workload:
        del bufs, out_host, dx_host
        x_dev = g_dev = None
        ffn = None
        params = []
        torch.cuda.empty_cache()
        for other in [w.strip() for w in args.extra_workload.split(",") if w.strip()]:
            if other != name and other in WORKLOADS:
                extra[other] = quick_measure(WORKLOADS[other], device, args, other)
            elif other == "attention_bf16_h768":
                extra[other] = attention_measure(device)
                torch.cuda.empty_cache()
            elif other == "leangpt_bf16_h768":
                try:
                    extra[other] = leangpt_measure(device)
                except Exception as e:  # the mirrored reference model must not take the headline number down
                    extra[other] = dict(unavailable=f"{type(e).__name__}: {e}")
                torch.cuda.empty_cache()

    if world > 1:
        lffn.set_grad_ready_hook(None)
        if reducer is not None:
            set_weight_grad_reducer(None)
        dist.destroy_process_group()
    if rank != 0:
        return

    peaks = load_peaks()
    tokens_per_s = total_tokens * args.steps / seconds
    tflops = tokens_per_s * flops_per_token(hidden, inter, wl) / 1e12
    achieved = gemm_flops / gemm_seconds / 1e12 if gemm_seconds > 0 else None
    traffic, traffic_note = captured_traffic(name, tokens)
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = host_threads()
        sample = 512 if hidden >= 4096 else 4096
        cpu_s, kind = cpu_baseline_time(hidden, inter, sample, 3, 1, threads, wl)
        cpu = dict(value=sample / cpu_s, unit="tokens/s", cores=threads, kind=kind,
                   sample=f"{sample} tokens of the {name} workload per step in fp32 on the host cores ("
                          + ("the reference's own LeanFFN, lean_transformer/ffn.py, ffn_custom_grad=True"
                             if kind == "reference" else "CPU restatement of the reference's LeanFFN")
                          + "), median of 3 steps after 1 warm-up")
    line = dict(
        metric="LeanFFN fwd+bwd tokens/sec", value=tokens_per_s, unit="tokens/s", n_gpus=world, steps=args.steps,
        warmup=args.warmup, ms_per_step=seconds / args.steps * 1e3, higher_is_better=True, scaling=wl["scaling"],
        vs_baseline=None, dtype="f32" if wl.get("fp32") else "bf16", data="synthetic",
        config=dict(workload=name, hidden=hidden, intermediate=inter, gated=True, activation="gelu_fused",
                    dropout=wl["dropout"], total_tokens=total_tokens, tokens_per_gpu=tokens,
                    parameters=("fp32 masters + bf16 compute (autocast)" if wl["mixed"] else
                                "fp32, products as three TF32 tensor-core products" if wl.get("fp32") else "bf16"),
                    parallelism=f"dp{world} token partition" + (
                        "" if world == 1 else ", weight gradients reduce-scattered inside their GEMMs (NVLink peer atomics) "
                        "+ copy-engine all-gather, NCCL for the small tensors" if reducer is not None
                        else ", bf16 gradient all-reduce (NCCL) overlapped with backward"),
                    l2="inputs and activations exceed the 126 MB L2 (no flush needed)",
                    step="forward + backward" + (" + gradient all-reduce" if world > 1 else "")),
        tflops=tflops, pct_of_bf16_peak_measured_burst=100.0 * tflops / world / peaks["bf16"],
        pct_of_bf16_peak_datasheet=100.0 * tflops / world / 2250.0,
        roofline=dict(bound="tensor", achieved=achieved, peak=peaks["bf16_sustained"], unit="TFLOP/s",
                      frac=(achieved / peaks["bf16_sustained"]) if achieved else None,
                      traffic=traffic, traffic_note=traffic_note,
                      kernel="gemm_tcgen05_kernel (all GEMM launches of the timed region)", launches=gemm_launches,
                      peak_source=f"bf16_tflops_sustained of {peaks['source']} peaks (kernel timed inside a long step)"),
        cpu_baseline=cpu,
        e2e=dict(value=total_tokens * args.steps / e_seconds, unit="tokens/s",
                 h2d_bytes_per_step=(x_host.numel() * x_host.element_size() + g_host.numel() * g_host.element_size()) * world,
                 d2h_bytes_per_step=(out_host_bytes + 4) * world, ms_per_step=e_seconds / args.steps * 1e3,
                 api="LeanFFN.forward / Tensor.backward with pinned host inputs (double-buffered uploads); the output, "
                     "the input gradient and the loss return to pinned host memory every step",
                 last_loss=losses[-1] if losses else None),
        gpu_launches=launches, clocks=clocks, checksum=checksum,
        tokens_per_s_per_sm_mhz=(tokens_per_s / clocks["sm_mhz"]) if clocks and clocks.get("sm_mhz") else None)
    if world > 1:
        line["comm"] = dict(exposed_allreduce_ms_per_step=exposed_ms,
                            sms_left_free_during_exchange=2 if reducer is not None else args.comm_sms,
                            grad_exchange=exchange_note,
                            note="time the compute stream of rank 0 waited for gradient all-reduces after its last kernel")
    if extra:
        line["other_workloads"] = extra
    print(json.dumps(line), flush=True)


def quick_measure(wl, device, args, name=""):
    """Device-resident fwd+bwd rate of a second workload on one GPU (reported next to the headline)."""
    import lean_transformer_b200 as L
    from lean_transformer_b200 import ops

    ffn = build_module(wl, device)
    tokens, hidden = wl.get("tokens_per_rank") or wl["total_tokens"], wl["hidden"]
    x = torch.randn(tokens, hidden, device=device).to(torch.float32 if (wl["mixed"] or wl.get("fp32")) else torch.bfloat16)
    g = torch.randn(tokens, hidden, device=device).to(torch.float32 if wl.get("fp32") else torch.bfloat16)
    params = list(ffn.parameters())

    from lean_transformer_b200.blocksparse.linear import clear_cast_cache

    def step():
        if wl["mixed"]:
            clear_cast_cache()
        for p in params:
            p.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=wl["mixed"]):
            out = ffn(x.detach().requires_grad_(True))
        out.backward(g)

    for _ in range(5):
        step()
    torch.cuda.synchronize()
    n = 20 if tokens * hidden >= (1 << 27) else 50
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ops.launch_count
    with ops.GemmTimer() as timer:
        a.record()
        for _ in range(n):
            step()
        b.record()
        torch.cuda.synchronize()
    L.check_device_status(device)
    s = a.elapsed_time(b) * 1e-3 / n
    gemm_flops, gemm_seconds, gemm_launches = timer.summary()
    peaks = load_peaks()
    achieved = gemm_flops / gemm_seconds / 1e12 if gemm_seconds > 0 else None
    traffic, traffic_note = captured_traffic(name, tokens)
    return dict(tokens_per_s=tokens / s, ms_per_step=s * 1e3, tflops=tokens / s * flops_per_token(hidden, wl["inter"], wl) / 1e12,
                steps=n, warmup=5, gpu_launches_per_step=(ops.launch_count - launches0) / n,
                roofline=dict(bound="tensor", achieved=achieved, peak=peaks["bf16_sustained"], unit="TFLOP/s",
                              frac=(achieved / peaks["bf16_sustained"]) if achieved else None, traffic=traffic,
                              traffic_note=traffic_note, launches=gemm_launches,
                              kernel="all GEMM launches of the timed region (CUDA events around each launch)"),
                config=dict(hidden=hidden, intermediate=wl["inter"], tokens=tokens, dropout=wl["dropout"],
                            parameters=("fp32 masters + bf16 compute" if wl["mixed"] else
                                        "fp32 (TF32x3 tensor cores)" if wl.get("fp32") else "bf16")))


def attention_measure(device, batch=32, seq=2048, heads=16, head_dim=48, steps=20, warmup=3):
    """The attention core of the 12-layer GPT configuration (hidden 768, 16 heads, 32 x 2048 tokens) on its own: rotary + causal attention over batch x seq tokens, heads x
    head_dim (this package's RotaryAttentionCore: leanffn_rotary + leanffn_attention_forward / backward), forward +
    backward, device-resident.  FLOPs: 4 * seq^2 * head_dim per head and batch row forward, 2.5 x that backward, halved
    by the causal rule.  The kernels are bound by the tensor cores' operand feed and the exponentials, so the fraction
    of the dense-GEMM peak reported here is low by construction."""
    import lean_transformer_b200 as L
    from lean_transformer_b200 import ops

    hidden = heads * head_dim
    torch.manual_seed(0)
    core = L.RotaryAttentionCore(hidden, heads).to(device).train()
    qkv = torch.randn(batch, seq, 3 * hidden, device=device).to(torch.bfloat16)
    g = torch.randn(batch, seq, hidden, device=device).to(torch.bfloat16)
    mask = ((1.0 - torch.ones(seq, seq, device=device).tril()) * -10000.0).view(1, 1, seq, seq)

    def step():
        leaf = qkv.detach().requires_grad_(True)
        q, k, v = leaf.split(hidden, dim=-1)
        out, _ = core(q, k, v, mask)
        out.backward(g)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ops.launch_count
    a.record()
    for _ in range(steps):
        step()
    b.record()
    torch.cuda.synchronize()
    L.check_device_status(device)
    s = a.elapsed_time(b) * 1e-3 / steps
    launches_per_step = (ops.launch_count - launches0) / steps
    flops = 3.5 * 4.0 * seq * seq * head_dim * heads * batch / 2
    peaks = load_peaks()
    achieved = flops / s / 1e12

    def timed(fn, n=10):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n):
            fn()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / n

    # the kernels alone (no rotary, no autograd bookkeeping), and the library's fused attention on the same shape for
    # context (torch.nn.functional.scaled_dot_product_attention: whichever flash / cuDNN kernel torch picks)
    scale = head_dim ** -0.5
    q, k, v = qkv.split(hidden, dim=-1)
    out, lse = ops.attention_forward(q, k, v, heads, scale, None, True)
    fwd_ms = timed(lambda: ops.attention_forward(q, k, v, heads, scale, None, True))
    bwd_ms = timed(lambda: ops.attention_backward(g, q, k, v, out, lse, heads, scale, None, True))
    library = None
    try:
        import torch.nn.functional as F
        q4, k4, v4 = (t.reshape(batch, seq, heads, head_dim).transpose(1, 2).contiguous().requires_grad_() for t in (q, k, v))
        g4 = g.reshape(batch, seq, heads, head_dim).transpose(1, 2).contiguous()
        lib_fwd = timed(lambda: F.scaled_dot_product_attention(q4, k4, v4, is_causal=True))
        lib_both = timed(lambda: torch.autograd.grad(F.scaled_dot_product_attention(q4, k4, v4, is_causal=True),
                                                     (q4, k4, v4), g4))
        library = dict(forward_ms=lib_fwd, forward_backward_ms=lib_both)
    except Exception as e:  # context only
        library = dict(unavailable=f"{type(e).__name__}: {e}")
    return dict(tokens_per_s=batch * seq / s, ms_per_step=s * 1e3, tflops=achieved, steps=steps, warmup=warmup,
                forward_kernel_ms=fwd_ms, backward_kernels_ms=bwd_ms, library_sdpa=library,
                gpu_launches_per_step=launches_per_step,
                roofline=dict(bound="tensor", achieved=achieved, peak=peaks["bf16_sustained"], unit="TFLOP/s",
                              frac=achieved / peaks["bf16_sustained"], traffic=None,
                              kernel="rotary + attention forward + backward (CUDA events around the whole step)"),
                config=dict(batch=batch, seq_len=seq, heads=heads, head_dim=head_dim, mask="causal (detected)",
                            dtype="bf16"))


def leangpt_measure(device, steps=3, warmup=1, batch=32, seq=2048):
    """The full-model configuration: the REFERENCE's own 12-layer LeanGPT (hidden 768, 16 heads, rotary, GeGLU, tied embeddings,
    vocab 10 000; imported from the mirror oracle/_ref) on the GPU under autocast(bf16), forward + backward on 32 x 2048
    random token ids with labels = ids, timed three times on the same weights: with the reference's own modules (stock
    PyTorch CUDA operators); with its LeanFFN / GeneralizedLinear modules and the attention blocks' LayerNorm and
    projections swapped for this package's (integration.convert_model, attention core still the reference's); and with
    the attention cores swapped too.  Embeddings, LM head and loss stay the reference's code in all runs.
    Also reports the time spent inside the FFN modules and inside the attention cores (CUDA events around their forward
    and backward)."""
    from oracle import ref_harness

    ref = ref_harness.import_reference()
    if ref is None:
        return dict(unavailable="the reference mirror oracle/_ref is absent (python oracle/build_ref.py builds it "
                                "where the reference checkout exists)")
    import lean_transformer_b200 as L
    from lean_transformer_b200.integration import convert_model

    torch.manual_seed(0)
    config = ref.gpt.LeanGPTConfig(vocab_size=10000, hidden_size=768, num_hidden_layers=12, num_attention_heads=16,
                                   position_embedding_type="rotary", hidden_act_gated=True, tie_word_embeddings=True)
    model = ref.gpt.LeanGPTModel(config).to(device).train()
    ids = torch.randint(0, 10000, (batch, seq), device=device, generator=torch.Generator(device=device).manual_seed(0))
    params = list(model.parameters())
    tokens = batch * seq

    def modules_named(name):
        return [m for m in model.modules() if type(m).__name__ == name]

    def timed(n_steps):
        events, core_events = [], []

        def hooks(store):
            def pre(_m, *_a):
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                store.append([e, None])

            def post(_m, *_a):
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                store[-1][1] = e
            return pre, post

        handles = []
        for store, mods in ((events, modules_named("LeanFFN")), (core_events, modules_named("RotaryAttentionCore"))):
            pre, post = hooks(store)
            for m in mods:
                handles += [m.register_forward_pre_hook(pre), m.register_forward_hook(post),
                            m.register_full_backward_pre_hook(pre), m.register_full_backward_hook(post)]
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        losses = []
        a.record()
        for _ in range(n_steps):
            for p in params:
                p.grad = None
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = model(input_ids=ids, labels=ids).loss
            loss.backward()
            losses.append(loss.detach())
        b.record()
        torch.cuda.synchronize()
        for h in handles:
            h.remove()
        ffn_ms = sum(s.elapsed_time(e) for s, e in events if e is not None) / n_steps
        core_ms = sum(s.elapsed_time(e) for s, e in core_events if e is not None) / n_steps
        return a.elapsed_time(b) / n_steps, ffn_ms, core_ms, float(losses[-1])

    out = dict(config=dict(model="LeanGPT (reference lean_transformer/models/gpt.py)", layers=12, hidden=768, heads=16,
                           intermediate=3072, gated=True, vocab=10000, batch=batch, seq_len=seq, tokens=tokens,
                           dtype="autocast bf16, fp32 parameters", steps=steps, warmup=warmup))
    # three runs of the same model object: the reference's modules; FFN blocks, linear layers and the attention
    # blocks' LayerNorm / projections swapped (attention core still the reference's stock operators); everything swapped
    for label in ("reference_modules", "swapped_ffn_and_linears", "swapped_with_attention_core"):
        if label == "swapped_ffn_and_linears":
            convert_model(model, convert_attention_core=False)
        elif label == "swapped_with_attention_core":
            convert_model(model)
        timed(warmup)
        launches = L.ops.launch_count
        ms, ffn_ms, core_ms, loss = timed(steps)
        out[label] = dict(ms_per_step=ms, tokens_per_s=tokens / ms * 1e3, ffn_ms_per_step=ffn_ms,
                          ffn_share=ffn_ms / ms, attention_core_ms_per_step=core_ms, loss=loss,
                          leanffn_b200_launches_per_step=(L.ops.launch_count - launches) / steps)
    L.check_device_status(device)
    # attention core: 4 * len * len * head_dim FLOPs per head and batch row forward, 2.5 x that backward, halved by
    # the causal rule
    core_flops = 12 * batch * 16 * 3.5 * 4 * seq * seq * 48 / 2
    out["swapped_with_attention_core"]["attention_core_tflops"] = (
        core_flops / max(out["swapped_with_attention_core"]["attention_core_ms_per_step"], 1e-9) / 1e9)
    out["speedup_attention_core"] = (out["swapped_ffn_and_linears"]["attention_core_ms_per_step"]
                                     / max(out["swapped_with_attention_core"]["attention_core_ms_per_step"], 1e-9))
    out["speedup_whole_step_with_attention_core"] = (out["reference_modules"]["ms_per_step"]
                                                     / out["swapped_with_attention_core"]["ms_per_step"])
    ffn_flops = 12 * tokens * flops_per_token(768, 3072)
    out["swapped_ffn_and_linears"]["ffn_tflops"] = ffn_flops / out["swapped_ffn_and_linears"]["ffn_ms_per_step"] / 1e9
    out["reference_modules"]["ffn_tflops"] = ffn_flops / out["reference_modules"]["ffn_ms_per_step"] / 1e9
    out["speedup_whole_step"] = out["reference_modules"]["ms_per_step"] / out["swapped_ffn_and_linears"]["ms_per_step"]
    out["speedup_ffn_modules"] = (out["reference_modules"]["ffn_ms_per_step"]
                                  / out["swapped_ffn_and_linears"]["ffn_ms_per_step"])
    return out


def leangpt_converted_steps(device, steps=2, batch=32, seq=2048):
    """The converted 12-layer GPT alone (no reference runs): ``steps`` forward + backward passes, for launch lists."""
    from oracle import ref_harness

    ref = ref_harness.import_reference()
    if ref is None:
        raise RuntimeError("the mirrored reference package (oracle/_ref) is missing")
    import lean_transformer_b200 as L
    from lean_transformer_b200.integration import convert_model

    torch.manual_seed(0)
    config = ref.gpt.LeanGPTConfig(vocab_size=10000, hidden_size=768, num_hidden_layers=12, num_attention_heads=16,
                                   position_embedding_type="rotary", hidden_act_gated=True, tie_word_embeddings=True)
    model = convert_model(ref.gpt.LeanGPTModel(config).to(device).train())
    ids = torch.randint(0, 10000, (batch, seq), device=device, generator=torch.Generator(device=device).manual_seed(0))
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for step in range(steps):
        if step == 1 or steps == 1:
            a.record()  # the first pass (library initialisation, allocator growth) is not timed when there are more
        for p in model.parameters():
            p.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
    b.record()
    torch.cuda.synchronize()
    L.check_device_status(device)
    return dict(workload="leangpt_bf16_h768 (converted model only)", steps=steps,
                ms_per_step=a.elapsed_time(b) / max(steps - 1, 1), loss=float(loss.detach()))


def epilogue_ablation(device):
    """What each phase of the fused GeGLU-backward epilogue costs: times the input-gradient product of config 2
    (16 384 x 1024 . 1024 x 4096) and of config 5 at 8192 tokens with phases of its epilogue left out.  Needs a
    MEASUREMENT build of the library, which reads the mask from LEANFFN_ABLATE on every call (results are wrong on
    purpose, nothing here is a bench number):

        LEANFFN_NVCC_EXTRA=-DLEANFFN_ABLATE_RUNTIME=1 python lean_transformer_b200/build.py --force
        python bench.py --epilogue-ablation

    Mask bits: 1 no residual / pre-activation loads, 2 no global stores, 4 no activation arithmetic, 8 no column
    sums, 16 no shared-memory transposition, 32 no tensor-memory read."""
    from lean_transformer_b200 import _native as N
    from lean_transformer_b200 import ops

    def timed(fn, n=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n * 1e3

    report = {}
    for tokens, hidden, inter, tag in ((16384, 1024, 4096, "config2"), (8192, 8192, 32768, "config5_8192_tokens")):
        torch.manual_seed(0)
        dy = torch.randn(tokens, hidden, device=device).bfloat16()
        w2 = (torch.randn(hidden, inter, device=device) * 0.02).bfloat16()
        pre = torch.randn(tokens, 2 * inter, device=device).bfloat16()
        dpre, hid = torch.empty_like(pre), torch.empty(tokens, inter, device=device, dtype=torch.bfloat16)
        partial = torch.empty((tokens + 31) // 32, 2 * inter, device=device)
        plain = torch.empty(tokens, inter, device=device, dtype=torch.bfloat16)
        entry = {}
        for mask in (0, 1, 2, 4, 8, 16, 32, 3, 7, 63):
            os.environ["LEANFFN_ABLATE"] = str(mask)
            entry[f"mask_{mask}_us"] = timed(lambda: ops.gemm(dy, w2, b_mn_major=True, epilogue=N.EPI_GLU_BWD, act=0, aux=pre,
                                                              out=dpre, out2=hid, colsum=partial))
        os.environ["LEANFFN_ABLATE"] = "0"
        entry["plain_store_us"] = timed(lambda: ops.gemm(dy, w2, b_mn_major=True, out=plain))
        report[tag] = entry
    print(json.dumps(dict(epilogue_ablation=report, note="measurement build only; mask 0 = the complete epilogue")), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="dense_bf16_h8192")
    ap.add_argument("--extra-workload", default="mixed_bf16_h1024,dense_fp32_h768,pixelfly_bf16_h4096,attention_bf16_h768,leangpt_bf16_h768",
                    help="comma-separated workloads measured device-resident on one GPU after the headline one and "
                         "reported under other_workloads ('' = none)")
    ap.add_argument("--comm-sms", type=int, default=20, help="SMs left to NCCL while GEMMs run (N > 1)")
    ap.add_argument("--grad-exchange", choices=("nccl", "fused"), default="fused",
                    help="N > 1: all-reduce every gradient with NCCL, or reduce-scatter the dense weight gradients inside "
                         "their GEMMs (peer atomics over NVLink + copy-engine hand-out) and keep NCCL for the small ones")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tokens", type=int, default=0,
                    help="override the workload's token count (smaller cases for ncu captures; not a bench number)")
    ap.add_argument("--skip-e2e", action="store_true", help="device-resident timing only (profiling runs)")
    ap.add_argument("--attention-only", action="store_true",
                    help="measure the attention-core workload alone (attention_bf16_h768) and print its line "
                         "(profiling runs)")
    ap.add_argument("--leangpt-only", action="store_true",
                    help="run --steps forward + backward passes of the converted 12-layer GPT and nothing else "
                         "(profiling runs)")
    ap.add_argument("--epilogue-ablation", action="store_true",
                    help="time the GeGLU-backward product with phases of its epilogue left out (measurement build of "
                         "the library only; see epilogue_ablation)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    if args.attention_only:
        torch.cuda.set_device(0)
        print(json.dumps(dict(workload="attention_bf16_h768",
                              **attention_measure(torch.device("cuda", 0), steps=args.steps, warmup=args.warmup))),
              flush=True)
        return
    if args.leangpt_only:
        torch.cuda.set_device(0)
        print(json.dumps(leangpt_converted_steps(torch.device("cuda", 0), steps=max(args.steps, 1))), flush=True)
        return
    if args.epilogue_ablation:
        torch.cuda.set_device(0)
        epilogue_ablation(torch.device("cuda", 0))
        return
    wl = dict(WORKLOADS[args.workload])
    if args.tokens:
        wl["total_tokens" if "total_tokens" in wl else "tokens_per_rank"] = args.tokens
    if args.impl == "reference":
        run_reference_arm(args, wl, args.workload)
    else:
        run_ours(args, wl, args.workload)


if __name__ == "__main__":
    main()
