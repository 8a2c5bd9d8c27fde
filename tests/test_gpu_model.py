"""The reference's own LeanGPT model with this package's kernels swapped in (needs a B200 and the reference mirror
that ``oracle/build_ref.py`` makes; skipped where the mirror is absent).

Pattern of the reference's tests/test_modifications.py:10-78 and tests/test_triton.py:62-97: one model, one batch,
one seed; run it with the reference's implementation, swap, run again with every memory-saving option toggled, and
compare logits, loss and every parameter gradient.  The model exercises the features the conversion has to keep:
matrices shared between layer groups with per-layer adapters, rotary attention, GeGLU, gradient checkpointing, the
``ffn_custom_grad`` switch, tied embeddings.
"""
import pytest
import torch

from conftest import BF16_ATOL, BF16_RTOL, FP32_ATOL, FP32_RTOL, assert_close, record_closeness

pytestmark = pytest.mark.gpu


def _reference():
    from oracle import ref_harness
    ref = ref_harness.import_reference()
    if ref is None:
        pytest.skip("oracle/_ref has not been built (python oracle/build_ref.py on a machine with the reference)")
    return ref


def _tiny_gpt(ref, **overrides):
    kw = dict(vocab_size=200, hidden_size=128, embedding_size=128, num_hidden_layers=4, num_hidden_groups=2,
              num_attention_heads=4, intermediate_size=256, position_embedding_type="rotary", hidden_act_gated=True,
              tie_word_embeddings=True, share_large_matrices=True, adapter_dim=8, hidden_dropout_prob=0.0)
    kw.update(overrides)
    return ref.gpt.LeanGPTModel(ref.gpt.LeanGPTConfig(**kw))


def _run(model, ids, autocast=False, seed=1337):
    model.zero_grad(set_to_none=True)
    torch.manual_seed(seed)
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast):
        out = model(input_ids=ids, labels=ids)
    out.loss.backward()
    grads = {n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None}
    return out.logits.detach().float().clone(), float(out.loss.detach()), grads


def _compare(got, want, rtol, atol, label, outlier_frac=0.0):
    assert_close(got[0], want[0], rtol, atol, f"{label}:logits", scale_atol=True, outlier_frac=outlier_frac)
    assert abs(got[1] - want[1]) <= atol + rtol * abs(want[1]), f"{label}: loss {got[1]} vs {want[1]}"
    assert set(got[2]) == set(want[2]), f"{label}: parameters with gradients differ"
    for name, ref_grad in want[2].items():
        assert_close(got[2][name], ref_grad, rtol, atol, f"{label}:grad {name}", scale_atol=True,
                     outlier_frac=outlier_frac)


def test_tiny_gpt_swapped_ffn_matches_reference_fp32(cuda_device):
    import lean_transformer_b200 as L
    from lean_transformer_b200.integration import convert_model

    ref = _reference()
    torch.manual_seed(0)
    model = _tiny_gpt(ref).to(cuda_device).train()
    ids = torch.randint(0, 200, (3, 48), generator=torch.Generator().manual_seed(5)).to(cuda_device)
    model.set_optimizations(ffn_custom_grad=True)
    want = _run(model, ids)  # the reference's own kernels (stock PyTorch CUDA operators), fp32
    convert_model(model, convert_attention_core=False)  # plain fp32: the attention kernels are bf16-only
    assert sum(isinstance(m, L.LeanFFN) for m in model.modules()) == 2
    launches = L.ops.launch_count
    for checkpoints, custom in ((False, True), (False, False), (True, True), (2, True)):
        model.set_optimizations(gradient_checkpointing=checkpoints, ffn_custom_grad=custom)
        got = _run(model, ids)
        _compare(got, want, FP32_RTOL, FP32_ATOL, f"gpt fp32 ckpt={checkpoints} custom={custom}")
    assert L.ops.launch_count > launches, "the converted model did not launch this package's kernels"
    L.check_device_status(cuda_device)


def test_tiny_gpt_swapped_ffn_matches_reference_bf16(cuda_device):
    """Same under autocast(bf16): the swapped model against the reference's fp32 run, with the reference's own
    autocast run recorded beside it as the noise floor."""
    from lean_transformer_b200.integration import convert_model

    ref = _reference()
    torch.manual_seed(0)
    model = _tiny_gpt(ref).to(cuda_device).train()
    ids = torch.randint(0, 200, (4, 64), generator=torch.Generator().manual_seed(6)).to(cuda_device)
    want = _run(model, ids)
    floor = _run(model, ids, autocast=True)
    convert_model(model)
    import lean_transformer_b200 as L
    assert sum(isinstance(m, L.RotaryAttentionCore) for m in model.modules()) >= 1
    got = _run(model, ids, autocast=True)
    # Through four layers the rounding noise of bf16 arithmetic compounds (the reference's own autocast run misses the
    # single-layer bound on some tensors by 1.7x), so each tensor is checked against that run: the swapped model's
    # rms distance from the fp32 run may be at most twice the reference-autocast run's, and no element may lie
    # beyond 3x the single-layer bound.
    assert abs(got[1] - want[1]) <= BF16_ATOL + BF16_RTOL * abs(want[1])
    pairs = [("logits", got[0], floor[0], want[0])] + [(f"grad {n}", got[2][n], floor[2][n], r) for n, r in want[2].items()]
    for name, ours, theirs, ref in pairs:
        mine = record_closeness(ours, ref, BF16_RTOL, BF16_ATOL, f"gpt bf16:{name}")
        record_closeness(theirs, ref, BF16_RTOL, BF16_ATOL, f"twin:gpt bf16:{name}")
        rms = lambda t: float((t.double().cpu() - ref.double().cpu()).pow(2).mean().sqrt())  # noqa: E731
        floor_rms = rms(theirs)
        assert rms(ours) <= 2.0 * floor_rms + 1e-3 * max(mine["rms_ref"], 1e-6), \
            f"{name}: rms error {rms(ours):.4g} vs {floor_rms:.4g} for the reference's own autocast run"
        assert mine["scaled_worst"] <= 3.0, f"{name}: an element lies {mine['scaled_worst']:.2f}x beyond the bound"


def test_dropout_runs_are_consistent_across_optimizations(cuda_device):
    """tests/test_modifications.py: with dropout 0.1 and one seed, checkpointing and the custom-gradient switch must
    not change logits or gradients (the dropout masks are regenerated, not re-drawn)."""
    from lean_transformer_b200.integration import convert_model

    ref = _reference()
    torch.manual_seed(0)
    model = convert_model(_tiny_gpt(ref, hidden_dropout_prob=0.1).to(cuda_device).train(),
                          convert_attention_core=False)
    ids = torch.randint(0, 200, (2, 32), generator=torch.Generator().manual_seed(7)).to(cuda_device)
    model.set_optimizations(gradient_checkpointing=False, checkpoint_last=False, checkpoint_attention_core=False,
                            ffn_custom_grad=False)
    want = _run(model, ids)
    for checkpoints, last, attn, custom in ((False, False, True, True), (True, True, False, True), (3, False, True, True)):
        model.set_optimizations(gradient_checkpointing=checkpoints, checkpoint_last=last,
                                checkpoint_attention_core=attn, ffn_custom_grad=custom)
        got = _run(model, ids)
        _compare(got, want, FP32_RTOL, FP32_ATOL, f"dropout ckpt={checkpoints} custom={custom}")
    other = _run(model, ids, seed=4242)
    assert not torch.allclose(other[0], want[0], rtol=1e-3, atol=1e-5), "dropout ignored the seed"


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_attention_shell_matches_reference_block(cuda_device, mode):
    """lean_transformer/attn.py:11-82 with a rotary core, shared block-sparse-free GeneralizedLinear projections and an
    fp32 residual stream: the reference block on stock operators against the same block after convert_model (its
    LayerNorm, qkv projection and out projection + dropout + residual on this package's kernels; in bf16 mode the rotary
    attention core too, in plain fp32 its own core)."""
    import lean_transformer_b200 as L
    from lean_transformer_b200.integration import convert_model

    ref = _reference()
    torch.manual_seed(3)
    hidden, heads = 256, 8
    GM, GL = ref.linear.GeneralizedMatrix, ref.linear.GeneralizedLinear
    block = ref.attn.LeanSelfAttention(hidden, heads, dropout=0.0, attention_core=ref.attn.RotaryAttentionCore(hidden, heads),
                                       qkv_proj=GL(GM(hidden, 3 * hidden, None, 16), adapter_dim=8),
                                       out_proj=GL(GM(hidden, hidden, None, 0))).to(cuda_device).train()
    with torch.no_grad():
        block.qkv_proj.adapter_second.normal_(0, 0.02)
    x = torch.randn(3, 96, hidden, device=cuda_device)
    g = torch.randn(3, 96, hidden, device=cuda_device)
    mask = torch.zeros(3, 1, 96, 96, device=cuda_device)
    mask[1, :, :, 80:] = -10000.0
    def run(module, autocast):
        module.zero_grad(set_to_none=True)
        inp = x.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast):
            (out,) = module(inp, mask)
        (out.float() * g).sum().backward()
        return out.detach(), inp.grad, {n: p.grad.clone() for n, p in module.named_parameters() if p.grad is not None}

    want = run(block, False)  # the reference's own fp32 run is the yardstick
    floor = run(block, True) if mode == "bf16" else None
    new = convert_model(block, convert_attention_core=mode == "bf16")
    assert isinstance(new, L.LeanSelfAttention) and isinstance(new, ref.attn.LeanSelfAttention)
    assert isinstance(new.qkv_proj, L.GeneralizedLinear)
    if mode == "bf16":
        assert isinstance(new.attention_core, L.RotaryAttentionCore)
        assert isinstance(new.attention_core, ref.attn.RotaryAttentionCore)
        assert new.attention_core.rotary_emb is block.attention_core.rotary_emb
    else:
        assert new.attention_core is block.attention_core
    launches = L.ops.launch_count
    got = run(new, mode == "bf16")
    assert L.ops.launch_count - launches >= 8
    assert got[0].dtype == torch.float32  # fp32 residual stream: attn.py:77
    rtol, atol = (BF16_RTOL, BF16_ATOL) if mode == "bf16" else (FP32_RTOL, FP32_ATOL)
    budget = dict(outlier_frac=1e-4, outlier_cap=2.0) if mode == "bf16" else {}
    assert_close(got[0], want[0], rtol, atol, f"attention {mode}:out", branch=want[0] - x, scale_atol=True, **budget)
    assert_close(got[1], want[1], rtol, atol, f"attention {mode}:grad_input", scale_atol=True, **budget)
    assert set(got[2]) == set(want[2])
    for name in want[2]:
        assert_close(got[2][name], want[2][name], rtol, atol, f"attention {mode}:grad {name}", scale_atol=True, **budget)
        if mode == "bf16":
            record_closeness(floor[2][name], want[2][name], rtol, atol, f"twin:attention bf16:grad {name}")
    L.check_device_status(cuda_device)
