"""Parity of every C-ABI kernel against the CPU oracle on the same seeded inputs (needs a B200)."""
import numpy as np
import pytest
import torch

from conftest import BF16_ATOL, BF16_RTOL, FP32_ATOL, FP32_RTOL, assert_close, load_golden
from oracle import leanffn_oracle as O

pytestmark = pytest.mark.gpu

ACTS = {"gelu_tanh": 0, "gelu_erf": 1, "relu": 2, "silu": 3, "tanh": 4, "sigmoid": 5, "identity": 6}


@pytest.fixture(scope="module")
def ops():
    from lean_transformer_b200 import ops as _ops
    return _ops


def _cpu64(t):
    return t.detach().double().cpu()


# ---- LayerNorm ------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,cols", [(1, 8), (5, 37), (37, 100), (512, 32), (333, 768), (1024, 1024), (65, 4096), (9, 8192),
                                       (3, 16388)])
@pytest.mark.parametrize("mode", ["f32", "f32->bf16", "bf16"])
def test_layer_norm_forward(ops, cuda_device, rows, cols, mode):
    torch.manual_seed(rows * 7 + cols)
    xdt = torch.bfloat16 if mode == "bf16" else torch.float32
    ydt = torch.float32 if mode == "f32" else torch.bfloat16
    x = (torch.randn(rows, cols) * 1.5 + 0.3).to(xdt)
    gamma = (1 + 0.2 * torch.randn(cols)).to(xdt)
    beta = (0.2 * torch.randn(cols)).to(xdt)
    y = ops.layer_norm_forward(x.to(cuda_device), gamma.to(cuda_device), beta.to(cuda_device), 1e-12, ydt)
    ref = O.layer_norm_forward(_cpu64(x), _cpu64(gamma), _cpu64(beta), 1e-12)
    if ydt == torch.float32:
        assert_close(y, ref, FP32_RTOL, FP32_ATOL, "ln fwd")
    else:
        assert_close(y, ref, BF16_RTOL, BF16_ATOL, "ln fwd")
    ops.check_device_status(cuda_device)


def test_layer_norm_constant_rows_and_empty(ops, cuda_device):
    x = torch.full((5, 64), 2.5, device=cuda_device)
    beta = torch.linspace(-1, 1, 64, device=cuda_device)
    y = ops.layer_norm_forward(x, torch.ones(64, device=cuda_device), beta, 1e-12, torch.float32)
    assert torch.equal(y, beta.expand(5, 64))  # zero variance: exactly beta, like the reference's F.layer_norm
    empty = ops.layer_norm_forward(torch.empty(0, 64, device=cuda_device), None, None, 1e-5, torch.float32)
    assert empty.shape == (0, 64)


@pytest.mark.parametrize("rows,cols", [(37, 100), (512, 32), (700, 768), (2048, 1024), (130, 4096), (20, 8192)])
def test_layer_norm_backward_fp32(ops, cuda_device, rows, cols):
    torch.manual_seed(cols)
    x, dy, res = torch.randn(rows, cols), torch.randn(rows, cols), torch.randn(rows, cols)
    gamma = 1 + 0.2 * torch.randn(cols)
    dx, dg, db = ops.layer_norm_backward(dy.to(cuda_device), x.to(cuda_device), gamma.to(cuda_device), 1e-12,
                                         res.to(cuda_device), torch.float32)
    rdx, rdg, rdb = O.layer_norm_backward(_cpu64(dy), _cpu64(x), _cpu64(gamma), 1e-12)
    assert_close(dx, rdx + _cpu64(res), FP32_RTOL, FP32_ATOL, "dx")
    assert_close(dg, rdg, FP32_RTOL, FP32_ATOL, "dgamma", scale_atol=True)
    assert_close(db, rdb, FP32_RTOL, FP32_ATOL, "dbeta", scale_atol=True)


def test_layer_norm_backward_mixed(ops, cuda_device):
    """bf16 incoming gradient, fp32 residual stream (the autocast configuration)."""
    torch.manual_seed(3)
    rows, cols = 1024, 1024
    x, gamma = torch.randn(rows, cols), 1 + 0.2 * torch.randn(cols)
    dy = torch.randn(rows, cols).bfloat16()
    dx, dg, db = ops.layer_norm_backward(dy.to(cuda_device), x.to(cuda_device), gamma.to(cuda_device), 1e-12,
                                         dy.to(cuda_device), torch.float32)
    rdx, rdg, rdb = O.layer_norm_backward(_cpu64(dy), _cpu64(x), _cpu64(gamma), 1e-12)
    assert dx.dtype == torch.float32
    assert_close(dx, rdx + _cpu64(dy), FP32_RTOL, FP32_ATOL, "dx")
    assert_close(dg, rdg, FP32_RTOL, FP32_ATOL, "dgamma", scale_atol=True)
    assert_close(db, rdb, FP32_RTOL, FP32_ATOL, "dbeta", scale_atol=True)


# ---- activations ----------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(ACTS))
@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activation_forward_backward(ops, cuda_device, name, gated, dtype):
    torch.manual_seed(11)
    rows, inter = 130, 96
    pre = (torch.randn(rows, 2 * inter if gated else inter) * 2).to(dtype)
    dhid = torch.randn(rows, inter).to(dtype)
    hid = ops.activation_forward(pre.to(cuda_device), gated, ACTS[name])
    dpre, hid2 = ops.activation_backward(dhid.to(cuda_device), pre.to(cuda_device), gated, ACTS[name], want_hid=True)
    ref_hid = O.apply_activation(_cpu64(pre), name, gated)
    ref_dpre = O.apply_activation_backward(_cpu64(dhid), _cpu64(pre), name, gated)
    rtol, atol = (FP32_RTOL, FP32_ATOL) if dtype == torch.float32 else (BF16_RTOL, BF16_ATOL)
    assert_close(hid, ref_hid, rtol, atol, "hid")
    assert_close(dpre, ref_dpre, rtol, atol, "dpre")
    assert torch.equal(hid, hid2)  # rematerialisation is bit-identical to the forward


# ---- dropout ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("p,seed,offset,n", [(0.1, 0, 0, 4096), (0.5, 1234, 64, 777), (0.9, 2**40 + 5, 3, 1001),
                                            (0.25, 7, 2**33, 512)])
def test_dropout_mask_is_the_oracle_philox_mask(ops, cuda_device, p, seed, offset, n):
    mask = ops.dropout_mask(n, p, seed, offset, cuda_device).cpu().numpy().astype(bool)
    assert np.array_equal(mask, O.dropout_keep_mask(n, p, seed, offset))  # bit-exact integer work
    x = torch.randn(n, device=cuda_device)
    y = ops.dropout(x, p, seed, offset)
    expect = torch.where(torch.from_numpy(mask).to(cuda_device), x / (1 - p), torch.zeros_like(x))
    assert_close(y, expect, 1e-6, 1e-7, "dropout values")
    res = torch.randn(n, device=cuda_device)
    y2 = ops.dropout(x.bfloat16(), p, seed, offset, out_dtype=torch.float32, residual=res)
    assert_close(y2, torch.where(torch.from_numpy(mask).to(cuda_device), x.bfloat16().float() / (1 - p),
                                 torch.zeros_like(x)) + res, 1e-6, 1e-6, "dropout + residual")


@pytest.mark.parametrize("rows,cols,p,in_dtype,out_dtype", [
    (16384, 1024, 0.1, torch.bfloat16, torch.bfloat16), (1000, 512, 0.3, torch.float32, torch.bfloat16),
    (37, 8192, 0.0, torch.float32, torch.bfloat16), (515, 100, 0.2, torch.float32, torch.float32),
    (64, 256, 0.5, torch.bfloat16, torch.float32), (1, 8, 0.1, torch.float32, torch.float32)])
def test_dropout_with_column_sums(ops, cuda_device, rows, cols, p, in_dtype, out_dtype):
    """Mask + cast + column sums in one pass equals the two separate kernels bit for bit (y) and the oracle."""
    torch.manual_seed(rows + cols)
    x = torch.randn(rows, cols, device=cuda_device).to(in_dtype)
    seed, offset = 11, 4 * 123
    y, sums = ops.dropout_colsum(x, p, seed, offset, out_dtype=out_dtype)
    assert torch.equal(y, ops.dropout(x, p, seed, offset, out_dtype=out_dtype))
    keep = torch.from_numpy(O.dropout_keep_mask(rows * cols, p, seed, offset)).view(rows, cols).double()
    ref = _cpu64(x) * keep / (1 - p)
    assert_close(y, ref, 1e-2 if out_dtype == torch.bfloat16 else 1e-6, 1e-6, "masked values")
    assert_close(sums, _cpu64(y).sum(0), 1e-5, 1e-3, "column sums of the rounded output")
    y2, sums2 = ops.dropout_colsum(x, p, seed, offset + 1, out_dtype=out_dtype)  # unaligned stream offset: two kernels
    assert_close(sums2, _cpu64(y2).sum(0), 1e-5, 1e-3, "fallback path")


def test_dropout_rate_and_identity(ops, cuda_device):
    x = torch.ones(1 << 22, device=cuda_device)
    for p in (0.1, 0.5):
        keep = float((ops.dropout(x, p, 99, 0) != 0).float().mean())
        assert abs(keep - (1 - p)) < 2e-3
    assert torch.equal(ops.dropout(x, 0.0, 5, 0), x)


# ---- reductions, casts, transposes ---------------------------------------------------------------
@pytest.mark.parametrize("rows,cols,dtype", [(1, 5, torch.float32), (5000, 777, torch.float32), (16384, 1024, torch.bfloat16),
                                            (100, 8192, torch.bfloat16), (70000, 64, torch.float32)])
def test_column_sum(ops, cuda_device, rows, cols, dtype):
    torch.manual_seed(1)
    x = torch.randn(rows, cols).to(dtype)
    out = ops.column_sum(x.to(cuda_device))
    assert_close(out, _cpu64(x).sum(0), FP32_RTOL, FP32_ATOL, "column sum", scale_atol=True)
    again = ops.column_sum(x.to(cuda_device))
    assert torch.equal(out, again)  # deterministic reduction order


def test_cast_and_transpose(ops, cuda_device):
    x = torch.randn(300, 200)
    assert torch.equal(ops.cast(x.to(cuda_device), torch.bfloat16).cpu(), x.bfloat16())
    assert torch.equal(ops.transpose(x.to(cuda_device)).cpu(), x.t().contiguous())
    xb = torch.randn(129, 65).bfloat16()
    assert torch.equal(ops.transpose(xb.to(cuda_device)).cpu(), xb.t().contiguous())


# ---- GEMM --------------------------------------------------------------------------------------------
def _gemm_inputs(M, N, K, a_mn, b_mn, dtype, device, scale=1.0):
    A = (torch.randn(M, K) * scale).to(dtype)
    B = (torch.randn(N, K) * scale).to(dtype)
    As = (A.t().contiguous() if a_mn else A).to(device)
    Bs = (B.t().contiguous() if b_mn else B).to(device)
    return A, B, As, Bs


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (200, 136, 100), (64, 64, 16), (300, 77, 513)])
def test_gemm_fp32_simt(ops, cuda_device, a_mn, b_mn, M, N, K):
    torch.manual_seed(M + N + K)
    A, B, As, Bs = _gemm_inputs(M, N, K, a_mn, b_mn, torch.float32, cuda_device)
    bias = torch.randn(N)
    D = ops.gemm(As, Bs, a_mn_major=a_mn, b_mn_major=b_mn, bias=bias.to(cuda_device), force_simt=True)
    assert_close(D, _cpu64(A) @ _cpu64(B).t() + bias.double(), FP32_RTOL, FP32_ATOL, "fp32 gemm", scale_atol=True)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(64, 64, 32), (200, 136, 100), (1000, 776, 520), (300, 264, 4100), (256, 512, 16384)])
def test_gemm_fp32_on_tensor_cores(ops, cuda_device, a_mn, b_mn, M, N, K):
    """fp32 products as three TF32 products over one reduction axis, sliced so that the accumulators' truncation
    stays below the fp32-mode tolerance whatever the length of the axis."""
    from lean_transformer_b200 import ops as raw_ops
    torch.manual_seed(M + N + K)
    A, B, As, Bs = _gemm_inputs(M, N, K, a_mn, b_mn, torch.float32, cuda_device)
    bias = torch.randn(N)
    before = raw_ops.launch_count
    D = ops.gemm(As, Bs, a_mn_major=a_mn, b_mn_major=b_mn, bias=bias.to(cuda_device))
    assert raw_ops.launch_count - before == 3  # two splits + ONE product that walks the slices itself
    ref = _cpu64(A) @ _cpu64(B).t() + bias.double()
    assert_close(D, ref, FP32_RTOL, FP32_ATOL, "fp32 gemm on tensor cores", scale_atol=True)
    # and with a tighter, K-independent bound: 3e-5 of the largest entry
    assert (D.double().cpu() - ref).abs().max() <= 3e-5 * ref.abs().max()
    ops.check_device_status(cuda_device)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 128), (200, 136, 104), (1000, 776, 520), (64, 64, 32),
                                   (2048, 1024, 4096), (4096, 8192, 256)])
def test_gemm_bf16_tensor_core(ops, cuda_device, a_mn, b_mn, M, N, K):
    """All three operand-majorness variants of the tcgen05 kernel, ragged edges included, against the
    oracle product of the same bf16-rounded inputs; fp32 output isolates accumulation from output rounding."""
    torch.manual_seed(M + 3 * N + 7 * K)
    A, B, As, Bs = _gemm_inputs(M, N, K, a_mn, b_mn, torch.bfloat16, cuda_device)
    ref = _cpu64(A) @ _cpu64(B).t()
    D32 = ops.gemm(As, Bs, a_mn_major=a_mn, b_mn_major=b_mn, out_dtype=torch.float32)
    assert_close(D32, ref, 1e-4, 1e-4, "bf16 gemm, fp32 out", scale_atol=True)
    D16 = ops.gemm(As, Bs, a_mn_major=a_mn, b_mn_major=b_mn)
    assert_close(D16, ref, BF16_RTOL, BF16_ATOL, "bf16 gemm, bf16 out", scale_atol=True)
    # the SIMT kernel on the same inputs agrees too (cross-check of the two device paths)
    Ds = ops.gemm(As, Bs, a_mn_major=a_mn, b_mn_major=b_mn, out_dtype=torch.float32, force_simt=True)
    assert_close(Ds, ref, 1e-4, 1e-4, "simt gemm on bf16 inputs", scale_atol=True)
    ops.check_device_status(cuda_device)


@pytest.mark.parametrize("a_mn,b_mn,M,N,K", [
    (True, True, 768, 768, 65536),     # the output-projection weight gradient of the 12-layer GPT: 18 tiles, 8 parts
    (True, True, 768, 3072, 16384),    # 72 tiles: 2 parts
    (False, False, 200, 520, 32768),   # ragged tiles, K-major operands
    (False, True, 256, 256, 20000),    # a reduction length that the parts do not divide evenly
])
def test_gemm_split_k_accumulates_in_fp32(ops, cuda_device, a_mn, b_mn, M, N, K):
    """Dense bf16 products with an fp32 result, few output tiles and a long reduction run as split-K (the parts add
    into a zeroed result): same values as the unsplit product up to fp32 summation order."""
    torch.manual_seed(0)
    a = (torch.randn((K, M) if a_mn else (M, K), device=cuda_device) * 0.1).to(torch.bfloat16)
    b = (torch.randn((K, N) if b_mn else (N, K), device=cuda_device) * 0.1).to(torch.bfloat16)
    out = torch.full((M, N), 7.0, device=cuda_device)  # the call must zero it itself
    got = ops.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out=out, out_dtype=torch.float32)
    A = (a.t() if a_mn else a).double().cpu()
    B = (b.t() if b_mn else b).double().cpu()
    ref = A @ B.t()
    assert_close(got, ref, 1e-4, 1e-4, f"split-k gemm {M}x{N}x{K}", scale_atol=True)


def test_gemm_rejects_bad_arguments(ops, cuda_device):
    a = torch.randn(8, 8, device=cuda_device)
    with pytest.raises(AssertionError):
        ops.gemm(a, torch.randn(8, 9, device=cuda_device))  # reduction mismatch
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.gemm(a.cpu(), a.cpu())
    with pytest.raises(TypeError):
        ops.gemm(a.half(), a.half())
    out = ops.gemm(torch.empty(0, 8, device=cuda_device), a)  # zero rows is a no-op
    assert out.shape == (0, 8)


@pytest.mark.parametrize("gated", [True, False])
def test_gemm_fused_epilogues_bf16(ops, cuda_device, gated):
    from lean_transformer_b200 import _native as N
    torch.manual_seed(5)
    T, H, I = 777, 512, 1024
    width = 2 * I if gated else I
    x = torch.randn(T, H).bfloat16()
    W1 = (torch.randn(width, H) * 0.05).bfloat16()
    b1 = torch.randn(width) * 0.1
    pre = torch.empty(T, width, device=cuda_device, dtype=torch.bfloat16)
    hid = torch.empty(T, I, device=cuda_device, dtype=torch.bfloat16)
    ops.gemm(x.to(cuda_device), W1.to(cuda_device), bias=b1.to(cuda_device),
             epilogue=N.EPI_GLU_FWD if gated else N.EPI_ACT_FWD, act=0, out=pre, out2=hid)
    pre_ref = _cpu64(x) @ _cpu64(W1).t() + b1.double()
    assert_close(pre, pre_ref, BF16_RTOL, BF16_ATOL, "pre")
    assert_close(hid, O.apply_activation(_cpu64(pre), "gelu_tanh", gated), BF16_RTOL, BF16_ATOL, "hid from stored pre")
    assert torch.equal(hid, ops.activation_forward(pre, gated, 0))  # fused == stand-alone kernel, bit for bit

    # output GEMM: bias + dropout + fp32 residual, bf16 result
    W2 = (torch.randn(H, I) * 0.05).bfloat16()
    b2, res = torch.randn(H) * 0.1, torch.randn(T, H)
    p, seed, offset = 0.1, 77, 4096
    out = ops.gemm(hid, W2.to(cuda_device), bias=b2.to(cuda_device), epilogue=N.EPI_DROPOUT_RESIDUAL,
                   aux=res.to(cuda_device), dropout_p=p, seed=seed, elem_offset=offset)
    keep = torch.from_numpy(O.dropout_keep_mask(T * H, p, seed, offset)).view(T, H).double()
    ref = (_cpu64(hid) @ _cpu64(W2).t() + b2.double()) * keep / (1 - p) + res.double()
    assert_close(out, ref, BF16_RTOL, BF16_ATOL, "dropout + residual epilogue")

    # dgrad with the activation backward in the epilogue
    dy = torch.randn(T, H).bfloat16()
    dpre = torch.empty_like(pre)
    hid2 = torch.empty_like(hid)
    ops.gemm(dy.to(cuda_device), W2.to(cuda_device), b_mn_major=True,
             epilogue=N.EPI_GLU_BWD if gated else N.EPI_ACT_BWD, act=0, aux=pre, out=dpre, out2=hid2)
    dhid = _cpu64(dy) @ _cpu64(W2)
    assert_close(dpre, O.apply_activation_backward(dhid, _cpu64(pre), "gelu_tanh", gated), BF16_RTOL, BF16_ATOL, "dpre")
    assert torch.equal(hid2, hid)
    # the same product also emits per-32-row partial column sums of dPre (the input projection's bias gradient):
    # nothing else changes, and the partials add up to the column sums of the stored (rounded) result
    dpre2, hid3 = torch.empty_like(pre), torch.empty_like(hid)
    partial = torch.full(((T + 31) // 32, width), float("nan"), device=cuda_device)
    ops.gemm(dy.to(cuda_device), W2.to(cuda_device), b_mn_major=True,
             epilogue=N.EPI_GLU_BWD if gated else N.EPI_ACT_BWD, act=0, aux=pre, out=dpre2, out2=hid3, colsum=partial)
    assert torch.equal(dpre2, dpre) and torch.equal(hid3, hid)
    assert not torch.isnan(partial).any()
    assert_close(partial[3], _cpu64(dpre[96:128]).sum(0), 1e-5, 1e-4, "one group of 32 rows")
    assert_close(ops.column_sum(partial), _cpu64(dpre).sum(0), 1e-5, 1e-3, "bias gradient from the epilogue")
    # the SIMT path keeps the contract (all sums in the first partial row)
    partial.fill_(float("nan"))
    ops.gemm(dy.to(cuda_device), W2.to(cuda_device), b_mn_major=True, force_simt=True,
             epilogue=N.EPI_GLU_BWD if gated else N.EPI_ACT_BWD, act=0, aux=pre, out=dpre2, out2=hid3, colsum=partial)
    assert_close(ops.column_sum(partial), _cpu64(dpre2).sum(0), 1e-5, 1e-3, "bias gradient, SIMT path")
    ops.check_device_status(cuda_device)


@pytest.mark.parametrize("rank", [128, 8, 60])
def test_gemm_low_rank_continuation(ops, cuda_device, rank):
    torch.manual_seed(rank)
    T, H, Nout = 300, 256, 512
    for dtype, rtol, atol in [(torch.float32, FP32_RTOL, FP32_ATOL), (torch.bfloat16, BF16_RTOL, BF16_ATOL)]:
        x, W = torch.randn(T, H).to(dtype), (torch.randn(Nout, H) * 0.1).to(dtype)
        L1, L2 = (torch.randn(rank, H) * 0.1).to(dtype), (torch.randn(Nout, rank) * 0.1).to(dtype)
        hid = ops.gemm(x.to(cuda_device), L1.to(cuda_device))
        out = ops.gemm(x.to(cuda_device), W.to(cuda_device), a2=hid, b2=L2.to(cuda_device))
        ref = _cpu64(x) @ _cpu64(W).t() + _cpu64(hid) @ _cpu64(L2).t()
        assert_close(out, ref, rtol, atol, f"low-rank continuation {dtype}", scale_atol=True)


# ---- block-sparse ------------------------------------------------------------------------------------
def test_blocksparse_golden_fixture(cuda_device):
    """The reference's own outputs for a rectangular pixelfly layout with block 12 (fp32 mode)."""
    import lean_transformer_b200 as L
    b = {k: torch.from_numpy(v) for k, v in load_golden("blocksparse_matmul").items()}
    x, w, g = b["x"].float().to(cuda_device), b["weight"].float().to(cuda_device), b["g"].float().to(cuda_device)
    out = L.blocksparse_matmul(x, w, b["forward_indices"].to(cuda_device))
    assert_close(out, b["out"], FP32_RTOL, FP32_ATOL, "forward")
    dx, dw = L.blocksparse_matmul_backward(g, x, w, b["backward_indices"].to(cuda_device))
    assert_close(dx, b["grad_input"], FP32_RTOL, FP32_ATOL, "dx")
    assert_close(dw, b["grad_weight"], FP32_RTOL, FP32_ATOL, "dw")
    # autograd through the functional API gives the same gradients
    x2, w2 = x.clone().requires_grad_(), w.clone().requires_grad_()
    L.blocksparse_matmul(x2, w2, b["forward_indices"].to(cuda_device)).backward(g)
    assert torch.equal(x2.grad, dx) and torch.equal(w2.grad, dw)


@pytest.mark.parametrize("in_f,out_f,bs,dtype", [
    (128, 512, 16, torch.float32), (96, 384, 24, torch.float32), (512, 128, 64, torch.float32),
    (512, 2048, 128, torch.bfloat16), (2048, 512, 128, torch.bfloat16), (1024, 1024, 256, torch.bfloat16),
    (512, 512, 64, torch.bfloat16), (4096, 1024, 128, torch.bfloat16)])
def test_blocksparse_native_vs_oracle(cuda_device, in_f, out_f, bs, dtype):
    import lean_transformer_b200 as L
    from lean_transformer_b200.blocksparse import layout as LY
    torch.manual_seed(in_f + bs)
    lay = LY.get_blocksparse_layout(out_f, in_f, f"pixelfly(block_size={bs})")
    fwd, bwd = LY.get_indices_from_layout(lay)
    w = (torch.randn(in_f, bwd.shape[1], bs) * 0.05).to(dtype)
    T = 333
    x, dy = torch.randn(2, T, in_f).to(dtype), torch.randn(2, T, out_f).to(dtype)
    out = L.blocksparse_matmul(x.to(cuda_device), w.to(cuda_device), fwd.to(cuda_device))
    dx, dw = L.blocksparse_matmul_backward(dy.to(cuda_device), x.to(cuda_device), w.to(cuda_device), bwd.to(cuda_device))
    ref_out = O.blocksparse_matmul(_cpu64(x), _cpu64(w), fwd)
    ref_dx, ref_dw = O.blocksparse_matmul_backward(_cpu64(dy), _cpu64(x), _cpu64(w), bwd)
    rtol, atol = (FP32_RTOL, FP32_ATOL) if dtype == torch.float32 else (BF16_RTOL, BF16_ATOL)
    assert_close(out, ref_out, rtol, atol, "out", scale_atol=True)
    assert_close(dx, ref_dx, rtol, atol, "dx", scale_atol=True)
    assert_close(dw, ref_dw, rtol, atol, "dw", scale_atol=True)
    from lean_transformer_b200 import ops as _ops
    _ops.check_device_status(cuda_device)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_blocksparse_fused_epilogues_match_unfused(cuda_device, dtype):
    """Block-sparse products with the gated activation (forward), dropout + residual (forward) and the activation
    backward (input gradient) in their epilogues against the same product followed by the stand-alone kernels."""
    from lean_transformer_b200 import _native as N, ops
    from lean_transformer_b200.blocksparse import layout as LY
    from lean_transformer_b200.blocksparse.native_backend import (_bs_dgrad, _bs_forward, gate_and_linear_blocks_pair_up,
                                                                  native_tables)
    torch.manual_seed(3)
    bs, hidden, inter, tokens = 128, 512, 2048, 400
    fwd1, bwd1 = LY.get_indices_from_layout(LY.get_blocksparse_layout(2 * inter, hidden, f"pixelfly(block_size={bs})"))
    fwd2, bwd2 = LY.get_indices_from_layout(LY.get_blocksparse_layout(hidden, inter, f"pixelfly(block_size={bs})"))
    fwd1, bwd1, fwd2, bwd2 = (t.to(cuda_device) for t in (fwd1, bwd1, fwd2, bwd2))
    w1 = (torch.randn(hidden, bwd1.shape[1], bs, device=cuda_device) * 0.05).to(dtype)
    w2 = (torch.randn(inter, bwd2.shape[1], bs, device=cuda_device) * 0.05).to(dtype)
    b1 = torch.randn(2 * inter, device=cuda_device) * 0.1
    x = torch.randn(tokens, hidden, device=cuda_device).to(dtype)
    t1, t2 = native_tables(fwd1, bwd1, w1.shape[1]), native_tables(fwd2, bwd2, w2.shape[1])
    assert gate_and_linear_blocks_pair_up(t1[0])

    pre_ref = _bs_forward(x, w1, t1[0], 2 * inter, bias=b1)
    hid_ref = ops.activation_forward(pre_ref, True, 0)
    if dtype == torch.bfloat16:  # fp32 runs on the SIMT kernel, which applies the activation as a second pass anyway
        pre, hid = torch.empty_like(pre_ref), torch.empty_like(hid_ref)
        _bs_forward(x, w1, t1[0], 2 * inter, out=pre, bias=b1, epilogue=N.EPI_GLU_FWD, act=0, out2=hid)
        assert torch.equal(pre, pre_ref) and torch.equal(hid, hid_ref)

    res = torch.randn(tokens, hidden, device=cuda_device).to(dtype)
    plain = _bs_forward(hid_ref, w2, t2[0], hidden)
    want = ops.dropout(plain, 0.25, 11, 64, residual=res)
    got = _bs_forward(hid_ref, w2, t2[0], hidden, epilogue=N.EPI_DROPOUT_RESIDUAL, aux=res, dropout_p=0.25, seed=11,
                      elem_offset=64)
    rtol, atol = (BF16_RTOL, BF16_ATOL) if dtype == torch.bfloat16 else (FP32_RTOL, FP32_ATOL)
    assert_close(got, want.double().cpu(), rtol, atol, "dropout + residual in the sparse forward")
    assert torch.equal(got == res, want == res)  # same elements dropped

    dy = torch.randn(tokens, hidden, device=cuda_device).to(dtype)
    dhid = _bs_dgrad(dy, w2, t2[1], inter)
    dpre_ref, hid_again = ops.activation_backward(dhid, pre_ref, True, 0, want_hid=True)
    dpre, hid2 = torch.empty_like(pre_ref), torch.empty_like(hid_ref)
    _bs_dgrad(dy, w2, t2[1], inter, epilogue=N.EPI_GLU_BWD, act=0, aux=pre_ref, out=dpre, out2=hid2)
    assert torch.equal(hid2, hid_ref)
    assert_close(dpre, dpre_ref.double().cpu(), rtol, atol, "activation backward in the sparse input gradient")
    ops.check_device_status(cuda_device)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("world", [1, 2, 3])
def test_gemm_scatter_epilogue_on_one_gpu(ops, cuda_device, out_dtype, world):
    """The reduce-scatter epilogue with every "replica" in this GPU's memory: two products are added into the
    replicas; each replica must hold the sum of both in the 256-row blocks it owns and stay untouched elsewhere."""
    from lean_transformer_b200 import dist as ldist
    torch.manual_seed(world)
    M, N, K, shift = 1024 + 128, 384, 512, 8
    a = [torch.randn(K, M, device=cuda_device).bfloat16() for _ in range(2)]   # weight-gradient form: both MN-major
    b = [torch.randn(K, N, device=cuda_device).bfloat16() for _ in range(2)]
    replicas = [torch.full((M, N), 7.0, device=cuda_device, dtype=out_dtype) for _ in range(world)]
    for rank, rep in enumerate(replicas):  # what begin_step does: zero the owned blocks
        for blk in ldist.owned_row_blocks(M, world, rank, shift):
            rep[blk << shift:(blk + 1) << shift] = 0
    addresses = [r.data_ptr() for r in replicas]
    for i in range(2):
        ops.gemm(a[i], b[i], a_mn_major=True, b_mn_major=True, out=replicas[0], scatter=(addresses, shift))
    torch.cuda.synchronize()
    total = sum(a[i].double().t() @ b[i].double() for i in range(2)).cpu()
    for rank, rep in enumerate(replicas):
        owned = torch.zeros(M, dtype=torch.bool)
        for blk in ldist.owned_row_blocks(M, world, rank, shift):
            owned[blk << shift:(blk + 1) << shift] = True
        got = rep.double().cpu()
        assert torch.equal(got[~owned], torch.full_like(got[~owned], 7.0)), "rows of other owners were touched"
        assert_close(got[owned], total[owned], BF16_RTOL, BF16_ATOL, f"replica {rank}", scale_atol=True)
    # scattered products exist on the tensor-core path only
    with pytest.raises(Exception):
        ops.gemm(a[0].float(), b[0].float(), a_mn_major=True, b_mn_major=True, out=replicas[0].float(),
                 scatter=(addresses, shift))
    ops.check_device_status(cuda_device)


def test_copy_2d_moves_owned_blocks(ops, cuda_device):
    from lean_transformer_b200 import dist as ldist
    rows, cols, world, rank, shift = 2048, 24, 4, 1, 8
    src = torch.randn(rows, cols, device=cuda_device)
    dst = torch.zeros_like(src)
    start, pitch, width, height = ldist.handout_plan(rows, cols, 4, world, rank, shift)
    ops.copy_2d(dst.data_ptr() + start, pitch, src.data_ptr() + start, pitch, width, height)
    torch.cuda.synchronize()
    owned = torch.zeros(rows, dtype=torch.bool)
    for blk in ldist.owned_row_blocks(rows, world, rank, shift):
        owned[blk << shift:(blk + 1) << shift] = True
    assert torch.equal(dst.cpu()[owned], src.cpu()[owned]) and not dst.cpu()[~owned].any()


@pytest.mark.parametrize("bs,dtype", [(16, torch.float32), (128, torch.bfloat16)])
def test_row_major_block_order_operator(cuda_device, bs, dtype):
    """The 'triton' weight order ([1, nnz, bs, bs] in layout.nonzero() order) with an UNBALANCED layout,
    against a dense masked product."""
    from lean_transformer_b200.blocksparse.triton_backend import TritonMatmulForLinearLayer
    torch.manual_seed(bs)
    lay = torch.tensor([[1, 0, 1, 0], [0, 1, 0, 0], [1, 1, 1, 1], [0, 0, 0, 1], [0, 1, 1, 0], [1, 0, 0, 0]], dtype=torch.bool)
    op = TritonMatmulForLinearLayer(lay, bs)
    nnz = int(lay.sum())
    w = (torch.randn(1, nnz, bs, bs) * 0.1).to(dtype)
    dense = torch.zeros(lay.shape[0] * bs, lay.shape[1] * bs, dtype=torch.float64)
    for f, (o, j) in enumerate(lay.nonzero().tolist()):
        dense[o * bs:(o + 1) * bs, j * bs:(j + 1) * bs] = w[0, f].double()
    T = 200
    x = torch.randn(T, lay.shape[1] * bs).to(dtype).to(cuda_device).requires_grad_()
    wd = w.to(cuda_device).requires_grad_()
    out = op(x, wd)
    g = torch.randn(T, lay.shape[0] * bs).to(dtype)
    out.backward(g.to(cuda_device))
    rtol, atol = (FP32_RTOL, FP32_ATOL) if dtype == torch.float32 else (BF16_RTOL, BF16_ATOL)
    assert_close(out, _cpu64(x) @ dense.t(), rtol, atol, "out", scale_atol=True)
    assert_close(x.grad, _cpu64(g) @ dense, rtol, atol, "dx", scale_atol=True)
    dw_dense = _cpu64(g).t() @ _cpu64(x)
    ref_dw = torch.stack([dw_dense[o * bs:(o + 1) * bs, j * bs:(j + 1) * bs] for o, j in lay.nonzero().tolist()])[None]
    assert_close(wd.grad, ref_dw, rtol, atol, "dw", scale_atol=True)
    with pytest.raises(ValueError):
        op.forward_functional(x.detach(), torch.zeros(nnz, bs, bs, device=cuda_device, dtype=dtype))


# ---- argument alignment and the bounded device wait ---------------------------------------------------------
def test_views_offset_by_one_element_take_the_scalar_paths(ops, cuda_device):
    """A C-ABI host may pass any view: a base address that is not a multiple of the vector width must give the
    same numbers through element-wise loads (column sum, LayerNorm forward) or a clean error code, never a
    misaligned-address fault."""
    from lean_transformer_b200 import _native as N
    torch.manual_seed(3)
    for dtype in (torch.float32, torch.bfloat16):
        flat = torch.randn(300 * 64 + 8, device=cuda_device).to(dtype)
        aligned = flat[:300 * 64].view(300, 64)
        shifted = flat[1:1 + 300 * 64].view(300, 64)  # ld % 4 == 0, base off by one element
        assert shifted.data_ptr() % 8 != 0
        expect = _cpu64(shifted).sum(0)
        assert_close(ops.column_sum(shifted), expect, 1e-5, 1e-4, f"column sum of a shifted view ({dtype})")
        assert_close(ops.column_sum(aligned), _cpu64(aligned).sum(0), 1e-5, 1e-4, "aligned view")
        sub = aligned[:, 1:61]  # odd first column, ld 64
        assert_close(ops.column_sum(sub), _cpu64(sub).sum(0), 1e-5, 1e-4, "column window")
    # LayerNorm forward: a shifted (contiguous) matrix goes through the scalar kernel
    flat = torch.randn(40 * 128 + 4, device=cuda_device)
    x = flat[1:1 + 40 * 128].view(40, 128)
    gamma, beta = torch.randn(128, device=cuda_device), torch.randn(128, device=cuda_device)
    ref = O.layer_norm_forward(_cpu64(x), _cpu64(gamma), _cpu64(beta), 1e-12)
    assert_close(ops.layer_norm_forward(x, gamma, beta, 1e-12, torch.float32), ref, FP32_RTOL, FP32_ATOL, "shifted LN")
    # LayerNorm backward and the activations reject such pointers before launching anything
    y = torch.empty(40, 128, device=cuda_device)
    code = N.lib.leanffn_layer_norm_backward(x.data_ptr(), N.F32, x.data_ptr(), N.F32, None, N.F32, None, 0, y.data_ptr(),
                                             N.F32, None, None, None, 40, 128, 1e-5, None)
    assert code == -3 and "align" in N.status_string(code)
    code = N.lib.leanffn_activation_forward(x.data_ptr(), y.data_ptr(), N.F32, 40, 64, 1, 0, None)
    assert code == -3
    torch.cuda.synchronize()


def test_bounded_wait_runs_out_and_reports(ops, cuda_device):
    """A device-side wait that nothing satisfies must return with a status code the host can read; the context
    stays usable.  The probe waits ~1e5 SM clocks on an mbarrier without arrivals, through the same bounded-wait
    and status-word code the GEMM roles use."""
    from lean_transformer_b200 import _native as N
    word = ops.status_word(cuda_device)
    ops.check_device_status(cuda_device)  # clean before
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    N.check(N.lib.leanffn_selftest_wait_timeout(word.data_ptr(), 100000, stream), "selftest")
    torch.cuda.synchronize()
    assert int(word.item()) == 3  # LEANFFN_DEV_TIMEOUT_EPILOGUE
    with pytest.raises(RuntimeError, match="timed out"):
        ops.check_device_status(cuda_device)
    ops.check_device_status(cuda_device)  # the check cleared the word
    # a real product with a short (but sufficient) wait limit still completes, and ordinary calls work afterwards
    a = torch.randn(512, 256, device=cuda_device).bfloat16()
    b = torch.randn(384, 256, device=cuda_device).bfloat16()
    out = ops.gemm(a, b)
    ops.check_device_status(cuda_device)
    assert_close(out, _cpu64(a) @ _cpu64(b).T, BF16_RTOL, BF16_ATOL, "gemm after the probe", scale_atol=True)
    assert N.lib.leanffn_selftest_wait_timeout(None, 1000, stream) == -1


def test_peer_barrier_signals_and_gives_up_within_its_limit(ops, cuda_device):
    """leanffn_peer_barrier with the flag arrays of two "ranks" placed on this one GPU and the peer's arrival written
    by the host: the kernel signals the peer, sees the arrival and returns; without the arrival it gives up after the
    limit, records LEANFFN_DEV_TIMEOUT_PEER and returns (no hang, no trap), and the context stays usable."""
    import ctypes
    from lean_transformer_b200 import _native as N
    flags = torch.zeros(2, 4, 8, dtype=torch.int32, device=cuda_device)  # [rank][channel][source rank]
    table = (ctypes.c_void_p * 8)(flags[0].data_ptr(), flags[1].data_ptr())
    word = ops.status_word(cuda_device)
    ops.check_device_status(cuda_device)
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    flags[0, 1, 1] = 7  # rank 1 has arrived at epoch 7 of channel 1
    N.check(N.lib.leanffn_peer_barrier(table, 0, 2, 1, 7, 100000, word.data_ptr(), stream), "peer barrier")
    torch.cuda.synchronize()
    assert int(word.item()) == 0 and int(flags[1, 1, 0]) == 7  # our signal reached the peer's array
    # a later epoch that the peer never reaches: bounded wait
    N.check(N.lib.leanffn_peer_barrier(table, 0, 2, 1, 8, 100000, word.data_ptr(), stream), "peer barrier")
    torch.cuda.synchronize()
    assert int(word.item()) == 4 and int(flags[1, 1, 0]) == 8
    with pytest.raises(RuntimeError, match="peer rank"):
        ops.check_device_status(cuda_device)
    # epochs compare modulo 2^32: arrival at epoch 1 after the counter wrapped satisfies a wait for epoch 0
    flags[0, 2, 1] = 1
    N.check(N.lib.leanffn_peer_barrier(table, 0, 2, 2, 0, 100000, word.data_ptr(), stream), "peer barrier")
    torch.cuda.synchronize()
    ops.check_device_status(cuda_device)
    assert N.lib.leanffn_peer_barrier(table, 2, 2, 0, 1, 0, None, stream) == -2   # rank outside the world
    assert N.lib.leanffn_peer_barrier(table, 0, 1, 0, 1, 0, None, stream) == 0    # a world of one: nothing to do
