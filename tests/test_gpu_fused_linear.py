"""linear -> dropout -> + residual as one product (the tail of the reference's attention block, attn.py:74-78)
against the same arithmetic in float64 with the kernel's own dropout mask injected."""
import pytest
import torch

from conftest import BF16_ATOL, BF16_RTOL, FP32_ATOL, FP32_RTOL, assert_close
from oracle import leanffn_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["fp32", "autocast"])
@pytest.mark.parametrize("kind", ["dense", "pixelfly"])
def test_linear_dropout_residual(cuda_device, mode, kind):
    import lean_transformer_b200 as L
    tokens, fin, fout, p = 300, 512, 512, 0.2
    torch.manual_seed(3)
    if kind == "dense":
        linear = torch.nn.Linear(fin, fout).to(cuda_device)
        dense_weight = lambda: linear.weight.detach().double().cpu()  # noqa: E731
    else:
        from lean_transformer_b200.blocksparse import convert as C
        linear = L.GeneralizedLinear(L.GeneralizedMatrix(fin, fout, "pixelfly(block_size=128)", 0)).to(cuda_device)
        dense_weight = lambda: C.native_weight_to_dense(linear.matrix.weight.detach().double().cpu(),  # noqa: E731
                                                        linear.matrix.backward_indices.cpu(), fout)
    with torch.no_grad():
        linear.bias.normal_(0, 0.1)
    x = torch.randn(2, tokens // 2, fin, device=cuda_device, requires_grad=True)
    res = torch.randn(2, tokens // 2, fout, device=cuda_device, requires_grad=True)   # fp32 residual stream
    g = torch.randn(2, tokens // 2, fout, device=cuda_device)

    torch.manual_seed(77)  # the mask is keep(seed = 77, element offset = 0)
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=mode == "autocast"):
        out = L.linear_dropout_residual(x, linear, res, p=p, training=True)
    assert out.dtype == torch.float32 and out.shape == res.shape
    out.backward(g)
    L.check_device_status(cuda_device)

    keep = torch.from_numpy(O.dropout_keep_mask(tokens * fout, p, 77, 0)).view(tokens, fout).double()
    W, b = dense_weight(), linear.bias.detach().double().cpu()
    x64, g64 = x.detach().double().cpu().view(tokens, fin), g.double().cpu().view(tokens, fout)
    if mode == "autocast":  # the kernel multiplies bf16 copies of x and W
        x64, W = x64.float().bfloat16().double(), W.float().bfloat16().double()
    lin = x64 @ W.t() + b
    ref_out = lin * keep / (1 - p) + res.detach().double().cpu().view(tokens, fout)
    gy = g64 * keep / (1 - p)
    rtol, atol = (BF16_RTOL, BF16_ATOL) if mode == "autocast" else (FP32_RTOL, FP32_ATOL)
    branch = lin * keep / (1 - p)
    assert_close(out.view(tokens, fout), ref_out, rtol, atol, "out", branch=branch, scale_atol=True)
    assert_close(x.grad.view(tokens, fin), gy @ W, rtol, atol, "dx", scale_atol=True)
    assert torch.equal(res.grad, g)
    assert_close(linear.bias.grad, gy.sum(0), rtol, atol, "db", scale_atol=True)
    if kind == "dense":
        assert_close(linear.weight.grad, gy.t() @ x64, rtol, atol, "dW", scale_atol=True)
    else:
        from lean_transformer_b200.blocksparse import convert as C
        got = C.native_weight_to_dense(linear.matrix.weight.grad.double().cpu(), linear.matrix.backward_indices.cpu(), fout)
        mask = C.native_weight_to_dense(torch.ones_like(linear.matrix.weight.grad, dtype=torch.float64).cpu(),
                                        linear.matrix.backward_indices.cpu(), fout)
        assert_close(got, (gy.t() @ x64) * mask, rtol, atol, "dW", scale_atol=True)
    # eval mode / p = 0: plain linear + residual
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16, enabled=mode == "autocast"):
        plain = L.linear_dropout_residual(x, linear, res, p=p, training=False)
    assert_close(plain.view(tokens, fout), lin + res.detach().double().cpu().view(tokens, fout), rtol, atol, "eval",
                 branch=lin, scale_atol=True)
