"""The allocation-free column sum (leanffn_column_sum_static) against the regular entry point.

Some users of the C ABI cannot give the library scratch memory: a Go / Rust / C++ host that binds only the
shared library has no tensor allocator, and a process whose own pool owns the whole device (or that must not
hit cudaMalloc's implicit synchronisation inside its step loop) cannot allocate per call.  For them the
partial sums live in a fixed array inside the library.  This test drives that entry point through ctypes
exactly as such a host would (raw pointers, no scratch argument) and checks it, twice in a row because the
array is shared between calls and keeps the previous call's contents.

The file name sorts last so that a run stopping at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _column_sum_both(N, x):
    rows, cols = x.shape
    stream = torch.cuda.current_stream(x.device).cuda_stream
    dt = N.BF16 if x.dtype == torch.bfloat16 else N.F32
    out_static = torch.full((cols,), float("nan"), dtype=torch.float32, device=x.device)
    code = N.lib.leanffn_column_sum_static(x.data_ptr(), dt, x.stride(0), out_static.data_ptr(), rows, cols, stream)
    assert code == 0, N.status_string(code)
    out_ref = torch.empty(cols, dtype=torch.float32, device=x.device)
    nbytes = N.lib.leanffn_column_sum_scratch_bytes(rows, cols)
    scratch = torch.empty(max(nbytes, 4) // 4, dtype=torch.float32, device=x.device)
    code = N.lib.leanffn_column_sum(x.data_ptr(), dt, x.stride(0), out_ref.data_ptr(), scratch.data_ptr(), rows, cols,
                                    stream)
    assert code == 0, N.status_string(code)
    torch.cuda.synchronize(x.device)
    return out_static, out_ref


def test_static_scratch_column_sum_matches_regular_entry_point(cuda_device):
    from lean_transformer_b200 import _native as N

    assert N.lib.leanffn_column_sum_static_capacity() == 1 << 18
    torch.manual_seed(0)
    # two calls in a row with different shapes and dtypes: the second must not see the first one's partials
    first = torch.randn(16384, 1024, device=cuda_device).bfloat16()
    second = torch.randn(5000, 777, device=cuda_device)
    for x in (first, second, first):
        got, ref = _column_sum_both(N, x)
        # same kernels, same reduction order: identical bits; the usual fp32 tolerance as a backstop
        assert torch.equal(got, ref)
        torch.testing.assert_close(got, x.float().sum(0), rtol=1e-4, atol=1e-4 * float(x.float().abs().sum(0).max()))
    # a sliced (strided) input and a single-chunk problem
    wide = torch.randn(40, 4096, device=cuda_device)
    got, ref = _column_sum_both(N, wide[:, 128:2048])
    assert torch.equal(got, ref)


def test_static_scratch_rejects_what_does_not_fit(cuda_device):
    from lean_transformer_b200 import _native as N

    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    out = torch.zeros(65536 + 128, dtype=torch.float32, device=cuda_device)
    big = torch.empty(1, dtype=torch.float32, device=cuda_device)  # never dereferenced: the call is rejected first
    code = N.lib.leanffn_column_sum_static(big.data_ptr(), N.F32, 65536 + 128, out.data_ptr(), 4096, 65536 + 128, stream)
    assert code == -7 and "maximum" in N.status_string(code)  # beyond 65536 columns: refused before any launch
    assert N.lib.leanffn_column_sum_static(big.data_ptr(), N.F32, 4, out.data_ptr(), 8, 16, stream) == -2  # ld < cols
    assert N.lib.leanffn_column_sum_static(None, N.F32, 16, out.data_ptr(), 8, 16, stream) == -1
    # zero rows: defined result (zeros), still no allocation
    out.fill_(1.0)
    assert N.lib.leanffn_column_sum_static(None, N.F32, 16, out.data_ptr(), 0, 16, stream) == 0
    torch.cuda.synchronize(cuda_device)
    assert float(out[:16].abs().sum()) == 0.0 and float(out[16]) == 1.0
