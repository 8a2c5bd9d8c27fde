"""Tensor-level wrappers over the C ABI: they take CUDA ``torch.Tensor``s, allocate outputs and
scratch through torch's caching allocator, and launch on torch's current stream.  PyTorch is used for
device memory and streams only; every computation is a kernel of ``libleanffn_b200.so``.
"""
from typing import Optional, Tuple

import torch

from . import _native as N

_DTYPES = {torch.float32: N.F32, torch.bfloat16: N.BF16}
_status_words = {}

# Bookkeeping for benchmarks: kernels launched by this package, an optional per-GEMM CUDA-event timer and the
# persistent-grid cap used while a collective shares the GPU.
launch_count = 0
_gemm_timer = None
_max_ctas = 0


def set_max_ctas(n: int):
    """Cap the tensor-core GEMM's persistent grid at ``n`` CTAs (0 = one per SM)."""
    global _max_ctas
    _max_ctas = int(n)


class GemmTimer:
    """Times every GEMM launch of the library while it is active (``with GemmTimer() as t: ...``): the C ABI records
    a CUDA-event pair around each ``leanffn_gemm`` kernel on the launching stream, also for the launches made inside
    the whole-block calls, together with the launch's algorithmic FLOPs (2 * M * N * K_effective), so a benchmark
    can report the kernel's achieved rate.  Launches beyond ``capacity`` are counted, not timed."""

    def __init__(self, capacity: int = 8192):
        import ctypes
        handle = ctypes.c_void_p()
        N.check(N.lib.leanffn_timer_create(int(capacity), ctypes.byref(handle)), "leanffn_timer_create")
        self.handle = handle

    def __enter__(self):
        global _gemm_timer
        N.check(N.lib.leanffn_timer_reset(self.handle), "leanffn_timer_reset")
        _gemm_timer = self
        return self

    def __exit__(self, *exc):
        global _gemm_timer
        _gemm_timer = None

    def summary(self):
        """(total_flops, total_seconds, launches) of the timed launches; waits for their events."""
        import ctypes
        flops, seconds = ctypes.c_double(), ctypes.c_double()
        timed, dropped = ctypes.c_int32(), ctypes.c_int32()
        N.check(N.lib.leanffn_timer_summary(self.handle, ctypes.byref(flops), ctypes.byref(seconds), ctypes.byref(timed),
                                            ctypes.byref(dropped)), "leanffn_timer_summary")
        self.dropped = dropped.value
        return flops.value, seconds.value, timed.value

    def __del__(self):
        try:
            N.lib.leanffn_timer_destroy(self.handle)
        except Exception:
            pass


def _timer_handle():
    return _gemm_timer.handle if _gemm_timer is not None else None



def _dt(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}: the kernels take float32 and bfloat16") from None


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "lean_transformer_b200 runs on CUDA tensors only (sm_100a kernels); got a tensor on "
                f"{t.device}. There is no CPU path."
            )


def _count(n: int = 1):
    global launch_count
    launch_count += n


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def status_word(device) -> torch.Tensor:
    """int32 device word that kernels write when a bounded wait gives up."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _status_words[key]


def check_device_status(device=None):
    """Synchronising check of the device-side status word; raises if a kernel reported a timeout."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    word = status_word(device)
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise RuntimeError(f"device-side status {code}: {N.DEV_STATUS_NAMES.get(code, 'unknown')}")


# ---- row kernels ----------------------------------------------------------------------------------
def layer_norm_forward(x: torch.Tensor, gamma: Optional[torch.Tensor], beta: Optional[torch.Tensor], eps: float,
                       out_dtype: torch.dtype, dropout_p: float = 0.0, seed: int = 0, elem_offset: int = 0,
                       residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(x, gamma, beta, residual)
    assert x.dim() == 2 and x.is_contiguous()
    rows, cols = x.shape
    y = torch.empty((rows, cols), dtype=out_dtype, device=x.device)
    if gamma is not None:
        assert gamma.is_contiguous() and gamma.numel() == cols
        assert beta is None or (beta.dtype == gamma.dtype and beta.is_contiguous())
    if residual is not None:
        assert residual.shape == x.shape and residual.is_contiguous()
    pdt = _dt(gamma) if gamma is not None else (_dt(beta) if beta is not None else N.F32)
    N.check(N.lib.leanffn_layer_norm_forward(
        _ptr(x), _dt(x), _ptr(gamma), _ptr(beta), pdt, _ptr(y), _dt(y), rows, cols, float(eps), float(dropout_p),
        int(seed), int(elem_offset), _ptr(residual), _dt(residual) if residual is not None else 0, _stream(x)),
        "leanffn_layer_norm_forward")
    _count()
    return y


def layer_norm_backward(dy: torch.Tensor, x: torch.Tensor, gamma: Optional[torch.Tensor], eps: float,
                        dresidual: Optional[torch.Tensor], dx_dtype: Optional[torch.dtype], need_dx: bool = True,
                        need_param_grads: bool = True
                        ) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], Optional[torch.Tensor]]:
    _require_cuda(dy, x, gamma, dresidual)
    assert dy.dim() == 2 and dy.is_contiguous() and x.is_contiguous() and dy.shape == x.shape
    rows, cols = x.shape
    dx = torch.empty((rows, cols), dtype=dx_dtype or x.dtype, device=x.device) if need_dx else None
    dgamma = dbeta = scratch = None
    if need_param_grads:
        dgb = torch.empty((2, cols), dtype=torch.float32, device=x.device)
        dgamma, dbeta = dgb[0], dgb[1]
        nbytes = N.lib.leanffn_layer_norm_backward_scratch_bytes(rows, cols)
        scratch = torch.empty(max(nbytes, 4) // 4, dtype=torch.float32, device=x.device)
    if dresidual is not None:
        assert dresidual.shape == x.shape and dresidual.is_contiguous()
    N.check(N.lib.leanffn_layer_norm_backward(
        _ptr(dy), _dt(dy), _ptr(x), _dt(x), _ptr(gamma), _dt(gamma) if gamma is not None else N.F32,
        _ptr(dresidual), _dt(dresidual) if dresidual is not None else 0, _ptr(dx), _dt(dx) if dx is not None else 0,
        _ptr(dgamma), _ptr(dbeta), _ptr(scratch), rows, cols, float(eps), _stream(x)),
        "leanffn_layer_norm_backward")
    _count(3 if need_param_grads else 1)
    return dx, dgamma, dbeta


def activation_forward(pre: torch.Tensor, gated: bool, act: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(pre, out)
    assert pre.dim() == 2 and pre.is_contiguous()
    rows = pre.shape[0]
    inter = pre.shape[1] // 2 if gated else pre.shape[1]
    hid = out if out is not None else torch.empty((rows, inter), dtype=pre.dtype, device=pre.device)
    assert hid.shape == (rows, inter) and hid.dtype == pre.dtype and hid.is_contiguous()
    N.check(N.lib.leanffn_activation_forward(_ptr(pre), _ptr(hid), _dt(pre), rows, inter, int(gated), act,
                                             _stream(pre)), "leanffn_activation_forward")
    _count()
    return hid


def activation_backward(dhid: torch.Tensor, pre: torch.Tensor, gated: bool, act: int, want_hid: bool = False,
                        out: Optional[torch.Tensor] = None, hid_out: Optional[torch.Tensor] = None):
    _require_cuda(dhid, pre, out, hid_out)
    assert pre.dim() == 2 and pre.is_contiguous() and dhid.is_contiguous() and dhid.dtype == pre.dtype
    rows = pre.shape[0]
    inter = pre.shape[1] // 2 if gated else pre.shape[1]
    assert dhid.shape == (rows, inter)
    dpre = out if out is not None else torch.empty_like(pre)
    assert dpre.shape == pre.shape and dpre.dtype == pre.dtype and dpre.is_contiguous()
    hid = hid_out if hid_out is not None else (torch.empty_like(dhid) if want_hid else None)
    assert hid is None or (hid.shape == dhid.shape and hid.dtype == dhid.dtype and hid.is_contiguous())
    N.check(N.lib.leanffn_activation_backward(_ptr(dhid), _ptr(pre), _ptr(dpre), _ptr(hid), _dt(pre), rows, inter,
                                              int(gated), act, _stream(pre)), "leanffn_activation_backward")
    _count()
    return dpre, hid


def dropout(x: torch.Tensor, p: float, seed: int, elem_offset: int, out_dtype: Optional[torch.dtype] = None,
            residual: Optional[torch.Tensor] = None):
    """y = dropout(x) [+ residual]; p == 0 makes it a cast (+ add)."""
    _require_cuda(x, residual)
    assert x.is_contiguous()
    y = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    if residual is not None:
        assert residual.is_contiguous() and residual.numel() == x.numel()
    N.check(N.lib.leanffn_dropout(_ptr(x), _dt(x), _ptr(y), _dt(y), x.numel(), float(p), int(seed), int(elem_offset),
                                  _ptr(residual), _dt(residual) if residual is not None else 0, _stream(x)),
            "leanffn_dropout")
    _count()
    return y


def dropout_colsum(x: torch.Tensor, p: float, seed: int, elem_offset: int, out_dtype: Optional[torch.dtype] = None):
    """(y, colsum): y = dropout(x) cast to ``out_dtype`` and the fp32 column sums of y, one pass over x."""
    _require_cuda(x)
    assert x.dim() == 2 and x.is_contiguous()
    rows, cols = x.shape
    y = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    out = torch.empty(cols, dtype=torch.float32, device=x.device)
    nbytes = N.lib.leanffn_dropout_colsum_scratch_bytes(rows, cols)
    scratch = torch.empty(max(nbytes, 4) // 4, dtype=torch.float32, device=x.device)
    N.check(N.lib.leanffn_dropout_colsum(_ptr(x), _dt(x), _ptr(y), _dt(y), rows, cols, float(p), int(seed),
                                         int(elem_offset), _ptr(out), _ptr(scratch), _stream(x)), "leanffn_dropout_colsum")
    _count(3)
    return y, out


def dropout_mask(numel: int, p: float, seed: int, elem_offset: int, device) -> torch.Tensor:
    mask = torch.empty(numel, dtype=torch.uint8, device=device)
    _require_cuda(mask)
    N.check(N.lib.leanffn_dropout_mask(_ptr(mask), numel, float(p), int(seed), int(elem_offset), _stream(mask)),
            "leanffn_dropout_mask")
    return mask


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
        return x
    _require_cuda(x)
    x = x.contiguous()
    y = torch.empty(x.shape, dtype=dtype, device=x.device)
    N.check(N.lib.leanffn_cast(_ptr(x), _dt(x), _ptr(y), _dt(y), x.numel(), _stream(x)), "leanffn_cast")
    _count()
    return y


def column_sum(x: torch.Tensor) -> torch.Tensor:
    _require_cuda(x)
    assert x.dim() == 2 and x.stride(1) == 1
    rows, cols = x.shape
    out = torch.empty(cols, dtype=torch.float32, device=x.device)
    nbytes = N.lib.leanffn_column_sum_scratch_bytes(rows, cols)
    scratch = torch.empty(max(nbytes, 4) // 4, dtype=torch.float32, device=x.device)
    N.check(N.lib.leanffn_column_sum(_ptr(x), _dt(x), x.stride(0), _ptr(out), _ptr(scratch), rows, cols, _stream(x)),
            "leanffn_column_sum")
    _count(2)
    return out


def transpose(x: torch.Tensor) -> torch.Tensor:
    _require_cuda(x)
    assert x.dim() == 2 and x.stride(1) == 1
    rows, cols = x.shape
    y = torch.empty((cols, rows), dtype=x.dtype, device=x.device)
    N.check(N.lib.leanffn_transpose(_ptr(x), _dt(x), x.stride(0), _ptr(y), rows, cols, _stream(x)),
            "leanffn_transpose")
    return y


# ---- fp32 products on the tensor cores ---------------------------------------------------------------
# fp32 mode multiplies on the tensor cores as three TF32 products folded into one reduction axis (see
# leanffn_split_tf32 in the header); shapes the kernel does not take (tiny, odd or strided ones) use the SIMT kernel.
_fp32_tensor_cores = True
# Reduction-axis elements per slice.  The tensor cores truncate their fp32 accumulator after every instruction, a
# bias that grows with the number of instructions that add into a full-size accumulator.  Each slice multiplies the
# two small cross terms first and the large hi x hi term last (see leanffn_split_tf32), so only a third of a slice's
# instructions see a full-size accumulator.  Measured on the 4096-token fp32 configuration against an fp64 run, as
# the worst |error| / (1e-4 + 1e-4 |ref|) over all outputs and gradients: 1.84 at 1024, 0.99 at 384, 0.59 at 256,
# 0.38 at 128 (exact fp32 FMA arithmetic: 1.08); step time 2.5 / 2.9 / 3.4 / 5.0 ms.
_TF32_SLICE = 256


def set_fp32_tensor_cores(enabled: bool) -> bool:
    """Switch fp32 products between the TF32x3 tensor-core path (default) and the fp32 SIMT kernel."""
    global _fp32_tensor_cores
    previous, _fp32_tensor_cores = _fp32_tensor_cores, bool(enabled)
    return previous


def _split_tf32(x: torch.Tensor, role: int, slice_width: int) -> torch.Tensor:
    rows, cols = x.shape
    out = torch.empty((rows, 3 * cols), dtype=torch.float32, device=x.device)
    N.check(N.lib.leanffn_split_tf32(_ptr(x), x.stride(0), _ptr(out), rows, cols, role, slice_width, _stream(x)),
            "leanffn_split_tf32")
    _count()
    return out


def _gemm_fp32_tensor(a, b, a_mn_major, b_mn_major, out, out_dtype, bias, epilogue, act, out2, aux, dropout_p, seed,
                      elem_offset):
    """fp32 product on the tensor cores with the fused-epilogue semantics of ``gemm``; NotImplemented if the shape
    or the arguments do not fit (the caller then takes the SIMT kernel)."""
    m, k = (a.shape[1], a.shape[0]) if a_mn_major else a.shape
    n = b.shape[1] if b_mn_major else b.shape[0]
    wide = 2 * n if epilogue == N.EPI_GLU_BWD else n
    if m < 64 or n < 64 or k < 32 or k % 4 or n % 8 or (out_dtype not in (None, torch.float32)):
        return NotImplemented
    if out is not None and (out.dtype != torch.float32 or not out.is_contiguous() or out.shape != (m, wide)):
        return NotImplemented
    if bias is not None and bias.dtype != torch.float32:
        return NotImplemented
    if aux is not None and (aux.dtype != torch.float32 or not aux.is_contiguous()):
        return NotImplemented
    backward_kind = epilogue in (N.EPI_GLU_BWD, N.EPI_ACT_BWD)
    a_k = transpose(a) if a_mn_major else a
    b_k = transpose(b) if b_mn_major else b
    plain = out if (out is not None and not backward_kind) else torch.empty((m, n), dtype=torch.float32, device=a.device)
    # the accumulators truncate: the reduction axis is cut into short slices that the kernel accumulates one by one,
    # keeping the running fp32 sum in the result (one launch; the split kernels lay the slices out)
    slice_width = _TF32_SLICE if _TF32_SLICE % 32 == 0 else 0
    a3 = _split_tf32(a_k, 0, slice_width or k)
    b3 = _split_tf32(b_k, 1, slice_width or k)
    d = N.GemmDesc()
    d.M, d.N, d.K = int(m), int(n), int(3 * k)
    d.in_dtype = N.TF32
    d.A, d.lda = a3.data_ptr(), 3 * k
    d.B, d.ldb = b3.data_ptr(), 3 * k
    d.epilogue = N.EPI_STORE
    d.D, d.ldd, d.d_dtype = _ptr(plain), n, N.F32
    if bias is not None and not backward_kind:
        d.bias, d.bias_dtype = _ptr(bias), N.F32
    d.tf32_k_slice = 3 * slice_width
    d.status_word = _ptr(status_word(a.device))
    d.max_ctas = _max_ctas
    d.timer = _timer_handle()
    _count()
    N.check(N.lib.leanffn_gemm(d, _stream(a)), "leanffn_gemm")
    if epilogue == N.EPI_STORE:
        return plain
    if epilogue == N.EPI_DROPOUT_RESIDUAL:
        if dropout_p == 0.0 and aux is None:
            return plain
        return dropout(plain, dropout_p, seed, elem_offset, residual=aux)
    gated = epilogue in (N.EPI_GLU_FWD, N.EPI_GLU_BWD)
    if not backward_kind:
        activation_forward(plain, gated, act, out=out2)
        return plain
    dpre, _ = activation_backward(plain, aux, gated, act, want_hid=out2 is not None, out=out, hid_out=out2)
    return dpre


# ---- GEMM -----------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool = False, b_mn_major: bool = False,
         M: Optional[int] = None, N_: Optional[int] = None, K: Optional[int] = None,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
         bias: Optional[torch.Tensor] = None, epilogue: int = N.EPI_STORE, act: int = 0,
         out2: Optional[torch.Tensor] = None, aux: Optional[torch.Tensor] = None,
         a2: Optional[torch.Tensor] = None, b2: Optional[torch.Tensor] = None,
         dropout_p: float = 0.0, seed: int = 0, elem_offset: int = 0,
         bs_mode: int = 0, bs_block: int = 0, bs_nnz: int = 0, bs_num_blocks: int = 0,
         bs_index: Optional[torch.Tensor] = None, bs_count: Optional[torch.Tensor] = None,
         force_simt: bool = False, scatter=None, bs_wgrad_pairs: bool = False,
         colsum: Optional[torch.Tensor] = None) -> torch.Tensor:
    """D = A(m,k) . B(n,k) with the fused epilogues of ``leanffn_gemm`` (see include/leanffn_b200.h).

    Dense operands are 2-D with unit inner stride: a K-major A is [M, K], an MN-major A is [K, M];
    a K-major B is [N, K] (so D = A @ B.T), an MN-major B is [K, N].

    ``scatter = (replica_addresses, block_shift)``: instead of being stored, the result is added into the replica
    of ``out`` that owns each row block (``out`` is this rank's replica; see ``scatter_world`` in the header).

    ``colsum`` (activation-backward epilogues, bf16): fp32 ``[ceil(M / 32), columns of out]`` buffer that receives
    per-32-row partial column sums of the result; ``column_sum(colsum)`` is then the bias gradient.
    """
    _require_cuda(a, b, out, bias, out2, aux, a2, b2, bs_index, bs_count)
    assert a.dim() == 2 and a.stride(1) == 1 and a.dtype == b.dtype
    if (a.dtype == torch.float32 and _fp32_tensor_cores and not force_simt and bs_mode == 0 and a2 is None
            and scatter is None and colsum is None and b.dim() == 2 and b.stride(1) == 1):
        result = _gemm_fp32_tensor(a, b, a_mn_major, b_mn_major, out, out_dtype, bias, epilogue, act, out2, aux,
                                   dropout_p, seed, elem_offset)
        if result is not NotImplemented:
            return result
    d = N.GemmDesc()
    if bs_mode == 0:
        assert b.dim() == 2 and b.stride(1) == 1
        m, k = (a.shape[1], a.shape[0]) if a_mn_major else a.shape
        n, kb = (b.shape[1], b.shape[0]) if b_mn_major else b.shape
        assert k == kb, f"reduction mismatch: {k} vs {kb}"
        d.ldb = b.stride(0)
    else:
        assert b.is_contiguous() and M is not None and N_ is not None and K is not None
        m, n, k = M, N_, K
        assert bs_index is not None and bs_index.dtype == torch.int32 and bs_index.is_contiguous()
        d.ldb = b.stride(0) if bs_mode == 3 else bs_block
    d.M, d.N, d.K = int(m), int(n), int(k)
    d.in_dtype = _dt(a)
    d.A, d.lda = _ptr(a), a.stride(0)
    d.B = _ptr(b)
    d.a_mn_major, d.b_mn_major = int(a_mn_major), int(b_mn_major)
    if a2 is not None:
        assert b2 is not None and a2.stride(1) == 1 and b2.stride(1) == 1 and a2.dtype == a.dtype == b2.dtype
        d.A2, d.B2, d.lda2, d.ldb2 = _ptr(a2), _ptr(b2), a2.stride(0), b2.stride(0)
        d.K2 = a2.shape[0] if a_mn_major else a2.shape[1]
    d.bs_mode, d.bs_block, d.bs_nnz, d.bs_num_blocks = bs_mode, bs_block, bs_nnz, bs_num_blocks
    d.bs_index = _ptr(bs_index)
    if bs_count is not None:
        assert bs_count.dtype == torch.int32 and bs_count.is_contiguous()
        d.bs_count = _ptr(bs_count)
    d.epilogue, d.act = epilogue, act
    if out is None:
        cols = 2 * n if epilogue == N.EPI_GLU_BWD else n
        out = torch.empty((m, cols), dtype=out_dtype or a.dtype, device=a.device)
    assert out.stride(-1) == 1
    d.D, d.ldd, d.d_dtype = _ptr(out), out.stride(0) if out.dim() == 2 else n, _dt(out)
    if out2 is not None:
        assert out2.dtype == out.dtype and out2.stride(1) == 1
        d.D2, d.ldd2 = _ptr(out2), out2.stride(0)
    if bias is not None:
        assert bias.is_contiguous()
        d.bias, d.bias_dtype = _ptr(bias), _dt(bias)
    if aux is not None:
        assert aux.stride(1) == 1
        d.aux, d.ldaux, d.aux_dtype = _ptr(aux), aux.stride(0), _dt(aux)
    d.dropout_p, d.seed, d.elem_offset = float(dropout_p), int(seed), int(elem_offset)
    d.status_word = _ptr(status_word(a.device))
    d.force_simt = int(force_simt)
    d.max_ctas = _max_ctas
    d.bs_wgrad_pairs = int(bs_wgrad_pairs)
    if colsum is not None:
        assert colsum.dtype == torch.float32 and colsum.dim() == 2 and colsum.stride(1) == 1
        assert colsum.shape[0] == (m + 31) // 32 and colsum.shape[1] == out.shape[-1]
        d.colsum_partial, d.ld_colsum = _ptr(colsum), colsum.stride(0)
    if scatter is not None:
        addresses, shift = scatter
        assert 1 <= len(addresses) <= 8 and epilogue == N.EPI_STORE and bias is None and out.dim() == 2
        d.scatter_world, d.scatter_block_shift = len(addresses), int(shift)
        for i, address in enumerate(addresses):
            d.scatter_D[i] = int(address)
    global launch_count
    launch_count += 1
    d.timer = _timer_handle()
    N.check(N.lib.leanffn_gemm(d, _stream(a)), "leanffn_gemm")
    return out


def copy_2d(dst_ptr: int, dst_pitch: int, src_ptr: int, src_pitch: int, width_bytes: int, height: int, stream=None):
    """Strided device-to-device copy by raw addresses (``leanffn_copy_2d``); with peer addresses it runs on a copy
    engine.  ``stream``: a ``torch.cuda.Stream`` (default: the current one)."""
    handle = (stream or torch.cuda.current_stream()).cuda_stream
    N.check(N.lib.leanffn_copy_2d(int(dst_ptr), int(dst_pitch), int(src_ptr), int(src_pitch), int(width_bytes),
                                  int(height), handle), "leanffn_copy_2d")


# ---- the whole block in one call ------------------------------------------------------------------------------------
def ffn_workspace(desc, backward: bool, device) -> torch.Tensor:
    nbytes = N.lib.leanffn_ffn_workspace_bytes(desc, int(backward))
    if nbytes == 0:
        raise RuntimeError("leanffn_ffn_workspace_bytes rejected the block descriptor")
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


def ffn_forward(desc, x, out, pre_activation, i2h_lowrank_hid, h2o_lowrank_hid, launches: int):
    """``leanffn_ffn_forward`` on torch tensors; ``launches`` = kernels the call enqueues (bookkeeping only)."""
    workspace = ffn_workspace(desc, False, x.device)
    desc.status_word = _ptr(status_word(x.device))
    desc.max_ctas = _max_ctas
    desc.timer = _timer_handle()
    N.check(N.lib.leanffn_ffn_forward(desc, _ptr(x), _ptr(out), _ptr(pre_activation), _ptr(i2h_lowrank_hid),
                                      _ptr(h2o_lowrank_hid), _ptr(workspace), _stream(x)), "leanffn_ffn_forward")
    _count(launches)


def ffn_backward(desc, grad_out, x, pre_activation, i2h_lowrank_hid, h2o_lowrank_hid, grads, launches: int):
    workspace = ffn_workspace(desc, True, x.device)
    desc.status_word = _ptr(status_word(x.device))
    desc.max_ctas = _max_ctas
    desc.timer = _timer_handle()
    N.check(N.lib.leanffn_ffn_backward(desc, _ptr(grad_out), _ptr(x), _ptr(pre_activation), _ptr(i2h_lowrank_hid),
                                       _ptr(h2o_lowrank_hid), grads, _ptr(workspace), _stream(x)), "leanffn_ffn_backward")
    _count(launches)


# ---- attention core ---------------------------------------------------------------------------------------------------
def _rows_view(t: torch.Tensor) -> torch.Tensor:
    """[batch, len, width] tensor whose (batch, len) rows lie at one pitch (e.g. a slice of a fused qkv output); anything
    else is made contiguous."""
    if t.dim() != 3:
        raise ValueError(f"expected [batch, len, hidden], got {tuple(t.shape)}")
    if t.stride(2) == 1 and t.stride(0) == t.shape[1] * t.stride(1) and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


def rotary(x: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], heads: int, *, inverse: bool = False,
           out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotary embedding of x [batch, len, heads * head_dim] with fp32 tables [>= len, head_dim] (``leanffn_rotary``);
    ``inverse`` applies the transposed rotation (gradients).  Without tables: a dtype conversion into a contiguous
    tensor.  ``out``: write into this tensor instead (same shape; a column slice of a wider tensor is fine)."""
    _require_cuda(x)
    x = _rows_view(x)
    batch, length, width = x.shape
    head_dim = width // heads
    if cos is not None:
        if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.stride(-1) != 1 or sin.stride() != cos.stride():
            raise ValueError("rotary tables must be float32 with unit inner stride and equal pitches")
        if cos.shape[0] < length or cos.shape[-1] != head_dim:
            raise ValueError(f"rotary tables {tuple(cos.shape)} do not cover length {length} x head_dim {head_dim}")
    if out is None:
        y = torch.empty(batch, length, width, dtype=out_dtype, device=x.device)
    else:
        y = out
        if y.shape != x.shape or y.stride(2) != 1 or y.stride(0) != length * y.stride(1):
            raise ValueError(f"rotary output {tuple(y.shape)} / strides {y.stride()} does not match the input rows")
    N.check(N.lib.leanffn_rotary(_ptr(x), _dt(x), x.stride(1), _ptr(cos), _ptr(sin), 0 if cos is None else cos.stride(0),
                                 _ptr(y), _dt(y), y.stride(1), batch, length, heads, head_dim, int(inverse), _stream(x)),
            "leanffn_rotary")
    _count()
    return y


def _mask_strides(mask: Optional[torch.Tensor], batch: int, heads: int, q_len: int, kv_len: int):
    """(tensor kept alive, strides over batch / head / query) of an additive mask broadcastable to
    [batch, heads, q_len, kv_len]."""
    if mask is None:
        return None, (0, 0, 0)
    if not torch.is_floating_point(mask):
        raise TypeError("expected float mask with negative values for masked items")
    if mask.dim() == 3:
        mask = mask.unsqueeze(1)
    if mask.dim() != 4:
        raise ValueError(f"attention mask must be [batch, (heads), q_len, kv_len], got {tuple(mask.shape)}")
    if mask.dtype != torch.float32 or mask.shape[-1] != kv_len or mask.stride(-1) != 1:
        mask = mask.to(torch.float32).expand(*mask.shape[:-1], kv_len).contiguous()
    for size, full in zip(mask.shape[:3], (batch, heads, q_len)):
        if size not in (1, full):
            raise ValueError(f"attention mask {tuple(mask.shape)} does not broadcast to "
                             f"[{batch}, {heads}, {q_len}, {kv_len}]")
    strides = tuple(0 if mask.shape[i] == 1 else mask.stride(i) for i in range(3))
    return mask, strides


def _attention_desc(q, k, v, heads, scale, mask, causal, dropout_p=0.0, seed=0, elem_offset=0):
    batch, q_len, width = q.shape
    kv_len = k.shape[1]
    if width % heads != 0:
        raise ValueError(f"hidden size {width} is not a multiple of {heads} heads")
    head_dim = width // heads
    if head_dim % 16 != 0 or head_dim > 128:
        raise NotImplementedError(f"attention kernels take head sizes that are multiples of 16 up to 128, got {head_dim}")
    for t in (q, k, v):
        if t.dtype != torch.bfloat16:
            raise TypeError("attention kernels compute in bfloat16 (run under autocast or pass bfloat16 tensors)")
    if k.shape != v.shape or k.shape[0] != batch or k.shape[2] != width:
        raise ValueError(f"query {tuple(q.shape)}, key {tuple(k.shape)}, value {tuple(v.shape)} do not match")
    mask, (sb, sh, sq) = _mask_strides(mask, batch, heads, q_len, kv_len)
    d = N.AttentionDesc()
    d.batch, d.heads, d.q_len, d.kv_len, d.head_dim = batch, heads, q_len, kv_len, head_dim
    d.causal, d.scale = int(causal), float(scale)
    d.dropout_p, d.seed, d.elem_offset = float(dropout_p), int(seed), int(elem_offset)
    d.q, d.k, d.v = _ptr(q), _ptr(k), _ptr(v)
    d.ld_q, d.ld_k, d.ld_v = q.stride(1), k.stride(1), v.stride(1)
    d.mask, d.mask_stride_b, d.mask_stride_h, d.mask_stride_q = _ptr(mask), sb, sh, sq
    d.status_word = _ptr(status_word(q.device))
    return d, mask


def attention_forward(q, k, v, heads: int, scale: float, mask=None, causal: bool = False, dropout_p: float = 0.0,
                      seed: int = 0, elem_offset: int = 0):
    """softmax(scale * q.k^T + mask).v per head (``leanffn_attention_forward``).  q [batch, q_len, hidden], k / v
    [batch, kv_len, hidden] bfloat16 (slices of one qkv tensor are taken in place).  ``dropout_p`` > 0 drops attention
    probabilities with the Philox mask of (seed, elem_offset) over the [batch, heads, q_len, kv_len] index space.
    Returns (out bfloat16 [batch, q_len, hidden], lse float32 [batch, heads, q_len] for the backward pass)."""
    _require_cuda(q, k, v, mask)
    q, k, v = _rows_view(q), _rows_view(k), _rows_view(v)
    d, mask = _attention_desc(q, k, v, heads, scale, mask, causal, dropout_p, seed, elem_offset)
    out = torch.empty(q.shape, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(q.shape[0], heads, q.shape[1], dtype=torch.float32, device=q.device)
    d.out, d.ld_out, d.lse = _ptr(out), out.stride(1), _ptr(lse)
    N.check(N.lib.leanffn_attention_forward(d, _stream(q)), "leanffn_attention_forward")
    _count()
    return out, lse


def attention_backward(d_out, q, k, v, out, lse, heads: int, scale: float, mask=None, causal: bool = False,
                       dropout_p: float = 0.0, seed: int = 0, elem_offset: int = 0, out_dk=None, out_dv=None):
    """Gradients of ``attention_forward`` (``leanffn_attention_backward``) for the same (mask, causal, dropout_p, seed,
    elem_offset): (dq float32 [batch, q_len, hidden], dk, dv bfloat16 [batch, kv_len, hidden]).  ``out_dk`` / ``out_dv``:
    bfloat16 tensors to write dk / dv into (row views of a wider tensor are fine)."""
    _require_cuda(d_out, q, k, v, out, lse, mask)
    q, k, v, d_out = _rows_view(q), _rows_view(k), _rows_view(v), _rows_view(d_out)
    if d_out.dtype != torch.bfloat16:
        d_out = d_out.to(torch.bfloat16)
    d, mask = _attention_desc(q, k, v, heads, scale, mask, causal, dropout_p, seed, elem_offset)
    dq = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    dk = out_dk if out_dk is not None else torch.empty(k.shape, dtype=torch.bfloat16, device=q.device)
    dv = out_dv if out_dv is not None else torch.empty(k.shape, dtype=torch.bfloat16, device=q.device)
    for t in (dk, dv):
        if t.dtype != torch.bfloat16 or t.shape != k.shape or t.stride(2) != 1 or t.stride(0) != t.shape[1] * t.stride(1):
            raise ValueError("dk / dv outputs must be bfloat16 row views of the key shape")
    delta = torch.empty_like(lse)
    d.out, d.ld_out, d.lse = _ptr(out), out.stride(1), _ptr(lse)
    d.d_out, d.ld_dout, d.delta, d.dq_accum = _ptr(d_out), d_out.stride(1), _ptr(delta), _ptr(dq)
    d.dk, d.dv, d.ld_dk, d.ld_dv = _ptr(dk), _ptr(dv), dk.stride(1), dv.stride(1)
    N.check(N.lib.leanffn_attention_backward(d, _stream(q)), "leanffn_attention_backward")
    _count(3)
    return dq, dk, dv
