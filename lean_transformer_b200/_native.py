"""ctypes binding of ``libleanffn_b200.so`` (declared in ``include/leanffn_b200.h``).

The library is the only compute path of this package.  If it is missing or does not load, importing
this module raises: there is no PyTorch / CPU fallback behind it.
"""
import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int32, c_int64, c_size_t, c_uint64, c_void_p
from pathlib import Path

LIB_NAME = "libleanffn_b200.so"
# LEANFFN_LIBRARY names another build of the same library (for example a measurement build); default: next to this file
LIB_PATH = Path(os.environ["LEANFFN_LIBRARY"]).resolve() if os.environ.get("LEANFFN_LIBRARY") else \
    Path(__file__).resolve().parent / LIB_NAME

# element types / activations / epilogues: keep in sync with include/leanffn_b200.h
F32, BF16, TF32 = 0, 1, 2
ABI_VERSION = 4
ACT_GELU_TANH, ACT_GELU_ERF, ACT_RELU, ACT_SILU, ACT_TANH, ACT_SIGMOID, ACT_IDENTITY = range(7)
EPI_STORE, EPI_GLU_FWD, EPI_ACT_FWD, EPI_DROPOUT_RESIDUAL, EPI_GLU_BWD, EPI_ACT_BWD = range(6)
DEV_STATUS_NAMES = {0: "ok", 1: "TMA producer wait timed out", 2: "MMA wait timed out", 3: "epilogue wait timed out",
                    4: "wait for a peer rank timed out"}


class GemmDesc(ctypes.Structure):
    """Mirror of ``leanffn_gemm_desc``."""

    _fields_ = [
        ("M", c_int32), ("N", c_int32), ("K", c_int32), ("in_dtype", c_int32),
        ("A", c_void_p), ("lda", c_int64), ("a_mn_major", c_int32), ("b_mn_major", c_int32),
        ("B", c_void_p), ("ldb", c_int64),
        ("A2", c_void_p), ("B2", c_void_p), ("lda2", c_int64), ("ldb2", c_int64), ("K2", c_int32),
        ("bs_mode", c_int32), ("bs_block", c_int32), ("bs_nnz", c_int32), ("bs_num_blocks", c_int32),
        ("bs_index", c_void_p), ("bs_count", c_void_p),
        ("epilogue", c_int32), ("act", c_int32),
        ("D", c_void_p), ("ldd", c_int64), ("d_dtype", c_int32),
        ("D2", c_void_p), ("ldd2", c_int64),
        ("bias", c_void_p), ("bias_dtype", c_int32),
        ("aux", c_void_p), ("ldaux", c_int64), ("aux_dtype", c_int32),
        ("dropout_p", c_float), ("seed", c_uint64), ("elem_offset", c_uint64),
        ("status_word", c_void_p), ("force_simt", c_int32), ("max_ctas", c_int32),
        ("scatter_world", c_int32), ("scatter_block_shift", c_int32), ("scatter_D", c_void_p * 8),
        ("bs_wgrad_pairs", c_int32), ("wait_limit_cycles", c_int64),
        ("colsum_partial", c_void_p), ("ld_colsum", c_int64), ("timer", c_void_p),
        ("tf32_k_slice", c_int32),
    ]


class LinearDesc(ctypes.Structure):
    """Mirror of ``leanffn_linear_desc``."""

    _fields_ = [
        ("weight", c_void_p), ("bias", c_void_p), ("bias_dtype", c_int32), ("rank", c_int32),
        ("lowrank_first", c_void_p), ("lowrank_second", c_void_p),
        ("bs_block", c_int32), ("bs_num_blocks", c_int32),
        ("fwd_index", c_void_p), ("fwd_count", c_void_p), ("fwd_nnz", c_int32), ("dgrad_nnz", c_int32),
        ("dgrad_index", c_void_p), ("dgrad_count", c_void_p), ("wgrad_index", c_void_p),
        ("wgrad_pairs", c_int32), ("fuse_gated_forward", c_int32),
    ]


class FfnDesc(ctypes.Structure):
    """Mirror of ``leanffn_ffn_desc``."""

    _fields_ = [
        ("tokens", c_int64), ("hidden", c_int32), ("intermediate", c_int32),
        ("gated", c_int32), ("act", c_int32), ("residual", c_int32),
        ("compute_dtype", c_int32), ("io_dtype", c_int32), ("grad_out_dtype", c_int32), ("param_dtype", c_int32),
        ("eps", c_float), ("dropout_p", c_float), ("seed", c_uint64), ("elem_offset", c_uint64),
        ("ln_weight", c_void_p), ("ln_bias", c_void_p),
        ("i2h", LinearDesc), ("h2o", LinearDesc),
        ("status_word", c_void_p), ("max_ctas", c_int32), ("timer", c_void_p),
    ]


class FfnGrads(ctypes.Structure):
    """Mirror of ``leanffn_ffn_grads``."""

    _fields_ = [(name, c_void_p) for name in (
        "grad_input", "grad_ln_weight", "grad_ln_bias", "grad_i2h_weight", "grad_i2h_bias", "grad_i2h_lowrank_first",
        "grad_i2h_lowrank_second", "grad_h2o_weight", "grad_h2o_bias", "grad_h2o_lowrank_first",
        "grad_h2o_lowrank_second")]


class AttentionDesc(ctypes.Structure):
    """Mirror of ``leanffn_attention_desc``."""

    _fields_ = [
        ("batch", c_int32), ("heads", c_int32), ("q_len", c_int32), ("kv_len", c_int32), ("head_dim", c_int32),
        ("causal", c_int32), ("scale", c_float), ("dropout_p", c_float),
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("ld_q", c_int64), ("ld_k", c_int64), ("ld_v", c_int64),
        ("mask", c_void_p), ("mask_stride_b", c_int64), ("mask_stride_h", c_int64), ("mask_stride_q", c_int64),
        ("out", c_void_p), ("ld_out", c_int64), ("lse", c_void_p),
        ("d_out", c_void_p), ("ld_dout", c_int64), ("delta", c_void_p), ("dq_accum", c_void_p),
        ("dk", c_void_p), ("dv", c_void_p), ("ld_dk", c_int64), ("ld_dv", c_int64),
        ("status_word", c_void_p), ("wait_limit_cycles", c_int64), ("seed", c_uint64), ("elem_offset", c_uint64),
    ]


_SIGNATURES = {
    "leanffn_attention_forward": (c_int32, [POINTER(AttentionDesc), c_void_p]),
    "leanffn_attention_backward": (c_int32, [POINTER(AttentionDesc), c_void_p]),
    "leanffn_rotary": (c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int32, c_int64,
                                 c_int32, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "leanffn_abi_version": (c_int32, []),
    "leanffn_status_string": (c_char_p, [c_int32]),
    "leanffn_layer_norm_forward": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_int32, c_void_p, c_int32, c_int64,
                                             c_int64, c_float, c_float, c_uint64, c_uint64, c_void_p, c_int32,
                                             c_void_p]),
    "leanffn_layer_norm_backward_scratch_bytes": (c_size_t, [c_int64, c_int64]),
    "leanffn_layer_norm_backward": (c_int32, [c_void_p, c_int32, c_void_p, c_int32, c_void_p, c_int32, c_void_p, c_int32,
                                              c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                              c_float, c_void_p]),
    "leanffn_activation_forward": (c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_int64, c_int32, c_int32, c_void_p]),
    "leanffn_activation_backward": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int64,
                                              c_int32, c_int32, c_void_p]),
    "leanffn_dropout": (c_int32, [c_void_p, c_int32, c_void_p, c_int32, c_int64, c_float, c_uint64, c_uint64, c_void_p,
                                  c_int32, c_void_p]),
    "leanffn_dropout_colsum_scratch_bytes": (c_size_t, [c_int64, c_int64]),
    "leanffn_dropout_colsum": (c_int32, [c_void_p, c_int32, c_void_p, c_int32, c_int64, c_int64, c_float, c_uint64,
                                         c_uint64, c_void_p, c_void_p, c_void_p]),
    "leanffn_dropout_mask": (c_int32, [c_void_p, c_int64, c_float, c_uint64, c_uint64, c_void_p]),
    "leanffn_column_sum_scratch_bytes": (c_size_t, [c_int64, c_int64]),
    "leanffn_column_sum": (c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "leanffn_column_sum_static_capacity": (c_int64, []),
    "leanffn_column_sum_static": (c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_int64, c_int64, c_void_p]),
    "leanffn_cast": (c_int32, [c_void_p, c_int32, c_void_p, c_int32, c_int64, c_void_p]),
    "leanffn_transpose": (c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_int64, c_int64, c_void_p]),
    "leanffn_copy_2d": (c_int32, [c_void_p, c_uint64, c_void_p, c_uint64, c_uint64, c_uint64, c_void_p]),
    "leanffn_split_tf32": (c_int32, [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int32, c_int64, c_void_p]),
    "leanffn_gemm": (c_int32, [POINTER(GemmDesc), c_void_p]),
    "leanffn_selftest_wait_timeout": (c_int32, [c_void_p, c_int64, c_void_p]),
    "leanffn_peer_barrier": (c_int32, [POINTER(c_void_p), c_int32, c_int32, c_int32, ctypes.c_uint32, c_int64, c_void_p,
                                       c_void_p]),
    "leanffn_timer_create": (c_int32, [c_int32, POINTER(c_void_p)]),
    "leanffn_timer_reset": (c_int32, [c_void_p]),
    "leanffn_timer_summary": (c_int32, [c_void_p, POINTER(ctypes.c_double), POINTER(ctypes.c_double), POINTER(c_int32),
                                        POINTER(c_int32)]),
    "leanffn_timer_destroy": (c_int32, [c_void_p]),
    "leanffn_ffn_workspace_bytes": (c_size_t, [POINTER(FfnDesc), c_int32]),
    "leanffn_ffn_forward": (c_int32, [POINTER(FfnDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p]),
    "leanffn_ffn_backward": (c_int32, [POINTER(FfnDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       POINTER(FfnGrads), c_void_p, c_void_p]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)


class NativeLibraryError(RuntimeError):
    pass


def _load():
    if not LIB_PATH.exists():
        raise NativeLibraryError(
            f"{LIB_PATH} is missing. Build it with `python -m lean_transformer_b200.build` (needs nvcc); "
            "this package has no fallback path without its CUDA library."
        )
    try:
        lib = ctypes.CDLL(os.fspath(LIB_PATH))
    except OSError as e:  # pragma: no cover - depends on the machine
        raise NativeLibraryError(f"could not load {LIB_PATH}: {e}") from e
    for name, (restype, argtypes) in _SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise NativeLibraryError(f"{LIB_PATH} does not export {name}") from e
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.leanffn_abi_version() != ABI_VERSION:
        raise NativeLibraryError("libleanffn_b200.so has an unexpected ABI version; rebuild it")
    return lib


lib = _load()


def status_string(code: int) -> str:
    return lib.leanffn_status_string(int(code)).decode()


def check(code: int, what: str):
    """Raise if a C-ABI call reported a non-zero status."""
    if code != 0:
        raise RuntimeError(f"{what} failed with status {code}: {status_string(code)}")
