"""Block-sparse layouts (host side): the registry and descriptor strings of the reference
(lean_transformer/blocksparse/layout.py:15-53), its pixelfly / hypercube generators (:56-153) and
the conversion of a boolean layout into the index tensors the module stores (:177-210), plus the
pair tables the CUDA kernels consume.

The generators are written directly in terms of block coordinates: a butterfly of size n with the
first ``n_factors`` factors connects positions r and c iff r == c or r ^ c is a single bit below
``n_factors``.
"""
import ast
import math
from typing import Callable, Dict, Optional, Tuple

import torch

from ..utils import get_logger

logger = get_logger(__name__)
REGISTERED_LAYOUTS: Dict[str, Callable] = {}


def register_blocksparse_layout(name: str):
    """Decorator: make ``fn(out_features, in_features, *args, **kwargs) -> BoolTensor`` available under ``name``."""

    def _register(fn: Callable):
        if name in REGISTERED_LAYOUTS:
            logger.warning(f"Overwriting layout {name} with {fn}.")
        REGISTERED_LAYOUTS[name] = fn
        return fn

    return _register


def get_blocksparse_layout(out_features: int, in_features: int, layout: str) -> torch.BoolTensor:
    """Evaluate a descriptor such as ``"pixelfly(block_size=128)"`` into a boolean
    [out_features // block, in_features // block] incidence matrix."""
    assert "(" in layout and layout.endswith(")"), "descriptor format must be name(foo=123, bar='456')"
    call = ast.parse(layout.strip(), mode="eval").body
    if not isinstance(call, ast.Call) or not isinstance(call.func, ast.Name):
        raise ValueError(f"cannot parse layout descriptor {layout!r}")
    name = call.func.id
    if name not in REGISTERED_LAYOUTS:
        raise ValueError(f"Unknown layout name {name}, supported layouts: {tuple(REGISTERED_LAYOUTS.keys())}")
    args = [ast.literal_eval(node) for node in call.args]
    kwargs = {kw.arg: ast.literal_eval(kw.value) for kw in call.keywords}
    return REGISTERED_LAYOUTS[name](out_features, in_features, *args, **kwargs)


def _butterfly_mask(size: int, n_factors: int) -> torch.Tensor:
    """[size, size] bool: r ~ c iff they are equal or differ in exactly one of the low ``n_factors`` bits."""
    idx = torch.arange(size)
    diff = idx[:, None] ^ idx[None, :]
    single_low_bit = torch.zeros(size, size, dtype=torch.bool)
    for bit in range(n_factors):
        single_low_bit |= diff == (1 << bit)
    return single_low_bit | (diff == 0)


def _deinterleave(layout: torch.Tensor) -> torch.Tensor:
    """Non-stretched rectangular layouts: regroup the longer axis so the square pattern repeats as tiles."""
    out_blocks, in_blocks = layout.shape
    if out_blocks > in_blocks:
        ratio = out_blocks // in_blocks
        return layout.view(out_blocks // ratio, ratio, in_blocks).permute(1, 0, 2).reshape(out_blocks, in_blocks)
    if out_blocks < in_blocks:
        ratio = in_blocks // out_blocks
        return layout.view(out_blocks, in_blocks // ratio, ratio).permute(0, 2, 1).reshape(out_blocks, in_blocks)
    return layout


@register_blocksparse_layout("pixelfly")
def get_butterfly_layout(out_features: int, in_features: int, block_size: int = 256,
                         butterfly_size: Optional[int] = None, n_factors: Optional[int] = None,
                         stretch: bool = False) -> torch.BoolTensor:
    """Sum of blocky butterfly factors (https://arxiv.org/abs/2112.00029), without the low-rank term.

    :param block_size: the layout is made of dense [block_size x block_size] blocks
    :param butterfly_size: logical butterfly size; defaults to the shorter side in blocks (rounded up to
      a power of two).  A smaller value tiles the pattern.
    :param n_factors: number of butterfly factors, default log2(butterfly_size)
    :param stretch: stretch the pattern over a rectangular matrix instead of repeating the square one
    """
    if butterfly_size is None:
        butterfly_size = 2 ** int(math.ceil(math.log2(min(in_features, out_features) / block_size)))
    assert out_features % in_features == 0 or in_features % out_features == 0, \
        "if matrix is not square, the longer dimension must be a multiple of the shorter dimension"
    assert out_features % block_size == 0 and in_features % block_size == 0
    log_n = int(math.log2(butterfly_size))
    n_factors = log_n if n_factors is None else n_factors
    if butterfly_size != 2 ** log_n or butterfly_size < 2:
        raise NotImplementedError("butterfly_size must be a power of 2")
    if not (1 <= n_factors <= log_n):
        raise NotImplementedError("n_factors must be a between 1 and log_2(butterfly_size)")

    mask = _butterfly_mask(butterfly_size, n_factors)
    out_blocks, in_blocks = out_features // block_size, in_features // block_size
    # Feature f of an axis with F features belongs to butterfly position f // (F // butterfly_size); a block is
    # active iff any of its features meets any feature of the other block through the mask.
    rep_out, rep_in = out_features // butterfly_size, in_features // butterfly_size
    assert rep_out > 0 and rep_in > 0, "butterfly_size exceeds the matrix size"

    def positions(num_blocks: int, rep: int) -> Tuple[torch.Tensor, torch.Tensor]:
        first = (torch.arange(num_blocks) * block_size) // rep
        last = ((torch.arange(num_blocks) + 1) * block_size - 1) // rep
        return first, last

    of, ol = positions(out_blocks, rep_out)
    jf, jl = positions(in_blocks, rep_in)
    # inclusive 2-D prefix sums of the mask give "any" over position rectangles
    csum = torch.zeros(butterfly_size + 1, butterfly_size + 1, dtype=torch.int64)
    csum[1:, 1:] = mask.to(torch.int64).cumsum(0).cumsum(1)
    r0, r1 = of[:, None], ol[:, None] + 1
    c0, c1 = jf[None, :], jl[None, :] + 1
    layout = (csum[r1, c1] - csum[r0, c1] - csum[r1, c0] + csum[r0, c0]) > 0
    if not stretch:
        layout = _deinterleave(layout)
    return layout


@register_blocksparse_layout("hypercube")
def get_hypercube_layout(out_features: int, in_features: int, block_size: int, stretch: bool = False,
                         folded: bool = False) -> torch.BoolTensor:
    """Pixelfly seen as a hypercube graph over blocks; ``folded`` adds the edge between antipodal nodes
    (https://en.wikipedia.org/wiki/Folded_cube_graph)."""
    smaller = min(out_features, in_features)
    assert math.log2(smaller / block_size).is_integer(), """layout dimension must be a power of 2"""
    assert out_features % smaller == 0 and in_features % smaller == 0
    dim = int(math.ceil(math.log2(smaller / block_size)))
    layout = get_butterfly_layout(smaller, smaller, block_size, n_factors=dim, stretch=False).clone()
    side = 2 ** dim
    assert layout.shape == (side, side)
    if folded:
        nodes = torch.arange(side)
        antipodes = (side - 1) - nodes  # all `dim` bits flipped
        assert not layout[nodes, antipodes].any()
        layout[nodes, antipodes] = True
    reps_out, reps_in = out_features // smaller, in_features // smaller
    if stretch:
        return layout[:, None, :, None].repeat(1, reps_out, 1, reps_in).flatten(-2, -1).flatten(0, 1)
    return layout.repeat(reps_out, reps_in)


def butterfly_factor_to_matrix(twiddle: torch.Tensor, factor_index: int) -> torch.Tensor:
    """Dense [n, n] matrix of one butterfly factor with base b: twiddle is [n // b, b, b]; factor
    ``factor_index`` mixes positions whose base-b digit number ``factor_index`` differs
    (lean_transformer/blocksparse/layout.py:156-174)."""
    n_div_b, b, b2 = twiddle.shape
    assert b == b2
    n = n_div_b * b
    log_b_n = int(round(math.log(n) / math.log(b)))
    assert n == b ** log_b_n, f"n must be a power of {b}"
    assert 0 <= factor_index <= log_b_n
    stride = b ** factor_index
    out = torch.zeros(n, n, dtype=twiddle.dtype)
    pos = torch.arange(n)
    low, digit, high = pos % stride, (pos // stride) % b, pos // (stride * b)
    group = high * stride + low  # which [b x b] twiddle block this position uses
    for other in range(b):
        src = high * stride * b + other * stride + low
        out[pos, src] = twiddle[group, digit, other]
    return out


def get_indices_from_layout(layout: torch.BoolTensor) -> Tuple[torch.IntTensor, torch.LongTensor]:
    """Boolean [out_blocks, in_blocks] layout -> (forward_indices int32 [out_blocks, per_row],
    backward_indices int64 [in_blocks, per_col]).  Weight block (j, a) of input block j goes to output block
    backward_indices[j, a]; forward_indices[i] lists the flat ids j * per_col + a feeding output block i.
    The layout must be balanced (same count in every row, same count in every column)."""
    layout = layout.bool()
    out_blocks, in_blocks = layout.shape
    per_row, per_col = layout.sum(1).unique(), layout.sum(0).unique()
    assert len(per_row) == 1, "butterfly layout must have the same number of blocks per row"
    assert len(per_col) == 1, "butterfly layout must have the same number of blocks per row"
    per_row, per_col = int(per_row.item()), int(per_col.item())
    # slot of output block i among the active outputs of input block j (ascending output order)
    slot = layout.to(torch.int64).cumsum(0) - 1  # [out_blocks, in_blocks]
    out_idx, in_idx = layout.nonzero(as_tuple=True)  # row-major: sorted by output block, then input block
    forward = (in_idx * per_col + slot[out_idx, in_idx]).view(out_blocks, per_row)
    in_sorted, out_sorted = layout.t().nonzero(as_tuple=True)
    backward = out_sorted.view(in_blocks, per_col)
    return forward.to(torch.int32), backward.to(torch.int64)


# ---- tables for the CUDA kernels -------------------------------------------------------------------
def tables_from_native_indices(forward_indices: torch.Tensor, backward_indices: torch.Tensor):
    """int32 pair tables for the three block-sparse products over the native weight order
    (weight block id f = j * blocks_per_input + a):
      forward [out_blocks, per_row, 2] = (f, j);  dgrad [in_blocks, per_col, 2] = (f, o);
      wgrad [num_blocks, 2] = (o, j)."""
    in_blocks, per_col = backward_indices.shape
    f_fwd = forward_indices.to(torch.int64)
    fwd = torch.stack([f_fwd, f_fwd // per_col], dim=-1)
    f_bwd = torch.arange(in_blocks * per_col, device=backward_indices.device).view(in_blocks, per_col)
    dgrad = torch.stack([f_bwd, backward_indices.to(torch.int64)], dim=-1)
    wgrad = torch.stack([backward_indices.to(torch.int64).flatten(), f_bwd.flatten() // per_col], dim=-1)
    return (fwd.to(torch.int32).contiguous(), dgrad.to(torch.int32).contiguous(),
            wgrad.to(torch.int32).contiguous())


def tables_from_layout_row_major(layout: torch.Tensor):
    """Pair tables for weights stored in ``layout.nonzero()`` order (the Triton operator's order): rows may
    hold different numbers of blocks, so each table comes with a per-row count.
    Returns (fwd, fwd_count, dgrad, dgrad_count, wgrad)."""
    layout = layout.bool().cpu()
    out_blocks, in_blocks = layout.shape
    out_idx, in_idx = layout.nonzero(as_tuple=True)
    nnz = out_idx.numel()
    block_id = torch.arange(nnz)
    row_counts, col_counts = layout.sum(1), layout.sum(0)
    max_row, max_col = max(int(row_counts.max()), 1), max(int(col_counts.max()), 1)
    fwd = torch.zeros(out_blocks, max_row, 2, dtype=torch.int32)
    dgrad = torch.zeros(in_blocks, max_col, 2, dtype=torch.int32)
    row_pos = torch.zeros(out_blocks, dtype=torch.int64)
    col_pos = torch.zeros(in_blocks, dtype=torch.int64)
    for f, o, j in zip(block_id.tolist(), out_idx.tolist(), in_idx.tolist()):
        fwd[o, row_pos[o], 0], fwd[o, row_pos[o], 1] = f, j
        dgrad[j, col_pos[j], 0], dgrad[j, col_pos[j], 1] = f, o
        row_pos[o] += 1
        col_pos[j] += 1
    wgrad = torch.stack([out_idx, in_idx], dim=-1).to(torch.int32)
    return fwd, row_counts.to(torch.int32), dgrad, col_counts.to(torch.int32), wgrad.contiguous()
