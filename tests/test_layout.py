"""Host-side layout code against golden layouts / index tensors produced by the reference, plus the
properties the reference's own tests pin (tests/test_layout.py densities, tests/test_butterfly.py support)."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from lean_transformer_b200.blocksparse import layout as L


def test_layouts_and_indices_match_reference():
    blob = load_golden("layouts")
    specs = [s.split("|") for s in blob["specs"].tolist()]
    assert len(specs) >= 9
    for n, (out_f, in_f, desc) in enumerate(specs):
        lay = L.get_blocksparse_layout(int(out_f), int(in_f), desc)
        assert np.array_equal(lay.numpy().astype(bool), blob[f"layout_{n}"].astype(bool)), desc
        if f"forward_{n}" in blob:
            fwd, bwd = L.get_indices_from_layout(lay)
            assert fwd.dtype == torch.int32 and bwd.dtype == torch.int64
            assert np.array_equal(fwd.numpy(), blob[f"forward_{n}"]), desc
            assert np.array_equal(bwd.numpy(), blob[f"backward_{n}"]), desc
        else:
            with pytest.raises(AssertionError):
                L.get_indices_from_layout(lay)


def test_pixelfly_closed_form_for_benchmark_shapes():
    """For power-of-two shapes the layout is popcount((r mod m) xor (c mod m)) <= 1 with m the shorter side."""
    for out_f, in_f in [(32768, 4096), (4096, 16384)]:
        lay = L.get_blocksparse_layout(out_f, in_f, "pixelfly(block_size=128)")
        m = min(lay.shape)
        r, c = torch.arange(lay.shape[0])[:, None] % m, torch.arange(lay.shape[1])[None, :] % m
        x = r ^ c
        expect = (x & (x - 1)) == 0
        assert torch.equal(lay, expect)
        assert int(lay.sum(1)[0]) * m // lay.shape[1] == int(np.log2(m)) + 1


@pytest.mark.parametrize("desc,density", [("pixelfly(block_size=4)", 0.5), ("pixelfly(block_size=2)", 0.3125),
                                          ("hypercube(block_size=2, folded=True)", 0.375)])
def test_layout_density_constants(desc, density):
    # square 32 x 32 matrices give the densities the reference asserts for its ALBERT test model
    lay = L.get_blocksparse_layout(32, 32, desc)
    assert abs(float(lay.float().mean()) - density) < 1e-9


def test_descriptor_parsing_and_registry():
    with pytest.raises(ValueError):
        L.get_blocksparse_layout(64, 64, "no_such_layout(8)")
    with pytest.raises(AssertionError):
        L.get_blocksparse_layout(64, 64, "pixelfly")
    with pytest.raises(NotImplementedError):
        L.get_blocksparse_layout(64, 64, "pixelfly(8, 3)")

    @L.register_blocksparse_layout("diag_for_test")
    def diag(out_features, in_features, block_size, width=1):
        n = out_features // block_size
        i = torch.arange(n)
        return (i[:, None] - i[None, :]).abs() % n < width

    lay = L.get_blocksparse_layout(64, 64, "diag_for_test(8, width=2)")
    assert lay.shape == (8, 8) and int(lay.sum()) == 8 + 14


def test_pair_tables_cover_every_block_once():
    lay = L.get_blocksparse_layout(512, 128, "pixelfly(block_size=16)")
    fwd, bwd = L.get_indices_from_layout(lay)
    t_fwd, t_dgrad, t_wgrad = L.tables_from_native_indices(fwd, bwd)
    per_col = bwd.shape[1]
    # forward: (f, j) with j = f // per_col and layout[i, j] set
    for i in range(t_fwd.shape[0]):
        for f, j in t_fwd[i].tolist():
            assert j == f // per_col and lay[i, j] and int(bwd[j, f % per_col]) == i
    # dgrad rows list each block of an input block once; wgrad is the same map seen from the block
    assert sorted(t_dgrad[..., 0].flatten().tolist()) == list(range(t_wgrad.shape[0]))
    for f, (o, j) in enumerate(t_wgrad.tolist()):
        assert lay[o, j] and j == f // per_col
    # row-major (Triton operator) order: unbalanced layouts are allowed
    lay2 = torch.tensor([[1, 0, 1], [0, 1, 0], [1, 1, 1], [0, 0, 1]], dtype=torch.bool)
    fwd2, c2, dgrad2, dc2, wgrad2 = L.tables_from_layout_row_major(lay2)
    assert c2.tolist() == [2, 1, 3, 1] and dc2.tolist() == [2, 2, 3]
    nz = lay2.nonzero().tolist()
    assert wgrad2.tolist() == nz
    for o in range(4):
        for t in range(int(c2[o])):
            f, j = fwd2[o, t].tolist()
            assert nz[f] == [o, j]


def test_native_index_buffers_are_validated_before_any_kernel_uses_them():
    """Entries of the index buffers become addresses inside the kernels: corrupt buffers must raise on the host."""
    import pytest
    from lean_transformer_b200.blocksparse.native_backend import _validate_indices
    layout = L.get_blocksparse_layout(512, 256, "pixelfly(block_size=32)")
    fwd, bwd = L.get_indices_from_layout(layout)
    per_input = bwd.shape[1]
    _validate_indices(fwd, bwd, per_input)
    _validate_indices(fwd, None, per_input)
    _validate_indices(None, bwd, per_input)
    bad = fwd.clone(); bad[0, 0] = fwd.numel() + 3  # out of range
    with pytest.raises(ValueError):
        _validate_indices(bad, None, per_input)
    bad = fwd.clone(); bad[0, 0] = bad[0, 1]  # not a permutation
    with pytest.raises(ValueError):
        _validate_indices(bad, bwd, per_input)
    bad = bwd.clone(); bad[0, 0] = -1
    with pytest.raises(ValueError):
        _validate_indices(fwd, bad, per_input)
    bad = bwd.clone(); bad[0, 0] = (int(bad[0, 0]) + 1) % fwd.shape[0]  # disagrees with forward_indices
    with pytest.raises(ValueError):
        _validate_indices(fwd, bad, per_input)
    with pytest.raises(ValueError):
        _validate_indices(fwd, bwd, per_input + 1)
