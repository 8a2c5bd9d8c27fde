"""Block-order converters (native <-> Triton <-> dense) against the oracle's block-by-block definition."""
import pytest
import torch

from oracle import leanffn_oracle as O


@pytest.mark.parametrize("out_f,in_f,bs,spec", [(256, 64, 16, "pixelfly"), (64, 256, 16, "pixelfly"), (128, 128, 32, "pixelfly"),
                                                  (256, 128, 8, "hypercube(folded=True)"), (512, 128, 64, "pixelfly")])
def test_native_triton_dense_round_trips(out_f, in_f, bs, spec):
    from lean_transformer_b200.blocksparse import convert as C, layout as LY
    name = f"{spec[:-1]}, block_size={bs})" if spec.endswith(")") else f"{spec}(block_size={bs})"
    layout = LY.get_blocksparse_layout(out_f, in_f, name)
    fwd, bwd = LY.get_indices_from_layout(layout)
    gen = torch.Generator().manual_seed(out_f + bs)
    native = torch.randn(in_f, bwd.shape[1], bs, generator=gen, dtype=torch.float64)
    dense = C.native_weight_to_dense(native, bwd, out_f)
    # the dense matrix is what the oracle's native product computes
    x = torch.randn(7, in_f, generator=gen, dtype=torch.float64)
    assert torch.allclose(O.blocksparse_matmul(x, native, fwd), x @ dense.t(), rtol=1e-12, atol=1e-12)
    # its support is exactly the layout
    support = dense.reshape(out_f // bs, bs, in_f // bs, bs).abs().amax(dim=(1, 3)) > 0
    assert torch.equal(support, layout.to(torch.bool))
    triton = C.native_to_triton_weight(native, bwd, layout)
    assert triton.shape == (1, int(layout.sum()), bs, bs)
    assert torch.equal(C.triton_weight_to_dense(triton, layout), dense)
    assert torch.equal(C.triton_to_native_weight(triton, bwd, layout), native)
    assert torch.equal(C.dense_to_native_weight(dense, bwd, bs), native)
    # blocks sit in layout.nonzero() order
    coords = layout.nonzero()
    k = int(coords.shape[0]) // 2
    o, i = coords[k].tolist()
    assert torch.equal(triton[0, k], dense[o * bs:(o + 1) * bs, i * bs:(i + 1) * bs])


def test_mismatched_layout_is_rejected():
    from lean_transformer_b200.blocksparse import convert as C, layout as LY
    layout = LY.get_blocksparse_layout(128, 128, "pixelfly(block_size=16)")
    _, bwd = LY.get_indices_from_layout(layout)
    other = layout.clone()
    o, i = (~layout).nonzero()[0].tolist()
    other[o, i] = True
    with pytest.raises(ValueError):
        C.native_to_triton_permutation(bwd, other)


def test_round_trips_on_random_balanced_layouts():
    """Circulant layouts with a random set of offsets are balanced (same number of blocks per row and per column), the
    case the native order supports; the converters must round-trip on all of them."""
    from hypothesis import given, settings, strategies as st

    from lean_transformer_b200.blocksparse import convert as C, layout as LY

    @settings(max_examples=40, deadline=None)
    @given(st.integers(2, 12), st.integers(1, 3), st.sets(st.integers(0, 11), min_size=1, max_size=5), st.integers(0, 2**31))
    def check(n, reps, offsets, seed):
        offsets = sorted({o % n for o in offsets})
        base = torch.zeros(n, n, dtype=torch.bool)
        rows = torch.arange(n)
        for o in offsets:
            base[rows, (rows + o) % n] = True
        layout = base.repeat(reps, 1)  # [reps*n out blocks, n in blocks]: still balanced
        fwd, bwd = LY.get_indices_from_layout(layout)
        bs = 4
        gen = torch.Generator().manual_seed(seed)
        native = torch.randn(n * bs, bwd.shape[1], bs, generator=gen, dtype=torch.float64)
        dense = C.native_weight_to_dense(native, bwd, layout.shape[0] * bs)
        triton = C.native_to_triton_weight(native, bwd, layout)
        assert torch.equal(C.triton_weight_to_dense(triton, layout), dense)
        assert torch.equal(C.triton_to_native_weight(triton, bwd, layout), native)
        x = torch.randn(3, n * bs, generator=gen, dtype=torch.float64)
        assert torch.allclose(O.blocksparse_matmul(x, native, fwd), x @ dense.t(), rtol=1e-12, atol=1e-12)

    check()
