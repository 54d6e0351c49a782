"""The oracle and the input generators against vectors produced by the reference's own modules.

For every verification case of the reference (5 nominal seeds, its fuzz list, its accuracy list) the
generator must reproduce the reference's inputs bit for bit and the float64 restatement must reproduce
the reference's truth (sampled positions, NaN/Inf counts, selected index sets)."""
import numpy as np
import pytest

from oracle import ref64
from tests._golden import check_inputs, check_truth, golden, sha
from verified_metal_kernels_b200 import ops

BIG = {("prefix", "L2_3"), ("prefix", "L3_1"), ("spec", "L2_3"), ("spec", "L3_2"), ("dsa", "L2_4"), ("dsa", "L3_2")}


def _cases(opname):
    op = ops.load_op(opname)
    return [pytest.param(opname, layer, i, shape, dist, seed, id=f"{opname}-{layer}_{i}")
            for layer, i, shape, dist, seed in ops.cases(op)]


ALL = _cases("prefix") + _cases("spec") + _cases("dsa")


@pytest.mark.parametrize("opname,layer,i,shape,dist,seed", ALL)
def test_generator_and_truth_match_reference(opname, layer, i, shape, dist, seed):
    op = ops.load_op(opname)
    key = f"{layer}_{i}"
    inp = op.make_inputs(shape, seed=seed, dist=dist)
    check_inputs(opname, key, inp)
    g = golden(opname)
    if opname == "spec":
        assert np.array_equal(inp["bits"], g[f"{key}/bits"])
    if opname == "dsa":
        if inp["lens"] is not None:
            assert np.array_equal(inp["lens"], g[f"{key}/lens"])
        s, sel = ref64.dsa_ref_select64(inp["iq"], inp["ik"], inp["w"], inp["lens"])
        np.testing.assert_allclose(s.reshape(-1)[g[f"{key}/score_idx"]], g[f"{key}/score_val"], rtol=1e-9, atol=1e-14)
        for b in range(s.shape[0]):
            gk = f"{key}/gap/{b}"
            # identical sets wherever the boundary is not a float64 near-tie
            if gk not in g.files or (g[gk][0] - g[gk][1]) > 1e-12 * max(1.0, abs(g[gk][0])):
                assert sha(np.sort(sel[b]).astype(np.int32)) == str(g[f"{key}/sel_sha/{b}"])
        out = ref64.dsa_ref64(inp["q"], inp["kv"], inp["iq"], inp["ik"], inp["w"], inp["lens"], sel=sel)
    else:
        out = ref64.REF64[opname](**inp)
    check_truth(opname, key, out)


def test_spec_wide_masks_reduce_to_reference_layout():
    """A (B,kd,1)-word mask and the reference's (B,kd) layout give the same visibility."""
    op = ops.load_op("spec")
    inp = op.make_inputs(dict(B=2, L=300, k=8), seed=5)
    a = ref64.spec_allowed(inp["bits"], 300, 8)
    b = ref64.spec_allowed(inp["bits"][:, :, None], 300, 8)
    assert np.array_equal(a, b)
    # every draft sees itself and never a later draft; chain rows are lower-triangular
    tail = a[:, :, -8:]
    assert tail[:, np.arange(8), np.arange(8)].all()
    assert not np.triu(tail, 1).any()


def test_spec_depth_capped_trees():
    op = ops.load_op("spec")
    rng = np.random.default_rng(0)
    for _ in range(20):
        masks = op.tree_bits(64, rng, max_depth=8)
        assert max(bin(m).count("1") for m in masks) <= 8
        assert all((m >> i) & 1 for i, m in enumerate(masks))
    packed = op.pack_bits([masks], 64)
    assert packed.shape == (1, 64, 2) and packed.dtype == np.int32
    a = ref64.spec_allowed(packed, 100, 64)[0, :, -64:]
    for i, m in enumerate(masks):
        assert [bool((m >> j) & 1) for j in range(64)] == a[i].tolist()


def test_prefix_ragged_reduces_to_dense():
    op = ops.load_op("prefix")
    inp = op.make_inputs(dict(N=3, P=50, S=9), seed=2)
    full = ref64.prefix_ref64(**inp)
    same = ref64.prefix_ref64(**inp, slens=np.array([9, 9, 9], dtype=np.int32))
    assert np.array_equal(full, same)
    cut = ref64.prefix_ref64(**inp, slens=np.array([0, 4, 9], dtype=np.int32))
    assert np.array_equal(cut[2], full[2]) and not np.allclose(cut[0], full[0])
    short = {k: (v[:, :, :4] if k in ("ks", "vs") else v) for k, v in inp.items()}
    np.testing.assert_allclose(cut[1], ref64.prefix_ref64(**short)[1], rtol=1e-12)
