"""The paged-cache helpers of the op definitions (extensions beyond the reference): scattering a cache into a
shuffled page pool and reading it back through the page table gives the cache back, and everything the table
does not cover is the fill value."""
import numpy as np

from verified_metal_kernels_b200 import ops


def test_spec_pages_round_trip():
    op = ops.load_op("spec")
    inp = op.make_inputs(dict(B=3, L=300, k=8), seed=2)
    kp, vp, table = op.to_pages(inp["k"], inp["v"], 64, seed=1)
    B, Hkv, L, D = inp["k"].shape
    assert table.shape == (B, 5) and len(set(table.ravel().tolist())) == B * 5
    for b in range(B):
        back = np.concatenate([kp[table[b, i]] for i in range(5)], axis=1)
        assert np.array_equal(back[:, :L], inp["k"][b])
        assert np.isnan(back[:, L:].astype(np.float32)).all()
    used = np.zeros(kp.shape[0], bool)
    used[table.ravel()] = True
    assert np.isnan(vp[~used].astype(np.float32)).all()


def test_prefix_pages_round_trip():
    op = ops.load_op("prefix")
    inp = op.make_inputs(dict(N=4, P=200, S=70, ragged=True), seed=3)
    kpg, vpg, ptab, stab = op.to_pages(inp["kp"], inp["vp"], inp["ks"], inp["vs"], inp["slens"], 64, seed=9)
    back = np.concatenate([vpg[p] for p in ptab], axis=1)
    assert np.array_equal(back[:, :200], inp["vp"])
    for n in range(4):
        s = int(inp["slens"][n])
        back = np.concatenate([kpg[p] for p in stab[n]], axis=1)
        assert np.array_equal(back[:, :s], inp["ks"][n][:, :s])
    assert len(set(ptab.tolist()) | set(stab.ravel().tolist())) == len(ptab) + stab.size
