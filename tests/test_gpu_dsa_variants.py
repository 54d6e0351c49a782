"""The two stage-1 implementations of `dsa` (tcgen05 + tensor memory, the default; warp-level mma.sync)
against the float64 scores and against each other."""
import numpy as np
import pytest
import torch

from oracle import judge, ref64
from tests import _verify
from verified_metal_kernels_b200 import load_kernel, ops
from verified_metal_kernels_b200.kernels import dsa_b200

pytestmark = pytest.mark.gpu
op = ops.load_op("dsa")


@pytest.fixture(autouse=True)
def _variant():
    dsa_b200.set_indexer_variant("tcgen05")
    yield
    dsa_b200.set_indexer_variant("tcgen05")


@pytest.mark.parametrize("B,L", [(1, 2049), (2, 4096), (3, 10007), (1, 65536), (5, 40000)])
def test_scores(B, L):
    inp = op.make_inputs(dict(B=B, L=L), seed=23)
    d = _verify.device_inputs("dsa", inp)
    s = dsa_b200.indexer(d["iq"], d["ik"], d["w"]).cpu().numpy().astype(np.float64)
    _verify.assert_clean_status()
    s64 = ref64.dsa_scores64(inp["iq"], inp["ik"], inp["w"])
    assert np.abs(s - s64).max() <= 2e-6 * np.abs(s64).max()
    dsa_b200.set_indexer_variant("mma")
    s0 = dsa_b200.indexer(d["iq"], d["ik"], d["w"]).cpu().numpy().astype(np.float64)
    _verify.assert_clean_status()
    assert np.abs(s0 - s64).max() <= 2e-6 * np.abs(s64).max()
    assert np.abs(s - s0).max() <= 2e-6 * np.abs(s64).max()


@pytest.mark.parametrize("variant", ["tcgen05", "mma"])
def test_ragged_and_full_op(variant):
    dsa_b200.set_indexer_variant(variant)
    inp = op.make_inputs(dict(B=3, L=9000), seed=12, dist="ragged")
    out, res, _ = _verify.run_kernel(load_kernel("dsa"), "dsa", inp, return_selection=True)
    _verify.assert_clean_status()
    _, idx, cnt = res
    idx, cnt = idx.cpu().numpy(), cnt.cpu().numpy()
    s64 = ref64.dsa_scores64(inp["iq"], inp["ik"], inp["w"])
    for b in range(3):
        assert judge.select_check(idx[b], cnt[b], s64[b], int(inp["lens"][b]))["ok"]
    sel = [idx[b, :cnt[b]].astype(np.int64) for b in range(3)]
    t = ref64.dsa_ref64(inp["q"], inp["kv"], inp["iq"], inp["ik"], inp["w"], inp["lens"], sel=sel)
    assert judge.judge_l2(out, t, half=True)["ok"]


@pytest.mark.parametrize("B,dist", [(1, "randn"), (3, "large"), (8, "randn"), (40, "needle")])
def test_attend_variants_agree(B, dist):
    """Stage 3 on tcgen05 (Q in tensor memory, output accumulated in registers; one CTA per request and value
    half, or a cluster of two per request) against the warp-level kernel and the oracle, on random selections
    with short and full counts."""
    L = 3000
    rng = np.random.default_rng(100 + B)
    inp = op.make_inputs(dict(B=B, L=L), seed=43, dist=dist)
    cnt = rng.integers(1, 2049, B).astype(np.int32)
    cnt[0] = 2048
    if B > 1:
        cnt[1] = 1
    if B > 2:
        cnt[2] = 65
    idx = np.zeros((B, 2048), dtype=np.int32)
    sel = []
    for b in range(B):
        sel.append(np.sort(rng.choice(L, cnt[b], replace=False)))
        idx[b, :cnt[b]] = sel[b]
    d = _verify.device_inputs("dsa", inp)
    ti, tc_ = torch.from_numpy(idx).cuda(), torch.from_numpy(cnt).cuda()
    outs = {}
    for v in ("tcgen05_pair", "tcgen05", "tcgen05_tma", "mma"):
        dsa_b200.set_attend_variant(v)
        try:
            outs[v] = dsa_b200.attend(d["q"], d["kv"], ti, tc_).float().cpu().numpy()
        finally:
            dsa_b200.set_attend_variant(dsa_b200.DEFAULT_ATTEND_VARIANT)
    _verify.assert_clean_status()
    t = ref64.dsa_ref64(inp["q"], inp["kv"], None, None, None, sel=sel)
    for v, o in outs.items():
        rep = judge.judge_l2(o, t, half=True, dist=dist)
        assert rep["ok"] and rep["err_max"] <= 2e-3, (v, rep)
    assert judge.nerr(outs["tcgen05"], outs["mma"])[0] <= 2e-3
    assert judge.nerr(outs["tcgen05_pair"], outs["tcgen05"])[0] <= 2e-3
    # the two gathers fill the same shared-memory tiles, so everything after them sees the same bits
    assert np.array_equal(outs["tcgen05"], outs["tcgen05_tma"], equal_nan=True)


def test_select_cluster_sizes_agree():
    """The top-k selection splits a long row over 1, 2, 4 or 8 CTAs (the batch size decides): the selected positions
    and counts are the same, with and without the indexer's fused histogram."""
    B, L = 3, 40000
    inp = op.make_inputs(dict(B=B, L=L), seed=5, dist="ragged")
    d = _verify.device_inputs("dsa", inp)
    scores, hist = dsa_b200.indexer_hist(d["iq"], d["ik"], d["w"], d.get("lens"))
    outs = {}
    try:
        for cs in (0, 1, 2, 4, 8):
            dsa_b200.set_select_cluster(cs)
            i1, c1 = dsa_b200.select(scores, d.get("lens"), hist)
            i2, c2 = dsa_b200.select(scores, d.get("lens"))
            outs[cs] = (i1.cpu().numpy(), c1.cpu().numpy())
            assert np.array_equal(outs[cs][1], c2.cpu().numpy())
            for b in range(B):
                n = int(outs[cs][1][b])
                assert np.array_equal(outs[cs][0][b, :n], i2.cpu().numpy()[b, :n])
    finally:
        dsa_b200.set_select_cluster(0)
    _verify.assert_clean_status()
    s64 = ref64.dsa_scores64(inp["iq"], inp["ik"], inp["w"])
    for cs, (idx, cnt) in outs.items():
        for b in range(B):
            assert judge.select_check(idx[b], cnt[b], s64[b], int(inp["lens"][b]))["ok"], cs
            n = int(cnt[b])
            assert np.array_equal(idx[b, :n], outs[0][0][b, :n]), cs


def test_select_crowded_boundary_bin_and_ties_stay_exact():
    """Scores whose boundary bin is crowded and unevenly spread (one warp's span holds far more than its share),
    and scores with many entries equal to the threshold: the selection is still the exact top-2048 with ties to the
    lowest positions, whichever path the kernel takes."""
    L = 131072
    g = torch.Generator(device="cuda").manual_seed(5)
    crowded = torch.randn(L, device="cuda", generator=g) * 0.1
    # 2.0 .. 2.49 share the top 11 key bits: 6000 such values, a third of them inside one warp's span of 4096
    crowded[torch.randperm(L, device="cuda", generator=g)[:4000]] = 2.0 + 0.49 * torch.rand(4000, device="cuda", generator=g)
    crowded[8192:8192 + 2000] = 2.0 + 0.49 * torch.rand(2000, device="cuda", generator=g)
    crowded[torch.randperm(L, device="cuda", generator=g)[:1500]] = 3.0 + torch.rand(1500, device="cuda", generator=g)
    tied = torch.randn(L, device="cuda", generator=g) * 0.1
    tied[torch.randperm(L, device="cuda", generator=g)[:2000]] = 5.0 + torch.rand(2000, device="cuda", generator=g)
    tied[torch.randperm(L, device="cuda", generator=g)[:150]] = 4.25            # 150 equal values around the threshold
    scores = torch.stack([crowded, tied]).contiguous()
    order = torch.sort(scores, dim=1, descending=True, stable=True).indices[:, :2048]
    want = torch.sort(order, dim=1).values.to(torch.int32)
    try:
        for cs in (0, 1, 4):
            dsa_b200.set_select_cluster(cs)
            idx, cnt = dsa_b200.select(scores)
            assert bool((cnt == 2048).all()) and torch.equal(idx, want), cs
    finally:
        dsa_b200.set_select_cluster(0)
    _verify.assert_clean_status()
