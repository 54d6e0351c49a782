"""`dsa` on the GPU through the C ABI: the fused op against the float64 oracle by the reference's three
layers, the integer stage (top-2048 index set) bit for bit, and each stage on its own."""
import numpy as np
import pytest
import torch

from oracle import judge, ref64
from tests import _verify
from verified_metal_kernels_b200 import _lib, load_kernel, ops
from verified_metal_kernels_b200.kernels import dsa_b200

pytestmark = pytest.mark.gpu
op = ops.load_op("dsa")


def _id(c):
    layer, i, shape, dist, seed = c
    return f"{layer}_{i}-" + "x".join(f"{k}{v}" for k, v in shape.items()) + f"-{dist}"


@pytest.mark.parametrize("case", ops.cases(op), ids=_id)
def test_reference_cases(case):
    layer, i, shape, dist, seed = case
    inp = op.make_inputs(shape, seed=seed, dist=dist)
    out, res, _ = _verify.run_kernel(load_kernel("dsa"), "dsa", inp, return_selection=True)
    _verify.assert_clean_status()
    _, idx, cnt = res
    idx, cnt = idx.cpu().numpy(), cnt.cpu().numpy()
    B, L = inp["ik"].shape[0], inp["ik"].shape[1]
    # integer stage: the selected set against the float64 scores
    s64 = ref64.dsa_scores64(inp["iq"], inp["ik"], inp["w"])
    for b in range(B):
        n = L if inp["lens"] is None else int(inp["lens"][b])
        rep = judge.select_check(idx[b], cnt[b], s64[b], n)
        assert rep["ok"], (b, rep)
        assert (np.diff(idx[b, :cnt[b]]) > 0).all(), "indices must be ascending"
    # floating-point stage, judged on the kernel's own (verified) selection for L2 so that a float64
    # near-tie at the boundary cannot turn into an output difference, and on the oracle's for L1/L3
    if layer == "L2":
        sel = [idx[b, :cnt[b]].astype(np.int64) for b in range(B)]
        t = ref64.dsa_ref64(inp["q"], inp["kv"], inp["iq"], inp["ik"], inp["w"], inp["lens"], sel=sel)
        rep = judge.judge_l2(out, t, half=True, dist=dist)
        assert rep["ok"], rep
        rep2 = judge.judge_l2(out, _verify.truth("dsa", inp), half=True, dist=dist)
        assert rep2["ok"] or dist == "nan_inf", rep2
    else:
        rep = _verify.judge_case("dsa", layer, dist, out, inp)
        assert rep["ok"], rep


def _scores_case(name, L, rng):
    if name == "randn":
        return rng.standard_normal(L).astype(np.float32)
    if name == "ties":                      # heavy ties straddling the boundary
        return rng.integers(0, 7, L).astype(np.float32)
    if name == "all_equal":
        return np.full(L, 0.25, dtype=np.float32)
    if name == "negative":
        return -np.abs(rng.standard_normal(L)).astype(np.float32) - 1.0
    if name == "nan_some":
        s = rng.standard_normal(L).astype(np.float32)
        s[rng.choice(L, L // 10, replace=False)] = np.nan
        return s
    if name == "tiny_spread":               # keys differing only in the low radix digits
        return (1.0 + rng.integers(0, 4000, L) * 2.0 ** -23).astype(np.float32)
    if name == "signed_zero":
        s = np.zeros(L, dtype=np.float32)
        s[::2] = -0.0
        s[rng.choice(L, 100, replace=False)] = 1.0
        return s
    raise KeyError(name)


@pytest.mark.parametrize("name", ["randn", "ties", "all_equal", "negative", "nan_some", "tiny_spread", "signed_zero"])
@pytest.mark.parametrize("L", [2049, 5000, 70001])
def test_select_stage_exact(name, L):
    """Stage 2 alone on adversarial score vectors: exactly 2048 distinct ascending positions; nothing
    left out beats anything taken; ties at the boundary go to the lowest positions; NaN ranks last."""
    rng = np.random.default_rng(L + len(name))
    s = np.stack([_scores_case(name, L, rng) for _ in range(3)])
    lens = np.array([L, L - 7, 2049], dtype=np.int32)
    idx, cnt = dsa_b200.select(torch.from_numpy(s).cuda(), torch.from_numpy(lens).cuda())
    idx, cnt = idx.cpu().numpy(), cnt.cpu().numpy()
    for b in range(3):
        n = int(lens[b])
        if n <= 2048:
            assert cnt[b] == n and idx[b, :n].tolist() == list(range(n))
            continue
        assert cnt[b] == 2048
        sel = idx[b]
        assert (np.diff(sel) > 0).all() and sel[0] >= 0 and sel[-1] < n
        key = np.where(np.isnan(s[b, :n]), -np.inf, s[b, :n]).astype(np.float64)
        chosen = np.zeros(n, dtype=bool)
        chosen[sel] = True
        thr = key[sel].min()
        assert (key[~chosen] <= thr).all()
        # among entries equal to the threshold the lowest positions are taken
        eq = np.flatnonzero(key == thr)
        take = chosen[eq]
        assert take[:take.sum()].all()


def test_select_identity_when_short():
    s = torch.randn(4, 2048, device="cuda")
    lens = torch.tensor([2048, 1, 100, 2047], dtype=torch.int32, device="cuda")
    idx, cnt = dsa_b200.select(s, lens)
    assert cnt.tolist() == [2048, 1, 100, 2047]
    for b, n in enumerate(cnt.tolist()):
        assert idx[b, :n].tolist() == list(range(n))


@pytest.mark.parametrize("B,L", [(1, 2049), (2, 4096), (3, 10007), (1, 65536)])
def test_indexer_stage(B, L):
    """Stage 1 alone: fp32 scores within fp32 accumulation error of the float64 scores."""
    inp = op.make_inputs(dict(B=B, L=L), seed=17)
    d = _verify.device_inputs("dsa", inp)
    s = dsa_b200.indexer(d["iq"], d["ik"], d["w"]).cpu().numpy().astype(np.float64)
    _verify.assert_clean_status()
    s64 = ref64.dsa_scores64(inp["iq"], inp["ik"], inp["w"])
    assert np.abs(s - s64).max() <= 2e-6 * np.abs(s64).max()


@pytest.mark.parametrize("B,L,dist", [(2, 4096, "randn"), (3, 9000, "ragged"), (1, 70001, "randn"), (2, 40000, "needle")])
def test_fused_histogram_and_select_from_it(B, L, dist):
    """The histogram the indexer accumulates is exactly the histogram of the top 11 key bits of the scores
    it wrote, and the select that starts from it returns the same list as the select that builds its own."""
    inp = op.make_inputs(dict(B=B, L=L), seed=29, dist=dist)
    d = _verify.device_inputs("dsa", inp)
    scores, hist = dsa_b200.indexer_hist(d["iq"], d["ik"], d["w"], d["lens"])
    _verify.assert_clean_status()
    s, h = scores.cpu().numpy(), hist.cpu().numpy()
    for b in range(B):
        n = L if inp["lens"] is None else int(inp["lens"][b])
        if n <= 2048:
            assert (h[b] == 0).all()
            continue
        u = (s[b, :n] + np.float32(0.0)).view(np.uint32)
        key = np.where(u & 0x80000000, ~u, u | 0x80000000).astype(np.uint32)
        assert np.array_equal(np.bincount(key >> 21, minlength=2048), h[b])
    a_idx, a_cnt = dsa_b200.select(scores, d["lens"], hist=hist)
    b_idx, b_cnt = dsa_b200.select(scores, d["lens"])
    assert torch.equal(a_idx, b_idx) and torch.equal(a_cnt, b_cnt)


def test_indexer_ragged_leaves_tail_untouched():
    inp = op.make_inputs(dict(B=3, L=6000), seed=18, dist="ragged")
    d = _verify.device_inputs("dsa", inp)
    s = dsa_b200.indexer(d["iq"], d["ik"], d["w"], d["lens"]).cpu().numpy()
    s64 = ref64.dsa_scores64(inp["iq"], inp["ik"], inp["w"])
    for b, n in enumerate(inp["lens"]):
        if n > 2048:
            assert np.abs(s[b, :n] - s64[b, :n]).max() <= 2e-6 * np.abs(s64).max()
        assert (s[b, n:] == 0).all()


@pytest.mark.parametrize("B", [1, 3, 8, 40])
def test_attend_stage(B):
    """Stage 3 alone on random (not top-k) selections, including short and empty-tail ones."""
    L = 3000
    rng = np.random.default_rng(B)
    inp = op.make_inputs(dict(B=B, L=L), seed=19)
    cnt = rng.integers(1, 2049, B).astype(np.int32)
    cnt[0] = 2048
    if B > 1:
        cnt[1] = 1
    idx = np.zeros((B, 2048), dtype=np.int32)
    sel = []
    for b in range(B):
        sel.append(np.sort(rng.choice(L, cnt[b], replace=False)))
        idx[b, :cnt[b]] = sel[b]
    d = _verify.device_inputs("dsa", inp)
    out = dsa_b200.attend(d["q"], d["kv"], torch.from_numpy(idx).cuda(), torch.from_numpy(cnt).cuda())
    _verify.assert_clean_status()
    t = ref64.dsa_ref64(inp["q"], inp["kv"], None, None, None, sel=sel)
    rep = judge.judge_l2(out.float().cpu().numpy(), t, half=True)
    assert rep["ok"] and rep["err_max"] <= 2e-3, rep


def test_deterministic_and_inputs_untouched():
    inp = op.make_inputs(dict(B=2, L=8192), seed=0)
    fn = load_kernel("dsa")
    o1, _, dinp = _verify.run_kernel(fn, "dsa", inp)
    snap = {k: v.clone() for k, v in dinp.items() if v is not None}
    o2 = fn(**dinp).float().cpu().numpy()
    assert np.array_equal(o1, o2)
    for k, v in snap.items():
        assert torch.equal(v, dinp[k]), f"input {k} was modified"


@pytest.mark.parametrize("B,L", [(8, 32768), (3, 9000)])
def test_back_to_back_fused_calls_equal_the_staged_calls(B, L):
    """Stage 3 starts before stage 2 has finished (a dependent launch) and reads the lists only after it has.
    Two different inputs alternate through the same workspace with no synchronisation between the calls: a
    list read too early would be the other input's, and the output would differ from the staged result."""
    fn = load_kernel("dsa")
    cases = []
    for seed in (41, 42):
        d = _verify.device_inputs("dsa", op.make_inputs(dict(B=B, L=L), seed=seed))
        scores, hist = dsa_b200.indexer_hist(d["iq"], d["ik"], d["w"], d["lens"])
        torch.cuda.synchronize()
        idx, cnt = dsa_b200.select(scores, d["lens"], hist=hist)
        torch.cuda.synchronize()
        want = dsa_b200.attend(d["q"], d["kv"], idx, cnt)
        torch.cuda.synchronize()
        cases.append((d, want))
    assert not torch.equal(cases[0][1], cases[1][1])
    outs = []
    for it in range(24):
        d, _ = cases[it & 1]
        outs.append(fn(**d))
    torch.cuda.synchronize()
    _verify.assert_clean_status()
    for it, o in enumerate(outs):
        assert torch.equal(o, cases[it & 1][1]), f"call {it} differs from the staged result"


def test_argument_errors():
    inp = op.make_inputs(dict(B=1, L=64), seed=0)
    d = _verify.device_inputs("dsa", inp)
    fn = load_kernel("dsa")
    with pytest.raises(TypeError):
        fn(**{**d, "w": d["w"].half()})
    with pytest.raises(ValueError):
        fn(**{**d, "ik": d["ik"][:, :32]})
    L = _lib.lib()
    rc = L.vmk_dsa_decode(d["q"].data_ptr(), d["kv"].data_ptr(), d["iq"].data_ptr(), d["ik"].data_ptr(),
                          d["w"].data_ptr(), None, d["q"].data_ptr(), None, None, 1, 64, d["kv"].data_ptr(), 64, None,
                          None)
    assert rc == -3


def test_gather_compacts_selected_rows_from_device_and_from_pinned_host_memory():
    """vmk_dsa_gather: kv_sel[b, j] = kv[b, idx[b, j]] for j < cnt[b] and idx_sel = 0..cnt-1, whether the
    cache is a device tensor or page-locked host memory read in place."""
    B, L = 3, 5000
    g = torch.Generator().manual_seed(5)
    kv = torch.randn(B, L, 576, generator=g).to(torch.float16)
    cnt = torch.tensor([2048, 1, 777], dtype=torch.int32)
    idx = torch.zeros(B, 2048, dtype=torch.int32)
    for b in range(B):
        idx[b, :cnt[b]] = torch.sort(torch.randperm(L, generator=g)[:cnt[b]]).values.to(torch.int32)
    for src in (kv.cuda(), kv.pin_memory()):
        kv_sel, idx_sel = dsa_b200.gather(src, idx.cuda(), cnt.cuda())
        torch.cuda.synchronize()
        for b in range(B):
            n = int(cnt[b])
            assert torch.equal(kv_sel[b, :n].cpu(), kv[b, idx[b, :n].long()])
            assert torch.equal(idx_sel[b, :n].cpu(), torch.arange(n, dtype=torch.int32))
    _verify.assert_clean_status()


@pytest.mark.parametrize("dist", ["randn", "ragged"])
def test_host_resident_cache_gives_the_same_bits_as_the_device_call(dist):
    """kernel(...) with page-locked host tensors leaves the latent cache on the host and reads only the
    selected rows; output and selection must equal the all-on-device call bit for bit."""
    inp = op.make_inputs(dict(B=3, L=9000), seed=21, dist=dist)
    d = _verify.device_inputs("dsa", inp)
    out_d, idx_d, cnt_d = dsa_b200.kernel(**d, return_selection=True)
    host = {k: (None if v is None else v.cpu().pin_memory()) for k, v in d.items()}
    out_h, idx_h, cnt_h = dsa_b200.kernel(**host, return_selection=True)
    torch.cuda.synchronize()
    assert not out_h.is_cuda
    assert torch.equal(out_h, out_d.cpu())
    assert torch.equal(cnt_h, cnt_d)
    for b in range(3):
        assert torch.equal(idx_h[b, :cnt_h[b]], idx_d[b, :cnt_d[b]])
    # an unpinned cache is copied whole and must agree too
    host["kv"] = d["kv"].cpu()
    assert torch.equal(dsa_b200.kernel(**host), out_d.cpu())
    _verify.assert_clean_status()


@pytest.mark.parametrize("shape,dist,page_size,bf16", [
    (dict(B=3, L=9000), "ragged", 128, False),
    (dict(B=2, L=6000), "randn", 512, False),
    (dict(B=40, L=3000), "ragged", 128, False),       # units cut by range boundaries in stage 3
    (dict(B=2, L=7000), "ragged", 256, True),
], ids=lambda x: str(x))
def test_paged_cache_equals_the_contiguous_call_bit_for_bit(shape, dist, page_size, bf16):
    """vmk_dsa_decode_paged on shuffled page pools (index keys and latent rows paged alike; unused pages and rows
    NaN) against vmk_dsa_decode on the contiguous tensors: same selection, same output bits."""
    inp = op.make_inputs(shape, seed=71, dist=dist)
    B, L = shape["B"], shape["L"]
    if inp.get("lens") is None:
        inp["lens"] = np.full(B, L, dtype=np.int32)
    if bf16:
        inp = ops.as_bf16("dsa", inp)
    d = ops.to_torch(ops.cand_inputs("dsa", inp), "cuda", bf16="dsa" if bf16 else None)
    ref, ridx, rcnt = dsa_b200.kernel(**d, return_selection=True)
    kvp, ikp, table = op.to_pages(inp["kv"], inp["ik"], inp["lens"], page_size, seed=9)
    tt = lambda a: (torch.from_numpy(a).cuda().to(torch.bfloat16) if bf16 else torch.from_numpy(a).cuda())
    out, idx, cnt = dsa_b200.kernel_paged(d["q"], tt(kvp), d["iq"], tt(ikp), d["w"], torch.from_numpy(table).cuda(),
                                          d["lens"], return_selection=True)
    torch.cuda.synchronize()
    _verify.assert_clean_status()
    assert torch.equal(cnt, rcnt)
    for b in range(B):
        assert torch.equal(idx[b, :cnt[b]], ridx[b, :rcnt[b]]), b
    assert torch.equal(out, ref)
