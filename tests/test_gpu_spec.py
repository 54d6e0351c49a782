"""`spec` on the GPU through the C ABI, judged by the reference's criteria against the float64 oracle."""
import numpy as np
import pytest
import torch

from oracle import judge
from tests import _verify
from verified_metal_kernels_b200 import _lib, load_kernel, ops

pytestmark = pytest.mark.gpu
op = ops.load_op("spec")


def _id(c):
    layer, i, shape, dist, seed = c
    return f"{layer}_{i}-" + "x".join(f"{k}{v}" for k, v in shape.items()) + f"-{dist}"


@pytest.mark.parametrize("case", ops.cases(op), ids=_id)
def test_reference_cases(case):
    layer, i, shape, dist, seed = case
    inp = op.make_inputs(shape, seed=seed, dist=dist)
    out, _, _ = _verify.run_kernel(load_kernel("spec"), "spec", inp)
    _verify.assert_clean_status()
    rep = _verify.judge_case("spec", layer, dist, out, inp)
    assert rep["ok"], rep


@pytest.mark.parametrize("shape,dist", op.FUZZ_EXT, ids=lambda x: str(x))
def test_wide_mask_extension(shape, dist):
    inp = op.make_inputs(shape, seed=13, dist=dist)
    out, _, _ = _verify.run_kernel(load_kernel("spec"), "spec", inp)
    _verify.assert_clean_status()
    rep = judge.judge_l2(out, _verify.truth("spec", inp), half=True, dist=dist)
    assert rep["ok"], rep


def test_word_layout_equivalence():
    """(B,kd) int32 masks and the same masks as (B,kd,1) / zero-extended (B,kd,2) words agree bit for bit."""
    inp = op.make_inputs(dict(B=2, L=700, k=8), seed=21)
    fn = load_kernel("spec")
    d = _verify.device_inputs("spec", inp)
    a = fn(**d)
    b = fn(**{**d, "bits": d["bits"][:, :, None].contiguous()})
    wide = torch.zeros(2, 8, 2, dtype=torch.int32, device="cuda")
    wide[:, :, 0] = d["bits"]
    c = fn(**{**d, "bits": wide})
    assert torch.equal(a, b) and torch.equal(a, c)


def test_tree_config_small_cache():
    """The 64-node depth-capped tree configuration at a cache length the oracle finishes quickly."""
    shape = dict(B=4, L=4096, k=64, max_depth=8)
    inp = op.make_inputs(shape, seed=0)
    out, _, _ = _verify.run_kernel(load_kernel("spec"), "spec", inp)
    _verify.assert_clean_status()
    t = _verify.truth("spec", inp)
    rep = judge.judge_l3(out, t, _verify.standard_op(op, "L3_REF", inp))
    assert rep["ok"], rep


def test_chain_equals_prefix_of_causal():
    """Chain masks: draft row i must equal plain attention over the first L-kd+i+1 positions."""
    shape = dict(B=1, L=600, k=8)
    inp = op.make_inputs(shape, seed=3, dist="chain")
    out, _, _ = _verify.run_kernel(load_kernel("spec"), "spec", inp)
    from oracle import ref64
    for i in range(8):
        n = 600 - 8 + i + 1
        one = dict(q=inp["q"][:, i:i + 1], k=inp["k"][:, :, :n], v=inp["v"][:, :, :n],
                   bits=np.ones((1, 1), dtype=np.int32))
        t = ref64.spec_ref64(**one)
        assert judge.nerr(out[:, i:i + 1], t)[0] <= 2e-3


def test_deterministic_and_inputs_untouched():
    inp = op.make_inputs(dict(B=1, L=8192, k=8), seed=0, dist="chain")
    fn = load_kernel("spec")
    o1, _, dinp = _verify.run_kernel(fn, "spec", inp)
    snap = {k: v.clone() for k, v in dinp.items()}
    o2 = fn(**dinp).float().cpu().numpy()
    assert np.array_equal(o1, o2)
    for k, v in snap.items():
        assert torch.equal(v, dinp[k]), f"input {k} was modified"


def test_partial_split_and_merge():
    shape = dict(B=2, L=5000, k=8)
    inp = op.make_inputs(shape, seed=6)
    d = _verify.device_inputs("spec", inp)
    full = load_kernel("spec")(**d)
    L = _lib.lib()
    B, kd, Hq, D = d["q"].shape
    Hkv, Lk = d["k"].shape[1], d["k"].shape[2]
    rows = B * kd * Hq
    cuts = [0, 2500, 4995, Lk]      # the last rank owns only draft positions and 3 cache positions
    pm = torch.empty(len(cuts) - 1, rows, device="cuda")
    pl = torch.empty_like(pm)
    po = torch.empty(len(cuts) - 1, rows, D, device="cuda")
    ws = torch.empty(L.vmk_spec_workspace_bytes(B, kd, Hq, Hkv, D, Lk), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for r in range(len(cuts) - 1):
        rc = L.vmk_spec_partial(d["q"].data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(), d["bits"].data_ptr(), 1, B, kd,
                                Hq, Hkv, D, Lk, cuts[r], cuts[r + 1], pm[r].data_ptr(), pl[r].data_ptr(),
                                po[r].data_ptr(), ws.data_ptr(), ws.numel(), None, st)
        assert rc == 0, _lib.error_string(rc)
    merged = torch.empty(rows, D, dtype=torch.float16, device="cuda")
    assert L.vmk_lse_merge(pm.data_ptr(), pl.data_ptr(), po.data_ptr(), len(cuts) - 1, rows, D, merged.data_ptr(), st) == 0
    torch.cuda.synchronize()
    a, b = merged.float().cpu().numpy().reshape(B, kd, Hq, D), full.float().cpu().numpy()
    assert np.abs(a - b).max() <= 2e-3
    rep = judge.judge_l2(a, _verify.truth("spec", inp), half=True)
    assert rep["ok"], rep


def test_argument_errors():
    inp = op.make_inputs(dict(B=1, L=64, k=4), seed=0)
    d = _verify.device_inputs("spec", inp)
    fn = load_kernel("spec")
    with pytest.raises(TypeError):
        fn(**{**d, "bits": d["bits"].long()})
    with pytest.raises(ValueError):
        fn(**{**d, "v": d["v"][:, :, :32]})
    L = _lib.lib()
    ws = torch.empty(1 << 22, dtype=torch.uint8, device="cuda")
    # more drafts than one mask word can describe
    rc = L.vmk_spec_verify(d["q"].data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(), d["bits"].data_ptr(), 1,
                           d["q"].data_ptr(), 1, 40, 32, 8, 128, 64, ws.data_ptr(), ws.numel(), None, None)
    assert rc == -2


@pytest.mark.parametrize("shape,page_size,tc", [
    (dict(B=2, L=1000, k=8), 64, True),        # warp-level kernel, last page 40/64 full
    (dict(B=3, L=5000, k=8), 128, True),
    (dict(B=2, L=3000, k=32), 64, True),       # 128 stacked rows: tcgen05 kernel, every 64-key box its own page
    (dict(B=2, L=3000, k=32), 256, True),
    (dict(B=2, L=3000, k=32), 256, False),     # the same shape forced onto the warp-level kernel
], ids=lambda x: str(x))
def test_paged_cache_equals_the_contiguous_call_bit_for_bit(shape, page_size, tc):
    """vmk_spec_verify_paged on a shuffled page pool (unused pages and the unused tail of every last page
    filled with NaN) against vmk_spec_verify on the same cache stored contiguously, and against the oracle."""
    from verified_metal_kernels_b200.kernels import spec_b200
    inp = op.make_inputs(shape, seed=31)
    d = _verify.device_inputs("spec", inp)
    kp, vp, table = op.to_pages(inp["k"], inp["v"], page_size, seed=5)
    lib = _lib.lib()
    lib.vmk_attn_set_tc(1 if tc else 0)
    try:
        ref = spec_b200.kernel(**d)
        out = spec_b200.kernel_paged(d["q"], torch.from_numpy(kp).cuda(), torch.from_numpy(vp).cuda(),
                                     torch.from_numpy(table).cuda(), shape["L"], d["bits"])
        torch.cuda.synchronize()
    finally:
        lib.vmk_attn_set_tc(1)
    _verify.assert_clean_status()
    assert torch.equal(out, ref)
    rep = judge.judge_l2(out.float().cpu().numpy(), _verify.truth("spec", inp), half=True)
    assert rep["ok"], rep


def test_paged_cache_rejects_bad_geometry():
    from verified_metal_kernels_b200.kernels import spec_b200
    inp = op.make_inputs(dict(B=1, L=500, k=8), seed=1)
    d = _verify.device_inputs("spec", inp)
    kp, vp, table = op.to_pages(inp["k"], inp["v"], 64, seed=5)
    kp, vp, table = torch.from_numpy(kp).cuda(), torch.from_numpy(vp).cuda(), torch.from_numpy(table).cuda()
    with pytest.raises(ValueError):
        spec_b200.kernel_paged(d["q"], kp, vp, table[:, :4].contiguous(), 500, d["bits"])   # table covers 256 keys
    with pytest.raises(ValueError):
        spec_b200.kernel_paged(d["q"], kp[:, :, :48].contiguous(), vp[:, :, :48].contiguous(), table, 500, d["bits"])
