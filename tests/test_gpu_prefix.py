"""`prefix` on the GPU through the C ABI, judged by the reference's criteria against the float64 oracle."""
import numpy as np
import pytest
import torch

from oracle import judge, ref64
from tests import _verify
from verified_metal_kernels_b200 import _lib, load_kernel, ops

pytestmark = pytest.mark.gpu
op = ops.load_op("prefix")


def _id(c):
    layer, i, shape, dist, seed = c
    return f"{layer}_{i}-" + "x".join(f"{k}{v}" for k, v in shape.items()) + f"-{dist}"


@pytest.mark.parametrize("case", ops.cases(op), ids=_id)
def test_reference_cases(case):
    layer, i, shape, dist, seed = case
    inp = op.make_inputs(shape, seed=seed, dist=dist)
    out, _, _ = _verify.run_kernel(load_kernel("prefix"), "prefix", inp)
    _verify.assert_clean_status()
    rep = _verify.judge_case("prefix", layer, dist, out, inp)
    assert rep["ok"], rep


@pytest.mark.parametrize("shape,dist", op.FUZZ_EXT, ids=lambda x: str(x))
def test_ragged_suffix_extension(shape, dist):
    inp = op.make_inputs(shape, seed=11, dist=dist)
    assert inp["slens"].min() >= 0 and inp["slens"].max() <= shape["S"]
    out, _, _ = _verify.run_kernel(load_kernel("prefix"), "prefix", inp)
    _verify.assert_clean_status()
    rep = judge.judge_l2(out, _verify.truth("prefix", inp), half=True, dist=dist)
    assert rep["ok"], rep


def test_ragged_ignores_padding_contents():
    """Keys beyond slens[n] must not influence the result even when they hold Inf / NaN."""
    shape = dict(N=5, P=200, S=96, ragged=True)
    inp = op.make_inputs(shape, seed=4)
    inp["slens"][:] = [0, 1, 63, 64, 96]
    clean, _, _ = _verify.run_kernel(load_kernel("prefix"), "prefix", inp)
    dirty = dict(inp)
    dirty["ks"], dirty["vs"] = inp["ks"].copy(), inp["vs"].copy()
    for n, sl in enumerate(inp["slens"]):
        dirty["ks"][n, :, sl:] = np.nan
        dirty["vs"][n, :, sl:] = np.inf
    out, _, _ = _verify.run_kernel(load_kernel("prefix"), "prefix", dirty)
    assert np.array_equal(clean, out)
    rep = judge.judge_l2(out, _verify.truth("prefix", inp), half=True)
    assert rep["ok"], rep


def test_deterministic_and_inputs_untouched():
    inp = op.make_inputs(dict(N=8, P=4096, S=256), seed=0)
    fn = load_kernel("prefix")
    o1, _, dinp = _verify.run_kernel(fn, "prefix", inp)
    snap = {k: v.clone() for k, v in dinp.items() if v is not None}
    o2 = fn(**dinp).float().cpu().numpy()
    assert np.array_equal(o1, o2)
    for k, v in snap.items():
        assert torch.equal(v, dinp[k]), f"input {k} was modified"


def test_other_head_geometry():
    """Hq/Hkv other than 32/8 (the generator's optional overrides, reference ops/prefix.py:18)."""
    for Hq, Hkv in ((16, 16), (8, 1), (24, 4)):
        shape = dict(N=3, P=500, S=70, Hq=Hq, Hkv=Hkv)
        inp = op.make_inputs(shape, seed=9)
        out, _, _ = _verify.run_kernel(load_kernel("prefix"), "prefix", inp)
        rep = judge.judge_l2(out, _verify.truth("prefix", inp), half=True)
        assert rep["ok"], (Hq, Hkv, rep)


def test_host_buffers_round_trip():
    """kernel(...) given pinned host tensors copies in, computes on the GPU and returns a host tensor."""
    inp = op.make_inputs(dict(N=4, P=1024, S=64), seed=1)
    host = {k: torch.from_numpy(v).pin_memory() for k, v in inp.items()}
    out = load_kernel("prefix")(**host)
    assert not out.is_cuda
    dev, _, _ = _verify.run_kernel(load_kernel("prefix"), "prefix", inp)
    assert np.array_equal(out.float().numpy(), dev)


def test_partial_split_and_merge():
    """Key-range partials (the multi-GPU KV split) merged by vmk_lse_merge equal the one-call result."""
    shape = dict(N=6, P=3000, S=130)
    inp = op.make_inputs(shape, seed=5)
    d = _verify.device_inputs("prefix", inp)
    full = load_kernel("prefix")(**d)
    L = _lib.lib()
    N, Hq, D = d["q"].shape
    Hkv, P = d["kp"].shape[0], d["kp"].shape[1]
    S = d["ks"].shape[2]
    rows = N * Hq
    cuts = [0, 1000, 1900, P]
    pm = torch.empty(len(cuts) - 1, rows, device="cuda")
    pl = torch.empty_like(pm)
    po = torch.empty(len(cuts) - 1, rows, D, device="cuda")
    ws = torch.empty(L.vmk_prefix_workspace_bytes(N, Hq, Hkv, D, P, S), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for r in range(len(cuts) - 1):
        rc = L.vmk_prefix_partial(d["q"].data_ptr(), d["kp"].data_ptr(), d["vp"].data_ptr(), d["ks"].data_ptr(),
                                  d["vs"].data_ptr(), None, N, Hq, Hkv, D, P, S, cuts[r], cuts[r + 1], int(r == 1),
                                  pm[r].data_ptr(), pl[r].data_ptr(), po[r].data_ptr(), ws.data_ptr(), ws.numel(),
                                  None, st)
        assert rc == 0, _lib.error_string(rc)
    merged = torch.empty(rows, D, dtype=torch.float16, device="cuda")
    rc = L.vmk_lse_merge(pm.data_ptr(), pl.data_ptr(), po.data_ptr(), len(cuts) - 1, rows, D, merged.data_ptr(), st)
    assert rc == 0
    torch.cuda.synchronize()
    a, b = merged.float().cpu().numpy().reshape(N, Hq, D), full.float().cpu().numpy()
    assert np.abs(a - b).max() <= 2e-3
    rep = judge.judge_l2(a, _verify.truth("prefix", inp), half=True)
    assert rep["ok"], rep


def test_argument_errors():
    inp = op.make_inputs(dict(N=2, P=64, S=8), seed=0)
    d = _verify.device_inputs("prefix", inp)
    fn = load_kernel("prefix")
    with pytest.raises(TypeError):
        fn(**{**d, "q": d["q"].float()})
    with pytest.raises(ValueError):
        fn(**{**d, "vp": d["vp"][:, :10]})
    with pytest.raises(ValueError):
        fn(**{**d, "kp": d["kp"].transpose(0, 1)})
    L = _lib.lib()
    rc = L.vmk_prefix_decode(d["q"].data_ptr(), d["kp"].data_ptr(), d["vp"].data_ptr(), d["ks"].data_ptr(),
                             d["vs"].data_ptr(), None, d["q"].data_ptr(), 2, 32, 8, 128, 64, 8, d["q"].data_ptr(), 16,
                             None, None)
    assert rc == -3       # workspace too small
    rc = L.vmk_prefix_decode(d["q"].data_ptr(), d["kp"].data_ptr(), d["vp"].data_ptr(), d["ks"].data_ptr(),
                             d["vs"].data_ptr(), None, d["q"].data_ptr(), 2, 32, 8, 64, 64, 8, d["q"].data_ptr(), 1 << 30,
                             None, None)
    assert rc == -2       # head dimension other than 128


@pytest.mark.parametrize("shape,page_size,ragged", [
    (dict(N=4, P=1000, S=77), 64, False),        # warp-level kernel for both roles
    (dict(N=5, P=3000, S=300), 128, True),
    (dict(N=40, P=2100, S=200), 64, True),       # 160 stacked rows per KV head: tcgen05 kernel on the prefix
    (dict(N=40, P=2100, S=200), 256, False),
], ids=lambda x: str(x))
def test_paged_cache_equals_the_contiguous_call_bit_for_bit(shape, page_size, ragged):
    """vmk_prefix_decode_paged on one shuffled page pool holding the shared prefix and every suffix (unused
    pages and rows filled with NaN) against vmk_prefix_decode on contiguous tensors."""
    from verified_metal_kernels_b200.kernels import prefix_b200
    inp = op.make_inputs(dict(shape, ragged=True) if ragged else shape, seed=17)
    d = _verify.device_inputs("prefix", inp)
    N, S = shape["N"], shape["S"]
    slens = inp.get("slens")
    ref = prefix_b200.kernel(**d)
    kpg, vpg, ptab, stab = op.to_pages(inp["kp"], inp["vp"], inp["ks"], inp["vs"], slens, page_size, seed=3)
    sl = torch.from_numpy(np.full(N, S, dtype=np.int32) if slens is None else np.asarray(slens, dtype=np.int32)).cuda()
    out = prefix_b200.kernel_paged(d["q"], torch.from_numpy(kpg).cuda(), torch.from_numpy(vpg).cuda(),
                                   torch.from_numpy(ptab).cuda(), shape["P"], torch.from_numpy(stab).cuda(), sl)
    torch.cuda.synchronize()
    _verify.assert_clean_status()
    assert torch.equal(out, ref)
