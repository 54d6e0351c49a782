"""bf16 tensors (an extension: the reference's kernels read fp16 only): `dsa` through the C ABI against the
float64 oracle on the bf16-rounded inputs.  Tolerances: the reference's fuzz criterion (same NaN/Inf pattern,
normalised max error <= 1e-2); the selection must be exact wherever the float64 scores are separated."""
import numpy as np
import pytest
import torch

from oracle import judge, ref64
from tests import _verify
from verified_metal_kernels_b200 import ops
from verified_metal_kernels_b200.kernels import dsa_b200

pytestmark = pytest.mark.gpu
dsa = ops.load_op("dsa")


@pytest.mark.parametrize("shape,dist", [(dict(B=2, L=5003), "randn"), (dict(B=3, L=9000), "ragged"),
                                        (dict(B=2, L=6000), "needle"), (dict(B=2, L=6000), "large"),
                                        (dict(B=1, L=2048), "randn"), (dict(B=2, L=6000), "nan_inf"),
                                        (dict(B=40, L=3000), "randn")], ids=lambda x: str(x))
def test_dsa_bf16_against_the_oracle(shape, dist):
    inp = ops.as_bf16("dsa", dsa.make_inputs(shape, seed=11, dist=dist))
    d = ops.to_torch(ops.cand_inputs("dsa", inp), "cuda", bf16="dsa")
    assert d["kv"].dtype == torch.bfloat16
    out, idx, cnt = dsa_b200.kernel(**d, return_selection=True)
    torch.cuda.synchronize()
    _verify.assert_clean_status()
    assert out.dtype == torch.bfloat16
    B, L = shape["B"], shape["L"]
    idx, cnt = idx.cpu().numpy(), cnt.cpu().numpy()
    s64 = ref64.dsa_scores64(inp["iq"], inp["ik"], inp["w"])
    lens = inp.get("lens")
    for b in range(B):
        n = L if lens is None else int(lens[b])
        assert judge.select_check(idx[b], cnt[b], s64[b], n)["ok"], b
    sel = [idx[b, :cnt[b]].astype(np.int64) for b in range(B)]
    truth = ref64.dsa_ref64(inp["q"], inp["kv"], inp["iq"], inp["ik"], inp["w"], lens, sel=sel)
    rep = judge.judge_l2(out.float().cpu().numpy(), truth, half=True, dist=dist)
    assert rep["ok"], rep


def test_dsa_bf16_host_resident_cache_gives_the_same_bits():
    inp = ops.as_bf16("dsa", dsa.make_inputs(dict(B=2, L=7000), seed=5))
    d = ops.to_torch(ops.cand_inputs("dsa", inp), "cuda", bf16="dsa")
    out_d = dsa_b200.kernel(**d)
    host = {k: (None if v is None else v.cpu().pin_memory()) for k, v in d.items()}
    out_h = dsa_b200.kernel(**host)
    torch.cuda.synchronize()
    assert out_h.dtype == torch.bfloat16 and torch.equal(out_h, out_d.cpu())


def test_dsa_bf16_needs_the_tensor_memory_kernels():
    """The warp-level cross-check variants are fp16 only: asking them for bf16 is refused, not miscomputed."""
    from verified_metal_kernels_b200 import _lib
    inp = ops.as_bf16("dsa", dsa.make_inputs(dict(B=1, L=3000), seed=1))
    d = ops.to_torch(ops.cand_inputs("dsa", inp), "cuda", bf16="dsa")
    dsa_b200.set_attend_variant("mma")
    try:
        with pytest.raises(_lib.VmkError) as e:
            dsa_b200.kernel(**d)
        assert e.value.code == -2
    finally:
        dsa_b200.set_attend_variant(dsa_b200.DEFAULT_ATTEND_VARIANT)


prefix = ops.load_op("prefix")
spec = ops.load_op("spec")


@pytest.mark.parametrize("shape,dist", [(dict(N=4, P=1000, S=77), "randn"), (dict(N=8, P=4096, S=256), "randn"),
                                        (dict(N=6, P=777, S=300, ragged=True), "randn"),
                                        (dict(N=3, P=640, S=5), "large"),
                                        (dict(N=40, P=2100, S=200), "randn"),            # tcgen05 kernel on the prefix
                                        (dict(N=70, P=5000, S=64, ragged=True), "randn")], ids=lambda x: str(x))
def test_prefix_bf16_against_the_oracle(shape, dist):
    from verified_metal_kernels_b200.kernels import prefix_b200
    inp = ops.as_bf16("prefix", prefix.make_inputs(shape, seed=23, dist=dist))
    d = ops.to_torch(ops.cand_inputs("prefix", inp), "cuda", bf16="prefix")
    out = prefix_b200.kernel(**d)
    torch.cuda.synchronize()
    _verify.assert_clean_status()
    assert out.dtype == torch.bfloat16
    truth = ref64.REF64["prefix"](**{k: inp.get(k) for k in ops.KEYS["prefix"]})
    rep = judge.judge_l2(out.float().cpu().numpy(), truth, half=True, dist=dist)
    assert rep["ok"], rep
    # bf16 keeps 8 significand bits: the output rounding alone is 2^-9 of the row's magnitude
    assert rep["err_max"] <= 6e-3, rep


@pytest.mark.parametrize("shape,dist", [(dict(B=2, L=1500, k=8), "randn"), (dict(B=1, L=8192, k=8), "chain"),
                                        (dict(B=2, L=700, k=16), "large"),
                                        (dict(B=2, L=3000, k=32), "randn"),               # tcgen05 kernel
                                        (dict(B=1, L=4096, k=64, max_depth=8), "randn")], ids=lambda x: str(x))
def test_spec_bf16_against_the_oracle(shape, dist):
    from verified_metal_kernels_b200.kernels import spec_b200
    inp = ops.as_bf16("spec", spec.make_inputs(shape, seed=29, dist=dist))
    d = ops.to_torch(ops.cand_inputs("spec", inp), "cuda", bf16="spec")
    out = spec_b200.kernel(**d)
    torch.cuda.synchronize()
    _verify.assert_clean_status()
    assert out.dtype == torch.bfloat16
    truth = ref64.REF64["spec"](**{k: inp.get(k) for k in ops.KEYS["spec"]})
    rep = judge.judge_l2(out.float().cpu().numpy(), truth, half=True, dist=dist)
    assert rep["ok"] and rep["err_max"] <= 6e-3, rep


def test_paged_bf16_equals_contiguous_bf16_bit_for_bit():
    from verified_metal_kernels_b200.kernels import spec_b200
    inp = ops.as_bf16("spec", spec.make_inputs(dict(B=2, L=3000, k=32), seed=3))
    d = ops.to_torch(ops.cand_inputs("spec", inp), "cuda", bf16="spec")
    ref = spec_b200.kernel(**d)
    kp, vp, table = spec.to_pages(inp["k"], inp["v"], 128, seed=5)
    out = spec_b200.kernel_paged(d["q"], torch.from_numpy(kp).cuda().to(torch.bfloat16),
                                 torch.from_numpy(vp).cuda().to(torch.bfloat16), torch.from_numpy(table).cuda(), 3000,
                                 d["bits"])
    torch.cuda.synchronize()
    assert out.dtype == torch.bfloat16 and torch.equal(out, ref)
