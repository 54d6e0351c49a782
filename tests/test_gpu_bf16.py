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
        dsa_b200.set_attend_variant("tcgen05")
