"""The tcgen05 (tensor-memory) split-KV attention kernel against the warp-level kernel and the oracle on
shapes whose stacked rows exceed 64, where the tensor-memory kernel is selected."""
import numpy as np
import pytest
import torch

from oracle import judge
from tests import _verify
from verified_metal_kernels_b200 import _lib, load_kernel, ops

pytestmark = pytest.mark.gpu


def _both(opname, inp):
    L = _lib.lib()
    fn = load_kernel(opname)
    d = _verify.device_inputs(opname, inp)
    outs = []
    for on in (1, 0):
        L.vmk_attn_set_tc(on)
        try:
            outs.append(fn(**d).float().cpu().numpy())
        finally:
            L.vmk_attn_set_tc(1)
    _verify.assert_clean_status()
    return outs


@pytest.mark.parametrize("shape,dist", [(dict(N=17, P=1000, S=50), "randn"), (dict(N=40, P=4097, S=33), "randn"),
                                        (dict(N=64, P=9000, S=0), "large"), (dict(N=100, P=130, S=7), "randn"),
                                        (dict(N=32, P=1, S=1), "randn"), (dict(N=33, P=3000, S=200), "nan_inf"),
                                        (dict(N=48, P=5000, S=300, ragged=True), "needle_prefix")],
                         ids=lambda x: str(x))
def test_prefix_tensor_memory_kernel(shape, dist):
    op = ops.load_op("prefix")
    if shape["S"] == 0:
        shape = dict(shape, S=1)
        inp = op.make_inputs(shape, seed=31, dist=dist)
        inp["slens"] = np.zeros(shape["N"], dtype=np.int32)      # every suffix empty
    else:
        inp = op.make_inputs(shape, seed=31, dist=dist)
    tc, warp = _both("prefix", inp)
    t = _verify.truth("prefix", inp)
    rep = judge.judge_l2(tc, t, half=True, dist=dist, std=warp)
    assert rep["ok"], rep
    assert judge.nerr(tc, warp)[0] <= 2e-3


@pytest.mark.parametrize("shape,dist", [(dict(B=2, L=2000, k=64, max_depth=8), "randn"), (dict(B=1, L=4096, k=31), "randn"),
                                        (dict(B=1, L=129, k=20), "chain"), (dict(B=3, L=5000, k=17), "needle_masked"),
                                        (dict(B=1, L=64, k=64), "chain"), (dict(B=2, L=3000, k=32), "large"),
                                        (dict(B=2, L=3000, k=24), "nan_inf")], ids=lambda x: str(x))
def test_spec_tensor_memory_kernel(shape, dist):
    op = ops.load_op("spec")
    inp = op.make_inputs(shape, seed=37, dist=dist)
    tc, warp = _both("spec", inp)
    t = _verify.truth("spec", inp)
    rep = judge.judge_l2(tc, t, half=True, dist=dist, std=warp)
    assert rep["ok"], rep
    assert judge.nerr(tc, warp)[0] <= 2e-3


def test_lazy_rescale_with_growing_maxima():
    """Scores that keep growing along the cache force the deferred rescaling of the accumulator."""
    op = ops.load_op("spec")
    inp = op.make_inputs(dict(B=1, L=4096, k=32), seed=41)
    k = inp["k"].astype(np.float32)
    k *= np.linspace(0.2, 6.0, 4096, dtype=np.float32)[None, None, :, None]
    inp["k"] = k.astype(np.float16)
    tc, warp = _both("spec", inp)
    rep = judge.judge_l2(tc, _verify.truth("spec", inp), half=True)
    assert rep["ok"] and rep["err_max"] <= 2e-3, rep
