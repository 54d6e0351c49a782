"""Stage 1 of `dsa` with the index queries and keys in fp8 (an extension: the reference's op takes fp16): against
the float64 scores of the DEQUANTISED inputs, then the whole op through select and sparse attention."""
import numpy as np
import pytest
import torch

from oracle import judge, ref64
from tests import _verify
from verified_metal_kernels_b200 import ops
from verified_metal_kernels_b200.kernels import dsa_b200

pytestmark = pytest.mark.gpu
op = ops.load_op("dsa")


def _deq(q8, scale):
    return (q8.view(torch.float8_e4m3fn).float() * scale.unsqueeze(-1)).cpu().numpy()


@pytest.mark.parametrize("shape,dist", [(dict(B=2, L=5003), "randn"), (dict(B=3, L=9000), "ragged"),
                                        (dict(B=2, L=6000), "needle"), (dict(B=1, L=131072), "randn")],
                         ids=lambda x: str(x))
def test_fp8_index_keys(shape, dist):
    inp = op.make_inputs(shape, seed=81, dist=dist)
    d = _verify.device_inputs("dsa", inp)
    iq8, iqs = dsa_b200.quantize_e4m3(d["iq"])
    ik8, iks = dsa_b200.quantize_e4m3(d["ik"])
    scores, hist = dsa_b200.indexer_hist_fp8(iq8, iqs, ik8, iks, d["w"], d["lens"])
    out, idx, cnt = dsa_b200.kernel_fp8_index(d["q"], d["kv"], iq8, iqs, ik8, iks, d["w"], d["lens"], return_selection=True)
    torch.cuda.synchronize()
    _verify.assert_clean_status()
    B, L = shape["B"], shape["L"]
    s64 = ref64.dsa_scores64(_deq(iq8, iqs), _deq(ik8, iks), inp["w"])
    lens = inp.get("lens")
    sc = scores.cpu().numpy()
    for b in range(B):
        n = L if lens is None else int(lens[b])
        span = float(s64[b, :n].max() - s64[b, :n].min())
        # products of e4m3 values are exact and the sums are fp32, as for fp16 inputs (requests of at most 2048
        # positions are not scored: everything is selected)
        if n > 2048:
            assert np.abs(sc[b, :n] - s64[b, :n]).max() <= 2e-6 * span, b
        assert judge.select_check(idx[b].cpu().numpy(), int(cnt[b]), s64[b], n)["ok"], b
        assert int(hist[b].sum()) == (n if n > 2048 else 0)
    sel = [idx[b, :cnt[b]].cpu().numpy().astype(np.int64) for b in range(B)]
    truth = ref64.dsa_ref64(inp["q"], inp["kv"], inp["iq"], inp["ik"], inp["w"], lens, sel=sel)
    assert judge.judge_l2(out.float().cpu().numpy(), truth, half=True)["ok"]


def test_fp8_index_host_tensors_and_host_cache():
    """kernel_fp8_index with host tensors: everything copied in, or the page-locked latent cache read in place
    (only the selected rows cross the link): the same bits as the device-resident call, returned on the host."""
    inp = op.make_inputs(dict(B=2, L=6000), seed=82, dist="ragged")
    d = _verify.device_inputs("dsa", inp)
    iq8, iqs = dsa_b200.quantize_e4m3(d["iq"])
    ik8, iks = dsa_b200.quantize_e4m3(d["ik"])
    ref = dsa_b200.kernel_fp8_index(d["q"], d["kv"], iq8, iqs, ik8, iks, d["w"], d["lens"])
    torch.cuda.synchronize()
    host = [t.cpu() for t in (d["q"], d["kv"], iq8, iqs, ik8, iks, d["w"], d["lens"])]
    out_copy = dsa_b200.kernel_fp8_index(*host)
    assert not out_copy.is_cuda and torch.equal(out_copy, ref.cpu())
    host[1] = host[1].pin_memory()
    out_in_place = dsa_b200.kernel_fp8_index(*host)
    assert not out_in_place.is_cuda and torch.equal(out_in_place, ref.cpu())
    _verify.assert_clean_status()
