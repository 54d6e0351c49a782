"""The projection in front of dsa stage 1 (vmk_dsa_index_project): index queries and head weights from the
activation, against the float64 statement; then the whole op fed by it."""
import numpy as np
import pytest
import torch

from oracle import judge, ref64
from tests import _verify
from verified_metal_kernels_b200 import ops
from verified_metal_kernels_b200.kernels import dsa_b200

pytestmark = pytest.mark.gpu


def _weights(Dx, seed, dtype=np.float16):
    rng = np.random.default_rng(seed)
    sc = Dx ** -0.5
    wq = (rng.standard_normal((8192, Dx), dtype=np.float32) * sc).astype(dtype)
    ww = (rng.standard_normal((64, Dx), dtype=np.float32) * sc).astype(dtype)
    return wq, ww


@pytest.mark.parametrize("B,Dx", [(1, 64), (5, 1536), (128, 1536), (200, 520), (3, 7168)])
def test_projection_against_float64(B, Dx):
    rng = np.random.default_rng(B * 7 + Dx)
    x = rng.standard_normal((B, Dx), dtype=np.float32).astype(np.float16)
    wq, ww = _weights(Dx, 1)
    t_iq, t_w = ref64.dsa_index_project64(x, wq, ww, 0.37)
    iq, w = dsa_b200.index_project(torch.from_numpy(x).cuda(), torch.from_numpy(wq).cuda(), torch.from_numpy(ww).cuda(), 0.37)
    torch.cuda.synchronize()
    _verify.assert_clean_status()
    assert tuple(iq.shape) == (B, 64, 128) and tuple(w.shape) == (B, 64) and w.dtype == torch.float32
    iq, w = iq.float().cpu().numpy(), w.cpu().numpy()
    # fp32 accumulation of exact fp16 products, rounded once to fp16: within one rounding of the float64 value
    # (plus the fp32 accumulation error of Dx terms, which is absolute: it matters for the values near zero)
    tol = 2.0 ** -10 * np.abs(t_iq) + 2e-5 * np.abs(t_iq).max()
    assert (np.abs(iq - t_iq) <= tol).all(), float(np.abs(iq - t_iq).max())
    # fp32 accumulation over Dx terms
    assert np.abs(w - t_w).max() <= 2e-5 * max(1.0, np.abs(t_w).max())


def test_projection_bf16_and_special_values():
    B, Dx = 9, 256
    rng = np.random.default_rng(3)
    x32 = ops.round_bf16(rng.standard_normal((B, Dx), dtype=np.float32))
    wq32, ww32 = (ops.round_bf16(a.astype(np.float32)) for a in _weights(Dx, 2, np.float32))
    x32[4, 7] = np.nan                                   # request 4 becomes NaN everywhere, the others stay clean
    to = lambda a: torch.from_numpy(a).cuda().to(torch.bfloat16)
    iq, w = dsa_b200.index_project(to(x32), to(wq32), to(ww32), 1.0)
    torch.cuda.synchronize()
    _verify.assert_clean_status()
    t_iq, t_w = ref64.dsa_index_project64(x32, wq32, ww32, 1.0)
    iq, w = iq.float().cpu().numpy(), w.cpu().numpy()
    assert np.isnan(iq[4]).all() and np.isnan(w[4]).all()
    keep = [b for b in range(B) if b != 4]
    assert np.isfinite(iq[keep]).all()
    assert (np.abs(iq[keep] - t_iq[keep]) <= 2.0 ** -7 * np.abs(t_iq[keep]) + 2e-5 * np.abs(t_iq[keep]).max()).all()
    assert np.abs(w[keep] - t_w[keep]).max() <= 2e-5 * max(1.0, np.abs(t_w[keep]).max())


def test_whole_op_fed_by_the_projection():
    """kernel_projected = projection + the three stages.  The truth takes the projection's own outputs as its iq and
    w (they are the op's inputs; their rounding is the projection's), so the selection must be exact as usual."""
    B, L, Dx = 3, 6000, 512
    op = ops.load_op("dsa")
    inp = op.make_inputs(dict(B=B, L=L), seed=11)
    rng = np.random.default_rng(12)
    x = rng.standard_normal((B, Dx), dtype=np.float32).astype(np.float16)
    wq, ww = _weights(Dx, 13)
    d = _verify.device_inputs("dsa", inp)
    cu = lambda a: torch.from_numpy(a).cuda()
    scale = (64 * 128) ** -0.5
    out, idx, cnt = dsa_b200.kernel_projected(d["q"], d["kv"], cu(x), cu(wq), cu(ww), d["ik"], scale, return_selection=True)
    iq, w = dsa_b200.index_project(cu(x), cu(wq), cu(ww), scale)
    torch.cuda.synchronize()
    _verify.assert_clean_status()
    iq_h, w_h = iq.cpu().numpy(), w.cpu().numpy()
    s64 = ref64.dsa_scores64(iq_h, inp["ik"], w_h)
    for b in range(B):
        assert judge.select_check(idx[b].cpu().numpy(), int(cnt[b]), s64[b], L)["ok"], b
    sel = [idx[b, :int(cnt[b])].cpu().numpy().astype(np.int64) for b in range(B)]
    truth = ref64.dsa_ref64(inp["q"], inp["kv"], iq_h, inp["ik"], w_h, None, sel=sel)
    rep = judge.judge_l2(out.float().cpu().numpy(), truth, half=True)
    assert rep["ok"] and rep["err_max"] <= 2e-3, rep
