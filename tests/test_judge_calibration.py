"""Calibration of the judge on the CPU with deliberately wrong kernels, after the reference's negative
fixtures (reference wrong_kernels/prefix_cheat_fp16.py:13-33: scores, probabilities and sums kept in fp16;
wrong_kernels/spec_cheat_nomax.py:19-28: softmax without subtracting the maximum).  The judge must accept
a correct fp32 composition and reject both cheats in the layers the reference documents
(README.md:109-112): the fp16 cascade in the float64 layers, the no-max softmax in the fuzz layer only."""
import math

import numpy as np
import pytest
import torch

from oracle import judge, ref64
from verified_metal_kernels_b200 import ops


def _t(inp, keys):
    return [torch.from_numpy(inp[k]) for k in keys]


def prefix_correct(q, kp, vp, ks, vs):
    N, Hq, d = q.shape
    Hkv = kp.shape[0]
    G = Hq // Hkv
    k = torch.cat([kp[None].expand(N, *kp.shape), ks], 2).float()
    v = torch.cat([vp[None].expand(N, *vp.shape), vs], 2).float()
    s = torch.einsum("nhgd,nhld->nhgl", q.float().reshape(N, Hkv, G, d), k) / math.sqrt(d)
    return torch.einsum("nhgl,nhld->nhgd", torch.softmax(s, -1), v).reshape(N, Hq, d).half()


def prefix_cheat_fp16(q, kp, vp, ks, vs):
    """Cascade with scores, probabilities and sums in fp16."""
    N, Hq, d = q.shape
    Hkv = kp.shape[0]
    G = Hq // Hkv
    sc = 1 / math.sqrt(d)
    h = lambda x: x.half()
    qp = q.reshape(N, Hkv, G, d).permute(1, 0, 2, 3).reshape(Hkv, N * G, d)
    s1 = h(h(qp.float() @ kp.float().transpose(-1, -2)) * sc)
    m1 = s1.max(-1, keepdim=True).values
    p1 = h(torch.exp(h(s1 - m1).float()))
    l1 = h(p1.float().sum(-1, keepdim=True))
    o1 = h(p1.float() @ vp.float()).reshape(Hkv, N, G, d).permute(1, 0, 2, 3)
    m1 = m1.reshape(Hkv, N, G, 1).permute(1, 0, 2, 3)
    l1 = l1.reshape(Hkv, N, G, 1).permute(1, 0, 2, 3)
    s2 = h(h(q.reshape(N, Hkv, G, d).float() @ ks.float().transpose(-1, -2)) * sc)
    m2 = s2.max(-1, keepdim=True).values
    p2 = h(torch.exp(h(s2 - m2).float()))
    l2 = h(p2.float().sum(-1, keepdim=True))
    o2 = h(p2.float() @ vs.float())
    m = torch.maximum(m1, m2)
    a, b = h(torch.exp((m1 - m).float())), h(torch.exp((m2 - m).float()))
    return h((o1 * a + o2 * b).float() / (l1 * a + l2 * b).float()).reshape(N, Hq, d)


def _spec_scores(q, k, bits):
    B, kd, Hq, d = q.shape
    Hkv, L = k.shape[1], k.shape[2]
    G = Hq // Hkv
    qf = q.reshape(B, kd, Hkv, G, d).permute(0, 2, 1, 3, 4).reshape(B, Hkv, kd * G, d)
    s = (qf.float() @ k.float().transpose(-1, -2)) * (1 / math.sqrt(d))
    m = ops.load_op("spec").mask_torch(bits, L, kd).repeat_interleave(G, dim=1)[:, None]
    return s, m, (B, kd, Hq, d, Hkv, G)


def spec_correct(q, k, v, bits):
    s, m, (B, kd, Hq, d, Hkv, G) = _spec_scores(q, k, bits)
    p = torch.softmax(s.masked_fill(~m, float("-inf")), -1)
    return (p @ v.float()).reshape(B, Hkv, kd, G, d).permute(0, 2, 1, 3, 4).reshape(B, kd, Hq, d).half()


def spec_cheat_nomax(q, k, v, bits):
    """exp() of the raw scores: overflows on large inputs."""
    s, m, (B, kd, Hq, d, Hkv, G) = _spec_scores(q, k, bits)
    e = torch.where(m, torch.exp(s), torch.zeros_like(s))
    p = (e / e.sum(-1, keepdim=True)).half()
    return (p.float() @ v.float()).reshape(B, Hkv, kd, G, d).permute(0, 2, 1, 3, 4).reshape(B, kd, Hq, d).half()


def test_prefix_fp16_cascade_is_rejected_and_fp32_accepted():
    """The cheat agrees with the standard op at nominal inputs (layer 1) but is rejected by the float64
    layers: the fuzz layer on large magnitudes, the accuracy layer on large magnitudes and needles."""
    op = ops.load_op("prefix")
    keys = ["q", "kp", "vp", "ks", "vs"]
    rep = {}
    for name, shape, dist in (("nominal", dict(N=4, P=2048, S=256), "randn"), ("large", dict(N=4, P=3000, S=200), "large"),
                              ("needle", dict(N=4, P=8192, S=512), "needle_prefix")):
        inp = op.make_inputs(shape, seed=3, dist=dist)
        t = ref64.prefix_ref64(**inp)
        good = prefix_correct(*_t(inp, keys)).float().numpy()
        bad = prefix_cheat_fp16(*_t(inp, keys)).float().numpy()
        assert judge.judge_l2(good, t, dist=dist)["ok"] and judge.judge_l3(good, t, good)["ok"]
        rep[name] = dict(l1=judge.judge_l1(bad, good), l2=judge.judge_l2(bad, t, dist=dist), l3=judge.judge_l3(bad, t, good))
    assert rep["nominal"]["l1"]["ok"] and rep["nominal"]["l2"]["ok"]
    assert not rep["large"]["l2"]["ok"] and not rep["large"]["l3"]["ok"], rep["large"]
    assert rep["needle"]["l2"]["ok"] and not rep["needle"]["l3"]["ok"], rep["needle"]


def test_spec_nomax_fails_only_on_large_inputs():
    op = ops.load_op("spec")
    keys = ["q", "k", "v", "bits"]
    inp = op.make_inputs(dict(B=2, L=3000, k=8), seed=14, dist="large")
    t = ref64.spec_ref64(**inp)
    good = spec_correct(*_t(inp, keys)).float().numpy()
    bad = spec_cheat_nomax(*_t(inp, keys)).float().numpy()
    assert judge.judge_l2(good, t, dist="large")["ok"]
    rep = judge.judge_l2(bad, t, dist="large")
    assert not rep["ok"] and not rep["pattern_ok"]          # NaN where the truth is finite
    inp = op.make_inputs(dict(B=2, L=3000, k=8), seed=13, dist="randn")
    t = ref64.spec_ref64(**inp)
    bad = spec_cheat_nomax(*_t(inp, keys)).float().numpy()
    assert judge.judge_l2(bad, t)["ok"] and judge.judge_l1(bad, spec_correct(*_t(inp, keys)).float().numpy())["ok"]


def test_nerr_and_pattern_follow_the_reference_definitions():
    r = np.array([0.5, 2.0, np.nan, np.inf, 70000.0])
    o = np.array([0.6, 2.0, np.nan, np.inf, np.inf])
    em, ea = judge.nerr(o, r)                    # jointly finite: first two entries, scale max(1, 2.0)
    assert abs(em - 0.05) < 1e-12 and abs(ea - 0.025) < 1e-12
    n, i = judge.pattern(r, half=True)           # 70000 is beyond fp16: counts as Inf
    assert n.tolist() == [False, False, True, False, False] and i.tolist() == [False, False, False, True, True]
    assert judge.judge_l2(o, r)["ok"] is False   # error 0.05 > 1e-2
    assert judge.judge_l2(np.array([0.5, 2.0, np.nan, np.inf, np.inf]), r)["ok"]


def test_select_check_accepts_near_ties_and_rejects_wrong_sets():
    rng = np.random.default_rng(0)
    s = rng.standard_normal(5000)
    top = np.argsort(-s)[:2048]
    assert judge.select_check(np.sort(top), 2048, s, 5000)["ok"]
    wrong = top.copy()
    wrong[0] = np.argsort(-s)[4000]              # a clearly worse position
    assert not judge.select_check(np.sort(wrong), 2048, s, 5000)["ok"]
    s2 = s.copy()
    s2[np.argsort(-s)[2048]] = s[np.argsort(-s)[2047]] + 1e-12    # near-tie at the boundary: either is fine
    swapped = np.sort(np.r_[np.argsort(-s)[:2047], np.argsort(-s)[2048]])
    assert judge.select_check(swapped, 2048, s2, 5000)["ok"]
    assert not judge.select_check(np.sort(top)[:-1], 2047, s, 5000)["ok"]
