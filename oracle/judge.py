"""Acceptance criteria of the reference verifier, restated (test infrastructure only).

Three layers, as in the reference verify.py:160-241:
  L1  allclose(atol=rtol=1e-2, equal_nan=True) against the platform's standard op;
  L2  against the float64 truth: NaN and Inf masks equal after rounding the truth to fp16 (fp32 when
      the kernel returned float32) -- for NaN/Inf inputs a mismatch may instead match the standard op's
      pattern -- and normalised max error <= 1e-2;
  L3  max and mean normalised error <= 2 * max(standard op's error, 2^-11).
"Normalised" divides by max(1, max|truth|) over jointly finite entries."""
import numpy as np

L2_TOL = 1e-2
L3_FLOOR = 2.0 ** -11


def nerr(o, r):
    """(max, mean) normalised error over entries finite in both (reference verify.py:160-166)."""
    o, r = np.asarray(o, dtype=np.float64), np.asarray(r, dtype=np.float64)
    fin = np.isfinite(r) & np.isfinite(o)
    if not fin.any():
        return 0.0, 0.0
    scale = max(1.0, float(np.abs(r[fin]).max()))
    d = np.abs(o[fin] - r[fin]) / scale
    return float(d.max()), float(d.mean())


def pattern(a, half=True):
    """NaN and Inf masks after rounding to the output precision (reference verify.py:169-171):
    truth values beyond the fp16 range count as Inf."""
    with np.errstate(over="ignore", invalid="ignore"):
        a = np.asarray(a).astype(np.float16 if half else np.float32)
    return np.isnan(a), np.isinf(a)


def judge_l1(out, std):
    out, std = np.asarray(out, dtype=np.float64), np.asarray(std, dtype=np.float64)
    if out.shape != std.shape:
        return dict(ok=False, error=f"shape {out.shape} != {std.shape}")
    ok = bool(np.allclose(out, std, atol=1e-2, rtol=1e-2, equal_nan=True))
    with np.errstate(invalid="ignore"):
        diff = np.abs(out - std)
    return dict(ok=ok, maxdiff=float(np.nanmax(diff)) if diff.size and not np.isnan(diff).all() else 0.0)


def judge_l2(out, truth, half=True, dist="randn", std=None):
    out, truth = np.asarray(out, dtype=np.float64), np.asarray(truth, dtype=np.float64)
    if out.shape != truth.shape:
        return dict(ok=False, error=f"shape {out.shape} != {truth.shape}")
    pn, pi = pattern(out, half)
    rn, ri = pattern(truth, half)
    pat = bool((pn == rn).all() and (pi == ri).all())
    rep = {}
    if not pat and dist == "nan_inf" and std is not None:
        sn, si = pattern(np.asarray(std, dtype=np.float64), half)
        pat = bool((pn == sn).all() and (pi == si).all())
        rep["pattern_vs"] = "std_op"
    if not pat:
        rep["pattern_detail"] = dict(nan_got=int(pn.sum()), nan_exp=int(rn.sum()), inf_got=int(pi.sum()),
                                     inf_exp=int(ri.sum()))
    em, ea = nerr(out, truth)
    rep.update(ok=bool(pat and em <= L2_TOL), pattern_ok=pat, err_max=em, err_mean=ea)
    return rep


def judge_l3(out, truth, std):
    em, ea = nerr(out, truth)
    sm, sa = nerr(std, truth)
    ok = em <= 2 * max(sm, L3_FLOOR) and ea <= 2 * max(sa, L3_FLOOR)
    return dict(ok=bool(ok), err_max=em, err_mean=ea, std_err_max=sm, std_err_mean=sa)


def select_check(idx, cnt, scores64, n, topk=2048, rel_eps=2e-6):
    """Integer-stage check for `dsa`: idx[:cnt] must be a duplicate-free set of valid positions which
    contains every position whose float64 score clears the top-k boundary by more than eps and none
    that falls short of it by more than eps; when the boundary gap itself exceeds eps the set must be
    exactly the float64 top-k.  eps = rel_eps * max|score| bounds the fp32 accumulation error of the
    64-head, 128-wide indexer sum; it is far below the fp16 rounding the acceptance bar allows."""
    idx = np.asarray(idx)[:int(cnt)].astype(np.int64)
    s = np.asarray(scores64)[:n]
    rep = dict(cnt=int(cnt))
    want = min(n, topk)
    if int(cnt) != want or len(np.unique(idx)) != want or (idx < 0).any() or (idx >= n).any():
        rep.update(ok=False, error=f"cnt {cnt} (want {want}), unique {len(np.unique(idx))}, range "
                                   f"[{idx.min() if idx.size else 0},{idx.max() if idx.size else 0}] n={n}")
        return rep
    if n <= topk:
        rep.update(ok=bool((np.sort(idx) == np.arange(n)).all()), exact=True)
        return rep
    srt = np.sort(s)[::-1]
    thr_in, thr_out = srt[topk - 1], srt[topk]
    eps = rel_eps * max(1e-30, float(np.abs(s).max()))
    chosen = np.zeros(n, dtype=bool)
    chosen[idx] = True
    must = s > thr_in + eps
    never = s < thr_out - eps
    exact_set = set(np.argpartition(-s, topk - 1)[:topk].tolist())
    rep.update(gap=float(thr_in - thr_out), eps=eps, exact=bool(set(idx.tolist()) == exact_set),
               missed=int((must & ~chosen).sum()), wrong=int((never & chosen).sum()))
    ok = rep["missed"] == 0 and rep["wrong"] == 0
    if thr_in - thr_out > eps:
        ok = ok and rep["exact"]
    rep["ok"] = bool(ok)
    return rep
