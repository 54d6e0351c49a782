"""Float64 ground truth for the three ops (NumPy only; test infrastructure, never on the product path).

Each function follows the arithmetic of the reference definition it cites and accepts the extensions
this repository adds (ragged suffix lengths, multi-word draft masks), which reduce to the reference's
behaviour when absent.
"""
import math

import numpy as np

TOPK = 2048          # reference ops/dsa.py:15
DC = 512             # latent (value) width, reference ops/dsa.py:15
DSA_SCALE = 1.0 / math.sqrt(128 + 64)   # reference ops/dsa.py:17


def _f64(x):
    return np.asarray(x).astype(np.float32).astype(np.float64) if np.asarray(x).dtype == np.float16 \
        else np.asarray(x).astype(np.float64)


def _softmax_rows_times(s, v):
    """Row softmax of s (r, l) applied to v (l, d), with the reference's max-subtracted form
    (reference ops/prefix.py:65-69).  NaN / Inf propagate exactly as in NumPy."""
    with np.errstate(invalid="ignore", over="ignore"):
        s = s - s.max(-1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(-1, keepdims=True)
        return p @ v


# ------------------------------------------------------------------------------------------ prefix
def prefix_ref64(q, kp, vp, ks, vs, slens=None, **_):
    """Shared-prefix decode truth (reference ops/prefix.py:57-70).

    q (N,Hq,D); kp,vp (Hkv,P,D); ks,vs (N,Hkv,S,D).  Request n attends the P shared keys followed by
    its own suffix keys.  `slens` (N,) is this repository's extension: only the first slens[n] suffix
    keys of request n exist.  Computed per (request, kv head) so the (N,Hkv,P+S,D) float64 copies the
    reference materialises are never built; the arithmetic per row is the same."""
    q, kp, vp, ks, vs = (_f64(x) for x in (q, kp, vp, ks, vs))
    N, Hq, d = q.shape
    Hkv = kp.shape[0]
    G = Hq // Hkv
    out = np.empty((N, Hq, d))
    inv = 1.0 / math.sqrt(d)
    for n in range(N):
        sl = ks.shape[2] if slens is None else int(np.asarray(slens)[n])
        for h in range(Hkv):
            k = np.concatenate([kp[h], ks[n, h, :sl]], axis=0)
            v = np.concatenate([vp[h], vs[n, h, :sl]], axis=0)
            s = (q[n, h * G:(h + 1) * G] @ k.T) * inv
            out[n, h * G:(h + 1) * G] = _softmax_rows_times(s, v)
    return out


# ------------------------------------------------------------------------------------------ spec
def spec_allowed(bits, L, kd):
    """(B,kd,L) bool visibility (reference ops/spec.py:59-66).  Every row sees the L-kd cache
    positions; draft row i sees draft j iff bit j of its mask is set.  `bits` is (B,kd) int32 as in the
    reference, or (B,kd,W) little-endian 32-bit words (this repository's extension for kd > 32)."""
    bits = np.asarray(bits)
    B = bits.shape[0]
    a = np.ones((B, kd, L), dtype=bool)
    j = np.arange(kd)
    if bits.ndim == 2:
        w = bits.astype(np.int64)
        a[:, :, L - kd:] = ((w[:, :, None] >> j[None, None, :]) & 1).astype(bool)
    else:
        w = bits.astype(np.int64) & 0xFFFFFFFF
        a[:, :, L - kd:] = ((w[:, :, j // 32] >> (j % 32)[None, None, :]) & 1).astype(bool)
    return a


def spec_ref64(q, k, v, bits, **_):
    """Speculative-verification truth (reference ops/spec.py:69-82): masked scores are -inf, float64
    softmax over all L positions.  q (B,kd,Hq,D); k,v (B,Hkv,L,D)."""
    q, k, v = (_f64(x) for x in (q, k, v))
    B, kd, Hq, d = q.shape
    Hkv, L = k.shape[1], k.shape[2]
    G = Hq // Hkv
    a = spec_allowed(bits, L, kd)
    out = np.empty((B, kd, Hq, d))
    inv = 1.0 / math.sqrt(d)
    for b in range(B):
        for h in range(Hkv):
            qq = q[b, :, h * G:(h + 1) * G].reshape(kd * G, d)          # rows ordered (draft i, group g)
            s = (qq @ k[b, h].T) * inv
            s = np.where(np.repeat(a[b], G, axis=0), s, -np.inf)
            out[b, :, h * G:(h + 1) * G] = _softmax_rows_times(s, v[b, h]).reshape(kd, G, d)
    return out


# ------------------------------------------------------------------------------------------ dsa
def dsa_scores64(iq, ik, w):
    """Indexer scores (B,L): sum_h w[b,h] * relu(iq[b,h] . ik[b,l]) (reference ops/dsa.py:53-58)."""
    iq, ik = _f64(iq), _f64(ik)
    w = np.asarray(w).astype(np.float64)
    B, L = ik.shape[0], ik.shape[1]
    s = np.empty((B, L))
    step = 16384
    for b in range(B):
        for l0 in range(0, L, step):
            t = ik[b, l0:l0 + step] @ iq[b].T                         # (l, Hi)
            s[b, l0:l0 + step] = np.maximum(t, 0) @ w[b]
    return s


def dsa_ref_select64(iq, ik, w, lens=None):
    """Scores and the selected index set per request (reference ops/dsa.py:53-66): all n valid
    positions when n <= 2048, else an (unordered) top-2048 by score."""
    s = dsa_scores64(iq, ik, w)
    B, L = s.shape
    sel = []
    for b in range(B):
        n = L if lens is None else int(np.asarray(lens)[b])
        if n <= TOPK:
            sel.append(np.arange(n))
        else:
            sel.append(np.argpartition(-s[b, :n], TOPK - 1)[:TOPK])
    return s, sel


def dsa_ref64(q, kv, iq, ik, w, lens=None, sel=None, **_):
    """DeepSeek sparse attention decode truth (reference ops/dsa.py:69-83): absorbed-MLA softmax over
    the selected latent rows, scale 1/sqrt(192), value = first 512 latent columns."""
    if sel is None:
        _, sel = dsa_ref_select64(iq, ik, w, lens)
    q = _f64(q)
    B, H = q.shape[0], q.shape[1]
    out = np.zeros((B, H, DC))
    for b in range(B):
        rows = _f64(np.asarray(kv)[b, sel[b]])
        out[b] = _softmax_rows_times((q[b] @ rows.T) * DSA_SCALE, rows[:, :DC])
    return out


def dsa_index_project64(x, wq, ww, w_scale=1.0):
    """The projection in front of the indexer, which the reference keeps outside its op (ops/dsa.py:8-9) and has no
    truth for: iq (B,64,128) = x @ wq^T and w (B,64) = w_scale * x @ ww^T in float64, unrounded.  x (B,Dx);
    wq (8192,Dx), ww (64,Dx) stored (out features, in features)."""
    x, wq, ww = _f64(x), _f64(wq), _f64(ww)
    iq = (x @ wq.T).reshape(x.shape[0], 64, 128)
    return iq, float(w_scale) * (x @ ww.T)


REF64 = dict(prefix=prefix_ref64, spec=spec_ref64, dsa=dsa_ref64)


def decode_ref64(q, k, v, lens, **_):
    """Plain single-token decode (an op the reference measures but does not define, POST.md:42): request b's
    query attends keys [0, lens[b]) of its own cache.  Same arithmetic as spec_ref64 (ops/spec.py:69-82) with one
    unmasked row per request.  q (B,Hq,D), k/v (B,Hkv,L,D) -> (B,Hq,D) float64."""
    q, k, v = _f64(q), _f64(k), _f64(v)
    B, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    out = np.empty((B, Hq, D), dtype=np.float64)
    for b in range(B):
        n = int(lens[b])
        qb = q[b].reshape(Hkv, G, D)
        for h in range(Hkv):
            s = (qb[h] @ k[b, h, :n].T) / np.sqrt(D)
            out[b, h * G:(h + 1) * G] = _softmax_rows_times(s, v[b, h, :n])
    return out
