"""Op `prefix`: shared-prefix decode.  N requests share a P-token prefix, each has its own S-token
suffix, one decode token per request.

    q (N,Hq,D) fp16      kp, vp (Hkv,P,D) fp16      ks, vs (N,Hkv,S,D) fp16      out (N,Hq,D) fp16

Follows the reference definition ops/prefix.py (generator 15-44, shape lists 11-12 and 147-153).
Extension: an optional `slens` (N,) int32 gives each request's true suffix length (<= S); the
reference has only dense suffixes."""
import numpy as np

NAME = "prefix"
HQ, HKV, D = 32, 8, 128
L1_SHAPE = dict(N=4, P=2048, S=256)
BENCH_SHAPES = [dict(N=8, P=8192, S=512), dict(N=16, P=16384, S=1024), dict(N=32, P=4096, S=256)]
# BASELINE configurations: the CPU-runnable case and the multi-GPU sweep case.
CONFIG_SMALL = dict(N=8, P=4096, S=256)
CONFIG_SWEEP = dict(N=256, P=32768, S=2048, ragged=True)


def make_inputs(shape, seed=0, dist="randn", with_ref_layouts=False):
    """Seeded inputs, bit-identical to the reference generator (ops/prefix.py:15-44): one
    default_rng(seed); float32 normal draws in the order q, kp, vp, ks, vs; the distribution transform;
    then rounding to fp16.  Returns NumPy arrays.  shape["ragged"] (extension) adds `slens` drawn
    uniformly from [0, S] by a separate default_rng(seed + 1), so the tensors stay those of the dense case."""
    rng = np.random.default_rng(seed)
    N, P, S = shape["N"], shape["P"], shape["S"]
    Hq, Hkv, d = shape.get("Hq", HQ), shape.get("Hkv", HKV), shape.get("D", D)
    G = Hq // Hkv
    t = {name: rng.standard_normal(dims, dtype=np.float32)
         for name, dims in (("q", (N, Hq, d)), ("kp", (Hkv, P, d)), ("vp", (Hkv, P, d)),
                            ("ks", (N, Hkv, S, d)), ("vs", (N, Hkv, S, d)))}
    if dist == "large":
        for name in ("q", "kp", "ks"):
            t[name] = t[name] * 8
    elif dist == "needle_prefix":          # one dominant shared key per kv head
        for h in range(Hkv):
            t["kp"][h, rng.integers(0, P)] = t["q"][:, h * G:(h + 1) * G].mean((0, 1)) * 6.0
    elif dist == "needle_suffix":          # one dominant private key per (request, kv head), values shifted
        for n in range(N):
            for h in range(Hkv):
                t["ks"][n, h, rng.integers(0, S)] = t["q"][n, h * G:(h + 1) * G].mean(0) * 6.0
                t["vs"][n, h] += 3.0
    elif dist == "nan_inf":
        t["ks"][N - 1, 0, S - 1, 0] = np.nan
        t["vp"][1, P // 2, 7] = np.inf
    elif dist == "tiny":
        for name, f in (("q", 1e-4), ("kp", 1e-4), ("vp", 1e-6), ("ks", 1e-4), ("vs", 1e-6)):
            t[name] = t[name] * f
    elif dist != "randn":
        raise ValueError(f"unknown dist {dist!r}")
    out = {name: a.astype(np.float16) for name, a in t.items()}
    if shape.get("ragged"):
        out["slens"] = np.random.default_rng(seed + 1).integers(0, S + 1, (N,)).astype(np.int32)
    if with_ref_layouts:
        out.update(build_layouts(out["kp"], out["vp"], out["ks"], out["vs"]))
    return out


def build_layouts(kp, vp, ks, vs):
    """Layouts the standard ops read, never passed to kernel() (reference ops/prefix.py:47-54): per-request full
    caches kf, vf (N,Hkv,P+S,D) for the non-sharing op, and the unified caches ku, vu (1,Hkv,P+N*S,D) -- the
    shared prefix once, then every request's suffix in turn -- for the block-masked op.  NumPy arrays or torch
    tensors."""
    N, Hkv, S, d = ks.shape
    if isinstance(kp, np.ndarray):
        kf = np.concatenate([np.broadcast_to(kp[None], (N,) + kp.shape), ks], axis=2)
        vf = np.concatenate([np.broadcast_to(vp[None], (N,) + vp.shape), vs], axis=2)
        ku = np.concatenate([kp, ks.transpose(1, 0, 2, 3).reshape(Hkv, N * S, d)], axis=1)[None]
        vu = np.concatenate([vp, vs.transpose(1, 0, 2, 3).reshape(Hkv, N * S, d)], axis=1)[None]
        return dict(kf=kf, vf=vf, ku=ku, vu=vu)
    import torch
    kf = torch.cat([kp[None].expand(N, *kp.shape), ks], dim=2)
    vf = torch.cat([vp[None].expand(N, *vp.shape), vs], dim=2)
    ku = torch.cat([kp, ks.permute(1, 0, 2, 3).reshape(Hkv, N * S, d)], dim=1)[None]
    vu = torch.cat([vp, vs.permute(1, 0, 2, 3).reshape(Hkv, N * S, d)], dim=1)[None]
    return dict(kf=kf, vf=vf, ku=ku, vu=vu)


# ------------------------------------------------------------------ standard ops (torch; opponents, not product)
def torch_naive(q, kp, vp, ks, vs, slens=None, kf=None, vf=None, **_):
    """Non-sharing engine: fused SDPA over per-request full caches (reference ops/prefix.py:121-123)."""
    import torch
    import torch.nn.functional as F
    if kf is None:
        lay = build_layouts(kp, vp, ks, vs)
        kf, vf = lay["kf"], lay["vf"]
    mask = None
    if slens is not None:
        P, S = kp.shape[1], ks.shape[2]
        pos = torch.arange(P + S, device=q.device)[None, :]
        mask = (pos < (P + slens.to(q.device).long())[:, None])[:, None, None, :]
    return F.scaled_dot_product_attention(q[:, :, None, :], kf, vf, attn_mask=mask, enable_gqa=True)[:, :, 0, :]


def torch_unified(q, kp, vp, ks, vs, slens=None, ku=None, vu=None, **_):
    """One fused SDPA call over the unified cache with a block mask: the N*G stacked rows of a kv head all see
    the shared prefix, and row (n, g) sees only request n's suffix block (reference ops/prefix.py:126-138, its
    strongest library opponent on this op).  The prefix is read once per kv head."""
    import torch
    import torch.nn.functional as F
    N, Hq, d = q.shape
    Hkv, P = kp.shape[0], kp.shape[1]
    S, G = ks.shape[2], Hq // kp.shape[0]
    if ku is None:
        lay = build_layouts(kp, vp, ks, vs)
        ku, vu = lay["ku"], lay["vu"]
    owner = torch.arange(N * G, device=q.device)[:, None] // G           # request of each stacked row
    col = torch.arange(P + N * S, device=q.device)[None, :]
    end = (owner + 1) * S if slens is None else owner * S + slens.to(q.device).long()[owner[:, 0]][:, None]
    mask = (col < P) | ((col >= P + owner * S) & (col < P + end))
    stacked = q.reshape(N, Hkv, G, d).permute(1, 0, 2, 3).reshape(1, Hkv, N * G, d)
    o = F.scaled_dot_product_attention(stacked, ku, vu, attn_mask=mask)
    return o.reshape(Hkv, N, G, d).permute(1, 0, 2, 3).reshape(N, Hq, d)


def torch_cascade(q, kp, vp, ks, vs, slens=None, **_):
    """The sharing algorithm written with library matmuls: prefix scores for all stacked rows at once, suffix
    scores per request, two fp32 softmax partials merged by log-sum-exp (the reference's `mlx_cascade`,
    ops/prefix.py:100-118, in torch).  Reads every byte once, like kernel(); P and the scores round-trip HBM."""
    import torch
    N, Hq, d = q.shape
    Hkv, S = kp.shape[0], ks.shape[2]
    G = Hq // Hkv
    sc = d ** -0.5
    qh = q.reshape(N, Hkv, G, d)
    qs = qh.permute(1, 0, 2, 3).reshape(Hkv, N * G, d)
    s1 = torch.matmul(qs, kp.transpose(1, 2)).float() * sc                   # (Hkv, N*G, P)
    m1 = s1.amax(-1, keepdim=True)
    p1 = torch.exp(s1 - m1)
    l1 = p1.sum(-1, keepdim=True)
    o1 = torch.matmul(p1.to(q.dtype), vp).float()
    to_req = lambda t: t.reshape(Hkv, N, G, -1).permute(1, 0, 2, 3)
    o1, m1, l1 = to_req(o1), to_req(m1), to_req(l1)
    s2 = torch.matmul(qh, ks.transpose(2, 3)).float() * sc                   # (N, Hkv, G, S)
    if slens is not None:
        dead = torch.arange(S, device=q.device)[None, :] >= slens.to(q.device).long()[:, None]
        s2 = s2.masked_fill(dead[:, None, None, :], float("-inf"))
    m2 = s2.amax(-1, keepdim=True)
    p2 = torch.exp(s2 - torch.where(torch.isinf(m2), torch.zeros_like(m2), m2))
    l2 = p2.sum(-1, keepdim=True)
    o2 = torch.matmul(p2.to(q.dtype), vs).float()
    m = torch.maximum(m1, m2)
    a, b = torch.exp(m1 - m), torch.exp(m2 - m)
    return ((o1 * a + o2 * b) / (l1 * a + l2 * b)).to(q.dtype).reshape(N, Hq, d)


TORCH_REFS = dict(torch_naive=torch_naive, torch_unified=torch_unified, torch_cascade=torch_cascade)
L1_REF = "torch_naive"
L3_REF = "torch_naive"

FUZZ = [(dict(N=1, P=1, S=1), "randn"), (dict(N=3, P=1000, S=77), "randn"), (dict(N=5, P=4097, S=33), "randn"),
        (dict(N=2, P=65536, S=4096), "randn"), (dict(N=33, P=300, S=10), "randn"), (dict(N=64, P=2048, S=64), "randn"),
        (dict(N=4, P=3000, S=200), "large"), (dict(N=4, P=3000, S=200), "needle_prefix"),
        (dict(N=4, P=3000, S=200), "needle_suffix"), (dict(N=4, P=3000, S=200), "nan_inf"),
        (dict(N=4, P=3000, S=200), "tiny"), (dict(N=7, P=8, S=1), "randn")]
L3_CASES = [(dict(N=8, P=1024, S=128), "randn"), (dict(N=8, P=32768, S=1024), "randn"),
            (dict(N=4, P=8192, S=512), "large"), (dict(N=4, P=8192, S=512), "needle_prefix"),
            (dict(N=4, P=8192, S=512), "needle_suffix")]
# Extension cases (no counterpart in the reference): ragged suffix lengths, including zero-length.
FUZZ_EXT = [(dict(N=6, P=777, S=300, ragged=True), "randn"), (dict(N=16, P=2048, S=512, ragged=True), "randn"),
            (dict(N=3, P=64, S=5, ragged=True), "large")]


def rows(shape):
    """Decode rows (query tokens) one call produces."""
    return shape["N"]


def algorithmic_bytes(shape, slens=None):
    """Compulsory HBM traffic of one call: every input byte once, every output byte once."""
    N, P, S = shape["N"], shape["P"], shape["S"]
    Hq, Hkv, d = shape.get("Hq", HQ), shape.get("Hkv", HKV), shape.get("D", D)
    suffix_tokens = int(np.sum(slens)) if slens is not None else N * S
    return 2 * Hkv * P * d * 2 + 2 * Hkv * d * 2 * suffix_tokens + 2 * N * Hq * d * 2


def to_pages(kp, vp, ks, vs, slens, page_size, seed=0, spare=3, fill=np.nan):
    """Extension beyond the reference (contiguous prefix and suffixes): scatters the shared prefix
    kp, vp (Hkv,P,D) and the private suffixes ks, vs (N,Hkv,S,D) (first slens[n] keys of each) into one
    shuffled page pool.  Returns (k_pages, v_pages (pages,Hkv,page_size,D), prefix_table (T_p,) int32,
    suffix_table (N,T_s) int32).  Unused pages and the unused rows of last pages hold `fill`."""
    Hkv, P, D = kp.shape
    N, S = ks.shape[0], ks.shape[2]
    slens = np.full(N, S, dtype=np.int32) if slens is None else np.asarray(slens)
    Tp, Ts = -(-P // page_size), max(1, -(-S // page_size))
    pages = Tp + N * Ts + spare
    perm = np.random.default_rng(seed).permutation(pages).astype(np.int32)
    ptab, stab = perm[:Tp].copy(), perm[Tp:Tp + N * Ts].reshape(N, Ts).copy()
    kpg = np.full((pages, Hkv, page_size, D), fill, dtype=kp.dtype)
    vpg = np.full((pages, Hkv, page_size, D), fill, dtype=vp.dtype)
    for i in range(Tp):
        n = min(page_size, P - i * page_size)
        kpg[ptab[i], :, :n] = kp[:, i * page_size:i * page_size + n]
        vpg[ptab[i], :, :n] = vp[:, i * page_size:i * page_size + n]
    for r in range(N):
        for i in range(Ts):
            n = min(page_size, int(slens[r]) - i * page_size)
            if n <= 0:
                break
            kpg[stab[r, i], :, :n] = ks[r, :, i * page_size:i * page_size + n]
            vpg[stab[r, i], :, :n] = vs[r, :, i * page_size:i * page_size + n]
    return kpg, vpg, ptab, stab
