"""Op `spec`: speculative verification.  kd draft tokens (a chain or a tree) are verified in one pass
against a cache of L tokens whose last kd positions are the drafts themselves.

    q (B,kd,Hq,D) fp16      k, v (B,Hkv,L,D) fp16      bits (B,kd) int32      out (B,kd,Hq,D) fp16

Bit j of bits[b,i] says draft i may attend draft j (ancestors and itself).  Follows the reference
definition ops/spec.py (mask builders 14-25, generator 28-56, shape lists 10-11 and 153-159).
Extension: for kd > 32 `bits` is (B,kd,W) int32 with W = ceil(kd/32) little-endian words, and
shape["max_depth"] caps the depth of generated trees; the reference holds kd <= 32."""
import numpy as np

NAME = "spec"
HQ, HKV, D = 32, 8, 128
L1_SHAPE = dict(B=2, L=4096, k=8)
BENCH_SHAPES = [dict(B=1, L=8192, k=8), dict(B=1, L=32768, k=8), dict(B=4, L=16384, k=4), dict(B=1, L=32768, k=16)]
CONFIG_CHAIN = dict(B=1, L=8192, k=8)                       # with dist="chain"
CONFIG_TREE = dict(B=4, L=32768, k=64, max_depth=8)         # wide-mask extension


def chain_bits(kd):
    """Causal chain: draft i sees drafts 0..i (reference ops/spec.py:14-15).  Python ints, any kd."""
    return [(1 << (i + 1)) - 1 for i in range(kd)]


def tree_bits(kd, rng, max_depth=None):
    """Random tree: node i's parent is uniform over earlier nodes, mask = ancestors-or-self
    (reference ops/spec.py:18-25).  With max_depth (extension) the parent is uniform over earlier nodes
    whose depth is below the cap; without it the draws are exactly the reference's."""
    masks, depth = [], []
    for i in range(kd):
        if i == 0:
            par = -1
        elif max_depth is None:
            par = int(rng.integers(0, i))
        else:
            ok = [j for j in range(i) if depth[j] < max_depth - 1]
            par = ok[int(rng.integers(0, len(ok)))]
        masks.append((1 << i) | (masks[par] if par >= 0 else 0))
        depth.append(depth[par] + 1 if par >= 0 else 0)
    return masks


def pack_bits(rows, kd):
    """List (per batch) of lists of Python-int masks -> int32 array: (B,kd) when kd <= 32 (the
    reference's layout, ops/spec.py:56), else (B,kd,W) little-endian words."""
    B = len(rows)
    if kd <= 32:
        a = np.array([[m & 0xFFFFFFFF for m in r] for r in rows], dtype=np.uint32).reshape(B, kd)
        return a.view(np.int32)
    W = (kd + 31) // 32
    a = np.array([[[(m >> (32 * w)) & 0xFFFFFFFF for w in range(W)] for m in r] for r in rows], dtype=np.uint32)
    return a.reshape(B, kd, W).view(np.int32)


def make_inputs(shape, seed=0, dist="randn"):
    """Seeded inputs, bit-identical to the reference generator (ops/spec.py:28-56): float32 normal
    draws q, k, v; then the per-batch masks from the SAME generator; then the distribution transform;
    then fp16 rounding.  Returns NumPy arrays."""
    rng = np.random.default_rng(seed)
    B, L, kd = shape["B"], shape["L"], shape["k"]
    Hq, Hkv, d = shape.get("Hq", HQ), shape.get("Hkv", HKV), shape.get("D", D)
    G = Hq // Hkv
    q = rng.standard_normal((B, kd, Hq, d), dtype=np.float32)
    k = rng.standard_normal((B, Hkv, L, d), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, L, d), dtype=np.float32)
    if dist == "chain":
        masks = [chain_bits(kd) for _ in range(B)]
    else:
        masks = [tree_bits(kd, rng, shape.get("max_depth")) for _ in range(B)]
    if dist == "large":
        q, k = q * 8.0, k * 8.0
    elif dist == "needle_masked":          # dominant key on the last draft, which row 0 must not see
        j = kd - 1
        for b in range(B):
            if (masks[b][0] >> j) & 1 == 0:
                for h in range(Hkv):
                    k[b, h, L - kd + j] = q[b, 0, h * G:(h + 1) * G].mean(0) * 8.0
                    v[b, h, L - kd + j] += 50.0
    elif dist == "needle_boundary":        # dominant key on the last cache position before the drafts
        for b in range(B):
            for h in range(Hkv):
                k[b, h, L - kd - 1] = q[b, :, h * G:(h + 1) * G].mean((0, 1)) * 6.0
    elif dist == "nan_inf":
        k[0, 0, L // 2, 3] = np.nan
    elif dist == "tiny":
        q, k, v = q * 1e-4, k * 1e-4, v * 1e-6
    elif dist not in ("randn", "chain"):
        raise ValueError(f"unknown dist {dist!r}")
    return dict(q=q.astype(np.float16), k=k.astype(np.float16), v=v.astype(np.float16), bits=pack_bits(masks, kd))


def mask_torch(bits, L, kd):
    """(B,kd,L) bool visibility on the device of `bits` (reference ops/spec.py:123-127, widened)."""
    import torch
    j = torch.arange(kd, device=bits.device)
    w = bits.long() & 0xFFFFFFFF
    if bits.dim() == 2:
        tail = ((w[:, :, None] >> j[None, None, :]) & 1).bool()
    else:
        tail = ((w[:, :, j // 32] >> (j % 32)[None, None, :]) & 1).bool()
    head = torch.ones(bits.shape[0], kd, L - kd, dtype=torch.bool, device=bits.device)
    return torch.cat([head, tail], -1)


# ------------------------------------------------------------------ standard ops (torch; opponents, not product)
def torch_sdpa(q, k, v, bits, **_):
    """Fused SDPA with a dense boolean (B,1,kd,L) mask (reference ops/spec.py:130-133)."""
    import torch.nn.functional as F
    m = mask_torch(bits, k.shape[2], q.shape[1])[:, None]
    return F.scaled_dot_product_attention(q.transpose(1, 2), k, v, attn_mask=m, enable_gqa=True).transpose(1, 2)


def torch_sdpa_fold(q, k, v, bits, **_):
    """GQA folded into kd*G rows per kv head (reference ops/spec.py:136-144)."""
    import torch.nn.functional as F
    B, kd, Hq, d = q.shape
    Hkv, L = k.shape[1], k.shape[2]
    G = Hq // Hkv
    qf = q.reshape(B, kd, Hkv, G, d).permute(0, 2, 1, 3, 4).reshape(B, Hkv, kd * G, d)
    m = mask_torch(bits, L, kd).repeat_interleave(G, dim=1)[:, None]
    o = F.scaled_dot_product_attention(qf, k, v, attn_mask=m)
    return o.reshape(B, Hkv, kd, G, d).permute(0, 2, 1, 3, 4).reshape(B, kd, Hq, d)


TORCH_REFS = dict(torch_sdpa=torch_sdpa, torch_sdpa_fold=torch_sdpa_fold)
L1_REF = "torch_sdpa"
L3_REF = "torch_sdpa"

FUZZ = [(dict(B=1, L=8, k=8), "randn"), (dict(B=1, L=9, k=1), "randn"), (dict(B=2, L=4097, k=8), "randn"),
        (dict(B=1, L=100000, k=16), "randn"), (dict(B=3, L=777, k=5), "randn"), (dict(B=1, L=4096, k=31), "randn"),
        (dict(B=2, L=3000, k=8), "chain"), (dict(B=2, L=3000, k=8), "large"), (dict(B=2, L=3000, k=8), "needle_masked"),
        (dict(B=2, L=3000, k=8), "needle_boundary"), (dict(B=2, L=3000, k=8), "nan_inf"), (dict(B=2, L=3000, k=8), "tiny"),
        (dict(B=8, L=2049, k=4), "randn"), (dict(B=1, L=31, k=31), "needle_masked")]
L3_CASES = [(dict(B=1, L=1024, k=8), "randn"), (dict(B=1, L=32768, k=8), "randn"), (dict(B=1, L=65536, k=16), "randn"),
            (dict(B=2, L=8192, k=8), "large"), (dict(B=2, L=8192, k=8), "needle_boundary")]
# Extension cases (no counterpart in the reference): kd > 32 with multi-word masks.
FUZZ_EXT = [(dict(B=2, L=2000, k=64, max_depth=8), "randn"), (dict(B=1, L=64, k=64), "chain"),
            (dict(B=1, L=5000, k=33), "randn"), (dict(B=2, L=1500, k=48, max_depth=8), "needle_masked")]


def rows(shape):
    return shape["B"] * shape["k"]


def algorithmic_bytes(shape):
    B, L, kd = shape["B"], shape["L"], shape["k"]
    Hq, Hkv, d = shape.get("Hq", HQ), shape.get("Hkv", HKV), shape.get("D", D)
    return 2 * B * Hkv * L * d * 2 + 2 * B * kd * Hq * d * 2 + 4 * B * kd * ((kd + 31) // 32)


def to_pages(k, v, page_size, seed=0, spare=3, fill=np.nan):
    """Extension beyond the reference (which stores one contiguous cache per request): scatters k, v
    (B,Hkv,L,D) into a shuffled page pool.  Returns (k_pages, v_pages (pages,Hkv,page_size,D), page_table
    (B,T) int32).  The pool holds `spare` unused pages, and the unused rows of every last page, filled with
    `fill`: a kernel that read them would show it."""
    B, Hkv, L, D = k.shape
    T = -(-L // page_size)
    pages = B * T + spare
    rng = np.random.default_rng(seed)
    perm = rng.permutation(pages)[:B * T].astype(np.int32).reshape(B, T)
    kp = np.full((pages, Hkv, page_size, D), fill, dtype=k.dtype)
    vp = np.full((pages, Hkv, page_size, D), fill, dtype=v.dtype)
    for b in range(B):
        for i in range(T):
            n = min(page_size, L - i * page_size)
            kp[perm[b, i], :, :n] = k[b, :, i * page_size:i * page_size + n]
            vp[perm[b, i], :, :n] = v[b, :, i * page_size:i * page_size + n]
    return kp, vp, perm
