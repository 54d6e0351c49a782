"""Op definition of plain single-token decode (an extension: the reference measures this op, POST.md:42,47,
but defines no ops/decode.py).  Shapes follow the reference's attention ops: 32 query heads, 8 KV heads,
head dim 128 (ops/spec.py:9).  q (B,Hq,D), k/v (B,Hkv,L,D) fp16, lens (B,) int32."""
import numpy as np

NAME = "decode"
HQ, HKV, D = 32, 8, 128
CONFIG_BENCH = dict(B=64, L=32768)      # 8.6 GB of K and V at full lengths
FUZZ = [(dict(B=1, L=1), "randn"), (dict(B=3, L=700), "ragged"), (dict(B=2, L=4097), "randn"),
        (dict(B=5, L=3000), "ragged"), (dict(B=2, L=2000), "large"), (dict(B=2, L=1000), "nan_pad"),
        (dict(B=17, L=900), "ragged")]


def make_inputs(shape, seed=0, dist="randn"):
    """Seeded inputs in the style of the reference's generators: float32 normal draws q, k, v, then the
    distribution transform, then fp16 rounding.  "ragged": lens ~ U[1, L] with lens[0] = L; "nan_pad": ragged
    with every row at or beyond lens[b] set to NaN (a kernel that read them would show it)."""
    rng = np.random.default_rng(seed)
    B, L = shape["B"], shape["L"]
    q = rng.standard_normal((B, HQ, D), dtype=np.float32)
    k = rng.standard_normal((B, HKV, L, D), dtype=np.float32)
    v = rng.standard_normal((B, HKV, L, D), dtype=np.float32)
    lens = np.full(B, L, dtype=np.int32)
    if dist in ("ragged", "nan_pad"):
        lens = rng.integers(1, L + 1, (B,)).astype(np.int32)
        lens[0] = L
    if dist == "large":
        q, k = q * 4.0, k * 4.0
    if dist == "nan_pad":
        for b in range(B):
            k[b, :, lens[b]:] = np.nan
            v[b, :, lens[b]:] = np.nan
    return dict(q=q.astype(np.float16), k=k.astype(np.float16), v=v.astype(np.float16), lens=lens)


def algorithmic_bytes(shape, lens=None):
    B, L = shape["B"], shape["L"]
    keys = B * L if lens is None else int(np.sum(lens))
    return 2 * HKV * D * 2 * keys + 2 * B * HQ * D * 2


def to_pages(k, v, lens, page_size, seed=0, spare=3, fill=np.nan):
    """Scatters each request's first lens[b] keys into a shuffled page pool: (k_pages, v_pages
    (pages,Hkv,page_size,D), page_table (B,T) int32, -1 where a request has no page)."""
    B, Hkv, L, Dh = k.shape
    T = -(-L // page_size)
    need = [-(-int(n) // page_size) for n in lens]
    pages = sum(need) + spare
    perm = np.random.default_rng(seed).permutation(pages).astype(np.int32)
    kp = np.full((pages, Hkv, page_size, Dh), fill, dtype=k.dtype)
    vp = np.full((pages, Hkv, page_size, Dh), fill, dtype=v.dtype)
    table = np.full((B, T), -1, dtype=np.int32)
    nxt = 0
    for b in range(B):
        for i in range(need[b]):
            pg = perm[nxt]
            nxt += 1
            table[b, i] = pg
            n = min(page_size, int(lens[b]) - i * page_size)
            kp[pg, :, :n] = k[b, :, i * page_size:i * page_size + n]
            vp[pg, :, :n] = v[b, :, i * page_size:i * page_size + n]
    return kp, vp, table
