"""One-process-per-GPU sharding of the three ops.

`dsa` and `spec` own a cache per batch element and `prefix` a suffix per request, so those units are
split across ranks with no data-path collective: each rank computes the outputs of its own units.
The one exchange this path ever needs is the merge of split partials (m, l, o) when a single shared
key range is divided between ranks (a long shared prefix, or one long speculative cache): each rank
computes partials over its key range with vmk_*_partial, the partials are all-gathered through
torch.distributed, and every rank merges locally with vmk_lse_merge.  Partials arrive in local memory
through the collective; no kernel reads a peer's memory."""
import os


def world():
    """(rank, local_rank, world_size) from the torchrun environment (1 process when absent)."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def unit_range(n_units, rank, world_size):
    """Contiguous [lo, hi) of `n_units` independent units owned by `rank`; sizes differ by at most one,
    and ranks beyond n_units get an empty range."""
    base, extra = divmod(n_units, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def key_range(n_keys, rank, world_size, align=64):
    """Contiguous [lo, hi) of a shared key range owned by `rank`, boundaries aligned to `align` keys."""
    blocks = (n_keys + align - 1) // align
    lo, hi = unit_range(blocks, rank, world_size)
    return min(lo * align, n_keys), min(hi * align, n_keys)


def shard_inputs(opname, inputs, rank, world_size):
    """The slice of a full input dict that `rank` owns (views, no copies) and its unit range.
    prefix: requests (the shared prefix is replicated); spec, dsa: batch elements."""
    if opname == "prefix":
        lo, hi = unit_range(inputs["q"].shape[0], rank, world_size)
        out = dict(inputs)
        for k in ("q", "ks", "vs", "slens"):
            if inputs.get(k) is not None:
                out[k] = inputs[k][lo:hi]
        return out, (lo, hi)
    lo, hi = unit_range(inputs["q"].shape[0], rank, world_size)
    return {k: (None if v is None else v[lo:hi]) for k, v in inputs.items()}, (lo, hi)


def gather_partials(pm, pl, po, group=None):
    """All-gather of one rank's (m (rows,), l (rows,), o (rows,D)) partials -> stacked (W,rows[,D])
    tensors on every rank.  Works on any torch.distributed backend (NCCL on GPUs, Gloo on CPU)."""
    import torch
    import torch.distributed as dist
    w = dist.get_world_size(group)
    gm = [torch.empty_like(pm) for _ in range(w)]
    gl = [torch.empty_like(pl) for _ in range(w)]
    go = [torch.empty_like(po) for _ in range(w)]
    dist.all_gather(gm, pm.contiguous(), group=group)
    dist.all_gather(gl, pl.contiguous(), group=group)
    dist.all_gather(go, po.contiguous(), group=group)
    return torch.stack(gm), torch.stack(gl), torch.stack(go)


def merge_partials_reference(gm, gl, go):
    """Host-side statement of the log-sum-exp merge (what vmk_lse_merge computes on the GPU), used by
    the CPU multi-process tests: m is in the base-2 scaled-score domain."""
    import torch
    M = gm.max(dim=0).values
    w = torch.where(torch.isinf(gm) & (gm < 0), torch.zeros_like(gm), torch.exp2(gm - M))
    return (w[..., None] * go).sum(0) / (w * gl).sum(0)[..., None]


def prefix_kv_split(q, kp, vp, ks, vs, slens=None, group=None):
    """Shared-prefix decode with the PREFIX keys split across ranks (every rank holds all requests'
    queries; rank r reads only its slice of kp/vp, and rank 0 also reads the suffixes).  One all-gather
    of (m, l, o), then a local merge.  Returns (N,Hq,D) fp16 on every rank."""
    import torch
    import torch.distributed as dist
    from . import _lib
    rank, w = dist.get_rank(group), dist.get_world_size(group)
    N, Hq, D = q.shape
    Hkv, P = kp.shape[0], kp.shape[1]
    S = ks.shape[2]
    lo, hi = key_range(P, rank, w)
    L = _lib.lib()
    dev = q.device
    rows = N * Hq
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream()
        pm = torch.empty(rows, dtype=torch.float32, device=dev)
        pl = torch.empty(rows, dtype=torch.float32, device=dev)
        po = torch.empty(rows, D, dtype=torch.float32, device=dev)
        ws = _lib.workspace(L.vmk_prefix_workspace_bytes(N, Hq, Hkv, D, P, S), dev, stream.cuda_stream)
        rc = L.vmk_prefix_partial(_lib.ptr(q), _lib.ptr(kp), _lib.ptr(vp), _lib.ptr(ks), _lib.ptr(vs), _lib.ptr(slens),
                                  N, Hq, Hkv, D, P, S, lo, hi, int(rank == 0), _lib.ptr(pm), _lib.ptr(pl), _lib.ptr(po),
                                  _lib.ptr(ws), ws.numel(), _lib.ptr(_lib.status_word(dev)), stream.cuda_stream)
        _lib.check(rc, "vmk_prefix_partial")
        gm, gl, go = gather_partials(pm, pl, po, group)
        out = torch.empty(N, Hq, D, dtype=torch.float16, device=dev)
        rc = L.vmk_lse_merge(_lib.ptr(gm), _lib.ptr(gl), _lib.ptr(go), w, rows, D, _lib.ptr(out), stream.cuda_stream)
        _lib.check(rc, "vmk_lse_merge")
    return out


def spec_kv_split(q, k, v, bits, group=None):
    """Speculative verification of ONE long cache split by position across ranks (every rank holds the
    full tensors or at least its slice; rank r reads keys [lo, hi) only).  One all-gather of (m, l, o),
    then a local merge.  Returns (B,kd,Hq,D) fp16 on every rank."""
    import torch
    import torch.distributed as dist
    from . import _lib
    rank, w = dist.get_rank(group), dist.get_world_size(group)
    B, kd, Hq, D = q.shape
    Hkv, Lk = k.shape[1], k.shape[2]
    words = 1 if bits.dim() == 2 else bits.shape[2]
    lo, hi = key_range(Lk, rank, w)
    L = _lib.lib()
    dev = q.device
    rows = B * kd * Hq
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream()
        pm = torch.empty(rows, dtype=torch.float32, device=dev)
        pl = torch.empty(rows, dtype=torch.float32, device=dev)
        po = torch.empty(rows, D, dtype=torch.float32, device=dev)
        ws = _lib.workspace(L.vmk_spec_workspace_bytes(B, kd, Hq, Hkv, D, Lk), dev, stream.cuda_stream)
        rc = L.vmk_spec_partial(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(bits), words, B, kd, Hq, Hkv, D, Lk, lo,
                                hi, _lib.ptr(pm), _lib.ptr(pl), _lib.ptr(po), _lib.ptr(ws), ws.numel(),
                                _lib.ptr(_lib.status_word(dev)), stream.cuda_stream)
        _lib.check(rc, "vmk_spec_partial")
        gm, gl, go = gather_partials(pm, pl, po, group)
        out = torch.empty(B, kd, Hq, D, dtype=torch.float16, device=dev)
        rc = L.vmk_lse_merge(_lib.ptr(gm), _lib.ptr(gl), _lib.ptr(go), w, rows, D, _lib.ptr(out), stream.cuda_stream)
        _lib.check(rc, "vmk_lse_merge")
    return out
