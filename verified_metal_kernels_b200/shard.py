"""One-process-per-GPU sharding of the three ops.

`dsa` and `spec` own a cache per batch element and `prefix` a suffix per request, so those units are
split across ranks with no data-path collective: each rank computes the outputs of its own units.
Where a single shared key range must be divided (the shared prefix of `prefix`; one long speculative
cache when there are more ranks than batch elements) each rank computes partials over its slice, ONE
collective moves packed (m, l, o[128]) records -- an all-to-all that hands every rank only the rows it
owns, or an all-gather when every rank wants everything -- and a local merge finishes.  Partials arrive in
local memory through the collective (NCCL on GPUs, Gloo in the CPU tests); no kernel reads a peer's memory.

The reference splits keys inside one GPU and merges the same way (kernels/prefix_opus55_v8.py:211-261 is
its merge, 320-331 its split plan); this module is that plan taken across GPUs."""
import os

RECORD = 130      # floats per packed partial record: m, l, o[128]


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


# ---------------------------------------------------------------------------------------------------------
# packed records and their exchange
# ---------------------------------------------------------------------------------------------------------
def pack_records(m, l, o):
    """(rows,), (rows,), (rows, D) -> (rows, D + 2) records (m, l, o[D]): the layout that crosses between ranks."""
    import torch
    return torch.cat([m[..., None], l[..., None], o], dim=-1).contiguous()


def exchange_records(send, in_rows, out_rows, group=None, out=None):
    """ONE all-to-all of packed records.  `send` (sum(in_rows), R) holds the rows for rank 0, then for rank 1, ...;
    the result (sum(out_rows), R) holds the rows received from rank 0, then from rank 1, ... (`out`, when given,
    is a contiguous tensor of that shape to receive into).  Works on NCCL and on Gloo."""
    import torch
    import torch.distributed as dist
    n_out = int(sum(out_rows))
    if out is None:
        out = torch.empty((n_out, send.shape[1]), dtype=send.dtype, device=send.device)
    assert out.is_contiguous() and out.shape[0] == n_out and send.shape[0] == int(sum(in_rows))
    dist.all_to_all_single(out, send.contiguous(), [int(x) for x in out_rows], [int(x) for x in in_rows], group=group)
    return out


def gather_records(rec, group=None):
    """ONE all-gather of a rank's packed records (rows, R) -> (W, rows, R) on every rank."""
    import torch
    import torch.distributed as dist
    w = dist.get_world_size(group)
    got = torch.empty((w * rec.shape[0],) + tuple(rec.shape[1:]), dtype=rec.dtype, device=rec.device)
    dist.all_gather_into_tensor(got, rec.contiguous(), group=group)      # rank r's rows at [r * rows, (r + 1) * rows)
    return got.view((w,) + tuple(rec.shape))


def gather_partials(pm, pl, po, group=None):
    """All-gather of separate (m (rows,), l (rows,), o (rows,D)) partials as one packed buffer; returns
    (W,rows), (W,rows), (W,rows,D) views of the gathered records."""
    got = gather_records(pack_records(pm, pl, po), group)
    return got[..., 0], got[..., 1], got[..., 2:]


def merge_partials_reference(gm, gl, go):
    """Host-side statement of the log-sum-exp merge (what vmk_lse_merge computes on the GPU), used by
    the CPU multi-process tests: m is in the base-2 scaled-score domain."""
    import torch
    M = gm.max(dim=0).values
    w = torch.where(torch.isinf(gm) & (gm < 0), torch.zeros_like(gm), torch.exp2(gm - M))
    return (w[..., None] * go).sum(0) / (w * gl).sum(0)[..., None]


def merge_records_reference(rec):
    """merge_partials_reference on packed records (parts, rows, D+2) -> (rows, D)."""
    return merge_partials_reference(rec[..., 0], rec[..., 1], rec[..., 2:])


class CudaPartials:
    """The partial computations and the merge on the GPU, through the C ABI (the `compute` object of
    prefix_hybrid / spec_split; the CPU tests pass a float64 NumPy object with the same methods)."""

    def __init__(self, bf16=False):
        self.bf16 = int(bool(bf16))

    @staticmethod
    def _ctx(t):
        import torch
        from . import _lib
        dev = t.device
        stream = torch.cuda.current_stream(dev)
        return _lib, _lib.lib(), dev, stream.cuda_stream

    def empty(self, shape, like):
        import torch
        return torch.empty(shape, dtype=torch.float32, device=like.device)

    def prefix_records(self, q_all, kp, vp, h0):
        """Records (N * Hq_cov, 130), row (n, head) at n * Hq_cov + head, of every request of q_all (N, Hq, D) over
        this rank's slice kp, vp (Hkv_cov, P_r, D) of the shared prefix, which holds kv heads [h0, h0 + Hkv_cov)."""
        _lib, L, dev, st = self._ctx(q_all)
        N, Hq, D = q_all.shape
        Hkv_cov, Pr = kp.shape[0], kp.shape[1]
        G = self.G
        Hq_cov = Hkv_cov * G
        rec = self.empty((N * Hq_cov, RECORD), q_all)
        nbytes = L.vmk_prefix_workspace_bytes(N, Hq_cov, Hkv_cov, D, Pr, 0)
        ws = _lib.workspace(nbytes, dev, st)
        q_ptr = q_all.data_ptr() + h0 * G * D * q_all.element_size()
        rc = L.vmk_prefix_partial_packed(q_ptr, Hq, _lib.ptr(kp), _lib.ptr(vp), None, None, None, N, Hq_cov, Hkv_cov, D,
                                         Pr, 0, 0, Pr, 0, self.bf16, _lib.ptr(rec), _lib.ptr(ws), ws.numel(),
                                         _lib.ptr(_lib.status_word(dev)), st)
        _lib.check(rc, "vmk_prefix_partial_packed (shared prefix)")
        return rec

    def suffix_records(self, q_loc, ks, vs, slens, out):
        """Records of this rank's own requests over their private suffixes, written into `out` (n * Hq, 130)."""
        _lib, L, dev, st = self._ctx(q_loc)
        n, Hq, D = q_loc.shape
        Hkv, S = ks.shape[1], ks.shape[2]
        nbytes = L.vmk_prefix_workspace_bytes(n, Hq, Hkv, D, 64, S)
        ws = _lib.workspace(nbytes, dev, st)
        rc = L.vmk_prefix_partial_packed(_lib.ptr(q_loc), Hq, None, None, _lib.ptr(ks), _lib.ptr(vs), _lib.ptr(slens), n,
                                         Hq, Hkv, D, 64, S, 0, 0, 1, self.bf16, _lib.ptr(out), _lib.ptr(ws), ws.numel(),
                                         _lib.ptr(_lib.status_word(dev)), st)
        _lib.check(rc, "vmk_prefix_partial_packed (suffixes)")

    def spec_records(self, q, k, v, bits, has_drafts):
        """Records (B * kd * Hq, 130) of q (B, kd, Hq, D) over k, v (B, Hkv, Ls, D), a slice of the cache that ends
        with the kd draft positions (has_drafts) or holds none of them."""
        _lib, L, dev, st = self._ctx(q)
        B, kd, Hq, D = q.shape
        Hkv, Ls = k.shape[1], k.shape[2]
        words = 1 if bits.dim() == 2 else bits.shape[2]
        rec = self.empty((B * kd * Hq, RECORD), q)
        ws = _lib.workspace(L.vmk_spec_workspace_bytes(B, kd, Hq, Hkv, D, Ls), dev, st)
        rc = L.vmk_spec_partial_packed(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(bits), words, B, kd, Hq, Hkv, D,
                                       Ls, 0, Ls, -1 if has_drafts else Ls, self.bf16, _lib.ptr(rec), _lib.ptr(ws),
                                       ws.numel(), _lib.ptr(_lib.status_word(dev)), st)
        _lib.check(rc, "vmk_spec_partial_packed")
        return rec

    def merge(self, buf):
        """(parts, rows, 130) records -> (rows, 128) in the call's 16-bit type."""
        import torch
        _lib, L, dev, st = self._ctx(buf)
        parts, rows = buf.shape[0], buf.shape[1]
        out = torch.empty((rows, RECORD - 2), dtype=torch.bfloat16 if self.bf16 else torch.float16, device=dev)
        if rows:
            rc = L.vmk_lse_merge_packed(_lib.ptr(buf), parts, rows, RECORD - 2, self.bf16, _lib.ptr(out), st)
            _lib.check(rc, "vmk_lse_merge_packed")
        return out


# ---------------------------------------------------------------------------------------------------------
# prefix: hybrid sharding.  Suffixes are owned by request; the shared prefix is split between the ranks, by kv
# head when the head count divides (8 heads over 8, 4 or 2 GPUs) and by key range otherwise.  Every rank computes
# prefix partials for ALL requests on its slice and suffix partials for ITS requests; one all-to-all hands each
# rank the prefix partials of its own requests; a local merge finishes.  Bytes read per rank ~ 1/W of the op's.
# ---------------------------------------------------------------------------------------------------------
class PrefixHybridPlan:
    """Who reads what.  mode 'head': rank r reads kv heads heads[r] = [h0, h1) over every key; mode 'key': every
    head over keys keys[r] = [lo, hi) (64-aligned).  req[r] = [lo, hi) are the requests rank r owns."""

    def __init__(self, N, Hq, Hkv, P, world_size, mode=None):
        self.N, self.Hq, self.Hkv, self.P, self.world = N, Hq, Hkv, P, world_size
        self.G = Hq // Hkv
        self.req = [unit_range(N, r, world_size) for r in range(world_size)]
        if mode is None:
            mode = "head" if Hkv % world_size == 0 else "key"
        if mode == "head" and Hkv % world_size != 0:
            raise ValueError("the head split needs a kv-head count that the world size divides")
        self.mode = mode
        if mode == "head":
            per = Hkv // world_size
            self.heads = [(r * per, (r + 1) * per) for r in range(world_size)]
            self.keys = [(0, P)] * world_size
        else:
            self.heads = [(0, Hkv)] * world_size
            self.keys = [key_range(P, r, world_size) for r in range(world_size)]

    def q_heads_covered(self, rank):
        h0, h1 = self.heads[rank]
        return (h1 - h0) * self.G

    def prefix_slice(self, kp, rank):
        """This rank's slice of a full (Hkv, P, D) prefix tensor (a view for the head split, a copy otherwise)."""
        (h0, h1), (lo, hi) = self.heads[rank], self.keys[rank]
        return kp[h0:h1] if self.mode == "head" else kp[:, lo:hi].contiguous()

    def send_rows(self, rank):
        """Rows of this rank's prefix records that go to each destination (its requests x the heads I cover)."""
        return [(hi - lo) * self.q_heads_covered(rank) for lo, hi in self.req]

    def recv_rows(self, rank):
        """Rows received from each source (my requests x the heads that source covers)."""
        lo, hi = self.req[rank]
        return [(hi - lo) * self.q_heads_covered(s) for s in range(self.world)]

    def parts(self):
        """Partials merged per output row: one (head split) or W (key split) prefix partials plus the suffix's."""
        return 2 if self.mode == "head" else self.world + 1

    def bytes_read(self, rank, slens, S, elt=2, D=128):
        """Algorithmic input bytes of rank `rank`: its prefix slice, its requests' suffixes, every query."""
        (h0, h1), (klo, khi) = self.heads[rank], self.keys[rank]
        lo, hi = self.req[rank]
        suf = float(sum(slens[lo:hi])) if slens is not None else float((hi - lo) * S)
        return 2 * (h1 - h0) * (khi - klo) * D * elt + 2 * self.Hkv * D * elt * suf + self.N * self.Hq * D * elt


def prefix_hybrid(q_all, kp_slice, vp_slice, ks_loc, vs_loc, slens_loc, plan, group=None, compute=None,
                  side_stream=None, check=False):
    """Shared-prefix decode over `plan.world` ranks with ONE exchange.

    q_all (N, Hq, D): every request's query, on every rank (2 MB at N = 256).  kp_slice, vp_slice: this rank's
    slice of the shared prefix, (Hkv / W, P, D) for the head split or (Hkv, P_r, D) for the key split
    (plan.prefix_slice).  ks_loc, vs_loc (n_loc, Hkv, S, D), slens_loc (n_loc) or None: the private suffixes of the
    requests this rank owns, plan.req[rank].  Returns out (n_loc, Hq, D), the outputs of those requests.

    Steps: prefix records for all N requests on the slice; suffix records for the own requests (on `side_stream`,
    a torch.cuda.Stream, when given: the first is tensor-bound, the second HBM-bound); one all-to-all of
    (rows, 130) fp32 records so that each rank receives only its own requests' rows; vmk_lse_merge_packed.
    check=True synchronises and raises VmkError if the device status word is non-zero."""
    import torch
    import torch.distributed as dist
    rank = dist.get_rank(group)
    if compute is None:
        compute = CudaPartials()
    compute.G = plan.G
    lo, hi = plan.req[rank]
    n_loc, Hq, W = hi - lo, plan.Hq, plan.world
    D = q_all.shape[2]
    rows = n_loc * Hq
    parts = plan.parts()
    buf = compute.empty((parts, rows, RECORD), q_all)

    has_suffix = ks_loc is not None and n_loc > 0 and ks_loc.shape[2] > 0
    cuda = q_all.is_cuda
    if has_suffix:
        q_loc = q_all[lo:hi]
        if side_stream is not None and cuda:
            main = torch.cuda.current_stream(q_all.device)
            side_stream.wait_stream(main)
            buf.record_stream(side_stream)
            with torch.cuda.stream(side_stream):
                compute.suffix_records(q_loc, ks_loc, vs_loc, slens_loc, buf[parts - 1])
        else:
            compute.suffix_records(q_loc, ks_loc, vs_loc, slens_loc, buf[parts - 1])
    elif rows:
        buf[parts - 1].zero_()
        buf[parts - 1, :, 0] = float("-inf")

    send = compute.prefix_records(q_all, kp_slice, vp_slice, plan.heads[rank][0])
    if plan.mode == "key":
        exchange_records(send, plan.send_rows(rank), plan.recv_rows(rank), group, out=buf[:W].view(W * rows, RECORD))
    else:
        recv = exchange_records(send, plan.send_rows(rank), plan.recv_rows(rank), group)
        if rows:
            hq_cov = plan.q_heads_covered(rank)
            buf[0].view(n_loc, W, hq_cov, RECORD).copy_(recv.view(W, n_loc, hq_cov, RECORD).permute(1, 0, 2, 3))
    if has_suffix and side_stream is not None and cuda:
        torch.cuda.current_stream(q_all.device).wait_stream(side_stream)
    out = compute.merge(buf).view(n_loc, Hq, D)
    if check and cuda:
        from . import _lib
        _lib.raise_on_status(q_all.device, "prefix_hybrid")
    return out


# ---------------------------------------------------------------------------------------------------------
# spec: batch elements over the ranks; with more ranks than elements, each element's cache is split by position
# over a group of ranks, and one all-to-all inside the group leaves every member with the merged result of its
# share of the output rows.
# ---------------------------------------------------------------------------------------------------------
class SpecSplitPlan:
    """world_size ranks over B batch elements with rows_per_elem = kd * Hq output rows each and caches of L keys.
    world_size <= B: elems[r] = [lo, hi) whole elements, no exchange (split is False).  Otherwise rank r works on
    element elem[r] with the ranks members[elem[r]]; as member j of g it reads keys keys[r] = [lo, hi) and owns the
    merged output rows own_rows[r] = [r0, r1) of that element."""

    def __init__(self, B, rows_per_elem, L, world_size):
        self.B, self.rows, self.L, self.world = B, rows_per_elem, L, world_size
        self.split = world_size > B
        if not self.split:
            self.elems = [unit_range(B, r, world_size) for r in range(world_size)]
            return
        self.elem = [r * B // world_size for r in range(world_size)]
        self.members = [[r for r in range(world_size) if self.elem[r] == b] for b in range(B)]
        self.keys, self.own_rows = [], []
        for r in range(world_size):
            grp = self.members[self.elem[r]]
            j = grp.index(r)
            self.keys.append(key_range(L, j, len(grp)))
            self.own_rows.append(unit_range(rows_per_elem, j, len(grp)))

    def has_drafts(self, rank):
        """The drafts are the last positions of the cache: the member whose slice ends at L holds them."""
        return self.keys[rank][1] == self.L

    def send_rows(self, rank):
        grp = self.members[self.elem[rank]]
        return [(self.own_rows[d][1] - self.own_rows[d][0]) if d in grp else 0 for d in range(self.world)]

    def recv_rows(self, rank):
        grp = self.members[self.elem[rank]]
        mine = self.own_rows[rank][1] - self.own_rows[rank][0]
        return [mine if s in grp else 0 for s in range(self.world)]


def spec_split(q, k_slice, v_slice, bits, plan, group=None, compute=None, check=False):
    """Speculative verification of ONE batch element whose cache is split by position over a group of ranks
    (plan.split must hold).  q (1, kd, Hq, D) and bits (1, kd[, W]) are the element's; k_slice, v_slice
    (1, Hkv, hi - lo, D) are this rank's keys plan.keys[rank] of its cache.  Returns (rows, D) and the range
    [r0, r1) of the element's kd * Hq output rows they are (row = draft * Hq + head)."""
    import torch.distributed as dist
    rank = dist.get_rank(group)
    if compute is None:
        compute = CudaPartials()
    grp = plan.members[plan.elem[rank]]
    r0, r1 = plan.own_rows[rank]
    kd_rows = plan.rows
    lo, hi = plan.keys[rank]
    assert k_slice.shape[2] == hi - lo and q.shape[0] == 1 and q.shape[1] * q.shape[2] == kd_rows
    if plan.has_drafts(rank) and hi - lo < q.shape[1]:
        raise ValueError("the slice that ends the cache must hold all draft positions")
    rec = compute.spec_records(q, k_slice, v_slice, bits, plan.has_drafts(rank))
    buf = exchange_records(rec, plan.send_rows(rank), plan.recv_rows(rank), group)
    out = compute.merge(buf.view(len(grp), r1 - r0, RECORD))
    if check and q.is_cuda:
        from . import _lib
        _lib.raise_on_status(q.device, "spec_split")
    return out, (r0, r1)


def spec_kv_split(q, k, v, bits, group=None, check=True):
    """Speculative verification with every cache split by position across ALL ranks (every rank holds the full
    tensors or at least its slice; rank r reads keys [lo, hi) only).  One all-gather of packed records, then a
    local merge.  Returns (B,kd,Hq,D) fp16 on every rank."""
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
        rec = torch.empty(rows, RECORD, dtype=torch.float32, device=dev)
        ws = _lib.workspace(L.vmk_spec_workspace_bytes(B, kd, Hq, Hkv, D, Lk), dev, stream.cuda_stream)
        rc = L.vmk_spec_partial_packed(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(bits), words, B, kd, Hq, Hkv, D, Lk,
                                       lo, hi, -1, 0, _lib.ptr(rec), _lib.ptr(ws), ws.numel(),
                                       _lib.ptr(_lib.status_word(dev)), stream.cuda_stream)
        _lib.check(rc, "vmk_spec_partial_packed")
        got = gather_records(rec, group)
        out = torch.empty(B, kd, Hq, D, dtype=torch.float16, device=dev)
        rc = L.vmk_lse_merge_packed(_lib.ptr(got), w, rows, D, 0, _lib.ptr(out), stream.cuda_stream)
        _lib.check(rc, "vmk_lse_merge_packed")
        if check:
            _lib.raise_on_status(dev, "spec_kv_split")
    return out
