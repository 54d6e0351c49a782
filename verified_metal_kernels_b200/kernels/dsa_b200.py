"""Kernel module for op `dsa` (DeepSeek sparse attention decode) on B200.

Drop-in for the reference's kernel module contract (reference kernels/dsa_opus55_v7.py:946, called as
fn(**inputs) by verify.py:139 with lens=None when absent); indexer, top-2048 select and sparse MLA
attention are sm_100a CUDA behind libvmk_b200's C ABI."""
import torch

from .. import _lib
from ._common import need, stage_in

H, DK, DC, HI, DI, TOPK = 128, 576, 512, 64, 128, 2048

# A page-locked host `kv` is read in place by stage 3's gather (only the selected rows cross the link).  False
# makes kernel() copy it to the device whole, like every other host input.
HOST_CACHE_IN_PLACE = True


def _half(t, name="q"):
    """The call's 16-bit type, taken from one of its tensors: fp16 (the reference's) or bf16."""
    if not isinstance(t, torch.Tensor) or t.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"{name}: expected a float16 or bfloat16 tensor")
    return t.dtype


def _sfx(dt):
    return "_bf16" if dt == torch.bfloat16 else ""


def _check(q, kv, iq, ik, w, lens):
    dt = _half(q)
    need(q, "q", dt, dims=3)
    B = q.shape[0]
    need(q, "q", dt, shape=(B, H, DK))
    need(kv, "kv", dt, dims=3)
    L = kv.shape[1]
    need(kv, "kv", dt, shape=(B, L, DK))
    need(iq, "iq", dt, shape=(B, HI, DI))
    need(ik, "ik", dt, shape=(B, L, DI))
    need(w, "w", torch.float32, shape=(B, HI))
    if lens is not None:
        need(lens, "lens", torch.int32, shape=(B,))
    return B, L


def kernel(q, kv, iq, ik, w, lens=None, return_selection=False, check=False):
    """q (B,128,576), kv (B,L,576), iq (B,64,128), ik (B,L,128) fp16 (or all four bf16), w (B,64) fp32, lens
    (B,) int32 or None -> (B,128,512) of the same 16-bit type.  With return_selection=True also returns (idx (B,2048) int32 ascending,
    cnt (B,) int32), the integer stage's result.  Inputs are not modified; host tensors are copied in
    and the result is returned on the host.

    A page-locked host `kv` is NOT copied whole: the index keys go to the device, stages 1 and 2 run there,
    and stage 3 is fed by `gather`, which reads only the selected rows out of host memory (2048 of L rows per
    request over the link).  The result is bit-identical to the all-on-device call.

    Device status: calls with host tensors synchronise and raise VmkDeviceStatusError when a kernel reported a
    bounded wait that ran out (the output is then invalid) or a clamped index; device-resident calls do so only
    with check=True (otherwise call check_status(device) after synchronising)."""
    if (HOST_CACHE_IN_PLACE and isinstance(kv, torch.Tensor) and not kv.is_cuda and kv.is_pinned() and kv.dim() == 3 and kv.shape[1] > TOPK
            and kv.dtype in (torch.float16, torch.bfloat16) and kv.is_contiguous()):
        return _kernel_host_cache(q, kv, iq, ik, w, lens, return_selection)
    (q, kv, iq, ik, w, lens), host = stage_in([q, kv, iq, ik, w, lens])
    B, L = _check(q, kv, iq, ik, w, lens)
    lib = _lib.lib()
    dev = q.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream()
        out = torch.empty(B, H, DC, dtype=q.dtype, device=dev)
        idx = torch.empty(B, TOPK, dtype=torch.int32, device=dev) if return_selection else None
        cnt = torch.empty(B, dtype=torch.int32, device=dev) if return_selection else None
        nbytes = lib.vmk_dsa_workspace_bytes(B, L)
        ws = _lib.workspace(nbytes, dev, stream.cuda_stream)
        rc = getattr(lib, "vmk_dsa_decode" + _sfx(q.dtype))(_lib.ptr(q), _lib.ptr(kv), _lib.ptr(iq), _lib.ptr(ik), _lib.ptr(w), _lib.ptr(lens),
                                _lib.ptr(out), _lib.ptr(idx), _lib.ptr(cnt), B, L, _lib.ptr(ws), ws.numel(),
                                _lib.ptr(_lib.status_word(dev)), stream.cuda_stream)
    _lib.check(rc, "vmk_dsa_decode")
    out = _lib.finish(out, host, check, dev, "vmk_dsa_decode")
    return (out, idx, cnt) if return_selection else out


def kernel_paged(q, kv_pages, iq, ik_pages, w, page_table, lens, return_selection=False, check=False):
    """`dsa` over a paged cache: kv_pages (pages,page_size,576) and ik_pages (pages,page_size,128) are pools paged
    alike, page_table (B,T) int32 maps positions [i * page_size, (i + 1) * page_size) of request b to page
    page_table[b, i]; lens (B,) int32 are the cache lengths (required); page_size a multiple of 128 and
    T * page_size > 2048.  fp16 or bf16.  The result (and the selection, in logical positions) equals kernel() on
    the de-paged tensors bit for bit."""
    dt = _half(q)
    need(q, "q", dt, dims=3)
    B = q.shape[0]
    need(q, "q", dt, shape=(B, H, DK))
    need(kv_pages, "kv_pages", dt, dims=3)
    pages, page_size = kv_pages.shape[0], kv_pages.shape[1]
    need(kv_pages, "kv_pages", dt, shape=(pages, page_size, DK))
    need(ik_pages, "ik_pages", dt, shape=(pages, page_size, DI))
    need(iq, "iq", dt, shape=(B, HI, DI))
    need(w, "w", torch.float32, shape=(B, HI))
    need(page_table, "page_table", torch.int32, dims=2)
    T = page_table.shape[1]
    need(page_table, "page_table", torch.int32, shape=(B, T))
    need(lens, "lens", torch.int32, shape=(B,))
    L = T * page_size
    if page_size % 128 != 0 or L <= TOPK:
        raise ValueError("page_size must be a multiple of 128 and the table must cover more than 2048 positions")
    lib = _lib.lib()
    dev = q.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream()
        out = torch.empty(B, H, DC, dtype=dt, device=dev)
        idx = torch.empty(B, TOPK, dtype=torch.int32, device=dev) if return_selection else None
        cnt = torch.empty(B, dtype=torch.int32, device=dev) if return_selection else None
        ws = _lib.workspace(lib.vmk_dsa_workspace_bytes(B, L), dev, stream.cuda_stream)
        rc = lib.vmk_dsa_decode_paged(_lib.ptr(q), _lib.ptr(kv_pages), _lib.ptr(iq), _lib.ptr(ik_pages), _lib.ptr(w),
                                      _lib.ptr(page_table), pages, page_size, T, _lib.ptr(lens), _lib.ptr(out),
                                      _lib.ptr(idx), _lib.ptr(cnt), B, L, 1 if dt == torch.bfloat16 else 0,
                                      _lib.ptr(ws), ws.numel(), _lib.ptr(_lib.status_word(dev)), stream.cuda_stream)
    _lib.check(rc, "vmk_dsa_decode_paged")
    out = _lib.finish(out, False, check, dev, "vmk_dsa_decode_paged")
    return (out, idx, cnt) if return_selection else out


def _kernel_host_cache(q, kv, iq, ik, w, lens, return_selection):
    """The op with the latent cache left in page-locked host memory (see kernel)."""
    (q, iq, ik, w, lens), _ = stage_in([q, iq, ik, w, lens])
    B, L = kv.shape[0], kv.shape[1]
    if tuple(kv.shape) != (B, L, DK):
        raise ValueError(f"kv: expected shape {(B, L, DK)}, got {tuple(kv.shape)}")
    need(q, "q", kv.dtype, shape=(B, H, DK))
    scores, hist = indexer_hist(iq, ik, w, lens)
    idx, cnt = select(scores, lens, hist)
    kv_sel, idx_sel = gather(kv, idx, cnt)
    out = _lib.finish(attend(q, kv_sel, idx_sel, cnt), True, True, q.device, "dsa (host-resident cache)")
    return (out, idx, cnt) if return_selection else out


def gather(kv, idx, cnt):
    """Compaction of the selected rows: (kv_sel (B,2048,576) fp16, idx_sel (B,2048) int32 = 0..cnt-1) on the
    device of `idx`.  `kv` (B,L,576) fp16 is a device tensor or a page-locked host tensor, which the kernel
    reads in place."""
    if not isinstance(kv, torch.Tensor) or kv.dtype not in (torch.float16, torch.bfloat16) or kv.dim() != 3 or kv.shape[2] != DK:
        raise TypeError("kv: expected a (B,L,576) fp16 or bf16 tensor")
    if not kv.is_contiguous() or not (kv.is_cuda or kv.is_pinned()):
        raise ValueError("kv: expected a C-contiguous device tensor or page-locked host tensor")
    B, L = kv.shape[0], kv.shape[1]
    need(idx, "idx", torch.int32, shape=(B, TOPK))
    need(cnt, "cnt", torch.int32, shape=(B,))
    lib = _lib.lib()
    dev = idx.device
    with torch.cuda.device(dev):
        kv_sel = torch.empty(B, TOPK, DK, dtype=kv.dtype, device=dev)
        idx_sel = torch.empty(B, TOPK, dtype=torch.int32, device=dev)
        rc = lib.vmk_dsa_gather(kv.data_ptr(), _lib.ptr(idx), _lib.ptr(cnt), _lib.ptr(kv_sel), _lib.ptr(idx_sel), B, L,
                                _lib.ptr(_lib.status_word(dev)), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "vmk_dsa_gather")
    return kv_sel, idx_sel


def indexer(iq, ik, w, lens=None):
    """Stage 1 alone: fp32 scores (B,L); positions at or beyond lens[b], and everything when L <= 2048,
    are left as NaN-free zeros."""
    B, L = ik.shape[0], ik.shape[1]
    need(iq, "iq", torch.float16, shape=(B, HI, DI))
    need(ik, "ik", torch.float16, shape=(B, L, DI))
    need(w, "w", torch.float32, shape=(B, HI))
    lib = _lib.lib()
    with torch.cuda.device(ik.device):
        scores = torch.zeros(B, L, dtype=torch.float32, device=ik.device)
        rc = lib.vmk_dsa_indexer(_lib.ptr(iq), _lib.ptr(ik), _lib.ptr(w), _lib.ptr(lens), _lib.ptr(scores), B, L,
                                 _lib.ptr(_lib.status_word(ik.device)), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "vmk_dsa_indexer")
    return scores


def indexer_hist(iq, ik, w, lens=None):
    """Stage 1 with the fused first radix level: (scores (B,L) fp32, hist (B,2048) int32)."""
    B, L = ik.shape[0], ik.shape[1]
    dt = _half(ik, "ik")
    need(iq, "iq", dt, shape=(B, HI, DI))
    need(ik, "ik", dt, shape=(B, L, DI))
    need(w, "w", torch.float32, shape=(B, HI))
    lib = _lib.lib()
    with torch.cuda.device(ik.device):
        scores = torch.zeros(B, L, dtype=torch.float32, device=ik.device)
        hist = torch.empty(B, 2048, dtype=torch.int32, device=ik.device)
        rc = getattr(lib, "vmk_dsa_indexer_hist" + _sfx(dt))(_lib.ptr(iq), _lib.ptr(ik), _lib.ptr(w), _lib.ptr(lens), _lib.ptr(scores),
                                      _lib.ptr(hist), B, L, _lib.ptr(_lib.status_word(ik.device)),
                                      torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "vmk_dsa_indexer_hist")
    return scores, hist


def quantize_e4m3(x):
    """Row-wise fp8 quantisation of a (..., 128) tensor: (bytes of torch.float8_e4m3fn values as uint8, fp32 scale
    per row) with x ~ scale * e4m3, scale = max|row| / 448 (1 for an all-zero row)."""
    amax = x.float().abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (x.float() / scale.unsqueeze(-1)).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).contiguous(), scale.contiguous()


def indexer_hist_fp8(iq8, iq_scale, ik8, ik_scale, w, lens=None):
    """Stage 1 on fp8 index queries and keys (see quantize_e4m3): (scores (B,L) fp32, hist (B,2048) int32)."""
    need(ik8, "ik8", torch.uint8, dims=3)
    B, L = ik8.shape[0], ik8.shape[1]
    need(ik8, "ik8", torch.uint8, shape=(B, L, DI))
    need(iq8, "iq8", torch.uint8, shape=(B, HI, DI))
    need(iq_scale, "iq_scale", torch.float32, shape=(B, HI))
    need(ik_scale, "ik_scale", torch.float32, shape=(B, L))
    need(w, "w", torch.float32, shape=(B, HI))
    lib = _lib.lib()
    with torch.cuda.device(ik8.device):
        scores = torch.zeros(B, L, dtype=torch.float32, device=ik8.device)
        hist = torch.empty(B, 2048, dtype=torch.int32, device=ik8.device)
        rc = lib.vmk_dsa_indexer_hist_fp8(_lib.ptr(iq8), _lib.ptr(iq_scale), _lib.ptr(ik8), _lib.ptr(ik_scale), _lib.ptr(w),
                                          _lib.ptr(lens), _lib.ptr(scores), _lib.ptr(hist), B, L,
                                          _lib.ptr(_lib.status_word(ik8.device)), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "vmk_dsa_indexer_hist_fp8")
    return scores, hist


def index_project(x, wq, ww, w_scale=1.0):
    """The projection in front of stage 1 (outside the reference's op, ops/dsa.py:8-9): x (B,Dx) activation,
    wq (8192,Dx) and ww (64,Dx) weights stored (out, in), all fp16 or all bf16 -> (iq (B,64,128) of the same type,
    w (B,64) fp32 = w_scale * x @ ww^T), the `iq` and `w` inputs of kernel()."""
    dt = _half(x, "x")
    need(x, "x", dt, dims=2)
    B, Dx = x.shape
    need(wq, "wq", dt, shape=(HI * DI, Dx))
    need(ww, "ww", dt, shape=(HI, Dx))
    if Dx % 8 != 0:
        raise ValueError("Dx must be a multiple of 8")
    dev = x.device
    with torch.cuda.device(dev):
        iq = torch.empty(B, HI, DI, dtype=dt, device=dev)
        w = torch.empty(B, HI, dtype=torch.float32, device=dev)
        rc = _lib.lib().vmk_dsa_index_project(_lib.ptr(x), _lib.ptr(wq), _lib.ptr(ww), float(w_scale), _lib.ptr(iq),
                                              _lib.ptr(w), B, Dx, 1 if dt == torch.bfloat16 else 0,
                                              _lib.ptr(_lib.status_word(dev)), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "vmk_dsa_index_project")
    return iq, w


def kernel_projected(q, kv, x, wq, ww, ik, w_scale=1.0, lens=None, return_selection=False, check=False):
    """The op with the indexer's queries and head weights computed here from the activation x (B,Dx) and the
    projection weights (see index_project), then the usual three stages."""
    iq, w = index_project(x, wq, ww, w_scale)
    return kernel(q, kv, iq, ik, w, lens, return_selection=return_selection, check=check)


def kernel_fp8_index(q, kv, iq8, iq_scale, ik8, ik_scale, w, lens=None, return_selection=False):
    """The op with the index queries and keys in fp8 (q and kv stay fp16 or bf16): stage 1 on fp8, then the
    usual select and sparse attention.  Host tensors are copied in and the result comes back on the host; a
    page-locked host `kv` is read in place (only the selected rows cross the link), as in kernel()."""
    if (HOST_CACHE_IN_PLACE and isinstance(kv, torch.Tensor) and not kv.is_cuda and kv.is_pinned() and kv.dim() == 3
            and kv.shape[1] > TOPK and kv.dtype in (torch.float16, torch.bfloat16) and kv.is_contiguous()):
        (q, iq8, iq_scale, ik8, ik_scale, w, lens), _ = stage_in([q, iq8, iq_scale, ik8, ik_scale, w, lens])
        scores, hist = indexer_hist_fp8(iq8, iq_scale, ik8, ik_scale, w, lens)
        idx, cnt = select(scores, lens, hist)
        kv_sel, idx_sel = gather(kv, idx, cnt)
        out = _lib.finish(attend(q, kv_sel, idx_sel, cnt), True, True, q.device, "dsa, fp8 index keys (host-resident cache)")
        return (out, idx, cnt) if return_selection else out
    (q, kv, iq8, iq_scale, ik8, ik_scale, w, lens), host = stage_in([q, kv, iq8, iq_scale, ik8, ik_scale, w, lens])
    scores, hist = indexer_hist_fp8(iq8, iq_scale, ik8, ik_scale, w, lens)
    idx, cnt = select(scores, lens, hist)
    out = _lib.finish(attend(q, kv, idx, cnt), host, False, q.device, "dsa, fp8 index keys")
    return (out, idx, cnt) if return_selection else out


def select(scores, lens=None, hist=None):
    """Stage 2 alone: (idx (B,2048) int32 ascending, cnt (B,) int32).  `hist` is stage 1's fused histogram."""
    need(scores, "scores", torch.float32, dims=2)
    B, L = scores.shape
    lib = _lib.lib()
    with torch.cuda.device(scores.device):
        idx = torch.empty(B, TOPK, dtype=torch.int32, device=scores.device)
        cnt = torch.empty(B, dtype=torch.int32, device=scores.device)
        if hist is None:
            rc = lib.vmk_dsa_select(_lib.ptr(scores), _lib.ptr(lens), _lib.ptr(idx), _lib.ptr(cnt), B, L,
                                    torch.cuda.current_stream().cuda_stream)
        else:
            rc = lib.vmk_dsa_select_hist(_lib.ptr(scores), _lib.ptr(hist), _lib.ptr(lens), _lib.ptr(idx), _lib.ptr(cnt),
                                         B, L, torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "vmk_dsa_select")
    return idx, cnt


def attend(q, kv, idx, cnt):
    """Stage 3 alone: absorbed-MLA attention over given selections."""
    B, L = kv.shape[0], kv.shape[1]
    dt = _half(q)
    need(q, "q", dt, shape=(B, H, DK))
    need(kv, "kv", dt, shape=(B, L, DK))
    need(idx, "idx", torch.int32, shape=(B, TOPK))
    need(cnt, "cnt", torch.int32, shape=(B,))
    lib = _lib.lib()
    dev = q.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream()
        out = torch.empty(B, H, DC, dtype=dt, device=dev)
        ws = _lib.workspace(lib.vmk_dsa_attend_workspace_bytes(B), dev, stream.cuda_stream)
        rc = getattr(lib, "vmk_dsa_attend" + _sfx(dt))(_lib.ptr(q), _lib.ptr(kv), _lib.ptr(idx), _lib.ptr(cnt), _lib.ptr(out), B, L,
                                _lib.ptr(ws), ws.numel(), _lib.ptr(_lib.status_word(dev)), stream.cuda_stream)
    _lib.check(rc, "vmk_dsa_attend")
    return out


def set_indexer_variant(name):
    """Chooses the stage-1 implementation: "mma" (mma.sync, warp-level) or "tcgen05" (tensor memory)."""
    rc = _lib.lib().vmk_dsa_set_indexer_variant({"mma": 0, "tcgen05": 1}[name])
    _lib.check(rc, "vmk_dsa_set_indexer_variant")


ATTEND_VARIANTS = {"mma": 0, "tcgen05": 1, "tcgen05_tma": 2, "tcgen05_pair": 3}
DEFAULT_ATTEND_VARIANT = "tcgen05_pair"


def set_select_cluster(csize):
    """CTAs per request of the top-k selection on long rows: 1, 2, 4 or 8; 0 (the default) = the largest size whose
    CTAs fit in one wave.  The selected set does not depend on it."""
    _lib.check(_lib.lib().vmk_dsa_set_select_cluster(int(csize)), "vmk_dsa_set_select_cluster")


def set_attend_variant(name):
    """Chooses the stage-3 implementation: "mma" (warp-level mma.sync), "tcgen05" (tensor memory, one CTA per
    request and value half, rows gathered by cp.async from four warps), "tcgen05_tma" (the same with the rows
    gathered by TMA tile::gather4) or "tcgen05_pair" (tensor memory, a cluster of two CTAs per request that share
    the score product: the default)."""
    rc = _lib.lib().vmk_dsa_set_attend_variant(ATTEND_VARIANTS[name])
    _lib.check(rc, "vmk_dsa_set_attend_variant")
