"""Kernel module for plain single-token decode on B200: one query per request over that request's own cache.

Not one of the reference's three ops: it measures this op beside them (POST.md:42,47: at parity with the
platform's kernel, bandwidth-bound) and names it as the natural fourth op on the same main loop.  Here it
is the `spec` main loop with one row per request, no draft mask and per-request lengths."""
import torch

from .. import _lib
from ._common import need, stage_in


def _common(q, lens):
    if not isinstance(q, torch.Tensor) or q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("q: expected a float16 or bfloat16 tensor")
    need(q, "q", q.dtype, dims=3)
    B = q.shape[0]
    need(lens, "lens", torch.int32, shape=(B,))
    return q.dtype, B


def kernel(q, k, v, lens, check=False):
    """q (B,Hq,D), k/v (B,Hkv,L,D) fp16 or bf16, lens (B,) int32 with 1 <= lens[b] <= L -> (B,Hq,D).
    Rows at or beyond lens[b] are never used.  Host tensors are copied in and the result returned on the host
    (with the device status word checked; device-resident calls check it only with check=True)."""
    (q, k, v, lens), host = stage_in([q, k, v, lens])
    dt, B = _common(q, lens)
    Hq, D = q.shape[1], q.shape[2]
    need(k, "k", dt, dims=4)
    Hkv, L = k.shape[1], k.shape[2]
    need(k, "k", dt, shape=(B, Hkv, L, D))
    need(v, "v", dt, shape=(B, Hkv, L, D))
    lib = _lib.lib()
    dev = q.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream()
        out = torch.empty_like(q)
        nbytes = lib.vmk_decode_workspace_bytes(B, Hq, Hkv, D, L)
        if nbytes == 0:
            raise _lib.VmkError(-2, "decode: unsupported shape")
        ws = _lib.workspace(nbytes, dev, stream.cuda_stream)
        rc = lib.vmk_decode(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(lens), _lib.ptr(out), B, Hq, Hkv, D, L,
                            1 if dt == torch.bfloat16 else 0, _lib.ptr(ws), ws.numel(),
                            _lib.ptr(_lib.status_word(dev)), stream.cuda_stream)
    _lib.check(rc, "vmk_decode")
    return _lib.finish(out, host, check, dev, "vmk_decode")


def kernel_paged(q, k_pages, v_pages, page_table, lens, check=False):
    """The same over a paged cache: k_pages / v_pages (pages,Hkv,page_size,D), page_table (B,T) int32, lens (B,)
    int32 with lens[b] <= T * page_size; page_size a multiple of 64."""
    dt, B = _common(q, lens)
    Hq, D = q.shape[1], q.shape[2]
    need(k_pages, "k_pages", dt, dims=4)
    pages, Hkv, page_size = k_pages.shape[0], k_pages.shape[1], k_pages.shape[2]
    need(k_pages, "k_pages", dt, shape=(pages, Hkv, page_size, D))
    need(v_pages, "v_pages", dt, shape=(pages, Hkv, page_size, D))
    need(page_table, "page_table", torch.int32, dims=2)
    T = page_table.shape[1]
    need(page_table, "page_table", torch.int32, shape=(B, T))
    if page_size % 64 != 0:
        raise ValueError("page_size must be a multiple of 64")
    L = T * page_size
    lib = _lib.lib()
    dev = q.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream()
        out = torch.empty_like(q)
        nbytes = lib.vmk_decode_workspace_bytes(B, Hq, Hkv, D, L)
        if nbytes == 0:
            raise _lib.VmkError(-2, "decode: unsupported shape")
        ws = _lib.workspace(nbytes, dev, stream.cuda_stream)
        rc = lib.vmk_decode_paged(_lib.ptr(q), _lib.ptr(k_pages), _lib.ptr(v_pages), _lib.ptr(page_table), pages,
                                  page_size, T, _lib.ptr(lens), _lib.ptr(out), B, Hq, Hkv, D, L,
                                  1 if dt == torch.bfloat16 else 0, _lib.ptr(ws), ws.numel(),
                                  _lib.ptr(_lib.status_word(dev)), stream.cuda_stream)
    _lib.check(rc, "vmk_decode_paged")
    return _lib.finish(out, False, check, dev, "vmk_decode_paged")
