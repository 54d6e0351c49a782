"""Kernel module for op `spec` (speculative chain / tree verification) on B200.

Drop-in for the reference's kernel module contract (reference kernels/spec_opus55_v7.py:467, called as
fn(**inputs) by verify.py:139); the work is done by sm_100a CUDA behind libvmk_b200's C ABI."""
import torch

from .. import _lib
from ._common import need, stage_in


def kernel(q, k, v, bits, check=False):
    """q (B,kd,Hq,D), k/v (B,Hkv,L,D) fp16 (or all bf16), bits (B,kd) int32 -- or (B,kd,W) int32 words for kd > 32 --
    -> (B,kd,Hq,D) fp16.  The drafts are the last kd cache positions; bit j of bits[b,i] set means
    draft i attends draft j.  Inputs are not modified; host tensors are copied in and the result is
    returned on the host (that path synchronises and raises VmkDeviceStatusError on a non-zero device status
    word; a device-resident call checks only with check=True, else use check_status(device) after synchronising)."""
    (q, k, v, bits), host = stage_in([q, k, v, bits])
    if not isinstance(q, torch.Tensor) or q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("q: expected a float16 or bfloat16 tensor")
    dt = q.dtype                                   # fp16 (the reference's) or bf16, the same for q, k and v
    need(q, "q", dt, dims=4)
    B, kd, Hq, D = q.shape
    need(k, "k", dt, dims=4)
    Hkv, Lk = k.shape[1], k.shape[2]
    need(k, "k", dt, shape=(B, Hkv, Lk, D))
    need(v, "v", dt, shape=(B, Hkv, Lk, D))
    if not isinstance(bits, torch.Tensor) or bits.dtype != torch.int32:
        raise TypeError("bits: expected an int32 tensor")
    if bits.dim() == 2:
        need(bits, "bits", torch.int32, shape=(B, kd))
        words = 1
    else:
        need(bits, "bits", torch.int32, dims=3)
        words = bits.shape[2]
        need(bits, "bits", torch.int32, shape=(B, kd, words))
    L = _lib.lib()
    dev = q.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream()
        out = torch.empty_like(q)
        nbytes = L.vmk_spec_workspace_bytes(B, kd, Hq, Hkv, D, Lk)
        if nbytes == 0:
            raise _lib.VmkError(-2, "spec: unsupported shape")
        ws = _lib.workspace(nbytes, dev, stream.cuda_stream)
        rc = (L.vmk_spec_verify_bf16 if dt == torch.bfloat16 else L.vmk_spec_verify)(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(bits), words, _lib.ptr(out), B, kd, Hq,
                               Hkv, D, Lk, _lib.ptr(ws), ws.numel(), _lib.ptr(_lib.status_word(dev)),
                               stream.cuda_stream)
    _lib.check(rc, "vmk_spec_verify")
    return _lib.finish(out, host, check, dev, "vmk_spec_verify")


def kernel_paged(q, k_pages, v_pages, page_table, L, bits, check=False):
    """`spec` over a paged cache: k_pages / v_pages (pages, Hkv, page_size, D) fp16 are one pool for every
    request, page_table (B, T) int32 maps keys [i * page_size, (i + 1) * page_size) of request b to page
    page_table[b, i]; L is the (common) cache length, T * page_size >= L, page_size a multiple of 64.
    q, bits and the result as in kernel(); the result equals kernel() on the de-paged cache bit for bit."""
    if not isinstance(q, torch.Tensor) or q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("q: expected a float16 or bfloat16 tensor")
    dt = q.dtype
    need(q, "q", dt, dims=4)
    B, kd, Hq, D = q.shape
    need(k_pages, "k_pages", dt, dims=4)
    pages, Hkv, page_size = k_pages.shape[0], k_pages.shape[1], k_pages.shape[2]
    need(k_pages, "k_pages", dt, shape=(pages, Hkv, page_size, D))
    need(v_pages, "v_pages", dt, shape=(pages, Hkv, page_size, D))
    need(page_table, "page_table", torch.int32, dims=2)
    T = page_table.shape[1]
    need(page_table, "page_table", torch.int32, shape=(B, T))
    if page_size % 64 != 0 or T * page_size < L or L <= 0:
        raise ValueError("page_size must be a multiple of 64 and the table must cover L keys")
    if not isinstance(bits, torch.Tensor) or bits.dtype != torch.int32:
        raise TypeError("bits: expected an int32 tensor")
    words = 1 if bits.dim() == 2 else bits.shape[2]
    need(bits, "bits", torch.int32, shape=(B, kd) if bits.dim() == 2 else (B, kd, words))
    lib = _lib.lib()
    dev = q.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream()
        out = torch.empty_like(q)
        nbytes = lib.vmk_spec_workspace_bytes(B, kd, Hq, Hkv, D, L)
        if nbytes == 0:
            raise _lib.VmkError(-2, "spec: unsupported shape")
        ws = _lib.workspace(nbytes, dev, stream.cuda_stream)
        rc = lib.vmk_spec_verify_paged(_lib.ptr(q), _lib.ptr(k_pages), _lib.ptr(v_pages), _lib.ptr(page_table), pages,
                                       page_size, T, _lib.ptr(bits), words, _lib.ptr(out), B, kd, Hq, Hkv, D, L,
                                       1 if dt == torch.bfloat16 else 0,
                                       _lib.ptr(ws), ws.numel(), _lib.ptr(_lib.status_word(dev)), stream.cuda_stream)
    _lib.check(rc, "vmk_spec_verify_paged")
    return _lib.finish(out, False, check, dev, "vmk_spec_verify_paged")
