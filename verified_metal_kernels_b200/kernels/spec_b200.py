"""Kernel module for op `spec` (speculative chain / tree verification) on B200.

Drop-in for the reference's kernel module contract (reference kernels/spec_opus55_v7.py:467, called as
fn(**inputs) by verify.py:139); the work is done by sm_100a CUDA behind libvmk_b200's C ABI."""
import torch

from .. import _lib
from ._common import need, stage_in


def kernel(q, k, v, bits):
    """q (B,kd,Hq,D), k/v (B,Hkv,L,D) fp16, bits (B,kd) int32 -- or (B,kd,W) int32 words for kd > 32 --
    -> (B,kd,Hq,D) fp16.  The drafts are the last kd cache positions; bit j of bits[b,i] set means
    draft i attends draft j.  Inputs are not modified; host tensors are copied in and the result is
    returned on the host."""
    (q, k, v, bits), host = stage_in([q, k, v, bits])
    need(q, "q", torch.float16, dims=4)
    B, kd, Hq, D = q.shape
    need(k, "k", torch.float16, dims=4)
    Hkv, Lk = k.shape[1], k.shape[2]
    need(k, "k", torch.float16, shape=(B, Hkv, Lk, D))
    need(v, "v", torch.float16, shape=(B, Hkv, Lk, D))
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
        rc = L.vmk_spec_verify(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(bits), words, _lib.ptr(out), B, kd, Hq,
                               Hkv, D, Lk, _lib.ptr(ws), ws.numel(), _lib.ptr(_lib.status_word(dev)),
                               stream.cuda_stream)
    _lib.check(rc, "vmk_spec_verify")
    return out.cpu() if host else out
