"""Kernel module for op `prefix` (shared-prefix decode) on B200.

Drop-in for the reference's kernel module contract: a top-level `kernel(...)` taking the op's inputs as
keyword arguments (reference kernels/prefix_opus55_v8.py:282, called as fn(**inputs) by verify.py:139).
The work is done by hand-written sm_100a CUDA reached through libvmk_b200's C ABI."""
import torch

from .. import _lib
from ._common import need, stage_in


def kernel(q, kp, vp, ks, vs, slens=None):
    """q (N,Hq,D), kp/vp (Hkv,P,D), ks/vs (N,Hkv,S,D) fp16 -> (N,Hq,D) fp16 on the inputs' device.

    `slens` (N,) int32, optional: true suffix length per request.  Inputs are not modified.  Host (CPU)
    tensors are accepted: they are copied to the current CUDA device first and the result is returned
    on the host, which is the end-to-end path measured by bench.py."""
    (q, kp, vp, ks, vs, slens), host = stage_in([q, kp, vp, ks, vs, slens])
    need(q, "q", torch.float16, dims=3)
    N, Hq, D = q.shape
    need(kp, "kp", torch.float16, dims=3)
    Hkv, P = kp.shape[0], kp.shape[1]
    need(vp, "vp", torch.float16, shape=(Hkv, P, D))
    need(ks, "ks", torch.float16, dims=4)
    S = ks.shape[2]
    need(ks, "ks", torch.float16, shape=(N, Hkv, S, D))
    need(vs, "vs", torch.float16, shape=(N, Hkv, S, D))
    if slens is not None:
        need(slens, "slens", torch.int32, shape=(N,))
    L = _lib.lib()
    dev = q.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream()
        out = torch.empty_like(q)
        nbytes = L.vmk_prefix_workspace_bytes(N, Hq, Hkv, D, P, S)
        if nbytes == 0:
            raise _lib.VmkError(-2, "prefix: unsupported shape")
        ws = _lib.workspace(nbytes, dev, stream.cuda_stream)
        rc = L.vmk_prefix_decode(_lib.ptr(q), _lib.ptr(kp), _lib.ptr(vp), _lib.ptr(ks) if S > 0 else None,
                                 _lib.ptr(vs) if S > 0 else None, _lib.ptr(slens), _lib.ptr(out), N, Hq, Hkv, D, P, S,
                                 _lib.ptr(ws), ws.numel(), _lib.ptr(_lib.status_word(dev)), stream.cuda_stream)
    _lib.check(rc, "vmk_prefix_decode")
    return out.cpu() if host else out
