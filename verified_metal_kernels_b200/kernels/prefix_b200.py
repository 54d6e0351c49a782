"""Kernel module for op `prefix` (shared-prefix decode) on B200.

Drop-in for the reference's kernel module contract: a top-level `kernel(...)` taking the op's inputs as
keyword arguments (reference kernels/prefix_opus55_v8.py:282, called as fn(**inputs) by verify.py:139).
The work is done by hand-written sm_100a CUDA reached through libvmk_b200's C ABI."""
import torch

from .. import _lib
from ._common import need, stage_in


def kernel(q, kp, vp, ks, vs, slens=None, check=False):
    """q (N,Hq,D), kp/vp (Hkv,P,D), ks/vs (N,Hkv,S,D) fp16 (or all bf16) -> (N,Hq,D) of the same type on the
    inputs' device.

    `slens` (N,) int32, optional: true suffix length per request.  Inputs are not modified.  Host (CPU)
    tensors are accepted: they are copied to the current CUDA device first and the result is returned
    on the host, which is the end-to-end path measured by bench.py.

    Device status: a call with host tensors synchronises anyway and raises VmkDeviceStatusError if a kernel
    reported a bounded wait that ran out (the output is then invalid) or a clamped index.  A device-resident call
    returns without synchronising; pass check=True to synchronise and check here, or call
    verified_metal_kernels_b200.check_status(device) after synchronising."""
    (q, kp, vp, ks, vs, slens), host = stage_in([q, kp, vp, ks, vs, slens])
    if not isinstance(q, torch.Tensor) or q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("q: expected a float16 or bfloat16 tensor")
    dt = q.dtype                                   # fp16 (the reference's) or bf16, the same for all five tensors
    need(q, "q", dt, dims=3)
    N, Hq, D = q.shape
    need(kp, "kp", dt, dims=3)
    Hkv, P = kp.shape[0], kp.shape[1]
    need(vp, "vp", dt, shape=(Hkv, P, D))
    need(ks, "ks", dt, dims=4)
    S = ks.shape[2]
    need(ks, "ks", dt, shape=(N, Hkv, S, D))
    need(vs, "vs", dt, shape=(N, Hkv, S, D))
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
        rc = (L.vmk_prefix_decode_bf16 if dt == torch.bfloat16 else L.vmk_prefix_decode)(_lib.ptr(q), _lib.ptr(kp), _lib.ptr(vp), _lib.ptr(ks) if S > 0 else None,
                                 _lib.ptr(vs) if S > 0 else None, _lib.ptr(slens), _lib.ptr(out), N, Hq, Hkv, D, P, S,
                                 _lib.ptr(ws), ws.numel(), _lib.ptr(_lib.status_word(dev)), stream.cuda_stream)
    _lib.check(rc, "vmk_prefix_decode")
    return _lib.finish(out, host, check, dev, "vmk_prefix_decode")


def kernel_paged(q, k_pages, v_pages, prefix_table, P, suffix_table=None, slens=None, check=False):
    """`prefix` over a paged cache: k_pages / v_pages (pages, Hkv, page_size, D) fp16 are one pool; the shared
    prefix is P keys in pages prefix_table (T_p,) int32; request n's private suffix is slens[n] keys in pages
    suffix_table[n] ((N, T_s) int32).  page_size a multiple of 64.  Returns (N,Hq,D) fp16, equal to kernel() on
    the de-paged tensors bit for bit."""
    if not isinstance(q, torch.Tensor) or q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("q: expected a float16 or bfloat16 tensor")
    dt = q.dtype
    need(q, "q", dt, dims=3)
    N, Hq, D = q.shape
    need(k_pages, "k_pages", dt, dims=4)
    pages, Hkv, page_size = k_pages.shape[0], k_pages.shape[1], k_pages.shape[2]
    need(k_pages, "k_pages", dt, shape=(pages, Hkv, page_size, D))
    need(v_pages, "v_pages", dt, shape=(pages, Hkv, page_size, D))
    need(prefix_table, "prefix_table", torch.int32, dims=1)
    Tp = prefix_table.shape[0]
    if page_size % 64 != 0 or P <= 0 or Tp * page_size < P:
        raise ValueError("page_size must be a multiple of 64 and prefix_table must cover P keys")
    S, Ts = 0, 0
    if suffix_table is not None:
        need(suffix_table, "suffix_table", torch.int32, dims=2)
        Ts = suffix_table.shape[1]
        need(suffix_table, "suffix_table", torch.int32, shape=(N, Ts))
        need(slens, "slens", torch.int32, shape=(N,))
        S = Ts * page_size
    lib = _lib.lib()
    dev = q.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream()
        out = torch.empty_like(q)
        nbytes = lib.vmk_prefix_workspace_bytes(N, Hq, Hkv, D, P, S)
        if nbytes == 0:
            raise _lib.VmkError(-2, "prefix: unsupported shape")
        ws = _lib.workspace(nbytes, dev, stream.cuda_stream)
        rc = lib.vmk_prefix_decode_paged(_lib.ptr(q), _lib.ptr(k_pages), _lib.ptr(v_pages), pages, page_size,
                                         _lib.ptr(prefix_table), Tp, _lib.ptr(suffix_table), Ts, _lib.ptr(slens),
                                         _lib.ptr(out), N, Hq, Hkv, D, P, S, 1 if dt == torch.bfloat16 else 0,
                                         _lib.ptr(ws), ws.numel(),
                                         _lib.ptr(_lib.status_word(dev)), stream.cuda_stream)
    _lib.check(rc, "vmk_prefix_decode_paged")
    return _lib.finish(out, False, check, dev, "vmk_prefix_decode_paged")
