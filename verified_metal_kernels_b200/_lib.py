"""ctypes binding of libvmk_b200.so (the C ABI declared in include/vmk_b200.h).

The library is built in-tree by build.py.  There is no fallback: if it is missing or a call fails, the
kernel modules raise."""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, os.environ.get("VMK_LIB_NAME", "libvmk_b200.so"))

_c = ctypes
_vp, _i, _sz = _c.c_void_p, _c.c_int, _c.c_size_t

# name -> (restype, argtypes): one entry per symbol declared in include/vmk_b200.h
SIGNATURES = {
    "vmk_version": (_i, []),
    "vmk_error_string": (_c.c_char_p, [_i]),
    "vmk_prefix_workspace_bytes": (_sz, [_i] * 6),
    "vmk_prefix_decode": (_i, [_vp] * 7 + [_i] * 6 + [_vp, _sz, _vp, _vp]),
    "vmk_prefix_decode_bf16": (_i, [_vp] * 7 + [_i] * 6 + [_vp, _sz, _vp, _vp]),
    "vmk_spec_workspace_bytes": (_sz, [_i] * 6),
    "vmk_spec_verify": (_i, [_vp] * 4 + [_i] + [_vp] + [_i] * 6 + [_vp, _sz, _vp, _vp]),
    "vmk_spec_verify_bf16": (_i, [_vp] * 4 + [_i] + [_vp] + [_i] * 6 + [_vp, _sz, _vp, _vp]),
    "vmk_prefix_decode_paged": (_i, [_vp] * 3 + [_i] * 2 + [_vp, _i, _vp, _i, _vp, _vp] + [_i] * 7 + [_vp, _sz, _vp, _vp]),
    "vmk_set_batch_invariant": (_i, [_i]),
    "vmk_decode_workspace_bytes": (_sz, [_i] * 5),
    "vmk_decode": (_i, [_vp] * 5 + [_i] * 6 + [_vp, _sz, _vp, _vp]),
    "vmk_decode_paged": (_i, [_vp] * 4 + [_i] * 3 + [_vp, _vp] + [_i] * 6 + [_vp, _sz, _vp, _vp]),
    "vmk_spec_verify_paged": (_i, [_vp] * 4 + [_i] * 3 + [_vp, _i, _vp] + [_i] * 7 + [_vp, _sz, _vp, _vp]),
    "vmk_spec_verify_noalloc": (_i, [_vp] * 4 + [_i] + [_vp] + [_i] * 6 + [_vp, _vp]),
    "vmk_dsa_workspace_bytes": (_sz, [_i] * 2),
    "vmk_dsa_decode": (_i, [_vp] * 9 + [_i] * 2 + [_vp, _sz, _vp, _vp]),
    "vmk_dsa_indexer_hist_fp8": (_i, [_vp] * 8 + [_i] * 2 + [_vp, _vp]),
    "vmk_dsa_decode_paged": (_i, [_vp] * 6 + [_i] * 3 + [_vp] * 4 + [_i] * 3 + [_vp, _sz, _vp, _vp]),
    "vmk_dsa_decode_bf16": (_i, [_vp] * 9 + [_i] * 2 + [_vp, _sz, _vp, _vp]),
    "vmk_dsa_indexer": (_i, [_vp] * 5 + [_i] * 2 + [_vp, _vp]),
    "vmk_dsa_select": (_i, [_vp] * 4 + [_i] * 2 + [_vp]),
    "vmk_dsa_indexer_hist": (_i, [_vp] * 6 + [_i] * 2 + [_vp, _vp]),
    "vmk_dsa_indexer_hist_bf16": (_i, [_vp] * 6 + [_i] * 2 + [_vp, _vp]),
    "vmk_dsa_select_hist": (_i, [_vp] * 5 + [_i] * 2 + [_vp]),
    "vmk_dsa_attend_workspace_bytes": (_sz, [_i]),
    "vmk_dsa_attend": (_i, [_vp] * 5 + [_i] * 2 + [_vp, _sz, _vp, _vp]),
    "vmk_dsa_attend_bf16": (_i, [_vp] * 5 + [_i] * 2 + [_vp, _sz, _vp, _vp]),
    "vmk_dsa_gather": (_i, [_vp] * 5 + [_i] * 2 + [_vp, _vp]),
    "vmk_dsa_index_project": (_i, [_vp] * 3 + [_c.c_float] + [_vp] * 2 + [_i] * 3 + [_vp, _vp]),
    "vmk_lse_merge": (_i, [_vp] * 3 + [_i] * 3 + [_vp, _vp]),
    "vmk_prefix_partial": (_i, [_vp] * 6 + [_i] * 9 + [_vp] * 3 + [_vp, _sz, _vp, _vp]),
    "vmk_spec_partial": (_i, [_vp] * 4 + [_i] + [_i] * 8 + [_vp] * 3 + [_vp, _sz, _vp, _vp]),
    "vmk_prefix_partial_packed": (_i, [_vp, _i] + [_vp] * 5 + [_i] * 10 + [_vp, _vp, _sz, _vp, _vp]),
    "vmk_spec_partial_packed": (_i, [_vp] * 4 + [_i] * 11 + [_vp, _vp, _sz, _vp, _vp]),
    "vmk_lse_merge_packed": (_i, [_vp] + [_i] * 4 + [_vp, _vp]),
    "vmk_attn_set_tc": (_i, [_i]),
    "vmk_prefix_set_side_by_side": (_i, [_i]),
    "vmk_dsa_set_indexer_variant": (_i, [_i]),
    "vmk_dsa_set_attend_variant": (_i, [_i]),
    "vmk_dsa_set_select_cluster": (_i, [_i]),
}
# exported by debug builds only (-DVMK_MLA_TIMING, -DVMK_TC_TIMING, -DVMK_SEL_TIMING, -DVMK_ATTN_TIMING): device-side event traces
DEBUG_EXPORTS = ("vmk_debug_mla_trace", "vmk_debug_pair_trace", "vmk_debug_tc_trace", "vmk_debug_sel_timing", "vmk_debug_attn_marks")

_lib = None


class VmkError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        super().__init__(f"{what}: libvmk_b200 error {code} ({error_string(code)})")


class VmkDeviceStatusError(VmkError):
    """The device status word was non-zero after a call: bit 0 = a bounded device-side wait ran out (the CTA that
    gave up wrote no result, so the WHOLE call's output is invalid), bit 1 = an index or length outside its tensor
    was clamped."""

    def __init__(self, status, what):
        self.code, self.status = None, status
        bits = [n for b, n in ((1, "a bounded device-side wait ran out: the output is invalid"),
                               (2, "an out-of-range index or length was clamped")) if status & b]
        RuntimeError.__init__(self, f"{what}: device status word {status} ({'; '.join(bits) or 'unknown bits'})")


def lib():
    """The loaded library (loads it on first use; raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m verified_metal_kernels_b200.build` "
                               "(nvcc, sm_100a); there is no fallback path")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def error_string(code):
    return lib().vmk_error_string(int(code)).decode()


def check(code, what):
    if code != 0:
        raise VmkError(code, what)


def ptr(t):
    """Device (or host) address of a torch tensor, or None."""
    return None if t is None else t.data_ptr()


class Workspace:
    """Grow-only device scratch buffer per (device, stream), plus the device status word."""

    def __init__(self):
        self._bufs = {}

    def get(self, nbytes, device, stream_id):
        import torch
        key = (device.index, stream_id)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
            self._bufs[key] = buf
        return buf


_workspace = Workspace()
_status = {}


def workspace(nbytes, device, stream_id):
    return _workspace.get(nbytes, device, stream_id)


def status_word(device):
    import torch
    s = _status.get(device.index)
    if s is None:
        s = torch.zeros(1, dtype=torch.int32, device=device)
        _status[device.index] = s
    return s


def read_status(device):
    """Synchronises and returns the device status word (0 = clean; bit 0 = a bounded wait ran out,
    bit 1 = an index was clamped), then clears it."""
    s = status_word(device)
    v = int(s.item())
    if v:
        s.zero_()
    return v


def raise_on_status(device, what):
    """Synchronises, reads and clears the device status word; raises VmkDeviceStatusError when it is non-zero."""
    v = read_status(device)
    if v:
        raise VmkDeviceStatusError(v, what)


def finish(out, host, check, device, what):
    """Common tail of the kernel modules.  A call made with host tensors returns a host tensor: the copy back
    synchronises, so the status word is read there and a non-zero word raises.  A device-resident call returns
    without synchronising; it checks only when asked (check=True), otherwise the caller reads the word with
    check_status(device) once it has synchronised."""
    if host:
        out = out.cpu()
    if host or check:
        raise_on_status(device, what)
    return out
