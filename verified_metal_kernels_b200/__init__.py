"""B200-native (sm_100a) implementation of the attention-decode ops `prefix`, `spec` and `dsa`.

    ops/      the op contract: shapes, seeded input generators, standard-op opponents
    kernels/  one module per op exposing `kernel(...)` with the reference signature
    csrc/     hand-written CUDA + the C ABI (include/vmk_b200.h), built into libvmk_b200.so
    shard.py  one-process-per-GPU sharding of the three ops

The float64 ground truth and the acceptance criteria live outside the package, under oracle/."""
from . import ops  # noqa: F401

KERNEL_MODULES = {"prefix": "verified_metal_kernels_b200.kernels.prefix_b200",
                  "spec": "verified_metal_kernels_b200.kernels.spec_b200",
                  "dsa": "verified_metal_kernels_b200.kernels.dsa_b200"}


def load_kernel(opname):
    """The op's `kernel` callable (imports torch and loads libvmk_b200.so)."""
    import importlib
    return importlib.import_module(KERNEL_MODULES[opname]).kernel


def check_status(device=None):
    """Synchronises `device` (default: the current CUDA device), reads and clears the status word the kernels OR
    bits into, and raises VmkDeviceStatusError when it is non-zero (bit 0: a bounded device-side wait ran out and
    the whole call's output is invalid; bit 1: an out-of-range index or length was clamped).  Calls made with host
    tensors do this themselves; device-resident calls leave it to the caller, who knows when it synchronises."""
    import torch
    from . import _lib
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _lib.raise_on_status(dev, "check_status")
