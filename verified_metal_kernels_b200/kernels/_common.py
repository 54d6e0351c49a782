"""Argument checks shared by the kernel modules."""
import torch


def need(t, name, dtype, shape=None, dims=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name}: expected a torch tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise ValueError(f"{name}: expected a CUDA tensor (the kernels have no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{name}: expected dtype {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise ValueError(f"{name}: expected {dims} dimensions, got shape {tuple(t.shape)}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: expected a C-contiguous tensor")
    return t


def stage_in(tensors):
    """Host tensors (pinned or not) -> device copies on the current stream; device tensors pass through.
    Returns (device tensors, any_host)."""
    out, any_host = [], False
    for t in tensors:
        if t is not None and not t.is_cuda:
            any_host = True
            t = t.to("cuda", non_blocking=True)
        out.append(t)
    return out, any_host
