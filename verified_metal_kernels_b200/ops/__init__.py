"""Op definitions (the contract): names, dimensions, seeded input generators, shape lists and the
standard-op opponents, mirroring the attribute names of the reference's ops/<op>.py modules."""
import importlib

OPS = ("prefix", "spec", "dsa")

# Keyword arguments each op's kernel(...) receives (reference verify.py:35-37).  Optional keys that a
# generator did not produce are passed as None.
KEYS = {"prefix": ["q", "kp", "vp", "ks", "vs", "slens"],
        "spec": ["q", "k", "v", "bits"],
        "dsa": ["q", "kv", "iq", "ik", "w", "lens"]}


# The 16-bit tensors of each op (everything else keeps its type whatever the 16-bit type is).
HALF_KEYS = {"prefix": ["q", "kp", "vp", "ks", "vs"], "spec": ["q", "k", "v"], "dsa": ["q", "kv", "iq", "ik"]}


def round_bf16(a):
    """float array -> float32 array of the nearest bf16 values (round to nearest even; NaN and Inf kept)."""
    import numpy as np
    x = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((x + np.uint32(0x7FFF) + ((x >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000))
    nan = ((x & np.uint32(0x7F800000)) == np.uint32(0x7F800000)) & ((x & np.uint32(0x007FFFFF)) != 0)
    r = np.where(nan, np.uint32(0x7FC00000) | (x & np.uint32(0x80000000)), r).astype(np.uint32)
    return r.view(np.float32)


def as_bf16(name, inputs):
    """Extension beyond the reference (its kernels are fp16-only): the same seeded inputs with the 16-bit
    tensors rounded to bf16 instead of fp16.  They are returned as float32 arrays holding bf16 values, which is
    what the float64 oracle reads; to_torch(..., bf16=name) turns them into torch.bfloat16."""
    out = dict(inputs)
    for k in HALF_KEYS[name]:
        if out.get(k) is not None:
            out[k] = round_bf16(out[k])
    return out


def load_op(name):
    if name not in OPS:
        raise ValueError(f"unknown op {name!r}; expected one of {OPS}")
    return importlib.import_module(f"{__name__}.{name}")


def cand_inputs(name, inputs):
    """The subset of a generator's output that is handed to kernel(**...) (reference verify.py:44-45)."""
    return {k: inputs.get(k) for k in KEYS[name]}


def cases(op):
    """(layer, index, shape, dist, seed) for every verification case (reference verify.py:48-53):
    L1 = 5 seeds at the nominal shape, L2 = the fuzz list with seed 7+i, L3 = the accuracy list, seed 3."""
    out = [("L1", i, op.L1_SHAPE, "randn", 100 + i) for i in range(5)]
    out += [("L2", i, s, d, 7 + i) for i, (s, d) in enumerate(op.FUZZ)]
    out += [("L3", i, s, d, 3) for i, (s, d) in enumerate(op.L3_CASES)]
    return out


def to_torch(inputs, device, bf16=None):
    """Move a generator's NumPy dict to torch tensors on `device` (None entries stay None).  bf16 = an op name:
    that op's 16-bit tensors (float32 arrays of bf16 values, see as_bf16) become torch.bfloat16."""
    import torch
    out = {}
    for k, v in inputs.items():
        out[k] = None if v is None else torch.from_numpy(v).to(device)
        if bf16 is not None and v is not None and k in HALF_KEYS[bf16]:
            out[k] = out[k].to(torch.bfloat16)
    return out
