"""Op definitions (the contract): names, dimensions, seeded input generators, shape lists and the
standard-op opponents, mirroring the attribute names of the reference's ops/<op>.py modules."""
import importlib

OPS = ("prefix", "spec", "dsa")

# Keyword arguments each op's kernel(...) receives (reference verify.py:35-37).  Optional keys that a
# generator did not produce are passed as None.
KEYS = {"prefix": ["q", "kp", "vp", "ks", "vs", "slens"],
        "spec": ["q", "k", "v", "bits"],
        "dsa": ["q", "kv", "iq", "ik", "w", "lens"]}


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


def to_torch(inputs, device):
    """Move a generator's NumPy dict to torch tensors on `device` (None entries stay None)."""
    import torch
    out = {}
    for k, v in inputs.items():
        out[k] = None if v is None else torch.from_numpy(v).to(device)
    return out
