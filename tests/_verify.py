"""Runs an op's kernel(...) on verification cases and judges the result with the oracle, following the
reference verifier's three layers (reference verify.py:129-241).  Test infrastructure."""
import numpy as np
import torch

from oracle import judge, ref64
from verified_metal_kernels_b200 import _lib, ops


def device_inputs(opname, inp, device="cuda"):
    return ops.to_torch(ops.cand_inputs(opname, inp), device)


def run_kernel(fn, opname, inp, device="cuda", **extra):
    """kernel(**inputs) on the device; returns the first output as a NumPy float array plus the raw result."""
    dinp = device_inputs(opname, inp, device)
    res = fn(**dinp, **extra)
    out = res[0] if isinstance(res, (tuple, list)) else res
    torch.cuda.synchronize()
    return out.float().cpu().numpy(), res, dinp


def standard_op(op, which, inp, device="cuda"):
    """The platform standard op (torch SDPA composition) on the same inputs."""
    fn = getattr(op, getattr(op, which))
    keys = ops.KEYS[op.NAME]
    dinp = {k: (None if inp.get(k) is None else torch.from_numpy(inp[k]).to(device)) for k in keys}
    return fn(**dinp).float().cpu().numpy()


def truth(opname, inp):
    return ref64.REF64[opname](**{k: inp.get(k) for k in ops.KEYS[opname]})


def judge_case(opname, layer, dist, out, inp, device="cuda"):
    """The verdict dict for one case; `ok` is the pass flag."""
    op = ops.load_op(opname)
    if layer == "L1":
        return judge.judge_l1(out, standard_op(op, "L1_REF", inp, device))
    t = truth(opname, inp)
    if layer == "L2":
        rep = judge.judge_l2(out, t, half=True, dist=dist)
        if not rep["ok"] and not rep["pattern_ok"] and dist == "nan_inf":
            rep = judge.judge_l2(out, t, half=True, dist=dist, std=standard_op(op, "L3_REF", inp, device))
        return rep
    return judge.judge_l3(out, t, standard_op(op, "L3_REF", inp, device))


def assert_clean_status(device="cuda"):
    st = _lib.read_status(torch.device(device, torch.cuda.current_device()))
    assert st == 0, f"device status word {st}: a bounded wait ran out (bit 0) or an index was clamped (bit 1)"
