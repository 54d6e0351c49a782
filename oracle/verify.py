"""Three-layer verifier for one kernel module (test infrastructure; the B200 counterpart of the
reference's verify.py).

    python -m oracle.verify verified_metal_kernels_b200/kernels/prefix_b200.py
    python -m oracle.verify my_kernel.py --op dsa --json report.json

A kernel module is a Python file with a top-level `def kernel(...)` taking the op's inputs as keyword
arguments (torch CUDA tensors).  As in the reference (verify.py:129-148, 174-241, 268-308) the module is
imported and run on every verification case in a CHILD process, which saves its raw outputs; the verdict
is computed in THIS process, which never imports the kernel, by regenerating the same inputs from their
seeds.  Layers: L1 allclose(1e-2) against the standard op (torch SDPA on the GPU), L2 NaN/Inf pattern and
normalised error <= 1e-2 against the float64 oracle, L3 error <= 2 x max(standard op's error, 2^-11).
Exit code 0 = CORRECT, 1 = REJECTED, 2 = usage error."""
import argparse
import importlib.util
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import judge, ref64                      # noqa: E402
from verified_metal_kernels_b200 import ops          # noqa: E402


def import_kernel(path):
    spec = importlib.util.spec_from_file_location("candidate_kernel", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.kernel


def rel_is_package(path):
    return os.path.relpath(os.path.abspath(path), ROOT).startswith("verified_metal_kernels_b200" + os.sep)


def load_kernel_any(path):
    """Kernel modules inside the package use relative imports: import those by module name."""
    rel = os.path.relpath(os.path.abspath(path), ROOT)
    if rel.startswith("verified_metal_kernels_b200" + os.sep):
        import importlib
        return importlib.import_module(rel[:-3].replace(os.sep, ".")).kernel
    return import_kernel(path)


def child_outputs(opname, kernel_path, out):
    """The only function that imports the kernel.  Saves raw outputs (.npz) and per-case status (.json)."""
    import torch
    fn = load_kernel_any(kernel_path)
    op = ops.load_op(opname)
    arrays, meta = {}, {}
    for layer, i, shape, dist, seed in ops.cases(op):
        key = f"{layer}_{i}"
        inp = ops.to_torch(ops.cand_inputs(opname, op.make_inputs(shape, seed=seed, dist=dist)), "cuda")
        t0 = time.time()
        try:
            o = fn(**inp)
            o = o[0] if isinstance(o, (tuple, list)) else o
            torch.cuda.synchronize()
            if rel_is_package(kernel_path):         # this library's kernels report device-side trouble in a status word
                import verified_metal_kernels_b200
                verified_metal_kernels_b200.check_status(o.device)      # raises: the case fails like any exception
            arrays[key] = o.float().cpu().numpy()
            meta[key] = dict(ok=True, dtype=str(o.dtype), s=time.time() - t0)
        except Exception as e:                      # any exception is a failed case
            meta[key] = dict(ok=False, error=f"{type(e).__name__}: {str(e)[:1500]}")
    np.savez(out + ".npz", **arrays)
    json.dump(meta, open(out + ".json", "w"))


def standard(op, which, inp):
    import torch
    fn = getattr(op, getattr(op, which))
    d = {k: (None if inp.get(k) is None else torch.from_numpy(inp[k]).cuda()) for k in ops.KEYS[op.NAME]}
    return fn(**d).float().cpu().numpy()


def judge_all(opname, outpath):
    op = ops.load_op(opname)
    meta = json.load(open(outpath + ".json"))
    arrs = np.load(outpath + ".npz")
    rep = dict(L1=[], L2=[], L3=[])
    for layer, i, shape, dist, seed in ops.cases(op):
        key = f"{layer}_{i}"
        case = dict(case=key, shape=shape, dist=dist)
        m = meta.get(key, dict(ok=False, error="missing (child crashed or timed out before this case)"))
        if not m["ok"]:
            case.update(ok=False, error=m["error"])
            rep[layer].append(case)
            continue
        inp = op.make_inputs(shape, seed=seed, dist=dist)
        out = arrs[key].astype(np.float64)
        half = "float32" not in m["dtype"]
        if layer == "L1":
            case.update(judge.judge_l1(out, standard(op, "L1_REF", inp)))
        else:
            truth = ref64.REF64[opname](**{k: inp.get(k) for k in ops.KEYS[opname]})
            if layer == "L2":
                r = judge.judge_l2(out, truth, half=half, dist=dist)
                if not r["ok"] and dist == "nan_inf" and not r.get("pattern_ok", True):
                    r = judge.judge_l2(out, truth, half=half, dist=dist, std=standard(op, "L3_REF", inp))
                case.update(r)
            else:
                case.update(judge.judge_l3(out, truth, standard(op, "L3_REF", inp)))
        rep[layer].append(case)
    for layer in ("L1", "L2", "L3"):
        rep[f"{layer}_pass"] = sum(bool(c["ok"]) for c in rep[layer])
        rep[f"{layer}_n"] = len(rep[layer])
    rep["verdict"] = "CORRECT" if all(rep[f"{l}_pass"] == rep[f"{l}_n"] for l in ("L1", "L2", "L3")) else "REJECTED"
    return rep


def summary(rep, max_fail=6):
    lines = [f"L1 (standard op, nominal shape)  {rep['L1_pass']}/{rep['L1_n']}",
             f"L2 (fuzzing vs float64)          {rep['L2_pass']}/{rep['L2_n']}",
             f"L3 (numerical error vs float64)  {rep['L3_pass']}/{rep['L3_n']}", f"=> {rep['verdict']}"]
    fails = [c for l in ("L1", "L2", "L3") for c in rep[l] if not c["ok"]]
    for c in fails[:max_fail]:
        lines.append("  FAIL " + json.dumps({k: v for k, v in c.items() if k != "ok"}, default=str)[:700])
    return "\n".join(lines)


def infer_op(path):
    base = os.path.basename(path)
    for opname in ops.OPS:
        if base.startswith(opname + "_"):
            return opname
    return None


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if argv and argv[0] == "--child":               # internal: --child OP KERNEL OUT
        child_outputs(argv[1], argv[2], argv[3])
        return 0
    ap = argparse.ArgumentParser(description="Three-layer verifier (see the module docstring).")
    ap.add_argument("kernel", help="path to the kernel file (a module with `def kernel(...)`)")
    ap.add_argument("--op", choices=sorted(ops.OPS), help="op name (default: inferred from the file name)")
    ap.add_argument("--json", help="write the full report to this file")
    ap.add_argument("--timeout", type=int, default=1800, help="child process timeout in seconds")
    a = ap.parse_args(argv)
    opname = a.op or infer_op(a.kernel)
    if opname is None:
        print("cannot infer the op from the file name; pass --op", file=sys.stderr)
        return 2
    kpath = os.path.abspath(a.kernel)
    t0 = time.time()
    with tempfile.TemporaryDirectory() as td:
        out = os.path.join(td, "outputs")
        p = subprocess.run([sys.executable, "-m", "oracle.verify", "--child", opname, kpath, out], cwd=ROOT,
                           timeout=a.timeout)
        if p.returncode != 0 or not os.path.exists(out + ".json"):
            print(f"child process failed (exit code {p.returncode}) before saving its outputs\n=> REJECTED")
            return 1
        rep = judge_all(opname, out)
    rep.update(kernel=a.kernel, op=opname, seconds=round(time.time() - t0, 1))
    print(summary(rep))
    if a.json:
        json.dump(rep, open(a.json, "w"), indent=1, default=str)
    return 0 if rep["verdict"] == "CORRECT" else 1


if __name__ == "__main__":
    sys.exit(main())
