"""Access to the committed golden vectors (tests/golden/*.npz, written by tests/golden/make_golden.py
from the reference project's own modules)."""
import hashlib
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_cache = {}


def golden(opname):
    if opname not in _cache:
        _cache[opname] = np.load(os.path.join(HERE, "golden", f"{opname}.npz"))
    return _cache[opname]


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(np.asarray(a)).tobytes()).hexdigest()


def check_inputs(opname, key, inp):
    g = golden(opname)
    for name, a in inp.items():
        k = f"{key}/sha/{name}"
        if a is None or k not in g.files:
            continue
        assert sha(a) == str(g[k]), f"{opname} {key}: generated `{name}` differs from the reference generator"


def check_truth(opname, key, out, rtol=1e-9, atol=1e-12):
    """Compare a float64 result with the reference's truth at the recorded sample positions."""
    g = golden(opname)
    out = np.asarray(out, dtype=np.float64)
    assert tuple(g[f"{key}/shape"]) == out.shape
    got = out.reshape(-1)[g[f"{key}/out_idx"]]
    exp = g[f"{key}/out_val"]
    assert (np.isnan(got) == np.isnan(exp)).all() and (np.isinf(got) == np.isinf(exp)).all()
    fin = np.isfinite(exp)
    np.testing.assert_allclose(got[fin], exp[fin], rtol=rtol, atol=atol)
    assert [int(np.isnan(out).sum()), int(np.isinf(out).sum())] == list(g[f"{key}/nan_inf"])
