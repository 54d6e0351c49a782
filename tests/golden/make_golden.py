"""Generate tests/golden/*.npz by running the reference project's own op definitions.

Run in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/reference

The reference's generator and float64 truth are pure NumPy apart from wrapping arrays in `mlx.core`,
which is not installable here; the stand-in package next to this script supplies those few names.  For
every verification case (5 nominal seeds, the fuzz list, the accuracy list) the script records

  * a SHA-256 of every generated input array (pins the generator bit for bit),
  * the float64 truth at a fixed pseudo-random subsample of output positions plus its NaN/Inf counts
    (pins the arithmetic), and
  * for `dsa`: the float64 indexer score at sampled positions, the score gap at the top-2048 boundary
    and a SHA-256 of the sorted selected indices.

The fixtures travel with the repository; the reference does not."""
import hashlib
import importlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SAMPLE = 2048


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(np.asarray(a)).tobytes()).hexdigest()


def sample_idx(size, key):
    rng = np.random.default_rng(abs(hash_str(key)) % (2 ** 32))
    return np.sort(rng.choice(size, size=min(SAMPLE, size), replace=False))


def hash_str(s):
    return int(hashlib.sha256(s.encode()).hexdigest()[:8], 16)


def main(ref_root):
    sys.path.insert(0, os.path.join(HERE, "_mlx_standin"))
    sys.path.insert(0, ref_root)
    for opname in ("prefix", "spec", "dsa"):
        op = importlib.import_module(f"ops.{opname}")
        cases = [("L1", i, op.L1_SHAPE, "randn", 100 + i) for i in range(5)]
        cases += [("L2", i, s, d, 7 + i) for i, (s, d) in enumerate(op.FUZZ)]
        cases += [("L3", i, s, d, 3) for i, (s, d) in enumerate(op.L3_CASES)]
        rec = {}
        for layer, i, shape, dist, seed in cases:
            key = f"{layer}_{i}"
            kw = dict(with_ref_layouts=False) if opname == "prefix" else {}
            inp = op.make_inputs(shape, seed=seed, dist=dist, **kw)
            for name, a in inp.items():
                if a is not None:
                    rec[f"{key}/sha/{name}"] = np.array(sha(a))
            if opname == "spec":
                rec[f"{key}/bits"] = np.asarray(inp["bits"])
            if opname == "dsa":
                if inp["lens"] is not None:
                    rec[f"{key}/lens"] = np.asarray(inp["lens"])
                s, sel = op.ref_select64(inp["iq"], inp["ik"], inp["w"], inp["lens"])
                B, L = s.shape
                si = sample_idx(s.size, f"dsa/{key}/scores")
                rec[f"{key}/score_idx"] = si
                rec[f"{key}/score_val"] = s.reshape(-1)[si]
                for b in range(B):
                    rec[f"{key}/sel_sha/{b}"] = np.array(sha(np.sort(np.asarray(sel[b])).astype(np.int32)))
                    n = L if inp["lens"] is None else int(np.asarray(inp["lens"])[b])
                    if n > op.TOPK:
                        srt = np.sort(s[b, :n])[::-1]
                        rec[f"{key}/gap/{b}"] = np.array([srt[op.TOPK - 1], srt[op.TOPK]])
                out = op.ref64(**{k: inp[k] for k in ("q", "kv", "iq", "ik", "w", "lens")}, sel=sel)
            else:
                out = op.ref64(**inp)
            out = np.asarray(out, dtype=np.float64)
            oi = sample_idx(out.size, f"{opname}/{key}/out")
            rec[f"{key}/shape"] = np.array(out.shape)
            rec[f"{key}/out_idx"] = oi
            rec[f"{key}/out_val"] = out.reshape(-1)[oi]
            rec[f"{key}/nan_inf"] = np.array([int(np.isnan(out).sum()), int(np.isinf(out).sum())])
            print(opname, key, shape, dist, "ok", flush=True)
        np.savez_compressed(os.path.join(HERE, f"{opname}.npz"), **rec)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python make_golden.py <path of a checkout of the reference project>")
    main(sys.argv[1])
