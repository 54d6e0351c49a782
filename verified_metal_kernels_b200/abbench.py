"""Interleaved A/B benchmark of one op configuration: this library's kernel(...) against the library
compositions of the same op (ops/<op>.py: TORCH_REFS), timed in the same rounds on the same GPU.

The method is the reference's (bench.py:61-76 chain, 99-111 interleaving, 114-126 statistics, 181-192 checks):
  * a candidate is timed as a CHAIN of `layers` calls over up to 8 distinct input sets (within 1.5 GiB), each
    call's query being the previous call's output, so that no call can start before the one before it ended;
  * here the chain of every candidate is captured once in a CUDA graph, so host launch overhead is off the clock
    for the kernel and for its opponents alike (a candidate that cannot be captured is timed eagerly and marked);
  * the L2 is flushed (a buffer of twice its size is rewritten) before every timed chain;
  * candidates run in `rounds` rounds, each round in a freshly shuffled order; reported per candidate: median,
    p10, p90 of the per-layer time, and per opponent the median over rounds of time(opponent) / time(kernel);
  * before any timing the kernel's output on the benchmark inputs is compared with the standard op
    (atol = rtol = 1e-2) and the inputs are checked for modification;
  * every sample is kept (save_samples writes results/bench_<op>.json)."""
import json
import os
import random
import statistics

import numpy as np

L2_FLUSH_BYTES = 256 << 20        # twice the 126 MB L2
SET_BUDGET = 3 << 29              # 1.5 GiB of distinct input sets per configuration


def device_inputs(opname, shape, seed, device="cuda", mask="tree"):
    """Synthetic inputs of one configuration created on the device, with the distributions of the op's generator
    (fp16 roundings of N(0,1); dsa head weights N(0,1) * (64*128)^-1/2; spec masks from the generator's own chain /
    tree functions; ragged prefix suffix lengths U[0,S]).  Same shapes and value distributions as
    ops.<op>.make_inputs, not the same bits: that generator draws on the host, which takes seconds per set."""
    import torch
    from . import ops
    op = ops.load_op(opname)
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))

    def r16(*dims):
        out = torch.empty(*dims, dtype=torch.float16, device=device)
        flat, step = out.view(-1), 1 << 28
        for i in range(0, flat.numel(), step):
            n = min(step, flat.numel() - i)
            flat[i:i + n] = torch.randn(n, generator=g, device=device, dtype=torch.float32).half()
        return out

    if opname == "prefix":
        N, P, S = shape["N"], shape["P"], shape["S"]
        Hq, Hkv, d = shape.get("Hq", op.HQ), shape.get("Hkv", op.HKV), shape.get("D", op.D)
        inp = dict(q=r16(N, Hq, d), kp=r16(Hkv, P, d), vp=r16(Hkv, P, d), ks=r16(N, Hkv, S, d), vs=r16(N, Hkv, S, d))
        if shape.get("ragged"):
            inp["slens"] = torch.randint(0, S + 1, (N,), generator=g, device=device, dtype=torch.int32)
        return inp
    if opname == "spec":
        B, L, kd = shape["B"], shape["L"], shape["k"]
        Hq, Hkv, d = shape.get("Hq", op.HQ), shape.get("Hkv", op.HKV), shape.get("D", op.D)
        rng = np.random.default_rng(seed)
        masks = [op.chain_bits(kd) if mask == "chain" else op.tree_bits(kd, rng, shape.get("max_depth")) for _ in range(B)]
        return dict(q=r16(B, kd, Hq, d), k=r16(B, Hkv, L, d), v=r16(B, Hkv, L, d),
                    bits=torch.from_numpy(op.pack_bits(masks, kd)).to(device))
    if opname == "dsa":
        B, L = shape["B"], shape["L"]
        return dict(q=r16(B, op.H, op.DK), kv=r16(B, L, op.DK), iq=r16(B, op.HI, op.DI), ik=r16(B, L, op.DI),
                    w=torch.randn(B, op.HI, generator=g, device=device, dtype=torch.float32) * (op.HI ** -0.5 * op.DI ** -0.5),
                    lens=None)
    raise ValueError(opname)


def set_bytes(inp):
    import torch
    return sum(v.numel() * v.element_size() for v in inp.values() if isinstance(v, torch.Tensor))


def checksum(inp):
    """A cheap fingerprint of every tensor of an input set (sum of its bytes read as integers), on the device."""
    import torch
    out = {}
    for k, v in inp.items():
        if isinstance(v, torch.Tensor):
            flat = v.contiguous().view(torch.uint8).view(-1)
            n8 = flat.numel() // 8 * 8
            s = int(flat[:n8].view(torch.int64).sum().item()) if n8 else 0
            out[k] = s + int(flat[n8:].to(torch.int64).sum().item())
    return out


def interleaved(runners, rounds, warmup=3, seed=0):
    """{name: [seconds per layer]}: `warmup` untimed runs of each candidate, then `rounds` rounds in shuffled order."""
    rng = random.Random(seed)
    names = list(runners)
    for n in names:
        for _ in range(warmup):
            runners[n]()
    times = {n: [] for n in names}
    for _ in range(rounds):
        order = names[:]
        rng.shuffle(order)
        for n in order:
            times[n].append(runners[n]())
    return times


def summary(samples_us):
    t = sorted(samples_us)
    return dict(median_us=statistics.median(t), p10_us=t[int(0.1 * len(t))], p90_us=t[max(int(0.9 * len(t)) - 1, 0)], n=len(t))


def ratio_median(times, a, b):
    """Median over rounds of time(b) / time(a): above 1 means a is faster than b."""
    return statistics.median([y / x for x, y in zip(times[a], times[b])])


class ChainRunner:
    """One candidate's chain of `layers` calls (output -> next query), replayed from a CUDA graph after an L2
    flush and timed with CUDA events; returns seconds per layer."""

    def __init__(self, fn, sets, layers, chain, flush):
        import torch
        self.torch, self.layers, self.flush, self.graph, self.eager = torch, layers, flush, None, None
        n = len(sets)

        def run_chain():
            q = sets[0]["q"]
            for i in range(layers):
                kw = dict(sets[i % n])
                kw["q"] = q
                q = chain(fn(**kw), kw)
            return q

        run_chain()
        torch.cuda.synchronize()
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.keep = run_chain()
            self.graph = g
        except Exception as e:                       # timed eagerly instead: host launch overhead is then on the clock
            torch.cuda.synchronize()
            self.eager, self.why = run_chain, f"{type(e).__name__}: {str(e)[:120]}"
        self.n = 0

    def __call__(self):
        torch = self.torch
        self.n += 1
        self.flush.fill_(self.n & 0xff)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        if self.graph is not None:
            self.graph.replay()
        else:
            self.eager()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e-3 / self.layers


def bench_config(opname, shape, kernel_fn, rounds=30, layers=16, mask="tree", opponents=True, flush=None,
                 kernel_kwargs=None, opponent_budget=24 << 30, std_name=None):
    """One configuration.  Returns a dict with the kernel's per-layer statistics (`median_us`, `p10_us`, `p90_us`),
    `output_ok` / `inputs_unmodified` from the pre-timing check, `vs_torch` = {opponent: ratio_median} and
    `opponents_us`, the number of distinct input sets, and `samples_us` for every candidate."""
    import torch
    from . import ops
    op = ops.load_op(opname)
    chain = getattr(op, "chain_torch", None) or (lambda out, kw: out)
    if flush is None:
        flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")
    first = device_inputs(opname, shape, 0, mask=mask)
    n_distinct = int(max(1, min(8, SET_BUDGET // max(set_bytes(first), 1))))
    sets = [first] + [device_inputs(opname, shape, s, mask=mask) for s in range(1, n_distinct)]
    keys = ops.KEYS[opname]
    wrapped = lambda **kw: kernel_fn(**{k: kw.get(k) for k in keys}, **(kernel_kwargs or {}))
    row = dict(shape=dict(shape), n_distinct=n_distinct, n_chain=layers, rounds=rounds)

    # output check on the benchmark inputs themselves, and input-modification check
    std = getattr(op, std_name or op.L1_REF)
    before = checksum(first)
    out = wrapped(**first)
    ref = std(**first)
    torch.cuda.synchronize()
    row["inputs_unmodified"] = checksum(first) == before
    row["output_ok"] = bool(torch.allclose(out.float(), ref.float(), atol=1e-2, rtol=1e-2, equal_nan=True))
    row["max_abs_diff_vs_standard_op"] = float((out.float() - ref.float()).abs().nan_to_num(0).max().item())
    del out, ref

    cands = {"kernel": ChainRunner(wrapped, sets, layers, chain, flush)}
    skipped = {}
    if opponents:
        lay = None
        if opname == "prefix":
            extra = sum(2 * s["ks"].shape[0] * s["kp"].numel() * 2 + 2 * s["ks"].numel() * 2 for s in sets)
            if extra <= opponent_budget:
                lay = [dict(s, **op.build_layouts(s["kp"], s["vp"], s["ks"], s["vs"])) for s in sets]
        for name, f in op.TORCH_REFS.items():
            use = sets
            if opname == "prefix" and name in ("torch_naive", "torch_unified"):
                if lay is None:
                    skipped[name] = "its cache layouts would not fit the memory budget of the benchmark"
                    continue
                use = lay
            try:
                cands[name] = ChainRunner(f, use, layers, chain, flush)
            except Exception as e:
                torch.cuda.synchronize()
                skipped[name] = f"{type(e).__name__}: {str(e)[:120]}"
    times = interleaved(cands, rounds)
    us = {n: [x * 1e6 for x in t] for n, t in times.items()}
    row.update(summary(us["kernel"]))
    row["timing"] = "per layer of a %d-layer chain (output -> next query), CUDA graph, L2 flushed, %d shuffled rounds" % (layers, rounds)
    refs = [n for n in us if n != "kernel"]
    if refs:
        row["vs_torch"] = {n: ratio_median(times, "kernel", n) for n in refs}
        row["opponents_us"] = {n: summary(us[n]) for n in refs}
        best = min(refs, key=lambda n: row["opponents_us"][n]["median_us"])
        row["strongest_ref"], row["speedup"] = best, row["vs_torch"][best]
    eager = {n: c.why for n, c in cands.items() if c.graph is None}
    if eager:
        row["timed_eagerly"] = eager
    if skipped:
        row["skipped"] = skipped
    row["samples_us"] = us
    del cands, sets
    torch.cuda.empty_cache()
    return row


def geomean(xs):
    xs = [x for x in xs if x and x > 0]
    return float(np.exp(np.mean(np.log(xs)))) if xs else None


def save_samples(opname, rows, root):
    """results/bench_<op>.json under `root`: every configuration's row with all its samples (reference bench.py:226,283)."""
    d = os.path.join(root, "results")
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, f"bench_{opname}.json")
    with open(path, "w") as f:
        json.dump(dict(op=opname, configs=rows), f)
    return path
