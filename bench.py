"""Benchmark of the B200 decode kernels on the multi-GPU sweep workload.

    python bench.py                                   # 1 GPU, dsa B=128 L=131072 (+ per-op lines with opponents)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus 8 --steps 20 --warmup 3       # ONE batch of 128 requests cut over the ranks (strong scaling)
    ... bench.py --gpus 8 --scaling weak              # headline = every rank its own batch of 128 instead
    python bench.py --impl reference                  # the float64 NumPy truth timed on the host cores

A step is one pass of the op over the whole batch.  The headline op is `dsa` on the sweep configuration
(batch 128, cache 131072): rows/s where a row is one request's complete output.  Requests are independent
units: they are spread over the ranks with no collective on the data path.  On more than one GPU the headline is
the STRONG scaling of that one batch (16 requests per GPU at N=8, where the fixed latencies of the three stages
weigh more); the line's `weak` object carries the same measurement with 128 requests per rank.  The `ops` object
holds the other configurations: on one GPU every configuration of the op list with its library opponents timed
in the same shuffled rounds; on N GPUs the `prefix` sweep under hybrid sharding (suffixes by request, the shared
prefix by kv head, one all-to-all of packed partials) and the speculative tree (by batch element, beyond four
ranks with every cache split in two).
Inputs are synthetic (seeded N(0,1) rounded to fp16, head weights N(0,1)/sqrt(64*128), as the op's generator
draws them).  The dsa inputs are far larger than the 126 MB L2; every other timing flushes L2 first.

Before any timing every rank checks one of its own requests against the float64 oracle and its inputs for
modification afterwards (`output_ok`).  Rank 0 prints one JSON line.  `value` is timed with inputs resident in
HBM; `e2e` through the kernel module's public call with pinned HOST tensors (copies inside the timed region);
`roofline` is for the dominant kernel (the indexer) from CUDA events inside this run; `cpu_baseline` is the
float64 oracle on a bounded sample on the host cores.  A non-zero device status word makes the run exit 1."""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "dsa decode rows/s (batch 128, cache 131072)"
UNIT = "rows/s"
DSA = dict(B=128, L=131072)
PREFIX = dict(N=256, P=32768, S=2048, ragged=True)
SPEC = dict(B=4, L=32768, k=64, max_depth=8)
FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0           # the figure the metric is quoted against
E2E_MAX = 32
DELAY_BYTES = 1 << 30              # a 1 GiB fill ahead of each multi-GPU side step: flushes L2 and lets the host run ahead


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def ncu_traffic():
    """DRAM bytes per indexer launch from the committed ncu capture (profiles/traffic.json), or None."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(path):
        try:
            return json.load(open(path))
        except Exception:
            return None
    return None


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) every few milliseconds
    while the timed region runs; falls back to polling nvidia-smi when NVML cannot be loaded."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index, period=0.002):
        self.index, self.period, self.rows, self.stop_flag, self.thread = index, period, [], False, None
        self.max_mhz, self.err = None, None

    def _loop_nvml(self):
        import pynvml as nv
        nv.nvmlInit()
        h = nv.nvmlDeviceGetHandleByIndex(self.index)
        self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                try:
                    rs = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                self.rows.append((time.perf_counter(), float(mhz), int(rs)))
            except Exception as e:          # keep sampling; report the last error
                self.err = repr(e)
            time.sleep(self.period)

    def _loop_smi(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.active"
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                f = [x.strip() for x in out.strip().split(",")]
                self.max_mhz = float(f[1])
                self.rows.append((time.perf_counter(), float(f[0]), int(f[2], 16)))
            except Exception as e:
                self.err = repr(e)
                time.sleep(0.05)

    def _loop(self):
        try:
            self._loop_nvml()
        except Exception as e:
            self.err = repr(e)
            self._loop_smi()

    def start(self, ready_timeout=10.0):
        """Starts the sampling thread and waits for its first sample (NVML start-up can take longer than a
        short timed region)."""
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()
        t_end = time.perf_counter() + ready_timeout
        while not self.rows and self.thread.is_alive() and time.perf_counter() < t_end:
            time.sleep(0.001)

    def mark(self):
        return time.perf_counter()

    def stop(self, t0=None, t1=None):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=10)
        rows = [r for r in self.rows if (t0 is None or r[0] >= t0) and (t1 is None or r[0] <= t1)]
        window = "timed region"
        if len(rows) < 3:                       # region shorter than a few samples: widen to the loaded period
            rows, window = self.rows, "warm-up + timed region"
        bits = 0
        for r in rows:
            bits |= r[2]
        sm = [r[1] for r in rows]
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_mhz_min=min(sm) if sm else None, sm_max_mhz=self.max_mhz,
                    reasons=[n for b, n in self.REASONS.items() if bits & b], samples=len(sm), window=window,
                    sampler_error=self.err)


# ------------------------------------------------------------------------------------------------ inputs
def dsa_inputs(B, L, device, seed):
    """Synthetic dsa inputs on the device with the generator's distributions (chunked to bound memory)."""
    from verified_metal_kernels_b200 import abbench
    return abbench.device_inputs("dsa", dict(B=B, L=L), seed, device)


RANK_MS = []          # per call of timed_steps under torch.distributed: ms per step of every rank


def timed_steps(fn, steps, warmup, dist, torch, sampler=None):
    """W warm-up calls, then K timed calls between barrier + synchronize; returns (max-over-ranks seconds
    for the K steps, per-step milliseconds on this rank)."""
    if sampler:
        sampler.start()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t_begin = time.perf_counter()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record()
    for i in range(steps):
        fn()
        ev[i + 1].record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop(t_begin, time.perf_counter()) if sampler else None
    total_ms = ev[0].elapsed_time(ev[-1])
    per = [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]
    if dist is not None:
        # every rank's own time for the K steps: the step is their maximum, the spread says where a loss comes from
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        every = torch.empty(dist.get_world_size(), device="cuda", dtype=torch.float64)
        dist.all_gather_into_tensor(every, t)
        RANK_MS.append([round(float(x) / steps, 5) for x in every.tolist()])
        total_ms = float(every.max().item())
    return total_ms / 1e3, per, clocks


def stage_times(inp, steps, torch):
    """Average device time of each dsa stage (CUDA events on the launching stream), same inputs."""
    from verified_metal_kernels_b200.kernels import dsa_b200
    out = {}
    scores = dsa_b200.indexer(inp["iq"], inp["ik"], inp["w"])
    idx, cnt = dsa_b200.select(scores)
    torch.cuda.synchronize()

    def avg(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    from verified_metal_kernels_b200 import _lib
    L = _lib.lib()
    B, Lk = inp["ik"].shape[0], inp["ik"].shape[1]
    st = torch.cuda.current_stream().cuda_stream
    status = _lib.status_word(inp["ik"].device)
    hist = torch.empty(B, 2048, dtype=torch.int32, device=scores.device)
    out["indexer_ms"] = avg(lambda: L.vmk_dsa_indexer_hist(inp["iq"].data_ptr(), inp["ik"].data_ptr(),
                                                           inp["w"].data_ptr(), None, scores.data_ptr(), hist.data_ptr(),
                                                           B, Lk, status.data_ptr(), st))
    out["select_ms"] = avg(lambda: L.vmk_dsa_select_hist(scores.data_ptr(), hist.data_ptr(), None, idx.data_ptr(),
                                                         cnt.data_ptr(), B, Lk, st))
    out["attend_ms"] = avg(lambda: dsa_b200.attend(inp["q"], inp["kv"], idx, cnt))
    # stage 1 on fp8 index queries and keys (a different input format, reported beside the fp16 stage)
    iq8, iqs, ik8, iks = fp8_index(inp, torch)
    out["indexer_fp8_ms"] = avg(lambda: L.vmk_dsa_indexer_hist_fp8(iq8.data_ptr(), iqs.data_ptr(), ik8.data_ptr(),
                                                                   iks.data_ptr(), inp["w"].data_ptr(), None,
                                                                   scores.data_ptr(), hist.data_ptr(), B, Lk,
                                                                   status.data_ptr(), st))
    return out


def fp8_index(inp, torch):
    """The index queries and keys of `inp` quantised to e4m3 bytes with positive fp32 scales (per head / per position)."""
    from verified_metal_kernels_b200.kernels import dsa_b200
    B, Lk = inp["ik"].shape[0], inp["ik"].shape[1]
    iq8, iqs = dsa_b200.quantize_e4m3(inp["iq"])
    ik8 = torch.empty(B, Lk, 128, dtype=torch.uint8, device=inp["ik"].device)
    iks = torch.empty(B, Lk, dtype=torch.float32, device=inp["ik"].device)
    for b0 in range(0, B, 8):                              # in pieces: the float copy of ik is 4 x its size
        ik8[b0:b0 + 8], iks[b0:b0 + 8] = dsa_b200.quantize_e4m3(inp["ik"][b0:b0 + 8])
    return iq8, iqs, ik8, iks


# ------------------------------------------------------------------------------------------------ output checks
def _host(t):
    return None if t is None else t.detach().cpu().numpy()


def check_dsa_request(inp, out, idx, cnt, b):
    """Request b of a dsa call against the float64 oracle: the selected set (exact wherever the float64 scores
    are separated by more than fp32 accumulation error) and the output (normalised max error <= 1e-2)."""
    from oracle import judge, ref64
    one = {k: _host(v[b:b + 1]) for k, v in inp.items() if v is not None}
    L = one["ik"].shape[1]
    s64 = ref64.dsa_scores64(one["iq"], one["ik"], one["w"])
    sel_rep = judge.select_check(_host(idx[b]), int(cnt[b]), s64[0], L)
    sel = [_host(idx[b, :int(cnt[b])]).astype(np.int64)]
    truth = ref64.dsa_ref64(one["q"], one["kv"], one["iq"], one["ik"], one["w"], None, sel=sel)
    rep = judge.judge_l2(_host(out[b:b + 1].float()), truth, half=True)
    return bool(sel_rep["ok"] and rep["ok"]), dict(selection_exact=sel_rep.get("exact"), err_max=rep.get("err_max"))


def all_ranks_ok(ok, dist, torch):
    if dist is None:
        return bool(ok)
    t = torch.tensor([1 if ok else 0], device="cuda", dtype=torch.int32)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(int(t.item()))


# ------------------------------------------------------------------------------------------------ one-GPU op lines
def ab_line(opname, name, shape, torch, rounds, mask="tree", opponents=True, std_name=None):
    """One configuration on one GPU through the interleaved A/B method (verified_metal_kernels_b200/abbench.py):
    per-layer time of a 16-layer CUDA-graph chain with L2 flushed, the library opponents in the same shuffled
    rounds, plus the time of one plain kernel(...) call (host launch overhead included)."""
    from verified_metal_kernels_b200 import abbench, load_kernel, ops
    op = ops.load_op(opname)
    fn = load_kernel(opname)
    flush = torch.empty(abbench.L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")
    row = abbench.bench_config(opname, shape, fn, rounds=rounds, mask=mask, opponents=opponents, flush=flush,
                               std_name=std_name)
    inp = abbench.device_inputs(opname, shape, 0, mask=mask)
    sl = _host(inp.get("slens")) if opname == "prefix" and inp.get("slens") is not None else None
    nbytes = op.algorithmic_bytes(shape, sl) if opname == "prefix" else op.algorithmic_bytes(shape)
    keys = ops.KEYS[opname]
    times = []
    for i in range(8):
        flush.fill_(i & 0xff)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn(**{k: inp.get(k) for k in keys})
        b.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(a.elapsed_time(b))
    ms_call = statistics.median(times)
    if opname == "prefix":
        flops = 4.0 * shape["N"] * 32 * 128 * (shape["P"] + (float(sl.mean()) if sl is not None else shape["S"]))
    elif opname == "spec":
        flops = 4.0 * shape["B"] * shape["k"] * 32 * 128 * shape["L"]
    else:
        flops = 2.0 * 64 * 128 * shape["L"] * shape["B"] + 2.0 * 128 * (576 + 512) * min(2048, shape["L"]) * shape["B"]
    peak, kind = peaks()
    ms = row["median_us"] * 1e-3
    gbs = nbytes / (ms * 1e-3) / 1e9
    line = dict(workload=name, algorithmic_mb=nbytes / 1e6, peak=f"of {kind}", l2="flushed before every timed chain",
                timing=row["timing"], ms=ms, p10_ms=row["p10_us"] * 1e-3, p90_ms=row["p90_us"] * 1e-3,
                rows_per_s=op.rows(shape) / (ms * 1e-3), hbm_gbs=gbs, hbm_frac=gbs / peak,
                hbm_frac_of_8tbs=gbs / NOMINAL_HBM_GBS, tflops=flops / (ms * 1e-3) / 1e12,
                ms_single_call=ms_call, single_call_hbm_frac=nbytes / (ms_call * 1e-3) / 1e9 / peak,
                output_ok=bool(row["output_ok"] and row["inputs_unmodified"]), n_distinct=row["n_distinct"])
    for k in ("vs_torch", "opponents_us", "strongest_ref", "speedup", "skipped", "timed_eagerly"):
        if k in row:
            line[k] = row[k]
    return line, row


def side_line(config, torch, steps):
    """rows/s and HBM fraction of the two extension configurations on one GPU (`decode`, `spec_tree_paged`), and of
    any named configuration for profiling (`--side-only`): L2 flushed between iterations, one call and a chain."""
    from verified_metal_kernels_b200 import abbench, ops
    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    r16 = lambda *s: torch.randn(*s, generator=g, device="cuda", dtype=torch.float32).half()
    named = dict(prefix_small=("prefix", dict(N=8, P=4096, S=256), "tree"), prefix_sweep=("prefix", PREFIX, "tree"),
                 spec_chain=("spec", dict(B=1, L=8192, k=8), "chain"), spec_tree=("spec", SPEC, "tree"),
                 dsa_small=("dsa", dict(B=8, L=32768), "tree"))
    if config in named:
        opname, shape, mask = named[config]
        return ab_line(opname, config, shape, torch, max(steps, 3), mask=mask, opponents=False)[0]
    if config == "spec_tree_paged":
        from verified_metal_kernels_b200.kernels import spec_b200
        op = ops.load_op("spec")
        shape = SPEC
        B, L, kd = shape["B"], shape["L"], shape["k"]
        base = abbench.device_inputs("spec", shape, 0)
        # the same cache as a shuffled pool of 64-key pages (the smallest page the kernels take)
        page = 64
        T = L // page
        perm = torch.randperm(B * T + 7, generator=g, device="cuda")[:B * T].to(torch.int32).reshape(B, T)
        inp = dict(q=base["q"], k_pages=r16(B * T + 7, 8, page, 128), v_pages=r16(B * T + 7, 8, page, 128),
                   page_table=perm.contiguous(), L=L, bits=base["bits"])
        nbytes, rows, fn, opname = op.algorithmic_bytes(shape), B * kd, spec_b200.kernel_paged, "spec"
        name = f"spec tree depth<=8 B={B} k={kd} L={L}, paged cache (page {page})"
        flops = 4.0 * B * kd * 32 * 128 * L
    elif config in ("decode", "decode_small"):
        # plain single-token decode (extension op): 64 requests with caches of 16k..32k keys
        from verified_metal_kernels_b200.kernels import decode_b200
        from verified_metal_kernels_b200.ops import decode as op
        opname = "decode"
        shape = op.CONFIG_BENCH if config == "decode" else dict(B=8, L=16384)     # the small one is for profiling
        B, L = shape["B"], shape["L"]
        lens = torch.randint(L // 2, L + 1, (B,), generator=g, device="cuda", dtype=torch.int32)
        inp = dict(q=r16(B, 32, 128), k=r16(B, 8, L, 128), v=r16(B, 8, L, 128), lens=lens)
        nbytes = op.algorithmic_bytes(shape, lens.cpu().numpy())
        rows, name, fn = B, f"decode B={B} L~U[{L // 2},{L}]", decode_b200.kernel
        flops = 4.0 * 32 * 128 * float(lens.sum())
    else:
        raise SystemExit(f"unknown configuration {config!r}")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    times = []
    for i in range(steps + 3):
        flush.fill_(i & 0xff)                     # evict the inputs from L2 between iterations
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn(**inp)
        b.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(a.elapsed_time(b))
    ms_call = statistics.median(times)
    ms = None
    try:
        ms = chain_time(fn, inp, flush, torch, steps)
    except Exception as e:                        # a capture problem must not lose the per-call number
        chain_err = f"{type(e).__name__}: {str(e)[:200]}"
    peak, kind = peaks()
    line = dict(workload=name, algorithmic_mb=nbytes / 1e6, peak=f"of {kind}", l2="flushed between iterations",
                ms_single_call=ms_call, single_call_hbm_frac=nbytes / (ms_call * 1e-3) / 1e9 / peak)
    if ms is None:
        ms, line["chain_error"] = ms_call, chain_err
        line["timing"] = "CUDA events around one kernel(...) call, host launch overhead included"
    else:
        line["timing"] = "per layer of a 16-layer chain (output -> next query) replayed as a CUDA graph"
    line.update(rows_per_s=rows / (ms * 1e-3), ms=ms, hbm_gbs=nbytes / (ms * 1e-3) / 1e9,
                hbm_frac=nbytes / (ms * 1e-3) / 1e9 / peak, hbm_frac_of_8tbs=nbytes / (ms * 1e-3) / 1e9 / NOMINAL_HBM_GBS,
                tflops=flops / (ms * 1e-3) / 1e12)
    return line


def chain_time(fn, inp, flush, torch, rounds, layers=16):
    """Median time per layer of a `layers`-long chain over up to 8 distinct copies of the inputs (within
    1.5 GiB), replayed from a CUDA graph; the L2 is flushed before every replay."""
    per_set = sum(v.numel() * v.element_size() for v in inp.values() if isinstance(v, torch.Tensor))
    n_distinct = int(max(1, min(8, (3 << 29) // max(per_set, 1))))
    g = torch.Generator(device="cuda")
    g.manual_seed(77)
    sets = [inp]
    for _ in range(1, n_distinct):
        cp = {}
        for k, v in inp.items():
            if not isinstance(v, torch.Tensor) or not v.is_floating_point():
                cp[k] = v
            else:
                cp[k] = torch.randn(v.shape, generator=g, device="cuda", dtype=torch.float32).to(v.dtype)
        sets.append(cp)

    def run_chain():
        q = sets[0]["q"]
        for i in range(layers):
            kw = dict(sets[i % n_distinct])
            kw["q"] = q
            q = fn(**kw)
        return q

    run_chain()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run_chain()
    times = []
    for i in range(rounds + 2):
        flush.fill_(i & 0xff)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(a.elapsed_time(b) / layers)
    return statistics.median(times)


def single_gpu_ops(torch, rounds):
    """Every configuration of the op list on one GPU: the five named ones (C1-C4 and the prefix sweep), the two
    extension lines, and the reference's own benchmark shapes (its ops/<op>.py: BENCH_SHAPES) with the geometric
    mean of the speed-up over the strongest library opponent per op, as the reference reports it."""
    from verified_metal_kernels_b200 import abbench, ops
    out, saved = {}, {"prefix": [], "spec": [], "dsa": []}
    # (the sweep's per-request caches for the non-sharing opponent would be 36 GB: its standard op for the output
    # check is the library cascade, and the opponents that need those layouts are skipped by the memory budget)
    named = [("prefix_small", "prefix", dict(N=8, P=4096, S=256), "tree", None),
             ("spec_chain", "spec", dict(B=1, L=8192, k=8), "chain", None),
             ("spec_tree", "spec", SPEC, "tree", None),
             ("dsa_small", "dsa", dict(B=8, L=32768), "tree", None),
             ("prefix_sweep", "prefix", PREFIX, "tree", "torch_cascade")]
    for key, opname, shape, mask, std_name in named:
        try:
            out[key], row = ab_line(opname, f"{opname} {json.dumps(shape)}", shape, torch, rounds, mask=mask,
                                    std_name=std_name)
            saved[opname].append(row)
        except Exception as e:
            out[key] = dict(error=f"{type(e).__name__}: {str(e)[:300]}")
            torch.cuda.synchronize()
    for c in ("spec_tree_paged", "decode"):
        out[c] = side_line(c, torch, 10)
    ref = {}
    for opname in ("prefix", "spec", "dsa"):
        rows_ = []
        for shape in ops.load_op(opname).BENCH_SHAPES:
            try:
                line, row = ab_line(opname, f"{opname} {json.dumps(shape)}", shape, torch, rounds)
                saved[opname].append(row)
                rows_.append({k: line.get(k) for k in ("workload", "ms", "p10_ms", "p90_ms", "rows_per_s", "hbm_frac",
                                                       "hbm_frac_of_8tbs", "vs_torch", "strongest_ref", "speedup",
                                                       "output_ok", "skipped")})
            except Exception as e:
                rows_.append(dict(workload=f"{opname} {json.dumps(shape)}", error=f"{type(e).__name__}: {str(e)[:300]}"))
                torch.cuda.synchronize()
        sp = [r.get("speedup") for r in rows_ if r.get("speedup")]
        ref[opname] = dict(shapes=rows_, geomean_speedup_vs_strongest_torch_ref=abbench.geomean(sp),
                           min=min(sp) if sp else None, max=max(sp) if sp else None)
    out["reference_bench_shapes"] = ref
    try:
        for opname, rows_ in saved.items():
            abbench.save_samples(opname, rows_, ROOT)
        out["samples_saved_to"] = "results/bench_<op>.json"
    except Exception as e:
        out["samples_saved_to"] = f"not saved: {type(e).__name__}"
    return out


# ------------------------------------------------------------------------------------------------ multi-GPU op lines
def timed_side_steps(step, steps, dist, torch, delay):
    """Per-step device time of a multi-GPU side configuration: before each step a 1 GiB fill (flushes L2 and gives
    the host time to enqueue the whole step, so that launch overhead is off the clock) and a tiny all-reduce (the
    ranks start together); CUDA events around the step; per step the MAX over ranks; returns the median in ms."""
    tiny = torch.zeros(1, device="cuda")
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    ev = []
    for i in range(steps):
        delay.fill_(i & 0xff)
        dist.all_reduce(tiny)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        ev.append((a, b))
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) for a, b in ev], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.median().item()), [float(x) for x in t.tolist()]


def multi_prefix(torch, dist, rank, world, steps, delay):
    """The prefix sweep under hybrid sharding: suffixes by request, the shared prefix by kv head (by key range when
    the head count does not divide), one all-to-all of packed partials, local merge."""
    from oracle import judge, ref64
    from verified_metal_kernels_b200 import abbench, load_kernel, ops, shard
    op = ops.load_op("prefix")
    N, P, S, Hq, Hkv, D = PREFIX["N"], PREFIX["P"], PREFIX["S"], op.HQ, op.HKV, op.D
    plan = shard.PrefixHybridPlan(N, Hq, Hkv, P, world)
    lo, hi = plan.req[rank]
    g = torch.Generator(device="cuda")

    def r16(seed, *dims):
        g.manual_seed(seed)
        return torch.randn(*dims, generator=g, device="cuda", dtype=torch.float32).half()

    q_all = r16(11, N, Hq, D)                                                     # the same on every rank
    slens_all = np.random.default_rng(1).integers(0, S + 1, (N,)).astype(np.int32)
    (h0, h1), (k0, k1) = plan.heads[rank], plan.keys[rank]
    # the shared prefix is generated head by head from per-head seeds, so any rank can rebuild any slice
    kp = torch.stack([r16(1000 + h, P, D) for h in range(h0, h1)])[:, k0:k1].contiguous()
    vp = torch.stack([r16(2000 + h, P, D) for h in range(h0, h1)])[:, k0:k1].contiguous()
    ks, vs = r16(3000 + rank, hi - lo, Hkv, S, D), r16(4000 + rank, hi - lo, Hkv, S, D)
    slens = torch.from_numpy(slens_all[lo:hi]).cuda()
    side = torch.cuda.Stream()
    comp = shard.CudaPartials()

    def step(ss=side):
        return shard.prefix_hybrid(q_all, kp, vp, ks, vs, slens, plan, compute=comp, side_stream=ss)

    # the other way to shard this op: by request alone, the shared prefix replicated (every rank reads all of it
    # but stacks only its own requests' rows on it); no exchange at all
    fn = load_kernel("prefix")
    kp_all = torch.stack([r16(1000 + h, P, D) for h in range(Hkv)])
    vp_all = torch.stack([r16(2000 + h, P, D) for h in range(Hkv)])
    q_loc = q_all[lo:hi].contiguous()

    def step_req():
        return fn(q=q_loc, kp=kp_all, vp=vp_all, ks=ks, vs=vs, slens=slens) if hi > lo else None

    # output check: this rank's first request against the float64 oracle on the full prefix, both ways
    ok, err = True, None
    inputs = dict(q=q_all, kp=kp, vp=vp, ks=ks, vs=vs, kp_all=kp_all, vp_all=vp_all)
    before = abbench.checksum(inputs)
    out = step()
    out_req = step_req()
    torch.cuda.synchronize()
    if hi > lo:
        truth = ref64.prefix_ref64(_host(q_all[lo:lo + 1]), _host(kp_all), _host(vp_all), _host(ks[:1]), _host(vs[:1]),
                                   slens_all[lo:lo + 1])
        rep = judge.judge_l2(_host(out[:1].float()), truth, half=True)
        rep2 = judge.judge_l2(_host(out_req[:1].float()), truth, half=True)
        ok, err = bool(rep["ok"] and rep2["ok"]), max(rep.get("err_max", 0.0), rep2.get("err_max", 0.0))
    t_side, _ = timed_side_steps(step, steps, dist, torch, delay)
    t_one, _ = timed_side_steps(lambda: step(None), steps, dist, torch, delay)
    t_req, _ = timed_side_steps(step_req, steps, dist, torch, delay)
    ok = ok and abbench.checksum(inputs) == before
    ok = all_ranks_ok(ok, dist, torch)
    t_hyb = min(t_side, t_one)
    ms = min(t_hyb, t_req)
    nbytes = op.algorithmic_bytes(PREFIX, slens_all)
    per_rank = max(plan.bytes_read(r, slens_all, S) for r in range(world))
    peak, kind = peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    hybrid = f"hybrid: suffixes by request, prefix by {plan.mode} x{world}, one all-to-all of packed (m,l,o) records"
    by_req = f"requests x{world}, shared prefix replicated, no exchange"
    return dict(workload=f"prefix N={N} P={P} S~U[0,{S}]", sharding=hybrid if t_hyb <= t_req else by_req, ms=ms,
                ms_hybrid=t_hyb, ms_hybrid_suffix_on_side_stream=t_side, ms_hybrid_single_stream=t_one, ms_by_request=t_req,
                shardings=dict(hybrid=hybrid, by_request=by_req),
                rows_per_s=N / (ms * 1e-3), algorithmic_mb=nbytes / 1e6, hybrid_max_bytes_per_gpu_mb=per_rank / 1e6,
                by_request_bytes_per_gpu_mb=(2 * Hkv * P * D * 2 + nbytes / world) / 1e6,
                hbm_gbs_aggregate=gbs, hbm_frac=gbs / (peak * world), hbm_frac_of_8tbs=gbs / (NOMINAL_HBM_GBS * world),
                peak=f"of {kind}", timing="median over steps of the max over ranks; CUDA events; 1 GiB fill + tiny all-reduce before each step",
                exchange_bytes_per_rank=int(sum(plan.send_rows(rank)) * shard.RECORD * 4), output_ok=ok, err_max=err)


def multi_spec(torch, dist, rank, world, steps, delay):
    """The speculative tree: batch elements over the ranks; with more ranks than elements each cache is split by
    position inside a group of ranks (one all-to-all of packed partials inside the group)."""
    from oracle import judge, ref64
    from verified_metal_kernels_b200 import abbench, load_kernel, ops, shard
    op = ops.load_op("spec")
    B, L, kd, Hq, Hkv, D = SPEC["B"], SPEC["L"], SPEC["k"], op.HQ, op.HKV, op.D
    plan = shard.SpecSplitPlan(B, kd * Hq, L, world)
    rng = np.random.default_rng(0)
    bits_all = op.pack_bits([op.tree_bits(kd, rng, SPEC["max_depth"]) for _ in range(B)], kd)
    g = torch.Generator(device="cuda")

    def r16(seed, *dims):
        g.manual_seed(seed)
        return torch.randn(*dims, generator=g, device="cuda", dtype=torch.float32).half()

    # element b: q from seed 100 + b; its cache from per-head seeds, so that any rank can rebuild any element
    def elem_q(b):
        return r16(100 + b, 1, kd, Hq, D)

    def elem_kv(b, which, lo, hi):
        return torch.stack([r16(1000 * which + 16 * b + h, L, D) for h in range(Hkv)])[None, :, lo:hi].contiguous()

    comp = shard.CudaPartials()
    ok, err = True, None
    if plan.split:
        b = plan.elem[rank]
        lo, hi = plan.keys[rank]
        q, bits = elem_q(b), torch.from_numpy(bits_all[b:b + 1]).cuda()
        k, v = elem_kv(b, 1, lo, hi), elem_kv(b, 2, lo, hi)
        step = lambda: shard.spec_split(q, k, v, bits, plan, compute=comp)
        inputs = dict(q=q, k=k, v=v)
        out, (r0, r1) = step()
        torch.cuda.synchronize()
        # check the first draft row this rank owns (all its heads in the range) against the full cache
        i0 = r0 // Hq
        kf, vf = _host(elem_kv(b, 1, 0, L)), _host(elem_kv(b, 2, 0, L))
        truth = ref64.spec_ref64(_host(q), kf, vf, bits_all[b:b + 1])[0].reshape(kd * Hq, D)
        r_hi = min(r1, (i0 + 2) * Hq)
        rep = judge.judge_l2(_host(out[:r_hi - r0].float()), truth[r0:r_hi], half=True)
        ok, err = bool(rep["ok"]), rep.get("err_max")
        del kf, vf
        mode = f"cache split in {world // B} by position inside groups of ranks, one all-to-all of packed (m,l,o) records per group"
        xbytes = int(sum(plan.send_rows(rank)) * shard.RECORD * 4)
    else:
        lo, hi = plan.elems[rank]
        fn = load_kernel("spec")
        xbytes = 0
        mode = f"batch elements x{world}, no exchange"
        if hi > lo:
            q = torch.cat([elem_q(b) for b in range(lo, hi)])
            k = torch.cat([elem_kv(b, 1, 0, L) for b in range(lo, hi)])
            v = torch.cat([elem_kv(b, 2, 0, L) for b in range(lo, hi)])
            bits = torch.from_numpy(bits_all[lo:hi]).cuda()
            step = lambda: fn(q=q, k=k, v=v, bits=bits)
            inputs = dict(q=q, k=k, v=v)
            out = step()
            torch.cuda.synchronize()
            # the first two draft rows of this rank's first element against the float64 oracle
            full = ref64.spec_ref64(_host(q[:1]), _host(k[:1]), _host(v[:1]), bits_all[lo:lo + 1])[:, :2]
            rep = judge.judge_l2(_host(out[:1, :2].float()), full, half=True)
            ok, err = bool(rep["ok"]), rep.get("err_max")
            del full
        else:
            step, inputs = (lambda: None), {}
    before = abbench.checksum(inputs)
    ms, _ = timed_side_steps(step, steps, dist, torch, delay)
    ok = ok and abbench.checksum(inputs) == before
    extra = {}
    if plan.split:
        # the alternative with more ranks than elements: whole elements on the first B ranks, the others idle (no
        # exchange, so none of its fixed cost); the faster of the two is the line's `ms`
        fn = load_kernel("spec")
        if rank < B:
            qw, bw = elem_q(rank), torch.from_numpy(bits_all[rank:rank + 1]).cuda()
            kw_, vw = elem_kv(rank, 1, 0, L), elem_kv(rank, 2, 0, L)
            step_whole = lambda: fn(q=qw, k=kw_, v=vw, bits=bw)
        else:
            step_whole = lambda: None
        ms_whole, _ = timed_side_steps(step_whole, steps, dist, torch, delay)
        extra = dict(ms_cache_split=ms, ms_whole_elements_on_first_ranks=ms_whole,
                     shardings=dict(cache_split=mode, whole_elements=f"batch elements on {B} of {world} ranks, no exchange"))
        if ms_whole < ms:
            ms, mode, xbytes = ms_whole, extra["shardings"]["whole_elements"], 0
    ok = all_ranks_ok(ok, dist, torch)
    nbytes = op.algorithmic_bytes(SPEC)
    flops = 4.0 * B * kd * Hq * D * L
    peak, kind = peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    used = min(world, max(B, world if plan.split else B))
    return dict(extra, workload=f"spec tree depth<=8 B={B} k={kd} L={L}", sharding=mode, ms=ms, rows_per_s=B * kd / (ms * 1e-3),
                algorithmic_mb=nbytes / 1e6, hbm_gbs_aggregate=gbs, hbm_frac=gbs / (peak * world),
                hbm_frac_of_8tbs=gbs / (NOMINAL_HBM_GBS * world), tflops_aggregate=flops / (ms * 1e-3) / 1e12,
                gpus_with_work=(B if xbytes == 0 else world) if plan.split else used, peak=f"of {kind}",
                timing="median over steps of the max over ranks; CUDA events; 1 GiB fill + tiny all-reduce before each step",
                exchange_bytes_per_rank=xbytes, output_ok=ok, err_max=err)


# ------------------------------------------------------------------------------------------------ CPU arm
def blas_threads(n=None):
    """Sets (when n is given) and returns the BLAS thread count NumPy's matmuls use.  A launcher that starts one
    process per GPU exports OMP_NUM_THREADS=1; the CPU arm runs on one rank alone and takes every core it may."""
    try:
        import threadpoolctl
        if n is not None:
            threadpoolctl.threadpool_limits(limits=int(n))
        info = [p for p in threadpoolctl.threadpool_info() if p.get("user_api") == "blas"]
        return max([int(p.get("num_threads", 1)) for p in info] or [1])
    except Exception:
        return None


def cpu_sample(n_requests, L):
    """Float64 oracle on `n_requests` requests of the dsa workload; returns seconds."""
    from oracle import ref64
    from verified_metal_kernels_b200 import ops
    op = ops.load_op("dsa")
    inp = op.make_inputs(dict(B=n_requests, L=L), seed=0)
    t0 = time.perf_counter()
    ref64.dsa_ref64(inp["q"], inp["kv"], inp["iq"], inp["ik"], inp["w"], None)
    return time.perf_counter() - t0


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def reference_arm(a):
    """The reference's CPU implementation of the path: its float64 NumPy truth as restated in oracle/ (the
    reference is a Python package that cannot travel to the GPU box; the restatement replaces its einsum
    contractions by BLAS matmuls of the same float64 arithmetic, which is faster, so the ratio against it is
    conservative).  One request per step, on every host core the process may use."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cores = host_cores()
    threads = blas_threads(cores)
    for _ in range(min(a.warmup, 1)):
        cpu_sample(1, DSA["L"])
    t = [cpu_sample(1, DSA["L"]) for _ in range(a.steps)]
    sec = sum(t) / len(t)
    v = 1.0 / sec
    line = dict(metric=METRIC, value=v, unit=UNIT, impl="reference", n_gpus=a.gpus, steps=a.steps, warmup=min(a.warmup, 1),
                ms_per_step=sec * 1e3, higher_is_better=True, scaling=a.scaling or ("weak" if a.gpus == 1 else "strong"),
                vs_baseline=None, dtype="f64", data="synthetic",
                config=dict(workload="dsa B=128 L=131072 (sample: 1 request per step)"),
                cpu_baseline=dict(value=v, unit=UNIT, cores=cores, blas_threads=threads, kind="port",
                                  sample="1 of 128 requests (B=1, L=131072) per step, float64 NumPy oracle, BLAS matmuls"),
                e2e=dict(value=v, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------------ main
def e2e_leg(fn, inp, Bl, L, world, steps, dist, torch):
    """The same op through the public kernel(...) call with pinned HOST tensors (at most E2E_MAX requests per call)."""
    from verified_metal_kernels_b200.kernels import dsa_b200
    Be = min(max(Bl, 1), E2E_MAX)
    host = {}
    for k, v in inp.items():
        if v is not None:
            host[k] = torch.empty(v[:Be].shape, dtype=v.dtype, pin_memory=True)
            host[k].copy_(v[:Be])
        else:
            host[k] = None
    torch.cuda.synchronize()
    all_bytes = sum(v.numel() * v.element_size() for v in host.values() if v is not None)
    kv_bytes = host["kv"].numel() * host["kv"].element_size()
    # the kernel module leaves a page-locked latent cache on the host and reads only the selected rows
    in_place = dsa_b200.HOST_CACHE_IN_PLACE and L > 2048
    h2d = all_bytes - kv_bytes + Be * min(L, 2048) * 576 * 2 if in_place else all_bytes
    d2h = Be * 128 * 512 * 2
    e_steps = min(steps, 5)
    run_h = (lambda: fn(**host)) if Bl > 0 else (lambda: None)
    esec, _, _ = timed_steps(run_h, e_steps, 1, dist, torch)
    e_rows = Be
    if dist is not None:
        t = torch.tensor([Be if Bl > 0 else 0], device="cuda", dtype=torch.int64)
        dist.all_reduce(t)
        e_rows = int(t.item())
    e2e = dict(value=e_rows * e_steps / esec, unit=UNIT, h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
               steps=e_steps, sample=f"{Be} requests per call per rank (of {Bl}), pinned host tensors in, host tensor out"
               + ("; the latent cache stays in host memory and stage 3 reads its 2048 selected rows per request "
                  "from there, every other input is copied" if in_place else ""))
    if in_place:
        # the same call with the cache copied to the device whole, for comparison
        dsa_b200.HOST_CACHE_IN_PLACE = False
        try:
            fsec, _, _ = timed_steps(run_h, e_steps, 1, dist, torch)
        finally:
            dsa_b200.HOST_CACHE_IN_PLACE = True
        e2e["copy_everything"] = dict(value=e_rows * e_steps / fsec, unit=UNIT, h2d_bytes_per_step=all_bytes)
        # the same call with the index queries and keys as e4m3 bytes + scales (a different input format, reported
        # beside): the index keys are most of what crosses the link, and this halves them
        iq8, iqs, ik8, iks = fp8_index({k: inp[k][:Be] for k in ("iq", "ik")}, torch)
        h8 = []
        for t in (iq8, iqs, ik8, iks):
            h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            h.copy_(t)
            h8.append(h)
        del iq8, iqs, ik8, iks
        torch.cuda.synchronize()
        run_8 = ((lambda: dsa_b200.kernel_fp8_index(host["q"], host["kv"], h8[0], h8[1], h8[2], h8[3], host["w"]))
                 if Bl > 0 else (lambda: None))
        gsec, _, _ = timed_steps(run_8, e_steps, 1, dist, torch)
        small = sum(host[k].numel() * host[k].element_size() for k in ("q", "w")) + sum(h.numel() * h.element_size() for h in h8)
        e2e["fp8_index"] = dict(value=e_rows * e_steps / gsec, unit=UNIT,
                                h2d_bytes_per_step=small + Be * min(L, 2048) * 576 * 2)
    return e2e


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=DSA["B"], help="total dsa batch (default: the sweep's 128)")
    ap.add_argument("--cache", type=int, default=DSA["L"], help="dsa cache length (default: the sweep's 131072)")
    ap.add_argument("--scaling", default=None, choices=["weak", "strong"],
                    help="N>1: strong = --batch requests in total, cut over the ranks (default); weak = --batch "
                         "requests per rank as the headline.  Both are measured and printed either way")
    ap.add_argument("--batch-invariant", action="store_true",
                    help="time the library with vmk_set_batch_invariant(1) (fixed kernels and cut points)")
    ap.add_argument("--no-side", action="store_true", help="skip the per-op lines (`ops`)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--spec-batch", type=int, default=SPEC["B"], help="batch elements of the speculative-tree line (default: "
                    "the configuration's 4; with fewer elements than ranks the caches are split by position)")
    ap.add_argument("--rounds", type=int, default=30, help="shuffled rounds per configuration of the per-op lines")
    ap.add_argument("--attend-variant", default=None, choices=["mma", "tcgen05", "tcgen05_tma", "tcgen05_pair"],
                    help="dsa stage 3 implementation (default: the library's, tcgen05_pair); for A/B runs")
    ap.add_argument("--side-only", default=None, help="time only one configuration (prefix_small, spec_chain, "
                    "spec_tree, dsa_small, prefix_sweep, decode, decode_small, spec_tree_paged) on one GPU and print "
                    "its line; used for profiling")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3) if a.impl == "ours" else a.warmup
    if a.impl == "reference":
        return reference_arm(a)
    SPEC["B"] = a.spec_batch

    import torch
    from verified_metal_kernels_b200 import _lib, abbench, build, load_kernel, ops, shard
    from verified_metal_kernels_b200.kernels import dsa_b200
    rank, local_rank, world = shard.world()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    build.build()
    if a.batch_invariant:
        _lib.lib().vmk_set_batch_invariant(1)
    if a.attend_variant:
        dsa_b200.set_attend_variant(a.attend_variant)
    if a.side_only:
        print(json.dumps(side_line(a.side_only, torch, a.steps)))
        return 0
    scaling = a.scaling or ("weak" if world == 1 else "strong")
    fn = load_kernel("dsa")
    op = ops.load_op("dsa")
    B, L = a.batch, a.cache
    lo, hi = shard.unit_range(B, rank, world)
    inp_full = dsa_inputs(B, L, "cuda", seed=1000 + rank)          # this rank's own 128 requests (the weak batch)
    n_strong = hi - lo
    inp_strong = {k: (None if v is None else v[:max(n_strong, 1)]) for k, v in inp_full.items()}   # its share of ONE batch

    # ---- output check before any timing: one request of this rank against the float64 oracle
    before = abbench.checksum({k: v for k, v in inp_strong.items() if v is not None})
    out, idx, cnt = dsa_b200.kernel(**inp_strong, return_selection=True)
    torch.cuda.synchronize()
    ok, detail = check_dsa_request(inp_strong, out, idx, cnt, 0)
    del out, idx, cnt

    def timed(inp_, n_local, sampler=None):
        run = (lambda: fn(**inp_)) if n_local > 0 else (lambda: None)
        return timed_steps(run, a.steps, a.warmup, dist, torch, sampler)

    sampler = ClockSampler(torch.cuda.current_device()) if rank == 0 else None
    results = {}
    clocks_by_rank = {}
    if world == 1:
        results["weak"] = timed(inp_full, B, sampler) + (B, B)
    else:
        order = ["strong", "weak"] if scaling == "strong" else ["weak", "strong"]
        rank_ms = {}
        for i, kind in enumerate(order):
            # every rank samples its own GPU's clock in both runs: when the step (the maximum over the ranks) is
            # slower than one GPU's, the per-rank times and clocks say which GPUs and why
            smp = sampler if (i == 0 and rank == 0) else ClockSampler(torch.cuda.current_device())
            if kind == "strong":
                results[kind] = timed(inp_strong, n_strong, smp) + (B, n_strong)
            else:
                results[kind] = timed(inp_full, B, smp) + (B * world, B)
            rank_ms[kind] = RANK_MS[-1]
            mine = results[kind][2] or {}
            every = [None] * world
            dist.all_gather_object(every, dict(sm_mhz=mine.get("sm_mhz"), sm_mhz_min=mine.get("sm_mhz_min"),
                                               reasons=mine.get("reasons")))
            clocks_by_rank[kind] = every
    status = _lib.read_status(dev)
    ok = ok and abbench.checksum({k: v for k, v in inp_strong.items() if v is not None}) == before
    ok = all_ranks_ok(ok, dist, torch)
    head = "weak" if world == 1 else scaling
    sec, per, clocks, B_total, Bl = results[head]
    value = B_total * a.steps / sec
    inp = inp_full if head == "weak" else inp_strong

    e2e = None if a.no_e2e else e2e_leg(fn, inp, Bl, L, world, a.steps, dist, torch)
    status |= _lib.read_status(dev)

    launches = 3 + (1 if _lib.lib().vmk_dsa_attend_workspace_bytes(max(Bl, 1)) > 256 else 0)
    metric = METRIC if (B, L) == (DSA["B"], DSA["L"]) else f"dsa decode rows/s (batch {B}, cache {L})"
    line = dict(metric=metric, value=value, unit=UNIT, n_gpus=world, steps=a.steps, warmup=a.warmup,
                ms_per_step=sec * 1e3 / a.steps, higher_is_better=True, scaling=head, vs_baseline=None, dtype="f16",
                data="synthetic",
                config=dict(workload=f"dsa B={B} L={L}" + (" (8-GPU sweep configuration)" if (B, L) == (DSA["B"], DSA["L"]) else ""),
                            parallelism=f"batch-sharded x{world}", global_batch=B_total, per_rank_batch=Bl,
                            l2="inputs (GBs per rank) far larger than the 126 MB L2; no flush"),
                clocks=clocks, e2e=e2e, gpu_launches=launches * a.steps, device_status=status,
                output_ok=ok, output_check=dict(what="request 0 of every rank against the float64 oracle (selection + output), "
                                                "inputs unmodified after the run", rank0=detail))
    for kind, (s_, _, _, bt, bl) in results.items():
        if kind != head or world > 1:
            line[kind] = dict(value=bt * a.steps / s_, unit=UNIT, ms_per_step=s_ * 1e3 / a.steps, global_batch=bt,
                              per_rank_batch=bl, scaling=kind)
            if world > 1:
                line[kind]["ms_per_step_by_rank"] = rank_ms[kind]
                line[kind]["clocks_by_rank"] = clocks_by_rank[kind]

    if world > 1:
        # the stages one by one on every rank's own 128 requests: when some GPUs are slower than others on the whole
        # step (ms_per_step_by_rank), this says in which stage
        mine = stage_times(inp_full, min(a.steps, 10), torch)
        every = [None] * world
        dist.all_gather_object(every, {k: round(v, 5) for k, v in mine.items()})
        if "weak" in line:
            line["weak"]["stages_ms_by_rank"] = every

    side_ops = None
    if world > 1 and not a.no_side:
        # side configurations on all ranks (collectives inside): the big dsa inputs go first
        del inp, inp_strong
        keep = {k: (None if v is None else v[:max(n_strong, 1)].clone()) for k, v in inp_full.items()}
        del inp_full
        torch.cuda.empty_cache()
        delay = torch.empty(DELAY_BYTES, dtype=torch.uint8, device="cuda")
        side_ops = {}
        for key, f in (("prefix_sweep", multi_prefix), ("spec_tree", multi_spec)):
            try:
                side_ops[key] = f(torch, dist, rank, world, max(a.steps, 10), delay)
            except Exception as e:                 # every rank raises or none does (same code path), so no rank is left waiting
                side_ops[key] = dict(error=f"{type(e).__name__}: {str(e)[:300]}")
        del delay
        status |= _lib.read_status(dev)
        line["device_status"] = status
        inp_full = keep
        inp = keep

    if rank == 0:
        st_inp = inp if world > 1 else inp
        st = stage_times(st_inp, min(a.steps, 10), torch)
        Bs = st_inp["ik"].shape[0]
        peak, kind = peaks()
        alg = Bs * L * 128 * 2                       # the ik stream: every byte once
        ach = alg / (st["indexer_ms"] * 1e-3) / 1e9
        tr = ncu_traffic()
        line["roofline"] = dict(kernel="dsa indexer", bound="hbm", achieved=ach, peak=peak, unit="GB/s", frac=ach / peak,
                                frac_of_8tbs=ach / NOMINAL_HBM_GBS, batch=Bs,
                                peak_source=f"of {kind}", traffic=(tr["indexer_bytes_per_position"] * Bs * L if tr else None),
                                algorithmic_bytes=alg, launch_ms=st["indexer_ms"])
        total_alg = op.algorithmic_bytes(dict(B=B_total, L=L))
        gbs = total_alg / (sec / a.steps) / 1e9
        line["stages_ms"] = dict(st, batch=Bs)
        line["op_hbm"] = dict(algorithmic_bytes=total_alg, gbs=gbs, frac=gbs / (peak * world),
                              frac_of_8tbs=gbs / (NOMINAL_HBM_GBS * world), gpus=world)
        if world == 1 and not a.no_side:
            # the whole op with fp8 index keys (a different input format: reported beside the headline)
            try:
                iq8, iqs, ik8, iks = fp8_index(inp, torch)
                f8 = lambda: dsa_b200.kernel_fp8_index(inp["q"], inp["kv"], iq8, iqs, ik8, iks, inp["w"])
                fsec, _, _ = timed_steps(f8, min(a.steps, 10), 3, None, torch)
                n8 = min(a.steps, 10)
                alg8 = total_alg - B * L * 128 + B * L * 4
                line["fp8_index"] = dict(value=B * n8 / fsec, unit=UNIT, ms_per_step=fsec * 1e3 / n8,
                                         algorithmic_bytes=alg8, hbm_frac=alg8 / (fsec / n8) / 1e9 / peak,
                                         note="index queries and keys as e4m3 bytes + fp32 scales; q, kv fp16")
                del iq8, iqs, ik8, iks
            except Exception as e:
                line["fp8_index"] = dict(error=f"{type(e).__name__}: {str(e)[:200]}")
            del inp, inp_full, inp_strong, st_inp
            torch.cuda.empty_cache()
            line["ops"] = single_gpu_ops(torch, a.rounds)
        elif side_ops is not None:
            line["ops"] = side_ops
        if not a.no_cpu and world == 1:
            n = 2
            threads = blas_threads(host_cores())
            t = cpu_sample(n, L)
            line["cpu_baseline"] = dict(value=n / t, unit=UNIT, cores=host_cores(), blas_threads=threads, kind="port",
                                        sample=f"{n} of {B} requests (L={L}), float64 NumPy oracle, {t:.1f} s")
        line["device_status"] |= _lib.read_status(dev)
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    bad = line["device_status"] != 0 or not line["output_ok"]
    if bad and rank == 0:
        sys.stderr.write(f"bench.py: INVALID run (device_status={line['device_status']}, output_ok={line['output_ok']})\n")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
