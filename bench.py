"""Benchmark of the B200 decode kernels on the multi-GPU sweep workload.

    python bench.py                                   # 1 GPU, dsa B=128 L=131072 (+ prefix / spec side lines)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus 8 --steps 20 --warmup 3       # every rank its own batch of 128 requests (weak scaling)
    ... bench.py --gpus 8 --scaling strong            # ONE batch of 128 requests cut over the ranks
    python bench.py --impl reference                  # the float64 NumPy truth timed on the host cores

A step is one pass of the op over the whole batch.  The headline op is `dsa` on the sweep configuration
(batch 128, cache 131072): rows/s where a row is one request's complete output.  Requests are independent
units: they are spread over the ranks with no collective on the data path.  By default every rank holds
the configuration's 128 requests (weak scaling: the global batch is 128 x N); `--scaling strong` cuts one
batch of 128 over the ranks instead (16 per GPU at N=8, where the fixed latencies of the three stages weigh
more).
Inputs are synthetic (seeded N(0,1) rounded to fp16, head weights N(0,1)/sqrt(64*128), as the op's
generator draws them) and far larger than the 126 MB L2, so no flush is needed between steps.

Rank 0 prints one JSON line.  `value` is timed with inputs resident in HBM; `e2e` is timed through the
kernel module's public call with pinned HOST tensors (host->device copies and the device->host read of
the result inside the timed region); `roofline` is for the dominant kernel (the indexer) from CUDA
events inside this run; `cpu_baseline` is the float64 oracle on a bounded sample on the host cores."""
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
PREFIX = dict(N=256, P=32768, S=2048)
SPEC = dict(B=4, L=32768, k=64)
FALLBACK_HBM_GBS = 6650.0
E2E_MAX = 32


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
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=self.max_mhz,
                    reasons=[n for b, n in self.REASONS.items() if bits & b], samples=len(sm), window=window,
                    sampler_error=self.err)


# ------------------------------------------------------------------------------------------------ inputs
def dsa_inputs(B, L, device, seed):
    """Synthetic dsa inputs on the device with the generator's distributions (chunked to bound memory)."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)

    def randn16(*shape):
        out = torch.empty(*shape, dtype=torch.float16, device=device)
        flat = out.view(-1)
        step = 1 << 28
        for i in range(0, flat.numel(), step):
            n = min(step, flat.numel() - i)
            flat[i:i + n] = torch.randn(n, generator=g, device=device, dtype=torch.float32).half()
        return out

    return dict(q=randn16(B, 128, 576), kv=randn16(B, L, 576), iq=randn16(B, 64, 128), ik=randn16(B, L, 128),
                w=torch.randn(B, 64, generator=g, device=device, dtype=torch.float32) * (64 ** -0.5 * 128 ** -0.5),
                lens=None)


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
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
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
    out["indexer_ms"] = avg(lambda: L.vmk_dsa_indexer(inp["iq"].data_ptr(), inp["ik"].data_ptr(), inp["w"].data_ptr(),
                                                      None, scores.data_ptr(), B, Lk, status.data_ptr(), st))
    hist = torch.empty(B, 2048, dtype=torch.int32, device=scores.device)
    out["indexer_ms"] = avg(lambda: L.vmk_dsa_indexer_hist(inp["iq"].data_ptr(), inp["ik"].data_ptr(),
                                                           inp["w"].data_ptr(), None, scores.data_ptr(), hist.data_ptr(),
                                                           B, Lk, status.data_ptr(), st))
    out["select_ms"] = avg(lambda: L.vmk_dsa_select_hist(scores.data_ptr(), hist.data_ptr(), None, idx.data_ptr(),
                                                         cnt.data_ptr(), B, Lk, st))
    out["attend_ms"] = avg(lambda: dsa_b200.attend(inp["q"], inp["kv"], idx, cnt))
    # stage 1 on fp8 index queries and keys (a different input format, reported beside the fp16 stage)
    iq8, iqs = dsa_b200.quantize_e4m3(inp["iq"])
    ik8 = torch.empty(B, Lk, 128, dtype=torch.uint8, device=scores.device)
    iks = torch.empty(B, Lk, dtype=torch.float32, device=scores.device)
    for b0 in range(0, B, 8):                              # in pieces: the float copy of ik is 4 x its size
        ik8[b0:b0 + 8], iks[b0:b0 + 8] = dsa_b200.quantize_e4m3(inp["ik"][b0:b0 + 8])
    out["indexer_fp8_ms"] = avg(lambda: L.vmk_dsa_indexer_hist_fp8(iq8.data_ptr(), iqs.data_ptr(), ik8.data_ptr(),
                                                                   iks.data_ptr(), inp["w"].data_ptr(), None,
                                                                   scores.data_ptr(), hist.data_ptr(), B, Lk,
                                                                   status.data_ptr(), st))
    return out


def side_line(config, torch, steps):
    """rows/s and HBM fraction of one named configuration on one GPU, L2 flushed between iterations.
    Configurations: prefix_small, spec_chain, spec_tree, spec_tree_paged, dsa_small (the single-GPU ones),
    prefix_sweep and decode (the extension op)."""
    from verified_metal_kernels_b200 import load_kernel, ops
    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    r16 = lambda *s: torch.randn(*s, generator=g, device="cuda", dtype=torch.float32).half()
    if config in ("prefix_small", "prefix_sweep"):
        opname = "prefix"
        op = ops.load_op(opname)
        shape = dict(N=8, P=4096, S=256) if config == "prefix_small" else PREFIX
        N, P, S = shape["N"], shape["P"], shape["S"]
        inp = dict(q=r16(N, 32, 128), kp=r16(8, P, 128), vp=r16(8, P, 128), ks=r16(N, 8, S, 128), vs=r16(N, 8, S, 128))
        sl = None
        if config == "prefix_sweep":
            inp["slens"] = torch.randint(0, S + 1, (N,), generator=g, device="cuda", dtype=torch.int32)
            sl = inp["slens"].cpu().numpy()
        nbytes = op.algorithmic_bytes(shape, sl)
        rows = N
        name = f"prefix N={N} P={P} " + (f"S~U[0,{S}]" if sl is not None else f"S={S}")
        flops = 4.0 * N * 32 * 128 * (P + (float(sl.mean()) if sl is not None else S))
    elif config in ("spec_chain", "spec_tree", "spec_tree_paged"):
        opname = "spec"
        op = ops.load_op(opname)
        shape = dict(B=1, L=8192, k=8) if config == "spec_chain" else SPEC
        B, L, kd = shape["B"], shape["L"], shape["k"]
        rng = np.random.default_rng(0)
        masks = [op.chain_bits(kd) if config == "spec_chain" else op.tree_bits(kd, rng, 8) for _ in range(B)]
        inp = dict(q=r16(B, kd, 32, 128), k=r16(B, 8, L, 128), v=r16(B, 8, L, 128),
                   bits=torch.from_numpy(op.pack_bits(masks, kd)).cuda())
        nbytes = op.algorithmic_bytes(shape)
        rows = B * kd
        name = f"spec {'chain' if config == 'spec_chain' else 'tree depth<=8'} B={B} k={kd} L={L}"
        flops = 4.0 * B * kd * 32 * 128 * L
        if config == "spec_tree_paged":
            # the same cache as a shuffled pool of 64-key pages (the smallest page the kernels take)
            page = 64
            T = L // page
            perm = torch.randperm(B * T + 7, generator=g, device="cuda")[:B * T].to(torch.int32).reshape(B, T)
            inp = dict(q=inp["q"], k_pages=r16(B * T + 7, 8, page, 128), v_pages=r16(B * T + 7, 8, page, 128),
                       page_table=perm.contiguous(), L=L, bits=inp["bits"])
            name += f", paged cache (page {page})"
    elif config in ("decode", "decode_small"):
        # plain single-token decode (extension op): 64 requests with caches of 16k..32k keys
        from verified_metal_kernels_b200.ops import decode as op
        opname = "decode"
        shape = op.CONFIG_BENCH if config == "decode" else dict(B=8, L=16384)     # the small one is for profiling
        B, L = shape["B"], shape["L"]
        lens = torch.randint(L // 2, L + 1, (B,), generator=g, device="cuda", dtype=torch.int32)
        inp = dict(q=r16(B, 32, 128), k=r16(B, 8, L, 128), v=r16(B, 8, L, 128), lens=lens)
        nbytes = op.algorithmic_bytes(shape, lens.cpu().numpy())
        rows, name = B, f"decode B={B} L~U[{L // 2},{L}]"
        flops = 4.0 * 32 * 128 * float(lens.sum())
    else:
        opname = "dsa"
        op = ops.load_op(opname)
        shape = dict(B=8, L=32768)
        inp = dsa_inputs(shape["B"], shape["L"], "cuda", seed=5)
        nbytes = op.algorithmic_bytes(shape)
        rows, name = shape["B"], "dsa B=8 L=32768"
        flops = 2.0 * 64 * 128 * shape["L"] * shape["B"] + 2.0 * 128 * (576 + 512) * 2048 * shape["B"]
    if opname == "decode":
        from verified_metal_kernels_b200.kernels import decode_b200
        fn = decode_b200.kernel
    else:
        fn = load_kernel(opname)
    if config == "spec_tree_paged":
        from verified_metal_kernels_b200.kernels import spec_b200
        fn = spec_b200.kernel_paged
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
    # The reference's timing method (bench.py:61-76 there): a chain of 16 "layers" on distinct input sets, each
    # layer's query being the previous layer's output, here captured once in a CUDA graph and replayed after an
    # L2 flush, so that host launch overhead is off the clock.
    ms = None
    try:
        ms = chain_time(opname, fn, inp, flush, torch, steps)
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
                hbm_frac=nbytes / (ms * 1e-3) / 1e9 / peak, tflops=flops / (ms * 1e-3) / 1e12)
    return line


def chain_time(opname, fn, inp, flush, torch, rounds, layers=16):
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
            if not isinstance(v, torch.Tensor) or not v.is_floating_point() or k in ("w",):
                cp[k] = v
            else:
                cp[k] = torch.randn(v.shape, generator=g, device="cuda", dtype=torch.float32).to(v.dtype)
        sets.append(cp)

    def run_chain():
        q = sets[0]["q"]
        for i in range(layers):
            kw = dict(sets[i % n_distinct])
            kw["q"] = q
            out = fn(**kw)
            q = torch.cat([out, kw["q"][..., 512:]], dim=-1) if opname == "dsa" else out
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


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_sample(n_requests, L):
    """Float64 oracle on `n_requests` requests of the dsa workload; returns (seconds, cores used)."""
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
    """The reference's CPU implementation of the path: its float64 NumPy truth, restated in oracle/ (the
    reference is a Python package that cannot travel to the GPU box).  One request per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    for _ in range(min(a.warmup, 1)):
        cpu_sample(1, DSA["L"])
    t = [cpu_sample(1, DSA["L"]) for _ in range(a.steps)]
    sec = sum(t) / len(t)
    v = 1.0 / sec
    line = dict(metric=METRIC, value=v, unit=UNIT, impl="reference", n_gpus=a.gpus, steps=a.steps, warmup=min(a.warmup, 1),
                ms_per_step=sec * 1e3, higher_is_better=True, scaling=a.scaling, vs_baseline=None, dtype="f64",
                data="synthetic", config=dict(workload="dsa B=128 L=131072 (sample: 1 request per step)"),
                cpu_baseline=dict(value=v, unit=UNIT, cores=host_cores(), kind="port",
                                  sample="1 of 128 requests (B=1, L=131072) per step, NumPy float64, BLAS threads"),
                e2e=dict(value=v, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=DSA["B"], help="total dsa batch (default: the sweep's 128)")
    ap.add_argument("--cache", type=int, default=DSA["L"], help="dsa cache length (default: the sweep's 131072)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="N>1: weak = --batch requests per rank (default), strong = --batch requests in total")
    ap.add_argument("--batch-invariant", action="store_true",
                    help="time the library with vmk_set_batch_invariant(1) (fixed kernels and cut points)")
    ap.add_argument("--no-side", action="store_true", help="skip the prefix / spec side lines")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--side-only", default=None, help="time only one side configuration (prefix_small, spec_chain, "
                    "spec_tree, dsa_small, prefix_sweep) on one GPU and print its line; used for profiling")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3) if a.impl == "ours" else a.warmup
    if a.impl == "reference":
        return reference_arm(a)

    import torch
    from verified_metal_kernels_b200 import _lib, build, load_kernel, ops, shard
    rank, local_rank, world = shard.world()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    build.build()
    if a.batch_invariant:
        _lib.lib().vmk_set_batch_invariant(1)
    if a.side_only:
        print(json.dumps(side_line(a.side_only, torch, a.steps)))
        return 0
    fn = load_kernel("dsa")
    op = ops.load_op("dsa")
    B, L = a.batch, a.cache
    if a.scaling == "weak":
        Bl, B_total = B, B * world                       # this rank's own requests; global batch grows with N
    else:
        lo, hi = shard.unit_range(B, rank, world)
        Bl, B_total = hi - lo, B
    inp = dsa_inputs(max(Bl, 1), L, "cuda", seed=1000 + rank)
    run = (lambda: fn(**inp)) if Bl > 0 else (lambda: None)

    sampler = ClockSampler(torch.cuda.current_device()) if rank == 0 else None
    sec, per, clocks = timed_steps(run, a.steps, a.warmup, dist, torch, sampler)
    status = _lib.read_status(torch.device("cuda", torch.cuda.current_device()))
    value = B_total * a.steps / sec

    # end to end: pinned host tensors in, host tensor out, through the public kernel(...) call
    e2e = None
    if not a.no_e2e:
        # Pinned host copies of (a bounded slice of) this rank's batch: at most E2E_MAX requests per call, so
        # that host memory and the pinning time stay modest; rows/s is per-request work either way.
        Be = min(max(Bl, 1), E2E_MAX)
        host = {}
        for k, v in inp.items():
            if v is not None:
                host[k] = torch.empty(v[:Be].shape, dtype=v.dtype, pin_memory=True)
                host[k].copy_(v[:Be])
            else:
                host[k] = None
        torch.cuda.synchronize()
        from verified_metal_kernels_b200.kernels import dsa_b200
        all_bytes = sum(v.numel() * v.element_size() for v in host.values() if v is not None)
        kv_bytes = host["kv"].numel() * host["kv"].element_size()
        # the kernel module leaves a page-locked latent cache on the host and reads only the selected rows
        in_place = dsa_b200.HOST_CACHE_IN_PLACE and L > 2048
        h2d = all_bytes - kv_bytes + Be * min(L, 2048) * 576 * 2 if in_place else all_bytes
        d2h = Be * 128 * 512 * 2
        e_steps = min(a.steps, 5)
        run_h = (lambda: fn(**host)) if Bl > 0 else (lambda: None)
        esec, _, _ = timed_steps(run_h, e_steps, 1, dist, torch)
        e_rows = Be * world if Bl > 0 else 0
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
        del host

    launches = 3 + (1 if _lib.lib().vmk_dsa_attend_workspace_bytes(max(Bl, 1)) > 256 else 0)
    metric = METRIC if (B, L) == (DSA["B"], DSA["L"]) else f"dsa decode rows/s (batch {B}, cache {L})"
    line = dict(metric=metric, value=value, unit=UNIT, n_gpus=world, steps=a.steps, warmup=a.warmup,
                ms_per_step=sec * 1e3 / a.steps, higher_is_better=True, scaling=a.scaling, vs_baseline=None, dtype="f16",
                data="synthetic",
                config=dict(workload=f"dsa B={B} L={L}" + (" (8-GPU sweep configuration)" if (B, L) == (DSA["B"], DSA["L"]) else ""), parallelism=f"batch-sharded x{world}",
                            global_batch=B_total, per_rank_batch=Bl, l2="inputs (GBs per rank) far larger than the 126 MB L2; no flush"),
                clocks=clocks, e2e=e2e, gpu_launches=launches * a.steps, device_status=status)

    if rank == 0:
        st = stage_times(inp, min(a.steps, 10), torch)
        peak, kind = peaks()
        alg = Bl * L * 128 * 2                       # the ik stream: every byte once
        ach = alg / (st["indexer_ms"] * 1e-3) / 1e9
        tr = ncu_traffic()
        line["roofline"] = dict(kernel="dsa indexer", bound="hbm", achieved=ach, peak=peak, unit="GB/s", frac=ach / peak,
                                peak_source=f"of {kind}", traffic=(tr["indexer_bytes_per_position"] * Bl * L if tr else None),
                                algorithmic_bytes=alg, launch_ms=st["indexer_ms"])
        total_alg = op.algorithmic_bytes(dict(B=Bl, L=L))
        line["stages_ms"] = st
        line["op_hbm"] = dict(algorithmic_bytes=total_alg, gbs=total_alg / (sec / a.steps) / 1e9,
                              frac=total_alg / (sec / a.steps) / 1e9 / peak)
        if not a.no_side and world == 1:
            del inp
            torch.cuda.empty_cache()
            line["ops"] = {c: side_line(c, torch, 10)
                           for c in ("prefix_small", "spec_chain", "spec_tree", "spec_tree_paged", "dsa_small", "prefix_sweep", "decode")}
        if not a.no_cpu and world == 1:
            n = 2
            t = cpu_sample(n, L)
            line["cpu_baseline"] = dict(value=n / t, unit=UNIT, cores=host_cores(), kind="port",
                                        sample=f"{n} of {B} requests (L={L}), float64 NumPy oracle, {t:.1f} s")
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
