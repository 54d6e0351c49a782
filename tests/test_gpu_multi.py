"""Multi-GPU paths on real GPUs (skipped with fewer than two): request / batch sharding needs no exchange; the
hybrid `prefix` sharding and the `spec` cache split exchange packed (m, l, o) records through NCCL once and merge
locally.  Each rank is a child process; NVLS is off."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["VMK_ROOT"])
from oracle import judge, ref64
from verified_metal_kernels_b200 import load_kernel, ops, shard
rank, local, world = shard.world()
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
try:
    # 1. prefix, hybrid sharding: suffixes by request, the shared prefix by kv head and then by key range, ONE
    #    all-to-all of packed (m, l, o) records, local merge.  Small (warp-level kernels) and with 40 requests x 4
    #    heads = 160 stacked rows (tcgen05 kernel); ragged suffixes, one of them empty; the suffix pass also on a
    #    side stream.  Every rank judges the outputs of its own requests against float64.
    op = ops.load_op("prefix")
    side = torch.cuda.Stream()
    for shape, seed in ((dict(N=6, P=5000, S=130, ragged=True), 5), (dict(N=40, P=3000, S=200, ragged=True), 8)):
        inp = op.make_inputs(shape, seed=seed)
        inp["slens"][1] = 0
        truth = ref64.prefix_ref64(**inp)
        d = ops.to_torch(ops.cand_inputs("prefix", inp), "cuda")
        N, Hq = d["q"].shape[0], d["q"].shape[1]
        Hkv, P = d["kp"].shape[0], d["kp"].shape[1]
        for mode, ss in (("head", None), ("key", None), ("head", side)):
            plan = shard.PrefixHybridPlan(N, Hq, Hkv, P, world, mode=mode)
            lo, hi = plan.req[rank]
            out = shard.prefix_hybrid(d["q"], plan.prefix_slice(d["kp"], rank), plan.prefix_slice(d["vp"], rank),
                                      d["ks"][lo:hi], d["vs"][lo:hi], d["slens"][lo:hi], plan, side_stream=ss, check=True)
            assert tuple(out.shape) == (hi - lo, Hq, 128)
            rep = judge.judge_l2(out.float().cpu().numpy(), truth[lo:hi], half=True)
            assert rep["ok"], (shape, mode, rep)
    # 2a. spec: one long cache split by position over all ranks, one all-gather, everyone gets everything
    op = ops.load_op("spec")
    inp = op.make_inputs(dict(B=1, L=20000, k=8), seed=6)
    d = ops.to_torch(ops.cand_inputs("spec", inp), "cuda")
    out = shard.spec_kv_split(d["q"], d["k"], d["v"], d["bits"])
    rep = judge.judge_l2(out.float().cpu().numpy(), ref64.spec_ref64(**inp), half=True)
    assert rep["ok"], rep
    # 2b. spec with more ranks than batch elements: the element's cache split inside its group of ranks, each rank
    #     holding only its slice, one all-to-all, each member left with its share of the merged rows (wide masks)
    inp = op.make_inputs(dict(B=1, L=9000, k=40, max_depth=8), seed=9)
    truth = ref64.spec_ref64(**inp)[0].reshape(40 * 32, 128)
    d = ops.to_torch(ops.cand_inputs("spec", inp), "cuda")
    plan = shard.SpecSplitPlan(1, 40 * 32, 9000, world)
    lo, hi = plan.keys[rank]
    out, (r0, r1) = shard.spec_split(d["q"], d["k"][:, :, lo:hi].contiguous(), d["v"][:, :, lo:hi].contiguous(), d["bits"],
                                     plan, check=True)
    rep = judge.judge_l2(out.float().cpu().numpy(), truth[r0:r1], half=True)
    assert rep["ok"], rep
    # 3. dsa sharded by batch element: every rank checks its own slice, no collective on the data path
    op = ops.load_op("dsa")
    inp = op.make_inputs(dict(B=3, L=5003), seed=7)
    mine, (lo, hi) = shard.shard_inputs("dsa", inp, rank, world)
    if hi > lo:
        out = load_kernel("dsa")(**ops.to_torch(ops.cand_inputs("dsa", mine), "cuda"))
        t = ref64.dsa_ref64(**{k: inp[k] for k in ("q", "kv", "iq", "ik", "w")})[lo:hi]
        rep = judge.judge_l2(out.float().cpu().numpy(), t, half=True)
        assert rep["ok"], rep
    torch.cuda.synchronize()
    dist.barrier()
    print(f"rank {rank} ok")
finally:
    dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_kv_split_and_batch_sharding_two_ranks(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, VMK_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)], env=env,
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-3000:]
    assert "rank 0 ok" in p.stdout and "rank 1 ok" in p.stdout
