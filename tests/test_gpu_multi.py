"""Multi-GPU paths on real GPUs (skipped with fewer than two): request sharding needs no exchange; the
KV split exchanges (m, l, o) through NCCL and merges locally.  Each rank is a child process."""
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
    # 1. prefix with the shared prefix split by position across ranks
    op = ops.load_op("prefix")
    inp = op.make_inputs(dict(N=6, P=5000, S=130), seed=5)
    d = ops.to_torch(ops.cand_inputs("prefix", inp), "cuda")
    out = shard.prefix_kv_split(d["q"], d["kp"], d["vp"], d["ks"], d["vs"])
    rep = judge.judge_l2(out.float().cpu().numpy(), ref64.prefix_ref64(**inp), half=True)
    assert rep["ok"], rep
    # 2. spec: one long cache split by position
    op = ops.load_op("spec")
    inp = op.make_inputs(dict(B=1, L=20000, k=8), seed=6)
    d = ops.to_torch(ops.cand_inputs("spec", inp), "cuda")
    out = shard.spec_kv_split(d["q"], d["k"], d["v"], d["bits"])
    rep = judge.judge_l2(out.float().cpu().numpy(), ref64.spec_ref64(**inp), half=True)
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
