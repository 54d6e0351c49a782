"""Host logic of the multi-GPU path on CPU: unit / key partitioning, and the (m, l, o) exchange + merge
run as two Gloo ranks whose partials come from the float64 oracle restricted to each rank's keys."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from verified_metal_kernels_b200 import ops, shard


def test_unit_range_partitions_everything():
    for n in (0, 1, 4, 7, 128, 129):
        for w in (1, 2, 3, 8):
            spans = [shard.unit_range(n, r, w) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def test_key_range_is_block_aligned():
    for n in (1, 63, 64, 65, 4097, 32768):
        for w in (1, 2, 8):
            spans = [shard.key_range(n, r, w) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(lo % 64 == 0 or lo == n for lo, _ in spans)


def test_shard_inputs_views():
    op = ops.load_op("prefix")
    inp = op.make_inputs(dict(N=5, P=16, S=4, ragged=True), seed=0)
    parts = [shard.shard_inputs("prefix", inp, r, 2) for r in range(2)]
    assert [p[1] for p in parts] == [(0, 3), (3, 5)]
    assert parts[1][0]["q"].shape[0] == 2 and parts[1][0]["kp"] is inp["kp"]
    assert np.array_equal(np.concatenate([p[0]["slens"] for p in parts]), inp["slens"])
    dsa = ops.load_op("dsa").make_inputs(dict(B=3, L=8), seed=0)
    d0, span = shard.shard_inputs("dsa", dsa, 1, 2)
    assert span == (2, 3) and d0["kv"].shape[0] == 1 and d0["lens"] is None


def _partial64(q, k, v, lo, hi, allowed=None):
    """Un-normalised (m, l, o) of softmax(q k^T / sqrt(d)) v over keys [lo, hi), m in the base-2 domain."""
    d = q.shape[-1]
    s = (q @ k[lo:hi].T) / np.sqrt(d) * np.log2(np.e)
    if allowed is not None:
        s = np.where(allowed[:, lo:hi], s, -np.inf)
    if hi == lo:
        return np.full(q.shape[0], -np.inf), np.zeros(q.shape[0]), np.zeros_like(q)
    m = s.max(-1)
    mu = np.where(np.isinf(m), 0.0, m)
    p = np.exp2(s - mu[:, None])
    return m, p.sum(-1), p @ v[lo:hi]


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)                      # same data on every rank
        rows, keys, d = 12, 300, 128
        q, k, v = rng.standard_normal((rows, d)), rng.standard_normal((keys, d)), rng.standard_normal((keys, d))
        allowed = rng.random((rows, keys)) > 0.2
        allowed[:, 0] = True
        lo, hi = shard.key_range(keys, rank, world)
        m, l, o = _partial64(q, k, v, lo, hi, allowed)
        gm, gl, go = shard.gather_partials(torch.from_numpy(m), torch.from_numpy(l), torch.from_numpy(o))
        out = shard.merge_partials_reference(gm, gl, go).numpy()
        s = np.where(allowed, (q @ k.T) / np.sqrt(d), -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        ref = (p / p.sum(-1, keepdims=True)) @ v
        np.save(os.path.join(tmp, f"err{rank}.npy"), np.abs(out - ref).max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_partial_exchange_and_merge_gloo(tmp_path, world):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert float(np.load(tmp_path / f"err{r}.npy")) < 1e-12


def _worker_missing_rank(rank, world, port, tmp):
    """Rank 1 never joins the collective: rank 0 must get an error from the process-group timeout."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    if rank == 1:
        return                                            # leaves between steps, nothing in flight
    t = torch.zeros(4)
    try:
        shard.gather_partials(t, t.clone(), torch.zeros(4, 2))
        open(os.path.join(tmp, "unexpected_success"), "w").close()
    except Exception as e:
        open(os.path.join(tmp, "failed_as_expected"), "w").write(type(e).__name__)


def test_missing_rank_surfaces_as_error(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker_missing_rank, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "failed_as_expected").exists() and not (tmp_path / "unexpected_success").exists()
