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


class NumpyPartials:
    """The `compute` object of shard.prefix_hybrid / shard.spec_split in float64 NumPy: the same records the CUDA
    entry points produce (m in the base-2 scaled-score domain), so the exchange and merge logic runs on CPU."""

    def empty(self, shape, like):
        return torch.empty(shape, dtype=torch.float64)

    @staticmethod
    def _rec(q, k, v, allowed=None):
        m, l, o = _partial64(q, k, v, 0, k.shape[0], allowed)
        return np.concatenate([m[:, None], l[:, None], o], axis=1)

    def prefix_records(self, q_all, kp, vp, h0):
        q, kp, vp = q_all.numpy(), kp.numpy(), vp.numpy()
        N, G = q.shape[0], self.G
        hq_cov = kp.shape[0] * G
        rec = np.empty((N, hq_cov, shard.RECORD))
        for j in range(kp.shape[0]):
            rows = q[:, (h0 + j) * G:(h0 + j + 1) * G].reshape(N * G, -1)
            rec[:, j * G:(j + 1) * G] = self._rec(rows, kp[j], vp[j]).reshape(N, G, shard.RECORD)
        return torch.from_numpy(rec.reshape(N * hq_cov, shard.RECORD))

    def suffix_records(self, q_loc, ks, vs, slens, out):
        q, ks, vs = q_loc.numpy(), ks.numpy(), vs.numpy()
        n, Hq, G = q.shape[0], q.shape[1], self.G
        rec = np.empty((n, Hq, shard.RECORD))
        for i in range(n):
            sl = ks.shape[2] if slens is None else int(slens[i])
            for h in range(ks.shape[1]):
                rec[i, h * G:(h + 1) * G] = self._rec(q[i, h * G:(h + 1) * G], ks[i, h, :sl], vs[i, h, :sl])
        out.copy_(torch.from_numpy(rec.reshape(n * Hq, shard.RECORD)))

    def spec_records(self, q, k, v, bits, has_drafts):
        from oracle import ref64
        q, k, v = q.numpy(), k.numpy(), v.numpy()
        B, kd, Hq, d = q.shape
        Hkv, Ls = k.shape[1], k.shape[2]
        G = Hq // Hkv
        allowed = ref64.spec_allowed(bits.numpy(), Ls, kd) if has_drafts else np.ones((B, kd, Ls), dtype=bool)
        rec = np.empty((B, kd, Hq, shard.RECORD))
        for b in range(B):
            for h in range(Hkv):
                rows = q[b, :, h * G:(h + 1) * G].reshape(kd * G, d)
                r = self._rec(rows, k[b, h], v[b, h], np.repeat(allowed[b], G, axis=0))
                rec[b, :, h * G:(h + 1) * G] = r.reshape(kd, G, shard.RECORD)
        return torch.from_numpy(rec.reshape(B * kd * Hq, shard.RECORD))

    def merge(self, buf):
        return shard.merge_records_reference(buf)


def _worker_prefix_hybrid(rank, world, port, tmp, mode):
    """Suffixes by request, the shared prefix by kv head (mode 'head') or by key range ('key'), one all-to-all of
    packed records, local merge: every rank's outputs for its own requests against the float64 oracle."""
    from oracle import ref64
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        op = ops.load_op("prefix")
        inp = op.make_inputs(dict(N=7, P=330, S=40, ragged=True), seed=3)       # same data on every rank
        inp["slens"][2] = 0                                                        # a request without a suffix
        truth = ref64.prefix_ref64(**inp)
        f64 = {k: torch.from_numpy(np.asarray(v, dtype=np.float64)) for k, v in inp.items() if k != "slens"}
        N, Hq = inp["q"].shape[0], inp["q"].shape[1]
        Hkv, P = inp["kp"].shape[0], inp["kp"].shape[1]
        plan = shard.PrefixHybridPlan(N, Hq, Hkv, P, world, mode=mode)
        assert plan.mode == mode and plan.parts() == (2 if mode == "head" else world + 1)
        lo, hi = plan.req[rank]
        out = shard.prefix_hybrid(f64["q"], plan.prefix_slice(f64["kp"], rank), plan.prefix_slice(f64["vp"], rank),
                                  f64["ks"][lo:hi], f64["vs"][lo:hi], inp["slens"][lo:hi], plan,
                                  compute=NumpyPartials())
        err = np.abs(out.numpy() - truth[lo:hi]).max() if hi > lo else 0.0
        # what each rank reads adds up to the op's algorithmic input bytes (+ the replicated queries)
        total = sum(plan.bytes_read(r, inp["slens"], 40) for r in range(world))
        alg = 2 * Hkv * P * 128 * 2 + 2 * Hkv * 128 * 2 * int(inp["slens"].sum()) + world * N * Hq * 128 * 2
        assert total == alg, (total, alg)
        np.save(os.path.join(tmp, f"err{rank}.npy"), err)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,mode", [(2, "head"), (4, "head"), (2, "key"), (3, "key")])
def test_prefix_hybrid_gloo(tmp_path, world, mode):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker_prefix_hybrid, args=(world, port, str(tmp_path), mode), nprocs=world, join=True)
    for r in range(world):
        assert float(np.load(tmp_path / f"err{r}.npy")) < 1e-12


def _worker_spec_split(rank, world, port, tmp, B):
    """More ranks than batch elements: every element's cache split by position over a group of ranks, one
    all-to-all inside the group, each member left with the merged result of its share of the rows."""
    from oracle import ref64
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        op = ops.load_op("spec")
        kd, L = 6, 300
        inp = op.make_inputs(dict(B=B, L=L, k=kd), seed=4)                # random tree masks
        truth = ref64.spec_ref64(**inp)
        Hq = inp["q"].shape[2]
        plan = shard.SpecSplitPlan(B, kd * Hq, L, world)
        assert plan.split
        b = plan.elem[rank]
        lo, hi = plan.keys[rank]
        t = lambda a: torch.from_numpy(np.asarray(a, dtype=np.float64))
        out, (r0, r1) = shard.spec_split(t(inp["q"][b:b + 1]), t(inp["k"][b:b + 1, :, lo:hi]), t(inp["v"][b:b + 1, :, lo:hi]),
                                         torch.from_numpy(inp["bits"][b:b + 1]), plan, compute=NumpyPartials())
        ref = truth[b].reshape(kd * Hq, -1)[r0:r1]
        np.save(os.path.join(tmp, f"err{rank}.npy"), np.abs(out.numpy() - ref).max() if r1 > r0 else 0.0)
        # the members of a group cover the cache and the rows exactly once
        grp = plan.members[b]
        assert [plan.keys[g] for g in grp][0][0] == 0 and [plan.keys[g] for g in grp][-1][1] == L
        assert sum(plan.own_rows[g][1] - plan.own_rows[g][0] for g in grp) == kd * Hq
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,B", [(2, 1), (4, 2), (3, 1)])
def test_spec_split_gloo(tmp_path, world, B):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker_spec_split, args=(world, port, str(tmp_path), B), nprocs=world, join=True)
    for r in range(world):
        assert float(np.load(tmp_path / f"err{r}.npy")) < 1e-12


def test_spec_split_plan_without_split():
    plan = shard.SpecSplitPlan(4, 64 * 32, 32768, 2)
    assert not plan.split and plan.elems == [(0, 2), (2, 4)]
    plan = shard.SpecSplitPlan(4, 64 * 32, 32768, 8)
    assert plan.split and plan.members[1] == [2, 3] and plan.keys[3] == (16384, 32768) and plan.has_drafts(3)
    assert not plan.has_drafts(2) and plan.own_rows[2] == (0, 1024) and plan.own_rows[3] == (1024, 2048)
    assert plan.send_rows(2) == [0, 0, 1024, 1024, 0, 0, 0, 0] and plan.recv_rows(3) == [0, 0, 1024, 1024, 0, 0, 0, 0]


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
