"""vmk_spec_verify_noalloc: the entry point for hosts that may not allocate device memory around the
call (its scratch is a static array inside the library).  Called through the C ABI and compared with
vmk_spec_verify on the same inputs, twice in a row with different inputs, so that whatever the first
call left in the shared array is there when the second one runs.  Collected last on purpose."""
import numpy as np
import pytest
import torch

from oracle import judge, ref64
from verified_metal_kernels_b200 import _lib, ops

pytestmark = pytest.mark.gpu
SCRATCH = 32 << 20


def _run_pair(L, shape, seed, dist):
    op = ops.load_op("spec")
    host = op.make_inputs(shape, seed=seed, dist=dist)
    inp = ops.to_torch(host, "cuda")
    q, k, v, bits = inp["q"], inp["k"], inp["v"], inp["bits"]
    B, kd, Hq, D = q.shape
    Hkv, Lk = k.shape[1], k.shape[2]
    words = 1 if bits.dim() == 2 else bits.shape[2]
    st = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    need = L.vmk_spec_workspace_bytes(B, kd, Hq, Hkv, D, Lk)
    assert 0 < need <= SCRATCH
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    ref = torch.empty_like(q)
    rc = L.vmk_spec_verify(q.data_ptr(), k.data_ptr(), v.data_ptr(), bits.data_ptr(), words, ref.data_ptr(), B, kd, Hq, Hkv,
                           D, Lk, ws.data_ptr(), ws.numel(), status.data_ptr(), st)
    assert rc == 0, _lib.error_string(rc)
    out = torch.full_like(q, float("nan"))
    rc = L.vmk_spec_verify_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), bits.data_ptr(), words, out.data_ptr(), B, kd,
                                   Hq, Hkv, D, Lk, status.data_ptr(), st)
    assert rc == 0, _lib.error_string(rc)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # and directly against the float64 truth, with the acceptance criterion of the parity tests
    rep = judge.judge_l2(out.float().cpu().numpy(), ref64.spec_ref64(**host), half=True)
    assert rep["ok"], rep
    return out, ref


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    L = _lib.lib()
    # two different problems back to back: split partials (several splits) first, then a tree with wide rows
    out1, ref1 = _run_pair(L, dict(B=1, L=8192, k=8), 0, "chain")
    out2, ref2 = _run_pair(L, dict(B=2, L=3000, k=40, max_depth=8), 5, "randn")
    for out, ref in ((out1, ref1), (out2, ref2)):
        assert not torch.isnan(out).any()
        # same kernels, same plan, same summation order: the results are identical, which is well inside
        # the 1e-2 normalised tolerance the parity tests use
        assert torch.equal(out, ref)


def test_noalloc_refuses_shapes_beyond_its_static_buffer():
    L = _lib.lib()
    B, kd, Hq, Hkv, D, Lk = 64, 64, 32, 8, 128, 4096
    assert L.vmk_spec_workspace_bytes(B, kd, Hq, Hkv, D, Lk) > SCRATCH
    x = torch.zeros(16, dtype=torch.float16, device="cuda")      # never dereferenced: the size check comes first
    rc = L.vmk_spec_verify_noalloc(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 2, x.data_ptr(), B, kd, Hq, Hkv,
                                   D, Lk, None, None)
    assert rc == -6
    assert "static buffer" in _lib.error_string(rc)
