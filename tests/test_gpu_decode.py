"""Plain single-token decode (extension op) on the GPU through the C ABI against the float64 oracle: ragged
lengths, NaN beyond the lengths, bf16, and the paged form bit for bit against the contiguous one."""
import numpy as np
import pytest
import torch

from oracle import judge, ref64
from tests import _verify
from verified_metal_kernels_b200 import ops
from verified_metal_kernels_b200.kernels import decode_b200
from verified_metal_kernels_b200.ops import decode as op

pytestmark = pytest.mark.gpu


def _dev(inp, bf16=False):
    d = {k: torch.from_numpy(v).cuda() for k, v in inp.items()}
    if bf16:
        for k in ("q", "k", "v"):
            d[k] = d[k].to(torch.bfloat16)
    return d


@pytest.mark.parametrize("shape,dist", op.FUZZ, ids=lambda x: str(x))
def test_decode_against_the_oracle(shape, dist):
    inp = op.make_inputs(shape, seed=41, dist=dist)
    out = decode_b200.kernel(**_dev(inp))
    torch.cuda.synchronize()
    _verify.assert_clean_status()
    truth = ref64.decode_ref64(**inp)
    rep = judge.judge_l2(out.float().cpu().numpy(), truth, half=True)
    assert rep["ok"] and rep["err_max"] <= 2e-3, rep


@pytest.mark.parametrize("page_size", [64, 256])
def test_decode_paged_equals_contiguous_bit_for_bit(page_size):
    inp = op.make_inputs(dict(B=6, L=2500), seed=43, dist="ragged")
    d = _dev(inp)
    ref = decode_b200.kernel(**d)
    kp, vp, table = op.to_pages(inp["k"], inp["v"], inp["lens"], page_size, seed=2)
    out = decode_b200.kernel_paged(d["q"], torch.from_numpy(kp).cuda(), torch.from_numpy(vp).cuda(),
                                   torch.from_numpy(table).cuda(), d["lens"])
    torch.cuda.synchronize()
    _verify.assert_clean_status()
    assert torch.equal(out, ref)


def test_decode_bf16():
    inp = op.make_inputs(dict(B=4, L=3000), seed=47, dist="ragged")
    for k in ("q", "k", "v"):
        inp[k] = ops.round_bf16(inp[k])
    out = decode_b200.kernel(**_dev(inp, bf16=True))
    torch.cuda.synchronize()
    assert out.dtype == torch.bfloat16
    rep = judge.judge_l2(out.float().cpu().numpy(), ref64.decode_ref64(**inp), half=True)
    assert rep["ok"] and rep["err_max"] <= 6e-3, rep


def test_decode_equals_spec_with_one_unmasked_draft():
    """With full lengths the op is `spec` with k = 1: same kernel, same bits."""
    from verified_metal_kernels_b200.kernels import spec_b200
    inp = op.make_inputs(dict(B=3, L=1800), seed=53)
    d = _dev(inp)
    out = decode_b200.kernel(**d)
    bits = torch.ones(3, 1, dtype=torch.int32, device="cuda")
    ref = spec_b200.kernel(d["q"].unsqueeze(1).contiguous(), d["k"], d["v"], bits)
    assert torch.equal(out, ref[:, 0])
