"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, and answers
the host-only entry points (sizes, error strings, argument validation that precedes any launch)."""
import ctypes
import os
import re

import pytest

from verified_metal_kernels_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.lib()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "vmk_b200.h")).read()
    return sorted(set(re.findall(r"VMK_API[^;]*?\b(vmk_\w+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    syms = header_symbols()
    assert len(syms) >= 14
    assert sorted(_lib.SIGNATURES) == syms
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for s in syms:
        assert hasattr(raw, s), f"{s} declared in include/vmk_b200.h but not exported"


def test_nothing_is_exported_that_the_header_does_not_declare(lib):
    """Every dynamic symbol named vmk_* is declared in the header, except the trace readers of debug builds."""
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = {ln.split()[-1] for ln in out.splitlines() if ln.split() and ln.split()[-1].startswith("vmk_")}
    assert exported, "no vmk_* symbol found in the dynamic symbol table"
    extra = exported - set(header_symbols()) - set(_lib.DEBUG_EXPORTS)
    assert not extra, f"exported but not declared in include/vmk_b200.h: {sorted(extra)}"


def test_every_declaration_cites_the_reference():
    text = open(os.path.join(ROOT, "include", "vmk_b200.h")).read()
    assert text.count("kernels/") >= 6 and "verify.py:" in text


def test_version_and_error_strings(lib):
    assert lib.vmk_version() >= 100
    seen = {_lib.error_string(c) for c in (0, -1, -2, -3, -4, -5)}
    assert len(seen) == 6 and "unknown" not in " ".join(seen)
    assert "unknown" in _lib.error_string(-99)


def test_workspace_sizes(lib):
    assert lib.vmk_prefix_workspace_bytes(8, 32, 8, 128, 4096, 256) > 0
    assert lib.vmk_prefix_workspace_bytes(8, 32, 8, 64, 4096, 256) == 0       # D != 128
    assert lib.vmk_prefix_workspace_bytes(8, 32, 7, 128, 4096, 256) == 0       # Hq % Hkv
    assert lib.vmk_spec_workspace_bytes(4, 64, 32, 8, 128, 32768) > 0
    a, b = lib.vmk_dsa_workspace_bytes(8, 32768), lib.vmk_dsa_workspace_bytes(8, 65536)
    assert b - a == 8 * 32768 * 4                                               # fp32 scores grow with L
    assert lib.vmk_dsa_workspace_bytes(0, 10) == 0
    big = lib.vmk_prefix_workspace_bytes(256, 32, 8, 128, 32768, 2048)
    assert 0 < big < 2 << 30


def test_bad_arguments_are_rejected_before_any_launch(lib):
    assert lib.vmk_prefix_decode(None, None, None, None, None, None, None, 1, 32, 8, 128, 8, 8, None, 0, None, None) == -1
    assert lib.vmk_spec_verify(None, None, None, None, 1, None, 1, 4, 32, 8, 128, 64, None, 0, None, None) == -1
    assert lib.vmk_dsa_decode(None, None, None, None, None, None, None, None, None, 1, 64, None, 0, None, None) == -1
    assert lib.vmk_dsa_select(None, None, None, None, 1, 64, None) == -1
    assert lib.vmk_lse_merge(None, None, None, 2, 4, 128, None, None) == -1
    assert lib.vmk_lse_merge_packed(None, 2, 4, 128, 0, None, None) == -1
    assert lib.vmk_lse_merge_packed(256, 2, 4, 64, 0, 256, None) == -2             # D != 128
    assert lib.vmk_prefix_partial_packed(None, 32, None, None, None, None, None, 1, 32, 8, 128, 8, 8, 0, 8, 1, 0, None,
                                         None, 0, None, None) == -1
    # a slice of heads wider than the tensor it is cut from
    assert lib.vmk_prefix_partial_packed(256, 4, 256, 256, 256, 256, None, 1, 8, 2, 128, 8, 8, 0, 8, 1, 0, 256,
                                         256, 1 << 20, None, None) == -1
    assert lib.vmk_spec_partial_packed(None, None, None, None, 1, 1, 4, 32, 8, 128, 64, 0, 64, -1, 0, None, None, 0,
                                       None, None) == -1
    # misaligned pointer
    assert lib.vmk_prefix_decode(8, 16, 16, 16, 16, None, 16, 1, 32, 8, 128, 8, 8, 256, 1 << 20, None, None) == -1
    # dsa: a bad LATE argument (the output pointer of stage 3) is refused before stage 1 enqueues anything -- here,
    # without a GPU, an enqueue would come back as a launch failure (-4) instead
    assert lib.vmk_dsa_decode(256, 256, 256, 256, 256, None, 8, None, None, 2, 4096, 256, 1 << 30, None, None) == -1
    assert lib.vmk_dsa_decode(256, 256, 256, 256, 256, None, None, None, None, 2, 4096, 256, 1 << 30, None, None) == -1
    assert lib.vmk_dsa_indexer_hist(256, 256, 256, None, 256, 256, 0, 4096, None, None) == -1          # B = 0
    assert lib.vmk_dsa_indexer_hist(256, 256, 256, None, 256, 256, 70000, 4096, None, None) == -1      # B > 65535


def test_kernel_modules_refuse_cpu_only_use():
    import numpy as np
    import torch
    from verified_metal_kernels_b200 import load_kernel, ops
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    inp = ops.load_op("spec").make_inputs(dict(B=1, L=16, k=2), seed=0)
    with pytest.raises((RuntimeError, ValueError, AssertionError)):
        load_kernel("spec")(**ops.to_torch(inp, "cpu"))


def test_build_is_keyed_by_content_not_by_file_times(monkeypatch):
    """A copy of the tree to another machine does not keep file times, and one rank per GPU may call the build
    at the same moment: the library is rebuilt only when the hash of its sources and flags differs from the
    stamp written beside it, under a file lock."""
    from verified_metal_kernels_b200 import build
    build.build()
    assert os.path.exists(build.LIB + ".stamp")
    assert not build.needs_build()
    os.utime(build.deps()[0])                                  # a newer source file alone is not a reason
    assert not build.needs_build()
    monkeypatch.setenv("VMK_EXTRA_NVCC_FLAGS", "-DVMK_SOME_FLAG")
    assert build.needs_build()                                 # other flags are


def test_variant_switches_refuse_unknown_values(lib):
    """The process-wide switches are host-side state: unknown values are refused and change nothing."""
    assert lib.vmk_dsa_set_attend_variant(7) == -1 and lib.vmk_dsa_set_attend_variant(-1) == -1
    assert lib.vmk_dsa_set_select_cluster(3) == -1 and lib.vmk_dsa_set_select_cluster(16) == -1
    for v in (0, 1, 2, 3):
        assert lib.vmk_dsa_set_attend_variant(v) == 0
    for c in (1, 2, 4, 8, 0):
        assert lib.vmk_dsa_set_select_cluster(c) == 0
    assert lib.vmk_dsa_set_attend_variant(3) == 0          # back to the defaults
