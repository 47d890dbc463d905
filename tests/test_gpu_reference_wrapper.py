"""Acceptance test of the drop-in boundary: the reference's OWN, unmodified Python module (wgpkernels/int8/__init__.py of WGPKernels,
placed under oracle/_ref/ by oracle/Makefile) loads this repository's library through its ctypes table (:66-95), passes its own
known-answer test (:542-576) on it, and its linear() gives what this repository's module gives."""
import sys
from pathlib import Path

import pytest
import torch

from wgpkernels_b200 import build as builder
from wgpkernels_b200 import workloads

pytestmark = pytest.mark.gpu
REF_ROOT = Path(__file__).resolve().parents[1] / "oracle" / "_ref"


@pytest.fixture(scope="module")
def reference_module(tmp_path_factory):
    if not (REF_ROOT / "wgpkernels" / "int8" / "__init__.py").exists():
        pytest.skip("the reference's Python wrapper was not placed under oracle/_ref (no reference checkout at build time)")
    sys.path.insert(0, str(REF_ROOT))
    try:
        from wgpkernels import int8 as reference_wq  # the reference's module, byte for byte
    finally:
        sys.path.remove(str(REF_ROOT))
    reference_wq.load_library(builder.library_file())
    return reference_wq


def test_reference_selftest_passes_on_this_library(reference_module):
    assert reference_module.weight_groups_supported()
    assert reference_module.selftest() is None


def test_reference_linear_matches_this_module(reference_module, wq):
    """linear() of the reference's module on this library, on bands of the benchmark configurations (its own path policy and tile tuner
    run: every variant number it may pick must be served), against this repository's module on the same tensors."""
    for name, rows, mode in (("c1", 700, "block"), ("c2", 300, "block"), ("c4", 520, "block"), ("c1", 300, "exact"), ("c0", 40, None)):
        c = workloads.make(name, rows=rows).to(torch.device("cuda", 0))
        kwargs = dict(act=c.act, act_weight=c.act_weight, eps=c.eps)
        residual = None if c.residual is None else c.residual.clone()
        got = reference_module.linear(c.x, c.weight, c.scale, c.bias, mode=mode, residual=residual, residual_scale=c.residual_scale, **kwargs)
        path = mode or reference_module.choose_path(c.x, c.weight, c.scale, c.bias, **kwargs)
        expected = wq.linear(c.x, c.weight, c.scale, c.bias, mode=path, residual=c.residual, residual_scale=c.residual_scale, **kwargs)
        torch.cuda.synchronize()
        error = float((got.float() - expected.float()).norm() / expected.float().norm())
        assert error < 1e-3, (name, path, error)
    assert wq.debug_status() == 0
