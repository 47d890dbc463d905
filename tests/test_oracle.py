"""The CPU oracle against the golden vectors produced by the reference's own Python code, and its internal
consistency (the properties the reference's quantization formulas imply)."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import int8_oracle as oracle
from tests import golden_cases
from wgpkernels_b200 import workloads

CASES = golden_cases.selftest_cases()


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.id)
def test_linear_reference_matches_reference_output(case):
    """oracle.linear_reference restates wgpkernels/int8/__init__.py:523-539: same PyTorch FP32 steps, so the same values."""
    y = oracle.linear_reference(case.x, case.w, case.scale, case.bias, case.group, case.act, case.act_weight, case.eps, case.residual,
                                case.residual_scale, case.path in ("lines", "small"))
    assert oracle.relative_error(y, case.ref) < 1e-6


def test_rotation_reference_matches_reference_output():
    x, outputs = golden_cases.rotation_vectors()
    for group, expected in outputs.items():
        assert torch.equal(oracle.rotate_reference(x, group), expected)
        # the in-kernel form (unnormalised digits, then 1 / sqrt(group)) is the same rotation
        mine = oracle.rotate_unnormalised(x.numpy(), group) * np.float32(group ** -0.5)
        assert oracle.relative_error(mine, expected) < 1e-6


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.id)
def test_path_restatement_within_selftest_bar(case):
    """The restated kernel arithmetic of every path passes the reference's own selftest bar against the reference output."""
    path = case.path.removesuffix("+g")
    y = oracle.linear(path, case.x, case.w, case.scale, case.bias, case.group, case.act, case.act_weight, case.eps, case.residual,
                      case.residual_scale)
    assert y.dtype == case.dtype
    assert oracle.relative_error(y, case.ref) < case.tolerance


def test_exact_path_within_two_tenths_of_a_percent():
    """The hi/lo split reproduces the FP32 dequantize-and-matmul within 0.2% even with outlier channels."""
    c = workloads.make("c0", rows=16)
    ref = oracle.linear_reference(c.x, c.weight, c.scale, c.bias)
    y = oracle.linear("exact", c.x, c.weight, c.scale, c.bias)
    assert oracle.relative_error(y, ref) < 2e-3
    # one INT8 pass with a scale per row is far worse on the same input; per-block scales sit between
    row = oracle.relative_error(oracle.linear("row", c.x, c.weight, c.scale, c.bias), ref)
    block = oracle.relative_error(oracle.linear("block", c.x, c.weight, c.scale, c.bias), ref)
    assert oracle.relative_error(y, ref) < block < row


def test_config0_matches_reference_output():
    """BASELINE config 0 (M=64, K=N=5120, seed 0): the seeded inputs are the ones the fixture was made from and the restated
    FP32 reference gives the reference's output."""
    golden = golden_cases.config0()
    c = workloads.make("c0")
    bits = lambda t: (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).contiguous().numpy().tobytes()
    digests = [hashlib.sha256(bits(t)).hexdigest() for t in (c.x, c.weight, c.scale, c.bias)]
    if digests != [str(d) for d in golden["digests"]]:
        pytest.skip("this PyTorch build draws different random numbers than the one the fixture was made with")
    y = oracle.linear_reference(c.x, c.weight, c.scale, c.bias)
    assert oracle.relative_error(y[:, :256], golden["y_slice"]) < 1e-6
    assert abs(float(y.double().norm()) - float(golden["y_norm"])) < 1e-6 * float(golden["y_norm"])
    block = oracle.linear("block", c.x, c.weight, c.scale, c.bias)
    assert oracle.relative_error(block[:, :256], golden["y_slice"]) < 3e-2


@pytest.mark.parametrize("act", [None, "rms_norm", "swiglu", "gelu"])
@pytest.mark.parametrize("group", [0, 64])
def test_block_quantizer_properties(act, group):
    g = torch.Generator().manual_seed(3)
    k = 384 + 8  # ragged last block
    k = 448 if group else k
    x = torch.randn(9, 2 * k if act == "swiglu" else k, generator=g).to(torch.bfloat16)
    x[3] = 0  # an all-zero row: scale 0, codes 0
    w = (torch.rand(k, generator=g) + 0.5).to(torch.bfloat16) if act == "rms_norm" else None
    q, scale = oracle.quantize_blocks(x, group, act, w, 1e-6)
    assert q.shape == (9, k) and scale.shape == (9, -(-k // 128))
    assert np.abs(q.astype(np.int32)).max() <= 127
    v = oracle.rotate_unnormalised(oracle.apply_act(x, act, w, 1e-6), group)
    for b in range(scale.shape[1]):
        block = v[:, b * 128:(b + 1) * 128]
        amax = np.abs(block).max(axis=1)
        assert np.array_equal(scale[:, b], (amax * oracle._norm_of(group)).astype(np.float32) / np.float32(127))
        assert np.all(np.abs(q[:, b * 128:(b + 1) * 128].astype(np.int32)).max(axis=1)[amax > 0] == 127)  # the maximum maps to +-127
        err = np.abs(block * oracle._norm_of(group) - q[:, b * 128:(b + 1) * 128] * scale[:, b:b + 1])
        assert np.all(err <= scale[:, b:b + 1] * 0.5001)
    assert not q[3].any() and not scale[3].any()


def test_hilo_reconstruction_error():
    """x ~= scale * (hi + lo / 254) to within scale / 508 (half a step of the low part)."""
    g = torch.Generator().manual_seed(4)
    x = torch.randn(5, 1024, generator=g).to(torch.bfloat16)
    hi, lo, scale = oracle.quantize_rows(x, 0, True)
    v = oracle.to_f32(x).astype(np.float64)
    rebuilt = scale[:, None].astype(np.float64) * (hi.astype(np.float64) + lo.astype(np.float64) / 254)
    assert np.all(np.abs(rebuilt - v) <= scale[:, None] / 508 * 1.001)
    assert np.abs(lo.astype(np.int32)).max() <= 127


def test_rms_tree_is_a_sum_of_squares():
    g = torch.Generator().manual_seed(5)
    for k in (256, 5120, 20000):
        x = torch.randn(3, k, generator=g).numpy()
        ss = oracle.rms_sum_squares(x)
        exact = (x.astype(np.float64) ** 2).sum(axis=1)
        assert np.all(np.abs(ss - exact) < 1e-5 * exact)


def test_block_sums_are_exact_integers():
    g = torch.Generator().manual_seed(6)
    a = torch.randint(-127, 128, (17, 320), dtype=torch.int8, generator=g).numpy()
    w = torch.randint(-127, 128, (24, 320), dtype=torch.int8, generator=g).numpy()
    s = oracle.block_sums(a, w)
    assert s.shape == (3, 17, 24)
    for b in range(3):
        expected = a[:, b * 128:(b + 1) * 128].astype(np.int64) @ w[:, b * 128:(b + 1) * 128].astype(np.int64).T
        assert np.array_equal(s[b], expected)
    assert np.array_equal(s.sum(axis=0), oracle.full_sums(a, w))
