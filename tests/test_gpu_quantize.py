"""Activation preparation kernels on the GPU: bit-exact against the reference's own CUDA library, and against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import int8_oracle as oracle
from tests import reflib
from tests.gpu_common import codes_close, randn

pytestmark = pytest.mark.gpu
ACTS = [None, "rms_norm", "swiglu", "gelu"]
# (M, K): ragged last block, register-resident rows of every size class, and a row longer than the register kernels hold
SHAPES = [(1, 8), (7, 264), (33, 2048), (5, 5120), (130, 1024 + 128 + 8), (3, 13824), (2, 16384 + 512)]


def make_x(m, k, act, dtype, seed):
    x = randn((m, 2 * k if act == "swiglu" else k), dtype, seed, 1.5)
    if m > 2:
        x[1] = 0  # an all-zero row
        x[2, ::7] *= 40  # outliers
    return x


def weight_of(k, act, dtype, seed):
    return (randn((k,), torch.float32, seed) * 0.1 + 1).to(dtype) if act == "rms_norm" else None


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
def test_quantize_blocks_matches_reference_library(wq, shape, act, dtype):
    m, k = shape
    x = make_x(m, k, act, dtype, 11).cuda()
    w = weight_of(k, act, dtype, 12)
    w = None if w is None else w.cuda()
    q, s = wq.quantize_blocks(x, 0, act, w, 1e-6)
    q_ref, s_ref = reflib.quantize_blocks(x, 0, act, w, 1e-6)
    assert torch.equal(q, q_ref)
    assert torch.equal(s, s_ref)


@pytest.mark.parametrize("group", [16, 64, 256])
@pytest.mark.parametrize("act", [None, "rms_norm", "gelu"])
def test_quantize_blocks_rotated_matches_reference_library(wq, group, act):
    m, k = 9, 1024 + 256
    x = make_x(m, k, act, torch.bfloat16, 13).cuda()
    w = weight_of(k, act, torch.bfloat16, 14)
    w = None if w is None else w.cuda()
    q, s = wq.quantize_blocks(x, group, act, w, 1e-6)
    q_ref, s_ref = reflib.quantize_blocks(x, group, act, w, 1e-6)
    assert torch.equal(q, q_ref) and torch.equal(s, s_ref)


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("shape", [(7, 264), (5, 5120), (2, 16384 + 512)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_quantize_blocks_matches_oracle(wq, shape, act):
    m, k = shape
    x = make_x(m, k, act, torch.bfloat16, 15)
    w = weight_of(k, act, torch.bfloat16, 16)
    q, s = wq.quantize_blocks(x.cuda(), 0, act, None if w is None else w.cuda(), 1e-6)
    q_cpu, s_cpu = oracle.quantize_blocks(x, 0, act, w, 1e-6)
    if act in (None, "rms_norm"):  # IEEE operations only: identical
        assert codes_close(q, q_cpu, 1e-5)
        assert np.allclose(s.cpu().numpy(), s_cpu, rtol=3e-7, atol=0)
    else:  # expf / tanhf of the CUDA math library vs the host's
        assert codes_close(q, q_cpu, 2e-3)
        assert np.allclose(s.cpu().numpy(), s_cpu, rtol=2e-6, atol=0)


@pytest.mark.parametrize("hilo", [False, True])
@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("shape", [(1, 8), (7, 264), (5, 5120), (3, 13824), (2, 16384 + 512)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_quantize_rows_matches_reference_library(wq, shape, act, hilo):
    m, k = shape
    x = make_x(m, k, act, torch.bfloat16, 17).cuda()
    w = weight_of(k, act, torch.bfloat16, 18)
    w = None if w is None else w.cuda()
    hi, lo, s = wq.quantize(x, 0, hilo, act, w, 1e-6)
    hi_ref, lo_ref, s_ref = reflib.quantize(x, 0, hilo, act, w, 1e-6)
    assert torch.equal(hi, hi_ref) and torch.equal(s, s_ref)
    assert (lo is None) == (not hilo)
    if hilo:
        assert torch.equal(lo, lo_ref)


def test_quantize_rows_matches_oracle(wq):
    x = make_x(6, 3072, None, torch.bfloat16, 19)
    hi, lo, s = wq.quantize(x.cuda(), 0, True)
    hi_cpu, lo_cpu, s_cpu = oracle.quantize_rows(x, 0, True)
    assert np.array_equal(hi.cpu().numpy(), hi_cpu) and np.array_equal(lo.cpu().numpy(), lo_cpu)
    assert np.array_equal(s.cpu().numpy(), s_cpu)


def test_quantize_fp32_input(wq):
    x = randn((5, 520), torch.float32, 20).cuda()
    q, s = wq.quantize_blocks(x)
    q_ref, s_ref = reflib.quantize_blocks(x)
    assert torch.equal(q, q_ref) and torch.equal(s, s_ref)
    hi, lo, s = wq.quantize(x, 0, True)
    hi_ref, lo_ref, s_ref = reflib.quantize(x, 0, True)
    assert torch.equal(hi, hi_ref) and torch.equal(lo, lo_ref) and torch.equal(s, s_ref)


def test_strided_rows(wq):
    """Rows may be a column slice of a wider tensor (row stride larger than K)."""
    wide = randn((9, 1024), torch.bfloat16, 21).cuda()
    x = wide[:, 256:768]
    q, s = wq.quantize_blocks(x)
    q2, s2 = wq.quantize_blocks(x.contiguous())
    assert torch.equal(q, q2) and torch.equal(s, s2)


@pytest.mark.parametrize("group", [0, 16, 64, 256])
@pytest.mark.parametrize("act", ACTS)
def test_transform_rows_matches_reference_library(wq, act, group):
    m, k = 5, 2048 + 256
    x = make_x(m, k, act, torch.bfloat16, 22).cuda()
    w = weight_of(k, act, torch.bfloat16, 23)
    w = None if w is None else w.cuda()
    assert torch.equal(wq.transform_rows(x, group, act, w, 1e-6), reflib.transform_rows(x, group, act, w, 1e-6))


@pytest.mark.parametrize("group", [16, 64, 256])
def test_rotate_groups(wq, group):
    x = randn((6, 1280), torch.float16, 24).cuda()
    out = wq.rotate_groups(x, group)
    assert torch.equal(out, reflib.rotate_groups(x, group))
    expected = oracle.rotate_reference(x.float().cpu(), group)
    assert oracle.relative_error(out.cpu(), expected) < 1e-3


def test_large_row_count(wq):
    """More rows than the reference's per-call limit of 65535, in one call."""
    x = randn((70000, 256), torch.bfloat16, 25).cuda()
    q, s = wq.quantize_blocks(x)
    q_ref, s_ref = reflib.quantize_blocks(x)
    assert torch.equal(q, q_ref) and torch.equal(s, s_ref)


@pytest.mark.parametrize("act", [None, "rms_norm", "gelu"])
def test_quantizers_at_row_windows(wq, act):
    """wq8_quantize_at / wq8_quantize_blocks_at: for several values of the device counter the codes and scales equal the plain entry
    points' on the matching slice of input rows (the outputs always start at row 0)."""
    total, m, k, first, step = 120, 20, 1024 + 128, 3, 25
    x = make_x(total, k, act, torch.bfloat16, 21).cuda()
    w = weight_of(k, act, torch.bfloat16, 22)
    w = None if w is None else w.cuda()
    lib, stream = wq._require(), wq._stream(x.device)
    acts = {None: 0, "rms_norm": 1, "gelu": 3}
    for count in (0, 1, 3):
        counter = torch.tensor([count], dtype=torch.int64, device="cuda")
        rows = x[first + count * step:first + count * step + m]
        q, s = torch.empty((m, k), dtype=torch.int8, device="cuda"), torch.empty((m, -(-k // 128)), dtype=torch.float32, device="cuda")
        assert lib.wq8_quantize_blocks_at(x.data_ptr(), q.data_ptr(), s.data_ptr(), m, k, x.stride(0), 1, 0, acts[act], wq._ptr(w), 1e-6, None,
                                          counter.data_ptr(), first, step, stream) == 0
        q_plain, s_plain = wq.quantize_blocks(rows, 0, act, w, 1e-6)
        assert torch.equal(q, q_plain) and torch.equal(s, s_plain)
        hi, lo, rs = (torch.empty((m, k), dtype=torch.int8, device="cuda"), torch.empty((m, k), dtype=torch.int8, device="cuda"),
                      torch.empty(m, dtype=torch.float32, device="cuda"))
        assert lib.wq8_quantize_at(x.data_ptr(), hi.data_ptr(), lo.data_ptr(), rs.data_ptr(), m, k, x.stride(0), 1, 0, acts[act], wq._ptr(w), 1e-6,
                                   counter.data_ptr(), first, step, stream) == 0
        hi_plain, lo_plain, rs_plain = wq.quantize(rows, 0, True, act, w, 1e-6)
        assert torch.equal(hi, hi_plain) and torch.equal(lo, lo_plain) and torch.equal(rs, rs_plain)
    # no counter: row 0, whatever first and step say
    q, s = torch.empty((m, k), dtype=torch.int8, device="cuda"), torch.empty((m, -(-k // 128)), dtype=torch.float32, device="cuda")
    assert lib.wq8_quantize_blocks_at(x.data_ptr(), q.data_ptr(), s.data_ptr(), m, k, x.stride(0), 1, 0, acts[act], wq._ptr(w), 1e-6, None, None, 7, 9,
                                      stream) == 0
    q_plain, s_plain = wq.quantize_blocks(x[:m], 0, act, w, 1e-6)
    assert torch.equal(q, q_plain) and torch.equal(s, s_plain)
