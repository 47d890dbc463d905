"""The tcgen05 INT8 GEMM on the GPU: exact INT32 block sums, every mode against the CPU oracle and against the reference's own CUDA
library, tails, in-place residual, determinism, and row / column partition invariance at full size."""
import numpy as np
import pytest
import torch

from oracle import int8_oracle as oracle
from tests import reflib
from tests.gpu_common import rand_int8, randn, rel
from wgpkernels_b200 import workloads

pytestmark = pytest.mark.gpu

MODES = {"row": 0, "exact": 1, "block": 10, "block-w8": 20, "block-n128": 15, "block+g": 12, "block+g-w8": 22, "block+g-n128": 13, "exact+g": 14}
REF_VARIANT = {"row": 2, "exact": 1, "block": 10, "block-w8": 10, "block-n128": 10, "block+g": 12, "block+g-w8": 12, "block+g-n128": 12,
               "exact+g": 14}


def operands(mode, m, n, k, dtype, seed, residual=False):
    """Random INT8 operands with the scale layout of `mode`, on the CPU."""
    base = mode.removesuffix("-w8").removesuffix("-n128")
    kb = -(-k // 128)
    g = torch.Generator().manual_seed(seed)
    a = rand_int8((m, k), seed)
    a_lo = rand_int8((m, k), seed + 1) if base.startswith("exact") else None
    sa = torch.rand((m, kb) if base.startswith("block") else (m,), generator=g) * 0.02 + 0.001
    b = rand_int8((n, k), seed + 2)
    sb = torch.rand((n, kb) if base.endswith("+g") else (n,), generator=g) * 0.01 + 0.0005
    bias = randn((n,), dtype, seed + 3)
    res = randn((m, n), dtype, seed + 4, 4.0) if residual else None
    rs = torch.rand(n, generator=g).to(dtype) if residual else None
    return base, a, a_lo, sa, b, sb, bias, res, rs


def run(wq, mode, a, a_lo, sa, b, sb, bias, res, rs, dtype, out=None):
    dev = lambda t: None if t is None else t.cuda()
    return wq.gemm(dev(a), dev(a_lo), dev(sa), dev(b), dev(sb), dev(bias), dtype, 0, MODES[mode], out=out, residual=dev(res) if out is None else out,
                   residual_scale=dev(rs))


@pytest.mark.parametrize("shape", [(40, 96, 256), (128, 256, 128), (129, 257 * 8, 384), (300, 520, 1024 + 16), (1, 8, 16)], ids=str)
def test_block_sums_are_exact(wq, shape):
    """The INT32 sums the tensor cores leave in tensor memory, per 128-element block of K, bit for bit."""
    m, n, k = shape
    a, b = rand_int8((m, k), 1), rand_int8((n, k), 2)
    sums = wq.debug_block_sums(a.cuda(), b.cuda())
    assert wq.debug_status() == 0
    assert np.array_equal(sums.cpu().numpy(), oracle.block_sums(a.numpy(), b.numpy()))


def test_block_sums_extreme_values(wq):
    """All operands at +-127: the largest block sums (128 * 127 * 127) the conversion must hold."""
    m, n, k = 128, 256, 512
    a = torch.full((m, k), 127, dtype=torch.int8)
    b = torch.full((n, k), -127, dtype=torch.int8)
    b[::2] = 127
    sums = wq.debug_block_sums(a.cuda(), b.cuda())
    assert np.array_equal(sums.cpu().numpy(), oracle.block_sums(a.numpy(), b.numpy()))
    sa, sb = torch.ones(m, 4), torch.ones(n)
    y = wq.gemm(a.cuda(), None, sa.cuda(), b.cuda(), sb.cuda(), None, torch.bfloat16, 0, 10)
    y2 = wq.gemm(a.cuda(), None, sa.cuda(), b.cuda(), sb.cuda(), None, torch.bfloat16, 0, 20)
    expected = oracle.gemm("block", a.numpy(), None, sa.numpy(), b.numpy(), sb.numpy())
    assert torch.equal(y.cpu(), expected) and torch.equal(y2.cpu(), expected)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("residual", [False, True], ids=["plain", "residual"])
@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("shape", [(40, 96, 256), (130, 264, 640), (257, 520, 1024 + 48)], ids=str)
def test_modes_match_oracle(wq, shape, mode, residual, dtype):
    m, n, k = shape
    base, a, a_lo, sa, b, sb, bias, res, rs = operands(mode, m, n, k, dtype, 31, residual)
    y = run(wq, mode, a, a_lo, sa, b, sb, bias, res, rs, dtype)
    assert wq.debug_status() == 0
    expected = oracle.gemm(base, a.numpy(), None if a_lo is None else a_lo.numpy(), sa.numpy(), b.numpy(), sb.numpy(), bias, res, rs, dtype)
    # same FP32 operation order as the oracle: identical up to the rare double rounding of the oracle's emulated FMA
    mismatch = (y.cpu() != expected).float().mean().item()
    assert mismatch < 1e-3, mismatch
    assert rel(y, expected) < 2e-5


@pytest.mark.parametrize("mode", list(MODES))
def test_modes_match_reference_library(wq, mode):
    m, n, k = 1000, 1536, 2048
    dtype = torch.bfloat16
    base, a, a_lo, sa, b, sb, bias, res, rs = operands(mode, m, n, k, dtype, 41, True)
    y = run(wq, mode, a, a_lo, sa, b, sb, bias, res, rs, dtype)
    dev = lambda t: None if t is None else t.cuda()
    y_ref = reflib.gemm(dev(a), dev(a_lo), dev(sa), dev(b), dev(sb), dev(bias), dtype, REF_VARIANT[mode], 0, dev(res), dev(rs))
    assert rel(y, y_ref) < 1e-3
    assert (y != y_ref).float().mean().item() < 1e-3


def test_odd_output_width(wq):
    """N not a multiple of 8: element-wise stores."""
    m, n, k = 70, 100 + 3, 256
    base, a, a_lo, sa, b, sb, bias, res, rs = operands("block", m, n, k, torch.bfloat16, 51, True)
    y = run(wq, "block", a, a_lo, sa, b, sb, bias, res, rs, torch.bfloat16)
    expected = oracle.gemm("block", a.numpy(), None, sa.numpy(), b.numpy(), sb.numpy(), bias, res, rs, torch.bfloat16)
    assert rel(y, expected) < 2e-5


def test_in_place_residual_and_determinism(wq):
    m, n, k = 300, 768, 1024
    base, a, a_lo, sa, b, sb, bias, res, rs = operands("block", m, n, k, torch.bfloat16, 61, True)
    y = run(wq, "block", a, a_lo, sa, b, sb, bias, res, rs, torch.bfloat16)
    target = res.cuda().clone()
    y2 = run(wq, "block", a, a_lo, sa, b, sb, bias, res, rs, torch.bfloat16, out=target)
    assert y2.data_ptr() == target.data_ptr()
    assert torch.equal(y, y2)
    assert torch.equal(y, run(wq, "block", a, a_lo, sa, b, sb, bias, res, rs, torch.bfloat16))


def test_weight_row_ranges(wq):
    """A row range of the weight (and of its scales and bias) computes the matching output columns, bit for bit."""
    m, n, k = 200, 1024, 512
    base, a, a_lo, sa, b, sb, bias, res, rs = operands("block", m, n, k, torch.bfloat16, 71)
    a, sa, b, sb, bias = a.cuda(), sa.cuda(), b.cuda(), sb.cuda(), bias.cuda()
    full = wq.gemm(a, None, sa, b, sb, bias, torch.bfloat16, 0, 10)
    part = wq.gemm(a, None, sa, b[256:640], sb[256:640], bias[256:640], torch.bfloat16, 0, 10)
    assert torch.equal(full[:, 256:640], part)
    rows = wq.gemm(a[64:150], None, sa[64:150], b, sb, bias, torch.bfloat16, 0, 10)
    assert torch.equal(full[64:150], rows)


@pytest.mark.parametrize("name", ["c1", "c2"])
def test_full_size_rows_against_oracle(wq, name):
    """BASELINE configs 1 and 2 at full width (N, K) on a band of rows that spans tile boundaries, through linear():
    the INT8 codes and scales feed the oracle's GEMM, so only the FP32 accumulation order of the GEMM is compared."""
    c = workloads.make(name, rows=300)
    g = c.to("cuda")
    y = wq.linear(g.x, g.weight, g.scale, g.bias, mode="block", act=c.act, act_weight=g.act_weight, eps=c.eps, residual=g.residual,
                  residual_scale=g.residual_scale)
    assert wq.debug_status() == 0
    q, sa = wq.quantize_blocks(g.x, 0, c.act, g.act_weight, c.eps)
    expected = oracle.gemm("block", q.cpu().numpy(), None, sa.cpu().numpy(), c.weight.numpy(), c.scale.numpy(), c.bias, c.residual, c.residual_scale,
                           torch.bfloat16)
    assert (y.cpu() != expected).float().mean().item() < 1e-3
    assert rel(y, expected) < 2e-5
    reference = oracle.linear_reference(c.x, c.weight, c.scale, c.bias, 0, c.act, c.act_weight, c.eps, c.residual, c.residual_scale)
    assert rel(y, reference) < 3e-2  # the block path's own quantization error against FP32, the reference's selftest bar


def test_full_size_partition_invariance(wq):
    """BASELINE config 1 at full size (M = 32760): every output element is computed by the same instruction sequence wherever its
    tile lies, so row bands and column bands of the problem reproduce the full result bit for bit; the band results are themselves
    checked against the oracle by the test above."""
    c = workloads.make("c1").to("cuda")
    prepared = wq.prepare(c.x, 0, "block", c.act, c.act_weight, c.eps)
    full = wq.linear_prepared(prepared, c.weight, c.scale, c.bias)
    assert wq.debug_status() == 0
    band = wq.linear_prepared(prepared.rows(12345, 12345 + 700), c.weight, c.scale, c.bias)
    assert torch.equal(full[12345:12345 + 700], band)
    cols = wq.linear_prepared(prepared, c.weight[7680:9216], c.scale[7680:9216], None)
    assert torch.equal(full[:, 7680:9216], cols)
    checksum = full.float().sum(dim=0)
    assert torch.isfinite(checksum).all()
    again = wq.linear_prepared(prepared, c.weight, c.scale, c.bias)
    assert torch.equal(full, again)


@pytest.mark.parametrize("mode", ["row", "exact", "block", "block+g", "exact+g"])
@pytest.mark.parametrize("residual", [False, True], ids=["plain", "residual"])
def test_column_ranges_and_several_outputs(wq, mode, residual):
    """out / residual as column ranges of wider matrices, and a list of outputs (what an N-sharded rank passes: its columns inside the
    full-width buffers of all ranks): every destination equals the contiguous result bit for bit, nothing else is touched."""
    m, n, k, dtype = 300, 520, 640, torch.bfloat16
    base, a, a_lo, sa, b, sb, bias, res, rs = operands(mode, m, n, k, dtype, 77, residual)
    dev = lambda t: None if t is None else t.cuda()
    expected = wq.gemm(dev(a), dev(a_lo), dev(sa), dev(b), dev(sb), dev(bias), dtype, 0, MODES[mode], residual=dev(res), residual_scale=dev(rs))
    wide = [torch.full((m, 1024), 7.0, dtype=dtype, device="cuda") for _ in range(3)]  # the destinations share one row stride
    offsets = [64, 256, 8]
    views = [w[:, o:o + n] for w, o in zip(wide, offsets)]
    wide_residual = None
    if residual:
        wide_residual = torch.zeros((m, 2048), dtype=dtype, device="cuda")
        wide_residual[:, 1024:1024 + n] = res.cuda()
    got = wq.gemm(dev(a), dev(a_lo), dev(sa), dev(b), dev(sb), dev(bias), dtype, 0, MODES[mode], out=views,
                  residual=None if wide_residual is None else wide_residual[:, 1024:1024 + n], residual_scale=dev(rs))
    torch.cuda.synchronize()
    assert got.data_ptr() == views[0].data_ptr()
    for w, o in zip(wide, offsets):
        assert torch.equal(w[:, o:o + n], expected)
        assert bool((w[:, :o] == 7.0).all()) and bool((w[:, o + n:] == 7.0).all())
    # one strided output, odd width (element-wise epilogue)
    odd = torch.full((m, 1000), 7.0, dtype=dtype, device="cuda")
    expected_odd = wq.gemm(dev(a), dev(a_lo), dev(sa), dev(b[:515]), dev(sb[:515]), dev(bias[:515]), dtype, 0, MODES[mode])
    wq.gemm(dev(a), dev(a_lo), dev(sa), dev(b[:515]), dev(sb[:515]), dev(bias[:515]), dtype, 0, MODES[mode], out=odd[:, 3:518])
    assert torch.equal(odd[:, 3:518], expected_odd) and bool((odd[:, :3] == 7.0).all()) and bool((odd[:, 518:] == 7.0).all())
    assert wq.debug_status() == 0


def test_segments_entry_point(wq):
    """wq8_gemm_segments of the C ABI: three weights of one quantized input, each output equal to wq8_gemm's on that weight."""
    import ctypes
    m, rows, k, dtype = 300, 264, 640, torch.bfloat16
    base, a, _, sa, b, sb, bias, _, _ = operands("block", m, 3 * rows, k, dtype, 91)
    ga, gsa, gb, gsb, gbias = a.cuda(), sa.cuda(), b.cuda(), sb.cuda(), bias.cuda()
    weights = [gb[s * rows:(s + 1) * rows] for s in range(3)]
    scales = [gsb[s * rows:(s + 1) * rows].contiguous() for s in range(3)]
    biases = [gbias[:rows].contiguous(), None, gbias[rows:2 * rows].contiguous()]
    outputs = [torch.empty((m, rows), dtype=dtype, device="cuda") for _ in range(3)]
    lib = wq._require()
    p, i = ctypes.c_void_p, ctypes.c_int
    lib.wq8_gemm_segments.argtypes = [p, p, p, p, p, p, p, i, i, i, i, i, i, i, i, p, p, p]
    pointers = lambda tensors: (ctypes.c_void_p * 4)(*[None if t is None else t.data_ptr() for t in tensors])
    code = lib.wq8_gemm_segments(ga.data_ptr(), None, gsa.data_ptr(), pointers(weights), pointers(scales), pointers(biases), pointers(outputs), 3, rows,
                                 m, k, 1, 10, 148, 0, None, None, wq._stream(ga.device))
    assert code == 0
    for weight, scale, bias_s, out in zip(weights, scales, biases, outputs):
        assert torch.equal(out, wq.gemm(ga, None, gsa, weight, scale, bias_s, dtype, 0, 10))
    assert lib.wq8_gemm_segments(ga.data_ptr(), None, gsa.data_ptr(), pointers(weights), pointers(scales), pointers(biases), pointers(outputs), 5, rows,
                                 m, k, 1, 10, 148, 0, None, None, wq._stream(ga.device)) == -4


def test_segments_through_the_module(wq):
    """linear_prepared_segments: one launch for the q / k / v weights of one prepared input, 'block' and 'exact', each output equal to
    linear_prepared on that weight; tiles of 256 and of 128 output channels; rows that are not a multiple of the tile."""
    assert wq.segments_supported()
    m, rows, k, dtype = 333, 200, 512, torch.bfloat16
    x = randn((m, k), dtype, 5).cuda()
    weights = [rand_int8((rows, k), 60 + s).cuda() for s in range(3)]
    scales = [(torch.rand(rows, generator=torch.Generator().manual_seed(70 + s)) * 0.01 + 0.001).cuda() for s in range(3)]
    biases = [randn((rows,), dtype, 80).cuda(), None, randn((rows,), dtype, 82).cuda()]
    for path in ("block", "exact", "row"):
        prepared = wq.prepare(x, 0, path)
        outputs = [torch.full((m, rows), 3.0, dtype=dtype, device="cuda") for _ in range(3)]
        wq.linear_prepared_segments(prepared, weights, scales, biases, outputs)
        for weight, scale, bias, out in zip(weights, scales, biases, outputs):
            zero = torch.zeros(rows, dtype=dtype, device="cuda") if bias is None else bias
            assert torch.equal(out, wq.linear_prepared(prepared, weight, scale, zero)), path
    assert wq.debug_status() == 0


def _gemm_at(wq, a, a_lo, sa, b, sb, bias, residual, rscale, y, m, variant, counter, first, step, span, scale_step, in_first, in_step):
    lib = wq._require()
    n, k = b.shape
    ptr = lambda t: None if t is None else t.data_ptr()
    sizes = (__import__("ctypes").c_int64 * 2)()
    lib.wq8_gemm_workspace(m, n, k, variant, 148, 0, sizes)
    workspace = torch.empty(max(int(sizes[0]), 16), dtype=torch.uint8, device=a.device)
    code = lib.wq8_gemm_at(a.data_ptr(), ptr(a_lo), sa.data_ptr(), b.data_ptr(), sb.data_ptr(), ptr(bias), ptr(residual), ptr(rscale), y.data_ptr(), m, n, k,
                           1, variant, 148, 0, workspace.data_ptr(), None, ptr(counter), first, step, span, scale_step, in_first, in_step,
                           wq._stream(a.device))
    assert code == 0, code
    torch.cuda.synchronize()


@pytest.mark.parametrize("mode", ["block", "exact", "row", "block+g"])
def test_gemm_at_row_windows(wq, mode):
    """wq8_gemm_at: for several values of the device counter, the window of output rows (written in place over the residual, with one
    residual gate per span of rows) equals the plain GEMM on the matching row slices; rows outside the window are untouched."""
    dtype, n, k = torch.bfloat16, 264, 640
    m, total_in, total_out = 300, 900, 1000                      # 300 = 2 tiles + a tail of 44 rows
    first, step, in_first, in_step, span = 24, 320, 40, 280, 128  # windows: outputs [24 + 320 c, ...), inputs [40 + 280 c, ...)
    base, a, a_lo, sa, b, sb, bias, _, _ = operands(mode, total_in, n, k, dtype, 17)
    dev = lambda t: None if t is None else t.cuda()
    a, a_lo, sa, b, sb, bias = map(dev, (a, a_lo, sa, b, sb, bias))
    gates = (torch.rand(-(-total_out // span), n, generator=torch.Generator().manual_seed(3)) + 0.5).to(dtype).cuda()
    untouched = randn((total_out, n), dtype, 19, 4.0).cuda()
    for count in (0, 1, 2):
        counter = torch.tensor([count], dtype=torch.int64, device="cuda")
        out0, in0 = first + count * step, in_first + count * in_step
        y = untouched.clone()
        _gemm_at(wq, a, a_lo, sa, b, sb, bias, y, gates, y, m, MODES[mode], counter, first, step, span, n, in_first, in_step)
        expected = untouched.clone()
        starts = [out0] + [r for r in range(out0 + 1, out0 + m) if r % span == 0]  # one plain GEMM per span of rows (its gate)
        for start in starts:
            stop = min((start // span + 1) * span, out0 + m)
            rows_in = slice(in0 + start - out0, in0 + stop - out0)
            expected[start:stop] = wq.gemm(a[rows_in], None if a_lo is None else a_lo[rows_in], sa[rows_in], b, sb, bias, dtype, 0, MODES[mode],
                                           residual=untouched[start:stop].clone(), residual_scale=gates[start // span].contiguous())
        assert torch.equal(y, expected), (mode, count, float((y.float() - expected.float()).abs().max()))
    # no counter: the plain entry point
    y = torch.empty((m, n), dtype=dtype, device="cuda")
    _gemm_at(wq, a, a_lo, sa, b, sb, bias, None, None, y, m, MODES[mode], None, 5, 7, 0, 0, 9, 11)
    assert torch.equal(y, wq.gemm(a[:m], None if a_lo is None else a_lo[:m], sa[:m], b, sb, bias, dtype, 0, MODES[mode]))
    assert wq.debug_status() == 0


def test_bounded_wait_gives_up_and_reports(wq):
    """A wait on a barrier that nothing completes: the kernel returns by itself, the status word holds the code, and the next GEMM is
    correct (the context stays usable)."""
    returned, status = wq.debug_wait_probe(clocks=2_000_000, code=9)
    assert returned == 2 and status == 9
    assert wq.debug_status() == 0  # cleared by the read
    a, b = rand_int8((64, 256), 1), rand_int8((96, 256), 2)
    sums = wq.debug_block_sums(a.cuda(), b.cuda())
    assert np.array_equal(sums.cpu().numpy(), oracle.block_sums(a.numpy(), b.numpy())) and wq.debug_status() == 0
