"""Few-token weight-streaming kernels ('lines', 'small') on the GPU against the CPU oracle and the reference's own CUDA library."""
import pytest
import torch

from oracle import int8_oracle as oracle
from tests import reflib
from tests.gpu_common import rand_int8, randn, rel

pytestmark = pytest.mark.gpu


def case(m, n, k, dtype, seed, residual):
    g = torch.Generator().manual_seed(seed)
    x = randn((m, k), dtype, seed)
    x[:, :4] = 1000.0 if dtype == torch.bfloat16 else 100.0  # massive-activation channels
    w = rand_int8((n, k), seed + 1)
    sw = torch.rand(n, generator=g) * 0.002 + 0.0001
    bias = randn((n,), dtype, seed + 2)
    res = randn((m, n), dtype, seed + 3, 4.0) if residual else None
    rs = torch.rand(n, generator=g).to(dtype) if residual else None
    return x, w, sw, bias, res, rs


def cuda(*tensors):
    return [None if t is None else t.cuda() for t in tensors]


@pytest.fixture(params=["planes", "converted"])
def kernel(request, wq, monkeypatch):
    """Both few-token kernels for shapes of at most 8 tokens: 'planes' (activations as INT8 digit planes, the Python module's choice) and
    'converted' (weights converted to the activation type: what wq8_gemv_lines / wq8_small of the C ABI run, and every larger shape)."""
    if request.param == "converted":
        monkeypatch.setattr(wq, "_stream_planes", lambda *args: False)
    return request.param


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("residual", [False, True], ids=["plain", "residual"])
@pytest.mark.parametrize("shape", [(1, 96, 256), (2, 100, 260), (3, 4096, 1024), (4, 520, 4096 + 64), (4, 28672, 4096), (1, 4096, 14336)], ids=str)
def test_lines(wq, kernel, shape, residual, dtype):
    m, n, k = shape
    x, w, sw, bias, res, rs = case(m, n, k, dtype, 101, residual)
    gx, gw, gsw, gbias, gres, grs = cuda(x, w, sw, bias, res, rs)
    y = wq.gemv_lines(gx, gw, gsw, gbias, gres, grs)
    expected = oracle.weight_only(x, w.numpy(), sw.numpy(), bias, res, rs, dtype)
    assert rel(y, expected) < 1e-3
    y_ref = reflib.gemv_lines(gx, gw, gsw, gbias, gres, grs)
    assert rel(y, y_ref) < 1e-3
    assert torch.equal(y, wq.gemv_lines(gx, gw, gsw, gbias, gres, grs))  # fixed-order reductions: run to run identical
    assert wq.debug_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("residual", [False, True], ids=["plain", "residual"])
@pytest.mark.parametrize("shape", [(5, 96, 256), (8, 1000, 1024), (16, 28672, 4096), (16, 4096, 14336), (32, 4096, 14336), (32, 1024, 8192), (9, 40, 64),
                                   (24, 2048, 4096)], ids=str)
def test_small(wq, kernel, shape, residual, dtype):
    m, n, k = shape
    x, w, sw, bias, res, rs = case(m, n, k, dtype, 111, residual)
    gx, gw, gsw, gbias, gres, grs = cuda(x, w, sw, bias, res, rs)
    y = wq.small(gx, gw, gsw, gbias, gres, grs)
    expected = oracle.weight_only(x, w.numpy(), sw.numpy(), bias, res, rs, dtype)
    assert rel(y, expected) < 1e-3
    y_ref = reflib.small(gx, gw, gsw, gbias, gres, grs)
    assert rel(y, y_ref) < 1e-3
    assert torch.equal(y, wq.small(gx, gw, gsw, gbias, gres, grs))  # fixed-order reductions: run to run identical
    # the split-K counters are left zeroed
    assert not wq._counters[0].any().item()
    assert wq.debug_status() == 0


def test_small_in_place_residual(wq):
    x, w, sw, bias, res, rs = case(12, 1024, 2048, torch.bfloat16, 121, True)
    gx, gw, gsw, gbias, gres, grs = cuda(x, w, sw, bias, res, rs)
    y = wq.small(gx, gw, gsw, gbias, gres, grs)
    target = gres.clone()
    wq.small(gx, gw, gsw, gbias, target, grs, out=target)
    assert torch.equal(y, target)


def test_strided_activation(wq):
    wide = randn((4, 4096), torch.bfloat16, 131).cuda()
    x = wide[:, 1024:3072]
    w = rand_int8((256, 2048), 132).cuda()
    sw = torch.full((256,), 0.001).cuda()
    assert torch.equal(wq.gemv_lines(x, w, sw), wq.gemv_lines(x.contiguous(), w, sw))
    assert torch.equal(wq.small(x, w, sw), wq.small(x.contiguous(), w, sw))


def test_planes_keep_small_values_next_to_large_ones(wq):
    """The digit planes share one power of two per 128 values: values down to 2^-14 of the largest of their run are exact, so a run that
    mixes 1000.0 with values around 0.5 still gives the FP32 result."""
    m, n, k = 4, 512, 4096
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16)
    x[:, ::128] = 1000.0
    w = rand_int8((n, k), 6)
    w[:, ::128] = 0  # the large values do not contribute: the result is made of the small ones only
    sw = torch.full((n,), 0.001)
    y = wq.gemv_lines(x.cuda(), w.cuda(), sw.cuda())
    expected = (x.double() @ w.double().T * 0.001).to(torch.bfloat16)
    assert rel(y, expected) < 2e-3
    assert wq.debug_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("tokens", [1, 4, 8])
@pytest.mark.parametrize("shape", [(28672, 4096), (4096, 14336)], ids=["up", "down"])
def test_planes_with_an_outlier_in_every_run(wq, shape, tokens, dtype):
    """The worst case of the digit-plane kernel: every run of 128 activations holds one value 2^10 times larger than the rest and all
    weights are live, so the small values carry the fewest digits.  Bar: 1e-3 against the reference's own CUDA kernels, which multiply
    the unrewritten activations; and the planes must actually be the kernel that ran."""
    n, k = shape
    g = torch.Generator().manual_seed(77)
    x = torch.randn(tokens, k, generator=g)
    x[:, 5::128] *= 1024.0
    x = x.to(dtype)
    w = rand_int8((n, k), 78)
    sw = torch.rand(n, generator=g) * 0.002 + 0.0001
    bias = randn((n,), dtype, 79)
    gx, gw, gsw, gbias = cuda(x, w, sw, bias)
    assert wq._require().wq8_stream_planes_workspace(tokens, n, k, 148) > 0
    for entry, reference in ((wq.gemv_lines, reflib.gemv_lines), (wq.small, reflib.small)):
        if entry is wq.gemv_lines and tokens > 4:
            continue
        y = entry(gx, gw, gsw, gbias)
        assert rel(y, reference(gx, gw, gsw, gbias)) < 1e-3
        exact = (x.double() @ (w.double() * sw.double()[:, None]).T + bias.double())
        assert rel(y, exact.float()) < 4e-3  # the output's own rounding to 8 or 11 bits
    assert wq.debug_status() == 0
