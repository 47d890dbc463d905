"""wq8_small_static: the few-token linear for callers that cannot allocate device memory.

Some users of this library never get to call an allocator on the GPU: a host that talks to the .so through a bare FFI and only owns
the input and output buffers it was given, a serving loop whose memory budget is fixed before the first request, code that runs while a
CUDA graph is being captured.  wq8_small needs scratch (K-split partial sums and tile counters) that such callers cannot supply, so
wq8_small_static keeps that scratch in a static buffer inside the library.  This test calls it through the C ABI, twice in a row on
shapes that do use scratch (digit planes, partial sums of K ranges shared by several CTAs, tile counters), and holds it to the output
of the existing entry point (the buffer keeps the previous call's contents: the
second call must not be disturbed by them).  Collected last on purpose.
"""
import ctypes

import pytest
import torch

from oracle import int8_oracle as oracle
from tests.gpu_common import rand_int8, randn, rel

pytestmark = pytest.mark.gpu
_DTYPES = {torch.float16: 0, torch.bfloat16: 1}


def bind(wq):
    lib = wq._require()
    p, i, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    lib.wq8_small_static.argtypes = [p, i64, p, p, p, p, p, p, i, i, i, i, i, p]
    lib.wq8_small_static.restype = i
    return lib


def static_small(wq, lib, x, w, sw, bias=None, residual=None, rscale=None):
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n), dtype=x.dtype, device=x.device)
    ptr = lambda t: None if t is None else t.data_ptr()
    code = lib.wq8_small_static(x.data_ptr(), x.stride(0), w.data_ptr(), sw.data_ptr(), ptr(bias), ptr(residual), ptr(rscale), y.data_ptr(), m, n, k,
                                _DTYPES[x.dtype], wq._sm_count(x.device), wq._stream(x.device))
    assert code == 0, f"wq8_small_static returned {code}"
    return y


@pytest.mark.parametrize("shape", [(16, 1024, 8192), (32, 4096, 14336), (4, 512, 4096), (8, 28672, 4096), (16, 1024, 8192 + 64)], ids=str)
def test_static_scratch_matches_caller_scratch(wq, shape):
    m, n, k = shape
    lib = bind(wq)
    g = torch.Generator().manual_seed(7)
    x = randn((m, k), torch.bfloat16, 201)
    w = rand_int8((n, k), 202)
    sw = torch.rand(n, generator=g) * 0.002 + 0.0001
    bias = randn((n,), torch.bfloat16, 203)
    res = randn((m, n), torch.bfloat16, 204, 4.0)
    rs = torch.rand(n, generator=g).to(torch.bfloat16)
    gx, gw, gsw, gbias, gres, grs = (t.cuda() for t in (x, w, sw, bias, res, rs))
    sizes = (ctypes.c_int64 * 2)()
    lib.wq8_small_workspace(m, n, k, wq._sm_count(gx.device), sizes)
    usual = wq.small(gx, gw, gsw, gbias, gres, grs)               # the usual entry point (up to 8 tokens the module runs another kernel)
    first = static_small(wq, lib, gx, gw, gsw, gbias, gres, grs)
    second = static_small(wq, lib, gx, gw, gsw, gbias, gres, grs)  # the buffer still holds the first call's partial sums
    torch.cuda.synchronize()
    assert torch.equal(first, second)
    assert rel(first, usual) < 1e-3
    if m > 8:  # above 8 tokens the module calls wq8_small itself: the same kernel on caller scratch, hence the same bits
        assert torch.equal(first, usual)
    assert rel(second, oracle.weight_only(x, w.numpy(), sw.numpy(), bias, res, rs, torch.bfloat16)) < 1e-3
    # a different shape in between, then the first one again: nothing left over from either
    half_k = k // 2 // 128 * 128
    half = gx[:, :half_k].contiguous(), gw[:, :half_k].contiguous(), gsw
    other = static_small(wq, lib, *half)
    assert torch.equal(other, static_small(wq, lib, *half)) and rel(other, wq.small(*half)) < 1e-3
    assert torch.equal(static_small(wq, lib, gx, gw, gsw, gbias, gres, grs), first)
    if shape in ((16, 1024, 8192), (16, 1024, 8192 + 64)):
        assert sizes[0] > 0  # this shape does exercise the scratch


def test_static_scratch_rejects_what_does_not_fit(wq):
    lib = bind(wq)
    one = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    # planning for a (fictitious) 4096-SM device: two pieces of partial sums per CTA, 128 MiB, far more than the 8 MiB buffer
    assert lib.wq8_small_static(one, 65536, one, one, None, None, None, one, 32, 4096, 65536, 1, 4096, None) == -5
    assert lib.wq8_small_static(one, 256, one, one, None, None, None, one, 33, 96, 256, 1, 148, None) == -2
    assert lib.wq8_small_static(one, 256, one, one, None, None, None, one, 0, 96, 256, 1, 148, None) == 0
