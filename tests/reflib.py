"""Thin ctypes caller of the reference's own CUDA library (oracle/_ref/libwgp_int8_ref.so, built by oracle/Makefile from the
unmodified reference source).  GPU parity tests compare this repository's kernels with it on the same inputs.  Test infrastructure only."""
import ctypes
from pathlib import Path

import pytest
import torch

PATH = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libwgp_int8_ref.so"
_DTYPES = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
_ACTS = {None: 0, "rms_norm": 1, "swiglu": 2, "gelu": 3}
_lib = None


def load():
    """The reference library, or a skip when it was not built (no reference checkout at build time)."""
    global _lib
    if _lib is None:
        if not PATH.exists():
            pytest.skip("reference CUDA library not built (oracle/_ref)")
        lib = ctypes.CDLL(str(PATH))
        assert lib.wq8_abi() == 11
        p, i, i64, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
        lib.wq8_quantize.argtypes = [p, p, p, p, i, i, i64, i, i, i, p, f, p]
        lib.wq8_quantize_blocks.argtypes = [p, p, p, i, i, i64, i, i, i, p, f, p, p]
        lib.wq8_transform_rows.argtypes = [p, p, i, i, i64, i, i, i, p, f, p]
        lib.wq8_rotate_groups.argtypes = [p, p, i, i, i64, i, i, p]
        lib.wq8_gemm.argtypes = [p, p, p, p, p, p, p, p, p, i, i, i, i, i, i, i, p, p, p]
        lib.wq8_gemm_workspace.argtypes = [i, i, i, i, i, i, p]
        lib.wq8_gemm_workspace.restype = None
        lib.wq8_small.argtypes = [p, i64, p, p, p, p, p, p, i, i, i, i, i, p, p, p]
        lib.wq8_small_workspace.argtypes = [i, i, i, i, p]
        lib.wq8_small_workspace.restype = None
        lib.wq8_gemv_lines.argtypes = [p, i64, p, p, p, p, p, p, i, i, i, i, p]
        _lib = lib
    return _lib


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(t):
    return torch._C._cuda_getCurrentRawStream(t.device.index)


def _ok(code):
    assert code == 0, f"reference library returned {code}"


def _width(x, act):
    return x.shape[1] // 2 if act == "swiglu" else x.shape[1]


def quantize_blocks(x, group=0, act=None, act_weight=None, eps=0.0):
    lib = load()
    m, k = x.shape[0], _width(x, act)
    q = torch.empty((m, k), dtype=torch.int8, device=x.device)
    scale = torch.empty((m, (k + 127) // 128), dtype=torch.float32, device=x.device)
    inv_rms = torch.empty(m, dtype=torch.float32, device=x.device)
    for start in range(0, m, 65535):  # the reference puts rows on the grid's y axis
        rows = min(65535, m - start)
        _ok(lib.wq8_quantize_blocks(x[start:].data_ptr(), q[start:].data_ptr(), scale[start:].data_ptr(), rows, k, x.stride(0), _DTYPES[x.dtype],
                                    group, _ACTS[act], _ptr(act_weight), eps, inv_rms[start:].data_ptr(), _stream(x)))
    return q, scale


def quantize(x, group=0, hilo=False, act=None, act_weight=None, eps=0.0):
    lib = load()
    m, k = x.shape[0], _width(x, act)
    hi = torch.empty((m, k), dtype=torch.int8, device=x.device)
    lo = torch.empty_like(hi) if hilo else None
    scale = torch.empty(m, dtype=torch.float32, device=x.device)
    _ok(lib.wq8_quantize(x.data_ptr(), hi.data_ptr(), _ptr(lo), scale.data_ptr(), m, k, x.stride(0), _DTYPES[x.dtype], group, _ACTS[act],
                         _ptr(act_weight), eps, _stream(x)))
    return hi, lo, scale


def transform_rows(x, group=0, act=None, act_weight=None, eps=0.0):
    lib = load()
    m, k = x.shape[0], _width(x, act)
    out = torch.empty((m, k), dtype=x.dtype, device=x.device)
    _ok(lib.wq8_transform_rows(x.data_ptr(), out.data_ptr(), m, k, x.stride(0), _DTYPES[x.dtype], group, _ACTS[act], _ptr(act_weight), eps, _stream(x)))
    return out


def rotate_groups(x, group):
    lib = load()
    out = torch.empty_like(x)
    _ok(lib.wq8_rotate_groups(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], x.stride(0), _DTYPES[x.dtype], group, _stream(x)))
    return out


def gemm(a, a_lo, sa, b, sb, bias, out_dtype, variant, split=0, residual=None, residual_scale=None, out=None):
    """The reference GEMM with one of its own variants (row 0/2/6, exact 1/7, block 10/11, block+g 12/13, exact+g 14)."""
    lib = load()
    m, k = a.shape
    n = b.shape[0]
    sms = torch.cuda.get_device_properties(a.device).multi_processor_count
    y = torch.empty((m, n), dtype=out_dtype, device=a.device) if out is None else out
    sizes = (ctypes.c_int64 * 2)()
    lib.wq8_gemm_workspace(m, n, k, variant, sms, split, sizes)
    slots = torch.empty(max(sizes[0], 16), dtype=torch.uint8, device=a.device)
    counters = torch.zeros(max(sizes[1] // 4, 1), dtype=torch.int32, device=a.device)
    _ok(lib.wq8_gemm(a.data_ptr(), _ptr(a_lo), sa.data_ptr(), b.data_ptr(), sb.data_ptr(), _ptr(bias), _ptr(residual), _ptr(residual_scale),
                     y.data_ptr(), m, n, k, _DTYPES[out_dtype], variant, sms, split, slots.data_ptr(), counters.data_ptr(), _stream(a)))
    return y


def small(x, w, sw, bias=None, residual=None, residual_scale=None):
    lib = load()
    m, k = x.shape
    n = w.shape[0]
    sms = torch.cuda.get_device_properties(x.device).multi_processor_count
    y = torch.empty((m, n), dtype=x.dtype, device=x.device)
    sizes = (ctypes.c_int64 * 2)()
    lib.wq8_small_workspace(m, n, k, sms, sizes)
    slots = torch.empty(max(sizes[0] // 4, 4), dtype=torch.float32, device=x.device)
    counters = torch.zeros(max(sizes[1] // 4, 1), dtype=torch.int32, device=x.device)
    _ok(lib.wq8_small(x.data_ptr(), x.stride(0), w.data_ptr(), sw.data_ptr(), _ptr(bias), _ptr(residual), _ptr(residual_scale), y.data_ptr(), m, n, k,
                      _DTYPES[x.dtype], sms, slots.data_ptr(), counters.data_ptr(), _stream(x)))
    return y


def gemv_lines(x, w, sw, bias=None, residual=None, residual_scale=None):
    lib = load()
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n), dtype=x.dtype, device=x.device)
    _ok(lib.wq8_gemv_lines(x.data_ptr(), x.stride(0), w.data_ptr(), sw.data_ptr(), _ptr(bias), _ptr(residual), _ptr(residual_scale), y.data_ptr(), m, n, k,
                           _DTYPES[x.dtype], _stream(x)))
    return y
