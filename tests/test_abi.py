"""The C-ABI library: it builds, loads without a GPU, exports every symbol include/wq8.h declares, identifies itself with the
reference's ABI number, and rejects bad arguments with the reference's error codes before touching the device."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

from wgpkernels_b200 import build as builder

ROOT = Path(__file__).resolve().parents[1]
p, i, i64, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float


@pytest.fixture(scope="module")
def lib():
    handle = ctypes.CDLL(str(builder.build()))
    handle.wq8_quantize.argtypes = [p, p, p, p, i, i, i64, i, i, i, p, f, p]
    handle.wq8_quantize_blocks.argtypes = [p, p, p, i, i, i64, i, i, i, p, f, p, p]
    handle.wq8_transform_rows.argtypes = [p, p, i, i, i64, i, i, i, p, f, p]
    handle.wq8_rotate_groups.argtypes = [p, p, i, i, i64, i, i, p]
    handle.wq8_gemm.argtypes = [p, p, p, p, p, p, p, p, p, i, i, i, i, i, i, i, p, p, p]
    handle.wq8_gemm_workspace.argtypes = [i, i, i, i, i, i, p]
    handle.wq8_gemm_workspace.restype = None
    handle.wq8_small.argtypes = [p, i64, p, p, p, p, p, p, i, i, i, i, i, p, p, p]
    handle.wq8_small_workspace.argtypes = [i, i, i, i, p]
    handle.wq8_small_workspace.restype = None
    handle.wq8_gemv_lines.argtypes = [p, i64, p, p, p, p, p, p, i, i, i, i, p]
    return handle


def declared_symbols():
    text = "\n".join((ROOT / "include").glob("*.h").__next__().read_text().splitlines())
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wq8_\w+)\s*\(", text)))


def test_header_symbols_are_exported():
    library = builder.build()
    listing = subprocess.run(["nm", "-D", "--defined-only", str(library)], capture_output=True, text=True, check=True).stdout
    exported = {line.split()[-1] for line in listing.splitlines() if " T " in line}
    declared = declared_symbols()
    assert len(declared) >= 17
    assert not [name for name in declared if name not in exported]
    # nothing but the C ABI leaves the library (hidden visibility, static CUDA runtime)
    assert all(name.startswith("wq8_") for name in exported), sorted(exported)[:10]


def test_reference_entry_points_present(lib):
    """The names the reference's ctypes table binds (wgpkernels/int8/__init__.py:73-89 of WGPKernels)."""
    for name in ("wq8_abi", "wq8_features", "wq8_quantize", "wq8_quantize_blocks", "wq8_transform_rows", "wq8_l2_flush", "wq8_l2_flush_release",
                 "wq8_gemm", "wq8_gemm_workspace", "wq8_gemm_select", "wq8_small", "wq8_small_workspace", "wq8_gemv_lines", "wq8_rotate_groups"):
        assert hasattr(lib, name), name


def test_identification(lib):
    assert lib.wq8_abi() == 11
    assert lib.wq8_features() & 1


def test_empty_calls_return_zero(lib):
    assert lib.wq8_quantize_blocks(None, None, None, 0, 256, 256, 1, 0, 0, None, 0.0, None, None) == 0
    assert lib.wq8_quantize(None, None, None, None, 0, 256, 256, 1, 0, 0, None, 0.0, None) == 0
    assert lib.wq8_transform_rows(None, None, 0, 256, 256, 1, 0, 0, None, 0.0, None) == 0
    assert lib.wq8_gemm(None, None, None, None, None, None, None, None, None, 0, 96, 256, 1, 10, 148, 0, None, None, None) == 0
    assert lib.wq8_small(None, 256, None, None, None, None, None, None, 0, 96, 256, 1, 148, None, None, None) == 0
    assert lib.wq8_gemv_lines(None, 256, None, None, None, None, None, None, 0, 96, 256, 1, None) == 0


def test_argument_errors(lib):
    one = ctypes.c_void_p(16)  # never dereferenced: the checks come first
    # a low part must accompany exactly the hi/lo variants
    assert lib.wq8_gemm(one, None, one, one, one, None, None, None, one, 8, 96, 256, 1, 1, 148, 0, None, None, None) == -2
    assert lib.wq8_gemm(one, one, one, one, one, None, None, None, one, 8, 96, 256, 1, 10, 148, 0, None, None, None) == -2
    assert lib.wq8_gemm(one, None, one, one, one, None, None, None, one, 8, 96, 250, 1, 10, 148, 0, None, None, None) == -2  # K % 16
    assert lib.wq8_gemm(one, None, one, one, one, None, None, None, one, 8, 96, 256, 2, 10, 148, 0, None, None, None) == -1  # fp32 output
    assert lib.wq8_gemm(one, None, one, one, one, None, None, None, one, 8, 96, 256, 1, 99, 148, 0, None, None, None) == -3  # variant
    assert lib.wq8_small(one, 256, one, one, None, None, None, one, 33, 96, 256, 1, 148, None, None, None) == -2
    assert lib.wq8_small(one, 256, one, one, None, None, None, one, 8, 96, 200, 1, 148, None, None, None) == -2
    assert lib.wq8_gemv_lines(one, 256, one, one, None, None, None, one, 5, 96, 256, 1, None) == -2
    assert lib.wq8_gemv_lines(one, 256, one, one, None, None, None, one, 2, 96, 254, 1, None) == -2
    assert lib.wq8_quantize_blocks(one, one, one, 4, 256, 256, 1, 32, 0, None, 0.0, None, None) == -1  # group
    assert lib.wq8_quantize_blocks(one, one, one, 4, 256, 256, 1, 0, 7, None, 0.0, None, None) == -1   # act
    assert lib.wq8_quantize_blocks(one, one, one, 4, 256, 256, 2, 0, 1, None, 0.0, None, None) == -1   # fp32 input takes no op
    assert lib.wq8_quantize(one, one, None, one, 4, 256, 256, 5, 0, 0, None, 0.0, None) == -1          # dtype
    assert lib.wq8_rotate_groups(one, one, 4, 256, 256, 1, 0, None) == -1


def test_workspace_queries(lib):
    sizes = (ctypes.c_int64 * 2)()
    lib.wq8_gemm_workspace(32760, 15360, 5120, 10, 148, 1, sizes)
    assert sizes[0] >= 0 and sizes[1] >= 0 and sizes[1] <= 4096
    # K a multiple of 128: the tensor-core kernel -- digit planes (96 rows for 9-32 token slots... 48 for 16), their powers of two and two
    # pieces of partial sums per CTA, each rounded up to 256 bytes; one counter per tile of 128 output channels
    lib.wq8_small_workspace(16, 1024, 14336, 148, sizes)
    assert sizes[0] == 48 * 14336 + (14336 // 128) * 16 * 4 + 148 * 2 * 128 * 16 * 4 and sizes[1] == 4 * 8
    lib.wq8_small_workspace(16, 28672, 4096, 148, sizes)
    assert sizes[0] == 48 * 4096 + (4096 // 128) * 16 * 4 + 148 * 2 * 128 * 16 * 4 and sizes[1] == 4 * 224
    lib.wq8_small_workspace(3, 256, 256, 148, sizes)  # fewer (tile, K block) pairs than SMs: one CTA per pair
    assert sizes[0] == 32 * 256 + 256 + 4 * 2 * 128 * 8 * 4 and sizes[1] == 8
    # K not a multiple of 128: the direct-load kernel; few channels split K across CTAs, many do not
    lib.wq8_small_workspace(16, 1024, 14336 + 64, 148, sizes)
    assert sizes[0] > 0 and 0 < sizes[1] <= 4096
    lib.wq8_small_workspace(16, 28672, 4096 + 64, 148, sizes)
    assert sizes[0] == 0 and sizes[1] == 0


def test_additions_check_their_arguments(lib):
    """The entry points this library adds: argument checks that come before any CUDA call, and the workspace sizes."""
    i, i64, p = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p
    lib.wq8_gemm_multi.argtypes = [p, p, p, p, p, p, p, i64, p, p, i, i64, i, i, i, i, i, i, p, p]
    lib.wq8_stream_planes_workspace.argtypes = [i, i, i, i]
    lib.wq8_stream_planes_workspace.restype = i64
    lib.wq8_stream_planes.argtypes = [p, i64, p, p, p, p, p, p, i, i, i, i, i, p, p]
    lib.wq8_gemm_segments.argtypes = [p, p, p, p, p, p, p, i, i, i, i, i, i, i, i, p, p, p]
    one = ctypes.c_void_p(16)
    targets = (ctypes.c_void_p * 8)(*([16] * 8))
    assert lib.wq8_gemm_multi(one, None, one, one, one, None, None, 0, None, targets, 0, 96, 8, 96, 256, 1, 10, 148, None, None) == -2   # no destination
    assert lib.wq8_gemm_multi(one, None, one, one, one, None, None, 0, None, targets, 9, 96, 8, 96, 256, 1, 10, 148, None, None) == -2   # too many
    assert lib.wq8_gemm_multi(one, None, one, one, one, None, None, 0, None, targets, 2, 64, 8, 96, 256, 1, 10, 148, None, None) == -2   # row stride < N
    assert lib.wq8_gemm_multi(one, None, one, one, one, None, None, 0, None, None, 1, 96, 8, 96, 256, 1, 10, 148, None, None) == -2
    assert lib.wq8_gemm_multi(None, None, None, None, None, None, None, 0, None, None, 0, 0, 0, 96, 256, 1, 10, 148, None, None) == 0    # empty
    assert lib.wq8_stream_planes_workspace(4, 4096, 4096, 148) == 8 * 3 * 4096 + (4096 // 128) * 8 * 4
    assert lib.wq8_stream_planes_workspace(9, 4096, 4096, 148) == 0      # more than 8 tokens
    assert lib.wq8_stream_planes_workspace(4, 4096, 4096 + 64, 148) == 0  # K not a multiple of 128
    assert lib.wq8_stream_planes_workspace(4, 4096, 512, 148) == 0        # too few K segments
    assert lib.wq8_stream_planes(one, 4096, one, one, None, None, None, one, 9, 4096, 4096, 1, 148, one, None) == -2
    assert lib.wq8_stream_planes(one, 4096, one, one, None, None, None, one, 4, 4096, 4096, 1, 148, None, None) == -2  # no workspace
    assert lib.wq8_stream_planes(one, 4096, one, one, None, None, None, one, 4, 4096, 4096, 2, 148, one, None) == -1
    four = (ctypes.c_void_p * 4)(16, 16, 16, 16)
    assert lib.wq8_gemm_segments(one, None, one, four, four, four, four, 5, 96, 8, 256, 1, 10, 148, 0, None, None, None) == -4
    assert lib.wq8_gemm_segments(one, None, one, four, four, four, four, 2, 100, 8, 256, 1, 10, 148, 0, None, None, None) == -4  # rows % 8
    assert lib.wq8_gemm_segments(one, None, one, four, four, four, four, 2, 96, 8, 256, 1, 12, 148, 0, None, None, None) == -4   # group scales
    sizes = (ctypes.c_int64 * 2)()
    lib.wq8_gemm_workspace(8, 300, 640, 12, 148, 0, sizes)
    assert sizes[0] == 5 * 512 * 4 and sizes[1] == 0
    lib.wq8_gemm_workspace(8, 300, 640, 10, 148, 1, sizes)
    assert sizes[0] == 0 and sizes[1] == 0


def test_unaligned_operands_are_refused_not_launched(lib):
    """Every few-token kernel reads x and w with vector loads: operands that are not aligned for them come back as -2 before any
    launch (bogus, never dereferenced pointers)."""
    i, i64, p = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p
    lib.wq8_small_static.argtypes = [p, i64, p, p, p, p, p, p, i, i, i, i, i, p]
    aligned, by8, by4, odd = p(4096), p(4096 + 8), p(4096 + 4), p(4096 + 1)
    # wq8_small and its static-scratch form: x and w 16-byte aligned, row stride a multiple of 8
    assert lib.wq8_small(aligned, 256, by8, aligned, None, None, None, aligned, 8, 96, 256, 1, 148, None, None, None) == -2
    assert lib.wq8_small(by8, 256, aligned, aligned, None, None, None, aligned, 8, 96, 256, 1, 148, None, None, None) == -2
    assert lib.wq8_small(aligned, 252, aligned, aligned, None, None, None, aligned, 8, 96, 256, 1, 148, None, None, None) == -2
    assert lib.wq8_small_static(aligned, 256, by8, aligned, None, None, None, aligned, 8, 96, 256, 1, 148, None) == -2
    assert lib.wq8_small_static(by8, 256, aligned, aligned, None, None, None, aligned, 8, 96, 256, 1, 148, None) == -2
    # wq8_gemv_lines with K % 64 != 0 runs the general kernel: x 8-byte aligned, row stride a multiple of 4, w 4-byte aligned
    assert lib.wq8_gemv_lines(by4, 100, aligned, aligned, None, None, None, aligned, 2, 96, 100, 1, None) == -2
    assert lib.wq8_gemv_lines(aligned, 102, aligned, aligned, None, None, None, aligned, 2, 96, 100, 1, None) == -2
    assert lib.wq8_gemv_lines(aligned, 100, odd, aligned, None, None, None, aligned, 2, 96, 100, 1, None) == -2
    # and an unaligned w with K % 64 == 0 takes the general kernel only if it is 4-byte aligned
    assert lib.wq8_gemv_lines(aligned, 256, odd, aligned, None, None, None, aligned, 2, 96, 256, 1, None) == -2


def test_row_window_entry_points_check_their_arguments(lib):
    i, i64, p, ll = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_longlong
    lib.wq8_gemm_at.argtypes = [p, p, p, p, p, p, p, p, p, i, i, i, i, i, i, i, p, p, p, ll, ll, ll, ll, ll, ll, p]
    lib.wq8_quantize_at.argtypes = [p, p, p, p, i, i, i64, i, i, i, p, f, p, ll, ll, p]
    lib.wq8_quantize_blocks_at.argtypes = [p, p, p, i, i, i64, i, i, i, p, f, p, p, ll, ll, p]
    one = p(16)
    assert lib.wq8_gemm_at(None, None, None, None, None, None, None, None, None, 0, 96, 256, 1, 10, 148, 0, None, None, one, 0, 1, 0, 0, 0, 0, None) == 0
    assert lib.wq8_gemm_at(one, None, one, one, one, None, None, None, one, 8, 96, 256, 1, 1, 148, 0, None, None, one, 0, 1, 0, 0, 0, 0, None) == -2   # no low part
    assert lib.wq8_gemm_at(one, None, one, one, one, None, None, None, one, 8, 96, 256, 1, 10, 148, 0, None, None, one, 0, 1, -1, 0, 0, 0, None) == -2  # span
    assert lib.wq8_gemm_at(one, None, one, one, one, None, None, None, one, 8, 96, 256, 1, 99, 148, 0, None, None, one, 0, 1, 0, 0, 0, 0, None) == -3
    assert lib.wq8_quantize_at(None, None, None, None, 0, 256, 256, 1, 0, 0, None, 0.0, one, 0, 1, None) == 0
    assert lib.wq8_quantize_at(one, one, None, one, 4, 256, 256, 5, 0, 0, None, 0.0, one, 0, 1, None) == -1
    assert lib.wq8_quantize_blocks_at(one, one, one, 4, 250, 256, 1, 0, 0, None, 0.0, None, one, 0, 1, None) == -2
