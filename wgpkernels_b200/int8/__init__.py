"""INT8 weight linears on B200: Y = op(X) @ (W * scales).T + bias, optionally residual + residual_scale * (...).

Host-side mirror of the reference's `wgpkernels.int8` module (wgpkernels/int8/__init__.py of WGPKernels): the same public
functions, arguments, return values and errors, over this package's own sm_100a library (`libwgp_int8.so`, the same `wq8_*` C ABI,
loaded with ctypes).  W is the checkpoint's INT8 (N, K) matrix; it is never dequantized or copied.

Paths (same names and meaning as the reference):
  'lines' / 'small'  1-4 / up to 32 tokens: unquantized activations, weights streamed once and converted exactly on the fly;
  'exact'            INT8 x INT8 on the exact split x ~= scale * (hi + lo / 254): two tensor-core passes, full precision;
  'block'            one INT8 pass with one FP32 scale per token and 128-element block of K;
  'row'              one INT8 pass with one scale per token, on request only.
linear() picks the fastest full-precision path while it costs at most EXACT_TOLERANCE more than 'block' (always with precise=True);
the choice is timed once per GPU, shape, input operation and token-count bucket and cached on disk.

There is no CPU or PyTorch fallback: every function raises if the CUDA library is not loaded.
"""
import ctypes
import functools
import json
import os
import time
from contextvars import ContextVar
from pathlib import Path

import torch

# Rows are quantized in chunks whose INT8 copy stays below this many bytes.  The reference keeps 16 MiB (consumer GPUs); with 180 GB
# of HBM one chunk covers a whole video-length activation, so the GEMM runs as one persistent launch.
SCRATCH_BYTES = 1 << 30
MAX_GRID_Y = 65535  # kept for callers that chunk rows themselves; this library's quantizers take any row count
EXACT_TOLERANCE = 0.10
EXACT_ROWS, LINE_ROWS, SMALL_ROWS = 64, 2, 16            # untimed choices (CUDA graph capture, compilation)
LINE_MAX_ROWS, SMALL_MAX_ROWS, DECIDE_MAX_ROWS = 4, 32, 4096
ACTS = {None: 0, "rms_norm": 1, "swiglu": 2, "gelu": 3}
ABI = 11
_COUNTERS = 1024
_DTYPES = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}

_lib = None
_weight_groups = False
_sms = {}
_counters = {}          # device index -> zeroed split-K counters shared by its streams
_stream_counters = {}   # raw stream handle -> counters of a stream prepared with prepare_stream()
_sizes = (ctypes.c_int64 * 2)()


def default_library_path():
    return Path(__file__).with_name("libwgp_int8.so")


def weight_groups_supported():
    """Whether the loaded library takes weight scales per output channel and 128-element block of K, (N, ceil(K / 128))."""
    return _weight_groups


def segments_supported():
    """Whether the loaded library computes several linears of one input in one GEMM."""
    return False


def _require():
    if _lib is None:
        raise RuntimeError("wgpkernels_b200.int8: the CUDA library is not loaded; build it (python -m wgpkernels_b200.build) and call load_library()")
    return _lib


def load_library(path=None):
    """Loads libwgp_int8.so (raises when it is missing or has another ABI) and allocates the per-device split-K counters."""
    global _lib, _weight_groups
    location = Path(path or default_library_path()).resolve()
    if not location.exists():
        raise RuntimeError(f"INT8 library not found at {location}; build it with `python -m wgpkernels_b200.build`")
    lib = ctypes.CDLL(str(location))
    if lib.wq8_abi() != ABI:
        raise RuntimeError("INT8 GEMM library ABI mismatch; rebuild it")
    _weight_groups = bool(lib.wq8_features() & 1)
    p, i, i64, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
    lib.wq8_quantize.argtypes = [p, p, p, p, i, i, i64, i, i, i, p, f, p]
    lib.wq8_quantize_blocks.argtypes = [p, p, p, i, i, i64, i, i, i, p, f, p, p]
    lib.wq8_transform_rows.argtypes = [p, p, i, i, i64, i, i, i, p, f, p]
    lib.wq8_rotate_groups.argtypes = [p, p, i, i, i64, i, i, p]
    lib.wq8_gemm.argtypes = [p, p, p, p, p, p, p, p, p, i, i, i, i, i, i, i, p, p, p]
    lib.wq8_gemm_workspace.argtypes = [i, i, i, i, i, i, p]
    lib.wq8_gemm_workspace.restype = None
    lib.wq8_gemm_multi.argtypes = [p, p, p, p, p, p, p, i64, p, p, i, i64, i, i, i, i, i, i, p, p]
    lib.wq8_gemm_select.argtypes = [i, i, i, i, i]
    lib.wq8_small.argtypes = [p, i64, p, p, p, p, p, p, i, i, i, i, i, p, p, p]
    lib.wq8_small_workspace.argtypes = [i, i, i, i, p]
    lib.wq8_small_workspace.restype = None
    lib.wq8_gemv_lines.argtypes = [p, i64, p, p, p, p, p, p, i, i, i, i, p]
    lib.wq8_stream_planes_workspace.argtypes = [i, i, i, i]
    lib.wq8_stream_planes_workspace.restype = i64
    lib.wq8_stream_planes.argtypes = [p, i64, p, p, p, p, p, p, i, i, i, i, i, p, p]
    lib.wq8_l2_flush.argtypes = [i, i64, p]
    lib.wq8_l2_flush_release.restype = None
    lib.wq8_debug_block_sums.argtypes = [p, p, p, i, i, i, i, p]
    if torch.cuda.is_available():
        for index in range(torch.cuda.device_count()):
            _counters.setdefault(index, torch.zeros(_COUNTERS, dtype=torch.int32, device=torch.device("cuda", index)))
    _lib = lib
    return lib


def _check(code):
    if code:
        raise RuntimeError(f"INT8 GEMM launch failed (CUDA error {code})")


def _ptr(tensor):
    return None if tensor is None else tensor.data_ptr()


def _stream(device):
    return torch._C._cuda_getCurrentRawStream(device.index)


def _sm_count(device):
    count = _sms.get(device.index)
    if count is None:
        count = _sms[device.index] = torch.cuda.get_device_properties(device).multi_processor_count
    return count


def prepare_stream(stream):
    """Gives `stream` its own split-K counters so that its launches may overlap those of the device's other streams.  Call it outside
    CUDA graph capture, before the stream's first launch."""
    if stream.cuda_stream not in _stream_counters:
        counters = torch.zeros(_COUNTERS, dtype=torch.int32, device=stream.device)
        torch.cuda.current_stream(stream.device).synchronize()
        _stream_counters[stream.cuda_stream] = counters


def _zeroed_counters(device, size, stream):
    if size > _COUNTERS * 4:
        raise RuntimeError("INT8 GEMM split-K counters exceeded")
    counters = _stream_counters.get(stream)
    if counters is None:
        counters = _counters.get(device.index)
        if counters is None:
            counters = _counters[device.index] = torch.zeros(_COUNTERS, dtype=torch.int32, device=device)
    return counters


def _width(x, act):
    """K of the linear that x feeds: SwiGLU rows hold the gate and the value halves."""
    return x.shape[1] // 2 if act == "swiglu" else x.shape[1]


def _check_input(x, act):
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("the activation must be 2-D with unit column stride")
    if act not in ACTS:
        raise ValueError(f"unknown input operation {act!r}")


# ---------------------------------------------------------------------------------------------------------------------
# activation preparation
# ---------------------------------------------------------------------------------------------------------------------
def quantize_blocks(x, group=0, act=None, act_weight=None, eps=0.0):
    """INT8 of op(x) with one FP32 scale per row and 128-element block of K: (q (M, K), scales (M, ceil(K / 128)))."""
    lib = _require()
    _check_input(x, act)
    m, k = x.shape[0], _width(x, act)
    q = torch.empty((m, k), dtype=torch.int8, device=x.device)
    scale = torch.empty((m, (k + 127) // 128), dtype=torch.float32, device=x.device)
    _check(lib.wq8_quantize_blocks(x.data_ptr(), q.data_ptr(), scale.data_ptr(), m, k, x.stride(0), _DTYPES[x.dtype], group, ACTS[act],
                                   _ptr(act_weight), eps, None, _stream(x.device)))
    return q, scale


def quantize(x, group=0, hilo=False, act=None, act_weight=None, eps=0.0):
    """Row-wise INT8 of op(x): (hi, lo or None, FP32 row scales); with hilo, op(x) ~= scale * (hi + lo / 254)."""
    lib = _require()
    _check_input(x, act)
    m, k = x.shape[0], _width(x, act)
    hi = torch.empty((m, k), dtype=torch.int8, device=x.device)
    lo = torch.empty_like(hi) if hilo else None
    scale = torch.empty(m, dtype=torch.float32, device=x.device)
    _check(lib.wq8_quantize(x.data_ptr(), hi.data_ptr(), _ptr(lo), scale.data_ptr(), m, k, x.stride(0), _DTYPES[x.dtype], group, ACTS[act],
                            _ptr(act_weight), eps, _stream(x.device)))
    return hi, lo, scale


def transform_rows(x, group=0, act=None, act_weight=None, eps=0.0):
    """op(x), rotated, rounded once to x's dtype: the unquantized activation of the few-token paths."""
    lib = _require()
    _check_input(x, act)
    m, k = x.shape[0], _width(x, act)
    out = torch.empty((m, k), dtype=x.dtype, device=x.device)
    _check(lib.wq8_transform_rows(x.data_ptr(), out.data_ptr(), m, k, x.stride(0), _DTYPES[x.dtype], group, ACTS[act], _ptr(act_weight), eps,
                                  _stream(x.device)))
    return out


def rotate_groups(x, group):
    """ConvRot rotation in groups of 16, 64 or 256, rounded once to the input dtype."""
    lib = _require()
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    _check(lib.wq8_rotate_groups(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], x.stride(0), _DTYPES[x.dtype], group, _stream(x.device)))
    return out


class Prepared:
    """An activation prepared for one path: the unquantized rows of 'lines' / 'small', or the INT8 rows and scales of 'exact' / 'block' /
    'row'.  Rows can be sliced; one preparation serves every weight with the same K and group."""
    __slots__ = ("path", "x", "lo", "scale", "dtype")

    def __init__(self, path, x, lo, scale, dtype):
        self.path, self.x, self.lo, self.scale, self.dtype = path, x, lo, scale, dtype

    def rows(self, start, stop):
        cut = lambda t: None if t is None else t[start:stop]
        return Prepared(self.path, self.x[start:stop], cut(self.lo), cut(self.scale), self.dtype)


def prepare(x, group=0, path="block", act=None, act_weight=None, eps=0.0):
    """op(x) prepared once for `path`; x: 2-D BF16 / FP16, rows 16-byte aligned; act_weight in x's dtype."""
    if path in ("lines", "small"):
        ready = transform_rows(x, group, act, act_weight, eps) if act else rotate_groups(x, group) if group else x
        return Prepared(path, ready, None, None, x.dtype)
    if path == "block":
        q, scale = quantize_blocks(x, group, act, act_weight, eps)
        return Prepared(path, q, None, scale, x.dtype)
    if path not in ("exact", "row"):
        raise ValueError(f"unknown path {path!r}")
    hi, lo, scale = quantize(x, group, path == "exact", act, act_weight, eps)
    return Prepared(path, hi, lo, scale, x.dtype)


# ---------------------------------------------------------------------------------------------------------------------
# tile tuner and its cache
# ---------------------------------------------------------------------------------------------------------------------
# (variant, split) candidates per mode; the first is the untuned default.  The variant numbers keep the reference's MODE meaning
# (row 0/2/6, exact 1/7, block 10/11, block+g 12/13, exact+g 14); what differs between the variants of a mode is this library's own:
# 10 / 12 convert block sums with the exact magic-number add, 11 / 13 with the conversion instruction.
_CANDIDATES = {"row": ((0, 0),), "exact": ((1, 0),), "block": ((10, 0), (11, 0)), "exact+g": ((14, 0),), "block+g": ((12, 0), (13, 0))}
_MODES = {0: "row", 2: "row", 6: "row", 1: "exact", 7: "exact", 10: "block", 11: "block", 12: "block+g", 13: "block+g", 14: "exact+g"}
_TUNING_VERSION = 1
_TUNING_PATH = Path(os.environ.get("WGPKERNELS_B200_CACHE") or Path.home() / ".cache" / "wgpkernels_b200" / "int8_tuning.json")
_tuned = None
_path_tuning = ContextVar("wgpkernels_b200_int8_path_tuning", default=False)


@functools.cache
def _device_name(index):
    return torch.cuda.get_device_name(index)


def _rows_bucket(m):
    """Multiples of 64 up to 4096 rows, then the next power of two up to 16384: tile and wave counts only matter for a few waves."""
    return -(-m // 64) * 64 if m <= 4096 else min(1 << (m - 1).bit_length(), 16384)


def _path_bucket(m):
    return m if m <= 16 else -(-m // 8) * 8 if m <= 128 else _rows_bucket(m)


def _cache():
    global _tuned
    if _tuned is None:
        try:
            payload = json.loads(_TUNING_PATH.read_text(encoding="utf-8"))
            _tuned = payload["configs"] if payload.get("version") == _TUNING_VERSION else {}
        except (OSError, ValueError, KeyError, AttributeError):
            _tuned = {}
    return _tuned


def _save_cache():
    try:
        _TUNING_PATH.parent.mkdir(parents=True, exist_ok=True)
        temporary = _TUNING_PATH.with_suffix(f".{os.getpid()}.tmp")
        temporary.write_text(json.dumps({"version": _TUNING_VERSION, "configs": _tuned}, indent=1), encoding="utf-8")
        os.replace(temporary, _TUNING_PATH)  # ranks of a multi-GPU job write the same file
    except OSError as error:
        print(f"[WGPKernels-B200] Could not save the INT8 tuning cache {_TUNING_PATH}: {error}")


def _capturing():
    return torch.cuda.is_current_stream_capturing() or torch.compiler.is_compiling()


def _best_of(launches, device):
    """Best time in ms of each launch(): one warm-up each, then three rounds in alternating order, each timed launch after a read of
    twice the L2 size from the library's own buffer (cold weights, as inside a model); back-to-back launches without that buffer."""
    lib = _require()
    names = list(launches)
    for name in names:
        launches[name]()
    flush_bytes, stream = 2 * torch.cuda.get_device_properties(device).L2_cache_size, _stream(device)
    cold = lib.wq8_l2_flush(device.index, flush_bytes, stream) == 0
    timings = {name: float("inf") for name in names}
    try:
        for round_index in range(3):
            for name in (names if round_index % 2 == 0 else names[::-1]):
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                if cold:
                    _check(lib.wq8_l2_flush(device.index, flush_bytes, stream))
                else:
                    torch.cuda._sleep(1_000_000)
                repeats = 1 if cold else 3
                start.record()
                for _ in range(repeats):
                    launches[name]()
                end.record()
                end.synchronize()
                timings[name] = min(timings[name], start.elapsed_time(end) / repeats)
    finally:
        lib.wq8_l2_flush_release()
    return timings


def _tuned_config(a, a_lo, sa, b, sb, bias, y, mode):
    """((variant, split), tuned?) of this shape bucket: cached, else timed on this call's operands (y may be overwritten), else the
    untuned default while a CUDA graph is captured or a graph is compiled."""
    (m, k), n = a.shape, b.shape[0]
    key = f"{mode}|{_rows_bucket(m)}x{n}x{k}|{_device_name(b.device.index)}"
    config = _cache().get(key)
    if config is not None:
        return tuple(config), True
    candidates = _CANDIDATES[mode]
    if _capturing():
        return candidates[0], False
    if len(candidates) == 1:
        _tuned[key] = list(candidates[0])
        return candidates[0], True
    started = time.time()
    log = not _path_tuning.get()
    label = f"INT8 GEMM {mode} {m}x{n}x{k}"
    if log:
        print(f"[WGPKernels-B200] Autotuning {label}...", flush=True)
    timings = _best_of({config: (lambda config: lambda: gemm(a, a_lo, sa, b, sb, bias, y.dtype, config[1], config[0], y))(config)
                        for config in candidates}, b.device)
    best_ms, best = min((ms, config) for config, ms in timings.items())
    _tuned[key] = list(best)
    _save_cache()
    if log:
        print(f"[WGPKernels-B200] Selected {label}: variant {best[0]}, split {best[1]} ({best_ms * 1000:.1f} us; tuned in "
              f"{time.time() - started:.2f} s).", flush=True)
    return best, True


_plans = {}  # (mode, M, N, K, device) -> (variant, split, workspace bytes, counter bytes)


def _plan(a, a_lo, sa, b, sb, bias, y, mode, scratch_output):
    (m, k), n = a.shape, b.shape[0]
    shape = (mode, m, n, k, b.device.index)
    plan = _plans.get(shape)
    if plan is not None:
        return plan
    (variant, split), tuned = _tuned_config(a, a_lo, sa, b, sb, bias, torch.empty_like(y) if scratch_output else y, mode)
    _require().wq8_gemm_workspace(m, n, k, variant, _sm_count(b.device), split, _sizes)
    plan = (variant, split, _sizes[0], _sizes[1])
    if tuned:
        _plans[shape] = plan
    return plan


def _weight_scale_groups(sb):
    if sb.dim() != 2:
        return False
    if not _weight_groups:
        raise RuntimeError("This INT8 library predates per-(n, k-block) weight scales; rebuild it")
    return True


def gemm(a, a_lo, sa, b, sb, bias, out_dtype, split=None, variant=None, out=None, mode=None, residual=None, residual_scale=None):
    """INT8 x INT8 GEMM with the fused epilogue.  mode: 'row' (sa per row), 'exact' (a_lo given) or 'block' (sa per row and 128-element
    block); inferred when omitted.  sb: (N) per channel, or (N, ceil(K / 128)) with 'exact' / 'block'.  residual (M, N) and residual_scale (N)
    in out_dtype: Y = residual + residual_scale * (A @ B.T + bias); out may be the residual.  out and residual may be column ranges of wider
    matrices (unit column stride, row stride a multiple of 8); out may also be a list of up to 8 such (M, N) views of equal row stride,
    which all receive the output (the ranks' buffers of an N-sharded layer, the peers' ones mapped into this process)."""
    lib = _require()
    m, k = a.shape
    n = b.shape[0]
    if k % 16:
        raise ValueError("K must be a multiple of 16")
    if out_dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("the output dtype must be float16 or bfloat16")
    sms = _sm_count(a.device)
    targets = list(out) if isinstance(out, (list, tuple)) else None
    y = torch.empty((m, n), dtype=out_dtype, device=a.device) if out is None else targets[0] if targets else out
    strided = targets is not None or y.stride(0) != n or (residual is not None and residual.stride(0) != n)
    if strided:
        targets = targets or [y]
        if not 1 <= len(targets) <= 8:
            raise ValueError("between 1 and 8 outputs")
        for t in targets:
            if tuple(t.shape) != (m, n) or t.dtype != out_dtype or t.stride(1) != 1 or t.stride(0) != y.stride(0):
                raise ValueError("every output must be an (M, N) view of the output dtype with unit column stride and the same row stride")
        if residual is not None and (tuple(residual.shape) != (m, n) or residual.stride(1) != 1):
            raise ValueError("the residual must be an (M, N) view with unit column stride")
    if variant is None and split is None:
        mode = mode or ("exact" if a_lo is not None else "block" if sa.dim() == 2 else "row")
        if _weight_scale_groups(sb):
            if mode == "row":
                raise ValueError("Weights with per-(n, k-block) scales run the 'block' or 'exact' path")
            mode += "+g"
        tuning_y = torch.empty((m, n), dtype=out_dtype, device=a.device) if strided else y  # the tuner may overwrite its output
        variant, split, workspace_bytes, counter_bytes = _plan(a, a_lo, sa, b, sb, bias, tuning_y, mode, residual is not None and not strided)
        del tuning_y
    else:
        split = 1 if split is None else split
        lib.wq8_gemm_workspace(m, n, k, variant, sms, split, _sizes)
        workspace_bytes, counter_bytes = _sizes[0], _sizes[1]
    workspace = torch.empty(workspace_bytes, dtype=torch.uint8, device=a.device) if workspace_bytes else None
    stream = _stream(a.device)
    counters = _zeroed_counters(a.device, counter_bytes, stream).data_ptr() if counter_bytes else None
    if strided:
        pointers = (ctypes.c_void_p * len(targets))(*[t.data_ptr() for t in targets])
        _check(lib.wq8_gemm_multi(a.data_ptr(), _ptr(a_lo), sa.data_ptr(), b.data_ptr(), sb.data_ptr(), _ptr(bias), _ptr(residual),
                                  residual.stride(0) if residual is not None else 0, _ptr(residual_scale), pointers, len(targets), y.stride(0),
                                  m, n, k, _DTYPES[out_dtype], variant, sms, _ptr(workspace), stream))
        return y
    _check(lib.wq8_gemm(a.data_ptr(), _ptr(a_lo), sa.data_ptr(), b.data_ptr(), sb.data_ptr(), _ptr(bias), _ptr(residual), _ptr(residual_scale),
                        y.data_ptr(), m, n, k, _DTYPES[out_dtype], variant, sms, split, _ptr(workspace), counters, stream))
    return y


def _stream_planes(lib, x, weight, scale, bias, residual, residual_scale, y):
    """At most 8 tokens: the activations split into INT8 digit planes (exact to 2^-14 of the largest of every 128 values), the weights on
    INT8 tensor cores as they are.  False when the shape or the alignment is not this kernel's."""
    m, k = x.shape
    n, sms = weight.shape[0], _sm_count(x.device)
    if m > 8 or x.stride(0) % 4 or x.data_ptr() % 8 or weight.data_ptr() % 16:
        return False
    size = lib.wq8_stream_planes_workspace(m, n, k, sms)
    if not size:
        return False
    workspace = torch.empty(size, dtype=torch.uint8, device=x.device)
    _check(lib.wq8_stream_planes(x.data_ptr(), x.stride(0), weight.data_ptr(), scale.data_ptr(), _ptr(bias), _ptr(residual), _ptr(residual_scale),
                                 y.data_ptr(), m, n, k, _DTYPES[x.dtype], sms, workspace.data_ptr(), _stream(x.device)))
    return True


def small(x, weight, scale, bias=None, residual=None, residual_scale=None, out=None):
    """Weight-only INT8 for at most 32 tokens: unquantized activations, FP32 accumulation.  K multiple of 64."""
    lib = _require()
    m, k = x.shape
    n = weight.shape[0]
    sms = _sm_count(x.device)
    y = torch.empty((m, n), dtype=x.dtype, device=x.device) if out is None else out
    if _stream_planes(lib, x, weight, scale, bias, residual, residual_scale, y):
        return y
    lib.wq8_small_workspace(m, n, k, sms, _sizes)
    slots = torch.empty(_sizes[0] // 4, dtype=torch.float32, device=x.device) if _sizes[0] else None
    stream = _stream(x.device)
    counters = _zeroed_counters(x.device, _sizes[1], stream).data_ptr() if _sizes[1] else None
    _check(lib.wq8_small(x.data_ptr(), x.stride(0), weight.data_ptr(), scale.data_ptr(), _ptr(bias), _ptr(residual), _ptr(residual_scale),
                         y.data_ptr(), m, n, k, _DTYPES[x.dtype], sms, _ptr(slots), counters, stream))
    return y


def gemv_lines(x, weight, scale, bias=None, residual=None, residual_scale=None, out=None):
    """One to four tokens, unquantized activations (K multiple of 4)."""
    lib = _require()
    m, k = x.shape
    y = torch.empty((m, weight.shape[0]), dtype=x.dtype, device=x.device) if out is None else out
    if _stream_planes(lib, x, weight, scale, bias, residual, residual_scale, y):
        return y
    _check(lib.wq8_gemv_lines(x.data_ptr(), x.stride(0), weight.data_ptr(), scale.data_ptr(), _ptr(bias), _ptr(residual), _ptr(residual_scale),
                              y.data_ptr(), m, weight.shape[0], k, _DTYPES[x.dtype], _stream(x.device)))
    return y


def linear_prepared(prepared, weight, scale, bias=None, residual=None, residual_scale=None, out=None):
    """Y = prepared @ (weight * scale).T + bias (or residual + residual_scale * (...)); weight: INT8 (N, K) matrix or a row range of one."""
    if prepared.path in ("lines", "small") and scale.dim() == 2:
        raise ValueError("Weights with per-(n, k-block) scales run the 'block' or 'exact' path")
    if prepared.path == "lines":
        return gemv_lines(prepared.x, weight, scale, bias, residual, residual_scale, out)
    if prepared.path == "small":
        return small(prepared.x, weight, scale, bias, residual, residual_scale, out)
    return gemm(prepared.x, prepared.lo, prepared.scale, weight, scale, bias, prepared.dtype, out=out, mode=prepared.path, residual=residual,
                residual_scale=residual_scale)


def linear_prepared_segments(prepared, weights, scales, biases, outputs):
    """outputs[s] = prepared @ (weights[s] * scales[s]).T + biases[s] for several weights of one prepared input."""
    for weight, scale, bias, out in zip(weights, scales, biases, outputs):
        linear_prepared(prepared, weight, scale, bias, out=out)
    return outputs


# ---------------------------------------------------------------------------------------------------------------------
# whole linear and the path policy
# ---------------------------------------------------------------------------------------------------------------------
def _gemm_path(x, weight, scale, bias, group, mode, act=None, act_weight=None, eps=0.0, residual=None, residual_scale=None, out=None):
    """'exact', 'block' or 'row' over row chunks whose quantized activations stay within SCRATCH_BYTES."""
    m, k = x.shape[0], weight.shape[1]
    out = torch.empty((m, weight.shape[0]), dtype=x.dtype, device=x.device) if out is None else out
    row_bytes = (2 * k if mode == "exact" else k) + 4 * (-(-k // 128) if mode == "block" else 1)
    rows = max(128, SCRATCH_BYTES // row_bytes // 128 * 128)
    for start in range(0, m, rows):
        stop = min(start + rows, m)
        prepared = prepare(x[start:stop], group, mode, act, act_weight, eps)
        rows_out = [t[start:stop] for t in out] if isinstance(out, (list, tuple)) else out[start:stop]
        linear_prepared(prepared, weight, scale, bias, None if residual is None else residual[start:stop], residual_scale, rows_out)
        del prepared
    return out


def _run(path, x, weight, scale, bias, group, act=None, act_weight=None, eps=0.0, residual=None, residual_scale=None, out=None):
    if path in ("lines", "small"):
        return linear_prepared(prepare(x, group, path, act, act_weight, eps), weight, scale, bias, residual, residual_scale, out)
    return _gemm_path(x, weight, scale, bias, group, path, act, act_weight, eps, residual, residual_scale, out)


def _precise_paths(m, k, groups=False):
    """Full-precision candidates; group-scaled weights only have 'exact'."""
    candidates = []
    if m <= LINE_MAX_ROWS and k % 4 == 0 and not groups:
        candidates.append("lines")
    if m <= SMALL_MAX_ROWS and k % 64 == 0 and not groups:
        candidates.append("small")
    return candidates + ["exact"]


def _static_path(m, k, precise, groups=False):
    if m <= LINE_ROWS and k % 4 == 0 and not groups:
        return "lines"
    if m <= SMALL_ROWS and k % 64 == 0 and not groups:
        return "small"
    return "exact" if precise or m <= EXACT_ROWS else "block"


_paths = {}  # (M, N, K, group, act, precise, device, grouped weights) -> path


def choose_path(x, weight, scale, bias=None, group=0, precise=False, act=None, act_weight=None, eps=0.0):
    """The fastest full-precision path while it costs at most EXACT_TOLERANCE more than 'block' (always one with precise=True), timed on
    this call's input once per GPU, shape, input operation and token-count bucket."""
    (m, k), n = (x.shape[0], weight.shape[1]), weight.shape[0]
    if m > DECIDE_MAX_ROWS and not precise:
        return "block"
    groups = _weight_scale_groups(scale)
    shape = (m, n, k, group, act, precise, x.device.index, groups)
    path = _paths.get(shape)
    if path is not None:
        return path
    key = (f"path{'+precise' if precise else ''}|{_path_bucket(m)}x{n}x{k}|g{group}{f'|{act}' if act else ''}{'|wgroups' if groups else ''}"
           f"|{_device_name(x.device.index)}")
    path = _cache().get(key)
    if path is not None:
        _paths[shape] = path
        return path
    if _capturing():
        return _static_path(m, k, precise, groups)
    candidates = _precise_paths(m, k, groups) + ([] if precise else ["block"])
    label = f"INT8 path {m}x{n}x{k}{f' ConvRot {group}' if group else ''}{f' {act}' if act else ''}{' (precise)' if precise else ''}"
    started = time.time()
    print(f"[WGPKernels-B200] Autotuning {label}...", flush=True)
    token = _path_tuning.set(True)
    try:
        timings = _best_of({path: (lambda path: lambda: _run(path, x, weight, scale, bias, group, act, act_weight, eps))(path) for path in candidates},
                           x.device)
    finally:
        _path_tuning.reset(token)
    full_ms, path = min((timings[p], p) for p in candidates if p != "block")
    if not precise and full_ms > (1 + EXACT_TOLERANCE) * timings["block"]:
        path = "block"
    _tuned[key] = _paths[shape] = path
    _save_cache()
    print(f"[WGPKernels-B200] Selected {label}: {path} ({timings[path] * 1000:.1f} us; tuned in {time.time() - started:.2f} s).", flush=True)
    return path


def linear(x, weight, scale, bias=None, group=0, precise=False, mode=None, act=None, act_weight=None, eps=0.0, residual=None, residual_scale=None,
           out=None):
    """Y = op(X) @ (INT8 weight * FP32 scales).T + bias for 2-D BF16 / FP16 X (rows 16-byte aligned, unit column stride), or residual +
    residual_scale * (...) (contiguous, X's dtype; out may be the residual).  act: None, 'rms_norm' (act_weight: K values in X's dtype or
    None; eps), 'swiglu' (X rows: gate | value) or 'gelu' (tanh approximation).  mode forces a path ('lines', 'small', 'exact', 'block',
    'row'); by default the path is chosen by choose_path()."""
    _check_input(x, act)
    path = mode or choose_path(x, weight, scale, bias, group, precise, act, act_weight, eps)
    return _run(path, x, weight, scale, bias, group, act, act_weight, eps, residual, residual_scale, out)


# ---------------------------------------------------------------------------------------------------------------------
# known-answer test
# ---------------------------------------------------------------------------------------------------------------------
def _reference(x, w, s, bias, group, act, act_weight, eps, residual, residual_scale, round_input):
    """FP32 PyTorch statement of linear() on x's device; round_input rounds op(x) to x's dtype as the few-token paths do."""
    v = x.float()
    if act == "swiglu":
        gate, value = v.chunk(2, dim=-1)
        v = torch.nn.functional.silu(gate) * value
    elif act == "rms_norm":
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * (1 if act_weight is None else act_weight.float())
    elif act == "gelu":
        v = torch.nn.functional.gelu(v, approximate="tanh")
    if group:
        v = _reference_rotation(v, group)
    if round_input:
        v = v.to(x.dtype).float()
    scale = s.repeat_interleave(128, dim=1)[:, :w.shape[1]] if s.dim() == 2 else s[:, None]
    out = v @ (w.float() * scale).T + bias.float()
    return out if residual is None else residual.float() + (1 if residual_scale is None else residual_scale.float()) * out


def _reference_rotation(v, group):
    h = torch.tensor([[1.0, 1, 1, -1], [1, 1, -1, 1], [1, -1, 1, 1], [-1, 1, 1, 1]], device=v.device)
    rotation = h
    while rotation.shape[0] < group:
        rotation = torch.kron(rotation, h)
    return (v.reshape(v.shape[0], -1, group) @ (rotation * group ** -0.5)).reshape(v.shape)


SELFTEST_CASES = ((1, "lines", 0, None, False), (5, "small", 0, None, False), (5, "small", 64, None, False), (40, "exact", 0, None, False),
                  (40, "block", 256, None, False), (40, "row", 16, None, False), (2, "lines", 0, "swiglu", True), (5, "small", 64, "rms_norm", True),
                  (40, "exact", 256, "rms_norm", False), (40, "block", 0, "swiglu", True), (40, "block", 16, "rms_norm", True),
                  (40, "exact", 64, None, True), (3, "lines", 64, "gelu", False), (5, "small", 0, "gelu", True), (40, "exact", 16, "gelu", False),
                  (40, "block", 256, "gelu", True), (40, "exact+g", 0, None, True), (40, "block+g", 64, "rms_norm", False),
                  (40, "block+g", 0, None, True))


def selftest(device=None):
    """Runs every kernel once on small inputs with fixed configurations (no tuning): None when the results match PyTorch, else a reason.
    Same case list and pass bars as the reference's selftest (relative Frobenius error 5e-3 on the full-precision paths, 3e-2 on
    'block' / 'row')."""
    _require()
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    generator = torch.Generator(device=device).manual_seed(0)
    variants = {"exact": 1, "block": 10, "row": 0, "exact+g": 14, "block+g": 12}
    for dtype in (torch.bfloat16, torch.float16):
        w = torch.randint(-127, 128, (96, 256), dtype=torch.int8, device=device, generator=generator)
        s = torch.rand(96, device=device, generator=generator) / 127
        s_groups = torch.rand(96, 2, device=device, generator=generator) / 127
        bias = torch.randn(96, dtype=dtype, device=device, generator=generator)
        norm_weight = (torch.rand(256, device=device, generator=generator) + 0.5).to(dtype)
        for m, path, group, act, with_residual in SELFTEST_CASES:
            x = torch.randn(m, 512 if act == "swiglu" else 256, dtype=dtype, device=device, generator=generator)
            act_weight = norm_weight if act == "rms_norm" else None
            residual = torch.randn(m, 96, dtype=dtype, device=device, generator=generator) * 4 if with_residual else None
            residual_scale = torch.rand(96, dtype=dtype, device=device, generator=generator) if with_residual else None
            scale = s_groups if path.endswith("+g") else s
            ref = _reference(x, w, scale, bias, group, act, act_weight, 1e-6, residual, residual_scale, path in ("lines", "small"))
            prepared = prepare(x, group, path.removesuffix("+g"), act, act_weight, 1e-6)
            if path in ("lines", "small"):
                y = linear_prepared(prepared, w, scale, bias, residual, residual_scale, residual)
            else:
                y = gemm(prepared.x, prepared.lo, prepared.scale, w, scale, bias, dtype, 0, variants[path], out=residual, residual=residual,
                         residual_scale=residual_scale)
            error = ((y.float() - ref).norm() / ref.norm()).item()
            if not error < (5e-3 if path in ("lines", "small", "exact", "exact+g") else 3e-2):
                return (f"{path} kernel mismatch ({dtype}, {m} rows, group {group}, {act or 'no input op'}{', residual' if with_residual else ''}): "
                        f"relative error {error:.3g}")
    torch.cuda.synchronize(device)
    return None


def debug_block_sums(a, b):
    """Exact INT32 block dot products (ceil(K / 128), M, N) computed by the tensor-core pipeline (parity tests)."""
    lib = _require()
    m, k = a.shape
    n = b.shape[0]
    sums = torch.empty(((k + 127) // 128, m, n), dtype=torch.int32, device=a.device)
    _check(lib.wq8_debug_block_sums(a.data_ptr(), b.data_ptr(), sums.data_ptr(), m, n, k, _sm_count(a.device), _stream(a.device)))
    return sums


def debug_status():
    """Status word of the GEMM pipeline (0 = no bounded wait gave up); synchronizes the device."""
    return _require().wq8_debug_status()


def debug_mma_peak(kind="i8", groups=4000, random_operands=True, device=None):
    """Issue-rate probe of the tensor pipe on the current device: (TOPS of the whole GPU, SM MHz during the probe, clocks per group of
    four M128 N256 MMAs).  kind "i8" (tcgen05 kind::i8) or "bf16" (kind::f16).  A measurement tool: allocates and synchronizes."""
    lib = _require()
    lib.wq8_debug_mma_peak.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.wq8_debug_mma_peak.restype = ctypes.c_int
    results = (ctypes.c_double * 3)()
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    _check(lib.wq8_debug_mma_peak(0 if kind == "i8" else 1, -groups if random_operands else groups, _sm_count(device), results))
    return results[0], results[1], results[2]
