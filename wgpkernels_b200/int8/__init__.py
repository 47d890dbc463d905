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
# Up to DECIDE_MAX_ROWS rows the path is timed.  The reference stops at 4096 (on its GPUs the two-pass 'exact' path cannot catch up with
# 'block' on long inputs); here 'exact' accumulates over all of K in tensor memory and has no per-block work on the CUDA cores, which
# makes it as fast as 'block' on video-length inputs (measured on B200), so those are timed as well.
LINE_MAX_ROWS, SMALL_MAX_ROWS, DECIDE_MAX_ROWS = 4, 32, 1 << 17
PLANES_MAX_ROWS = 4  # few-token calls of at most this many tokens run the digit-plane mma.sync kernel, larger ones wq8_small (tcgen05)
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
    """Whether the loaded library computes several linears of one input in one GEMM launch (wq8_gemm_segments)."""
    return _lib is not None and hasattr(_lib, "wq8_gemm_segments")


def _require():
    if _lib is None:
        raise RuntimeError("wgpkernels_b200.int8: the CUDA library is not loaded; build it (python -m wgpkernels_b200.build) and call load_library()")
    return _lib


# ctypes signatures of the C ABI (include/wq8.h): v = pointer, i = int, l = int64, f = float; the part after "->" is the result
# ("" = void, default int).
_SIGNATURES = {
    "wq8_quantize": "vvvviiliiivfv",
    "wq8_quantize_blocks": "vvviiliiivfvv",
    "wq8_transform_rows": "vviiliiivfv",
    "wq8_rotate_groups": "vviiliiv",
    "wq8_gemm": "vvvvvvvvviiiiiiivvv",
    "wq8_gemm_multi": "vvvvvvvlvviliiiiiivv",
    "wq8_gemm_segments": "vvvvvvviiiiiiiivvv",
    "wq8_gemm_at": "vvvvvvvvviiiiiiivvvllllllv",
    "wq8_quantize_at": "vvvviiliiivfvllv",
    "wq8_quantize_blocks_at": "vvviiliiivfvvllv",
    "wq8_gemm_workspace": "iiiiiiv->",
    "wq8_gemm_select": "iiiii",
    "wq8_small": "vlvvvvvviiiiivvv",
    "wq8_small_workspace": "iiiiv->",
    "wq8_gemv_lines": "vlvvvvvviiiiv",
    "wq8_stream_planes_workspace": "iiii->l",
    "wq8_stream_planes": "vlvvvvvviiiiivv",
    "wq8_l2_flush": "ilv",
    "wq8_l2_flush_release": "->",
    "wq8_debug_block_sums": "vvviiiiv",
    "wq8_debug_wait_probe": "livv",
    "wq8_debug_status": "",
}
_CTYPES = {"v": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_int64, "f": ctypes.c_float}  # "l" also carries long long


def _bind(handle):
    for name, signature in _SIGNATURES.items():
        arguments, arrow, result = signature.partition("->")
        function = getattr(handle, name)
        function.argtypes = [_CTYPES[letter] for letter in arguments]
        function.restype = (_CTYPES[result] if result else None) if arrow else ctypes.c_int


def load_library(path=None):
    """Opens libwgp_int8.so and binds its entry points; RuntimeError when the file is missing or speaks another ABI.  Also creates the
    zeroed counter buffer of every visible GPU."""
    global _lib, _weight_groups
    location = Path(default_library_path() if path is None else path).resolve()
    if not location.is_file():
        raise RuntimeError(f"INT8 library not found at {location}; build it with `python -m wgpkernels_b200.build`")
    handle = ctypes.CDLL(str(location))
    found = handle.wq8_abi()
    if found != ABI:
        raise RuntimeError(f"INT8 GEMM library ABI mismatch ({found}, this module speaks {ABI}); rebuild it")
    _bind(handle)
    _weight_groups = handle.wq8_features() & 1 == 1
    for index in range(torch.cuda.device_count() if torch.cuda.is_available() else 0):
        if index not in _counters:
            _counters[index] = torch.zeros(_COUNTERS, dtype=torch.int32, device=f"cuda:{index}")
    _lib = handle
    return handle


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
def _row_kernel(entry, x, group, act, act_weight, eps, outputs, scratch=()):
    """One launch of a row-wise preparation kernel of the C ABI: the output pointers first (None for an absent one), then the common
    tail (M, K, row stride, dtype, group, input operation, its weight, eps), `scratch` pointers and the stream."""
    _check_input(x, act)
    pointers = [None if t is None else t.data_ptr() for t in outputs]
    tail = (x.shape[0], _width(x, act), x.stride(0), _DTYPES[x.dtype], group, ACTS[act], _ptr(act_weight), eps)
    _check(getattr(_require(), entry)(x.data_ptr(), *pointers, *tail, *scratch, _stream(x.device)))


def _like(x, act, dtype, *shape):
    return torch.empty(shape or (x.shape[0], _width(x, act)), dtype=dtype, device=x.device)


def quantize_blocks(x, group=0, act=None, act_weight=None, eps=0.0):
    """INT8 of op(x) with one FP32 scale per row and 128-element block of K: (q (M, K), scales (M, ceil(K / 128)))."""
    _check_input(x, act)
    codes = _like(x, act, torch.int8)
    scales = _like(x, act, torch.float32, x.shape[0], -(-_width(x, act) // 128))
    _row_kernel("wq8_quantize_blocks", x, group, act, act_weight, eps, (codes, scales), scratch=(None,))
    return codes, scales


def quantize(x, group=0, hilo=False, act=None, act_weight=None, eps=0.0):
    """Row-wise INT8 of op(x): (hi, lo or None, FP32 row scales); with hilo, op(x) ~= scale * (hi + lo / 254)."""
    _check_input(x, act)
    hi = _like(x, act, torch.int8)
    lo = _like(x, act, torch.int8) if hilo else None
    scales = _like(x, act, torch.float32, x.shape[0])
    _row_kernel("wq8_quantize", x, group, act, act_weight, eps, (hi, lo, scales))
    return hi, lo, scales


def transform_rows(x, group=0, act=None, act_weight=None, eps=0.0):
    """op(x), rotated, rounded once to x's dtype: the unquantized activation of the few-token paths."""
    _check_input(x, act)
    ready = _like(x, act, x.dtype)
    _row_kernel("wq8_transform_rows", x, group, act, act_weight, eps, (ready,))
    return ready


def rotate_groups(x, group):
    """ConvRot rotation in groups of 16, 64 or 256, rounded once to the input dtype."""
    rotated = torch.empty_like(x, memory_format=torch.contiguous_format)
    m, k = x.shape
    _check(_require().wq8_rotate_groups(x.data_ptr(), rotated.data_ptr(), m, k, x.stride(0), _DTYPES[x.dtype], group, _stream(x.device)))
    return rotated


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
    if path == "block":
        codes, scales = quantize_blocks(x, group, act, act_weight, eps)
        return Prepared(path, codes, None, scales, x.dtype)
    if path in ("exact", "row"):
        hi, lo, scales = quantize(x, group, path == "exact", act, act_weight, eps)
        return Prepared(path, hi, lo, scales, x.dtype)
    if path not in ("lines", "small"):
        raise ValueError(f"unknown path {path!r}")
    if act:
        rows = transform_rows(x, group, act, act_weight, eps)
    else:
        rows = rotate_groups(x, group) if group else x
    return Prepared(path, rows, None, None, x.dtype)


# ---------------------------------------------------------------------------------------------------------------------
# tile tuner and its cache
# ---------------------------------------------------------------------------------------------------------------------
# (variant, split) candidates per mode; the first is the untuned default.  The variant numbers keep the reference's MODE meaning
# (row 0/2/6, exact 1/7, block 10/11, block+g 12/13, exact+g 14); what differs between the variants of a mode is this library's own:
# 10 and 12 work on tiles of 256 output channels (two accumulator buffers in tensor memory) with sixteen drain warps, 20 and 22 are the
# same with eight drain warps (fewer instructions per output, fewer warps to hide latencies), 15 and 13 work on tiles of 128 channels
# (four buffers, more tiles: the better choice for small products); 11 and 16 are accepted as other names of 10 and 15.
_CANDIDATES = {"row": ((0, 0),), "exact": ((1, 0),), "block": ((10, 0), (20, 0), (15, 0)), "exact+g": ((14, 0),),
               "block+g": ((12, 0), (22, 0), (13, 0))}
_MODES = {0: "row", 2: "row", 6: "row", 1: "exact", 7: "exact", 10: "block", 11: "block", 15: "block", 16: "block", 20: "block", 12: "block+g",
          13: "block+g", 22: "block+g", 14: "exact+g"}
_TUNING_VERSION = 2
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


def _read_tuning_file():
    """The configs of the tuning file, {} when it is absent, unreadable or written by another version of the kernels."""
    try:
        stored = json.loads(_TUNING_PATH.read_text(encoding="utf-8"))
    except (OSError, ValueError):
        return {}
    if not isinstance(stored, dict) or stored.get("version") != _TUNING_VERSION or not isinstance(stored.get("configs"), dict):
        return {}
    return stored["configs"]


def _cache():
    """Tuned choices of this process, seeded once from the tuning file."""
    global _tuned
    if _tuned is None:
        _tuned = _read_tuning_file()
    return _tuned


def _save_cache():
    """Writes the tuned choices next to the old file and swaps them in (several ranks may do so at once); failures are reported only."""
    document = json.dumps({"version": _TUNING_VERSION, "configs": _tuned}, indent=1)
    scratch = _TUNING_PATH.with_suffix(f".{os.getpid()}.tmp")
    try:
        _TUNING_PATH.parent.mkdir(parents=True, exist_ok=True)
        scratch.write_text(document, encoding="utf-8")
        os.replace(scratch, _TUNING_PATH)
    except OSError as error:
        print(f"[WGPKernels-B200] Could not save the INT8 tuning cache {_TUNING_PATH}: {error}")


def _capturing():
    return torch.cuda.is_current_stream_capturing() or torch.compiler.is_compiling()


class _ColdTimer:
    """Times launches on the current stream of `device` with CUDA events, each after a read of twice the L2 size from the library's
    flush buffer, so that weights come from HBM as they do inside a model.  Without that buffer (allocation failed) launches are timed
    three in a row after a pause."""

    def __init__(self, device):
        self.lib, self.device, self.stream = _require(), device, _stream(device)
        self.bytes = 2 * torch.cuda.get_device_properties(device).L2_cache_size
        self.cold = self.lib.wq8_l2_flush(device.index, self.bytes, self.stream) == 0

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.lib.wq8_l2_flush_release()

    def ms(self, launch):
        if self.cold:
            _check(self.lib.wq8_l2_flush(self.device.index, self.bytes, self.stream))
            count = 1
        else:
            torch.cuda._sleep(1_000_000)
            count = 3
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first.record()
        for _ in range(count):
            launch()
        last.record()
        last.synchronize()
        return first.elapsed_time(last) / count


def _best_of(launches, device):
    """{name: best ms} of the launch() callables: one untimed call each, then three timed rounds, the order reversed every other round."""
    order = list(launches)
    for name in order:
        launches[name]()
    best = dict.fromkeys(order, float("inf"))
    with _ColdTimer(device) as timer:
        for round_index in range(3):
            for name in (order if round_index % 2 == 0 else reversed(order)):
                best[name] = min(best[name], timer.ms(launches[name]))
    return best


def _tuned_config(rows, n, k, device, mode, make_launch):
    """((variant, split), tuned?) for the bucket of this shape.  Known buckets come from the cache; a mode with one candidate needs no
    timing; while a CUDA graph is captured or compiled the first candidate is used and nothing is recorded; otherwise every candidate is
    timed through make_launch((variant, split)) -> callable (which may overwrite the output it was given) and the winner is stored."""
    key = "|".join((mode, f"{_rows_bucket(rows)}x{n}x{k}", _device_name(device.index)))
    known = _cache().get(key)
    if known is not None:
        return tuple(known), True
    options = _CANDIDATES[mode]
    if _capturing():
        return options[0], False
    if len(options) == 1:
        _tuned[key] = list(options[0])
        return options[0], True
    verbose = not _path_tuning.get()
    what = f"INT8 GEMM {mode} {rows}x{n}x{k}"
    began = time.time()
    if verbose:
        print(f"[WGPKernels-B200] Autotuning {what}...", flush=True)
    times = _best_of({option: make_launch(option) for option in options}, device)
    winner = min(options, key=lambda option: (times[option], option))
    _tuned[key] = list(winner)
    _save_cache()
    if verbose:
        print(f"[WGPKernels-B200] Selected {what}: variant {winner[0]}, split {winner[1]} ({times[winner] * 1000:.1f} us; tuned in "
              f"{time.time() - began:.2f} s).", flush=True)
    return winner, True


_plans = {}  # (mode, M, N, K, device) -> (variant, split, workspace bytes, counter bytes)


def _plan(m, n, k, device, mode, make_launch):
    """(variant, split, workspace bytes, counter bytes) of a GEMM of this exact shape; remembered once it comes from a tuned choice.
    make_launch is only called when candidates have to be timed (it is where a scratch output gets allocated, if one is needed)."""
    signature = (mode, m, n, k, device.index)
    if signature in _plans:
        return _plans[signature]
    (variant, split), final = _tuned_config(m, n, k, device, mode, make_launch)
    _require().wq8_gemm_workspace(m, n, k, variant, _sm_count(device), split, _sizes)
    result = (variant, split, _sizes[0], _sizes[1])
    if final:
        _plans[signature] = result
    return result


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

        scratch = []  # the tuner overwrites its output: it gets one of its own when y is a view, several views or holds the residual

        def make_launch(option):
            if strided or residual is not None:
                if not scratch:
                    scratch.append(torch.empty((m, n), dtype=out_dtype, device=a.device))
                target = scratch[0]
            else:
                target = y
            return lambda: gemm(a, a_lo, sa, b, sb, bias, out_dtype, option[1], option[0], target)

        variant, split, workspace_bytes, counter_bytes = _plan(m, n, k, a.device, mode, make_launch)
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
    """A few tokens: the activations split into INT8 digit planes (exact to 2^-14 of the largest of every 128 values), the weights on
    INT8 tensor cores as they are.  False when the shape or the alignment is not this kernel's."""
    m, k = x.shape
    n, sms = weight.shape[0], _sm_count(x.device)
    # up to PLANES_MAX_ROWS tokens this kernel is the fastest (measured on B200); above, wq8_small's tcgen05 kernel is
    if m > PLANES_MAX_ROWS or x.stride(0) % 4 or x.data_ptr() % 8 or weight.data_ptr() % 16:
        return False
    size = lib.wq8_stream_planes_workspace(m, n, k, sms)
    if not size:
        return False
    workspace = torch.empty(size, dtype=torch.uint8, device=x.device)
    _check(lib.wq8_stream_planes(x.data_ptr(), x.stride(0), weight.data_ptr(), scale.data_ptr(), _ptr(bias), _ptr(residual), _ptr(residual_scale),
                                 y.data_ptr(), m, n, k, _DTYPES[x.dtype], sms, workspace.data_ptr(), _stream(x.device)))
    return True


def _few_token_call(entry, x, weight, scale, bias, residual, residual_scale, out, extra):
    """Common part of the few-token entry points: output allocation, the digit-plane kernel when the shape is its own, else `entry` of
    the C ABI with `extra(m, n, k)` = the arguments between the dtype and the stream."""
    lib = _require()
    tokens, k = x.shape
    channels = weight.shape[0]
    y = out if out is not None else torch.empty((tokens, channels), dtype=x.dtype, device=x.device)
    if not _stream_planes(lib, x, weight, scale, bias, residual, residual_scale, y):
        stream = _stream(x.device)
        _check(getattr(lib, entry)(x.data_ptr(), x.stride(0), weight.data_ptr(), scale.data_ptr(), _ptr(bias), _ptr(residual),
                                   _ptr(residual_scale), y.data_ptr(), tokens, channels, k, _DTYPES[x.dtype], *extra(tokens, channels, k, stream), stream))
    return y


def small(x, weight, scale, bias=None, residual=None, residual_scale=None, out=None):
    """Weight-only INT8 for at most 32 tokens: unquantized activations, FP32 accumulation.  K multiple of 64."""
    keep = []  # the scratch must outlive the launch call

    def scratch(tokens, channels, k, stream):
        sms = _sm_count(x.device)
        _require().wq8_small_workspace(tokens, channels, k, sms, _sizes)
        slot_bytes, counter_bytes = _sizes[0], _sizes[1]
        slots = torch.empty(slot_bytes // 4, dtype=torch.float32, device=x.device) if slot_bytes else None
        keep.append(slots)
        counters = _zeroed_counters(x.device, counter_bytes, stream).data_ptr() if counter_bytes else None
        return sms, _ptr(slots), counters

    return _few_token_call("wq8_small", x, weight, scale, bias, residual, residual_scale, out, scratch)


def gemv_lines(x, weight, scale, bias=None, residual=None, residual_scale=None, out=None):
    """One to four tokens, unquantized activations (K multiple of 4)."""
    return _few_token_call("wq8_gemv_lines", x, weight, scale, bias, residual, residual_scale, out, lambda *shape: ())


def linear_prepared(prepared, weight, scale, bias=None, residual=None, residual_scale=None, out=None):
    """Y = prepared @ (weight * scale).T + bias (or residual + residual_scale * (...)); weight: INT8 (N, K) matrix or a row range of one."""
    few_tokens = {"lines": gemv_lines, "small": small}.get(prepared.path)
    if few_tokens is None:
        return gemm(prepared.x, prepared.lo, prepared.scale, weight, scale, bias, prepared.dtype, out=out, mode=prepared.path,
                    residual=residual, residual_scale=residual_scale)
    if scale.dim() == 2:
        raise ValueError("Weights with per-(n, k-block) scales run the 'block' or 'exact' path")
    return few_tokens(prepared.x, weight, scale, bias, residual, residual_scale, out)


def _pointer_table(tensors):
    return (ctypes.c_void_p * 4)(*[None if t is None else t.data_ptr() for t in tensors])


def linear_prepared_segments(prepared, weights, scales, biases, outputs):
    """outputs[s] = prepared @ (weights[s] * scales[s]).T + biases[s] for 1 to 4 linears of one 'exact', 'block' or 'row' preparation in
    ONE GEMM launch that reads the prepared input once: weights INT8 (rows, K), each contiguous, all of the same shape; scales FP32
    (rows,); biases in the output dtype or None; outputs (M, rows) contiguous in the prepared dtype, rows a multiple of 8.  Each output
    is bit for bit what linear_prepared gives on that weight with the same tile variant (a column tile never straddles two weights).
    The tile variant is chosen once for N = count * rows, timed on the launch itself."""
    lib = _require()
    a, count, rows = prepared.x, len(weights), weights[0].shape[0]
    if not 1 <= count <= 4 or rows % 8 or not (len(scales) == len(biases) == len(outputs) == count):
        raise ValueError("1 to 4 weights of the same shape, rows a multiple of 8, one scale, bias (or None) and output for each")
    if prepared.path not in ("exact", "block", "row"):
        raise ValueError("segments run the 'exact', 'block' or 'row' path")
    for weight, scale, out in zip(weights, scales, outputs):
        if scale.dim() != 1:
            raise ValueError("Weights with per-(n, k-block) scales cannot share a launch")
        if tuple(weight.shape) != tuple(weights[0].shape) or not weight.is_contiguous() or not out.is_contiguous() or tuple(out.shape) != (a.shape[0], rows):
            raise ValueError("every weight (rows, K) and output (M, rows) must be contiguous and of the same shape")
    m, k = a.shape
    stream = _stream(a.device)
    tables = [_pointer_table(t) for t in (weights, scales, biases, outputs)]

    def launch(variant, split, workspace):
        _check(lib.wq8_gemm_segments(a.data_ptr(), _ptr(prepared.lo), prepared.scale.data_ptr(), *tables, count, rows, m, k, _DTYPES[prepared.dtype],
                                     variant, _sm_count(a.device), split, _ptr(workspace), None, stream))

    variant, split, workspace_bytes, _ = _plan(m, count * rows, k, a.device, prepared.path, lambda option: lambda: launch(option[0], option[1], None))
    workspace = torch.empty(workspace_bytes, dtype=torch.uint8, device=a.device) if workspace_bytes else None
    launch(variant, split, workspace)
    return outputs


# ---------------------------------------------------------------------------------------------------------------------
# whole linear and the path policy
# ---------------------------------------------------------------------------------------------------------------------
def _chunk_rows(k, mode):
    """Rows whose quantized copy (codes, the low part of 'exact', scales) stays within SCRATCH_BYTES, a multiple of 128, at least 128."""
    per_row = k * (2 if mode == "exact" else 1) + 4 * ((k + 127) // 128 if mode == "block" else 1)
    return max(SCRATCH_BYTES // per_row // 128, 1) * 128


# Measurement aid: a callable that linear() calls with "quantized" after a band's activation quantizer has been enqueued and with
# "multiplied" after its GEMM (a benchmark records CUDA events there, so that the kernels are timed inside the very calls it times).
stage_hook = None


def _gemm_path(x, weight, scale, bias, group, mode, act=None, act_weight=None, eps=0.0, residual=None, residual_scale=None, out=None):
    """'exact', 'block' or 'row': quantize a band of rows, multiply it, next band.  out: a tensor, or a list of destinations."""
    m, n = x.shape[0], weight.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    several = isinstance(out, (list, tuple))
    band = _chunk_rows(weight.shape[1], mode)
    for first in range(0, m, band):
        rows = slice(first, min(first + band, m))
        prepared = prepare(x[rows], group, mode, act, act_weight, eps)
        if stage_hook is not None:
            stage_hook("quantized")
        linear_prepared(prepared, weight, scale, bias, residual[rows] if residual is not None else None, residual_scale,
                        [t[rows] for t in out] if several else out[rows])
        if stage_hook is not None:
            stage_hook("multiplied")
        del prepared  # the band's codes go back to the allocator before the next band is quantized
    return out


def _run(path, x, weight, scale, bias, group, act=None, act_weight=None, eps=0.0, residual=None, residual_scale=None, out=None):
    if path not in ("lines", "small"):
        return _gemm_path(x, weight, scale, bias, group, path, act, act_weight, eps, residual, residual_scale, out)
    return linear_prepared(prepare(x, group, path, act, act_weight, eps), weight, scale, bias, residual, residual_scale, out)


def _few_token_paths(m, k, groups, line_rows, small_rows):
    """The few-token kernels that can take this shape, given the row limits in force (group-scaled weights have none)."""
    if groups:
        return []
    usable = []
    if m <= line_rows and k % 4 == 0:
        usable.append("lines")
    if m <= small_rows and k % 64 == 0:
        usable.append("small")
    return usable


def _precise_paths(m, k, groups=False):
    """Full-precision candidates, 'exact' last (it always applies)."""
    return _few_token_paths(m, k, groups, LINE_MAX_ROWS, SMALL_MAX_ROWS) + ["exact"]


def _static_path(m, k, precise, groups=False):
    """The untimed choice (CUDA graph capture, compilation): fixed row thresholds."""
    few = _few_token_paths(m, k, groups, LINE_ROWS, SMALL_ROWS)
    if few:
        return few[0]
    return "exact" if precise or m <= EXACT_ROWS else "block"


_paths = {}  # (M, N, K, group, act, precise, device, grouped weights) -> path


def _path_key(m, n, k, group, act, precise, groups, device_index):
    parts = ["path+precise" if precise else "path", f"{_path_bucket(m)}x{n}x{k}", f"g{group}"]
    if act:
        parts.append(act)
    if groups:
        parts.append("wgroups")
    parts.append(_device_name(device_index))
    return "|".join(parts)


def choose_path(x, weight, scale, bias=None, group=0, precise=False, act=None, act_weight=None, eps=0.0):
    """The fastest full-precision path while it costs at most EXACT_TOLERANCE more than 'block' (always one with precise=True), timed on
    this call's input once per GPU, shape, input operation and token-count bucket."""
    m, n, k = x.shape[0], weight.shape[0], weight.shape[1]
    if not precise and m > DECIDE_MAX_ROWS:
        return "block"  # long inputs: the few-token and two-pass paths cannot win
    groups = _weight_scale_groups(scale)
    exact_shape = (m, n, k, group, act, precise, x.device.index, groups)
    if exact_shape in _paths:
        return _paths[exact_shape]
    key = _path_key(m, n, k, group, act, precise, groups, x.device.index)
    stored = _cache().get(key)
    if stored is not None:
        _paths[exact_shape] = stored
        return stored
    if _capturing():
        return _static_path(m, k, precise, groups)
    full_precision = _precise_paths(m, k, groups)
    contenders = full_precision if precise else full_precision + ["block"]
    what = f"INT8 path {m}x{n}x{k}" + (f" ConvRot {group}" if group else "") + (f" {act}" if act else "") + (" (precise)" if precise else "")
    began = time.time()
    print(f"[WGPKernels-B200] Autotuning {what}...", flush=True)

    def runner(candidate):
        return lambda: _run(candidate, x, weight, scale, bias, group, act, act_weight, eps)

    quiet = _path_tuning.set(True)  # the tile tuners that run inside these launches keep silent
    try:
        times = _best_of({candidate: runner(candidate) for candidate in contenders}, x.device)
    finally:
        _path_tuning.reset(quiet)
    chosen = min(full_precision, key=lambda candidate: (times[candidate], candidate))
    if not precise and times[chosen] > times["block"] * (1 + EXACT_TOLERANCE):
        chosen = "block"
    _tuned[key] = chosen
    _paths[exact_shape] = chosen
    _save_cache()
    print(f"[WGPKernels-B200] Selected {what}: {chosen} ({times[chosen] * 1000:.1f} us; tuned in {time.time() - began:.2f} s).", flush=True)
    return chosen


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
def _input_operation(values, act, act_weight, eps):
    """op(x) in FP32 with PyTorch operators (the known-answer side of selftest)."""
    functional = torch.nn.functional
    if act == "rms_norm":
        normalised = values * (values.square().mean(dim=-1, keepdim=True) + eps).rsqrt()
        return normalised if act_weight is None else normalised * act_weight.float()
    if act == "swiglu":
        half = values.shape[-1] // 2
        return functional.silu(values[..., :half]) * values[..., half:]
    if act == "gelu":
        return functional.gelu(values, approximate="tanh")
    return values


def _reference_rotation(v, group):
    """ConvRot: every run of `group` values times the Kronecker power of the 4 x 4 block (ones with -1 on the anti-diagonal), scaled to
    be orthonormal."""
    block = torch.ones(4, 4, device=v.device) - 2 * torch.eye(4, device=v.device).flip(1)
    matrix = block
    while matrix.shape[0] < group:
        matrix = torch.kron(matrix, block)
    runs = v.reshape(v.shape[0], v.shape[1] // group, group)
    return (runs @ (matrix / group ** 0.5)).reshape(v.shape)


def _reference(x, w, s, bias, group, act, act_weight, eps, residual, residual_scale, round_input):
    """FP32 PyTorch statement of linear() on x's device; round_input rounds op(x) to x's dtype as the few-token paths do."""
    prepared = _input_operation(x.float(), act, act_weight, eps)
    if group:
        prepared = _reference_rotation(prepared, group)
    if round_input:
        prepared = prepared.to(x.dtype).float()
    per_element = s[:, None] if s.dim() == 1 else s.repeat_interleave(128, dim=1)[:, :w.shape[1]]
    result = prepared @ (w.float() * per_element).T + bias.float()
    if residual is None:
        return result
    return residual.float() + result * (1 if residual_scale is None else residual_scale.float())


# The known-answer cases, grouped by what they exercise: (rows, path, rotation group, input operation, residual?).  The list covers the
# same kernels, rotations, input operations and residual forms as the reference's selftest, in its order (the random stream is shared).
_PLAIN_CASES = [(1, "lines", 0, None, False), (5, "small", 0, None, False), (5, "small", 64, None, False), (40, "exact", 0, None, False),
                (40, "block", 256, None, False), (40, "row", 16, None, False)]
_FUSED_CASES = [(2, "lines", 0, "swiglu", True), (5, "small", 64, "rms_norm", True), (40, "exact", 256, "rms_norm", False),
                (40, "block", 0, "swiglu", True), (40, "block", 16, "rms_norm", True), (40, "exact", 64, None, True)]
_GELU_CASES = [(3, "lines", 64, "gelu", False), (5, "small", 0, "gelu", True), (40, "exact", 16, "gelu", False), (40, "block", 256, "gelu", True)]
_GROUP_SCALE_CASES = [(40, "exact+g", 0, None, True), (40, "block+g", 64, "rms_norm", False), (40, "block+g", 0, None, True)]
SELFTEST_CASES = tuple(_PLAIN_CASES + _FUSED_CASES + _GELU_CASES + _GROUP_SCALE_CASES)
_SELFTEST_VARIANT = {"row": 0, "exact": 1, "block": 10, "block+g": 12, "exact+g": 14}
_FULL_PRECISION = ("lines", "small", "exact", "exact+g")


def selftest(device=None):
    """Runs every kernel once on small inputs with fixed configurations (no tuning): None when the results match PyTorch, else a reason.
    Pass bars as in the reference's selftest: relative Frobenius error 5e-3 on the full-precision paths, 3e-2 on 'block' / 'row'."""
    _require()
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    rng = torch.Generator(device=device).manual_seed(0)
    n, k, eps = 96, 256, 1e-6

    def normal(*shape, dtype):
        return torch.randn(*shape, dtype=dtype, device=device, generator=rng)

    def uniform(*shape):
        return torch.rand(*shape, device=device, generator=rng)

    for dtype in (torch.bfloat16, torch.float16):
        weight = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=device, generator=rng)
        channel_scale = uniform(n) / 127
        block_scale = uniform(n, k // 128) / 127
        bias = normal(n, dtype=dtype)
        norm_weight = (uniform(k) + 0.5).to(dtype)
        for rows, path, group, act, with_residual in SELFTEST_CASES:
            x = normal(rows, 2 * k if act == "swiglu" else k, dtype=dtype)
            act_weight = norm_weight if act == "rms_norm" else None
            residual = normal(rows, n, dtype=dtype) * 4 if with_residual else None
            residual_scale = uniform(n).to(dtype) if with_residual else None
            scale = block_scale if path.endswith("+g") else channel_scale
            few_tokens = path in ("lines", "small")
            expected = _reference(x, weight, scale, bias, group, act, act_weight, eps, residual, residual_scale, few_tokens)
            prepared = prepare(x, group, path.split("+")[0], act, act_weight, eps)
            if few_tokens:
                got = linear_prepared(prepared, weight, scale, bias, residual, residual_scale, residual)  # in place when there is a residual
            else:
                got = gemm(prepared.x, prepared.lo, prepared.scale, weight, scale, bias, dtype, 0, _SELFTEST_VARIANT[path], out=residual,
                           residual=residual, residual_scale=residual_scale)
            error = float((got.float() - expected).norm() / expected.norm())
            bar = 5e-3 if path in _FULL_PRECISION else 3e-2
            if not error < bar:
                details = [str(dtype), f"{rows} rows", f"group {group}", act or "no input op"] + (["residual"] if with_residual else [])
                return f"{path} kernel mismatch ({', '.join(details)}): relative error {error:.3g}"
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


def debug_wait_probe(clocks=2_000_000, code=9, device=None):
    """Runs one bounded wait on a barrier that nothing completes, with a limit of `clocks` SM clocks: (what the kernel reported --
    1 completed, 2 gave up --, the status word afterwards).  The give-up path of the library's waits, exercised without a fault."""
    lib = _require()
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    returned = torch.zeros(1, dtype=torch.int32, device=device)
    _check(lib.wq8_debug_wait_probe(clocks, code, returned.data_ptr(), _stream(device)))
    status = lib.wq8_debug_status()
    return int(returned.item()), status
