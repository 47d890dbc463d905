"""Benchmark of the INT8 weight linear.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c4] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

A step is one whole linear of the workload through the public API (`wgpkernels_b200.int8.linear`: activation quantizer with the fused
input operation + INT8 GEMM with the fused epilogue) on seeded synthetic tensors of the benchmark configuration's shapes.  The default
workload is the fused-QKV projection of a 14B video DiT on the 'block' path: M = 32760 tokens, K = 5120, N = 15360, rms_norm fused,
bf16 output.  Metric: effective INT8 TOPS = 2 M N K / time, whole job.

  value      inputs resident in HBM; CUDA events around exactly K steps after W warm-up steps; max over ranks
  e2e        the same linear with HOST buffers through the package's call for them (wgpkernels_b200.host.HostLinear: pinned x -> device,
             linear, y -> pinned host, pipelined over 4096-row chunks on three streams), copies inside the timed region
  roofline   the GEMM kernel alone (events around its launches): achieved TOPS against the tensor-core peak
  cpu_baseline  the FP32 dequantize-and-matmul statement of the linear (the reference's own CPU path, restated) on the host cores,
             on a bounded band of rows of the same workload

With N > 1 the output channels are sharded over the ranks (each keeps N / g rows of the weight), every rank quantizes the replicated
activation and its GEMM writes its (M, N / g) output columns into the full-width buffers of all ranks (--gather fused, TMA stores over
NVLink from the tile epilogue) or the slices are all-gathered over NCCL afterwards (--gather nccl): total work is fixed ("strong"
scaling).  Only the JSON line goes to stdout; tuner messages go to stderr.

With N = 1 the same line also carries `paths`: the other paths the metric names, each a short run of its own (exact / row on the
default workload, configurations 2 and 4, the few-token paths of configuration 3 in GB/s, the fused q / k / v launch against three
launches) and `reference_cuda`: the reference's own CUDA library (built from its sources into oracle/_ref/, a baseline leg like
cpu_baseline, never on the product path) on the same tensors.  --no-paths skips them.
With N > 1 the line carries `parity` (a band of rows of every rank's gathered output against the unsharded linear computed on that
rank: mismatches must be 0), `sharded_consumer` (the output kept column-sharded, no exchange: what a consumer sharded the same way
reads) and `token_sharded` (rows sharded, weight replicated, no exchange), and e2e runs the row-sharded host pipeline.

--impl reference times the CPU statement of the linear only (rank 0; the other ranks exit).
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from wgpkernels_b200 import workloads  # noqa: E402

METRIC, UNIT = "int8_linear_effective_tops", "TOPS"
FEW_TOKEN = {"c3u": "SwiGLU MLP up projection: K=4096 N=28672", "c3d": "SwiGLU MLP down projection: K=14336 N=4096, act=swiglu on a (M, 28672) input"}
DESCRIPTIONS = {
    "c1": "block path, fused QKV projection of a 14B video DiT: M=32760 K=5120 N=15360, act=rms_norm, bf16 out",
    "c2": "block path, FFN down projection: M=32760 K=13824 N=5120, act=gelu, in-place residual, bf16 out",
    "c4": "block path, group-128 weight scales: M=16384 K=3072 N=12288, bf16 out",
}


def measured_peaks():
    try:
        return json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except (OSError, ValueError):
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.process = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                                            stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None

    def stop(self):
        if self.process is None:
            return None
        self.process.terminate()
        try:
            self.process.wait(5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        self.file.flush()
        self.file.seek(0)
        rows = [[cell.strip() for cell in line.split(",")] for line in self.file.read().splitlines() if line.count(",") >= 6]
        self.file.close()
        os.unlink(self.file.name)
        clocks = sorted(int(float(r[0])) for r in rows if r[0].replace(".", "").isdigit())
        if not clocks:
            return None
        busy = [c for c in clocks if c > 0]
        reasons = [name for position, name in ((3, "hw_slowdown"), (4, "hw_thermal_slowdown"), (5, "sw_thermal_slowdown"), (6, "sw_power_cap"))
                   if any(r[position].lower().startswith("active") for r in rows)]
        max_mhz = max((int(float(r[1])) for r in rows if r[1].replace(".", "").isdigit()), default=None)
        power = max((float(r[2]) for r in rows if r[2].replace(".", "").isdigit()), default=None)
        return {"sm_mhz": busy[len(busy) // 2], "sm_max_mhz": max_mhz, "samples": len(rows), "power_w_max": power, "reasons": reasons}


def profiled_traffic(name, mode, rows):
    """(DRAM bytes of one GEMM launch, where the figure comes from): dram__bytes_read + write of the committed ncu summary of the same
    kernel on a small case (its `traffic:` line names the workload, path, rows and bytes), scaled by the rows -- codes once, weights once
    per band of row tiles, outputs once all grow with the rows.  (None, why) when no summary covers this kernel."""
    import re
    for summary in sorted((ROOT / "profiles").glob("gemm_i8_tc_*.md")):
        found = re.search(r"^traffic: workload=(\w+) path=(\w+) rows=(\d+) dram_bytes=(\d+)", summary.read_text(), flags=re.M)
        if found and found.group(1) == name and found.group(2) == mode:
            return int(found.group(4)) * rows / int(found.group(3)), f"profiles/{summary.name}: {found.group(4)} bytes at {found.group(3)} rows, scaled by the rows"
    return None, "no committed ncu summary of this kernel and path"


def tensor_pipe_probe(device, groups=4000):
    """(INT8 TOPS of the whole GPU, SM MHz, clocks per group of four M128 N256 MMAs) from the probe library built beside the product
    library: MMAs alone on resident pseudo-random operands, all SMs.  A measurement tool: allocates and synchronizes."""
    import ctypes
    from wgpkernels_b200 import build as builder
    lib = ctypes.CDLL(str(builder.probe_library_file()))
    lib.wq8_probe_mma_peak.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    results = (ctypes.c_double * 3)()
    code = lib.wq8_probe_mma_peak(0, -groups, torch.cuda.get_device_properties(device).multi_processor_count, results)
    if code:
        raise RuntimeError(f"tensor-pipe probe failed ({code})")
    return results[0], results[1], results[2]


def cpu_reference_tops(name, rows, repeats):
    """The FP32 dequantize-and-matmul statement of the linear on the host cores, on the first `rows` rows of the workload."""
    from oracle import int8_oracle as oracle
    c = workloads.make(name, rows=rows)

    def once():
        return oracle.linear_reference(c.x, c.weight, c.scale, c.bias, 0, c.act, c.act_weight, c.eps, c.residual, c.residual_scale)

    once()
    times = []
    for _ in range(repeats):
        started = time.perf_counter()
        once()
        times.append(time.perf_counter() - started)
    best = sorted(times)[len(times) // 2]
    return c.ops / best / 1e12, best, c


def host_threads():
    """Every core this process may run on: launchers (torchrun) set OMP_NUM_THREADS=1, which would make a CPU baseline of rank 0 eight
    or more times slower than the same code started by hand."""
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    torch.set_num_threads(max(cores, 1))
    return torch.get_num_threads()


def run_reference(args, rank):
    if rank != 0:
        return
    threads = host_threads()
    rows = 512
    tops, seconds, c = cpu_reference_tops(args.workload, rows, max(args.steps, 1))
    sample = f"first {rows} of {workloads.make.__name__}('{args.workload}') rows, full K and N, FP32 dequantize + matmul (PyTorch CPU), median of {max(args.steps, 1)}"
    line = {"impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {DESCRIPTIONS[args.workload]}", "sample": sample},
            "cpu_baseline": {"value": tops, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), file=RESULT_STREAM, flush=True)


def measure_few_tokens(wq, device, workload, tokens, path, steps, warmup):
    """One few-token linear (BASELINE config 3) through the public API, L2 flushed before every timed launch (the 59-117 MB of weights
    would otherwise stay in the 126 MB L2), each launch with its own events: median ms, achieved GB/s on the algorithmic bytes, and the
    same byte count read by a plain streaming kernel timed the same way."""
    c = workloads.make(workload, rows=tokens)
    g = c.to(device)
    lib, stream = wq._require(), wq._stream(device)
    # 8 x L2: cold weights for the timed launch, and a flush long enough (about 0.15 ms) for the host to queue the next launch meanwhile
    flush_bytes = 8 * torch.cuda.get_device_properties(device).L2_cache_size

    def launch():
        return wq.linear(g.x, g.weight, g.scale, None, mode=path, act=c.act, precise=True)

    for _ in range(max(warmup, 3)):
        launch()
    # The host queues all steps without waiting: while the GPU runs a step's flush the next launches are already in the stream, so the
    # events of a step bracket its kernels and not the host's launch path (a launch into an idle GPU would time mostly that).
    def cold_ms(body):
        marks = []
        torch.cuda.synchronize()
        for _ in range(steps):
            wq._check(lib.wq8_l2_flush(device.index, flush_bytes, stream))
            first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            first.record()
            body()
            last.record()
            marks.append((first, last))
        torch.cuda.synchronize()
        return sorted(first.elapsed_time(last) for first, last in marks)[len(marks) // 2]

    ms = cold_ms(launch)
    # The same bytes read by a plain streaming kernel (the library's flush kernel on the cold start of its own buffer): what a launch
    # of this size can reach at all.  A 60-120 MB read lasts 10-20 us at the HBM rate, so launch, ramp-up and tail weigh on it.
    probe_ms = cold_ms(lambda: wq._check(lib.wq8_l2_flush(device.index, c.n * c.k, stream)))
    lib.wq8_l2_flush_release()
    n, k, m = c.n, c.k, tokens
    # algorithmic bytes of one call: weights once, scales, activations in, outputs out (the swiglu transform reads 2 x and writes 1 x more)
    moved = n * k + 4 * n + 2 * m * k + 2 * m * n + (6 * m * k if c.act == "swiglu" else 0)
    if path == "exact":
        moved += 3 * m * k  # the hi / lo INT8 copies written and read
    return {"ms": ms, "gbs": moved / (ms * 1e-3) / 1e9, "algorithmic_bytes": moved, "tops": 2 * m * n * k / (ms * 1e-3) / 1e12, "plain_read_ms": probe_ms,
            "n": n, "k": k, "act": c.act}


def run_few_tokens(args, rank):
    """Weight-streaming paths (BASELINE config 3): achieved HBM GB/s of one linear at 1-32 tokens, replicas only (rank 0 measures)."""
    if rank != 0:
        return
    from wgpkernels_b200 import int8 as wq
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    wq.load_library()
    m = args.tokens
    path = args.path or ("lines" if m <= 4 else "small")
    sampler = ClockSampler(0)
    r = measure_few_tokens(wq, device, args.workload, m, path, args.steps, args.warmup)
    clocks = sampler.stop()
    peaks = measured_peaks()
    peak = peaks["hbm_gbs"] if peaks else 6650.0
    line = {"metric": f"int8_{path}_weight_stream_gbs", "value": r["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": r["ms"], "higher_is_better": True, "scaling": "replicas only", "vs_baseline": None, "dtype": "bf16 x int8 -> f32" if path != "exact" else "int8",
            "data": "synthetic", "config": {"workload": f"{args.workload}: {FEW_TOKEN[args.workload]}", "tokens": m, "path": path,
                                            "l2": "flushed before every timed launch (read of 8 x L2 bytes)"},
            "effective_tops": r["tops"], "gpu_launches": args.steps * (2 if r["act"] or path == "exact" else 1), "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": r["gbs"], "peak": peak, "unit": "GB/s", "frac": r["gbs"] / peak, "traffic": None,
                         "algorithmic_bytes": r["algorithmic_bytes"], "peak_source": "MEASURED_PEAKS hbm_gbs, of measured" if peaks else "of fallback",
                         "plain_read": {"ms": r["plain_read_ms"], "gbs": r["n"] * r["k"] / (r["plain_read_ms"] * 1e-3) / 1e9,
                                        "frac_of_it": r["plain_read_ms"] / r["ms"] * r["algorithmic_bytes"] / (r["n"] * r["k"]),
                                        "what": "a plain read kernel over the weight's byte count, cold, same events"}}}
    print(json.dumps(line), file=RESULT_STREAM, flush=True)


def events_ms(body, steps, warmup=2):
    """Median-free mean ms of body() over `steps` back-to-back calls on the current stream (single GPU legs of `paths`)."""
    for _ in range(warmup):
        body()
    torch.cuda.synchronize()
    first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first.record()
    for _ in range(steps):
        body()
    last.record()
    torch.cuda.synchronize()
    return first.elapsed_time(last) / steps


class ReferenceCuda:
    """The reference's own CUDA library (oracle/_ref/libwgp_int8_ref.so, built from its unmodified source by oracle/Makefile) called
    through ctypes with the reference's own signatures: a BASELINE leg, like cpu_baseline -- never on the product path, never inside
    the timed region of `value`."""

    def __init__(self):
        import ctypes
        self.ctypes = ctypes
        path = ROOT / "oracle" / "_ref" / "libwgp_int8_ref.so"
        self.lib = ctypes.CDLL(str(path)) if path.exists() else None
        if self.lib is not None:
            p, i, i64, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
            self.lib.wq8_quantize_blocks.argtypes = [p, p, p, i, i, i64, i, i, i, p, f, p, p]
            self.lib.wq8_gemm.argtypes = [p, p, p, p, p, p, p, p, p, i, i, i, i, i, i, i, p, p, p]
            self.lib.wq8_gemm_workspace.argtypes = [i, i, i, i, i, i, p]
            self.lib.wq8_gemm_workspace.restype = None

    def linear_ms(self, g, act_code, eps, steps):
        """Quantizer + GEMM of the reference (variant 10, its untuned default for the block path) on the workload g: (quantizer ms, GEMM ms)."""
        ctypes, lib = self.ctypes, self.lib
        m, k, n = g.x.shape[0], g.weight.shape[1], g.weight.shape[0]
        device, stream = g.x.device, torch._C._cuda_getCurrentRawStream(g.x.device.index)
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        q = torch.empty((m, k), dtype=torch.int8, device=device)
        sa = torch.empty((m, (k + 127) // 128), dtype=torch.float32, device=device)
        scratch = torch.empty(m, dtype=torch.float32, device=device)
        y = torch.empty((m, n), dtype=g.x.dtype, device=device)
        sizes = (ctypes.c_int64 * 2)()
        lib.wq8_gemm_workspace(m, n, k, 10, sms, 0, sizes)
        slots = torch.empty(max(sizes[0], 16), dtype=torch.uint8, device=device)
        counters = torch.zeros(max(sizes[1] // 4, 1), dtype=torch.int32, device=device)
        ptr = lambda t: None if t is None else t.data_ptr()

        def quantize():
            for start in range(0, m, 65535):  # the reference puts rows on the grid's y axis
                rows = min(65535, m - start)
                code = lib.wq8_quantize_blocks(g.x[start:].data_ptr(), q[start:].data_ptr(), sa[start:].data_ptr(), rows, k, g.x.stride(0), 1, 0, act_code,
                                               ptr(g.act_weight), eps, scratch[start:].data_ptr(), stream)
                assert code == 0, code

        def gemm():
            code = lib.wq8_gemm(q.data_ptr(), None, sa.data_ptr(), g.weight.data_ptr(), g.scale.data_ptr(), ptr(g.bias), None, None, y.data_ptr(), m, n, k, 1, 10,
                                sms, 0, slots.data_ptr(), counters.data_ptr(), stream)
            assert code == 0, code

        return events_ms(quantize, steps), events_ms(gemm, steps)


def measure_paths(wq, device, c1, steps):
    """The other paths the metric names, each a short run of its own on one GPU: {name: {...}}.  c1: the default workload on the device."""
    paths = {}
    peaks = measured_peaks()
    tensor_peak = 2 * (peaks["bf16_tflops_sustained"] if peaks else 1400.0)
    hbm_peak = peaks["hbm_gbs"] if peaks else 6650.0

    def linear_entry(c, mode, ms, extra=None):
        tops = 2 * c.m * c.n * c.k / (ms * 1e-3) / 1e12
        entry = {"ms": ms, "tops": tops, "frac_of_tensor_peak": tops / tensor_peak, "mode": mode}
        entry.update(extra or {})
        return entry

    def whole(c, mode):
        residual = c.residual
        return lambda: wq.linear(c.x, c.weight, c.scale, c.bias, mode=mode, act=c.act, act_weight=c.act_weight, eps=c.eps, residual=residual,
                                 residual_scale=c.residual_scale, out=residual)

    # configuration 1 on the full-precision and the row paths
    for mode in ("exact", "row"):
        paths[f"c1_{mode}"] = linear_entry(c1, mode, events_ms(whole(c1, mode), steps))
    # the fused q / k / v form of configuration 1: one preparation, then one launch over the three (5120, K) weights against three launches
    prepared = wq.prepare(c1.x, 0, "block", c1.act, c1.act_weight, c1.eps)
    third = c1.n // 3
    weights = [c1.weight[s * third:(s + 1) * third] for s in range(3)]
    scales = [c1.scale[s * third:(s + 1) * third].contiguous() for s in range(3)]
    biases = [None if c1.bias is None else c1.bias[s * third:(s + 1) * third].contiguous() for s in range(3)]
    outputs = [torch.empty((c1.m, third), dtype=c1.x.dtype, device=device) for _ in range(3)]
    one_launch = events_ms(lambda: wq.linear_prepared_segments(prepared, weights, scales, biases, outputs), steps)
    three_launches = events_ms(lambda: [wq.linear_prepared(prepared, w, s, b, out=o) for w, s, b, o in zip(weights, scales, biases, outputs)], steps)
    paths["c1_qkv_segments"] = {"one_launch_ms": one_launch, "three_launches_ms": three_launches, "tops": 2 * c1.m * c1.n * c1.k / (one_launch * 1e-3) / 1e12,
                                "what": "GEMM only, q / k / v weights (3 x 5120 rows) of one prepared input: wq8_gemm_segments against three wq8_gemm"}
    del prepared, outputs
    # configuration 2: gelu + in-place residual
    c2 = workloads.make("c2").to(device)
    master = c2.residual.clone()
    ms = events_ms(lambda: (c2.residual.copy_(master), whole(c2, "block")()), steps)
    restore = events_ms(lambda: c2.residual.copy_(master), steps)
    quant = events_ms(lambda: wq.prepare(c2.x, 0, "block", c2.act, c2.act_weight, c2.eps), steps)
    quant_bytes = c2.m * c2.k * 3 + 4 * c2.m * ((c2.k + 127) // 128)
    paths["c2_block"] = linear_entry(c2, "block", ms - restore, {"quantizer_ms": quant, "quantizer_gbs": quant_bytes / (quant * 1e-3) / 1e9,
                                                                 "quantizer_frac_of_hbm": quant_bytes / (quant * 1e-3) / 1e9 / hbm_peak})
    del c2, master
    # configuration 4: group-128 weight scales, one preparation for three weights
    c4 = workloads.make("c4").to(device)
    for mode in ("block", "exact"):
        pairs = [(c4.weight, c4.scale)] + list(c4.extra_weights)

        def three(mode=mode, pairs=pairs):
            prepared = wq.prepare(c4.x, 0, mode)
            for weight, scale in pairs:
                wq.linear_prepared(prepared, weight, scale, c4.bias)

        ms = events_ms(three, steps)
        paths[f"c4_{mode}+g"] = {"ms": ms, "weights": len(pairs), "tops": 2 * c4.m * c4.n * c4.k * len(pairs) / (ms * 1e-3) / 1e12, "mode": mode + "+g",
                                 "frac_of_tensor_peak": 2 * c4.m * c4.n * c4.k * len(pairs) / (ms * 1e-3) / 1e12 / tensor_peak,
                                 "what": "prepare() once + linear_prepared on every weight"}
    del c4
    # configuration 3: few tokens, GB/s with a cold L2
    for workload in ("c3u", "c3d"):
        for tokens in (1, 4, 16, 32):
            path = "lines" if tokens <= 4 else "small"
            r = measure_few_tokens(wq, device, workload, tokens, path, max(steps, 10), 3)
            paths[f"{workload}_{tokens}"] = {"ms": r["ms"], "gbs": r["gbs"], "frac_of_hbm": r["gbs"] / hbm_peak, "path": path, "plain_read_ms": r["plain_read_ms"]}
    return paths


RESULT_STREAM = sys.stdout  # the one JSON line goes here; everything else the process prints (tuner messages) goes to stderr


def main():
    # Libraries under this process write to file descriptor 1 directly (NCCL prints its version there): the descriptor itself is pointed at
    # stderr and the JSON line goes to a copy of the original stdout.
    global RESULT_STREAM
    sys.stdout.flush()
    RESULT_STREAM = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    sys.stdout = sys.stderr
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--workload", default="c1", choices=sorted(DESCRIPTIONS) + sorted(FEW_TOKEN))
    parser.add_argument("--tokens", type=int, default=1, help="token count of the few-token workloads (c3u, c3d)")
    parser.add_argument("--gather", choices=["fused", "nccl"], default="fused", help="N > 1: how the output slices reach every rank: written "
                        "by the GEMM's tile epilogue into all ranks' buffers (fused), or an NCCL all-gather after the GEMM")
    parser.add_argument("--mode", choices=["block", "exact", "row"], default="block", help="path of the block workloads (default: the "
                        "'block' path the headline names; 'exact' is the two-pass full-precision path, 'row' one scale per token)")
    parser.add_argument("--rows", type=int, default=None, help="rows of the block workloads (default: the configuration's own; a smaller "
                        "case of the same shape is what a profiler capture wants)")
    parser.add_argument("--path", default=None, help="path of the few-token workloads: lines, small or exact (default: by token count)")
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--no-paths", action="store_true", help="skip the short runs of the other paths (`paths`, `reference_cuda`)")
    args = parser.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if args.workload in FEW_TOKEN:
        return run_few_tokens(args, rank)
    if args.impl == "reference":
        return run_reference(args, rank)

    import torch.distributed as dist
    from wgpkernels_b200 import dist as wdist
    from wgpkernels_b200 import int8 as wq
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    wq.load_library()
    warmup = max(args.warmup, 3)

    # ---- workload: the full problem; with several ranks every rank also keeps its output-channel slice of the weight ----------------
    name = args.workload
    _, k, n_total = workloads.SHAPES[name]
    c = workloads.make(name, rows=args.rows)
    m = c.m
    ops = 2 * m * n_total * k
    full = c.to(device)
    start, stop = wdist.shard_bounds(n_total, world, rank)
    if world > 1:
        layer = wdist.ShardedLinear.from_full(full.weight, full.scale, full.bias)
        cut = slice(start, stop)
        local_residual = None if full.residual is None else full.residual[:, cut]
        local_rscale = None if full.residual_scale is None else full.residual_scale[cut].contiguous()
    else:
        layer = None
    g = full
    in_place = g.residual is not None
    residual_master = g.residual.clone() if in_place else None
    common = dict(mode=args.mode, act=c.act, act_weight=g.act_weight, eps=c.eps)

    def step(x):
        if in_place:
            g.residual.copy_(residual_master)  # restore the tensor the epilogue overwrites (outside the operator, inside the step)
        if layer is None:
            return wq.linear(x, g.weight, g.scale, g.bias, residual=g.residual, residual_scale=g.residual_scale, out=g.residual if in_place else None, **common)
        if args.gather == "fused":  # every rank's GEMM writes its columns into all ranks' (M, N) buffers: no collective on the data
            return layer(x, gather="fused", residual=local_residual, residual_scale=local_rscale, **common)
        return layer(x, gather="full", residual=local_residual, residual_scale=local_rscale, **common)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(body, steps):
        """ms of `steps` iterations of body(), events on the current stream, max over ranks."""
        barrier()
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first.record()
        for _ in range(steps):
            body()
        last.record()
        barrier()
        ms = first.elapsed_time(last)
        if world > 1:
            slowest = torch.tensor([ms], device=device)
            dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
            ms = slowest.item()
        return ms

    for _ in range(warmup):
        y = step(g.x)
    sampler = ClockSampler(local_rank) if rank == 0 else None

    # ---- value: inputs resident in HBM ------------------------------------------------------------------------------------
    # One GPU: the quantizer and the GEMM are timed inside these very calls (events recorded from linear()'s stage hook).
    inner = []
    if world == 1:
        def hooked_step():
            begin = torch.cuda.Event(enable_timing=True)
            begin.record()
            stamps = [begin]
            wq.stage_hook = lambda tag: (stamps.append(torch.cuda.Event(enable_timing=True)), stamps[-1].record())
            step(g.x)
            wq.stage_hook = None
            inner.append(stamps)
        total_ms = timed(hooked_step, args.steps)
    else:
        total_ms = timed(lambda: step(g.x), args.steps)

    # ---- kernel breakdown: events around the quantizer and the GEMM of every step -------------------------------------------
    marks = []
    own = (g.weight, g.scale, g.bias) if layer is None else (layer.weight, layer.scale, layer.bias)
    own_residual = g.residual if layer is None else local_residual
    own_rscale = g.residual_scale if layer is None else local_rscale

    def split_step():
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        prepared = wq.prepare(g.x, 0, args.mode, c.act, g.act_weight, c.eps)
        e1.record()
        wq.linear_prepared(prepared, *own, own_residual, own_rscale, None)
        e2.record()
        marks.append((e0, e1, e2))

    if inner and all(len(stamps) == 3 for stamps in inner):
        quant_ms = sum(a.elapsed_time(b) for a, b, _ in inner) / len(inner)
        gemm_ms = sum(b.elapsed_time(d) for _, b, d in inner) / len(inner)
    else:  # several ranks (the step's GEMM also stores to the peers), or more than one band of rows: a pass of its own
        timed(split_step, args.steps)
        quant_ms = sum(a.elapsed_time(b) for a, b, _ in marks) / len(marks)
        gemm_ms = sum(b.elapsed_time(d) for _, b, d in marks) / len(marks)
    status = wq.debug_status()

    # ---- several ranks: is the gathered output the unsharded linear's?  and the forms without an exchange -----------------------
    parity = sharded_consumer = token_sharded = None
    if world > 1:
        band = slice(max(m // 2 - 320, 0), min(m // 2 + 320, m))  # rows on both sides of tile edges, all N columns
        gathered = step(g.x)
        torch.cuda.synchronize()
        if in_place:
            g.residual.copy_(residual_master)
        expected = wq.linear(g.x[band], g.weight, g.scale, g.bias, residual=None if g.residual is None else g.residual[band].clone(),
                             residual_scale=g.residual_scale, **common)
        mismatches = (gathered[band] != expected).sum().to(torch.int64)
        dist.all_reduce(mismatches)
        parity = {"rows": band.stop - band.start, "columns": n_total, "ranks": world, "mismatches": int(mismatches.item()),
                  "what": "every rank: its gathered (M, N) output on this band of rows against the unsharded linear computed on that rank, element for element"}
        consumer_step = lambda: layer(g.x, gather=None, residual=local_residual, residual_scale=local_rscale, **common)
        for _ in range(2):
            consumer_step()  # the tile tuner runs on the first call of a shape: outside the timed region
        consumer_ms = timed(consumer_step, args.steps)
        sharded_consumer = {"ms_per_step": consumer_ms / args.steps, "value": ops * args.steps / (consumer_ms * 1e-3) / 1e12, "unit": UNIT,
                            "what": "output kept column-sharded (M, N / g) on each rank, no exchange: the form a consumer sharded the same way reads "
                                    "(attention heads of a fused q / k / v projection)"}
        per_rank = -(-m // world)
        rows = slice(min(rank * per_rank, m), min((rank + 1) * per_rank, m))
        token_residual = None if g.residual is None else g.residual[rows]
        token_step = lambda: wq.linear(g.x[rows], g.weight, g.scale, g.bias, residual=token_residual, residual_scale=g.residual_scale, **common)
        for _ in range(2):
            token_step()
        token_ms = timed(token_step, args.steps)
        token_sharded = {"ms_per_step": token_ms / args.steps, "value": ops * args.steps / (token_ms * 1e-3) / 1e12, "unit": UNIT,
                         "what": "rows sharded (M / g tokens per rank), weight replicated, full-width output rows on their rank, no exchange"}

    # ---- e2e: host buffers, copies inside the timed region ----------------------------------------------------------------------
    e2e = None
    if not args.no_e2e:
        if world == 1:
            # the package's call for host-resident activations: copy in, linear and copy out pipelined over chunks of 4096 rows
            from wgpkernels_b200.host import HostLinear
            host_x = c.x.pin_memory()
            host_y = torch.empty((m, n_total), dtype=c.x.dtype).pin_memory()
            host_linear = HostLinear(g.weight, g.scale, g.bias, chunk_rows=4096)
            h2d, d2h = host_x.numel() * host_x.element_size(), host_y.numel() * host_y.element_size()

            def e2e_step():
                host_linear(host_x, host_y, residual=g.residual, residual_scale=g.residual_scale, **common)
            call = "wgpkernels_b200.host.HostLinear (pinned host x -> pinned host y, 4096-row chunks pipelined on three streams)"
        else:
            # rows sharded over the ranks, host buffers shared by the processes: every GPU moves and multiplies its own band only
            from wgpkernels_b200.host import ShardedHostLinear
            sharded_host = ShardedHostLinear(g.weight, g.scale, g.bias, rows=m, k=g.x.shape[1], dtype=c.x.dtype, chunk_rows=2048,
                                             tag=os.environ.get("MASTER_PORT", "0"))
            if rank == 0:
                sharded_host.x.copy_(c.x)
            barrier()
            h2d, d2h = sharded_host.h2d_bytes, sharded_host.d2h_bytes
            band_residual = None if g.residual is None else g.residual[sharded_host.start:sharded_host.stop]

            def e2e_step():
                sharded_host(residual=band_residual, residual_scale=g.residual_scale, **common)
            call = ("wgpkernels_b200.host.ShardedHostLinear (host x and y shared by the ranks; rank r copies in, multiplies and copies out rows "
                    "[r M / g, (r + 1) M / g) with the replicated weight, 2048-row chunks pipelined on three streams)")

        for _ in range(2):
            e2e_step()
        e2e_steps = max(3, min(args.steps, 10))
        e2e_ms = timed(e2e_step, e2e_steps)
        e2e = {"value": ops * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_ms / e2e_steps, "call": call}
        if world > 1:
            check = wq.linear(g.x[sharded_host.start:sharded_host.stop], g.weight, g.scale, g.bias, residual=band_residual, residual_scale=g.residual_scale,
                              **common) if not in_place else None
            if check is not None:
                wrong = (sharded_host.y[sharded_host.start:sharded_host.stop].to(device) != check).sum().to(torch.int64)
                dist.all_reduce(wrong)
                e2e["mismatches"] = int(wrong.item())
            sharded_host.close()
    clocks = sampler.stop() if sampler else None

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- report ----------------------------------------------------------------------------------------------------------------------
    peaks = measured_peaks()
    local_ops = 2 * m * (stop - start) * k
    achieved = local_ops / (gemm_ms * 1e-3) / 1e12
    if peaks:
        # the step is a long-running loop under the power cap: the sustained figure; kind::i8 issues at twice the 16-bit rate
        peak, peak_source = 2 * peaks["bf16_tflops_sustained"], "2 x MEASURED_PEAKS bf16_tflops_sustained (INT8 MMA rate = 2 x BF16), of measured"
    else:
        peak, peak_source = 2 * 1400.0, "2 x 1.4 PFLOP/s sustained bf16, of fallback"
    traffic, traffic_source = profiled_traffic(name, args.mode, m) if world == 1 else (None, None)
    local_m_bytes = m * k * (2 if args.mode == "exact" else 1) + 4 * m * ((k + 127) // 128 if args.mode == "block" else 1) + (stop - start) * k + 4 * (stop - start) + 2 * m * (stop - start)
    launches_per_step = 2 + (1 if g.scale.dim() == 2 else 0)  # quantizer, GEMM, and the regrouping of group-scaled weight scales
    quant_bytes = m * k * (2 if c.act != "swiglu" else 4) + m * k * (2 if args.mode == "exact" else 1) + 4 * m * ((k + 127) // 128 if args.mode == "block" else 1)
    line = {
        "metric": METRIC, "value": ops * args.steps / (total_ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "tokens_per_s": m * args.steps / (total_ms * 1e-3),
        "config": {"workload": f"{name}: {DESCRIPTIONS[name]}", "path": args.mode, "global_rows": m, "n": n_total, "k": k,
                   "parallelism": "single GPU" if world == 1 else (f"output channels sharded x{world}, replicated activation, output written into every rank's buffer by the GEMM epilogue (TMA "
                                   "stores over NVLink)" if args.gather == "fused" else
                                   f"output channels sharded x{world}, replicated activation, NCCL all_gather of the output"),
                   "l2": "no flush: the operands of a step (x, q, W, y: > 1 GB) exceed the 126 MB L2"},
        "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
        "roofline": {"kernel": f"gemm_i8_tc ({args.mode} mode)", "bound": "tensor", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                     "peak_source": peak_source, "nominal_dense_int8_tops": 4500.0, "traffic": traffic, "traffic_source": traffic_source,
                     "algorithmic_bytes": local_m_bytes, "kernel_ms": gemm_ms,
                     "quantizer": {"kernel_ms": quant_ms, "bound": "hbm", "achieved": quant_bytes / (quant_ms * 1e-3) / 1e9, "unit": "GB/s",
                                   "peak": peaks["hbm_gbs"] if peaks else 6650.0, "frac": quant_bytes / (quant_ms * 1e-3) / 1e9 / (peaks["hbm_gbs"] if peaks else 6650.0),
                                   "algorithmic_bytes": quant_bytes}},
        "device_status": status,
    }
    if world > 1:
        line["parity"], line["sharded_consumer"], line["token_sharded"] = parity, sharded_consumer, token_sharded
        line["sharding_policy"] = dict(wdist.worth_sharding(m, n_total, k, world),
                                       what="estimate for the replicated output: every rank receives (g - 1) / g of the (M, N) output over NVLink, "
                                            "which bounds the step whatever the GEMM does")
    if world == 1:
        # this library's own probe of the INT8 tensor pipe (MMAs alone on resident pseudo-random operands), measured now on this GPU: the
        # ceiling of any kind::i8 kernel at the clocks this board holds under that load
        probe_tops, probe_mhz, _ = tensor_pipe_probe(device)
        line["roofline"]["tensor_probe"] = {"int8_tops": probe_tops, "sm_mhz": probe_mhz, "frac": achieved / probe_tops,
                                            "what": "tcgen05 kind::i8 M128 N256 issue rate, all SMs, pseudo-random operands"}
        line["roofline"]["frac_of_probe"] = achieved / probe_tops
        if not args.no_paths and name == "c1" and args.rows is None:
            line["paths"] = measure_paths(wq, device, g, max(3, min(args.steps, 5)))
            reference = ReferenceCuda()
            if reference.lib is not None:
                ref_quant, ref_gemm = reference.linear_ms(g, {None: 0, "rms_norm": 1, "swiglu": 2, "gelu": 3}[c.act], c.eps, 3)
                line["reference_cuda"] = {"quantizer_ms": ref_quant, "gemm_ms": ref_gemm, "tops": ops / ((ref_quant + ref_gemm) * 1e-3) / 1e12,
                                          "speedup": (ref_quant + ref_gemm) / (total_ms / args.steps),
                                          "what": "the reference's own CUDA library (its block path: quantizer + variant 10 GEMM, sm_100 build of its mma.sync "
                                                  "kernels) on the same tensors and GPU, outside every timed region of this line"}
            else:
                line["reference_cuda"] = {"unavailable": "oracle/_ref/libwgp_int8_ref.so was not built (no reference checkout at build time)"}
    if not args.no_cpu_baseline and world == 1:
        rows = 512
        threads = host_threads()
        tops, seconds, _ = cpu_reference_tops(name, rows, 3)
        line["cpu_baseline"] = {"value": tops, "unit": UNIT, "cores": threads, "kind": "port", "seconds": seconds,
                                "sample": f"first {rows} rows of the workload, full K and N; FP32 dequantize + matmul (PyTorch CPU), median of 3"}
    print(json.dumps(line), file=RESULT_STREAM, flush=True)
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and parity["mismatches"]:
        sys.exit(3)


if __name__ == "__main__":
    main()
