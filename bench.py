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


def run_reference(args, rank):
    if rank != 0:
        return
    threads = torch.get_num_threads()
    rows = 512
    tops, seconds, c = cpu_reference_tops(args.workload, rows, max(args.steps, 1))
    sample = f"first {rows} of {workloads.make.__name__}('{args.workload}') rows, full K and N, FP32 dequantize + matmul (PyTorch CPU), median of {max(args.steps, 1)}"
    line = {"impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {DESCRIPTIONS[args.workload]}", "sample": sample},
            "cpu_baseline": {"value": tops, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), file=RESULT_STREAM, flush=True)


def run_few_tokens(args, rank):
    """Weight-streaming paths (BASELINE config 3): achieved HBM GB/s of one linear at 1-32 tokens, replicas only (rank 0 measures).
    The weights (59-117 MB) would fit the 126 MB L2, so L2 is flushed before every timed launch and each launch has its own events."""
    if rank != 0:
        return
    from wgpkernels_b200 import int8 as wq
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    wq.load_library()
    m = args.tokens
    path = args.path or ("lines" if m <= 4 else "small")
    c = workloads.make(args.workload, rows=m)
    g = c.to(device)
    lib, stream = wq._require(), wq._stream(device)
    # 8 x L2: cold weights for the timed launch, and a flush long enough (about 0.15 ms) for the host to queue the next launch meanwhile
    flush_bytes = 8 * torch.cuda.get_device_properties(device).L2_cache_size

    def launch():
        return wq.linear(g.x, g.weight, g.scale, None, mode=path, act=c.act, precise=True)

    for _ in range(max(args.warmup, 3)):
        launch()
    sampler = ClockSampler(0)
    # The host queues all steps without waiting: while the GPU runs a step's flush the next launches are already in the stream, so the
    # events of a step bracket its kernels and not the host's launch path (a launch into an idle GPU would time mostly that).
    marks = []
    torch.cuda.synchronize()
    for _ in range(args.steps):
        wq._check(lib.wq8_l2_flush(0, flush_bytes, stream))
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first.record()
        launch()
        last.record()
        marks.append((first, last))
    torch.cuda.synchronize()
    times = [first.elapsed_time(last) for first, last in marks]
    # The same bytes read by a plain streaming kernel (the library's flush kernel on the cold start of its own buffer), timed the same
    # way: what a launch of this size can reach at all.  A 60-120 MB read lasts 10-20 us at the HBM rate, so launch, ramp-up and tail
    # are a large part of any such launch.
    probe_marks = []
    for _ in range(args.steps):
        wq._check(lib.wq8_l2_flush(0, flush_bytes, stream))
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first.record()
        wq._check(lib.wq8_l2_flush(0, c.n * c.k, stream))
        last.record()
        probe_marks.append((first, last))
    torch.cuda.synchronize()
    probe_ms = sorted(first.elapsed_time(last) for first, last in probe_marks)[len(probe_marks) // 2]
    lib.wq8_l2_flush_release()
    clocks = sampler.stop()
    ms = sorted(times)[len(times) // 2]
    n, k = c.n, c.k
    # algorithmic bytes of one call: weights once, scales, activations in, outputs out (the swiglu transform reads 2 x and writes 1 x more)
    moved = n * k + 4 * n + 2 * m * k + 2 * m * n + (6 * m * k if c.act == "swiglu" else 0)
    if path == "exact":
        moved += 3 * m * k  # the hi / lo INT8 copies written and read
    peaks = measured_peaks()
    peak = peaks["hbm_gbs"] if peaks else 6650.0
    achieved = moved / (ms * 1e-3) / 1e9
    line = {"metric": f"int8_{path}_weight_stream_gbs", "value": achieved, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms, "higher_is_better": True, "scaling": "replicas only", "vs_baseline": None, "dtype": "bf16 x int8 -> f32" if path != "exact" else "int8",
            "data": "synthetic", "config": {"workload": f"{args.workload}: {FEW_TOKEN[args.workload]}", "tokens": m, "path": path,
                                            "l2": "flushed before every timed launch (read of 8 x L2 bytes)"},
            "effective_tops": 2 * m * n * k / (ms * 1e-3) / 1e12, "gpu_launches": args.steps * (2 if c.act or path == "exact" else 1), "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                         "algorithmic_bytes": moved, "peak_source": "MEASURED_PEAKS hbm_gbs, of measured" if peaks else "of fallback",
                         "plain_read": {"ms": probe_ms, "gbs": c.n * c.k / (probe_ms * 1e-3) / 1e9, "frac_of_it": probe_ms / ms * moved / (c.n * c.k),
                                        "what": "a plain read kernel over the weight's byte count, cold, same events"}}}
    print(json.dumps(line), file=RESULT_STREAM, flush=True)


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

    # ---- workload: full problem on one GPU, an output-channel slice per rank otherwise --------------------------------------
    name = args.workload
    _, k, n_total = workloads.SHAPES[name]
    start, stop = wdist.shard_bounds(n_total, world, rank)
    c = workloads.make(name, rows=args.rows, n_offset=start, n_rows=stop - start)
    m = c.m
    ops = 2 * m * n_total * k
    host_x = c.x.pin_memory()
    g = c.to(device)
    layer = wdist.ShardedLinear(g.weight, g.scale, g.bias, n_total) if world > 1 else None
    in_place = g.residual is not None
    residual_master = g.residual.clone() if in_place else None

    def step(x):
        if in_place:
            g.residual.copy_(residual_master)  # restore the tensor the epilogue overwrites (outside the operator, inside the step)
        if layer is None:
            return wq.linear(x, g.weight, g.scale, g.bias, mode=args.mode, act=c.act, act_weight=g.act_weight, eps=c.eps, residual=g.residual,
                             residual_scale=g.residual_scale, out=g.residual if in_place else None)
        if args.gather == "fused":  # every rank's GEMM writes its columns into all ranks' (M, N) buffers: no collective on the data
            return layer(x, gather="fused", mode=args.mode, act=c.act, act_weight=g.act_weight, eps=c.eps, residual=g.residual,
                         residual_scale=g.residual_scale)
        return layer(x, gather="full", mode=args.mode, act=c.act, act_weight=g.act_weight, eps=c.eps, residual=g.residual,
                     residual_scale=g.residual_scale, out=g.residual if in_place else None)

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
    total_ms = timed(lambda: step(g.x), args.steps)

    # ---- kernel breakdown: events around the quantizer and the GEMM of every step -------------------------------------------
    marks = []

    def split_step():
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        prepared = wq.prepare(g.x, 0, args.mode, c.act, g.act_weight, c.eps)
        e1.record()
        wq.linear_prepared(prepared, g.weight, g.scale, g.bias, g.residual, g.residual_scale, g.residual if in_place else None)
        e2.record()
        marks.append((e0, e1, e2))

    timed(split_step, args.steps)
    quant_ms = sum(a.elapsed_time(b) for a, b, _ in marks) / len(marks)
    gemm_ms = sum(b.elapsed_time(d) for _, b, d in marks) / len(marks)
    status = wq.debug_status()

    # ---- e2e: host buffers, copies inside the timed region ----------------------------------------------------------------------
    e2e = None
    if not args.no_e2e:
        host_y = torch.empty((m, n_total if world > 1 else g.weight.shape[0]), dtype=c.x.dtype).pin_memory()
        device_x = torch.empty_like(g.x)

        if world == 1:
            # the package's call for host-resident activations: copy in, linear and copy out pipelined over chunks of 4096 rows
            from wgpkernels_b200.host import HostLinear
            host_linear = HostLinear(g.weight, g.scale, g.bias, chunk_rows=4096)

            def e2e_step():
                host_linear(host_x, host_y, residual=g.residual, residual_scale=g.residual_scale, mode=args.mode, act=c.act,
                            act_weight=g.act_weight, eps=c.eps)
        else:
            def e2e_step():
                device_x.copy_(host_x, non_blocking=True)
                host_y.copy_(step(device_x), non_blocking=True)

        for _ in range(2):
            e2e_step()
        e2e_steps = max(3, min(args.steps, 10))
        e2e_ms = timed(e2e_step, e2e_steps)
        e2e = {"value": ops * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": host_x.numel() * host_x.element_size(),
               "d2h_bytes_per_step": host_y.numel() * host_y.element_size(), "ms_per_step": e2e_ms / e2e_steps,
               "call": "wgpkernels_b200.host.HostLinear (pinned host x -> pinned host y, 4096-row chunks pipelined on three streams)" if world == 1
               else "pinned host x -> device, ShardedLinear, device -> pinned host y"}
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
    # DRAM bytes of one GEMM launch: the ncu capture of the same kernel at M = 4096 rows of c1 (dram__bytes_read + write = 275.2 MB, its
    # summary is committed under profiles/) scaled by the rows: codes once, weights once per band of 2048 rows, outputs once.
    traffic, traffic_source = None, None
    if name == "c1" and world == 1 and args.mode == "block":
        traffic = 275.245e6 * m / 4096
        traffic_source = "ncu capture at 4096 rows (275.2 MB) x rows / 4096"
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
                                   "peak": peaks["hbm_gbs"] if peaks else 6650.0, "algorithmic_bytes": quant_bytes}},
        "device_status": status,
    }
    if world == 1:
        # this library's own probe of the INT8 tensor pipe (MMAs alone on resident pseudo-random operands), measured now on this GPU: the
        # ceiling of any kind::i8 kernel at the clocks this board holds under that load
        probe_tops, probe_mhz, _ = tensor_pipe_probe(device)
        line["roofline"]["tensor_probe"] = {"int8_tops": probe_tops, "sm_mhz": probe_mhz, "frac": achieved / probe_tops,
                                            "what": "tcgen05 kind::i8 M128 N256 issue rate, all SMs, pseudo-random operands"}
    if not args.no_cpu_baseline and world == 1:
        rows = 512
        tops, seconds, _ = cpu_reference_tops(name, rows, 3)
        line["cpu_baseline"] = {"value": tops, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "seconds": seconds,
                                "sample": f"first {rows} rows of the workload, full K and N; FP32 dequantize + matmul (PyTorch CPU), median of 3"}
    print(json.dumps(line), file=RESULT_STREAM, flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
