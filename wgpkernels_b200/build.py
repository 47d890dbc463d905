"""Ahead-of-time build of libwgp_int8.so for B200 (sm_100a), written next to the package's `int8` module:

    python -m wgpkernels_b200.build [--output PATH] [--verbose] [--jobs N] [--force]

A second, tiny library, libwgp_int8_probe.so, is built beside it: the tensor-pipe issue-rate probe that only the benchmark loads.

One architecture only: the GEMM uses tcgen05 / tensor-memory instructions that exist on sm_100a alone, so there is no PTX fallback.
The CUDA runtime is linked statically and only the C ABI is exported, so the library depends on the driver alone (the same properties
as the reference's build, wgpkernels/build.py:55-65 of WGPKernels).
"""
import argparse
import os
import subprocess
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
SOURCES = ("api.cu", "quantize.cu", "stream.cu", "stream_tc.cu", "gemm_tc.cu")
PROBE_SOURCES = ("probe.cu",)
HEADERS = ("common.cuh", "tc_ptx.cuh")
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")


def library_file():
    return PACKAGE / "int8" / "libwgp_int8.so"


def probe_library_file():
    return PACKAGE / "int8" / "libwgp_int8_probe.so"


def _stale(target, sources):
    if not target.exists():
        return True
    newest = max(p.stat().st_mtime for p in sources)
    return target.stat().st_mtime < newest


def build(output=None, nvcc="nvcc", verbose=False, jobs=None, force=False, sources=SOURCES):
    """Compiles `sources` into the shared library `output` (default: the product library; the probe library is built with it)."""
    if output is None and sources is SOURCES:
        build(probe_library_file(), nvcc, verbose, jobs, force, PROBE_SOURCES)
    target = Path(output or library_file()).resolve()
    csrc = PACKAGE / "csrc"
    inputs = [csrc / name for name in sources] + [csrc / name for name in HEADERS]
    if not force and not _stale(target, inputs):
        return target
    target.parent.mkdir(parents=True, exist_ok=True)
    common = [nvcc, "-O3", "-std=c++17", "-lineinfo", *ARCH_FLAGS, "-Xcompiler", "-fPIC,-fvisibility=hidden", "--cudart", "static"]
    if verbose:
        common += ["-Xptxas", "-v"]
    with tempfile.TemporaryDirectory(prefix="wgpkernels-b200-") as work:
        def compile_one(name):
            obj = Path(work) / (name + ".o")
            done = subprocess.run([*common, "-c", str(csrc / name), "-o", str(obj)], capture_output=True, text=True)
            if verbose or done.returncode:
                print(done.stdout + done.stderr)
            if done.returncode:
                raise RuntimeError(f"nvcc failed on {name}")
            return obj
        with ThreadPoolExecutor(max_workers=jobs or min(len(sources), os.cpu_count() or 1)) as pool:
            objects = list(pool.map(compile_one, sources))
        built = Path(work) / target.name
        subprocess.run([nvcc, "-shared", *ARCH_FLAGS, "--cudart", "static", "-Xcompiler", "-fPIC,-fvisibility=hidden",
                        *map(str, objects), "-o", str(built)], check=True)
        target.write_bytes(built.read_bytes())
    return target


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--output", type=Path, default=None)
    parser.add_argument("--nvcc", default="nvcc")
    parser.add_argument("--verbose", action="store_true", help="print register and shared memory usage (-Xptxas -v)")
    parser.add_argument("--jobs", type=int, default=None)
    parser.add_argument("--force", action="store_true")
    args = parser.parse_args()
    print(f"Built {build(args.output, args.nvcc, args.verbose, args.jobs, args.force)}")


if __name__ == "__main__":
    main()
