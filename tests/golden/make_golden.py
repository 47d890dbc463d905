"""Generates tests/golden/*.npz from the reference's own Python code (run in a container that has the
reference checkout; the GPU box does not):

    python tests/golden/make_golden.py /path/to/WGPKernels

The reference has no golden vectors of its own; its only known-answer check is ``selftest()``
(wgpkernels/int8/__init__.py:542-576), which compares its kernels with ``_reference`` (:523-539) on a fixed
case list (:547-552).  This script imports the reference, rebuilds that case list with a CPU generator
(seed 0; the reference draws on the GPU, which cannot be reproduced without one), and stores the inputs
together with the outputs of the reference's ``_reference`` / ``_reference_rotation``.  The tests then pin
``oracle/int8_oracle.py`` to these outputs.

Files written:
  selftest_cases.npz  inputs + reference outputs of the 19 selftest cases, bf16 and fp16
  config0.npz         BASELINE config 0 (M=64, K=N=5120, seed 0): output slice + checksums of the seeded inputs
"""
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden.py /path/to/WGPKernels   (the reference checkout)")
REFERENCE = Path(sys.argv[1])
sys.path.insert(0, str(REFERENCE))

from wgpkernels import int8 as ref  # noqa: E402  (the reference; imports without its CUDA library)
from wgpkernels_b200 import workloads  # noqa: E402

CASES = ((1, "lines", 0, None, False), (5, "small", 0, None, False), (5, "small", 64, None, False), (40, "exact", 0, None, False),
         (40, "block", 256, None, False), (40, "row", 16, None, False), (2, "lines", 0, "swiglu", True), (5, "small", 64, "rms_norm", True),
         (40, "exact", 256, "rms_norm", False), (40, "block", 0, "swiglu", True), (40, "block", 16, "rms_norm", True), (40, "exact", 64, None, True),
         (3, "lines", 64, "gelu", False), (5, "small", 0, "gelu", True), (40, "exact", 16, "gelu", False), (40, "block", 256, "gelu", True),
         (40, "exact+g", 0, None, True), (40, "block+g", 64, "rms_norm", False), (40, "block+g", 0, None, True))


def bits(t):
    """Raw storage of a 16-bit float tensor (NumPy has no bfloat16)."""
    return t.view(torch.int16).numpy() if t.dtype in (torch.bfloat16, torch.float16) else t.numpy()


def selftest_cases():
    out = {"cases": np.array([f"{m}|{path}|{group}|{act}|{int(res)}" for m, path, group, act, res in CASES])}
    generator = torch.Generator().manual_seed(0)
    for dtype, tag in ((torch.bfloat16, "bf16"), (torch.float16, "fp16")):
        w = torch.randint(-127, 128, (96, 256), dtype=torch.int8, generator=generator)
        s = torch.rand(96, generator=generator) / 127
        s_groups = torch.rand(96, 2, generator=generator) / 127
        bias = torch.randn(96, generator=generator).to(dtype)
        norm_weight = (torch.rand(256, generator=generator) + 0.5).to(dtype)
        out.update({f"{tag}.w": w.numpy(), f"{tag}.s": s.numpy(), f"{tag}.s_groups": s_groups.numpy(), f"{tag}.bias": bits(bias),
                    f"{tag}.norm_weight": bits(norm_weight)})
        for index, (m, path, group, act, with_residual) in enumerate(CASES):
            x = torch.randn(m, 512 if act == "swiglu" else 256, generator=generator).to(dtype)
            act_weight = norm_weight if act == "rms_norm" else None
            residual = (torch.randn(m, 96, generator=generator) * 4).to(dtype) if with_residual else None
            residual_scale = torch.rand(96, generator=generator).to(dtype) if with_residual else None
            scale = s_groups if path.endswith("+g") else s
            y = ref._reference(x, w, scale, bias, group, act, act_weight, 1e-6, residual, residual_scale, path in ("lines", "small"))
            out[f"{tag}.{index}.x"] = bits(x)
            if with_residual:
                out[f"{tag}.{index}.residual"] = bits(residual)
                out[f"{tag}.{index}.residual_scale"] = bits(residual_scale)
            out[f"{tag}.{index}.ref"] = y.numpy()
    v = torch.randn(7, 512, generator=generator)
    out["rotation.x"] = v.numpy()
    for group in (16, 64, 256):
        out[f"rotation.{group}"] = ref._reference_rotation(v, group).numpy()
    np.savez_compressed(HERE / "selftest_cases.npz", **out)


def digest(t):
    return hashlib.sha256(bits(t.contiguous()).tobytes()).hexdigest()


def config0():
    c = workloads.make("c0")
    y = ref._reference(c.x, c.weight, c.scale, c.bias, 0, None, None, 0.0, None, None, False)
    np.savez_compressed(HERE / "config0.npz", y_slice=y[:, :256].numpy(), y_norm=np.float64(y.double().norm().item()),
                        y_sum=np.float64(y.double().sum().item()),
                        digests=np.array([digest(c.x), digest(c.weight), digest(c.scale), digest(c.bias)]))


if __name__ == "__main__":
    selftest_cases()
    config0()
    print("wrote", *(p.name for p in sorted(HERE.glob("*.npz"))))
