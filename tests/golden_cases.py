"""Loader of the committed golden vectors (tests/golden/*.npz, written by tests/golden/make_golden.py)."""
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"
DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16}


def _tensor(array, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(array))
    return t.view(dtype) if dtype is not None and t.dtype == torch.int16 else t


class SelftestCase:
    """One case of the reference's selftest list with the inputs it was drawn with and the output of the reference's
    FP32 PyTorch computation."""

    def __init__(self, data, tag, index, spec):
        m, path, group, act, with_residual = spec.split("|")
        self.tag, self.index, self.dtype = tag, index, DTYPES[tag]
        self.m, self.path, self.group = int(m), path, int(group)
        self.act = None if act == "None" else act
        self.w = _tensor(data[f"{tag}.w"])
        self.scale = _tensor(data[f"{tag}.s_groups" if path.endswith("+g") else f"{tag}.s"])
        self.bias = _tensor(data[f"{tag}.bias"], self.dtype)
        self.act_weight = _tensor(data[f"{tag}.norm_weight"], self.dtype) if self.act == "rms_norm" else None
        self.x = _tensor(data[f"{tag}.{index}.x"], self.dtype)
        self.residual = self.residual_scale = None
        if int(with_residual):
            self.residual = _tensor(data[f"{tag}.{index}.residual"], self.dtype)
            self.residual_scale = _tensor(data[f"{tag}.{index}.residual_scale"], self.dtype)
        self.ref = _tensor(data[f"{tag}.{index}.ref"])
        self.eps = 1e-6
        # the pass bars of the reference's selftest (wgpkernels/int8/__init__.py:573)
        self.tolerance = 5e-3 if path in ("lines", "small", "exact", "exact+g") else 3e-2

    @property
    def id(self):
        return f"{self.tag}-{self.index}-{self.path}-m{self.m}-g{self.group}-{self.act}-{'res' if self.residual is not None else 'nores'}"


def selftest_cases(tags=("bf16", "fp16")):
    data = np.load(GOLDEN / "selftest_cases.npz")
    specs = [str(s) for s in data["cases"]]
    return [SelftestCase(data, tag, index, spec) for tag in tags for index, spec in enumerate(specs)]


def rotation_vectors():
    data = np.load(GOLDEN / "selftest_cases.npz")
    return _tensor(data["rotation.x"]), {g: _tensor(data[f"rotation.{g}"]) for g in (16, 64, 256)}


def config0():
    return np.load(GOLDEN / "config0.npz")
