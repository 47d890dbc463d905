"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

No dataset is involved: every tensor is drawn from a ``torch.Generator`` on the CPU (one generator per
tensor, so that a tensor does not change when another one's shape does) and moved to the device afterwards,
so a CPU checker and the GPU see identical bits.

Weights follow the checkpoints the reference serves (Quanto INT8: symmetric per-output-channel absmax;
group-128 checkpoints: one scale per channel and 128-element block of K).  Bias, residual scale and
RMSNorm weight are held in the activation dtype, as the C ABI reads them.

  c0  M=64    K=5120   N=5120   no input op                       (the CPU-runnable case)
  c1  M=32760 K=5120   N=15360  rms_norm, fused QKV projection    (block path)
  c2  M=32760 K=13824  N=5120   gelu + in-place residual          (block path)
  c3u M<=32   K=4096   N=28672  SwiGLU MLP up   (lines / small / exact, precise)
  c3d M<=32   K=14336  N=4096   SwiGLU MLP down, act=swiglu on a (M, 28672) input
  c4  M=16384 K=3072   N=12288  group-128 weight scales, three weights per prepare()
"""
from dataclasses import dataclass, field
from typing import Optional

import torch


# (M, K, N) of each configuration at full size
SHAPES = {"c0": (64, 5120, 5120), "c1": (32760, 5120, 15360), "c2": (32760, 13824, 5120), "c3u": (1, 4096, 28672), "c3d": (1, 14336, 4096),
          "c4": (16384, 3072, 12288)}


@dataclass
class Workload:
    name: str
    x: torch.Tensor
    weight: torch.Tensor
    scale: torch.Tensor
    bias: Optional[torch.Tensor] = None
    act: Optional[str] = None
    act_weight: Optional[torch.Tensor] = None
    eps: float = 0.0
    residual: Optional[torch.Tensor] = None
    residual_scale: Optional[torch.Tensor] = None
    mode: Optional[str] = None
    precise: bool = False
    extra_weights: list = field(default_factory=list)  # further (weight, scale) pairs sharing one prepare()

    @property
    def m(self):
        return self.x.shape[0]

    @property
    def k(self):
        return self.weight.shape[1]

    @property
    def n(self):
        return self.weight.shape[0]

    @property
    def ops(self):
        """Effective operations of one linear: 2 M N K."""
        return 2 * self.m * self.n * self.k

    def to(self, device):
        move = lambda t: None if t is None else t.to(device)
        return Workload(self.name, move(self.x), move(self.weight), move(self.scale), move(self.bias), self.act, move(self.act_weight),
                        self.eps, move(self.residual), move(self.residual_scale), self.mode, self.precise,
                        [(move(w), move(s)) for w, s in self.extra_weights])


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def quantized_weight(n, k, seed=0, groups=False, std=0.02, n_offset=0, n_total=None):
    """INT8 weight + FP32 scales from W_fp ~ N(0, std): scales = absmax / 127 per row (or per row and 128-block),
    W = round(W_fp / scale) clipped to [-127, 127].  n_offset / n_total draw rows [n_offset, n_offset + n) of the
    (n_total, k) matrix, so that a shard holds exactly the rows of the unsharded weight."""
    n_total = n if n_total is None else n_total
    w_fp = torch.randn(n_total, k, generator=_gen(1000 + seed)) * std
    w_fp = w_fp[n_offset:n_offset + n]
    if groups:
        kb = -(-k // 128)
        padded = torch.zeros(n, kb * 128)
        padded[:, :k] = w_fp
        blocks = padded.view(n, kb, 128)
        scale = blocks.abs().amax(dim=2) / 127
        q = torch.round(blocks / scale.clamp_min(1e-30)[:, :, None]).clamp_(-127, 127).to(torch.int8).view(n, kb * 128)[:, :k].contiguous()
        return q, scale.contiguous()
    scale = w_fp.abs().amax(dim=1) / 127
    q = torch.round(w_fp / scale.clamp_min(1e-30)[:, None]).clamp_(-127, 127).to(torch.int8)
    return q.contiguous(), scale.contiguous()


def _activations(m, k, seed, std=1.0, outliers=0, factor=1.0, magnitude=None, dtype=torch.bfloat16):
    x = torch.randn(m, k, generator=_gen(2000 + seed)) * std
    if outliers:
        channels = torch.randperm(k, generator=_gen(3000 + seed))[:outliers]
        if magnitude is None:
            x[:, channels] *= factor
        else:
            x[:, channels] = torch.sign(x[:, channels]) * magnitude
    return x.to(dtype)


def make(name, rows=None, dtype=torch.bfloat16, seed=0, n_offset=0, n_rows=None):
    """Workload `name` ('c0', 'c1', 'c2', 'c3u', 'c3d', 'c4').  rows: a smaller token count (parity tests and
    bounded CPU samples use the first rows of the same distribution).  n_offset / n_rows: the output-channel slice
    of an N-sharded run (weights, scales and bias of those channels only)."""
    def weight(n, k, wseed=0, groups=False):
        count = n if n_rows is None else n_rows
        w, s = quantized_weight(count, k, seed + wseed, groups, n_offset=n_offset, n_total=n)
        return w, s

    def bias_of(n):
        b = (torch.randn(n, generator=_gen(4000 + seed)) * 0.01).to(dtype)
        return b[n_offset:n_offset + (n if n_rows is None else n_rows)].contiguous()

    if name == "c0":
        m, k, n = rows or 64, 5120, 5120
        w, s = weight(n, k)
        return Workload(name, _activations(m, k, seed, outliers=8, factor=50.0, dtype=dtype), w, s, bias_of(n))
    if name == "c1":
        m, k, n = rows or 32760, 5120, 15360
        w, s = weight(n, k)
        act_weight = (1 + torch.randn(k, generator=_gen(5000 + seed)) * 0.1).to(dtype)
        return Workload(name, _activations(m, k, seed, outliers=26, factor=100.0, dtype=dtype), w, s, None, "rms_norm", act_weight, 1e-6,
                        mode="block")
    if name == "c2":
        m, k, n = rows or 32760, 13824, 5120
        w, s = weight(n, k)
        count = n if n_rows is None else n_rows
        residual = torch.randn(m, count, generator=_gen(6000 + seed)).to(dtype)
        return Workload(name, _activations(m, k, seed, std=1.5, dtype=dtype), w, s, bias_of(n), "gelu", None, 0.0, residual,
                        torch.full((count,), 0.7, dtype=dtype), mode="block")
    if name == "c3u":
        m, k, n = rows or 1, 4096, 2 * 14336
        w, s = weight(n, k)
        return Workload(name, _activations(m, k, seed, outliers=4, magnitude=1000.0, dtype=dtype), w, s, None, precise=True)
    if name == "c3d":
        m, k, n = rows or 1, 14336, 4096
        w, s = weight(n, k)
        return Workload(name, _activations(m, 2 * k, seed, outliers=4, magnitude=1000.0, dtype=dtype), w, s, None, "swiglu", precise=True)
    if name == "c4":
        m, k, n = rows or 16384, 3072, 12288
        w, s = weight(n, k, 0, True)
        extra = [weight(n, k, wseed, True) for wseed in (1, 2)]
        return Workload(name, _activations(m, k, seed, outliers=31, factor=64.0, dtype=dtype), w, s, None, mode="block", extra_weights=extra)
    raise ValueError(f"unknown workload {name!r}")
