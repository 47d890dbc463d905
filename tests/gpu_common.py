"""Shared pieces of the GPU parity tests."""
import numpy as np
import torch

from oracle import int8_oracle as oracle


def rel(y, ref):
    return oracle.relative_error(y.detach().float().cpu(), ref.detach().float().cpu() if isinstance(ref, torch.Tensor) else ref)


def randn(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def rand_int8(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(-127, 128, shape, dtype=torch.int8, generator=g)


def codes_close(q_gpu, q_cpu, max_fraction):
    """INT8 codes equal except for one-step differences on at most max_fraction of the elements (libm ulps at rounding ties)."""
    diff = np.abs(q_gpu.cpu().numpy().astype(np.int32) - np.asarray(q_cpu).astype(np.int32))
    return diff.max(initial=0) <= 1 and (diff != 0).mean() <= max_fraction
