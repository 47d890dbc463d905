"""Output-channel (N) sharding of the INT8 linear over the GPUs of one node: one process per GPU, `torch.distributed` (NCCL over
NVLink / NVSwitch) for the one exchange step.

The reference is single-GPU; this is an addition.  Rank r keeps rows [r N / g, (r + 1) N / g) of the INT8 weight with their scales
and bias (loaded once; the weight never moves).  The activation is present on every rank (replicated by the caller, or broadcast from
rank 0 here); every rank quantizes it itself -- recomputing the quantization costs less than moving the INT8 copy over NVLink -- and
runs the GEMM on its own output channels.  The one collective is the all-gather of the (M, N / g) output slices.

`gather="fused"` removes that collective: the output buffer of every rank lives in symmetric memory (mapped into all processes of
the node), and the GEMM of a rank writes its output columns into the full-width (M, N) buffer of every rank from its tile epilogue (one
TMA store per destination and 32 x 32 block of outputs, over NVLink for the peers), so the transfer runs under the tensor-core work
tile by tile.  Nothing is ever loaded from a peer.  Two small NCCL all-reduces order the step against the readers on the other ranks.

Whether sharding pays is a property of the shape: the GEMM shrinks by g but every rank must receive (g - 1) / g of the (M, N) output,
so `worth_sharding()` compares the two and `ShardedLinear` can keep the output sharded (`gather=None`) for a consumer that is sharded
the same way (attention heads of a fused QKV projection).
"""
from dataclasses import dataclass

import torch
import torch.distributed as dist


def shard_bounds(n, world_size, rank, multiple=8):
    """[start, stop) of rank's output channels: equal slices, each a multiple of `multiple` channels (the GEMM stores 16 bytes at a
    time), the remainder going to the last rank."""
    if n % multiple:
        raise ValueError(f"N = {n} must be a multiple of {multiple} to be sharded")
    units = n // multiple
    per_rank = -(-units // world_size)
    start = min(rank * per_rank, units) * multiple
    stop = min((rank + 1) * per_rank, units) * multiple
    return start, stop


# Measured on B200 (one node, NVSwitch): effective INT8 throughput of the block path's GEMM on one GPU, the replicated activation
# quantizer's HBM rate, and the bytes per second one GPU receives from its peers' TMA stores.
MEASURED_TOPS, MEASURED_QUANTIZER_GBS, MEASURED_LINK_GBS = 1800.0, 2800.0, 770.0


def worth_sharding(m, n, k, world_size, tops=MEASURED_TOPS, link_gbs=MEASURED_LINK_GBS, output_bytes=2, quantizer_gbs=MEASURED_QUANTIZER_GBS):
    """Estimated times in ms of the linear on one GPU and sharded over `world_size` GPUs with the full output replicated on every rank,
    and which number of ranks (a power of two up to world_size) is the fastest.  Sharded: the GEMM shrinks by g, the activation
    quantizer does not (every rank quantizes all of x), and every rank receives (g - 1) / g of the (M, N) output over NVLink, which
    the fused gather overlaps with the GEMM: step = quantizer + max(GEMM / g, incoming bytes / link rate)."""
    quantize_ms = 3.0 * m * k / (quantizer_gbs * 1e9) * 1e3
    gemm_ms = 2.0 * m * n * k / (tops * 1e12) * 1e3

    def step_ms(g):
        gather = (g - 1) / g * m * n * output_bytes / (link_gbs * 1e9) * 1e3
        return quantize_ms + max(gemm_ms / g, gather)

    candidates = [1]
    while candidates[-1] * 2 <= world_size:
        candidates.append(candidates[-1] * 2)
    best = min(candidates, key=lambda g: (step_ms(g), g))
    gather_ms = (world_size - 1) / world_size * m * n * output_bytes / (link_gbs * 1e9) * 1e3
    return {"single_ms": step_ms(1), "sharded_ms": step_ms(world_size), "gather_ms": gather_ms, "shard": step_ms(world_size) < step_ms(1),
            "best_ranks": best, "best_ms": step_ms(best), "bound": "nvlink" if gather_ms > gemm_ms / world_size else "tensor"}


FUSED_MIN_ROWS = 32  # up to here the linear is a few-token weight stream (lines / small): no tile epilogue to store from


@dataclass
class ShardedLinear:
    """The rank's slice of one INT8 linear.  weight (N_local, K) int8, scale (N_local,) or (N_local, ceil(K / 128)) fp32, bias (N_local,).
    linear: the local operator, `wgpkernels_b200.int8.linear` by default (injected so that the partition and gather logic can be tested
    with CPU ranks)."""
    weight: torch.Tensor
    scale: torch.Tensor
    bias: torch.Tensor = None
    n_total: int = 0
    group: object = None  # torch.distributed process group (None: the default group)
    linear: object = None

    def __post_init__(self):
        self.world_size = dist.get_world_size(self.group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        self.n_total = self.n_total or self.weight.shape[0] * self.world_size
        self.start, self.stop = shard_bounds(self.n_total, self.world_size, self.rank)
        if self.stop - self.start != self.weight.shape[0]:
            raise ValueError(f"rank {self.rank} holds {self.weight.shape[0]} channels, its slice is [{self.start}, {self.stop})")
        equal = self.n_total % (8 * self.world_size) == 0
        if not equal:
            raise ValueError("N must split into equal slices of a multiple of 8 channels (all_gather moves equal chunks)")
        if self.linear is None:
            from wgpkernels_b200 import int8
            self.linear = int8.linear
        self._gathered = None
        self._symmetric = {}  # (M, dtype, which of the two alternating sets) -> (own buffer, views of every rank's buffer, barrier token)
        self._fused_calls = {}  # (M, dtype) -> calls of fused() so far

    @classmethod
    def from_full(cls, weight, scale, bias=None, group=None, linear=None):
        """Slices an unsharded weight (every rank passes the same full tensors; only the slice is kept)."""
        world_size = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        start, stop = shard_bounds(weight.shape[0], world_size, rank)
        return cls(weight[start:stop].contiguous(), scale[start:stop].contiguous(), None if bias is None else bias[start:stop].contiguous(),
                   weight.shape[0], group, linear)

    def local(self, x, residual=None, residual_scale=None, **kwargs):
        """This rank's output columns (M, N_local).  residual / residual_scale: the rank's own columns."""
        return self.linear(x, self.weight, self.scale, self.bias, residual=residual, residual_scale=residual_scale, **kwargs)

    def policy(self, m):
        """worth_sharding() for this layer's shape and group size at m rows: the estimate of what sharding gains, the number of ranks
        that would serve a replicated output best, and what bounds it."""
        return worth_sharding(m, self.n_total, self.weight.shape[1], self.world_size)

    def symmetric_output(self, m, dtype, device, which=0):
        """(own (M, N) buffer, [view of rank r's buffer for every r], token) in symmetric memory; a collective call the first time.
        which: 0 or 1, the two sets of buffers fused() alternates between."""
        key = (m, dtype, which)
        if key not in self._symmetric:
            import torch.distributed._symmetric_memory as symmetric_memory
            own = symmetric_memory.empty((m, self.n_total), dtype=dtype, device=device)
            handle = symmetric_memory.rendezvous(own, self.group if self.group is not None else dist.group.WORLD)
            views = [own if r == self.rank else handle.get_buffer(r, (m, self.n_total), dtype) for r in range(self.world_size)]
            self._symmetric[key] = (own, views, torch.zeros(1, device=device), handle)
        return self._symmetric[key][:3]

    def fused(self, x, residual=None, residual_scale=None, **kwargs):
        """(M, N) on every rank, each rank's GEMM writing its columns into all ranks' buffers.  The result is one of this layer's two
        buffers for (M, dtype), used in turn: it stays valid until the call AFTER the next one with the same M is made (work that reads
        it must be on the stream before that call).  One 4-byte all-reduce per call orders everything: it ends the call, so it follows
        the rank's stores and, on the same stream, whatever the rank enqueued earlier -- the readers of the other buffer set included;
        nobody starts the next call's stores into that other set before every rank has reached this point.
        residual / residual_scale: the rank's own columns, (M, N / g) with any row stride and (N / g)."""
        mode = kwargs.setdefault("mode", "block")
        if mode not in ("block", "exact", "row"):
            raise ValueError(f"the fused gather runs the 'block', 'exact' or 'row' path (every rank the same one), not {mode!r}")
        calls = self._fused_calls.get((x.shape[0], x.dtype), 0)
        self._fused_calls[(x.shape[0], x.dtype)] = calls + 1
        own, views, token = self.symmetric_output(x.shape[0], x.dtype, x.device, calls & 1)
        # own buffer first, then the peers starting from the next rank, so that the ranks do not all store to the same GPU at once
        order = [(self.rank + d) % self.world_size for d in range(self.world_size)]
        outputs = [views[r][:, self.start:self.stop] for r in order]
        kwargs.pop("out", None)
        self.linear(x, self.weight, self.scale, self.bias, residual=residual, residual_scale=residual_scale, out=outputs, **kwargs)
        dist.all_reduce(token, group=self.group)  # every rank's stores have been issued and completed before anyone reads
        return own

    def __call__(self, x, gather="full", broadcast_input=False, residual=None, residual_scale=None, **kwargs):
        """gather: 'full' -> (M, N) on every rank; 'blocked' -> (g, M, N / g), rank-major (what the all-gather delivers, no extra copy);
        'fused' -> (M, N) on every rank without a collective on the data (see fused(); block / exact / row paths only);
        'auto' -> (M, N) on every rank by the cheaper of the two routes: 'fused' for more than FUSED_MIN_ROWS rows on a path the fused
        epilogue runs ('block' when none is named), the NCCL all-gather ('full') for the few-token paths, whose outputs are a few KB;
        None -> the local (M, N / g) slice only.  residual / residual_scale: the rank's own columns.
        broadcast_input: x is valid on rank 0 only and is broadcast first."""
        if broadcast_input and self.world_size > 1:
            dist.broadcast(x, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0, group=self.group)
        if gather == "auto":
            gather = "fused" if x.shape[0] > FUSED_MIN_ROWS and kwargs.get("mode", "block") in ("block", "exact", "row") else "full"
        if gather == "fused" and self.world_size > 1:
            return self.fused(x, residual=residual, residual_scale=residual_scale, **kwargs)
        if gather == "fused":
            gather = "full"
        y = self.local(x, residual=residual, residual_scale=residual_scale, **kwargs)
        if gather is None or self.world_size == 1:
            return y if gather != "blocked" else y.unsqueeze(0)
        m, n_local = y.shape
        if self._gathered is None or self._gathered.shape != (self.world_size, m, n_local) or self._gathered.dtype != y.dtype:
            self._gathered = torch.empty((self.world_size, m, n_local), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(self._gathered.view(self.world_size * m, n_local), y.contiguous(), group=self.group)
        if gather == "blocked":
            return self._gathered
        return unshard(self._gathered)


def unshard(blocked, out=None):
    """(g, M, N / g) rank-major slices -> (M, N) row-major."""
    g, m, n_local = blocked.shape
    out = torch.empty((m, g * n_local), dtype=blocked.dtype, device=blocked.device) if out is None else out
    out.view(m, g, n_local).copy_(blocked.permute(1, 0, 2))
    return out
