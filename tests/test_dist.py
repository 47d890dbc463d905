"""N-sharding logic with two CPU ranks on the gloo backend: the partition, the gather and the unshard reproduce the unsharded linear.
The local operator is the CPU checker here (the partition logic does not depend on where the slice is computed)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from wgpkernels_b200 import dist as wdist


def test_shard_bounds_cover_all_channels():
    for n, g in ((15360, 8), (5120, 4), (12288, 2), (96, 2), (104, 4)):
        pieces = [wdist.shard_bounds(n, g, r) for r in range(g)]
        assert pieces[0][0] == 0 and pieces[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))
        assert all((stop - start) % 8 == 0 for start, stop in pieces)
    with pytest.raises(ValueError):
        wdist.shard_bounds(100, 2, 0)


def test_sharding_policy():
    """The all-gather of the output bounds the sharded time: long K pays, short K does not."""
    wide = wdist.worth_sharding(32760, 15360, 5120, 8)
    assert wide["gather_ms"] > wide["single_ms"] / 8  # config 1: the gather, not the GEMM, is what is left
    deep = wdist.worth_sharding(32760, 5120, 13824, 2)
    assert deep["shard"]
    assert wide["bound"] == "nvlink" and wide["best_ranks"] < 8  # replicating a 1 GB output to 8 GPUs loses to fewer ranks
    assert deep["best_ranks"] == 2
    small = wdist.worth_sharding(64, 5120, 512, 8)
    assert small["best_ms"] <= small["single_ms"]


def test_unshard():
    blocked = torch.arange(2 * 3 * 4).view(2, 3, 4)
    full = wdist.unshard(blocked)
    assert full.shape == (3, 8)
    assert torch.equal(full[:, :4], blocked[0]) and torch.equal(full[:, 4:], blocked[1])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world_size, port, failures):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world_size)
    try:
        from oracle import int8_oracle as oracle
        from wgpkernels_b200 import workloads
        c = workloads.make("c0", rows=24)
        c.weight, c.scale, c.bias = c.weight[:256].contiguous(), c.scale[:256].contiguous(), c.bias[:256].contiguous()

        def cpu_linear(x, weight, scale, bias, residual=None, residual_scale=None, mode="block", **kwargs):
            return oracle.linear(mode, x, weight.numpy(), scale.numpy(), bias, residual=residual, rscale=residual_scale, **kwargs)

        full = cpu_linear(c.x, c.weight, c.scale, c.bias)
        layer = wdist.ShardedLinear.from_full(c.weight, c.scale, c.bias, linear=cpu_linear)
        assert layer.weight.shape[0] == 256 // world_size
        # rank 0 owns the input; the others start from garbage and receive it
        x = c.x.clone() if rank == 0 else torch.zeros_like(c.x)
        y = layer(x, gather="full", broadcast_input=True)
        assert torch.equal(y, full), "gathered output differs from the unsharded linear"
        blocked = layer(c.x, gather="blocked")
        assert blocked.shape == (world_size, 24, 256 // world_size)
        assert torch.equal(blocked[rank], full[:, layer.start:layer.stop])
        local = layer(c.x, gather=None)
        assert torch.equal(local, full[:, layer.start:layer.stop])
        # fused gather: the rank's columns go into every rank's full-width buffer (stand-ins for the symmetric-memory views here),
        # its own buffer first, nothing else is touched
        views = [torch.zeros(24, 256, dtype=full.dtype) for _ in range(world_size)]
        order = []

        def writing_linear(x, weight, scale, bias, residual=None, residual_scale=None, out=None, **kwargs):
            result = cpu_linear(x, weight, scale, bias, residual=residual, residual_scale=residual_scale, **kwargs)
            if out is None:
                return result
            for target in out:
                order.append(next(i for i, view in enumerate(views) if view.data_ptr() == target.data_ptr() - target.storage_offset() * target.element_size()))
                target.copy_(result)
            return out

        fused_layer = wdist.ShardedLinear.from_full(c.weight, c.scale, c.bias, linear=writing_linear)
        fused_layer.symmetric_output = lambda m, dtype, device, which=0: (views[rank], views, torch.zeros(1))
        returned = fused_layer(c.x, gather="fused", out=torch.empty(1))  # a caller's `out` is ignored: the result is the layer's buffer
        assert returned is views[rank]
        try:  # the fused gather never times paths: a few-token path (or none given and a tuner picking one) is refused
            fused_layer(c.x, gather="fused", mode="lines")
            raise AssertionError("mode='lines' must be refused by the fused gather")
        except ValueError:
            pass
        assert order == [(rank + d) % world_size for d in range(world_size)]
        # 'auto': few rows (a weight stream, nothing to store from) go through the all-gather, more rows through the fused epilogue
        calls = len(order)
        wdist.FUSED_MIN_ROWS = 8
        assert torch.equal(fused_layer(c.x[:4], gather="auto"), full[:4]) and len(order) == calls
        assert fused_layer(c.x, gather="auto") is views[rank] and len(order) == calls + world_size
        assert fused_layer.policy(32760)["best_ranks"] >= 1
        for view in views:
            assert torch.equal(view[:, fused_layer.start:fused_layer.stop], full[:, fused_layer.start:fused_layer.stop])
            untouched = torch.ones(256, dtype=torch.bool)
            untouched[fused_layer.start:fused_layer.stop] = False
            assert not view[:, untouched].any()
        # a shard built from its own slice of a seeded weight equals the slice of the full weight
        w_slice, s_slice = workloads.quantized_weight(128, 5120, 0, n_offset=rank * 128, n_total=5120)
        assert torch.equal(w_slice, workloads.quantized_weight(5120, 5120, 0)[0][rank * 128:(rank + 1) * 128])
    except Exception as error:  # noqa: BLE001
        failures.put(f"rank {rank}: {type(error).__name__}: {error}")
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_linear_matches_unsharded():
    context = mp.get_context("spawn")
    failures = context.Queue()
    port = _free_port()
    workers = [context.Process(target=_rank_main, args=(rank, 2, port, failures)) for rank in range(2)]
    for w in workers:
        w.start()
    for w in workers:
        w.join(300)
        assert w.exitcode == 0, "a rank did not finish"
    assert failures.empty(), failures.get()
