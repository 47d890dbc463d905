"""N-sharded linear on 2, 4 and 8 GPUs of one box (as many as the box has; skipped with one): the fused gather, in which every rank's
GEMM writes its output columns into all ranks' symmetric-memory buffers, and the NCCL all-gather, both bit for bit against the unsharded
linear on the same operands; the row-sharded host pipeline against the same."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["WQ_REPO"])
os.environ["WGPKERNELS_B200_CACHE"] = os.path.join(os.environ["WQ_TMP"], "tuning_" + os.environ["RANK"] + ".json")  # read at import
from wgpkernels_b200 import int8 as wq, dist as wdist, workloads
rank = int(os.environ["RANK"]); torch.cuda.set_device(rank); device = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=device)
wq.load_library()
for name, rows in (("c1", 1000), ("c2", 700), ("c4", 520)):
    full = workloads.make(name, rows=rows).to(device)
    expected = wq.linear(full.x, full.weight, full.scale, full.bias, mode="block", act=full.act, act_weight=full.act_weight, eps=full.eps,
                         residual=full.residual, residual_scale=full.residual_scale)
    layer = wdist.ShardedLinear.from_full(full.weight, full.scale, full.bias)
    cut = slice(layer.start, layer.stop)
    residual = None if full.residual is None else full.residual[:, cut]
    rscale = None if full.residual_scale is None else full.residual_scale[cut].contiguous()
    for gather in ("fused", "full", "fused", "auto", "fused"):  # alternating buffer sets: the result of a call outlives the next call
        got = layer(full.x, gather=gather, mode="block", act=full.act, act_weight=full.act_weight, eps=full.eps, residual=residual,
                    residual_scale=rscale)
        torch.cuda.synchronize()
        if got.shape != expected.shape or not torch.equal(got, expected):  # say where: whose columns, which rows
            bad = (got != expected).nonzero()
            width = expected.shape[1] // dist.get_world_size()
            raise AssertionError((name, gather, rank, "mismatches", int(bad.shape[0]), "columns of ranks", sorted(set((bad[:, 1] // width).tolist())),
                                  "rows", sorted(set(bad[:, 0].tolist()))[:12], "columns", sorted(set(bad[:, 1].tolist()))[:12],
                                  "max difference", float((got.float() - expected.float()).abs().max())))
    for mode in ("exact", "row"):
        if full.scale.dim() == 2 and mode == "row":
            continue
        expected = wq.linear(full.x, full.weight, full.scale, full.bias, mode=mode, act=full.act, act_weight=full.act_weight, eps=full.eps,
                             residual=full.residual, residual_scale=full.residual_scale)
        got = layer(full.x, gather="fused", mode=mode, act=full.act, act_weight=full.act_weight, eps=full.eps, residual=residual, residual_scale=rscale)
        torch.cuda.synchronize()
        assert torch.equal(got, expected), (name, mode, rank)
    if full.scale.dim() == 1:  # few tokens: 'auto' takes the all-gather route
        few = layer(full.x[:4], gather="auto", mode="lines", act=full.act, act_weight=full.act_weight, eps=full.eps)
        alone = wq.linear(full.x[:4], full.weight, full.scale, full.bias, mode="lines", act=full.act, act_weight=full.act_weight, eps=full.eps)
        torch.cuda.synchronize()
        # the few-token kernels split K by the shape of N: a slice's sums are added in another order than the whole matrix's
        assert float((few.float() - alone.float()).norm()) <= 1e-3 * float(alone.float().norm()), (name, "auto, few tokens", rank)
    try:
        layer(full.x[:4], gather="fused", mode="lines")
        raise AssertionError("few-token paths must be refused by the fused gather")
    except ValueError:
        pass
    assert wq.debug_status() == 0
# host pipeline, rows sharded over the ranks: every rank's band of the output equals the unsharded linear's
from wgpkernels_b200.host import ShardedHostLinear
full = workloads.make("c1", rows=1000).to(device)
expected = wq.linear(full.x, full.weight, full.scale, full.bias, mode="block", act=full.act, act_weight=full.act_weight, eps=full.eps)
host = ShardedHostLinear(full.weight, full.scale, full.bias, rows=1000, k=full.k, dtype=full.x.dtype, chunk_rows=128, tag=os.environ["MASTER_PORT"])
if rank == 0:
    host.x.copy_(full.x.cpu())
dist.barrier()
host(mode="block", act=full.act, act_weight=full.act_weight, eps=full.eps)
torch.cuda.synchronize()
dist.barrier()
assert torch.equal(host.y.to(device), expected), rank
host.close()
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok")
'''


def _world_sizes():
    count = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return [size for size in (2, 4, 8) if size <= count] or [2]


@pytest.mark.parametrize("world", _world_sizes())
def test_sharded_linear_equals_unsharded(tmp_path, world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    workers = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WQ_REPO=repo,
                   WQ_TMP=str(tmp_path))
        workers.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outputs = []
    for worker in workers:
        try:
            out, _ = worker.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            worker.kill()
            out, _ = worker.communicate()
        outputs.append(out)
    for rank, (worker, out) in enumerate(zip(workers, outputs)):
        assert worker.returncode == 0 and f"rank {rank} ok" in out, out[-3000:]
