"""N-sharded linear on two GPUs of one box (skipped with fewer): the fused gather, in which every rank's GEMM writes its output
columns into all ranks' symmetric-memory buffers, and the NCCL all-gather, both against the unsharded linear on the same operands."""
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
    for gather in ("fused", "full", "fused"):
        got = layer(full.x, gather=gather, mode="block", act=full.act, act_weight=full.act_weight, eps=full.eps, residual=residual,
                    residual_scale=rscale)
        torch.cuda.synchronize()
        assert got.shape == expected.shape and torch.equal(got, expected), (name, gather, rank, float((got.float() - expected.float()).abs().max()))
    assert wq.debug_status() == 0
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok")
'''


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_fused_and_nccl_gather(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    workers = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WQ_REPO=repo)
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
