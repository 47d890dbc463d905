"""HostLinear: the pipelined host-to-host linear equals the plain linear on the same rows, for a ragged last chunk, with a residual, and
called twice in a row on the same buffers."""
import pytest
import torch

from wgpkernels_b200 import workloads
from wgpkernels_b200.host import HostLinear

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["c1", "c2"])
def test_host_linear_matches_device_linear(wq, name):
    c = workloads.make(name, rows=1000)
    g = c.to(torch.device("cuda", 0))
    n = g.weight.shape[0]
    kwargs = dict(mode="block", act=c.act, act_weight=g.act_weight, eps=c.eps, residual_scale=g.residual_scale)
    expected = wq.linear(g.x, g.weight, g.scale, g.bias, residual=g.residual, **kwargs)
    host_x = c.x.pin_memory()
    host_y = torch.empty((c.m, n), dtype=c.x.dtype).pin_memory()
    layer = HostLinear(g.weight, g.scale, g.bias, chunk_rows=384)  # 1000 rows: two whole chunks and one of 232
    for _ in range(2):
        host_y.zero_()
        layer(host_x, host_y, residual=g.residual, **kwargs)
        torch.cuda.synchronize()
        assert torch.equal(host_y, expected.cpu())
    with pytest.raises(ValueError):
        layer(c.x, host_y, **kwargs)  # not pinned
    assert wq.debug_status() == 0
