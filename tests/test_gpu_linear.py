"""The public API on the GPU: selftest(), the reference's selftest cases against the golden outputs of the reference's own FP32
computation, prepare() reuse, the path policy and the error behaviour."""
import pytest
import torch

from oracle import int8_oracle as oracle
from tests import golden_cases
from tests.gpu_common import rel
from wgpkernels_b200 import workloads

pytestmark = pytest.mark.gpu
CASES = golden_cases.selftest_cases()


def test_selftest_passes(wq):
    assert wq.selftest() is None
    assert wq.debug_status() == 0


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.id)
def test_golden_selftest_cases(wq, case):
    """linear(mode=path) on the inputs the golden outputs were made from, within the reference's own pass bars; and against the CPU
    restatement of the same path within 1e-3."""
    dev = lambda t: None if t is None else t.cuda()
    path = case.path.removesuffix("+g")
    y = wq.linear(dev(case.x), dev(case.w), dev(case.scale), dev(case.bias), group=case.group, mode=path, act=case.act, act_weight=dev(case.act_weight),
                  eps=case.eps, residual=dev(case.residual), residual_scale=dev(case.residual_scale))
    assert y.dtype == case.dtype and y.shape == (case.m, 96)
    assert rel(y, case.ref) < case.tolerance
    expected = oracle.linear(path, case.x, case.w.numpy(), case.scale.numpy(), case.bias, case.group, case.act, case.act_weight, case.eps, case.residual,
                             case.residual_scale)
    assert rel(y, expected) < 1e-3


def test_exact_path_precision(wq):
    """'exact' within 0.2% of the FP32 dequantize-and-matmul on activations with outlier channels (BASELINE config 0)."""
    c = workloads.make("c0")
    g = c.to("cuda")
    reference = oracle.linear_reference(c.x, c.weight, c.scale, c.bias)
    y = wq.linear(g.x, g.weight, g.scale, g.bias, mode="exact")
    assert rel(y, reference) < 2e-3
    block = wq.linear(g.x, g.weight, g.scale, g.bias, mode="block")
    row = wq.linear(g.x, g.weight, g.scale, g.bias, mode="row")
    assert rel(y, reference) < rel(block, reference) < rel(row, reference)
    assert rel(block, oracle.linear("block", c.x, c.weight.numpy(), c.scale.numpy(), c.bias)) < 1e-3


def test_prepare_once_for_three_weights(wq):
    """BASELINE config 4 (group-128 weight scales) on a band of rows: one prepare() per path, three weights."""
    c = workloads.make("c4", rows=384)
    g = c.to("cuda")
    for path in ("block", "exact"):
        prepared = wq.prepare(g.x, 0, path)
        for (w, s), (w_cpu, s_cpu) in zip([(g.weight, g.scale)] + g.extra_weights, [(c.weight, c.scale)] + c.extra_weights):
            y = wq.linear_prepared(prepared, w, s)
            expected = oracle.linear(path, c.x, w_cpu.numpy(), s_cpu.numpy())
            assert rel(y, expected) < 1e-3
            if path == "exact":
                assert rel(y, oracle.linear_reference(c.x, w_cpu, s_cpu)) < 2e-3
    assert wq.debug_status() == 0


def test_few_token_config(wq):
    """BASELINE config 3: SwiGLU MLP up / down at 1, 4, 16, 32 tokens on the precise paths."""
    for name in ("c3u", "c3d"):
        for m, path in ((1, "lines"), (4, "lines"), (16, "small"), (32, "small"), (32, "exact")):
            c = workloads.make(name, rows=m)
            g = c.to("cuda")
            y = wq.linear(g.x, g.weight, g.scale, None, mode=path, act=c.act, precise=True)
            reference = oracle.linear_reference(c.x, c.weight, c.scale, None, 0, c.act, None, 0.0, None, None, path in ("lines", "small"))
            # the output is rounded to bf16 (2^-9 relative per element); the FP32 reference is not
            assert rel(y, reference) < 4e-3, (name, m, path)
            assert rel(y, oracle.linear(path, c.x, c.weight.numpy(), c.scale.numpy(), None, 0, c.act)) < 1e-3, (name, m, path)


def test_choose_path_and_cache(wq, tmp_path, monkeypatch):
    monkeypatch.setattr(wq, "_TUNING_PATH", tmp_path / "tuning.json")
    monkeypatch.setattr(wq, "_tuned", None)
    wq._paths.clear()
    wq._plans.clear()
    c = workloads.make("c3u", rows=4).to("cuda")
    path = wq.choose_path(c.x, c.weight, c.scale, precise=True)
    assert path in ("lines", "small", "exact")
    assert (tmp_path / "tuning.json").exists()
    assert wq.choose_path(c.x, c.weight, c.scale, precise=True) == path
    big = workloads.make("c0", rows=5000).to("cuda")
    assert wq.choose_path(big.x, big.weight, big.scale) in ("block", "exact")  # timed: 'exact' keeps up with 'block' on this GPU
    monkeypatch.setattr(wq, "DECIDE_MAX_ROWS", 4096)
    wq._paths.clear()
    monkeypatch.setattr(wq, "_tuned", {})
    assert wq.choose_path(big.x, big.weight, big.scale) == "block"             # past the limit: 'block' without timing
    y = wq.linear(c.x, c.weight, c.scale, precise=True)
    assert y.shape == (4, c.weight.shape[0])


def test_cuda_graph_replay(wq):
    """After one eager call per shape the linear can be captured and replayed."""
    c = workloads.make("c0", rows=256).to("cuda")
    out = torch.empty((256, c.n), dtype=torch.bfloat16, device="cuda")
    eager = wq.linear(c.x, c.weight, c.scale, c.bias, mode="block").clone()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        wq.linear(c.x, c.weight, c.scale, c.bias, mode="block", out=out)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)


def test_errors(wq):
    c = workloads.make("c0", rows=8).to("cuda")
    groups = torch.ones((c.n, c.k // 128), device="cuda")
    with pytest.raises(ValueError):
        wq.linear_prepared(wq.prepare(c.x, 0, "small"), c.weight, groups)
    hi, _, row_scale = wq.quantize(c.x)
    with pytest.raises(ValueError):
        wq.gemm(hi, None, row_scale, c.weight, groups, None, torch.bfloat16, mode="row")
    with pytest.raises(RuntimeError):
        wq.gemm(hi, None, row_scale, c.weight, c.scale, None, torch.bfloat16, 0, 99)
    with pytest.raises(ValueError):
        wq.linear(c.x, c.weight, c.scale, act="relu")
