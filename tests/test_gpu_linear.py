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


def test_graph_loop_over_row_windows(wq):
    """The use the *_at entry points exist for: ONE captured quantize + GEMM body replayed while a device counter advances walks a long
    input window by window; the result equals the eager linear on the whole input."""
    import ctypes
    c = workloads.make("c0", rows=640).to("cuda")
    window, n, k = 160, c.n, c.k
    lib = wq._require()
    expected = wq.linear(c.x, c.weight, c.scale, c.bias, mode="block")
    out = torch.zeros_like(expected)
    codes = torch.empty((window, k), dtype=torch.int8, device="cuda")
    scales = torch.empty((window, k // 128), dtype=torch.float32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int64, device="cuda")
    one = torch.ones(1, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        stream = wq._stream(c.x.device)
        assert lib.wq8_quantize_blocks_at(c.x.data_ptr(), codes.data_ptr(), scales.data_ptr(), window, k, c.x.stride(0), 1, 0, 0, None, 0.0, None,
                                          counter.data_ptr(), 0, window, stream) == 0
        assert lib.wq8_gemm_at(codes.data_ptr(), None, scales.data_ptr(), c.weight.data_ptr(), c.scale.data_ptr(), c.bias.data_ptr(), None, None,
                               out.data_ptr(), window, n, k, 1, 10, 148, 0, None, None, counter.data_ptr(), 0, window, 0, 0, 0, 0, stream) == 0
        counter.add_(one)
    for _ in range(640 // window):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, expected)
    assert wq.debug_status() == 0


def test_row_bands_through_small_scratch(wq, monkeypatch):
    """_gemm_path with a scratch limit that forces several bands of rows (three or more, the last one ragged), with a residual written
    in place and with a list of destinations: identical to the one-band result."""
    c = workloads.make("c2", rows=700).to("cuda")
    kwargs = dict(act=c.act, act_weight=c.act_weight, eps=c.eps, residual_scale=c.residual_scale)
    for mode in ("block", "exact"):
        whole = wq.linear(c.x, c.weight, c.scale, c.bias, mode=mode, residual=c.residual, **kwargs)
        monkeypatch.setattr(wq, "SCRATCH_BYTES", 256 * (c.k * (2 if mode == "exact" else 1) + 4 * (c.k // 128)))  # bands of 256 rows
        assert wq._chunk_rows(c.k, mode) == 256
        in_place = c.residual.clone()
        banded = wq.linear(c.x, c.weight, c.scale, c.bias, mode=mode, residual=in_place, out=in_place, **kwargs)
        assert banded.data_ptr() == in_place.data_ptr() and torch.equal(banded, whole), mode
        # the stage hook (what the benchmark records its events from) is called once per band and stage, in order
        tags = []
        monkeypatch.setattr(wq, "stage_hook", tags.append)
        wq.linear(c.x, c.weight, c.scale, c.bias, mode=mode, residual=c.residual, **kwargs)
        assert tags == ["quantized", "multiplied"] * 3, tags
        monkeypatch.setattr(wq, "stage_hook", None)
        wide = [torch.zeros((700, c.n + 64), dtype=c.x.dtype, device="cuda") for _ in range(2)]
        wq.linear(c.x, c.weight, c.scale, c.bias, mode=mode, residual=c.residual, out=[t[:, 32:32 + c.n] for t in wide], **kwargs)
        for t in wide:
            assert torch.equal(t[:, 32:32 + c.n], whole) and not t[:, :32].any() and not t[:, 32 + c.n:].any()
        monkeypatch.undo()


@pytest.mark.parametrize("name,rows", [("c1", 1500), ("c2", 900), ("c4", 1100)])
def test_config_bands_match_reference_library(wq, name, rows):
    """Bands of the benchmark configurations (their outlier channels, input operations, group scales) against the reference's own CUDA
    library on the same tensors: codes and scales bit for bit, outputs within 1e-3 relative Frobenius."""
    from tests import reflib
    c = workloads.make(name, rows=rows).to("cuda")
    q, s = wq.quantize_blocks(c.x, 0, c.act, c.act_weight, c.eps)
    q_ref, s_ref = reflib.quantize_blocks(c.x, 0, c.act, c.act_weight, c.eps)
    assert torch.equal(q, q_ref) and torch.equal(s, s_ref)
    grouped = c.scale.dim() == 2
    y = wq.gemm(q, None, s, c.weight, c.scale, c.bias, c.x.dtype, mode="block", residual=c.residual, residual_scale=c.residual_scale)
    y_ref = reflib.gemm(q_ref, None, s_ref, c.weight, c.scale, c.bias, c.x.dtype, 12 if grouped else 10, residual=c.residual,
                        residual_scale=c.residual_scale)
    assert rel(y, y_ref) < 1e-3, name
    hi, lo, rs = wq.quantize(c.x, 0, True, c.act, c.act_weight, c.eps)
    hi_ref, lo_ref, rs_ref = reflib.quantize(c.x, 0, True, c.act, c.act_weight, c.eps)
    assert torch.equal(hi, hi_ref) and torch.equal(lo, lo_ref) and torch.equal(rs, rs_ref)
    y = wq.gemm(hi, lo, rs, c.weight, c.scale, c.bias, c.x.dtype, mode="exact", residual=c.residual, residual_scale=c.residual_scale)
    y_ref = reflib.gemm(hi_ref, lo_ref, rs_ref, c.weight, c.scale, c.bias, c.x.dtype, 14 if grouped else 1, residual=c.residual,
                        residual_scale=c.residual_scale)
    assert rel(y, y_ref) < 1e-3, name
