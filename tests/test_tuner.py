"""Host-side policy of the INT8 module without a GPU: buckets, the on-disk cache, the path rule (fastest full-precision path unless
it costs more than 10% over 'block'), the untimed fallbacks used during CUDA graph capture, and the loud failure without a library."""
import json

import pytest
import torch

from wgpkernels_b200 import int8 as wq


@pytest.fixture
def tuner(tmp_path, monkeypatch):
    """The module with a private cache file, a fake device name and a recorded fake timer."""
    monkeypatch.setattr(wq, "_TUNING_PATH", tmp_path / "cache" / "int8_tuning.json")
    monkeypatch.setattr(wq, "_tuned", None)
    monkeypatch.setattr(wq, "_weight_groups", True)
    monkeypatch.setattr(wq, "_device_name", lambda index: "Fake B200")
    monkeypatch.setattr(wq, "_capturing", lambda: False)
    wq._paths.clear()
    wq._plans.clear()
    calls = []

    def fake_best_of(launches, device):
        calls.append(sorted(map(str, launches)))
        return {name: fake_best_of.times[name] for name in launches}

    fake_best_of.times = {}
    monkeypatch.setattr(wq, "_best_of", fake_best_of)
    wq.calls, wq.fake = calls, fake_best_of
    yield wq
    wq._paths.clear()
    wq._plans.clear()


def operands(m, k=256, n=96, groups=False):
    x = torch.zeros(m, k, dtype=torch.bfloat16)
    w = torch.zeros(n, k, dtype=torch.int8)
    s = torch.ones(n, k // 128) if groups else torch.ones(n)
    return x, w, s


def test_buckets():
    assert [wq._rows_bucket(m) for m in (1, 64, 65, 4096, 4097, 8192, 8193, 32760, 100000)] == [64, 64, 128, 4096, 8192, 8192, 16384, 16384, 16384]
    assert [wq._path_bucket(m) for m in (1, 16, 17, 24, 128, 129, 4096)] == [1, 16, 24, 24, 128, 192, 4096]


def test_cache_round_trip_and_version(tuner):
    tuner._cache()["key"] = [10, 0]
    tuner._save_cache()
    payload = json.loads(tuner._TUNING_PATH.read_text())
    assert payload == {"version": tuner._TUNING_VERSION, "configs": {"key": [10, 0]}}
    tuner._tuned = None
    assert tuner._cache() == {"key": [10, 0]}
    tuner._TUNING_PATH.write_text(json.dumps({"version": tuner._TUNING_VERSION + 1, "configs": {"key": [11, 0]}}))
    tuner._tuned = None
    assert tuner._cache() == {}  # another version's tile ids are never read
    tuner._TUNING_PATH.write_text("{not json")
    tuner._tuned = None
    assert tuner._cache() == {}


def test_unwritable_cache_is_reported_not_raised(tuner, capsys):
    blocker = tuner._TUNING_PATH.parent
    blocker.parent.mkdir(parents=True, exist_ok=True)
    blocker.write_text("a file where the cache directory should be")
    tuner._cache()["key"] = "block"
    tuner._save_cache()
    assert "Could not save" in capsys.readouterr().out


def test_many_rows_take_block_without_timing(tuner):
    x, w, s = operands(140000)
    assert tuner.choose_path(x, w, s) == "block"
    assert tuner.calls == []
    tuner.fake.times = {"exact": 2.0}
    assert tuner.choose_path(x, w, s, precise=True) == "exact"  # precise: never 'block', whatever the size


def test_ten_percent_rule(tuner):
    x, w, s = operands(3)
    tuner.fake.times = {"lines": 1.09, "small": 1.2, "exact": 3.0, "block": 1.0}
    assert tuner.choose_path(x, w, s) == "lines"
    assert tuner.calls == [["block", "exact", "lines", "small"]]
    key = "path|3x96x256|g0|Fake B200"
    assert json.loads(tuner._TUNING_PATH.read_text())["configs"][key] == "lines"
    # memoised: no second timing
    assert tuner.choose_path(x, w, s) == "lines" and len(tuner.calls) == 1
    x, w, s = operands(24)
    tuner.fake.times = {"small": 1.2, "exact": 3.0, "block": 1.0}
    assert tuner.choose_path(x, w, s) == "block"  # 20% slower than block: not worth it
    tuner.fake.times = {"small": 1.2, "exact": 3.0}
    assert tuner.choose_path(x, w, s, precise=True) == "small"
    assert "path+precise|24x96x256|g0|Fake B200" in tuner._cache()


def test_candidates(tuner):
    assert tuner._precise_paths(4, 256) == ["lines", "small", "exact"]
    assert tuner._precise_paths(5, 256) == ["small", "exact"]
    assert tuner._precise_paths(4, 100) == ["lines", "exact"]
    assert tuner._precise_paths(40, 256) == ["exact"]
    assert tuner._precise_paths(2, 256, groups=True) == ["exact"]  # group-scaled weights have no few-token kernel
    x, w, s = operands(3, groups=True)
    tuner.fake.times = {"exact": 1.0, "block": 2.0}
    assert tuner.choose_path(x, w, s) == "exact"
    assert "path|3x96x256|g0|wgroups|Fake B200" in tuner._cache()
    x, w, s = operands(3)
    tuner.fake.times = {"lines": 1.0, "small": 2.0, "exact": 3.0, "block": 4.0}
    tuner.choose_path(x, w, s, group=64, act="gelu")
    assert "path|3x96x256|g64|gelu|Fake B200" in tuner._cache()


def test_capture_uses_static_thresholds_and_caches_nothing(tuner, monkeypatch):
    monkeypatch.setattr(tuner, "_capturing", lambda: True)
    picks = [tuner.choose_path(*operands(m)) for m in (1, 2, 3, 16, 17, 64, 65)]
    assert picks == ["lines", "lines", "small", "small", "exact", "exact", "block"]
    assert tuner.choose_path(*operands(500), precise=True) == "exact"
    assert tuner.choose_path(*operands(2, groups=True)) == "exact"
    assert tuner.calls == [] and tuner._cache() == {} and tuner._paths == {}
    a, b = torch.zeros(100, 256, dtype=torch.int8), torch.zeros(96, 256, dtype=torch.int8)
    config, tuned = tuner._tuned_config(100, 96, 256, a.device, "block", lambda option: None)
    assert config == tuner._CANDIDATES["block"][0] and not tuned


def test_tile_tuner_picks_the_fastest_candidate(tuner):
    a, b = torch.zeros(100, 256, dtype=torch.int8), torch.zeros(96, 256, dtype=torch.int8)
    tuner.fake.times = {(10, 0): 2.0, (20, 0): 2.5, (15, 0): 1.0}
    config, tuned = tuner._tuned_config(100, 96, 256, a.device, "block", lambda option: None)
    assert config == (15, 0) and tuned
    assert tuner._cache()["block|128x96x256|Fake B200"] == [15, 0]
    tuner.fake.times = {(10, 0): 0.5, (20, 0): 2.5, (15, 0): 1.0}
    assert tuner._tuned_config(100, 96, 256, a.device, "block", lambda option: None)[0] == (15, 0)  # cached
    # a mode with one candidate needs no timing
    before = len(tuner.calls)
    assert tuner._tuned_config(100, 96, 256, a.device, "exact", lambda option: None) == ((1, 0), True)
    assert len(tuner.calls) == before
    assert set(tuner._MODES[v] for mode, candidates in tuner._CANDIDATES.items() for v, _ in candidates if tuner._MODES[v] != mode) == set()


def test_no_library_no_result(monkeypatch):
    """Nothing computes without the CUDA library: there is no CPU path to fall back to."""
    monkeypatch.setattr(wq, "_lib", None)
    x, w, s = operands(4)
    for call in (lambda: wq.linear(x, w, s, mode="block"), lambda: wq.quantize_blocks(x), lambda: wq.quantize(x), lambda: wq.transform_rows(x),
                 lambda: wq.gemv_lines(x, w, s), lambda: wq.small(x, w, s), lambda: wq.selftest("cpu")):
        with pytest.raises(RuntimeError, match="not loaded"):
            call()
    with pytest.raises(RuntimeError, match="not found"):
        wq.load_library("/nonexistent/libwgp_int8.so")


def test_prepared_rows_slice_every_part():
    p = wq.Prepared("exact", torch.arange(12).view(6, 2), torch.arange(12).view(6, 2) + 100, torch.arange(6.0), torch.bfloat16)
    part = p.rows(2, 5)
    assert part.path == "exact" and part.dtype == torch.bfloat16
    assert part.x.shape == (3, 2) and part.lo[0, 0] == 104 and part.scale.tolist() == [2.0, 3.0, 4.0]
    assert wq.Prepared("lines", torch.zeros(4, 2), None, None, torch.float16).rows(1, 2).scale is None
