"""Host-side helpers of the shared host buffers (no GPU): the mapping shared by processes, the parsing of a GPU's CPU list and the
first-touch placement with the thread's affinity put back."""
import os

import torch

from wgpkernels_b200 import host


def test_shared_mapping_is_the_same_bytes_in_two_mappings(tmp_path):
    path = f"/dev/shm/wgpkernels_b200_test_{os.getpid()}"
    try:
        first = host._shared_mapping(path, (6, 16), torch.bfloat16, True)
        second = host._shared_mapping(path, (6, 16), torch.bfloat16, False)
        assert first.shape == (6, 16) and float(first.float().abs().sum()) == 0.0  # a new file reads as zeros
        first[2:4] = 1.5
        assert torch.equal(second, first) and float(second[3, 5]) == 1.5
    finally:
        os.unlink(path)


def test_touch_near_writes_zeros_and_restores_the_affinity(monkeypatch):
    before = os.sched_getaffinity(0)
    one = {min(before)}
    seen = []
    monkeypatch.setattr(host, "_cpus_near", lambda device: one)
    real = os.sched_setaffinity
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cpus: (seen.append(set(cpus)), real(pid, cpus)))
    band = torch.ones(5, 8, dtype=torch.bfloat16)
    host._touch_near(0, (band[1:3], band[4:]))
    assert seen == [one, set(before)] and os.sched_getaffinity(0) == before
    assert float(band[1:3].float().sum()) == 0.0 and float(band[4:].float().sum()) == 0.0 and float(band[0].float().sum()) == 8.0


def test_cpus_near_without_a_gpu_is_unknown():
    assert host._cpus_near(0) is None or isinstance(host._cpus_near(0), set)
