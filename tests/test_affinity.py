"""CPU-socket binding helper: decisions against a fake NVML answer, without changing this process for real."""

import os

import pytest

from moonep_b200.utils import affinity


@pytest.fixture
def fake_sched(monkeypatch):
    state = {"allowed": set(range(8)), "set_calls": []}
    monkeypatch.setattr(os, "sched_getaffinity", lambda pid: set(state["allowed"]), raising=False)
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cpus: state["set_calls"].append(set(cpus)), raising=False)
    monkeypatch.delenv("MOONEP_NO_AFFINITY", raising=False)
    return state


def test_binds_to_the_intersection(fake_sched, monkeypatch):
    monkeypatch.setattr(affinity, "gpu_cpu_set", lambda index: {4, 5, 6, 7, 12, 13})
    out = affinity.bind_to_gpu_socket(0)
    assert out == {"applied": True, "cpus": 4} and fake_sched["set_calls"] == [{4, 5, 6, 7}]


def test_leaves_the_process_alone_when_it_should(fake_sched, monkeypatch):
    monkeypatch.setattr(affinity, "gpu_cpu_set", lambda index: None)
    assert affinity.bind_to_gpu_socket(0)["applied"] is False
    monkeypatch.setattr(affinity, "gpu_cpu_set", lambda index: {9})  # none of the GPU's CPUs is available here
    assert affinity.bind_to_gpu_socket(0)["applied"] is False
    monkeypatch.setattr(affinity, "gpu_cpu_set", lambda index: set(range(16)))  # already inside the GPU's set
    assert affinity.bind_to_gpu_socket(0)["applied"] is False
    monkeypatch.setenv("MOONEP_NO_AFFINITY", "1")
    monkeypatch.setattr(affinity, "gpu_cpu_set", lambda index: {1, 2, 3})
    assert affinity.bind_to_gpu_socket(0)["applied"] is False
    assert fake_sched["set_calls"] == []


def test_reading_nvml_never_raises():
    assert affinity.gpu_cpu_set(0) is None or isinstance(affinity.gpu_cpu_set(0), set)
