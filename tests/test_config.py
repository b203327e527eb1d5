"""Environment switches: defaults, overrides and rejected values (``moonep_b200/config.py``)."""

import pytest

from moonep_b200 import config


def test_copy_path_defaults_and_overrides(monkeypatch):
    for name in ("MOONEP_COPY_PATH", "MOONEP_SEND_PATH", "MOONEP_PULL_PATH", "MOONEP_GRAD_PATH", "MOONEP_PREFETCH_PATH"):
        monkeypatch.delenv(name, raising=False)
    assert config.copy_path("send") == "bulk" and config.copy_path("pull") == "ldst" and config.copy_path("grad") == "ldst"
    assert config.copy_path("prefetch") == "async" and not config.copy_path_is_set("prefetch")
    monkeypatch.setenv("MOONEP_COPY_PATH", "ldst")
    assert config.copy_path("send") == "ldst"
    assert config.copy_path("prefetch") == "async", "the prefetch keeps its ring whatever the general switch says"
    monkeypatch.setenv("MOONEP_PREFETCH_PATH", "ldst")
    assert config.copy_path("prefetch") == "ldst" and config.copy_path_is_set("prefetch")
    monkeypatch.setenv("MOONEP_SEND_PATH", "async")  # only the prefetch has a cp.async ring
    with pytest.raises(ValueError):
        config.copy_path("send")
    monkeypatch.setenv("MOONEP_GRAD_PATH", "tma")
    with pytest.raises(ValueError):
        config.copy_path("grad")


@pytest.mark.parametrize(
    "fn,name,default",
    [
        (config.local_rows_by_expand, "MOONEP_LOCAL_ROWS", True),
        (config.local_home_by_fold, "MOONEP_LOCAL_HOME", True),
        (config.fuse_plan_publish, "MOONEP_FUSE_PUBLISH", False),
        (config.backward_overlap, "MOONEP_BWD_OVERLAP", False),
        (config.pdl_allowed, "MOONEP_PDL", True),
    ],
)
def test_boolean_switches(fn, name, default, monkeypatch):
    monkeypatch.delenv(name, raising=False)
    assert fn() is default
    monkeypatch.setenv(name, "0")
    assert fn() is False
    monkeypatch.setenv(name, "1")
    assert fn() is True
