"""Buffer layout, padding helpers, constants shared with the native library, environment switches."""

import ctypes

import pytest
import torch

from moonep_b200 import config, constants
from moonep_b200.layout import align_up, check_encoding_bounds, compute_layout, pad_dim0_for_alignment, pad_to_granularity


@pytest.mark.parametrize("S,H,K,E,R,B,P", [(4096, 7168, 8, 256, 8, None, 128), (1, 16, 1, 1, 1, None, 8),
                                           (33, 48, 2, 4, 2, 1, 1), (256, 16, 1, 2050, 2, 1, 1), (8192, 4096, 6, 64, 8, 4, 128)])  # fmt: skip
def test_meta_layout_follows_the_reference_formulas(S, H, K, E, R, B, P):
    lay = compute_layout(S, H, K, E, R, B=B, token_padding=P)
    epn = E // R
    Bv = epn if B is None else B
    N = S * K
    assert lay["NvS"] == N + (P - 1) * 2 * epn and lay["N"] == N and lay["B"] == Bv
    planning_out = 3 * E * R + R * (E + Bv) + 2 * R * (E + Bv) + R * Bv + 2 * R
    n4 = align_up(N, 4)
    assert lay["WEIGHTS_OFF"] == 0 and lay["TPE_OFF"] == align_up(lay["NvS"], 4)
    assert lay["PLAN_OFF"] == align_up(lay["TPE_OFF"] + R * E, 4)
    assert lay["TOPK0_OFF"] == align_up(lay["PLAN_OFF"] + planning_out, 4)
    assert lay["ORDER_OFF"] == lay["TOPK0_OFF"] + n4 and lay["ORDER0_OFF"] == lay["ORDER_OFF"] + n4
    assert lay["BARRIER_OFF"] == lay["ORDER0_OFF"] + n4 and lay["SRC_INFO_OFF"] == lay["BARRIER_OFF"] + 3
    # additions live past the reference's logical end and inside the padded chunk
    assert lay["SYNC_OFF"] >= lay["SRC_INFO_OFF"] + lay["NvS"] and lay["LINK_OFF"] > lay["SYNC_OFF"]
    assert lay["meta_chunk_padded"] >= lay["LINK_OFF"] + lay["NvS"]
    assert (lay["meta_chunk_padded"] * 4) % 128 == 0 and (lay["NvS_padded"] * H * 2) % 128 == 0
    assert lay["NvS_padded"] >= lay["NvS"]
    check_encoding_bounds(lay)


def test_vmm_granularity_padding():
    lay = compute_layout(4096, 7168, 8, 256, 8, gran_bytes=2 << 20)
    assert (lay["NvS_padded"] * 7168 * 2) % (2 << 20) == 0 and (lay["meta_chunk_padded"] * 4) % (2 << 20) == 0
    assert pad_dim0_for_alignment([3, 48], torch.bfloat16) * 96 % 128 == 0
    assert pad_to_granularity(1, 128) == 128 and pad_to_granularity(256, 128) == 256


def test_encoding_bounds_are_enforced():
    with pytest.raises(AssertionError):
        check_encoding_bounds(compute_layout(8, 16, 33, 64, 2))  # K > 32
    with pytest.raises(AssertionError):
        check_encoding_bounds({"R": 2, "S": 1, "K": 1, "NvS": 1 << 24})
    with pytest.raises(AssertionError):
        compute_layout(8, 16, 2, 10, 4)  # E not a multiple of R


def test_constants_match_the_native_header():
    from moonep_b200.ops import _lib

    text = (_lib.CSRC / "moonep.h").read_text()

    def c_define(name):
        for line in text.splitlines():
            parts = line.split()
            if len(parts) >= 3 and parts[0] == "#define" and parts[1] == name:
                return int(parts[2], 0)
        raise KeyError(name)

    assert c_define("MOONEP_KIDX_BITS") == constants.KIDX_BITS and c_define("MOONEP_NVS_BITS") == constants.NVS_BITS
    assert c_define("MOONEP_MAX_TOPK") == constants.MAX_TOPK and c_define("MOONEP_MAX_RANKS") == constants.MAX_RANKS
    assert c_define("MOONEP_NUM_FLAG_FAMILIES") == constants.NUM_FLAG_FAMILIES
    assert c_define("MOONEP_PLAN_BLOCK") == constants.PLAN_BLOCK
    for fam in ("READY", "TPE", "PLAN", "SENT", "COMB", "GRAD_READY", "GRAD_DONE"):
        assert c_define(f"MOONEP_FLAG_{fam}") == getattr(constants, f"FLAG_{fam}")
    lib = _lib.load()
    assert lib.moonep_version() == c_define("MOONEP_VERSION")
    assert lib.moonep_planner_table_words(8, 256, 32) == 2 * 256 + 3 * 8 * 256 + 64 + 16
    g = ctypes.c_ulonglong(0)
    if not torch.cuda.is_available():  # without a driver the allocator reports an error instead of crashing
        assert lib.moonep_vmm_granularity(0, ctypes.byref(g)) != 0 and b"driver" in lib.moonep_last_error()


def test_environment_switches(monkeypatch):
    monkeypatch.delenv("MOONEP_PLANNER", raising=False)
    monkeypatch.delenv("MOONEP_TD_PLANNING_TRITON", raising=False)
    assert config.planner_on_gpu()
    monkeypatch.setenv("MOONEP_TD_PLANNING_TRITON", "0")
    assert not config.planner_on_gpu()
    monkeypatch.setenv("MOONEP_PLANNER", "gpu")
    assert config.planner_on_gpu()
    monkeypatch.setenv("MOONEP_COPY_PATH", "ldst")
    assert config.copy_path("send") == "ldst" and config.copy_path("pull") == "ldst"
    monkeypatch.setenv("MOONEP_SEND_PATH", "bulk")
    assert config.copy_path("send") == "bulk"
    monkeypatch.setenv("MOONEP_PULL_PATH", "nope")
    with pytest.raises(ValueError):
        config.copy_path("pull")
    monkeypatch.setenv("MOONEP_NUM_SMS_DEDUP", "200")
    with pytest.raises(ValueError):
        config.num_sms_dedup(148)
    monkeypatch.setenv("MOONEP_NUM_SMS_DEDUP", "7")
    assert config.num_sms_dedup(148) == 7
    monkeypatch.setenv("MOONEP_TIMEOUT_MS", "250")
    assert config.timeout_ms() == 250
    monkeypatch.setenv("MOONEP_LOCAL_SMS", "1000")
    assert config.local_sms(148) == 148


def test_symmetric_tensor_helpers_on_an_emulated_world():
    from moonep_b200.parallel.symm import (create_nvl_dist_tensor, create_nvl_single_owner_tensor, nvl_dist_peer_row,
                                           release_nvl_dist_tensor, view_nvl_dist_rows)  # fmt: skip
    from moonep_b200.parallel.world import LocalWorld

    lw = LocalWorld(3, "cpu")

    def body(r):
        w = lw.view(r)
        full = create_nvl_dist_tensor([2, 4, 8], torch.float32, w)
        rows = full.shape[0] // 3
        full[r * rows : (r + 1) * rows].fill_(float(r + 1))
        w.step()
        v = view_nvl_dist_rows(full, 3, rows)
        ok = all(float(nvl_dist_peer_row(full, p, r, 3, rows).mean()) == p + 1 for p in range(3)) and v.shape[:2] == (3, rows)
        owner = create_nvl_single_owner_tensor([2, 4, 8], torch.float32, 1, w)
        if r == 1:
            owner.fill_(7.0)
        w.step()
        ok = ok and float(owner.mean()) == 7.0 and owner.shape == (2, 4, 8)
        w.step()
        release_nvl_dist_tensor(full)
        return ok

    assert all(lw.run(body))
