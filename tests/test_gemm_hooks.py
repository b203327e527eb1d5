"""Tile-by-tile hand-off hooks of the CTA-pair grouped GEMM (per-row arrival flags, per-slot weight flags, per-row-block
output counters).  The waits are bounded: a flag that nothing sets makes the kernel give up after its budget, record a
status and return (no hang, no trap)."""

import pytest
import torch

from moonep_b200.ops.grouped_gemm import GemmHooks, grouped_gemm, grouped_gemm_reference


def _case(rows_per_group, K, N, seed=0):
    g = torch.Generator().manual_seed(seed)
    ends, total = [], 0
    for r in rows_per_group:
        total += r
        ends.append(total)
    G = len(rows_per_group)
    x = (torch.randn(total + 256, K, generator=g) * 0.5).to(torch.bfloat16).cuda()
    w = (torch.randn(G, N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    cu = torch.tensor(ends, dtype=torch.int32, device="cuda")
    return x, w, cu, total


def _hooks(row_flags=None, row_epoch=0, slot_flags=None, slot_epoch=0, first=0, done=None, tables=None, tables_epoch=0):
    h = GemmHooks()
    if row_flags is not None:
        h.row_flags, h.row_epoch = row_flags.data_ptr(), row_epoch
    if slot_flags is not None:
        h.slot_flags, h.slot_epoch, h.slot_first_group = slot_flags.data_ptr(), slot_epoch, first
    if done is not None:
        h.done_counter = done.data_ptr()
    if tables is not None:
        h.tables_ready, h.tables_epoch = tables.data_ptr(), tables_epoch
    return h


@pytest.mark.gpu
def test_hooked_gemm_equals_plain_and_counts_finished_tiles():
    rows = [256, 0, 128, 384, 128]
    x, w, cu, total = _case(rows, 256, 512)
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    row_flags = torch.full((x.shape[0],), 5, dtype=torch.int32, device="cuda")  # every row arrived in epoch 5
    slot_flags = torch.tensor([3, 3], dtype=torch.int32, device="cuda")  # groups 3 and 4 use "prefetched" weights
    tables = torch.tensor([9], dtype=torch.int32, device="cuda")
    done = torch.zeros((x.shape[0] + 127) // 128, dtype=torch.int32, device="cuda")
    h = _hooks(row_flags, 5, slot_flags, 3, 3, done, tables, 9)
    y = grouped_gemm(x, w, cu, status=status, pair=True, hooks=h)
    y0 = grouped_gemm(x, w, cu, status=status, pair=True)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, status.tolist()
    assert torch.equal(y[:total], y0[:total])
    want = grouped_gemm_reference(x, w, cu)
    assert (y[:total].float() - want[:total].float()).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item())
    # every 128-row block with rows was finished by 4 epilogue warps per column tile (N / 256 tiles)
    blocks = total // 128
    assert done[:blocks].tolist() == [4 * (512 // 256)] * blocks and int(done[blocks:].sum()) == 0
    # a second call counts on
    grouped_gemm(x, w, cu, status=status, pair=True, hooks=h)
    torch.cuda.synchronize()
    assert done[:blocks].tolist() == [8 * (512 // 256)] * blocks


@pytest.mark.gpu
@pytest.mark.parametrize("what", ["rows", "slot", "tables"])
def test_hooked_gemm_gives_up_on_a_flag_nothing_sets(what, monkeypatch):
    monkeypatch.setenv("MOONEP_TIMEOUT_MS", "200")
    rows = [128, 256, 128]
    x, w, cu, total = _case(rows, 128, 256, seed=1)
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    row_flags = torch.full((x.shape[0],), 2, dtype=torch.int32, device="cuda")
    slot_flags = torch.tensor([2], dtype=torch.int32, device="cuda")
    tables = torch.tensor([2], dtype=torch.int32, device="cuda")
    if what == "rows":
        row_flags[200] = 1  # one row of the second block never arrives in epoch 2
    elif what == "slot":
        slot_flags[0] = 1  # the prefetch of the last group's weights never completes
    else:
        tables[0] = 1  # the planner tables never come out
    h = _hooks(row_flags, 2, slot_flags, 2, 2, None, tables, 2)
    grouped_gemm(x, w, cu, status=status, pair=True, hooks=h)
    torch.cuda.synchronize()  # returns: the wait is bounded
    st = status.tolist()
    assert st[0] == 1 and st[1] == 15, f"expected a timeout recorded by the CTA-pair GEMM, got {st}"
    assert st[2] == {"rows": 11, "slot": 12, "tables": 10}[what], st
    # the device is still usable and the same call succeeds once the flag is there
    status.zero_()
    row_flags.fill_(2)
    slot_flags.fill_(2)
    tables.fill_(2)
    y = grouped_gemm(x, w, cu, status=status, pair=True, hooks=h)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    want = grouped_gemm_reference(x, w, cu)
    assert (y[:total].float() - want[:total].float()).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item())


def test_group_without_weights_is_an_error_on_the_reference_path():
    x = torch.randn(256, 64).to(torch.bfloat16)
    w = torch.randn(1, 256, 64).to(torch.bfloat16)
    cu = torch.tensor([128, 256], dtype=torch.int32)
    gm = torch.tensor([0, -1], dtype=torch.int32)  # the second group has rows but its expert is not on this rank
    with pytest.raises(IndexError):
        grouped_gemm_reference(x, w, cu, group_map=gm)
    gm_ok = torch.tensor([0, 0], dtype=torch.int32)
    assert grouped_gemm_reference(x, w, cu, group_map=gm_ok).shape == (256, 256)


@pytest.mark.gpu
@pytest.mark.parametrize("pair", [False, True])
def test_group_without_weights_is_reported_by_the_kernels(pair):
    x, w, cu, total = _case([128, 128], 64, 256, seed=2)
    gm = torch.tensor([0, -1], dtype=torch.int32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    grouped_gemm(x, w[:1].contiguous(), cu, status=status, pair=pair, group_map=gm)
    torch.cuda.synchronize()
    st = status.tolist()
    assert st[0] == 2 and st[2] == 13, f"expected an index error for the group without weights, got {st}"
