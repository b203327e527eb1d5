"""The measurement kernel behind ``bench.py --config p2p_peak`` (SM-driven bulk-copy ring) copies what it is given."""

import pytest
import torch


@pytest.mark.gpu
@pytest.mark.parametrize("nbytes,chunk,grid,fence_warps", [(1 << 20, 4096, 4, 0), (3 * 14336 * 7 + 16, 14336, 3, 2),
                                                           (48, 16, 1, 0)])  # fmt: skip
def test_peer_store_kernel_copies_its_input(nbytes, chunk, grid, fence_warps):
    from moonep_b200.ops import _lib

    lib = _lib.load()
    src = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device="cuda")
    dst = torch.zeros(nbytes + 64, dtype=torch.uint8, device="cuda")
    words = torch.zeros(grid * 4 * 32, dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.moonep_peer_store_bench(dst.data_ptr(), src.data_ptr(), nbytes, chunk, grid, err.data_ptr(), 2000, fence_warps,
                                     words.data_ptr() if fence_warps else None, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.moonep_last_error().decode()
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert torch.equal(dst[:nbytes], src) and not bool(dst[nbytes:].any()), "copy differs or ran past the end"
    # refused before any launch: sizes that are not multiples of 16 bytes
    assert lib.moonep_peer_store_bench(dst.data_ptr(), src.data_ptr(), 24, 16, 1, err.data_ptr(), 2000, 0, None,
                                       torch.cuda.current_stream().cuda_stream) != 0
