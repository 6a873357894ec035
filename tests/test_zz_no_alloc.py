"""The allocation-free scan entry point against the workspace-taking one.

``d3gs_scan_tiles_static`` exists for callers that have no way to get device memory at call time (their
budget sits in another engine's pool, they run in a frame loop that cannot afford cudaMalloc's device-wide
stall, or they are plain C hosts without an allocator): it keeps its tile-status scratch in a fixed array
inside the library.  Both entry points run the same kernel, so their integer outputs must be identical.  The
array is shared by every call and keeps the previous call's contents, hence two calls in a row with different
sizes: the second one must not be disturbed by what the first one left behind.

This file sorts last on purpose, so that a run that stops at the first failure has already run everything else.
"""
import numpy as np
import pytest
import torch

from d3gs_research_b200 import _lib

pytestmark = pytest.mark.gpu


def _scan_with_workspace(lib, x):
    n = x.numel()
    out = torch.empty_like(x)
    sync = torch.zeros(2, dtype=torch.int64, device=x.device)
    ws = torch.empty(lib.d3gs_scan_workspace_bytes(n) + 64, dtype=torch.uint8, device=x.device)
    _lib.check(lib.d3gs_scan_tiles(x.data_ptr(), out.data_ptr(), n, sync.data_ptr(), ws.data_ptr(), ws.numel(),
                                   sync.data_ptr() + 8, torch.cuda.current_stream().cuda_stream), "d3gs_scan_tiles")
    total, status = sync.tolist()
    assert status == 0
    return out, total


def _scan_static(lib, x):
    n = x.numel()
    out = torch.empty_like(x)
    sync = torch.zeros(2, dtype=torch.int64, device=x.device)
    _lib.check(lib.d3gs_scan_tiles_static(x.data_ptr(), out.data_ptr(), n, sync.data_ptr(), sync.data_ptr() + 8,
                                          torch.cuda.current_stream().cuda_stream), "d3gs_scan_tiles_static")
    total, status = sync.tolist()
    assert status == 0
    return out, total


def test_static_scratch_scan_matches_workspace_scan_twice_in_a_row(cuda_device):
    lib = _lib.load()
    g = torch.Generator().manual_seed(77)
    # many tiles; then fewer tiles and a ragged tail, reusing the same scratch; then more tiles again than the call
    # before cleared
    for n in (3_000_017, 70_001, 1_500_003):
        x = torch.randint(0, 40, (n,), generator=g, dtype=torch.int32).to(cuda_device)
        ref, ref_total = _scan_with_workspace(lib, x)
        got, got_total = _scan_static(lib, x)
        assert got_total == ref_total == int(x.sum(dtype=torch.int64))
        assert torch.equal(got, ref)       # integer work: bit-exact
        np.testing.assert_array_equal(got[-5:].cpu().numpy(), np.cumsum(x.cpu().numpy().astype(np.int64))[-5:])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs a second GPU")
def test_static_scratch_scan_on_a_second_device(cuda_device):
    """Every GPU that loads the library holds its own copy of the array; its address is looked up per device."""
    lib = _lib.load()
    g = torch.Generator().manual_seed(78)
    x = torch.randint(0, 40, (200_003,), generator=g, dtype=torch.int32)
    for dev in (torch.device("cuda", 1), torch.device("cuda", 0)):
        with torch.cuda.device(dev):
            xd = x.to(dev)
            ref, ref_total = _scan_with_workspace(lib, xd)
            got, got_total = _scan_static(lib, xd)
            assert got_total == ref_total and torch.equal(got, ref)


def test_static_scratch_scan_rejects_sizes_beyond_its_capacity(cuda_device):
    lib = _lib.load()
    cap = lib.d3gs_scan_tiles_static_max_items()
    assert cap == 1 << 24
    sync = torch.zeros(2, dtype=torch.int64, device=cuda_device)
    dummy = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    rc = lib.d3gs_scan_tiles_static(dummy.data_ptr(), dummy.data_ptr(), cap + 1, sync.data_ptr(), sync.data_ptr() + 8,
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == -1 and "at most" in _lib.last_error()
    # n == 0 is valid and only clears the total
    sync.fill_(5)
    _lib.check(lib.d3gs_scan_tiles_static(None, None, 0, sync.data_ptr(), sync.data_ptr() + 8,
                                          torch.cuda.current_stream().cuda_stream), "empty scan")
    assert sync.tolist()[0] == 0
