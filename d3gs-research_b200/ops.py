"""Point-cloud operators of the initialisation path (d3sim/algos/d3gs/ops.py).

``simple_knn(points, k, use_64bit=False)`` has the reference's signature and result: a ``[n, k]`` float tensor of
the distances from every point to its ``k`` nearest other points, ascending.  The work is done by
``d3gs_simple_knn`` of the sm_100a library (Morton codes, radix sort, boxes of 256 sorted points, one CTA per
box); there is no host fallback.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib


def simple_knn(points: torch.Tensor, k: int, use_64bit: bool = False) -> torch.Tensor:
    assert points.is_contiguous() and points.dim() == 2 and points.shape[1] >= 3     # ops.py:18
    assert points.dtype == torch.float32, "points must be float32"
    if not points.is_cuda:
        raise RuntimeError("simple_knn runs on the GPU: pass a CUDA tensor")
    lib = _lib.load()
    n = points.shape[0]
    dev = points.device
    out = torch.empty([n, k], dtype=torch.float32, device=dev)
    if n == 0:
        return out
    bits = 21 if use_64bit else 10                                                   # ops.py:29
    pmin = points[:, :3].min(0).values.contiguous()                                  # ops.py:21-22
    pmax = points[:, :3].max(0).values.contiguous()
    ws = torch.empty(lib.d3gs_simple_knn_workspace_bytes(n, bits), dtype=torch.uint8, device=dev)
    status = torch.zeros(2, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(lib.d3gs_simple_knn(points.data_ptr(), points.stride(0), n, int(k), bits, pmin.data_ptr(),
                                   pmax.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(), status.data_ptr(),
                                   stream), "d3gs_simple_knn")
    if int(status[0].item()) != 0:
        raise RuntimeError(f"d3gs_simple_knn: device status {int(status[0].item()):#x} (a bounded wait of the sort gave up)")
    return out
