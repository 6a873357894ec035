"""Fused Adam: drop-in for ``d3sim.ops.optim.adam.GaussianAdam``.

``GaussianAdam`` stays a ``torch.optim.Adam`` subclass with the torch state keys ``step`` (CPU tensor),
``exp_avg`` and ``exp_avg_sq`` (d3sim/ops/optim/adam.py:382-418), so optimizer-state surgery written
for the reference (d3sim/algos/d3gs/strategy.py:19-66) keeps working.  Where the reference launches
one kernel per parameter tensor (six per iteration, adam.py:415-417), ``step()`` here covers all
tensors of the optimizer in one launch, and ``fused_step`` covers SEVERAL optimizers plus the
densification statistics (d3sim/algos/d3gs/origin/strategy.py:93-122) in one launch.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Iterable

import torch

from . import _lib

MAX_SEGMENTS = 8


def _segments_of(optim: "GaussianAdam") -> list[_lib.AdamSegment]:
    segs = []
    for group in optim.param_groups:
        assert not group.get("fused", False), "construct GaussianAdam with fused=False (the reference does)"
        assert not group.get("amsgrad", False) and not group.get("maximize", False), "amsgrad/maximize not built"
        beta1, beta2 = group["betas"]
        for p in group["params"]:
            if p.grad is None:
                continue
            assert p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and p.grad.is_contiguous()
            state = optim.state[p]
            if len(state) == 0:
                state["step"] = torch.tensor(0.0, dtype=torch.float32)
                state["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                state["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            state["step"] += 1
            step = float(state["step"])
            # bias corrections on the host in double (adam.py:55-57)
            bc1 = 1.0 - math.pow(beta1, step)
            bc2_sqrt = math.sqrt(1.0 - math.pow(beta2, step))
            s = _lib.AdamSegment()
            s.param, s.grad = p.data_ptr(), p.grad.data_ptr()
            s.exp_avg, s.exp_avg_sq = state["exp_avg"].data_ptr(), state["exp_avg_sq"].data_ptr()
            s.count = p.numel()
            s.lr, s.beta1, s.beta2, s.eps = float(group["lr"]), float(beta1), float(beta2), float(group["eps"])
            s.bias_correction1, s.bias_correction2_sqrt = bc1, bc2_sqrt
            s.grad_scale, s.weight_decay = 1.0, float(group["weight_decay"])
            segs.append(s)
    return segs


def _launch(segs: list[_lib.AdamSegment], stats: _lib.DensifyStats | None, device,
            peers: "_lib.PeerSet | None" = None):
    """``peers``: gradients are summed over every rank's buffer and parameters stored into every rank's
    buffer through peer mappings (``d3gs_adam_stats_step_peers``)."""
    lib = _lib.load()
    stream = torch.cuda.current_stream(device).cuda_stream
    first = True
    for k in range(0, max(len(segs), 1), MAX_SEGMENTS):
        chunk = segs[k:k + MAX_SEGMENTS]
        arr = (_lib.AdamSegment * max(len(chunk), 1))(*chunk)
        st = C.byref(stats) if (stats is not None and first) else None
        if peers is None:
            _lib.check(lib.d3gs_adam_stats_step(arr, len(chunk), st, stream), "d3gs_adam_stats_step")
        else:
            _lib.check(lib.d3gs_adam_stats_step_peers(arr, len(chunk), st, C.byref(peers), stream),
                       "d3gs_adam_stats_step_peers")
        first = False


class GaussianAdam(torch.optim.Adam):
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        segs = _segments_of(self)
        if segs:
            _launch(segs, None, self.param_groups[0]["params"][0].device)
        return loss


def make_stats_struct(state, radii: torch.Tensor, duv: torch.Tensor, width: int, height: int,
                      need_max_radii: bool, loss_batch: int = 0) -> _lib.DensifyStats:
    """``duv`` is [B,N,2]: dense, or a strided view (last two dims' strides (s, 1)) of the packed per-splat
    gradient array, which is then read in place."""
    assert duv.ndim == 3 and duv.shape[2] == 2 and radii.is_contiguous()
    b, n, _ = duv.shape
    if not (duv.stride(2) == 1 and duv.stride(0) == n * duv.stride(1) and duv.stride(1) % 2 == 0
            and duv.data_ptr() % 8 == 0):
        duv = duv.contiguous()
    assert radii.numel() == b * n and state.duv_ndc_length.shape[0] == n
    st = _lib.DensifyStats()
    st.duv, st.radii = duv.data_ptr(), radii.data_ptr()
    st.duv_stride = int(duv.stride(1))
    st.duv_ndc_length, st.count, st.max_radii = (state.duv_ndc_length.data_ptr(), state.count.data_ptr(),
                                                 state.max_radii.data_ptr())
    st.num, st.batch, st.width, st.height, st.need_max_radii = n, b, int(width), int(height), int(need_max_radii)
    st.loss_batch = int(loss_batch)
    st._keepalive = (duv, radii, state)   # the struct holds raw addresses only
    return st


@torch.no_grad()
def fused_step(optims: Iterable[GaussianAdam], stats: _lib.DensifyStats | None = None):
    """One launch for all the given optimizers (and the densification statistics, when given)."""
    segs, dev = [], None
    for o in optims:
        s = _segments_of(o)
        if s and dev is None:
            dev = o.param_groups[0]["params"][0].device
        segs += s
    if dev is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    if segs or stats is not None:
        _launch(segs, stats, dev)
