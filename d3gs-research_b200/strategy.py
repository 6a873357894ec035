"""Densification statistics: drop-in for the hot-path part of ``GaussianStrategyOrigin``.

``GaussianTrainState`` (d3sim/algos/d3gs/strategy.py:88-110) and ``GaussianStrategyOrigin.update``
(d3sim/algos/d3gs/origin/strategy.py:75-122) are provided.  The densify / prune / opacity-reset
policy (origin/strategy.py:159-363) runs every 100+ iterations outside the training step and is not
part of this library.
"""
from __future__ import annotations

import dataclasses

import torch

from . import _lib
from .adam import make_stats_struct
from .render import GaussianSplatOutput


@dataclasses.dataclass
class GaussianTrainState:
    duv_ndc_length: torch.Tensor
    count: torch.Tensor
    max_radii: torch.Tensor
    scene_scale: float = 1.0

    @classmethod
    def create(cls, num_gaussian: int, scene_scale: float = 1.0, device=None):
        z = lambda: torch.zeros(num_gaussian, dtype=torch.float32, device=device)
        return cls(duv_ndc_length=z(), count=z(), max_radii=z(), scene_scale=scene_scale)

    def reset(self):
        self.duv_ndc_length.zero_()
        self.count.zero_()
        self.max_radii.zero_()


@dataclasses.dataclass
class GaussianStrategyOrigin:
    reset_opacity_thresh: float = 0.01
    prune_opacity_thresh: float = 0.005
    grow_grad2d: float = 0.0002
    grow_scale3d: float = 0.01
    grow_scale2d: float = 0.05
    prune_scale3d: float = 0.1
    prune_scale2d: float = 0.15
    refine_scale2d_stop_iter: int = 0
    refine_start_iter: int = 500
    refine_stop_iter: int = 15_000
    reset_opacity_every: int = 3000
    refine_every: int = 100
    absgrad: bool = False
    revised_opacity: bool = False
    verbose: bool = False

    def rescale_steps_by_batch_size(self, batch_size: int):
        self.refine_start_iter //= batch_size
        self.refine_stop_iter //= batch_size
        self.refine_every //= batch_size
        self.reset_opacity_every //= batch_size

    def stats_struct(self, state: GaussianTrainState, out: GaussianSplatOutput, duv: torch.Tensor):
        width, height = out.image_shape_wh
        assert out.radii is not None and out.sparse_gaussian_ids is None
        # the kernel indexes radii flat as view*N + gaussian (origin/strategy.py:102-104); the op returns
        # radii 1-D (render.py:642) and both 1-D and [B,N] are accepted here
        return make_stats_struct(state, out.radii.reshape(-1), duv, width, height,
                                 self.refine_scale2d_stop_iter > 0)

    @torch.no_grad()
    def update(self, state: GaussianTrainState, out: GaussianSplatOutput, duv: torch.Tensor):
        assert duv.ndim == 3
        st = self.stats_struct(state, out, duv)
        lib = _lib.load()
        _lib.check(lib.d3gs_densify_stats(st, torch.cuda.current_stream(duv.device).cuda_stream), "d3gs_densify_stats")

    def refine_gs(self, *args, **kwargs):
        raise NotImplementedError("densification / pruning policy is outside the training-step library")
