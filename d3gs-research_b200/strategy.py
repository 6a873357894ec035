"""Densification statistics: drop-in for the hot-path part of ``GaussianStrategyOrigin``.

``GaussianTrainState`` (d3sim/algos/d3gs/strategy.py:88-110), ``GaussianStrategyOrigin.update``
(d3sim/algos/d3gs/origin/strategy.py:75-122), the densify / prune policy ``refine_gs``
(origin/strategy.py:159-363, with the optimizer-state surgery of strategy.py:131-178) and the opacity reset
(origin/trainer.py:388-417, strategy.py:181-202).

``refine_gs`` here is three launches around one host read (classify -> four scans -> apply) instead of the
reference's chain of boolean-mask indexing, concatenations and per-tensor optimizer gathers; the output order
[survivors | duplicates | first split copies | second split copies], the thresholds and the split geometry are
the reference's.
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

    def _refine_config(self, state: GaussianTrainState, step: int, fused: bool) -> _lib.RefineConfig:
        rc = _lib.RefineConfig()
        rc.prune_opacity_thresh, rc.grow_grad2d = self.prune_opacity_thresh, self.grow_grad2d
        rc.grow_scale3d, rc.grow_scale2d = self.grow_scale3d, self.grow_scale2d
        rc.prune_scale3d, rc.prune_scale2d = self.prune_scale3d, self.prune_scale2d
        rc.scene_scale = float(state.scene_scale)
        rc.prune_too_big = int(step > self.reset_opacity_every)          # origin/strategy.py:178
        rc.refine_by_radii = int(step < self.refine_scale2d_stop_iter)    # origin/strategy.py:177
        rc.fused_activations = int(fused)
        return rc

    @torch.no_grad()
    def refine_tensors(self, model, moments: "dict[str, tuple[torch.Tensor, torch.Tensor]] | None",
                       state: GaussianTrainState, step: int, generator: "torch.Generator | None" = None,
                       normals: "torch.Tensor | None" = None):
        """Densify and prune.  ``model``: a Gaussian model container with raw (fused-activation) or activated
        parameters; ``moments``: field name -> (exp_avg, exp_avg_sq) shaped like the field, or None.
        Returns ``(new_model, new_moments, src_index, (n_keep, n_dup_kept, n_split_kept, n_split))``; nothing is
        modified in place.  ``normals`` ([2 * n_split, 3]) replaces the ``torch.randn`` draw of
        origin/strategy.py:286 (tests); ``generator`` seeds that draw (identical on every rank of a
        data-parallel job)."""
        import ctypes as C
        lib = _lib.load()
        n, dev = len(model), model.xyz.device
        assert model.color_sh_base is not None, "refinement is built for the split SH layout (color_sh_base + color_sh)"
        stream = torch.cuda.current_stream(dev).cuda_stream
        fused = bool(getattr(model, "has_fused_activations", False))
        rc = self._refine_config(state, step, fused)
        cols = torch.empty([4, n], dtype=torch.int32, device=dev)
        flags = torch.empty(n, dtype=torch.uint8, device=dev)
        mstruct = _model_struct(model)
        _lib.check(lib.d3gs_refine_classify(C.byref(mstruct), C.byref(rc), state.duv_ndc_length.data_ptr(),
                                            state.count.data_ptr(), state.max_radii.data_ptr(), cols.data_ptr(),
                                            flags.data_ptr(), stream), "d3gs_refine_classify")
        totals_dev = torch.zeros(4, dtype=torch.int64, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        ws = torch.empty(max(int(lib.d3gs_scan_workspace_bytes(n)), 16), dtype=torch.uint8, device=dev)
        for k in range(4):   # stream-ordered: the scans may share the workspace
            _lib.check(lib.d3gs_scan_tiles(cols[k].data_ptr(), cols[k].data_ptr(), n, totals_dev.data_ptr() + 8 * k,
                                           ws.data_ptr(), ws.numel(), status.data_ptr(), stream), "d3gs_scan_tiles")
        totals = [int(v) for v in totals_dev.tolist()] if n > 0 else [0, 0, 0, 0]
        if int(status.item()) != 0:
            raise RuntimeError("scan of the refinement columns gave up on a bounded wait")
        n_keep, n_dup, n_split_kept, n_split = totals
        n_out = n_keep + n_dup + 2 * n_split_kept
        if normals is None:
            normals = torch.randn(2 * n_split, 3, device=dev, generator=generator)
        assert normals.shape == (2 * n_split, 3) and normals.is_contiguous() and normals.dtype == torch.float32
        if getattr(model, "flat", None) is not None:
            new_model = type(model).create_flat(n_out, device=dev, cur_sh_degree=model.cur_sh_degree)
        else:
            new_model = type(model).zeros_like(model, num=n_out, not_param=True)
        new_model.act_applied = model.act_applied
        mom = None
        new_moments = None
        fields = ("xyz", "quaternion_xyzw", "scale", "opacity", "color_sh_base", "color_sh")
        if moments is not None:
            mom = _lib.RefineMoments()
            new_moments = {}
            for f, name in enumerate(fields):
                if name not in moments or getattr(model, name) is None:
                    continue
                m, v = moments[name]
                shape = (n_out,) + tuple(getattr(model, name).shape[1:])
                assert m.is_contiguous() and v.is_contiguous() and m.numel() == getattr(model, name).numel()
                nm, nv = torch.empty(shape, dtype=torch.float32, device=dev), torch.empty(shape, dtype=torch.float32, device=dev)
                mom.exp_avg_src[f], mom.exp_avg_sq_src[f] = m.data_ptr(), v.data_ptr()
                mom.exp_avg_dst[f], mom.exp_avg_sq_dst[f] = nm.data_ptr(), nv.data_ptr()
                new_moments[name] = (nm, nv)
        src_index = torch.empty(n_out, dtype=torch.int32, device=dev)
        dstruct = _model_struct(new_model)
        tot = (C.c_int64 * 4)(*totals)
        _lib.check(lib.d3gs_refine_apply(C.byref(mstruct), C.byref(dstruct), C.byref(rc),
                                         C.byref(mom) if mom is not None else None, cols.data_ptr(), flags.data_ptr(),
                                         normals.data_ptr() if n_split > 0 else None, tot, src_index.data_ptr(), stream),
                   "d3gs_refine_apply")
        return new_model, new_moments, src_index, (n_keep, n_dup, n_split_kept, n_split)

    @torch.no_grad()
    def refine_gs(self, model, optimizers, state: GaussianTrainState, step: int,
                  generator: "torch.Generator | None" = None):
        """origin/strategy.py:159-363 with the reference's signature: ``optimizers`` maps field names to
        single-tensor optimizers (``create_origin_3dgs_optimizers``).  The model, the optimizers' parameters and
        moments and the train state are replaced in place; the state is reset."""
        moments = {}
        for name, opt in optimizers.items():
            p = opt.param_groups[0]["params"][0]
            st = opt.state.get(p, {})
            if "exp_avg" in st:
                moments[name] = (st["exp_avg"].contiguous(), st["exp_avg_sq"].contiguous())
        new_model, new_moments, _, _ = self.refine_tensors(model, moments or None, state, step, generator)
        for name, t in new_model.get_all_tensor_fields().items():
            old = getattr(model, name)
            setattr(model, name, torch.nn.Parameter(t) if isinstance(old, torch.nn.Parameter) else t)
        if getattr(new_model, "flat", None) is not None:
            model.flat = new_model.flat
        for name, opt in optimizers.items():   # strategy.py:17-66: swap the parameter, keep "step", replace the moments
            p_old = opt.param_groups[0]["params"][0]
            st = opt.state.pop(p_old, {})
            p_new = getattr(model, name)
            opt.param_groups[0]["params"] = [p_new]
            if new_moments is not None and name in new_moments:
                st["exp_avg"], st["exp_avg_sq"] = new_moments[name]
            if st:
                opt.state[p_new] = st
        n_out = len(model)
        new_state = GaussianTrainState.create(n_out, state.scene_scale, device=model.xyz.device)
        state.duv_ndc_length, state.count, state.max_radii = new_state.duv_ndc_length, new_state.count, new_state.max_radii
        return model

    @torch.no_grad()
    def reset_opacity(self, model, optimizers=None):
        """origin/trainer.py:388-417: opacity <- logit(min(opacity_act, reset_opacity_thresh)) in place and the
        opacity optimizer's moments zeroed (reset_param_in_optim, strategy.py:181-202)."""
        lib = _lib.load()
        dev = model.opacity.device
        m = v = None
        if optimizers is not None and "opacity" in optimizers:
            opt = optimizers["opacity"]
            st = opt.state.get(opt.param_groups[0]["params"][0], {})
            m, v = st.get("exp_avg"), st.get("exp_avg_sq")
        _lib.check(lib.d3gs_reset_opacity(model.opacity.data_ptr(), len(model), float(self.reset_opacity_thresh),
                                          int(bool(getattr(model, "has_fused_activations", False))), _lib.ptr(m),
                                          _lib.ptr(v), torch.cuda.current_stream(dev).cuda_stream), "d3gs_reset_opacity")


def _model_struct(model) -> "_lib.Model":
    from .render import GaussianSplatOp
    return GaussianSplatOp._model_struct(model)
