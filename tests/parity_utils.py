"""Shared helpers of the parity tests: build the same seeded scene for the CPU oracle and the GPU library."""
from __future__ import annotations

import numpy as np
import torch

import d3gs_research_b200 as d3
from d3gs_research_b200 import scenes
from oracle import oracle as O


def small_scene(n=2000, width=160, height=112, sh_degree=3, seed=0, views=1, log_scale=("normal", -2.6, 0.6),
                pos=("uniform", 3.0), cam_radius=9.0, base="cfg1", sh_gain=4.0):
    b = scenes.CONFIGS[base]
    cfg = scenes.SceneConfig(**{**b.__dict__, "n": n, "width": width, "height": height, "sh_degree": sh_degree,
                                "log_scale": log_scale, "pos": pos, "cam_radius": cam_radius, "num_views": views,
                                "cam_layout": "sphere" if views > 1 else b.cam_layout})
    sc = scenes.make_scene(cfg, seed=seed)
    if sh_degree > 0:
        sc["sh_rest"] = (sc["sh_rest"] * sh_gain).contiguous()
    return sc


def oracle_scene(sc) -> O.Scene:
    return O.Scene(*(sc[k].numpy().copy() for k in ("xyz", "quat", "scale", "opacity", "sh_base", "sh_rest")),
                   cams=np.ascontiguousarray(sc["cams"]).copy())


def oracle_cfg(sc, op_cfg: "d3.GaussianSplatConfig", training=True) -> O.OpConfig:
    c = sc["cfg"]
    return O.OpConfig(width=c.width, height=c.height, sh_degree=c.sh_degree, early_filter=int(op_cfg.early_filter_algo),
                      training=training, clamp_mask_reference_order=op_cfg.clamp_mask_reference_order,
                      near=op_cfg.near, far=op_cfg.far, scale_global=op_cfg.scale_global,
                      key_shift=18 if op_cfg.enable_32bit_sort else 32, depth_prec=op_cfg.depth_32bit_prec,
                      anti_aliasing=op_cfg.enable_anti_aliasing, inv_depth=op_cfg.render_inv_depth)


def gpu_model(sc, device, flat=True, requires_grad=False):
    m = d3.GaussianModelOriginFused.from_tensors(sc["xyz"], sc["quat"], sc["scale"], sc["opacity"], sc["sh_base"],
                                                 sc["sh_rest"], device=device, cur_sh_degree=sc["cfg"].sh_degree,
                                                 flat=flat)
    if requires_grad:
        m.set_requires_grad(True)
    return m


def gpu_cameras(sc, device):
    c = sc["cfg"]
    fx, fy, cx, cy = sc["intrinsics"]
    cams = [d3.BasicPinholeCamera.from_params(m, fx, fy, cx, cy, c.width, c.height) for m in sc["cam2worlds"]]
    if len(cams) == 1:
        return cams[0]
    from d3gs_research_b200.render import CameraBundle
    return CameraBundle.from_pinhole_cams(cams, device=device)


def rel_inf(a, b, floor=1e-12):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / (np.abs(b).max() + floor))


def assert_close(a, b, tol, name, floor_frac=1e-3):
    """|a-b| <= tol * max(|b|, floor) elementwise with floor = floor_frac * max|b|, plus the inf-norm ratio."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    assert a.shape == b.shape, f"{name}: shape {a.shape} vs {b.shape}"
    scale = np.abs(b).max()
    if scale == 0:
        assert np.abs(a).max() == 0, f"{name}: expected all zeros"
        return
    err = np.abs(a - b)
    bound = tol * np.maximum(np.abs(b), floor_frac * scale)
    bad = err > bound
    assert not bad.any(), (f"{name}: {int(bad.sum())}/{bad.size} elements off, max err {err.max():.3e} "
                           f"(scale {scale:.3e}, rel-inf {err.max() / scale:.3e}, tol {tol})")


def assert_bit_equal(got, ref, name):
    """Integer / bit-pattern equality with the mismatch count in the message (the target is 0)."""
    g = got.cpu().numpy() if hasattr(got, "cpu") else np.asarray(got)
    r = np.asarray(ref)
    assert g.shape == r.shape, f"{name}: shape {g.shape} vs {r.shape}"
    if g.dtype != r.dtype:
        assert g.dtype.itemsize == r.dtype.itemsize, f"{name}: dtype {g.dtype} vs {r.dtype}"
        g = g.view(r.dtype)
    bad = int(np.count_nonzero(g != r))
    assert bad == 0, f"{name}: {bad} of {g.size} elements differ from the oracle (first at {np.flatnonzero(g != r)[:5]})"


def assert_update_close(dp, dp_ref, g_ref, lr, name, tol=1e-3, first_step=True, resolved_frac=None,
                        max_unresolved=0.02, p_before=None, ulps=1.0):
    """Adam update ``p_after - p_before`` against the oracle's, relative to the update's own scale.

    Adam normalises the gradient (``lr * m_hat / (sqrt(v_hat) + eps)``; the very first step is ``lr * sign(g)``),
    so an element whose gradient lies below the resolution of the fp32 sums -- where the gradient tolerance itself
    admits a sign change -- can legitimately move by a different amount.  Elements whose oracle gradient exceeds
    ``resolved_frac * max|g|`` must match within ``tol * lr`` (the scale of an Adam update); the others may differ, but
    must stay within the step bound (first step: ``|update| <= lr``) and must be few.  ``resolved_frac`` defaults
    to 1e-5 for a first step (only the gradient's sign matters there) and to 1e-3 afterwards (the floor below
    which the gradient comparison itself is absolute, not relative).  ``p_before``: the parameter is stored in
    fp32, so its update is quantised by the spacing of the parameter itself (one ulp of a position near 16 is
    1.2 % of the position learning rate); ``ulps`` spacings of ``p_before`` are added to the bound."""
    if resolved_frac is None:
        resolved_frac = 1e-5 if first_step else 1e-3
    dp = np.asarray(dp, np.float64)
    dp_ref = np.asarray(dp_ref, np.float64)
    g = np.abs(np.asarray(g_ref, np.float64))
    assert dp.shape == dp_ref.shape == g.shape, f"{name}: shapes {dp.shape} {dp_ref.shape} {g.shape}"
    assert np.abs(dp_ref).max() > 0.5 * lr, f"{name}: the oracle's update is empty"
    assert np.abs(dp).max() > 0.5 * lr, f"{name}: the parameters did not move"
    resolved = g > resolved_frac * g.max()
    err = np.abs(dp - dp_ref)
    bound = np.full(dp.shape, tol * lr)       # relative to the update's own scale: Adam moves an element by about lr
    if p_before is not None:
        bound = bound + ulps * np.spacing(np.abs(np.asarray(p_before, np.float32))).astype(np.float64)
    bad = resolved & (err > bound)
    assert not bad.any(), (f"{name}: {int(bad.sum())}/{int(resolved.sum())} resolved elements off, max err "
                           f"{err[resolved].max():.3e} against lr {lr:.3e}")
    loose = ~resolved
    if first_step:
        step_bound = lr * (1.0 + 1e-3)
        if p_before is not None:     # the stored parameter rounds the step to its own spacing
            step_bound = step_bound + np.spacing(np.abs(np.asarray(p_before, np.float32))).astype(np.float64)[loose]
        assert (np.abs(dp[loose]) <= step_bound).all(), f"{name}: an update exceeds the first-step bound lr"
    differing = loose & (err > bound)
    moved = max(int(np.count_nonzero(dp_ref)), 1)
    assert differing.sum() <= max_unresolved * moved, \
        f"{name}: {int(differing.sum())} unresolved elements differ ({differing.sum() / moved:.2%} of the moved ones)"
