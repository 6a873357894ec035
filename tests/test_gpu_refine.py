"""Densification / pruning / opacity reset against the numpy restatement of the reference's refine_gs
(d3sim/algos/d3gs/origin/strategy.py:159-363) and of its optimizer-state surgery (strategy.py:131-202).

Bit-exact: which Gaussians are duplicated, split and pruned, the order of the output rows, the copied
parameters and the gathered / zeroed Adam moments.  Within 1e-6 relative: the positions and log-scales of the
split children (a rotation-matrix product and a logarithm in float32)."""
import numpy as np
import pytest
import torch

import d3gs_research_b200 as d3
from d3gs_research_b200.strategy import GaussianStrategyOrigin, GaussianTrainState
from oracle import oracle as O

pytestmark = pytest.mark.gpu

NAMES = {"xyz": "xyz", "quat": "quaternion_xyzw", "scale": "scale", "opacity": "opacity", "sh_base": "color_sh_base",
         "sh_rest": "color_sh"}


def _scene(n, seed, dev):
    g = torch.Generator().manual_seed(seed)
    t = {"xyz": torch.randn(n, 3, generator=g) * 2, "quat": torch.randn(n, 4, generator=g),
         "scale": torch.randn(n, 3, generator=g) * 0.9 - 3.6, "opacity": torch.randn(n, generator=g) * 3.0 - 1.0,
         "sh_base": torch.randn(n, 3, generator=g), "sh_rest": torch.randn(n, 15, 3, generator=g) * 0.1}
    state = {"duv_ndc_length": torch.rand(n, generator=g) * 0.01, "count": torch.randint(0, 20, (n,), generator=g).float(),
             "max_radii": torch.rand(n, generator=g) * 0.2}
    moments = {k: (torch.randn(v.shape, generator=g), torch.rand(v.shape, generator=g)) for k, v in t.items()}
    model = d3.GaussianModelOriginFused.from_tensors(t["xyz"], t["quat"], t["scale"], t["opacity"], t["sh_base"],
                                                     t["sh_rest"], device=dev)
    return t, state, moments, model


@pytest.mark.parametrize("step,scale2d_stop", [(600, 0), (3500, 0), (700, 5000)])
def test_refine_matches_reference_policy(cuda_device, step, scale2d_stop):
    n = 20011
    t, state, moments, model = _scene(n, 7 + step, cuda_device)
    strat = GaussianStrategyOrigin(refine_scale2d_stop_iter=scale2d_stop)
    rc = O.RefineConfig(refine_scale2d_stop_iter=scale2d_stop)
    scene_scale = 3.0
    np_model = {k: v.numpy().copy() for k, v in t.items()}
    np_state = {k: v.numpy().copy() for k, v in state.items()}
    np_mom = {k: (m.numpy().copy(), v.numpy().copy()) for k, (m, v) in moments.items()}
    dup, split, _ = O.refine_masks(rc, np_model, np_state, scene_scale, step)
    n_split = int(split.sum())
    assert dup.sum() > 100 and n_split > 100
    normals = torch.randn(2 * n_split, 3, generator=torch.Generator().manual_seed(1))
    ref_model, ref_mom, ref_inds, ref_ndup, _ = O.refine_gs(rc, np_model, np_mom, np_state, scene_scale, step, normals.numpy())

    st = GaussianTrainState(duv_ndc_length=state["duv_ndc_length"].to(cuda_device), count=state["count"].to(cuda_device),
                            max_radii=state["max_radii"].to(cuda_device), scene_scale=scene_scale)
    gmom = {NAMES[k]: (m.to(cuda_device), v.to(cuda_device)) for k, (m, v) in moments.items()}
    new_model, new_mom, src_index, totals = strat.refine_tensors(model, gmom, st, step, normals=normals.to(cuda_device))
    torch.cuda.synchronize()
    assert totals[3] == n_split and len(new_model) == len(ref_inds)
    np.testing.assert_array_equal(src_index.cpu().numpy(), ref_inds)
    n_keep, n_dupk = totals[0], totals[1]
    for k, name in NAMES.items():
        got = getattr(new_model, name).cpu().numpy()
        if k in ("xyz", "scale"):   # split children are computed, everything before them is a copy
            np.testing.assert_array_equal(got[:n_keep + n_dupk], ref_model[k][:n_keep + n_dupk], err_msg=k)
            np.testing.assert_allclose(got[n_keep + n_dupk:], ref_model[k][n_keep + n_dupk:], rtol=2e-6, atol=2e-6, err_msg=k)
        else:
            np.testing.assert_array_equal(got, ref_model[k], err_msg=k)
        np.testing.assert_array_equal(new_mom[name][0].cpu().numpy(), ref_mom[k][0], err_msg=f"exp_avg {k}")
        np.testing.assert_array_equal(new_mom[name][1].cpu().numpy(), ref_mom[k][1], err_msg=f"exp_avg_sq {k}")
    assert float(new_mom["xyz"][0][n_keep:].abs().max()) == 0.0      # new Gaussians start with zero moments


def test_refine_gs_updates_model_optimizers_and_state(cuda_device):
    from d3gs_research_b200.tools import create_origin_3dgs_optimizers
    from d3gs_research_b200 import config_def
    n = 5003
    t, state, _, model = _scene(n, 3, cuda_device)
    model = model.to_parameter()
    optims, _ = create_origin_3dgs_optimizers(model, config_def.Optimizer(), 1, 1.0)
    for name, opt in optims.items():   # give every optimizer a state
        p = opt.param_groups[0]["params"][0]
        p.grad = torch.randn_like(p)
        opt.step()
    strat = GaussianStrategyOrigin()
    st = GaussianTrainState(duv_ndc_length=state["duv_ndc_length"].to(cuda_device), count=state["count"].to(cuda_device),
                            max_radii=state["max_radii"].to(cuda_device), scene_scale=3.0)
    strat.refine_gs(model, optims, st, 600, generator=torch.Generator(device=cuda_device).manual_seed(5))
    n_out = len(model)
    assert n_out != n and st.count.shape[0] == n_out and float(st.count.abs().sum()) == 0.0
    for name, opt in optims.items():
        p = opt.param_groups[0]["params"][0]
        assert p is getattr(model, name) and p.shape[0] == n_out
        assert opt.state[p]["exp_avg"].shape == p.shape and "step" in opt.state[p]
        p.grad = torch.randn_like(p)
        opt.step()                     # the optimizers keep working on the new tensors
    # the refined model renders
    op = d3.GaussianSplatOp(d3.GaussianSplatConfig())
    cam = d3.BasicPinholeCamera.from_params(np.eye(4, dtype=np.float32), 200.0, 200.0, 80.0, 56.0, 160, 112)
    model.act_applied = True
    out, _ = op.forward(model, cam, training=False)
    assert bool(torch.isfinite(out.color).all())


def test_reset_opacity(cuda_device):
    t, _, _, model = _scene(4099, 9, cuda_device)
    ref = O.reset_opacity(t["opacity"].numpy(), 0.01)
    GaussianStrategyOrigin().reset_opacity(model)
    np.testing.assert_array_equal(model.opacity.cpu().numpy(), ref)


def test_trainer_refine_between_steps(cuda_device):
    """Train, densify/prune, reset opacities, train on: the trainer's buffers follow the new Gaussian count."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from d3gs_research_b200.config_def import EarlyFilterAlgo
    from d3gs_research_b200.trainer import SplatTrainer
    from parity_utils import gpu_cameras, gpu_model, small_scene
    sc = small_scene(n=6001, width=176, height=128, sh_degree=3, seed=2)
    model = gpu_model(sc, cuda_device)
    tr = SplatTrainer(model, d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT), lambda_dssim=0.2,
                      batch_size=1)
    cams = gpu_cameras(sc, cuda_device)
    target = torch.rand(1, 3, 128, 176, generator=torch.Generator().manual_seed(4)).to(cuda_device)
    for _ in range(3):
        tr.step(cams, target)
    assert float(tr.state.count.sum()) > 0
    n0 = len(model)
    moved = tr.exp_avg.clone()
    strat = GaussianStrategyOrigin(grow_grad2d=float(torch.quantile((tr.state.duv_ndc_length / tr.state.count.clamp(min=1)), 0.7)))
    tr.state.scene_scale = 3.0
    totals = tr.refine(strat, step=600, generator=torch.Generator(device=cuda_device).manual_seed(0))
    n1 = len(model)
    assert n1 == totals[0] + totals[1] + 2 * totals[2] and n1 != n0 and totals[1] + totals[2] > 0
    assert tr.exp_avg.numel() == tr.flat_total and tr.state.count.shape[0] == n1 and model.flat.numel() >= 59 * n1
    # survivors keep their moments: the first n_keep rows of every field are gathered rows of the old buffer
    assert float(tr._field_views(tr.exp_avg)["xyz"][:totals[0]].abs().sum()) > 0
    assert float(tr._field_views(tr.exp_avg)["xyz"][totals[0]:].abs().sum()) == 0.0
    tr.reset_opacity(strat)
    from math import log
    assert float(model.opacity.max()) <= log(0.01 / 0.99) + 1e-4
    assert float(tr._field_views(tr.exp_avg)["opacity"].abs().sum()) == 0.0
    for _ in range(2):
        info = tr.step(cams, target)
    torch.cuda.synchronize()
    assert bool(torch.isfinite(model.flat).all()) and bool(torch.isfinite(info["out"].color).all())
    assert moved.numel() != tr.exp_avg.numel()
