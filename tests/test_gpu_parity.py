"""GPU parity: the sm_100a library (through its C ABI / the operator API) against the CPU oracle.

Bars (from the task's north star): bit-exact for tile-touch counts, sort keys/values, tile ranges and
n_contrib; <= 1e-4 relative for images; <= 1e-3 relative for gradients, Adam updates and statistics.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import d3gs_research_b200 as d3
from d3gs_research_b200 import _lib
from d3gs_research_b200.config_def import EarlyFilterAlgo
from d3gs_research_b200.render import GaussianSplatGradients
from oracle import oracle as O
from parity_utils import assert_close, assert_update_close, gpu_cameras, gpu_model, oracle_cfg, oracle_scene, small_scene

pytestmark = pytest.mark.gpu

IMG_TOL = 1e-4
GRAD_TOL = 1e-3


def _run_forward(sc, device, early_filter, training=True, binning="sort", **cfg_kw):
    op_cfg = d3.GaussianSplatConfig(early_filter_algo=early_filter, **cfg_kw)
    op = d3.GaussianSplatOp(op_cfg)
    op.binning = binning
    op.debug_capture = True
    model = gpu_model(sc, device)
    model.act_applied = True
    cams = gpu_cameras(sc, device)
    out, ctx = op.forward(model, cams, training=training)
    torch.cuda.synchronize()
    ocfg = oracle_cfg(sc, op_cfg, training)
    osc = oracle_scene(sc)
    ref = O.forward(ocfg, osc)
    return op, model, cams, out, ctx, ocfg, osc, ref


@pytest.mark.parametrize("early_filter", [EarlyFilterAlgo.NONE, EarlyFilterAlgo.AABB, EarlyFilterAlgo.ELLIPSE,
                                          EarlyFilterAlgo.OBB, EarlyFilterAlgo.OBB_DFVT])
@pytest.mark.parametrize("sh_degree,views", [(3, 1), (0, 1), (2, 3)])
@pytest.mark.parametrize("binning", ["sort", "bucket"])
def test_binning_bit_exact(cuda_device, early_filter, sh_degree, views, binning):
    """Both ways of building the sorted per-tile lists -- key duplication + radix sort + range extraction like the
    reference, and per-tile buckets sorted in shared memory -- against the oracle, bit for bit."""
    sc = small_scene(n=6000, width=200, height=136, sh_degree=sh_degree, seed=3 + sh_degree, views=views)
    op, model, cams, out, ctx, ocfg, osc, ref = _run_forward(sc, cuda_device, early_filter, binning=binning)
    assert op.last_binning == binning
    dbg = {k: v.cpu().numpy() for k, v in op.debug.items()}
    # K1: integer outputs bit-exact, float context bit-exact on visible Gaussians
    np.testing.assert_array_equal(dbg["tiles_touched"], ref.prep["tiles_touched"])
    np.testing.assert_array_equal(ctx.radii.cpu().numpy(), ref.prep["radii"])
    vis = ref.prep["radii"] > 0
    assert vis.sum() > 100
    for name, got in (("depths", ctx.depths), ("uvs", ctx.uvs), ("conic_opacity", ctx.conic_opacity),
                      ("cov2d", ctx.cov2d_vecs), ("rgb", ctx.rgb_gaussian)):
        g = got.cpu().numpy()[vis]
        r = ref.prep[name][vis]
        np.testing.assert_array_equal(g.view(np.uint32), r.view(np.uint32), err_msg=name)
    np.testing.assert_array_equal(ctx.sh_to_rgb_ne_0.cpu().numpy()[vis], ref.prep["ne0"][vis])
    # K2/K3/K4/K5
    assert op.last_num_rendered == ref.num_rendered
    if binning == "sort":     # the bucket path has no scan over the Gaussians and no unsorted key list
        np.testing.assert_array_equal(dbg["scan"], ref.scan)
        np.testing.assert_array_equal(dbg["keys"].view(np.uint64), ref.keys)
        np.testing.assert_array_equal(dbg["values"], ref.vals)
    np.testing.assert_array_equal(dbg["sorted_keys"].view(np.uint64), ref.sorted_keys)
    np.testing.assert_array_equal(dbg["sorted_values"], ref.sorted_ids)
    np.testing.assert_array_equal(ctx.workload_ranges.cpu().numpy(), ref.ranges)
    # K6
    np.testing.assert_array_equal(out.n_contrib.cpu().numpy(), ref.n_contrib)
    assert_close(out.color.cpu().numpy(), ref.color, IMG_TOL, "color")
    assert_close(out.T.cpu().numpy(), ref.T, IMG_TOL, "T")


@pytest.mark.parametrize("views", [1, 3])
def test_binning_bit_exact_32bit_keys(cuda_device, views):
    """enable_32bit_sort (render.py:227-228, 737, 767-770, 851-854): key = tile << 18 | 18-bit quantised depth,
    sorted on 32 bits.  Keys, sorted lists, ranges and contributor counts must equal the oracle's bit for bit;
    the image follows (a different depth order than with 64-bit keys, the same one as the oracle's)."""
    sc = small_scene(n=6000, width=200, height=136, sh_degree=2, seed=17, views=views)
    op, model, cams, out, ctx, ocfg, osc, ref = _run_forward(sc, cuda_device, EarlyFilterAlgo.OBB_DFVT,
                                                             enable_32bit_sort=True)
    assert ocfg.key_shift == 18
    dbg = {k: v.cpu().numpy() for k, v in op.debug.items()}
    assert int(dbg["keys"].max()) < 2 ** 32 and op.last_num_rendered == ref.num_rendered
    np.testing.assert_array_equal(dbg["keys"].view(np.uint64), ref.keys)
    np.testing.assert_array_equal(dbg["values"], ref.vals)
    np.testing.assert_array_equal(dbg["sorted_keys"].view(np.uint64), ref.sorted_keys)
    np.testing.assert_array_equal(dbg["sorted_values"], ref.sorted_ids)
    np.testing.assert_array_equal(ctx.workload_ranges.cpu().numpy(), ref.ranges)
    np.testing.assert_array_equal(out.n_contrib.cpu().numpy(), ref.n_contrib)
    assert_close(out.color.cpu().numpy(), ref.color, IMG_TOL, "color")


@pytest.mark.parametrize("early_filter", [EarlyFilterAlgo.NONE, EarlyFilterAlgo.AABB, EarlyFilterAlgo.ELLIPSE,
                                          EarlyFilterAlgo.OBB_DFVT])
@pytest.mark.parametrize("binning", ["sort", "bucket"])
def test_binning_bit_exact_large_gaussians(cuda_device, early_filter, binning):
    """Gaussians that cover hundreds of tiles take the warp-cooperative paths of the tile count and of the key
    emission; the unsorted key list must still come out in the reference's per-Gaussian row-major order."""
    sc = small_scene(n=500, width=400, height=304, sh_degree=1, seed=11, log_scale=("normal", -0.9, 0.8))
    op, model, cams, out, ctx, ocfg, osc, ref = _run_forward(sc, cuda_device, early_filter, binning=binning)
    assert op.last_binning == binning
    dbg = {k: v.cpu().numpy() for k, v in op.debug.items()}
    assert ref.prep["tiles_touched"].max() > 200, "the scene has no screen-filling Gaussian"
    np.testing.assert_array_equal(dbg["tiles_touched"], ref.prep["tiles_touched"])
    if binning == "sort":
        np.testing.assert_array_equal(dbg["scan"], ref.scan)
        np.testing.assert_array_equal(dbg["keys"].view(np.uint64), ref.keys)
        np.testing.assert_array_equal(dbg["values"], ref.vals)
    np.testing.assert_array_equal(dbg["sorted_keys"].view(np.uint64), ref.sorted_keys)
    np.testing.assert_array_equal(dbg["sorted_values"], ref.sorted_ids)
    np.testing.assert_array_equal(ctx.workload_ranges.cpu().numpy(), ref.ranges)
    np.testing.assert_array_equal(out.n_contrib.cpu().numpy(), ref.n_contrib)


def test_forward_inference_background(cuda_device):
    sc = small_scene(n=3000, width=96, height=80, sh_degree=1, seed=11)
    op_cfg = d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.NONE, bg_color=np.array([0.2, 0.5, 0.9], np.float32),
                                    scale_global=0.8)
    op = d3.GaussianSplatOp(op_cfg)
    model = gpu_model(sc, cuda_device)
    out = d3.rasterize_gaussians(model, gpu_cameras(sc, cuda_device), op, training=False)
    ocfg = oracle_cfg(sc, op_cfg, training=False)
    osc = oracle_scene(sc)
    ref = O.forward(ocfg, osc)
    color, T, nc = O.raster_fwd(ocfg, 1, ref.ranges, ref.sorted_ids, ref.prep, bg=op_cfg.bg_color)
    np.testing.assert_array_equal(out.n_contrib.cpu().numpy(), nc)
    assert_close(out.color.cpu().numpy(), color, IMG_TOL, "color+bg")


@pytest.mark.parametrize("early_filter,views,ref_order", [(EarlyFilterAlgo.NONE, 1, True), (EarlyFilterAlgo.OBB_DFVT, 1, True),
                                                           (EarlyFilterAlgo.OBB, 3, True), (EarlyFilterAlgo.NONE, 2, False)])
def test_backward_gradients(cuda_device, early_filter, views, ref_order):
    sc = small_scene(n=5000, width=176, height=120, sh_degree=3, seed=21, views=views)
    op_cfg = d3.GaussianSplatConfig(early_filter_algo=early_filter, clamp_mask_reference_order=ref_order)
    op = d3.GaussianSplatOp(op_cfg)
    model = gpu_model(sc, cuda_device)
    model.act_applied = True
    cams = gpu_cameras(sc, cuda_device)
    out, ctx = op.forward(model, cams, training=True)
    g = torch.Generator().manual_seed(7)
    c = sc["cfg"]
    drgb = torch.randn(views, c.height, c.width, 3, generator=g)
    dT = torch.randn(views, c.height, c.width, generator=g)
    grad = GaussianSplatGradients(drgb=drgb.to(cuda_device), dT=dT.to(cuda_device))
    gm, duv, _ = op.backward(model, cams, ctx, out, grad, return_uv_grad=True)
    torch.cuda.synchronize()
    ocfg = oracle_cfg(sc, op_cfg)
    osc = oracle_scene(sc)
    ref = O.forward(ocfg, osc)
    O.backward(ocfg, osc, ref, drgb.numpy(), dT.numpy())
    assert_close(duv.reshape(-1, 2).cpu().numpy(), ref.raster_grads["duv"], GRAD_TOL, "duv")
    for name, ours in (("xyz", gm.xyz), ("quat", gm.quaternion_xyzw), ("scale", gm.scale), ("opacity", gm.opacity),
                       ("sh_base", gm.color_sh_base), ("sh_rest", gm.color_sh)):
        assert_close(ours.cpu().numpy(), ref.grads[name], GRAD_TOL, f"grad {name}")


@pytest.mark.parametrize("early_filter,views", [(EarlyFilterAlgo.OBB_DFVT, 1), (EarlyFilterAlgo.NONE, 2)])
def test_anti_aliasing_parity(cuda_device, early_filter, views):
    """enable_anti_aliasing (render.py:391-406, 449-462, 3295-3309; gs3d.py:592-683): the compensated opacity and
    the un-guarded conic must equal the oracle's bit for bit (they decide tile counts and contributors), the
    gradients, including the compensation's path into the covariance, within the gradient tolerance."""
    sc = small_scene(n=5000, width=176, height=120, sh_degree=3, seed=23, views=views)
    op, model, cams, out, ctx, ocfg, osc, ref = _run_forward(sc, cuda_device, early_filter, enable_anti_aliasing=True)
    assert ocfg.anti_aliasing
    base = O.forward(oracle_cfg(sc, d3.GaussianSplatConfig(early_filter_algo=early_filter)), osc)
    assert not np.array_equal(base.prep["conic_opacity"], ref.prep["conic_opacity"])   # the option changes the result
    dbg = {k: v.cpu().numpy() for k, v in op.debug.items()}
    np.testing.assert_array_equal(dbg["tiles_touched"], ref.prep["tiles_touched"])
    np.testing.assert_array_equal(ctx.radii.cpu().numpy(), ref.prep["radii"])
    vis = ref.prep["radii"] > 0
    np.testing.assert_array_equal(ctx.conic_opacity.cpu().numpy()[vis].view(np.uint32),
                                  ref.prep["conic_opacity"][vis].view(np.uint32))
    np.testing.assert_array_equal(dbg["sorted_values"], ref.sorted_ids)
    np.testing.assert_array_equal(out.n_contrib.cpu().numpy(), ref.n_contrib)
    assert_close(out.color.cpu().numpy(), ref.color, IMG_TOL, "color")
    g = torch.Generator().manual_seed(7)
    c = sc["cfg"]
    drgb = torch.randn(views, c.height, c.width, 3, generator=g)
    dT = torch.randn(views, c.height, c.width, generator=g)
    gm, duv, _ = op.backward(model, cams, ctx, out, GaussianSplatGradients(drgb=drgb.to(cuda_device), dT=dT.to(cuda_device)),
                             return_uv_grad=True)
    torch.cuda.synchronize()
    O.backward(ocfg, osc, ref, drgb.numpy(), dT.numpy())
    for name, ours in (("xyz", gm.xyz), ("quat", gm.quaternion_xyzw), ("scale", gm.scale), ("opacity", gm.opacity),
                       ("sh_base", gm.color_sh_base), ("sh_rest", gm.color_sh)):
        assert_close(ours.cpu().numpy(), ref.grads[name], GRAD_TOL, f"grad {name}")


@pytest.mark.parametrize("inv,gather,views", [(False, True, 2), (True, True, 1), (False, False, 1)])
def test_render_depth_parity(cuda_device, inv, gather, views):
    """render_depth / render_inv_depth (render.py:582, 1824, 1948-1967, 2244-2255, 3053-3057): the blended depth
    value in training, its normalised form at inference, and the gradient a depth loss sends to the parameters.
    With render_inv_depth the depth array holds 1/z and, as in the reference, the sort keys are built from it."""
    sc = small_scene(n=4000, width=160, height=104, sh_degree=2, seed=29, views=views)
    op_cfg = d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT, render_depth=True, render_inv_depth=inv)
    op = d3.GaussianSplatOp(op_cfg)
    op.gather_records = gather
    op.debug_capture = True
    model = gpu_model(sc, cuda_device)
    model.act_applied = True
    cams = gpu_cameras(sc, cuda_device)
    out, ctx = op.forward(model, cams, training=True)
    ocfg = oracle_cfg(sc, op_cfg)
    osc = oracle_scene(sc)
    ref = O.forward(ocfg, osc, render_depth=True)
    np.testing.assert_array_equal(op.debug["sorted_values"].cpu().numpy(), ref.sorted_ids)
    np.testing.assert_array_equal(out.n_contrib.cpu().numpy(), ref.n_contrib)
    assert_close(out.depth.cpu().numpy(), ref.depth, IMG_TOL, "depth")
    assert_close(out.color.cpu().numpy(), ref.color, IMG_TOL, "color")
    # inference: depth_accum / (1e-10 + 1 - T)
    out_inf, _ = op.forward(model, cams, training=False)
    ref_inf = O.forward(oracle_cfg(sc, op_cfg, training=False), osc, render_depth=True)
    assert_close(out_inf.depth.cpu().numpy(), ref_inf.depth, 5e-4, "normalised depth")
    g = torch.Generator().manual_seed(13)
    c = sc["cfg"]
    drgb = torch.randn(views, c.height, c.width, 3, generator=g)
    ddepth = torch.randn(views, c.height, c.width, generator=g)
    gm, duv, _ = op.backward(model, cams, ctx, out,
                             GaussianSplatGradients(drgb=drgb.to(cuda_device), dT=None, ddepth=ddepth.to(cuda_device)),
                             return_uv_grad=True)
    torch.cuda.synchronize()
    O.backward(ocfg, osc, ref, drgb.numpy(), None, ddepth.numpy())
    assert_close(duv.reshape(-1, 2).cpu().numpy(), ref.raster_grads["duv"], GRAD_TOL, "duv")
    for name, ours in (("xyz", gm.xyz), ("quat", gm.quaternion_xyzw), ("scale", gm.scale), ("opacity", gm.opacity),
                       ("sh_base", gm.color_sh_base), ("sh_rest", gm.color_sh)):
        assert_close(ours.cpu().numpy(), ref.grads[name], GRAD_TOL, f"grad {name}")


@pytest.mark.parametrize("rgba", [False, True])
def test_disable_builtin_rgb(cuda_device, rgba):
    """disable_builtin_rgb (config_def.py:116-132, render.py:667): the colour output has no channels (or the alpha
    alone) and the custom features carry the appearance; the SH coefficients receive no gradient."""
    sc = small_scene(n=2000, width=96, height=64, sh_degree=1, seed=37)
    op_cfg = d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT, disable_builtin_rgb=True, render_rgba=rgba)
    assert op_cfg.num_channels == (1 if rgba else 0)
    op = d3.GaussianSplatOp(op_cfg)
    model = gpu_model(sc, cuda_device)
    model.act_applied = True
    cams = gpu_cameras(sc, cuda_device)
    g = torch.Generator().manual_seed(19)
    feat = torch.randn(2000, 3, generator=g)
    out, ctx = op.forward(model, cams, training=True, custom_features=feat.to(cuda_device))
    assert tuple(out.color.shape) == (1, 64, 96, 1 if rgba else 0)
    ocfg = oracle_cfg(sc, op_cfg)
    osc = oracle_scene(sc)
    ref = O.forward(ocfg, osc, custom_features=feat.numpy())
    if rgba:
        assert_close(out.color[..., 0].cpu().numpy(), 1.0 - ref.T, IMG_TOL, "alpha")
    assert_close(out.custom_features.cpu().numpy(), ref.custom_image, IMG_TOL, "custom features")
    dcol = torch.randn(out.color.shape, generator=g)
    dfi = torch.randn(1, 64, 96, 3, generator=g)
    gm, _, dfeat = op.backward(model, cams, ctx, out, GaussianSplatGradients(
        drgb=dcol.to(cuda_device), dT=None, dcustom_features=dfi.to(cuda_device)))
    torch.cuda.synchronize()
    O.backward(ocfg, osc, ref, np.zeros((1, 64, 96, 3), np.float32), -dcol[..., 0].numpy() if rgba else None, None, dfi.numpy())
    assert float(gm.color_sh.abs().max()) == 0.0 and float(gm.color_sh_base.abs().max()) == 0.0
    assert_close(dfeat.cpu().numpy(), ref.raster_grads["dcustom"], GRAD_TOL, "dcustom_features")
    for name, ours in (("xyz", gm.xyz), ("opacity", gm.opacity)):
        assert_close(ours.cpu().numpy(), ref.grads[name], GRAD_TOL, f"grad {name}")


@pytest.mark.parametrize("nfeat,depth,views", [(4, False, 1), (3, True, 2), (1, False, 1)])
def test_custom_features_parity(cuda_device, nfeat, depth, views):
    """custom_features [B*N,F] -> out.custom_features [B,H,W,F] (render.py:241-245, 1920-1923, 2268-2270) and the
    gradients of a loss on that image: dcustom_features per Gaussian and the share that reaches the Gaussians'
    parameters through the blend weights (1952-1971); through the operator and through rasterize_gaussians."""
    sc = small_scene(n=3000, width=128, height=88, sh_degree=1, seed=31, views=views)
    op_cfg = d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT, render_depth=depth)
    op = d3.GaussianSplatOp(op_cfg)
    model = gpu_model(sc, cuda_device)
    model.act_applied = True
    cams = gpu_cameras(sc, cuda_device)
    g = torch.Generator().manual_seed(17)
    c = sc["cfg"]
    feat = torch.randn(views * 3000, nfeat, generator=g)
    out, ctx = op.forward(model, cams, training=True, custom_features=feat.to(cuda_device))
    assert tuple(out.custom_features.shape) == (views, c.height, c.width, nfeat)
    ocfg = oracle_cfg(sc, op_cfg)
    osc = oracle_scene(sc)
    ref = O.forward(ocfg, osc, render_depth=depth, custom_features=feat.numpy())
    assert_close(out.custom_features.cpu().numpy(), ref.custom_image, IMG_TOL, "custom features")
    drgb = torch.randn(views, c.height, c.width, 3, generator=g)
    dfi = torch.randn(views, c.height, c.width, nfeat, generator=g)
    dd = torch.randn(views, c.height, c.width, generator=g) if depth else None
    grads = GaussianSplatGradients(drgb=drgb.to(cuda_device), dT=None, ddepth=None if dd is None else dd.to(cuda_device),
                                   dcustom_features=dfi.to(cuda_device))
    gm, duv, dfeat = op.backward(model, cams, ctx, out, grads, return_uv_grad=True)
    torch.cuda.synchronize()
    O.backward(ocfg, osc, ref, drgb.numpy(), None, None if dd is None else dd.numpy(), dfi.numpy())
    assert_close(dfeat.cpu().numpy(), ref.raster_grads["dcustom"], GRAD_TOL, "dcustom_features")
    assert_close(duv.reshape(-1, 2).cpu().numpy(), ref.raster_grads["duv"], GRAD_TOL, "duv")
    for name, ours in (("xyz", gm.xyz), ("scale", gm.scale), ("opacity", gm.opacity), ("sh_base", gm.color_sh_base)):
        assert_close(ours.cpu().numpy(), ref.grads[name], GRAD_TOL, f"grad {name}")
    if views == 1 and not depth:   # the autograd entry point carries the features and their gradient
        m2 = gpu_model(sc, cuda_device, requires_grad=True)
        f2 = feat.to(cuda_device).requires_grad_(True)
        o2 = d3.rasterize_gaussians(m2, cams, d3.GaussianSplatOp(op_cfg), training=True, custom_features=f2)
        ((o2.color * drgb.to(cuda_device)).sum() + (o2.custom_features * dfi.to(cuda_device)).sum()).backward()
        assert_close(f2.grad.cpu().numpy(), ref.raster_grads["dcustom"], GRAD_TOL, "autograd dcustom_features")


@pytest.mark.parametrize("width,height,views", [(177, 121, 1), (64, 33, 2)])
def test_record_staging_modes_agree(cuda_device, width, height, views):
    """The raster kernels stage their records either by gathering from the per-Gaussian table the preprocess
    writes (default) or by streaming per-pair records written by d3gs_pack_splats.  Both must give the same
    image, transmittance and contributor counts bit for bit (odd image sizes: the second pixel of a lane
    falls outside), the oracle's contributor counts, and the same gradients up to the order of the float atomics."""
    sc = small_scene(n=4000, width=width, height=height, sh_degree=3, seed=33, views=views)
    op_cfg = d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT)
    g = torch.Generator().manual_seed(9)
    drgb = torch.randn(views, height, width, 3, generator=g).to(cuda_device)
    res = {}
    for gather in (True, False):
        op = d3.GaussianSplatOp(op_cfg)
        op.gather_records = gather
        model = gpu_model(sc, cuda_device)
        model.act_applied = True
        cams = gpu_cameras(sc, cuda_device)
        out, ctx = op.forward(model, cams, training=True)
        assert ctx.records_by_id == gather
        gm, duv, _ = op.backward(model, cams, ctx, out, GaussianSplatGradients(drgb=drgb, dT=None), return_uv_grad=True)
        torch.cuda.synchronize()
        res[gather] = (out.color.clone(), out.T.clone(), out.n_contrib.clone(), duv.clone(), gm.xyz.clone(),
                       gm.color_sh.clone())
    for k in range(3):
        assert torch.equal(res[True][k], res[False][k])
    for k, name in ((3, "duv"), (4, "xyz"), (5, "sh_rest")):
        assert_close(res[True][k].cpu().numpy(), res[False][k].cpu().numpy(), GRAD_TOL, name)
    ref = O.forward(oracle_cfg(sc, op_cfg), oracle_scene(sc))
    np.testing.assert_array_equal(res[True][2].cpu().numpy(), ref.n_contrib)


@pytest.mark.parametrize("nchw,rgba,training", [(True, False, True), (False, True, True), (True, True, True),
                                                  (True, True, False)])
def test_output_formats_nchw_rgba(cuda_device, nchw, rgba, training):
    """use_nchw / render_rgba (render.py:696-705, 1623-1668, 2222-2300): the alpha channel is the blended
    constant 1, sum of alpha_i T_i = 1 - T; its gradient reaches the splats like a colour channel's.  The
    PER_GAUSSIAN backward choice of the reference gives the same gradients as DEFAULT and is accepted."""
    from d3gs_research_b200.config_def import RasterizeBackwardAlgo
    views = 2
    sc = small_scene(n=3000, width=96, height=72, sh_degree=3, seed=11, views=views)
    op_cfg = d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT, use_nchw=nchw, render_rgba=rgba,
                                    rasterize_backward_algo=RasterizeBackwardAlgo.PER_GAUSSIAN)
    op = d3.GaussianSplatOp(op_cfg)
    assert op.is_nchw == nchw and op.is_rgba == rgba
    model = gpu_model(sc, cuda_device)
    model.act_applied = True
    cams = gpu_cameras(sc, cuda_device)
    out, ctx = op.forward(model, cams, training=training)
    ch = 4 if rgba else 3
    assert tuple(out.color.shape) == ((views, ch, 72, 96) if nchw else (views, 72, 96, ch))
    ocfg = oracle_cfg(sc, op_cfg, training=training)
    osc = oracle_scene(sc)
    ref = O.forward(ocfg, osc)
    if training:
        ref_color, ref_T = ref.color, ref.T
    else:
        ref_color, ref_T, _ = O.raster_fwd(ocfg, views, ref.ranges, ref.sorted_ids, ref.prep, bg=op_cfg.bg_color)
    expect = np.concatenate([ref_color, 1.0 - ref_T[..., None]], axis=-1) if rgba else ref_color
    if nchw:
        expect = np.ascontiguousarray(expect.transpose(0, 3, 1, 2))
    assert_close(out.color.cpu().numpy(), expect, IMG_TOL, "formatted colour")
    if not training:
        assert ctx is None
        return
    g = torch.Generator().manual_seed(3)
    dcol = torch.randn(out.color.shape, generator=g)
    dT = torch.randn(views, 72, 96, generator=g)
    gm, duv, _ = op.backward(model, cams, ctx, out, GaussianSplatGradients(drgb=dcol.to(cuda_device), dT=dT.to(cuda_device)),
                             return_uv_grad=True)
    torch.cuda.synchronize()
    d = dcol.permute(0, 2, 3, 1) if nchw else dcol
    dT_ref = dT - d[..., 3] if rgba else dT
    O.backward(ocfg, osc, ref, d[..., :3].contiguous().numpy(), dT_ref.contiguous().numpy())
    assert_close(duv.reshape(-1, 2).cpu().numpy(), ref.raster_grads["duv"], GRAD_TOL, "duv")
    for name, ours in (("xyz", gm.xyz), ("opacity", gm.opacity), ("sh_rest", gm.color_sh)):
        assert_close(ours.cpu().numpy(), ref.grads[name], GRAD_TOL, f"grad {name}")


def test_autograd_api_and_unsplit_nonflat_models(cuda_device):
    """rasterize_gaussians + loss.backward() through the public API; non-flat tensors."""
    sc = small_scene(n=3000, width=128, height=96, sh_degree=2, seed=5)
    op_cfg = d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT)
    op = d3.GaussianSplatOp(op_cfg)
    model = gpu_model(sc, cuda_device, flat=False).to_parameter()
    cams = gpu_cameras(sc, cuda_device)
    holder = torch.empty(1, len(model), 2, device=cuda_device, requires_grad=True)
    out = d3.rasterize_gaussians(model, cams, op, training=True, uv_grad_holder=holder)
    g = torch.Generator().manual_seed(9)
    w = torch.randn(out.color.shape, generator=g).to(cuda_device)
    (out.color * w).sum().backward()
    ocfg = oracle_cfg(sc, op_cfg)
    osc = oracle_scene(sc)
    ref = O.forward(ocfg, osc)
    O.backward(ocfg, osc, ref, w.cpu().numpy())
    assert_close(model.xyz.grad.cpu().numpy(), ref.grads["xyz"], GRAD_TOL, "xyz.grad")
    assert_close(model.color_sh.grad.cpu().numpy(), ref.grads["sh_rest"], GRAD_TOL, "color_sh.grad")
    assert_close(model.opacity.grad.cpu().numpy(), ref.grads["opacity"], GRAD_TOL, "opacity.grad")
    assert_close(holder.grad.reshape(-1, 2).cpu().numpy(), ref.raster_grads["duv"], GRAD_TOL, "uv_grad_holder.grad")


def test_empty_and_degenerate_inputs(cuda_device):
    """No visible Gaussian -> (out, None) like render.py:706-729; zero Gaussians; all masked."""
    sc = small_scene(n=500, width=64, height=48, sh_degree=0, seed=1)
    sc["xyz"] = sc["xyz"] + torch.tensor([0.0, 0.0, 1000.0])   # everything behind / outside the frustum
    op = d3.GaussianSplatOp(d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.NONE))
    model = gpu_model(sc, cuda_device)
    model.act_applied = True
    out, ctx = op.forward(model, gpu_cameras(sc, cuda_device), training=True)
    assert ctx is None and op.last_num_rendered == 0
    sc2 = small_scene(n=800, width=64, height=48, sh_degree=0, seed=2)
    m2 = gpu_model(sc2, cuda_device)
    m2.act_applied = True
    mask = torch.ones(800, dtype=torch.bool, device=cuda_device)
    out, ctx = op.forward(m2, gpu_cameras(sc2, cuda_device), training=True, mask=mask)
    assert ctx is None


@pytest.mark.parametrize("n", [0, 1, 31, 4095, 4096, 4097, 70001, 1 << 20])
def test_scan_matches_cumsum(cuda_device, n):
    lib = _lib.load()
    g = torch.Generator().manual_seed(n)
    x = torch.randint(0, 50, (max(n, 1),), generator=g, dtype=torch.int32)[:n]
    xd = x.to(cuda_device)
    out = torch.empty_like(xd)
    sync = torch.zeros(2, dtype=torch.int64, device=cuda_device)
    ws = torch.empty(lib.d3gs_scan_workspace_bytes(n) + 64, dtype=torch.uint8, device=cuda_device)
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.d3gs_scan_tiles(xd.data_ptr(), out.data_ptr(), n, sync.data_ptr(), ws.data_ptr(), ws.numel(),
                                   sync.data_ptr() + 8, st), "scan")
    total, status = sync.tolist()
    assert status == 0
    ref = np.cumsum(x.numpy().astype(np.int64))
    assert total == (int(ref[-1]) if n else 0)
    np.testing.assert_array_equal(out.cpu().numpy(), ref.astype(np.int32))


@pytest.mark.parametrize("n,end_bit", [(1, 45), (300, 41), (4096, 45), (4097, 47), (123457, 45), (1 << 21, 50),
                                       (50000, 64), (50000, 8), (50000, 13)])
def test_radix_sort_stable_bit_range(cuda_device, n, end_bit):
    lib = _lib.load()
    rng = np.random.default_rng(n + end_bit)
    keys = rng.integers(0, 2 ** 63, size=n, dtype=np.uint64)
    if end_bit < 64:
        # few distinct values in the sorted range => many ties => stability is exercised
        keys = (keys & ~np.uint64((1 << end_bit) - 1)) | (rng.integers(0, 1 << min(end_bit, 12), size=n, dtype=np.uint64)
                                                          << np.uint64(max(end_bit - 12, 0)))
    vals = np.arange(n, dtype=np.int32)
    kd = torch.from_numpy(keys.view(np.int64)).to(cuda_device)
    vd = torch.from_numpy(vals).to(cuda_device)
    ka, va = torch.empty_like(kd), torch.empty_like(vd)
    ws = torch.empty(lib.d3gs_sort_workspace_bytes(n, 0, end_bit), dtype=torch.uint8, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    in_alt = C.c_int32(0)
    _lib.check(lib.d3gs_sort_pairs(kd.data_ptr(), ka.data_ptr(), vd.data_ptr(), va.data_ptr(), n, 0, end_bit,
                                   ws.data_ptr(), ws.numel(), C.byref(in_alt), status.data_ptr(),
                                   torch.cuda.current_stream().cuda_stream), "sort")
    ks, vs = (ka, va) if in_alt.value else (kd, vd)
    assert int(status.item()) == 0
    mask = np.uint64((1 << end_bit) - 1) if end_bit < 64 else np.uint64(2 ** 64 - 1)
    order = np.argsort(keys & mask, kind="stable")
    np.testing.assert_array_equal(ks.cpu().numpy().view(np.uint64), keys[order])
    np.testing.assert_array_equal(vs.cpu().numpy(), vals[order])


def test_bucket_sort_every_list_length(cuda_device):
    """d3gs_bucket_prepare + d3gs_bucket_sort through the C ABI: tiles whose lists have every interesting length
    (empty, one entry, the class boundaries of the three kernel instances, the capacity) come out ordered by
    (depth bits, index) with the reference's keys and ranges; a list beyond the capacity is refused."""
    lib = _lib.load()
    cap = int(lib.d3gs_bucket_sort_capacity())
    lengths = [0, 1, 2, 3, 31, 0, 511, 512, 513, 1000, 2047, 2048, 2049, 5000, 0, cap - 1, cap, 7]
    rng = np.random.default_rng(5)
    counts = np.array(lengths, np.int32)
    incl = np.cumsum(counts).astype(np.int32)
    total = int(incl[-1])
    # few distinct depths -> many ties, broken by the index; entries shuffled inside every tile's range
    depth = rng.integers(0, 200, size=total, dtype=np.uint64) + np.uint64(0x3F000000)
    ids = rng.permutation(total).astype(np.uint64)
    entries = (depth << np.uint64(32)) | ids
    st = torch.cuda.current_stream().cuda_stream
    dev = cuda_device
    d_counts, d_incl = torch.from_numpy(counts).to(dev), torch.from_numpy(incl).to(dev)
    ranges = torch.empty(len(lengths), 2, dtype=torch.int32, device=dev)
    cursor = torch.empty(len(lengths), dtype=torch.int32, device=dev)
    maxc = torch.zeros(1, dtype=torch.int64, device=dev)
    _lib.check(lib.d3gs_bucket_prepare(d_counts.data_ptr(), d_incl.data_ptr(), len(lengths), ranges.data_ptr(),
                                       cursor.data_ptr(), maxc.data_ptr(), 0, st), "prepare")
    assert int(maxc.item()) == cap
    start = incl - counts
    exp_ranges = np.stack([np.where(counts > 0, start, 0), np.where(counts > 0, incl, 0)], axis=1).astype(np.int32)
    np.testing.assert_array_equal(ranges.cpu().numpy(), exp_ranges)
    np.testing.assert_array_equal(cursor.cpu().numpy(), start)
    # pair buffers sized before the count was known and too small: every range is left empty, the longest list is
    # still reported; a capacity that holds the pairs changes nothing
    r2 = torch.full_like(ranges, -1)
    _lib.check(lib.d3gs_bucket_prepare(d_counts.data_ptr(), d_incl.data_ptr(), len(lengths), r2.data_ptr(),
                                       cursor.data_ptr(), maxc.data_ptr(), total - 1, st), "prepare (too small)")
    assert int(maxc.item()) == cap and int(r2.abs().sum().item()) == 0
    _lib.check(lib.d3gs_bucket_prepare(d_counts.data_ptr(), d_incl.data_ptr(), len(lengths), r2.data_ptr(),
                                       cursor.data_ptr(), maxc.data_ptr(), total, st), "prepare (fits)")
    np.testing.assert_array_equal(r2.cpu().numpy(), exp_ranges)
    d_entries = torch.from_numpy(entries.view(np.int64)).to(dev)
    vals = torch.full((total,), -1, dtype=torch.int32, device=dev)
    keys = torch.zeros(total, dtype=torch.int64, device=dev)
    _lib.check(lib.d3gs_bucket_sort(d_entries.data_ptr(), ranges.data_ptr(), len(lengths), cap, vals.data_ptr(),
                                    keys.data_ptr(), st), "sort")
    got_v, got_k = vals.cpu().numpy(), keys.cpu().numpy().view(np.uint64)
    for t, (a, b) in enumerate(zip(start, incl)):
        e = np.sort(entries[a:b])
        np.testing.assert_array_equal(got_v[a:b], (e & np.uint64(0xFFFFFFFF)).astype(np.int32), err_msg=f"tile {t}")
        np.testing.assert_array_equal(got_k[a:b], (np.uint64(t) << np.uint64(32)) | (e >> np.uint64(32)), err_msg=f"tile {t}")
    # keys are optional
    vals2 = torch.empty_like(vals)
    _lib.check(lib.d3gs_bucket_sort(d_entries.data_ptr(), ranges.data_ptr(), len(lengths), cap, vals2.data_ptr(), None, st),
               "sort without keys")
    assert torch.equal(vals, vals2)
    assert lib.d3gs_bucket_sort(d_entries.data_ptr(), ranges.data_ptr(), len(lengths), cap + 1, vals2.data_ptr(), None,
                                st) == -3
    assert "radix" in _lib.last_error() or "sort_pairs" in _lib.last_error()


def test_bucket_binning_falls_back_on_long_lists(cuda_device):
    """A tile list longer than the bucket sort's shared-memory capacity makes the operator take the radix-sort
    path for that launch; the result is the oracle's either way."""
    sc = small_scene(n=40000, width=64, height=48, sh_degree=0, seed=41, pos=("uniform", 0.4), log_scale=("normal", -3.0, 0.3))
    op, model, cams, out, ctx, ocfg, osc, ref = _run_forward(sc, cuda_device, EarlyFilterAlgo.OBB_DFVT, binning="bucket")
    longest = int((ref.ranges[:, 1] - ref.ranges[:, 0]).max())
    assert longest > _lib.load().d3gs_bucket_sort_capacity(), longest
    assert op.last_binning == "sort"
    np.testing.assert_array_equal(op.debug["sorted_values"].cpu().numpy(), ref.sorted_ids)
    np.testing.assert_array_equal(ctx.workload_ranges.cpu().numpy(), ref.ranges)
    np.testing.assert_array_equal(out.n_contrib.cpu().numpy(), ref.n_contrib)


def test_launch_ahead_binning_matches_and_repeats(cuda_device):
    """From the second launch of a shape on, the bucket path queues binning and rasterisation before the host has
    read the pair count.  Same lists, ranges and image as the first (waited-for) launch and the oracle -- also when
    the guess was wrong: buffers too small for the pairs, the tile-sort class of the longest list not launched, and
    a longest list beyond the sort capacity (radix path)."""
    # dense enough that some tile list is longer than 512 entries (second sort class)
    sc = small_scene(n=30000, width=200, height=136, sh_degree=1, seed=9, log_scale=("normal", -2.6, 0.3))
    op, model, cams, out, ctx, ocfg, osc, ref = _run_forward(sc, cuda_device, EarlyFilterAlgo.OBB_DFVT, binning="bucket")
    longest = int((ref.ranges[:, 1] - ref.ranges[:, 0]).max())
    assert 512 < longest <= _lib.load().d3gs_bucket_sort_capacity(), longest
    (key, guess), = op._ahead.items()
    assert guess[0] >= ref.num_rendered and guess[1] >= longest

    def same(tag, repeated):
        o, c = op.forward(model, cams, training=True)
        torch.cuda.synchronize()
        assert op.last_binning == "bucket" and op.launches_repeated == repeated, (tag, op.launches_repeated)
        assert op.last_num_rendered == ref.num_rendered
        np.testing.assert_array_equal(c.gaussian_idx_sorted.cpu().numpy(), ref.sorted_ids, err_msg=tag)
        np.testing.assert_array_equal(op.debug["sorted_keys"].cpu().numpy(), ref.sorted_keys.view(np.int64), err_msg=tag)
        np.testing.assert_array_equal(c.workload_ranges.cpu().numpy(), ref.ranges, err_msg=tag)
        np.testing.assert_array_equal(o.n_contrib.cpu().numpy(), ref.n_contrib, err_msg=tag)
        assert torch.equal(o.color, out.color) and torch.equal(o.T, out.T), tag

    same("guess holds", 0)
    op._ahead[key] = (1024, guess[1])          # fewer entries than pairs: nothing written, launch repeated
    assert ref.num_rendered > 1024
    same("pair buffers too small", 1)
    op._ahead[key] = (guess[0], 100)           # only the first sort class launched: long lists left unsorted, repeated
    same("sort class missing", 2)
    same("guess holds again", 2)
    op.launch_ahead = False
    same("waited for", 2)
    # a list beyond the sort capacity, met by a launch that ran ahead: the radix path takes over
    sc2 = small_scene(n=40000, width=64, height=48, sh_degree=0, seed=41, pos=("uniform", 0.4), log_scale=("normal", -3.0, 0.3))
    op2, model2, cams2, out2, ctx2, _, _, ref2 = _run_forward(sc2, cuda_device, EarlyFilterAlgo.OBB_DFVT, binning="bucket")
    assert op2.last_binning == "sort" and not op2._ahead
    tiles = ref2.ranges.shape[0]
    op2._ahead[(model2.xyz.device, 1, 40000, tiles)] = (1 << 21, 16384)
    o2, c2 = op2.forward(model2, cams2, training=True)
    torch.cuda.synchronize()
    assert op2.last_binning == "sort" and op2.launches_repeated == 1
    np.testing.assert_array_equal(c2.gaussian_idx_sorted.cpu().numpy(), ref2.sorted_ids)
    np.testing.assert_array_equal(o2.n_contrib.cpu().numpy(), ref2.n_contrib)
    assert torch.equal(o2.color, out2.color)


@pytest.mark.parametrize("direct", [True, False])
def test_atomic_add_count_matches_the_oracle(cuda_device, direct, capsys):
    """measure_atomic_add_count (config_def.py:134): the instrumented raster backward counts its groups of global
    atomic adds.  With direct adds a group is (4 x 2 pixel block, splat) with a valid pixel -- counted exactly by the
    oracle; with per-tile accumulation it is (tile, splat) with a non-zero sum.  The oracle also gives the count of
    the reference's own reduction unit (a warp = 16 x 2 pixels).  Gradients are those of the plain kernel."""
    sc = small_scene(n=6000, width=200, height=136, sh_degree=1, seed=21)
    grads = {}
    for measure in (False, True):
        op_cfg = d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT, measure_atomic_add_count=measure)
        op = d3.GaussianSplatOp(op_cfg)
        op.raster_grad_direct = direct
        model = gpu_model(sc, cuda_device)
        model.act_applied = True
        cams = gpu_cameras(sc, cuda_device)
        out, ctx = op.forward(model, cams, training=True)
        g = torch.Generator(device="cpu").manual_seed(3)
        drgb = torch.randn(out.color.shape, generator=g).to(cuda_device)
        rg = op.rasterize_forward_backward(model, ctx, out, GaussianSplatGradients(drgb=drgb, dT=None))
        torch.cuda.synchronize()
        grads[measure] = [t.cpu().numpy() for t in (rg.duv, rg.dconic, rg.dopacity, rg.dcolor)]
    assert "atomic add count:" in capsys.readouterr().out
    for a, b in zip(grads[False], grads[True]):
        assert_close(b, a, 1e-4, "instrumented vs plain gradient", floor_frac=1e-3)   # float adds in another order
    ocfg = oracle_cfg(sc, op_cfg, True)
    ref = O.forward(ocfg, oracle_scene(sc))
    nc = out.n_contrib.cpu().numpy()
    np.testing.assert_array_equal(nc, ref.n_contrib)
    st = op.last_atomic_stats
    assert st["direct"] == direct and st["sort_pairs"] == ref.num_rendered
    groups_42, pixels = O.count_accumulations(ocfg, 1, ref.ranges, ref.sorted_ids, ref.prep, nc, block_wh=(4, 2))
    groups_warp, _ = O.count_accumulations(ocfg, 1, ref.ranges, ref.sorted_ids, ref.prep, nc, block_wh=(16, 2))
    groups_tile, _ = O.count_accumulations(ocfg, 1, ref.ranges, ref.sorted_ids, ref.prep, nc, block_wh=(16, 16))
    assert groups_tile <= groups_warp <= groups_42 <= pixels
    # a warp pass handles one splat for each of its eight lane groups (every group walks its own survivor list)
    assert groups_42 / 8 <= st["warp_passes"] <= groups_42
    if direct:
        assert op.last_atomic_add_count == groups_42
    else:   # a sum that cancels to exactly zero is not flushed: at most the oracle's count, and nearly all of it
        assert 0.999 * groups_tile <= op.last_atomic_add_count <= groups_tile


@pytest.mark.parametrize("shape", [(1, 40, 56), (2, 97, 130), (1, 16, 16), (1, 5, 7)])
def test_l1_dssim_loss_and_gradient(cuda_device, shape):
    b, h, w = shape
    g = torch.Generator().manual_seed(h * w)
    x = torch.rand(b, h, w, 3, generator=g)
    y = torch.rand(b, 3, h, w, generator=g)
    from d3gs_research_b200.fused_ssim import l1_dssim_forward_backward
    res, dx = l1_dssim_forward_backward(x.to(cuda_device), y.to(cuda_device), 0.2)
    ref, rdx = O.l1_dssim(x.numpy(), y.numpy(), 0.2)
    assert abs(res.item() - float(ref[0])) <= 1e-5 * max(1.0, abs(float(ref[0])))
    assert_close(dx.cpu().numpy(), rdx, 1e-4, "dL/dcolor", floor_frac=1e-2)


def test_fused_ssim_loss_api_matches_conv2d(cuda_device):
    from dense_reference import ssim_l1_loss_torch
    g = torch.Generator().manual_seed(4)
    x = torch.rand(2, 3, 75, 93, generator=g).to(cuda_device).requires_grad_(True)
    y = torch.rand(2, 3, 75, 93, generator=g).to(cuda_device)
    loss = d3.fused_ssim_loss(x, y)
    loss.backward()
    xr = x.detach().double().cpu().requires_grad_(True)
    _, _, ssim_ref = ssim_l1_loss_torch(xr, y.double().cpu())
    ssim_ref.backward()
    assert abs(loss.item() - ssim_ref.item()) < 1e-5
    assert_close(x.grad.cpu().numpy(), xr.grad.numpy(), 1e-3, "dssim/dx", floor_frac=1e-2)
    # NHWC prediction, same values
    xn = x.detach().permute(0, 2, 3, 1).contiguous().requires_grad_(True)
    d3.fused_ssim_loss(xn, y, pred_is_nhwc=True).backward()
    assert_close(xn.grad.permute(0, 3, 1, 2).cpu().numpy(), x.grad.cpu().numpy(), 1e-5, "nhwc grad")


def test_adam_and_densify_stats(cuda_device):
    n, b = 5003, 2
    g = torch.Generator().manual_seed(12)
    sc = small_scene(n=n, width=64, height=48, sh_degree=3, seed=8)
    model = gpu_model(sc, cuda_device).to_parameter()
    names = dict(xyz="xyz", quaternion_xyzw="quat", scale="scale", opacity="opacity", color_sh_base="sh_base",
                 color_sh="sh_rest")
    host = {k: sc[v].numpy().copy() for k, v in names.items()}
    initial = {k: v.copy() for k, v in host.items()}
    optims, _ = d3.create_origin_3dgs_optimizers(model, d3.Optimizer(), batch_size=1, spatial_lr_scale=1.0)
    state = d3.GaussianTrainState.create(n, device=cuda_device)
    strat = d3.GaussianStrategyOrigin(refine_scale2d_stop_iter=10)
    hm = {k: np.zeros_like(v) for k, v in host.items()}
    hv = {k: np.zeros_like(v) for k, v in host.items()}
    hstate = dict(duv_ndc_length=np.zeros(n, np.float32), count=np.zeros(n, np.float32), max_radii=np.zeros(n, np.float32))
    from d3gs_research_b200.adam import fused_step
    from d3gs_research_b200.render import GaussianSplatOutput
    for step in (1, 2, 3):
        grads = {k: (torch.randn(v.shape, generator=g) * (torch.rand(v.shape, generator=g) > 0.3)).numpy().astype(np.float32)
                 for k, v in host.items()}
        for k in host:
            getattr(model, k).grad = torch.from_numpy(grads[k]).to(cuda_device)
        duv = torch.randn(b, n, 2, generator=g) * 1e-3
        radii = torch.randint(0, 30, (b * n,), generator=g, dtype=torch.int32) * (torch.rand(b * n, generator=g) > 0.4)
        radii = radii.to(torch.int32)
        out = GaussianSplatOutput(custom_features=None, T=torch.empty(b, 48, 64, device=cuda_device), color=None,
                                  radii=radii.to(cuda_device))
        duv_d = duv.to(cuda_device)      # must outlive the launch: the struct only holds its address
        st = strat.stats_struct(state, out, duv_d)
        if step == 2:   # separate launches: six optimizers then the statistics
            for o in optims.values():
                o.step()
            strat.update(state, out, duv_d)
        else:           # one fused launch
            fused_step(optims.values(), st)
        lrs = dict(xyz=1.6e-4, color_sh_base=2.5e-3, color_sh=2.5e-3 / 20, opacity=0.05, scale=5e-3, quaternion_xyzw=1e-3)
        for k in host:
            O.adam(host[k].reshape(-1), grads[k].reshape(-1), hm[k].reshape(-1), hv[k].reshape(-1), lrs[k], 0.9, 0.999,
                   1e-15, step)
        O.densify_stats(b, n, 64, 48, True, duv.numpy(), radii.numpy(), hstate["duv_ndc_length"], hstate["count"],
                        hstate["max_radii"])
    torch.cuda.synchronize()
    lrs = dict(xyz=1.6e-4, color_sh_base=2.5e-3, color_sh=2.5e-3 / 20, opacity=0.05, scale=5e-3, quaternion_xyzw=1e-3)
    for k in host:
        # the UPDATE over the three steps (a tolerance relative to the parameter's magnitude would hide it: three
        # position steps move at most 5e-4 of a coordinate near 3); three steps -> three roundings of the parameter
        moved = getattr(model, k).detach().cpu().numpy() - initial[k]
        assert_update_close(moved, host[k] - initial[k], np.ones_like(host[k]), lrs[k], f"update {k}", first_step=False,
                            p_before=initial[k], ulps=3.0)
        assert_close(optims[k].state[getattr(model, k)]["exp_avg"].cpu().numpy(), hm[k], GRAD_TOL, f"exp_avg {k}")
        assert_close(optims[k].state[getattr(model, k)]["exp_avg_sq"].cpu().numpy(), hv[k], GRAD_TOL, f"exp_avg_sq {k}")
    for k in hstate:
        assert_close(getattr(state, k).cpu().numpy(), hstate[k], GRAD_TOL, f"stats {k}")


@pytest.mark.parametrize("n,sh_degree", [(3000, 3), (2501, 1)])
def test_fused_backward_adam_matches_separate_kernels(cuda_device, n, sh_degree):
    """The single-rank trainer applies Adam inside the preprocess backward; it must leave the parameters and
    moments that the gradient buffer + optimizer kernel leave.  The per-splat gradients come out of
    floating-point atomics, so the two runs differ in the last bits of some gradients: the moments (linear in
    the gradient) are compared tightly, the parameters over the bulk (Adam's normalised step amplifies a
    last-bit difference of a near-zero gradient)."""
    from d3gs_research_b200.trainer import SplatTrainer
    sc = small_scene(n=n, width=176, height=128, sh_degree=sh_degree, seed=5)
    op_cfg = d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT)
    target = torch.rand(1, 3, 128, 176, generator=torch.Generator().manual_seed(2)).to(cuda_device)
    res = {}
    for fused in (True, False):
        model = gpu_model(sc, cuda_device)
        model.cur_sh_degree = sh_degree
        init = model.flat.clone()
        tr = SplatTrainer(model, op_cfg, lambda_dssim=0.2, batch_size=1, fuse_backward_adam=fused)
        assert tr.fused_adam == fused
        for _ in range(2):
            tr.step(gpu_cameras(sc, cuda_device), target)
        torch.cuda.synchronize()
        res[fused] = (model.flat.clone(), tr.exp_avg.clone(), tr.exp_avg_sq.clone(), tr.state.count.clone())
    assert float((res[True][0] - init).abs().max()) > 0
    assert torch.equal(res[True][3], res[False][3])
    for k, name in ((1, "exp_avg"), (2, "exp_avg_sq")):
        assert_close(res[True][k].cpu().numpy(), res[False][k].cpu().numpy(), GRAD_TOL, name)
    d = (res[True][0] - res[False][0]).abs()
    scale = (res[True][0] - init).abs().max()
    assert float((d > 1e-4 * scale).float().mean()) < 1e-3


def _full_size_invariants(cuda_device, cfg_name, training):
    from d3gs_research_b200 import scenes
    sc = scenes.make_scene(cfg_name, seed=0, views=1)
    op = d3.GaussianSplatOp(d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT))
    op.binning = "sort"     # the invariants below involve the unsorted key list
    op.debug_capture = True
    model = gpu_model(sc, cuda_device)
    model.act_applied = True
    out, ctx = op.forward(model, gpu_cameras(sc, cuda_device), training=training)
    torch.cuda.synchronize()
    d = op.debug
    K = op.last_num_rendered
    tt = d["tiles_touched"].long()
    assert int(tt.sum()) == K and int(d["scan"][-1]) == K
    assert torch.equal(torch.cumsum(tt, 0).int(), d["scan"])
    sk = d["sorted_keys"]
    assert bool((sk[1:] >= sk[:-1]).all()), "sorted keys are not non-decreasing"
    # the sort is a permutation of the emitted pairs and agrees with torch's stable sort
    ref_k, ref_i = torch.sort(d["keys"], stable=True)
    assert torch.equal(ref_k, sk)
    assert torch.equal(d["values"][ref_i], d["sorted_values"])
    # every tile's range holds exactly that tile's keys
    tiles = (sk >> 32).int()
    r = d["ranges"] if ctx is None else ctx.workload_ranges
    counts = torch.bincount(tiles.long(), minlength=r.shape[0]).int()
    assert torch.equal(r[:, 1] - r[:, 0], counts)
    nz = counts > 0
    assert bool((tiles[r[nz, 0].long()] == torch.nonzero(nz).flatten().int()).all())
    # raster invariants
    T = out.T
    assert bool(((T >= 0) & (T <= 1)).all())
    assert bool((out.n_contrib >= 0).all())
    assert bool(torch.isfinite(out.color).all())
    # no pixel can have contributed beyond the end of its tile's list
    h, w = T.shape[-2], T.shape[-1]
    tiles_x = (w + 15) // 16
    ty, tx = torch.meshgrid(torch.arange(h, device=T.device) // 16, torch.arange(w, device=T.device) // 16,
                            indexing="ij")
    per_pixel = (r[:, 1] - r[:, 0])[(ty * tiles_x + tx).flatten().long()].view(h, w)
    assert bool((out.n_contrib[0] < torch.clamp(per_pixel, min=1)).all())
    return K, out


def test_full_size_properties_cfg3(cuda_device):
    """BASELINE size (3 M Gaussians, 1080p): size-independent invariants of the binning and raster stages."""
    K, _ = _full_size_invariants(cuda_device, "cfg3", training=True)
    assert K > 1_000_000


def test_full_size_properties_cfg4_render(cuda_device):
    """Largest configuration (6 M Gaussians, 3840x2160, forward only): the same invariants in inference mode,
    where the background is composited and the colour clamped to [0, 1]."""
    K, out = _full_size_invariants(cuda_device, "cfg4", training=False)
    assert K > 5_000_000
    assert bool(((out.color >= 0) & (out.color <= 1)).all())


@pytest.mark.parametrize("n,k,use_64bit", [(1, 3, False), (3, 3, False), (257, 1, False), (5000, 3, False),
                                           (20000, 3, True), (20000, 6, False), (4097, 8, True)])
def test_simple_knn_against_the_oracle(cuda_device, n, k, use_64bit):
    """d3gs_simple_knn (ops.py:14-183) against the oracle's exhaustive search, bit for bit: the same distance
    expression in the same order on both sides, and the k smallest values do not depend on the search order.
    Clustered points (most boxes are culled for most CTAs), a duplicate pair, n not a multiple of the box size, and
    fewer than k other points (the missing neighbours stay at sqrt(FLT_MAX), as in the reference)."""
    from d3gs_research_b200.ops import simple_knn
    rng = np.random.default_rng(n + k)
    pts = np.concatenate([rng.normal(size=(n - n // 3, 3)) * 3.0,
                          rng.normal(size=(n // 3, 3)) * 0.02 + np.array([5.0, -2.0, 1.0])]).astype(np.float32)
    if n > 10:
        pts[9] = pts[2]
    # a wider row than xyz: the stride is honoured
    wide = np.concatenate([pts, rng.normal(size=(n, 2)).astype(np.float32)], axis=1)
    got = simple_knn(torch.from_numpy(wide).to(cuda_device), k, use_64bit).cpu().numpy()
    ref = O.simple_knn(wide, k)
    np.testing.assert_array_equal(got.view(np.uint32), ref.view(np.uint32))
    if n > 10:
        assert got[9, 0] == 0.0 and got[2, 0] == 0.0


def test_point_cloud_init_scales(cuda_device):
    """tools.py:64-90: a regular grid has its three nearest neighbours at the grid spacing."""
    from d3gs_research_b200.tools import init_original_3dgs_model, points_to_gaussian_init_scale
    pts = np.stack(np.meshgrid(np.arange(4.0), np.arange(4.0), np.arange(4.0), indexing="ij"), -1).reshape(-1, 3) * 0.5
    s = points_to_gaussian_init_scale(torch.from_numpy(pts.astype(np.float32)).to(cuda_device))
    assert torch.allclose(s, torch.full_like(s, float(np.log(0.5))), atol=1e-5)
    m2 = d3.GaussianModelOriginFused.create_flat(64, device=cuda_device)
    init_original_3dgs_model(m2, pts, np.full((64, 3), 0.5))
    assert m2.cur_sh_degree == 0 and float(m2.color_sh_base.abs().max()) == 0.0 and float(m2.quaternion_xyzw[:, 3].min()) == 1.0
    assert abs(float(torch.sigmoid(m2.opacity[0])) - 0.1) < 1e-6
    assert torch.allclose(m2.scale, torch.full_like(m2.scale, float(np.log(0.5))), atol=1e-5)


def test_sh_degree_schedule_steps_match_the_oracle(cuda_device):
    """train.py:299-302: the active SH degree rises by one every 1000 // batch_size iterations.  A trainer whose
    batch size makes that period one iteration steps at degree 0, 1, 2, 3; every step's Adam update must be the
    oracle's for that degree (bands above the active degree get no gradient, their moments only decay)."""
    from d3gs_research_b200.strategy import GaussianStrategyOrigin
    from d3gs_research_b200.trainer import SplatTrainer
    sc = small_scene(n=4000, width=160, height=112, sh_degree=3, seed=23)
    op_cfg = d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT)
    osc = oracle_scene(sc)
    model = gpu_model(sc, cuda_device)
    model.cur_sh_degree = 0
    cams = gpu_cameras(sc, cuda_device)
    target = sc["target"][:1].contiguous()
    tgt = target.to(cuda_device)
    fields = ("xyz", "quat", "scale", "opacity", "sh_base", "sh_rest")
    attr = dict(xyz="xyz", quat="quaternion_xyzw", scale="scale", opacity="opacity", sh_base="color_sh_base", sh_rest="color_sh")
    tr = SplatTrainer(model, op_cfg, lambda_dssim=0.2, batch_size=1)
    tr.batch_size = 1000          # only the schedule reads it after construction: 1000 // 1000 = every iteration
    st = GaussianStrategyOrigin(refine_start_iter=10 ** 6)
    adam_state = {k: (np.zeros_like(getattr(osc, k)), np.zeros_like(getattr(osc, k))) for k in fields}
    m_views, v_views = tr._field_views(tr.exp_avg), tr._field_views(tr.exp_avg_sq)
    for step in range(4):
        assert model.cur_sh_degree == step
        # both sides start the step from the oracle's state, so that only this step's gradient differs
        before = {k: getattr(osc, k).copy() for k in fields}
        with torch.no_grad():
            for k in fields:
                getattr(model, attr[k]).copy_(torch.from_numpy(before[k]).to(cuda_device))
                m_views[attr[k]].copy_(torch.from_numpy(adam_state[k][0]).to(cuda_device))
                v_views[attr[k]].copy_(torch.from_numpy(adam_state[k][1]).to(cuda_device))
        ocfg = oracle_cfg(sc, op_cfg, True)
        ocfg.sh_degree = step
        ref = O.run_iteration(ocfg, osc, target.numpy(), 0.2, adam_state=adam_state, step=step + 1)
        if step < 3:     # bands above the active degree: no gradient
            assert not ref.grads["sh_rest"][:, (step + 1) ** 2 - 1:].any()
        tr.step(cams, tgt)
        tr.op.check_status()
        torch.cuda.synchronize()
        for k in fields:
            after = getattr(model, attr[k]).detach().cpu().numpy()
            if k == "sh_rest" and step == 0:     # degree 0: no band above the base is active, nothing may move
                assert not (getattr(osc, k) - before[k]).any() and not (after - before[k]).any()
                continue
            assert_update_close(after - before[k], getattr(osc, k) - before[k], ref.grads[k], O.ADAM_LRS[k],
                                f"degree {step} Adam update {k}", first_step=step == 0, p_before=before[k])
        fired = tr.end_of_iteration(step, st)
        assert fired == (["up_sh"] if step < 3 else [])
    assert model.cur_sh_degree == 3


def _rigid_T(rng, angle, shift):
    """A [4,3] transform in the cam2world_T layout: rows 0-2 the transposed rotation, row 3 the translation."""
    axis = rng.normal(size=3)
    axis /= np.linalg.norm(axis)
    a = rng.uniform(-angle, angle)
    K = np.array([[0, -axis[2], axis[1]], [axis[2], 0, -axis[0]], [-axis[1], axis[0], 0]])
    R = np.eye(3) + np.sin(a) * K + (1 - np.cos(a)) * (K @ K)
    return np.concatenate([R.T, rng.uniform(-shift, shift, size=(1, 3))], axis=0).astype(np.float32)


@pytest.mark.parametrize("views", [1, 3])
def test_instance_rendering_forward_and_backward(cuda_device, views):
    """instance2world_T (render.py:207-220, 346-354, 3031-3039): Gaussians with instance_id >= 0 are rendered through
    the camera taken into their object's frame, per view's frame id.  Binning bit-exact, image and the gradients of
    the Gaussians' own parameters against the oracle; Gaussians of no instance behave as without the argument."""
    sc = small_scene(n=5000, width=200, height=136, sh_degree=2, seed=31, views=views)
    rng = np.random.default_rng(8)
    n = sc["cfg"].n
    inst = rng.integers(-1, 3, size=n).astype(np.int32)               # -1: world Gaussian; 0..2: an object
    frames = 4
    T = np.stack([np.stack([_rigid_T(rng, 0.25, 0.3) for _ in range(3)]) for _ in range(frames)])   # [4,3,4,3]
    frame_ids = np.array([2, 0, 3][:views], np.int32)
    op_cfg = d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT)
    op = d3.GaussianSplatOp(op_cfg)
    op.debug_capture = True
    model = gpu_model(sc, cuda_device)
    model.act_applied = True
    model.instance_id = torch.from_numpy(inst).to(cuda_device)
    cams = gpu_cameras(sc, cuda_device)
    if views == 1:
        cams.frame_local_id = int(frame_ids[0])
    else:
        cams.frame_ids = torch.from_numpy(frame_ids).to(cuda_device)
    T_dev = torch.from_numpy(T).to(cuda_device)
    out, ctx = op.forward(model, cams, training=True, instance2world_T=T_dev)
    torch.cuda.synchronize()
    ocfg = oracle_cfg(sc, op_cfg, True)
    osc = oracle_scene(sc)
    osc.instance_id, osc.instance2world_T, osc.frame_ids = inst, T, frame_ids
    ref = O.forward(ocfg, osc)
    plain = O.forward(ocfg, oracle_scene(sc))
    assert (ref.prep["radii"] != plain.prep["radii"]).sum() > 100, "the transforms should move many Gaussians"
    world = np.tile(inst < 0, views)
    np.testing.assert_array_equal(ref.prep["radii"][world], plain.prep["radii"][world])
    np.testing.assert_array_equal(op.debug["tiles_touched"].cpu().numpy(), ref.prep["tiles_touched"])
    np.testing.assert_array_equal(ctx.radii.cpu().numpy(), ref.prep["radii"])
    np.testing.assert_array_equal(op.debug["sorted_values"].cpu().numpy(), ref.sorted_ids)
    np.testing.assert_array_equal(ctx.workload_ranges.cpu().numpy(), ref.ranges)
    np.testing.assert_array_equal(out.n_contrib.cpu().numpy(), ref.n_contrib)
    assert_close(out.color.cpu().numpy(), ref.color, IMG_TOL, "color")
    g = torch.Generator(device="cpu").manual_seed(5)
    drgb = torch.randn(out.color.shape, generator=g)
    O.backward(ocfg, osc, ref, drgb.numpy())
    gm, duv, _ = op.backward(model, cams, ctx, out, GaussianSplatGradients(drgb=drgb.to(cuda_device), dT=None),
                             return_uv_grad=True, instance2world_T=T_dev)
    torch.cuda.synchronize()
    for k, attr in (("xyz", "xyz"), ("quat", "quaternion_xyzw"), ("scale", "scale"), ("opacity", "opacity"),
                    ("sh_base", "color_sh_base"), ("sh_rest", "color_sh")):
        assert_close(getattr(gm, attr).cpu().numpy(), ref.grads[k], GRAD_TOL, f"grad {k}", floor_frac=1e-2)
    # and through the autograd entry point
    m2 = gpu_model(sc, cuda_device, requires_grad=True)
    m2.instance_id = model.instance_id
    out2 = d3.rasterize_gaussians(m2, cams, d3.GaussianSplatOp(op_cfg), training=True, instance2world_T=T_dev)
    (out2.color * drgb.to(cuda_device)).sum().backward()
    assert_close(m2.xyz.grad.cpu().numpy(), ref.grads["xyz"], GRAD_TOL, "autograd grad xyz", floor_frac=1e-2)
    # render.py:3840-3891: the "dynamic" entry point is the same call for a model without proxy fields; it wants a
    # camera bundle with frame ids when instances are rendered, and refuses user-defined proxy inputs
    op3 = d3.GaussianSplatOp(op_cfg)
    if views > 1:
        out3 = d3.rasterize_gaussians_dynamic(model, cams, op3, training=True, instance2world_T=T_dev)
        assert torch.equal(out3.color, out.color) and torch.equal(out3.n_contrib, out.n_contrib)
    else:
        with pytest.raises(AssertionError):
            d3.rasterize_gaussians_dynamic(model, cams, op3, training=True, instance2world_T=T_dev)
        out3 = d3.rasterize_gaussians_dynamic(model, cams, op3, training=True)
        assert out3.color.shape == out.color.shape
    with pytest.raises(NotImplementedError):
        d3.rasterize_gaussians_dynamic(model, cams, op3, prep_inputs={"x": 1})


@pytest.mark.parametrize("views", [1, 3])
def test_sparse_mode_matches_dense(cuda_device, views):
    """sparse_mode (config_def.py:119; render.py:235-238, 478-499, 2860-2903): the tensors kept for the backward and
    the returned gradient model hold the visible items / the Gaussians some view saw; values are the dense ones."""
    sc = small_scene(n=5000, width=200, height=136, sh_degree=2, seed=37, views=views)
    model = gpu_model(sc, cuda_device)
    model.act_applied = True
    cams = gpu_cameras(sc, cuda_device)
    n = sc["cfg"].n
    # the scene's Gaussians all lie in view: a mask (render.py:270-272, non-zero = skip) takes a third of the items out
    mask = (torch.rand(views * n, generator=torch.Generator().manual_seed(2)) < 0.33).to(cuda_device)
    res = {}
    for sparse in (False, True):
        op = d3.GaussianSplatOp(d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT, sparse_mode=sparse))
        out, ctx = op.forward(model, cams, training=True, mask=mask)
        g = torch.Generator(device="cpu").manual_seed(5)
        drgb = torch.randn(out.color.shape, generator=g).to(cuda_device)
        gm, duv, _ = op.backward(model, cams, ctx, out, GaussianSplatGradients(drgb=drgb, dT=None), return_uv_grad=True)
        torch.cuda.synchronize()
        res[sparse] = (out, ctx, gm, duv)
    (od, cd, gd, duvd), (os_, cs, gs, duvs) = res[False], res[True]
    assert torch.equal(os_.color, od.color) and torch.equal(os_.T, od.T) and torch.equal(os_.n_contrib, od.n_contrib)
    flat = torch.nonzero(cd.radii != 0).flatten()
    assert 100 < flat.numel() < views * n
    assert torch.equal(os_.sparse_gaussian_ids.long(), flat % n) and torch.equal(os_.sparse_batch_ids.long(), flat // n)
    assert os_.radii.shape[0] == flat.numel() and torch.equal(os_.radii, cd.radii[flat])
    for name in ("depths", "uvs", "conic_opacity", "rgb_gaussian", "cov2d_vecs", "sh_to_rgb_ne_0", "splat_records"):
        assert torch.equal(getattr(cs, name), getattr(cd, name)[flat]), name
    # the sorted lists are the dense ones with the indices renumbered
    assert torch.equal(flat[cs.gaussian_idx_sorted.long()], cd.gaussian_idx_sorted.long())
    assert torch.equal(cs.workload_ranges, cd.workload_ranges)
    # gradients: rows of the Gaussians some view saw, ascending; everything else is zero in the dense model
    seen = torch.nonzero((cd.radii.view(views, n) != 0).any(0)).flatten()
    assert torch.equal(gs.sparse_gaussian_ids.long(), seen) and len(gs) == seen.numel()
    for attr in ("xyz", "quaternion_xyzw", "scale", "opacity", "color_sh_base", "color_sh"):
        dense = getattr(gd, attr)
        # the float atomics of the raster backward add in another order: not bit-equal
        assert_close(getattr(gs, attr).cpu().numpy(), dense[seen].cpu().numpy(), GRAD_TOL, f"sparse grad {attr}", floor_frac=1e-2)
        rest = torch.ones(n, dtype=torch.bool, device=cuda_device)
        rest[seen] = False
        assert not dense[rest].any()
    got = duvs.reshape(-1, 2).cpu().numpy()
    assert_close(got, duvd.reshape(-1, 2)[flat].cpu().numpy(), GRAD_TOL, "sparse duv", floor_frac=1e-2)
