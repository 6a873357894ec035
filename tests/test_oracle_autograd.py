"""The CPU oracle's forward image and all 59 parameter gradients against torch autograd on an independent
dense float64 renderer (tests/dense_reference.py)."""
import numpy as np
import pytest
import torch

from dense_reference import render_dense
from oracle import oracle as O
from parity_utils import oracle_scene, small_scene


@pytest.mark.parametrize("deg,early_filter,ref_order,aa", [(0, 0, True, False), (3, 0, True, False), (3, 3, True, False),
                                                             (2, 1, False, False), (1, 0, True, True), (3, 4, True, True),
                                                             (2, 2, True, False)])
def test_oracle_matches_dense_autograd(deg, early_filter, ref_order, aa):
    """aa: enable_anti_aliasing, the opacity compensation of render.py:449-462 and its gradient (3295-3309)."""
    W, H = 48, 40
    sc = small_scene(n=150, width=W, height=H, sh_degree=deg, seed=10 + deg, log_scale=("normal", -1.8, 0.5), sh_gain=6.0)
    osc = oracle_scene(sc)
    cfg = O.OpConfig(width=W, height=H, sh_degree=deg, early_filter=early_filter, clamp_mask_reference_order=ref_order,
                     anti_aliasing=aa)
    res = O.forward(cfg, osc)
    g = torch.Generator().manual_seed(5)
    drgb = torch.randn(1, H, W, 3, generator=g).numpy().astype(np.float32)
    dT = torch.randn(1, H, W, generator=g).numpy().astype(np.float32)
    O.backward(cfg, osc, res, drgb, dT)
    params = {k: torch.tensor(getattr(osc, k), dtype=torch.float64, requires_grad=True)
              for k in ("xyz", "quat", "scale", "opacity", "sh_base", "sh_rest")}
    C, T, vis = render_dense(params, osc.cams[0], W, H, deg, clamp_mask_reference_order=ref_order, anti_aliasing=aa)
    assert int(vis.sum()) == int((res.prep["radii"] > 0).sum())
    assert np.abs(C.detach().numpy() - res.color[0]).max() < 2e-5
    assert np.abs(T.detach().numpy() - res.T[0]).max() < 2e-5
    loss = (C * torch.tensor(drgb[0], dtype=torch.float64)).sum() + (T * torch.tensor(dT[0], dtype=torch.float64)).sum()
    loss.backward()
    for k, p in params.items():
        ref = p.grad.numpy()
        scale = np.abs(ref).max()
        if scale == 0:
            assert np.abs(res.grads[k]).max() == 0
        else:
            assert np.abs(res.grads[k] - ref).max() / scale < 2e-4, k


def test_view_batch_gradient_is_sum_over_views():
    """render.py:3182-3199: the gradient of a view batch is the plain sum of the per-view gradients."""
    sc = small_scene(n=300, width=64, height=48, sh_degree=1, seed=2, views=2)
    osc = oracle_scene(sc)
    cfg = O.OpConfig(width=64, height=48, sh_degree=1)
    g = torch.Generator().manual_seed(1)
    drgb = torch.randn(2, 48, 64, 3, generator=g).numpy().astype(np.float32)
    both = O.backward(cfg, osc, O.forward(cfg, osc), drgb)
    acc = None
    for v in range(2):
        one = O.Scene(osc.xyz, osc.quat, osc.scale, osc.opacity, osc.sh_base, osc.sh_rest, cams=osc.cams[v:v + 1].copy())
        r = O.backward(cfg, one, O.forward(cfg, one), drgb[v:v + 1])
        acc = {k: r.grads[k].astype(np.float64) + (0 if acc is None else acc[k]) for k in r.grads}
    for k in acc:
        np.testing.assert_allclose(both.grads[k], acc[k], rtol=1e-4, atol=1e-6 * max(1e-12, np.abs(acc[k]).max()))


def test_oracle_32bit_sort_keys():
    """enable_32bit_sort (render.py:737, 767-770, 851-854): key = tile << 18 | (uint32(depth / 0.001) & 0x3FFFF),
    sorted on 32 bits; same pairs and ranges as the 64-bit keys, tiles in the same order, depths quantised."""
    sc = small_scene(n=800, width=96, height=64, sh_degree=1, seed=6, views=2)
    osc = oracle_scene(sc)
    r64 = O.forward(O.OpConfig(width=96, height=64, sh_degree=1, early_filter=4), osc)
    r32 = O.forward(O.OpConfig(width=96, height=64, sh_degree=1, early_filter=4, key_shift=18), osc)
    assert r32.num_rendered == r64.num_rendered and int(r32.keys.max()) < 2 ** 32
    np.testing.assert_array_equal(r32.vals, r64.vals)
    np.testing.assert_array_equal(r32.keys >> np.uint64(18), r64.keys >> np.uint64(32))
    depth = r64.keys.astype(np.uint32).view(np.float32)      # low 32 bits of the 64-bit keys are the depth's bits
    np.testing.assert_array_equal(r32.keys & np.uint64(0x3FFFF),
                                  ((depth / np.float32(0.001)).astype(np.uint32) & 0x3FFFF).astype(np.uint64))
    assert bool((r32.sorted_keys[1:] >= r32.sorted_keys[:-1]).all())
    np.testing.assert_array_equal(r32.ranges, r64.ranges)     # the same tiles hold the same number of pairs
    order = np.argsort(r32.keys, kind="stable")
    np.testing.assert_array_equal(r32.sorted_ids, r32.vals[order])


@pytest.mark.parametrize("inv", [False, True])
def test_oracle_depth_matches_dense_autograd(inv):
    """render_depth / render_inv_depth: the blended depth value and the gradient it sends to every parameter
    (render.py:582, 1824, 1948-1967, 3053-3057)."""
    W, H, deg = 48, 40, 1
    sc = small_scene(n=150, width=W, height=H, sh_degree=deg, seed=12, log_scale=("normal", -1.8, 0.5), sh_gain=6.0)
    osc = oracle_scene(sc)
    cfg = O.OpConfig(width=W, height=H, sh_degree=deg, early_filter=0, inv_depth=inv)
    res = O.forward(cfg, osc, render_depth=True)
    g = torch.Generator().manual_seed(8)
    drgb = torch.randn(1, H, W, 3, generator=g).numpy().astype(np.float32)
    ddepth = torch.randn(1, H, W, generator=g).numpy().astype(np.float32)
    O.backward(cfg, osc, res, drgb, None, ddepth)
    params = {k: torch.tensor(getattr(osc, k), dtype=torch.float64, requires_grad=True)
              for k in ("xyz", "quat", "scale", "opacity", "sh_base", "sh_rest")}
    C, T, vis, D = render_dense(params, osc.cams[0], W, H, deg, depth_mode="inv" if inv else "z")
    assert np.abs(C.detach().numpy() - res.color[0]).max() < 2e-5
    scale_d = np.abs(D.detach().numpy()).max()
    assert np.abs(D.detach().numpy() - res.depth[0]).max() < 2e-5 * max(scale_d, 1.0)
    loss = (C * torch.tensor(drgb[0], dtype=torch.float64)).sum() + (D * torch.tensor(ddepth[0], dtype=torch.float64)).sum()
    loss.backward()
    for k, p in params.items():
        ref = p.grad.numpy()
        scale = np.abs(ref).max()
        assert np.abs(res.grads[k] - ref).max() / scale < 2e-4, k


def test_oracle_custom_features_match_dense_autograd():
    """custom_features [B*N,F] blended into [B,H,W,F] and the gradients of a loss on that image: to the features
    themselves and, through the blend weights, to the Gaussians (render.py:241-245, 1920-1923, 1952-1971)."""
    W, H, deg, F = 48, 40, 0, 4
    sc = small_scene(n=150, width=W, height=H, sh_degree=deg, seed=14, log_scale=("normal", -1.8, 0.5), sh_gain=6.0)
    osc = oracle_scene(sc)
    cfg = O.OpConfig(width=W, height=H, sh_degree=deg, early_filter=3)
    g = torch.Generator().manual_seed(9)
    feat = torch.randn(150, F, generator=g).numpy().astype(np.float32)
    res = O.forward(cfg, osc, custom_features=feat)
    drgb = torch.randn(1, H, W, 3, generator=g).numpy().astype(np.float32)
    dfeat_img = torch.randn(1, H, W, F, generator=g).numpy().astype(np.float32)
    O.backward(cfg, osc, res, drgb, None, None, dfeat_img)
    params = {k: torch.tensor(getattr(osc, k), dtype=torch.float64, requires_grad=True)
              for k in ("xyz", "quat", "scale", "opacity", "sh_base", "sh_rest")}
    ft = torch.tensor(feat, dtype=torch.float64, requires_grad=True)
    C, T, vis, Fi = render_dense(params, osc.cams[0], W, H, deg, custom=ft)
    assert np.abs(Fi.detach().numpy() - res.custom_image[0]).max() < 2e-5
    loss = (C * torch.tensor(drgb[0], dtype=torch.float64)).sum() + (Fi * torch.tensor(dfeat_img[0], dtype=torch.float64)).sum()
    loss.backward()
    ref = ft.grad.numpy()
    assert np.abs(res.raster_grads["dcustom"] - ref).max() / np.abs(ref).max() < 2e-4
    for k in ("xyz", "quat", "scale", "opacity"):
        ref = params[k].grad.numpy()
        assert np.abs(res.grads[k] - ref).max() / np.abs(ref).max() < 2e-4, k


def test_early_filters_drop_only_tiles_that_contribute_nothing():
    """The filters (render.py:1017-1327) only remove (tile, splat) pairs in which no pixel reaches alpha_eps, so the
    image is the unfiltered one bit for bit; the exact ellipse test (ELLIPSE) keeps no more pairs than its
    bounding boxes (AABB, OBB) do."""
    sc = small_scene(n=3000, width=200, height=136, sh_degree=1, seed=6, log_scale=("normal", -2.2, 0.7))
    osc = oracle_scene(sc)
    res = {f: O.forward(O.OpConfig(width=200, height=136, sh_degree=1, early_filter=f), osc) for f in (0, 1, 2, 3)}
    for f in (1, 2, 3):
        np.testing.assert_array_equal(res[f].color.view(np.uint32), res[0].color.view(np.uint32))
        np.testing.assert_array_equal(res[f].T.view(np.uint32), res[0].T.view(np.uint32))
    k = {f: r.num_rendered for f, r in res.items()}
    assert k[2] <= k[3] <= k[0] and k[2] <= k[1] <= k[0] and k[2] < 0.9 * k[0], k
    # pair by pair: what ELLIPSE keeps, both boxes keep
    for other in (1, 3):
        kept = set(zip((res[2].sorted_keys >> np.uint64(32)).tolist(), res[2].sorted_ids.tolist()))
        box = set(zip((res[other].sorted_keys >> np.uint64(32)).tolist(), res[other].sorted_ids.tolist()))
        assert kept <= box, other
