"""The CPU oracle against vectors generated from the reference's own pure-torch helpers
(tests/golden/make_golden.py -> tests/golden/ref_vectors.npz) and against torch references."""
import os

import numpy as np
import torch

from oracle import oracle as O

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz"))


def test_sh_eval_matches_reference_eval_sh():
    coeff = G["sh_coeff"]                      # [n,16,3] coefficient-major
    base, rest = coeff[:, 0, :].copy(), np.ascontiguousarray(coeff[:, 1:, :])
    for deg in range(4):
        ours = O.sh_eval(deg, G["sh_dirs"], base, rest) - 0.5
        np.testing.assert_allclose(ours, G[f"sh_rgb_deg{deg}"], rtol=2e-5, atol=2e-6)


def test_rotation_and_covariance_match_reference():
    cov6, rot = O.cov3d(G["quat_xyzw"], G["scale_act"])
    np.testing.assert_allclose(rot, G["rot"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(cov6, G["cov6"], rtol=2e-5, atol=1e-9)


def test_ssim_and_l1_match_reference_loss_utils():
    for xk, sk in (("img_x", "ssim"), ("img_x2", "ssim2")):
        x_nhwc = np.ascontiguousarray(G[xk].transpose(0, 2, 3, 1))
        out, _ = O.l1_dssim(x_nhwc, np.ascontiguousarray(G["img_y"]), 0.2, want_grad=False)
        assert abs(float(out[2]) - float(G[sk])) < 2e-6, (out, G[sk])
        if xk == "img_x":
            assert abs(float(out[1]) - float(G["l1"])) < 1e-6
            assert abs(float(out[0]) - (0.8 * float(G["l1"]) + 0.2 * (1 - float(G["ssim"])))) < 2e-6


def test_lr_schedule_matches_reference():
    from d3gs_research_b200.tools import get_expon_lr_func
    f = get_expon_lr_func(lr_init=1.6e-4, lr_final=1.6e-6, lr_delay_mult=0.01, max_steps=30000)
    vals = np.array([f(int(s)) for s in G["lr_steps"]])
    np.testing.assert_allclose(vals, G["lr_values"], rtol=1e-12)


def test_loss_gradient_matches_torch_autograd():
    from dense_reference import ssim_l1_loss_torch
    g = torch.Generator().manual_seed(3)
    x = torch.rand(1, 3, 29, 41, generator=g, dtype=torch.float64, requires_grad=True)
    y = torch.rand(1, 3, 29, 41, generator=g, dtype=torch.float64)
    loss, _, _ = ssim_l1_loss_torch(x, y, 0.2)
    loss.backward()
    out, dx = O.l1_dssim(np.ascontiguousarray(x.detach().numpy().transpose(0, 2, 3, 1).astype(np.float32)),
                         y.numpy().astype(np.float32), 0.2)
    assert abs(float(out[0]) - loss.item()) < 2e-6
    ref = x.grad.numpy().transpose(0, 2, 3, 1)
    assert np.abs(dx - ref).max() < 2e-3 * np.abs(ref).max()


def test_adam_matches_torch_optim():
    g = torch.Generator().manual_seed(5)
    p0 = torch.randn(1000, generator=g)
    p = p0.clone().requires_grad_(True)
    opt = torch.optim.Adam([p], lr=1.6e-4, eps=1e-15, betas=(0.9, 0.999))
    hp, hm, hv = p0.numpy().copy(), np.zeros(1000, np.float32), np.zeros(1000, np.float32)
    for step in range(1, 6):
        gr = torch.randn(1000, generator=g)
        p.grad = gr.clone()
        opt.step()
        O.adam(hp, gr.numpy(), hm, hv, 1.6e-4, 0.9, 0.999, 1e-15, step)
    np.testing.assert_allclose(hp, p.detach().numpy(), rtol=1e-5, atol=1e-7)


def test_transcendentals_are_accurate():
    xs = np.linspace(-20, 10, 2001).astype(np.float32)
    got = np.array([O.lib().oracle_expf(float(v)) for v in xs])
    np.testing.assert_allclose(got, np.exp(xs.astype(np.float64)), rtol=3e-7)
    xs = np.linspace(-12, 0, 2001).astype(np.float32)
    got = np.array([O.lib().oracle_exp_blend(float(v)) for v in xs])
    np.testing.assert_allclose(got, np.exp(xs.astype(np.float64)), rtol=1.5e-6)
    xs = np.exp(np.linspace(-8, 3, 2001)).astype(np.float32)
    got = np.array([O.lib().oracle_logf(float(v)) for v in xs])
    np.testing.assert_allclose(got, np.log(xs.astype(np.float64)), rtol=3e-7, atol=3e-7)


def test_sort_is_stable_and_ranges_cover_tiles():
    rng = np.random.default_rng(0)
    keys = (rng.integers(0, 50, 5000, dtype=np.uint64) << np.uint64(32)) | rng.integers(0, 7, 5000, dtype=np.uint64)
    vals = np.arange(5000, dtype=np.int32)
    ks, vs = O.sort_pairs(keys, vals, 32 + 6)
    order = np.argsort(keys, kind="stable")
    np.testing.assert_array_equal(ks, keys[order])
    np.testing.assert_array_equal(vs, vals[order])
    r = O.tile_ranges(ks, 64)
    tiles = (ks >> np.uint64(32)).astype(np.int64)
    for t in range(64):
        idx = np.nonzero(tiles == t)[0]
        if len(idx):
            assert r[t, 0] == idx[0] and r[t, 1] == idx[-1] + 1
        else:
            assert tuple(r[t]) == (0, 0)


def test_oracle_simple_knn_against_sklearn():
    """The reference checks simple_knn against sklearn's NearestNeighbors (ops.py:186-206); so does the oracle."""
    from sklearn.neighbors import NearestNeighbors
    rng = np.random.default_rng(11)
    pts = np.concatenate([rng.normal(size=(1500, 3)), rng.normal(size=(500, 3)) * 0.05 + 2.0]).astype(np.float32)
    pts[7] = pts[3]                                    # a duplicate: its nearest other point is at distance 0
    for k in (1, 3, 6):
        got = O.simple_knn(pts, k)
        dist, _ = NearestNeighbors(n_neighbors=k + 1, algorithm="brute").fit(pts.astype(np.float64)).kneighbors(pts.astype(np.float64))
        np.testing.assert_allclose(got, dist[:, 1:], rtol=2e-5, atol=1e-7)
        assert (np.diff(got, axis=1) >= 0).all() and got[7, 0] == 0.0 and got[3, 0] == 0.0
