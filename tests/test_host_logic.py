"""Host-side logic that needs no GPU: configuration, containers, cameras, scenes, data-parallel semantics."""
import os
import sys

import numpy as np
import pytest
import torch

import d3gs_research_b200 as d3
from d3gs_research_b200 import scenes
from d3gs_research_b200.model import FLAT_ORDER, carve_flat


def test_config_defaults_follow_reference():
    c = d3.GaussianSplatConfig()
    assert c.tile_size == (16, 16) and c.near == 0.2 and c.far == 10000.0 and c.alpha_eps == 1.0 / 255.0
    assert c.gaussian_lowpass_filter == 0.3 and c.gaussian_std_sigma == 3.0 and c.projected_clamp_factor == 1.3
    assert c.early_filter_algo == d3.EarlyFilterAlgo.OBB_DFVT and c.num_channels == 3 and c.block_size == 256
    assert c.unsupported_options() == []
    t = d3.Train(batch_size=4)
    t.rescale_steps_by_batch_size(4)
    assert t.iterations == 7500 and t.optim.position_lr_max_steps == 7500 and t.strategy.refine_every == 25


@pytest.mark.parametrize("kw", [dict(transmittance_is_double=True), dict(move_opacity_in_grad_to_prep=True),
                                dict(tile_size=(8, 8)), dict(tile_size=(16, 8))])
def test_unsupported_options_raise_at_construction(kw):
    from d3gs_research_b200.render import GaussianSplatOp
    with pytest.raises(NotImplementedError):
        GaussianSplatOp(d3.GaussianSplatConfig(**kw))


def test_output_format_options_are_accepted():
    c = d3.GaussianSplatConfig(use_nchw=True, render_rgba=True, enable_32bit_sort=True, enable_anti_aliasing=True,
                               render_depth=True, render_inv_depth=True,
                               rasterize_backward_algo=d3.RasterizeBackwardAlgo.PER_GAUSSIAN)
    assert c.unsupported_options() == [] and c.num_channels == 4


def test_flat_model_views_and_containers():
    from d3gs_research_b200.model import flat_layout
    assert flat_layout(12)[1] == 59 * 12                       # no padding when n is a multiple of 4
    n = 10
    layout, total = flat_layout(n)
    assert total == 600 and all(off % 4 == 0 for off, _, _ in layout.values())   # every field on a 16-byte boundary
    flat = torch.arange(total, dtype=torch.float32)
    v = carve_flat(flat, n)
    assert [tuple(v[k].shape) for k in FLAT_ORDER] == [(n, 3), (n, 4), (n, 3), (n,), (n, 3), (n, 15, 3)]
    assert v["xyz"].data_ptr() == flat.data_ptr() and v["quaternion_xyzw"][0, 0] == 32
    assert v["color_sh"][-1, -1, -1] == layout["color_sh"][0] + 450 - 1
    m = d3.GaussianModelOriginFused.create_flat(n, device="cpu")
    assert len(m) == n and m.color_sh_degree == 3 and m.has_fused_activations and m.flat.numel() == total
    assert m.get_unique_kernel_key() == "3_3_normalize_exponential_sigmoid_False"
    z = d3.GaussianModelOriginFused.zeros_like(m, num=4, not_param=True)
    assert len(z) == 4 and z.color_sh.shape == (4, 15, 3)
    assert len(m.concat(z)) == 14 and len(m[2:5]) == 3
    mp = m.to_parameter()
    assert isinstance(mp.xyz, torch.nn.Parameter) and set(mp.get_all_parameter_fields()) >= {"xyz", "opacity"}
    o = d3.GaussianModelOrigin.zeros(3, 3, split=True)
    o.scale.fill_(0.5)
    act = o.create_model_with_act()
    assert act.act_applied and torch.allclose(act.scale, torch.exp(torch.tensor(0.5))) and not o.has_fused_activations
    assert torch.allclose(act.opacity, torch.tensor(0.5))


def test_camera_packing_matches_reference_layout():
    from d3gs_research_b200.render import CameraBundle, _camera_rows
    c2w = scenes.look_at_cam2world([1.0, 2.0, 8.0])
    cam = d3.BasicPinholeCamera.from_params(c2w, 500.0, 510.0, 320.0, 240.0, 640, 480)
    row = _camera_rows(cam)[0]
    np.testing.assert_allclose(row[:12].reshape(4, 3), c2w[:3].T, rtol=1e-6)      # render.py:205
    np.testing.assert_allclose(row[12:], [500, 510, 320, 240])
    np.testing.assert_allclose(cam.focal_length, [500, 510])
    b = CameraBundle.from_pinhole_cams([cam, cam], device="cpu")
    assert tuple(b.cam2world_T.shape) == (2, 4, 3) and tuple(b.focal_xy_ppoint.shape) == (2, 4)
    np.testing.assert_allclose(b.host_params()[1], row, rtol=1e-6)
    # forward axis +z, looking at the origin: the origin projects to the principal point
    R, c = c2w[:3, :3], c2w[:3, 3]
    pc = R.T @ (np.zeros(3) - c)
    assert pc[2] > 0 and abs(pc[0]) < 1e-9 and abs(pc[1]) < 1e-9


def test_scene_generators_are_seeded_and_shaped():
    a = scenes.make_scene("cfg0", seed=0)
    b = scenes.make_scene("cfg0", seed=0)
    assert a["xyz"].shape == (10_000, 3) and torch.equal(a["xyz"], b["xyz"]) and torch.equal(a["target"], b["target"])
    assert a["target"].shape == (1, 3, 256, 256) and float(a["sh_rest"].abs().max()) == 0.0
    c3 = scenes.make_scene("cfg3", seed=0, n=1000, views=8, width=64, height=36)
    assert c3["cams"].shape == (8, 16) and c3["target"].shape == (8, 3, 36, 64)
    assert abs(float(c3["quat"].norm(dim=1).mean()) - 1.0) < 1e-5
    c4 = scenes.CONFIGS["cfg4"]
    assert c4.n == 6_000_000 and (c4.width, c4.height) == (3840, 2160) and c4.num_views == 64


def test_optimizer_factory_hyperparameters():
    m = d3.GaussianModelOriginFused.create_flat(8, device="cpu").to_parameter()
    opts, sched = d3.create_origin_3dgs_optimizers(m, d3.Optimizer(), batch_size=4, spatial_lr_scale=2.0)
    assert set(opts) == {"xyz", "color_sh_base", "color_sh", "opacity", "scale", "quaternion_xyzw"}
    g = opts["xyz"].param_groups[0]
    assert abs(g["lr"] - 1.6e-4 * 2.0 * 2.0) < 1e-12 and abs(g["eps"] - 1e-15 / 2.0) < 1e-24
    assert g["betas"] == (1 - 4 * (1 - 0.9), 1 - 4 * (1 - 0.999))
    assert abs(opts["color_sh"].param_groups[0]["lr"] - 0.0025 * 2.0 / 20.0) < 1e-12
    assert abs(sched(0) - 1.6e-4 * 4.0) < 1e-12        # no delay steps: the delay multiplier is inactive
    assert abs(sched(30000) - 1.6e-6 * 4.0) < 1e-12


def _dp_worker(rank, world, port, q):
    """Each rank computes its own view's gradient with the loss scaled by 1/world; all-reduce (sum) must equal
    the gradient of the reference's batched loss (mean over B*C*H*W, train.py:170-172)."""
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from oracle import oracle as O
    from parity_utils import oracle_scene, small_scene
    sc = small_scene(n=400, width=64, height=48, sh_degree=1, seed=4, views=world)
    osc = oracle_scene(sc)
    cfg = O.OpConfig(width=64, height=48, sh_degree=1)
    tgt = sc["target"].numpy()
    one = O.Scene(osc.xyz, osc.quat, osc.scale, osc.opacity, osc.sh_base, osc.sh_rest, cams=osc.cams[rank:rank + 1].copy())
    res = O.forward(cfg, one)
    _, dx = O.l1_dssim(res.color, np.ascontiguousarray(tgt[rank:rank + 1]), 0.2)
    O.backward(cfg, one, res, dx / world)
    flat = torch.from_numpy(np.concatenate([res.grads[k].reshape(-1) for k in ("xyz", "quat", "scale", "opacity", "sh_base", "sh_rest")]))
    dist.all_reduce(flat)
    if rank == 0:
        full = O.forward(cfg, osc)
        _, dxf = O.l1_dssim(full.color, np.ascontiguousarray(tgt), 0.2)       # mean over B*C*H*W
        O.backward(cfg, osc, full, dxf)
        ref = np.concatenate([full.grads[k].reshape(-1) for k in ("xyz", "quat", "scale", "opacity", "sh_base", "sh_rest")])
        q.put(float(np.abs(flat.numpy() - ref).max() / np.abs(ref).max()))
    dist.barrier()
    dist.destroy_process_group()


def test_data_parallel_allreduce_equals_batched_gradient_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_dp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    err = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert err < 1e-5, err


def test_shard_layout_and_field_clipping():
    from d3gs_research_b200.trainer import clip_fields, shard_layout
    n = 1001
    total = 59 * n
    for world in (1, 2, 3, 8):
        s, padded = shard_layout(total, world)
        assert s % 4 == 0 and padded == s * world and padded >= total and padded - total < 4 * world + world
    offsets, off = {}, 0
    for name, per in zip(FLAT_ORDER, (3, 4, 3, 1, 3, 45)):
        offsets[name] = (off, per * n)
        off += per * n
    s, padded = shard_layout(total, 3)
    covered = np.zeros(padded, dtype=np.int32)
    for r in range(3):
        for name, a, cnt in clip_fields(offsets, r * s, (r + 1) * s):
            o, c = offsets[name]
            assert o <= a and a + cnt <= o + c and r * s <= a and a + cnt <= (r + 1) * s
            covered[a:a + cnt] += 1
    assert (covered[:total] == 1).all() and (covered[total:] == 0).all()   # every parameter in exactly one slice


def _shard_worker(rank, world, port, q):
    """Reduce-scatter + sliced update + in-place all-gather must leave every replica with exactly the
    parameters of all-reduce + replicated update."""
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from d3gs_research_b200.trainer import clip_fields, shard_layout, sharded_update
    n = 37
    total = 59 * n
    s, padded = shard_layout(total, world)
    offsets, off = {}, 0
    for name, per in zip(FLAT_ORDER, (3, 4, 3, 1, 3, 45)):
        offsets[name] = (off, per * n)
        off += per * n
    lrs = {name: 0.01 * (k + 1) for k, name in enumerate(FLAT_ORDER)}
    g0 = torch.Generator().manual_seed(7)
    param0 = torch.zeros(padded)
    param0[:total] = torch.randn(total, generator=g0)

    def adam(p, g, m, v, lr, t):
        m.mul_(0.9).add_(g, alpha=0.1)
        v.mul_(0.999).addcmul_(g, g, value=0.001)
        p.addcdiv_(m / (1 - 0.9 ** t), (v / (1 - 0.999 ** t)).sqrt_().add_(1e-15), value=-lr)

    # replicated: all-reduce, every rank updates everything
    pr, mr, vr = param0.clone(), torch.zeros(padded), torch.zeros(padded)
    # sharded: moments exist for this rank's slice only
    ps, ms, vs, gs = param0.clone(), torch.zeros(s), torch.zeros(s), torch.zeros(s)
    for t in (1, 2, 3):
        grad = torch.zeros(padded)
        grad[:total] = torch.randn(total, generator=torch.Generator().manual_seed(100 * t + rank))
        full = grad.clone()
        dist.all_reduce(full)
        for name, (o, c) in offsets.items():
            adam(pr[o:o + c], full[o:o + c], mr[o:o + c], vr[o:o + c], lrs[name], t)

        def apply(lo, hi, grad_shard):
            for name, a, cnt in clip_fields(offsets, lo, hi):
                adam(ps[a:a + cnt], grad_shard[a - lo:a - lo + cnt], ms[a - lo:a - lo + cnt], vs[a - lo:a - lo + cnt],
                     lrs[name], t)
        sharded_update(grad, ps, gs, rank, None, apply)
    q.put((rank, bool(torch.equal(ps, pr)), float(ps[total:].abs().max()) if padded > total else 0.0))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_optimizer_equals_replicated_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_shard_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=180) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == [(0, True, 0.0), (1, True, 0.0)], got


def test_ply_roundtrip_and_point_cloud_init(tmp_path):
    from d3gs_research_b200.tools import (init_original_3dgs_model, load_3dgs_origin_model, points_to_gaussian_init_scale,
                                          save_3dgs_origin_model)
    n = 37
    g = torch.Generator().manual_seed(3)
    m = d3.GaussianModelOriginFused.from_tensors(torch.randn(n, 3, generator=g), torch.randn(n, 4, generator=g),
                                                 torch.randn(n, 3, generator=g), torch.randn(n, generator=g),
                                                 torch.randn(n, 3, generator=g), torch.randn(n, 15, 3, generator=g), device="cpu")
    path = str(tmp_path / "m.ply")
    save_3dgs_origin_model(m, path)
    head = open(path, "rb").read(400).decode("ascii", "replace")
    assert head.startswith("ply\nformat binary_little_endian 1.0\nelement vertex 37\nproperty float x\n")
    assert "property float f_rest_44" in open(path, "rb").read(4000).decode("ascii", "replace")
    for split in (True, False):
        r = load_3dgs_origin_model(path, fused=True, split=split, device="cpu")
        assert torch.equal(r.xyz, m.xyz) and torch.equal(r.quaternion_xyzw, m.quaternion_xyzw)
        assert torch.equal(r.scale, m.scale) and torch.equal(r.opacity, m.opacity) and r.cur_sh_degree == 3
        if split:
            assert torch.equal(r.color_sh_base, m.color_sh_base) and torch.equal(r.color_sh, m.color_sh)
        else:
            assert torch.equal(r.color_sh[:, 0], m.color_sh_base) and torch.equal(r.color_sh[:, 1:], m.color_sh)
    # the file layout is the Inria one: rot_0 is w, f_rest is channel-major
    from d3gs_research_b200.tools import _read_ply_vertices
    v = _read_ply_vertices(path)
    assert np.allclose(v["rot_0"], m.quaternion_xyzw[:, 3].numpy()) and np.allclose(v["f_rest_1"], m.color_sh[:, 1, 0].numpy())
    assert np.allclose(v["f_rest_15"], m.color_sh[:, 0, 1].numpy())
    # point-cloud initialisation needs the neighbour search of the CUDA library: no host fallback
    pts = np.stack(np.meshgrid(np.arange(4.0), np.arange(4.0), np.arange(4.0), indexing="ij"), -1).reshape(-1, 3) * 0.5
    with pytest.raises(RuntimeError, match="GPU"):
        points_to_gaussian_init_scale(torch.from_numpy(pts.astype(np.float32)))


def test_end_of_iteration_fires_like_the_reference_period_events():
    """train.py:68-74 registers up_sh (1000 // batch), update_gs (refine_every) and reset_opacity
    (reset_opacity_every); core/train.py:76-87 fires an event when (cur_step + 1) % interval == 0; the handlers'
    own conditions are train.py:299-320.  Batch size 4: SH degree up after iterations 250, 500, 750; refinement
    every 25 iterations strictly between 125 and 3750; opacity reset every 750 iterations before 3750."""
    from types import SimpleNamespace
    from d3gs_research_b200.strategy import GaussianStrategyOrigin
    from d3gs_research_b200.trainer import SplatTrainer
    tr = SplatTrainer.__new__(SplatTrainer)
    tr.batch_size = 4
    tr.model = SimpleNamespace(cur_sh_degree=0)
    tr.grad_model = SimpleNamespace(cur_sh_degree=0)
    calls = []
    tr.refine = lambda strategy, step, generator=None: calls.append(("refine", step))
    tr.reset_opacity = lambda strategy: calls.append(("reset", None))
    st = GaussianStrategyOrigin()
    st.rescale_steps_by_batch_size(4)
    assert (st.refine_every, st.refine_start_iter, st.refine_stop_iter, st.reset_opacity_every) == (25, 125, 3750, 750)
    fired = {}
    for cur in range(4000):
        ev = tr.end_of_iteration(cur, st)
        if ev:
            fired[cur + 1] = ev
    ups = [s for s, ev in fired.items() if "up_sh" in ev]
    assert ups == [250, 500, 750] and tr.model.cur_sh_degree == 3 and tr.grad_model.cur_sh_degree == 3
    refines = [s for s, ev in fired.items() if "update_gs" in ev]
    assert refines == list(range(150, 3750, 25)) and [c[1] for c in calls if c[0] == "refine"] == refines
    resets = [s for s, ev in fired.items() if "reset_opacity" in ev]
    assert resets == [750, 1500, 2250, 3000]
    assert fired[750] == ["up_sh", "update_gs", "reset_opacity"]      # the reference's registration order


def _count_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from d3gs_research_b200.trainer import check_same_count
    check_same_count(1000, torch.device("cpu"))                 # equal counts pass
    try:
        check_same_count(1000 + 4 * rank, torch.device("cpu"))  # rank 1 holds four more
        q.put((rank, "no error"))
    except RuntimeError as e:
        q.put((rank, "between 1000 and 1004" in str(e)))
    dist.barrier()
    dist.destroy_process_group()


def test_ranks_with_different_gaussian_counts_are_refused_gloo():
    """The host check before the first exchange: all ranks raise, with the range of counts in the message."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 33500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_count_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=180) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == [(0, True), (1, True)], got
