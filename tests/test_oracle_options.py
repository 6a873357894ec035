"""CPU checks of oracle restatements that the reference offers no fixture for: instance rendering and the
atomic-add count."""
import numpy as np

from oracle import oracle as O
from parity_utils import oracle_scene, small_scene


def _rigid_T(rng, angle, shift):
    """[4,3] in the cam2world_T layout: rows 0-2 the transposed rotation, row 3 the translation."""
    axis = rng.normal(size=3)
    axis /= np.linalg.norm(axis)
    a = rng.uniform(-angle, angle)
    K = np.array([[0, -axis[2], axis[1]], [axis[2], 0, -axis[0]], [-axis[1], axis[0], 0]])
    R = np.eye(3) + np.sin(a) * K + (1 - np.cos(a)) * (K @ K)
    return np.concatenate([R.T, rng.uniform(-shift, shift, size=(1, 3))], axis=0).astype(np.float32)


def test_instance_rendering_equals_gaussians_moved_into_the_world_frame():
    """render.py:346-354: cam2instance = inverse(instance2world) @ cam2world.  Rendering Gaussians that live in an
    object's frame must put them where the same Gaussians, moved into the world frame by the object's transform
    (x_w = R x + t), land; identity transforms and Gaussians of no instance change nothing."""
    sc = small_scene(n=3000, width=200, height=136, sh_degree=0, seed=31, views=1)
    rng = np.random.default_rng(8)
    n = sc["cfg"].n
    cfg = O.OpConfig(width=200, height=136, sh_degree=0, early_filter=0)
    plain = O.preprocess_fwd(cfg, oracle_scene(sc))
    T = _rigid_T(rng, 0.25, 0.3)[None, None]                     # one frame, one instance
    osc = oracle_scene(sc)
    osc.instance_id, osc.instance2world_T, osc.frame_ids = np.zeros(n, np.int32), T, np.zeros(1, np.int32)
    inst = O.preprocess_fwd(cfg, osc)
    R, t = T[0, 0, :3].T.astype(np.float64), T[0, 0, 3].astype(np.float64)
    moved = oracle_scene(sc)
    moved.xyz = (moved.xyz.astype(np.float64) @ R.T + t).astype(np.float32)
    world = O.preprocess_fwd(cfg, moved)
    vis = (inst["radii"] > 0) & (world["radii"] > 0)
    assert vis.sum() > 0.95 * (inst["radii"] > 0).sum() > 1000
    assert np.abs(inst["uvs"][vis] - world["uvs"][vis]).max() < 1e-3            # pixels
    assert np.abs(inst["depths"][vis] - world["depths"][vis]).max() < 1e-4
    assert (inst["radii"] != plain["radii"]).sum() > 100                       # the transform did move them
    # identity transform, and instance id -1, are the plain render bit for bit
    osc.instance2world_T = np.concatenate([np.eye(3), np.zeros((1, 3))]).astype(np.float32)[None, None]
    same = O.preprocess_fwd(cfg, osc)
    osc.instance2world_T, osc.instance_id = T, np.full(n, -1, np.int32)
    none = O.preprocess_fwd(cfg, osc)
    for k in ("radii", "tiles_touched", "uvs", "depths", "conic_opacity", "rgb"):
        np.testing.assert_array_equal(same[k], plain[k], err_msg=k)
        np.testing.assert_array_equal(none[k], plain[k], err_msg=k)


def test_atomic_add_count_by_reducing_block():
    """measure_atomic_add_count (config_def.py:134): one count per (reducing lane set, splat) with a valid pixel.
    Larger lane sets merge counts: a tile <= a warp of the reference (16 x 2 pixels) <= 4 x 2 pixels <= single
    pixels; counting by single pixels is the number of valid (pixel, splat) pairs."""
    sc = small_scene(n=3000, width=160, height=112, sh_degree=1, seed=4)
    osc = oracle_scene(sc)
    cfg = O.OpConfig(width=160, height=112, sh_degree=1, early_filter=4)
    res = O.forward(cfg, osc)
    counts = {b: O.count_accumulations(cfg, 1, res.ranges, res.sorted_ids, res.prep, res.n_contrib, block_wh=b)
              for b in ((16, 16), (16, 2), (4, 2), (1, 1))}
    groups = [counts[b][0] for b in ((16, 16), (16, 2), (4, 2), (1, 1))]
    assert groups == sorted(groups) and groups[0] > 0
    pixels = {c[1] for c in counts.values()}
    assert len(pixels) == 1 and counts[(1, 1)][0] == counts[(1, 1)][1]
    assert groups[0] <= res.num_rendered          # at most one count per (tile, splat) pair
