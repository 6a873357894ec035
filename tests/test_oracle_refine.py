"""The oracle's refine_gs (numpy) against a second, independent restatement written with torch boolean-mask
indexing in the order of the reference's own code (d3sim/algos/d3gs/origin/strategy.py:242-347): duplicate /
split index lists, [dupli | split | split] concatenation, pruning of originals and of new Gaussians, optimizer
gather + zero of the new range (strategy.py:131-178).  The reference itself cannot be imported here (it needs
pccm/cumm), so this pins the bookkeeping of the oracle, not the reference: parity for this function stays
"unpinned" in the sense of the oracle header."""
import numpy as np
import torch

from oracle import oracle as O


def _torch_refine(rc, t, mom, state, scene_scale, step, normals):
    exp = lambda a: torch.from_numpy(O._act_exp(a.numpy()))
    log = lambda a: torch.from_numpy(O._act_log(a.numpy()))
    sig = lambda a: 1.0 / (1.0 + exp(-a))
    n = t["xyz"].shape[0]
    scales, opacity = exp(t["scale"]), sig(t["opacity"])
    grad_high = (state["duv_ndc_length"] / torch.clamp(state["count"], min=1.0)) >= rc.grow_grad2d
    smax = scales.max(dim=1).values
    is_small = smax <= np.float32(rc.grow_scale3d) * np.float32(scene_scale)
    is_dupli = grad_high & is_small
    prune = opacity < rc.prune_opacity_thresh
    if step > rc.reset_opacity_every:
        prune = prune | (smax > np.float32(rc.prune_scale3d) * np.float32(scene_scale))
    is_split = grad_high & ~is_small
    origin_prune = prune | is_split
    dup_inds, split_inds = torch.nonzero(is_dupli).view(-1), torch.nonzero(is_split).view(-1)
    n_dup, n_split = len(dup_inds), len(split_inds)
    new_inds = torch.cat([dup_inds, split_inds, split_inds])
    new = {k: v[new_inds].clone() for k, v in t.items()}
    new_prune = torch.empty(n_dup + 2 * n_split, dtype=torch.bool)
    new_prune[:n_dup] = origin_prune[is_dupli]
    q = new["quat"][n_dup:]
    q = q / torch.sqrt(((q[:, 0] * q[:, 0] + q[:, 1] * q[:, 1]) + q[:, 2] * q[:, 2]) + q[:, 3] * q[:, 3])[:, None]
    x, y, z, w = q.unbind(1)
    R = torch.stack([torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y)], 1),
                     torch.stack([2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x)], 1),
                     torch.stack([2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)], 1)], 1)
    s_act = exp(new["scale"][n_dup:])
    v = normals * s_act
    new_xyz = ((R[:, :, 0] * v[:, 0:1] + R[:, :, 1] * v[:, 1:2]) + R[:, :, 2] * v[:, 2:3]) + new["xyz"][n_dup:]
    new_scaling = s_act / 1.6
    child_prune = sig(new["opacity"][n_dup:]) < rc.prune_opacity_thresh
    if step > rc.reset_opacity_every:
        child_prune = child_prune | (new_scaling.max(dim=1).values > np.float32(rc.prune_scale3d) * np.float32(scene_scale))
    new["xyz"][n_dup:] = new_xyz
    new["scale"][n_dup:] = log(new_scaling)
    new_prune[n_dup:] = child_prune
    res = {k: torch.cat([t[k][~origin_prune], new[k][~new_prune]]) for k in t}
    inds = torch.cat([torch.arange(n)[~origin_prune], new_inds[~new_prune]])
    n_keep = int((~origin_prune).sum())
    res_mom = {}
    for k, (m, vv) in mom.items():
        m2, v2 = m[inds].clone(), vv[inds].clone()
        m2[n_keep:].zero_()
        v2[n_keep:].zero_()
        res_mom[k] = (m2, v2)
    return res, res_mom, inds


def test_oracle_refine_matches_torch_mask_indexing():
    n, step, scene_scale = 3001, 3500, 3.0
    g = torch.Generator().manual_seed(0)
    t = {"xyz": torch.randn(n, 3, generator=g), "quat": torch.randn(n, 4, generator=g),
         "scale": torch.randn(n, 3, generator=g) * 0.9 - 3.6, "opacity": torch.randn(n, generator=g) * 3.0 - 1.0,
         "sh_base": torch.randn(n, 3, generator=g), "sh_rest": torch.randn(n, 15, 3, generator=g)}
    state = {"duv_ndc_length": torch.rand(n, generator=g) * 0.01, "count": torch.randint(0, 20, (n,), generator=g).float(),
             "max_radii": torch.rand(n, generator=g) * 0.2}
    mom = {k: (torch.randn(v.shape, generator=g), torch.rand(v.shape, generator=g)) for k, v in t.items()}
    rc = O.RefineConfig()
    np_t = {k: v.numpy().copy() for k, v in t.items()}
    np_s = {k: v.numpy().copy() for k, v in state.items()}
    _, split, _ = O.refine_masks(rc, np_t, np_s, scene_scale, step)
    normals = torch.randn(2 * int(split.sum()), 3, generator=g)
    model, moments, inds, n_dup, n_split = O.refine_gs(rc, np_t, {k: (m.numpy().copy(), v.numpy().copy()) for k, (m, v) in mom.items()},
                                                       np_s, scene_scale, step, normals.numpy())
    ref, ref_mom, ref_inds = _torch_refine(rc, t, mom, state, scene_scale, step, normals)
    assert n_dup > 10 and n_split > 10 and len(inds) != n
    np.testing.assert_array_equal(inds, ref_inds.numpy())
    for k in t:
        np.testing.assert_allclose(model[k], ref[k].numpy(), rtol=1e-6, atol=1e-6, err_msg=k)
        np.testing.assert_array_equal(moments[k][0], ref_mom[k][0].numpy())
        np.testing.assert_array_equal(moments[k][1], ref_mom[k][1].numpy())


def test_oracle_reset_opacity_clamps_to_threshold():
    o = np.array([-9.0, -4.6, 0.0, 5.0], np.float32)
    r = O.reset_opacity(o, 0.01)
    lim = np.log(0.01 / 0.99)
    assert abs(r[0] - (-9.0)) < 1e-5 and np.all(r[1:] <= lim + 1e-5) and abs(r[3] - lim) < 1e-5
