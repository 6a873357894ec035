"""ctypes driver for the CPU oracle (oracle/d3gs_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of bench.py.  The product package never imports it.

All functions take and return numpy arrays.  ``Scene`` bundles the Gaussian parameters in the
reference's layout (d3sim/algos/d3gs/origin/model.py:36-44) and ``run_iteration`` chains the
stages in the order of the reference's training step (d3sim/algos/d3gs/train.py:162-217).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import time
from dataclasses import dataclass, field, replace as dataclass_replace

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libd3gs_oracle.so")
_SRC = os.path.join(_HERE, "d3gs_oracle.cpp")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with g++ (OpenMP when the compiler has it)."""
    if not force and os.path.exists(_SO) and os.path.getmtime(_SO) >= os.path.getmtime(_SRC):
        return _SO
    os.makedirs(os.path.dirname(_SO), exist_ok=True)
    base = ["-O2", "-fPIC", "-shared", "-std=c++17", "-ffp-contract=off", "-fno-fast-math",
            "-Wno-unknown-pragmas", "-o", _SO, _SRC]
    errs = []
    for cxx in ("/usr/bin/g++", "g++"):
        for omp in (["-fopenmp"], []):
            r = subprocess.run([cxx] + omp + base, capture_output=True, text=True)
            if r.returncode == 0:
                return _SO
            errs.append(r.stderr[-400:])
    raise RuntimeError("could not build the CPU oracle:\n" + "\n".join(errs))


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.oracle_scan_inclusive.restype = ctypes.c_int64
        _lib.oracle_num_threads.restype = ctypes.c_int
        for f in ("oracle_expf", "oracle_logf", "oracle_exp_blend"):
            getattr(_lib, f).restype = ctypes.c_float
            getattr(_lib, f).argtypes = [ctypes.c_float]
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int | None = None) -> int:
    """Use ``n`` OpenMP threads from now on (default: every core this process may run on), whatever
    OMP_NUM_THREADS says -- torch.distributed.run exports OMP_NUM_THREADS=1 to its workers."""
    if n is None:
        try:
            n = len(os.sched_getaffinity(0))
        except AttributeError:
            n = os.cpu_count() or 1
    lib().oracle_set_num_threads(ctypes.c_int(int(n)))
    return num_threads()


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(ctypes.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


@dataclass
class OpConfig:
    """Scalar options of the splat operator (defaults: config_def.py:77-161)."""
    width: int = 256
    height: int = 256
    tile: int = 16
    near: float = 0.2
    far: float = 10000.0
    eps: float = 1e-6
    eigen_eps: float = 0.1
    clamp_factor: float = 1.3
    sigma: float = 3.0
    lowpass: float = 0.3
    alpha_eps: float = 1.0 / 255.0
    t_eps: float = 0.0001
    early_filter: int = 0          # EarlyFilterAlgo value
    sh_degree: int = 3
    training: bool = True
    scale_global: float = 1.0
    clamp_mask_reference_order: bool = True
    fused_activations: bool = True
    key_shift: int = 32            # 18: enable_32bit_sort (render.py:737, 767-770)
    depth_prec: float = 0.001      # depth_32bit_prec
    anti_aliasing: bool = False    # enable_anti_aliasing (render.py:391-406, 449-462)
    inv_depth: bool = False        # render_inv_depth: the depth array holds 1/z (render.py:582)

    def vec(self) -> np.ndarray:
        return np.array([self.width, self.height, self.tile, self.near, self.far, self.eps, self.eigen_eps,
                         self.clamp_factor, self.sigma, self.lowpass, self.alpha_eps, self.t_eps,
                         self.early_filter, self.sh_degree, int(self.training), self.scale_global,
                         int(self.clamp_mask_reference_order), int(self.fused_activations), self.key_shift,
                         self.depth_prec, int(self.anti_aliasing), int(self.inv_depth), 0, 0], dtype=np.float32)

    @property
    def tiles_xy(self):
        return (self.width + self.tile - 1) // self.tile, (self.height + self.tile - 1) // self.tile


@dataclass
class Scene:
    xyz: np.ndarray
    quat: np.ndarray
    scale: np.ndarray
    opacity: np.ndarray
    sh_base: np.ndarray
    sh_rest: np.ndarray          # [N,15,3]
    cams: np.ndarray             # [B,16]
    # instance rendering (render.py:207-220, 346-354); all three or none
    instance_id: np.ndarray | None = None          # [N] int32, < 0 = world Gaussian
    instance2world_T: np.ndarray | None = None     # [num_frame, num_instance, 4, 3]
    frame_ids: np.ndarray | None = None            # [B] int32

    @property
    def n(self):
        return self.xyz.shape[0]

    @property
    def b(self):
        return self.cams.shape[0]


def bit_length(n: int) -> int:
    """DeviceSort.get_higher_msb (csrc/devsort.py:129-149)."""
    return int(n).bit_length()


class _instances:
    """Switches the C library's instance context on for the calls inside the block."""

    def __init__(self, sc: Scene):
        self.sc = sc

    def __enter__(self):
        sc = self.sc
        if sc.instance_id is not None:
            self.keep = (np.ascontiguousarray(sc.instance_id, np.int32), _f32(sc.instance2world_T),
                         np.ascontiguousarray(sc.frame_ids, np.int32))
            assert self.keep[1].ndim == 4 and self.keep[1].shape[2:] == (4, 3) and self.keep[2].size == sc.b
            lib().oracle_set_instances(_p(self.keep[0]), _p(self.keep[1]), ctypes.c_int(self.keep[1].shape[1]),
                                       _p(self.keep[2]), ctypes.c_int(sc.b))

    def __exit__(self, *exc):
        lib().oracle_set_instances(None, None, ctypes.c_int(0), None, ctypes.c_int(0))


def preprocess_fwd(cfg: OpConfig, sc: Scene, mask=None):
    with _instances(sc):
        return _preprocess_fwd(cfg, sc, mask)


def _preprocess_fwd(cfg: OpConfig, sc: Scene, mask=None):
    BN = sc.b * sc.n
    out = dict(
        tiles_touched=np.zeros(BN, np.int32), radii=np.zeros(BN, np.int32),
        depths=np.zeros(BN, np.float32), uvs=np.zeros((BN, 2), np.float32),
        conic_opacity=np.zeros((BN, 4), np.float32), rgb=np.zeros((BN, 3), np.float32),
        cov2d=np.zeros((BN, 3), np.float32), ne0=np.zeros(BN, np.uint8))
    cv = cfg.vec()
    lib().oracle_preprocess_fwd(_p(cv), ctypes.c_int(sc.b), ctypes.c_int(sc.n), _p(sc.cams), _p(sc.xyz), _p(sc.quat),
                                _p(sc.scale), _p(sc.opacity), _p(sc.sh_base), _p(sc.sh_rest), _p(mask),
                                _p(out["tiles_touched"]), _p(out["radii"]), _p(out["depths"]), _p(out["uvs"]),
                                _p(out["conic_opacity"]), _p(out["rgb"]), _p(out["cov2d"]), _p(out["ne0"]))
    return out


def scan_inclusive(tiles_touched):
    out = np.empty_like(tiles_touched)
    total = lib().oracle_scan_inclusive(ctypes.c_int64(tiles_touched.size), _p(tiles_touched), _p(out))
    return out, int(total)


def duplicate_keys(cfg: OpConfig, b: int, n: int, scan, total, prep):
    keys = np.zeros(total, np.uint64)
    vals = np.zeros(total, np.int32)
    cv = cfg.vec()
    lib().oracle_duplicate_keys(_p(cv), ctypes.c_int(b), ctypes.c_int(n), _p(scan), _p(prep["radii"]),
                                _p(prep["depths"]), _p(prep["uvs"]), _p(prep["conic_opacity"]), _p(keys), _p(vals))
    return keys, vals


def sort_pairs(keys, vals, end_bit: int):
    ko = np.empty_like(keys)
    vo = np.empty_like(vals)
    lib().oracle_sort_pairs(ctypes.c_int64(keys.size), ctypes.c_int(end_bit), _p(keys), _p(vals), _p(ko), _p(vo))
    return ko, vo


def tile_ranges(sorted_keys, num_tiles: int, shift: int = 32):
    r = np.zeros((num_tiles, 2), np.int32)
    lib().oracle_tile_ranges(ctypes.c_int64(sorted_keys.size), _p(sorted_keys), _p(r), ctypes.c_int(shift))
    return r


def raster_fwd(cfg: OpConfig, b: int, ranges, sorted_ids, prep, bg=None):
    H, W = cfg.height, cfg.width
    color = np.zeros((b, H, W, 3), np.float32)
    T = np.zeros((b, H, W), np.float32)
    nc = np.zeros((b, H, W), np.int32)
    bg = _f32(np.zeros(3) if bg is None else bg)
    cv = cfg.vec()
    lib().oracle_raster_fwd(_p(cv), ctypes.c_int(b), _p(ranges), _p(sorted_ids), _p(prep["uvs"]),
                            _p(prep["conic_opacity"]), _p(prep["rgb"]), _p(bg), _p(color), _p(T), _p(nc))
    return color, T, nc


def raster_bwd(cfg: OpConfig, b: int, bn: int, ranges, sorted_ids, prep, color, T, nc, drgb, dT=None):
    duv = np.zeros((bn, 2), np.float32)
    dconic = np.zeros((bn, 3), np.float32)
    dop = np.zeros(bn, np.float32)
    dcol = np.zeros((bn, 3), np.float32)
    cv = cfg.vec()
    drgb = _f32(drgb)
    dT = None if dT is None else _f32(dT)
    lib().oracle_raster_bwd(_p(cv), ctypes.c_int(b), ctypes.c_int64(bn), _p(ranges), _p(sorted_ids), _p(prep["uvs"]),
                            _p(prep["conic_opacity"]), _p(prep["rgb"]), _p(color), _p(T), _p(nc), _p(drgb), _p(dT),
                            _p(duv), _p(dconic), _p(dop), _p(dcol))
    return dict(duv=duv, dconic=dconic, dopacity=dop, dcolor=dcol)


def simple_knn(points, k: int):
    """[n, k] float32: distances to the k nearest other points, ascending (ops.py:14-183)."""
    pts = _f32(points)
    out = np.zeros((pts.shape[0], k), np.float32)
    lib().oracle_simple_knn(_p(pts), ctypes.c_int64(pts.shape[1]), ctypes.c_int64(pts.shape[0]), ctypes.c_int(k), _p(out))
    return out


def count_accumulations(cfg: OpConfig, b: int, ranges, sorted_ids, prep, nc, block_wh=(16, 2)):
    """(groups, pixels): (pixel block, splat) pairs with a valid pixel -- what measure_atomic_add_count counts for a
    kernel whose lanes over ``block_wh`` pixels reduce before one group of global adds -- and valid (pixel, splat)
    pairs.  (16, 2) is a warp of the reference's 16 x 16 thread block."""
    out = np.zeros(2, np.int64)
    cv = cfg.vec()
    lib().oracle_count_accumulations(_p(cv), ctypes.c_int(b), _p(ranges), _p(sorted_ids), _p(prep["uvs"]),
                                     _p(prep["conic_opacity"]), _p(nc), ctypes.c_int(block_wh[0]),
                                     ctypes.c_int(block_wh[1]), _p(out))
    return int(out[0]), int(out[1])


def preprocess_bwd(cfg: OpConfig, sc: Scene, prep, rg, dz=None):
    with _instances(sc):
        return _preprocess_bwd(cfg, sc, prep, rg, dz)


def _preprocess_bwd(cfg: OpConfig, sc: Scene, prep, rg, dz=None):
    n = sc.n
    dz = None if dz is None else _f32(dz)   # [B*N]: d loss / d depth value of every splat (render_depth)
    g = dict(xyz=np.zeros((n, 3), np.float32), quat=np.zeros((n, 4), np.float32),
             scale=np.zeros((n, 3), np.float32), opacity=np.zeros(n, np.float32),
             sh_base=np.zeros((n, 3), np.float32), sh_rest=np.zeros((n, 15, 3), np.float32))
    cv = cfg.vec()
    lib().oracle_preprocess_bwd(_p(cv), ctypes.c_int(sc.b), ctypes.c_int(n), _p(sc.cams), _p(sc.xyz), _p(sc.quat),
                                _p(sc.scale), _p(sc.opacity), _p(sc.sh_rest), _p(prep["radii"]), _p(prep["cov2d"]),
                                _p(prep["ne0"]), _p(rg["duv"]), _p(rg["dconic"]), _p(rg["dopacity"]),
                                _p(rg["dcolor"]), _p(dz), _p(g["xyz"]), _p(g["quat"]),
                                _p(g["scale"]), _p(g["opacity"]),
                                _p(g["sh_base"]), _p(g["sh_rest"]))
    return g


def l1_dssim(x_nhwc, y_nchw, lambda_dssim: float = 0.2, want_grad: bool = True):
    b, h, w, _ = x_nhwc.shape
    out = np.zeros(3, np.float32)
    dx = np.zeros_like(x_nhwc) if want_grad else None
    lib().oracle_l1_dssim(ctypes.c_int(b), ctypes.c_int(h), ctypes.c_int(w), ctypes.c_float(lambda_dssim),
                          _p(x_nhwc), _p(y_nchw), _p(out), _p(dx))
    return out, dx


def adam(p, g, m, v, lr, beta1, beta2, eps, step):
    lib().oracle_adam(ctypes.c_int64(p.size), _p(p), _p(g), _p(m), _p(v), ctypes.c_float(lr), ctypes.c_float(beta1),
                      ctypes.c_float(beta2), ctypes.c_float(eps), ctypes.c_int(step))


def densify_stats(b, n, width, height, need_max_radii, duv, radii, duv_ndc_length, count, max_radii):
    lib().oracle_densify_stats(ctypes.c_int(b), ctypes.c_int(n), ctypes.c_int(width), ctypes.c_int(height),
                               ctypes.c_int(int(need_max_radii)), _p(duv), _p(radii), _p(duv_ndc_length),
                               _p(count), _p(max_radii))


# Per-tensor Adam learning rates of the reference's optimizer factory (tools.py:146-173).
ADAM_LRS = dict(xyz=1.6e-4, sh_base=2.5e-3, sh_rest=2.5e-3 / 20.0, opacity=0.05, scale=5e-3, quat=1e-3)


@dataclass
class IterationResult:
    prep: dict
    scan: np.ndarray
    num_rendered: int
    keys: np.ndarray
    vals: np.ndarray
    sorted_keys: np.ndarray
    sorted_ids: np.ndarray
    ranges: np.ndarray
    color: np.ndarray
    T: np.ndarray
    n_contrib: np.ndarray
    depth: np.ndarray | None = None          # render_depth: [B,H,W]
    custom_features: np.ndarray | None = None   # [B*N,F] input
    custom_image: np.ndarray | None = None      # [B,H,W,F] blend
    loss: np.ndarray | None = None
    drgb: np.ndarray | None = None
    raster_grads: dict | None = None
    grads: dict | None = None
    timings: dict = field(default_factory=dict)


def _aux_prep(prep, values3):
    """Depth and custom features are blended like a colour (render.py:1824, 1920-1923: accum += weight * value):
    a copy of the per-Gaussian context whose colour is the given [B*N,3] values."""
    p2 = dict(prep)
    p2["rgb"] = _f32(values3)
    return p2


def _depth_values(prep):
    v = np.zeros_like(prep["rgb"])
    v[:, 0] = prep["depths"]
    return v


def _feature_groups(feat):
    """[B*N,F] -> list of [B*N,3] (zero padded)."""
    feat = _f32(feat)
    pad = (-feat.shape[1]) % 3
    if pad:
        feat = np.concatenate([feat, np.zeros((feat.shape[0], pad), np.float32)], axis=1)
    return [np.ascontiguousarray(feat[:, k:k + 3]) for k in range(0, feat.shape[1], 3)]


def raster_aux(cfg: OpConfig, b: int, ranges, sorted_ids, prep, values3):
    """Un-composited, un-clamped blend of three per-Gaussian channels."""
    acc, _, _ = raster_fwd(dataclass_replace(cfg, training=True), b, ranges, sorted_ids, _aux_prep(prep, values3))
    return acc


def raster_depth(cfg: OpConfig, b: int, ranges, sorted_ids, prep, T):
    """render.py:2244-2255: sum_i w_i depth_i in training, divided by (1e-10 + 1 - T) at inference."""
    acc = np.ascontiguousarray(raster_aux(cfg, b, ranges, sorted_ids, prep, _depth_values(prep))[..., 0])
    if cfg.training:
        return acc
    with np.errstate(invalid="ignore", divide="ignore"):   # in float32 1e-10 + 1 - T is 0 where nothing was blended: 0/0, as in the reference
        return acc / (np.float32(1e-10) + np.float32(1.0) - T)


def forward(cfg: OpConfig, sc: Scene, timings: dict | None = None, render_depth: bool = False,
            custom_features=None) -> IterationResult:
    """preprocess -> scan -> keys -> sort -> ranges -> raster (render.py:169-1015)."""
    tm = {} if timings is None else timings
    tx, ty = cfg.tiles_xy
    t0 = time.perf_counter()
    prep = preprocess_fwd(cfg, sc)
    t1 = time.perf_counter()
    scan, total = scan_inclusive(prep["tiles_touched"])
    keys, vals = duplicate_keys(cfg, sc.b, sc.n, scan, total, prep)
    t2 = time.perf_counter()
    end_bit = 32 if cfg.key_shift == 18 else 32 + bit_length(sc.b * tx * ty)   # render.py:851-854
    sk, sv = sort_pairs(keys, vals, end_bit)
    t3 = time.perf_counter()
    ranges = tile_ranges(sk, sc.b * tx * ty, cfg.key_shift)
    t4 = time.perf_counter()
    color, T, nc = raster_fwd(cfg, sc.b, ranges, sv, prep)
    t5 = time.perf_counter()
    tm.update(preprocess=t1 - t0, scan_keys=t2 - t1, sort=t3 - t2, ranges=t4 - t3, raster_fwd=t5 - t4)
    depth = raster_depth(cfg, sc.b, ranges, sv, prep, T) if render_depth else None
    feat_img = None
    if custom_features is not None:   # [B*N,F] -> [B,H,W,F] (render.py:241-245, 2268-2270)
        nf = custom_features.shape[1]
        feat_img = np.concatenate([raster_aux(cfg, sc.b, ranges, sv, prep, v) for v in _feature_groups(custom_features)],
                                  axis=-1)[..., :nf]
        feat_img = np.ascontiguousarray(feat_img)
    res = IterationResult(prep, scan, total, keys, vals, sk, sv, ranges, color, T, nc, depth=depth, timings=tm)
    res.custom_features, res.custom_image = custom_features, feat_img
    return res


def backward(cfg: OpConfig, sc: Scene, res: IterationResult, drgb, dT=None, ddepth=None, dcustom=None) -> IterationResult:
    """raster backward -> preprocess backward (render.py:2779-3374).  ddepth [B,H,W] / dcustom [B,H,W,F]: gradients
    of the rendered depth (training output, the un-normalised sum) and of the blended custom features; the raster
    backward is linear in the image gradients, so every extra channel group is one more pass with its values as
    the colour (render.py:1948-1971)."""
    t0 = time.perf_counter()
    res.drgb = _f32(drgb)
    bn = sc.b * sc.n
    res.raster_grads = raster_bwd(cfg, sc.b, bn, res.ranges, res.sorted_ids, res.prep, res.color, res.T,
                                  res.n_contrib, res.drgb, dT)

    def aux_pass(values3, blend3, dimg3):
        rg2 = raster_bwd(cfg, sc.b, bn, res.ranges, res.sorted_ids, _aux_prep(res.prep, values3), _f32(blend3), res.T,
                         res.n_contrib, _f32(dimg3), None)
        for k in ("duv", "dconic", "dopacity"):
            res.raster_grads[k] = res.raster_grads[k] + rg2[k]
        return rg2["dcolor"]

    dz = None
    if ddepth is not None:
        assert res.depth is not None and cfg.training
        col = np.zeros(res.color.shape, np.float32)
        col[..., 0] = res.depth
        dcol = np.zeros(res.color.shape, np.float32)
        dcol[..., 0] = ddepth
        dz = np.ascontiguousarray(aux_pass(_depth_values(res.prep), col, dcol)[:, 0])
        res.raster_grads["dz"] = dz
    if dcustom is not None:
        nf = res.custom_features.shape[1]
        pad = (-nf) % 3
        img = np.concatenate([res.custom_image, np.zeros(res.custom_image.shape[:3] + (pad,), np.float32)], axis=-1)
        dimg = np.concatenate([_f32(dcustom), np.zeros(res.custom_image.shape[:3] + (pad,), np.float32)], axis=-1)
        parts = [aux_pass(v, img[..., 3 * k:3 * k + 3], dimg[..., 3 * k:3 * k + 3])
                 for k, v in enumerate(_feature_groups(res.custom_features))]
        res.raster_grads["dcustom"] = np.ascontiguousarray(np.concatenate(parts, axis=1)[:, :nf])
    t1 = time.perf_counter()
    res.grads = preprocess_bwd(cfg, sc, res.prep, res.raster_grads, dz)
    t2 = time.perf_counter()
    res.timings.update(raster_bwd=t1 - t0, preprocess_bwd=t2 - t1)
    return res


def run_iteration(cfg: OpConfig, sc: Scene, target_nchw, lambda_dssim: float, adam_state: dict | None = None,
                  step: int = 1, betas=(0.9, 0.999), eps: float = 1e-15, lrs: dict | None = None,
                  stats: dict | None = None) -> IterationResult:
    """One full training iteration on the CPU: forward, loss, backward, Adam, densify statistics."""
    res = forward(cfg, sc)
    t0 = time.perf_counter()
    loss, drgb = l1_dssim(res.color, _f32(target_nchw), lambda_dssim)
    res.loss = loss
    res.timings["loss"] = time.perf_counter() - t0
    backward(cfg, sc, res, drgb)
    if adam_state is not None:
        t0 = time.perf_counter()
        lrs = ADAM_LRS if lrs is None else lrs
        for name in ("xyz", "quat", "scale", "opacity", "sh_base", "sh_rest"):
            p = getattr(sc, name)
            adam(p, res.grads[name], adam_state[name][0], adam_state[name][1], lrs[name], betas[0], betas[1], eps, step)
        res.timings["adam"] = time.perf_counter() - t0
    if stats is not None:
        duv = res.raster_grads["duv"]
        densify_stats(sc.b, sc.n, cfg.width, cfg.height, stats.get("need_max_radii", False), duv, res.prep["radii"],
                      stats["duv_ndc_length"], stats["count"], stats["max_radii"])
    return res


def sh_eval(deg: int, dirs, base, rest):
    """SH colour INCLUDING the +0.5 offset, no clamp (gs3d.py:151-201). rest: [n,15,3]."""
    n = dirs.shape[0]
    out = np.zeros((n, 3), np.float32)
    lib().oracle_sh_eval(ctypes.c_int(deg), ctypes.c_int(n), _p(_f32(dirs)), _p(_f32(base)), _p(_f32(rest)), _p(out))
    return out


def cov3d(quat_xyzw, scale_act):
    n = quat_xyzw.shape[0]
    cov6 = np.zeros((n, 6), np.float32)
    rot = np.zeros((n, 3, 3), np.float32)
    lib().oracle_cov3d(ctypes.c_int(n), _p(_f32(quat_xyzw)), _p(_f32(scale_act)), _p(cov6), _p(rot))
    return cov6, rot


# ---- densification / pruning / opacity reset (test infrastructure like the rest of this file) ----------------
def _act_exp(a):
    f = lib().oracle_expf
    return np.array([f(float(x)) for x in np.asarray(a, np.float32).ravel()], np.float32).reshape(np.shape(a))


def _act_log(a):
    f = lib().oracle_logf
    return np.array([f(float(x)) for x in np.asarray(a, np.float32).ravel()], np.float32).reshape(np.shape(a))


def _sigmoid(a):
    one = np.float32(1.0)
    return (one / (one + _act_exp(-np.asarray(a, np.float32)))).astype(np.float32)


@dataclass
class RefineConfig:
    """Thresholds of GaussianStrategyOrigin (d3sim/algos/d3gs/origin/strategy.py:21-35)."""
    reset_opacity_thresh: float = 0.01
    prune_opacity_thresh: float = 0.005
    grow_grad2d: float = 0.0002
    grow_scale3d: float = 0.01
    grow_scale2d: float = 0.05
    prune_scale3d: float = 0.1
    prune_scale2d: float = 0.15
    refine_scale2d_stop_iter: int = 0
    reset_opacity_every: int = 3000


def refine_masks(rc: RefineConfig, model: dict, state: dict, scene_scale: float, step: int):
    """The mask kernel of refine_gs (origin/strategy.py:195-241) on a fused-activation model (raw scale and
    opacity).  Returns (should_dupli, should_split, origin_prune)."""
    f32 = np.float32
    scale = _act_exp(model["scale"])
    opac = _sigmoid(model["opacity"])
    cnt = state["count"].astype(f32)
    grad_high = (state["duv_ndc_length"].astype(f32) / np.maximum(cnt, f32(1.0))) >= f32(rc.grow_grad2d)
    smax = scale.max(axis=1)
    small = smax <= f32(rc.grow_scale3d) * f32(scene_scale)
    dup = grad_high & small
    large = ~small
    prune = opac < f32(rc.prune_opacity_thresh)
    if step > rc.reset_opacity_every:
        prune = prune | (smax > f32(rc.prune_scale3d) * f32(scene_scale))
    if step < rc.refine_scale2d_stop_iter:
        large = large | (state["max_radii"] > f32(rc.grow_scale2d))
        prune = prune | (state["max_radii"] > f32(rc.prune_scale2d))
    split = grad_high & large
    return dup, split, prune | split


def refine_gs(rc: RefineConfig, model: dict, moments: dict, state: dict, scene_scale: float, step: int, normals):
    """refine_gs (origin/strategy.py:159-363) + select_gs_optimizer_by_mask / zero_optimizer_by_range
    (strategy.py:131-178) with numpy.  ``model``: name -> array (raw parameters, first axis N); ``moments``: name ->
    (exp_avg, exp_avg_sq); ``normals``: [2 * n_split, 3] standard normal draws (torch.randn in the reference).
    Returns (new_model, new_moments, res_inds, n_dupli, n_split)."""
    f32 = np.float32
    dup, split, origin_prune = refine_masks(rc, model, state, scene_scale, step)
    n = model["xyz"].shape[0]
    dup_inds, split_inds = np.nonzero(dup)[0], np.nonzero(split)[0]
    n_dup, n_split = len(dup_inds), len(split_inds)
    assert normals.shape == (2 * n_split, 3)
    new_inds = np.concatenate([dup_inds, split_inds, split_inds])
    new = {k: v[new_inds].copy() for k, v in model.items()}
    new_prune = np.zeros(n_dup + 2 * n_split, dtype=bool)
    new_prune[:n_dup] = origin_prune[dup_inds]
    # split children (origin/strategy.py:286-331)
    sl = slice(n_dup, None)
    q = new["quat"][sl].astype(f32)
    qn = np.sqrt(((q[:, 0] * q[:, 0] + q[:, 1] * q[:, 1]) + q[:, 2] * q[:, 2]) + q[:, 3] * q[:, 3]).astype(f32)
    q = (q / qn[:, None]).astype(f32)
    x, y, z, w = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
    two, one = f32(2.0), f32(1.0)
    R = np.empty((len(q), 3, 3), f32)
    R[:, 0, 0] = one - two * (y * y + z * z); R[:, 0, 1] = two * (x * y - w * z); R[:, 0, 2] = two * (x * z + w * y)
    R[:, 1, 0] = two * (x * y + w * z); R[:, 1, 1] = one - two * (x * x + z * z); R[:, 1, 2] = two * (y * z - w * x)
    R[:, 2, 0] = two * (x * z - w * y); R[:, 2, 1] = two * (y * z + w * x); R[:, 2, 2] = one - two * (x * x + y * y)
    s_act = _act_exp(new["scale"][sl])
    v = (normals.astype(f32) * s_act).astype(f32)
    new_xyz = (((R[:, :, 0] * v[:, 0:1] + R[:, :, 1] * v[:, 1:2]) + R[:, :, 2] * v[:, 2:3]) + new["xyz"][sl]).astype(f32)
    new_scaling = (s_act / f32(1.6)).astype(f32)
    child_prune = _sigmoid(new["opacity"][sl]) < f32(rc.prune_opacity_thresh)
    if step > rc.reset_opacity_every:
        child_prune = child_prune | (new_scaling.max(axis=1) > f32(rc.prune_scale3d) * f32(scene_scale))
    if step < rc.refine_scale2d_stop_iter:
        child_prune = child_prune | (state["max_radii"][new_inds[sl]] > f32(rc.prune_scale2d))
    new["xyz"][sl] = new_xyz
    new["scale"][sl] = _act_log(new_scaling)
    new_prune[sl] = child_prune
    keep_o, keep_n = ~origin_prune, ~new_prune
    res_model = {k: np.concatenate([model[k][keep_o], new[k][keep_n]]) for k in model}
    res_inds = np.concatenate([np.arange(n)[keep_o], new_inds[keep_n]])
    n_keep = int(keep_o.sum())
    res_moments = {}
    for k, (m, vv) in moments.items():
        mm, v2 = m[res_inds].copy(), vv[res_inds].copy()
        mm[n_keep:] = 0
        v2[n_keep:] = 0
        res_moments[k] = (mm, v2)
    return res_model, res_moments, res_inds, n_dup, n_split


def reset_opacity(opacity_raw, thresh: float):
    """origin/trainer.py:388-417: logit(min(sigmoid(opacity), thresh))."""
    o = np.minimum(_sigmoid(opacity_raw), np.float32(thresh)).astype(np.float32)
    return _act_log((o / (np.float32(1.0) - o)).astype(np.float32))
