"""Optimizer factory and learning-rate schedule of the reference training setup.

Mirrors d3sim/algos/d3gs/tools.py:92-125 (``get_expon_lr_func``) and 146-173
(``create_origin_3dgs_optimizers``): six single-tensor ``GaussianAdam`` optimizers with
lr = {xyz 1.6e-4*extent, sh_base 2.5e-3, sh 2.5e-3/20, opacity 0.05, scale 5e-3, quat 1e-3} * sqrt(B),
eps = 1e-15/sqrt(B), betas = (1 - B*0.1, 1 - B*0.001).
"""
from __future__ import annotations

import math

import numpy as np

from . import config_def
from .adam import GaussianAdam
from .model import GaussianModelOriginBase


def get_expon_lr_func(lr_init, lr_final, lr_delay_steps=0, lr_delay_mult=1.0, max_steps=1000000):
    def helper(step):
        if step < 0 or (lr_init == 0.0 and lr_final == 0.0):
            return 0.0
        if lr_delay_steps > 0:
            delay_rate = lr_delay_mult + (1 - lr_delay_mult) * np.sin(0.5 * np.pi * np.clip(step / lr_delay_steps, 0, 1))
        else:
            delay_rate = 1.0
        t = np.clip(step / max_steps, 0, 1)
        log_lerp = np.exp(np.log(lr_init) * (1 - t) + np.log(lr_final) * t)
        return delay_rate * log_lerp

    return helper


def create_origin_3dgs_optimizers(model: GaussianModelOriginBase, optim_cfg: config_def.Optimizer, batch_size: int,
                                  spatial_lr_scale: float, fused: bool = True):
    bs_scale = math.sqrt(batch_size)
    pgs = [
        {"params": [model.xyz], "lr": optim_cfg.position_lr_init * spatial_lr_scale * bs_scale, "name": "xyz"},
        {"params": [model.color_sh_base], "lr": optim_cfg.feature_lr * bs_scale, "name": "color_sh_base"},
        {"params": [model.color_sh], "lr": optim_cfg.feature_lr * bs_scale / 20.0, "name": "color_sh"},
        {"params": [model.opacity], "lr": optim_cfg.opacity_lr * bs_scale, "name": "opacity"},
        {"params": [model.scale], "lr": optim_cfg.scaling_lr * bs_scale, "name": "scale"},
        {"params": [model.quaternion_xyzw], "lr": optim_cfg.rotation_lr * bs_scale, "name": "quaternion_xyzw"},
    ]
    optimizers = {
        pg["name"]: GaussianAdam([{"params": pg["params"], "lr": pg["lr"], "name": pg["name"]}], fused=False,
                                 eps=1e-15 / bs_scale,
                                 betas=(1 - batch_size * (1 - 0.9), 1 - batch_size * (1 - 0.999)))
        for pg in pgs
    }
    schedule = get_expon_lr_func(lr_init=optim_cfg.position_lr_init * spatial_lr_scale * bs_scale,
                                 lr_final=optim_cfg.position_lr_final * spatial_lr_scale * bs_scale,
                                 lr_delay_mult=optim_cfg.position_lr_delay_mult,
                                 max_steps=optim_cfg.position_lr_max_steps)
    return optimizers, schedule


# ---- model I/O and initialisation (d3sim/algos/d3gs/tools.py:14-90) --------------------------------------------
SH_C0 = 0.28209479177387814


def rgb_to_sh(rgb):
    return (rgb - 0.5) / SH_C0


def inverse_sigmoid(x):
    import torch
    return torch.log(x / (1 - x))


_PLY_FIELDS = (["x", "y", "z", "nx", "ny", "nz"] + [f"f_dc_{i}" for i in range(3)] + [f"f_rest_{i}" for i in range(45)] +
               ["opacity"] + [f"scale_{i}" for i in range(3)] + [f"rot_{i}" for i in range(4)])


def _read_ply_vertices(path: str) -> np.ndarray:
    """Vertex table of a binary little-endian PLY as a numpy structured array (the reference reads it with the
    plyfile package, tools.py:21-22; only float/double/int/uchar scalar properties occur in these files)."""
    types = {"float": "<f4", "float32": "<f4", "double": "<f8", "float64": "<f8", "int": "<i4", "int32": "<i4",
             "uint": "<u4", "uint32": "<u4", "short": "<i2", "ushort": "<u2", "char": "i1", "uchar": "u1",
             "int8": "i1", "uint8": "u1", "int16": "<i2", "uint16": "<u2"}
    with open(path, "rb") as f:
        if f.readline().strip() != b"ply":
            raise ValueError(f"{path}: not a PLY file")
        fmt, count, props, in_vertex = None, None, [], False
        while True:
            line = f.readline()
            if not line:
                raise ValueError(f"{path}: truncated PLY header")
            tok = line.decode("ascii", "replace").split()
            if not tok:
                continue
            if tok[0] == "format":
                fmt = tok[1]
            elif tok[0] == "element":
                in_vertex = tok[1] == "vertex"
                if in_vertex:
                    count = int(tok[2])
                elif count is not None and not props:
                    raise ValueError(f"{path}: vertex element has no properties")
            elif tok[0] == "property" and in_vertex:
                if tok[1] == "list":
                    raise ValueError(f"{path}: list properties in the vertex element are not supported")
                props.append((tok[2], types[tok[1]]))
            elif tok[0] == "end_header":
                break
        if fmt != "binary_little_endian":
            raise ValueError(f"{path}: only binary_little_endian PLY is supported (got {fmt})")
        if count is None:
            raise ValueError(f"{path}: no vertex element")
        data = np.fromfile(f, dtype=np.dtype(props), count=count)
    if data.shape[0] != count:
        raise ValueError(f"{path}: expected {count} vertices, file holds {data.shape[0]}")
    return data


def load_3dgs_origin_model(ply_path: str, fused: bool = True, split: bool = True, device="cuda"):
    """tools.py:20-64: an Inria-layout 3DGS checkpoint -> model.  File conventions: ``f_rest`` is stored
    channel-major ([3][15]) and becomes coefficient-major [15,3]; ``rot`` is (w,x,y,z) and becomes (x,y,z,w)."""
    import torch
    from .model import GaussianModelOrigin, GaussianModelOriginFused
    v = _read_ply_vertices(ply_path)
    missing = [k for k in _PLY_FIELDS if k not in v.dtype.names and not k.startswith("n")]
    if missing:
        raise ValueError(f"{ply_path}: missing properties {missing[:5]}...")
    f32 = np.float32
    xyz = np.stack([v["x"], v["y"], v["z"]], axis=1).astype(f32)
    f_dc = np.stack([v[f"f_dc_{i}"] for i in range(3)], axis=1)
    f_rest = np.stack([v[f"f_rest_{i}"] for i in range(45)], axis=1).reshape(-1, 3, 15).transpose(0, 2, 1).reshape(len(v), -1)
    sh = np.ascontiguousarray(np.concatenate([f_dc, f_rest], axis=1).astype(f32)).reshape(-1, 16, 3)
    rots = np.ascontiguousarray(np.stack([v[f"rot_{i}"] for i in range(4)], axis=1).astype(f32)[:, [1, 2, 3, 0]])
    scales = np.stack([v[f"scale_{i}"] for i in range(3)], axis=1).astype(f32)
    opacity = v["opacity"].astype(f32)
    cls = GaussianModelOriginFused if fused else GaussianModelOrigin
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    if split:
        return cls.from_tensors(t(xyz), t(rots), t(scales), t(opacity), t(sh[:, 0]), t(sh[:, 1:]), device=device,
                                cur_sh_degree=3)
    m = cls(xyz=t(xyz).to(device), quaternion_xyzw=t(rots).to(device), scale=t(scales).to(device),
            opacity=t(opacity).to(device), color_sh=t(sh).to(device), color_sh_base=None, cur_sh_degree=3)
    return m


def save_3dgs_origin_model(model: GaussianModelOriginBase, ply_path: str) -> None:
    """Writes the raw parameters in the layout ``load_3dgs_origin_model`` reads (the Inria checkpoint layout)."""
    n = len(model)
    c = lambda x: x.detach().cpu().numpy().astype(np.float32)
    if model.color_sh_base is not None:
        sh = np.concatenate([c(model.color_sh_base)[:, None, :], c(model.color_sh)], axis=1)
    else:
        sh = c(model.color_sh)
    if sh.shape[1] < 16:
        sh = np.concatenate([sh, np.zeros((n, 16 - sh.shape[1], 3), np.float32)], axis=1)
    rec = np.zeros(n, dtype=[(k, "<f4") for k in _PLY_FIELDS])
    xyz, rot, sc = c(model.xyz), c(model.quaternion_xyzw), c(model.scale)
    for i, k in enumerate("xyz"):
        rec[k] = xyz[:, i]
    for i in range(3):
        rec[f"f_dc_{i}"] = sh[:, 0, i]
        rec[f"scale_{i}"] = sc[:, i]
    rest = sh[:, 1:, :].transpose(0, 2, 1).reshape(n, 45)          # coefficient-major -> channel-major
    for i in range(45):
        rec[f"f_rest_{i}"] = rest[:, i]
    rec["opacity"] = c(model.opacity)
    for i, src in enumerate((3, 0, 1, 2)):                          # (x,y,z,w) -> (w,x,y,z)
        rec[f"rot_{i}"] = rot[:, src]
    header = "ply\nformat binary_little_endian 1.0\nelement vertex %d\n" % n
    header += "".join(f"property float {k}\n" for k in _PLY_FIELDS) + "end_header\n"
    with open(ply_path, "wb") as f:
        f.write(header.encode("ascii"))
        rec.tofile(f)


def points_to_gaussian_init_scale(points):
    """tools.py:64-71: log of the root mean squared distance to the three nearest neighbours, for all three axes."""
    import torch
    from .ops import simple_knn
    knn_res = simple_knn(points.contiguous(), min(3, max(points.shape[0] - 1, 1)))
    dist2 = torch.clamp_min(torch.square(knn_res).mean(1), 0.0000001)
    return torch.log(torch.sqrt(dist2))[..., None].repeat(1, 3)


def init_original_3dgs_model(model: GaussianModelOriginBase, points: np.ndarray, points_rgb: np.ndarray):
    """tools.py:73-90: SfM points -> initial Gaussians (DC colour from RGB, isotropic kNN scale, identity
    rotation, opacity 0.1, SH degree 0)."""
    import torch
    with torch.no_grad():
        assert model.xyz.shape[0] == points.shape[0]
        dev = model.xyz.device
        pts = torch.from_numpy(points.astype(np.float32)).to(dev).contiguous()
        col = rgb_to_sh(torch.from_numpy(points_rgb.astype(np.float32)).to(dev))
        if model.color_sh_base is None:
            model.color_sh[:, 0] = col
        else:
            model.color_sh_base[:] = col
        model.scale[:] = points_to_gaussian_init_scale(pts)
        quat = torch.zeros((pts.shape[0], 4), device=dev)
        quat[:, 3] = 1
        model.quaternion_xyzw[:] = quat
        model.opacity[:] = inverse_sigmoid(0.1 * torch.ones(pts.shape[0], dtype=torch.float32, device=dev))
        model.cur_sh_degree = 0
        model.xyz[:] = pts
