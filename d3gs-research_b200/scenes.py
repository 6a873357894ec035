"""Seeded synthetic scenes with the shapes and value distributions of the benchmark configs.

The reference measures on Mip-NeRF-360 "garden" (d3sim/algos/d3gs/train.py:362-371,
scripts/d3gs/d3gs_dev.py); that dataset is not available offline, so these generators stand in
for it.  Every draw comes from one ``torch.Generator(device="cpu")`` in a fixed order (positions,
log-scales, quaternions, opacity logits, SH DC, SH rest, target) so that a CPU checker and the GPU
see identical bits.

Camera convention (csrc/camera.py:307-333, ``pos_cam_to_uv_no_distort<2,0,1>``): +z forward,
+x right, +y down; ``cam2world`` is a 4x4 matrix; focal from the vertical field of view,
``f = 0.5*H/tan(vfov/2)`` with square pixels, principal point at the image centre.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch


@dataclass
class SceneConfig:
    name: str
    n: int
    width: int
    height: int
    vfov_deg: float
    cam_radius: float
    pos: tuple            # ("normal", sigma) | ("uniform", half_extent)
    log_scale: tuple      # ("normal", mean, std) | ("mixture", (w, mean, std), ...)
    opacity: tuple        # (mean, std)
    sh_degree: int
    loss: str             # "l1" | "l1_dssim"
    target: str           # "uniform" | "blobs"
    num_views: int = 1
    cam_layout: str = "axis"   # "axis" | "sphere" | "ring"
    elevation_deg: float = 0.0


CONFIGS = {
    # Tiny scene that the CPU checker runs in full
    "cfg0": SceneConfig("cfg0", 10_000, 256, 256, 60.0, 8.0, ("normal", 2.0), ("normal", -3.0, 0.5), (0.0, 1.0),
                        0, "l1", "uniform"),
    "cfg1": SceneConfig("cfg1", 100_000, 800, 800, 50.0, 12.0, ("uniform", 5.0), ("normal", -4.0, 0.6), (0.0, 1.5),
                        3, "l1", "uniform", cam_layout="sphere"),
    "cfg2": SceneConfig("cfg2", 1_000_000, 1297, 840, 55.0, 15.0, ("normal", 6.0), ("normal", -4.0, 0.6), (0.0, 1.5),
                        3, "l1_dssim", "blobs", cam_layout="sphere"),
    "cfg3": SceneConfig("cfg3", 3_000_000, 1920, 1080, 60.0, 20.0, ("normal", 8.0), ("normal", -4.5, 0.7), (0.0, 1.5),
                        3, "l1_dssim", "blobs", num_views=8, cam_layout="ring", elevation_deg=15.0),
    "cfg4": SceneConfig("cfg4", 6_000_000, 3840, 2160, 70.0, 25.0, ("normal", 10.0),
                        ("mixture", (0.9, -5.0, 0.5), (0.1, -1.5, 0.5)), (0.5, 1.0),
                        3, "none", "none", num_views=64, cam_layout="sphere"),
}


def look_at_cam2world(eye, target=(0.0, 0.0, 0.0), up=(0.0, -1.0, 0.0)) -> np.ndarray:
    """4x4 camera-to-world with +z forward, +x right, +y down."""
    eye = np.asarray(eye, np.float64)
    fwd = np.asarray(target, np.float64) - eye
    fwd /= np.linalg.norm(fwd)
    upv = np.asarray(up, np.float64)
    if abs(np.dot(fwd, upv)) > 0.999:
        upv = np.array([0.0, 0.0, 1.0])
    down = -upv
    right = np.cross(down, fwd)
    right /= np.linalg.norm(right)
    down = np.cross(fwd, right)
    m = np.eye(4)
    m[:3, 0], m[:3, 1], m[:3, 2], m[:3, 3] = right, down, fwd, eye
    return m


def camera_positions(cfg: SceneConfig, gen: torch.Generator) -> list[np.ndarray]:
    r = cfg.cam_radius
    if cfg.cam_layout == "axis":
        return [np.array([0.0, 0.0, r])]
    if cfg.cam_layout == "ring":
        el = math.radians(cfg.elevation_deg)
        return [np.array([r * math.cos(el) * math.cos(2 * math.pi * k / cfg.num_views), -r * math.sin(el),
                          r * math.cos(el) * math.sin(2 * math.pi * k / cfg.num_views)])
                for k in range(cfg.num_views)]
    # golden-spiral points on a sphere (deterministic, evenly spread)
    out = []
    for k in range(cfg.num_views):
        zc = 1.0 - 2.0 * (k + 0.5) / max(cfg.num_views, 1)
        rad = math.sqrt(max(0.0, 1.0 - zc * zc))
        phi = k * math.pi * (3.0 - math.sqrt(5.0)) + 0.7
        out.append(np.array([r * rad * math.cos(phi), r * zc, r * rad * math.sin(phi)]))
    return out


def pack_camera(cam2world: np.ndarray, fx: float, fy: float, cx: float, cy: float) -> np.ndarray:
    """16 floats: cam2world[:3].T flattened ([4,3], render.py:136) followed by fx, fy, cx, cy."""
    c2w_t = np.ascontiguousarray(cam2world[:3].T, dtype=np.float64).reshape(12)
    return np.concatenate([c2w_t, [fx, fy, cx, cy]]).astype(np.float32)


def intrinsics(cfg: SceneConfig):
    f = 0.5 * cfg.height / math.tan(math.radians(cfg.vfov_deg) / 2.0)
    return f, f, cfg.width / 2.0, cfg.height / 2.0


def make_scene(cfg: SceneConfig | str, seed: int = 0, n: int | None = None, views: int | None = None,
               width: int | None = None, height: int | None = None):
    """Returns a dict of CPU float32 torch tensors plus the packed cameras.

    ``n``/``views``/``width``/``height`` override the config (bounded samples keep the config's
    distributions and camera geometry; a smaller image keeps the field of view).
    """
    if isinstance(cfg, str):
        cfg = CONFIGS[cfg]
    if n is not None or views is not None or width is not None or height is not None:
        cfg = SceneConfig(**{**cfg.__dict__, "n": n or cfg.n, "num_views": views or cfg.num_views,
                             "width": width or cfg.width, "height": height or cfg.height})
    g = torch.Generator(device="cpu").manual_seed(seed)
    N = cfg.n

    def randn(*shape):
        return torch.randn(*shape, generator=g, dtype=torch.float32)

    if cfg.pos[0] == "normal":
        xyz = randn(N, 3) * cfg.pos[1]
    else:
        xyz = (torch.rand(N, 3, generator=g, dtype=torch.float32) * 2.0 - 1.0) * cfg.pos[1]
    if cfg.log_scale[0] == "normal":
        scale = randn(N, 3) * cfg.log_scale[2] + cfg.log_scale[1]
    else:
        comp = torch.rand(N, generator=g, dtype=torch.float32)
        z = randn(N, 3)
        w0, m0, s0 = cfg.log_scale[1]
        _, m1, s1 = cfg.log_scale[2]
        first = (comp < w0)[:, None]
        scale = torch.where(first, z * s0 + m0, z * s1 + m1)
    quat = randn(N, 4)
    quat = quat / quat.norm(dim=1, keepdim=True)
    opacity = randn(N) * cfg.opacity[1] + cfg.opacity[0]
    sh_base = randn(N, 3) * 0.5
    sh_rest = randn(N, 15, 3) * 0.05 if cfg.sh_degree > 0 else torch.zeros(N, 15, 3)
    fx, fy, cx, cy = intrinsics(cfg)
    eyes = camera_positions(cfg, g)[: cfg.num_views]
    cam2worlds = [look_at_cam2world(e) for e in eyes]
    cams = np.stack([pack_camera(m, fx, fy, cx, cy) for m in cam2worlds])
    H, W = cfg.height, cfg.width
    if cfg.target == "uniform":
        target = torch.rand(cfg.num_views, H, W, 3, generator=g, dtype=torch.float32).permute(0, 3, 1, 2).contiguous()
    elif cfg.target == "blobs":
        target = blob_target(cfg.num_views, H, W, g)
    else:
        target = None
    return dict(cfg=cfg, xyz=xyz.contiguous(), quat=quat.contiguous(), scale=scale.contiguous(),
                opacity=opacity.contiguous(), sh_base=sh_base.contiguous(), sh_rest=sh_rest.contiguous(),
                cams=cams, cam2worlds=cam2worlds, intrinsics=(fx, fy, cx, cy), target=target)


def blob_target(views: int, H: int, W: int, g: torch.Generator) -> torch.Tensor:
    """Smooth target: per channel the sum of 16 random 2-D Gaussian blobs, clipped to [0,1]. NCHW."""
    ys = torch.arange(H, dtype=torch.float32)[:, None]
    xs = torch.arange(W, dtype=torch.float32)[None, :]
    out = torch.zeros(views, 3, H, W)
    for v in range(views):
        for c in range(3):
            p = torch.rand(16, 4, generator=g, dtype=torch.float32)
            for k in range(16):
                mx, my = p[k, 0] * W, p[k, 1] * H
                sg = (0.05 + 0.2 * p[k, 2]) * min(H, W)
                amp = 0.2 + 0.6 * p[k, 3]
                out[v, c] += amp * torch.exp(-((xs - mx) ** 2 + (ys - my) ** 2) / (2 * sg * sg))
    return out.clamp_(0.0, 1.0).contiguous()
