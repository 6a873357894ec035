"""Minimal pinhole camera carrier with the attributes the splat operator reads.

Mirrors the part of d3sim/data/scene_def/camera.py:54-61, 184-190, 285-290 and
d3sim/data/scene_def/base.py:137-196 that ``GaussianSplatOp.forward`` touches: ``intrinsic`` (4x4),
``pose.to_world`` (camera-to-world 4x4), ``image_shape_wh``, ``focal_length``, ``principal_point``
and ``frame_local_id``.  Image loading, distortion and lazy transforms are dataset plumbing and
are not part of this library.
"""
from __future__ import annotations

import dataclasses

import numpy as np


@dataclasses.dataclass
class Pose:
    to_world: np.ndarray = dataclasses.field(default_factory=lambda: np.eye(4))
    to_vehicle: np.ndarray = dataclasses.field(default_factory=lambda: np.eye(4))


@dataclasses.dataclass(kw_only=True)
class BasicPinholeCamera:
    image_shape_wh: tuple[int, int]
    intrinsic: np.ndarray = dataclasses.field(default_factory=lambda: np.eye(4))
    pose: Pose = dataclasses.field(default_factory=Pose)
    frame_local_id: int | None = None
    id: str = ""

    @property
    def focal_length(self) -> np.ndarray:
        return np.array([self.intrinsic[0, 0], self.intrinsic[1, 1]], np.float32)

    @property
    def principal_point(self) -> np.ndarray:
        return np.array([self.intrinsic[0, 2], self.intrinsic[1, 2]], np.float32)

    @property
    def fov_xy(self) -> np.ndarray:
        return 2 * np.arctan(0.5 * np.array(self.image_shape_wh, np.float32) / self.focal_length)

    @classmethod
    def from_params(cls, cam2world: np.ndarray, fx: float, fy: float, cx: float, cy: float, width: int, height: int,
                    frame_local_id: int | None = None):
        k = np.eye(4, dtype=np.float64)
        k[0, 0], k[1, 1], k[0, 2], k[1, 2] = fx, fy, cx, cy
        return cls(image_shape_wh=(int(width), int(height)), intrinsic=k, pose=Pose(to_world=np.asarray(cam2world)),
                   frame_local_id=frame_local_id)
