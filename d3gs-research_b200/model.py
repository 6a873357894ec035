"""Gaussian model containers in the reference's layout.

Mirrors d3sim/algos/d3gs/origin/model.py:34-269, 435-465 and the struct-of-tensors helpers of
d3sim/core/pytorch/hmt.py:62-199 that the operator and the optimizer factory rely on.  Two model
classes exist in the reference and both are provided:

* ``GaussianModelOriginFused``: raw parameters; ``normalize`` / ``exp`` / ``sigmoid`` are applied
  INSIDE the kernels (origin/model.py:453-462).  This is what the reference trains with
  (d3sim/algos/d3gs/train.py:384).
* ``GaussianModelOrigin``: activations applied by torch ops in ``create_model_with_act``
  (origin/model.py:248-269); the kernels then treat the tensors as already activated.

``create_flat`` additionally places all six parameter tensors in ONE contiguous allocation (in
the order xyz, quaternion, scale, opacity, sh_base, sh) so that the 59-float-per-Gaussian gradient
is one buffer for the data-parallel all-reduce and one span for the fused Adam launch.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any

import torch

TENSOR_FIELDS = ("xyz", "quaternion_xyzw", "scale", "opacity", "color_sh", "color_sh_base")
# order of the fields inside a flat allocation; also the order of the Adam segments
FLAT_ORDER = ("xyz", "quaternion_xyzw", "scale", "opacity", "color_sh_base", "color_sh")


def flat_field_sizes(n: int, sh_rest: int = 15) -> dict[str, tuple[int, tuple]]:
    return {"xyz": (3 * n, (n, 3)), "quaternion_xyzw": (4 * n, (n, 4)), "scale": (3 * n, (n, 3)),
            "opacity": (n, (n,)), "color_sh_base": (3 * n, (n, 3)), "color_sh": (sh_rest * 3 * n, (n, sh_rest, 3))}


def flat_layout(n: int, sh_rest: int = 15, align: int = 4) -> tuple[dict[str, tuple[int, int, tuple]], int]:
    """``({name: (offset, count, shape)}, total)`` of the six tensors inside one flat float32 buffer.

    Every field starts on a multiple of ``align`` elements (16 bytes: the kernels read quaternions and
    SH rows with vector loads), so ``total`` is 59*n plus at most 3 elements of padding per field; it is
    exactly 59*n when n is a multiple of 4."""
    out, off = {}, 0
    for name in FLAT_ORDER:
        cnt, shape = flat_field_sizes(n, sh_rest)[name]
        out[name] = (off, cnt, shape)
        off = -(-(off + cnt) // align) * align
    return out, off


def carve_flat(flat: torch.Tensor, n: int, sh_rest: int = 15) -> dict[str, torch.Tensor]:
    """Views of the six model tensors inside one flat float32 buffer laid out by ``flat_layout`` (a longer
    buffer carries padding at its end, e.g. to a whole number of optimizer slices)."""
    layout, total = flat_layout(n, sh_rest)
    assert total <= flat.numel()
    return {name: flat[off:off + cnt].view(*shape) for name, (off, cnt, shape) in layout.items()}


@dataclasses.dataclass(kw_only=True)
class GaussianModelOriginBase:
    xyz: torch.Tensor
    quaternion_xyzw: torch.Tensor
    scale: torch.Tensor
    opacity: torch.Tensor
    color_sh: torch.Tensor
    color_sh_base: torch.Tensor | None
    instance_id: torch.Tensor | None = None
    act_applied: bool = False
    cur_sh_degree: int = 0
    # not in the reference: the flat parameter buffer when the model was made by ``create_flat``
    flat: torch.Tensor | None = dataclasses.field(default=None, repr=False, compare=False)

    # ---- struct-of-tensors helpers (hmt.py) ----------------------------------------------------
    def get_all_tensor_fields(self) -> dict[str, torch.Tensor]:
        return {k: getattr(self, k) for k in TENSOR_FIELDS + ("instance_id",) if getattr(self, k) is not None}

    def get_all_non_tensor_fields(self) -> dict[str, Any]:
        return {"act_applied": self.act_applied, "cur_sh_degree": self.cur_sh_degree}

    def get_all_parameter_fields(self) -> dict[str, torch.nn.Parameter]:
        return {k: v for k, v in self.get_all_tensor_fields().items() if isinstance(v, torch.nn.Parameter)}

    def __len__(self) -> int:
        return int(self.xyz.shape[0])

    def __getitem__(self, idx) -> "GaussianModelOriginBase":
        t = {k: v[idx] for k, v in self.get_all_tensor_fields().items()}
        if self.color_sh_base is None:
            t["color_sh_base"] = None
        return type(self)(**t, **self.get_all_non_tensor_fields())

    def concat(self, other: "GaussianModelOriginBase") -> "GaussianModelOriginBase":
        t = {}
        for k, v in self.get_all_tensor_fields().items():
            cat = torch.cat([v, getattr(other, k)], dim=0)
            t[k] = torch.nn.Parameter(cat) if isinstance(v, torch.nn.Parameter) else cat
        if self.color_sh_base is None:
            t["color_sh_base"] = None
        return type(self)(**t, **self.get_all_non_tensor_fields())

    def to_parameter(self):
        rep = {k: torch.nn.Parameter(v) for k, v in self.get_all_tensor_fields().items() if v.is_floating_point()}
        return dataclasses.replace(self, **rep)

    def to_device(self, device):
        t = {}
        for k, v in self.get_all_tensor_fields().items():
            r = v.to(device)
            t[k] = torch.nn.Parameter(r) if isinstance(v, torch.nn.Parameter) else r
        if self.color_sh_base is None:
            t["color_sh_base"] = None
        return type(self)(**t, **self.get_all_non_tensor_fields())

    @classmethod
    def zeros_like(cls, model: "GaussianModelOriginBase", num: int | None = None, not_param: bool = False,
                   external_tensors: dict[str, torch.Tensor] | None = None):
        t = {}
        for k, v in model.get_all_tensor_fields().items():
            if external_tensors is not None and k in external_tensors:
                t[k] = external_tensors[k]
            elif num is not None:
                t[k] = torch.zeros(num, *v.shape[1:], dtype=v.dtype, device=v.device)
            else:
                t[k] = torch.zeros_like(v)
            if isinstance(v, torch.nn.Parameter) and not not_param:
                t[k] = torch.nn.Parameter(t[k])
        if model.color_sh_base is None:
            t["color_sh_base"] = None
        return cls(**t, **model.get_all_non_tensor_fields())

    # ---- model API (origin/model.py:50-156) ----------------------------------------------------
    @property
    def xyz_act(self) -> torch.Tensor:
        return self.xyz

    @property
    def quaternion_xyzw_act(self) -> torch.Tensor:
        raise NotImplementedError

    @property
    def scale_act(self) -> torch.Tensor:
        raise NotImplementedError

    @property
    def opacity_act(self) -> torch.Tensor:
        raise NotImplementedError

    def inverse_scale_act(self, scale_act: torch.Tensor) -> torch.Tensor:
        return torch.log(scale_act)

    @property
    def fused_quaternion_xyzw_act_op(self) -> tuple[str, str]:
        return ("identity", "identity")

    @property
    def fused_scale_act_op(self) -> tuple[str, str]:
        return ("identity", "identity")

    @property
    def fused_opacity_act_op(self) -> tuple[str, str]:
        return ("identity", "identity")

    @property
    def has_fused_activations(self) -> bool:
        return self.fused_scale_act_op[0] != "identity"

    @property
    def color_sh_act(self) -> torch.Tensor:
        return self.color_sh

    @property
    def color_sh_base_act(self) -> torch.Tensor | None:
        return self.color_sh_base

    @property
    def color_sh_degree(self) -> int:
        dim = self.color_sh.shape[1] + (1 if self.color_sh_base is not None else 0)
        res = int(math.sqrt(dim)) - 1
        assert (res + 1) * (res + 1) == dim
        return res

    def get_unique_kernel_key(self):
        return (f"{self.color_sh_degree}_{self.cur_sh_degree}_{self.fused_quaternion_xyzw_act_op[0]}"
                f"_{self.fused_scale_act_op[0]}_{self.fused_opacity_act_op[0]}_{self.color_sh_base is None}")

    def get_proxy_field_dict(self):
        res = {k: getattr(self, k) for k in ("xyz", "quaternion_xyzw", "scale", "opacity", "color_sh")}
        if self.color_sh_base is not None:
            res["color_sh_base"] = self.color_sh_base
        return res

    def set_requires_grad(self, requires_grad: bool):
        for k in TENSOR_FIELDS:
            v = getattr(self, k)
            if v is not None:
                v.requires_grad_(requires_grad)

    def clear_grad(self):
        for k in TENSOR_FIELDS:
            v = getattr(self, k)
            if v is not None:
                v.grad = None

    def create_model_with_act(self):
        if self.act_applied:
            return dataclasses.replace(self)
        return dataclasses.replace(self, xyz=self.xyz_act, quaternion_xyzw=self.quaternion_xyzw_act,
                                   scale=self.scale_act, opacity=self.opacity_act, color_sh=self.color_sh_act,
                                   color_sh_base=self.color_sh_base_act, act_applied=True)

    @classmethod
    def empty(cls, N: int, max_num_degree: int, split: bool = False, dtype: torch.dtype = torch.float32,
              device: torch.device | str = "cuda"):
        k = (max_num_degree + 1) ** 2 - (1 if split else 0)
        return cls(xyz=torch.empty(N, 3, dtype=dtype, device=device),
                   quaternion_xyzw=torch.empty(N, 4, dtype=dtype, device=device),
                   scale=torch.empty(N, 3, dtype=dtype, device=device),
                   opacity=torch.empty(N, dtype=dtype, device=device),
                   color_sh_base=torch.empty(N, 3, dtype=dtype, device=device) if split else None,
                   color_sh=torch.empty(N, k, 3, dtype=dtype, device=device), cur_sh_degree=0)

    @classmethod
    def zeros(cls, N: int, max_num_degree: int, split: bool = False, dtype: torch.dtype = torch.float32,
              device: torch.device | str = "cpu", opacity: torch.Tensor | None = None):
        k = (max_num_degree + 1) ** 2 - (1 if split else 0)
        return cls(xyz=torch.zeros(N, 3, dtype=dtype, device=device),
                   quaternion_xyzw=torch.zeros(N, 4, dtype=dtype, device=device),
                   scale=torch.zeros(N, 3, dtype=dtype, device=device),
                   opacity=opacity if opacity is not None else torch.zeros(N, dtype=dtype, device=device),
                   color_sh_base=torch.zeros(N, 3, dtype=dtype, device=device) if split else None,
                   color_sh=torch.zeros(N, k, 3, dtype=dtype, device=device), cur_sh_degree=0)

    @classmethod
    def create_flat(cls, N: int, device: torch.device | str = "cuda", cur_sh_degree: int = 3):
        """Degree-3 split model whose six tensors are views of one flat buffer (``flat_layout``)."""
        flat = torch.zeros(flat_layout(N)[1], dtype=torch.float32, device=device)
        views = carve_flat(flat, N)
        return cls(**views, cur_sh_degree=cur_sh_degree, flat=flat)

    @classmethod
    def from_tensors(cls, xyz, quaternion_xyzw, scale, opacity, color_sh_base, color_sh, device="cuda",
                     cur_sh_degree: int = 3, flat: bool = True):
        """Build a model on ``device`` from CPU/GPU tensors (``color_sh`` = the 15 higher-order coefficients)."""
        n = xyz.shape[0]
        if flat and color_sh.shape[1] == 15:
            m = cls.create_flat(n, device=device, cur_sh_degree=cur_sh_degree)
            for k, v in (("xyz", xyz), ("quaternion_xyzw", quaternion_xyzw), ("scale", scale), ("opacity", opacity),
                         ("color_sh_base", color_sh_base), ("color_sh", color_sh)):
                getattr(m, k).copy_(v.to(device))
            return m
        return cls(xyz=xyz.to(device).contiguous(), quaternion_xyzw=quaternion_xyzw.to(device).contiguous(),
                   scale=scale.to(device).contiguous(), opacity=opacity.to(device).contiguous(),
                   color_sh_base=color_sh_base.to(device).contiguous(), color_sh=color_sh.to(device).contiguous(),
                   cur_sh_degree=cur_sh_degree)


@dataclasses.dataclass(kw_only=True)
class GaussianModelOrigin(GaussianModelOriginBase):
    """Activations applied by torch (origin/model.py:248-269)."""

    @property
    def quaternion_xyzw_act(self) -> torch.Tensor:
        if self.act_applied:
            return self.quaternion_xyzw
        return torch.nn.functional.normalize(self.quaternion_xyzw, p=2, dim=-1)

    @property
    def scale_act(self) -> torch.Tensor:
        return self.scale if self.act_applied else torch.exp(self.scale)

    @property
    def opacity_act(self) -> torch.Tensor:
        return self.opacity if self.act_applied else torch.sigmoid(self.opacity)


@dataclasses.dataclass(kw_only=True)
class GaussianModelOriginFused(GaussianModelOriginBase):
    """Activations fused into the kernels (origin/model.py:435-465)."""

    @property
    def quaternion_xyzw_act(self) -> torch.Tensor:
        return self.quaternion_xyzw

    @property
    def scale_act(self) -> torch.Tensor:
        return self.scale

    @property
    def opacity_act(self) -> torch.Tensor:
        return self.opacity

    @property
    def fused_quaternion_xyzw_act_op(self) -> tuple[str, str]:
        return ("normalize", "normalize_grad_out")

    @property
    def fused_scale_act_op(self) -> tuple[str, str]:
        return ("exponential", "exponential_grad_out")

    @property
    def fused_opacity_act_op(self) -> tuple[str, str]:
        return ("sigmoid", "sigmoid_grad_out")
