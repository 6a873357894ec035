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
