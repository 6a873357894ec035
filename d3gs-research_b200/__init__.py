"""B200-native 3D-Gaussian-splatting training step behind the d3sim.algos.d3gs operator API.

The compute path is the sm_100a shared library ``libd3gs_b200.so`` (C ABI in include/d3gs_b200.h); the
modules here mirror the reference's Python operator interface on top of it.  Importing the package
does not load the library; constructing an operator or calling an op does, and fails loudly if the
library has not been built.
"""
__version__ = "0.1.0"

from .config_def import (Config, EarlyFilterAlgo, GaussianSplatConfig, Model, Optimizer,  # noqa: F401
                         RasterizeBackwardAlgo, Strategy, Train)
from .camera import BasicPinholeCamera, Pose  # noqa: F401
from .model import GaussianModelOrigin, GaussianModelOriginBase, GaussianModelOriginFused  # noqa: F401


def __getattr__(name):
    # torch-dependent modules are imported on first use
    import importlib
    table = {
        "GaussianSplatOp": "render", "rasterize_gaussians": "render", "rasterize_gaussians_dynamic": "render",
        "CameraBundle": "render", "GaussianSplatOutput": "render", "GaussianSplatOpContext": "render",
        "GaussianSplatGradients": "render", "fused_ssim_loss": "fused_ssim", "l1_dssim_loss": "fused_ssim",
        "l1_loss": "fused_ssim", "GaussianAdam": "adam", "fused_step": "adam", "GaussianTrainState": "strategy",
        "GaussianStrategyOrigin": "strategy", "create_origin_3dgs_optimizers": "tools", "SplatTrainer": "trainer",
    }
    if name in table:
        return getattr(importlib.import_module(f"{__name__}.{table[name]}"), name)
    raise AttributeError(name)
