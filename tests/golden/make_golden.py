"""Generates tests/golden/ref_vectors.npz by importing the reference's own pure-torch helper modules.

Run where the reference tree is available:  python tests/golden/make_golden.py <path to the d3gs-research checkout>
The modules are loaded by file path (the d3sim package itself cannot be imported: its JIT dependencies are
absent) and called unmodified.  ``build_rotation`` hard-codes device="cuda" for its temporaries; torch.zeros is
wrapped for the duration of the call so that the same code runs on the CPU.

Pinned here:
  * SH evaluation            d3sim/algos/d3gs/origin/data/utils/sh_utils.py:57-112   (eval_sh)
  * quaternion -> rotation   d3sim/algos/d3gs/origin/data/utils/general_utils.py:78-99
  * covariance R S S^T R^T   general_utils.py:101-110 (build_scaling_rotation), 64-76 (strip_symmetric)
  * SSIM and L1              d3sim/algos/d3gs/origin/data/utils/loss_utils.py:17-63
  * position lr schedule     general_utils.py:39-76 (get_expon_lr_func)
"""
import contextlib
import importlib.util
import os
import sys

import numpy as np
import torch


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


@contextlib.contextmanager
def zeros_on_cpu():
    orig = torch.zeros

    def patched(*a, **k):
        k.pop("device", None)
        return orig(*a, **k)

    torch.zeros = patched
    try:
        yield
    finally:
        torch.zeros = orig


def main(ref_root):
    u = os.path.join(ref_root, "d3sim/algos/d3gs/origin/data/utils")
    sh_utils = load(os.path.join(u, "sh_utils.py"), "ref_sh_utils")
    general = load(os.path.join(u, "general_utils.py"), "ref_general_utils")
    loss_utils = load(os.path.join(u, "loss_utils.py"), "ref_loss_utils")
    g = torch.Generator().manual_seed(1234)
    out = {}
    # SH: reference layout sh[..., C, (deg+1)^2]; d3sim stores coefficient-major [N, 16, 3] (tools.py:31-33)
    n = 48
    dirs = torch.randn(n, 3, generator=g)
    dirs = dirs / dirs.norm(dim=1, keepdim=True)
    coeff = torch.randn(n, 16, 3, generator=g)            # coefficient-major
    out["sh_dirs"], out["sh_coeff"] = dirs.numpy(), coeff.numpy()
    for deg in range(4):
        out[f"sh_rgb_deg{deg}"] = sh_utils.eval_sh(deg, coeff.permute(0, 2, 1), dirs).numpy()
    # rotation / covariance: the reference takes (w, x, y, z); d3sim stores (x, y, z, w) (tools.py:37)
    quat_xyzw = torch.randn(n, 4, generator=g)
    scale_act = torch.exp(torch.randn(n, 3, generator=g) * 0.5 - 2.0)
    wxyz = quat_xyzw[:, [3, 0, 1, 2]]
    with zeros_on_cpu():
        R = general.build_rotation(wxyz)
        L = general.build_scaling_rotation(scale_act, wxyz)
        cov6 = general.strip_symmetric(L @ L.transpose(1, 2))
    out["quat_xyzw"], out["scale_act"], out["rot"], out["cov6"] = (quat_xyzw.numpy(), scale_act.numpy(), R.numpy(),
                                                                   cov6.numpy())
    # SSIM / L1 (NCHW)
    x = torch.rand(2, 3, 37, 45, generator=g)
    y = torch.rand(2, 3, 37, 45, generator=g)
    out["img_x"], out["img_y"] = x.numpy(), y.numpy()
    out["ssim"] = np.float64(loss_utils.ssim(x, y).item())
    out["l1"] = np.float64(loss_utils.l1_loss(x, y).item())
    xs = (x * 0.25 + 0.5 * y).clamp(0, 1)       # a correlated pair: SSIM far from 0
    out["img_x2"] = xs.numpy()
    out["ssim2"] = np.float64(loss_utils.ssim(xs, y).item())
    # lr schedule
    f = general.get_expon_lr_func(lr_init=1.6e-4, lr_final=1.6e-6, lr_delay_mult=0.01, max_steps=30000)
    steps = np.array([0, 1, 10, 100, 1000, 7000, 15000, 29999, 30000, 40000])
    out["lr_steps"], out["lr_values"] = steps, np.array([f(int(s)) for s in steps], np.float64)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("D3SIM_REFERENCE", "reference"))
