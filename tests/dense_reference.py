"""Independent dense reference renderer in torch float64 with autograd.

It evaluates the splatting equations pixel by pixel over ALL Gaussians (no tiles lists, no sort
keys, no hand-written gradients) and lets torch differentiate them.  It is used to validate the
CPU oracle's forward image and all 59 parameter gradients on tiny scenes; formulas follow the
reference's comments ("cov3d = R @ S @ S.T @ R.T" d3sim/csrc/gs3d.py:370, "Projected Cov =
J @ W @ Cov @ W.T @ J.T" gs3d.py:463-465, blend rules d3sim/algos/d3gs/render.py:1762-1808).
"""
from __future__ import annotations

import math

import torch

SH_C0 = 0.28209479177387814
SH_C1 = 0.4886025119029199
SH_C2 = [1.0925484305920792, -1.0925484305920792, 0.31539156525252005, -1.0925484305920792, 0.5462742152960396]
SH_C3 = [-0.5900435899266435, 2.890611442640554, -0.4570457994644658, 0.3731763325901154, -0.4570457994644658,
         1.445305721320277, -0.5900435899266435]


def sh_basis(deg, d):
    x, y, z = d[:, 0], d[:, 1], d[:, 2]
    b = [torch.full_like(x, SH_C0)]
    if deg > 0:
        b += [-SH_C1 * y, SH_C1 * z, -SH_C1 * x]
    if deg > 1:
        xx, yy, zz, xy, yz, xz = x * x, y * y, z * z, x * y, y * z, x * z
        b += [SH_C2[0] * xy, SH_C2[1] * yz, SH_C2[2] * (2 * zz - xx - yy), SH_C2[3] * xz, SH_C2[4] * (xx - yy)]
    if deg > 2:
        b += [SH_C3[0] * y * (3 * xx - yy), SH_C3[1] * xy * z, SH_C3[2] * y * (4 * zz - xx - yy),
              SH_C3[3] * z * (2 * zz - 3 * xx - 3 * yy), SH_C3[4] * x * (4 * zz - xx - yy),
              SH_C3[5] * z * (xx - yy), SH_C3[6] * x * (xx - 3 * yy)]
    return torch.stack(b, dim=1)


def render_dense(params, cam16, W, H, sh_degree, clamp_mask_reference_order=True, tile=16, near=0.2, far=1e4,
                 lowpass=0.3, alpha_eps=1.0 / 255.0, t_eps=1e-4, anti_aliasing=False, depth_mode=None, custom=None):
    """params: dict of float64 leaf tensors (xyz, quat, scale, opacity, sh_base, sh_rest).
    Returns color [H,W,3], T [H,W], n_valid (visible mask [N]); with depth_mode "z" or "inv" also the blended
    depth value sum_i w_i d_i [H,W] (d3sim/algos/d3gs/render.py:1824, 2244-2255 in training).  "inv": the depth
    value is 1/z AND, as in the reference, that value is what the splats are sorted by (render.py:582, 773).
    custom: [N,F] float64 features blended like colours; their image [H,W,F] is appended to the result."""
    xyz, quat, scale, opac = params["xyz"], params["quat"], params["scale"], params["opacity"]
    cam16 = torch.as_tensor(cam16, dtype=torch.float64)
    Rt = cam16[:9].reshape(3, 3)            # rows: columns of R_c2w  == world->cam rotation
    c = cam16[9:12]
    fx, fy, cx, cy = [float(v) for v in cam16[12:16]]
    d = xyz - c
    pc = d @ Rt.T
    z = pc[:, 2]
    u = pc[:, 0] / z * fx + cx - 0.5
    v = pc[:, 1] / z * fy + cy - 0.5
    q = quat / quat.norm(dim=1, keepdim=True)
    s = torch.exp(scale)
    o = torch.sigmoid(opac)
    x_, y_, z_, w_ = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
    R = torch.stack([
        1 - 2 * (y_ * y_ + z_ * z_), 2 * (x_ * y_ - w_ * z_), 2 * (x_ * z_ + w_ * y_),
        2 * (x_ * y_ + w_ * z_), 1 - 2 * (x_ * x_ + z_ * z_), 2 * (y_ * z_ - w_ * x_),
        2 * (x_ * z_ - w_ * y_), 2 * (y_ * z_ + w_ * x_), 1 - 2 * (x_ * x_ + y_ * y_)], dim=1).reshape(-1, 3, 3)
    M = R * s[:, None, :]
    Sigma = M @ M.transpose(1, 2)
    tanx, tany = 0.5 * W / fx, 0.5 * H / fy
    limx, limy = (1.3 * tanx * z).abs(), (1.3 * tany * z).abs()
    tx = torch.minimum(limx, torch.maximum(-limx, pc[:, 0]))
    ty = torch.minimum(limy, torch.maximum(-limy, pc[:, 1]))
    # the clamp limit is treated as a constant w.r.t. z in the reference's gradient (gs3d.py:524-529)
    tx = torch.where((pc[:, 0] < -limx) | (pc[:, 0] > limx), tx.detach(), tx)
    ty = torch.where((pc[:, 1] < -limy) | (pc[:, 1] > limy), ty.detach(), ty)
    zero = torch.zeros_like(z)
    J = torch.stack([fx / z, zero, -fx * tx / (z * z), zero, fy / z, -fy * ty / (z * z)], dim=1).reshape(-1, 2, 3)
    Tm = J @ Rt
    cov = Tm @ Sigma @ Tm.transpose(1, 2)
    a = cov[:, 0, 0] + lowpass
    b = cov[:, 0, 1]
    cc = cov[:, 1, 1] + lowpass
    det = a * cc - b * b
    # forward uses 1/(det+1e-6), the backward differentiates 1/det with a 1e-8 guard on det^2
    # (gs3d.py:549 vs 575); on well-conditioned inputs both agree far below the test tolerance.
    det_inv = 1.0 / (det + 1e-6)
    ca, cb, ccn = cc * det_inv, -b * det_inv, a * det_inv
    if anti_aliasing:
        # d3sim/csrc/gs3d.py:592-619, d3sim/algos/d3gs/render.py:449-462: no eps guard on the inverse, the
        # determinant before the low-pass drives radius and validity, opacity *= sqrt(max(2.5e-5, det/det_lowpass))
        det_l = det
        det = (a - lowpass) * (cc - lowpass) - b * b
        ca, cb, ccn = cc / det_l, -b / det_l, a / det_l
        o = o * torch.sqrt(torch.clamp(det / det_l, min=0.000025))
    with torch.no_grad():
        mid = 0.5 * (a + cc)
        sq = torch.sqrt(torch.clamp(mid * mid - det, min=0.1))
        radius = torch.ceil(3.0 * torch.sqrt(torch.maximum(mid + sq, mid - sq)))
        tiles_x, tiles_y = (W + tile - 1) // tile, (H + tile - 1) // tile
        rminx = torch.clamp(torch.trunc((u - radius) / tile), 0, tiles_x)
        rminy = torch.clamp(torch.trunc((v - radius) / tile), 0, tiles_y)
        rmaxx = torch.clamp(torch.trunc((u + radius + tile - 1) / tile), 0, tiles_x)
        rmaxy = torch.clamp(torch.trunc((v + radius + tile - 1) / tile), 0, tiles_y)
        area = (rmaxx - rminx) * (rmaxy - rminy)
        visible = (det > 0) & (z >= near) & (z <= far) & (area > 0) & (o > alpha_eps)
    dirn = d / d.norm(dim=1, keepdim=True)
    basis = sh_basis(sh_degree, dirn)
    coeffs = torch.cat([params["sh_base"][:, None, :], params["sh_rest"]], dim=1)[:, : basis.shape[1], :]
    rgb_raw = (basis[:, :, None] * coeffs).sum(1) + 0.5
    neg = rgb_raw < 0
    rgb = torch.where(neg, torch.zeros_like(rgb_raw), rgb_raw)
    if clamp_mask_reference_order:
        # the reference gates channel k's gradient by bit k of (r<0)<<2 | (g<0)<<1 | (b<0)
        # (d3sim/algos/d3gs/render.py:608 vs 3344-3350): channel 0 is gated by b<0, channel 2 by r<0
        gate = torch.stack([neg[:, 2], neg[:, 1], neg[:, 0]], dim=1)
        rgb_val = rgb.detach()
        rgb = torch.where(gate, rgb_val, rgb_val + (rgb_raw - rgb_raw.detach()))
    dval = (1.0 / z) if depth_mode == "inv" else z
    order = torch.argsort((dval if depth_mode == "inv" else z).detach(), stable=True)
    ys, xs = torch.meshgrid(torch.arange(H, dtype=torch.float64), torch.arange(W, dtype=torch.float64), indexing="ij")
    tyi, txi = (ys // tile), (xs // tile)
    T = torch.ones(H, W, dtype=torch.float64)
    C = torch.zeros(H, W, 3, dtype=torch.float64)
    D = torch.zeros(H, W, dtype=torch.float64)
    Fi = None if custom is None else torch.zeros(H, W, custom.shape[1], dtype=torch.float64)
    done = torch.zeros(H, W, dtype=torch.bool)
    for g in order.tolist():
        if not bool(visible[g]):
            continue
        in_rect = (txi >= rminx[g]) & (txi < rmaxx[g]) & (tyi >= rminy[g]) & (tyi < rmaxy[g])
        dx, dy = u[g] - xs, v[g] - ys
        power = -0.5 * (ca[g] * dx * dx + ccn[g] * dy * dy) - cb[g] * dx * dy
        G = torch.exp(power)
        alpha = torch.clamp(o[g] * G, max=0.99)
        with torch.no_grad():
            ok = in_rect & ~done & (alpha >= alpha_eps)
            nT = T * (1 - alpha)
            should_done = ok & (nT < t_eps)
            done = done | should_done
            ok = ok & ~should_done & (power <= 0)
        w = torch.where(ok, alpha * T, torch.zeros_like(T))
        C = C + w[:, :, None] * rgb[g]
        D = D + w * dval[g]
        if custom is not None:
            Fi = Fi + w[:, :, None] * custom[g]
        T = torch.where(ok, T * (1 - alpha), T)
    extra = (() if depth_mode is None else (D,)) + (() if custom is None else (Fi,))
    return (C, T, visible) + extra


def ssim_l1_loss_torch(x_nchw, y_nchw, lambda_dssim=0.2, window_size=11, sigma=1.5):
    """0.8*L1 + 0.2*(1-SSIM) in the conv2d formulation of d3sim/ops/image/fused_ssim.py:63-81."""
    import torch.nn.functional as F
    ch = x_nchw.shape[1]
    g = torch.tensor([math.exp(-(i - window_size // 2) ** 2 / float(2 * sigma ** 2)) for i in range(window_size)],
                     dtype=x_nchw.dtype)
    g = g / g.sum()
    win = (g[:, None] @ g[None, :])[None, None].expand(ch, 1, window_size, window_size).contiguous()
    pad = window_size // 2
    mu1 = F.conv2d(x_nchw, win, padding=pad, groups=ch)
    mu2 = F.conv2d(y_nchw, win, padding=pad, groups=ch)
    s11 = F.conv2d(x_nchw * x_nchw, win, padding=pad, groups=ch) - mu1 * mu1
    s22 = F.conv2d(y_nchw * y_nchw, win, padding=pad, groups=ch) - mu2 * mu2
    s12 = F.conv2d(x_nchw * y_nchw, win, padding=pad, groups=ch) - mu1 * mu2
    C1, C2 = 0.01 ** 2, 0.03 ** 2
    ssim = ((2 * mu1 * mu2 + C1) * (2 * s12 + C2)) / ((mu1 * mu1 + mu2 * mu2 + C1) * (s11 + s22 + C2))
    l1 = (x_nchw - y_nchw).abs().mean()
    return (1 - lambda_dssim) * l1 + lambda_dssim * (1 - ssim.mean()), l1, ssim.mean()
