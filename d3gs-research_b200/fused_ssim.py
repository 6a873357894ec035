"""Fused SSIM and fused L1 + D-SSIM loss: drop-in for ``d3sim.ops.image.fused_ssim``.

``fused_ssim_loss(pred, target, window_size=11, size_average=True, pred_is_nhwc=False)`` keeps the
reference signature (d3sim/ops/image/fused_ssim.py:411-416) and its autograd behaviour
(``_FusedSSIMMap``, 379-409).  ``l1_dssim_loss`` is the fused form of the reference's training loss
``(1-lambda)*l1_loss(color, gt) + lambda*(1 - fused_ssim_loss(color, gt))`` (d3sim/algos/d3gs/train.py:
169-172): it consumes the rasteriser's NHWC colour directly and produces dL/dcolor in NHWC in two
kernel launches.
"""
from __future__ import annotations

import torch

from . import _lib


def _stream(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def ssim_forward(images_x: torch.Tensor, images_y: torch.Tensor, window_size: int, training: bool = True,
                 imgx_is_nhwc: bool = False):
    """fused_ssim.py:93-238.  Returns (ssim_map NCHW, (dmu1, dmu11, dmu12))."""
    assert window_size == 11, "only the 11x11 window is built"
    assert images_x.is_contiguous() and images_y.is_contiguous()
    assert images_x.ndim == 4 and images_y.ndim == 4
    assert images_x.size(-1 if imgx_is_nhwc else -3) == 3 and images_y.size(-3) == 3, "3 channels"
    lib = _lib.load()
    b, _, h, w = images_y.shape
    ssim_res = torch.empty_like(images_y)
    mus = tuple(torch.empty_like(images_y) for _ in range(3)) if training else (None, None, None)
    _lib.check(lib.d3gs_ssim_forward(images_x.data_ptr(), images_y.data_ptr(), b, h, w, int(imgx_is_nhwc),
                                     ssim_res.data_ptr(), _lib.ptr(mus[0]), _lib.ptr(mus[1]), _lib.ptr(mus[2]),
                                     _stream(images_y)), "d3gs_ssim_forward")
    return ssim_res, mus


def ssim_backward(dssim_map: torch.Tensor, mu_tensors, images_x: torch.Tensor, images_y: torch.Tensor,
                  window_size: int, imgx_is_nhwc: bool = False):
    """fused_ssim.py:240-377."""
    lib = _lib.load()
    b, _, h, w = images_y.shape
    dimages_x = torch.empty_like(images_x)
    _lib.check(lib.d3gs_ssim_backward(dssim_map.data_ptr(), mu_tensors[0].data_ptr(), mu_tensors[1].data_ptr(),
                                      mu_tensors[2].data_ptr(), images_x.data_ptr(), images_y.data_ptr(), b, h, w,
                                      int(imgx_is_nhwc), dimages_x.data_ptr(), _stream(images_y)), "d3gs_ssim_backward")
    return dimages_x


class _FusedSSIMMap(torch.autograd.Function):
    @staticmethod
    def forward(ctx, images_x, images_y, window_size: int, training: bool = True, imgx_is_nhwc: bool = False):
        res, mus = ssim_forward(images_x.detach(), images_y.detach(), window_size, training, imgx_is_nhwc)
        if training:
            ctx.save_for_backward(images_x, images_y, *mus)
        ctx.window_size = window_size
        ctx.imgx_is_nhwc = imgx_is_nhwc
        return res

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dssim_map):
        x, y, *mus = ctx.saved_tensors
        dx = ssim_backward(dssim_map.contiguous(), mus, x, y, ctx.window_size, ctx.imgx_is_nhwc)
        return dx, None, None, None, None


def fused_ssim_loss(pred: torch.Tensor, target: torch.Tensor, window_size: int = 11, size_average: bool = True,
                    pred_is_nhwc: bool = False):
    res = _FusedSSIMMap.apply(pred, target, window_size, True, pred_is_nhwc)
    if size_average:
        return res.mean()
    return res.mean(1).mean(1).mean(1)


class L1DSSIMResult:
    """Lazy loss value: the sums stay on the device until ``loss()``/``item()`` is asked for."""

    def __init__(self, sums: torch.Tensor, n: int, lambda_dssim: float):
        self.sums, self.n, self.lambda_dssim = sums, n, lambda_dssim

    def loss(self) -> torch.Tensor:
        l1 = self.sums[0] / self.n
        ssim = self.sums[1] / self.n
        return ((1.0 - self.lambda_dssim) * l1 + self.lambda_dssim * (1.0 - ssim)).float()

    def item(self) -> float:
        return float(self.loss().item())


def l1_dssim_forward_backward(color_nhwc: torch.Tensor, target_nchw: torch.Tensor, lambda_dssim: float = 0.2,
                              grad_scale: float = 1.0, want_grad: bool = True, scratch: torch.Tensor | None = None,
                              sums: torch.Tensor | None = None, dcolor: torch.Tensor | None = None):
    """Loss sums and dL/dcolor (NHWC) of (1-lambda)*mean|x-y| + lambda*(1-mean SSIM), pre-multiplied by
    ``grad_scale``.  Returns ``(L1DSSIMResult, dcolor | None)``."""
    assert color_nhwc.is_contiguous() and target_nchw.is_contiguous()
    b, h, w, c = color_nhwc.shape
    assert c == 3 and tuple(target_nchw.shape) == (b, 3, h, w)
    lib = _lib.load()
    dev = color_nhwc.device
    if sums is None:
        sums = torch.empty(2, dtype=torch.float64, device=dev)
    nbytes = lib.d3gs_l1_dssim_scratch_bytes(b, h, w)
    if want_grad:
        if scratch is None or scratch.numel() * scratch.element_size() < nbytes:
            scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        if dcolor is None:
            dcolor = torch.empty_like(color_nhwc)
    _lib.check(lib.d3gs_l1_dssim_forward_backward(color_nhwc.data_ptr(), target_nchw.data_ptr(), b, h, w,
                                                  float(lambda_dssim), float(grad_scale), sums.data_ptr(),
                                                  _lib.ptr(dcolor) if want_grad else None,
                                                  _lib.ptr(scratch) if want_grad else None,
                                                  scratch.numel() * scratch.element_size() if want_grad else 0,
                                                  _stream(color_nhwc)), "d3gs_l1_dssim_forward_backward")
    return L1DSSIMResult(sums, b * 3 * h * w, lambda_dssim), (dcolor if want_grad else None)


class _L1DSSIMLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, color_nhwc, target_nchw, lambda_dssim: float):
        res, dcolor = l1_dssim_forward_backward(color_nhwc.detach().contiguous(), target_nchw.detach().contiguous(),
                                                lambda_dssim)
        ctx.save_for_backward(dcolor)
        return res.loss()

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dloss):
        (dcolor,) = ctx.saved_tensors
        return dcolor * dloss, None, None


def l1_dssim_loss(color_nhwc: torch.Tensor, target_nchw: torch.Tensor, lambda_dssim: float = 0.2) -> torch.Tensor:
    """Scalar training loss with autograd: ``(1-l)*L1 + l*(1-SSIM)`` for NHWC colour and NCHW target."""
    return _L1DSSIMLoss.apply(color_nhwc, target_nchw, lambda_dssim)


def l1_loss(network_output: torch.Tensor, gt: torch.Tensor) -> torch.Tensor:
    """d3sim/algos/d3gs/losses.py:19-20."""
    return torch.abs(network_output - gt).mean()
