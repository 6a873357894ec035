"""One training iteration of 3D Gaussian splatting as a fused sequence of library calls.

``SplatTrainer.step`` performs what the reference's ``Trainer.train`` loop body does per iteration
(d3sim/algos/d3gs/train.py:162-217): rasterize (training) -> 0.8*L1 + 0.2*(1-SSIM) -> backward ->
Adam on the six parameter tensors -> densification statistics.  It drives the operator directly
(no autograd graph), keeps the 59-float-per-Gaussian gradient in one flat buffer, and issues Adam
plus statistics as one launch.

Data-parallel over views (one process per GPU, ``torch.distributed`` NCCL): every rank holds the full
Gaussian set and renders its own camera.  The reference's batch semantics are kept exactly: its loss
is a mean over B*C*H*W (train.py:170-172), so every per-view gradient carries 1/B and the per-Gaussian
gradient of the batch is the plain sum over views (render.py:3182-3199, origin/model.py:422-431).
Here each rank scales its loss gradient by 1/world_size and the flat gradient buffer is summed over the
ranks between the preprocess backward and the Adam launch.  With ``shard_optimizer`` (the default for
more than one rank) the sum is a reduce-scatter: every rank owns one contiguous slice of the flat
parameter buffer together with its Adam moments, updates only that slice, and an in-place all-gather
brings the updated slices back to every replica.  The bytes on the wire equal those of an all-reduce,
while the Adam launch, which is bound by HBM bandwidth, shrinks by the number of ranks.
Optimizer hyper-parameters are scaled with the global batch like tools.py:146-163.
"""
from __future__ import annotations

import math

import torch

from . import _lib, config_def
from .adam import _launch as _launch_adam
from .adam import make_stats_struct
from .fused_ssim import l1_dssim_forward_backward
from .model import FLAT_ORDER, GaussianModelOriginBase, carve_flat, flat_field_sizes
from .render import GaussianSplatGradients, GaussianSplatOp
from .strategy import GaussianTrainState
from .tools import get_expon_lr_func


def shard_layout(total: int, world: int, align: int = 4) -> tuple[int, int]:
    """``(shard_len, padded_total)``: equal slices of a flat buffer, each a multiple of ``align`` elements
    (16 bytes for float32) so that every slice starts on a vector boundary; the tail slice is padding."""
    s = -(-total // world)
    s = -(-s // align) * align
    return s, s * world


def clip_fields(offsets: dict, lo: int, hi: int) -> list[tuple[str, int, int]]:
    """Intersect the fields ``name -> (offset, count)`` of a flat buffer with the slice [lo, hi):
    ``[(name, start, count)]`` with ``start`` an absolute element index, empty intersections dropped."""
    out = []
    for name, (off, cnt) in offsets.items():
        a, b = max(off, lo), min(off + cnt, hi)
        if b > a:
            out.append((name, a, b - a))
    return out


def sharded_update(grad_flat: torch.Tensor, param_flat: torch.Tensor, grad_shard: torch.Tensor, rank: int,
                   group, apply_fn) -> None:
    """Reduce-scatter ``grad_flat`` (sum), let ``apply_fn(lo, hi, grad_shard)`` update ``param_flat[lo:hi]`` in
    place, then all-gather the slices in place.  Both flat buffers hold ``world * len(grad_shard)`` elements."""
    s = grad_shard.numel()
    lo, hi = rank * s, (rank + 1) * s
    torch.distributed.reduce_scatter_tensor(grad_shard, grad_flat, group=group)
    apply_fn(lo, hi, grad_shard)
    torch.distributed.all_gather_into_tensor(param_flat, param_flat[lo:hi], group=group)


class HostFeed:
    """Uploads per-step inputs that live in pinned host memory on a side stream, double buffered.

    ``push(host_tensor)`` starts the copy and returns ``(device_tensor, event)``; pass both to
    ``SplatTrainer.step`` so that the copy overlaps the preprocess/sort/raster kernels of the same step.
    A buffer is reused two pushes later; the copy into it first waits for the compute stream's work that
    was enqueued at the time of the push, which includes every reader of that buffer."""

    def __init__(self, device, slots: int = 2):
        self.device = device
        self.stream = torch.cuda.Stream(device=device)
        self.bufs: list[torch.Tensor | None] = [None] * slots
        self.k = 0

    def push(self, host: torch.Tensor):
        assert host.is_pinned(), "per-step inputs must be in pinned host memory for an asynchronous upload"
        i = self.k % len(self.bufs)
        self.k += 1
        if self.bufs[i] is None or self.bufs[i].shape != host.shape:
            self.bufs[i] = torch.empty(host.shape, dtype=host.dtype, device=self.device)
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            self.bufs[i].copy_(host, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return self.bufs[i], ev


class SplatTrainer:
    def __init__(self, model: GaussianModelOriginBase, op_cfg: config_def.GaussianSplatConfig,
                 lambda_dssim: float = 0.2, batch_size: int = 1, optim_cfg: config_def.Optimizer | None = None,
                 spatial_lr_scale: float = 1.0, process_group=None, need_max_radii: bool = False,
                 shard_optimizer: bool | None = None):
        """``batch_size`` is the GLOBAL number of views per iteration (= world size in data-parallel runs).
        ``shard_optimizer``: reduce-scatter + sliced Adam + all-gather instead of all-reduce + replicated
        Adam; default on when there is more than one rank."""
        assert model.has_fused_activations, "the trainer drives the fused-activation model"
        assert model.color_sh_base is not None and model.color_sh.shape[1] == 15, "degree-3 split SH layout"
        self.model = model
        self.pg = process_group
        self.world, self.rank = 1, 0
        if process_group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()):
            self.world = torch.distributed.get_world_size(process_group)
            self.rank = torch.distributed.get_rank(process_group)
        self.sharded = (self.world > 1) if shard_optimizer is None else (bool(shard_optimizer) and self.world > 1)
        n, dev = len(model), model.xyz.device
        total = 59 * n
        self.shard_len, padded = shard_layout(total, self.world) if self.sharded else (total, total)
        if model.flat is None or model.flat.numel() < padded:
            # move the parameters into one flat buffer (padded to a whole number of slices when the
            # optimizer is sharded); the model's tensors become views of it
            flat = torch.zeros(padded, dtype=torch.float32, device=dev)
            views = carve_flat(flat, n)
            for k in FLAT_ORDER:
                views[k].copy_(getattr(model, k).detach())
                setattr(model, k, views[k])
            model.flat = flat
        self.op = GaussianSplatOp(op_cfg)
        self.lambda_dssim = float(lambda_dssim)
        self.batch_size = int(batch_size)
        self.need_max_radii = need_max_radii
        self.grad_flat = torch.zeros(padded, dtype=torch.float32, device=dev)
        self.grad_model = type(model)(**carve_flat(self.grad_flat, n), cur_sh_degree=model.cur_sh_degree,
                                      act_applied=True, flat=self.grad_flat)
        # Adam moments: the whole buffer on one rank, only this rank's slice when sharded
        self.state_lo = self.rank * self.shard_len if self.sharded else 0
        self.grad_shard = torch.zeros(self.shard_len, dtype=torch.float32, device=dev) if self.sharded else None
        self.exp_avg = torch.zeros(self.shard_len, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.shard_len, dtype=torch.float32, device=dev)
        self.state = GaussianTrainState.create(n, device=dev)
        oc = optim_cfg or config_def.Optimizer()
        bs = math.sqrt(self.batch_size)                              # tools.py:147-163
        self.lrs = {"xyz": oc.position_lr_init * spatial_lr_scale * bs, "color_sh_base": oc.feature_lr * bs,
                    "color_sh": oc.feature_lr * bs / 20.0, "opacity": oc.opacity_lr * bs, "scale": oc.scaling_lr * bs,
                    "quaternion_xyzw": oc.rotation_lr * bs}
        self.eps = 1e-15 / bs
        self.betas = (1 - self.batch_size * (1 - 0.9), 1 - self.batch_size * (1 - 0.999))
        self.xyz_schedule = get_expon_lr_func(lr_init=oc.position_lr_init * spatial_lr_scale * bs,
                                              lr_final=oc.position_lr_final * spatial_lr_scale * bs,
                                              lr_delay_mult=oc.position_lr_delay_mult,
                                              max_steps=oc.position_lr_max_steps)
        self.use_xyz_schedule = False
        self.step_count = 0
        self._loss_scratch = None
        self._loss_sums = torch.zeros(2, dtype=torch.float64, device=dev)
        self._dcolor = None
        self._offsets = {}
        off = 0
        for name in FLAT_ORDER:
            cnt, _ = flat_field_sizes(n)[name]
            self._offsets[name] = (off, cnt)
            off += cnt

    # ------------------------------------------------------------------------------------------
    def _adam_segments(self):
        self.step_count += 1
        t = float(self.step_count)
        b1, b2 = self.betas
        bc1 = 1.0 - math.pow(b1, t)
        bc2s = math.sqrt(1.0 - math.pow(b2, t))
        if self.use_xyz_schedule:
            self.lrs["xyz"] = float(self.xyz_schedule(self.step_count))   # train.py:286-292
        segs = []
        esz = 4
        lo = self.state_lo
        grad = self.grad_shard if self.sharded else self.grad_flat   # both start at flat index `lo`
        for name, a, cnt in clip_fields(self._offsets, lo, lo + self.shard_len):
            s = _lib.AdamSegment()
            s.param = self.model.flat.data_ptr() + a * esz
            s.grad = grad.data_ptr() + (a - lo) * esz
            s.exp_avg = self.exp_avg.data_ptr() + (a - lo) * esz
            s.exp_avg_sq = self.exp_avg_sq.data_ptr() + (a - lo) * esz
            s.count = cnt
            s.lr, s.beta1, s.beta2, s.eps = float(self.lrs[name]), b1, b2, self.eps
            s.bias_correction1, s.bias_correction2_sqrt = bc1, bc2s
            s.grad_scale, s.weight_decay = 1.0, 0.0
            segs.append(s)
        return segs

    @torch.no_grad()
    def step(self, cameras, target_nchw: torch.Tensor, update: bool = True,
             target_ready: "torch.cuda.Event | None" = None) -> dict:
        """One iteration on this rank's view(s).  Returns ``{"out", "loss" (lazy), "num_rendered"}``.

        ``target_ready``: an event recorded after an asynchronous upload of ``target_nchw`` on another
        stream; the loss kernels wait for it, so the upload overlaps the forward pass."""
        model = self.model
        model.act_applied = True
        if self.op.timer is not None:
            self.op.timer.begin_step()
        out, ctx = self.op.forward(model, cameras, training=True)
        if ctx is None:  # nothing visible: zero gradient, still take part in the collective
            self.grad_flat.zero_()
            loss = None
            duv = None
        else:
            b, h, w, _ = out.color.shape
            nbytes = 3 * b * 3 * h * w * 4
            if self._loss_scratch is None or self._loss_scratch.numel() < nbytes:
                self._loss_scratch = torch.empty(nbytes, dtype=torch.uint8, device=out.color.device)
            if self._dcolor is None or self._dcolor.shape != out.color.shape:
                self._dcolor = torch.empty_like(out.color)
            if target_ready is not None:
                torch.cuda.current_stream(out.color.device).wait_event(target_ready)
            # the loss of a data-parallel batch is the mean over all ranks' views: 1/world per rank
            loss, dcolor = l1_dssim_forward_backward(out.color, target_nchw, self.lambda_dssim,
                                                     grad_scale=1.0 / self.world, scratch=self._loss_scratch,
                                                     sums=self._loss_sums, dcolor=self._dcolor)
            self.op._mark("l1_dssim")
            _, duv, _ =self.op.backward(model, cameras, ctx, out, GaussianSplatGradients(drgb=dcolor, dT=None),
                                         return_uv_grad=True, grad_out=self.grad_model)
        stats = None
        if update and duv is not None:
            w, h = out.image_shape_wh
            stats = make_stats_struct(self.state, out.radii, duv, w, h, self.need_max_radii,
                                      loss_batch=duv.shape[0] * self.world)
        if self.sharded and update:
            def apply(lo, hi, grad_shard):
                self.op._mark("reduce_scatter")
                _launch_adam(self._adam_segments(), stats, model.xyz.device)
                self.op._mark("adam_stats")
            sharded_update(self.grad_flat, model.flat, self.grad_shard, self.rank, self.pg, apply)
            self.op._mark("all_gather")
        else:
            if self.world > 1:
                torch.distributed.all_reduce(self.grad_flat, group=self.pg)
                self.op._mark("allreduce")
            if update:
                assert not self.sharded, "a sharded optimizer cannot apply a replicated update"
                _launch_adam(self._adam_segments(), stats, model.xyz.device)
                self.op._mark("adam_stats")
        return {"out": out, "loss": loss, "num_rendered": self.op.last_num_rendered}

    @torch.no_grad()
    def render(self, cameras) -> "torch.Tensor":
        """Forward-only rendering (inference mode: background composited, clamped)."""
        self.model.act_applied = True
        out, _ = self.op.forward(self.model, cameras, training=False)
        return out

    def reduce_stats(self):
        """All-reduce the densification statistics (each rank accumulates its own views' share)."""
        if self.world > 1:
            torch.distributed.all_reduce(self.state.duv_ndc_length, group=self.pg)
            torch.distributed.all_reduce(self.state.count, group=self.pg)
            torch.distributed.all_reduce(self.state.max_radii, op=torch.distributed.ReduceOp.MAX, group=self.pg)

    def parameter_checksum(self) -> torch.Tensor:
        """Sum of the raw parameter bits; replicas must agree after every update."""
        return self.model.flat[:59 * len(self.model)].view(torch.int32).sum(dtype=torch.int64)
