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
With ``peer_update`` (the default on NCCL when the buffers can be mapped) the three steps are one kernel
over NVLink memory of all ranks.  Preferred form (``"symm"``): the gradient, parameter and flag buffers are
torch symmetric memory (``SymmBuffer``); when the switch offers a multicast mapping the launch pulls its
slice of the gradient sum with one ``multimem.ld_reduce`` per element and pushes the new parameters with
one ``multimem.st``; without multicast it uses plain peer loads and stores.  The launches of the ranks are
ordered by flags inside the kernel (gradients ready / update done), so the step contains no host-side
collective at all.  Fallback form (``"ipc"``): ``PeerBuffer`` maps cudaMalloc buffers through CUDA IPC and
two one-element all-reduces order the launches.
Optimizer hyper-parameters are scaled with the global batch like tools.py:146-163.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib, config_def
from .adam import _launch as _launch_adam
from .adam import make_stats_struct
from .fused_ssim import l1_dssim_forward_backward
from .model import FLAT_ORDER, GaussianModelOriginBase, carve_flat, flat_layout
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


def check_same_count(n: int, device, group=None) -> None:
    """Data parallel with replicated Gaussians: every rank must hold the same number of them before the first
    exchange (the buffers the ranks share are cut by index).  Collective; raises on EVERY rank when they differ."""
    dist = torch.distributed
    t = torch.tensor([n, -n], dtype=torch.int64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    lo, hi = int(t[0].item()), -int(t[1].item())
    if lo != hi:
        raise RuntimeError(f"data-parallel ranks hold different Gaussian counts (between {lo} and {hi}; this rank {n}): "
                           "the replicas must be identical before the first gradient exchange")


class _DeviceSpan:
    """Lets torch alias raw device memory (``torch.as_tensor`` reads ``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, numel: int):
        self.__cuda_array_interface__ = {"shape": (numel,), "typestr": "<f4", "data": (ptr, False), "version": 2,
                                         "strides": None}


class PeerBuffer:
    """One float32 buffer per rank of a node, each mapped into every rank's process.

    ``tensor`` aliases this rank's buffer; ``ptrs[q]`` is rank q's buffer as mapped here.  Construction is
    collective over ``group``; it raises on every rank when any rank could not allocate or map."""

    def __init__(self, numel: int, device, group=None):
        dist = torch.distributed
        lib = _lib.load()
        self.numel, self.device, self.group = numel, device, group
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        self.world, self.rank = world, rank
        self.ptrs: list[int] = [0] * world
        self._own = 0
        ok = torch.ones(1, dtype=torch.int32, device=device)
        handle = C.create_string_buffer(_lib.PEER_HANDLE_BYTES)
        err = ""
        with torch.cuda.device(device):
            ptr = C.c_void_p()
            if lib.d3gs_peer_buffer_create(numel * 4, C.byref(ptr), handle) != 0:
                ok.zero_()
                err = _lib.last_error()
            else:
                self._own = ptr.value
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 0:
                self.close(collective=False)
                raise RuntimeError(f"peer buffer allocation failed on some rank ({err or 'not this one'})")
            handles = [None] * world
            dist.all_gather_object(handles, handle.raw, group=group)
            for q in range(world):
                if q == rank:
                    self.ptrs[q] = self._own
                    continue
                mapped = C.c_void_p()
                if lib.d3gs_peer_buffer_open(handles[q], C.byref(mapped)) != 0:
                    ok.zero_()
                    err = _lib.last_error()
                    break
                self.ptrs[q] = mapped.value
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 0:
                self.close(collective=False)
                raise RuntimeError(f"peer buffer mapping failed on some rank ({err or 'not this one'})")
        self.tensor = torch.as_tensor(_DeviceSpan(self._own, numel), device=device)
        assert self.tensor.data_ptr() == self._own, "torch copied the buffer instead of aliasing it"

    def close(self, collective: bool = True):
        """Unmap the peers' buffers, then (after every rank has unmapped) free this rank's."""
        lib = _lib.load()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for q, p in enumerate(self.ptrs):
                if p and q != self.rank:
                    lib.d3gs_peer_buffer_close(p)
            self.ptrs = [0] * self.world
            if collective:
                torch.distributed.barrier(group=self.group)
            if self._own:
                lib.d3gs_peer_buffer_destroy(self._own)
                self._own = 0
        self.tensor = None


class SymmBuffer:
    """One buffer per rank in torch symmetric memory (``torch.distributed._symmetric_memory``): every rank's
    copy is mapped into every process (``ptrs[q]``), and where the NVLink switch supports it the copies are also
    bound to one multicast address (``multicast_ptr``; 0 otherwise).  Construction is collective."""

    def __init__(self, numel: int, dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        dist = torch.distributed
        group = group if group is not None else dist.group.WORLD
        self.numel, self.device, self.group = numel, device, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:
            pass      # newer torch enables the group on first use
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        assert self.ptrs[self.rank] == self.tensor.data_ptr(), "symmetric memory: local pointer mismatch"
        mc = 0
        try:
            if self.handle.has_multicast_support(device.type, device.index):
                mc = int(self.handle.multicast_ptr)
        except Exception:
            mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.multicast_ptr = mc
        torch.cuda.synchronize(device)
        dist.barrier(group=group)     # every rank's buffer is zero before anybody writes into a peer's

    def close(self, collective: bool = True):
        torch.cuda.synchronize(self.device)
        if collective:
            torch.distributed.barrier(group=self.group)
        self.handle = None
        self.tensor = None


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
                 shard_optimizer: bool | None = None, peer_update: "bool | str | None" = None,
                 fuse_backward_adam: bool | None = None, multicast: bool | None = None,
                 fuse_exchange: bool | None = None):
        """``batch_size`` is the GLOBAL number of views per iteration (= world size in data-parallel runs).
        ``shard_optimizer``: reduce-scatter + sliced Adam + all-gather instead of all-reduce + replicated
        Adam; default on when there is more than one rank.  ``peer_update``: do the sharded update as one
        kernel over the ranks' mapped buffers: ``"symm"`` (torch symmetric memory, ordering by flags inside the
        kernel, switch multicast when available and ``multicast`` is not False), ``"ipc"`` / ``True`` (CUDA IPC
        buffers, plain peer accesses, two one-element all-reduces around the launch), ``False`` (NCCL
        reduce-scatter / all-gather).  Default on NCCL: ``"symm"``, then ``"ipc"``, then NCCL, whichever can be
        set up on every rank.
        ``fuse_exchange`` (with ``"symm"``; default on): the preprocess backward moves INTO the exchange launch.
        Every rank owns a contiguous range of the Gaussians; its launch reads every rank's per-splat raster
        gradients for that range over NVLink (65 bytes per Gaussian and peer instead of the 236 of the parameter
        gradient), runs the backward of all views, applies Adam and stores the new parameters into every
        replica.  ``step`` then needs the cameras of all ranks (``all_cameras``).
        ``fuse_backward_adam`` (single rank, one view per step; default on): the preprocess backward applies
        Adam as it produces the gradients, which are then never stored; ``grad_flat`` is not written."""
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
        if self.world > 1:
            check_same_count(n, dev, process_group)
        layout, total = flat_layout(n)
        self.flat_total = total
        self.shard_len, padded = shard_layout(total, self.world) if self.sharded else (total, total)
        self.peer_param = self.peer_grad = self.peer_flags = None
        self.multicast = False
        self.exchange = "nccl"      # how the gradient sum and the parameter broadcast travel: symm | ipc | nccl
        self._multicast_wanted = multicast
        can_peer = self.sharded and dev.type == "cuda" and self.world <= _lib.MAX_PEERS and \
            torch.distributed.get_backend(process_group) == "nccl"
        if peer_update is True:
            peer_update = "ipc"
        if peer_update in ("symm", "ipc"):
            assert can_peer, "peer_update needs a sharded optimizer on NCCL with at most 8 ranks"
            modes = [peer_update]
        elif peer_update is None and can_peer:
            modes = ["symm", "ipc"]
        else:
            modes = []
        for mode in modes:
            try:
                self._create_peer_buffers(mode, padded, dev)
                self.exchange = mode
                break
            except Exception:
                if peer_update is not None:
                    raise
                self._release_peer_buffers()
        if self.peer_param is not None or model.flat is None or model.flat.numel() < padded:
            # move the parameters into one flat buffer (padded to a whole number of slices when the
            # optimizer is sharded, inside the mapped buffer for the peer update); the model's tensors
            # become views of it
            flat = self.peer_param.tensor if self.peer_param is not None else \
                torch.zeros(padded, dtype=torch.float32, device=dev)
            views = carve_flat(flat, n)
            for k in FLAT_ORDER:
                views[k].copy_(getattr(model, k).detach())
                setattr(model, k, views[k])
            model.flat = flat
        if op_cfg.use_nchw or op_cfg.render_rgba or op_cfg.disable_builtin_rgb:
            raise NotImplementedError("SplatTrainer's fused loss reads the operator's NHWC RGB output: "
                                      "use_nchw / render_rgba are for GaussianSplatOp and rasterize_gaussians")
        self.op = GaussianSplatOp(op_cfg)
        self.fused_adam = (self.world == 1) if fuse_backward_adam is None else bool(fuse_backward_adam)
        assert not (self.fused_adam and self.world > 1), "the fused backward + Adam is the single-rank path"
        self.lambda_dssim = float(lambda_dssim)
        self.batch_size = int(batch_size)
        self.need_max_radii = need_max_radii
        self.grad_flat = self.peer_grad.tensor if self.peer_grad is not None else \
            torch.zeros(padded, dtype=torch.float32, device=dev)
        self._peerset = None
        self._epoch = 0
        self.peer_wait_limit = 0      # polls before a flag wait inside the exchange kernel gives up; 0 = default
        self.peer_lanes = 0           # fused exchange: lanes that share one Gaussian (1, 2, 4; 0 = the library's choice)
        self.fused_exchange = False
        self.peer_views = None
        if self.peer_param is not None:
            self._peerset = self._make_peerset(dev)
            self._bar = torch.zeros(1, dtype=torch.float32, device=dev)
        want_fx = self.exchange == "symm" if fuse_exchange is None else bool(fuse_exchange)
        assert not want_fx or self.exchange == "symm", "fuse_exchange needs the symmetric-memory exchange"
        if want_fx:
            self._setup_fused_exchange(n, dev)
        self.grad_model = type(model)(**carve_flat(self.grad_flat, n), cur_sh_degree=model.cur_sh_degree,
                                      act_applied=True, flat=self.grad_flat)
        # Adam moments: the whole buffer on one rank, only this rank's slice when sharded
        self.state_lo = self.rank * self.shard_len if self.sharded else 0
        self.grad_shard = torch.zeros(self.shard_len, dtype=torch.float32, device=dev) \
            if (self.sharded and self._peerset is None) else None
        if self.fused_exchange:     # moments of this rank's range of Gaussians, in the flat layout of that many Gaussians
            self.shard_len = flat_layout(self.range_len)[1]
            self.state_lo = 0
            self.grad_shard = None
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
        self._offsets = {name: (off, cnt) for name, (off, cnt, _) in layout.items()}

    # ------------------------------------------------------------------------------------------
    def _create_peer_buffers(self, mode: str, padded: int, dev) -> None:
        """Collective.  Raises on every rank when any rank could not set the buffers up."""
        dist = torch.distributed
        ok = torch.ones(1, dtype=torch.int32, device=dev)
        err = None
        try:
            if mode == "symm":
                self.peer_param = SymmBuffer(padded, torch.float32, dev, self.pg)
                self.peer_grad = SymmBuffer(padded, torch.float32, dev, self.pg)
                self.peer_flags = SymmBuffer(_lib.PEER_FLAG_WORDS, torch.int32, dev, self.pg)
            else:
                self.peer_param = PeerBuffer(padded, dev, self.pg)
                self.peer_grad = PeerBuffer(padded, dev, self.pg)
        except Exception as e:      # noqa: BLE001 -- any failure means "this mode is not available here"
            err = e
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.pg)
        if int(ok.item()) == 0:
            raise RuntimeError(f"peer buffers ({mode}) could not be set up on some rank: {err or 'not this one'}")

    def _release_peer_buffers(self) -> None:
        for b in (self.peer_flags, self.peer_grad, self.peer_param):
            if b is not None:
                try:
                    b.close(collective=False)
                except Exception:   # noqa: BLE001
                    pass
        self.peer_param = self.peer_grad = self.peer_flags = None

    def _make_peerset(self, dev) -> "_lib.PeerSet":
        ps = _lib.PeerSet()
        ps.world, ps.rank = self.world, self.rank
        for q in range(self.world):
            ps.grad[q], ps.param[q] = self.peer_grad.ptrs[q], self.peer_param.ptrs[q]
        ps.status = self.op._sync_words(dev).data_ptr() + 8   # the word every forward pass checks
        self.multicast = False
        if self.exchange == "symm":
            for q in range(self.world):
                ps.flags[q] = self.peer_flags.ptrs[q]
            gmc, pmc = self.peer_grad.multicast_ptr, self.peer_param.multicast_ptr
            if self._multicast_wanted is not False and gmc and pmc:
                ps.grad_mc, ps.param_mc = gmc, pmc
                self.multicast = True
            assert not (self._multicast_wanted is True and not self.multicast), \
                "multicast=True, but the symmetric buffers have no multicast mapping here"
        return ps

    def _setup_fused_exchange(self, n: int, dev) -> None:
        """Collective.  Ranges of Gaussians per rank (multiples of 256, the kernel's tile) and the symmetric buffer
        every rank writes its view's raster gradients and backward context into."""
        s = -(-n // self.world)
        self.range_len = -(-s // 256) * 256
        self.g_begin = min(self.rank * self.range_len, n)
        self.g_count = max(0, min(self.range_len, n - self.g_begin))
        sec = lambda nbytes: -(-nbytes // 256) * 256
        off_cov, off_rad = sec(n * 48), sec(n * 48) + sec(n * 12)
        off_ne0 = off_rad + sec(n * 4)
        total = off_ne0 + sec(n)
        self.peer_views = SymmBuffer(total // 4, torch.float32, dev, self.pg)
        raw = self.peer_views.tensor.view(torch.uint8)
        self.op.external = {
            "packed": raw[:n * 48].view(torch.float32).view(n, 12),
            "cov2d_vecs": raw[off_cov:off_cov + n * 12].view(torch.float32).view(n, 3),
            "radii": raw[off_rad:off_rad + n * 4].view(torch.int32),
            "sh_to_rgb_ne_0": raw[off_ne0:off_ne0 + n],
        }
        v = _lib.PeerViews()
        for q in range(self.world):
            base = self.peer_views.ptrs[q]
            v.splat_grads[q], v.cov2d_vecs[q] = base, base + off_cov
            v.radii[q], v.sh_to_rgb_ne_0[q] = base + off_rad, base + off_ne0
        self._views_struct = v
        self.fused_exchange = True

    def _fused_segments(self):
        """Six segments over this rank's range of Gaussians, moments in the range's own flat layout."""
        self.step_count += 1
        t = float(self.step_count)
        b1, b2 = self.betas
        bc1 = 1.0 - math.pow(b1, t)
        bc2s = math.sqrt(1.0 - math.pow(b2, t))
        if self.use_xyz_schedule:
            self.lrs["xyz"] = float(self.xyz_schedule(self.step_count))
        layout, _ = flat_layout(self.range_len)
        per = {"xyz": 3, "quaternion_xyzw": 4, "scale": 3, "opacity": 1, "color_sh_base": 3, "color_sh": 45}
        segs = []
        for name in FLAT_ORDER:
            off, _, _ = layout[name]
            s = _lib.AdamSegment()
            s.param = getattr(self.model, name).data_ptr() + self.g_begin * per[name] * 4
            s.grad = None
            s.exp_avg = self.exp_avg.data_ptr() + off * 4
            s.exp_avg_sq = self.exp_avg_sq.data_ptr() + off * 4
            s.count = per[name] * self.g_count
            s.lr, s.beta1, s.beta2, s.eps = float(self.lrs[name]), b1, b2, self.eps
            s.bias_correction1, s.bias_correction2_sqrt = bc1, bc2s
            s.grad_scale, s.weight_decay = 1.0, 0.0
            segs.append(s)
        return segs

    def _field_views(self, flat: torch.Tensor) -> dict:
        """Views of a flat buffer in this trainer's layout, shaped like the model's tensors."""
        return {name: flat[off:off + cnt].view(getattr(self.model, name).shape) for name, (off, cnt) in self._offsets.items()}

    @torch.no_grad()
    def refine(self, strategy, step: int, generator: "torch.Generator | None" = None) -> tuple:
        """Densify and prune between two training steps (``GaussianStrategyOrigin.refine_gs``,
        d3sim/algos/d3gs/origin/strategy.py:159-363; the trainer calls it every ``refine_every`` iterations
        between ``refine_start_iter`` and ``refine_stop_iter``, origin/trainer.py:377-386).  The model's tensors,
        the Adam moments, the gradient buffer and the statistics are rebuilt for the new Gaussian count.

        With several ranks the call is collective: the statistics are summed over the ranks first, every rank
        then takes the same decisions on its replica (the split children's normals come from a device generator
        seeded alike on all ranks), the sharded Adam moments are gathered for the call and cut into the new
        slices afterwards, and the buffers the ranks share (symmetric memory or CUDA IPC) are released and
        re-created for the new count.  Returns ``(n_keep, n_dup_kept, n_split_kept, n_split)``."""
        model, dev = self.model, self.model.xyz.device
        dist = torch.distributed
        if self.world > 1:
            self.reduce_stats()
            if generator is None:
                generator = torch.Generator(device=dev)
                generator.manual_seed(0x5EED0000 + int(step))
        full_m, full_v = self._gather_full_moments()   # the moments of the whole model, for the gather by source index
        m_views, v_views = self._field_views(full_m), self._field_views(full_v)
        moments = {name: (m_views[name], v_views[name]) for name in self._offsets}
        new_model, new_moments, _, totals = strategy.refine_tensors(model, moments, self.state, step, generator)
        n = len(new_model)
        if self.world > 1:   # the replicas must have taken the same decisions
            t = torch.tensor(list(totals), dtype=torch.int64, device=dev)
            lo, hi = t.clone(), t.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.pg)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.pg)
            assert bool((lo == hi).all().item()), f"ranks disagree on the refinement: {totals}"
        layout, total = flat_layout(n)
        self.flat_total = total
        self.shard_len, padded = shard_layout(total, self.world) if self.sharded else (total, total)
        self._offsets = {name: (off, cnt) for name, (off, cnt, _) in layout.items()}
        was_fused = self.fused_exchange
        if self.peer_param is not None:
            # the shared buffers have the old size: release them on every rank, then map new ones
            mode = self.exchange
            for k in FLAT_ORDER:
                setattr(model, k, None)
            model.flat = None
            self.grad_flat = self.grad_model = self._peerset = None
            self.op.external = None
            for b in (self.peer_views, self.peer_flags, self.peer_grad, self.peer_param):
                if b is not None:
                    b.close()
            self.peer_param = self.peer_grad = self.peer_flags = self.peer_views = None
            self.fused_exchange = False
            self._create_peer_buffers(mode, padded, dev)
            flat = self.peer_param.tensor
            self.grad_flat = self.peer_grad.tensor
        else:
            flat = torch.zeros(padded, dtype=torch.float32, device=dev)
            self.grad_flat = torch.zeros(padded, dtype=torch.float32, device=dev)
        views = carve_flat(flat, n)
        for k in FLAT_ORDER:
            views[k].copy_(getattr(new_model, k))
            setattr(model, k, views[k])
        model.flat = flat
        if self.peer_param is not None:
            self._peerset = self._make_peerset(dev)
            self._epoch = 0          # the new flag blocks start at zero
            if was_fused:
                self._setup_fused_exchange(n, dev)
        if self.fused_exchange:
            # this rank's range of Gaussians, field by field, into the range's own flat layout
            per = {"xyz": 3, "quaternion_xyzw": 4, "scale": 3, "opacity": 1, "color_sh_base": 3, "color_sh": 45}
            layout_s, self.shard_len = flat_layout(self.range_len)
            self.state_lo = 0
            self.exp_avg = torch.zeros(self.shard_len, dtype=torch.float32, device=dev)
            self.exp_avg_sq = torch.zeros(self.shard_len, dtype=torch.float32, device=dev)
            for name, (m, v) in new_moments.items():
                off_s = layout_s[name][0]
                lo, cnt = self.g_begin * per[name], self.g_count * per[name]
                self.exp_avg[off_s:off_s + cnt].copy_(m.reshape(-1)[lo:lo + cnt])
                self.exp_avg_sq[off_s:off_s + cnt].copy_(v.reshape(-1)[lo:lo + cnt])
            self.grad_shard = None
        else:
            # the new moments, in the flat layout, cut to this rank's slice
            new_m = torch.zeros(padded, dtype=torch.float32, device=dev)
            new_v = torch.zeros(padded, dtype=torch.float32, device=dev)
            for name, (m, v) in new_moments.items():
                off, cnt = self._offsets[name]
                new_m[off:off + cnt].copy_(m.reshape(-1))
                new_v[off:off + cnt].copy_(v.reshape(-1))
            self.state_lo = self.rank * self.shard_len if self.sharded else 0
            self.exp_avg = new_m[self.state_lo:self.state_lo + self.shard_len].clone()
            self.exp_avg_sq = new_v[self.state_lo:self.state_lo + self.shard_len].clone()
            self.grad_shard = torch.zeros(self.shard_len, dtype=torch.float32, device=dev) \
                if (self.sharded and self._peerset is None) else None
        self.grad_model = type(model)(**carve_flat(self.grad_flat, n), cur_sh_degree=model.cur_sh_degree,
                                      act_applied=True, flat=self.grad_flat)
        self.state = GaussianTrainState.create(n, self.state.scene_scale, device=dev)   # reset, origin/strategy.py:349
        if self.world > 1:
            torch.cuda.synchronize(dev)
            dist.barrier(group=self.pg)     # nobody starts a step before every replica is in place
        return totals

    def _gather_full_moments(self):
        """Both Adam moments of the whole model in the flat layout (collective when the optimizer is sharded)."""
        if not self.sharded:
            return self.exp_avg, self.exp_avg_sq
        dist, dev = torch.distributed, self.model.xyz.device
        if not self.fused_exchange:      # equal slices of the flat buffer
            out = []
            for src in (self.exp_avg, self.exp_avg_sq):
                full = torch.empty(self.shard_len * self.world, dtype=torch.float32, device=dev)
                dist.all_gather_into_tensor(full, src, group=self.pg)
                out.append(full)
            return out
        # ranges of Gaussians: the ranks' pieces of a field, in rank order, are the field
        layout_g, total = flat_layout(len(self.model))
        layout_s, _ = flat_layout(self.range_len)
        out = []
        for src in (self.exp_avg, self.exp_avg_sq):
            full = torch.zeros(total, dtype=torch.float32, device=dev)
            for name in FLAT_ORDER:
                off_s, cnt_s, _ = layout_s[name]
                off_g, cnt_g, _ = layout_g[name]
                gathered = torch.empty(self.world * cnt_s, dtype=torch.float32, device=dev)
                dist.all_gather_into_tensor(gathered, src[off_s:off_s + cnt_s].contiguous(), group=self.pg)
                full[off_g:off_g + cnt_g].copy_(gathered[:cnt_g])
            out.append(full)
        return out

    @torch.no_grad()
    def reset_opacity(self, strategy) -> None:
        """origin/trainer.py:388-417 on the trainer's buffers: clamp the opacities, zero their Adam moments.  With a
        sharded optimizer every rank clamps its own replica and zeroes the part of the opacity moments it holds."""
        off, cnt = self._offsets["opacity"]
        lib = _lib.load()
        dev = self.model.opacity.device
        if self.fused_exchange:      # this rank holds the opacity moments of its own range of Gaussians
            _lib.check(lib.d3gs_reset_opacity(self.model.opacity.data_ptr(), cnt, float(strategy.reset_opacity_thresh),
                                              int(self.model.has_fused_activations), None, None,
                                              torch.cuda.current_stream(dev).cuda_stream), "d3gs_reset_opacity")
            off_s = flat_layout(self.range_len)[0]["opacity"][0]
            self.exp_avg[off_s:off_s + self.range_len].zero_()
            self.exp_avg_sq[off_s:off_s + self.range_len].zero_()
            return
        lo, hi = max(off, self.state_lo), min(off + cnt, self.state_lo + self.shard_len)
        whole = lo == off and hi == off + cnt       # this rank holds the moments of every opacity
        _lib.check(lib.d3gs_reset_opacity(self.model.opacity.data_ptr(), cnt, float(strategy.reset_opacity_thresh),
                                          int(self.model.has_fused_activations),
                                          self.exp_avg.data_ptr() + (off - self.state_lo) * 4 if whole else None,
                                          self.exp_avg_sq.data_ptr() + (off - self.state_lo) * 4 if whole else None,
                                          torch.cuda.current_stream(dev).cuda_stream), "d3gs_reset_opacity")
        if not whole and hi > lo:
            self.exp_avg[lo - self.state_lo:hi - self.state_lo].zero_()
            self.exp_avg_sq[lo - self.state_lo:hi - self.state_lo].zero_()

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
        if self.grad_shard is not None:
            grad_ptr = self.grad_shard.data_ptr()              # reduce-scatter output: starts at flat index `lo`
        else:
            grad_ptr = self.grad_flat.data_ptr() + lo * esz    # this rank's flat gradient buffer
        for name, a, cnt in clip_fields(self._offsets, lo, lo + self.shard_len):
            s = _lib.AdamSegment()
            s.param = self.model.flat.data_ptr() + a * esz
            s.grad = grad_ptr + (a - lo) * esz
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
             target_ready: "torch.cuda.Event | None" = None, all_cameras=None) -> dict:
        """One iteration on this rank's view(s).  Returns ``{"out", "loss" (lazy), "num_rendered"}``.

        ``all_cameras`` (data parallel with the backward fused into the exchange): the cameras of all ranks in
        rank order, as a list of ``BasicPinholeCamera`` or a ``CameraBundle``.  Without it the ranks exchange
        their camera parameters through the process group every step (a small blocking collective).

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
            if self.fused_exchange and update:     # this view contributes nothing: radii == 0 everywhere
                self.op.external["radii"].zero_()
                return self._step_fused_exchange(cameras, all_cameras, None, out, None, None)
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
            if self.fused_exchange and update:
                return self._step_fused_exchange(cameras, all_cameras, ctx, out, dcolor, loss)
            fuse = self.fused_adam and update and out.color.shape[0] == 1
            w, h = out.image_shape_wh
            stats_fn = (lambda d: make_stats_struct(self.state, out.radii, d, w, h, self.need_max_radii,
                                                    loss_batch=d.shape[0] * self.world)) if fuse else None
            _, duv, _ = self.op.backward(model, cameras, ctx, out, GaussianSplatGradients(drgb=dcolor, dT=None),
                                         return_uv_grad=True, grad_out=None if fuse else self.grad_model,
                                         adam_segments=self._adam_segments() if fuse else None, stats_fn=stats_fn)
            if fuse:   # Adam and the densification statistics were part of the backward launch
                return {"out": out, "loss": loss, "num_rendered": self.op.last_num_rendered}
        stats = None
        if update and duv is not None:
            w, h = out.image_shape_wh
            stats = make_stats_struct(self.state, out.radii, duv, w, h, self.need_max_radii,
                                      loss_batch=duv.shape[0] * self.world)
        self.apply_gradients(stats, update)
        return {"out": out, "loss": loss, "num_rendered": self.op.last_num_rendered}

    def end_of_iteration(self, cur_step: int, strategy, generator: "torch.Generator | None" = None,
                         verbose: bool = False) -> list:
        """The reference trainer's period events for the iteration ``cur_step`` (0-based) that has just finished
        (d3sim/algos/d3gs/train.py:68-74, 299-320; d3sim/core/train.py:76-87: an event with interval p fires when
        ``(cur_step + 1) % p == 0``).  ``strategy``: a ``GaussianStrategyOrigin`` whose step counts were already
        rescaled for the batch size.

        * every ``1000 // batch_size`` iterations the active SH degree goes up by one until it is 3
          (train.py:299-302); the next forward and backward then evaluate one more band;
        * every ``refine_every`` iterations with ``refine_start_iter < cur_step + 1 < refine_stop_iter``:
          densify and prune (train.py:303-316);
        * every ``reset_opacity_every`` iterations before ``refine_stop_iter``: reset the opacities
          (train.py:318-320).

        Collective when there are several ranks (every rank calls it with the same ``cur_step``).  Returns the
        names of the events that fired, in the order the reference registers them."""
        fired = []
        step1 = cur_step + 1
        up_sh = max(1000 // self.batch_size, 1)
        if step1 % up_sh == 0 and self.model.cur_sh_degree < 3:
            self.model.cur_sh_degree += 1
            if self.grad_model is not None:
                self.grad_model.cur_sh_degree = self.model.cur_sh_degree
            fired.append("up_sh")
            if verbose:
                print(f"Up SH degree to {self.model.cur_sh_degree}")
        if step1 % max(strategy.refine_every, 1) == 0 and strategy.refine_start_iter < step1 < strategy.refine_stop_iter:
            self.refine(strategy, step1, generator)
            fired.append("update_gs")
            if verbose:
                print("REFINE GS!!!", len(self.model))
        if step1 % max(strategy.reset_opacity_every, 1) == 0 and step1 < strategy.refine_stop_iter:
            self.reset_opacity(strategy)
            fired.append("reset_opacity")
            if verbose:
                print("RESET GS OPACITY!!!", step1)
        return fired

    def _all_cameras(self, cameras, all_cameras):
        from .render import CameraBundle, _camera_rows
        if all_cameras is None:
            rows = torch.from_numpy(_camera_rows(cameras)).to(self.model.xyz.device)
            gathered = torch.empty(self.world * rows.numel(), dtype=rows.dtype, device=rows.device)
            torch.distributed.all_gather_into_tensor(gathered, rows.reshape(-1), group=self.pg)
            host = gathered.view(self.world, 16).cpu().numpy()
            return CameraBundle(None, cameras.image_shape_wh, None, None, host)
        if isinstance(all_cameras, (list, tuple)):
            key = id(all_cameras[0]), len(all_cameras)
            cached = getattr(self, "_cam_cache", None)
            if cached is None or cached[0] != key or cached[1] is not all_cameras:
                import numpy as np
                host = np.concatenate([_camera_rows(c) for c in all_cameras], axis=0)
                self._cam_cache = (key, all_cameras, CameraBundle(None, all_cameras[0].image_shape_wh, None, None, host))
            return self._cam_cache[2]
        return all_cameras

    def _step_fused_exchange(self, cameras, all_cameras, ctx, out, dcolor, loss) -> dict:
        """Raster backward of this rank's view into the shared buffer, then one launch that does the preprocess
        backward of all views for this rank's Gaussians, the gradient sum, Adam and the parameter broadcast."""
        model = self.model
        bundle = self._all_cameras(cameras, all_cameras)
        if ctx is not None:
            self.op.rasterize_forward_backward(model, ctx, out, GaussianSplatGradients(drgb=dcolor, dT=None), training=True)
        # The launch accumulates the statistics of this rank's Gaussians over ALL views (it reads every view's duv and
        # radii anyway): they come out summed over the ranks, each rank holding its own range; reduce_stats() (a
        # sum / max over ranks, the other ranges being zero here) puts them together when a refinement needs them.
        w, h = bundle.image_shape_wh
        st = _lib.DensifyStats()
        st.duv_ndc_length, st.count, st.max_radii = (self.state.duv_ndc_length.data_ptr(), self.state.count.data_ptr(),
                                                     self.state.max_radii.data_ptr())
        st.num, st.batch, st.width, st.height = len(model), self.world, int(w), int(h)
        st.need_max_radii, st.loss_batch = int(self.need_max_radii), self.world
        self._epoch += 1
        self._peerset.epoch = self._epoch
        self._peerset.wait_limit = int(self.peer_wait_limit)
        self._peerset.lanes_per_gaussian = int(self.peer_lanes)
        self.op.backward_adam_peers(model, bundle, self._views_struct, self.g_begin, self.g_count,
                                    self._fused_segments(), self._peerset, st)
        return {"out": out, "loss": loss, "num_rendered": self.op.last_num_rendered}

    @torch.no_grad()
    def apply_gradients(self, stats=None, update: bool = True) -> None:
        """Sum ``grad_flat`` over the ranks and take the Adam step (second half of ``step``)."""
        model = self.model
        if self._peerset is not None and update and self.exchange == "symm":
            # ordering by flags inside the launch: no host-side collective in the step
            self._epoch += 1
            self._peerset.epoch = self._epoch
            self._peerset.wait_limit = int(self.peer_wait_limit)
            _launch_adam(self._adam_segments(), stats, model.xyz.device, peers=self._peerset)
            self.op._mark("adam_stats")
        elif self._peerset is not None and update:
            torch.distributed.all_reduce(self._bar, group=self.pg)    # every rank's gradient is complete
            self.op._mark("barrier_grads")
            _launch_adam(self._adam_segments(), stats, model.xyz.device, peers=self._peerset)
            self.op._mark("adam_stats")
            torch.distributed.all_reduce(self._bar, group=self.pg)    # every rank's parameters are complete
            self.op._mark("barrier_params")
        elif self.sharded and update:
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

    @torch.no_grad()
    def render(self, cameras) -> "torch.Tensor":
        """Forward-only rendering (inference mode: background composited, clamped)."""
        self.model.act_applied = True
        out, _ = self.op.forward(self.model, cameras, training=False)
        return out

    def close(self):
        """Release the mapped peer buffers (collective).  The model's tensors are moved to ordinary memory."""
        if self.peer_param is None:
            return
        n = len(self.model)
        flat = self.model.flat.clone()
        views = carve_flat(flat, n)
        for k in FLAT_ORDER:
            setattr(self.model, k, views[k])
        self.model.flat = flat
        self.grad_flat = self.grad_model = None
        self._peerset = None
        self.op.external = None
        for b in (self.peer_views, self.peer_flags, self.peer_grad, self.peer_param):
            if b is not None:
                b.close()
        self.peer_param = self.peer_grad = self.peer_flags = self.peer_views = None

    def reduce_stats(self):
        """All-reduce the densification statistics (each rank accumulates its own views' share)."""
        if self.world > 1:
            torch.distributed.all_reduce(self.state.duv_ndc_length, group=self.pg)
            torch.distributed.all_reduce(self.state.count, group=self.pg)
            torch.distributed.all_reduce(self.state.max_radii, op=torch.distributed.ReduceOp.MAX, group=self.pg)

    def update_path_name(self) -> str:
        """Which of the update paths this trainer takes (for logs and benchmark records)."""
        if self.world == 1:
            return "single rank, Adam inside the preprocess backward" if self.fused_adam else \
                "single rank, gradient buffer + optimizer kernel"
        if self.fused_exchange:
            return ("sharded by Gaussian range, ONE launch over symmetric memory: preprocess backward of all ranks' views "
                    "from their raster gradients (peer loads), gradient sum, Adam, parameters stored to every replica; "
                    "launches ordered by flags inside the kernel")
        if self._peerset is not None and self.exchange == "symm":
            how = ("multimem.ld_reduce / multimem.st through the NVLink switch" if self.multicast else
                   "plain peer loads and stores (no multicast mapping)")
            return ("sharded, one kernel over symmetric memory: gradient slice summed and parameters broadcast by "
                    f"{how}, Adam on the slice, launches ordered by flags inside the kernel")
        if self._peerset is not None:
            return ("sharded, one kernel over NVLink peer memory (CUDA IPC): sum of all ranks' gradient slices, Adam, "
                    "store to all ranks' parameters; two one-element all-reduces order the launches")
        if self.sharded:
            return "sharded: reduce-scatter, Adam on 1/N slice, all-gather"
        return "replicated after all-reduce"

    def parameter_checksum(self) -> torch.Tensor:
        """Sum of the raw parameter bits; replicas must agree after every update."""
        return self.model.flat[:self.flat_total].view(torch.int32).sum(dtype=torch.int64)
