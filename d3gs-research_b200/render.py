"""The splat operator: drop-in for ``d3sim.algos.d3gs.render``.

Same public names, argument order, tensor shapes and dtypes as the reference
(d3sim/algos/d3gs/render.py): ``GaussianSplatOp(cfg).forward / .backward``,
``rasterize_gaussians``, ``rasterize_gaussians_dynamic``, ``CameraBundle``, ``GaussianSplatOutput``,
``GaussianSplatOpContext``, ``GaussianSplatGradients``.  Where the reference launches NVRTC-compiled
kernel strings through cumm (render.py:676-681, 839-840, 937-939, 2308-2309, 3361-3369) and calls a
pybind wrapper of cub's radix sort (render.py:845-887), this module calls the ahead-of-time
sm_100a library through its C ABI on torch's current stream.  All buffers are torch allocations;
the library allocates nothing.
"""
from __future__ import annotations

import copy
import ctypes as C
import dataclasses
from typing import Any

import numpy as np
import torch

from . import _lib
from .camera import BasicPinholeCamera
from .config_def import EarlyFilterAlgo, GaussianSplatConfig, RasterizeBackwardAlgo
from .model import GaussianModelOriginBase, carve_flat, flat_layout


def div_up(a: int, b: int) -> int:
    return (a + b - 1) // b


@dataclasses.dataclass
class GaussianSplatOpContext:
    """Per-(view, Gaussian) tensors kept for the backward pass (render.py:57-72)."""
    conic_opacity: torch.Tensor
    radii: torch.Tensor
    uvs: torch.Tensor
    rgb_gaussian: torch.Tensor | None
    gaussian_idx_sorted: torch.Tensor
    workload_ranges: torch.Tensor
    image_shape_wh: tuple[int, int]
    depths: torch.Tensor
    cov2d_vecs: torch.Tensor | None = None
    sh_to_rgb_ne_0: torch.Tensor | None = None
    per_gaussian_snap: Any = None
    # not in the reference: the sorted, contiguous 48-byte splat records the raster kernels stream, and the
    # order in which their CTAs take the tiles (longest lists first)
    splat_records: torch.Tensor | None = None
    tile_order: torch.Tensor | None = None
    records_by_id: bool = False   # splat_records is the per-Gaussian table (gathered by sorted id), not per pair
    raster_color: torch.Tensor | None = None   # the kernels' [B,H,W,3] colour when out.color is a re-formatted copy
    # Quantities blended like a colour (render_depth, custom_features), three channels per extra raster pass:
    # for every pass (records with those values in the colour slots, their [B,H,W,3] blend)
    aux_passes: list | None = None
    num_custom_feat: int = 0
    # sparse_mode: the per-item tensors above hold the kept items only; which Gaussian / view each is, and N
    sparse_gaussian_ids: torch.Tensor | None = None
    sparse_batch_ids: torch.Tensor | None = None
    num_gaussians: int = 0


@dataclasses.dataclass
class GaussianSplatOutput:
    """render.py:74-100.  ``color`` is NHWC [B,H,W,3]; in training it is not composited with a background."""
    custom_features: torch.Tensor | None
    T: torch.Tensor
    color: torch.Tensor
    depth: torch.Tensor | None = None
    n_contrib: torch.Tensor | None = None
    radii: torch.Tensor | None = None
    sparse_gaussian_ids: torch.Tensor | None = None
    sparse_batch_ids: torch.Tensor | None = None

    @property
    def image_shape_wh(self) -> tuple[int, int]:
        return (self.T.shape[2], self.T.shape[1])

    def select_batch(self, batch_idx: int):
        sl = slice(batch_idx, batch_idx + 1)
        return GaussianSplatOutput(
            custom_features=None if self.custom_features is None else self.custom_features[sl],
            T=self.T[sl], color=self.color[sl], depth=None if self.depth is None else self.depth[sl],
            n_contrib=None if self.n_contrib is None else self.n_contrib[sl],
            radii=None if self.radii is None else self.radii[sl])


@dataclasses.dataclass
class RasterizeGradientOutput:
    """render.py:103-111."""
    duv: torch.Tensor
    dconic: torch.Tensor
    dopacity: torch.Tensor
    dcolor: torch.Tensor | None
    dcustom_features: torch.Tensor | None = None
    dz: torch.Tensor | None = None
    # not in the reference: the [B*N,12] array the four tensors above are views of
    packed: torch.Tensor | None = None


@dataclasses.dataclass
class GaussianSplatGradients:
    """render.py:113-120."""
    drgb: torch.Tensor
    dT: torch.Tensor | None
    ddepth: torch.Tensor | None = None
    dcustom_features: torch.Tensor | None = None


@dataclasses.dataclass
class CameraParamBundle:
    focal_xy_ppoint: torch.Tensor
    image_shape_wh: tuple[int, int]
    frame_ids: torch.Tensor | None


@dataclasses.dataclass
class CameraBundle(CameraParamBundle):
    """A batch of pinhole cameras (render.py:122-150): ``cam2world_T`` [B,4,3], ``focal_xy_ppoint`` [B,4]."""
    cam2world_T: torch.Tensor = None
    _host: np.ndarray | None = dataclasses.field(default=None, repr=False, compare=False)

    @classmethod
    def from_pinhole_cams(cls, cams: list[BasicPinholeCamera], device: torch.device | str = "cuda"):
        c2w_t = np.stack([np.ascontiguousarray(cam.pose.to_world[:3].T) for cam in cams], axis=0).reshape(-1, 4, 3)
        fpp = np.concatenate([np.stack([cam.focal_length for cam in cams]).reshape(-1, 2),
                              np.stack([cam.principal_point for cam in cams]).reshape(-1, 2)], axis=1)
        frame_ids = None
        if cams[0].frame_local_id is not None:
            frame_ids = torch.tensor([cam.frame_local_id for cam in cams], dtype=torch.int32, device=device)
        host = np.concatenate([c2w_t.reshape(-1, 12), fpp], axis=1).astype(np.float32)
        return cls(torch.from_numpy(np.ascontiguousarray(fpp.astype(np.float32))).to(device), cams[0].image_shape_wh,
                   frame_ids, torch.from_numpy(np.ascontiguousarray(c2w_t.astype(np.float32))).to(device), host)

    def host_params(self) -> np.ndarray:
        """[B,16] float32 on the host (one device read, cached)."""
        if self._host is None:
            c2w = self.cam2world_T.detach().float().cpu().numpy().reshape(-1, 12)
            fpp = self.focal_xy_ppoint.detach().float().cpu().numpy().reshape(-1, 4)
            self._host = np.concatenate([c2w, fpp], axis=1).astype(np.float32)
        return self._host


def _camera_rows(cameras: BasicPinholeCamera | CameraBundle) -> np.ndarray:
    if isinstance(cameras, BasicPinholeCamera):
        k = cameras.intrinsic
        c2w_t = np.ascontiguousarray(cameras.pose.to_world[:3].T).reshape(12)     # render.py:205
        return np.concatenate([c2w_t, [k[0, 0], k[1, 1], k[0, 2], k[1, 2]]]).astype(np.float32)[None]
    return cameras.host_params()


def _sort_class(longest: int) -> int:
    """Which instance of the tile sort a list of this length needs (d3gs_bucket_sort: <= 512, <= 2048, larger)."""
    return 0 if longest <= 512 else (1 if longest <= 2048 else 2)


def _pair_capacity(n: int) -> int:
    """Allocation size for a buffer of n (tile, splat) pairs: n + n/8, rounded up to a multiple of 2^20."""
    q = 1 << 20
    return max(-(-(n + n // 8) // q) * q, q)


class _Workspace:
    """Grow-only scratch tensors so that the steady state performs no allocation for them."""

    def __init__(self):
        self.bufs: dict[str, torch.Tensor] = {}

    def get(self, name: str, nbytes: int, device) -> torch.Tensor:
        t = self.bufs.get(name)
        if t is None or t.numel() < nbytes or t.device != device:
            t = torch.empty(max(int(nbytes * 1.25), 256), dtype=torch.uint8, device=device)
            self.bufs[name] = t
        return t


class StageTimer:
    """CUDA-event marks on the launching stream, the counterpart of the reference's
    ``measure_and_print_torch(name, enable=cfg.verbose)`` blocks (render.py:250, 689, 739, 845, 896, 1004).
    ``mark(name)`` closes the stage ``name``; durations are read after a synchronize."""

    def __init__(self, prealloc: int = 0):
        """``prealloc``: number of events to create up front (a CUDA event is created by its first record; inside
        a timed loop that creation is host work between two launches)."""
        self.steps: list[list[tuple[str, torch.cuda.Event]]] = []
        self.pool: list[torch.cuda.Event] = []
        for _ in range(prealloc):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.pool.append(ev)

    def _event(self) -> torch.cuda.Event:
        ev = self.pool.pop() if self.pool else torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    def begin_step(self):
        self.steps.append([("begin", self._event())])

    def mark(self, name: str):
        if not self.steps:
            self.begin_step()
        self.steps[-1].append((name, self._event()))

    def summary(self, median: bool = False) -> dict[str, float]:
        """Milliseconds per stage over the recorded steps (call after torch.cuda.synchronize()): the mean, or
        the per-stage median, which ignores a one-off stall of a single step."""
        acc: dict[str, list[float]] = {}
        for marks in self.steps:
            per: dict[str, float] = {}
            for (_, e0), (name, e1) in zip(marks[:-1], marks[1:]):
                per[name] = per.get(name, 0.0) + e0.elapsed_time(e1)
            for k, v in per.items():
                acc.setdefault(k, []).append(v)
        if median:
            return {k: sorted(v)[len(v) // 2] for k, v in acc.items()}
        n = max(len(self.steps), 1)
        return {k: sum(v) / n for k, v in acc.items()}


class GaussianSplatOp:
    """render.py:152-167.  ``cfg`` is deep-copied: create a new op to change options."""

    # sort pairs per (view, Gaussian) below which the raster backward skips its shared-memory accumulation
    DIRECT_ATOMICS_PAIRS_PER_GAUSSIAN = 3.0

    def __init__(self, cfg: GaussianSplatConfig) -> None:
        self._cfg = copy.deepcopy(cfg)
        bad = self._cfg.unsupported_options()
        if bad:
            raise NotImplementedError("GaussianSplatConfig options not built in this library: " + ", ".join(bad))
        self._lib = _lib.load()
        self._ws = _Workspace()
        self._sync: dict[Any, torch.Tensor] = {}
        self.last_num_rendered = 0
        # when True, forward() keeps copies of the intermediate binning arrays in ``self.debug`` (tests)
        self.debug_capture = False
        # True: the preprocess writes one raster record per Gaussian and the raster kernels gather them by sorted
        # id; False: d3gs_pack_splats writes one record per sorted (tile, splat) pair and the raster kernels stream
        # them with bulk copies (one more pass over the pairs; same results)
        self.gather_records = True
        # Raster backward: True = every group of four lanes adds its per-splat sums to global memory directly,
        # False = per-tile accumulation in shared memory first, None = chosen per call from the number of sort
        # pairs per Gaussian (small splats -> direct).  Same gradients up to the order of the float additions.
        self.raster_grad_direct: bool | None = None
        # How the sorted per-tile lists are built.  "bucket": the preprocess counts the pairs of every tile, the
        # pairs are written straight into their tile's range and every tile's list is sorted in shared memory
        # (d3gs_bucket_*); "sort": key duplication, global radix sort and range extraction like the reference.
        # Same lists and ranges bit for bit.  "bucket" falls back to "sort" for a launch whose longest list does
        # not fit one CTA's shared memory, and is not used with 32-bit sort keys.
        self.binning = "bucket"
        self.last_binning = ""
        # Bucket binning only.  True: from the second launch of a shape on, the pair buffers are sized from the
        # previous launch's pair count (+ 12.5 %, quantised), the binning and raster kernels are queued at once and
        # check the count on the device, and the host reads the count (one copy on a side stream, as the reference's
        # one read per forward) while they run; a launch whose count outgrew the buffers, or whose longest list
        # outgrew the sort classes that were launched, is repeated with the true sizes (``launches_repeated``).
        # False: the host waits for the count before it launches, like the reference (render.py:695).
        self.launch_ahead = True
        self.launches_repeated = 0
        # measure_atomic_add_count: groups of global atomic adds of the last raster backward, and more detail
        self.last_atomic_add_count: int | None = None
        self.last_atomic_stats: dict = {}
        self._ahead: dict = {}
        self._readback: dict = {}
        # Optional caller-owned tensors for what a later stage on ANOTHER GPU reads (data-parallel training with
        # the backward fused into the exchange): keys "radii" [N] int32, "cov2d_vecs" [N,3], "sh_to_rgb_ne_0" [N]
        # uint8 (written by forward) and "packed" [N,12] (written by the raster backward); single-view launches.
        self.external: dict[str, torch.Tensor] | None = None
        self.debug: dict[str, torch.Tensor] = {}
        # optional StageTimer; None = no events recorded
        self.timer: StageTimer | None = None

    def _mark(self, name: str):
        if self.timer is not None:
            self.timer.mark(name)

    @property
    def is_nchw(self):
        return self._cfg.use_nchw

    @property
    def is_rgba(self):
        return self._cfg.render_rgba

    # ---- plumbing ---------------------------------------------------------------------------
    def _sync_words(self, device) -> torch.Tensor:
        """int64[4] on the device: [num_rendered, status bits, longest tile list, unused]; read back with one copy."""
        t = self._sync.get(device)
        if t is None:
            t = torch.zeros(4, dtype=torch.int64, device=device)
            self._sync[device] = t
        return t

    def _read_sync_words_async(self, dev, sync):
        """Copy the four sync words to pinned host memory on a side stream, ordered after what the current stream
        has queued so far.  Returns a function that waits for that copy alone and returns the words."""
        rb = self._readback.get(dev)
        if rb is None:
            rb = (torch.empty(4, dtype=torch.int64).pin_memory(), torch.cuda.Stream(dev), torch.cuda.Event(),
                  torch.cuda.Event())
            self._readback[dev] = rb
        host, side, ready, done = rb
        ready.record(torch.cuda.current_stream(dev))
        side.wait_event(ready)
        with torch.cuda.stream(side):
            host.copy_(sync, non_blocking=True)
            done.record(side)

        def wait():
            done.synchronize()
            return tuple(int(v) for v in host.tolist())
        return wait

    def check_status(self, device=None) -> None:
        """Read the device status word (one 8-byte copy), clear it and raise if a bounded wait of any kernel
        launched through this operator gave up.  ``forward`` checks the word with its own read-back, which
        covers everything launched before it; call this after the LAST forward / backward / optimizer launch of
        a run, where no further forward follows."""
        for dev, sync in self._sync.items():
            if device is not None and dev != device:
                continue
            status = int(sync[1].item())
            if status != 0:
                sync[1] = 0
                raise RuntimeError(f"d3gs_b200 device status {status:#x}: a bounded wait gave up "
                                   "(1 scan, 2 sort, 4 bulk copy); results of the previous call are invalid")

    def _op_config(self, model: GaussianModelOriginBase, cameras, training: bool,
                   instance2world_T: torch.Tensor | None = None) -> _lib.OpConfig:
        cfg = self._cfg
        rows = _camera_rows(cameras)
        if rows.shape[0] > _lib.MAX_VIEWS:
            raise NotImplementedError(f"at most {_lib.MAX_VIEWS} views per launch (got {rows.shape[0]})")
        w, h = cameras.image_shape_wh
        c = _lib.OpConfig()
        c.width, c.height = int(w), int(h)
        c.tile_x, c.tile_y = int(cfg.tile_size[0]), int(cfg.tile_size[1])
        c.near_plane, c.far_plane, c.eps = cfg.near, cfg.far, cfg.eps
        c.cov2d_radii_eigen_eps = cfg.cov2d_radii_eigen_eps
        c.projected_clamp_factor = cfg.projected_clamp_factor
        c.gaussian_std_sigma = cfg.gaussian_std_sigma
        c.gaussian_lowpass_filter = cfg.gaussian_lowpass_filter
        c.alpha_eps = cfg.alpha_eps
        c.transmittance_eps = cfg.transmittance_eps
        c.scale_global = cfg.scale_global
        c.early_filter_algo = int(cfg.early_filter_algo)
        c.sh_degree = int(model.cur_sh_degree)
        c.training = int(bool(training))
        c.clamp_mask_reference_order = int(bool(cfg.clamp_mask_reference_order))
        c.fused_activations = int(model.has_fused_activations)
        bg = np.asarray(cfg.bg_color, np.float32).reshape(-1)
        for k in range(3):
            c.bg_color[k] = float(bg[k])
        # enable_32bit_sort (render.py:227-228, 737, 767-770): 14 bits of tile index over an 18-bit quantised depth
        c.key_shift_bits = 18 if cfg.enable_32bit_sort else 32
        c.depth_32bit_prec = float(cfg.depth_32bit_prec)
        c.anti_aliasing = int(bool(cfg.enable_anti_aliasing))
        c.inv_depth = int(bool(cfg.render_inv_depth))
        c.num_views = rows.shape[0]
        if cfg.enable_32bit_sort:
            assert rows.shape[0] * div_up(int(w), 16) * div_up(int(h), 16) < 2 ** 14, \
                "32bit sort only support 14 bits tile idx"
        for b in range(rows.shape[0]):
            cam = c.cameras[b]
            for k in range(12):
                cam.cam2world_T[k] = float(rows[b, k])
            cam.fx, cam.fy, cam.cx, cam.cy = (float(v) for v in rows[b, 12:16])
        if instance2world_T is not None:   # render.py:207-220
            assert model.instance_id is not None, "instance_id must be provided in model when render with instance"
            if isinstance(cameras, CameraBundle):
                assert cameras.frame_ids is not None, "frame_ids must be provided when render with instance"
                frames = [int(v) for v in cameras.frame_ids.tolist()]
            else:
                assert cameras.frame_local_id is not None
                frames = [int(cameras.frame_local_id)]
            if instance2world_T.dim() == 3:        # one frame
                instance2world_T = instance2world_T.unsqueeze(0)
            assert instance2world_T.dim() == 4 and tuple(instance2world_T.shape[2:]) == (4, 3), \
                "instance2world_T must be 4D tensor [num_frame, num_instance, 4, 3]"
            assert max(frames) < instance2world_T.shape[0] and min(frames) >= 0
            ids = model.instance_id
            if ids.dtype != torch.int32 or not ids.is_contiguous():
                ids = ids.to(torch.int32).contiguous()
            tr = instance2world_T.detach()
            if tr.dtype != torch.float32 or not tr.is_contiguous():
                tr = tr.to(torch.float32).contiguous()
            assert ids.shape[0] == len(model) and ids.device == model.xyz.device and tr.device == model.xyz.device
            self._instance_keep = (ids, tr)       # the launches read them asynchronously
            c.instance_id, c.instance2world_T = ids.data_ptr(), tr.data_ptr()
            c.num_instance = int(tr.shape[1])
            for b, f in enumerate(frames):
                c.frame_ids[b] = f
        return c

    @staticmethod
    def _model_struct(model: GaussianModelOriginBase) -> _lib.Model:
        m = _lib.Model()
        m.num = len(model)
        for name in ("xyz", "quaternion_xyzw", "scale", "opacity", "color_sh"):
            t = getattr(model, name)
            assert t.is_contiguous() and t.dtype == torch.float32 and t.is_cuda, f"model.{name} must be contiguous fp32 CUDA"
        m.xyz, m.quaternion_xyzw = model.xyz.data_ptr(), model.quaternion_xyzw.data_ptr()
        m.scale, m.opacity = model.scale.data_ptr(), model.opacity.data_ptr()
        k = model.color_sh.shape[1]
        if model.color_sh_base is not None:
            assert model.color_sh_base.is_contiguous()
            m.sh_base, m.sh_base_stride = model.color_sh_base.data_ptr(), 3
            m.sh_rest, m.sh_rest_stride = model.color_sh.data_ptr(), k * 3
        else:   # un-split [N,(D+1)^2,3]: first coefficient is the base
            m.sh_base, m.sh_base_stride = model.color_sh.data_ptr(), k * 3
            m.sh_rest, m.sh_rest_stride = model.color_sh.data_ptr() + 12, k * 3
        return m

    @staticmethod
    def _ctx_struct(tiles_touched, radii, depths, uvs, conic_opacity, rgb, cov2d, ne0,
                    tile_mask=None, records=None, tile_counts=None) -> _lib.SplatContext:
        s = _lib.SplatContext()
        s.tiles_touched, s.radii, s.depths = _lib.ptr(tiles_touched), _lib.ptr(radii), _lib.ptr(depths)
        s.uvs, s.conic_opacity, s.rgb_gaussian = _lib.ptr(uvs), _lib.ptr(conic_opacity), _lib.ptr(rgb)
        s.cov2d_vecs, s.sh_to_rgb_ne_0 = _lib.ptr(cov2d), _lib.ptr(ne0)
        s.tile_mask = _lib.ptr(tile_mask)
        s.records = _lib.ptr(records)
        s.tile_counts = _lib.ptr(tile_counts)
        return s

    # ---- output formats (render.py:696-705, 1623-1668, 2222-2300) ------------------------------------
    def _format_color(self, color: torch.Tensor, final_T: torch.Tensor) -> torch.Tensor:
        """The kernels write NHWC RGB.  ``render_rgba`` appends the accumulated opacity: the reference blends a
        fourth channel of constant 1, sum_i alpha_i T_i, which telescopes to 1 - T_final (and stays inside [0,1],
        so the inference clamp with a zero background alpha changes nothing).  ``use_nchw`` permutes."""
        if self._cfg.disable_builtin_rgb:   # config_def.py:127-132: 0 colour channels, or the alpha alone
            assert not self._cfg.use_nchw, "only support nhwc if disable builtin rgb."   # render.py:667
            color = color[..., :0]
        if self._cfg.render_rgba:
            color = torch.cat([color, (1.0 - final_T).unsqueeze(-1)], dim=-1)
        if self._cfg.use_nchw:
            color = color.permute(0, 3, 1, 2).contiguous()
        return color

    def _unformat_grad(self, drgb: torch.Tensor, dT: torch.Tensor | None):
        """Inverse of ``_format_color`` for the incoming gradient: back to NHWC RGB; the alpha channel's gradient
        moves to the transmittance, d(1 - T)/dT = -1."""
        if self._cfg.use_nchw:
            drgb = drgb.permute(0, 2, 3, 1)
        if self._cfg.render_rgba:
            dalpha = drgb[..., -1]
            dT = -dalpha if dT is None else dT - dalpha
            drgb = drgb[..., :-1]
        if self._cfg.disable_builtin_rgb:   # no colour channels: the splat colours receive no gradient
            drgb = torch.zeros(drgb.shape[:3] + (3,), dtype=drgb.dtype, device=drgb.device)
        return drgb.contiguous(), dT

    # ---- forward (render.py:169-1015) ---------------------------------------------------------
    def forward(self, model: GaussianModelOriginBase, cameras: BasicPinholeCamera | CameraBundle,
                training: bool = False, instance2world_T: torch.Tensor | None = None,
                custom_features: torch.Tensor | None = None, mask: torch.Tensor | None = None,
                prep_user_inputs: dict[str, Any] | None = None):
        assert model.act_applied, "model must be activated before render"
        if prep_user_inputs is not None:
            raise NotImplementedError("proxy inputs are not built")
        lib = self._lib
        dev = model.xyz.device
        stream = torch.cuda.current_stream(dev).cuda_stream
        num = len(model)
        ocfg = self._op_config(model, cameras, training, instance2world_T)
        B, W, H = ocfg.num_views, ocfg.width, ocfg.height
        BN = B * num
        tiles_x, tiles_y = div_up(W, 16), div_up(H, 16)
        num_tiles = B * tiles_x * tiles_y
        i32, f32 = torch.int32, torch.float32
        ext = self.external if (self.external is not None and training and B == 1) else None
        depths = torch.empty(BN, dtype=f32, device=dev)
        radii = ext["radii"] if ext else torch.empty(BN, dtype=i32, device=dev)
        uvs = torch.empty([BN, 2], dtype=f32, device=dev)
        conic_opacity = torch.empty([BN, 4], dtype=f32, device=dev)
        rgb_gaussian = torch.empty([BN, 3], dtype=f32, device=dev)
        cov2d_vecs = (ext["cov2d_vecs"] if ext else torch.empty([BN, 3], dtype=f32, device=dev)) if training else None
        sh_ne0 = (ext["sh_to_rgb_ne_0"] if ext else torch.empty([BN], dtype=torch.uint8, device=dev)) if training else None
        if ext:
            assert radii.shape == (BN,) and cov2d_vecs.shape == (BN, 3) and sh_ne0.shape == (BN,)
        tiles_touched = torch.empty(BN, dtype=i32, device=dev)
        tile_mask = torch.empty(BN, dtype=torch.int64, device=dev)   # binning scratch, dropped after the key emission
        # per-Gaussian raster records, written by the preprocess and gathered by sorted id in the raster kernels
        gather = self.gather_records
        records = torch.empty([BN, 12], dtype=f32, device=dev) if gather else None
        use_bucket = self.binning == "bucket" and not self._cfg.enable_32bit_sort
        tile_counts = torch.empty(num_tiles, dtype=i32, device=dev) if use_bucket else None
        mstruct = self._model_struct(model)
        cstruct = self._ctx_struct(tiles_touched, radii, depths, uvs, conic_opacity, rgb_gaussian, cov2d_vecs, sh_ne0,
                                   tile_mask, records, tile_counts)
        mask_u8 = None
        if mask is not None:
            mask_u8 = mask.to(torch.uint8).contiguous()
            assert mask_u8.numel() == BN
        sync = self._sync_words(dev)
        _lib.check(lib.d3gs_preprocess_forward(C.byref(ocfg), C.byref(mstruct), _lib.ptr(mask_u8), C.byref(cstruct),
                                               sync.data_ptr() + 8, stream), "d3gs_preprocess_forward")
        self._mark("preprocess_fwd")
        if self.debug_capture:
            self.debug = {"tiles_touched": tiles_touched.clone()}
        workload_ranges = cursor = None
        final_T = torch.empty([B, H, W], dtype=f32, device=dev)
        n_contrib = torch.empty([B, H, W], dtype=i32, device=dev)
        out_color = torch.empty([B, H, W, 3], dtype=f32, device=dev)

        def scan_tiles_touched():   # cumsum + total (render.py:694-695)
            ws = self._ws.get("scan", lib.d3gs_scan_workspace_bytes(BN), dev)
            _lib.check(lib.d3gs_scan_tiles(tiles_touched.data_ptr(), tiles_touched.data_ptr(), BN, sync.data_ptr(),
                                           ws.data_ptr(), ws.numel(), sync.data_ptr() + 8, stream), "d3gs_scan_tiles")

        def bucket_prepare(pair_capacity):
            _lib.check(lib.d3gs_bucket_prepare(tile_counts.data_ptr(), tile_scan.data_ptr(), num_tiles,
                                               workload_ranges.data_ptr(), cursor.data_ptr(), sync.data_ptr() + 16,
                                               pair_capacity, stream), "d3gs_bucket_prepare")

        def bucket_lists(cap, sort_max, checked):
            """Entries -> sorted lists for pair buffers of ``cap`` entries; ``checked``: the kernels compare the pair
            count on the device with ``cap`` (the host has not read it yet)."""
            entries = torch.empty(cap, dtype=torch.int64, device=dev)
            ids = torch.empty(cap, dtype=i32, device=dev)
            keys = torch.empty(cap, dtype=torch.int64, device=dev) if self.debug_capture else None
            _lib.check(lib.d3gs_bucket_emit(C.byref(ocfg), num, C.byref(cstruct), cursor.data_ptr(), entries.data_ptr(),
                                            sync.data_ptr() if checked else None, cap if checked else 0, stream),
                       "d3gs_bucket_emit")
            self._mark("duplicate_keys")
            _lib.check(lib.d3gs_bucket_sort(entries.data_ptr(), workload_ranges.data_ptr(), num_tiles, sort_max,
                                            ids.data_ptr(), _lib.ptr(keys), stream), "d3gs_bucket_sort")
            self._mark("sort")
            return ids, keys

        def raster(ids):
            tile_order = torch.empty(num_tiles, dtype=i32, device=dev)
            _lib.check(lib.d3gs_tile_order(workload_ranges.data_ptr(), num_tiles, tile_order.data_ptr(), stream),
                       "d3gs_tile_order")
            self._mark("tile_order")
            _lib.check(lib.d3gs_raster_forward(C.byref(ocfg), workload_ranges.data_ptr(), tile_order.data_ptr(),
                                               records.data_ptr(), ids.data_ptr() if gather else None,
                                               out_color.data_ptr(), final_T.data_ptr(),
                                               n_contrib.data_ptr(), sync.data_ptr() + 8, stream), "d3gs_raster_forward")
            self._mark("raster_fwd")
            return tile_order

        gaussian_idx_sorted = tile_order = keys = None
        ahead = None
        sort_capacity = lib.d3gs_bucket_sort_capacity()
        if use_bucket:
            # the pair count is the total of the per-tile counts; their scan is every tile's range
            tile_scan = torch.empty(num_tiles, dtype=i32, device=dev)
            ws = self._ws.get("scan_tiles", lib.d3gs_scan_workspace_bytes(num_tiles), dev)
            _lib.check(lib.d3gs_scan_tiles(tile_counts.data_ptr(), tile_scan.data_ptr(), num_tiles, sync.data_ptr(),
                                           ws.data_ptr(), ws.numel(), sync.data_ptr() + 8, stream), "d3gs_scan_tiles")
            workload_ranges = torch.empty([num_tiles, 2], dtype=i32, device=dev)
            cursor = torch.empty(num_tiles, dtype=i32, device=dev)
            # Launch ahead of the read-back: buffers sized from the previous launch of the same shape, the kernels
            # check the count themselves, and the host reads the count while they run (and repeats if it was wrong).
            ahead = self._ahead.get((dev, B, num, num_tiles)) if (self.launch_ahead and gather) else None
            bucket_prepare(ahead[0] if ahead else 0)
        else:
            scan_tiles_touched()
        self._mark("scan")
        if ahead:
            words = self._read_sync_words_async(dev, sync)
            gaussian_idx_sorted, keys = bucket_lists(ahead[0], ahead[1], checked=True)
            tile_order = raster(gaussian_idx_sorted)
            num_rendered, status, longest, _ = words()
        else:
            # one device->host read per forward, as in the reference (render.py:695)
            num_rendered, status, longest, _ = (int(v) for v in sync.tolist())
        self._mark("host_readback_idle")
        if status != 0:
            sync[1] = 0
            raise RuntimeError(f"d3gs_b200 device status {status:#x}: a bounded wait gave up "
                               "(1 scan, 2 sort, 4 bulk copy, 8 peer flag); results of the previous call are invalid")
        if num_rendered >= 2 ** 31:
            raise RuntimeError(f"num_rendered {num_rendered} does not fit the int32 offsets")
        self.last_num_rendered = num_rendered
        if num_rendered == 0:   # render.py:706-729: outputs are left uninitialised, no context
            return GaussianSplatOutput(custom_features=None, T=final_T, color=self._format_color(out_color, final_T),
                                       depth=None, n_contrib=n_contrib), None
        if use_bucket and longest > sort_capacity:
            use_bucket = False          # a list too long for one CTA's shared memory: radix-sort path for this launch
            self.launches_repeated += bool(ahead)
            ahead = None
            scan_tiles_touched()
        self.last_binning = "bucket" if use_bucket else "sort"
        # Pair-sized buffers are allocated with a capacity quantised to 2^20 pairs above 1.125 x the count: the
        # count changes a little every training step, and exact sizes would make the caching allocator miss
        # and fall back to cudaMalloc (a device-wide stall of milliseconds) every few steps.
        cap = _pair_capacity(num_rendered)
        if use_bucket:
            # Instances of the tile sort to launch next time: those this launch's longest list needs -- no margin, an
            # instance nobody needs costs 20-30 us, a wrong guess one repeated launch -- but sticky: once a longer
            # list has been met the guess only comes down when the lists have shrunk to half of it, so that a
            # longest list hovering around an instance boundary does not repeat every other step.
            sort_guess = longest
            if ahead and longest > ahead[1] // 2:
                sort_guess = max(longest, ahead[1])
            self._ahead[(dev, B, num, num_tiles)] = (cap, min(sort_capacity, sort_guess))
            if ahead and (num_rendered > ahead[0] or _sort_class(longest) > _sort_class(ahead[1])):
                self.launches_repeated += 1
                bucket_prepare(0)       # the guess was too small: ranges and cursors again, then the chain below
                ahead = None
            if not ahead:
                gaussian_idx_sorted, keys = bucket_lists(cap, longest, checked=False)
            gaussian_idx_sorted = gaussian_idx_sorted[:num_rendered]
            if self.debug_capture:
                self.debug.update(sorted_keys=keys[:num_rendered], sorted_values=gaussian_idx_sorted,
                                  ranges=workload_ranges)
        else:
            keys = torch.empty(cap, dtype=torch.int64, device=dev)[:num_rendered]
            keys_alt = torch.empty(cap, dtype=torch.int64, device=dev)[:num_rendered]
            gaussian_idx = torch.empty(cap, dtype=i32, device=dev)[:num_rendered]
            gaussian_idx_alt = torch.empty(cap, dtype=i32, device=dev)[:num_rendered]
            _lib.check(lib.d3gs_duplicate_keys(C.byref(ocfg), num, tiles_touched.data_ptr(), C.byref(cstruct),
                                               keys.data_ptr(), gaussian_idx.data_ptr(), stream), "d3gs_duplicate_keys")
            self._mark("duplicate_keys")
            if self.debug_capture:
                self.debug.update(scan=tiles_touched.clone(), keys=keys.clone(), values=gaussian_idx.clone())
            end_bit = 32 if self._cfg.enable_32bit_sort else 32 + lib.d3gs_bit_length(num_tiles)   # render.py:851-854
            ws_sort = self._ws.get("sort", lib.d3gs_sort_workspace_bytes(num_rendered, 0, end_bit), dev)
            in_alt = C.c_int32(0)
            _lib.check(lib.d3gs_sort_pairs(keys.data_ptr(), keys_alt.data_ptr(), gaussian_idx.data_ptr(),
                                           gaussian_idx_alt.data_ptr(), num_rendered, 0, end_bit, ws_sort.data_ptr(),
                                           ws_sort.numel(), C.byref(in_alt), sync.data_ptr() + 8, stream),
                       "d3gs_sort_pairs")
            self._mark("sort")
            if in_alt.value:                                                   # render.py:884-887
                keys, keys_alt = keys_alt, keys
                gaussian_idx, gaussian_idx_alt = gaussian_idx_alt, gaussian_idx
            gaussian_idx_sorted = gaussian_idx
            if self.debug_capture:
                self.debug.update(sorted_keys=keys, sorted_values=gaussian_idx_sorted)
            workload_ranges = torch.empty([num_tiles, 2], dtype=i32, device=dev)
            _lib.check(lib.d3gs_tile_ranges(keys.data_ptr(), num_rendered, workload_ranges.data_ptr(), num_tiles,
                                            ocfg.key_shift_bits, stream), "d3gs_tile_ranges")
            self._mark("tile_ranges")
            if self.debug_capture:
                self.debug.update(ranges=workload_ranges)
        if not gather:   # one record per sorted pair, in list order
            records = torch.empty(cap * 12, dtype=f32, device=dev)[:num_rendered * 12].view(num_rendered, 12)
            _lib.check(lib.d3gs_pack_splats(gaussian_idx_sorted.data_ptr(), num_rendered, C.byref(cstruct),
                                            float(self._cfg.alpha_eps), records.data_ptr(), stream),
                       "d3gs_pack_splats")
            self._mark("pack_splats")
        if not ahead:
            tile_order = raster(gaussian_idx_sorted)
        # render.py:1824, 1920-1923, 2244-2270: the depth value and the custom features are blended exactly like
        # colour channels (accum += weight * value, never composited or clamped).  Each group of three channels
        # is one more forward pass over the same lists with the values in the records' colour slots.
        depth = out_feat = None
        aux_values = []
        if self._cfg.render_depth:
            aux_values.append(torch.stack([depths, torch.zeros_like(depths), torch.zeros_like(depths)], dim=1))
        nfeat = 0
        if custom_features is not None:
            assert not self._cfg.use_nchw, "custom feat don't support nchw, set use_nchw=False in config."
            nfeat = custom_features.shape[-1]
            assert custom_features.shape[0] == BN and custom_features.dim() == 2
            feat = custom_features.detach().to(f32)
            pad = (-nfeat) % 3
            if pad:
                feat = torch.cat([feat, torch.zeros([BN, pad], dtype=f32, device=dev)], dim=1)
            aux_values += [feat[:, k:k + 3] for k in range(0, nfeat + pad, 3)]
        aux_passes = []
        for vals in aux_values:
            recs = records.clone()
            recs[:, 8:11] = vals if gather else vals[gaussian_idx_sorted.long()]
            ocfg_a = _lib.OpConfig.from_buffer_copy(ocfg)
            ocfg_a.training = 1
            blend = torch.empty([B, H, W, 3], dtype=f32, device=dev)
            _lib.check(lib.d3gs_raster_forward(C.byref(ocfg_a), workload_ranges.data_ptr(), tile_order.data_ptr(),
                                               recs.data_ptr(), gaussian_idx_sorted.data_ptr() if gather else None,
                                               blend.data_ptr(), torch.empty_like(final_T).data_ptr(),
                                               torch.empty_like(n_contrib).data_ptr(), sync.data_ptr() + 8, stream),
                       "d3gs_raster_forward(aux)")
            aux_passes.append((recs, blend))
        if aux_passes:
            self._mark("raster_fwd_aux")
        if self._cfg.render_depth:
            depth = aux_passes[0][1][..., 0]
            depth = depth.contiguous() if training else depth / (1e-10 + 1.0 - final_T)
        if nfeat:
            groups = aux_passes[1:] if self._cfg.render_depth else aux_passes
            out_feat = torch.cat([b for _, b in groups], dim=-1)[..., :nfeat].contiguous()
        output = GaussianSplatOutput(custom_features=out_feat, T=final_T, color=self._format_color(out_color, final_T),
                                     depth=depth, n_contrib=n_contrib, radii=radii)
        if not training:
            return output, None
        ctx = GaussianSplatOpContext(conic_opacity=conic_opacity, radii=radii, uvs=uvs, rgb_gaussian=rgb_gaussian,
                                     gaussian_idx_sorted=gaussian_idx_sorted, workload_ranges=workload_ranges,
                                     image_shape_wh=(W, H), depths=depths, cov2d_vecs=cov2d_vecs,
                                     sh_to_rgb_ne_0=sh_ne0, splat_records=records, tile_order=tile_order,
                                     records_by_id=gather,
                                     raster_color=out_color if output.color is not out_color else None,
                                     aux_passes=aux_passes, num_custom_feat=nfeat, num_gaussians=num)
        if self._cfg.sparse_mode:
            self._compact_context(output, ctx, B, num, stream)
        return output, ctx

    def _compact_context(self, output: GaussianSplatOutput, ctx: GaussianSplatOpContext, B: int, num: int, stream) -> None:
        """sparse_mode (render.py:235-238, 478-499, 622-637): what is kept for the backward holds the visible
        (view, Gaussian) items only, in flat-index order; ``output.sparse_gaussian_ids`` / ``sparse_batch_ids`` name
        them and ``output.radii`` is compact too.  One more device->host read (the kept count, render.py:635)."""
        lib = self._lib
        assert ctx.records_by_id and not ctx.aux_passes, "sparse mode: no depth / custom-feature passes, gathered records"
        dev = ctx.radii.device
        BN = B * num
        i32, f32 = torch.int32, torch.float32
        flags = torch.empty(BN, dtype=i32, device=dev)
        _lib.check(lib.d3gs_sparse_flags(ctx.radii.data_ptr(), num, B, 0, flags.data_ptr(), stream), "d3gs_sparse_flags")
        scan = torch.empty(BN, dtype=i32, device=dev)
        total = torch.zeros(1, dtype=torch.int64, device=dev)
        ws = self._ws.get("scan", lib.d3gs_scan_workspace_bytes(BN), dev)
        _lib.check(lib.d3gs_scan_tiles(flags.data_ptr(), scan.data_ptr(), BN, total.data_ptr(), ws.data_ptr(), ws.numel(),
                                       self._sync_words(dev).data_ptr() + 8, stream), "d3gs_scan_tiles")
        kept = int(total.item())
        new = dict(radii=torch.empty(kept, dtype=i32, device=dev), depths=torch.empty(kept, dtype=f32, device=dev),
                   uvs=torch.empty([kept, 2], dtype=f32, device=dev),
                   conic_opacity=torch.empty([kept, 4], dtype=f32, device=dev),
                   rgb_gaussian=torch.empty([kept, 3], dtype=f32, device=dev),
                   cov2d_vecs=torch.empty([kept, 3], dtype=f32, device=dev),
                   sh_to_rgb_ne_0=torch.empty([kept], dtype=torch.uint8, device=dev),
                   splat_records=torch.empty([kept, 12], dtype=f32, device=dev))
        gids = torch.empty(kept, dtype=i32, device=dev)
        bids = torch.empty(kept, dtype=i32, device=dev)
        dense = self._ctx_struct(None, ctx.radii, ctx.depths, ctx.uvs, ctx.conic_opacity, ctx.rgb_gaussian, ctx.cov2d_vecs,
                                 ctx.sh_to_rgb_ne_0, None, ctx.splat_records)
        comp = self._ctx_struct(None, new["radii"], new["depths"], new["uvs"], new["conic_opacity"], new["rgb_gaussian"],
                                new["cov2d_vecs"], new["sh_to_rgb_ne_0"], None, new["splat_records"])
        _lib.check(lib.d3gs_sparse_compact(C.byref(dense), num, B, scan.data_ptr(), C.byref(comp), gids.data_ptr(),
                                           bids.data_ptr(), stream), "d3gs_sparse_compact")
        ids = ctx.gaussian_idx_sorted
        _lib.check(lib.d3gs_sparse_remap(ids.data_ptr(), ids.shape[0], scan.data_ptr(), stream), "d3gs_sparse_remap")
        for k, v in new.items():
            setattr(ctx, k, v)
        ctx.sparse_gaussian_ids, ctx.sparse_batch_ids = gids, bids
        output.radii = new["radii"]
        output.sparse_gaussian_ids, output.sparse_batch_ids = gids, bids

    # ---- raster backward (render.py:1329-2316 with grad) -----------------------------------------
    def rasterize_forward_backward(self, model, ctx: GaussianSplatOpContext, out: GaussianSplatOutput,
                                   grad: GaussianSplatGradients | None = None, training: bool = False,
                                   render_depth: bool = False, custom_features: torch.Tensor | None = None,
                                   cameras=None):
        if grad is None:
            raise NotImplementedError("forward rasterisation is part of GaussianSplatOp.forward")
        lib = self._lib
        dev = out.T.device
        stream = torch.cuda.current_stream(dev).cuda_stream
        B, H, W = out.T.shape
        BN = ctx.depths.shape[0]
        num = BN // B
        drgb = grad.drgb
        assert drgb.is_contiguous(), "drgb must be contiguous"
        dT = grad.dT
        if self._cfg.use_nchw or self._cfg.render_rgba or self._cfg.disable_builtin_rgb:
            drgb, dT = self._unformat_grad(drgb, dT)
        color = ctx.raster_color if ctx.raster_color is not None else out.color
        # packed per-splat gradients [BN,12]: dconic a b c, dopacity | dcolor r g b, 0 | duv x y, 0 0
        if self.external is not None and B == 1 and "packed" in self.external:
            packed = self.external["packed"]
            assert packed.shape == (BN, 12) and packed.is_contiguous()
        else:
            # sparse mode: the kept items are not a whole number of Gaussians per view, so the entry point's own
            # zero fill (num * B rows) may stop short of the last rows
            alloc = torch.zeros if ctx.sparse_gaussian_ids is not None else torch.empty
            packed = alloc([BN, 12], dtype=torch.float32, device=dev)
        ocfg = _lib.OpConfig()
        ocfg.width, ocfg.height, ocfg.tile_x, ocfg.tile_y = W, H, 16, 16
        ocfg.alpha_eps, ocfg.transmittance_eps = self._cfg.alpha_eps, self._cfg.transmittance_eps
        ocfg.num_views, ocfg.training = B, 1
        sync = self._sync_words(dev)
        if dT is not None:
            dT = dT.contiguous()
        direct = self.raster_grad_direct
        if direct is None:
            direct = ctx.gaussian_idx_sorted.shape[0] < self.DIRECT_ATOMICS_PAIRS_PER_GAUSSIAN * BN
        mode = (_lib.RASTER_RECORDS_BY_ID if ctx.records_by_id else 0) | (_lib.RASTER_DIRECT_ATOMICS if direct else 0)
        # config_def.py:134, render.py:1451-1453: count the groups of global atomic adds of this launch
        counts = torch.zeros(2, dtype=torch.int64, device=dev) if self._cfg.measure_atomic_add_count else None
        _lib.check(lib.d3gs_raster_backward(C.byref(ocfg), num, ctx.workload_ranges.data_ptr(), _lib.ptr(ctx.tile_order),
                                            ctx.splat_records.data_ptr(), mode,
                                            ctx.gaussian_idx_sorted.data_ptr(),
                                            color.data_ptr(), out.T.data_ptr(), out.n_contrib.data_ptr(),
                                            drgb.data_ptr(), _lib.ptr(dT), packed.data_ptr(), _lib.ptr(counts),
                                            sync.data_ptr() + 8, stream), "d3gs_raster_backward")
        self._mark("raster_bwd")
        if counts is not None:
            groups, passes = (int(v) for v in counts.tolist())
            self.last_atomic_add_count = groups
            self.last_atomic_stats = dict(atomic_add_groups=groups, warp_passes=passes, direct=bool(direct),
                                          sort_pairs=int(ctx.gaussian_idx_sorted.shape[0]))
            print(f"atomic add count: {groups}")     # render.py:2310-2311
        # render.py:1948-1971: the raster backward is linear in the image gradients of all blended channels; the
        # share of every auxiliary group is one more pass with that group's records, whose "colour" gradient is
        # the gradient of the blended values (dz for the depth, dcustom_features for the features)
        dz = dfeat = None
        aux = list(ctx.aux_passes or [])
        aux_grads = []
        if self._cfg.render_depth and aux:
            dd = None
            if grad.ddepth is not None:
                dd = torch.zeros([B, H, W, 3], dtype=torch.float32, device=dev)
                dd[..., 0] = grad.ddepth
            aux_grads.append(dd)
        else:
            assert grad.ddepth is None, "ddepth needs an operator configured with render_depth"
        nfeat = ctx.num_custom_feat
        if nfeat:
            df = grad.dcustom_features
            if df is not None:
                pad = (-nfeat) % 3
                if pad:
                    df = torch.cat([df, torch.zeros([B, H, W, pad], dtype=torch.float32, device=dev)], dim=-1)
            aux_grads += [None if df is None else df[..., k:k + 3].contiguous() for k in range(0, nfeat + (-nfeat) % 3, 3)]
        per_splat = []
        for (recs, blend), dimg in zip(aux, aux_grads):
            if dimg is None:
                per_splat.append(None)
                continue
            packed2 = torch.empty([BN, 12], dtype=torch.float32, device=dev)
            _lib.check(lib.d3gs_raster_backward(C.byref(ocfg), num, ctx.workload_ranges.data_ptr(),
                                                _lib.ptr(ctx.tile_order), recs.data_ptr(), mode,
                                                ctx.gaussian_idx_sorted.data_ptr(), blend.data_ptr(), out.T.data_ptr(),
                                                out.n_contrib.data_ptr(), dimg.data_ptr(), None, packed2.data_ptr(),
                                                None, sync.data_ptr() + 8, stream), "d3gs_raster_backward(aux)")
            packed[:, 0:4] += packed2[:, 0:4]
            packed[:, 8:10] += packed2[:, 8:10]
            per_splat.append(packed2[:, 4:7])
        if per_splat:
            self._mark("raster_bwd_aux")
        if self._cfg.render_depth and per_splat:
            if per_splat[0] is not None:
                packed[:, 7] = per_splat[0][:, 0]     # slot 7: dz, consumed by the preprocess backward
                dz = packed[:, 7]
            per_splat = per_splat[1:]
        if nfeat and any(p is not None for p in per_splat):
            dfeat = torch.cat([p if p is not None else torch.zeros([BN, 3], dtype=torch.float32, device=dev)
                               for p in per_splat], dim=1)[:, :nfeat].contiguous()
        # the reference's four tensors (render.py:1412-1418) are views of the packed array
        return RasterizeGradientOutput(duv=packed[:, 8:10], dconic=packed[:, 0:3], dopacity=packed[:, 3],
                                       dcolor=packed[:, 4:7], dcustom_features=dfeat, dz=dz, packed=packed)

    # ---- backward (render.py:2779-3374) --------------------------------------------------------
    def backward(self, model: GaussianModelOriginBase, cameras: BasicPinholeCamera | CameraBundle,
                 ctx: GaussianSplatOpContext, out: GaussianSplatOutput, grad: GaussianSplatGradients,
                 return_uv_grad: bool = False, instance2world_T: torch.Tensor | None = None,
                 custom_features: torch.Tensor | None = None, prep_user_inputs: dict[str, Any] | None = None,
                 grad_out: "GaussianModelOriginBase | None" = None, adam_segments=None, stats_fn=None):
        """Returns ``(grad_model, duv | None, dcustom_features)`` like the reference.

        ``grad_out`` (not in the reference) lets the caller supply the gradient container, e.g. views of
        a persistent flat buffer that is summed across ranks.  ``adam_segments`` (not in the reference): six
        ``_lib.AdamSegment`` for xyz, quaternion, scale, opacity, sh_base, sh_rest; the backward then applies
        Adam to the model in place instead of producing gradients (``grad_model`` is None); ``stats_fn(duv)``
        may then return a ``_lib.DensifyStats`` to accumulate in the same launch.
        """
        lib = self._lib
        rg = self.rasterize_forward_backward(model, ctx, out, grad, training=True)
        dev = model.xyz.device
        stream = torch.cuda.current_stream(dev).cuda_stream
        ocfg = self._op_config(model, cameras, True, instance2world_T)
        B = ocfg.num_views
        num = len(model)
        sparse = ctx.sparse_gaussian_ids is not None
        if sparse:
            # render.py:2857-2903: spread the kept rows over dense arrays of what the preprocess backward reads, run
            # it, then hand out the gradient rows of the Gaussians that some view saw
            assert adam_segments is None and grad_out is None, "sparse mode returns a compact gradient model"
            kept = ctx.sparse_gaussian_ids.shape[0]
            d_radii = torch.empty(B * num, dtype=torch.int32, device=dev)
            d_cov2d = torch.empty([B * num, 3], dtype=torch.float32, device=dev)
            d_ne0 = torch.empty(B * num, dtype=torch.uint8, device=dev)
            d_packed = torch.empty([B * num, 12], dtype=torch.float32, device=dev)
            _lib.check(lib.d3gs_sparse_expand(kept, num, B, ctx.sparse_gaussian_ids.data_ptr(), ctx.sparse_batch_ids.data_ptr(),
                                              ctx.radii.data_ptr(), ctx.cov2d_vecs.data_ptr(), ctx.sh_to_rgb_ne_0.data_ptr(),
                                              rg.packed.data_ptr(), d_radii.data_ptr(), d_cov2d.data_ptr(), d_ne0.data_ptr(),
                                              d_packed.data_ptr(), stream), "d3gs_sparse_expand")
            compact_rg, compact_ctx = rg, ctx
            ctx = dataclasses.replace(ctx, radii=d_radii, cov2d_vecs=d_cov2d, sh_to_rgb_ne_0=d_ne0, depths=None, uvs=None,
                                      conic_opacity=None, rgb_gaussian=None)
            rg = dataclasses.replace(rg, packed=d_packed)
        if adam_segments is not None:
            assert len(adam_segments) == 6 and B == 1
            assert instance2world_T is None, "the backward fused with Adam does not render instances"

            mstruct = self._model_struct(model)
            cstruct = self._ctx_struct(None, ctx.radii, ctx.depths, ctx.uvs, ctx.conic_opacity, ctx.rgb_gaussian,
                                       ctx.cov2d_vecs, ctx.sh_to_rgb_ne_0)
            arr = (_lib.AdamSegment * 6)(*adam_segments)
            duv = rg.packed.view(B, -1, 12)[:, :, 8:10]
            stats = stats_fn(duv) if stats_fn is not None else None
            _lib.check(lib.d3gs_preprocess_backward_adam(C.byref(ocfg), C.byref(mstruct), C.byref(cstruct),
                                                         rg.packed.data_ptr(), arr,
                                                         C.byref(stats) if stats is not None else None,
                                                         self._sync_words(dev).data_ptr() + 8, stream),
                       "d3gs_preprocess_backward_adam")
            self._mark("preprocess_bwd_adam")
            return None, (duv if return_uv_grad else None), rg.dcustom_features
        if grad_out is None:
            if model.flat is not None or (model.color_sh_base is not None and model.color_sh.shape[1] == 15):
                flat = torch.zeros(flat_layout(num)[1], dtype=torch.float32, device=dev)
                grad_out = type(model)(**carve_flat(flat, num), cur_sh_degree=model.cur_sh_degree, act_applied=True,
                                       flat=flat)
            else:
                t = {k: torch.empty_like(v) for k, v in model.get_all_tensor_fields().items() if v.is_floating_point()}
                if model.color_sh_base is None:
                    t["color_sh_base"] = None
                grad_out = type(model)(**t, cur_sh_degree=model.cur_sh_degree, act_applied=True)
        g = _lib.ModelGrad()
        g.xyz, g.quaternion_xyzw = grad_out.xyz.data_ptr(), grad_out.quaternion_xyzw.data_ptr()
        g.scale, g.opacity = grad_out.scale.data_ptr(), grad_out.opacity.data_ptr()
        k = grad_out.color_sh.shape[1]
        if grad_out.color_sh_base is not None:
            g.sh_base, g.sh_base_stride = grad_out.color_sh_base.data_ptr(), 3
            g.sh_rest, g.sh_rest_stride, g.sh_rest_floats = grad_out.color_sh.data_ptr(), k * 3, k * 3
        else:
            g.sh_base, g.sh_base_stride = grad_out.color_sh.data_ptr(), k * 3
            g.sh_rest, g.sh_rest_stride, g.sh_rest_floats = grad_out.color_sh.data_ptr() + 12, k * 3, k * 3 - 3
        mstruct = self._model_struct(model)
        cstruct = self._ctx_struct(None, ctx.radii, ctx.depths, ctx.uvs, ctx.conic_opacity, ctx.rgb_gaussian,
                                   ctx.cov2d_vecs, ctx.sh_to_rgb_ne_0)
        _lib.check(lib.d3gs_preprocess_backward(C.byref(ocfg), C.byref(mstruct), C.byref(cstruct),
                                                rg.packed.data_ptr(), C.byref(g), self._sync_words(dev).data_ptr() + 8,
                                                stream), "d3gs_preprocess_backward")
        self._mark("preprocess_bwd")
        if sparse:
            if B == 1:      # render.py:2904-2905: one view, the kept items are the Gaussians
                unique = compact_ctx.sparse_gaussian_ids
            else:           # render.py:2864-2903 collects them through a hash table; here: ascending
                flags = torch.empty(num, dtype=torch.int32, device=dev)
                _lib.check(lib.d3gs_sparse_flags(d_radii.data_ptr(), num, B, 1, flags.data_ptr(), stream), "d3gs_sparse_flags")
                scan = torch.empty(num, dtype=torch.int32, device=dev)
                total = torch.zeros(1, dtype=torch.int64, device=dev)
                ws = self._ws.get("scan", lib.d3gs_scan_workspace_bytes(num), dev)
                _lib.check(lib.d3gs_scan_tiles(flags.data_ptr(), scan.data_ptr(), num, total.data_ptr(), ws.data_ptr(),
                                               ws.numel(), self._sync_words(dev).data_ptr() + 8, stream), "d3gs_scan_tiles")
                unique = torch.empty(int(total.item()), dtype=torch.int32, device=dev)
                _lib.check(lib.d3gs_flagged_indices(flags.data_ptr(), scan.data_ptr(), num, unique.data_ptr(), stream),
                           "d3gs_flagged_indices")
            rows = unique.shape[0]
            t = {}
            for name, v in grad_out.get_all_tensor_fields().items():
                if not v.is_floating_point():
                    continue
                per = v[0].numel() if v.dim() > 1 else 1
                dst = torch.empty((rows,) + tuple(v.shape[1:]), dtype=v.dtype, device=dev)
                src = v if v.is_contiguous() else v.contiguous()
                _lib.check(lib.d3gs_gather_rows(src.data_ptr(), per, unique.data_ptr(), rows, dst.data_ptr(), stream),
                           "d3gs_gather_rows")
                t[name] = dst
            if grad_out.color_sh_base is None:
                t["color_sh_base"] = None
            grad_sparse = type(model)(**t, cur_sh_degree=model.cur_sh_degree, act_applied=True)
            grad_sparse.sparse_gaussian_ids = unique       # not in the reference: which Gaussian every row belongs to
            duv = compact_rg.packed[:, 8:10]
            return grad_sparse, ((duv.view(1, -1, 2) if B == 1 else duv) if return_uv_grad else None), rg.dcustom_features
        if return_uv_grad:
            # [B,N,2] strided view of the packed array (the reference returns duv.view(B,-1,2), render.py:3373)
            return grad_out, rg.packed.view(B, -1, 12)[:, :, 8:10], rg.dcustom_features
        return grad_out, None, rg.dcustom_features


    def backward_adam_peers(self, model: GaussianModelOriginBase, all_cameras, views: "_lib.PeerViews", g_begin: int,
                            g_count: int, adam_segments, peerset: "_lib.PeerSet", stats: "_lib.DensifyStats | None" = None) -> None:
        """Data-parallel training, one view per rank: the preprocess backward of ALL ranks' views for this rank's
        share of the Gaussians, the gradient sum, Adam and the parameter broadcast in one launch
        (``d3gs_preprocess_backward_adam_peers``).  ``all_cameras``: the cameras of all ranks in rank order;
        ``views``: every rank's raster gradients and context as mapped here (written by ``forward`` and
        ``rasterize_forward_backward`` of the ranks through ``external``)."""
        dev = model.xyz.device
        ocfg = self._op_config(model, all_cameras, True)
        assert ocfg.num_views == peerset.world and len(adam_segments) == 6
        mstruct = self._model_struct(model)
        arr = (_lib.AdamSegment * 6)(*adam_segments)
        _lib.check(self._lib.d3gs_preprocess_backward_adam_peers(C.byref(ocfg), C.byref(mstruct), C.byref(views), g_begin,
                                                                 g_count, arr, C.byref(stats) if stats is not None else None,
                                                                 C.byref(peerset),
                                                                 torch.cuda.current_stream(dev).cuda_stream),
                   "d3gs_preprocess_backward_adam_peers")
        self._mark("preprocess_bwd_adam_peers")


class _RasterizeGaussians(torch.autograd.Function):
    """Autograd glue with the reference's 18 forward arguments and 6 outputs (render.py:3376-3587).

    Saved state is keyed by name on ``ctx`` for non-tensors and by a fixed tuple for tensors; the
    reference's positional read-back of its saved tensors is not reproduced.
    """

    @staticmethod
    def forward(ctx, xyz, color_sh, color_sh_base, scale, quaternion_xyzw, opacity, cur_sh_degree, instance_id,
                custom_features, mask, model_cls, camera_params, cam2world_T, frame_ids, instance2world_T, training,
                op: GaussianSplatOp, uv_grad_holder=None):
        if isinstance(camera_params, CameraParamBundle) and not isinstance(camera_params, CameraBundle):
            cams = CameraBundle(camera_params.focal_xy_ppoint, camera_params.image_shape_wh, frame_ids, cam2world_T)
        else:
            cams = camera_params
        model = model_cls(xyz=xyz.detach(), color_sh=color_sh.detach(),
                          color_sh_base=None if color_sh_base is None else color_sh_base.detach(),
                          scale=scale.detach(), quaternion_xyzw=quaternion_xyzw.detach(), opacity=opacity.detach(),
                          cur_sh_degree=cur_sh_degree, instance_id=instance_id, act_applied=True)
        out, fwd_ctx = op.forward(model, cams, training, instance2world_T, custom_features, mask)
        ctx.has_ctx = fwd_ctx is not None
        if fwd_ctx is not None:
            ctx.fwd_ctx = fwd_ctx
            ctx.out = out
            ctx.model = model
            ctx.cams = cams
        ctx.op = op
        ctx.instance2world_T = instance2world_T
        ctx.return_uv_grad = uv_grad_holder is not None
        radii = out.radii if out.radii is not None else torch.zeros(0, dtype=torch.int32, device=xyz.device)
        ctx.mark_non_differentiable(out.n_contrib, radii)
        return out.color, out.depth, out.custom_features, out.T, out.n_contrib, radii

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, drgb, ddepth, dcustom_features, dT, dn_contrib, dradii):
        if not ctx.has_ctx:
            return (None,) * 18
        op: GaussianSplatOp = ctx.op
        if drgb is None:
            drgb = torch.zeros_like(ctx.out.color)
        if not drgb.is_contiguous():
            drgb = drgb.contiguous()
        gradient = GaussianSplatGradients(drgb=drgb, dT=dT, ddepth=ddepth, dcustom_features=dcustom_features)
        gm, duv, dfeat = op.backward(ctx.model, ctx.cams, ctx.fwd_ctx, ctx.out, gradient, ctx.return_uv_grad,
                                     ctx.instance2world_T)
        return (gm.xyz, gm.color_sh, gm.color_sh_base, gm.scale, gm.quaternion_xyzw, gm.opacity, None, None, dfeat,
                None, None, None, None, None, None, None, None, duv)


def rasterize_gaussians(model: GaussianModelOriginBase, cameras: BasicPinholeCamera | CameraBundle,
                        op: GaussianSplatOp, training=False, uv_grad_holder: torch.Tensor | None = None,
                        instance2world_T: torch.Tensor | None = None, custom_features: torch.Tensor | None = None,
                        mask: torch.Tensor | None = None) -> GaussianSplatOutput:
    """render.py:3783-3838."""
    model = model.create_model_with_act()
    c2w_t = frame_ids = None
    if isinstance(cameras, CameraBundle):
        c2w_t, frame_ids = cameras.cam2world_T, cameras.frame_ids
    res = _RasterizeGaussians.apply(model.xyz, model.color_sh, model.color_sh_base, model.scale,
                                    model.quaternion_xyzw, model.opacity, model.cur_sh_degree, model.instance_id,
                                    custom_features, mask, type(model), cameras, c2w_t, frame_ids, instance2world_T,
                                    training, op, uv_grad_holder)
    return GaussianSplatOutput(color=res[0], depth=res[1], custom_features=res[2], T=res[3], n_contrib=res[4],
                               radii=res[5])


def rasterize_gaussians_dynamic(model, cameras, op: GaussianSplatOp, training=False, uv_grad_holder=None,
                                instance2world_T=None, custom_features=None, prep_input_tensors=None,
                                prep_inputs=None, mask=None) -> GaussianSplatOutput:
    """render.py:3840-3891: the entry point of models whose parameters carry user-defined (proxy) fields.  The proxy
    extension inputs are user code spliced into JIT kernels in the reference and are not built; without them this
    is ``rasterize_gaussians`` with the reference's two preconditions."""
    assert op._cfg.use_proxy_model, "only v2 (proxy) is supported"                      # render.py:3852
    if instance2world_T is not None:
        assert isinstance(cameras, CameraBundle) and cameras.frame_ids is not None      # render.py:3859-3860
    if prep_input_tensors is not None or prep_inputs is not None:
        raise NotImplementedError("user-defined proxy inputs are not built")
    return rasterize_gaussians(model, cameras, op, training, uv_grad_holder, instance2world_T, custom_features, mask)
