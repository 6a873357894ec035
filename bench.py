"""Benchmark of the 3D-Gaussian-splatting training step (fwd + bwd + L1/D-SSIM + Adam).

    python bench.py --gpus N --steps K --warmup W            # this library on N GPUs (torchrun for N>1)
    python bench.py --impl reference --steps K --warmup W    # CPU restatement of the reference, host cores
    python bench.py --config cfg0|cfg1|cfg2|cfg3             # the other named training configurations (1 GPU)
    python bench.py --config cfg4 --gpus N                   # render sweep: 64 cameras, forward only

Default workload: the data-parallel configuration the headline metric is quoted on -- 3,000,000
Gaussians (SH degree 3, fp32), 1920x1080, one view per GPU with replicated Gaussians, loss 0.8*L1 +
0.2*(1-SSIM), 59-float-per-Gaussian gradients summed over the ranks, one fused Adam step.  Inputs are
seeded synthetic data with that configuration's shapes and distributions (the reference's own
measurement scene is not available offline).

One JSON line is printed by rank 0.  ``value`` is views/s over all GPUs with inputs resident in HBM: the
median over ``--repeats`` timed loops of ``--steps`` steps, every loop starting from the same snapshot of
parameters and optimizer state; ``e2e`` is the same step driven with host buffers (target image uploaded
from pinned memory and the loss read back every step; for the render sweep: cameras from the host, every
rendered image copied back to pinned host memory).
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "training iters/sec (fwd+bwd+SSIM+Adam) at 3M Gaussians 1080p; views/sec at 1/2/4/8 B200"
UNIT = "views/s"
WORKLOADS = {
    "cfg0": "cfg0: 10k Gaussians, SH0 fp32, 256x256, forward + backward under an L1 loss (no optimizer step)",
    "cfg1": "cfg1: 100k Gaussians, SH3 fp32, 800x800, L1 loss, fused Adam + densification statistics",
    "cfg2": "cfg2: 1M Gaussians, SH3 fp32, 1297x840, L1+D-SSIM, fused Adam",
    "cfg3": "cfg3: 3M Gaussians, SH3 fp32, 1920x1080, 1 view/GPU, L1+D-SSIM, gradient sum over ranks, fused Adam",
    "cfg4": "cfg4: 6M Gaussians (heavy-tailed scales), SH3 fp32, 3840x2160, forward-only render of 64 cameras, "
            "64/N views per GPU in launches of up to 8 views",
}
LAMBDA_DSSIM = {"cfg0": 0.0, "cfg1": 0.0, "cfg2": 0.2, "cfg3": 0.2}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="cfg3")
    ap.add_argument("--n", type=int, default=0, help="override the Gaussian count (profiling on small cases)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--peer-lanes", type=int, default=0, choices=[0, 1, 2, 4],
                    help="N>1, fused exchange: lanes that share one Gaussian in the exchange launch (0 = the library's choice)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "fused", "symm", "symm-nomc", "ipc", "nccl"],
                    help="N>1: how gradients are summed and parameters broadcast.  fused (the default when symmetric "
                         "memory can be set up): one launch does the preprocess backward of all ranks' views from their "
                         "raster gradients, the sum, Adam and the parameter broadcast; symm: gradient buffers summed by "
                         "one kernel over symmetric memory (switch multicast when available; -nomc: plain peer "
                         "accesses); ipc: the same over CUDA IPC buffers with NCCL barriers; nccl: reduce-scatter / "
                         "all-gather")
    ap.add_argument("--nccl-update", action="store_true",
                    help="N>1: sharded optimizer through NCCL reduce-scatter / all-gather instead of the peer-memory kernel")
    ap.add_argument("--separate-adam", action="store_true",
                    help="N=1: gradient buffer + optimizer kernel instead of Adam inside the preprocess backward")
    ap.add_argument("--replicated-adam", action="store_true",
                    help="N>1: all-reduce + full Adam on every rank instead of the sharded optimizer")
    ap.add_argument("--cpu-sample", type=int, default=1,
                    help="CPU baseline runs on 1/S of the Gaussians (1 = the whole workload, about 9 s on 16 cores)")
    ap.add_argument("--repeats", type=int, default=0,
                    help="timed loops of --steps steps, each from the same snapshot; the median is reported "
                         "(default 9 for the training configurations, 3 for the render sweep)")
    ap.add_argument("--long-steps", type=int, default=300,
                    help="also time one loop of this many steps from the snapshot (value_300: the work per step "
                         "drifts as training moves the Gaussians); 0 = skip")
    ap.add_argument("--binning", default="bucket", choices=["bucket", "sort"],
                    help="sorted per-tile lists from per-tile buckets sorted in shared memory, or from key "
                         "duplication + global radix sort + range extraction like the reference")
    ap.add_argument("--raster-grad-mode", default="auto", choices=["auto", "direct", "shared"],
                    help="raster backward: direct global atomics per lane group, per-tile accumulation in shared "
                         "memory, or chosen from the pairs per Gaussian")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------
# clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs.

    The values are the ones `nvidia-smi --query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.*` prints, read
    through NVML in this process (read-only queries).  A query holds a driver lock for 3.5 ms or more (up to
    30 ms was seen), during which kernel launches of the step stall: polling every 20 ms, or running nvidia-smi
    beside an 80 ms timed region, added 0.1-0.5 ms per step in one run out of three.  So the samples are taken
    where they cannot delay a launch: `sample()` is called by the timed loop after its last launch is enqueued
    and before it synchronises (the GPU is still executing the last step), and a background thread adds one
    sample every 500 ms for long runs.  nvidia-smi is the fallback when the NVML binding is missing; it is
    started before the warm-up so that its start-up cost is over when the timing begins.  Only samples taken
    between begin() and stop() are reported."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    # NVML clocks-event (throttle) reason bits
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[tuple[float, str]] = []
        self.samples: list[tuple[float, float, float, int]] = []   # (time, sm MHz, max MHz, reason bits)
        self.nvml = None
        self.running = False
        self.t_begin = None
        self.max_poll_ms = 0.0

    def start(self):
        """Start sampling (call before the warm-up)."""
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(self.gpu_index).uuid)
                uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if hasattr(uuid, "encode") else uuid)
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self.max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.running = True
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def begin(self):
        """The timed region starts now."""
        self.t_begin = time.monotonic()

    def sample(self):
        """One NVML sample now (no-op for the nvidia-smi fallback, which samples by itself)."""
        nv = self.nvml
        if nv is None:
            return
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        try:
            t0 = time.monotonic()
            sm = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
            bits = int(get_reasons(self.handle))
            self.samples.append((t0, sm, self.max_sm, bits))
            self.max_poll_ms = max(self.max_poll_ms, (time.monotonic() - t0) * 1e3)
        except Exception:
            pass

    def _poll(self):
        last = None
        while self.running:
            time.sleep(0.02)
            if self.t_begin is None:
                continue
            now = time.monotonic()
            if last is None:
                last = self.t_begin       # the first background sample comes 0.5 s into the timed region
            if self.running and now - last >= 0.5:
                last = now
                self.sample()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.monotonic(), line.strip()))

    def stop(self) -> dict:
        t_end = time.monotonic()
        t0 = self.t_begin if self.t_begin is not None else 0.0
        sm, mx, reasons = [], [], set()
        if self.nvml is not None:
            self.running = False
            self.thread.join(timeout=1)
            for ts, clk, mxc, bits in self.samples:
                if t0 <= ts <= t_end:
                    sm.append(clk)
                    mx.append(mxc)
                    reasons.update(nm for nm, bit in self.REASON_BITS.items() if bits & bit)
            source = "NVML"
        elif self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for ts, ln in self.lines:
                parts = [p.strip() for p in ln.split(",")]
                if len(parts) < 9 or not (t0 <= ts <= t_end + 0.15):
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for nm, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(nm)
            source = "nvidia-smi"
        else:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": source,
                "max_poll_ms": round(self.max_poll_ms, 3)}


# ---------------------------------------------------------------------------------------------
def algorithmic_bytes(stage: str, N: int, V: int, K: int, P: int, Tn: int, training: bool = True) -> float:
    """Compulsory bytes per launch of each stage (degree-3 SH); N (view, Gaussian) items, V visible ones,
    K sort pairs, P pixels, Tn tiles -- all summed over the views of the launch."""
    passes = 6
    ctx_bytes = 53 if training else 40      # per visible item: the context the later stages read (cov2d and the clamp mask only in training)
    table = {
        "preprocess_fwd": 44 * N + 192 * V + 8 * N + ctx_bytes * V + 48 * V,   # + the 48-byte raster record per visible Gaussian
        "scan": 8 * N,
        "duplicate_keys": 8 * N + 28 * V + 12 * K,
        "sort": (8 + 24 * passes) * K,
        "tile_ranges": 8 * K + 8 * Tn,
        "pack_splats": (4 + 40 + 48) * K,   # only when the records are packed per pair (GaussianSplatOp.gather_records off)
        "tile_order": 16 * Tn,
        "raster_fwd": 48 * K + 8 * Tn + 20 * P,
        "l1_dssim": 24 * P + 12 * P,
        "raster_bwd": 48 * K + 36 * P + 36 * K,
        "preprocess_bwd": (53 + 36) * V + 4 * N + 236 * V + 236 * N,
        "adam_stats": 1652 * N + 12 * N + 24 * N,
        # single-rank fused path: the per-unit figures of the two stages it replaces, so that the iteration total
        # stays comparable between update paths (see moved_bytes for what the launch itself has to move)
        "preprocess_bwd_adam": (53 + 36) * V + 4 * N + 236 * V + 236 * N + 1652 * N + 12 * N + 24 * N,
        # data parallel, backward fused into the exchange: per rank, what the replicated pipeline would move for
        # it -- the backward of its own view and Adam over all Gaussians (the same figure as the single-rank launch)
        "preprocess_bwd_adam_peers": (53 + 36) * V + 4 * N + 236 * V + 236 * N + 1652 * N + 12 * N + 24 * N,
        "densify_stats": 0,
    }
    return float(table.get(stage, 0.0))


BUCKET_BINNING = False    # set by the bench from the binning path the operator took
WORLD = 1                 # ranks of the run (the fused backward + exchange launch covers 1/WORLD of the Gaussians)


def moved_bytes(stage: str, N: int, V: int, K: int, P: int, Tn: int, training: bool = True) -> float:
    """Bytes the launch of a stage itself has to move.  Equal to the algorithmic bytes except for the fused
    backward + Adam launch, which neither writes nor re-reads the 236-byte-per-Gaussian gradient, and for the
    tile-bucket binning: the scan runs over the tiles, a pair is one 8-byte entry, the per-tile sort reads the
    entries once and writes 4-byte indices, and there is no range extraction."""
    if stage == "preprocess_bwd_adam":
        return float(89 * V + 1456 * N)
    if stage == "preprocess_bwd_adam_peers":
        # HBM side of one rank's launch: its share of parameters and moments, the raster gradients and context of
        # its Gaussians in every view (its own from HBM, the others' over NVLink), and the other ranks' parameter
        # stores arriving in this replica
        return float(89 * V + 1456 * N / WORLD + 236 * N * (WORLD - 1) / WORLD)
    if stage == "densify_stats":
        return float(24 * N + 12 * V)
    if BUCKET_BINNING:
        if stage == "scan":
            return float(8 * Tn + 20 * Tn)
        if stage == "duplicate_keys":
            return float(4 * N + 28 * V + 8 * K + 8 * K)    # + one cursor atomic per pair
        if stage == "sort":
            return float(8 * K + 4 * K + 8 * Tn)
        if stage == "preprocess_fwd":
            return algorithmic_bytes(stage, N, V, K, P, Tn, training) + 4 * K   # one count atomic per pair
    return algorithmic_bytes(stage, N, V, K, P, Tn, training)


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch, from `ncu --set full` captures of
# the small case `--n 750000` (N, V, K, P, Tn below); the summaries under profiles/ give the commands.
# A full-size launch is too large to capture under a 40-pass replay, so the figure is scaled to the bench's
# workload by the ratio of algorithmic bytes (traffic of these kernels grows with the units processed).
NCU_SMALL_CASE = dict(N=750000, V=574917, K=1068256, P=2073600, Tn=8160)
NCU_SMALL_TRAFFIC = {"raster_bwd": 152.06e6, "raster_fwd": 42.86e6, "adam_stats": 1244.93e6, "preprocess_bwd": 351.21e6,
                     "preprocess_fwd": 253.40e6, "preprocess_bwd_adam": 1104.75e6, "l1_dssim": 224.19e6, "pack_splats": 35.39e6, "duplicate_keys": 21.03e6}


def ncu_traffic(stage: str, N: int, V: int, K: int, P: int, Tn: int):
    if stage not in NCU_SMALL_TRAFFIC:
        return None
    small = moved_bytes(stage, **NCU_SMALL_CASE)
    return NCU_SMALL_TRAFFIC[stage] * moved_bytes(stage, N, V, K, P, Tn) / small


COMM_STAGES = ("host_readback_idle", "allreduce", "reduce_scatter", "all_gather", "barrier_grads", "barrier_params")


def load_peak():
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    kind = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
    return peak, kind


def roofline_block(stage_ms: dict, ms_per_step: float, N, V, K, P, Tn, training=True, with_traffic=True) -> dict:
    """Roofline of the stage with the largest share and of the whole step.  ``frac`` counts the bytes the launch
    itself has to move; ``frac_unfused_bytes`` the per-stage figures of the unfused pipeline (for a fused launch the
    sum of the stages it replaces, which can exceed 1: those bytes are saved, not moved)."""
    peak, peak_kind = load_peak()
    kernel_stages = {k: v for k, v in stage_ms.items() if k not in COMM_STAGES and v > 0}
    dom = max(kernel_stages, key=kernel_stages.get)
    sec = kernel_stages[dom] * 1e-3
    moved = moved_bytes(dom, N, V, K, P, Tn, training)
    unfused = algorithmic_bytes(dom, N, V, K, P, Tn, training)
    it_unfused = sum(algorithmic_bytes(s, N, V, K, P, Tn, training) for s in kernel_stages)
    it_moved = sum(moved_bytes(s, N, V, K, P, Tn, training) for s in kernel_stages)
    step_sec = ms_per_step * 1e-3
    per_stage = {s: round(moved_bytes(s, N, V, K, P, Tn, training) / (t * 1e-3) / 1e9 / peak, 4)
                 for s, t in kernel_stages.items() if moved_bytes(s, N, V, K, P, Tn, training) > 0}
    return {"bound": "hbm", "kernel": dom, "achieved": moved / sec / 1e9, "peak": peak, "unit": "GB/s",
            "frac": moved / sec / 1e9 / peak,
            "traffic": ncu_traffic(dom, N, V, K, P, Tn) if with_traffic else None,
            "traffic_source": "ncu dram bytes of the 750k-Gaussian case scaled by the bytes moved" if with_traffic else None,
            "peak_kind": peak_kind,
            "algorithmic_bytes_per_launch": moved,
            "unfused_bytes_per_launch": unfused,
            "frac_unfused_bytes": unfused / sec / 1e9 / peak,
            "stage_frac": per_stage,
            "iteration": {"algorithmic_bytes": it_unfused, "achieved": it_unfused / step_sec / 1e9,
                          "frac": it_unfused / step_sec / 1e9 / peak,
                          "moved_bytes": it_moved, "frac_moved_bytes": it_moved / step_sec / 1e9 / peak}}


def _oracle_scene(sc, views=1):
    import numpy as np
    from oracle import oracle as O
    return O.Scene(*(sc[k].numpy().copy() for k in ("xyz", "quat", "scale", "opacity", "sh_base", "sh_rest")),
                   cams=np.ascontiguousarray(sc["cams"][:views]).copy())


def cpu_baseline(cfg_name: str, sample: int, check: dict | None = None):
    """Times the CPU oracle on the configuration's workload for one view (all host threads this process may
    use).  ``sample`` > 1: on 1/sample of the Gaussians at full resolution, per-Gaussian stages scaled back.
    cfg4 (render sweep): one forward pass of camera 0; ``check``, when given, holds that camera's sorted values
    and tile ranges from the GPU, which are compared bit for bit with the oracle's here."""
    import numpy as np
    from d3gs_research_b200 import scenes
    from oracle import oracle as O
    cores = O.set_num_threads()
    full = scenes.CONFIGS[cfg_name]
    n = max(full.n // sample, 1000)
    render_only = cfg_name == "cfg4"
    # camera 0 of the configuration's camera set (the render sweep's cameras lie on a sphere whose sampling
    # depends on the number of views; the training configurations use their first camera)
    sc = scenes.make_scene(cfg_name, seed=0, n=n, views=None if render_only else 1)
    osc = _oracle_scene(sc)
    ocfg = O.OpConfig(width=full.width, height=full.height, sh_degree=full.sh_degree, early_filter=4,
                      training=not render_only)
    scale = full.n / n
    if render_only:
        t0 = time.perf_counter()
        res = O.forward(ocfg, osc)
        wall = time.perf_counter() - t0
        out = {"value": 1.0 / (wall * scale), "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"oracle/d3gs_oracle.cpp, forward pass of camera 0 at {full.width}x{full.height}, {n} of "
                         f"{full.n} Gaussians; measured {wall:.2f} s",
               "sample_seconds": wall, "stage_seconds": {k: round(v, 4) for k, v in res.timings.items()}}
        if check is not None and sample == 1:
            same_vals = bool(np.array_equal(check["sorted_values"], res.sorted_ids))
            same_ranges = bool(np.array_equal(check["ranges"], res.ranges))
            out["parity_camera0"] = {"sort_pairs": int(res.num_rendered), "sorted_values_bit_exact": same_vals,
                                     "tile_ranges_bit_exact": same_ranges,
                                     "n_contrib_bit_exact": bool(np.array_equal(check["n_contrib"], res.n_contrib[0]))}
        return out
    adam_state = None
    if cfg_name != "cfg0":
        adam_state = {k: (np.zeros_like(getattr(osc, k)), np.zeros_like(getattr(osc, k)))
                      for k in ("xyz", "quat", "scale", "opacity", "sh_base", "sh_rest")}
    stats = dict(duv_ndc_length=np.zeros(n, np.float32), count=np.zeros(n, np.float32), max_radii=np.zeros(n, np.float32))
    t0 = time.perf_counter()
    res = O.run_iteration(ocfg, osc, sc["target"][:1].numpy(), LAMBDA_DSSIM[cfg_name], adam_state=adam_state, step=1,
                          stats=stats)
    wall = time.perf_counter() - t0
    tm = res.timings
    per_pixel = tm.get("loss", 0.0)
    scaled = (wall - per_pixel) * scale + per_pixel
    return {"value": 1.0 / scaled, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"oracle/d3gs_oracle.cpp, 1 view at {full.width}x{full.height}, {n} of {full.n} Gaussians "
                      f"(1/{sample}); measured {wall:.2f} s, per-Gaussian stages scaled x{scale:.0f}, "
                      f"per-pixel loss stage ({per_pixel:.2f} s) unscaled",
            "sample_seconds": wall, "stage_seconds": {k: round(v, 4) for k, v in tm.items()}}


def run_reference(args):
    """Reference arm: the reference has no runnable implementation of this path here (its kernels are
    JIT-compiled through the absent cumm package and it has no CPU path), so its CPU restatement --
    the oracle -- is timed on the host cores with every thread this process may use (an inherited
    OMP_NUM_THREADS=1, which torch.distributed.run exports, is overridden)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 3))
    vals = []
    cb = None
    for _ in range(max(0, min(args.warmup, 1)) + steps):
        cb = cpu_baseline(args.config, args.cpu_sample)
        vals.append(cb["value"])
    vals = vals[-steps:]
    v = sum(vals) / len(vals)
    cb["value"] = v
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": min(args.warmup, 1), "ms_per_step": 1000.0 / v, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOADS[args.config],
                       "note": "CPU restatement of the reference kernels on host cores; one view per step"},
            "cpu_baseline": cb,
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def _median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def _dist_setup():
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    return world, rank, local_rank, dev


# ---------------------------------------------------------------------------------------------
def bench_train(args):
    global BUCKET_BINNING, WORLD
    import torch
    import torch.distributed as dist

    import d3gs_research_b200 as d3
    from d3gs_research_b200 import _lib, scenes
    from d3gs_research_b200.config_def import EarlyFilterAlgo
    from d3gs_research_b200.render import StageTimer
    from d3gs_research_b200.trainer import HostFeed, SplatTrainer

    world, rank, local_rank, dev = _dist_setup()
    lib = _lib.load()
    scfg = scenes.CONFIGS[args.config]
    n_override = args.n if args.n > 0 else None
    sc = scenes.make_scene(args.config, seed=0, n=n_override, views=max(world, 1))
    N = sc["xyz"].shape[0]
    W, H = scfg.width, scfg.height
    model = d3.GaussianModelOriginFused.from_tensors(sc["xyz"], sc["quat"], sc["scale"], sc["opacity"], sc["sh_base"],
                                                     sc["sh_rest"], device=dev, cur_sh_degree=scfg.sh_degree)
    op_cfg = d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT)
    do_update = args.config != "cfg0"           # cfg0 is forward + backward only
    peer_update = {"auto": None, "fused": "symm", "symm": "symm", "symm-nomc": "symm", "ipc": "ipc",
                   "nccl": False}[args.exchange]
    fuse_exchange = {"auto": None, "fused": True}.get(args.exchange, False)
    if args.nccl_update or args.replicated_adam or world == 1:
        peer_update = False if world > 1 else None
    trainer = SplatTrainer(model, op_cfg, lambda_dssim=LAMBDA_DSSIM[args.config], batch_size=world,
                           shard_optimizer=False if args.replicated_adam else None,
                           peer_update=peer_update, multicast=False if args.exchange == "symm-nomc" else None,
                           fuse_exchange=fuse_exchange if world > 1 else False,
                           fuse_backward_adam=False if (args.separate_adam or world > 1 or not do_update) else None)
    trainer.op.raster_grad_direct = {"auto": None, "direct": True, "shared": False}[args.raster_grad_mode]
    trainer.op.binning = args.binning
    trainer.peer_lanes = args.peer_lanes
    fx, fy, cx, cy = sc["intrinsics"]
    cam = d3.BasicPinholeCamera.from_params(sc["cam2worlds"][rank % len(sc["cam2worlds"])], fx, fy, cx, cy, W, H)
    # the cameras of all ranks of this step's batch, in rank order (a training loop knows the batch it draws)
    all_cams = [d3.BasicPinholeCamera.from_params(sc["cam2worlds"][r % len(sc["cam2worlds"])], fx, fy, cx, cy, W, H)
                for r in range(world)] if world > 1 else None
    target_host = sc["target"][rank % sc["target"].shape[0]][None].contiguous().pin_memory()
    target_dev = target_host.to(dev)
    repeats = args.repeats if args.repeats > 0 else 9

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    feed = HostFeed(dev)

    def timed(steps: int, e2e: bool, sample_clocks: bool = False):
        # one pinned slot per step: every step's loss sums are read back inside the timed region
        loss_host = torch.zeros(steps, 2, dtype=torch.float64).pin_memory()
        gc.collect()
        gc.disable()   # a generational collection in the launch loop stalls the queue for milliseconds
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = lib.d3gs_kernel_launch_count()
        e0.record()
        nxt = feed.push(target_host) if e2e else None
        for k in range(steps):
            if e2e:
                # this step's target image travels pinned host memory -> device on a side stream.  The upload
                # of step k+1 is started before step k is enqueued (two device slots), like a loader that
                # prefetches one batch: it overlaps a whole step; the loss kernels wait for its event.
                tgt, ready = nxt
                if k + 1 < steps:
                    nxt = feed.push(target_host)
                info = trainer.step(cam, tgt, update=do_update, target_ready=ready, all_cameras=all_cams)
                loss_host[k].copy_(trainer._loss_sums, non_blocking=True)   # this step's loss sums -> host
            else:
                info = trainer.step(cam, target_dev, update=do_update, all_cameras=all_cams)
        e1.record()
        launches = lib.d3gs_kernel_launch_count() - launches0
        if sample_clocks:   # everything is enqueued and the GPU is still executing: the query delays no launch
            sampler.sample()
        barrier()      # synchronises: all uploads consumed, all loss read-backs landed
        gc.enable()
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        # only two numbers of the last step leave the loop: a returned `info` would keep that step's buffers alive
        # through the next timed loop as a third generation beside the two the loop itself holds, and the caching
        # allocator would have to cudaMalloc them (a 7-22 ms stall, seen in one run out of four)
        counts = (int(info["num_rendered"]), int((info["out"].radii > 0).sum().item()))
        return float(t.item()), counts, int(launches)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # The warm-up keeps each step's result alive until the next one returns, exactly like the timed loops: the
    # second generation of output buffers is then already in the allocator's cache (without this the first
    # timed loop paid a cudaMalloc of up to 9 ms in its second step, one run out of four).
    info = None
    for _ in range(max(args.warmup, 3)):
        info = trainer.step(cam, target_dev, update=do_update, all_cameras=all_cams)
    for _ in range(3):      # warm the host-buffer path (side stream, staging buffers) as well
        tgt, ready = feed.push(target_host)
        info = trainer.step(cam, tgt, update=do_update, target_ready=ready, all_cameras=all_cams)
    # Every timed loop starts from the same parameters and optimizer state: training moves the Gaussians, so
    # the work per step drifts with the step count and the loops would not measure the same steps.
    snap = {"flat": trainer.model.flat.clone(), "m": trainer.exp_avg.clone(), "v": trainer.exp_avg_sq.clone(),
            "stats": [t.clone() for t in (trainer.state.duv_ndc_length, trainer.state.count, trainer.state.max_radii)],
            "step": trainer.step_count}

    def restore():
        trainer.model.flat.copy_(snap["flat"])
        trainer.exp_avg.copy_(snap["m"])
        trainer.exp_avg_sq.copy_(snap["v"])
        for dst, src in zip((trainer.state.duv_ndc_length, trainer.state.count, trainer.state.max_radii), snap["stats"]):
            dst.copy_(src)
        trainer.step_count = snap["step"]

    for _ in range(3):      # the same pattern once more after the snapshot's allocations
        info = trainer.step(cam, target_dev, update=do_update, all_cameras=all_cams)
    restore()
    info = None    # the timed loops hold two generations of step buffers, like the warm-up: no third one from here
    sampler.begin()
    dev_ms, e2e_ms = [], []
    K = V = launches = 0
    for _ in range(repeats):
        ms, (K, V), launches = timed(args.steps, e2e=False, sample_clocks=rank == 0)
        dev_ms.append(ms)
        restore()
    for _ in range(repeats):
        ms, _, _ = timed(args.steps, e2e=True, sample_clocks=rank == 0)
        e2e_ms.append(ms)
        restore()
    long_ms = None
    if args.long_steps > 0:
        long_ms, _, _ = timed(args.long_steps, e2e=False, sample_clocks=rank == 0)
        restore()
    clocks = sampler.stop() if rank == 0 else None
    # Per-stage times come from one more pass over the same steps: the event records between the launches
    # cost about 0.05 ms per step, which the timed loops above do not pay.
    trainer.op.timer = StageTimer(prealloc=20 * (args.steps + 1))
    torch.cuda.synchronize()
    timed(args.steps, e2e=False)
    stage_ms = trainer.op.timer.summary(median=True)   # per-stage median over the steps of the pass
    trainer.op.timer = None
    trainer.op.check_status()

    replicas_agree = None
    if world > 1:   # every replica must hold bit-identical parameters after the same updates
        c = trainer.parameter_checksum().reshape(1)
        c_lo, c_hi = c.clone(), c.clone()
        dist.all_reduce(c_lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(c_hi, op=dist.ReduceOp.MAX)
        replicas_agree = bool((c_lo == c_hi).item())
    P, Tn = W * H, ((W + 15) // 16) * ((H + 15) // 16)
    views = world
    ms_total, ms_e2e = _median(dev_ms), _median(e2e_ms)
    value = views * args.steps / (ms_total / 1e3)
    e2e_value = views * args.steps / (ms_e2e / 1e3)
    optimizer_kind = ("none (forward + backward only)" if not do_update else
                      ("single rank, Adam inside the preprocess backward" if trainer.fused_adam else
                       "single rank, gradient buffer + optimizer kernel") if world == 1 else
                      trainer.update_path_name())
    direct = trainer.op.raster_grad_direct
    if direct is None:
        direct = K < trainer.op.DIRECT_ATOMICS_PAIRS_PER_GAUSSIAN * N
    WORLD = world
    BUCKET_BINNING = trainer.op.last_binning == "bucket"
    binning_taken = trainer.op.last_binning
    trainer.close()    # unmap the peer buffers (collective) before the process group goes away
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOADS[args.config] if not n_override else f"{args.config} n={N}",
                   "gaussians": N, "visible": V, "sort_pairs": K, "resolution": [W, H], "views_per_gpu": 1,
                   "parallelism": f"dp{world} over views, replicated Gaussians",
                   "optimizer": optimizer_kind,
                   "raster_backward": "direct global atomics per lane group" if direct else "per-tile accumulation in shared memory",
                   "binning": "per-tile buckets sorted in shared memory" if binning_taken == "bucket" else
                              "key duplication + global radix sort + range extraction",
                   "replicas_agree": replicas_agree, "early_filter": "OBB_DFVT",
                   "l2": "inputs larger than L2 (params+grads+Adam state 2.8 GB per step)" if N >= 1_000_000 else
                         "working set below the 126 MB L2 at this size; no flush between steps (a training loop "
                         "re-reads its own parameters)"},
        "repeats": {"count": repeats, "ms_per_step_min": min(dev_ms) / args.steps, "ms_per_step_max": max(dev_ms) / args.steps,
                    "ms_per_step_median": ms_total / args.steps,
                    "e2e_ms_per_step_min": min(e2e_ms) / args.steps, "e2e_ms_per_step_max": max(e2e_ms) / args.steps},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(target_host.numel() * 4),
                "d2h_bytes_per_step": 16 + 16, "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": launches,   # kernels of this library launched inside one timed loop (counted by the library)
        "gpu_launches_per_step": launches / args.steps,
        "clocks": clocks,
        "stage_ms": {k: round(v, 4) for k, v in stage_ms.items()},
        "roofline": roofline_block(stage_ms, ms_total / args.steps, N, V, K, P, Tn, with_traffic=N >= 500_000),
    }
    if long_ms is not None:
        line["value_300"] = views * args.long_steps / (long_ms / 1e3)
        line["ms_per_step_300"] = long_ms / args.long_steps
        line["long_steps"] = args.long_steps
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args.config, args.cpu_sample)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
def bench_render(args):
    """cfg4: forward-only rendering of the configuration's 64 cameras, 64/N views per GPU in launches of up to
    8 views (one ``CameraBundle`` per launch; sort key = (view * tiles + tile) << 32 | depth).  A step is one pass
    over this rank's cameras.  No collective: the ranks render disjoint cameras."""
    global BUCKET_BINNING
    import numpy as np
    import torch
    import torch.distributed as dist

    import d3gs_research_b200 as d3
    from d3gs_research_b200 import _lib, scenes
    from d3gs_research_b200.config_def import EarlyFilterAlgo
    from d3gs_research_b200.render import CameraBundle, StageTimer

    world, rank, local_rank, dev = _dist_setup()
    lib = _lib.load()
    scfg = scenes.CONFIGS[args.config]
    n_override = args.n if args.n > 0 else None
    sc = scenes.make_scene(args.config, seed=0, n=n_override)
    N = sc["xyz"].shape[0]
    W, H = scfg.width, scfg.height
    total_views = scfg.num_views
    assert total_views % world == 0, "the camera set must split evenly over the ranks"
    per_rank = total_views // world
    group = min(8, per_rank)
    model = d3.GaussianModelOriginFused.from_tensors(sc["xyz"], sc["quat"], sc["scale"], sc["opacity"], sc["sh_base"],
                                                     sc["sh_rest"], device=dev, cur_sh_degree=scfg.sh_degree)
    model.act_applied = True
    op = d3.GaussianSplatOp(d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT))
    op.binning = args.binning
    fx, fy, cx, cy = sc["intrinsics"]
    my_cams = [d3.BasicPinholeCamera.from_params(sc["cam2worlds"][rank * per_rank + k], fx, fy, cx, cy, W, H)
               for k in range(per_rank)]
    groups = [my_cams[k:k + group] for k in range(0, per_rank, group)]
    bundles = [CameraBundle.from_pinhole_cams(g, device=dev) for g in groups]
    repeats = args.repeats if args.repeats > 0 else 3

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    copy_stream = torch.cuda.Stream(device=dev)
    host_images = [torch.empty(group, H, W, 3, dtype=torch.float32).pin_memory() for _ in range(2)]
    slot_free = [None, None]

    def timed(steps: int, e2e: bool, sample_clocks: bool = False):
        gc.collect()
        gc.disable()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = lib.d3gs_kernel_launch_count()
        e0.record()
        k_pairs = vis = 0
        slot = 0
        keep = []
        for _ in range(steps):
            for gi, cams in enumerate(groups):
                if e2e:
                    # the cameras come from the host every launch; the rendered images go back to pinned host
                    # memory on a side stream (two slots), overlapping the next launch
                    bundle = CameraBundle.from_pinhole_cams(cams, device=dev)
                    out, _ = op.forward(model, bundle, training=False)
                    done = torch.cuda.Event()
                    done.record()
                    copy_stream.wait_event(done)
                    with torch.cuda.stream(copy_stream):
                        host_images[slot][:len(cams)].copy_(out.color, non_blocking=True)
                        out.color.record_stream(copy_stream)
                    slot ^= 1
                else:
                    out, _ = op.forward(model, bundles[gi], training=False)
                k_pairs = op.last_num_rendered
            keep = out
        e1.record()
        launches = lib.d3gs_kernel_launch_count() - launches0
        if sample_clocks:
            sampler.sample()
        barrier()
        torch.cuda.current_stream().wait_stream(copy_stream)
        torch.cuda.synchronize()
        gc.enable()
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        vis = int((keep.radii > 0).sum().item())
        return float(t.item()), (int(k_pairs), vis), int(launches)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(min(args.warmup, 3), 2)):
        timed(1, e2e=False)
    timed(1, e2e=True)
    sampler.begin()
    dev_ms, e2e_ms = [], []
    K = V = launches = 0
    for _ in range(repeats):
        ms, (K, V), launches = timed(args.steps, e2e=False, sample_clocks=rank == 0)
        dev_ms.append(ms)
    for _ in range(repeats):
        ms, _, _ = timed(args.steps, e2e=True, sample_clocks=rank == 0)
        e2e_ms.append(ms)
    clocks = sampler.stop() if rank == 0 else None
    op.timer = StageTimer(prealloc=16 * len(groups) * 2 + 16)
    torch.cuda.synchronize()
    timed(1, e2e=False)
    # the timer holds one "step" per begin_step(); forward() marks into the last one: sum over the launches of a pass
    stage_ms = op.timer.summary(median=False)
    op.timer = None
    op.check_status()
    BUCKET_BINNING = op.last_binning == "bucket"
    binning_taken = op.last_binning
    # camera 0 of the whole set, rendered alone, for the bit-exact comparison with the CPU oracle
    check = None
    if rank == 0 and not args.no_cpu_baseline and not n_override:
        op.debug_capture = True
        out0, _ = op.forward(model, my_cams[0], training=False)
        torch.cuda.synchronize()
        check = {"sorted_values": op.debug["sorted_values"].cpu().numpy(), "ranges": op.debug["ranges"].cpu().numpy(),
                 "n_contrib": out0.n_contrib[0].cpu().numpy()}
        op.debug_capture = False
        op.debug = {}
    ms_total, ms_e2e = _median(dev_ms), _median(e2e_ms)
    value = total_views * args.steps / (ms_total / 1e3)
    e2e_value = total_views * args.steps / (ms_e2e / 1e3)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    B = len(groups[-1])
    P, Tn = W * H * B, ((W + 15) // 16) * ((H + 15) // 16) * B
    launches_per_pass = len(groups)
    per_launch_ms = {k: v / launches_per_pass for k, v in stage_ms.items()}
    line = {
        "metric": "render throughput, forward only: views/sec over the 64-camera sweep of cfg4 (6M Gaussians, 3840x2160)",
        "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(min(args.warmup, 3), 2) + 1,
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOADS[args.config] if not n_override else f"{args.config} n={N}",
                   "gaussians": N, "views_total": total_views, "views_per_gpu": per_rank, "views_per_launch": B,
                   "sort_pairs_per_launch": K, "visible_per_launch": V, "resolution": [W, H],
                   "sort_key_bits": 32 + int(Tn).bit_length(),
                   "parallelism": f"{world} ranks render disjoint cameras, replicated Gaussians, no collective",
                   "binning": "per-tile buckets sorted in shared memory" if binning_taken == "bucket" else
                              "key duplication + global radix sort + range extraction",
                   "early_filter": "OBB_DFVT", "l2": "inputs larger than L2 (several GB per launch)"},
        "repeats": {"count": repeats, "ms_per_step_min": min(dev_ms) / args.steps, "ms_per_step_max": max(dev_ms) / args.steps,
                    "ms_per_step_median": ms_total / args.steps},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 64 * per_rank,
                "d2h_bytes_per_step": per_rank * H * W * 3 * 4 + 16 * len(groups), "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": launches, "gpu_launches_per_step": launches / args.steps,
        "clocks": clocks,
        "stage_ms": {k: round(v, 4) for k, v in stage_ms.items()},
        "stage_ms_per_launch": {k: round(v, 4) for k, v in per_launch_ms.items()},
        "roofline": roofline_block(per_launch_ms, ms_total / args.steps / launches_per_pass, N * B, V, K, P, Tn,
                                   training=False, with_traffic=False),
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args.config, args.cpu_sample, check)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.config not in WORKLOADS:
        raise SystemExit(f"unknown --config {args.config}: one of {sorted(WORKLOADS)}")
    if args.impl == "reference":
        run_reference(args)
    elif args.config == "cfg4":
        bench_render(args)
    else:
        bench_train(args)


if __name__ == "__main__":
    main()
