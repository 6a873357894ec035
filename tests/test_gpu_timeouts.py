"""Every bounded wait of the kernels is made to RUN OUT, safely: the waiting code must give up, set its
D3GS_STATUS_* bit and return -- nothing faults, nothing waits for ever, and the next call works again.

How a wait is made to run out: ``d3gs_test_hooks(poll_limit, hold)`` gives every bounded wait a limit of a few
hundred polls and makes one CTA / tile withhold what others (or itself) wait for -- its look-back flag in the scan
and the sort, the bulk copy its own barrier expects elsewhere.  No copy is in flight when a kernel gives up on it
(it was never issued), and every index the kernels touch stays inside their buffers.  The waits on another rank's
flags are made to run out by simply never setting that rank's flag (one GPU plays rank 0 of a two-rank job).
"""
import ctypes as C

import numpy as np
import pytest
import torch

import d3gs_research_b200 as d3
from d3gs_research_b200 import _lib
from d3gs_research_b200.config_def import EarlyFilterAlgo
from d3gs_research_b200.render import GaussianSplatGradients
from parity_utils import gpu_cameras, gpu_model, small_scene

pytestmark = pytest.mark.gpu

SCAN, SORT, COPY, PEER = 1, 2, 4, 8
POLLS = 300


@pytest.fixture
def hooks():
    lib = _lib.load()

    def set_hooks(poll_limit, hold):
        lib.d3gs_test_hooks(poll_limit, hold)

    yield set_hooks
    lib.d3gs_test_hooks(0, -1)


def _stream():
    return torch.cuda.current_stream().cuda_stream


class hooked_only:
    """The hooks are in force only while the named entry point of the library runs (it reads them when it
    launches): the launches before and after it in the same operator call are left alone."""

    def __init__(self, name, poll_limit=POLLS, hold=0):
        self.lib, self.name, self.args = _lib.load(), name, (poll_limit, hold)

    def __enter__(self):
        lib, orig, args = self.lib, getattr(self.lib, self.name), self.args
        self.orig = orig

        def wrapper(*a):
            lib.d3gs_test_hooks(*args)
            try:
                return orig(*a)
            finally:
                lib.d3gs_test_hooks(0, -1)

        setattr(lib, self.name, wrapper)

    def __exit__(self, *exc):
        setattr(self.lib, self.name, self.orig)
        self.lib.d3gs_test_hooks(0, -1)


def test_scan_lookback_gives_up(cuda_device, hooks):
    lib = _lib.load()
    n = 3 * 4096 + 17
    x = torch.randint(0, 9, (n,), dtype=torch.int32, device=cuda_device)
    out = torch.empty_like(x)
    sync = torch.zeros(2, dtype=torch.int64, device=cuda_device)
    ws = torch.empty(lib.d3gs_scan_workspace_bytes(n), dtype=torch.uint8, device=cuda_device)

    def run():
        _lib.check(lib.d3gs_scan_tiles(x.data_ptr(), out.data_ptr(), n, sync.data_ptr(), ws.data_ptr(), ws.numel(),
                                       sync.data_ptr() + 8, _stream()), "scan")
        torch.cuda.synchronize()
        return int(sync[1].item())

    hooks(POLLS, 0)                      # the first tile never publishes its total
    assert run() & SCAN
    sync.zero_()
    hooks(0, -1)
    assert run() == 0
    assert torch.equal(out, torch.cumsum(x, 0).int())


def test_sort_lookback_gives_up(cuda_device, hooks):
    lib = _lib.load()
    n = 3 * 8192 + 5
    g = torch.Generator().manual_seed(3)
    keys = torch.randint(0, 2 ** 40, (n,), generator=g, dtype=torch.int64).to(cuda_device)
    vals = torch.arange(n, dtype=torch.int32, device=cuda_device)
    ws = torch.empty(lib.d3gs_sort_workspace_bytes(n, 0, 40), dtype=torch.uint8, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)

    def run():
        k, v = keys.clone(), vals.clone()
        ka, va = torch.empty_like(k), torch.empty_like(v)
        in_alt = C.c_int32(0)
        _lib.check(lib.d3gs_sort_pairs(k.data_ptr(), ka.data_ptr(), v.data_ptr(), va.data_ptr(), n, 0, 40, ws.data_ptr(),
                                       ws.numel(), C.byref(in_alt), status.data_ptr(), _stream()), "sort")
        torch.cuda.synchronize()
        return (ka, va) if in_alt.value else (k, v)

    hooks(POLLS, 0)                      # the first tile never publishes its digit counts
    run()
    assert int(status.item()) & SORT
    status.zero_()
    hooks(0, -1)
    ks, vs = run()
    assert int(status.item()) == 0
    ref_k, ref_i = torch.sort(keys, stable=True)
    assert torch.equal(ks, ref_k) and torch.equal(vs, vals[ref_i])


def _scene_op(device, gather=True):
    sc = small_scene(n=2048, width=96, height=64, sh_degree=3, seed=6)
    op = d3.GaussianSplatOp(d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT))
    op.gather_records = gather
    model = gpu_model(sc, device)
    model.act_applied = True
    return sc, op, model, gpu_cameras(sc, device)


def test_preprocess_forward_copy_gives_up(cuda_device):
    sc, op, model, cams = _scene_op(cuda_device)
    with hooked_only("d3gs_preprocess_forward"):       # CTA 0's coefficient rows are never copied
        with pytest.raises(RuntimeError, match="bounded wait"):
            op.forward(model, cams, training=True)
    out, ctx = op.forward(model, cams, training=True)      # the status word was cleared by the raise
    op.check_status()
    assert ctx is not None and bool(torch.isfinite(out.color).all())


def test_preprocess_backward_copy_gives_up(cuda_device):
    sc, op, model, cams = _scene_op(cuda_device)
    out, ctx = op.forward(model, cams, training=True)
    grad = GaussianSplatGradients(drgb=torch.ones_like(out.color), dT=None)
    with hooked_only("d3gs_preprocess_backward"):
        gm, _, _ = op.backward(model, cams, ctx, out, grad)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bounded wait"):
        op.check_status()
    gm, _, _ = op.backward(model, cams, ctx, out, grad)
    op.check_status()
    assert float(gm.xyz.abs().max()) > 0


def test_fused_backward_adam_copy_gives_up_and_takes_no_step(cuda_device):
    """The CTA whose staging copy never arrives must not apply Adam to its Gaussians."""
    from d3gs_research_b200.trainer import SplatTrainer
    sc = small_scene(n=2048, width=96, height=64, sh_degree=3, seed=6)
    model = gpu_model(sc, cuda_device)
    tr = SplatTrainer(model, d3.GaussianSplatConfig(early_filter_algo=EarlyFilterAlgo.OBB_DFVT), lambda_dssim=0.2)
    assert tr.fused_adam
    target = torch.rand(1, 3, 64, 96, generator=torch.Generator().manual_seed(1)).to(cuda_device)
    cams = gpu_cameras(sc, cuda_device)
    before = model.flat.clone()
    with hooked_only("d3gs_preprocess_backward_adam"):     # the step's forward, loss and raster launches are left alone
        tr.step(cams, target)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bounded wait"):
        tr.op.check_status()
    moved = (model.flat != before)
    xyz_moved = moved[:2048 * 3].view(2048, 3).any(dim=1)
    assert not bool(xyz_moved[:256].any()), "the CTA that gave up still updated its Gaussians"
    assert bool(xyz_moved[256:].any()), "the other CTAs must have taken their step"


def test_raster_record_copies_give_up(cuda_device):
    """The bulk-copy staging of the raster kernels (records packed per pair) in the forward and the backward."""
    sc, op, model, cams = _scene_op(cuda_device, gather=False)
    with hooked_only("d3gs_raster_forward"):
        out, ctx = op.forward(model, cams, training=True)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bounded wait"):
        op.check_status()
    out, ctx = op.forward(model, cams, training=True)
    op.check_status()
    with hooked_only("d3gs_raster_backward"):
        op.rasterize_forward_backward(model, ctx, out, GaussianSplatGradients(drgb=torch.ones_like(out.color), dT=None))
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bounded wait"):
        op.check_status()


def _two_rank_set(device, n, with_flags):
    """One GPU plays rank 0 of a two-rank job: both ranks' buffers live here, rank 1 never launches."""
    grads = [torch.randn(n, device=device) for _ in range(2)]
    params = [torch.zeros(n, device=device) for _ in range(2)]
    flags = [torch.zeros(_lib.PEER_FLAG_WORDS, dtype=torch.int32, device=device) for _ in range(2)]
    status = torch.zeros(2, dtype=torch.int32, device=device)
    ps = _lib.PeerSet()
    ps.world, ps.rank = 2, 0
    for q in range(2):
        ps.grad[q], ps.param[q] = grads[q].data_ptr(), params[q].data_ptr()
        if with_flags:
            ps.flags[q] = flags[q].data_ptr()
    ps.status = status.data_ptr()
    ps.epoch, ps.wait_limit = 1, POLLS
    m, v = torch.zeros(n // 2, device=device), torch.zeros(n // 2, device=device)
    seg = _lib.AdamSegment()
    seg.param, seg.grad = params[0].data_ptr(), grads[0].data_ptr()
    seg.exp_avg, seg.exp_avg_sq, seg.count = m.data_ptr(), v.data_ptr(), n // 2
    seg.lr, seg.beta1, seg.beta2, seg.eps = 1e-2, 0.9, 0.999, 1e-15
    seg.bias_correction1, seg.bias_correction2_sqrt, seg.grad_scale, seg.weight_decay = 0.1, 0.0316, 1.0, 0.0
    keep = (grads, params, flags, status, m, v)
    return ps, seg, keep


def test_peer_update_staging_copy_gives_up(cuda_device, hooks):
    lib = _lib.load()
    n = 1 << 16
    ps, seg, (grads, params, flags, status, m, v) = _two_rank_set(cuda_device, n, with_flags=False)
    arr = (_lib.AdamSegment * 1)(seg)
    hooks(POLLS, 0)                      # CTA 0 never issues its gradient copies
    _lib.check(lib.d3gs_adam_stats_step_peers(arr, 1, None, C.byref(ps), _stream()), "peers")
    torch.cuda.synchronize()
    assert int(status[0].item()) & COPY
    assert float(params[0][:16].abs().max()) == 0.0, "the chunk whose copy never arrived must stay unchanged"
    assert float(params[0][n // 4:n // 2].abs().max()) > 0 and torch.equal(params[0][:n // 2], params[1][:n // 2])


def test_peer_flags_never_arrive(cuda_device):
    """Rank 1 never announces its gradients: rank 0's launch gives up on the flag, changes nothing, reports."""
    lib = _lib.load()
    n = 1 << 16
    ps, seg, (grads, params, flags, status, m, v) = _two_rank_set(cuda_device, n, with_flags=True)
    arr = (_lib.AdamSegment * 1)(seg)
    _lib.check(lib.d3gs_adam_stats_step_peers(arr, 1, None, C.byref(ps), _stream()), "peers")
    torch.cuda.synchronize()
    assert int(status[0].item()) & PEER
    assert float(params[0].abs().max()) == 0.0 and float(m.abs().max()) == 0.0
    # rank 0 did announce itself to both ranks, and told both that it is done
    f1 = flags[1].cpu().numpy()
    assert f1[0] == 1 and f1[8] == 1 and (f1[16] & PEER)
    # with rank 1's flags in place (as if it had run) the next launch goes through
    status.zero_()
    ps.epoch = 2
    flags[0][1] = 2          # ready
    flags[0][8 + 1] = 2      # done
    torch.cuda.synchronize()
    _lib.check(lib.d3gs_adam_stats_step_peers(arr, 1, None, C.byref(ps), _stream()), "peers")
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0
    assert float(params[0][:n // 2].abs().max()) > 0 and torch.equal(params[0][:n // 2], params[1][:n // 2])
