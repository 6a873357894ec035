"""The C-ABI library loads, exports every symbol include/d3gs_b200.h declares, agrees with the binding on
struct sizes, and validates its arguments on the host (no GPU needed: nothing here launches a kernel)."""
import ctypes as C
import os
import re

from d3gs_research_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "d3gs_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(d3gs_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/d3gs_b200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature in _lib.py"
    assert set(_lib.SIGNATURES) == set(names)


def test_struct_sizes_match():
    lib = _lib.load()
    for k, st in enumerate(_lib._STRUCTS):
        assert lib.d3gs_struct_size(k) == C.sizeof(st), st.__name__
    assert lib.d3gs_struct_size(99) == 0


def test_helpers_and_workspace_queries():
    lib = _lib.load()
    assert b"sm_100a" in lib.d3gs_version()
    for n in (0, 1, 2, 255, 256, 8160, 32400, 2 ** 31 - 1):
        assert lib.d3gs_bit_length(n) == int(n).bit_length()      # DeviceSort.get_higher_msb, devsort.py:129-149
    assert lib.d3gs_scan_workspace_bytes(0) >= 16
    assert lib.d3gs_scan_workspace_bytes(10 ** 7) >= (10 ** 7 // 4096) * 8
    assert lib.d3gs_sort_workspace_bytes(10 ** 6, 0, 45) > 8 * 256 * 4
    assert lib.d3gs_l1_dssim_scratch_bytes(1, 1080, 1920) == 3 * 3 * 1080 * 1920 * 4


def test_argument_errors_are_reported_not_raised_on_device():
    lib = _lib.load()
    assert lib.d3gs_preprocess_forward(None, None, None, None, None, None) == -1
    assert "cfg" in _lib.last_error()
    cfg = _lib.OpConfig()
    cfg.width, cfg.height, cfg.tile_x, cfg.tile_y, cfg.num_views = 64, 64, 8, 8, 1
    assert lib.d3gs_preprocess_forward(C.byref(cfg), None, None, None, None, None) == -1
    assert "16x16" in _lib.last_error()
    in_alt = C.c_int32(0)
    assert lib.d3gs_sort_pairs(None, None, None, None, -5, 0, 45, None, 0, C.byref(in_alt), None, None) == -1
    assert lib.d3gs_sort_pairs(None, None, None, None, 10, 40, 30, None, 0, C.byref(in_alt), None, None) == -1
    assert "bit range" in _lib.last_error()
    seg = (_lib.AdamSegment * 1)()
    assert lib.d3gs_adam_stats_step(seg, 9, None, None) == -1
    assert lib.d3gs_ssim_forward(None, None, 1, 8, 8, 0, None, None, None, None, None) == -1
    try:
        _lib.check(-1, "demo")
    except RuntimeError as e:
        assert "demo failed" in str(e)
    else:
        raise AssertionError("check() must raise")
