"""ctypes binding of libd3gs_b200.so (declarations mirror include/d3gs_b200.h).

The library is the only compute path of this package: there is no CPU or torch fallback.
``load()`` raises if the shared object is missing, and every wrapper raises ``RuntimeError`` with
the library's message when an entry point reports an error -- the same way the reference's native
sort module surfaces ``TV_THROW_RT_ERR`` as a Python exception (d3sim/csrc/devsort.py:36, 90).
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libd3gs_b200.so")
MAX_VIEWS = 8

_lib = None


class Camera(C.Structure):
    _fields_ = [("cam2world_T", C.c_float * 12), ("fx", C.c_float), ("fy", C.c_float), ("cx", C.c_float),
                ("cy", C.c_float)]


class OpConfig(C.Structure):
    _fields_ = [("width", C.c_int32), ("height", C.c_int32), ("tile_x", C.c_int32), ("tile_y", C.c_int32),
                ("near_plane", C.c_float), ("far_plane", C.c_float), ("eps", C.c_float),
                ("cov2d_radii_eigen_eps", C.c_float), ("projected_clamp_factor", C.c_float),
                ("gaussian_std_sigma", C.c_float), ("gaussian_lowpass_filter", C.c_float), ("alpha_eps", C.c_float),
                ("transmittance_eps", C.c_float), ("scale_global", C.c_float), ("early_filter_algo", C.c_int32),
                ("sh_degree", C.c_int32), ("training", C.c_int32), ("clamp_mask_reference_order", C.c_int32),
                ("fused_activations", C.c_int32),
                ("bg_color", C.c_float * 3), ("key_shift_bits", C.c_int32), ("depth_32bit_prec", C.c_float), ("anti_aliasing", C.c_int32), ("inv_depth", C.c_int32),
                ("num_views", C.c_int32), ("cameras", Camera * MAX_VIEWS),
                ("instance_id", C.c_void_p), ("instance2world_T", C.c_void_p), ("num_instance", C.c_int32),
                ("frame_ids", C.c_int32 * MAX_VIEWS), ("reserved_", C.c_int32)]


class Model(C.Structure):
    _fields_ = [("num", C.c_int64), ("xyz", C.c_void_p), ("quaternion_xyzw", C.c_void_p), ("scale", C.c_void_p),
                ("opacity", C.c_void_p), ("sh_base", C.c_void_p), ("sh_rest", C.c_void_p),
                ("sh_base_stride", C.c_int32), ("sh_rest_stride", C.c_int32)]


class ModelGrad(C.Structure):
    _fields_ = [("xyz", C.c_void_p), ("quaternion_xyzw", C.c_void_p), ("scale", C.c_void_p), ("opacity", C.c_void_p),
                ("sh_base", C.c_void_p), ("sh_rest", C.c_void_p), ("sh_base_stride", C.c_int32),
                ("sh_rest_stride", C.c_int32), ("sh_rest_floats", C.c_int32), ("reserved", C.c_int32)]


class SplatContext(C.Structure):
    _fields_ = [("tiles_touched", C.c_void_p), ("radii", C.c_void_p), ("depths", C.c_void_p), ("uvs", C.c_void_p),
                ("conic_opacity", C.c_void_p), ("rgb_gaussian", C.c_void_p), ("cov2d_vecs", C.c_void_p),
                ("sh_to_rgb_ne_0", C.c_void_p), ("tile_mask", C.c_void_p), ("records", C.c_void_p),
                ("tile_counts", C.c_void_p)]


class AdamSegment(C.Structure):
    _fields_ = [("param", C.c_void_p), ("grad", C.c_void_p), ("exp_avg", C.c_void_p), ("exp_avg_sq", C.c_void_p),
                ("count", C.c_int64), ("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
                ("bias_correction1", C.c_float), ("bias_correction2_sqrt", C.c_float), ("grad_scale", C.c_float),
                ("weight_decay", C.c_float)]


class DensifyStats(C.Structure):
    _fields_ = [("duv", C.c_void_p), ("radii", C.c_void_p), ("duv_ndc_length", C.c_void_p), ("count", C.c_void_p),
                ("max_radii", C.c_void_p), ("num", C.c_int64), ("batch", C.c_int32), ("width", C.c_int32),
                ("height", C.c_int32), ("need_max_radii", C.c_int32), ("loss_batch", C.c_int32),
                ("duv_stride", C.c_int32)]


MAX_PEERS = 8
RASTER_RECORDS_BY_ID = 1
RASTER_DIRECT_ATOMICS = 2
PEER_HANDLE_BYTES = 64
PEER_FLAG_WORDS = 32
STATUS_PEER_TIMEOUT = 8


class PeerSet(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("grad", C.c_void_p * MAX_PEERS),
                ("param", C.c_void_p * MAX_PEERS), ("status", C.c_void_p), ("grad_mc", C.c_void_p),
                ("param_mc", C.c_void_p), ("flags", C.c_void_p * MAX_PEERS), ("epoch", C.c_uint32),
                ("wait_limit", C.c_uint32), ("lanes_per_gaussian", C.c_int32), ("reserved_", C.c_int32)]


class PeerViews(C.Structure):
    _fields_ = [("splat_grads", C.c_void_p * MAX_PEERS), ("radii", C.c_void_p * MAX_PEERS),
                ("cov2d_vecs", C.c_void_p * MAX_PEERS), ("sh_to_rgb_ne_0", C.c_void_p * MAX_PEERS)]


class RefineConfig(C.Structure):
    _fields_ = [("prune_opacity_thresh", C.c_float), ("grow_grad2d", C.c_float), ("grow_scale3d", C.c_float),
                ("grow_scale2d", C.c_float), ("prune_scale3d", C.c_float), ("prune_scale2d", C.c_float),
                ("scene_scale", C.c_float), ("prune_too_big", C.c_int32), ("refine_by_radii", C.c_int32),
                ("fused_activations", C.c_int32)]


class RefineMoments(C.Structure):
    _fields_ = [("exp_avg_src", C.c_void_p * 6), ("exp_avg_sq_src", C.c_void_p * 6), ("exp_avg_dst", C.c_void_p * 6),
                ("exp_avg_sq_dst", C.c_void_p * 6)]


_STRUCTS = [Camera, OpConfig, Model, ModelGrad, SplatContext, AdamSegment, DensifyStats, PeerSet, RefineConfig,
            RefineMoments, PeerViews]

_P, _I32, _I64, _F, _SZ = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); every symbol include/d3gs_b200.h declares
SIGNATURES = {
    "d3gs_version": (C.c_char_p, []),
    "d3gs_last_error": (_SZ, [C.c_char_p, _SZ]),
    "d3gs_bit_length": (_I32, [C.c_uint32]),
    "d3gs_struct_size": (_SZ, [_I32]),
    "d3gs_kernel_launch_count": (C.c_uint64, []),
    "d3gs_test_hooks": (None, [C.c_uint32, _I32]),
    "d3gs_preprocess_forward": (_I32, [C.POINTER(OpConfig), C.POINTER(Model), _P, C.POINTER(SplatContext), _P, _P]),
    "d3gs_scan_workspace_bytes": (_SZ, [_I64]),
    "d3gs_scan_tiles": (_I32, [_P, _P, _I64, _P, _P, _SZ, _P, _P]),
    "d3gs_scan_tiles_static_max_items": (_I64, []),
    "d3gs_scan_tiles_static": (_I32, [_P, _P, _I64, _P, _P, _P]),
    "d3gs_duplicate_keys": (_I32, [C.POINTER(OpConfig), _I64, _P, C.POINTER(SplatContext), _P, _P, _P]),
    "d3gs_sort_workspace_bytes": (_SZ, [_I64, _I32, _I32]),
    "d3gs_sort_pairs": (_I32, [_P, _P, _P, _P, _I64, _I32, _I32, _P, _SZ, C.POINTER(_I32), _P, _P]),
    "d3gs_bucket_sort_capacity": (_I64, []),
    "d3gs_sparse_flags": (_I32, [_P, _I64, _I32, _I32, _P, _P]),
    "d3gs_sparse_compact": (_I32, [C.POINTER(SplatContext), _I64, _I32, _P, C.POINTER(SplatContext), _P, _P, _P]),
    "d3gs_sparse_remap": (_I32, [_P, _I64, _P, _P]),
    "d3gs_sparse_expand": (_I32, [_I64, _I64, _I32, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "d3gs_flagged_indices": (_I32, [_P, _P, _I64, _P, _P]),
    "d3gs_gather_rows": (_I32, [_P, _I32, _P, _I64, _P, _P]),
    "d3gs_simple_knn_workspace_bytes": (C.c_size_t, [_I64, _I32]),
    "d3gs_simple_knn": (_I32, [_P, _I64, _I64, _I32, _I32, _P, _P, _P, _P, C.c_size_t, _P, _P]),
    "d3gs_bucket_prepare": (_I32, [_P, _P, _I64, _P, _P, _P, _I64, _P]),
    "d3gs_bucket_emit": (_I32, [C.POINTER(OpConfig), _I64, C.POINTER(SplatContext), _P, _P, _P, _I64, _P]),
    "d3gs_bucket_sort": (_I32, [_P, _P, _I64, _I64, _P, _P, _P]),
    "d3gs_tile_ranges": (_I32, [_P, _I64, _P, _I64, _I32, _P]),
    "d3gs_pack_splats": (_I32, [_P, _I64, C.POINTER(SplatContext), _F, _P, _P]),
    "d3gs_tile_order": (_I32, [_P, _I64, _P, _P]),
    "d3gs_raster_forward": (_I32, [C.POINTER(OpConfig), _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "d3gs_raster_backward": (_I32, [C.POINTER(OpConfig), _I64, _P, _P, _P, _I32, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "d3gs_preprocess_backward": (_I32, [C.POINTER(OpConfig), C.POINTER(Model), C.POINTER(SplatContext), _P,
                                        C.POINTER(ModelGrad), _P, _P]),
    "d3gs_ssim_forward": (_I32, [_P, _P, _I32, _I32, _I32, _I32, _P, _P, _P, _P, _P]),
    "d3gs_ssim_backward": (_I32, [_P, _P, _P, _P, _P, _P, _I32, _I32, _I32, _I32, _P, _P]),
    "d3gs_l1_dssim_scratch_bytes": (_SZ, [_I32, _I32, _I32]),
    "d3gs_l1_dssim_forward_backward": (_I32, [_P, _P, _I32, _I32, _I32, _F, _F, _P, _P, _P, _SZ, _P]),
    "d3gs_adam_stats_step": (_I32, [C.POINTER(AdamSegment), _I32, C.POINTER(DensifyStats), _P]),
    "d3gs_densify_stats": (_I32, [C.POINTER(DensifyStats), _P]),
    "d3gs_preprocess_backward_adam": (_I32, [C.POINTER(OpConfig), C.POINTER(Model), C.POINTER(SplatContext), _P,
                                             C.POINTER(AdamSegment), C.POINTER(DensifyStats), _P, _P]),
    "d3gs_preprocess_backward_adam_peers": (_I32, [C.POINTER(OpConfig), C.POINTER(Model), C.POINTER(PeerViews), _I64, _I64,
                                                   C.POINTER(AdamSegment), C.POINTER(DensifyStats), C.POINTER(PeerSet),
                                                   _P]),
    "d3gs_adam_stats_step_peers": (_I32, [C.POINTER(AdamSegment), _I32, C.POINTER(DensifyStats), C.POINTER(PeerSet), _P]),
    "d3gs_refine_classify": (_I32, [C.POINTER(Model), C.POINTER(RefineConfig), _P, _P, _P, _P, _P, _P]),
    "d3gs_refine_apply": (_I32, [C.POINTER(Model), C.POINTER(Model), C.POINTER(RefineConfig), C.POINTER(RefineMoments),
                                 _P, _P, _P, C.POINTER(C.c_int64), _P, _P]),
    "d3gs_reset_opacity": (_I32, [_P, _I64, _F, _I32, _P, _P, _P]),
    "d3gs_peer_buffer_create": (_I32, [_I64, C.POINTER(_P), _P]),
    "d3gs_peer_buffer_open": (_I32, [_P, C.POINTER(_P)]),
    "d3gs_peer_buffer_close": (_I32, [_P]),
    "d3gs_peer_buffer_destroy": (_I32, [_P]),
}


def load():
    """Load the shared library once; raise loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -c \"import __graft_entry__ as g; g.build()\"` "
            "(nvcc, sm_100a). This package has no fallback path.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    for k, st in enumerate(_STRUCTS):
        native = lib.d3gs_struct_size(k)
        if native != C.sizeof(st):
            raise RuntimeError(f"ABI mismatch for {st.__name__}: library {native} bytes, binding {C.sizeof(st)} bytes")
    _lib = lib
    return lib


def last_error() -> str:
    buf = C.create_string_buffer(512)
    load().d3gs_last_error(buf, 512)
    return buf.value.decode("utf-8", "replace")


def check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc}): {last_error()}")


def ptr(t):
    """Device pointer of a torch tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()
