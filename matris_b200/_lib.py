"""ctypes binding of libmatris_b200.so (the C ABI declared in include/matris_b200.h).

There is no fallback: if the library is missing or a call returns a non-zero
status, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libmatris_b200.so")

MB_OK = 0
MB_ERR_CAPACITY = 7
MB_GRAPH_EDGES_ONLY = 1
OUT_STORE, OUT_ADD, OUT_ATOMIC = 0, 1, 2

_vp, _i32, _i64, _f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float


class MbError(RuntimeError):
    pass


class IsolatedAtomError(ValueError):
    """Raised like the reference's GraphConverter (matris/graph/converter.py:108-113)."""


class MbGraph(C.Structure):
    _fields_ = [
        ("n_atoms", _i32), ("n_struct", _i32), ("n_cells", _i32),
        ("cap_edges", _i32), ("cap_triplets", _i32), ("flags", _i32),
        ("cutoff", C.c_double), ("line_cutoff", C.c_double), ("tol", C.c_double),
        ("cart", _vp), ("lattice", _vp), ("inv_lattice", _vp), ("atom_struct", _vp), ("grid", _vp),
        ("cell_ptr", _vp), ("cell_fill", _vp), ("cell_atoms", _vp), ("atom_cell", _vp), ("atom_wrap", _vp),
        ("scan_tmp", _vp), ("counts", _vp), ("key_unsorted", _vp), ("dist_unsorted", _vp), ("key", _vp),
        ("atom_counts", _vp), ("edge_rank", _vp), ("bond_counts", _vp), ("edge_flag", _vp),
        ("edge_ptr", _vp),
        ("center", _vp), ("neighbor", _vp), ("image", _vp), ("dist", _vp), ("rev", _vp), ("d2u", _vp),
        ("u2d", _vp), ("trip_ptr", _vp), ("trip_src_ptr", _vp),
        ("line_graph", _vp), ("trip_src_perm", _vp),
        ("run_if", _vp), ("cand_ptr", _vp), ("cand_nbr", _vp), ("cand_img", _vp), ("cand_counts", _vp),
    ]


class MbSrc(C.Structure):
    _fields_ = [("ptr", _vp), ("idx", _vp), ("ld", _i64), ("col", _i32), ("act", _i32)]


class MbColBlock(C.Structure):
    _fields_ = [
        ("n_src", _i32), ("out_act", _i32), ("src", MbSrc * 4),
        ("W", _vp), ("W_hi", _vp), ("W_lo", _vp), ("W_hi16", _vp), ("W_lo16", _vp), ("ldw", _i64), ("bias", _vp),
        ("gate", _vp), ("ld_gate", _i64), ("col_gate", _i32), ("pad0", _i32),
        ("res", _vp), ("res_w", _vp), ("ld_res", _i64), ("col_res", _i32), ("mode", _i32),
        ("out", _vp), ("out_idx", _vp), ("ld_out", _i64), ("col_out", _i32), ("out_scale", _f32),
    ]


class MbGemmDesc(C.Structure):
    _fields_ = [("n_rows", _i64), ("n_blocks", _i32), ("pad", _i32), ("blk", MbColBlock * 4)]


class MbGatedMlp(C.Structure):
    _fields_ = [
        ("n_rows", _i64), ("n_src", _i32), ("kind", _i32), ("src", MbSrc * 4),
        ("W1", _vp), ("W1_hi", _vp), ("W1_lo", _vp), ("W1_hi16", _vp), ("W1_lo16", _vp), ("ldw1", _i64), ("b1", _vp),
        ("W2", _vp), ("W2_hi", _vp), ("W2_lo", _vp), ("W2_hi16", _vp), ("W2_lo16", _vp), ("ldw2", _i64), ("b2", _vp),
        ("norm_core", _vp), ("norm_gate", _vp),
        ("z1", _vp), ("ld_z1", _i64), ("z2", _vp), ("ld_z2", _i64), ("h", _vp), ("ld_h", _i64),
        ("res", _vp), ("res_w", _vp), ("ld_res", _i64), ("out2", _vp), ("ld_out2", _i64),
    ]


# name -> argtypes (every function returns int status unless listed in _OTHER)
_SIGNATURES = {
    "mb_graph_build": [C.POINTER(MbGraph), _vp],
    "mb_graph_status": [C.POINTER(C.c_int32)],
    "mb_graph_skin_check": [_i32, _vp, _vp, C.c_double, _vp, _vp],
    "mb_graph_skin_commit": [_i32, _vp, _vp, _vp, _vp],
    "mb_gemm": [C.POINTER(MbGemmDesc), _vp],
    "mb_set_gemm_mode": [C.c_int],
    "mb_gemm_status": [C.POINTER(C.c_int), _vp],
    "mb_gemm_status_async": [_vp, _vp],
    "mb_gemm_status_clear": [_vp],
    "mb_selftest_wait_expiry": [_vp],
    "mb_bench_mma_rate": [C.c_int, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_int), _vp],
    "mb_gated_mlp_fwd": [C.POINTER(MbGatedMlp), _vp],
    "mb_gate_fwd": [_i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "mb_gate_bwd": [_i64, _vp, _vp, _vp, _vp, _vp, _vp],
    "mb_seg_attn_fwd": [_i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "mb_seg_attn_bwd": [_i64, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f32, _vp, _vp, _vp, _vp,
                        _vp, _vp, _vp],
    "mb_seg_smooth_sum_fwd": [_i32, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp],
    "mb_seg_smooth_sum_bwd_rows": [_i64, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp],
    "mb_seg_smooth_sum_bwd_env": [_i32, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "mb_mul_rows_gather": [_i64, _vp, _vp, _vp, _vp, _vp],
    "mb_pair_mean_res": [_i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "mb_scale_rows": [_i64, _vp, _vp, _vp, _i32, _vp],
    "mb_small_linear_fwd": [_i64, _i32, _vp, _vp, _vp, _vp],
    "mb_small_linear_bwd": [_i64, _i32, _vp, _vp, _vp, _i32, _vp],
    "mb_layernorm_fwd": [_i64, _vp, _vp, _vp, _vp, _vp],
    "mb_layernorm_bwd": [_i64, _vp, _vp, _vp, _vp, _vp],
    "mb_rmsnorm_fwd": [_i64, _vp, _vp, _vp, _vp],
    "mb_rmsnorm_bwd": [_i64, _vp, _vp, _vp, _vp, _vp],
    "mb_embedding": [_i64, _vp, _i32, _vp, _vp, _vp],
    "mb_head_dot_fwd": [_i64, _i32, _vp, _vp, _vp, _i32, _vp, _vp],
    "mb_head_dot_bwd": [_i64, _i32, _vp, _vp, _vp, _vp, _vp, _vp],
    "mb_silu_bwd": [_i64, _vp, _vp, _vp, _vp],
    "mb_segment_sum_scalar": [_i32, _vp, _vp, _vp, _vp],
    "mb_edge_geometry_fwd": [_i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "mb_edge_geometry_bwd": [_i32, _i32, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "mb_edge_geometry_bwd_static": [_i32, _i32, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "mb_bessel_fwd": [_i32, _vp, _vp, _vp, _f32, _vp, _f32, _i32, _vp, _vp, _vp],
    "mb_bessel_bwd": [_i32, _vp, _vp, _vp, _f32, _vp, _f32, _i32, _vp, _vp, _vp, _vp],
    "mb_angle_basis_fwd": [_i64, _vp, _vp, _f32, _f32, _vp, _vp],
    "mb_angle_basis_bwd": [_i64, _vp, _vp, _f32, _f32, _vp, _vp, _vp],
    "mb_gaussian_fwd": [_i32, _vp, _vp, _vp, _f32, _vp, _f32, _vp, _vp, _vp],
    "mb_gaussian_bwd": [_i32, _vp, _vp, _vp, _f32, _vp, _f32, _vp, _vp, _vp, _vp],
    "mb_fourier_basis_fwd": [_i64, _vp, _vp, _vp, _vp, _vp],
    "mb_fourier_basis_bwd": [_i64, _vp, _vp, _vp, _vp, _vp, _vp],
}
_OTHER = {
    "mb_version": (C.c_int, []),
    "mb_status_string": (C.c_char_p, [C.c_int]),
    "mb_last_cuda_error": (C.c_char_p, []),
    "mb_graph_scan_tmp_len": (C.c_size_t, [_i64]),
}

_lib = None
launch_count = 0  # number of C-ABI compute calls issued (each launches >= 1 kernel)


def load() -> C.CDLL:
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise MbError(f"{LIB_PATH} is missing: build it with `python -m matris_b200.build` "
                      "(there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = C.c_int
    for name, (restype, argtypes) in _OTHER.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status == MB_OK:
        return
    lib = load()
    msg = lib.mb_status_string(status).decode()
    if status == 5:
        raise IsolatedAtomError("Error: Detected isolated atom. Calculation stopped")
    if status == 2:
        msg += ": " + lib.mb_last_cuda_error().decode()
    raise MbError(f"{what} failed with status {status} ({msg})")


profile = None       # set to a list to record (name, start_event, end_event, meta) around every call
profile_meta = None  # filled by the caller (e.g. algorithmic FLOPs of a GEMM) just before call()


_bound: dict = {}  # entry points by name, bound on first use


def call(name: str, *args) -> None:
    """Call an int-returning entry point and raise on a non-zero status."""
    global launch_count, profile_meta
    fn = _bound.get(name)
    if fn is None:
        fn = _bound[name] = getattr(load(), name)
    launch_count += 1
    if profile is None:
        status = fn(*args)
        if status:
            check(status, name)
        return
    lib = load()
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    check(getattr(lib, name)(*args), name)
    e1.record()
    profile.append((name, e0, e1, profile_meta))
    profile_meta = None


def ptr(t):
    """Device pointer of a tensor (None -> NULL).  The tensor must be contiguous
    from its first element on; views with a column offset are addressed through
    the (ld, col) arguments instead."""
    return None if t is None else t.data_ptr()
