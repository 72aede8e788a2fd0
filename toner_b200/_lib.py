"""ctypes binding of libtoner_b200.so (the C ABI declared in include/toner_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libtoner_b200.so")

_lib: Optional[C.CDLL] = None


class TonerError(RuntimeError):
    """A C-ABI entry point returned a non-zero code."""


class Operand(C.Structure):
    _fields_ = [
        ("base", C.c_void_p), ("list", C.POINTER(C.c_void_p)),
        ("rows", C.c_int32), ("cols", C.c_int32),
        ("ld", C.c_int64), ("z_stride", C.c_int64),
        ("nz", C.c_int32), ("mn_major", C.c_int32),
        ("seg_z", C.c_int32 * 3), ("z_step", C.c_int32),
    ]


class CaptureJob(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("b", C.c_void_p), ("dst", C.c_void_p),
        ("batch_stride", C.c_int64), ("row_stride", C.c_int64),
        ("width", C.c_int32), ("kind", C.c_int32),
    ]


class GemmDesc(C.Structure):
    _fields_ = [
        ("a", Operand), ("b", Operand),
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("batch", C.c_int32),
        ("segs", C.c_int32), ("fmt", C.c_int32), ("tri", C.c_int32), ("mirror", C.c_int32), ("packed", C.c_int32),
        ("alpha", C.c_float), ("beta", C.c_float),
        ("alpha_a", C.c_void_p), ("alpha_b", C.c_void_p), ("beta_v", C.c_void_p), ("alpha_b_step", C.c_int32),
        ("c", C.c_void_p), ("ldc", C.c_int64), ("c_bs", C.c_int64),
        ("d", C.c_void_p), ("ldd", C.c_int64), ("d_bs", C.c_int64),
        ("d16", C.c_void_p), ("ld16", C.c_int64), ("d16_bs", C.c_int64), ("d16_fmt", C.c_int32),
        ("sumsq", C.c_void_p), ("maxabs", C.c_void_p), ("maxaff", C.c_void_p),
        ("aff_a", C.c_float), ("aff_b", C.c_float),
        ("tile_n", C.c_int32), ("promote", C.c_int32), ("raster", C.c_int32), ("promote_all", C.c_int32),
        ("split0", C.c_void_p), ("split1", C.c_void_p),
        ("split_ld", C.c_int64), ("split_bs", C.c_int64), ("split_plane", C.c_int64),
        ("split0_scale", C.c_float), ("split1_scale", C.c_float), ("split1_aff_a", C.c_float), ("split1_aff_b", C.c_float),
        ("maxres", C.c_void_p),
        ("upper_d", C.c_int32),
    ]


# name -> (restype, argtypes).  Every symbol include/toner_b200.h declares is listed here.
_vp, _i32, _i64, _f32, _sz = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_size_t
SIGNATURES = {
    "toner_init": (C.c_int, [C.c_int]),
    "toner_last_error": (C.c_char_p, []),
    "toner_sm_count": (C.c_int, []),
    "toner_launch_count": (C.c_longlong, []),
    "toner_device_status": (C.c_int, [_vp, C.POINTER(C.c_int)]),
    "toner_status_snapshot": (C.c_int, [_vp, _vp]),
    "toner_gemm": (C.c_int, [C.POINTER(GemmDesc), _vp]),
    "toner_set_gemm_sm_limit": (C.c_int, [_i32]),
    "toner_selftest_bounded_wait": (C.c_int, [C.c_longlong, _vp]),
    "toner_gemm_phase_cycles": (C.c_int, [C.c_int, _vp, C.POINTER(C.c_uint64)]),
    "toner_syrk_upper": (C.c_int, [C.POINTER(_vp), _vp, _i64, _i32, _i32, _i32, _i64, _vp, _i32, _f32, _f32, _vp]),
    "toner_unpack_ema": (C.c_int, [_vp, _vp, _i32, _i32, _f32, _f32, _vp]),
    "toner_inv_roots_workspace_bytes": (C.c_size_t, [_i32, _i32]),
    "toner_inv_roots_iterations": (C.c_int, [_i32, _f32, _i32]),
    "toner_inv_roots": (C.c_int, [_vp, _i32, _i32, _f32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "toner_inv_roots_iterations_for": (C.c_int, [_f32, _i32]),
    "toner_inv_roots_finish_order_for": (C.c_int, [_f32, _i32, _i32]),
    "toner_inv_roots_schedule": (C.c_int, [_f32, _i32, _i32, C.POINTER(C.c_double), _i32, C.POINTER(C.c_double), _i32,
                                           C.POINTER(_i32), C.POINTER(C.c_double)]),
    "toner_inv_roots_ex": (C.c_int, [_vp, _i32, _i32, _f32, _i32, _i32, _i32, _f32, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "toner_inv_roots_tracked": (C.c_int, [_vp, _i32, _i32, _f32, _i32, _i32, _i32, _f32, _i32, _vp, _vp, _vp, _vp, _vp, _vp,
                                          _vp, _vp, _i32, _vp, _i32, _vp, _vp, _sz, _vp]),
    "toner_ns_polar_workspace_bytes": (C.c_size_t, [_i32, _i32, _i32]),
    "toner_ns_polar": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _f32, _vp, _vp, _vp, _sz, _vp]),
    "toner_sumsq_scratch_bytes": (C.c_size_t, [_i32]),
    "toner_sumsq": (C.c_int, [_vp, _i32, _i32, _i32, _i64, _i64, _vp, _vp, _vp]),
    "toner_gather_rows": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _i64, _i64, _vp, _i32, _vp, _vp]),
    "toner_capture": (C.c_int, [_vp, _vp, _i32, _vp, _vp, _i32, _i32, _f32, _vp]),
    "toner_sumsq_static_max_batch": (C.c_int, []),
    "toner_sumsq_static": (C.c_int, [_vp, _i32, _i32, _i32, _i64, _i64, _vp, _vp]),
    "toner_muont_momentum": (C.c_int, [_vp, _vp, _vp, _i32, _i64, _f32, _i32, _vp, _vp]),
    "toner_muont_coeffs": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _f32, _f32, _f32, _vp, _vp, _vp]),
    "toner_scale_vec": (C.c_int, [_vp, _vp, _i32, _vp]),
    "toner_adamt_first_moment": (C.c_int, [_vp, _vp, _i32, _i64, _f32, _vp]),
    "toner_adamt_ratio": (C.c_int, [_vp, _vp, _vp, _i32, _i64, _f32, _f32, _f32, _vp, _vp]),
    "toner_adamt_coeffs": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _f32, _f32, _vp, _vp, _vp, _vp, _vp]),
    "toner_axpby": (C.c_int, [_vp, _vp, _vp, _i64, _f32, _f32, _vp]),
    "toner_scale_stack": (C.c_int, [_vp, _vp, _vp, _i32, _i64, _vp]),
    "toner_apply_delta": (C.c_int, [_vp, _vp, _i32, _i64, _vp]),
    "toner_apply_scaled": (C.c_int, [_vp, _vp, _i32, _i64, _f32, _f32, _vp]),
    "toner_split16": (C.c_int, [_vp, _vp, _i32, _i32, _i32, _i64, _i64, _f32, _f32, _vp, _vp, _vp, _vp, _vp]),
}


def load() -> C.CDLL:
    """Load the shared library once and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise TonerError(
            f"{LIB_PATH} is missing: build it with `python -m toner_b200.csrc.build` "
            "(toner_b200 has no CPU or PyTorch fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().toner_last_error()
        raise TonerError(f"{what} failed (code {code}): {msg.decode() if msg else 'unknown error'}")
