"""ctypes binding of libss2d_b200.so (include/ss2d_b200.h).

There is no CPU or eager fallback: if the library is missing or cannot be loaded the
import of any operator fails with an explicit error.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libss2d_b200.so")

SS2D_F32, SS2D_F16, SS2D_BF16 = 0, 1, 2
SS2D_OK = 0
SS2D_ENOTSUP = -6
ROUTES = 4

_i32, _i64, _vp, _f32 = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_float


class ScanParams(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ("u", "delta", "A", "B", "C", "D", "delta_bias", "out")] + \
               [(n, _i32) for n in ("in_dtype", "out_dtype", "delta_softplus", "delta_ratio")] + \
               [(n, _i64) for n in ("batch", "dim", "dstate", "seqlen", "n_groups",
                                    "u_batch_stride", "u_dim_stride", "delta_batch_stride", "delta_dim_stride",
                                    "out_batch_stride", "out_dim_stride",
                                    "B_batch_stride", "B_group_stride", "B_state_stride",
                                    "C_batch_stride", "C_group_stride", "C_state_stride")] + \
               [("checkpoints", _vp)]


class ScanBwdParams(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ("u", "delta", "A", "B", "C", "D", "delta_bias", "dout",
                                   "du", "ddelta", "dA", "dB", "dC", "dD", "ddelta_bias", "workspace")] + \
               [("workspace_bytes", _i64)] + \
               [(n, _i32) for n in ("in_dtype", "dout_dtype", "delta_softplus", "delta_ratio")] + \
               [(n, _i64) for n in ("batch", "dim", "dstate", "seqlen", "n_groups",
                                    "u_batch_stride", "u_dim_stride", "delta_batch_stride", "delta_dim_stride",
                                    "dout_batch_stride", "dout_dim_stride",
                                    "B_batch_stride", "B_group_stride", "B_state_stride",
                                    "C_batch_stride", "C_group_stride", "C_state_stride")] + \
               [("checkpoints", _vp)]


class CrossParams(ctypes.Structure):
    _fields_ = [("in_", _vp), ("out", _vp), ("dtype", _i32), ("scans", _i32),
                ("B", _i64), ("C", _i64), ("H", _i64), ("W", _i64)]


class CrossExParams(ctypes.Structure):
    _fields_ = [("in_", _vp), ("out", _vp), ("dtype", _i32), ("scans", _i32), ("in_channel_first", _i32),
                ("out_channel_first", _i32), ("one_by_one", _i32), ("reserved0", _i32),
                ("B", _i64), ("C", _i64), ("H", _i64), ("W", _i64)]


class CoreParams(ctypes.Structure):
    _fields_ = [("x", _vp), ("delta", _vp * ROUTES), ("Bm", _vp * ROUTES), ("Cm", _vp * ROUTES),
                ("A", _vp), ("Dskip", _vp), ("delta_bias", _vp), ("ln_weight", _vp), ("ln_bias", _vp),
                ("y", _vp), ("workspace", _vp), ("workspace_bytes", _i64),
                ("delta_batch_stride", _i64 * ROUTES), ("bc_batch_stride", _i64 * ROUTES),
                ("B", _i64), ("D", _i64), ("H", _i64), ("W", _i64), ("N", _i64),
                ("act_dtype", _i32), ("y_dtype", _i32), ("with_norm", _i32), ("ln_eps", _f32),
                ("x_batch_stride", _i64), ("x_channel_stride", _i64), ("y_batch_stride", _i64), ("y_channel_stride", _i64),
                ("delta_channel_stride", _i64 * ROUTES)]


class ExpandParams(ctypes.Structure):
    _fields_ = [("x_dbl", _vp), ("dt_weight", _vp), ("delta", _vp * ROUTES), ("bc", _vp * ROUTES),
                ("x_dbl_batch_stride", _i64), ("x_dbl_route_stride", _i64), ("x_dbl_row_stride", _i64),
                ("delta_batch_stride", _i64 * ROUTES), ("bc_batch_stride", _i64 * ROUTES),
                ("delta_channel_stride", _i64 * ROUTES), ("bc_row_stride", _i64 * ROUTES),
                ("B", _i64), ("D", _i64), ("R", _i64), ("N", _i64), ("H", _i64), ("W", _i64),
                ("act_dtype", _i32), ("reserved0", _i32), ("workspace", _vp), ("workspace_bytes", _i64)]


class PointwiseParams(ctypes.Structure):
    _fields_ = [("x", _vp), ("weight", _vp), ("bias", _vp), ("y", _vp),
                ("B", _i64), ("D", _i64), ("H", _i64), ("W", _i64), ("dtype", _i32), ("act", _i32),
                ("channel_major", _i32), ("reserved0", _i32)]


class NormParams(ctypes.Structure):
    _fields_ = [("in_", _vp), ("add", _vp), ("add_bias", _vp), ("sum_out", _vp), ("weight", _vp), ("bias", _vp),
                ("out", _vp), ("B", _i64), ("D", _i64), ("L", _i64), ("batch_stride", _i64), ("channel_stride", _i64),
                ("out_batch_stride", _i64), ("out_channel_stride", _i64), ("io_dtype", _i32), ("eps", _f32),
                ("skip_norm", _i32), ("descending", _i32)]


class StemParams(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ("x", "weight", "conv_bias", "ln_weight", "ln_bias", "y")] + \
               [(n, _i64) for n in ("B", "H", "W", "C0", "in_channels")] + \
               [("dtype", _i32), ("act", _i32), ("eps", _f32), ("reserved0", _i32)]


class RelayoutParams(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ("rows", "planes", "add", "bias", "ln_weight", "ln_bias", "sum_out")] + \
               [(n, _i64) for n in ("N", "C", "plane_stride")] + \
               [("rows_dtype", _i32), ("planes_dtype", _i32), ("eps", _f32), ("reserved0", _i32)]


class MlpParams(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ("x", "w1", "b1", "w2", "y")] + [(n, _i64) for n in ("C", "hidden", "N")] + \
               [("dtype", _i32), ("reserved0", _i32)]


class LinearParams(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ("x", "w", "bias", "out")] + \
               [(n, _i64) for n in ("M", "K", "N", "x_row_stride", "out_row_stride")] + [("dtype", _i32), ("reserved0", _i32)]


EXPORTS = {
    # name: (restype, argtypes)
    "ss2d_selective_scan_fwd": (ctypes.c_int, [ctypes.POINTER(ScanParams), _vp]),
    "ss2d_selective_scan_bwd": (ctypes.c_int, [ctypes.POINTER(ScanBwdParams), _vp]),
    "ss2d_selective_scan_bwd_workspace_bytes": (_i64, [ctypes.POINTER(ScanBwdParams)]),
    "ss2d_cross_scan": (ctypes.c_int, [ctypes.POINTER(CrossParams), _vp]),
    "ss2d_cross_merge": (ctypes.c_int, [ctypes.POINTER(CrossParams), _vp]),
    "ss2d_cross_scan_ex": (ctypes.c_int, [ctypes.POINTER(CrossExParams), _vp]),
    "ss2d_cross_merge_ex": (ctypes.c_int, [ctypes.POINTER(CrossExParams), _vp]),
    "ss2d_core_workspace_bytes": (_i64, [ctypes.POINTER(CoreParams)]),
    "ss2d_core_fwd": (ctypes.c_int, [ctypes.POINTER(CoreParams), _vp]),
    "ss2d_core_supported": (ctypes.c_int, [ctypes.POINTER(CoreParams)]),
    "ss2d_core_fwd_static": (ctypes.c_int, [ctypes.POINTER(CoreParams), _vp]),
    "ss2d_core_static_capacity": (_i64, []),
    "ss2d_layer_norm_cf": (ctypes.c_int, [ctypes.POINTER(NormParams), _vp]),
    "ss2d_route_expand": (ctypes.c_int, [ctypes.POINTER(ExpandParams), _vp]),
    "ss2d_route_expand_workspace_bytes": (_i64, [ctypes.POINTER(ExpandParams)]),
    "ss2d_stem_conv_norm_act": (ctypes.c_int, [ctypes.POINTER(StemParams), _vp]),
    "ss2d_pixels_norm_to_planes": (ctypes.c_int, [ctypes.POINTER(RelayoutParams), _vp]),
    "ss2d_planes_to_pixels": (ctypes.c_int, [ctypes.POINTER(RelayoutParams), _vp]),
    "ss2d_bias_act": (ctypes.c_int, [ctypes.POINTER(PointwiseParams), _vp]),
    "ss2d_dwconv3x3_act": (ctypes.c_int, [ctypes.POINTER(PointwiseParams), _vp]),
    "ss2d_mlp_supported": (ctypes.c_int, [ctypes.POINTER(MlpParams)]),
    "ss2d_mlp_fwd": (ctypes.c_int, [ctypes.POINTER(MlpParams), _vp]),
    "ss2d_linear_supported": (ctypes.c_int, [ctypes.POINTER(LinearParams)]),
    "ss2d_linear_fwd": (ctypes.c_int, [ctypes.POINTER(LinearParams), _vp]),
    "ss2d_set_debug_checks": (ctypes.c_int, [ctypes.c_int]),
    "ss2d_version": (ctypes.c_int, []),
    "ss2d_strerror": (ctypes.c_char_p, [ctypes.c_int]),
    "ss2d_launch_count": (_i64, []),
}

_lib = None


class Ss2dError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().ss2d_strerror(status).decode()
        super().__init__(f"{where}: {msg} (status {status})")


def lib():
    """The loaded library; raises if it has not been built (python vmamba_b200/build.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} not found. vmamba_b200 has no CPU or eager fallback: build the CUDA "
                "library first with `python vmamba_b200/build.py` (needs nvcc, targets sm_100a).")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(handle, name)   # AttributeError if a declared symbol is missing
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int, where: str):
    if status != SS2D_OK:
        raise Ss2dError(status, where)


def launch_count() -> int:
    return int(lib().ss2d_launch_count())
