"""ctypes front-end of the C oracle (oracle/ss2d_oracle.c) -- TEST INFRASTRUCTURE.

Same functions as oracle/ss2d_oracle.py, float32 in / float32 out, multi-threaded
with OpenMP.  Used where the numpy statement would take minutes (full-size
workloads, the timed CPU baseline).  Never imported by the `vmamba_b200` package.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libss2d_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "ss2d_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        i64, fp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        _lib.orc_cross_scan.argtypes = [fp, fp, i64, i64, i64, i64, ci]
        _lib.orc_cross_scan.restype = None
        _lib.orc_cross_merge.argtypes = [fp, fp, i64, i64, i64, i64, ci]
        _lib.orc_cross_merge.restype = None
        _lib.orc_selective_scan.argtypes = [fp] * 8 + [i64] * 5 + [ci]
        _lib.orc_selective_scan.restype = ci
        _lib.orc_layer_norm_cf.argtypes = [fp, fp, fp, fp, i64, i64, i64, ctypes.c_float]
        _lib.orc_layer_norm_cf.restype = None
    return _lib


def _c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def cross_scan(x, scans=0):
    x = _c(x)
    B, C, H, W = x.shape
    y = np.empty((B, 4, C, H * W), dtype=np.float32)
    lib().orc_cross_scan(_p(x), _p(y), B, C, H, W, scans)
    return y


def cross_merge(ys, scans=0):
    ys = _c(ys)
    B, K, C, H, W = ys.shape
    assert K == 4
    y = np.empty((B, C, H * W), dtype=np.float32)
    lib().orc_cross_merge(_p(ys), _p(y), B, C, H, W, scans)
    return y


def selective_scan(u, delta, A, B, C, D=None, delta_bias=None, delta_softplus=True):
    """fp32 state and output (the `oflex=True` form); callers round if they need to."""
    u, delta, A, B, C = _c(u), _c(delta), _c(A), _c(B), _c(C)
    Bt, K, N, L = B.shape
    KC = u.shape[1]
    assert KC % K == 0 and A.shape == (KC, N) and delta.shape == u.shape == (Bt, KC, L)
    D = None if D is None else _c(D)
    bias = None if delta_bias is None else _c(delta_bias)
    out = np.empty_like(u)
    rc = lib().orc_selective_scan(_p(u), _p(delta), _p(A), _p(B), _p(C), _p(D), _p(bias), _p(out),
                                  Bt, K, KC // K, N, L, int(bool(delta_softplus)))
    if rc != 0:
        raise ValueError("orc_selective_scan: unsupported d_state")
    return out


def layer_norm_cf(y, weight=None, bias=None, eps=1e-5):
    y = _c(y)
    shp = y.shape
    B, D = shp[0], shp[1]
    L = int(np.prod(shp[2:]))
    w = None if weight is None else _c(weight)
    b = None if bias is None else _c(bias)
    out = np.empty_like(y)
    lib().orc_layer_norm_cf(_p(y), _p(w), _p(b), _p(out), B, D, L, eps)
    return out
