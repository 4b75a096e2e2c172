"""Installs the vmamba_b200 operators into MzeroMiko/VMamba's own modules, source untouched.

The reference resolves `selective_scan_fn`, `cross_scan_fn`, `cross_merge_fn` (and the Function
classes) as module globals at call time (vmamba.py:1532-1557), so replacing the attributes of the
imported module is enough for the one-file distribution.  The full tree
(classification/models/vmamba.py:22-30) imports the helpers from modules named `csm_triton` and
`csms6s`; `preseed_sys_modules()` registers stand-ins under those names before that import.
"""
from __future__ import annotations

import sys
import types

from . import ops

_SURFACE = (
    "selective_scan_fn", "SelectiveScanCuda", "SelectiveScanOflex",
    "cross_scan_fn", "cross_merge_fn", "CrossScanF", "CrossMergeF",
    "CrossScanTritonF", "CrossMergeTritonF", "CrossScan", "CrossMerge",
)


def install(module) -> dict:
    """Point the operator names of an imported reference module (e.g. root `vmamba`) at this
    package.  Returns the replaced attributes so that `uninstall` can restore them."""
    saved = {}
    for name in _SURFACE:
        if hasattr(module, name) or name in ("selective_scan_fn", "cross_scan_fn", "cross_merge_fn"):
            saved[name] = getattr(module, name, None)
            setattr(module, name, getattr(ops, name))
    # the reference falls back to its python loop when this flag is False (vmamba.py:884)
    if hasattr(module, "WITH_SELECTIVESCAN_MAMBA"):
        saved["WITH_SELECTIVESCAN_MAMBA"] = module.WITH_SELECTIVESCAN_MAMBA
        module.WITH_SELECTIVESCAN_MAMBA = True
    module.__vmamba_b200_saved__ = saved
    return saved


def uninstall(module) -> None:
    for name, val in getattr(module, "__vmamba_b200_saved__", {}).items():
        if val is None:
            if hasattr(module, name):
                delattr(module, name)
        else:
            setattr(module, name, val)
    if hasattr(module, "__vmamba_b200_saved__"):
        del module.__vmamba_b200_saved__


def preseed_sys_modules() -> None:
    """Register `csm_triton` and `csms6s` stand-ins so that `classification/models/vmamba.py`
    picks up the CUDA-backed operators when it is imported afterwards."""
    csm = types.ModuleType("csm_triton")
    for name in ("cross_scan_fn", "cross_merge_fn", "CrossScanF", "CrossMergeF", "CrossScanTritonF",
                 "CrossMergeTritonF"):
        setattr(csm, name, getattr(ops, name))
    s6 = types.ModuleType("csms6s")
    for name in ("selective_scan_fn", "SelectiveScanCuda", "SelectiveScanOflex"):
        setattr(s6, name, getattr(ops, name))
    s6.selective_scan_flop_jit = ops.selective_scan_flop_jit
    s6.flops_selective_scan_fn = ops.flops_selective_scan_fn
    sys.modules.setdefault("csm_triton", csm)
    sys.modules.setdefault("csms6s", s6)


def preseed_extension_module() -> None:
    """Register the stand-in for the compiled extension `selective_scan_cuda_oflex`, so that the
    reference's OWN csms6s.py (imported unchanged afterwards) finds it and routes
    SelectiveScanCuda.forward / backward through this library (csms6s.py:9-14, 81, 97-99)."""
    sys.modules.setdefault("selective_scan_cuda_oflex", ops.selective_scan_cuda_oflex)
