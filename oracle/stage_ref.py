"""Stages the reference's own Python files for the GPU tests (test infrastructure only).

    python oracle/stage_ref.py [--ref /path/to/VMamba]

Copies, unmodified, the one-file distribution `vmamba.py` and, from `classification/models/`,
`csms6s.py`, `csm_triton.py` and the full `vmamba.py` (staged as `tree_vmamba.py`: it holds the
cascade scan mode, which the one-file distribution dropped) of a MzeroMiko/VMamba checkout into
`oracle/_ref/`.  That folder is git-ignored: nothing of the
reference enters the history, the copy only travels with the working tree to machines that have
no checkout (the GPU box), where `tests/test_gpu_reference_modules.py` and `bench.py` run the
unmodified modules on this library's operators.  Without a checkout the script does nothing and
those tests skip.

`load(name)` imports a staged file with stand-ins for the two third-party packages the reference
imports but does not need for inference (`timm`, `fvcore`).
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import shutil
import sys
import types
import warnings

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
_MODELS = os.path.join("classification", "models")
FILES = {"vmamba.py": "vmamba.py", "csms6s.py": os.path.join(_MODELS, "csms6s.py"),
         "csm_triton.py": os.path.join(_MODELS, "csm_triton.py"), "tree_vmamba.py": os.path.join(_MODELS, "vmamba.py")}


def default_checkout() -> str:
    """Where a VMamba checkout is looked for: $VMAMBA_REFERENCE, else a folder `reference` beside this repository."""
    return os.environ.get("VMAMBA_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def stage(ref_root: str | None = None) -> list:
    done = []
    ref_root = ref_root or default_checkout()
    if not os.path.isdir(ref_root):
        return done
    os.makedirs(REF_DIR, exist_ok=True)
    for name, rel in FILES.items():
        src = os.path.join(ref_root, rel)
        if os.path.exists(src):
            shutil.copyfile(src, os.path.join(REF_DIR, name))
            done.append(name)
    return done


def staged(name: str = "vmamba.py") -> bool:
    return os.path.exists(os.path.join(REF_DIR, name))


def _install_stubs():
    """Stand-ins for the timm / fvcore symbols that vmamba.py imports at module import (vmamba.py:1047-1048, 2161)."""
    import torch
    try:
        import timm  # noqa: F401
    except ImportError:
        timm = types.ModuleType("timm")
        models = types.ModuleType("timm.models")
        layers = types.ModuleType("timm.models.layers")

        class DropPath(torch.nn.Module):
            def __init__(self, drop_prob=0.0):
                super().__init__()
                self.drop_prob = drop_prob

            def forward(self, x):      # inference: identity
                return x

        layers.DropPath = DropPath
        layers.trunc_normal_ = torch.nn.init.trunc_normal_
        models.register_model = lambda fn: fn
        models.layers = layers
        timm.models = models
        sys.modules.update({"timm": timm, "timm.models": models, "timm.models.layers": layers})
    try:
        import fvcore  # noqa: F401
    except ImportError:
        fv = types.ModuleType("fvcore")
        nn = types.ModuleType("fvcore.nn")
        for name in ("FlopCountAnalysis", "flop_count_str", "flop_count", "parameter_count"):
            setattr(nn, name, None)
        fv.nn = nn
        sys.modules.update({"fvcore": fv, "fvcore.nn": nn})
    if "mamba2.ssd_minimal" not in sys.modules:
        # classification/models/vmamba.py:33-36 imports the chunked Mamba-2 scan of its `m0` family at module import;
        # that family is not staged, the name only has to resolve
        pkg, mod = types.ModuleType("mamba2"), types.ModuleType("mamba2.ssd_minimal")
        mod.selective_scan_chunk_fn = None
        pkg.ssd_minimal = mod
        sys.modules.update({"mamba2": pkg, "mamba2.ssd_minimal": mod})


def load(name: str = "vmamba.py", module_name: str | None = None):
    """Import a staged reference file under `module_name` (default: its own name without .py)."""
    path = os.path.join(REF_DIR, name)
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path}: run `python oracle/stage_ref.py` where a VMamba checkout is available")
    _install_stubs()
    module_name = module_name or name[:-3]
    spec = importlib.util.spec_from_file_location(module_name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[module_name] = mod
    sys.path.insert(0, REF_DIR)         # tree_vmamba.py falls back to `from csm_triton import ...` (vmamba.py:22-30)
    try:
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            spec.loader.exec_module(mod)
    finally:
        sys.path.remove(REF_DIR)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=None, help="VMamba checkout (default: $VMAMBA_REFERENCE or ../reference)")
    print("staged:", stage(ap.parse_args().ref))
