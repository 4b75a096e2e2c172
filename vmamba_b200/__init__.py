"""vmamba_b200: the SS2D core of VMamba as hand-written sm_100a CUDA behind the reference's
operator surface.  Importing the package loads libss2d_b200.so and fails loudly if it is absent."""
from . import _lib

_lib.lib()   # no CUDA library, no package: there is no CPU or eager fallback

from .ops import (CrossMerge, CrossMergeF, CrossMergeTritonF, CrossScan, CrossScanF, CrossScanTritonF,  # noqa: E402
                  SelectiveScanCuda, SelectiveScanOflex, cross_merge_fn, cross_merge_fwd, cross_scan_fn,
                  cross_scan_fwd, flops_selective_scan_fn, layer_norm_cf, selective_scan_bwd, selective_scan_cuda_oflex,
                  selective_scan_flop_jit, selective_scan_fn, selective_scan_fwd)
from .fused import CoreWeights, disable_fused, enable_fused, ss2d_core, ss2d_core_autograd  # noqa: E402
from .patch import install, preseed_extension_module, preseed_sys_modules, uninstall  # noqa: E402
from .runner import GraphedBackbone  # noqa: E402
from .backbone import AcceleratedVSSM, VSSMInfer, accelerate  # noqa: E402

__all__ = [
    "selective_scan_fn", "selective_scan_fwd", "selective_scan_bwd", "SelectiveScanCuda", "SelectiveScanOflex",
    "selective_scan_cuda_oflex", "flops_selective_scan_fn", "selective_scan_flop_jit",
    "cross_scan_fn", "cross_merge_fn", "cross_scan_fwd", "cross_merge_fwd",
    "CrossScanF", "CrossMergeF", "CrossScanTritonF", "CrossMergeTritonF", "CrossScan", "CrossMerge",
    "layer_norm_cf", "ss2d_core", "ss2d_core_autograd", "CoreWeights", "enable_fused", "disable_fused",
    "install", "uninstall", "preseed_sys_modules", "preseed_extension_module", "GraphedBackbone",
    "VSSMInfer", "AcceleratedVSSM", "accelerate",
]
