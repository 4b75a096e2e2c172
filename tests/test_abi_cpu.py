"""CPU-side checks of the C-ABI library: it loads, exports every declared symbol, the ctypes
mirrors match the C structs, and argument validation rejects bad calls before any launch."""
import ctypes
import os
import re
import subprocess

import pytest

from vmamba_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ss2d_b200.h")


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(ss2d_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert "ss2d_selective_scan_fwd" in names and "ss2d_core_fwd" in names
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} declared in include/ss2d_b200.h but not exported"
    assert set(names) == set(_lib.EXPORTS), "python binding and header disagree on the entry points"


def test_struct_layout_matches_header(tmp_path):
    prog = tmp_path / "sz.c"
    prog.write_text('#include "ss2d_b200.h"\n#include <stdio.h>\n#include <stddef.h>\nint main(){printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n",'
                    'sizeof(ss2d_scan_params),sizeof(ss2d_cross_params),sizeof(ss2d_core_params),sizeof(ss2d_norm_params),'
                    'offsetof(ss2d_core_params,delta_batch_stride),offsetof(ss2d_scan_params,batch),'
                    'sizeof(ss2d_expand_params),sizeof(ss2d_pointwise_params),offsetof(ss2d_expand_params,B),'
                    'offsetof(ss2d_norm_params,io_dtype),sizeof(ss2d_scan_bwd_params),offsetof(ss2d_scan_bwd_params,in_dtype),'
                    'offsetof(ss2d_scan_bwd_params,C_state_stride),sizeof(ss2d_linear_params),offsetof(ss2d_linear_params,dtype),'
                    'sizeof(ss2d_mlp_params),offsetof(ss2d_mlp_params,dtype));return 0;}\n')
    exe = tmp_path / "sz"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(prog), "-o", str(exe)])
    got = [int(t) for t in subprocess.check_output([str(exe)]).split()]
    want = [ctypes.sizeof(_lib.ScanParams), ctypes.sizeof(_lib.CrossParams), ctypes.sizeof(_lib.CoreParams),
            ctypes.sizeof(_lib.NormParams), _lib.CoreParams.delta_batch_stride.offset, _lib.ScanParams.batch.offset,
            ctypes.sizeof(_lib.ExpandParams), ctypes.sizeof(_lib.PointwiseParams), _lib.ExpandParams.B.offset,
            _lib.NormParams.io_dtype.offset, ctypes.sizeof(_lib.ScanBwdParams), _lib.ScanBwdParams.in_dtype.offset,
            _lib.ScanBwdParams.C_state_stride.offset, ctypes.sizeof(_lib.LinearParams), _lib.LinearParams.dtype.offset,
            ctypes.sizeof(_lib.MlpParams), _lib.MlpParams.dtype.offset]
    assert got == want


def test_version_and_strerror():
    L = _lib.lib()
    assert L.ss2d_version() == 1
    assert L.ss2d_strerror(0) == b"ok"
    assert b"NULL" in L.ss2d_strerror(-1)
    assert L.ss2d_strerror(-99) == b"unknown status"


def test_validation_rejects_before_launch():
    """None of these calls reaches a kernel launch, so they run without a GPU."""
    L = _lib.lib()
    before = _lib.launch_count()
    assert L.ss2d_selective_scan_fwd(None, None) == -1
    p = _lib.ScanParams()
    assert L.ss2d_selective_scan_fwd(p, None) == -1                 # null tensors
    buf = (ctypes.c_float * 64)()
    addr = ctypes.addressof(buf)
    for f in ("u", "delta", "A", "B", "C", "out"):
        setattr(p, f, addr)
    p.in_dtype = 7
    assert L.ss2d_selective_scan_fwd(p, None) == -3                 # bad dtype
    p.in_dtype, p.out_dtype = _lib.SS2D_BF16, _lib.SS2D_F16
    assert L.ss2d_selective_scan_fwd(p, None) == -3                 # out must be fp32 or the input type
    p.in_dtype = p.out_dtype = _lib.SS2D_F32
    assert L.ss2d_selective_scan_fwd(p, None) == -2                 # zero sizes
    p.batch, p.dim, p.dstate, p.seqlen, p.n_groups = 1, 6, 1, 8, 4
    assert L.ss2d_selective_scan_fwd(p, None) == -2                 # dim not a multiple of groups
    p.dim = 8
    p.dstate = 1000
    assert L.ss2d_selective_scan_fwd(p, None) == -6                 # d_state above the limit
    p.dstate = 1
    assert L.ss2d_selective_scan_fwd(p, None) == -5                 # strides smaller than the row
    for f in ("u_dim_stride", "delta_dim_stride", "out_dim_stride", "B_state_stride", "C_state_stride",
              "B_group_stride", "C_group_stride"):
        setattr(p, f, 8)
    p.u = addr + 2
    assert L.ss2d_selective_scan_fwd(p, None) == -4                 # misaligned fp32 pointer

    c = _lib.CrossParams()
    assert L.ss2d_cross_scan(c, None) == -1
    c.in_, c.out, c.dtype, c.scans = addr, addr, 0, 9
    assert L.ss2d_cross_scan(c, None) == -6
    c.scans = 0
    assert L.ss2d_cross_merge(c, None) == -2

    k = _lib.CoreParams()
    assert L.ss2d_core_fwd(k, None) == -1
    assert L.ss2d_core_workspace_bytes(k) == -1
    n = _lib.NormParams()
    assert L.ss2d_layer_norm_cf(n, None) == -1
    assert _lib.launch_count() == before


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU or eager fallback"):
        _lib.lib()


def test_operators_refuse_cpu_tensors():
    import torch
    import vmamba_b200 as vb
    x = torch.zeros(1, 2, 3, 4)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        vb.cross_scan_fn(x)
    with pytest.raises(NotImplementedError):
        vb.selective_scan_fn(x, x, x, x, x, backend="torch")
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        vb.cross_scan_fn(x, in_channel_first=False)
    with pytest.raises(NotImplementedError):         # one_by_one with a channel-last side: route sets 0-2 only
        vb.cross_scan_fn(torch.zeros(1, 3, 3, 4, 2), in_channel_first=False, out_channel_first=False, one_by_one=True, scans=3)


def test_install_patches_a_reference_like_module():
    """`install` swaps the operator names a reference module resolves at call time; `uninstall` restores them."""
    import types
    import vmamba_b200 as vb
    from vmamba_b200 import ops
    fake = types.ModuleType("vmamba")
    fake.selective_scan_fn = lambda *a, **k: "torch loop"
    fake.cross_scan_fn = lambda *a, **k: "torch"
    fake.cross_merge_fn = lambda *a, **k: "torch"
    fake.SelectiveScanCuda = object
    fake.WITH_SELECTIVESCAN_MAMBA = False
    vb.install(fake)
    assert fake.selective_scan_fn is ops.selective_scan_fn and fake.cross_scan_fn is ops.cross_scan_fn
    assert fake.cross_merge_fn is ops.cross_merge_fn and fake.SelectiveScanCuda is ops.SelectiveScanCuda
    assert fake.WITH_SELECTIVESCAN_MAMBA is True
    vb.uninstall(fake)
    assert fake.selective_scan_fn() == "torch loop" and fake.WITH_SELECTIVESCAN_MAMBA is False
    import sys
    saved = {k: sys.modules.pop(k, None) for k in ("csm_triton", "csms6s")}
    try:
        vb.preseed_sys_modules()
        assert sys.modules["csms6s"].selective_scan_fn is ops.selective_scan_fn
        assert sys.modules["csm_triton"].cross_scan_fn is ops.cross_scan_fn
        assert sys.modules["csms6s"].flops_selective_scan_fn is ops.flops_selective_scan_fn
    finally:
        for k, v in saved.items():
            sys.modules.pop(k, None)
            if v is not None:
                sys.modules[k] = v
    saved = sys.modules.pop("selective_scan_cuda_oflex", None)
    try:
        vb.preseed_extension_module()
        import selective_scan_cuda_oflex as ext      # what the reference's csms6s.py does (csms6s.py:9-14)
        assert ext is ops.selective_scan_cuda_oflex and callable(ext.fwd) and callable(ext.bwd)
    finally:
        sys.modules.pop("selective_scan_cuda_oflex", None)
        if saved is not None:
            sys.modules["selective_scan_cuda_oflex"] = saved


def test_flop_helpers_match_the_reference_formula():
    """9 B L D N (+ B D L for the D skip, + B D L for a z gate): csms6s.py:136-160; the jit handle reads
    the sizes of u and A from the traced inputs (csms6s.py:212-219)."""
    import vmamba_b200 as vb
    assert vb.flops_selective_scan_fn(B=2, L=3136, D=384, N=1) == 9 * 2 * 3136 * 384 + 2 * 384 * 3136
    assert vb.flops_selective_scan_fn(B=1, L=10, D=4, N=16, with_D=False, with_Z=True) == 9 * 10 * 4 * 16 + 4 * 10

    class _T:
        def __init__(self, sizes):
            self._s = sizes

        def type(self):
            return self

        def sizes(self):
            return self._s

    ins = [_T([2, 384, 3136]), _T([2, 384, 3136]), _T([384, 1])]
    assert vb.selective_scan_flop_jit(ins, None, verbose=False) == vb.flops_selective_scan_fn(B=2, L=3136, D=384, N=1)


def test_enable_fused_selects_supported_modules_only():
    import functools
    import torch
    import vmamba_b200 as vb

    class FakeSS2D(torch.nn.Module):
        def __init__(self, scan_mode="cross2d", channel_first=True, norm=True):
            super().__init__()
            self.channel_first = channel_first
            self.d_state, self.dt_rank = 1, 1
            self.x_proj = torch.nn.Linear(4, 12, bias=False)
            self.dt_projs = torch.nn.Linear(1, 16, bias=False)
            self.A_logs = torch.nn.Parameter(torch.zeros(16, 1))
            self.Ds = torch.nn.Parameter(torch.ones(16))
            self.dt_projs_bias = torch.nn.Parameter(torch.zeros(4, 4))
            self.out_norm = torch.nn.LayerNorm(4) if norm else torch.nn.Identity()
            self.forward_core = functools.partial(self._core, scan_mode=scan_mode)

        def _core(self, x, scan_mode="cross2d"):
            return x

    model = torch.nn.Sequential(FakeSS2D(), FakeSS2D(scan_mode="unidi"), FakeSS2D(channel_first=False), FakeSS2D(norm=False))
    assert vb.enable_fused(model) == 1
    x = torch.zeros(1, 4, 2, 2)
    assert model[0].forward_core(x) is x          # CPU tensor: falls through to the original core
    assert vb.disable_fused(model) == 1
    assert isinstance(model[0].forward_core, functools.partial)


def test_checkpoint_key_normalisation():
    """Older checkpoint namings are mapped as the reference's loaders map them (vmamba.py:1682-1697, 2061-2102)."""
    import torch
    from vmamba_b200.backbone import normalize_state_dict
    z = torch.zeros(1)
    old = {"model": {
        "module.patch_embed.proj.weight": z, "patch_embed.norm.bias": z,
        "layers.0.blocks.1.ln_1.weight": z, "layers.0.blocks.1.self_attention.x_proj_weight": z,
        "layers.0.blocks.1.self_attention.dt_projs_weight": z, "layers.0.blocks.1.self_attention.dt_projs_bias": z,
        "layers.2.downsample.norm.weight": z, "layers.2.downsample.reduction.weight": z,
        "norm.weight": z, "head.bias": z, "layers.0.blocks.0.op.A_logs": z}}
    new = normalize_state_dict(old)
    assert set(new) == {
        "patch_embed.0.weight", "patch_embed.2.bias", "layers.0.blocks.1.norm.weight",
        "layers.0.blocks.1.op.x_proj.weight", "layers.0.blocks.1.op.dt_projs.weight", "layers.0.blocks.1.op.dt_projs_bias",
        "layers.2.downsample.1.weight", "layers.2.downsample.2.weight", "classifier.norm.weight", "classifier.head.bias",
        "layers.0.blocks.0.op.A_logs"}
    same = normalize_state_dict(new)
    assert set(same) == set(new)


def test_tensor_core_planners_answer_without_a_gpu():
    """`ss2d_linear_supported` / `ss2d_mlp_supported` decide from the parameter block alone: what the tcgen05 kernels take,
    what goes to the library GEMM; nothing is launched."""
    import torch
    from vmamba_b200 import ops
    before = _lib.launch_count()
    bf = torch.bfloat16
    assert ops.linear_supported(32, 96, 128 * 3136, bf)            # x_proj of VMamba-T stage 0
    assert ops.linear_supported(56, 192, 128 * 784, torch.float16)
    assert ops.linear_supported(104, 384, 128 * 196, bf)
    assert not ops.linear_supported(200, 768, 128 * 49, bf)        # stage 3: the stacked weights leave no room for the ring
    assert not ops.linear_supported(32, 96, 1001, bf)              # rows not a multiple of 16 bytes
    assert not ops.linear_supported(32, 96, 1024, torch.float32)
    assert ops.mlp_supported(96, 384, 128 * 3136, bf)
    assert not ops.mlp_supported(192, 768, 128 * 784, bf)
    L = _lib.lib()
    assert L.ss2d_linear_fwd(None, None) == -1 and L.ss2d_linear_supported(None) == -1
    p = _lib.LinearParams()
    assert L.ss2d_linear_fwd(p, None) == -1                        # null tensors
    assert _lib.launch_count() == before


def test_backward_planner_picks_the_rows_kernels_by_row_count():
    """`ss2d_selective_scan_bwd_workspace_bytes` is the planner's answer without a launch: the lanes-are-rows kernels
    (one dB / dC partial per 32 rows of a group) are taken with the forward call's checkpoints and enough rows, the
    warp-per-row kernels (a partial per CTA of 8 rows, d_state > 1) otherwise."""
    L = _lib.lib()
    dummy = 0x10000                       # any aligned non-null address: the planner only looks at alignment

    def ws(batch, dim, N, seqlen, groups, ckpt):
        p = _lib.ScanBwdParams()
        for name in ("u", "delta", "A", "B", "C", "dout", "du", "ddelta", "dA", "dB", "dC"):
            setattr(p, name, dummy)
        p.in_dtype, p.dout_dtype, p.delta_softplus = 2, 0, 1          # bf16 rows, fp32 dout
        p.batch, p.dim, p.dstate, p.seqlen, p.n_groups = batch, dim, N, seqlen, groups
        p.u_batch_stride = p.delta_batch_stride = p.dout_batch_stride = dim * seqlen
        p.u_dim_stride = p.delta_dim_stride = p.dout_dim_stride = seqlen
        p.B_batch_stride = p.C_batch_stride = groups * N * seqlen
        p.B_group_stride = p.C_group_stride = N * seqlen
        p.B_state_stride = p.C_state_stride = seqlen
        p.checkpoints = dummy if ckpt else None
        return L.ss2d_selective_scan_bwd_workspace_bytes(p)

    def expect(batch, dim, N, seqlen, groups, parts):
        return 4 * (batch * dim * (N + 2) + batch * groups * parts * 2 * N * seqlen)

    before = _lib.launch_count()
    gs = 768
    # d_state 16: 6144 rows with checkpoints -> a partial per 32 rows; without checkpoints or with too few rows -> per 8 rows
    assert ws(2, 4 * gs, 16, 3136, 4, True) == expect(2, 4 * gs, 16, 3136, 4, gs // 32)
    assert ws(2, 4 * gs, 16, 3136, 4, False) == expect(2, 4 * gs, 16, 3136, 4, gs // 8)
    assert ws(1, 4 * gs, 16, 3136, 4, True) == expect(1, 4 * gs, 16, 3136, 4, gs // 8)
    # d_state 1: from 33 152 rows up
    assert ws(16, 4 * gs, 1, 784, 4, True) == expect(16, 4 * gs, 1, 784, 4, gs // 32)
    assert ws(8, 4 * gs, 1, 784, 4, True) != expect(8, 4 * gs, 1, 784, 4, gs // 32)
    assert ws(2, 4 * gs, 16, 0, 4, True) < 0                          # invalid sizes: no plan
    assert _lib.launch_count() == before


def test_accelerate_refuses_modules_that_are_not_on_a_gpu():
    import torch
    import vmamba_b200 as vb
    with pytest.raises(RuntimeError, match="CUDA"):
        vb.accelerate(torch.nn.Linear(4, 4))
