"""The UNMODIFIED reference modules on this library's operators, on a GPU.

`oracle/stage_ref.py` stages the reference's own `vmamba.py` and `csms6s.py` (git-ignored copies that travel
with the working tree); here its `VSSM` is built on the GPU, the operator names it resolves at call time are
pointed at the CUDA library (`install`, vmamba.py:1532-1557), then its SS2D cores are rebound to the fused
call (`enable_fused`, vmamba.py:1448), and the logits are compared with the CPU oracle on the model's own
state dict: max-rel error <= 1e-4 in fp32 and <= 2e-2 under bf16 autocast (the reference's mixed-precision
recipe, vmamba.py:2384).  The tests skip where no checkout was staged.
"""
import os
import sys
import zlib

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import ss2d_oracle as O  # noqa: E402
from oracle import stage_ref  # noqa: E402

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not stage_ref.staged("vmamba.py"),
                                                   reason="reference files not staged (python oracle/stage_ref.py)")]

TOL_F32, TOL_BF16 = 1e-4, 2e-2


@pytest.fixture(scope="module")
def vb():
    assert torch.cuda.is_available()
    import vmamba_b200
    return vmamba_b200


@pytest.fixture(scope="module")
def ref():
    return stage_ref.load("vmamba.py", "vmamba_reference_gpu")


def _model(ref, dims, depths, hw, ssm_ratio=1.0, seed=0):
    torch.manual_seed(seed)
    cfg = dict(depths=depths, dims=dims, drop_path_rate=0.1, patch_size=4, in_chans=3, num_classes=10,
               ssm_d_state=1, ssm_ratio=ssm_ratio, ssm_dt_rank="auto", ssm_act_layer="silu", ssm_conv=3,
               ssm_conv_bias=False, ssm_drop_rate=0.0, ssm_init="v0", forward_type="v05_noz", mlp_ratio=4.0,
               mlp_act_layer="gelu", mlp_drop_rate=0.0, gmlp=False, patch_norm=True, norm_layer="ln2d",
               downsample_version="v3", patchembed_version="v2", use_checkpoint=False, posembed=False,
               imgsize=hw[0])
    m = ref.VSSM(**cfg).eval()
    g = torch.Generator().manual_seed(seed + 5)
    with torch.no_grad():
        for name, p in m.named_parameters():        # random init leaves LayerNorms at (1, 0) and biases at 0
            if p.ndim == 1 and ("norm" in name or name.endswith(".bias")):
                p.add_(0.1 * torch.randn(p.shape, generator=g))
    img = torch.randn((2, 3) + tuple(hw), generator=g)
    return m, img


def _oracle_logits(m, img):
    from oracle import backbone_oracle as BO
    sd = {k: v.detach().float().cpu().numpy() for k, v in m.state_dict().items()}
    return BO.vssm_logits(img.numpy(), sd)


@pytest.mark.parametrize("dims,depths,hw,ratio", [(32, [1, 1, 2, 1], (64, 64), 1.0), (96, [1, 1, 1, 1], (224, 224), 1.0),
                                                  (16, [1, 1, 2, 1], (96, 64), 2.0)])
def test_reference_vssm_on_library_operators(vb, ref, dims, depths, hw, ratio):
    """install(): every SS2D of the reference runs cross_scan_fn / selective_scan_fn / cross_merge_fn of this library;
    then enable_fused(): every supported SS2D core runs `ss2d_core_fwd`."""
    m, img = _model(ref, dims, depths, hw, ratio)
    want = _oracle_logits(m, img)
    m = m.cuda()
    x = img.cuda()
    old = torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32
    torch.backends.cudnn.allow_tf32 = torch.backends.cuda.matmul.allow_tf32 = False
    vb.install(ref)
    try:
        from vmamba_b200 import _lib
        n0 = _lib.launch_count()
        with torch.no_grad():
            got = m(x)
        assert _lib.launch_count() > n0, "the reference's forward did not reach the CUDA library"
        assert O.max_rel_err(got.float().cpu().numpy(), want) <= TOL_F32
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            got16 = m(x)
        assert O.max_rel_err(got16.float().cpu().numpy(), want) <= TOL_BF16

        n = vb.enable_fused(m)
        assert n == sum(depths), f"{n} of {sum(depths)} SS2D modules took the fused core"
        with torch.no_grad():
            fused = m(x)
        assert O.max_rel_err(fused.float().cpu().numpy(), want) <= TOL_F32
        assert np.array_equal(fused.argmax(1).cpu().numpy(), want.argmax(1))
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            fused16 = m(x)
        assert O.max_rel_err(fused16.float().cpu().numpy(), want) <= TOL_BF16
        # a gradient asked for through a fused module takes the differentiable operators, not the fused call
        xg = x.clone().requires_grad_(True)
        m(xg).sum().backward()
        assert xg.grad is not None and torch.isfinite(xg.grad).all() and xg.grad.abs().max() > 0
        vb.disable_fused(m)
        xg2 = x.clone().requires_grad_(True)
        m(xg2).sum().backward()
        assert O.max_rel_err(xg.grad.cpu().numpy(), xg2.grad.cpu().numpy()) <= 1e-5
    finally:
        vb.disable_fused(m)
        vb.uninstall(ref)
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = old


def test_accelerate_hands_back_an_equivalent_inference_module(vb, ref):
    """accelerate(): a reference VSSM / Backbone_VSSM -> this library's backbone on the module's own weights; logits and
    feature maps against the CPU oracle, a family the backbone does not reproduce is refused."""
    m, img = _model(ref, 32, [1, 1, 2, 1], (64, 64), 1.0)
    want = _oracle_logits(m, img)
    m = m.cuda()
    fast = vb.accelerate(m)
    assert isinstance(fast, torch.nn.Module) and not fast.training
    got = fast(img.cuda())
    assert got.shape == want.shape and O.max_rel_err(got.float().cpu().numpy(), want) <= TOL_BF16
    old = torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32
    torch.backends.cudnn.allow_tf32 = torch.backends.cuda.matmul.allow_tf32 = False      # fp32 means fp32 in the library calls too
    try:
        _accelerate_fp32_checks(vb, ref, m, img, want)
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = old


def _accelerate_fp32_checks(vb, ref, m, img, want):
    fast = vb.accelerate(m)
    fast32 = vb.accelerate(m, dtype=torch.float32)
    assert O.max_rel_err(fast32(img.cuda()).float().cpu().numpy(), want) <= TOL_F32
    assert m.training is False and not hasattr(ref, "__vmamba_b200_saved__")      # the module is left as it was
    with pytest.raises(RuntimeError):
        fast.train()
    # the dense-prediction backbone: four LayerNorm'ed maps
    torch.manual_seed(1)
    bb = ref.Backbone_VSSM(out_indices=(0, 1, 2, 3), pretrained=None, depths=[1, 1, 2, 1], dims=32, drop_path_rate=0.0, patch_size=4,
                           in_chans=3, num_classes=10, ssm_d_state=1, ssm_ratio=1.0, ssm_dt_rank="auto", ssm_act_layer="silu",
                           ssm_conv=3, ssm_conv_bias=False, ssm_drop_rate=0.0, ssm_init="v0", forward_type="v05_noz",
                           mlp_ratio=4.0, mlp_act_layer="gelu", mlp_drop_rate=0.0, gmlp=False, patch_norm=True, norm_layer="ln2d",
                           downsample_version="v3", patchembed_version="v2", use_checkpoint=False, posembed=False,
                           imgsize=64).cuda().eval()
    fb = vb.accelerate(bb, dtype=torch.float32)
    vb.install(ref)
    try:
        with torch.no_grad():
            maps = bb(img.cuda())
    finally:
        vb.uninstall(ref)
    outs = fb(img.cuda())
    assert len(outs) == len(maps) == 4
    for a_, b_ in zip(outs, maps):
        assert a_.shape == b_.shape and O.max_rel_err(a_.float().cpu().numpy(), b_.float().cpu().numpy()) <= 2e-4
    # a block with a z branch (forward_type v05) is another family
    cfg = dict(depths=[1, 1, 1, 1], dims=16, drop_path_rate=0.0, patch_size=4, in_chans=3, num_classes=10, ssm_d_state=1,
               ssm_ratio=1.0, ssm_dt_rank="auto", ssm_act_layer="silu", ssm_conv=3, ssm_conv_bias=False, ssm_drop_rate=0.0,
               ssm_init="v0", forward_type="v05", mlp_ratio=4.0, mlp_act_layer="gelu", mlp_drop_rate=0.0, gmlp=False,
               patch_norm=True, norm_layer="ln2d", downsample_version="v3", patchembed_version="v2", use_checkpoint=False,
               posembed=False, imgsize=64)
    with pytest.raises(NotImplementedError):
        vb.accelerate(ref.VSSM(**cfg).cuda().eval())


@pytest.mark.skipif(not stage_ref.staged("csms6s.py"), reason="csms6s.py not staged")
def test_reference_csms6s_on_extension_stand_in(vb):
    """The reference's own csms6s.py, imported unchanged after `preseed_extension_module()`: its SelectiveScanCuda
    calls `selective_scan_cuda_oflex.fwd / bwd` (csms6s.py:9-14, 81, 97-99), which are this library's kernels."""
    saved = {k: sys.modules.pop(k, None) for k in ("selective_scan_cuda_oflex", "csms6s_reference_gpu")}
    try:
        vb.preseed_extension_module()
        cs = stage_ref.load("csms6s.py", "csms6s_reference_gpu")
        assert cs.WITH_SELECTIVESCAN_OFLEX
        rng = np.random.default_rng(3)
        Bt, K, D, N, L = 2, 4, 24, 1, 200
        u = rng.standard_normal((Bt, K * D, L), dtype=np.float32)
        delta = rng.standard_normal((Bt, K * D, L), dtype=np.float32)
        A = -np.exp(0.3 * rng.standard_normal((K * D, N), dtype=np.float32))
        Bm = rng.standard_normal((Bt, K, N, L), dtype=np.float32)
        Cm = rng.standard_normal((Bt, K, N, L), dtype=np.float32)
        Dp = rng.standard_normal(K * D).astype(np.float32)
        bias = (0.5 * rng.random(K * D)).astype(np.float32)
        want = O.selective_scan(u, delta, A, Bm, Cm, Dp, bias, True)
        t = lambda a: torch.from_numpy(a).cuda().requires_grad_(True)
        tu, td, tA, tB, tC, tD, tb = map(t, (u, delta, A, Bm, Cm, Dp, bias))
        from vmamba_b200 import _lib
        n0 = _lib.launch_count()
        out = cs.selective_scan_fn(tu, td, tA, tB, tC, tD, tb, True, True, backend="oflex")
        assert _lib.launch_count() > n0
        assert O.max_rel_err(out.detach().cpu().numpy(), want) <= TOL_F32
        out.sum().backward()
        # gradients against autograd through the reference's own pure-torch recurrence on the same inputs
        tu2, td2, tA2, tB2, tC2, tD2, tb2 = map(t, (u, delta, A, Bm, Cm, Dp, bias))
        cs.selective_scan_torch(tu2, td2, tA2, tB2, tC2, tD2, tb2, True, True).sum().backward()
        for a_, b_ in ((tu, tu2), (td, td2), (tA, tA2), (tB, tB2), (tC, tC2), (tD, tD2), (tb, tb2)):
            assert O.max_rel_err(a_.grad.cpu().numpy(), b_.grad.cpu().numpy()) <= 2e-4
    finally:
        for k, v in saved.items():
            sys.modules.pop(k, None)
            if v is not None:
                sys.modules[k] = v


def test_top1_like_for_like_against_reference_bf16(vb, ref):
    """Top-1 agreement measured like for like: this library's bf16 backbone against the reference's own pure-torch
    path under bf16 autocast on the same GPU (CrossScan / CrossMerge torch Functions and `selective_scan_torch`),
    on synthetic images.  Random-init logits are nearly flat, so near-ties flip on rounding alone: the assertion
    is on the images whose reference margin exceeds the measured logit noise; the raw figure is printed."""
    from vmamba_b200.backbone import VSSMInfer
    m, _ = _model(ref, 48, [1, 1, 2, 1], (64, 64), 1.0, seed=3)
    m = m.cuda()
    orig_scan, orig_merge = ref.cross_scan_fn, ref.cross_merge_fn
    ref.cross_scan_fn = lambda *a, **k: orig_scan(*a, **{**k, "force_torch": True})
    ref.cross_merge_fn = lambda *a, **k: orig_merge(*a, **{**k, "force_torch": True})
    try:
        g = torch.Generator().manual_seed(11)
        img = torch.randn((256, 3, 64, 64), generator=g).cuda()
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            want16 = torch.cat([m(img[i:i + 64]) for i in range(0, 256, 64)]).float()
        with torch.no_grad():
            want32 = torch.cat([m(img[i:i + 64]) for i in range(0, 256, 64)]).float()
    finally:
        ref.cross_scan_fn, ref.cross_merge_fn = orig_scan, orig_merge
    sd = {k: v.detach().float().cpu().numpy() for k, v in m.state_dict().items()}
    lib16 = VSSMInfer.from_state_dict(sd, dtype=torch.bfloat16)(img.to(torch.bfloat16)).float()
    noise = (want16 - want32).abs().max().item()                 # what bf16 does to the reference itself
    top2 = want16.topk(2, dim=1).values
    clear = (top2[:, 0] - top2[:, 1]) > 4 * noise
    agree = lib16.argmax(1) == want16.argmax(1)
    print(f"top-1 agreement library bf16 vs reference bf16: {agree.float().mean().item():.4f} raw, "
          f"{agree[clear].float().mean().item():.4f} on {int(clear.sum())} images with a clear margin; "
          f"reference bf16-vs-fp32 logit noise {noise:.3e}")
    assert (lib16 - want16).abs().max().item() <= 4 * noise + 1e-3
    assert int(clear.sum()) > 0 and bool(agree[clear].all())


# ------------------------------------------------------------------------------------------------
# every forward type of the reference's SS2D that runs in the reference itself, on this library
# ------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def tree():
    """The full `classification/models/vmamba.py` with its own `csm_triton.py` and `csms6s.py` (no compiled
    extension importable: its selective scan is the reference's torch recurrence)."""
    if not stage_ref.staged("tree_vmamba.py"):
        pytest.skip("classification/models/vmamba.py not staged")
    names = ("csm_triton", "csms6s", "selective_scan_cuda_oflex", "selective_scan_cuda_core", "selective_scan_cuda")
    saved = {k: sys.modules.pop(k, None) for k in names}
    try:
        mod = stage_ref.load("tree_vmamba.py", "vmamba_tree_reference_gpu")
        yield mod, sys.modules["csm_triton"], sys.modules["csms6s"]
    finally:
        for k in names:
            sys.modules.pop(k, None)
            if saved[k] is not None:
                sys.modules[k] = saved[k]


class _torch_path:
    """The reference's own eager path: its torch CrossScanF / CrossMergeF (csm_triton.py:182-273) and
    `selective_scan_torch` (csms6s.py:30-70), whatever backend the module asks for."""

    def __init__(self, tree):
        self.mod, self.csm, self.s6 = tree

    def __enter__(self):
        mod, csm, s6 = self.mod, self.csm, self.s6
        self.saved = mod.cross_scan_fn, mod.cross_merge_fn, mod.selective_scan_fn

        def scan(x, in_channel_first=True, out_channel_first=True, one_by_one=False, scans=0, force_torch=False):
            return csm.CrossScanF.apply(x, in_channel_first, out_channel_first, one_by_one, scans)

        def merge(y, in_channel_first=True, out_channel_first=True, one_by_one=False, scans=0, force_torch=False):
            return csm.CrossMergeF.apply(y, in_channel_first, out_channel_first, one_by_one, scans)

        eager = s6.selective_scan_fn        # bound now: for the one-file distribution `s6` is `mod` itself
        mod.cross_scan_fn, mod.cross_merge_fn = scan, merge
        mod.selective_scan_fn = lambda *a, **k: eager(*a, **{**k, "backend": "torch"})
        return self

    def __exit__(self, *exc):
        self.mod.cross_scan_fn, self.mod.cross_merge_fn, self.mod.selective_scan_fn = self.saved


FORWARD_TYPES = [
    # forward_type, d_state, channel_first, (H, W)
    ("v0", 16, False, (7, 9)), ("v0seq", 16, False, (7, 9)), ("v0", 1, False, (14, 14)),
    ("v01", 4, False, (7, 9)), ("v02", 1, False, (7, 9)), ("v03", 2, True, (7, 9)), ("v04", 1, False, (9, 7)),
    ("v05", 1, True, (14, 14)), ("v05_noz_oact", 1, True, (7, 9)), ("v05_nozact", 16, False, (7, 9)), ("v3", 1, True, (7, 9)),
    ("v051d", 1, True, (7, 9)), ("v052d", 1, False, (7, 9)),
    ("v052d3", 1, True, (8, 8)),        # the debug route set: only the one-file distribution has it (vmamba.py:62-68)
    ("v052dc", 1, True, (7, 9)), ("v052dc", 4, True, (14, 14)),
    ("v05_onsoftmax", 1, True, (7, 9)), ("v05_ondwconv3", 1, True, (7, 9)),
]


@pytest.mark.parametrize("ft,N,cf,hw", FORWARD_TYPES)
def test_reference_ss2d_forward_types_on_library(vb, tree, ref, ft, N, cf, hw):
    """One SS2D module of the reference per forward type (vmamba.py:425-445: v0, v0seq, v01-v05 and their
    postfixes, the one-direction / two-direction / debug route sets, the cascade row-then-column mode, v3), built by
    the reference and run unchanged with `install()`: output and gradients against the same module on the
    reference's eager path."""
    if ft == "v052d3":
        tree = (ref, ref, ref)
    mod = tree[0]
    torch.manual_seed(zlib.crc32(ft.encode()) % 1000)
    d_model = 24
    m = mod.SS2D(d_model=d_model, d_state=N, ssm_ratio=2.0, dt_rank="auto", d_conv=3, conv_bias=False,
                 forward_type=ft, channel_first=cf).cuda().eval()
    shape = (2, d_model) + hw if cf else (2,) + hw + (d_model,)
    x = torch.randn(shape, device="cuda")
    old = torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32
    torch.backends.cudnn.allow_tf32 = torch.backends.cuda.matmul.allow_tf32 = False
    params = [p for p in m.parameters() if p.requires_grad]
    try:
        with _torch_path(tree):
            xr = x.clone().requires_grad_(True)
            want = m(xr)
            gout = torch.randn_like(want)
            want_g = torch.autograd.grad(want, [xr] + params, gout, allow_unused=True)
        vb.install(mod)
        try:
            from vmamba_b200 import _lib
            n0 = _lib.launch_count()
            xg = x.clone().requires_grad_(True)
            got = m(xg)
            assert _lib.launch_count() > n0, "the module's forward did not reach the CUDA library"
            got_g = torch.autograd.grad(got, [xg] + params, gout, allow_unused=True)
            with torch.no_grad():
                plain = m(x)
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                got16 = m(x)
        finally:
            vb.uninstall(mod)
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = old
    w = want.detach().cpu().numpy()
    assert O.max_rel_err(got.detach().cpu().numpy(), w) <= TOL_F32
    assert O.max_rel_err(plain.cpu().numpy(), w) <= TOL_F32
    assert O.max_rel_err(got16.float().cpu().numpy(), w) <= 3e-2
    for a, b in zip(got_g, want_g):
        assert (a is None) == (b is None)
        if a is not None:
            assert O.max_rel_err(a.cpu().numpy(), b.cpu().numpy()) <= 5e-4


def test_reference_xv_forward_types_raise_in_the_reference(tree):
    """The `xv*` family hands 4-d B / C maps to `cross_scan_fn(..., one_by_one=True)` (vmamba.py:871-872), and both of
    the reference's Functions unpack five dimensions there (csm_triton.py:186, 406): the family does not run in
    the reference, so there is nothing to be a drop-in for."""
    mod = tree[0]
    m = mod.SS2D(d_model=16, d_state=1, ssm_ratio=2.0, dt_rank="auto", d_conv=3, conv_bias=False,
                 forward_type="xv1a", channel_first=True).cuda().eval()
    with pytest.raises(ValueError), torch.no_grad():
        m(torch.randn(2, 16, 6, 6, device="cuda"))
