"""Generate the golden fixtures in this folder from the UNMODIFIED reference.

Run where a checkout of MzeroMiko/VMamba is available:

    python tests/golden/make_golden.py [--ref /path/to/VMamba]

The reference's one-file distribution (`vmamba.py` at its repository root) is imported
on CPU.  Its two third-party imports that are not needed for inference (`timm`,
`fvcore`) are replaced by minimal stand-ins when they are not installed; with no CUDA
extension importable the reference's `selective_scan_fn` takes its pure-torch path
(`selective_scan_torch`) and `cross_scan_fn` / `cross_merge_fn` their torch Functions.
Nothing of the reference is copied: only inputs and the outputs it computed are stored.
The fixtures are what pins the CPU oracle (tests/test_oracle_golden.py) and, through it,
the CUDA kernels.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _install_stubs():
    """Stand-ins for timm / fvcore symbols that vmamba.py imports at module import."""
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

            def forward(self, x):  # inference: identity
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


def load_reference(ref_root: str):
    _install_stubs()
    path = os.path.join(ref_root, "vmamba.py")
    spec = importlib.util.spec_from_file_location("vmamba_reference", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["vmamba_reference"] = mod
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        spec.loader.exec_module(mod)
    return mod


def npf(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def digest(a: np.ndarray, stride: int = 997) -> dict:
    """Size-independent fingerprint of a large array: sums and a strided sample."""
    f = np.asarray(a, dtype=np.float32).reshape(-1)
    return dict(sum=np.float64(f.astype(np.float64).sum()),
                abssum=np.float64(np.abs(f).astype(np.float64).sum()),
                sample=f[::stride].copy(), stride=np.int64(stride), size=np.int64(f.size))


def config0_inputs(seed: int = 0, Bt=2, D=96, H=56, W=56, N=1):
    """The seeded single-op workload: draws, in this fixed order, x, raw delta, dt,
    Bs, Cs from one torch.Generator (value distributions of mamba_init)."""
    import math
    g = torch.Generator().manual_seed(seed)
    K, L = 4, H * W
    x = torch.randn((Bt, D, H, W), generator=g)
    delta = torch.randn((Bt, K * D, L), generator=g)
    dt = torch.exp(torch.rand(K * D, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3)).clamp(min=1e-4)
    delta_bias = dt + torch.log(-torch.expm1(-dt))
    A = -torch.exp(torch.log(torch.arange(1, N + 1, dtype=torch.float32).view(1, -1).repeat(K * D, 1)))
    Bs = torch.randn((Bt, K, N, L), generator=g)
    Cs = torch.randn((Bt, K, N, L), generator=g)
    Dp = torch.ones(K * D)
    return dict(x=x, delta=delta, A=A, Bs=Bs, Cs=Cs, D=Dp, delta_bias=delta_bias)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("VMAMBA_REFERENCE"), required="VMAMBA_REFERENCE" not in os.environ,
                    help="checkout of MzeroMiko/VMamba (or set VMAMBA_REFERENCE)")
    args = ap.parse_args()
    ref = load_reference(args.ref)
    torch.set_grad_enabled(False)

    # ---- 1. CrossScan / CrossMerge, all four scan modes, H != W -------------------
    g = torch.Generator().manual_seed(11)
    out = {}
    x = torch.randn((2, 3, 5, 7), generator=g)
    ys = torch.randn((2, 4, 3, 5, 7), generator=g)
    out["x"], out["ys"] = npf(x), npf(ys)
    for s in range(4):
        out[f"scan_s{s}"] = npf(ref.cross_scan_fn(x, True, True, False, s, True))
        out[f"merge_s{s}"] = npf(ref.cross_merge_fn(ys, True, True, False, s, True))
    # the printed known-answer case of the reference's checks: arange(16) as a 4x4 map
    xa = torch.arange(16, dtype=torch.float32).view(1, 1, 4, 4)
    out["arange_scan_s0"] = npf(ref.cross_scan_fn(xa, True, True, False, 0, True))
    out["arange_merge_s0"] = npf(ref.cross_merge_fn(out_t := ref.cross_scan_fn(xa, True, True, False, 0, True).view(1, 4, 1, 4, 4),
                                                    True, True, False, 0, True))
    np.savez_compressed(os.path.join(HERE, "csm_small.npz"), **out)

    # ---- 1b. layout flags (channel-last in / out) and one_by_one, through the reference's torch Functions ----
    outl = {}
    gl = torch.Generator().manual_seed(21)
    for (H, W) in ((5, 7), (6, 6)):
        xcf = torch.randn((2, 3, H, W), generator=gl)
        ycf = torch.randn((2, 4, 3, H, W), generator=gl)
        tag = f"{H}x{W}"
        outl[f"{tag}_x"], outl[f"{tag}_ys"] = npf(xcf), npf(ycf)
        for scans in (0, 1, 2, 3):
            if scans == 3 and H != W:
                continue
            for icf in (True, False):
                for ocf in (True, False):
                    xin = xcf if icf else xcf.permute(0, 2, 3, 1).contiguous()
                    yin = ycf if ocf else ycf.permute(0, 3, 4, 1, 2).contiguous()
                    outl[f"{tag}_scan_s{scans}_i{int(icf)}_o{int(ocf)}"] = npf(ref.cross_scan_fn(xin, icf, ocf, False, scans, True))
                    outl[f"{tag}_merge_s{scans}_i{int(icf)}_o{int(ocf)}"] = npf(ref.cross_merge_fn(yin, icf, ocf, False, scans, True))
            outl[f"{tag}_scan1b1_s{scans}"] = npf(ref.cross_scan_fn(ycf, True, True, True, scans, True))
            outl[f"{tag}_merge1b1_s{scans}"] = npf(ref.cross_merge_fn(ycf, True, True, True, scans, True))
            # one_by_one with a channel-last side: the torch Functions define scans 0 and 1 (their branch for 2 indexes the
            # wrong axes, csm_triton.py:117-123); for scans 1 with channel-first in and channel-last out their flatten(2, 3)
            # merges C with H before the permute, which the reference's GPU kernel does not: that combination is left out
            if scans in (0, 1):
                ycl = ycf.permute(0, 3, 4, 1, 2).contiguous()
                for icf in (True, False):
                    for ocf in (True, False):
                        if icf and ocf:
                            continue
                        key = f"s{scans}_i{int(icf)}_o{int(ocf)}"
                        if not (scans == 1 and icf and not ocf):
                            outl[f"{tag}_scan1b1_{key}"] = npf(ref.cross_scan_fn(ycf if icf else ycl, icf, ocf, True, scans, True))
                        outl[f"{tag}_merge1b1_{key}"] = npf(ref.cross_merge_fn(ycf if ocf else ycl, icf, ocf, True, scans, True))
    np.savez_compressed(os.path.join(HERE, "csm_layouts_small.npz"), **outl)

    # ---- 2. selective scan, small cases over the flag space ---------------------
    cases = [
        dict(name="c0", Bt=2, K=4, Cd=3, N=1, L=37, D=True, bias=True, sp=True, dt="f32", oflex=True),
        dict(name="c1", Bt=1, K=4, Cd=2, N=4, L=70, D=False, bias=True, sp=True, dt="f32", oflex=True),
        dict(name="c2", Bt=2, K=4, Cd=2, N=2, L=33, D=True, bias=False, sp=False, dt="f32", oflex=True),
        dict(name="c3", Bt=2, K=4, Cd=4, N=1, L=64, D=True, bias=True, sp=True, dt="bf16", oflex=True),
        dict(name="c4", Bt=1, K=4, Cd=4, N=2, L=50, D=True, bias=True, sp=True, dt="bf16", oflex=False),
        dict(name="c5", Bt=2, K=1, Cd=5, N=3, L=41, D=True, bias=True, sp=True, dt="f32", oflex=True),
        dict(name="c6", Bt=1, K=2, Cd=3, N=16, L=300, D=True, bias=True, sp=True, dt="f16", oflex=True),
    ]
    out = {"names": np.array([c["name"] for c in cases])}
    for c in cases:
        g = torch.Generator().manual_seed(100 + len(c["name"]) + ord(c["name"][1]))
        tdt = dict(f32=torch.float32, bf16=torch.bfloat16, f16=torch.float16)[c["dt"]]
        KC = c["K"] * c["Cd"]
        u = torch.randn((c["Bt"], KC, c["L"]), generator=g).to(tdt)
        delta = (0.5 * torch.rand((c["Bt"], KC, c["L"]), generator=g)).to(tdt) if not c["sp"] \
            else torch.randn((c["Bt"], KC, c["L"]), generator=g).to(tdt)
        A = -0.5 * torch.rand((KC, c["N"]), generator=g) - 0.05
        Bm = torch.randn((c["Bt"], c["K"], c["N"], c["L"]), generator=g).to(tdt)
        Cm = torch.randn((c["Bt"], c["K"], c["N"], c["L"]), generator=g).to(tdt)
        Dp = torch.randn(KC, generator=g) if c["D"] else None
        bias = (0.5 * torch.rand(KC, generator=g) - 2.0) if c["bias"] else None
        y = ref.selective_scan_torch(u, delta, A, Bm, Cm, Dp, bias, c["sp"], c["oflex"])
        assert y.dtype == (torch.float32 if c["oflex"] else tdt)
        n = c["name"]
        out.update({f"{n}_u": npf(u), f"{n}_delta": npf(delta), f"{n}_A": npf(A), f"{n}_B": npf(Bm),
                    f"{n}_C": npf(Cm), f"{n}_y": npf(y), f"{n}_sp": np.bool_(c["sp"]),
                    f"{n}_oflex": np.bool_(c["oflex"]), f"{n}_dtype": np.array(c["dt"])})
        if Dp is not None:
            out[f"{n}_D"] = npf(Dp)
        if bias is not None:
            out[f"{n}_bias"] = npf(bias)
    np.savez_compressed(os.path.join(HERE, "selscan_small.npz"), **out)

    # ---- 2b. gradients of the same cases: autograd through the reference's selective_scan_torch,
    #          which is what SelectiveScanCuda.backward (csms6s.py:89-109) has to reproduce ----------
    outb = {"names": np.array([c["name"] for c in cases])}
    for c in cases:
        g = torch.Generator().manual_seed(100 + len(c["name"]) + ord(c["name"][1]))
        tdt = dict(f32=torch.float32, bf16=torch.bfloat16, f16=torch.float16)[c["dt"]]
        KC = c["K"] * c["Cd"]
        u = torch.randn((c["Bt"], KC, c["L"]), generator=g).to(tdt)
        delta = (0.5 * torch.rand((c["Bt"], KC, c["L"]), generator=g)).to(tdt) if not c["sp"] \
            else torch.randn((c["Bt"], KC, c["L"]), generator=g).to(tdt)
        A = -0.5 * torch.rand((KC, c["N"]), generator=g) - 0.05
        Bm = torch.randn((c["Bt"], c["K"], c["N"], c["L"]), generator=g).to(tdt)
        Cm = torch.randn((c["Bt"], c["K"], c["N"], c["L"]), generator=g).to(tdt)
        Dp = torch.randn(KC, generator=g) if c["D"] else None
        bias = (0.5 * torch.rand(KC, generator=g) - 2.0) if c["bias"] else None
        leaves = [t for t in (u, delta, A, Bm, Cm, Dp, bias) if t is not None]
        with torch.enable_grad():
            for t in leaves:
                t.requires_grad_(True)
            y = ref.selective_scan_torch(u, delta, A, Bm, Cm, Dp, bias, c["sp"], c["oflex"])
            dout = torch.randn(y.shape, generator=torch.Generator().manual_seed(7 + ord(c["name"][1]))).to(y.dtype)
            y.backward(dout)
        n = c["name"]
        outb[f"{n}_dout"] = npf(dout)
        for nm, t in (("du", u), ("ddelta", delta), ("dA", A), ("dB", Bm), ("dC", Cm), ("dD", Dp), ("dbias", bias)):
            if t is not None:
                assert t.grad is not None and t.grad.dtype == t.dtype
                outb[f"{n}_{nm}"] = npf(t.grad)
    np.savez_compressed(os.path.join(HERE, "selscan_bwd_small.npz"), **outb)

    # ---- 3. SS2D module (forward_type v05_noz, channel-first), core in/out -------
    out = {}
    for tag, kw, shape in (
        ("m0", dict(d_model=16, d_state=1, ssm_ratio=1.0), (2, 16, 9, 11)),
        ("m1", dict(d_model=8, d_state=2, ssm_ratio=2.0), (1, 8, 6, 5)),
    ):
        torch.manual_seed(7)
        m = ref.SS2D(dt_rank="auto", act_layer=torch.nn.SiLU, d_conv=3, conv_bias=False,
                     forward_type="v05_noz", channel_first=True, initialize="v0", **kw).eval()
        # give out_norm and x_proj non-trivial values
        torch.nn.init.normal_(m.out_norm.weight, 1.0, 0.2)
        torch.nn.init.normal_(m.out_norm.bias, 0.0, 0.2)
        torch.nn.init.normal_(m.Ds, 1.0, 0.3)
        torch.nn.init.normal_(m.A_logs, 0.0, 0.5)
        setattr(m, "__DEBUG__", True)
        g = torch.Generator().manual_seed(3)
        xin = torch.randn(shape, generator=g)
        captured = {}
        orig_core = m.forward_core

        def core(x, _orig=orig_core, _cap=captured):
            _cap["x"] = x.clone()
            y = _orig(x)
            _cap["y"] = y.clone()
            return y

        m.forward_core = core
        yout = m(xin)
        data = getattr(m, "__data__")
        out.update({f"{tag}_in": npf(xin), f"{tag}_out": npf(yout),
                    f"{tag}_core_x": npf(captured["x"]), f"{tag}_core_y": npf(captured["y"]),
                    f"{tag}_us": npf(data["us"]), f"{tag}_dts": npf(data["dts"]),
                    f"{tag}_Bs": npf(data["Bs"]), f"{tag}_Cs": npf(data["Cs"]),
                    f"{tag}_ys": npf(data["ys"]), f"{tag}_merged": npf(data["y"]),
                    f"{tag}_d_state": np.int64(m.d_state), f"{tag}_dt_rank": np.int64(m.dt_rank)})
        for k, v in m.state_dict().items():
            out[f"{tag}_sd_{k}"] = npf(v)
    np.savez_compressed(os.path.join(HERE, "ss2d_module_small.npz"), **out)

    # ---- 3b. gradients of the same modules' cores: autograd through the reference's forward_core
    #          (CrossScan -> x_proj -> dt_projs -> selective_scan_torch -> CrossMerge -> out_norm) -------
    outg = {}
    for tag, kw, shape in (
        ("m0", dict(d_model=16, d_state=1, ssm_ratio=1.0), (2, 16, 9, 11)),
        ("m1", dict(d_model=8, d_state=2, ssm_ratio=2.0), (1, 8, 6, 5)),
    ):
        torch.manual_seed(7)
        m = ref.SS2D(dt_rank="auto", act_layer=torch.nn.SiLU, d_conv=3, conv_bias=False,
                     forward_type="v05_noz", channel_first=True, initialize="v0", **kw).eval()
        torch.nn.init.normal_(m.out_norm.weight, 1.0, 0.2)
        torch.nn.init.normal_(m.out_norm.bias, 0.0, 0.2)
        torch.nn.init.normal_(m.Ds, 1.0, 0.3)
        torch.nn.init.normal_(m.A_logs, 0.0, 0.5)
        d_inner = m.out_norm.weight.numel()
        g = torch.Generator().manual_seed(13)
        xc = torch.randn((shape[0], d_inner, shape[2], shape[3]), generator=g)
        gy = torch.randn((shape[0], d_inner, shape[2], shape[3]), generator=g)
        with torch.enable_grad():
            xc.requires_grad_(True)
            y = m.forward_core(xc)
            assert y.shape == gy.shape
            y.backward(gy)
        outg.update({f"{tag}_core_x": npf(xc), f"{tag}_core_gy": npf(gy), f"{tag}_core_y": npf(y), f"{tag}_core_gx": npf(xc.grad)})
        for k, v in m.named_parameters():
            if v.grad is not None:
                outg[f"{tag}_grad_{k}"] = npf(v.grad)
        m.zero_grad()
    np.savez_compressed(os.path.join(HERE, "ss2d_core_grads_small.npz"), **outg)

    # ---- 4. the full-size single-op workload (2,96,56,56), digests only ----------
    inp = config0_inputs(0)
    xs = ref.cross_scan_fn(inp["x"], True, True, False, 0, True)
    ys = ref.selective_scan_torch(xs.view(2, 384, 3136), inp["delta"], inp["A"], inp["Bs"], inp["Cs"],
                                  inp["D"], inp["delta_bias"], True, True)
    y = ref.cross_merge_fn(ys.view(2, 4, 96, 56, 56), True, True, False, 0, True)
    yn = torch.nn.functional.layer_norm(y.view(2, 96, 3136).permute(0, 2, 1), (96,)).permute(0, 2, 1)
    out = {}
    for name, arr in (("x", inp["x"]), ("delta", inp["delta"]), ("delta_bias", inp["delta_bias"]),
                      ("Bs", inp["Bs"]), ("Cs", inp["Cs"]), ("ys", ys), ("merged", y), ("normed", yn)):
        for k, v in digest(npf(arr)).items():
            out[f"{name}_{k}"] = v
    np.savez_compressed(os.path.join(HERE, "config0_digest.npz"), **out)

    # ---- 5. a small VSSM backbone of the VMamba-T family --------------------------
    torch.manual_seed(0)
    cfg = dict(depths=[1, 1, 2, 1], dims=8, drop_path_rate=0.1, patch_size=4, in_chans=3, num_classes=10,
               ssm_d_state=1, ssm_ratio=1.0, ssm_dt_rank="auto", ssm_act_layer="silu", ssm_conv=3,
               ssm_conv_bias=False, ssm_drop_rate=0.0, ssm_init="v0", forward_type="v05_noz", mlp_ratio=4.0,
               mlp_act_layer="gelu", mlp_drop_rate=0.0, gmlp=False, patch_norm=True, norm_layer="ln2d",
               downsample_version="v3", patchembed_version="v2", use_checkpoint=False, posembed=False,
               imgsize=64)
    model = ref.VSSM(**cfg).eval()
    # random-init leaves LayerNorms at (1, 0) and head biases at 0: perturb so that every
    # parameter matters to the output
    g = torch.Generator().manual_seed(5)
    for name, p in model.named_parameters():
        if p.ndim == 1 and ("norm" in name or name.endswith(".bias")):
            p.add_(0.1 * torch.randn(p.shape, generator=g))
    img = torch.randn((2, 3, 64, 64), generator=g)
    logits = model(img)
    out = {"img": npf(img), "logits": npf(logits)}
    for k, v in model.state_dict().items():
        out[f"sd_{k}"] = npf(v)
    out["cfg_depths"] = np.array(cfg["depths"])
    out["cfg_dims"] = np.array([8, 16, 32, 64])
    np.savez_compressed(os.path.join(HERE, "vssm_small.npz"), **out)

    bb = ref.Backbone_VSSM(out_indices=(0, 1, 2, 3), pretrained=None, norm_layer="ln2d",
                           **{k: v for k, v in cfg.items() if k != "norm_layer"}).eval()
    sd = {k: v for k, v in model.state_dict().items() if not k.startswith("classifier.")}
    missing = bb.load_state_dict(sd, strict=False)
    outs = bb(img)
    fo = {f"feat{i}": npf(o) for i, o in enumerate(outs)}
    for i in range(4):
        fo[f"sd_outnorm{i}.weight"] = npf(getattr(bb, f"outnorm{i}").weight)
        fo[f"sd_outnorm{i}.bias"] = npf(getattr(bb, f"outnorm{i}").bias)
    np.savez_compressed(os.path.join(HERE, "vssm_small_features.npz"), **fo)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
