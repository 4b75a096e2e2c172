"""Pins the CPU oracle (numpy and C statements) to outputs of the unmodified reference
stored under tests/golden/ (see tests/golden/make_golden.py).  CPU only."""
import os

import numpy as np
import pytest

from oracle import backbone_oracle as BO
from oracle import c_oracle as CO
from oracle import ss2d_oracle as O

G = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    return np.load(os.path.join(G, name))


@pytest.mark.parametrize("scans", [0, 1, 2, 3])
def test_cross_scan_merge_bit_exact(scans):
    g = load("csm_small.npz")
    for impl in (O, CO):
        assert np.array_equal(impl.cross_scan(g["x"], scans), g[f"scan_s{scans}"])
        assert np.array_equal(impl.cross_merge(g["ys"], scans), g[f"merge_s{scans}"])


def test_arange_known_answer():
    g = load("csm_small.npz")
    x = np.arange(16, dtype=np.float32).reshape(1, 1, 4, 4)
    xs = O.cross_scan(x, 0)
    assert np.array_equal(xs, g["arange_scan_s0"])
    # column-major route of a 4x4 arange starts 0,4,8,12,1,...
    assert xs[0, 1, 0, :5].tolist() == [0, 4, 8, 12, 1]
    assert np.array_equal(O.cross_merge(xs.reshape(1, 4, 1, 4, 4), 0), g["arange_merge_s0"])
    assert np.array_equal(O.cross_merge(xs.reshape(1, 4, 1, 4, 4), 0), 4 * x.reshape(1, 1, 16))


def test_cross_scan_merge_layout_flags_and_one_by_one():
    """Channel-last in / out and one_by_one against the reference's torch Functions (bit-exact data movement;
    the merge sums in the reference's order)."""
    g = load("csm_layouts_small.npz")
    for tag, (H, W) in (("5x7", (5, 7)), ("6x6", (6, 6))):
        x, ys = g[f"{tag}_x"], g[f"{tag}_ys"]
        for scans in (0, 1, 2, 3):
            if scans == 3 and H != W:
                continue
            for icf in (True, False):
                for ocf in (True, False):
                    xin = x if icf else np.ascontiguousarray(x.transpose(0, 2, 3, 1))
                    yin = ys if ocf else np.ascontiguousarray(ys.transpose(0, 3, 4, 1, 2))
                    key = f"s{scans}_i{int(icf)}_o{int(ocf)}"
                    assert np.array_equal(O.cross_scan_ex(xin, scans, icf, ocf), g[f"{tag}_scan_{key}"]), key
                    assert np.array_equal(O.cross_merge_ex(yin, scans, icf, ocf), g[f"{tag}_merge_{key}"]), key
            assert np.array_equal(O.cross_scan_ex(ys, scans, one_by_one=True), g[f"{tag}_scan1b1_s{scans}"]), scans
            assert np.array_equal(O.cross_merge_ex(ys, scans, one_by_one=True), g[f"{tag}_merge1b1_s{scans}"]), scans
            if scans > 1:
                continue
            ycl = np.ascontiguousarray(ys.transpose(0, 3, 4, 1, 2))     # one map per route, channel-last
            for icf, ocf in ((True, False), (False, True), (False, False)):
                key = f"s{scans}_i{int(icf)}_o{int(ocf)}"
                if f"{tag}_scan1b1_{key}" in g.files:       # scans 1, i1_o0: the torch path's C*H merge, not stored
                    got = O.cross_scan_ex(ys if icf else ycl, scans, icf, ocf, True)
                    assert np.array_equal(got, g[f"{tag}_scan1b1_{key}"]), key
                got = O.cross_merge_ex(ys if ocf else ycl, scans, icf, ocf, True)
                assert np.array_equal(got, g[f"{tag}_merge1b1_{key}"]), key


def _case(g, n):
    kw = dict(D=g[f"{n}_D"] if f"{n}_D" in g.files else None,
              delta_bias=g[f"{n}_bias"] if f"{n}_bias" in g.files else None,
              delta_softplus=bool(g[f"{n}_sp"]))
    return (g[f"{n}_u"], g[f"{n}_delta"], g[f"{n}_A"], g[f"{n}_B"], g[f"{n}_C"]), kw


@pytest.mark.parametrize("n", ["c0", "c1", "c2", "c3", "c4", "c5", "c6"])
def test_selective_scan_vs_reference(n):
    g = load("selscan_small.npz")
    args, kw = _case(g, n)
    oflex, dt = bool(g[f"{n}_oflex"]), str(g[f"{n}_dtype"])
    y = O.selective_scan(*args, oflex=oflex, dtype_in=dt, **kw)
    assert O.max_rel_err(y, g[f"{n}_y"]) <= 2e-6
    yc = CO.selective_scan(*args, **kw)
    if not oflex:
        yc = O._round_to(yc, dt)
    # rounding to bf16 may flip one ulp of the storage type
    assert O.max_rel_err(yc, g[f"{n}_y"]) <= (2e-6 if oflex else 8e-3)


@pytest.mark.parametrize("n", ["c0", "c1", "c2", "c3", "c4", "c5", "c6"])
def test_selective_scan_bwd_vs_reference_autograd(n):
    """The oracle's gradient formulas against autograd through the reference's selective_scan_torch."""
    g, gb = load("selscan_small.npz"), load("selscan_bwd_small.npz")
    (u, delta, A, B, C), kw = _case(g, n)
    dt = str(g[f"{n}_dtype"])
    grads = O.selective_scan_bwd(u, delta, A, B, C, kw["D"], kw["delta_bias"], gb[f"{n}_dout"],
                                 delta_softplus=kw["delta_softplus"], dtype_in=dt)
    # 16-bit storage: the reference rounds its gradients to the storage type too; one ulp may flip
    tol = 1e-5 if dt == "f32" else (8e-3 if dt == "bf16" else 2e-3)
    for name, got in zip(("du", "ddelta", "dA", "dB", "dC", "dD", "dbias"), grads):
        key = f"{n}_{name}"
        if got is None:
            assert key not in gb.files, name
            continue
        t = 1e-5 if name in ("dA", "dD", "dbias") else tol
        assert O.max_rel_err(got, gb[key]) <= t, (name, O.max_rel_err(got, gb[key]))


@pytest.mark.parametrize("tag", ["m0", "m1"])
def test_ss2d_core_vs_reference_module(tag):
    g = load("ss2d_module_small.npz")
    sd = {k[len(tag) + 4:]: g[k] for k in g.files if k.startswith(f"{tag}_sd_")}
    N, R = int(g[f"{tag}_d_state"]), int(g[f"{tag}_dt_rank"])
    y, parts = O.ss2d_core(g[f"{tag}_core_x"], sd["x_proj.weight"], sd["dt_projs.weight"], sd["dt_projs_bias"],
                           sd["A_logs"], sd["Ds"], sd["out_norm.weight"], sd["out_norm.bias"],
                           d_state=N, dt_rank=R, return_parts=True)
    assert np.array_equal(parts["xs"].reshape(g[f"{tag}_us"].shape), g[f"{tag}_us"])
    assert O.max_rel_err(parts["dts"], g[f"{tag}_dts"]) <= 2e-6
    assert O.max_rel_err(parts["ys"].reshape(g[f"{tag}_ys"].shape), g[f"{tag}_ys"]) <= 5e-6
    assert O.max_rel_err(parts["merged"].reshape(g[f"{tag}_merged"].shape), g[f"{tag}_merged"]) <= 5e-6
    assert O.max_rel_err(y, g[f"{tag}_core_y"]) <= 1e-5
    yc = BO.ss2d_core_c(g[f"{tag}_core_x"], sd, "", N, R)
    assert O.max_rel_err(yc, g[f"{tag}_core_y"]) <= 1e-5
    # whole module: in_proj -> dwconv -> SiLU -> core -> out_proj
    import torch
    out = BO.ss2d_forward(torch.from_numpy(g[f"{tag}_in"]), sd, "").numpy()
    assert O.max_rel_err(out, g[f"{tag}_out"]) <= 1e-5


def test_config0_full_size_digest():
    """The (2,96,56,56) single-op workload, regenerated from its seed, through the C oracle."""
    import sys
    sys.path.insert(0, G)
    from make_golden import config0_inputs, digest
    g = load("config0_digest.npz")
    inp = {k: v.numpy() for k, v in config0_inputs(0).items()}
    for name, key in (("x", "x"), ("delta", "delta"), ("delta_bias", "delta_bias"), ("Bs", "Bs"), ("Cs", "Cs")):
        d = digest(inp[key])
        assert np.array_equal(d["sample"], g[f"{name}_sample"]), f"seeded input {name} differs"
    xs = CO.cross_scan(inp["x"], 0)
    ys = CO.selective_scan(xs.reshape(2, 384, 3136), inp["delta"], inp["A"], inp["Bs"], inp["Cs"], inp["D"],
                           inp["delta_bias"], True)
    merged = CO.cross_merge(ys.reshape(2, 4, 96, 56, 56), 0)
    normed = CO.layer_norm_cf(merged)
    for name, arr in (("ys", ys), ("merged", merged), ("normed", normed)):
        d = digest(arr)
        ref = g[f"{name}_sample"]
        assert np.max(np.abs(d["sample"] - ref)) <= 2e-5 * np.max(np.abs(ref)), name
        assert abs(d["abssum"] - float(g[f"{name}_abssum"])) <= 1e-5 * float(g[f"{name}_abssum"]), name


def test_backbone_vs_reference():
    g = load("vssm_small.npz")
    sd = {k[3:]: g[k] for k in g.files if k.startswith("sd_")}
    logits = BO.vssm_logits(g["img"], sd)
    assert O.max_rel_err(logits, g["logits"]) <= 2e-5
    assert np.array_equal(logits.argmax(1), g["logits"].argmax(1))
    f = load("vssm_small_features.npz")
    sd.update({k[3:]: f[k] for k in f.files if k.startswith("sd_")})
    feats = BO.backbone_features(g["img"], sd)
    for i, o in enumerate(feats):
        assert o.shape == f[f"feat{i}"].shape
        assert O.max_rel_err(o, f[f"feat{i}"]) <= 2e-5


def test_bf16_rounding_helper():
    import torch
    a = np.random.default_rng(0).standard_normal(4096).astype(np.float32) * 37.0
    ref = torch.from_numpy(a).to(torch.bfloat16).float().numpy()
    assert np.array_equal(O.round_bf16(a), ref)
