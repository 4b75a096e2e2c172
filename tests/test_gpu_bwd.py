"""Parity of the backward operators (selective-scan gradients, CrossScan / CrossMerge adjoints)
with the reference's autograd results (golden fixtures) and with the CPU oracle.  Needs a GPU.

Tolerances: max|got-ref| / max|ref| <= 1e-4 for fp32 tensors, <= 2e-2 for 16-bit storage;
the CrossScan / CrossMerge adjoints are data movement (and fp32 sums in the reference's order): bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import ss2d_oracle as O

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
TOL = {"f32": 1e-4, "bf16": 2e-2, "f16": 2e-2}
TD = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
NAMES = ("du", "ddelta", "dA", "dB", "dC", "dD", "dbias")


@pytest.fixture(scope="module")
def vb():
    import vmamba_b200
    assert torch.cuda.is_available()
    return vmamba_b200


def dev(a, dtype=torch.float32):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to("cuda").to(dtype)


def host(t):
    return None if t is None else t.detach().float().cpu().numpy()


def _autograd(vb, u, delta, A, B, C, D, bias, dout, sp, oflex, dt):
    """Gradients through the public operator (SelectiveScanCuda.apply under selective_scan_fn)."""
    td = TD[dt]
    ts = [dev(u, td), dev(delta, td), dev(A), dev(B, td), dev(C, td), dev(D), dev(bias)]
    for t in ts:
        if t is not None:
            t.requires_grad_(True)
    y = vb.selective_scan_fn(*ts, sp, oflex)
    assert y.dtype == (torch.float32 if oflex else td)
    y.backward(dev(dout, y.dtype))
    return [None if t is None else host(t.grad) for t in ts]


@pytest.mark.parametrize("n", ["c0", "c1", "c2", "c3", "c4", "c5", "c6"])
def test_selective_scan_bwd_golden(vb, n):
    """Against autograd through the unmodified reference's selective_scan_torch (stored fixture)."""
    g, gb = np.load(os.path.join(G, "selscan_small.npz")), np.load(os.path.join(G, "selscan_bwd_small.npz"))
    dt = str(g[f"{n}_dtype"])
    D = g[f"{n}_D"] if f"{n}_D" in g.files else None
    bias = g[f"{n}_bias"] if f"{n}_bias" in g.files else None
    got = _autograd(vb, g[f"{n}_u"], g[f"{n}_delta"], g[f"{n}_A"], g[f"{n}_B"], g[f"{n}_C"], D, bias, gb[f"{n}_dout"],
                    bool(g[f"{n}_sp"]), bool(g[f"{n}_oflex"]), dt)
    for name, x in zip(NAMES, got):
        key = f"{n}_{name}"
        if x is None:
            assert key not in gb.files
            continue
        err = O.max_rel_err(x, gb[key])
        assert err <= TOL[dt], (name, err)


def _random_case(Bt, K, Cd, N, L, seed, with_D=True, with_bias=True):
    rng = np.random.default_rng(seed)
    KC = K * Cd
    u = rng.standard_normal((Bt, KC, L), dtype=np.float32)
    delta = rng.standard_normal((Bt, KC, L), dtype=np.float32)
    A = -np.exp(0.3 * rng.standard_normal((KC, N), dtype=np.float32))
    B = rng.standard_normal((Bt, K, N, L), dtype=np.float32)
    C = rng.standard_normal((Bt, K, N, L), dtype=np.float32)
    D = rng.standard_normal(KC).astype(np.float32) if with_D else None
    bias = (rng.standard_normal(KC).astype(np.float32) - 3.0) if with_bias else None
    dout = rng.standard_normal((Bt, KC, L), dtype=np.float32)
    return u, delta, A, B, C, D, bias, dout


@pytest.mark.parametrize("Bt,K,Cd,N,L", [(2, 4, 5, 1, 3136), (1, 4, 12, 1, 784), (3, 4, 3, 1, 49), (2, 4, 2, 1, 1),
                                          (2, 4, 9, 1, 197), (1, 2, 3, 16, 330), (2, 1, 2, 64, 70), (1, 4, 2, 1, 16384)])
def test_selective_scan_bwd_fp32_vs_oracle(vb, Bt, K, Cd, N, L):
    u, delta, A, B, C, D, bias, dout = _random_case(Bt, K, Cd, N, L, seed=L + N)
    ref = O.selective_scan_bwd(u, delta, A, B, C, D, bias, dout, True, "f32")
    got = _autograd(vb, u, delta, A, B, C, D, bias, dout, True, True, "f32")
    for name, x, r in zip(NAMES, got, ref):
        err = O.max_rel_err(x, r)
        assert err <= TOL["f32"], (name, err)


@pytest.mark.parametrize("L,dt,oflex,opt", [(200, "f32", True, True), (392, "bf16", True, True), (136, "bf16", False, True),
                                            (196, "f16", True, False), (16, "f32", True, True)])
def test_selective_scan_bwd_many_rows(vb, L, dt, oflex, opt):
    """d_state 1 with enough rows (26 x 4 x 384 = 39 936) for the lanes-are-rows backward kernel: rows of one chunk and a
    ragged second one (L = 200), several chunks (392), a 14 x 14 map (196), a single tile; every gradient against
    the oracle, and against the warp-per-row kernel on the first two images (too few rows for this one)."""
    Bt, K, Cd = 26, 4, 384
    u, delta, A, B, C, D, bias, dout = _random_case(Bt, K, Cd, 1, L, seed=L, with_D=opt, with_bias=opt)
    if dt != "f32":
        rnd = lambda a: O._round_to(a, dt)
        u, delta, B, C = rnd(u), rnd(delta), rnd(B), rnd(C)
        if not oflex:
            dout = rnd(dout)
    from vmamba_b200 import _lib
    n0 = _lib.launch_count()
    got = _autograd(vb, u, delta, A, B, C, D, bias, dout, True, oflex, dt)
    assert _lib.launch_count() == n0 + 3          # forward, backward, fold
    ref = O.selective_scan_bwd(u, delta, A, B, C, D, bias, dout, True, dt)
    for name, x, r in zip(NAMES, got, ref):
        assert (x is None) == (r is None), name
        if x is not None:
            err = O.max_rel_err(x, r)
            assert err <= TOL[dt], (name, err)
    few = _autograd(vb, u[:2], delta[:2], A, B[:2], C[:2], D, bias, dout[:2], True, oflex, dt)
    for name, x, y in zip(NAMES[:2] + NAMES[3:5], got[:2] + got[3:5], few[:2] + few[3:5]):      # du, ddelta, dB, dC: per image
        assert O.max_rel_err(x[:2], y) <= (2e-5 if dt == "f32" else TOL[dt]), name


@pytest.mark.parametrize("N,L,dt,oflex,opt", [(16, 200, "f32", True, True), (16, 392, "bf16", True, True),
                                              (16, 136, "bf16", False, True), (8, 196, "f16", True, False),
                                              (4, 16, "f32", True, True), (16, 72, "f32", True, False),
                                              (16, 3136, "bf16", True, True)])
def test_selective_scan_bwd_many_rows_states(vb, N, L, dt, oflex, opt):
    """d_state 4 / 8 / 16 with enough rows (3 x 4 x 800 = 9 600) for the lanes-are-rows backward kernel of those state
    counts: every gradient against the oracle (short rows) and against the warp-per-row kernel run image by image (too
    few rows for this one); one case without D and delta_bias."""
    Bt, K, Cd = 3, 4, 800
    u, delta, A, B, C, D, bias, dout = _random_case(Bt, K, Cd, N, L, seed=L + N, with_D=opt, with_bias=opt)
    if dt != "f32":
        rnd = lambda a: O._round_to(a, dt)
        u, delta, B, C = rnd(u), rnd(delta), rnd(B), rnd(C)
        if not oflex:
            dout = rnd(dout)
    got = _autograd(vb, u, delta, A, B, C, D, bias, dout, True, oflex, dt)
    if L <= 400:                                   # the oracle takes minutes on the long rows
        ref = O.selective_scan_bwd(u, delta, A, B, C, D, bias, dout, True, dt)
        for name, x, r in zip(NAMES, got, ref):
            assert (x is None) == (r is None), name
            if x is not None:
                err = O.max_rel_err(x, r)
                assert err <= TOL[dt], (name, err)
    sums = [0.0, 0.0, 0.0]                          # dA, dD, dbias: sums over the images
    for i in range(Bt):
        s = slice(i, i + 1)
        few = _autograd(vb, u[s], delta[s], A, B[s], C[s], D, bias, dout[s], True, oflex, dt)
        for name, x, y in zip(NAMES[:2] + NAMES[3:5], got[:2] + got[3:5], few[:2] + few[3:5]):  # du, ddelta, dB, dC: per image
            assert O.max_rel_err(x[s], y) <= (2e-5 if dt == "f32" else TOL[dt]), (name, i)
        sums = [None if b is None else a + b for a, b in zip(sums, (few[2], few[5], few[6]))]
    for name, x, y in zip(("dA", "dD", "dbias"), (got[2], got[5], got[6]), sums):
        assert (x is None) == (y is None), name
        if x is not None:
            assert O.max_rel_err(x, y) <= (1e-4 if dt == "f32" else TOL[dt]), name


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("oflex", [True, False])
def test_selective_scan_bwd_16bit_vs_oracle(vb, dt, oflex):
    u, delta, A, B, C, D, bias, dout = _random_case(2, 4, 6, 1, 784, seed=11)
    rnd = lambda a: O._round_to(a, dt)
    u, delta, B, C = rnd(u), rnd(delta), rnd(B), rnd(C)
    if not oflex:
        dout = rnd(dout)
    ref = O.selective_scan_bwd(u, delta, A, B, C, D, bias, dout, True, dt)
    got = _autograd(vb, u, delta, A, B, C, D, bias, dout, True, oflex, dt)
    for name, x, r in zip(NAMES, got, ref):
        err = O.max_rel_err(x, r)
        assert err <= TOL[dt], (name, err)


def test_selective_scan_bwd_optional_args_strided_and_deterministic(vb):
    u, delta, A, B, C, _, _, dout = _random_case(2, 4, 3, 2, 160, seed=3, with_D=False, with_bias=False)
    ref = O.selective_scan_bwd(u, delta, A, B, C, None, None, dout, False, "f32")
    from vmamba_b200 import ops
    big_u = torch.zeros((2, 12, 2 * 160), device="cuda")
    big_u[:, :, 8:8 + 160] = dev(u)
    big_g = torch.zeros((2, 24, 160), device="cuda")
    big_g[:, ::2] = dev(dout)
    args = (big_u[:, :, 8:8 + 160], dev(delta), dev(A), dev(B), dev(C), None, None, big_g[:, ::2], False)
    got = ops.selective_scan_bwd(*args)
    assert got[5] is None and got[6] is None
    for name, x, r in zip(NAMES, got, ref):
        if r is not None:
            assert O.max_rel_err(host(x), r) <= TOL["f32"], name
    again = ops.selective_scan_bwd(*args)
    for a_, b_ in zip(got, again):
        if a_ is not None:
            assert torch.equal(a_, b_)


def test_selective_scan_bwd_rejects_bad_arguments(vb):
    from vmamba_b200 import ops
    u, delta, A, B, C, D, bias, dout = (dev(t) for t in _random_case(1, 4, 2, 1, 32, seed=1))
    with pytest.raises(RuntimeError):
        ops.selective_scan_bwd(u, delta, A, B, C, D, bias, dout[:, :, :16], True)
    with pytest.raises(RuntimeError):
        ops.selective_scan_bwd(u.cpu(), delta, A, B, C, D, bias, dout, True)


@pytest.mark.parametrize("scans", [0, 1, 2, 3])
@pytest.mark.parametrize("shape", [(2, 5, 7, 9), (1, 3, 14, 14)])
def test_cross_scan_merge_adjoints(vb, scans, shape):
    """CrossScan.backward is CrossMerge.forward and vice versa (csm_triton.py:207-225, 248-273)."""
    if scans == 3 and shape[2] != shape[3]:
        pytest.skip("rotations need square maps")
    rng = np.random.default_rng(scans)
    Bt, Cc, H, W = shape
    x = rng.standard_normal(shape, dtype=np.float32)
    gy = rng.standard_normal((Bt, 4, Cc, H * W), dtype=np.float32)
    xt = dev(x).requires_grad_(True)
    ys = vb.cross_scan_fn(xt, True, True, False, scans)
    ys.backward(dev(gy))
    assert np.array_equal(host(xt.grad).reshape(Bt, Cc, H * W), O.cross_merge(gy.reshape(Bt, 4, Cc, H, W), scans))
    yt = dev(gy.reshape(Bt, 4, Cc, H, W)).requires_grad_(True)
    gm = rng.standard_normal((Bt, Cc, H * W), dtype=np.float32)
    m = vb.cross_merge_fn(yt, True, True, False, scans)
    m.backward(dev(gm))
    assert np.array_equal(host(yt.grad).reshape(Bt, 4, Cc, H * W), O.cross_scan(gm.reshape(Bt, Cc, H, W), scans))


@pytest.mark.parametrize("tag", ["m0", "m1"])
def test_core_training_chain_vs_reference_grads(vb, tag):
    """Forward + backward of the whole SS2D core through this package's autograd Functions against
    autograd through the unmodified reference module's forward_core (stored fixture): the output,
    the input gradient and the gradient of every parameter."""
    from vmamba_b200 import fused
    gm = np.load(os.path.join(G, "ss2d_module_small.npz"))
    gg = np.load(os.path.join(G, "ss2d_core_grads_small.npz"))
    sd = {k[len(tag) + 4:]: gm[k] for k in gm.files if k.startswith(f"{tag}_sd_")}
    N, R = int(gm[f"{tag}_d_state"]), int(gm[f"{tag}_dt_rank"])
    names = ("x_proj.weight", "dt_projs.weight", "dt_projs_bias", "A_logs", "Ds", "out_norm.weight", "out_norm.bias")
    params = [dev(sd[n]).requires_grad_(True) for n in names]
    x = dev(gg[f"{tag}_core_x"]).requires_grad_(True)
    y = fused.ss2d_core_autograd(x, *params, d_state=N, dt_rank=R)
    assert O.max_rel_err(host(y), gg[f"{tag}_core_y"]) <= 1e-4
    y.backward(dev(gg[f"{tag}_core_gy"]))
    assert O.max_rel_err(host(x.grad), gg[f"{tag}_core_gx"]) <= 1e-4
    for n, p_ in zip(names, params):
        ref = gg[f"{tag}_grad_{n}"]
        err = O.max_rel_err(host(p_.grad).reshape(ref.shape), ref)
        assert err <= 1e-4, (n, err)


def test_extension_module_surface(vb):
    """fwd / bwd of the stand-in for the compiled extension, called as the reference calls them
    (csms6s.py:81, 97-99): same values as the operator and its autograd."""
    u, delta, A, B, C, D, bias, dout = (dev(t) for t in _random_case(2, 4, 3, 1, 200, seed=9))
    ext = vb.selective_scan_cuda_oflex
    out, x, *rest = ext.fwd(u, delta, A, B, C, D, bias, True, 1, True)
    assert torch.equal(out, vb.selective_scan_fwd(u, delta, A, B, C, D, bias, True, True))
    assert tuple(x.shape) == (2, 12, 2, 1)      # states in front of elements 0 and 128
    du, ddelta, dA, dB, dC, dD, dbias, *rest = ext.bwd(u, delta, A, B, C, D, bias, dout, x, True, 1)
    ref = O.selective_scan_bwd(*(host(t) for t in (u, delta, A, B, C, D, bias, dout)), True, "f32")
    for name, got, r in zip(NAMES, (du, ddelta, dA, dB, dC, dD, dbias), ref):
        assert O.max_rel_err(host(got), r) <= TOL["f32"], name


@pytest.mark.parametrize("ratio", [2, 3])
def test_shared_delta_rows_forward_and_backward(vb, ratio):
    """delta with dim / ratio rows, row r / ratio serving channel r (selective_scan_oflex.cpp:59, 176-183, 348-352).
    The reference's pure-torch path has no such mode, so the oracle is fed the expanded delta and bias and its
    per-channel gradients are summed over the rows that shared an input row."""
    from vmamba_b200 import ops
    Bt, K, Cd, N, L = 2, 2, 3 * ratio, 2, 150
    u, delta_full, A, B, C, D, bias_full, dout = _random_case(Bt, K, Cd, N, L, seed=40 + ratio)
    KC = K * Cd
    delta = delta_full[:, ::ratio].copy()
    bias = bias_full[::ratio].copy()
    d_exp, b_exp = np.repeat(delta, ratio, axis=1), np.repeat(bias, ratio)
    ref_y = O.selective_scan(u, d_exp, A, B, C, D, b_exp, True, True, "f32")
    y = ops.selective_scan_fwd(dev(u), dev(delta), dev(A), dev(B), dev(C), dev(D), dev(bias), True, True)
    assert O.max_rel_err(host(y), ref_y) <= TOL["f32"]
    ref = list(O.selective_scan_bwd(u, d_exp, A, B, C, D, b_exp, dout, True, "f32"))
    ref[1] = ref[1].reshape(Bt, KC // ratio, ratio, L).sum(2)
    ref[6] = ref[6].reshape(KC // ratio, ratio).sum(1)
    got = ops.selective_scan_bwd(dev(u), dev(delta), dev(A), dev(B), dev(C), dev(D), dev(bias), dev(dout), True)
    assert tuple(got[1].shape) == (Bt, KC // ratio, L) and tuple(got[6].shape) == (KC // ratio,)
    for name, x, r in zip(NAMES, got, ref):
        assert O.max_rel_err(host(x), r) <= TOL["f32"], name


@pytest.mark.parametrize("N,L", [(1, 3136), (1, 200), (3, 300), (1, 90)])
def test_backward_with_and_without_forward_checkpoints(vb, N, L):
    """The step states written by the forward call give the same gradients as recomputing them (to fp32 rounding: the
    forward kernel composes the recurrence in 256-element steps, the recomputation in 128-element steps), and the
    checkpoints are the oracle's states in front of every 128th element."""
    from vmamba_b200 import ops
    u, delta, A, B, C, D, bias, dout = _random_case(2, 2, 3, N, L, seed=L)
    args = [dev(t) for t in (u, delta, A, B, C, D, bias)]
    out, ck = ops.selective_scan_fwd(*args, True, True, return_checkpoints=True)
    assert torch.equal(out, ops.selective_scan_fwd(*args, True, True))
    g1 = ops.selective_scan_bwd(*args, dev(dout), True)
    g2 = ops.selective_scan_bwd(*args, dev(dout), True, checkpoints=ck)
    for a_, b_ in zip(g1, g2):
        assert O.max_rel_err(host(a_), host(b_)) <= 1e-5
    # states by the oracle's recurrence
    dl = O.softplus(delta + bias[None, :, None])
    Bx = np.repeat(B, 3, axis=1).reshape(2, 6, N, L)
    h = np.zeros((2, 6, N), np.float32)
    want = np.zeros((2, 6, (L + 127) // 128, N), np.float32)
    for i in range(L):
        if i % 128 == 0:
            want[:, :, i // 128] = h
        h = np.exp(dl[:, :, i, None] * A[None]) * h + (dl[:, :, i] * u[:, :, i])[:, :, None] * Bx[..., i]
    assert O.max_rel_err(host(ck), want) <= 1e-4
