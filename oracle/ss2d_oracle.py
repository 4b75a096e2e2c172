"""CPU oracle for the SS2D core of VMamba -- TEST INFRASTRUCTURE, NOT A PRODUCT PATH.

This file restates, in plain numpy, the reference's pure-torch algorithm for the
SS2D hot path so that the CUDA kernels can be checked against it on machines where
the reference itself is not present.  Only tests, the smoke check and the
`cpu_baseline` / `--impl reference` legs of the benchmark may import it; the
package `vmamba_b200` never does.

Parity status: PINNED.  Every function here is compared (tests/test_oracle_golden.py)
against outputs of the unmodified reference (root `vmamba.py`, imported on CPU)
stored under tests/golden/ by tests/golden/make_golden.py.

Reference anchors (paths inside MzeroMiko/VMamba):
  cross_scan        vmamba.py:41-84    (cross_scan_fwd,  channel-first branch)
  cross_merge       vmamba.py:87-130   (cross_merge_fwd, channel-first branch)
  selective_scan    vmamba.py:791-834  (selective_scan_torch) == classification/models/csms6s.py:25-68
  layer_norm_cf     vmamba.py:1078-1093 (LayerNorm with channel_first=True)
  ss2d_core         vmamba.py:1504-1571 (SS2Dv2.forward_corev2, no_einsum/conv1d form)
  dt/A/D init       vmamba.py:1170-1237 (mamba_init)

Arrays are float32 numpy arrays.  bf16 is represented as float32 values that have
been rounded to the bf16 grid with `round_bf16` (numpy has no bf16 type).
"""
from __future__ import annotations

import math
import numpy as np

K_ROUTES = 4


# --------------------------------------------------------------------------- #
# dtype helpers
# --------------------------------------------------------------------------- #
def round_bf16(a: np.ndarray) -> np.ndarray:
    """Round float32 values to the nearest bfloat16 (ties to even), return float32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16) << 16
    out = r.astype(np.uint32).view(np.float32).reshape(a.shape).copy()
    nan = np.isnan(a)
    if nan.any():
        out[nan] = np.nan
    return out


def round_f16(a: np.ndarray) -> np.ndarray:
    return np.asarray(a, dtype=np.float32).astype(np.float16).astype(np.float32)


def _round_to(a: np.ndarray, dtype: str) -> np.ndarray:
    if dtype in ("f32", "fp32", "float32"):
        return np.asarray(a, dtype=np.float32)
    if dtype in ("bf16", "bfloat16"):
        return round_bf16(a)
    if dtype in ("f16", "fp16", "float16"):
        return round_f16(a)
    raise ValueError(f"unknown dtype tag {dtype!r}")


# --------------------------------------------------------------------------- #
# a1: CrossScan  (vmamba.py:41-84)
# --------------------------------------------------------------------------- #
def cross_scan(x: np.ndarray, scans: int = 0) -> np.ndarray:
    """(B, C, H, W) -> (B, 4, C, H*W).

    scans=0: route 0 row-major, route 1 column-major, routes 2/3 the same reversed
             (vmamba.py:45-49).
    scans=1: the row-major sequence repeated four times (vmamba.py:50-51).
    scans=2: row-major twice, then its reversal twice (vmamba.py:52-54).
    scans=3: row-major sequences of the map rotated by 0/90/180/270 degrees
             (vmamba.py:55-60).
    """
    B, C, H, W = x.shape
    L = H * W
    y = np.empty((B, 4, C, L), dtype=x.dtype)
    if scans == 0:
        y[:, 0] = x.reshape(B, C, L)
        y[:, 1] = x.transpose(0, 1, 3, 2).reshape(B, C, L)
        y[:, 2] = y[:, 0, :, ::-1]
        y[:, 3] = y[:, 1, :, ::-1]
    elif scans == 1:
        y[:] = x.reshape(B, 1, C, L)
    elif scans == 2:
        y[:, 0] = x.reshape(B, C, L)
        y[:, 1] = y[:, 0]
        y[:, 2] = y[:, 0, :, ::-1]
        y[:, 3] = y[:, 2]
    elif scans == 3:
        for k in range(4):
            y[:, k] = np.rot90(x, k, axes=(2, 3)).reshape(B, C, L)
    else:
        raise ValueError("scans must be 0, 1, 2 or 3")
    return y


# --------------------------------------------------------------------------- #
# a7: CrossMerge  (vmamba.py:87-130)
# --------------------------------------------------------------------------- #
def cross_merge(ys: np.ndarray, scans: int = 0) -> np.ndarray:
    """(B, 4, C, H, W) -> (B, C, H*W); the adjoint of cross_scan.

    The summation ORDER follows the reference so that fp32 results are bit-identical:
    scans=0: (y0 + flip(y2)) + transpose((y1 + flip(y3)))  (vmamba.py:92-94)
    scans=1: sum over the route axis, routes added in order 0,1,2,3 (vmamba.py:95-96)
    scans=2: (y0+flip(y2)) + (y1+flip(y3))                 (vmamba.py:97-99)
    scans=3: y0 + rot-90(y1) + rot-180(y2) + rot-270(y3)   (vmamba.py:100-105)
    """
    B, K, C, H, W = ys.shape
    assert K == 4
    L = H * W
    y = ys.reshape(B, K, C, L)
    if scans == 0:
        t = y[:, 0:2] + y[:, 2:4, :, ::-1]
        col = t[:, 1].reshape(B, C, W, H).transpose(0, 1, 3, 2).reshape(B, C, L)
        return t[:, 0] + col
    if scans == 1:
        return ((y[:, 0] + y[:, 1]) + y[:, 2]) + y[:, 3]
    if scans == 2:
        t = y[:, 0:2] + y[:, 2:4, :, ::-1]
        return t[:, 0] + t[:, 1]
    if scans == 3:
        oy = y[:, 0].copy()
        oy = oy + np.rot90(y[:, 1].reshape(B, C, W, H), -1, axes=(2, 3)).reshape(B, C, L)
        oy = oy + np.rot90(y[:, 2].reshape(B, C, H, W), -2, axes=(2, 3)).reshape(B, C, L)
        oy = oy + np.rot90(y[:, 3].reshape(B, C, W, H), -3, axes=(2, 3)).reshape(B, C, L)
        return oy
    raise ValueError("scans must be 0, 1, 2 or 3")


# --------------------------------------------------------------------------- #
# layout and one-by-one variants of CrossScan / CrossMerge  (vmamba.py:41-245)
# --------------------------------------------------------------------------- #
def cross_scan_ex(x: np.ndarray, scans: int = 0, in_channel_first: bool = True, out_channel_first: bool = True,
                  one_by_one: bool = False) -> np.ndarray:
    """CrossScan with the reference's layout flags.

    x: (B, C, H, W) or, channel-last, (B, H, W, C); one_by_one: (B, 4, C, H, W) or, channel-last, (B, H, W, 4, C),
    route k reads its own map x[:, k] (csm_triton.py:88-131).  Result (B, 4, C, L) or, with out_channel_first
    False, (B, L, 4, C) (csm_triton.py:420, the shapes the reference's GPU path allocates).  The reference's torch
    path returns the same memory for every combination but one_by_one, scans 1, channel-first in and channel-last
    out, where its `flatten(2, 3)` on the 5-d tensor merges C with H before the permute (csm_triton.py:101, 126);
    its GPU path (csm_triton.py:403-431) has no such case, and this restatement follows the GPU path there."""
    if one_by_one:
        xc = x if in_channel_first else np.ascontiguousarray(x.transpose(0, 3, 4, 1, 2))   # (B,H,W,4,C) -> (B,4,C,H,W)
        B, K, C, H, W = xc.shape
        assert K == 4
        y = np.stack([cross_scan(np.ascontiguousarray(xc[:, k]), scans)[:, k] for k in range(4)], axis=1)
        if scans == 1 and in_channel_first and out_channel_first:
            return xc.reshape(B, 4, C * H, W).copy()    # csm_triton.py:101: the torch path's shape, same memory
        return y if out_channel_first else np.ascontiguousarray(y.transpose(0, 3, 1, 2))
    xc = x if in_channel_first else np.ascontiguousarray(np.moveaxis(x, -1, 1))
    y = cross_scan(xc, scans)                                   # (B, 4, C, L)
    return y if out_channel_first else np.ascontiguousarray(y.transpose(0, 3, 1, 2))


def cross_merge_ex(ys: np.ndarray, scans: int = 0, in_channel_first: bool = True, out_channel_first: bool = True,
                   one_by_one: bool = False) -> np.ndarray:
    """CrossMerge with the reference's layout flags: `out_channel_first` names the layout of the routes ys
    ((B, 4, C, H, W) or (B, H, W, 4, C)), `in_channel_first` the layout of the result ((B, C, L) or (B, L, C)),
    as in cross_merge_fwd (vmamba.py:87-130).  one_by_one: every route is brought back to row-major order
    separately, no sum: (B, 4, C, L) or, with in_channel_first False, (B, L, 4, C) (csm_triton.py:134-179)."""
    if one_by_one:
        yc = ys if out_channel_first else np.ascontiguousarray(ys.transpose(0, 3, 4, 1, 2))
        B, K, C, H, W = yc.shape
        out = np.empty((B, 4, C, H * W), dtype=ys.dtype)
        for k in range(4):
            only = np.zeros_like(yc)
            only[:, k] = yc[:, k]
            out[:, k] = cross_merge(only, scans)                # x + 0 is exact: the un-permuted route k
        return out if in_channel_first else np.ascontiguousarray(out.transpose(0, 3, 1, 2))
    yc = ys if out_channel_first else np.ascontiguousarray(ys.transpose(0, 3, 4, 1, 2))     # (B,H,W,K,D) -> (B,K,D,H,W)
    y = cross_merge(yc, scans)                                  # (B, C, L)
    return y if in_channel_first else np.ascontiguousarray(y.transpose(0, 2, 1))


# --------------------------------------------------------------------------- #
# a5/a6: selective scan  (vmamba.py:791-834)
# --------------------------------------------------------------------------- #
def softplus(x: np.ndarray) -> np.ndarray:
    """torch.nn.functional.softplus with beta=1, threshold=20 (vmamba.py:816)."""
    x = np.asarray(x, dtype=np.float32)
    with np.errstate(over="ignore"):
        sp = np.log1p(np.exp(np.minimum(x, np.float32(20.0)))).astype(np.float32)
    return np.where(x > 20.0, x, sp).astype(np.float32)


def selective_scan(u, delta, A, B, C, D=None, delta_bias=None, delta_softplus=True,
                   oflex=True, dtype_in: str = "f32") -> np.ndarray:
    """Sequential recurrence, fp32 state (vmamba.py:805-834).

    u, delta: (Bt, K*Cd, L); A: (K*Cd, N); B, C: (Bt, K, N, L); D, delta_bias: (K*Cd,).
    h_n <- exp(delta' * A_n) * h_n + delta' * B_n * u ;  y = sum_n C_n h_n (+ D u)
    with delta' = softplus(delta + delta_bias).
    `dtype_in` names the storage type of u/delta/B/C; with a bias the sum
    delta + bias is formed in fp32 (the bias is fp32, vmamba.py:813-814); without one
    the softplus runs in the storage type (vmamba.py:815-816) and is rounded to it.
    Output fp32 when `oflex`, else rounded to `dtype_in` (vmamba.py:834).
    """
    u = np.asarray(u, dtype=np.float32)
    delta = np.asarray(delta, dtype=np.float32)
    A = np.asarray(A, dtype=np.float32)
    B = np.asarray(B, dtype=np.float32)
    C = np.asarray(C, dtype=np.float32)
    Bt, K, N, L = B.shape
    KC = u.shape[1]
    Cd = KC // K
    assert u.shape == (Bt, KC, L) and delta.shape == (Bt, KC, L)
    assert A.shape == (KC, N) and C.shape == B.shape

    if delta_bias is not None:
        delta = delta + np.asarray(delta_bias, dtype=np.float32)[None, :, None]
        if delta_softplus:
            delta = softplus(delta)
    elif delta_softplus:
        delta = _round_to(softplus(delta), dtype_in)

    Bx = np.repeat(B, Cd, axis=1).reshape(Bt, KC, N, L)   # (Bt, K, 1, N, L) repeated over Cd
    Cx = np.repeat(C, Cd, axis=1).reshape(Bt, KC, N, L)
    # note: np.repeat on axis 1 of (Bt, K, N, L) gives k-major order k0,k0,..,k1,.. == view(K,1)->repeat(Cd)
    h = np.zeros((Bt, KC, N), dtype=np.float32)
    y = np.empty((Bt, KC, L), dtype=np.float32)
    for i in range(L):
        dl = delta[:, :, i]                                   # (Bt, KC)
        dA = np.exp(dl[:, :, None] * A[None]).astype(np.float32)
        dBu = (dl * u[:, :, i])[:, :, None] * Bx[:, :, :, i]
        h = dA * h + dBu
        y[:, :, i] = np.sum(h * Cx[:, :, :, i], axis=-1, dtype=np.float32)
    out = y if D is None else y + u * np.asarray(D, dtype=np.float32)[None, :, None]
    out = out.astype(np.float32)
    return out if oflex else _round_to(out, dtype_in)


def selective_scan_bwd(u, delta, A, B, C, D, delta_bias, dout, delta_softplus=True, dtype_in: str = "f32"):
    """Gradients of `selective_scan` for an upstream gradient dout (Bt, K*Cd, L).

    What SelectiveScanCuda.backward returns (csms6s.py:89-109; shapes and types of the results
    as in selective_scan_oflex.cpp:308-353): du, ddelta like u; dA (K*Cd, N) fp32; dB, dC like B, C
    (accumulated in fp32 over the channels of a group, then rounded to the storage type);
    dD, ddelta_bias (K*Cd,) fp32, or None where the input was None.  With
    d' = softplus(delta + bias), a = exp(d' A), h_l = a_l h_{l-1} + d'_l B_l u_l, y_l = C_l . h_l + D u_l:
        dh_l  = C_l dout_l + a_{l+1} dh_{l+1}                    (reverse recurrence)
        dC_l  = sum_channels dout_l h_l          dB_l = sum_channels dh_l d'_l u_l
        du_l  = dout_l D + d'_l (B_l . dh_l)     dD   = sum_{b,l} dout_l u_l
        dd'_l = sum_n dh_l (B_l u_l + A a_l h_{l-1})             dA = sum_{b,l} dh_l d'_l a_l h_{l-1}
        ddelta_l = dd'_l * sigmoid(delta_l + bias) where softplus is applied below its threshold 20
    The forward states are recomputed exactly as in `selective_scan` (fp32).
    """
    u = np.asarray(u, dtype=np.float32)
    draw = np.asarray(delta, dtype=np.float32)
    A = np.asarray(A, dtype=np.float32)
    B = np.asarray(B, dtype=np.float32)
    C = np.asarray(C, dtype=np.float32)
    g = np.asarray(dout, dtype=np.float32)
    Bt, K, N, L = B.shape
    KC = u.shape[1]
    Cd = KC // K
    x = draw if delta_bias is None else draw + np.asarray(delta_bias, dtype=np.float32)[None, :, None]
    if delta_softplus:
        dl = softplus(x)
        if delta_bias is None:
            dl = _round_to(dl, dtype_in)
        with np.errstate(over="ignore"):
            dsp = np.where(x > 20.0, 1.0, 1.0 / (1.0 + np.exp(-x))).astype(np.float32)
    else:
        dl, dsp = x, np.ones_like(x)
    Bx = np.repeat(B, Cd, axis=1).reshape(Bt, KC, N, L)
    Cx = np.repeat(C, Cd, axis=1).reshape(Bt, KC, N, L)
    a = np.exp(dl[:, :, None, :] * A[None, :, :, None]).astype(np.float32)        # (Bt, KC, N, L)
    hs = np.empty((Bt, KC, N, L), dtype=np.float32)
    h = np.zeros((Bt, KC, N), dtype=np.float32)
    for i in range(L):
        h = a[..., i] * h + (dl[:, :, i] * u[:, :, i])[:, :, None] * Bx[..., i]
        hs[..., i] = h
    hprev = np.concatenate([np.zeros((Bt, KC, N, 1), np.float32), hs[..., :-1]], axis=-1)
    dh = np.empty_like(hs)
    e = np.zeros((Bt, KC, N), dtype=np.float32)      # a_{l+1} dh_{l+1}
    for i in range(L - 1, -1, -1):
        dh[..., i] = Cx[..., i] * g[:, :, None, i] + e
        e = a[..., i] * dh[..., i]
    dC = (g[:, :, None, :] * hs).reshape(Bt, K, Cd, N, L).sum(axis=2, dtype=np.float32)
    dB = (dh * (dl * u)[:, :, None, :]).reshape(Bt, K, Cd, N, L).sum(axis=2, dtype=np.float32)
    du = dl * np.sum(Bx * dh, axis=2, dtype=np.float32)
    ddl = np.sum(dh * (Bx * u[:, :, None, :] + A[None, :, :, None] * a * hprev), axis=2, dtype=np.float32)
    dA = np.sum(dh * a * hprev * dl[:, :, None, :], axis=(0, 3), dtype=np.float32)
    dD = None
    if D is not None:
        du = du + g * np.asarray(D, dtype=np.float32)[None, :, None]
        dD = np.sum(g * u, axis=(0, 2), dtype=np.float32)
    ddelta = (ddl * dsp).astype(np.float32)
    dbias = None if delta_bias is None else np.sum(ddelta, axis=(0, 2), dtype=np.float32)
    return (_round_to(du.astype(np.float32), dtype_in), _round_to(ddelta, dtype_in), dA,
            _round_to(dB, dtype_in), _round_to(dC, dtype_in), dD, dbias)


# --------------------------------------------------------------------------- #
# a8: channel-first LayerNorm  (vmamba.py:1078-1093)
# --------------------------------------------------------------------------- #
def layer_norm_cf(y: np.ndarray, weight=None, bias=None, eps: float = 1e-5) -> np.ndarray:
    """LayerNorm over axis 1 of a (B, D, ...) array (biased variance, as torch)."""
    y = np.asarray(y, dtype=np.float32)
    mean = y.mean(axis=1, keepdims=True, dtype=np.float32)
    var = ((y - mean) ** 2).mean(axis=1, keepdims=True, dtype=np.float32)
    out = (y - mean) / np.sqrt(var + np.float32(eps))
    shp = (1, -1) + (1,) * (y.ndim - 2)
    if weight is not None:
        out = out * np.asarray(weight, dtype=np.float32).reshape(shp)
    if bias is not None:
        out = out + np.asarray(bias, dtype=np.float32).reshape(shp)
    return out.astype(np.float32)


# --------------------------------------------------------------------------- #
# a1-a8 composed: SS2D core  (vmamba.py:1504-1571)
# --------------------------------------------------------------------------- #
def ss2d_core(x, x_proj_weight, dt_projs_weight, dt_projs_bias, A_logs, Ds,
              out_norm_weight=None, out_norm_bias=None, *, d_state: int, dt_rank: int,
              scans: int = 0, act_dtype: str = "f32", eps: float = 1e-5,
              with_out_norm: bool = True, return_parts: bool = False):
    """forward_corev2 for channel-first input, LayerNorm out-norm.

    x: (B, D, H, W) activation (already conv+SiLU'd).  x_proj_weight: (K*(R+2N), D);
    dt_projs_weight: (K*D, R); dt_projs_bias: (K, D) or (K*D,); A_logs: (K*D, N); Ds: (K*D,).
    `act_dtype` emulates autocast: with "bf16" the tensors the reference would hold in
    bf16 (xs, x_dbl, dts, Bs, Cs and the returned y) are rounded to bf16 at the same
    points; the recurrence, merge and LayerNorm stay fp32 (vmamba.py:1544-1571).
    """
    x = _round_to(x, act_dtype)
    Bt, D, H, W = x.shape
    K, N, R = K_ROUTES, int(d_state), int(dt_rank)
    L = H * W
    Wx = np.asarray(x_proj_weight, dtype=np.float32).reshape(K, R + 2 * N, D)
    Wdt = np.asarray(dt_projs_weight, dtype=np.float32).reshape(K, D, R)
    if act_dtype != "f32":   # autocast casts the conv weights to the activation dtype
        Wx, Wdt = _round_to(Wx, act_dtype), _round_to(Wdt, act_dtype)

    xs = cross_scan(x, scans)                                   # (B, K, D, L)   :1536
    x_dbl = np.einsum("kcd,bkdl->bkcl", Wx, xs, dtype=np.float32)   # grouped conv1d :1537
    x_dbl = _round_to(x_dbl, act_dtype)
    dts_low, Bs, Cs = x_dbl[:, :, :R], x_dbl[:, :, R:R + N], x_dbl[:, :, R + N:]   # :1538
    dts = np.einsum("kdr,bkrl->bkdl", Wdt, dts_low, dtype=np.float32)          # :1539-1540
    dts = _round_to(dts, act_dtype).reshape(Bt, K * D, L)
    As = -np.exp(np.asarray(A_logs, dtype=np.float32)).reshape(K * D, N)        # :1544
    Dsf = np.asarray(Ds, dtype=np.float32).reshape(K * D)
    bias = np.asarray(dt_projs_bias, dtype=np.float32).reshape(K * D)          # :1548
    ys = selective_scan(xs.reshape(Bt, K * D, L), dts, As, np.ascontiguousarray(Bs),
                        np.ascontiguousarray(Cs), Dsf, bias, True, True, act_dtype)   # :1553
    y = cross_merge(ys.reshape(Bt, K, D, H, W), scans).reshape(Bt, D, H, W)    # :1557
    merged = y
    if with_out_norm:
        y = layer_norm_cf(y, out_norm_weight, out_norm_bias, eps)              # :1569
    y = _round_to(y, act_dtype)                                                # :1571
    if return_parts:
        return y, dict(xs=xs, dts=dts, Bs=Bs, Cs=Cs, As=As, ys=ys, merged=merged)
    return y


# --------------------------------------------------------------------------- #
# seeded synthetic inputs (value distributions of mamba_init, vmamba.py:1170-1237)
# --------------------------------------------------------------------------- #
def make_scan_inputs(Bt: int, D: int, H: int, W: int, N: int = 1, seed: int = 0,
                     act_dtype: str = "f32"):
    """Synthetic operator-level inputs: x ~ N(0,1); raw delta ~ N(0,1);
    delta_bias = inverse-softplus(dt), dt log-uniform in [1e-3, 1e-1] (vmamba.py:1185-1190);
    A = -exp(A_log), A_log = log(1..N) (vmamba.py:1201-1203); B, C ~ N(0,1); D = 1."""
    rng = np.random.default_rng(seed)
    K, L = K_ROUTES, H * W
    x = rng.standard_normal((Bt, D, H, W), dtype=np.float32)
    delta = rng.standard_normal((Bt, K * D, L), dtype=np.float32)
    dt = np.exp(rng.random(K * D, dtype=np.float32) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    dt = np.maximum(dt, 1e-4).astype(np.float32)
    delta_bias = (dt + np.log(-np.expm1(-dt))).astype(np.float32)
    A = -np.tile(np.arange(1, N + 1, dtype=np.float32)[None], (K * D, 1))
    Bs = rng.standard_normal((Bt, K, N, L), dtype=np.float32)
    Cs = rng.standard_normal((Bt, K, N, L), dtype=np.float32)
    Dp = np.ones(K * D, dtype=np.float32)
    x, delta, Bs, Cs = (_round_to(t, act_dtype) for t in (x, delta, Bs, Cs))
    return dict(x=x, delta=delta, A=A, Bs=Bs, Cs=Cs, D=Dp, delta_bias=delta_bias)


def max_rel_err(got, ref) -> float:
    """max |got - ref| / max |ref| -- the 'max relative error' used for float parity."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    denom = max(float(np.max(np.abs(ref))), 1e-30)
    return float(np.max(np.abs(got - ref))) / denom
