"""CPU oracle for the VMamba backbones that exercise the SS2D core -- TEST INFRASTRUCTURE.

A functional restatement of the reference's inference forward for the `v05_noz`,
channel-first ("ln2d") model family (VMamba-T/S/B): the layers around the core use
torch CPU functional ops (the reference is torch), the SS2D core itself runs through
the oracle of this folder (C statement; numpy statement for small inputs).  It takes
a reference-format state dict (name -> float32 array) so that a checkpoint or a
random init of the reference can be evaluated without the reference's code.

Parity status: PINNED against tests/golden/vssm_small*.npz, produced by the
unmodified reference (tests/golden/make_golden.py).

Reference anchors (paths inside MzeroMiko/VMamba):
  patch embed v2        vmamba.py:1928-1942      downsample v3   vmamba.py:1964-1971
  VSSBlock._forward     vmamba.py:1766-1778      Mlp             vmamba.py:1151-1167
  SS2D.forwardv2        vmamba.py:1573-1589      forward_corev2  vmamba.py:1504-1571
  VSSM.forward          vmamba.py:2027-2035      classifier      vmamba.py:1881-1887
  Backbone_VSSM.forward vmamba.py:2133-2153
"""
from __future__ import annotations

import math
import re

import numpy as np
import torch
import torch.nn.functional as F

from . import c_oracle, ss2d_oracle


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))


def _ln_cf(x: torch.Tensor, w, b, eps=1e-5):
    """LayerNorm over channels of a (B, C, H, W) map (vmamba.py:1087-1093)."""
    y = F.layer_norm(x.permute(0, 2, 3, 1), (x.shape[1],), _t(w), _t(b), eps)
    return y.permute(0, 3, 1, 2)


def ss2d_core_c(x: np.ndarray, sd: dict, prefix: str, d_state: int, dt_rank: int) -> np.ndarray:
    """forward_corev2 through the C oracle, fp32 (vmamba.py:1504-1571)."""
    Bt, D, H, W = x.shape
    K, N, R, L = 4, d_state, dt_rank, H * W
    Wx = np.asarray(sd[prefix + "x_proj.weight"], np.float32).reshape(K, R + 2 * N, D)
    Wdt = np.asarray(sd[prefix + "dt_projs.weight"], np.float32).reshape(K, D, R)
    xs = c_oracle.cross_scan(x, 0)
    x_dbl = torch.einsum("kcd,bkdl->bkcl", _t(Wx), _t(xs))
    dts = torch.einsum("kdr,bkrl->bkdl", _t(Wdt), x_dbl[:, :, :R]).reshape(Bt, K * D, L).numpy()
    Bs = x_dbl[:, :, R:R + N].contiguous().numpy()
    Cs = x_dbl[:, :, R + N:].contiguous().numpy()
    As = -np.exp(np.asarray(sd[prefix + "A_logs"], np.float32))
    ys = c_oracle.selective_scan(xs.reshape(Bt, K * D, L), dts, As, Bs, Cs,
                                 np.asarray(sd[prefix + "Ds"], np.float32),
                                 np.asarray(sd[prefix + "dt_projs_bias"], np.float32).reshape(-1), True)
    y = c_oracle.cross_merge(ys.reshape(Bt, K, D, H, W), 0)
    y = c_oracle.layer_norm_cf(y, sd[prefix + "out_norm.weight"], sd[prefix + "out_norm.bias"], 1e-5)
    return y.reshape(Bt, D, H, W)


def ss2d_forward(x: torch.Tensor, sd: dict, prefix: str, use_numpy_core: bool = False) -> torch.Tensor:
    """SS2D.forwardv2 for forward_type v05_noz, channel-first (vmamba.py:1573-1589)."""
    w_in = _t(sd[prefix + "in_proj.weight"])
    D = w_in.shape[0]
    N = sd[prefix + "A_logs"].shape[1]
    R = sd[prefix + "dt_projs.weight"].shape[1]
    x = F.conv2d(x, w_in[:, :, None, None])
    x = F.conv2d(x, _t(sd[prefix + "conv2d.weight"]),
                 None if (prefix + "conv2d.bias") not in sd else _t(sd[prefix + "conv2d.bias"]),
                 padding=1, groups=D)
    x = F.silu(x)
    if use_numpy_core:
        y = ss2d_oracle.ss2d_core(x.numpy(), sd[prefix + "x_proj.weight"], sd[prefix + "dt_projs.weight"],
                                  sd[prefix + "dt_projs_bias"], sd[prefix + "A_logs"], sd[prefix + "Ds"],
                                  sd[prefix + "out_norm.weight"], sd[prefix + "out_norm.bias"],
                                  d_state=N, dt_rank=R)
    else:
        y = ss2d_core_c(x.numpy(), sd, prefix, N, R)
    return F.conv2d(_t(y), _t(sd[prefix + "out_proj.weight"])[:, :, None, None])


def block_forward(x: torch.Tensor, sd: dict, prefix: str) -> torch.Tensor:
    """VSSBlock._forward, pre-norm, eval mode (vmamba.py:1766-1778)."""
    x = x + ss2d_forward(_ln_cf(x, sd[prefix + "norm.weight"], sd[prefix + "norm.bias"]), sd, prefix + "op.")
    h = _ln_cf(x, sd[prefix + "norm2.weight"], sd[prefix + "norm2.bias"])
    h = F.conv2d(h, _t(sd[prefix + "mlp.fc1.weight"])[:, :, None, None], _t(sd[prefix + "mlp.fc1.bias"]))
    h = F.gelu(h)
    h = F.conv2d(h, _t(sd[prefix + "mlp.fc2.weight"])[:, :, None, None], _t(sd[prefix + "mlp.fc2.bias"]))
    return x + h


def _depths(sd: dict):
    n = {}
    for k in sd:
        m = re.match(r"layers\.(\d+)\.blocks\.(\d+)\.", k)
        if m:
            i, j = int(m.group(1)), int(m.group(2))
            n[i] = max(n.get(i, 0), j + 1)
    return [n[i] for i in sorted(n)]


def stem(img: torch.Tensor, sd: dict) -> torch.Tensor:
    """patch embed v2: conv3x3 s2 -> LN -> GELU -> conv3x3 s2 -> LN (vmamba.py:1928-1942)."""
    x = F.conv2d(img, _t(sd["patch_embed.0.weight"]), _t(sd["patch_embed.0.bias"]), stride=2, padding=1)
    x = F.gelu(_ln_cf(x, sd["patch_embed.2.weight"], sd["patch_embed.2.bias"]))
    x = F.conv2d(x, _t(sd["patch_embed.5.weight"]), _t(sd["patch_embed.5.bias"]), stride=2, padding=1)
    return _ln_cf(x, sd["patch_embed.7.weight"], sd["patch_embed.7.bias"])


def features(img: np.ndarray, sd: dict):
    """Per-stage block outputs (before downsample) and the final map."""
    x = stem(_t(img), sd)
    depths = _depths(sd)
    outs = []
    for i, depth in enumerate(depths):
        for j in range(depth):
            x = block_forward(x, sd, f"layers.{i}.blocks.{j}.")
        outs.append(x)
        if i < len(depths) - 1:     # downsample v3 (vmamba.py:1964-1971)
            x = F.conv2d(x, _t(sd[f"layers.{i}.downsample.1.weight"]), _t(sd[f"layers.{i}.downsample.1.bias"]),
                         stride=2, padding=1)
            x = _ln_cf(x, sd[f"layers.{i}.downsample.3.weight"], sd[f"layers.{i}.downsample.3.bias"])
    return outs, x


def vssm_logits(img: np.ndarray, sd: dict) -> np.ndarray:
    """VSSM.forward (vmamba.py:2027-2035) with the classifier of vmamba.py:1881-1887."""
    _, x = features(img, sd)
    x = _ln_cf(x, sd["classifier.norm.weight"], sd["classifier.norm.bias"])
    x = x.mean(dim=(2, 3))
    return F.linear(x, _t(sd["classifier.head.weight"]), _t(sd["classifier.head.bias"])).numpy()


def backbone_features(img: np.ndarray, sd: dict, out_indices=(0, 1, 2, 3)):
    """Backbone_VSSM.forward (vmamba.py:2133-2153): LN'd per-stage maps."""
    outs, _ = features(img, sd)
    return [_ln_cf(outs[i], sd[f"outnorm{i}.weight"], sd[f"outnorm{i}.bias"]).contiguous().numpy()
            for i in out_indices]


# --------------------------------------------------------------------------- #
# random init with the reference's distributions, for workloads whose weights
# cannot travel (VMamba-T/S/B are 30-89 M parameters)
# --------------------------------------------------------------------------- #
def random_state_dict(depths, dims, d_state=1, ssm_ratio=1.0, mlp_ratio=4.0, num_classes=1000,
                      in_chans=3, seed=0, with_outnorm=False) -> dict:
    """Random init in the value distributions the reference's one-file model ends up
    with: trunc-normal(std 0.02) for every Linear incl. x_proj / dt_projs
    (vmamba.py:1898-1905), LayerNorm (1, 0), PyTorch's default conv init, dt bias =
    inverse-softplus of log-uniform [1e-3, 1e-1], A_log = log(1..N), D = 1
    (vmamba.py:1170-1237).  Not bit-identical to any reference RNG stream."""
    g = torch.Generator().manual_seed(seed)
    sd = {}

    def tn(*shape):
        t = torch.empty(shape)
        torch.nn.init.trunc_normal_(t, std=0.02, generator=g)
        return t.numpy()

    def conv(cout, cin, k, groups=1, bias=True, name=""):
        fan_in = cin // groups * k * k
        bound = 1.0 / math.sqrt(fan_in)
        sd[name + ".weight"] = ((torch.rand((cout, cin // groups, k, k), generator=g) * 2 - 1) * bound).numpy()
        if bias:
            sd[name + ".bias"] = ((torch.rand(cout, generator=g) * 2 - 1) * bound).numpy()

    def ln(name, c):
        sd[name + ".weight"] = np.ones(c, np.float32)
        sd[name + ".bias"] = np.zeros(c, np.float32)

    conv(dims[0] // 2, in_chans, 3, name="patch_embed.0"); ln("patch_embed.2", dims[0] // 2)
    conv(dims[0], dims[0] // 2, 3, name="patch_embed.5"); ln("patch_embed.7", dims[0])
    for i, (depth, C) in enumerate(zip(depths, dims)):
        D, R, K, N = int(ssm_ratio * C), math.ceil(C / 16), 4, d_state
        for j in range(depth):
            p = f"layers.{i}.blocks.{j}."
            ln(p + "norm", C)
            sd[p + "op.A_logs"] = np.tile(np.log(np.arange(1, N + 1, dtype=np.float32))[None], (K * D, 1))
            sd[p + "op.Ds"] = np.ones(K * D, np.float32)
            dt = torch.exp(torch.rand((K, D), generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3)).clamp(min=1e-4)
            sd[p + "op.dt_projs_bias"] = (dt + torch.log(-torch.expm1(-dt))).numpy()
            ln(p + "op.out_norm", D)
            sd[p + "op.in_proj.weight"] = tn(D, C)
            conv(D, D, 3, groups=D, bias=False, name=p + "op.conv2d")
            sd[p + "op.x_proj.weight"] = tn(K * (R + 2 * N), D)
            sd[p + "op.dt_projs.weight"] = tn(K * D, R)
            sd[p + "op.out_proj.weight"] = tn(C, D)
            ln(p + "norm2", C)
            Hd = int(C * mlp_ratio)
            sd[p + "mlp.fc1.weight"] = tn(Hd, C); sd[p + "mlp.fc1.bias"] = np.zeros(Hd, np.float32)
            sd[p + "mlp.fc2.weight"] = tn(C, Hd); sd[p + "mlp.fc2.bias"] = np.zeros(C, np.float32)
        if i < len(depths) - 1:
            conv(dims[i + 1], C, 3, name=f"layers.{i}.downsample.1"); ln(f"layers.{i}.downsample.3", dims[i + 1])
        if with_outnorm:
            ln(f"outnorm{i}", C)
    ln("classifier.norm", dims[-1])
    sd["classifier.head.weight"] = tn(num_classes, dims[-1])
    sd["classifier.head.bias"] = np.zeros(num_classes, np.float32)
    return {k: np.ascontiguousarray(v, dtype=np.float32) for k, v in sd.items()}


CONFIGS = dict(
    # vmamba.py:2286-2300, 2250-2264, 2268-2282
    vmamba_tiny_s1l8=dict(depths=[2, 2, 8, 2], dims=[96, 192, 384, 768], d_state=1, ssm_ratio=1.0),
    vmamba_small_s2l15=dict(depths=[2, 2, 15, 2], dims=[96, 192, 384, 768], d_state=1, ssm_ratio=2.0),
    vmamba_base_s2l15=dict(depths=[2, 2, 15, 2], dims=[128, 256, 512, 1024], d_state=1, ssm_ratio=2.0),
)
