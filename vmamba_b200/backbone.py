"""Inference-only VMamba backbone around the fused SS2D core.

Host-side mirror of the reference's `VSSM` / `Backbone_VSSM` forward for the model family the
headline numbers are quoted on: forward_type "v05_noz", channel-first ("ln2d"), patch embed v2,
downsample v3, ssm_conv 3 without bias (vmamba.py:2250-2300).  It consumes a state dict in the
reference's own key layout (vmamba.py:1788-2035), so weights trained with or initialised by the
reference load unchanged.

Only the SS2D core and the channel-first LayerNorms are this package's kernels; the dense
contractions (1x1 projections, MLP, strided 3x3 convolutions) are library calls, the rest are
elementwise torch ops.  Precision follows the reference's autocast recipe: bf16 (or fp16/fp32)
activations into every contraction, fp32 LayerNorm statistics, fp32 residual stream, fp32 state in
the scan.
"""
from __future__ import annotations

import math
import re
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from . import ops
from .fused import CoreWeights, ss2d_core

# vmamba.py:2286-2300 (tiny), 2250-2264 (small), 2268-2282 (base)
CONFIGS = dict(
    vmamba_tiny_s1l8=dict(depths=[2, 2, 8, 2], dims=[96, 192, 384, 768], d_state=1, ssm_ratio=1.0),
    vmamba_small_s2l15=dict(depths=[2, 2, 15, 2], dims=[96, 192, 384, 768], d_state=1, ssm_ratio=2.0),
    vmamba_base_s2l15=dict(depths=[2, 2, 15, 2], dims=[128, 256, 512, 1024], d_state=1, ssm_ratio=2.0),
)


class _Block:
    __slots__ = ("n1w", "n1b", "w_in", "w_dw", "core", "w_out", "n2w", "n2b", "w1", "b1f", "w2", "b2f", "D")


def normalize_state_dict(sd: dict) -> dict:
    """Checkpoint keys in the current naming of the reference.  Applies the renames the reference's own
    loaders apply (`VSSM._load_from_state_dict`, vmamba.py:2061-2102; `SS2D._load_from_state_dict`,
    vmamba.py:1682-1697) and unwraps the {"model": ...} / {"state_dict": ...} containers its training
    script writes, so that older released checkpoints load as they do there.  Returns a new dict; tensors
    are shared, not copied."""
    for key in ("model", "state_dict", "model_ema"):
        if isinstance(sd.get(key), dict) and any(isinstance(v, torch.Tensor) or hasattr(v, "shape") for v in sd[key].values()):
            sd = sd[key]
            break
    out = {}
    prefix_map = [("patch_embed.proj", "patch_embed.0"), ("patch_embed.norm", "patch_embed.2")]
    top_map = [("norm.", "classifier.norm."), ("head.", "classifier.head.")]
    for k, v in sd.items():
        nk = k[len("module."):] if k.startswith("module.") else k       # DistributedDataParallel wrapper
        for src, dst in prefix_map:
            if nk.startswith(src):
                nk = dst + nk[len(src):]
        for src, dst in top_map:
            if nk.startswith(src):
                nk = dst + nk[len(src):]
        nk = re.sub(r"^(layers\.\d+\.blocks\.\d+)\.ln_1", r"\1.norm", nk)
        nk = re.sub(r"^(layers\.\d+\.blocks\.\d+)\.self_attention", r"\1.op", nk)
        nk = re.sub(r"^(layers\.\d+\.downsample)\.norm", r"\1.1", nk)
        nk = re.sub(r"^(layers\.\d+\.downsample)\.reduction", r"\1.2", nk)
        for src, dst in (("x_proj_weight", "x_proj.weight"), ("x_proj_bias", "x_proj.bias"),
                         ("dt_projs_weight", "dt_projs.weight")):
            if nk.endswith("." + src):
                nk = nk[:-len(src)] + dst
        out[nk] = v
    return out


class VSSMInfer:
    """Functional VMamba forward.  `VSSMInfer.from_state_dict(sd, dtype=torch.bfloat16)`."""

    def __init__(self):
        self.blocks: List[List[_Block]] = []
        self.down: List[Optional[dict]] = []
        self.stem: dict = {}
        self.head: Optional[dict] = None
        self.outnorm: Dict[int, tuple] = {}
        self.dtype = torch.bfloat16
        self.device = torch.device("cuda")

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_state_dict(sd: dict, dtype=torch.bfloat16, device="cuda") -> "VSSMInfer":
        dev = torch.device(device)
        m = VSSMInfer()
        m.dtype, m.device = dtype, dev
        sd = normalize_state_dict(sd)

        def T(name, dt=None):
            v = sd[name]
            v = torch.as_tensor(v) if not isinstance(v, torch.Tensor) else v
            return v.detach().to(device=dev, dtype=dt or torch.float32).contiguous()

        depths = {}
        for k in sd:
            mt = re.match(r"layers\.(\d+)\.blocks\.(\d+)\.", k)
            if mt:
                i, j = int(mt.group(1)), int(mt.group(2))
                depths[i] = max(depths.get(i, 0), j + 1)
        m.stem = dict(w0=T("patch_embed.0.weight", dtype), b0=T("patch_embed.0.bias", dtype).float(),
                      n0w=T("patch_embed.2.weight"), n0b=T("patch_embed.2.bias"),
                      w1=T("patch_embed.5.weight", dtype).contiguous(memory_format=torch.channels_last),
                      b1=T("patch_embed.5.bias", dtype).float(),
                      n1w=T("patch_embed.7.weight"), n1b=T("patch_embed.7.bias"))
        for i in sorted(depths):
            stage = []
            for j in range(depths[i]):
                p = f"layers.{i}.blocks.{j}."
                if p + "op.in_proj.bias" in sd or p + "op.conv2d.bias" in sd:
                    raise NotImplementedError("in_proj / conv2d biases are not part of the v05_noz family")
                b = _Block()
                b.n1w, b.n1b = T(p + "norm.weight"), T(p + "norm.bias")
                b.w_in = T(p + "op.in_proj.weight", dtype)
                b.D = b.w_in.shape[0]
                if sd[p + "op.out_proj.weight"].shape[1] != b.D:
                    raise NotImplementedError("models with a z branch (no '_noz') are not supported")
                b.w_dw = T(p + "op.conv2d.weight", dtype)
                N = sd[p + "op.A_logs"].shape[1]
                R = sd[p + "op.dt_projs.weight"].shape[1]
                b.core = CoreWeights.build(T(p + "op.x_proj.weight"), T(p + "op.dt_projs.weight"),
                                           T(p + "op.dt_projs_bias"), T(p + "op.A_logs"), T(p + "op.Ds"),
                                           T(p + "op.out_norm.weight"), T(p + "op.out_norm.bias"),
                                           d_state=N, dt_rank=R, dtype=dtype)
                b.w_out = T(p + "op.out_proj.weight", dtype)
                b.n2w, b.n2b = T(p + "norm2.weight"), T(p + "norm2.bias")
                b.w1, b.b1f = T(p + "mlp.fc1.weight", dtype), T(p + "mlp.fc1.bias", dtype).float()   # bias rounded as autocast does
                b.w2, b.b2f = T(p + "mlp.fc2.weight", dtype), T(p + "mlp.fc2.bias", dtype).float()
                stage.append(b)
            m.blocks.append(stage)
            q = f"layers.{i}.downsample."
            if q + "1.weight" in sd:
                m.down.append(dict(w=T(q + "1.weight", dtype).contiguous(memory_format=torch.channels_last),
                                   bf=T(q + "1.bias", dtype).float(),
                                   nw=T(q + "3.weight"), nb=T(q + "3.bias")))
            else:
                m.down.append(None)
            if f"outnorm{i}.weight" in sd:
                m.outnorm[i] = (T(f"outnorm{i}.weight"), T(f"outnorm{i}.bias"))
        if "classifier.head.weight" in sd:
            m.head = dict(nw=T("classifier.norm.weight"), nb=T("classifier.norm.bias"),
                          w=T("classifier.head.weight", dtype), b=T("classifier.head.bias", dtype))
        return m

    # ------------------------------------------------------------------ layers
    # Between the stem and the head every map is kept CHANNEL-MAJOR, (C, B, H, W): each 1x1 projection
    # is then ONE GEMM  (C_out x C_in) . (C_in x B*H*W)  whose long dimension is a multiple of 8 for any
    # map size (14x14 and 7x7 maps would otherwise give 128 small GEMMs with unaligned leading dimensions),
    # while every (channel, image) plane stays a contiguous run of H*W pixels for the scan kernels.
    def _ln(self, x, w, b, out_dtype=None, cm=True, out_cm=None):
        """channel-first LayerNorm (vmamba.py:1078-1093), fp32 statistics."""
        return ops.layer_norm_cf(x, w, b, 1e-5, out_dtype or self.dtype, channel_major=cm, out_channel_major=out_cm)

    @staticmethod
    def _pw(w, x):
        """1x1 convolution of a channel-major map as one GEMM (vmamba.py:1060-1064)."""
        C, B, H, W = x.shape
        return torch.matmul(w, x.view(C, B * H * W)).view(w.shape[0], B, H, W)

    def _block(self, x: torch.Tensor, h: torch.Tensor, b: _Block, nxt):
        """VSSBlock._forward, eval mode (vmamba.py:1766-1778).  x: fp32 residual stream (updated in
        place), h = norm(x) of this block.  Returns (x, norm_next(x)) where norm_next is the first
        norm of the following block (`nxt` = its weight/bias) or None at the end of a stage: both
        residual additions are fused into the LayerNorm that consumes their result."""
        h = self._pw(b.w_in, h)                                                   # in_proj          :1574
        h = ops.dwconv3x3_act(h, b.w_dw, None, "silu", channel_major=True)        # dwconv 3x3, SiLU :1582-1583
        h = ss2d_core(h, b.core, channel_major=True)                              # forward_core     :1584
        o = self._pw(b.w_out, h)                                                  # out_proj         :1588
        h = ops.layer_norm_cf(x, b.n2w, b.n2b, 1e-5, self.dtype, add=o, update=True, channel_major=True)   # :1772, 1777
        if ops.mlp_supported(h.shape[0], b.w1.shape[0], h.numel() // h.shape[0], h.dtype):
            m = ops.mlp_fused(h, b.w1, b.b1f, b.w2)                               # Mlp: fc1 + GELU + fc2, one kernel :1151-1167
        else:
            h = ops.bias_act_(self._pw(b.w1, h), b.b1f, "gelu", channel_major=True)   # Mlp fc1 + GELU   :1160-1163
            m = self._pw(b.w2, h)                                                 # fc2 (its bias joins the residual update)
        if nxt is None:          # end of a stage: the caller decides what consumes x + m + bias
            return x, (m, b.b2f)
        return x, ops.layer_norm_cf(x, nxt[0], nxt[1], 1e-5, self.dtype, add=m, add_bias=b.b2f, update=True,
                                    channel_major=True)

    @staticmethod
    def _conv_s2(rows, w_cl):
        """3x3 stride-2 convolution (library) of a pixel-major (B, H, W, C) map; returns pixel-major.
        The tensor is handed over as a channels-last view, so the library runs its pixel-major kernel
        without converting."""
        y = F.conv2d(rows.permute(0, 3, 1, 2), w_cl, None, stride=2, padding=1)
        y = y.permute(0, 2, 3, 1)
        return y if y.is_contiguous() else y.contiguous()

    def _stem(self, img):
        """patch embed v2 (vmamba.py:1928-1942): conv+LayerNorm+GELU in one kernel, the second convolution in
        the library on the pixel-major map, its bias + LayerNorm + the change to channel planes in one kernel."""
        s = self.stem
        img = img.to(self.dtype)
        if ops.stem_supported(img.shape[1], s["w0"].shape[0]):
            x = ops.stem_conv_norm_act(img, s["w0"], s["b0"], s["n0w"], s["n0b"])            # (B, H/2, W/2, C0)
        else:
            x = F.conv2d(img, s["w0"], None, stride=2, padding=1)
            x = F.gelu(ops.layer_norm_cf(None, s["n0w"], s["n0b"], 1e-5, self.dtype, add=x, add_bias=s["b0"]))
            x = x.permute(0, 2, 3, 1).contiguous()
        x = self._conv_s2(x, s["w1"])
        return ops.pixels_norm_to_planes(x, s["b1"], s["n1w"], s["n1b"])                     # -> (C, B, H, W) fp32

    def _stages(self, img, want_features=False, head_norm=None):
        """Runs the stages.  Returns (per-stage residual maps if wanted, last value):
        the last value is the classifier-normalised (B, C, H, W) map when `head_norm` is given."""
        x = self._stem(img)
        outs = []
        last = None
        for i, stage in enumerate(self.blocks):
            h = self._ln(x, stage[0].n1w, stage[0].n1b)
            pend = None
            for j, b in enumerate(stage):
                nxt = (stage[j + 1].n1w, stage[j + 1].n1b) if j + 1 < len(stage) else None
                x, h = self._block(x, h, b, nxt)
                if nxt is None:
                    pend = h            # (m, bias): the last residual update of the stage, not applied yet
            m, mb = pend
            d = self.down[i]
            if d is not None:
                # downsample v3 (vmamba.py:1964-1971): x + m + bias as the pixel-major 16-bit input of the strided
                # convolution in one pass (the sum goes back into x only when the stage's map is asked for: the
                # convolution's output replaces the residual stream); its bias + LayerNorm + the way back to planes in another
                xin = ops.planes_to_pixels(x, add=m, add_bias=mb, update=want_features, out_dtype=self.dtype)
                if want_features:
                    outs.append(x.clone())
                x = ops.pixels_norm_to_planes(self._conv_s2(xin, d["w"]), d["bf"], d["nw"], d["nb"])
            else:
                if head_norm is not None:     # classifier norm fused with the last residual update
                    last = ops.layer_norm_cf(x, head_norm[0], head_norm[1], 1e-5, torch.float32, add=m, add_bias=mb,
                                             update=True, channel_major=True, out_channel_major=False)
                else:
                    ops.layer_norm_cf(x, None, None, 1e-5, self.dtype, add=m, add_bias=mb, update=True,
                                      channel_major=True, normalize=False)
                if want_features:
                    outs.append(x)
        return outs, (last if last is not None else x)

    # ------------------------------------------------------------------ public
    @torch.no_grad()
    def __call__(self, img: torch.Tensor) -> torch.Tensor:
        """VSSM.forward (vmamba.py:2027-2035): (B, 3, H, W) -> (B, num_classes) logits."""
        if self.head is None:
            raise RuntimeError("this model was built without a classifier")
        hd = self.head
        _, x = self._stages(img, head_norm=(hd["nw"], hd["nb"]))
        return F.linear(x.mean(dim=(2, 3)).to(self.dtype), hd["w"], hd["b"])

    @torch.no_grad()
    def features(self, img: torch.Tensor, out_indices: Sequence[int] = (0, 1, 2, 3)):
        """Backbone_VSSM.forward (vmamba.py:2133-2153): LayerNorm'ed per-stage maps."""
        outs, _ = self._stages(img, want_features=True)
        res = []
        for i in out_indices:
            w, b = self.outnorm[i]
            res.append(self._ln(outs[i], w, b, torch.float32, out_cm=False))
        return res


class AcceleratedVSSM(torch.nn.Module):
    """A reference `VSSM` / `Backbone_VSSM` module replaced, for inference, by this library's backbone on the same
    weights: `forward(images)` returns what the module's own forward returns (logits, vmamba.py:2027-2035, or the list of
    LayerNorm'ed feature maps, vmamba.py:2133-2153).  Built by `accelerate`."""

    def __init__(self, fast: VSSMInfer, features: bool, out_indices: Sequence[int]):
        super().__init__()
        self.fast, self._features, self.out_indices = fast, features, tuple(out_indices)
        self.training = False

    @torch.no_grad()
    def forward(self, images: torch.Tensor):
        images = images.to(device=self.fast.device, dtype=self.fast.dtype)
        if self._features:
            return self.fast.features(images, self.out_indices)
        return self.fast(images)

    def train(self, mode: bool = True):
        if mode:
            raise RuntimeError("AcceleratedVSSM is an inference module: train the reference module on the operator "
                               "surface (vmamba_b200.install) instead")
        return super().train(False)


def accelerate(model: torch.nn.Module, dtype: torch.dtype = torch.bfloat16, check: bool = True) -> AcceleratedVSSM:
    """The one-call drop-in at model level: a reference `VSSM` (or `Backbone_VSSM`) of the `v05_noz` channel-first family
    on a CUDA device -> an inference module that runs this library's backbone (channel-major maps, fused SS2D core,
    tcgen05 x_proj and MLP kernels) on the module's own weights.

    With `check` the two are compared on two random 64 x 64 images in fp32 before the module is handed over (the
    reference side runs on this library's operator surface for the comparison); a model of another family, or one this
    library does not reproduce, raises NotImplementedError instead of returning something that computes something else.
    """
    import sys
    params = list(model.parameters())
    if not params or not params[0].is_cuda:
        raise RuntimeError("accelerate() expects a module on a CUDA device (there is no CPU path)")
    device = params[0].device
    features = hasattr(model, "out_indices") and not hasattr(model, "classifier")
    out_indices = tuple(getattr(model, "out_indices", (0, 1, 2, 3)))
    sd = model.state_dict()
    try:
        fast = VSSMInfer.from_state_dict(sd, dtype=dtype, device=device)
    except (KeyError, NotImplementedError, RuntimeError) as e:
        raise NotImplementedError(f"accelerate(): not a v05_noz channel-first VSSM this library reproduces ({e})") from e
    if check:
        from . import patch
        was_training = model.training
        ref_module = sys.modules.get(type(model).__module__)
        probe = VSSMInfer.from_state_dict(sd, dtype=torch.float32, device=device)
        g = torch.Generator(device="cpu").manual_seed(0)
        x = torch.randn((2, 3, 64, 64), generator=g).to(device)
        old = torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32
        torch.backends.cudnn.allow_tf32 = torch.backends.cuda.matmul.allow_tf32 = False
        installed = ref_module is not None and not hasattr(ref_module, "__vmamba_b200_saved__")
        try:
            if installed:
                patch.install(ref_module)
            model.eval()
            with torch.no_grad():
                want = model(x)
                got = probe.features(x, out_indices) if features else probe(x)
        except Exception as e:      # the reference module itself could not run this input on the operator surface
            raise NotImplementedError(f"accelerate(): the module did not run on the operator surface ({type(e).__name__}: {e})") from e
        finally:
            if installed:
                patch.uninstall(ref_module)
            model.train(was_training)
            torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = old
        pairs = list(zip(want, got)) if features else [(want, got)]
        for w_, g_ in pairs:
            err = (w_.float() - g_.float()).abs().max().item() / max(w_.float().abs().max().item(), 1e-30)
            if not (err <= 1e-3):
                raise NotImplementedError(f"accelerate(): this library's backbone does not reproduce the module "
                                          f"(max relative difference {err:.2e} on a 64 x 64 probe)")
        del probe
    return AcceleratedVSSM(fast, features, out_indices)
