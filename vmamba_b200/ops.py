"""Operator surface of the reference, backed by the sm_100a kernels of libss2d_b200.so.

Mirrors, name for name, what MzeroMiko/VMamba's modules resolve at call time:
  selective_scan_fn, SelectiveScanCuda (+ alias SelectiveScanOflex)   classification/models/csms6s.py:71-126,
                                                                       vmamba.py:837-885
  cross_scan_fn, cross_merge_fn, CrossScanF, CrossMergeF (+ aliases)  classification/models/csm_triton.py:182-273,
                                                                       403-517; vmamba.py:254-345, 481-601
Forward (inference) only.  Tensors must live on a CUDA device; there is no torch/CPU path here
(`backend="torch"` raises).  Argument meaning, output shapes/dtypes and the error behaviour on bad
shapes follow the reference.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import (CrossExParams, CrossParams, NormParams, PointwiseParams, RelayoutParams, ScanBwdParams, ScanParams, StemParams,
                   check, lib)

_DTYPES = {torch.float32: _lib.SS2D_F32, torch.float16: _lib.SS2D_F16, torch.bfloat16: _lib.SS2D_BF16}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}: expected float32, float16 or bfloat16") from None


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("vmamba_b200 operators run on CUDA tensors only (no CPU fallback); "
                               "use the oracle under oracle/ for CPU reference values")


def _ptr(t):
    return None if t is None else t.data_ptr()


# --------------------------------------------------------------------------------------------
# selective scan
# --------------------------------------------------------------------------------------------
def selective_scan_fwd(u, delta, A, B, C, D=None, delta_bias=None, delta_softplus=False, out_float=True,
                       return_checkpoints=False, out=None):
    """out = selective scan of (u, delta, A, B, C [, D, delta_bias]); see include/ss2d_b200.h.

    u, delta: (batch, K*C, L); A: (K*C, N); B, C: (batch, K, N, L); D, delta_bias: (K*C,) fp32.
    Output fp32 if `out_float` (the reference's "oflex") else u.dtype.  With `return_checkpoints` also the fp32
    states in front of every 128th element, (batch, K*C, ceil(L/128), N), which `selective_scan_bwd` accepts
    instead of recomputing them.  `out`: optional result tensor of that shape and type (any batch / row strides,
    elements of a row contiguous), e.g. a permuted view, so that the result lands in the caller's layout.
    """
    _require_cuda(u, delta, A, B, C, D, delta_bias)
    if u.dim() != 3 or delta.dim() != 3 or delta.shape[0] != u.shape[0] or delta.shape[2] != u.shape[2] \
            or delta.shape[1] == 0 or u.shape[1] % delta.shape[1] != 0:
        raise RuntimeError(f"u must be (batch, dim, L) and delta (batch, dim / r, L), got {tuple(u.shape)} {tuple(delta.shape)}")
    if B.dim() != 4 or C.shape != B.shape:
        raise RuntimeError("B and C must be (batch, n_groups, dstate, L) with equal shapes")
    batch, dim, L = u.shape
    _, K, N, Lb = B.shape
    if B.shape[0] != batch or Lb != L or dim % K != 0:
        raise RuntimeError("B/C shape does not match u")
    if tuple(A.shape) != (dim, N):
        raise RuntimeError(f"A must be (dim, dstate) = ({dim}, {N}), got {tuple(A.shape)}")
    if delta.dtype != u.dtype or B.dtype != u.dtype or C.dtype != u.dtype:
        raise RuntimeError("u, delta, B, C must share one dtype")
    if u.stride(-1) != 1:
        u = u.contiguous()
    if delta.stride(-1) != 1:
        delta = delta.contiguous()
    if B.stride(-1) != 1:
        B = B.contiguous()
    if C.stride(-1) != 1:
        C = C.contiguous()
    A = A.contiguous().float()
    D = None if D is None else D.contiguous().float()
    delta_bias = None if delta_bias is None else delta_bias.contiguous().float()
    if D is not None and D.numel() != dim:
        raise RuntimeError("D must have dim elements")
    ratio = dim // delta.shape[1]        # channels sharing one delta row (selective_scan_oflex.cpp:59)
    if delta_bias is not None and delta_bias.numel() != delta.shape[1]:
        raise RuntimeError("delta_bias must have one element per delta row")
    out_dtype = torch.float32 if out_float else u.dtype
    if out is None:
        out = torch.empty((batch, dim, L), device=u.device, dtype=out_dtype)
    elif tuple(out.shape) != (batch, dim, L) or out.dtype != out_dtype or out.stride(-1) != 1 or out.device != u.device:
        raise RuntimeError("out must be (batch, dim, L) of the result type on u's device with contiguous rows")
    p = ScanParams()
    p.u, p.delta, p.A, p.B, p.C, p.D, p.delta_bias, p.out = (_ptr(t) for t in (u, delta, A, B, C, D, delta_bias, out))
    p.in_dtype, p.out_dtype = dtype_code(u), dtype_code(out)
    p.delta_softplus, p.delta_ratio = int(bool(delta_softplus)), ratio
    p.batch, p.dim, p.dstate, p.seqlen, p.n_groups = batch, dim, N, L, K
    p.u_batch_stride, p.u_dim_stride = u.stride(0), u.stride(1)
    p.delta_batch_stride, p.delta_dim_stride = delta.stride(0), delta.stride(1)
    p.out_batch_stride, p.out_dim_stride = out.stride(0), out.stride(1)
    p.B_batch_stride, p.B_group_stride, p.B_state_stride = B.stride(0), B.stride(1), B.stride(2)
    p.C_batch_stride, p.C_group_stride, p.C_state_stride = C.stride(0), C.stride(1), C.stride(2)
    ckpt = None
    if return_checkpoints:
        ckpt = torch.empty((batch, dim, (L + 127) // 128, N), device=u.device, dtype=torch.float32)
        p.checkpoints = ckpt.data_ptr()
    with torch.cuda.device(u.device):
        check(lib().ss2d_selective_scan_fwd(p, _stream(u)), "ss2d_selective_scan_fwd")
    return (out, ckpt) if return_checkpoints else out


def selective_scan_bwd(u, delta, A, B, C, D, delta_bias, dout, delta_softplus=False, checkpoints=None):
    """Gradients (du, ddelta, dA, dB, dC, dD, ddelta_bias) of `selective_scan_fwd` for the upstream
    gradient dout (batch, dim, L), fp32 or u.dtype; dD / ddelta_bias are None where the input was None.
    `checkpoints`: what `selective_scan_fwd(..., return_checkpoints=True)` returned (optional).
    Shapes and types of the results as selective_scan_cuda_oflex.bwd returns them
    (selective_scan_oflex.cpp:308-353)."""
    _require_cuda(u, delta, A, B, C, D, delta_bias, dout)
    batch, dim, L = u.shape
    _, K, N, _ = B.shape
    if dout.shape != u.shape:
        raise RuntimeError(f"dout must have the shape of u, got {tuple(dout.shape)}")
    if dout.dtype not in (torch.float32, u.dtype):
        raise RuntimeError("dout must be fp32 or of u's dtype")
    cont = lambda t: t if t.stride(-1) == 1 else t.contiguous()
    u, delta, B, C, dout = cont(u), cont(delta), cont(B), cont(C), cont(dout)
    A = A.contiguous().float()
    D = None if D is None else D.contiguous().float()
    delta_bias = None if delta_bias is None else delta_bias.contiguous().float()
    du = torch.empty((batch, dim, L), device=u.device, dtype=u.dtype)
    ddelta = torch.empty_like(du)
    dA = torch.empty((dim, N), device=u.device, dtype=torch.float32)
    dB = torch.empty((batch, K, N, L), device=u.device, dtype=u.dtype)
    dC = torch.empty_like(dB)
    dD = None if D is None else torch.empty(dim, device=u.device, dtype=torch.float32)
    dbias = None if delta_bias is None else torch.empty(dim, device=u.device, dtype=torch.float32)
    p = ScanBwdParams()
    p.u, p.delta, p.A, p.B, p.C, p.D, p.delta_bias, p.dout = (_ptr(t) for t in (u, delta, A, B, C, D, delta_bias, dout))
    p.du, p.ddelta, p.dA, p.dB, p.dC, p.dD, p.ddelta_bias = (_ptr(t) for t in (du, ddelta, dA, dB, dC, dD, dbias))
    p.in_dtype, p.dout_dtype = dtype_code(u), dtype_code(dout)
    ratio = dim // delta.shape[1]
    p.delta_softplus, p.delta_ratio = int(bool(delta_softplus)), ratio
    p.batch, p.dim, p.dstate, p.seqlen, p.n_groups = batch, dim, N, L, K
    p.u_batch_stride, p.u_dim_stride = u.stride(0), u.stride(1)
    p.delta_batch_stride, p.delta_dim_stride = delta.stride(0), delta.stride(1)
    p.dout_batch_stride, p.dout_dim_stride = dout.stride(0), dout.stride(1)
    p.B_batch_stride, p.B_group_stride, p.B_state_stride = B.stride(0), B.stride(1), B.stride(2)
    p.C_batch_stride, p.C_group_stride, p.C_state_stride = C.stride(0), C.stride(1), C.stride(2)
    if checkpoints is not None:
        if checkpoints.dtype != torch.float32 or tuple(checkpoints.shape) != (batch, dim, (L + 127) // 128, N) \
                or not checkpoints.is_contiguous() or checkpoints.device != u.device:
            raise RuntimeError("checkpoints must be the fp32 (batch, dim, ceil(L/128), dstate) tensor of the forward call")
        p.checkpoints = checkpoints.data_ptr()
    need = int(lib().ss2d_selective_scan_bwd_workspace_bytes(p))
    if need < 0:
        raise RuntimeError("ss2d_selective_scan_bwd_workspace_bytes: invalid or unsupported arguments")
    ws = torch.empty(max(need, 16), device=u.device, dtype=torch.uint8)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    with torch.cuda.device(u.device):
        check(lib().ss2d_selective_scan_bwd(p, _stream(u)), "ss2d_selective_scan_bwd")
    if ratio > 1:       # rows that shared a delta row: their gradients add up (selective_scan_oflex.cpp:348-352)
        ddelta = ddelta.view(batch, dim // ratio, ratio, L).float().sum(2).to(u.dtype)
        if dbias is not None:
            dbias = dbias.view(dim // ratio, ratio).sum(1)
    return du, ddelta, dA, dB, dC, dD, dbias


class SelectiveScanCuda(torch.autograd.Function):
    """Same call signature, saved tensors and gradient tuple as the reference Function
    (csms6s.py:71-109)."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, u, delta, A, B, C, D=None, delta_bias=None, delta_softplus=False, oflex=True, backend=None):
        if backend == "torch":
            raise NotImplementedError("backend='torch' is not provided: vmamba_b200 has no eager/CPU path "
                                      "(reference values come from the oracle under oracle/)")
        if backend not in (None, "oflex", "mamba", "core"):
            raise ValueError(f"unknown selective-scan backend {backend!r}")
        ctx.delta_softplus = delta_softplus
        ctx.backend = backend
        ctx.has_D, ctx.has_bias = D is not None, delta_bias is not None
        # the step states go to the backward call, as the reference's `x` does (csms6s.py:81-86)
        out, ckpt = selective_scan_fwd(u, delta, A, B, C, D, delta_bias, delta_softplus, bool(oflex), return_checkpoints=True)
        saved = [u, delta, A, B, C, ckpt] + ([D] if ctx.has_D else []) + ([delta_bias] if ctx.has_bias else [])
        ctx.save_for_backward(*saved)
        return out

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, dout, *args):
        saved = list(ctx.saved_tensors)
        u, delta, A, B, C, ckpt = saved[:6]
        rest = saved[6:]
        D = rest.pop(0) if ctx.has_D else None
        delta_bias = rest.pop(0) if ctx.has_bias else None
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        du, ddelta, dA, dB, dC, dD, dbias = selective_scan_bwd(u, delta, A, B, C, D, delta_bias, dout, ctx.delta_softplus, ckpt)
        dA = dA.to(A.dtype)
        if dD is not None:
            dD = dD.to(D.dtype)
        if dbias is not None:
            dbias = dbias.to(delta_bias.dtype)
        return du, ddelta, dA, dB, dC, dD, dbias, None, None, None


SelectiveScanOflex = SelectiveScanCuda   # name used by older revisions of the reference


def selective_scan_fn(u, delta, A, B, C, D=None, delta_bias=None, delta_softplus=True, oflex=True, backend=None):
    """Drop-in for selective_scan_fn (csms6s.py:112-126, vmamba.py:872-885)."""
    if backend == "torch":
        raise NotImplementedError("backend='torch' is not provided: vmamba_b200 has no eager/CPU path "
                                  "(reference values come from the oracle under oracle/)")
    if torch.is_grad_enabled() and any(isinstance(t, torch.Tensor) and t.requires_grad for t in (u, delta, A, B, C, D, delta_bias)):
        return SelectiveScanCuda.apply(u, delta, A, B, C, D, delta_bias, delta_softplus, oflex, backend)
    with torch.autocast("cuda", enabled=False):
        return selective_scan_fwd(u, delta, A, B, C, D, delta_bias, delta_softplus, bool(oflex))


def flops_selective_scan_fn(B=1, L=256, D=768, N=16, with_D=True, with_Z=False, with_complex=False):
    """FLOP count of one selective scan as the reference counts it (csms6s.py:136-160): nine per
    (batch, position, channel, state) plus one per element for the D skip and for a z gate."""
    assert not with_complex
    flops = 9 * B * L * D * N
    if with_D:
        flops += B * D * L
    if with_Z:
        flops += B * D * L
    return flops


def selective_scan_flop_jit(inputs, outputs, backend="prefixsum", verbose=True):
    """fvcore / torch-jit FLOP handle for the Function (csms6s.py:212-219): sizes are read from the
    traced inputs u (B, D, L) and A (D, N)."""
    if backend == "naive":
        raise NotImplementedError("the 'naive' count belongs to the reference's python loop, which this package does not provide")
    B, D, L = inputs[0].type().sizes()
    N = inputs[2].type().sizes()[1]
    return flops_selective_scan_fn(B=B, L=L, D=D, N=N, with_D=True, with_Z=False)


class _ExtShim:
    """Stand-in for the compiled module `selective_scan_cuda_oflex` (pybind11 surface of
    selective_scan_oflex.cpp:357-360): `fwd` and `bwd` with the reference's argument lists, for code
    that calls the extension directly (csms6s.py:81, 97-99; test_selective_scan.py:62)."""
    __name__ = "selective_scan_cuda_oflex"

    @staticmethod
    def fwd(u, delta, A, B, C, D=None, delta_bias=None, delta_softplus=False, nrows=1, out_float=True):
        # the reference returns its chunk states `x` here and wants them back in bwd; so does this library, with
        # its own spacing: (batch, dim, ceil(L / 128), dstate)
        out, x = selective_scan_fwd(u, delta, A, B, C, D, delta_bias, delta_softplus, bool(out_float), return_checkpoints=True)
        return [out, x]

    @staticmethod
    def bwd(u, delta, A, B, C, D, delta_bias, dout, x=None, delta_softplus=False, nrows=1):
        L, N = u.shape[-1], A.shape[1]
        ok = x is not None and x.dtype == torch.float32 and tuple(x.shape) == (u.shape[0], u.shape[1], (L + 127) // 128, N)
        return list(selective_scan_bwd(u, delta, A, B, C, D, delta_bias, dout, delta_softplus, x.contiguous() if ok else None))


selective_scan_cuda_oflex = _ExtShim()


# --------------------------------------------------------------------------------------------
# CrossScan / CrossMerge
# --------------------------------------------------------------------------------------------
def _check_flags(in_channel_first, out_channel_first, one_by_one, scans):
    if one_by_one and not (in_channel_first and out_channel_first) and scans not in (0, 1, 2):
        raise NotImplementedError("vmamba_b200: one_by_one CrossScan/CrossMerge with a channel-last side is implemented for "
                                  "scans 0, 1 and 2, the route sets the reference's GPU kernel defines "
                                  "(csm_triton.py:313-336)")
    if scans not in (0, 1, 2, 3):
        raise NotImplementedError(f"vmamba_b200: scans={scans} is not implemented")


def _plain(in_channel_first, out_channel_first, one_by_one):
    return bool(in_channel_first) and bool(out_channel_first) and not one_by_one


def cross_scan_fwd(x: torch.Tensor, scans: int = 0, in_channel_first=True, out_channel_first=True,
                   one_by_one=False) -> torch.Tensor:
    """cross_scan_fwd / cross_scan1b1_fwd of the reference (vmamba.py:41-84, 130-183).  Default flags:
    (B, C, H, W) -> (B, 4, C, H*W) through the tuned kernels; channel-last sides and one_by_one through the
    index-only kernels (`ss2d_cross_scan_ex`)."""
    _require_cuda(x)
    _check_flags(in_channel_first, out_channel_first, one_by_one, scans)
    x = x.contiguous()
    if _plain(in_channel_first, out_channel_first, one_by_one):
        if x.dim() != 4:
            raise RuntimeError("cross_scan expects a (B, C, H, W) tensor")
        B, C, H, W = x.shape
        y = torch.empty((B, 4, C, H * W), device=x.device, dtype=x.dtype)
        p = CrossParams(x.data_ptr(), y.data_ptr(), dtype_code(x), scans, B, C, H, W)
        with torch.cuda.device(x.device):
            check(lib().ss2d_cross_scan(p, _stream(x)), "ss2d_cross_scan")
        return y
    if one_by_one:
        if in_channel_first:
            B, K, C, H, W = x.shape
        else:
            B, H, W, K, C = x.shape
        if K != 4:
            raise RuntimeError("one_by_one expects (B, 4, C, H, W) or (B, H, W, 4, C)")
        if not out_channel_first:
            oshape = (B, H * W, 4, C)
        elif in_channel_first and scans == 1:
            # the reference's `x.flatten(2, 3)` for scans 1 merges C with H (vmamba.py:142-143): same shape here
            oshape = (B, 4, C * H, W)
        else:
            oshape = (B, 4, C, H * W)
    elif in_channel_first:
        B, C, H, W = x.shape
    else:
        B, H, W, C = x.shape
    if not one_by_one:
        oshape = (B, 4, C, H * W) if out_channel_first else (B, H * W, 4, C)
    y = torch.empty(oshape, device=x.device, dtype=x.dtype)
    p = CrossExParams(x.data_ptr(), y.data_ptr(), dtype_code(x), scans, int(bool(in_channel_first)),
                      int(bool(out_channel_first)), int(bool(one_by_one)), 0, B, C, H, W)
    with torch.cuda.device(x.device):
        check(lib().ss2d_cross_scan_ex(p, _stream(x)), "ss2d_cross_scan_ex")
    return y


def cross_merge_fwd(ys: torch.Tensor, scans: int = 0, in_channel_first=True, out_channel_first=True,
                    one_by_one=False) -> torch.Tensor:
    """cross_merge_fwd / cross_merge1b1_fwd of the reference (vmamba.py:87-130, 186-245).  `out_channel_first` names
    the layout of ys ((B, 4, C, H, W) or (B, H, W, 4, C)), `in_channel_first` the layout of the result ((B, C, L)
    or (B, L, C)), as there."""
    _require_cuda(ys)
    _check_flags(in_channel_first, out_channel_first, one_by_one, scans)
    ys = ys.contiguous()
    if ys.dim() != 5:
        raise RuntimeError("cross_merge expects a 5-d tensor of four routes")
    if _plain(in_channel_first, out_channel_first, one_by_one):
        B, K, C, H, W = ys.shape
        if K != 4:
            raise RuntimeError("cross_merge expects (B, 4, C, H, W)")
        y = torch.empty((B, C, H * W), device=ys.device, dtype=ys.dtype)
        p = CrossParams(ys.data_ptr(), y.data_ptr(), dtype_code(ys), scans, B, C, H, W)
        with torch.cuda.device(ys.device):
            check(lib().ss2d_cross_merge(p, _stream(ys)), "ss2d_cross_merge")
        return y
    if out_channel_first:
        B, K, C, H, W = ys.shape
    else:
        B, H, W, K, C = ys.shape
    if K != 4:
        raise RuntimeError("cross_merge expects four routes")
    if one_by_one:
        oshape = (B, 4, C, H * W) if in_channel_first else (B, H * W, 4, C)
    else:
        oshape = (B, C, H * W) if in_channel_first else (B, H * W, C)
    y = torch.empty(oshape, device=ys.device, dtype=ys.dtype)
    p = CrossExParams(ys.data_ptr(), y.data_ptr(), dtype_code(ys), scans, int(bool(in_channel_first)),
                      int(bool(out_channel_first)), int(bool(one_by_one)), 0, B, C, H, W)
    with torch.cuda.device(ys.device):
        check(lib().ss2d_cross_merge_ex(p, _stream(ys)), "ss2d_cross_merge_ex")
    return y


class CrossScanF(torch.autograd.Function):
    """CrossScanF of the reference (csm_triton.py:182-225): forward the scan, backward the merge of the same flags."""

    @staticmethod
    def forward(ctx, x, in_channel_first=True, out_channel_first=True, one_by_one=False, scans=0):
        _check_flags(in_channel_first, out_channel_first, one_by_one, scans)
        ctx.flags = (bool(in_channel_first), bool(out_channel_first), bool(one_by_one), scans)
        if one_by_one:
            if in_channel_first:
                B, _, C, H, W = x.shape
            else:
                B, H, W, _, C = x.shape
        elif in_channel_first:
            B, C, H, W = x.shape
        else:
            B, H, W, C = x.shape
        ctx.shape = (B, C, H, W)
        return cross_scan_fwd(x, scans, in_channel_first, out_channel_first, one_by_one)

    @staticmethod
    def backward(ctx, ys):
        # the adjoint of the four-route copy is the four-route sum (csm_triton.py:207-225)
        icf, ocf, obo, scans = ctx.flags
        B, C, H, W = ctx.shape
        ys = ys.contiguous().view(B, 4, C, H, W) if ocf else ys.contiguous().view(B, H, W, 4, C)
        y = cross_merge_fwd(ys, scans, icf, ocf, obo)
        if obo:
            y = y.view(B, 4, C, H, W) if icf else y.view(B, H, W, 4, C)
        else:
            y = y.view(B, C, H, W) if icf else y.view(B, H, W, C)
        return y, None, None, None, None


class CrossMergeF(torch.autograd.Function):
    """CrossMergeF of the reference (csm_triton.py:228-273): forward the merge, backward the scan of the same flags."""

    @staticmethod
    def forward(ctx, ys, in_channel_first=True, out_channel_first=True, one_by_one=False, scans=0):
        _check_flags(in_channel_first, out_channel_first, one_by_one, scans)
        ctx.flags = (bool(in_channel_first), bool(out_channel_first), bool(one_by_one), scans)
        if out_channel_first:
            B, _, C, H, W = ys.shape
        else:
            B, H, W, _, C = ys.shape
        ctx.shape = (B, C, H, W)
        return cross_merge_fwd(ys, scans, in_channel_first, out_channel_first, one_by_one)

    @staticmethod
    def backward(ctx, x):
        # the adjoint of the four-route sum is the four-route copy (csm_triton.py:248-273)
        icf, ocf, obo, scans = ctx.flags
        B, C, H, W = ctx.shape
        if obo:
            if scans == 1 and icf and ocf:      # the forward passed the maps through; so does the adjoint
                return x.contiguous().view(B, 4, C, H, W), None, None, None, None
            xin = x.contiguous().view(B, 4, C, H, W) if icf else x.contiguous().view(B, H, W, 4, C)
        else:
            xin = x.contiguous().view(B, C, H, W) if icf else x.contiguous().view(B, H, W, C)
        xs = cross_scan_fwd(xin, scans, icf, ocf, obo)
        xs = xs.view(B, 4, C, H, W) if ocf else xs.view(B, H, W, 4, C)
        return xs, None, None, None, None


# the CUDA-backed Functions stand in for the reference's Triton Functions too
CrossScanTritonF, CrossMergeTritonF = CrossScanF, CrossMergeF
CrossScan, CrossMerge = CrossScanF, CrossMergeF


def cross_scan_fn(x, in_channel_first=True, out_channel_first=True, one_by_one=False, scans=0, force_torch=False):
    """Drop-in for cross_scan_fn (vmamba.py:577-588).  `force_torch` is accepted and ignored:
    there is one implementation."""
    _check_flags(in_channel_first, out_channel_first, one_by_one, scans)
    if torch.is_grad_enabled() and x.requires_grad:
        return CrossScanF.apply(x, in_channel_first, out_channel_first, one_by_one, scans)
    return cross_scan_fwd(x, scans, in_channel_first, out_channel_first, one_by_one)


def cross_merge_fn(y, in_channel_first=True, out_channel_first=True, one_by_one=False, scans=0, force_torch=False):
    """Drop-in for cross_merge_fn (vmamba.py:591-601)."""
    _check_flags(in_channel_first, out_channel_first, one_by_one, scans)
    if torch.is_grad_enabled() and y.requires_grad:
        return CrossMergeF.apply(y, in_channel_first, out_channel_first, one_by_one, scans)
    return cross_merge_fwd(y, scans, in_channel_first, out_channel_first, one_by_one)


# --------------------------------------------------------------------------------------------
# channel-first LayerNorm (out_norm of SS2D)
# --------------------------------------------------------------------------------------------
def layer_norm_cf(y, weight=None, bias=None, eps: float = 1e-5, out_dtype=None, *,
                  add: torch.Tensor = None, add_bias: torch.Tensor = None, update: bool = False,
                  channel_major: bool = False, out_channel_major=None, normalize: bool = True) -> torch.Tensor:
    """LayerNorm over the channel axis of an fp32 map, as LayerNorm(channel_first=True)
    (vmamba.py:1078-1093); output in `out_dtype` (default fp32).

    The map is (B, D, ...) or, with `channel_major`, (D, B, ...); `out_channel_major` (default: same
    as the input) picks the layout of the result, so the call also converts between the two.
    With `add` (a map of the output dtype, input layout) and/or `add_bias` (per channel), the sum
    y + add + add_bias is what gets normalised; `y` may be None (then `add` alone is the input, e.g. a
    16-bit convolution output).  `update=True` also writes the sum back into `y` (the residual
    update of VSSBlock._forward, vmamba.py:1772/1777, fused with the next norm).
    `normalize=False` skips the normalisation: the call is then a fused add + cast + layout change."""
    _require_cuda(y, weight, bias, add, add_bias)
    if y is None:
        if add is None or update:
            raise RuntimeError("layer_norm_cf needs y or add (and y for update=True)")
    else:
        if y.dtype != torch.float32:
            if update:
                raise RuntimeError("update=True needs an fp32 residual tensor")
            y = y.float()
        if not y.is_contiguous():
            if update:
                raise RuntimeError("update=True needs a contiguous residual tensor")
            y = y.contiguous()
    ref = y if y is not None else add
    if out_channel_major is None:
        out_channel_major = channel_major
    B, D = (ref.shape[1], ref.shape[0]) if channel_major else (ref.shape[0], ref.shape[1])
    L = ref[0, 0].numel()
    rest = tuple(ref.shape[2:])
    if out_dtype is None:
        out_dtype = torch.float32 if add is None else add.dtype
    out = torch.empty(((D, B) if out_channel_major else (B, D)) + rest, device=ref.device, dtype=out_dtype)
    w = None if weight is None else weight.contiguous().float()
    b = None if bias is None else bias.contiguous().float()
    if add is not None:
        if add.shape != ref.shape:
            raise RuntimeError("add must have the shape of the normalised map")
        add = add.contiguous().to(out.dtype)
    ab = None if add_bias is None else add_bias.contiguous().float()
    p = NormParams()
    p.in_, p.add, p.add_bias = _ptr(y), _ptr(add), _ptr(ab)
    p.sum_out = y.data_ptr() if update else None
    p.weight, p.bias, p.out = _ptr(w), _ptr(b), out.data_ptr()
    if channel_major and out_channel_major:
        # images of a channel are adjacent in both maps: one run of B*L pixels per channel
        p.B, p.D, p.L = 1, D, B * L
        p.batch_stride, p.channel_stride = D * B * L, B * L
        p.out_batch_stride, p.out_channel_stride = D * B * L, B * L
    else:
        p.B, p.D, p.L = B, D, L
        p.batch_stride, p.channel_stride = (L, B * L) if channel_major else (D * L, L)
        p.out_batch_stride, p.out_channel_stride = (L, B * L) if out_channel_major else (D * L, L)
    p.io_dtype, p.eps, p.skip_norm = dtype_code(out), eps, int(not normalize)
    with torch.cuda.device(ref.device):
        check(lib().ss2d_layer_norm_cf(p, _stream(ref)), "ss2d_layer_norm_cf")
    return out


# --------------------------------------------------------------------------------------------
# elementwise producers around the core
# --------------------------------------------------------------------------------------------
_ACTS = {None: 0, "none": 0, "gelu": 1, "silu": 2}


def _bdhw(x, channel_major):
    return (x.shape[1], x.shape[0], x.shape[2], x.shape[3]) if channel_major else tuple(x.shape)


def bias_act_(x: torch.Tensor, bias=None, act="gelu", channel_major: bool = False) -> torch.Tensor:
    """In place x <- act(x + bias[channel]) on a contiguous (B, D, H, W) map ((D, B, H, W) with
    `channel_major`): the bias addition and activation of Mlp.forward (vmamba.py:1160-1163) in one pass."""
    _require_cuda(x, bias)
    if x.dim() != 4 or not x.is_contiguous():
        raise RuntimeError("bias_act_ expects a contiguous 4-d tensor")
    B, D, H, W = _bdhw(x, channel_major)
    b = None if bias is None else bias.contiguous().float()
    if b is not None and b.numel() != D:
        raise RuntimeError("bias must have one value per channel")
    if channel_major:      # all images of a channel are one contiguous run: vector width independent of the map size
        B, H, W = 1, 1, B * H * W
    p = PointwiseParams(x.data_ptr(), None, _ptr(b), x.data_ptr(), B, D, H, W, dtype_code(x), _ACTS[act], int(channel_major), 0)
    with torch.cuda.device(x.device):
        check(lib().ss2d_bias_act(p, _stream(x)), "ss2d_bias_act")
    return x


def mlp_supported(C: int, hidden: int, n_pixels: int, dtype: torch.dtype) -> bool:
    """True when `mlp_fused` takes a channel-major (C, n_pixels) map itself (the library's planner decides)."""
    if dtype not in (torch.bfloat16, torch.float16):
        return False
    from ._lib import MlpParams
    fake = 4096                                   # an aligned address; the query dereferences nothing
    p = MlpParams(fake, fake, fake, fake, fake, C, hidden, n_pixels, _DTYPES[dtype], 0)
    return int(lib().ss2d_mlp_supported(p)) == 0


def mlp_fused(x: torch.Tensor, w1: torch.Tensor, b1: torch.Tensor, w2: torch.Tensor, out=None) -> torch.Tensor:
    """fc2(gelu(fc1(x) + b1)) of Mlp.forward (vmamba.py:1151-1167) on a channel-major (C, B, H, W) map in one
    kernel on the tcgen05 tensor cores; the fc2 bias is left to the residual update that follows.
    w1: (4C, C), b1: (4C,) fp32, w2: (C, 4C)."""
    _require_cuda(x, w1, b1, w2)
    if x.dim() != 4 or not x.is_contiguous():
        raise RuntimeError("mlp_fused expects a contiguous channel-major (C, B, H, W) map")
    from ._lib import MlpParams
    C = x.shape[0]
    N = x.numel() // C
    w1 = w1.contiguous().to(x.dtype)
    w2 = w2.contiguous().to(x.dtype)
    b1 = b1.contiguous().float()
    y = torch.empty_like(x) if out is None else out
    if y.shape != x.shape or y.dtype != x.dtype or not y.is_contiguous():
        raise RuntimeError("out must be a contiguous tensor of x's shape and dtype")
    p = MlpParams(x.data_ptr(), w1.data_ptr(), b1.data_ptr(), w2.data_ptr(), y.data_ptr(), C, w1.shape[0], N, dtype_code(x), 0)
    with torch.cuda.device(x.device):
        check(lib().ss2d_mlp_fwd(p, _stream(x)), "ss2d_mlp_fwd")
    return y


def linear_supported(M: int, K: int, n_pixels: int, dtype: torch.dtype) -> bool:
    """True when `linear_cf` takes a dense (K, n_pixels) map itself (the library's planner decides)."""
    if dtype not in (torch.bfloat16, torch.float16):
        return False
    from ._lib import LinearParams
    fake = 4096                                   # an aligned address; the query dereferences nothing
    p = LinearParams(fake, fake, None, fake, M, K, n_pixels, 0, 0, _DTYPES[dtype], 0)
    return int(lib().ss2d_linear_supported(p)) == 0


def linear_cf(x: torch.Tensor, w: torch.Tensor, bias=None, out=None) -> torch.Tensor:
    """w . x (+ bias) for a channel-major map x (K, ...) of contiguous pixels: the 1x1 projection of Linear2d.forward
    (vmamba.py:1062-1075) and, with the stacked weights of the four routes, x_proj of forward_corev2 on the
    un-scanned map (vmamba.py:1536-1538), on the tcgen05 tensor cores.  w: (M, K) with M <= 256; returns (M, ...)."""
    _require_cuda(x, w, bias)
    if not x.is_contiguous():
        raise RuntimeError("linear_cf expects a contiguous channel-major map")
    from ._lib import LinearParams
    K = x.shape[0]
    N = x.numel() // K
    w = w.contiguous().to(x.dtype)
    if w.dim() != 2 or w.shape[1] != K:
        raise RuntimeError("linear_cf expects weights of shape (M, K)")
    M = w.shape[0]
    b = None if bias is None else bias.contiguous().float()
    y = torch.empty((M,) + tuple(x.shape[1:]), device=x.device, dtype=x.dtype) if out is None else out
    if y.numel() != M * N or y.dtype != x.dtype or not y.is_contiguous():
        raise RuntimeError("out must be a contiguous (M, ...) tensor of x's dtype")
    p = LinearParams(x.data_ptr(), w.data_ptr(), None if b is None else b.data_ptr(), y.data_ptr(), M, K, N, 0, 0, dtype_code(x), 0)
    with torch.cuda.device(x.device):
        check(lib().ss2d_linear_fwd(p, _stream(x)), "ss2d_linear_fwd")
    return y


def dwconv3x3_act(x: torch.Tensor, weight: torch.Tensor, bias=None, act="silu", channel_major: bool = False) -> torch.Tensor:
    """act(depthwise 3x3 convolution, padding 1) of a (B, D, H, W) map ((D, B, H, W) with
    `channel_major`): conv2d + SiLU in front of the SS2D core (vmamba.py:1582-1583).
    weight: (D, 1, 3, 3) or (D, 3, 3)."""
    _require_cuda(x, weight, bias)
    if x.dim() != 4:
        raise RuntimeError("dwconv3x3_act expects a 4-d tensor")
    x = x.contiguous()
    B, D, H, W = _bdhw(x, channel_major)
    if weight.numel() != D * 9:
        raise RuntimeError("weight must be (D, 1, 3, 3)")
    w = weight.contiguous().to(x.dtype)
    b = None if bias is None else bias.contiguous().float()
    y = torch.empty_like(x)
    p = PointwiseParams(x.data_ptr(), w.data_ptr(), _ptr(b), y.data_ptr(), B, D, H, W, dtype_code(x), _ACTS[act], int(channel_major), 0)
    with torch.cuda.device(x.device):
        check(lib().ss2d_dwconv3x3_act(p, _stream(x)), "ss2d_dwconv3x3_act")
    return y


# --------------------------------------------------------------------------------------------
# patch embedding / downsampling seam: pixel-major (B, H, W, C) maps for the library's strided
# convolutions, channel planes (C, B, H, W) for the trunk
# --------------------------------------------------------------------------------------------
def stem_supported(in_channels: int, c0: int) -> bool:
    return in_channels == 3 and c0 in (32, 48, 64)


def stem_conv_norm_act(img: torch.Tensor, weight: torch.Tensor, conv_bias=None, ln_weight=None, ln_bias=None,
                       eps: float = 1e-5) -> torch.Tensor:
    """GELU(LayerNorm2d(conv3x3 stride 2 pad 1 (img) + bias)): the first three modules of the v2 patch
    embedding (vmamba.py:1928-1942) in one kernel.  img (B, 3, H, W) -> (B, H/2, W/2, C0) PIXEL-MAJOR."""
    _require_cuda(img, weight, conv_bias, ln_weight, ln_bias)
    img = img.contiguous()
    B, Cin, H, W = img.shape
    C0 = weight.shape[0]
    if tuple(weight.shape) != (C0, Cin, 3, 3):
        raise RuntimeError("weight must be (C0, in_channels, 3, 3)")
    w = weight.contiguous().to(img.dtype)
    f32 = lambda t: None if t is None else t.contiguous().float()
    cb, lw, lb = f32(conv_bias), f32(ln_weight), f32(ln_bias)
    y = torch.empty((B, (H + 1) // 2, (W + 1) // 2, C0), device=img.device, dtype=img.dtype)
    p = StemParams(img.data_ptr(), w.data_ptr(), _ptr(cb), _ptr(lw), _ptr(lb), y.data_ptr(), B, H, W, C0, Cin,
                   dtype_code(img), _ACTS["gelu"], eps, 0)
    with torch.cuda.device(img.device):
        check(lib().ss2d_stem_conv_norm_act(p, _stream(img)), "ss2d_stem_conv_norm_act")
    return y


def pixels_norm_to_planes(rows: torch.Tensor, bias=None, ln_weight=None, ln_bias=None, eps: float = 1e-5,
                          out_dtype=torch.float32) -> torch.Tensor:
    """LayerNorm over the last axis of a pixel-major (B, H, W, C) map (+ per-channel bias first),
    written as channel planes (C, B, H, W): the LayerNorm2d behind a strided convolution
    (vmamba.py:1940, 1969) and the layout change back to the trunk in one pass."""
    _require_cuda(rows, bias, ln_weight, ln_bias)
    if rows.dim() != 4 or not rows.is_contiguous():
        raise RuntimeError("pixels_norm_to_planes expects a contiguous (B, H, W, C) tensor")
    B, H, W, C = rows.shape
    f32 = lambda t: None if t is None else t.contiguous().float()
    bb, lw, lb = f32(bias), f32(ln_weight), f32(ln_bias)
    out = torch.empty((C, B, H, W), device=rows.device, dtype=out_dtype)
    p = RelayoutParams(rows.data_ptr(), out.data_ptr(), None, _ptr(bb), _ptr(lw), _ptr(lb), None, B * H * W, C, 0,
                       dtype_code(rows), dtype_code(out), eps, 0)
    with torch.cuda.device(rows.device):
        check(lib().ss2d_pixels_norm_to_planes(p, _stream(rows)), "ss2d_pixels_norm_to_planes")
    return out


def planes_to_pixels(planes: torch.Tensor, add=None, add_bias=None, update: bool = False, out_dtype=None) -> torch.Tensor:
    """fp32 channel planes (C, B, H, W) (+ add + add_bias[channel]) -> pixel-major (B, H, W, C) in
    `out_dtype` (default: add's dtype, else fp32).  `update=True` writes the sum back into `planes`
    (the last residual addition of a stage in front of the downsampling convolution, vmamba.py:1772/1777)."""
    _require_cuda(planes, add, add_bias)
    if planes.dim() != 4 or planes.dtype != torch.float32 or not planes.is_contiguous():
        raise RuntimeError("planes_to_pixels expects a contiguous fp32 (C, B, H, W) tensor")
    C, B, H, W = planes.shape
    if out_dtype is None:
        out_dtype = add.dtype if add is not None else torch.float32
    if add is not None:
        if add.shape != planes.shape:
            raise RuntimeError("add must have the shape of the planes")
        add = add.contiguous().to(out_dtype)
    ab = None if add_bias is None else add_bias.contiguous().float()
    rows = torch.empty((B, H, W, C), device=planes.device, dtype=out_dtype)
    p = RelayoutParams(rows.data_ptr(), planes.data_ptr(), _ptr(add), _ptr(ab), None, None,
                       planes.data_ptr() if update else None, B * H * W, C, 0, dtype_code(rows), dtype_code(planes), 0.0, 0)
    with torch.cuda.device(planes.device):
        check(lib().ss2d_planes_to_pixels(p, _stream(planes)), "ss2d_planes_to_pixels")
    return rows
