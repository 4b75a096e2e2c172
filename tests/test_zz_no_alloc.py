"""`ss2d_core_fwd_static`: the fused SS2D core for callers that cannot allocate device memory.

Some users of the C ABI only ever hold the tensors they were given: an operator slot in a serving
runtime receives its inputs and outputs already placed and has no allocator handle; a host program
written against the ABI from a language without CUDA bindings cannot call cudaMalloc at all; a
process with a device-memory budget fixed at start-up must not grow it.  `ss2d_core_fwd` asks such a
caller for an fp32 workspace it cannot provide, so the library also ships a variant whose scratch is
a 32 MiB static device array inside the library.  This test drives both entry points through the
C ABI on the same inputs, twice in a row with different shapes (the array is shared between calls and
keeps old contents), and checks that results agree and that an oversized problem is refused before
any launch.  Collected last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def _params(vb, x, proj, w, y, workspace=None):
    """Fill ss2d_core_params by hand, exactly as a foreign caller of the C ABI would."""
    from vmamba_b200 import _lib, ops
    bc = (proj[0], proj[1])
    dl = (proj[2], proj[3])
    p = _lib.CoreParams()
    p.x = x.data_ptr()
    N = w.d_state
    for k in range(4):
        j, i = k % 2, k // 2
        p.delta[k] = dl[j].data_ptr() + i * dl[j].stride(1) * x.element_size()
        p.delta_batch_stride[k] = dl[j].stride(0)
        base = bc[j].data_ptr() + i * bc[j].stride(1) * x.element_size()
        p.Bm[k], p.Cm[k] = base, base + N * bc[j].stride(2) * x.element_size()
        p.bc_batch_stride[k] = bc[j].stride(0)
    p.A, p.Dskip, p.delta_bias = w.A.data_ptr(), w.Ds.data_ptr(), w.dt_bias.data_ptr()
    p.ln_weight, p.ln_bias = w.ln_weight.data_ptr(), w.ln_bias.data_ptr()
    p.y = y.data_ptr()
    p.B, p.D, p.H, p.W, p.N = x.shape[0], x.shape[1], x.shape[2], x.shape[3], N
    p.act_dtype, p.y_dtype = ops.dtype_code(x), ops.dtype_code(y)
    p.with_norm, p.ln_eps = 1, 1e-5
    if workspace is not None:
        p.workspace, p.workspace_bytes = workspace.data_ptr(), workspace.numel()
    return p


def _case(vb, shape, dtype, seed):
    from vmamba_b200 import fused
    Bt, D, H, W = shape
    g = torch.Generator(device="cuda").manual_seed(seed)
    R, N, K = math.ceil(D / 16), 1, 4
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g)
    dt = torch.exp(torch.rand(K, D, device="cuda", generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    w = vb.CoreWeights.build(rnd(K * (R + 2 * N), D) / math.sqrt(D), rnd(K * D, R) * R ** -0.5,
                             dt + torch.log(-torch.expm1(-dt)), 0.2 * rnd(K * D, N), 1 + 0.2 * rnd(K * D),
                             1 + 0.2 * rnd(D), 0.2 * rnd(D), d_state=N, dt_rank=R, dtype=dtype)
    x = rnd(Bt, D, H, W).to(dtype)
    with torch.autocast("cuda", enabled=False):
        proj = fused.project(x, w)
    return x, proj, w


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_entry_matches_workspace_entry(dtype):
    import vmamba_b200 as vb
    from vmamba_b200 import _lib
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    assert L.ss2d_core_static_capacity() == 8 * 1024 * 1024
    # two calls in a row; the second, smaller one must not see anything of the first in the shared array
    for shape, seed in (((3, 48, 28, 28), 1), ((2, 32, 14, 14), 2)):
        x, proj, w = _case(vb, shape, dtype, seed)
        y_ref = torch.empty(shape, device="cuda", dtype=dtype)
        y_new = torch.full(shape, float("nan"), device="cuda", dtype=dtype)
        ws = torch.empty(x.numel() * 4, device="cuda", dtype=torch.uint8)
        assert L.ss2d_core_fwd(_params(vb, x, proj, w, y_ref, ws), stream) == 0
        assert L.ss2d_core_fwd_static(_params(vb, x, proj, w, y_new), stream) == 0
        torch.cuda.synchronize()
        ref, got = y_ref.float(), y_new.float()
        assert torch.isfinite(got).all()
        err = float((got - ref).abs().max() / ref.abs().max())
        assert err <= TOL[dtype], f"{shape}: max rel err {err:.3e}"
        assert torch.equal(y_new, y_ref), "same kernels on the same inputs: results must be bit-identical"


def test_static_scratch_entry_against_the_oracle_and_without_norm():
    """The same entry point against the CPU oracle (not only against its sibling), and its `with_norm = 0` form, which
    needs no scratch at all: the merged fp32 map goes straight to y, and strided y is refused as by `ss2d_core_fwd`."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import ss2d_oracle as O
    import vmamba_b200 as vb
    from vmamba_b200 import _lib, fused
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(3)
    Bt, D, H, W, N, K = 2, 24, 12, 20, 1, 4
    R = math.ceil(D / 16)
    x = rng.standard_normal((Bt, D, H, W), dtype=np.float32)
    wx = (rng.standard_normal((K * (R + 2 * N), D), dtype=np.float32) / np.sqrt(D)).astype(np.float32)
    wdt = (rng.standard_normal((K * D, R), dtype=np.float32) * R ** -0.5).astype(np.float32)
    dt = np.exp(rng.random((K, D), dtype=np.float32) * (np.log(0.1) - np.log(1e-3)) + np.log(1e-3))
    bias = (dt + np.log(-np.expm1(-dt))).astype(np.float32)
    A_logs = (0.2 * rng.standard_normal((K * D, N))).astype(np.float32)
    Ds = (1 + 0.2 * rng.standard_normal(K * D)).astype(np.float32)
    lw, lb = (1 + 0.2 * rng.standard_normal(D)).astype(np.float32), (0.2 * rng.standard_normal(D)).astype(np.float32)
    ref, parts = O.ss2d_core(x, wx, wdt, bias, A_logs, Ds, lw, lb, d_state=N, dt_rank=R, return_parts=True)
    dev = lambda a: torch.from_numpy(a).cuda()
    w = vb.CoreWeights.build(dev(wx), dev(wdt), dev(bias), dev(A_logs), dev(Ds), dev(lw), dev(lb), d_state=N, dt_rank=R,
                             dtype=torch.float32)
    xt = dev(x)
    proj = fused.project(xt, w)
    y = torch.full((Bt, D, H, W), float("nan"), device="cuda")
    assert L.ss2d_core_fwd_static(_params(vb, xt, proj, w, y), stream) == 0
    torch.cuda.synchronize()
    assert O.max_rel_err(y.cpu().numpy(), ref) <= 1e-4
    # without the LayerNorm: fp32 merged map, no scratch involved
    ym = torch.full((Bt, D, H, W), float("nan"), device="cuda")
    p = _params(vb, xt, proj, w, ym)
    p.with_norm = 0
    assert L.ss2d_core_workspace_bytes(p) == 0
    assert L.ss2d_core_fwd_static(p, stream) == 0
    torch.cuda.synchronize()
    assert O.max_rel_err(ym.cpu().numpy(), parts["merged"]) <= 1e-4
    # a strided y cannot take the dense merged map: refused, as by ss2d_core_fwd, before any launch
    p.y_batch_stride, p.y_channel_stride = H * W, Bt * H * W
    before = _lib.launch_count()
    assert L.ss2d_core_fwd_static(p, stream) == _lib.SS2D_ENOTSUP
    assert L.ss2d_core_fwd(p, stream) == _lib.SS2D_ENOTSUP
    assert _lib.launch_count() == before


def test_static_scratch_entry_rejects_oversized_and_bad_calls():
    from vmamba_b200 import _lib
    L = _lib.lib()
    assert L.ss2d_core_fwd_static(None, None) == -1
    buf = torch.zeros(4096, device="cuda")
    p = _lib.CoreParams()
    p.x = p.A = p.Dskip = p.delta_bias = p.y = buf.data_ptr()
    for k in range(4):
        p.delta[k] = p.Bm[k] = p.Cm[k] = buf.data_ptr()
    p.B, p.D, p.H, p.W, p.N = 1, 4096, 64, 64, 1          # 16.8 M map elements > 8.4 M capacity
    p.act_dtype, p.y_dtype, p.with_norm, p.ln_eps = _lib.SS2D_BF16, _lib.SS2D_BF16, 1, 1e-5
    before = _lib.launch_count()
    rc = L.ss2d_core_fwd_static(p, torch.cuda.current_stream().cuda_stream)
    assert rc == -9
    assert b"scratch" in L.ss2d_strerror(rc)
    assert _lib.launch_count() == before, "an oversized request must be refused before any launch"
