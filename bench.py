#!/usr/bin/env python
"""Benchmark: VMamba-T inference throughput (img/s, 224x224, bf16, batch 128 per GPU) on the
fused SS2D core, with the roofline of the dominant kernel and a CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N > 1 is launched with torchrun (one process per GPU); each rank runs its own replica on its own
batch shard (weak scaling, no collective on the data path) and the time is the max over ranks.
`--impl reference` times the CPU oracle (the port of the reference's pure-torch path) on the host
cores instead, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MODEL = "vmamba_tiny_s1l8"
BATCH = 128            # per GPU, the batch the reference quotes its throughput on
IMG = 224
NUM_CLASSES = 1000
UNIT = "img/s"
FEATURES = False       # config 3: the dense-prediction backbone returns four feature maps instead of logits
LABELS = {"vmamba_tiny_s1l8": "VMamba-T", "vmamba_small_s2l15": "VMamba-S", "vmamba_base_s2l15": "VMamba-B"}


def metric_name() -> str:
    what = "dense-prediction backbone, four feature maps" if FEATURES else "inference"
    return f"{LABELS.get(MODEL, MODEL)} img/s @{IMG}^2 bf16 (batch {BATCH} per GPU, {what})"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower() == "active":
                    reasons.add(name)
        sm.sort()
        busy = [v for v in sm if v > 0.5 * (mx[0] if mx else 1)] or sm
        med = busy[len(busy) // 2] if busy else None
        return {"sm_mhz": med, "sm_max_mhz": mx[0] if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
def synthetic_state_dict(seed: int = 0):
    """Random init of VMamba-T in the reference's value distributions (no checkpoint can travel)."""
    from oracle import backbone_oracle as BO     # host-side generator of the synthetic weights only
    cfg = BO.CONFIGS[MODEL]
    return BO.random_state_dict(cfg["depths"], cfg["dims"], cfg["d_state"], cfg["ssm_ratio"], 4.0, NUM_CLASSES, 3, seed,
                                with_outnorm=FEATURES)


def cpu_baseline(sd, n_images: int, repeats: int = 1):
    """The oracle's VMamba-T forward on the host cores; returns (img/s, cores, description)."""
    import numpy as np
    import torch
    from oracle import backbone_oracle as BO
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    rng = np.random.default_rng(1)
    img = rng.standard_normal((n_images, 3, IMG, IMG), dtype=np.float32)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        logits = BO.vssm_logits(img, sd)
        best = min(best, time.perf_counter() - t0)
    cpu_baseline.last = (img, logits)      # kept for the parity line of the GPU arm
    return n_images / best, cores, f"{n_images} images of the {BATCH}-image batch, fp32, full VMamba-T forward, {cores} threads"


def run_reference(args):
    """`--impl reference`: the CPU oracle on this box's host cores (rank 0 only)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    sd = synthetic_state_dict(0)
    n_img = 4
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_baseline(sd, 1)
    times = []
    val = cores = desc = None
    for _ in range(max(1, min(args.steps, 3))):
        v, cores, desc = cpu_baseline(sd, n_img)
        times.append(n_img / v)
    sec = sum(times) / len(times)
    val = n_img / sec
    line = {
        "impl": "reference", "metric": metric_name(), "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": len(times),
        "warmup": min(args.warmup, 1), "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{MODEL} inference, {IMG}x{IMG}, CPU oracle (port of the reference's pure-torch path); "
                               f"each step = {n_img} images", "batch_per_step": n_img},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
def time_events(fn, iters, warmup=3):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters   # ms


def roofline_of_core(model, peak_gbs, peak_kind, batch=None, iters=20):
    """Times the dominant kernel chain alone: the stage-0 SS2D scan+merge (+LayerNorm) of VMamba-T at
    batch 128 (x 77 MB + delta 308 MB per launch: larger than L2, so every launch streams from HBM)."""
    import torch
    from vmamba_b200 import fused
    w = model.blocks[0][0].core
    B, D, H, W = batch or 128, w.d_inner, 56, 56      # the 224x224 stage-0 map, whatever the benchmark's image size
    L = H * W
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((B, D, H, W), device="cuda", generator=g).to(model.dtype)
    proj = fused.project(x, w)
    ws = torch.empty(B * D * L * 4, device="cuda", dtype=torch.uint8)
    y = torch.empty((B, D, H, W), device="cuda", dtype=model.dtype)
    ym = torch.empty((B, D, H, W), device="cuda", dtype=torch.float32)
    t_chain = time_events(lambda: fused.scan_merge_norm(x, proj, w, with_norm=True, workspace=ws, out=y), iters)
    t_scan = time_events(lambda: fused.scan_merge_norm(x, proj, w, with_norm=False, out=ym), iters)
    s = x.element_size()
    N, K = w.d_state, 4
    alg = B * L * (D * s + K * D * s + 2 * K * N * s + D * s) + 4 * (K * D * N + 2 * K * D) + 2 * 4 * D
    scan_bytes = B * L * (D * s + K * D * s + 2 * K * N * s + D * 4)
    ach = alg / (t_chain * 1e-3) / 1e9
    # DRAM bytes of the chain's two kernels: an ncu capture of this very command line at batch 128 (one launch of each
    # kernel, caches left as the previous launch left them) gave 392 MB read + 164 MB written by the scan + merge kernel
    # and 128 MB read + 72 MB written by the LayerNorm kernel, 19.6 bytes per (pixel, channel); other batch sizes are
    # scaled by their (pixel, channel) count.
    traffic = 19.6 * B * D * L if (D == 96 and s == 2) else None
    return {
        "bound": "hbm", "achieved": ach, "peak": peak_gbs, "unit": "GB/s", "frac": ach / peak_gbs, "traffic": traffic,
        "peak_kind": f"of {peak_kind}",
        "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of core_route_kernel and layer_norm_cf_kernel, "
                          "batch 128, --cache-control none; scaled by (pixel, channel) count" if traffic else None,
        "kernel": "core_route_kernel + layer_norm_cf_kernel (fused SS2D scan+merge+LayerNorm chain)",
        "workload": f"stage 0 of {MODEL} at 224x224: B={B} D={D} H=W={H} bf16",
        "algorithmic_bytes_per_launch": alg, "chain_ms": t_chain,
        "scan_merge_kernel_ms": t_scan, "scan_merge_kernel_gbs": scan_bytes / (t_scan * 1e-3) / 1e9,
        "scan_merge_kernel_bytes": scan_bytes,
    }


def mlp_leg(model, batch=None, iters=20):
    """The fused MLP kernel (tcgen05) of the first stage-0 block alone, beside the three launches it replaces."""
    import torch
    from vmamba_b200 import ops
    b = model.blocks[0][0]
    C, B = b.w1.shape[1], batch or 128
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((C, B, 56, 56), device="cuda", generator=g).to(model.dtype)
    if not ops.mlp_supported(C, b.w1.shape[0], x.numel() // C, x.dtype):
        return None

    def unfused():
        h = torch.matmul(b.w1, x.view(C, -1)).view(b.w1.shape[0], B, 56, 56)
        ops.bias_act_(h, b.b1f, "gelu", channel_major=True)
        return torch.matmul(b.w2, h.view(b.w1.shape[0], -1))
    t_f = time_events(lambda: ops.mlp_fused(x, b.w1, b.b1f, b.w2), iters)
    t_u = time_events(unfused, iters)
    flops = 4.0 * C * b.w1.shape[0] * (x.numel() // C)
    tf_peak = None
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            tf_peak = float(json.load(f)["bf16_tflops"])
    tf = flops / (t_f * 1e-3) / 1e12
    return {"kernel": "mlp_fused_kernel (fc1 + bias + GELU + fc2, tcgen05)", "workload": f"C={C} hidden={b.w1.shape[0]} pixels={x.numel() // C} bf16",
            "ms": t_f, "tflops": tf, "peak_tflops": tf_peak, "frac_of_measured_bf16_peak": (tf / tf_peak) if tf_peak else None,
            "replaced_launches_ms": t_u, "note": "bound by the GELU epilogue on the FMA pipe, not by the tensor pipe"}


def xproj_leg(model, batch=None, iters=20, stage=0):
    """The x_proj kernel (`ss2d_linear_fwd`, tcgen05) of the first block of a stage alone, beside the library GEMM on
    the same operands; bytes = x read once + the projected rows written once."""
    import torch
    from vmamba_b200 import ops
    w = model.blocks[stage][0].core
    hw = 56 >> stage
    D, B = w.d_inner, batch or 128
    M = w.wx.shape[0]
    g = torch.Generator(device="cuda").manual_seed(0)
    # several input buffers in turn, so that a launch never finds its x in L2
    nb = max(2, int(400e6 // ((D + M) * B * hw * hw * 2)) + 1)
    xs = [torch.randn((D, B * hw * hw), device="cuda", generator=g).to(model.dtype) for _ in range(nb)]
    if not ops.linear_supported(M, D, xs[0].shape[1], xs[0].dtype):
        return None
    out = torch.empty((M, xs[0].shape[1]), device="cuda", dtype=model.dtype)
    state = {"i": 0}

    def own():
        state["i"] = (state["i"] + 1) % nb
        ops.linear_cf(xs[state["i"]], w.wx, out=out)

    def library():
        state["i"] = (state["i"] + 1) % nb
        torch.matmul(w.wx, xs[state["i"]], out=out)
    t_o = time_events(own, iters * nb)
    t_l = time_events(library, iters * nb)
    peak, kind = peaks()
    by = (D + M) * xs[0].shape[1] * 2
    return {"kernel": "linear_cf_kernel (x_proj, tcgen05 + TMA)", "workload": f"M={M} K={D} pixels={xs[0].shape[1]} bf16, {nb} input buffers in turn",
            "ms": t_o, "gbs": by / t_o / 1e6, "frac_of_measured_hbm": by / t_o / 1e6 / peak, "peak_kind": kind, "library_gemm_ms": t_l,
            "note": "timed launch by launch: includes the launch gap, which a captured graph does not have"}


def op_sweep(args):
    """Operator-surface sweep (the selective-scan op alone, bf16 u/delta/B/C, fp32 state and output) over
    d_state x channels x length, plus CrossScan / CrossMerge; one JSON line per cell with the achieved
    HBM bandwidth on the op's algorithmic bytes.  Inputs are sized to `--sweep-gb` GB per cell (the
    full-size sweep uses 40 GB; the value distributions and shapes are the same)."""
    import torch
    import vmamba_b200 as vb
    peak, kind = peaks()
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(0)
    K = 4
    for N in (1, 16):
        for D in (96, 384, 768):
            for L in (196, 3136, 16384, 65536):
                Bt = max(1, int(args.sweep_gb * 1e9 / (16 * L * (D + N))))
                # drawn in bf16 directly: an fp32 draw of a 20 GB tensor would need 40 GB more for a moment
                u = torch.randn((Bt, K * D, L), device="cuda", generator=g, dtype=torch.bfloat16)
                delta = torch.randn((Bt, K * D, L), device="cuda", generator=g, dtype=torch.bfloat16)
                Bm = torch.randn((Bt, K, N, L), device="cuda", generator=g, dtype=torch.bfloat16)
                Cm = torch.randn((Bt, K, N, L), device="cuda", generator=g, dtype=torch.bfloat16)
                A = -torch.arange(1, N + 1, device="cuda", dtype=torch.float32).repeat(K * D, 1)
                Dp = torch.ones(K * D, device="cuda")
                dt = torch.exp(torch.rand(K * D, device="cuda", generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
                bias = dt + torch.log(-torch.expm1(-dt))
                out = torch.empty((Bt, K * D, L), device="cuda", dtype=torch.float32)     # one output buffer for all launches
                ms = time_events(lambda: vb.selective_scan_fwd(u, delta, A, Bm, Cm, Dp, bias, True, True, out=out), args.steps)
                del out
                nbytes = Bt * L * (K * D * (2 * 2 + 4) + 2 * K * N * 2) + 4 * (K * D * N + 2 * K * D)
                gbs = nbytes / (ms * 1e-3) / 1e9
                print(json.dumps({"op": "selective_scan_fwd", "dtype": "bf16->f32", "d_state": N, "D": D, "L": L, "batch": Bt,
                                  "ms": ms, "algorithmic_bytes": nbytes, "achieved_gbs": gbs, "frac": gbs / peak,
                                  "peak_gbs": peak, "peak_kind": f"of {kind}"}), flush=True)
                if args.sweep_gb > 8:          # the gradient cell needs four more maps of this size: small sweeps only
                    del u, delta, Bm, Cm
                    continue
                # gradients of the same cell: reads u, delta, dout (fp32), B, C; writes du, ddelta, dB, dC
                from vmamba_b200 import ops as _ops
                dout = torch.randn((Bt, K * D, L), device="cuda", generator=g)
                _, ck = _ops.selective_scan_fwd(u, delta, A, Bm, Cm, Dp, bias, True, True, return_checkpoints=True)
                ms = time_events(lambda: _ops.selective_scan_bwd(u, delta, A, Bm, Cm, Dp, bias, dout, True, ck), args.steps)
                nbytes = Bt * L * (K * D * (2 * 2 + 4 + 2 * 2) + 4 * K * N * 2) + 4 * (2 * K * D * N + 4 * K * D)
                gbs = nbytes / (ms * 1e-3) / 1e9
                print(json.dumps({"op": "selective_scan_bwd", "dtype": "bf16, dout f32", "d_state": N, "D": D, "L": L, "batch": Bt,
                                  "ms": ms, "algorithmic_bytes": nbytes, "achieved_gbs": gbs, "frac": gbs / peak,
                                  "peak_gbs": peak, "peak_kind": f"of {kind}"}), flush=True)
                del u, delta, Bm, Cm, dout
    for (D, H) in ((96, 56), (384, 14), (96, 256)):
        Bt = max(1, int(min(args.sweep_gb, 8.0) * 1e9 / (10 * D * H * H)))
        x = torch.randn((Bt, D, H, H), device="cuda", generator=g).to(torch.bfloat16)
        ms = time_events(lambda: vb.cross_scan_fwd(x, 0), args.steps)
        nb = x.numel() * 2 * 5
        print(json.dumps({"op": "cross_scan", "dtype": "bf16", "D": D, "H": H, "batch": Bt, "ms": ms, "algorithmic_bytes": nb,
                          "achieved_gbs": nb / (ms * 1e-3) / 1e9, "frac": nb / (ms * 1e-3) / 1e9 / peak}), flush=True)
        ys = torch.randn((Bt, 4, D, H, H), device="cuda", generator=g)
        ms = time_events(lambda: vb.cross_merge_fwd(ys, 0), args.steps)
        nb = ys.numel() * 4 * 5 // 4
        print(json.dumps({"op": "cross_merge", "dtype": "f32", "D": D, "H": H, "batch": Bt, "ms": ms, "algorithmic_bytes": nb,
                          "achieved_gbs": nb / (ms * 1e-3) / 1e9, "frac": nb / (ms * 1e-3) / 1e9 / peak}), flush=True)
        del x, ys


def reference_modules_leg(local: int, steps: int = 5):
    """The UNMODIFIED reference modules (the staged copy of its one-file vmamba.py) on this library's operators:
    `install()` + `enable_fused()`, eager, bf16 autocast, batch 128 - the drop-in use of the library, reported
    beside the headline.  Also the top-1 agreement measured like for like: this library's bf16 backbone against the
    reference's own pure-torch path under bf16 autocast on the same GPU, same weights, 256 synthetic images.
    Returns None where no checkout was staged (oracle/stage_ref.py)."""
    import torch
    from oracle import stage_ref              # checker-side loader of the reference's own file; not a product path
    if not stage_ref.staged("vmamba.py"):
        return None
    import vmamba_b200 as vb
    from vmamba_b200.backbone import VSSMInfer
    ref = stage_ref.load("vmamba.py", "vmamba_reference_bench")
    torch.manual_seed(0)
    m = ref.vmamba_tiny_s1l8().eval().cuda(local)
    g = torch.Generator().manual_seed(7)
    out = {"model": "vmamba.py:vmamba_tiny_s1l8 (unmodified reference modules), eager, torch.autocast bf16"}
    # ---- like-for-like top-1: reference pure-torch bf16 autocast vs this library's bf16 backbone ----
    img = torch.randn((256, 3, IMG, IMG), generator=g).cuda(local)
    orig_scan, orig_merge = ref.cross_scan_fn, ref.cross_merge_fn
    ref.cross_scan_fn = lambda *a, **k: orig_scan(*a, **{**k, "force_torch": True})
    ref.cross_merge_fn = lambda *a, **k: orig_merge(*a, **{**k, "force_torch": True})
    try:
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            want16 = torch.cat([m(img[i:i + 32]) for i in range(0, 256, 32)]).float()
        with torch.no_grad():
            want32 = torch.cat([m(img[i:i + 32]) for i in range(0, 64, 32)]).float()
    finally:
        ref.cross_scan_fn, ref.cross_merge_fn = orig_scan, orig_merge
    sd = {k: v.detach().float().cpu().numpy() for k, v in m.state_dict().items()}
    lib = VSSMInfer.from_state_dict(sd, dtype=torch.bfloat16, device=f"cuda:{local}")
    lib16 = torch.cat([lib(img[i:i + 64].to(torch.bfloat16)) for i in range(0, 256, 64)]).float()
    noise = float((want16[:64] - want32).abs().max())
    top2 = want16.topk(2, dim=1).values
    clear = (top2[:, 0] - top2[:, 1]) > 4 * noise
    agree = lib16.argmax(1) == want16.argmax(1)
    out["top1_like_for_like"] = {
        "images": 256, "raw": float(agree.float().mean()), "clear_margin_images": int(clear.sum()),
        "clear_margin_agreement": float(agree[clear].float().mean()) if int(clear.sum()) else None,
        "reference_bf16_vs_fp32_logit_noise": noise, "max_abs_logit_diff": float((lib16 - want16).abs().max()),
        "comparator": "reference CrossScanF/CrossMergeF + selective_scan_torch under torch.autocast(bf16) on this GPU"}
    del lib, lib16, want16, want32
    # ---- throughput of the reference modules on the library: surface operators, then the fused core ----
    x = img[:BATCH] if BATCH <= 256 else img
    x = torch.randn((BATCH, 3, IMG, IMG), generator=g).cuda(local)
    vb.install(ref)
    try:
        def fwd():
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                return m(x)
        out["img_s_surface_operators"] = BATCH / (time_events(fwd, steps) * 1e-3)
        out["fused_modules"] = vb.enable_fused(m)
        out["img_s_fused_core"] = BATCH / (time_events(fwd, steps) * 1e-3)
    finally:
        vb.disable_fused(m)
        vb.uninstall(ref)
    # ---- one training step of the same module on the operator surface (forward, backward through SelectiveScanCuda /
    #      CrossScanF / CrossMergeF of this library, SGD update), eager, bf16 autocast ----
    vb.install(ref)
    try:
        m.train()
        opt = torch.optim.SGD(m.parameters(), lr=1e-4)
        tb = min(BATCH, 64)
        xt = x[:tb]

        def train_step():
            opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = m(xt).float().logsumexp(1).mean()
            loss.backward()
            opt.step()
        out["train_img_s_surface_operators"] = tb / (time_events(train_step, max(3, steps // 2)) * 1e-3)
        out["train_batch"] = tb
    except Exception as e:      # the inference lines above stand on their own
        out["train_img_s_surface_operators"] = None
        out["train_error"] = f"{type(e).__name__}: {e}"[:200]
    finally:
        m.eval()
        vb.uninstall(ref)
    # ---- the same module handed to accelerate(): this library's backbone on the module's weights, eager (no graph) ----
    fast = vb.accelerate(m)
    x16 = x.to(torch.bfloat16)
    out["img_s_accelerated_module"] = BATCH / (time_events(lambda: fast(x16), steps) * 1e-3)
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    import vmamba_b200  # noqa: F401  (fails loudly if the CUDA library is missing)
    from vmamba_b200 import _lib
    from vmamba_b200.backbone import VSSMInfer
    from vmamba_b200.runner import GraphedBackbone

    global MODEL, BATCH, IMG, FEATURES
    if args.config == 2:       # VMamba-S, global batch 256 sharded over the ranks
        MODEL, BATCH, IMG = "vmamba_small_s2l15", max(1, 256 // world), 224
    elif args.config == 3:     # VMamba-B as a dense-prediction backbone: 1024 x 1024, global batch 16, four feature maps
        MODEL, BATCH, IMG, FEATURES = "vmamba_base_s2l15", max(1, 16 // world), 1024, True
    if args.model:
        MODEL = args.model
    if args.batch:
        BATCH = args.batch
    if args.img:
        IMG = args.img
    sd = synthetic_state_dict(0)
    model = VSSMInfer.from_state_dict(sd, dtype=torch.bfloat16, device=f"cuda:{local}")
    if args.roofline_only:     # the dominant kernel chain alone (small cases for profiler captures)
        peak, kind = peaks()
        print(json.dumps({"roofline": roofline_of_core(model, peak, kind, args.roofline_batch, args.steps)}), flush=True)
        return

    if args.mlp_only:          # the fused MLP kernel alone (small cases for profiler captures)
        print(json.dumps({"mlp_fused": mlp_leg(model, args.roofline_batch, args.steps)}), flush=True)
        return

    if args.xproj_only:        # the x_proj kernel alone (small cases for profiler captures)
        print(json.dumps({"xproj": xproj_leg(model, args.roofline_batch, args.steps, args.stage)}), flush=True)
        return

    if args.forward_only:      # plain (un-graphed) forwards and nothing else: the case profiler captures use
        img = torch.randn((BATCH, 3, IMG, IMG), device=f"cuda:{local}").to(torch.bfloat16)
        for _ in range(max(1, args.steps)):
            out = model(img)
        torch.cuda.synchronize()
        print(json.dumps({"forward_only": True, "batch": BATCH, "forwards": max(1, args.steps), "logits": list(out.shape)}), flush=True)
        return

    # synthetic images: N(0,1), seeded per rank, bf16 in pinned host memory
    g = torch.Generator().manual_seed(1234 + rank)
    host_img = torch.randn((BATCH, 3, IMG, IMG), generator=g).to(torch.bfloat16).pin_memory()
    dev_img = host_img.cuda(non_blocking=True)
    torch.cuda.synchronize()

    # ---- one forward captured in a CUDA graph (static input / output buffers): the package's own runner ----
    runner = GraphedBackbone(model, (BATCH, 3, IMG, IMG), dtype=torch.bfloat16, features=FEATURES)
    runner.input.copy_(dev_img)
    dev_out = runner.output
    outs = dev_out if isinstance(dev_out, (list, tuple)) else [dev_out]
    host_outs = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
    host_out = host_outs if FEATURES else host_outs[0]
    d2h_bytes = sum(o.numel() * o.element_size() for o in outs)
    launches_per_forward = runner.launches_per_forward
    runner.replay()
    torch.cuda.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, steps, warmup):
        for _ in range(warmup):
            step_fn()
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            step_fn()
        e.record()
        barrier()
        ms = s.elapsed_time(e)
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def step_device():
        runner.replay()

    # End to end through the public call: every step uploads its batch from pinned host memory (on a copy
    # stream, into one of two staging buffers, so the upload of step i+1 overlaps the forward of step i),
    # runs the forward and reads its logits back into pinned host memory.
    def step_e2e():
        runner.infer_host(host_img, host_out)

    def timed_e2e(steps, warmup):
        for _ in range(warmup):
            step_e2e()
        barrier()
        runner.fence_uploads()                 # no upload starts before the timed region does
        return timed(step_e2e, steps, 0)

    warm = max(args.warmup, 3)
    # several timed regions of exactly `steps` steps each; the median region is the one reported
    n_regions = 3 if args.steps <= 100 else 1
    sampler = ClockSampler(local).start() if rank == 0 else None
    regions_dev = [timed(step_device, args.steps, warm if i == 0 else 0) for i in range(n_regions)]
    clocks = sampler.stop() if sampler else None
    regions_e2e = [timed_e2e(args.steps, warm if i == 0 else 1) for i in range(n_regions)]
    ms_dev = sorted(regions_dev)[n_regions // 2]
    ms_e2e = sorted(regions_e2e)[n_regions // 2]

    total_imgs = BATCH * world * args.steps
    value = total_imgs / (ms_dev * 1e-3)
    e2e = total_imgs / (ms_e2e * 1e-3)

    roof = cpu = parity = refmod = mlp = None
    if rank == 0:
        peak, kind = peaks()
        roof = roofline_of_core(model, peak, kind)
        mlp = mlp_leg(model)
        if world == 1 and not args.no_cpu_baseline and MODEL == "vmamba_tiny_s1l8" and IMG == 224:
            v, cores, desc = cpu_baseline(sd, 4)
            cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc}
            # the same images through the GPU model: parity of the benchmarked path with the oracle
            import numpy as np
            img_np, ref = cpu_baseline.last
            got16 = model(torch.from_numpy(img_np).cuda().to(torch.bfloat16)).float().cpu().numpy()
            old_tf32 = torch.backends.cudnn.allow_tf32
            torch.backends.cudnn.allow_tf32 = False
            m32 = VSSMInfer.from_state_dict(sd, dtype=torch.float32, device=f"cuda:{local}")
            got32 = m32(torch.from_numpy(img_np).cuda()).cpu().numpy()
            torch.backends.cudnn.allow_tf32 = old_tf32
            del m32
            if not args.no_reference_modules:
                refmod = reference_modules_leg(local)
            den = float(np.abs(ref).max())
            parity = {"images": int(ref.shape[0]), "oracle": "oracle/backbone_oracle.vssm_logits (fp32, CPU)",
                      "max_rel_err_fp32": float(np.abs(got32 - ref).max()) / den,
                      "max_rel_err_bf16": float(np.abs(got16 - ref).max()) / den,
                      "top1_agree_fp32": int((got32.argmax(1) == ref.argmax(1)).sum()),
                      "top1_agree_bf16": int((got16.argmax(1) == ref.argmax(1)).sum())}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    act_mb = BATCH * 96 * 56 * 56 * 2 / 1e6
    line = {
        "metric": metric_name(), "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
        "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{MODEL} (" + ("VMamba-T, dims 96/192/384/768, depths 2/2/8/2, " if MODEL == "vmamba_tiny_s1l8" else "") +
                               f"v05_noz, d_state 1) backbone inference, random init, {BATCH} images of 3x{IMG}x{IMG} per GPU per step",
                   "output": "four LayerNorm'ed feature maps (strides 4, 8, 16, 32)" if FEATURES else "logits",
                   "global_batch": BATCH * world, "parallelism": f"replicas x{world}, batch-sharded, no collective",
                   "l2": f"no flush needed: one stage-0 activation is {act_mb:.0f} MB and a step streams several GB, "
                         "far more than the 126 MB L2",
                   "precision": "bf16 activations into every contraction, fp32 LayerNorm statistics, fp32 residual "
                                "stream, fp32 scan state", "cuda_graph": True,
                   "published_reference": "1686 img/s on A100, fp32 without AMP (README.md:91) - other hardware and "
                                          "precision, so vs_baseline stays null"},
        "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": host_img.numel() * 2 * world,
                "d2h_bytes_per_step": d2h_bytes * world, "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": launches_per_forward * args.steps * world,
        "gpu_launches_per_step_per_gpu": launches_per_forward,
        "clocks": clocks, "roofline": roof,
        "timed_regions": {"count": n_regions, "steps_each": args.steps, "reported": "median region",
                          "device_ms": regions_dev, "e2e_ms": regions_e2e},
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if parity is not None:
        line["parity"] = parity
    if refmod is not None:
        line["reference_modules"] = refmod
    if mlp is not None:
        line["mlp_fused"] = mlp
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-modules", action="store_true", help="skip the leg that runs the staged reference modules")
    ap.add_argument("--config", type=int, default=1, choices=[1, 2, 3, 4],
                    help="benchmark configuration: 1 VMamba-T batch 128 per GPU (default); 2 VMamba-S, global batch 256 over the "
                         "ranks; 3 VMamba-B 1024x1024 dense-prediction backbone, global batch 16 over the ranks, four feature "
                         "maps read back; 4 the operator sweep with inputs sized by the 40 GB rule (1 GPU)")
    ap.add_argument("--model", default=None, help="vmamba_tiny_s1l8 (default) | vmamba_small_s2l15 | vmamba_base_s2l15")
    ap.add_argument("--batch", type=int, default=None, help="images per GPU per step (default 128)")
    ap.add_argument("--img", type=int, default=None, help="image side (default 224)")
    ap.add_argument("--op-sweep", action="store_true", help="selective-scan / CrossScan / CrossMerge operator sweep (1 GPU)")
    ap.add_argument("--sweep-gb", type=float, default=2.0, help="input gigabytes per sweep cell")
    ap.add_argument("--roofline-only", action="store_true", help="time only the fused SS2D core chain of stage 0")
    ap.add_argument("--roofline-batch", type=int, default=None, help="batch for --roofline-only (default 128)")
    ap.add_argument("--xproj-only", action="store_true", help="time only the x_proj kernel of a block (stage: --stage, batch: --roofline-batch)")
    ap.add_argument("--stage", type=int, default=0, help="stage whose first block --xproj-only takes (0..2)")
    ap.add_argument("--mlp-only", action="store_true", help="time only the fused MLP kernel of a stage-0 block (batch: --roofline-batch)")
    ap.add_argument("--forward-only", action="store_true", help="run --steps plain forwards of the model and exit (profiler captures)")
    args = ap.parse_args()
    if args.config == 4:
        args.op_sweep, args.sweep_gb = True, 40.0
    if args.op_sweep:
        op_sweep(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
