#!/usr/bin/env python
"""Benchmark of the SAPA upsampling hot path: upsampled Mpix/s and fraction of the HBM roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype f32|bf16|f16] [--workload cfg2|cfg5a|cfg5b]
    python bench.py --impl reference ...      # the CPU path of the reference on the host cores

A step is one fused SAPA-B forward (sim -> softmax -> atn, one kernel launch) over one batch of seeded
synthetic tensors.  Default workload ``cfg2``: B=8, C=256, 64x64 -> 128x128, d=64, K=5, s=2 per GPU
(batch-sharded, weak scaling: every rank runs the same per-GPU batch, no collective on the data path).
One pixel = one high-res output location across all C channels: Mpix = B*sH*sW / 1e6.

Prints ONE JSON line (rank 0).  ``value`` is measured with inputs resident in HBM; ``e2e`` goes through
the public Python op with pinned host buffers, host->device and device->host copies inside the timed
region.  ``roofline.achieved`` = algorithmic bytes per launch (every input read once + the output written
once, the attention map not counted) / measured launch duration.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: per-GPU shapes at N = 1 (cfg5* are split across ranks: strong scaling)
    "cfg2": dict(B=8, d=64, C=256, H=64, W=64, K=5, s=2, scaling="weak", shard="batch"),
    "cfg5a": dict(B=64, d=64, C=256, H=128, W=128, K=5, s=2, scaling="strong", shard="batch"),
    "cfg5b": dict(B=1, d=64, C=256, H=1024, W=1024, K=5, s=2, scaling="strong", shard="rows"),
}
DTYPES = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
L2_BYTES = 126 * 1024 * 1024
FALLBACK_HBM_GBS = 6650.0
# one metric string for both arms (the GPU kernels and --impl reference): the ratio between the arms is only defined
# when they measure the same thing on the same workload
METRIC = "upsampled Mpix/s (SAPA-B forward: sim -> softmax -> atn)"

def ncu_traffic(dtype_name, kernels):
    """dram__bytes_read.sum + dram__bytes_write.sum of one fused-forward launch at cfg2, from the tracked summary of an
    ncu capture (``profiles/fused_fwd_cfg2_traffic.json``); None when there is no capture for this element type or when the
    capture was made with another kernel than the one that just ran."""
    try:
        with open(os.path.join(ROOT, "profiles", "fused_fwd_cfg2_traffic.json")) as f:
            entry = json.load(f).get(dtype_name)
    except Exception:
        return None
    if not entry or entry.get("kernel") not in kernels:
        return None
    return int(entry["dram_bytes_read"]) + int(entry["dram_bytes_write"])


def algorithmic_bytes(w, esize):
    hi, lo = w["s"] * w["H"] * w["s"] * w["W"], w["H"] * w["W"]
    return (w["B"] * w["d"] * hi + w["B"] * w["d"] * lo + w["B"] * w["C"] * lo + w["B"] * w["C"] * hi) * esize


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler(threading.Thread):
    """Polls SM clock and throttle reasons through NVML (read-only) while the GPU is under load."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag, self.max_mhz, self.error = index, [], threading.Event(), None, None

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            try:      # NVML order can differ from CUDA order: look the device up by UUID
                h = pynvml.nvmlDeviceGetHandleByUUID("GPU-" + str(torch.cuda.get_device_properties(self.index).uuid))
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            while not self.stop_flag.is_set():
                try:
                    reasons = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    reasons = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                self.samples.append((time.perf_counter(), pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM), reasons))
                time.sleep(0.005)
        except Exception as exc:  # NVML missing: report it, do not fail the run
            self.error = repr(exc)

    def summary(self, t0, t1):
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        window = "timed region"
        if len(inside) < 3:
            inside, window = list(self.samples), "warm-up + timed region + identical trailing load"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0, "error": self.error}
        mhz = sorted(s[1] for s in inside)
        seen = set()
        for s in inside:
            for bit, name in self.REASONS.items():
                if s[2] & bit:
                    seen.add(name)
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(seen),
                "samples": len(inside), "window": window}


def make_inputs(w, dtype, device, seed, pinned=False):
    g = torch.Generator().manual_seed(seed)
    s = w["s"]
    shapes = dict(q=(w["B"], w["d"], s * w["H"], s * w["W"]), k=(w["B"], w["d"], w["H"], w["W"]),
                  v=(w["B"], w["C"], w["H"], w["W"]))
    out = {}
    for name, shape in shapes.items():
        t = torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype)
        out[name] = t.pin_memory() if pinned else t.to(device)
    return out


# ------------------------------------------------------------------ CPU path of the reference (oracle port)

def cpu_pass(w, nb, which, tensors):
    """One forward of the reference's CPU formulation on ``nb`` images; returns seconds."""
    from oracle import c_oracle, unfold_port
    q, k, v = (tensors[n][:nb] for n in ("q", "k", "v"))
    t0 = time.perf_counter()
    if which == "unfold":
        with torch.no_grad():
            unfold_port.sapa(q, k, v, w["K"], w["s"])
    else:
        c_oracle.sapa_forward(q.numpy(), k.numpy(), v.numpy(), w["K"], w["s"])
    return time.perf_counter() - t0


def cpu_baseline(w, budget_s=12.0):
    """Times both CPU restatements on the full per-GPU batch for about ``budget_s`` seconds each at most and
    reports the faster one.  float32, all host threads."""
    from oracle import c_oracle
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    c_oracle.set_num_threads(cores)
    tensors = make_inputs(w, torch.float32, "cpu", 0)
    nb = min(w["B"], 8)
    best = {}
    for which in ("unfold", "c"):
        cpu_pass(w, 1, which, tensors)                      # warm-up on one image
        times, spent = [], 0.0
        while spent < budget_s / 2 and len(times) < 5:
            t = cpu_pass(w, nb, which, tensors)
            times.append(t)
            spent += t
        best[which] = min(times)
    which = min(best, key=best.get)
    pix = nb * w["s"] * w["H"] * w["s"] * w["W"]
    threads = torch.get_num_threads() if which == "unfold" else c_oracle.num_threads()
    return {"value": pix / best[which] / 1e6, "unit": "Mpix/s", "cores": threads, "kind": "port",
            "sample": f"{nb} of {w['B']} images of the workload, float32, best of {len(times)} passes; "
                      f"unfold/einsum port {best['unfold'] * 1e3:.0f} ms, scalar C port (OpenMP) {best['c'] * 1e3:.0f} ms, "
                      f"faster one reported ({which}); host has {cores} logical cores"}


def run_reference(args, w):
    """--impl reference: the reference's CPU path (oracle port) on the host cores; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import c_oracle
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    c_oracle.set_num_threads(cores)
    tensors = make_inputs(w, torch.float32, "cpu", 0)
    # pick the faster restatement and a per-step sample that keeps the whole run within ~2 minutes
    t1 = {which: min(cpu_pass(w, 1, which, tensors) for _ in range(2)) for which in ("unfold", "c")}
    which = min(t1, key=t1.get)
    total_steps = args.steps + args.warmup
    nb = max(1, min(w["B"], int(120.0 / max(t1[which] * total_steps, 1e-9))))
    for _ in range(args.warmup):
        cpu_pass(w, nb, which, tensors)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pass(w, nb, which, tensors)
    dt = time.perf_counter() - t0
    pix = nb * w["s"] * w["H"] * w["s"] * w["W"]
    value = pix * args.steps / dt / 1e6
    threads = torch.get_num_threads() if which == "unfold" else c_oracle.num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": value,
        "unit": "Mpix/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": w["scaling"], "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config_dict(args, w),
        "note": "CPU path of the reference (F.unfold/einsum formulation or scalar C port, whichever is faster on this host)",
        "cpu_baseline": {"value": value, "unit": "Mpix/s", "cores": threads, "kind": "port",
                         "sample": f"each step = {nb} of {w['B']} images, float32, restatement '{which}'"},
        "e2e": {"value": value, "unit": "Mpix/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def config_dict(args, w):
    """The workload, identical in both arms."""
    return {"workload": f"{args.workload}: SAPA-B forward, B={w['B']} per GPU" if w["scaling"] == "weak"
            else f"{args.workload}: SAPA-B forward, B={w['B']} total ({w['shard']}-sharded)",
            "B": w["B"], "C": w["C"], "d": w["d"], "low_res": [w["H"], w["W"]],
            "high_res": [w["s"] * w["H"], w["s"] * w["W"]], "kernel_size": w["K"], "scale": w["s"],
            "sharding": w["shard"],
            "l2": "inputs and outputs rotate over buffer sets larger than the 126 MB L2 (GPU arm); the CPU arm "
                  "streams a batch far larger than the host caches"}


# ------------------------------------------------------------------ the reference's own CUDA extensions (GPU baseline)

def reference_cuda_ext_times(wl, device, time_path):
    """Device time of the UNMODIFIED reference extensions (``oracle/_ref``: qk_ext, av_ext, dqk, dav) on the cfg2 /
    cfg3 shapes in float32, called the way the reference's autograd Functions call them (sapa/sapa/sapa_func.py:24-26,
    44-46, 69-71, 89-91; deformsapa/deformsapa/deform_func.py), including their zero-filled outputs.  Outside every timed
    region of this library; reported next to it as the GPU baseline."""
    path = os.path.join(ROOT, "oracle", "_ref")
    names = ("qk_ext", "av_ext", "dqk", "dav")
    if not all(os.path.exists(os.path.join(path, n + ".so")) for n in names):
        return {"unavailable": "oracle/_ref is not built (python oracle/build_ref.py <reference checkout>)"}
    import importlib
    if path not in sys.path:
        sys.path.append(path)
    qk_ext, av_ext, dqk, dav = (importlib.import_module(n) for n in names)
    B, d, C, H, W, K, s = wl["B"], wl["d"], wl["C"], wl["H"], wl["W"], wl["K"], wl["s"]
    t = make_inputs(wl, torch.float32, device, seed=901)
    q, k, v = t["q"], t["k"], t["v"]
    go = torch.randn(B, C, s * H, s * W, device=device)
    state = {}

    def fwd():
        sim = q.new_zeros((B, K * K, s * H, s * W))
        qk_ext.forward(k, q, K, s, sim)
        attn = torch.softmax(sim, dim=1)
        out = v.new_zeros((B, C, s * H, s * W))
        av_ext.forward(v, attn, K, s, out)
        state["attn"] = attn

    def bwd():
        attn = state["attn"]
        gv, ga = torch.zeros_like(v), torch.zeros_like(attn)
        av_ext.backward(go, v, attn, K, s, gv, ga)
        gs = attn * (ga - (attn * ga).sum(dim=1, keepdim=True))
        gk, gq = torch.zeros_like(k), torch.zeros_like(q)
        qk_ext.backward(gs, k, q, K, s, gk, gq)

    G_, P_ = 4, 9
    off = torch.randn(B, G_ * P_ * 2, s * H, s * W, device=device) * 0.5

    def dfwd():
        sim = q.new_zeros((B, G_, P_, s * H, s * W))
        dqk.forward(q, k, off, P_, s, G_, sim)
        attn = torch.softmax(sim, dim=2)
        out = v.new_zeros((B, C, s * H, s * W))
        dav.forward(attn, v, off, P_, s, G_, out)

    pix = B * s * H * s * W
    res = {}
    for name, fn, steps in (("sapa_b_forward", fwd, 5), ("sapa_b_backward", bwd, 3), ("sapa_d_forward", dfwd, 3)):
        ms = time_path(fn, steps, warm=2)
        res[name] = {"ms": ms, "mpix_per_s": pix / (ms * 1e-3) / 1e6}
    res["note"] = "unmodified reference kernels compiled for sm_100a, float32, legacy default stream, same shapes"
    return res


# ------------------------------------------------------------------ BASELINE config 5 (strong scaling over the ranks)

def measure_config5(name, world, rank, device, dist, steps=10, warm=3):
    """SAPA-B fused forward in bfloat16 on the whole of config 5a (B=64, 128^2 -> 256^2, batch-sharded) or 5b (one
    1024^2 -> 2048^2 image in row slabs with a 2-row halo exchange) split over the ranks of this run; at N = 1 the whole
    workload runs on one GPU.  Inputs (1.2 GB) and output (2.1 GB) are far larger than L2.  Device time by CUDA events
    around `steps` steps between barriers, max over ranks."""
    import sapa_b200
    from sapa_b200 import sharding
    w = dict(WORKLOADS[name])
    K, s, dtype = w["K"], w["s"], torch.bfloat16
    wl = dict(w)
    if world > 1:
        if w["shard"] == "batch":
            sl = sharding.batch_slice(w["B"], world, rank)
            wl["B"] = sl.stop - sl.start
        else:
            sl = sharding.row_slice(w["H"], world, rank)
            wl["H"] = sl.stop - sl.start
    gen = torch.Generator(device=device).manual_seed(50 + rank)       # 1.2 G elements: drawn on the device
    shapes = dict(q=(wl["B"], wl["d"], s * wl["H"], s * wl["W"]), k=(wl["B"], wl["d"], wl["H"], wl["W"]),
                  v=(wl["B"], wl["C"], wl["H"], wl["W"]))
    t = {n: torch.randn(*sh, generator=gen, device=device, dtype=dtype) for n, sh in shapes.items()}
    out = torch.empty((wl["B"], wl["C"], s * wl["H"], s * wl["W"]), dtype=dtype, device=device)
    code = sapa_b200._lib.dtype_code(t["q"])
    slab = None
    if w["shard"] == "rows" and world > 1:
        slab = sharding.RowSlab(wl["B"], wl["d"], wl["C"], wl["H"], wl["W"], dtype, device, K, s)
        slab.key.copy_(t["k"])
        slab.value.copy_(t["v"])

    def step():
        if slab is not None:
            slab.forward(t["q"], out)
        else:
            sapa_b200._lib.call("sapa_fused_forward", device, t["q"], t["k"], t["v"], out, None, wl["B"], wl["d"], wl["C"],
                                wl["H"], wl["W"], K, s, code)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warm):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        tt = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    pix = w["B"] * s * w["H"] * s * w["W"]
    return {"mpix_per_s": pix / (ms * 1e-3) / 1e6, "ms_per_step": ms, "steps": steps, "dtype": "bf16", "n_gpus": world,
            "sharding": w["shard"], "scaling": "strong",
            "workload": f"{name}: B={w['B']}, C={w['C']}, d={w['d']}, {w['H']}x{w['W']} -> {s * w['H']}x{s * w['W']}"}


def measure_deform_rows(world, rank, device, dist, steps=5, warm=3):
    """SAPA-D fused forward, float32, on ONE 512^2 -> 1024^2 image (C=256, d=64, 4 groups x 9 points, offsets ~
    N(0, 0.5^2)) split into row slabs over the ranks of this run (`sharding.sapa_deform_row_sharded`: the halo depth is
    measured from the offsets at every step - a device reduction, a MAX all-reduce and a host read - then the halo rows of
    key / value travel to the neighbours and the padded slab runs as an image of its own).  At N = 1 the whole image runs
    through `deform_sapa_fused`.  Strong scaling; device time by CUDA events, max over ranks."""
    import sapa_b200
    from sapa_b200 import sharding
    B, C, d, H, W, G, P, s = 1, 256, 64, 512, 512, 4, 9, 2
    sl = sharding.row_slice(H, world, rank)
    Hl = sl.stop - sl.start
    gen = torch.Generator(device=device).manual_seed(70 + rank)
    q = torch.randn(B, d, s * Hl, s * W, generator=gen, device=device)
    k = torch.randn(B, d, Hl, W, generator=gen, device=device)
    v = torch.randn(B, C, Hl, W, generator=gen, device=device)
    off = 0.5 * torch.randn(B, 2 * G * P, s * Hl, s * W, generator=gen, device=device)
    halo = sharding.deform_halo_rows(off, local_rows=Hl) if world > 1 else None

    def step():
        with torch.no_grad():
            if world > 1:
                return sharding.sapa_deform_row_sharded(q, k, v, off, P, s, G)      # measures the halo depth itself
            return sapa_b200.deform_sapa_fused(q, k, v, off, P, s, G)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        for _ in range(warm):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        t = e0.elapsed_time(e1) / steps
        if world > 1:
            tt = torch.tensor([t], device=device, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = float(tt.item())
        return t

    ms_measured = timed(step)
    ms = ms_measured
    if world > 1:
        # resident padded key / value and a halo depth known beforehand (offsets bounded by the caller): nothing but the
        # halo rows moves and no host read happens inside the step
        del k, v
        slab = sharding.DeformRowSlab(B, d, C, Hl, W, max(halo, 2), device, P, G)
        gen2 = torch.Generator(device=device).manual_seed(70 + rank)
        slab.key.copy_(torch.randn(B, d, Hl, W, generator=gen2, device=device))
        slab.value.copy_(torch.randn(B, C, Hl, W, generator=gen2, device=device))
        out = torch.empty(B, C, s * Hl, s * W, device=device)
        ms = timed(lambda: slab.forward(q, off, halo=halo, out=out))
    pix = B * s * H * s * W
    return {"mpix_per_s": pix / (ms * 1e-3) / 1e6, "ms_per_step": ms, "steps": steps, "dtype": "f32", "n_gpus": world,
            "sharding": "rows", "scaling": "strong", "halo_rows": halo,
            "ms_per_step_halo_measured_every_step": ms_measured,
            "workload": f"SAPA-D fused forward: B={B}, C={C}, d={d}, groups={G}, points={P}, {H}x{W} -> {s * H}x{s * W}"}


# ------------------------------------------------------------------ GPU arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=200)
    ap.add_argument("--impl", default="sapa_b200", choices=["sapa_b200", "reference"])
    ap.add_argument("--dtype", default="f32", choices=list(DTYPES))
    ap.add_argument("--workload", default="cfg2", choices=list(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the additional (non-headline) measurements")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every step from Python instead of replaying a CUDA graph of one launch per buffer set")
    ap.add_argument("--only-path", default=None, choices=["backward", "deform"],
                    help="N = 1: run only the SAPA-B fused backward or the SAPA-D fused forward at the cfg2 shapes "
                         "(warm-up + --steps launches) and print a short JSON line; meant for profiler captures")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    w = dict(WORKLOADS[args.workload])

    if args.impl == "reference":
        run_reference(args, w)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the SAPA kernels have no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    import sapa_b200
    from sapa_b200 import sharding
    from sapa_b200.functions import fused_forward_raw

    dtype = DTYPES[args.dtype]
    esize = torch.empty((), dtype=dtype).element_size()
    K, s = w["K"], w["s"]

    # per-rank share of the workload
    wl = dict(w)
    halo = (0, 0)
    if w["scaling"] == "strong" and world > 1:
        if w["shard"] == "batch":
            sl = sharding.batch_slice(w["B"], world, rank)
            wl["B"] = sl.stop - sl.start
        else:
            sl = sharding.row_slice(w["H"], world, rank)
            wl["H"] = sl.stop - sl.start
    bytes_per_launch = algorithmic_bytes(wl, esize)
    pix_per_step_rank = wl["B"] * s * wl["H"] * s * wl["W"]

    if args.only_path is not None:
        assert world == 1, "--only-path is a single-GPU run"
        t = make_inputs(wl, dtype, device, seed=900)
        hi_px = s * wl["H"] * s * wl["W"]
        if args.only_path == "backward":
            g_out = torch.randn(wl["B"], wl["C"], s * wl["H"], s * wl["W"], device=device).to(dtype)
            _, attn_b = fused_forward_raw(t["q"], t["k"], t["v"], K, s, True)
            code = sapa_b200._lib.dtype_code(t["q"])
            gq, gk, gv = torch.empty_like(t["q"]), torch.empty_like(t["k"]), torch.empty_like(t["v"])
            nb = sapa_b200._lib.fused_backward_workspace(wl["B"], wl["H"], wl["W"], K, s, code)
            ws = torch.empty(nb, dtype=torch.uint8, device=device)

            def run_path():
                sapa_b200._lib.call("sapa_fused_backward", device, g_out, t["q"], t["k"], t["v"], attn_b, gq, gk, gv, ws, nb,
                                    wl["B"], wl["d"], wl["C"], wl["H"], wl["W"], K, s, code)
            launches = 3
        else:
            off = (torch.randn(wl["B"], 4 * 9 * 2, s * wl["H"], s * wl["W"], device=device) * 0.5).to(dtype)

            def run_path():
                sapa_b200.deform_sapa_fused(t["q"], t["k"], t["v"], off, 9, s, 4)
            launches = 1
        for _ in range(max(3, args.warmup)):
            run_path()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            run_path()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        print(json.dumps({"path": args.only_path, "dtype": args.dtype, "ms_per_step": ms, "steps": args.steps,
                          "mpix_per_s": wl["B"] * hi_px / (ms * 1e-3) / 1e6, "gpu_launches": launches * args.steps,
                          "l2": "same buffers every step (not flushed): for profiler captures, not a bench value"}), flush=True)
        return

    # rotating buffer sets so that no input is L2-resident from the previous iteration
    nsets = max(2, min(8, -(-3 * L2_BYTES // bytes_per_launch) + 1))
    sets = []
    for i in range(nsets):
        t = make_inputs(wl, dtype, device, seed=rank * 1000 + i)
        t["out"] = torch.empty((wl["B"], wl["C"], s * wl["H"], s * wl["W"]), dtype=dtype, device=device)
        sets.append(t)

    row_sharded = w["shard"] == "rows" and world > 1
    if row_sharded:       # key / value live in padded slabs (sharding.RowSlab); only the halo rows move per step
        for t in sets:
            t["slab"] = sharding.RowSlab(wl["B"], wl["d"], wl["C"], wl["H"], wl["W"], dtype, device, K, s)
            t["slab"].key.copy_(t["k"])
            t["slab"].value.copy_(t["v"])
            del t["k"], t["v"]

    def step(i):
        t = sets[i % nsets]
        if row_sharded:   # halo exchange (NCCL send/recv over NVLink) under the interior rows, then the border bands
            t["slab"].forward(t["q"], t["out"])
        else:
            sapa_b200._lib.call("sapa_fused_forward", device, t["q"], t["k"], t["v"], t["out"], None, wl["B"], wl["d"],
                                wl["C"], wl["H"], wl["W"], K, s, sapa_b200._lib.dtype_code(t["q"]))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # The timed loop replays a CUDA graph that holds one launch per buffer set (the launches and their order are the
    # same as in the eager loop; only the per-launch host work disappears).  Row-sharded steps contain an NCCL
    # exchange and stay eager; any failure to capture falls back to the eager loop.
    graph = None
    if not row_sharded and not args.no_graph:
        try:
            for i in range(nsets):
                step(i)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(nsets):
                    step(i)
            torch.cuda.synchronize()
        except Exception as exc:          # noqa: BLE001 - the eager loop measures the same thing
            print(f"bench: CUDA graph capture failed ({exc}); using the eager loop", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

    def run_steps(n):
        if graph is None:
            for i in range(n):
                step(i)
            return
        full, rest = divmod(n, nsets)
        for _ in range(full):
            graph.replay()
        for i in range(rest):
            step(i)

    step(0)
    kernels_per_step = sapa_b200._lib.last_kernels()     # which kernel the entry point chose (host-side record)
    sampler = ClockSampler(local)
    sampler.start()
    run_steps(args.warmup)
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.perf_counter()
    start.record()
    run_steps(args.steps)
    end.record()
    barrier()
    t_wall1 = time.perf_counter()
    elapsed_ms = start.elapsed_time(end)
    if world > 1:
        tt = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        elapsed_ms = float(tt.item())
        pp = torch.tensor([pix_per_step_rank], device=device, dtype=torch.float64)
        dist.all_reduce(pp, op=dist.ReduceOp.SUM)
        pix_per_step = float(pp.item())
    else:
        pix_per_step = float(pix_per_step_rank)
    # A timed region shorter than a few clock samples: run the identical load a little longer, untimed, only so that
    # the clocks can be sampled.  The decision and the number of extra steps derive from the max-reduced time, so
    # every rank takes the same path (a row-sharded step contains an exchange with the neighbouring ranks).
    if elapsed_ms < 40.0:
        extra = min(20000, int(300.0 / max(elapsed_ms / args.steps, 1e-3)) + 1)
        for i in range(0, extra, 64):
            run_steps(min(64, extra - i))
            torch.cuda.synchronize()
        barrier()
    sampler.stop_flag.set()
    sampler.join(timeout=2)
    clocks = sampler.summary(t_wall0, t_wall1)

    ms_per_step = elapsed_ms / args.steps
    value = pix_per_step / (ms_per_step * 1e-3) / 1e6

    # ---- the same kernel-only measurement for the other element types at the same shapes (not the headline; N = 1 only) ----
    other = {}
    if world == 1 and not args.no_extra and args.workload == "cfg2":
        for name in [n for n in DTYPES if n != args.dtype]:
            odt = DTYPES[name]
            osize = torch.empty((), dtype=odt).element_size()
            obytes = algorithmic_bytes(wl, osize)
            on = max(2, min(8, -(-3 * L2_BYTES // obytes) + 1))
            osets = []
            for i in range(on):
                t = make_inputs(wl, odt, device, seed=500 + i)
                t["out"] = torch.empty((wl["B"], wl["C"], s * wl["H"], s * wl["W"]), dtype=odt, device=device)
                osets.append(t)
            code = sapa_b200._lib.dtype_code(osets[0]["q"])

            def ostep(i):
                t = osets[i % on]
                sapa_b200._lib.call("sapa_fused_forward", device, t["q"], t["k"], t["v"], t["out"], None, wl["B"], wl["d"],
                                    wl["C"], wl["H"], wl["W"], K, s, code)
            osteps = max(3, min(args.steps, 300))
            for i in range(max(3, min(args.warmup, 20))):
                ostep(i)
            torch.cuda.synchronize()
            o0, o1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            o0.record()
            for i in range(osteps):
                ostep(i)
            o1.record()
            torch.cuda.synchronize()
            oms = o0.elapsed_time(o1) / osteps
            other[name] = {"value": pix_per_step_rank / (oms * 1e-3) / 1e6, "unit": "Mpix/s", "ms_per_step": oms, "steps": osteps,
                           "roofline_frac": obytes / (oms * 1e-3) / 1e9 / measured_peak()[0],
                           "algorithmic_bytes_per_launch": obytes}
            del osets

    # ---- the rest of the path at the same shapes: SAPA-B fused backward and SAPA-D fused forward (kernel time only) ----
    paths = {}
    if world == 1 and not args.no_extra and args.workload == "cfg2":
        peak_gbs = measured_peak()[0]

        def time_path(fn, steps, warm=5):
            for _ in range(warm):
                fn()
            torch.cuda.synchronize()
            flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=device)   # L2 flushed between iterations
            times = []
            for _ in range(steps):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            times.sort()
            return times[len(times) // 2]

        t = make_inputs(wl, dtype, device, seed=900)
        B_, d_, C_, H_, W_ = wl["B"], wl["d"], wl["C"], wl["H"], wl["W"]
        hi = s * H_ * s * W_
        g_out = torch.randn(B_, C_, s * H_, s * W_, device=device).to(dtype)
        out_b, attn_b = fused_forward_raw(t["q"], t["k"], t["v"], K, s, True)
        code = sapa_b200._lib.dtype_code(t["q"])
        gq, gk, gv = torch.empty_like(t["q"]), torch.empty_like(t["k"]), torch.empty_like(t["v"])
        nb = sapa_b200._lib.fused_backward_workspace(B_, H_, W_, K, s, code)
        ws = torch.empty(nb, dtype=torch.uint8, device=device)
        ms_b = time_path(lambda: sapa_b200._lib.call("sapa_fused_backward", device, g_out, t["q"], t["k"], t["v"], attn_b, gq, gk, gv,
                                                     ws, nb, B_, d_, C_, H_, W_, K, s, code), 20)
        # reads dOut, V, Q, K and the saved attention map; writes dV, dQ, dK
        bytes_b = (B_ * C_ * hi + B_ * C_ * H_ * W_ + B_ * d_ * hi + B_ * d_ * H_ * W_ + B_ * K * K * hi
                   + B_ * C_ * H_ * W_ + B_ * d_ * hi + B_ * d_ * H_ * W_) * esize
        paths["sapa_b_fused_backward"] = {"ms": ms_b, "launches": 3, "algorithmic_bytes": bytes_b,
                                          "achieved_gbs": bytes_b / (ms_b * 1e-3) / 1e9, "roofline_frac": bytes_b / (ms_b * 1e-3) / 1e9 / peak_gbs,
                                          "mpix_per_s": pix_per_step_rank / (ms_b * 1e-3) / 1e6}
        del out_b, gq, gk, gv, ws
        # the same forward on channels-last tensors (one warp per pixel, no tiles): same algorithmic bytes
        ql, kl, vl = (x.permute(0, 2, 3, 1).contiguous() for x in (t["q"], t["k"], t["v"]))
        with torch.no_grad():
            ms_n = time_path(lambda: sapa_b200.sapa_fused_nhwc(ql, kl, vl, K, s), 10)
        abytes = algorithmic_bytes(wl, esize)
        paths["sapa_b_fused_forward_channels_last"] = {"ms": ms_n, "launches": 1, "algorithmic_bytes": abytes,
                                                       "achieved_gbs": abytes / (ms_n * 1e-3) / 1e9,
                                                       "roofline_frac": abytes / (ms_n * 1e-3) / 1e9 / peak_gbs,
                                                       "mpix_per_s": pix_per_step_rank / (ms_n * 1e-3) / 1e6,
                                                       "kernels": sapa_b200._lib.last_kernels()}
        del ql, kl, vl
        # SAPA-D, config 3: 4 groups, 9 points, offsets ~ N(0, 0.5^2), q/k channels = d in total
        G_, P_ = 4, 9
        off = (torch.randn(B_, G_ * P_ * 2, s * H_, s * W_, device=device) * 0.5).to(dtype)
        ms_d = time_path(lambda: sapa_b200.deform_sapa_fused(t["q"], t["k"], t["v"], off, P_, s, G_), 10)
        bytes_d = (B_ * d_ * hi + B_ * d_ * H_ * W_ + 2 * B_ * G_ * P_ * hi + B_ * C_ * H_ * W_ + B_ * C_ * hi) * esize
        paths["sapa_d_fused_forward"] = {"ms": ms_d, "launches": 1, "algorithmic_bytes": bytes_d,
                                         "achieved_gbs": bytes_d / (ms_d * 1e-3) / 1e9, "roofline_frac": bytes_d / (ms_d * 1e-3) / 1e9 / peak_gbs,
                                         "mpix_per_s": pix_per_step_rank / (ms_d * 1e-3) / 1e6,
                                         "config": {"groups": G_, "points": P_, "offset_sigma": 0.5}}
        # SAPA-D fused backward at the same shapes (one kernel: both scatters, softmax gradient, summed offset gradient)
        qd, kd, vd, od = (x.detach().clone().requires_grad_() for x in (t["q"], t["k"], t["v"], off))
        out_d = sapa_b200.deform_sapa_fused(qd, kd, vd, od, P_, s, G_)
        ms_db = time_path(lambda: torch.autograd.grad(out_d, (qd, kd, vd, od), g_out, retain_graph=True), 10)
        bytes_db = (B_ * C_ * hi + 2 * (B_ * d_ * hi + B_ * d_ * H_ * W_ + B_ * C_ * H_ * W_) + 2 * (2 * B_ * G_ * P_ * hi)
                    + B_ * G_ * P_ * hi) * esize
        paths["sapa_d_fused_backward"] = {"ms": ms_db, "algorithmic_bytes": bytes_db, "achieved_gbs": bytes_db / (ms_db * 1e-3) / 1e9,
                                          "roofline_frac": bytes_db / (ms_db * 1e-3) / 1e9 / peak_gbs,
                                          "kernels": sapa_b200._lib.last_kernels(),
                                          "note": "torch.autograd.grad through deform_sapa_fused: sapa_deform_fused_backward plus the casts of "
                                                  "its float32 accumulation buffers; bytes = dOut, attention read; q, k, v, offsets read and "
                                                  "their gradients written"}
        del qd, kd, vd, od, out_d
        if dtype == torch.float32:      # the same two calls on bfloat16 tensors (16-bit operands, float32 similarities)
            h16 = [x.to(torch.bfloat16) for x in (t["q"], t["k"], t["v"], off, g_out)]
            ms_d16 = time_path(lambda: sapa_b200.deform_sapa_fused(h16[0], h16[1], h16[2], h16[3], P_, s, G_), 10)
            k16 = sapa_b200._lib.last_kernels()
            r16 = [x.detach().clone().requires_grad_() for x in h16[:4]]
            out16 = sapa_b200.deform_sapa_fused(*r16, P_, s, G_)
            ms_db16 = time_path(lambda: torch.autograd.grad(out16, r16, h16[4], retain_graph=True), 10)
            paths["sapa_d_fused_bf16"] = {"forward_ms": ms_d16, "backward_ms": ms_db16,
                                          "forward_roofline_frac": bytes_d / 2 / (ms_d16 * 1e-3) / 1e9 / peak_gbs,
                                          "backward_roofline_frac": bytes_db / 2 / (ms_db16 * 1e-3) / 1e9 / peak_gbs,
                                          "forward_kernels": k16, "backward_kernels": sapa_b200._lib.last_kernels()}
            del h16, r16, out16
        del t, off, g_out, attn_b
        # Decoder pyramid (stand-in wiring, random init, forward only, bf16, B = 16): features of 64 / 128 / 320 / 512
        # channels at 128^2 / 64^2 / 32^2 / 16^2, each projected to 256 channels by a 1x1 convolution, then three
        # chained SAPA modules (d = 32, K = 5) upsample 16^2 -> 32^2 -> 64^2 -> 128^2.  Whole-module time: GroupNorm
        # and the 1x1 convolutions are torch kernels, the attention is the fused kernel.
        torch.manual_seed(0)
        PB = 16
        feats = [torch.randn(PB, c, r, r, device=device, dtype=torch.bfloat16) for c, r in ((64, 128), (128, 64), (320, 32), (512, 16))]
        proj = [torch.nn.Conv2d(c, 256, 1).to(device, torch.bfloat16) for c in (64, 128, 320, 512)]
        ups = [sapa_b200.SAPA(256, embedding_dim=32).to(device, torch.bfloat16) for _ in range(3)]

        def pyramid():
            with torch.no_grad():
                ys = [p(f) for p, f in zip(proj, feats)]
                x = ys[3]
                for level, m in zip((2, 1, 0), ups):
                    x = m(ys[level], x)
                return x

        def upsampling_chain(ys):
            x = ys[3]
            for level, m in zip((2, 1, 0), ups):
                x = m(ys[level], x)
            return x

        def upsampling_only():
            with torch.no_grad():
                return upsampling_chain(ys_fixed)

        with torch.no_grad():
            ys_fixed = [p(f) for p, f in zip(proj, feats)]
        ms_p, ms_u = time_path(pyramid, 10), time_path(upsampling_only, 10)
        graphed = sapa_b200.GraphedForward(lambda *ys: upsampling_chain(ys), ys_fixed)
        ms_g_u = time_path(lambda: graphed(*graphed.inputs), 10)      # inputs already in the captured buffers: replay only
        del graphed
        for m in ups:
            m.fuse_projection = False
        ms_u_torch = time_path(upsampling_only, 10)
        pyr_pix = PB * (32 * 32 + 64 * 64 + 128 * 128)
        paths["decoder_pyramid_bf16"] = {"ms": ms_p, "ms_sapa_modules_only": ms_u, "ms_sapa_modules_graph_replay": ms_g_u,
                                         "ms_sapa_modules_torch_projections": ms_u_torch,
                                         "batch": PB, "mpix_per_s": pyr_pix / (ms_u * 1e-3) / 1e6,
                                         "note": "three chained SAPA modules: GroupNorm + 1x1 query / key projections as one tensor-core "
                                                 "GEMM each (sapa_project_forward) and the fused attention kernel; "
                                                 "ms_sapa_modules_graph_replay = the same captured once into a CUDA graph (GraphedForward) and replayed; "
                                                 "ms_sapa_modules_torch_projections = eager with torch's GroupNorm and convolution; "
                                                 "ms = with the four 256-channel feature projections (torch), mpix_per_s = upsampled pixels "
                                                 "of the three levels / ms_sapa_modules_only"}
        del feats, proj, ups, ys_fixed
        # GroupNorm(32) + 1x1 projection of the guidance features to the query at the cfg2 shapes: statistics pass, fold,
        # tcgen05 GEMM.  Bytes: x is read twice (the statistics must be complete before the first output), out written once.
        from sapa_b200.projection import project
        xg = torch.randn(B_, C_, s * H_, s * W_, device=device).to(dtype)
        gn = torch.nn.GroupNorm(32, C_).to(device, dtype)
        cv = torch.nn.Conv2d(C_, d_, 1).to(device, dtype)
        with torch.no_grad():
            ms_g = time_path(lambda: project(xg, gn, cv), 10)
            ms_t = time_path(lambda: cv(gn(xg)), 10)
        bytes_g = (2 * xg.numel() + B_ * d_ * hi) * esize
        paths["projection_groupnorm_1x1"] = {"ms": ms_g, "ms_torch_groupnorm_conv": ms_t, "launches": 3, "algorithmic_bytes": bytes_g,
                                             "achieved_gbs": bytes_g / (ms_g * 1e-3) / 1e9,
                                             "roofline_frac": bytes_g / (ms_g * 1e-3) / 1e9 / peak_gbs,
                                             "kernels": sapa_b200._lib.last_kernels(),
                                             "config": {"B": B_, "C": C_, "d": d_, "pixels": hi, "groups": 32}}
        del xg, gn, cv
        paths["reference_cuda_ext"] = reference_cuda_ext_times(wl, device, time_path)

    # ---- BASELINE config 5 at this N: batch-sharded and row-sharded bfloat16 forward, strong scaling ----
    config5 = {}
    if not args.no_extra and args.workload == "cfg2":
        for name in ("cfg5a", "cfg5b"):
            config5[name] = measure_config5(name, world, rank, device, dist)
        config5["sapa_d_rows"] = measure_deform_rows(world, rank, device, dist)

    # ---- end to end: public op, pinned host buffers in and out, copies inside the timed region ----
    e2e_steps = max(3, min(args.steps, 30))
    host_in = [make_inputs(wl, dtype, device, seed=7 + i, pinned=True) for i in range(2)]
    host_out = [torch.empty((wl["B"], wl["C"], s * wl["H"], s * wl["W"]), dtype=dtype).pin_memory() for _ in range(2)]
    s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    dev_in = [None, None]
    dev_out = [None, None]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_k = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_loop(n):
        for i in range(n):
            b = i % 2
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_k[b])                 # the kernel that last read this slot is done
                dev_in[b] = {k: v.to(device, non_blocking=True) for k, v in host_in[b].items()}
                ev_in[b].record(s_in)
            s_main.wait_event(ev_in[b])
            s_main.wait_event(ev_out[b])                 # the copy-out that last read this slot is done
            if row_sharded:
                dev_out[b] = sharding.sapa_fused_row_sharded(dev_in[b]["q"], dev_in[b]["k"], dev_in[b]["v"], K, s)
            else:
                dev_out[b] = sapa_b200.sapa_fused(dev_in[b]["q"], dev_in[b]["k"], dev_in[b]["v"], K, s)
            ev_k[b].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_k[b])
                host_out[b].copy_(dev_out[b], non_blocking=True)
                dev_out[b].record_stream(s_out)
                ev_out[b].record(s_out)
        s_main.wait_stream(s_in)
        s_main.wait_stream(s_out)

    e2e_loop(3)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_loop(e2e_steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        tt = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt.item())
    e2e_value = pix_per_step / (e2e_ms / e2e_steps * 1e-3) / 1e6
    h2d = sum(v.numel() * v.element_size() for v in host_in[0].values())
    d2h = host_out[0].numel() * host_out[0].element_size()

    if rank == 0:
        peak, peak_kind = measured_peak()
        achieved = bytes_per_launch / (ms_per_step * 1e-3) / 1e9
        traffic = ncu_traffic(args.dtype, kernels_per_step) if args.workload == "cfg2" and world == 1 else None
        line = {
            "metric": METRIC, "value": value, "unit": "Mpix/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": w["scaling"], "vs_baseline": None, "dtype": args.dtype,
            "data": "synthetic",
            "config": config_dict(args, w),
            "timing": {"l2": f"{nsets} rotating input/output sets ({nsets * bytes_per_launch / 1e6:.0f} MB) > 126 MB L2",
                       "launch": (f"CUDA graph of {nsets} launches (one per buffer set), replayed" if graph is not None
                                  else "one call per step from Python"),
                       "kernels_per_step": kernels_per_step},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "Mpix/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "how": "sapa_b200.sapa_fused on pinned host tensors, double-buffered "
                                               "H2D / kernel / D2H on three streams"},
            "gpu_launches": args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_source": f"of {peak_kind}",
                         "algorithmic_bytes_per_launch": bytes_per_launch,
                         "frac_of_8000_nominal": achieved / 8000.0},
        }
        if world == 1 and not args.no_extra and args.workload == "cfg2":
            line["other_dtypes"] = other
            line["other_paths"] = paths
        if config5:
            line["config5"] = config5
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(w)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
