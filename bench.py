#!/usr/bin/env python
"""Benchmark of the QKANLayer hot path: fused forward + backward, edge-evaluations per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (one "step" = one forward + one backward over one batch): a single
QKANLayer, batch 65536 per GPU, 256 -> 256, reps 3, float32, preacts / postact
weights / postact bias / theta all trainable, base term frozen at 0, fast readout.
Seeded synthetic inputs: x ~ U[-1,1], theta ~ U[-pi,pi], preacts weight 1 / bias 0,
postact weights ~ N(0, 1/sqrt(256)), upstream gradient ~ N(0,1).

Metric: edge-evaluations per second counted as B*in*out*reps per pass (a forward
plus backward step counts its edges once). For N > 1 the batch is sharded by rows
(every rank gets its own 65536 rows: weak scaling) and the parameter gradients
are summed with one NCCL all-reduce per step inside the timed region.

``--impl reference`` times the CPU restatement of the reference algorithm
(oracle/, float32, all host threads) on a bounded row sample of the same layer.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOAD = "qkan_layer_fwd_bwd B=65536/gpu 256->256 reps=3 fp32 (layer microbenchmark)"
B_PER_GPU, IN_DIM, OUT_DIM, REPS = 65536, 256, 256, 3
METRIC = "qkan_edge_evals_per_sec_fwd_bwd"
UNIT = "edge-reps/s"

# Algorithmic work per edge-evaluation (pz ansatz, trainable preacts, fast readout):
# FP32 lane-ops W_f and special-function ops W_m, forward and forward+backward.
def work_per_edge(reps: int, frozen: bool = False):
    """Pinned (FP32 lane-ops, SFU ops) per edge evaluation; `frozen` = preacts not trainable (data trig hoisted)."""
    if frozen:
        return {"fwd": (12 * reps + 10, 2), "fwd_bwd": (47 * reps + 44, 5)}
    return {"fwd": (11 * reps + 10, 2 * reps + 2), "fwd_bwd": (46 * reps + 44, 4 * reps + 5)}


VARIANTS = {"headline": "preacts trainable, fast readout, base term off",
            "base": "base term on (silu(x) @ base_weight, trainable)",
            "born": "Born readout (fast_measure=False)",
            "frozen": "preacts frozen (preact_trainable=False)"}


SM_COUNT, FP32_LANES, SFU_LANES, NOMINAL_GHZ = 148, 128, 16, 1.965

# dram__bytes_read.sum + dram__bytes_write.sum of one backward_kernel launch, from the ncu capture of a
# 16384-row case (52.2 MB + 161.6 MB, backward tile pinned to the full batch's) scaled by 4 to the 65536-row
# batch; the traffic is proportional to the batch (activations and per-tile partials).
# See profiles/forward_backward_kernels_batch16384.md.
BACKWARD_DRAM_BYTES_PER_LAUNCH = 4 * (52_166_912 + 161_625_344)


def issue_roofline_seconds(edges: float, reps: int, which: str, ghz: float = NOMINAL_GHZ,
                           frozen: bool = False) -> float:
    wf, wm = work_per_edge(reps, frozen)[which]
    per_edge_clk = max((wf + wm) / FP32_LANES, wm / SFU_LANES)
    return edges * per_edge_clk / (SM_COUNT * ghz * 1e9)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return json.load(fh), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs (read-only)."""

    def __init__(self, device_index: int, period_s: float = 0.02):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._period = period_s
        try:
            import pynvml

            pynvml.nvmlInit()
            import torch

            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self._nv = pynvml
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(self._period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def make_problem_numpy(seed: int, rows: int):
    """Seeded host-side inputs of the microbenchmark layer (float32)."""
    rng = np.random.default_rng(seed)
    return dict(
        x=rng.uniform(-1, 1, (rows, IN_DIM)).astype(np.float32),
        theta=rng.uniform(-math.pi, math.pi, (OUT_DIM, IN_DIM, REPS + 1, 2)).astype(np.float32),
        pw=np.ones((OUT_DIM, IN_DIM, REPS), np.float32),
        pb=np.zeros((OUT_DIM, IN_DIM, REPS), np.float32),
        postw=(rng.standard_normal((OUT_DIM, IN_DIM)) / math.sqrt(IN_DIM)).astype(np.float32),
        postb=np.zeros((OUT_DIM, IN_DIM), np.float32),
        gy=rng.standard_normal((rows, OUT_DIM)).astype(np.float32),
    )


def cpu_baseline(sample_rows: int, repeats: int = 1):
    """Times the CPU port of the reference algorithm (oracle/, float32) on `sample_rows` rows."""
    from oracle import oracle

    oracle.use_all_cores()
    p = make_problem_numpy(1234, sample_rows)
    args = [p["x"], p["theta"], p["pw"], p["pb"], p["postw"], p["postb"], None, None]
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True, dtype=np.float32)
    oracle.forward(*[a[:8] if i == 0 else a for i, a in enumerate(args)], **cfg)  # warm the library
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.forward(*args, **cfg)
        oracle.backward(*args, p["gy"], **cfg)
        best = min(best, time.perf_counter() - t0)
    edges = sample_rows * IN_DIM * OUT_DIM
    return {
        "value": edges * REPS / best, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
        "sample": f"{sample_rows} rows of the same 256->256 reps=3 layer, fwd+bwd, float32, "
                  f"{best:.2f} s on {oracle.num_threads()} OpenMP threads",
    }, best


def run_reference(args):
    """`--impl reference`: the CPU restatement of the reference algorithm on the host cores."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return 0
    rows = args.ref_rows
    for _ in range(max(args.warmup, 1)):
        cpu_baseline(min(rows, 32))
    times = []
    info = None
    for _ in range(args.steps):
        info, t = cpu_baseline(rows)
        times.append(t)
    total = float(sum(times))
    edges = rows * IN_DIM * OUT_DIM
    value = edges * REPS * args.steps / total
    info = dict(info, value=value)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": f"{rows} rows per step on the host CPU",
                   "batch_per_gpu": B_PER_GPU, "in_dim": IN_DIM, "out_dim": OUT_DIM, "reps": REPS},
        "cpu_baseline": info,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


def run_b200(args):
    import torch
    import torch.distributed as dist

    from qkan_b200 import functional as F
    from qkan_b200.parallel import GradBucket, layer_grad_shapes

    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    from qkan_b200.parallel import bind_host_thread_near_gpu

    all_cores = os.sched_getaffinity(0)
    numa_cores = bind_host_thread_near_gpu(local_rank)  # host buffers next to this rank's GPU
    if world > 1:
        # NCCL prints its version banner with printf when NCCL_DEBUG is set; stdout carries the one JSON line
        # only, so file descriptor 1 points at stderr while the communicator comes up
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.all_reduce(torch.zeros(1, device=dev))
            torch.cuda.synchronize()
        finally:
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    rows = args.batch if args.scaling == "weak" else (args.batch + world - 1) // world
    host = make_problem_numpy(100 + rank, rows)
    shared = make_problem_numpy(7, 8)  # parameters are replicated: same seed on every rank
    for k in ("theta", "pw", "pb", "postw", "postb"):
        host[k] = shared[k]
    t = {k: torch.from_numpy(v).to(dev) for k, v in host.items()}
    # the headline is the default; the other variants are the extra rows the microbenchmark names
    # (base term on, Born readout, frozen preacts) and skip the host-buffer and CPU legs
    variant = args.variant
    cfg = dict(preact_trainable=variant != "frozen", fast_measure=variant != "born", use_postact_bias=True)
    basew = None
    if variant == "base":
        basew = (0.5 * torch.randn(OUT_DIM, IN_DIM, generator=torch.Generator().manual_seed(5))).to(dev)
    if variant != "headline":
        args.no_e2e = args.no_cpu_baseline = True
    bucket = GradBucket(layer_grad_shapes(IN_DIM, OUT_DIM, REPS, preact_trainable=cfg["preact_trainable"],
                                          base=basew is not None), dev)
    gx = torch.empty_like(t["x"])
    outs = dict(bucket.views, x=gx)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)  # > 126 MB L2

    def step():
        y = F.layer_forward(t["x"], t["theta"], t["pw"], t["pb"], t["postw"], t["postb"], basew, None, **cfg)
        F.layer_backward(t["x"], t["theta"], t["pw"], t["pb"], t["postw"], t["postb"], basew, None,
                         t["gy"], out=outs, want=tuple(outs), **cfg)
        if world > 1:
            bucket.all_reduce()
        return y

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sync_all()

    # ---- timed region: K steps, one pair of CUDA events per step, L2 flushed in between ----
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    fwd_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    bwd_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    with ClockSampler(local_rank) as clocks:
        wall0 = time.perf_counter()
        for k in range(args.steps):
            flush.zero_()
            ev[k][0].record()
            fwd_ev[k][0].record()
            F.layer_forward(t["x"], t["theta"], t["pw"], t["pb"], t["postw"], t["postb"], basew, None, **cfg)
            fwd_ev[k][1].record()
            bwd_ev[k][0].record()
            F.layer_backward(t["x"], t["theta"], t["pw"], t["pb"], t["postw"], t["postb"], basew, None,
                             t["gy"], out=outs, want=tuple(outs), **cfg)
            bwd_ev[k][1].record()
            if world > 1:
                bucket.all_reduce()
            ev[k][1].record()  # the step ends when the all-reduced gradients are there
        sync_all()
        wall = time.perf_counter() - wall0
    total_ms = sum(a.elapsed_time(b) for a, b in ev)
    fwd_ms = sum(a.elapsed_time(b) for a, b in fwd_ev) / args.steps
    bwd_ms = sum(a.elapsed_time(b) for a, b in bwd_ev) / args.steps
    # gradient exchange as seen by this rank: from the end of its backward to the end of the all-reduce
    # (the collective itself plus the wait for the slowest rank)
    exchange_ms = sum(b[1].elapsed_time(e[1]) for b, e in zip(bwd_ev, ev)) / args.steps
    if world > 1:
        tt = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        total_ms = float(tt.item())
    ms_per_step = total_ms / args.steps
    edges_per_rank = rows * IN_DIM * OUT_DIM
    value = edges_per_rank * world * REPS / (ms_per_step * 1e-3)

    # ---- end-to-end leg: host buffers in, results back on the host, every step ----
    hx = torch.from_numpy(host["x"]).pin_memory()
    hgy = torch.from_numpy(host["gy"]).pin_memory()
    hy = torch.empty((rows, OUT_DIM), dtype=torch.float32).pin_memory()
    hgx = torch.empty((rows, IN_DIM), dtype=torch.float32).pin_memory()
    hgrads = torch.empty(bucket.flat.numel(), dtype=torch.float32).pin_memory()
    e2e_steps = 0 if args.no_e2e else max(3, min(args.steps, 10))

    from qkan_b200.host import HostLayerPipeline

    pipe = HostLayerPipeline(rows, IN_DIM, OUT_DIM, REPS, dev, n_chunks=args.e2e_chunks) if e2e_steps else None
    dev_params = {k: t[k] for k in ("theta", "pw", "pb", "postw", "postb")}

    def e2e_step():
        # public host-buffer API: chunked copy-in / kernels / copy-out pipeline on three streams
        pipe.step(hx, hgy, dev_params, hy, hgx, hgrads)

    for _ in range(2 if e2e_steps else 0):
        e2e_step()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    if pipe is not None:
        pipe.wait()  # the last step's copy-out belongs to the timed region
    e1.record()
    sync_all()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps if e2e_steps else float("nan")
    if world > 1:
        tt = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt.item())
    e2e_value = edges_per_rank * world * REPS / (e2e_ms * 1e-3)
    os.sched_setaffinity(0, all_cores)  # the CPU baseline below gets every core again
    h2d = hx.numel() * 4 + hgy.numel() * 4
    d2h = hy.numel() * 4 + hgx.numel() * 4 + hgrads.numel() * 4

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        clk = clocks.summary()
        work = work_per_edge(REPS, frozen=variant == "frozen")
        wf, wm = work["fwd_bwd"]
        # step-level issue roofline (fwd + bwd), and the dominant kernel (the fused backward) alone
        lane_ops = edges_per_rank * (wf + wm)
        achieved = lane_ops / (fwd_ms + bwd_ms) * 1e-9  # Tlane-op/s on this rank
        peak_issue = SM_COUNT * FP32_LANES * NOMINAL_GHZ * 1e-3  # 37.23 Tlane-op/s
        wfb, wmb = wf - work["fwd"][0], wm - work["fwd"][1]
        bwd_achieved = edges_per_rank * (wfb + wmb) / bwd_ms * 1e-9
        alg_bytes = 4 * (2 * rows * IN_DIM + 2 * rows * OUT_DIM + rows * IN_DIM) + 3 * bucket.nbytes()
        roofline = {
            "bound": "fp32_issue", "achieved": achieved, "peak": peak_issue, "unit": "Tlane-op/s",
            "frac": achieved / peak_issue,
            "roofline_ms": 1e3 * issue_roofline_seconds(edges_per_rank, REPS, "fwd_bwd", frozen=variant == "frozen"),
            "frac_at_sampled_clock": (achieved / (peak_issue * clk["sm_mhz"] / 1965.0)
                                      if clk.get("sm_mhz") else None),
            "peak_source": "148 SMs x 128 FP32 lanes x 1.965 GHz (issue roofline; SFU 16 lanes/SM)",
            "work_per_edge": {"fp32": wf, "sfu": wm},
            "dominant_kernel": {"name": "backward_kernel", "ms": bwd_ms, "achieved": bwd_achieved,
                                "frac": bwd_achieved / peak_issue,
                                "timed": "CUDA events around the backward C-ABI call (prep + colsum + backward + finish)"},
            "forward_ms": fwd_ms,
            "hbm": {"algorithmic_bytes_per_step": alg_bytes,
                    "achieved_gbs": alg_bytes / ((fwd_ms + bwd_ms) * 1e-3) * 1e-9,
                    "peak_gbs": peaks["hbm_gbs"], "peak_kind": peak_kind},
            "traffic": None,
        }
        if rows == B_PER_GPU and variant == "headline":
            roofline["traffic"] = BACKWARD_DRAM_BYTES_PER_LAUNCH
        if variant in ("base", "born"):
            roofline["note"] = "work per edge is the headline's pinned count; this variant has no pinned count of its own"
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu, _ = cpu_baseline(args.cpu_rows)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": (WORKLOAD if args.batch == B_PER_GPU else f"profiling-size run, batch {args.batch}")
                       + ("" if variant == "headline" else f" [variant: {VARIANTS[variant]}]"),
                       "batch_per_gpu": rows, "global_batch": rows * world,
                       "in_dim": IN_DIM, "out_dim": OUT_DIM, "reps": REPS,
                       "parallelism": f"dp{world}", "l2": "flushed between timed steps (256 MB write)",
                       "edge_evals_per_sec": value / REPS},
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
            "gradient_exchange_ms": exchange_ms if world > 1 else 0.0,
            "host_cores_near_gpu": numa_cores,
            "gpu_launches": (7 + (1 if basew is not None else 0)) * args.steps,
            "clocks": clk,
            "wall_s_timed_region": wall,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("b200", "reference"), default="b200")
    ap.add_argument("--scaling", choices=("weak", "strong"), default="weak")
    ap.add_argument("--cpu-rows", type=int, default=1024, help="rows of the CPU-baseline sample")
    ap.add_argument("--ref-rows", type=int, default=256, help="rows per step of --impl reference")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--e2e-chunks", type=int, default=3, help="row chunks of the host-buffer pipeline")
    ap.add_argument("--variant", choices=tuple(VARIANTS), default="headline",
                    help="extra rows of the microbenchmark; only the default is the benchmark line")
    ap.add_argument("--batch", type=int, default=B_PER_GPU,
                    help="rows per GPU; anything but the default is a profiling-size run, not the benchmark")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_b200(args)


if __name__ == "__main__":
    sys.exit(main())
