#!/usr/bin/env python
"""Benchmark of the QKANLayer hot path: fused forward + backward, edge-evaluations per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--config NAME]

Default workload, ``--config layer`` (one "step" = one forward + one backward over one batch): a single
QKANLayer, batch 65536 per GPU, 256 -> 256, reps 3, float32, preacts / postact weights / postact bias /
theta all trainable, base term frozen at 0, fast readout. Seeded synthetic inputs: x ~ U[-1,1],
theta ~ U[-pi,pi], preacts weight 1 / bias 0, postact weights ~ N(0, 1/sqrt(256)), upstream gradient ~ N(0,1).

Metric: edge-evaluations per second counted as B*in*out*reps per pass (a forward plus backward step counts
its edges once). For N > 1 the batch is sharded by rows (every rank gets its own 65536 rows: weak scaling;
``--scaling strong`` cuts the same 65536 rows into N shards) and the parameter gradients are summed with one
NCCL all-reduce per step inside the timed region.

Other workloads (``--config``): ``bf16_sweep`` (batch 8192, square layers 512 / 1024 / 2048, reps 1 / 2 / 4 / 8,
bfloat16 activations), ``mnist`` (QKAN [784,128,10] Adam training step, batch 1024 per GPU) and ``hqkan``
(a stack of twelve 768 -> 768 layers, reps 2, bfloat16 activations, 8192 rows per GPU, per-layer gradient
all-reduce overlapped with the backward) and ``hqkan_block`` (the launch-bound hybrid block, eager and as a
CUDA graph). Each prints one JSON line of the same form.

Baselines. ``--impl reference`` times the reference package's own ``exact`` solver (torch, CPU, all host
cores) on a bounded row sample of the same layer; the default run carries the same measurement as
``cpu_baseline`` and, under ``baselines``, the reference's own GPU solvers (``flash``: Triton, ``cute``: CUDA)
on this GPU. All of them import the unmodified reference from ``baseline/_ref`` (installed by
``baseline/install_ref.py``); when that folder is absent the CPU legs fall back to the C port under
``oracle/`` and the GPU arms report ``unavailable``.
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
import types

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOAD = "qkan_layer_fwd_bwd B=65536/gpu 256->256 reps=3 fp32 (layer microbenchmark)"
B_PER_GPU, IN_DIM, OUT_DIM, REPS = 65536, 256, 256, 3
METRIC = "qkan_edge_evals_per_sec_fwd_bwd"
UNIT = "edge-reps/s"
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


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
PEAK_ISSUE = SM_COUNT * FP32_LANES * NOMINAL_GHZ * 1e-3  # 37.22 Tlane-op/s


def backward_dram_bytes(rows: int, in_dim: int, out_dim: int, reps: int):
    """DRAM bytes of one backward_kernel launch, from one ncu capture scaled by the rows processed.

    Captured: 16384 x 256 -> 256, reps 3, float32, 256-row tiles: dram read 51.40 MB, write 162.19 MB. The
    traffic is x, grad_y, grad_x (algorithmic) plus the per-batch-tile gradient partials the kernel writes for
    the finishing kernel (not algorithmic), all proportional to the rows. Other shapes have no capture: None.
    """
    if (in_dim, out_dim, reps) != (256, 256, 3) or rows < 4096:
        return None
    return int((51_401_472 + 162_188_032) * rows / 16384)


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


def make_problem_numpy(seed: int, rows: int, in_dim: int = IN_DIM, out_dim: int = OUT_DIM, reps: int = REPS):
    """Seeded host-side inputs of the microbenchmark layer (float32)."""
    rng = np.random.default_rng(seed)
    return dict(
        x=rng.uniform(-1, 1, (rows, in_dim)).astype(np.float32),
        theta=rng.uniform(-math.pi, math.pi, (out_dim, in_dim, reps + 1, 2)).astype(np.float32),
        pw=np.ones((out_dim, in_dim, reps), np.float32),
        pb=np.zeros((out_dim, in_dim, reps), np.float32),
        postw=(rng.standard_normal((out_dim, in_dim)) / math.sqrt(in_dim)).astype(np.float32),
        postb=np.zeros((out_dim, in_dim), np.float32),
        gy=rng.standard_normal((rows, out_dim)).astype(np.float32),
    )


# ------------------------------------------------------------------------------------------------
# Baselines: the reference package itself (baseline/_ref), else the C port of its algorithm (oracle/)
# ------------------------------------------------------------------------------------------------
def load_reference():
    """Import the unmodified reference package from baseline/_ref; None when it is not installed there.

    The reference imports matplotlib at module level for its plotting helpers; an empty stand-in module is
    registered for the import when matplotlib is absent (nothing on the timed path touches it).
    """
    if not os.path.isdir(os.path.join(REF_DIR, "qkan")):
        return None
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    try:
        import matplotlib.pyplot  # noqa: F401
    except Exception:
        for name in ("matplotlib", "matplotlib.pyplot"):
            sys.modules.setdefault(name, types.ModuleType(name))
    try:
        import qkan

        return qkan
    except Exception as exc:  # pragma: no cover - depends on the box
        print(f"bench: reference import failed: {exc!r}", file=sys.stderr)
        return None


def reference_layer(qkan, solver: str, device: str, seed: int = 0):
    """The microbenchmark layer built by the reference's own QKANLayer, every gradient of the headline on."""
    import torch

    layer = qkan.QKANLayer(IN_DIM, OUT_DIM, reps=REPS, solver=solver, device=device, preact_trainable=True,
                           postact_weight_trainable=True, postact_bias_trainable=True, ba_trainable=False,
                           seed=seed)
    gen = torch.Generator().manual_seed(7)
    with torch.no_grad():
        layer.theta.copy_(((torch.rand(layer.theta.shape, generator=gen) * 2 - 1) * math.pi).to(device))
        layer.postact_weights.copy_((torch.randn(layer.postact_weights.shape, generator=gen)
                                     / math.sqrt(IN_DIM)).to(device))
    return layer


def cpu_reference_exact(sample_rows: int, chunk: int = 64):
    """Reference `exact` solver (torch eager, CPU, all host cores) on `sample_rows` rows in chunks of 64.

    The whole batch at once would need ~1.7 TB of autograd storage, so the rows go through in chunks, as a
    user of the reference on a CPU would have to. Returns (cpu_baseline dict, seconds) or None.
    """
    qkan = load_reference()
    if qkan is None:
        return None
    import torch

    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    layer = reference_layer(qkan, "exact", "cpu")
    gen = torch.Generator().manual_seed(11)
    x = torch.rand(sample_rows, IN_DIM, generator=gen) * 2 - 1
    gy = torch.randn(sample_rows, OUT_DIM, generator=gen)

    def run(rows_x, rows_gy):
        xx = rows_x.clone().requires_grad_(True)
        layer(xx).backward(rows_gy)

    run(x[:8], gy[:8])  # warm torch's thread pool
    layer.zero_grad()
    t0 = time.perf_counter()
    for b in range(0, sample_rows, chunk):
        run(x[b:b + chunk], gy[b:b + chunk])
    sec = time.perf_counter() - t0
    edges = sample_rows * IN_DIM * OUT_DIM
    return {
        "value": edges * REPS / sec, "unit": UNIT, "cores": cores, "kind": "reference",
        "sample": f"{sample_rows} rows of the same 256->256 reps=3 layer in {chunk}-row chunks, fwd+bwd, float32, "
                  f"reference QKANLayer(solver='exact', device='cpu'), {sec:.2f} s on {cores} torch threads",
    }, sec


def cpu_port(sample_rows: int):
    """Times the C/OpenMP port of the reference algorithm (oracle/, float32) on `sample_rows` rows."""
    from oracle import oracle

    oracle.use_all_cores()
    p = make_problem_numpy(1234, sample_rows)
    args = [p["x"], p["theta"], p["pw"], p["pb"], p["postw"], p["postb"], None, None]
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True, dtype=np.float32)
    oracle.forward(*[a[:8] if i == 0 else a for i, a in enumerate(args)], **cfg)  # warm the library
    t0 = time.perf_counter()
    oracle.forward(*args, **cfg)
    oracle.backward(*args, p["gy"], **cfg)
    sec = time.perf_counter() - t0
    edges = sample_rows * IN_DIM * OUT_DIM
    return {
        "value": edges * REPS / sec, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
        "sample": f"{sample_rows} rows of the same 256->256 reps=3 layer, fwd+bwd, float32, "
                  f"{sec:.2f} s on {oracle.num_threads()} OpenMP threads",
    }, sec


def cpu_baseline(ref_rows: int, port_rows: int):
    """The reference's exact solver when baseline/_ref is present, else the port; plus the port beside it."""
    got = cpu_reference_exact(ref_rows)
    if got is not None:
        info, _ = got
        try:
            port, _ = cpu_port(port_rows)
            info["port_beside_it"] = {k: port[k] for k in ("value", "cores", "sample")}
        except Exception as exc:  # the port is optional here
            info["port_beside_it"] = {"unavailable": repr(exc)[:200]}
        return info
    info, _ = cpu_port(port_rows)
    info["note"] = "baseline/_ref absent: C port of the reference algorithm"
    return info


def run_reference(args):
    """`--impl reference`: the reference's own CPU implementation of the path on the host cores."""
    if int(os.environ.get("RANK", 0)) != 0:
        return 0
    use_ref = load_reference() is not None
    rows = args.ref_rows
    timer = (lambda: cpu_reference_exact(rows)) if use_ref else (lambda: cpu_port(rows * 4))
    for _ in range(min(args.warmup, 1)):
        (cpu_reference_exact(64) if use_ref else cpu_port(32))
    times, info = [], None
    for _ in range(args.steps):
        info, t = timer()
        times.append(t)
    total = float(sum(times))
    step_rows = rows if use_ref else rows * 4
    value = step_rows * IN_DIM * OUT_DIM * REPS * args.steps / total
    info = dict(info, value=value)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": f"{step_rows} rows per step on the host CPU",
                   "batch_per_gpu": B_PER_GPU, "in_dim": IN_DIM, "out_dim": OUT_DIM, "reps": REPS},
        "cpu_baseline": info,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# The reference's GPU solvers index their backward state buffer (programs x (3 reps + 3) x 4 x block) with
# 32-bit integers (src/qkan/solver/flash/fused_ops.py:1270-1272, src/qkan/csrc/cute_kernels.cu:281-286): at this
# layer shape the offset passes 2^31 from batch 683 on, and a batch of 1024 ended in an illegal memory access.
# So forward+backward is timed at 512 rows, the largest power of two inside that limit, and forward only at 8192.
BASELINE_ROWS_FWD_BWD, BASELINE_ROWS_FWD = 512, 8192


def run_baseline_arm(solver: str):
    """Child process of the default run: one GPU solver of the reference on this GPU; prints one JSON dict."""
    import torch

    out = {"solver": solver}
    qkan = load_reference()
    if qkan is None:
        print(json.dumps({"solver": solver, "unavailable": "baseline/_ref is not installed"}))
        return 0
    dev = "cuda"

    def nerr(a, b):
        return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))

    try:
        gen = torch.Generator().manual_seed(3)
        layer = reference_layer(qkan, solver, dev)
        # the same 256 rows through this repository's kernels: the arms time the same function
        from qkan_b200 import functional as F

        x = (torch.rand(256, IN_DIM, generator=gen) * 2 - 1).to(dev)
        with torch.no_grad():
            y_ref = layer(x)
        y = F.layer_forward(x, layer.theta.detach(), layer.preacts_weight.detach(), layer.preacts_bias.detach(),
                            layer.postact_weights.detach(), layer.postact_bias.detach(), None, None,
                            preact_trainable=True, fast_measure=True, use_postact_bias=True)
        out["nerr_y_vs_b200_kernels"] = nerr(y_ref, y)
        for rows, with_bwd in ((BASELINE_ROWS_FWD_BWD, True), (BASELINE_ROWS_FWD, False)):
            x = (torch.rand(rows, IN_DIM, generator=gen) * 2 - 1).to(dev)
            gy = torch.randn(rows, OUT_DIM, generator=gen).to(dev)
            if with_bwd:
                x.requires_grad_(True)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            t_f = t_b = 0.0
            n_warm, n_timed = 3, 10
            for it in range(n_warm + n_timed):
                ev[0].record()
                if with_bwd:
                    y = layer(x)
                    ev[1].record()
                    y.backward(gy)
                    ev[2].record()
                    layer.zero_grad()
                    x.grad = None
                else:
                    with torch.no_grad():
                        layer(x)
                    ev[1].record()
                    ev[2].record()
                torch.cuda.synchronize()
                if it >= n_warm:
                    t_f += ev[0].elapsed_time(ev[1])
                    t_b += ev[1].elapsed_time(ev[2])
            t_f, t_b = t_f / n_timed, t_b / n_timed
            edges = rows * IN_DIM * OUT_DIM * REPS
            key = "fwd_bwd" if with_bwd else "fwd_only"
            out[key] = {"rows": rows, "fwd_ms": t_f, "bwd_ms": t_b if with_bwd else None,
                        "value": edges / ((t_f + t_b) * 1e-3), "unit": UNIT,
                        "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9}
            torch.cuda.reset_peak_memory_stats()
    except Exception as exc:
        out["unavailable"] = f"{type(exc).__name__}: {str(exc)[:400]}"
    print(json.dumps(out))
    return 0


def gpu_baselines(timeout_s: int = 240):
    """Runs each GPU solver of the reference in a child process (a fault there must not take this run down)."""
    result = {"note": "reference QKANLayer(solver=...) on this GPU, same 256->256 reps=3 fp32 layer; fwd+bwd at "
                      f"{BASELINE_ROWS_FWD_BWD} rows (their 32-bit state indexing ends at 682), forward only at "
                      f"{BASELINE_ROWS_FWD} rows; CUDA events, 10 timed iterations"}
    for solver in ("flash", "cute"):
        try:
            res = subprocess.run([sys.executable, os.path.abspath(__file__), "--baseline-arm", solver],
                                 capture_output=True, text=True, timeout=timeout_s, cwd=ROOT)
            lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
            if lines:
                result[solver] = json.loads(lines[-1])
            else:
                result[solver] = {"unavailable": f"exit {res.returncode}: {res.stderr[-400:]}"}
        except subprocess.TimeoutExpired:
            result[solver] = {"unavailable": f"no result within {timeout_s} s"}
        except Exception as exc:  # pragma: no cover
            result[solver] = {"unavailable": repr(exc)[:400]}
    return result


# ------------------------------------------------------------------------------------------------
# Common plumbing of the b200 arm
# ------------------------------------------------------------------------------------------------
class Run:
    """Process group, device, timing helpers shared by the workloads."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        self.torch, self.dist, self.args = torch, dist, args
        self.world = int(os.environ.get("WORLD_SIZE", 1))
        self.rank = int(os.environ.get("RANK", 0))
        self.local_rank = int(os.environ.get("LOCAL_RANK", 0))
        if self.world != args.gpus and self.world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        from qkan_b200.parallel import bind_host_thread_near_gpu

        self.all_cores = os.sched_getaffinity(0)
        self.numa_cores = bind_host_thread_near_gpu(self.local_rank)  # host buffers next to this rank's GPU
        if self.world > 1:
            # NCCL prints its version banner with printf when NCCL_DEBUG is set; stdout carries the one JSON
            # line only, so file descriptor 1 points at stderr while the communicator comes up
            sys.stdout.flush()
            saved_stdout = os.dup(1)
            os.dup2(2, 1)
            try:
                dist.init_process_group("nccl", device_id=self.dev)
                dist.all_reduce(torch.zeros(1, device=self.dev))
                torch.cuda.synchronize()
            finally:
                os.dup2(saved_stdout, 1)
                os.close(saved_stdout)
        self.flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=self.dev)  # > 126 MB L2

    def sync_all(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def event(self):
        return self.torch.cuda.Event(enable_timing=True)

    def max_over_ranks(self, value: float) -> float:
        if self.world == 1:
            return value
        t = self.torch.tensor([value], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def gather(self, values):
        """One list of floats per rank, on every rank."""
        t = self.torch.tensor(values, device=self.dev, dtype=self.torch.float64)
        if self.world == 1:
            return [t.tolist()]
        out = [self.torch.zeros_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t)
        return [o.tolist() for o in out]

    def time_steps(self, step, steps: int, warmup: int, marks: int = 0):
        """W warm-up steps, then K timed steps: the L2 is flushed before each, one CUDA-event pair brackets each.

        `step(rec)` runs one step; it may call rec() up to `marks` times to drop intermediate events. Returns
        (total ms as the max over ranks, per-mark mean ms on this rank, clock summary, wall seconds).
        """
        for _ in range(max(warmup, 3)):
            step(lambda: None)
        evs = [[self.event() for _ in range(marks + 2)] for _ in range(steps)]
        # the sampler starts (NVML initialisation, tens of milliseconds and not the same on every rank) before the
        # barrier, so that the ranks leave the barrier straight into the first timed step
        with ClockSampler(self.local_rank) as clocks:
            self.sync_all()
            wall0 = time.perf_counter()
            for k in range(steps):
                self.flush.zero_()
                cur = iter(evs[k][1:-1])
                evs[k][0].record()
                step(lambda: next(cur).record())
                evs[k][-1].record()
            self.sync_all()
            wall = time.perf_counter() - wall0
        total_ms = sum(e[0].elapsed_time(e[-1]) for e in evs)
        segs = [sum(e[j].elapsed_time(e[j + 1]) for e in evs) / steps for j in range(marks + 1)]
        return self.max_over_ranks(total_ms), total_ms, segs, clocks.summary(), wall

    def finish(self):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


def roofline_block(edges_per_rank, reps, frozen, fwd_ms, bwd_ms, clk, alg_bytes, traffic, note=None):
    peaks, peak_kind = measured_peaks()
    work = work_per_edge(reps, frozen=frozen)
    wf, wm = work["fwd_bwd"]
    achieved = edges_per_rank * (wf + wm) / (fwd_ms + bwd_ms) * 1e-9  # Tlane-op/s on this rank
    wfb, wmb = wf - work["fwd"][0], wm - work["fwd"][1]
    bwd_achieved = edges_per_rank * (wfb + wmb) / bwd_ms * 1e-9
    block = {
        "bound": "fp32_issue", "achieved": achieved, "peak": PEAK_ISSUE, "unit": "Tlane-op/s",
        "frac": achieved / PEAK_ISSUE,
        "roofline_ms": 1e3 * issue_roofline_seconds(edges_per_rank, reps, "fwd_bwd", frozen=frozen),
        "frac_at_sampled_clock": (achieved / (PEAK_ISSUE * clk["sm_mhz"] / 1965.0) if clk.get("sm_mhz") else None),
        "peak_source": "148 SMs x 128 FP32 lanes x 1.965 GHz (issue roofline; SFU 16 lanes/SM)",
        "work_per_edge": {"fp32": wf, "sfu": wm},
        "dominant_kernel": {"name": "backward_kernel", "ms": bwd_ms, "achieved": bwd_achieved,
                            "frac": bwd_achieved / PEAK_ISSUE,
                            "timed": "CUDA events around the backward C-ABI call (backward + finish launches)"},
        "forward_ms": fwd_ms,
        "hbm": {"algorithmic_bytes_per_step": alg_bytes,
                "achieved_gbs": alg_bytes / ((fwd_ms + bwd_ms) * 1e-3) * 1e-9,
                "peak_gbs": peaks["hbm_gbs"], "peak_kind": peak_kind},
        "traffic": traffic,
    }
    if note:
        block["note"] = note
    return block


# ------------------------------------------------------------------------------------------------
# --config layer (the headline)
# ------------------------------------------------------------------------------------------------
def dp_check(run: Run):
    """Data-parallel correctness on the bench's own path: world x 64 rows, sharded + all-reduced, against rank 0
    computing the whole mini batch. Normalised max error over every parameter gradient."""
    torch = run.torch
    from qkan_b200 import functional as F
    from qkan_b200.parallel import GradBucket, layer_grad_shapes

    rows = 64 * run.world
    host = make_problem_numpy(4242, rows, 64, 48, REPS)
    t = {k: torch.from_numpy(v).to(run.dev) for k, v in host.items()}
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True)
    prep = F.prepare_layer(t["theta"], t["pw"], t["pb"], t["postw"], t["postb"], None, None, in_dim=64, **cfg)
    shapes = layer_grad_shapes(64, 48, REPS)
    part, whole = GradBucket(shapes, run.dev), GradBucket(shapes, run.dev)
    b = 64 * run.rank
    F.backward_prepared(prep, t["x"][b:b + 64].contiguous(), t["gy"][b:b + 64].contiguous(),
                        out=dict(part.views), want=tuple(part.views))
    part.all_reduce()
    F.backward_prepared(prep, t["x"], t["gy"], out=dict(whole.views), want=tuple(whole.views))
    worst = 0.0
    for k in shapes:
        worst = max(worst, float((part[k] - whole[k]).abs().max() / whole[k].abs().max().clamp_min(1e-30)))
    worst = run.max_over_ranks(worst)
    return {"rows": rows, "nerr": worst, "ok": bool(worst <= 2e-6), "tolerance": 2e-6}


def run_layer(run: Run):
    torch, args, dev, world, rank = run.torch, run.args, run.dev, run.world, run.rank
    from qkan_b200 import functional as F
    from qkan_b200.parallel import GradBucket, layer_grad_shapes

    rows = args.batch if args.scaling == "weak" else (args.batch + world - 1) // world
    host = make_problem_numpy(100 + rank, rows)
    shared = make_problem_numpy(7, 8)  # parameters are replicated: same seed on every rank
    for k in ("theta", "pw", "pb", "postw", "postb"):
        host[k] = shared[k]
    t = {k: torch.from_numpy(v).to(dev) for k, v in host.items()}
    # the headline is the default; the other variants are the extra rows the microbenchmark names
    # (base term on, Born readout, frozen preacts) and skip the host-buffer, CPU and reference-GPU legs
    variant = args.variant
    cfg = dict(preact_trainable=variant != "frozen", fast_measure=variant != "born", use_postact_bias=True)
    basew = None
    if variant == "base":
        basew = (0.5 * torch.randn(OUT_DIM, IN_DIM, generator=torch.Generator().manual_seed(5))).to(dev)
    if variant != "headline":
        args.no_e2e = args.no_cpu_baseline = args.no_baselines = True
    bucket = GradBucket(layer_grad_shapes(IN_DIM, OUT_DIM, REPS, preact_trainable=cfg["preact_trainable"],
                                          base=basew is not None), dev)
    gx = torch.empty_like(t["x"])
    outs = dict(bucket.views, x=gx)

    def step(mark):
        # forward call = set-up + forward kernel; backward call = backward + finish: four launches
        prep = F.prepare_layer(t["theta"], t["pw"], t["pb"], t["postw"], t["postb"], basew, None,
                               in_dim=IN_DIM, **cfg)
        F.forward_prepared(prep, t["x"])
        mark()
        F.backward_prepared(prep, t["x"], t["gy"], out=outs, want=tuple(outs))
        mark()
        if world > 1:
            bucket.all_reduce()  # the step ends when the all-reduced gradients are there

    total_max_ms, total_ms, segs, clk, wall = run.time_steps(step, args.steps, args.warmup, marks=2)
    fwd_ms, bwd_ms, exchange_ms = segs
    ms_per_step = total_max_ms / args.steps
    edges_per_rank = rows * IN_DIM * OUT_DIM
    value = edges_per_rank * world * REPS / (ms_per_step * 1e-3)
    per_rank = run.gather([fwd_ms, bwd_ms, exchange_ms, total_ms / args.steps, clk.get("sm_mhz") or 0.0])
    check = dp_check(run)

    # ---- end-to-end leg: host buffers in, results back on the host, every step ----
    e2e = None
    if not args.no_e2e:
        from qkan_b200.host import HostLayerPipeline

        hx = torch.from_numpy(host["x"]).pin_memory()
        hgy = torch.from_numpy(host["gy"]).pin_memory()
        hy = torch.empty((rows, OUT_DIM), dtype=torch.float32).pin_memory()
        hgx = torch.empty((rows, IN_DIM), dtype=torch.float32).pin_memory()
        hgrads = torch.empty(bucket.flat.numel(), dtype=torch.float32).pin_memory()
        e2e_steps = max(3, min(args.steps, 20))
        pipe = HostLayerPipeline(rows, IN_DIM, OUT_DIM, REPS, dev, n_chunks=args.e2e_chunks)
        dev_params = {k: t[k] for k in ("theta", "pw", "pb", "postw", "postb")}
        for _ in range(2):
            pipe.step(hx, hgy, dev_params, hy, hgx, hgrads)
        run.sync_all()
        e0, e1 = run.event(), run.event()
        e0.record()
        for _ in range(e2e_steps):
            pipe.step(hx, hgy, dev_params, hy, hgx, hgrads)
        pipe.wait()  # the last step's copy-out belongs to the timed region
        e1.record()
        run.sync_all()
        e2e_ms = run.max_over_ranks(e0.elapsed_time(e1) / e2e_steps)
        e2e = {"value": edges_per_rank * world * REPS / (e2e_ms * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": hx.numel() * 4 + hgy.numel() * 4,
               "d2h_bytes_per_step": hy.numel() * 4 + hgx.numel() * 4 + hgrads.numel() * 4,
               "ms_per_step": e2e_ms, "gpu_launches_per_step": pipe.launches_per_step()}
    os.sched_setaffinity(0, run.all_cores)  # the CPU baseline below gets every core again

    if rank == 0:
        alg_bytes = 4 * (2 * rows * IN_DIM + 2 * rows * OUT_DIM + rows * IN_DIM) + 3 * bucket.nbytes()
        note = ("work per edge is the headline's pinned count; this variant has no pinned count of its own"
                if variant in ("base", "born") else None)
        roofline = roofline_block(edges_per_rank, REPS, variant == "frozen", fwd_ms, bwd_ms, clk, alg_bytes,
                                  backward_dram_bytes(rows, IN_DIM, OUT_DIM, REPS) if variant == "headline" else None,
                                  note)
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu = cpu_baseline(args.cpu_ref_rows, args.cpu_rows)
        baselines = None
        if world == 1 and not args.no_baselines:
            baselines = gpu_baselines()
            for solver in ("flash", "cute"):
                arm = baselines.get(solver, {})
                if "fwd_bwd" in arm:
                    arm["b200_over_this_arm_fwd_bwd"] = value / arm["fwd_bwd"]["value"]
                if "fwd_only" in arm:
                    arm["b200_over_this_arm_fwd"] = (edges_per_rank * REPS / (fwd_ms * 1e-3)) / arm["fwd_only"]["value"]
        launches_per_step = 4 + (1 if basew is not None else 0)
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
            "roofline": roofline, "cpu_baseline": cpu, "baselines": baselines,
            "e2e": e2e,
            "gradient_exchange_ms": exchange_ms if world > 1 else 0.0,
            "per_rank": {"columns": ["fwd_ms", "bwd_ms", "exchange_ms", "step_ms", "sm_mhz"], "rows": per_rank},
            "dp_check": check,
            "host_cores_near_gpu": run.numa_cores,
            "gpu_launches": launches_per_step * args.steps,
            "gpu_launches_per_step": {"device_resident": launches_per_step,
                                      "kernels": "prep, forward, backward, finish_grads"
                                                 + (", base_backward" if basew is not None else "")},
            "clocks": clk,
            "wall_s_timed_region": wall,
        }
        print(json.dumps(line))
    run.finish()
    return 0


# ------------------------------------------------------------------------------------------------
# --config bf16_sweep
# ------------------------------------------------------------------------------------------------
SWEEP_BATCH, SWEEP_WIDTHS, SWEEP_REPS = 8192, (512, 1024, 2048), (1, 2, 4, 8)


def run_bf16_sweep(run: Run):
    torch, args, dev, world, rank = run.torch, run.args, run.dev, run.world, run.rank
    from qkan_b200 import functional as F
    from qkan_b200.parallel import GradBucket, layer_grad_shapes

    rows = SWEEP_BATCH if args.scaling == "weak" else (SWEEP_BATCH + world - 1) // world
    cfg = dict(preact_trainable=True, fast_measure=True, use_postact_bias=True)
    table, clk_all, tot_edges_reps, tot_ms = [], None, 0.0, 0.0
    for width in (args.sweep_widths or SWEEP_WIDTHS):
        for reps in (args.sweep_reps or SWEEP_REPS):
            gen = torch.Generator().manual_seed(1000 * width + reps)
            x = torch.randn(rows, width, generator=torch.Generator().manual_seed(50 + rank)).clamp_(-3, 3)
            x = x.to(torch.bfloat16).to(dev)
            gy = torch.randn(rows, width, generator=torch.Generator().manual_seed(60 + rank)).to(torch.bfloat16).to(dev)
            theta = ((torch.rand(width, width, reps + 1, 2, generator=gen) * 2 - 1) * math.pi).to(dev)
            pw = torch.ones(width, width, reps, device=dev)
            pb = torch.zeros(width, width, reps, device=dev)
            postw = (torch.randn(width, width, generator=gen) / math.sqrt(width)).to(torch.bfloat16).to(dev)
            postb = torch.zeros(width, width, dtype=torch.bfloat16, device=dev)
            bucket = GradBucket(layer_grad_shapes(width, width, reps), dev)
            outs = dict(bucket.views, x=torch.empty_like(x))

            def step(mark):
                prep = F.prepare_layer(theta, pw, pb, postw, postb, None, None, in_dim=width, **cfg)
                F.forward_prepared(prep, x)
                mark()
                F.backward_prepared(prep, x, gy, out=outs, want=tuple(outs))
                mark()
                if world > 1:
                    bucket.all_reduce()

            total_max_ms, _, segs, clk, _ = run.time_steps(step, args.steps, args.warmup, marks=2)
            ms = total_max_ms / args.steps
            edges = rows * width * width
            roof_ms = 1e3 * issue_roofline_seconds(edges, reps, "fwd_bwd")
            table.append({"in_dim": width, "out_dim": width, "reps": reps, "rows_per_gpu": rows,
                          "fwd_ms": segs[0], "bwd_ms": segs[1], "exchange_ms": segs[2], "ms_per_step": ms,
                          "value": edges * world * reps / (ms * 1e-3), "roofline_ms": roof_ms,
                          "frac": roof_ms / (segs[0] + segs[1]), "sm_mhz": clk.get("sm_mhz")})
            tot_edges_reps += edges * world * reps
            tot_ms += ms
            clk_all = clk if clk_all is None else {**clk_all, "reasons": sorted(set(clk_all["reasons"]) | set(clk["reasons"]))}
            del x, gy, theta, pw, pb, postw, postb, bucket, outs
            torch.cuda.empty_cache()
    if rank == 0:
        fr = [r["frac"] for r in table]
        line = {
            "metric": METRIC, "value": tot_edges_reps / (tot_ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": tot_ms / len(table),
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16 I/O, f32 compute",
            "data": "synthetic",
            "config": {"workload": "bf16 layer sweep: batch 8192, square layers 512/1024/2048, reps 1/2/4/8, "
                                   "bf16 x / grad_y / postact tensors, fp32 theta and accumulation, fwd+bwd",
                       "rows_per_gpu": rows, "parallelism": f"dp{world}",
                       "l2": "flushed between timed steps (256 MB write)",
                       "value_is": "edge-reps of the whole sweep / summed step times"},
            "roofline": {"bound": "fp32_issue", "unit": "fraction of each shape's pinned issue roofline",
                         "frac": float(np.mean(fr)), "frac_min": min(fr), "frac_max": max(fr), "peak": PEAK_ISSUE},
            "rows": table, "gpu_launches": 4 * args.steps * len(table), "clocks": clk_all,
        }
        print(json.dumps(line))
    run.finish()
    return 0


# ------------------------------------------------------------------------------------------------
# --config mnist and --config hqkan: whole models through the public QKAN API
# ------------------------------------------------------------------------------------------------
def model_edges(widths):
    return sum(a * b for a, b in zip(widths[:-1], widths[1:]))


def run_mnist(run: Run):
    """MNIST-shaped classifier: QKAN [784,128,10], reps 3, float32, batch 1024 per GPU, cross-entropy, Adam 1e-3.
    A step is forward, loss, backward, gradient averaging over the ranks and the optimiser update."""
    torch, dist, args, dev, world, rank = run.torch, run.dist, run.args, run.dev, run.world, run.rank
    from qkan_b200 import QKAN
    from qkan_b200.parallel import OverlappedGradSync

    widths, reps, rows = [784, 128, 10], 3, 1024
    model = QKAN(widths, reps=reps, device=dev, seed=0)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    gen = torch.Generator().manual_seed(200 + rank)
    hx = torch.rand(rows, 784, generator=gen).pin_memory()          # pixels ~ U[0,1]
    hlab = torch.randint(0, 10, (rows,), generator=gen).pin_memory()  # labels uniform over 0..9
    x, lab = hx.to(dev), hlab.to(dev)
    loss_fn = torch.nn.CrossEntropyLoss()
    graphed = not args.eager
    if graphed:
        # forward + loss + backward replayed as one CUDA graph (the step is bound by launches at this size); the
        # gradients land in one flat buffer, averaged over the ranks with a single collective
        from qkan_b200.graph import make_graphed_train_step

        train = make_graphed_train_step(model, x, lab, loss_fn, opt, flat_grads=True)
        avg = dist.ReduceOp.AVG if world > 1 else None

        def step(mark, xx=x, ll=lab):
            loss = train(xx, ll)
            mark()
            if world > 1:
                dist.all_reduce(train.flat, op=avg)
            mark()
            opt.step()
            return loss
        grad_bytes = train.flat.numel() * 4
    else:
        sync = OverlappedGradSync(model)

        def step(mark, xx=x, ll=lab):
            sync.zero_grad()
            loss = loss_fn(model(xx), ll)
            mark()
            loss.backward()
            sync.finish()
            mark()
            opt.step()
            return loss
        grad_bytes = sync.nbytes()

    total_max_ms, _, segs, clk, wall = run.time_steps(step, args.steps, args.warmup, marks=2)
    ms = total_max_ms / args.steps

    def e2e_step():
        return float(step(lambda: None, hx.to(dev, non_blocking=True), hlab.to(dev, non_blocking=True)))

    for _ in range(3):
        e2e_step()
    run.sync_all()
    n_e2e = max(3, min(args.steps, 20))
    e0, e1 = run.event(), run.event()
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    run.sync_all()
    e2e_ms = run.max_over_ranks(e0.elapsed_time(e1) / n_e2e)
    if rank == 0:
        edges = rows * model_edges(widths)
        roof_ms = 1e3 * issue_roofline_seconds(edges, reps, "fwd_bwd", frozen=True)
        line = {
            "metric": METRIC, "value": edges * world * reps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "MNIST-shaped classifier QKAN [784,128,10] reps 3 fp32, batch 1024/GPU, "
                                   "cross-entropy, Adam lr 1e-3, whole training step (uniform pixels, uniform labels)",
                       "parallelism": f"dp{world}", "l2": "flushed between timed steps (256 MB write)",
                       "train_steps_per_sec": 1e3 / ms, "samples_per_sec": rows * world * 1e3 / ms},
            "roofline": {"bound": "launch/latency at this size; issue roofline for reference", "roofline_ms": roof_ms,
                         "frac": roof_ms / ms, "peak": PEAK_ISSUE, "unit": "Tlane-op/s",
                         "achieved": roof_ms / ms * PEAK_ISSUE,
                         "segments_ms": dict(zip(("graph_forward_loss_backward", "gradient_all_reduce", "optimizer")
                                                 if graphed else ("forward_loss", "backward_sync", "optimizer"), segs)),
                         "mode": "CUDA-graph replay of forward + loss + backward" if graphed else "eager"},
            "e2e": {"value": edges * world * reps / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": hx.numel() * 4 + hlab.numel() * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": 8 * args.steps, "gradient_bytes_per_step": grad_bytes, "clocks": clk,
            "wall_s_timed_region": wall,
        }
        print(json.dumps(line))
    run.finish()
    return 0


def run_hqkan(run: Run):
    """HQKANsformer-shaped stack: twelve QKAN [768 -> 768] layers, reps 2, bfloat16 activations, 8 x 1024 token rows
    per GPU; forward + backward with one gradient all-reduce per layer, launched as soon as that layer's
    gradients exist and overlapped with the backward of the layers before it."""
    torch, args, dev, world, rank = run.torch, run.args, run.dev, run.world, run.rank
    from qkan_b200 import QKAN
    from qkan_b200.parallel import OverlappedGradSync

    depth, width, reps, rows = args.hqkan_layers, 768, 2, 8192
    torch.manual_seed(0)
    layers = torch.nn.ModuleList([QKAN([width, width], reps=reps, device=dev, seed=l, ba_trainable=True)
                                  for l in range(depth)])
    sync = OverlappedGradSync(layers, groups=[[p for p in m.parameters() if p.requires_grad] for m in layers])
    x0 = (torch.randn(rows, width, generator=torch.Generator().manual_seed(300 + rank)) * 0.5).to(torch.bfloat16).to(dev)
    gy = torch.randn(rows, width, generator=torch.Generator().manual_seed(400 + rank)).to(torch.bfloat16).to(dev)

    def step(mark):
        sync.zero_grad()
        h = x0
        for m in layers:
            h = m(h)
        mark()
        h.backward(gy)
        sync.finish()

    total_max_ms, _, segs, clk, wall = run.time_steps(step, args.steps, args.warmup, marks=1)
    ms = total_max_ms / args.steps
    if rank == 0:
        edges = rows * depth * width * width
        roof_ms = 1e3 * issue_roofline_seconds(edges, reps, "fwd_bwd", frozen=True)
        line = {
            "metric": METRIC, "value": edges * world * reps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 I/O, f32 compute", "data": "synthetic",
            "config": {"workload": f"HQKANsformer-shaped stack: {depth} x QKAN [768->768] reps 2, bf16 activations, "
                                   "base term on, 8192 token rows/GPU, fwd+bwd, per-layer gradient all-reduce "
                                   "overlapped with the backward",
                       "parallelism": f"dp{world}", "l2": "flushed between timed steps (256 MB write)",
                       "tokens_per_sec": rows * world * 1e3 / ms},
            "roofline": {"bound": "fp32_issue", "roofline_ms": roof_ms, "frac": roof_ms / ms, "peak": PEAK_ISSUE,
                         "unit": "Tlane-op/s", "achieved": roof_ms / ms * PEAK_ISSUE,
                         "forward_ms": segs[0], "backward_sync_ms": segs[1],
                         "note": "pinned count of the frozen-preact circuit; the base term's two products are not counted"},
            "gpu_launches": 5 * depth * args.steps, "gradient_bytes_per_step": sync.nbytes(), "clocks": clk,
            "wall_s_timed_region": wall,
        }
        print(json.dumps(line))
    run.finish()
    return 0


def count_kernels(torch, fn):
    """(library kernels, all kernels) launched by one call of fn, from torch's profiler."""
    from torch.profiler import ProfilerActivity, profile

    fn()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        fn()
        torch.cuda.synchronize()
    names = [e.name for e in prof.events() if str(e.device_type).endswith("CUDA") and "memcpy" not in e.name.lower()
             and "memset" not in e.name.lower()]
    return sum(1 for n in names if "qk::" in n), len(names)


def run_hqkan_block(run: Run):
    """The launch-bound regime: the hybrid block Linear(768 -> w) -> QKAN[w, w] -> Linear(w -> 768) in bfloat16
    (qkan_b200.FusedHQKAN, w = 10, one repetition), forward + loss + backward, eager and captured in a CUDA graph."""
    torch, args, dev, rank = run.torch, run.args, run.dev, run.rank
    from qkan_b200 import FusedHQKAN
    from qkan_b200.graph import make_graphed_train_step

    table = []
    for rows in (8192, 1024):
        torch.manual_seed(0)
        block = FusedHQKAN(768, 10, reps=1, device=dev)
        x = torch.randn(rows, 768, device=dev, dtype=torch.bfloat16)
        tgt = torch.randn(rows, 768, device=dev, dtype=torch.bfloat16)
        loss_fn = lambda y, t: torch.nn.functional.mse_loss(y.float(), t.float())  # noqa: E731
        opt = torch.optim.SGD(block.parameters(), lr=0.0)

        def eager(mark=lambda: None):
            block.zero_grad(set_to_none=True)
            loss_fn(block(x), tgt).backward()

        lib_k, all_k = count_kernels(torch, eager)
        eager_ms = run.time_steps(eager, args.steps, args.warmup)[0] / args.steps
        graphed = make_graphed_train_step(block, x, tgt, loss_fn, opt)
        graph_ms = run.time_steps(lambda mark: graphed(x, tgt), args.steps, args.warmup)[0] / args.steps
        table.append({"rows": rows, "eager_us": 1e3 * eager_ms, "graphed_us": 1e3 * graph_ms,
                      "library_launches_per_step": lib_k, "all_kernels_per_step": all_k})
    if rank == 0:
        edges = sum(r["rows"] for r in table) * 100
        ms = sum(r["graphed_us"] for r in table) * 1e-3
        line = {
            "metric": METRIC, "value": edges / (ms * 1e-3), "unit": UNIT, "n_gpus": run.world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / len(table), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "hybrid block Linear(768->10) -> QKAN[10,10] reps 1 -> Linear(10->768), bf16, "
                                   "forward + MSE + backward at 8192 and 1024 rows, eager and CUDA-graph replay",
                       "l2": "flushed between timed steps (256 MB write)",
                       "library_kernels": "prep, forward, backward, base_backward, finish_grads"},
            "rows": table, "gpu_launches": sum(r["library_launches_per_step"] for r in table) * args.steps,
        }
        print(json.dumps(line))
    run.finish()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("b200", "reference"), default="b200")
    ap.add_argument("--config", choices=("layer", "bf16_sweep", "mnist", "hqkan", "hqkan_block"), default="layer",
                    help="workload; only the default is the benchmark line")
    ap.add_argument("--scaling", choices=("weak", "strong"), default="weak")
    ap.add_argument("--cpu-rows", type=int, default=1024, help="rows of the C-port CPU sample")
    ap.add_argument("--cpu-ref-rows", type=int, default=192, help="rows of the reference `exact` CPU sample")
    ap.add_argument("--ref-rows", type=int, default=128, help="rows per step of --impl reference")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-baselines", action="store_true", help="skip the reference's GPU solvers (profiling runs)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--e2e-chunks", type=int, default=3, help="row chunks of the host-buffer pipeline")
    ap.add_argument("--variant", choices=tuple(VARIANTS), default="headline",
                    help="extra rows of the microbenchmark; only the default is the benchmark line")
    ap.add_argument("--batch", type=int, default=B_PER_GPU,
                    help="rows per GPU; anything but the default is a profiling-size run, not the benchmark")
    ap.add_argument("--sweep-widths", type=int, nargs="*", help="bf16_sweep: subset of the layer widths")
    ap.add_argument("--sweep-reps", type=int, nargs="*", help="bf16_sweep: subset of the repetition counts")
    ap.add_argument("--hqkan-layers", type=int, default=12)
    ap.add_argument("--eager", action="store_true", help="mnist: eager step with per-layer gradient buckets instead of the CUDA-graph step")
    ap.add_argument("--baseline-arm", choices=("flash", "cute"), help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.baseline_arm:
        return run_baseline_arm(args.baseline_arm)
    if args.impl == "reference":
        return run_reference(args)
    run = Run(args)
    return {"layer": run_layer, "bf16_sweep": run_bf16_sweep, "mnist": run_mnist, "hqkan": run_hqkan,
            "hqkan_block": run_hqkan_block}[args.config](run)


if __name__ == "__main__":
    sys.exit(main())
