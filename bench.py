#!/usr/bin/env python
"""Benchmark of the gated-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Default workload: ``triangle_end_1024`` (triangle attention around the ending node, 1024 x 1024 pair
representation, 723 GFLOP per call). A "step" is ONE such problem: the pair-bias projection of the rows of z,
kutacc_af2_gating_attention on them, and with N > 1 (launched by torch.distributed.run, one rank per GPU)
the two collectives of the sharded flow: the rows are split over the ranks, each rank projects the pair bias
of its rows, the ranks all-gather the bias [4, 1024, 1024] and, after the attention, the output rows
(kutacc_af2_all_gather over NCCL). Total work is fixed as N grows (strong scaling). Rank 0 prints one JSON line:

  value / ms_per_step  whole-job TFLOP/s (algorithmic FLOPs, 2 per multiply-add) with inputs resident
                       in HBM, timed with CUDA events on the launching stream, max over ranks per step
  e2e                  the same problem with each rank's rows of z and of the mask in pinned HOST memory and its
                       output rows delivered to pinned host memory: copies inside the timed region; steps run
                       back to back with the next step's upload beside this step's kernels and download
                       (ms_per_step_alone = one step with nothing else in flight)
  roofline             the dominant kernel (the fused attention core), timed live with CUDA events
  compute_only         the same step with the output rows left sharded (the state the reference operator leaves)
  phases_ms            pair-bias projection, bias all-gather, attention, exposed part of the output gather
  cpu_baseline         the CPU restatement of the reference on the host cores (rank 0, N = 1 only)
  global_attention     N = 1 only: the extra-MSA global column attention (its one-pass kernel against the HBM copy)

Other workloads (``--workload``) that are not triangle shapes, and ``--scaling weak``, run every rank on its
own batch of rows with no collective (weak scaling).

--impl reference times the CPU restatement of the reference's algorithm on the host cores (the
reference's own ARM SVE sources do not compile on this x86 host) on a bounded sample of the same
workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

DEFAULT_WORKLOAD = "triangle_end_1024"
TRIANGLE = ("triangle_start_384", "triangle_end_1024")
METRIC = "gated_attention_tflops"
UNIT = "TFLOP/s"

# DRAM bytes (read + write) of one launch of the dominant kernel from an ncu capture, per workload;
# None until a capture exists for the current kernel. See profiles/.
NCU_TRAFFIC = {
    # attn_tc_kernel, ncu --set full, dram__bytes_read.sum + dram__bytes_write.sum of one launch
    "triangle_start_384": 152.5e6 + 22.0e6,
    # captured on 64 of the 1024 rows and scaled by the rows (the 8.4 MB pair bias does not scale):
    # profiles/attn_core_triangle_end_1024.md
    "triangle_end_1024": (75.7e6 - 8.4e6) * 16 + 8.4e6 + 5.3e6 * 16,
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while a region runs (read-only NVML)."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.samples, self.mem_samples, self.reasons, self.max_mhz = [], [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                self.mem_samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_MEM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "mem_mhz": statistics.median(self.mem_samples) if self.mem_samples else None,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def hbm_copy_gbs(torch, dev, n_bytes=1 << 30, reps=5):
    """Read + write bandwidth of a plain device copy on this GPU right now (the quantity the measured HBM peak
    was taken with): lets a reader tell a slow kernel from a slow box."""
    a = torch.empty(n_bytes, dtype=torch.uint8, device=dev)
    b = torch.empty_like(a)
    b.copy_(a)
    best = None
    for _ in range(reps):
        e0, e1 = _events(torch)
        e0.record()
        b.copy_(a)
        e1.record()
        e1.synchronize()
        ms = e0.elapsed_time(e1)
        best = ms if best is None else min(best, ms)
    del a, b
    torch.cuda.empty_cache()
    return 2.0 * n_bytes / (best * 1e-3) / 1e9


def config_for(name, world, scaling, slabs=None):
    """The `config` object of the JSON line: the same for both arms (`--impl ours` and `--impl reference`)."""
    from kutacc_b200 import workloads as W
    kind, dtype, B, S, H, D, c_z, seed = W.spec(name)
    if scaling == "strong":
        par = (f"rows of one problem over {world} GPU(s)"
               + ("; NCCL all-gather of the projected pair bias and of the output rows, output gather overlapped "
                  "slab by slab" if world > 1 else "; single GPU, no collective"))
    else:
        par = f"every rank runs the whole workload on its own rows ({world} GPU(s)), no collective"
    probe = W.Workload(name=name, kind=kind, dtype=dtype, B=B, S=S, H=H, D=D, seed=seed, c_z=c_z,
                       has_nb=bool(c_z) and kind == "gating")
    return {"workload": name, "B": B, "S": S, "H": H, "D": D, "C": H * D, "pair_bias": probe.has_nb,
            "gflop_per_call": probe.flops() / 1e9, "l2": "flushed between timed steps (256 MiB memset)",
            "parallelism": par}


def dominant_kernel(workload, rows=None):
    """(kernel name in the library's profile record, bound, algorithmic work per call, unit)."""
    B = workload.B if rows is None else rows
    if workload.kind == "gating":
        # Q.K^T and P.V: 4*B*S^2*C FLOPs, all inside the fused attention core
        return "attn_core", "tensor", 4.0 * B * workload.S * workload.S * workload.C, "TFLOP/s"
    # global attention: one kernel reads x once and writes out once: bandwidth bound
    return "global_fused", "hbm", 2.0 * B * workload.S * workload.C * 2, "GB/s"


def torch_cpu_gating(w, reps: int = 3):
    """The same operator written with torch CPU ops in the workload's dtype (oneDNN bf16 GEMMs), all host
    threads: a second, library-grade CPU number beside the restatement of the reference's own loops."""
    import torch
    dt = torch.bfloat16 if w.dtype == "bf16" else torch.float32
    A = {k: torch.from_numpy(v).to(dt) for k, v in w.arrays.items() if k in ("x", "wq", "wk", "wv", "wg", "wo", "bias", "nb")}
    bg, bo = torch.from_numpy(w.arrays["bg"]).to(dt), torch.from_numpy(w.arrays["bo"]).to(dt)
    B, S, H, D = w.B, w.S, w.H, w.D

    def run():
        x = A["x"]
        q = (x @ A["wq"].T).view(B, S, H, D).transpose(1, 2)
        k = (x @ A["wk"].T).view(B, S, H, D).transpose(1, 2)
        v = (x @ A["wv"].T).view(B, S, H, D).transpose(1, 2)
        gate = torch.sigmoid(x @ A["wg"].T + bg)
        logits = (q @ k.transpose(-1, -2)) * (1.0 / D ** 0.5) + A["bias"][:, None, None, :]
        if "nb" in A:
            logits = logits + A["nb"][None]
        p = torch.softmax(logits.float(), dim=-1).to(dt)
        avg = (p @ v).transpose(1, 2).reshape(B, S, H * D) * gate
        return avg @ A["wo"].T + bo

    with torch.no_grad():
        run()
        times = []
        for _ in range(reps):
            t0 = time.perf_counter()
            run()
            times.append(time.perf_counter() - t0)
    t = min(times)
    return {"value": w.flops(pair_bias=False) / t / 1e12, "unit": UNIT, "threads": torch.get_num_threads(),
            "ms_per_pass": t * 1e3, "sample_rows": w.B}


def cpu_baseline(name: str, budget_s: float = 12.0):
    """CPU restatement of the reference on a bounded sample (a subset of the batch rows). The pair bias is an
    input of the reference operator, so its projection is outside both the timed pass and the FLOP count."""
    from kutacc_b200 import workloads as W
    from oracle import cpu_oracle as O
    from tests import helpers
    kind, dtype, B, S, H, D, c_z, seed = W.spec(name)
    rows = min(B, 8)
    w = W.make(name, rows=rows)
    run = (lambda ww: helpers.oracle_exact(ww)) if dtype == "fp32" else (lambda ww: helpers.oracle_faithful(ww))
    t0 = time.perf_counter()
    run(w)
    t_probe = time.perf_counter() - t0
    # grow the sample so that one pass takes a few seconds, then repeat within the budget
    rows2 = int(min(B, max(rows, rows * 3.0 / max(t_probe, 1e-3))))
    if rows2 != rows:
        w = W.make(name, rows=rows2)
    times = []
    t_start = time.perf_counter()
    while len(times) < 5 and (time.perf_counter() - t_start < budget_s or not times):
        t0 = time.perf_counter()
        run(w)
        times.append(time.perf_counter() - t0)
    t = min(times)
    torch_cpu = None
    if kind == "gating":
        try:
            torch_cpu = torch_cpu_gating(w)
        except Exception as exc:                                       # a second opinion only: never fatal
            torch_cpu = {"error": str(exc)[:200]}
    return {"value": w.flops(pair_bias=False) / t / 1e12, "unit": UNIT, "cores": O.num_threads(), "kind": "port",
            "torch_cpu": torch_cpu,
            "sample": f"{w.B} of {B} batch rows of {name} (full sequence length {S}), best of {len(times)} runs, "
                      f"{t * 1e3:.1f} ms per pass",
            "ms_full_call_est": t * 1e3 * B / w.B}


def run_reference_arm(args):
    """The reference's CPU implementation, as restated in oracle/ (the ARM sources do not compile here)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return 0
    # torchrun gives every rank OMP_NUM_THREADS=1; rank 0 alone runs the CPU arm and may use every host core
    # (the OpenMP runtime reads the variable when the oracle library is loaded, below)
    if world > 1:
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    from kutacc_b200 import workloads as W
    from oracle import cpu_oracle as O
    from tests import helpers
    if world > 1:
        O.set_num_threads(os.cpu_count() or 1)
    name = args.workload
    kind, dtype, B, S, H, D, c_z, seed = W.spec(name)
    run = (lambda ww: helpers.oracle_exact(ww)) if dtype == "fp32" else (lambda ww: helpers.oracle_faithful(ww))
    probe = W.make(name, rows=min(B, 4))
    t0 = time.perf_counter()
    run(probe)
    t_row = (time.perf_counter() - t0) / probe.B
    total_steps = args.steps + args.warmup
    rows = int(max(1, min(B, 150.0 / max(total_steps, 1) / max(t_row, 1e-6))))
    w = W.make(name, rows=rows) if rows != probe.B else probe
    for _ in range(args.warmup):
        run(w)
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        run(w)
        times.append(time.perf_counter() - t0)
    t = sum(times) / len(times)
    val = w.flops(pair_bias=False) / t / 1e12
    sample = f"{rows} of {B} batch rows of {name} per step (full sequence length {S})"
    scaling = resolve_scaling(args, name)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": dtype, "data": "synthetic (seeded numpy, AlphaFold2 model shapes)",
        "config": config_for(name, max(world, args.gpus, 1), scaling),
        "note": "CPU restatement of the reference algorithm (oracle/), host cores only; ms_per_step is the time of the "
                "sampled rows, value is per-row throughput and does not depend on the sample size",
        "ms_full_call_est": t * 1e3 * B / rows,
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": O.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(json.dumps(line))
    return 0


def resolve_scaling(args, name):
    if args.scaling != "auto":
        return args.scaling
    return "strong" if name in TRIANGLE else "weak"


def _events(torch):
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def global_attention_extra(torch, api, W, runner, dev, peaks, steps=10):
    """The extra-MSA global column attention (one launch of the one-pass kernel) on this GPU: device time per
    call and the achieved fraction of the measured HBM copy bandwidth."""
    g = W.make("extra_msa_global")
    case = runner.DeviceCase(g, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    api.set_async(True)
    try:
        for _ in range(3):
            case.run()
        torch.cuda.synchronize()
        ms = []
        for _ in range(steps):
            flush.zero_()
            e0, e1 = _events(torch)
            e0.record()
            case.run()
            e1.record()
            e1.synchronize()
            ms.append(e0.elapsed_time(e1))
        api.synchronize()
        api.raise_if_error()
    finally:
        api.set_async(False)
    t = sum(ms) / len(ms)
    nbytes = 2.0 * g.B * g.S * g.C * 2
    gbs = nbytes / (t * 1e-3) / 1e9
    del case, flush
    torch.cuda.empty_cache()
    return {"workload": "extra_msa_global", "ms_per_call": t, "value": g.flops() / (t * 1e-3) / 1e12, "unit": UNIT,
            "roofline": {"kernel": "global_fused", "bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} (copy)",
                         "algorithmic_bytes": nbytes}}


def run_strong_scaling(args, torch, dist, api, W, runner, dev, world, rank, local_rank):
    """One triangle-attention problem split over the ranks: pair-bias projection, bias all-gather, attention
    on this rank's rows, output all-gather (kutacc_b200/sharding.py). Total work is fixed as N grows."""
    from kutacc_b200 import sharding
    w = W.make(args.workload, with_nb=False)
    if not (w.kind == "gating" and "wb" in w.arrays and w.B == w.S):
        raise SystemExit("--scaling strong needs a triangle workload (triangle_start_384, triangle_end_1024)")
    if args.sm_margin < 0:
        args.sm_margin = args.nccl_ctas if world > 1 else 0
    if world > 1:
        if args.nccl_ctas > 0:
            os.environ["KUTACC_NCCL_MAX_CTAS"] = str(args.nccl_ctas)
        uid = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            uid = torch.tensor(list(api.comm_unique_id()), dtype=torch.uint8, device=dev)
        dist.broadcast(uid, 0)
        api.comm_init(world, rank, 0, bytes(uid.cpu().tolist()))
    slabs = args.slabs if world > 1 else 1
    op = sharding.ShardedTriangleAttention(w, rank, world, slabs, dev, sm_margin=args.sm_margin,
                                           bias_gather_beside=not args.bias_gather_inline)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows_per_rank = w.B // world

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values):
        t = torch.tensor(values, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def timed(n, gather):
        out_ms, phases = [], []
        for _ in range(n):
            flush.zero_()
            barrier()                                                 # ranks enter the step together
            e0, e1 = _events(torch)
            e0.record()
            op.step(gather_output=gather)
            e1.record()
            e1.synchronize()
            out_ms.append(e0.elapsed_time(e1))
            phases.append(op.phase_ms())
        return out_ms, phases

    for _ in range(args.warmup):
        op.step(gather_output=not args.leave_sharded)
    barrier()
    launches0 = api.launch_count()
    with ClockSampler(local_rank) as clocks:
        step_ms, phases = timed(args.steps, not args.leave_sharded)
        barrier()
    launches = api.launch_count() - launches0
    api.synchronize()
    api.raise_if_error()
    step_ms = max_over_ranks(step_ms)                                  # per step, the slowest rank
    ms_per_step = sum(step_ms) / args.steps
    value = w.flops() / (ms_per_step * 1e-3) / 1e12
    names = list(phases[0])
    ph = max_over_ranks([sum(p[k] for p in phases) / len(phases) for k in names])
    phases_ms = {k: round(v, 4) for k, v in zip(names, ph)}

    # the same step with the output rows left sharded (what the reference operator itself leaves behind)
    n_co = max(3, min(args.steps, 10))
    co_ms, _ = timed(n_co, False)
    co = sum(max_over_ranks(co_ms)) / n_co
    compute_only = {"ms_per_step": co, "value": w.flops() / (co * 1e-3) / 1e12, "unit": UNIT,
                    "note": "output rows left sharded over the ranks (no output all-gather)"}

    # per-kernel CUDA events (they cost a few per cent of a step, so they run in a pass of their own)
    api.set_profile(True)
    api.profile_read()
    n_prof = max(3, min(args.steps, 10))
    timed(n_prof, not args.leave_sharded)
    barrier()
    prof = api.profile_read()
    api.set_profile(False)
    api.synchronize()
    api.raise_if_error()
    per_kernel = {}
    for n, ms in prof:
        per_kernel.setdefault(n, []).append(ms)
    peaks = measured_peaks()
    roofline = None
    if "attn_core" in per_kernel:
        k_ms = max_over_ranks([sum(per_kernel["attn_core"]) / n_prof])[0]      # the slowest rank's kernel time per step
        work = 4.0 * rows_per_rank * w.S * w.S * w.C
        achieved = work / (k_ms * 1e-3) / 1e12
        tot = max(sum(sum(v) for v in per_kernel.values()), 1e-9)
        traffic = NCU_TRAFFIC.get(args.workload)
        roofline = {"kernel": "attn_core", "bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
                    "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                    "traffic": traffic * rows_per_rank / w.B if traffic else None,
                    "peak_source": f"{peaks['source']} (burst bf16)", "kernel_ms_per_step": k_ms,
                    "launches_per_step": len(per_kernel["attn_core"]) / n_prof,
                    "algorithmic_flops_per_step_per_gpu": work,
                    "measured": "CUDA events around every kernel on its stream, per rank (slowest rank reported), in a "
                                "pass of the same steps directly after the timed region",
                    "time_share": {n: round(sum(v) / tot, 4) for n, v in per_kernel.items()}}
    checksum = float(op.out_full.float().abs().mean().item())
    del op
    torch.cuda.empty_cache()

    # end to end: this rank's rows of z and of the mask bias start in pinned host memory, its output rows end there
    e2e = None
    if not args.no_e2e:
        host = sharding.HostShardedTriangleAttention(w, rank, world, dev)
        # (a) one step on its own: upload, kernels and download of the same step, nothing else in flight
        for _ in range(2):
            host.step(prefetch=False)
        barrier()
        l_ms = []
        for _ in range(3):
            barrier()
            e0, e1 = _events(torch)
            e0.record()
            host.step(prefetch=False)
            e1.record()
            e1.synchronize()
            l_ms.append(e0.elapsed_time(e1))
        l_ms = max_over_ranks(l_ms)
        # (b) steps back to back, two in flight: a step sends the NEXT step's rows while its own kernels and
        # download run (the attention needs the pair bias of every row, so inside one step nothing can overlap the
        # upload). K uploads and K downloads lie inside the timed region: the first timed step's rows were sent by
        # the last warm-up step, and the region ends only when the rows the last step sent have arrived.
        n_e2e = max(3, min(args.steps, 10))
        for _ in range(2):
            host.step()
        barrier()
        e0, e1 = _events(torch)
        e0.record()
        for _ in range(n_e2e):
            host.step()
        host.drain()
        e1.record()
        e1.synchronize()
        api.synchronize()
        api.raise_if_error()
        em = max_over_ranks([e0.elapsed_time(e1)])[0] / n_e2e
        # host<->device copies alone, per rank, so that a host-side limit shows when N grows
        c_up, c_dn = [], []
        for _ in range(3):
            barrier()
            e0, e1 = _events(torch)
            e0.record()
            host.xs[0].copy_(host.hx, non_blocking=True)
            e1.record()
            e1.synchronize()
            c_up.append(e0.elapsed_time(e1))
            barrier()
            e0, e1 = _events(torch)
            e0.record()
            host.hout.copy_(host.xs[0], non_blocking=True)
            e1.record()
            e1.synchronize()
            c_dn.append(e0.elapsed_time(e1))
        up, dn = max_over_ranks([min(c_up)])[0], max_over_ranks([min(c_dn)])[0]
        e2e = {"value": w.flops() / (em * 1e-3) / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": host.h2d_bytes() * world, "d2h_bytes_per_step": host.d2h_bytes() * world,
               "ms_per_step": em, "steps_in_flight": 2, "steps_timed": n_e2e,
               "ms_per_step_alone": sum(l_ms) / len(l_ms),
               "result_mean_abs": float(host.hout.float().abs().mean()),
               "copies_alone_ms": {"h2d_rows": up, "d2h_rows": dn,
                                   "h2d_gbs_per_gpu": host.hx.numel() * 2 / (up * 1e-3) / 1e9,
                                   "d2h_gbs_per_gpu": host.hout.numel() * 2 / (dn * 1e-3) / 1e9},
               "note": "bytes are the whole job's (all ranks); every rank moves its own rows; the output rows stay "
                       "sharded in the node's host memory (nothing is gathered on the way out). value: steps back to "
                       "back, the upload of step i+1 beside the kernels and the download of step i; "
                       "ms_per_step_alone: one step with nothing else in flight"}
        del host
        torch.cuda.empty_cache()
    if world > 1:
        api.comm_fini()

    copy_now = hbm_copy_gbs(torch, dev) if rank == 0 else None
    cpu = glob = None
    if rank == 0 and world == 1:
        if not args.no_cpu_baseline:
            cpu = cpu_baseline(args.workload)
        if not args.no_global:
            glob = global_attention_extra(torch, api, W, runner, dev, peaks)
    if rank == 0:
        cfg = config_for(args.workload, world, "strong")
        emit(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": w.dtype, "data": "synthetic (seeded numpy, AlphaFold2 model shapes)",
            "config": cfg,
            "details": {"slabs": slabs, "sm_margin": args.sm_margin if world > 1 else 0,
                        "nccl_max_ctas": args.nccl_ctas if world > 1 else 0,
                        "output_gathered": (not args.leave_sharded) and world > 1, "rows_per_gpu": rows_per_rank,
                        "call_mode": "value: enqueue-only calls (kutacc_b200_set_async), device time by CUDA events; "
                                     "e2e: host rows in, host rows out"},
            "frac_of_bf16_peak": value / world / peaks["bf16_tflops"],
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches),
            "compute_only": compute_only, "phases_ms": phases_ms, "global_attention": glob,
            "result_mean_abs": checksum, "clocks": clocks.summary(), "hbm_copy_gbs_now": copy_now,
        }))
    return 0


_RESULT_FD = None


def keep_stdout_for_the_result():
    """Libraries loaded below write to the process's standard output on their own (NCCL prints its version line
    there when NCCL_DEBUG asks for it). The contract is ONE JSON line on stdout, so file descriptor 1 is pointed at
    stderr for the rest of the run and the result line goes to a saved copy of the original stdout."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line: str):
    sys.stdout.flush()
    if _RESULT_FD is None:
        print(line, flush=True)
    else:
        os.write(_RESULT_FD, (line + "\n").encode())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-global", action="store_true", help="skip the extra global-attention measurement (N = 1)")
    ap.add_argument("--rows", type=int, default=0,
                    help="profiling aid (weak mode): run only this many of the workload's batch rows (0 = all); the "
                         "JSON line then describes that smaller case and is not a benchmark result")
    ap.add_argument("--scaling", default="auto", choices=["auto", "weak", "strong"],
                    help="strong: one triangle workload split over the ranks with the two all-gathers (default for the "
                         "triangle workloads); weak: every rank runs the whole workload on its own rows, no "
                         "collective (default for the others)")
    ap.add_argument("--sm-margin", type=int, default=-1,
                    help="strong scaling: SMs the kernels leave to NCCL (default: the value of --nccl-ctas)")
    ap.add_argument("--nccl-ctas", type=int, default=0,
                    help="strong scaling: upper bound on the CTAs of the library's NCCL collectives (0 = NCCL's own choice, "
                         "which measured best on 2 GPUs: 1.99 ms against 2.07 ms with 16 CTAs and a margin of 16 SMs)")
    ap.add_argument("--leave-sharded", action="store_true",
                    help="strong scaling: skip the all-gather of the output rows in the headline figure too")
    ap.add_argument("--bias-gather-inline", action="store_true",
                    help="strong scaling: run the bias all-gather on the compute stream instead of beside the projections")
    ap.add_argument("--slabs", type=int, default=2, help="strong scaling: slabs the output gather is pipelined in")
    args = ap.parse_args()
    keep_stdout_for_the_result()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    args.steps = max(args.steps, 1)

    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import torch.distributed as dist
    from kutacc_b200 import api, build, runner
    from kutacc_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(dev))
    if not os.path.exists(api.LIB_PATH):
        build.build()
    api.lib()

    scaling = resolve_scaling(args, args.workload)
    if scaling == "strong" and args.rows <= 0:
        rc = run_strong_scaling(args, torch, dist, api, W, runner, dev, world, rank, local_rank)
        if world > 1:
            dist.destroy_process_group()
        return rc

    w = W.make(args.workload, rows=args.rows) if args.rows > 0 else W.make(args.workload)
    case = runner.DeviceCase(w, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # larger than the 126 MB L2

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Device-resident timing uses the library's enqueue-only mode (kutacc_b200_set_async): the call returns
    # when its kernels are queued and the CUDA events bracket device time only. The synchronous default of the
    # C ABI (what a caller of the reference sees) is what the end-to-end figure below measures.
    api.set_async(True)
    for _ in range(args.warmup):
        case.run()
    barrier()
    launches0 = api.launch_count()

    def timed_steps():
        out_ms = []
        for _ in range(args.steps):
            flush.zero_()                                             # evict L2 between timed steps
            e0, e1 = _events(torch)
            e0.record()
            case.run()
            e1.record()
            e1.synchronize()
            out_ms.append(e0.elapsed_time(e1))
        return out_ms

    with ClockSampler(local_rank) as clocks:
        step_ms = timed_steps()
        barrier()
    launches = api.launch_count() - launches0
    api.synchronize()
    api.raise_if_error()
    # Per-kernel CUDA events cost a few per cent of a step, so the timed region above runs without them; the
    # same K steps are repeated right away with the events on for the kernel breakdown.
    api.set_profile(True)
    api.profile_read()
    timed_steps()
    barrier()
    prof = api.profile_read()
    api.set_profile(False)
    api.synchronize()
    api.raise_if_error()
    api.set_async(False)
    total_ms = float(sum(step_ms))
    if world > 1:
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    # the pair bias is an input of this call (projected beforehand), so its projection is not counted
    flops_job = w.flops(pair_bias=False) * world
    value = flops_job / (ms_per_step * 1e-3) / 1e12

    # dominant kernel, timed live inside the same steps
    kname, bound, work, runit = dominant_kernel(w)
    per_kernel = {}
    for n, ms in prof:
        per_kernel.setdefault(n, []).append(ms)
    kshare = {n: sum(v) / max(sum(sum(x) for x in per_kernel.values()), 1e-9) for n, v in per_kernel.items()}
    peaks = measured_peaks()
    roofline = None
    if kname == "attn_core" and kname not in per_kernel and "attn_f32" in per_kernel:
        kname = "attn_f32"            # the fp32 shape runs the error-compensated tf32 kernel (three products per multiply)
    if kname == "global_fused" and kname not in per_kernel:
        kname = "global_out"          # shapes the one-pass kernel does not cover run the three-kernel path
    if kname in per_kernel:
        launches_per_step = len(per_kernel[kname]) / args.steps
        k_ms = sum(per_kernel[kname]) / args.steps                    # all launches of that kernel in one step
        achieved = work / (k_ms * 1e-3) / (1e12 if bound == "tensor" else 1e9)
        peak = peaks["bf16_tflops"] if bound == "tensor" else peaks["hbm_gbs"]
        traffic = NCU_TRAFFIC.get(args.workload)
        _, _, Bfull = W.spec(args.workload)[:3]
        roofline = {"kernel": kname, "bound": bound, "achieved": achieved, "peak": peak, "unit": runit,
                    "frac": achieved / peak, "traffic": traffic * w.B / Bfull if traffic else None,
                    "peak_source": f"{peaks['source']} ({'burst bf16' if bound == 'tensor' else 'copy'})",
                    "kernel_ms_per_step": k_ms, "launches_per_step": launches_per_step,
                    "measured": "CUDA events around every kernel on its stream, in a second pass of the same K steps "
                                "directly after the timed region (the events themselves cost a few per cent of a step)",
                    "time_share": {n: round(s, 4) for n, s in kshare.items()}}

    # end to end: every tensor in pinned host memory, copies inside the library call
    e2e = None
    if not args.no_e2e:
        host = runner.HostCase(w)
        for _ in range(2):
            host.run()
        barrier()
        e_ms = []
        for _ in range(max(3, min(args.steps, 10))):
            e0, e1 = _events(torch)
            e0.record()
            host.run()
            e1.record()
            e1.synchronize()
            e_ms.append(e0.elapsed_time(e1))
        em = float(sum(e_ms) / len(e_ms))
        if world > 1:
            t = torch.tensor([em], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            em = float(t.item())
        e2e = {"value": flops_job / (em * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": host.h2d_bytes(),
               "d2h_bytes_per_step": host.d2h_bytes(), "ms_per_step": em}
        checksum = float(host.out.float().abs().mean())               # read the result on the host
        e2e["result_mean_abs"] = checksum

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and args.rows <= 0:
        cpu = cpu_baseline(args.workload)

    if rank == 0:
        cfg = config_for(args.workload, world, "weak")
        if args.rows > 0:
            cfg["rows_run"] = w.B
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": w.dtype, "data": "synthetic (seeded numpy, AlphaFold2 model shapes)",
            "config": cfg,
            "details": {"call_mode": "value: enqueue-only calls (kutacc_b200_set_async), device time by CUDA events; "
                                     "e2e: the synchronous default with host buffers",
                        "flops": "the pair bias is an input of the timed call: its projection is neither run nor counted"},
            "frac_of_bf16_peak": value / world / peaks["bf16_tflops"],
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches),
            "clocks": clocks.summary(), "hbm_copy_gbs_now": hbm_copy_gbs(torch, dev),
        }
        emit(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
