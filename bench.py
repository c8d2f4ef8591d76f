#!/usr/bin/env python
"""Benchmark of the NVFP4 GEMM -> grouped GEMM -> fused-MoE path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload W]

One JSON line on stdout (rank 0). The headline `value` is the dense GEMM; the same line carries
the other half of the metric and the remaining configurations as extra objects:

  value / e2e / roofline   N = 1: M = N = K = 8192 NVFP4 GEMM, FP16 output (the shape the "% of FP4
                           peak" target is quoted on). N > 1: M = 16384, N = 28672, K = 8192 with B
                           split by columns over the ranks, no collective (strong scaling).
  "sustained"              (N = 1) the same GEMM launched back to back for >= 2 s, with the SM clock
                           sampled meanwhile, against the sustained cuBLAS bf16 figure.
  "sweep"                  (N = 1) M = 16 / 128 / 256 / 1024 / 4096 at N = 4096, K = 8192 through
                           the default dispatcher, and the grouped GEMM of 8 experts x 2048 rows
                           (Dirichlet(0.5) split, per-expert alpha): mean / P50 / P95 per call,
                           TFLOP/s, algorithmic GB/s, both roofline fractions, a CPU-oracle figure.
  "moe"                    the DeepSeek-V3-shaped fused-MoE layer (hidden 7168, intermediate 2048,
                           256 experts, top-8) in tokens/s. N = 1: T = 4096 on one GPU. N > 1:
                           expert parallel over the ranks, a weak reading (T = 4096 per rank) and a
                           strong one (T = 4096 in total), each with the phases of the slowest rank.

`--workload gemm8192 | gemm4096 | gemm_nshard | moe | gemm_m16 | gemm_sweep | grouped_c3` runs one
workload alone (gemm4096 is the small case for profiler captures).

A step is one pass of the hot path over one batch. `value` is device-timed with the inputs
resident in HBM; `e2e` times the same call with host buffers (pinned host -> device copy of the
step's inputs, the call through the C ABI, device -> host copy of the result). Operands are seeded
normal data (BF16-rounded) quantised to NVFP4 by this library's row quantiser. The CPU oracle is
only ever the thing measured in the `cpu_baseline` / `cpu_tflops` / `--impl reference` legs.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "NVFP4 GEMM TFLOPS (% FP4 peak); fused-MoE tokens/s at 1/2/4/8 B200"
NOMINAL_FP4_TFLOPS = 9000.0      # dense FP4 per B200 (vendor figure without sparsity)
FALLBACK_BF16_TFLOPS = 1590.0    # used only when MEASURED_PEAKS.json is absent
FALLBACK_BF16_SUSTAINED = 1400.0
FALLBACK_HBM_GBS = 6650.0
L2_NOTE = "256 MiB flush write between timed steps"


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return {"bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
        except Exception:
            pass
    return {"bf16_tflops": FALLBACK_BF16_TFLOPS, "bf16_tflops_sustained": FALLBACK_BF16_SUSTAINED,
            "hbm_gbs": FALLBACK_HBM_GBS, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._proc = None
        self._thread = None

    def start(self):
        query = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                 "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={query}",
                                           "--format=csv,noheader,nounits", "-lms", "20"],
                                          stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self._proc = None
            return self
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()
        t0 = time.time()
        while not self.samples and time.time() - t0 < 5.0:
            time.sleep(0.02)
        return self

    def _read(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                self.samples.append((time.time(), float(parts[0])))
                self.max_mhz = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    self.reasons.add(name)

    def stop(self, window=None):
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except Exception:
                self._proc.kill()
        if self._thread is not None:
            self._thread.join(timeout=5)
        vals = [v for (t, v) in self.samples if window is None or window[0] <= t <= window[1]]
        note = "samples inside the timed region"
        if not vals and self.samples:  # region shorter than the sampling period: nearest sample
            mid = 0.5 * (window[0] + window[1])
            vals = [min(self.samples, key=lambda s: abs(s[0] - mid))[1]]
            note = "timed region shorter than the sampling period: nearest sample"
        med = float(np.median(vals)) if vals else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(vals), "note": note}


# --------------------------------------------------------------------------- data


def align(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def scale_k_padded(k: int) -> int:
    return align((k + 15) // 16, 4)


def quantized_normal(rows: int, k: int, seed: int, device, sigma: float = 1.0, chunk_rows: int = 4096):
    """Seeded N(0, sigma^2) values, rounded to BF16 and quantised to NVFP4 by the library's row
    quantiser (one UE4M3 scale = amax / 6 per 16 values). Returns (payload [rows, k / 2], scale region
    of align128(rows) * scale_k_padded(k) bytes in the block-scaled layout, padding zero)."""
    import sm120_nvfp4_b200 as ops
    g = torch.Generator(device=device).manual_seed(seed)
    skp = scale_k_padded(k)
    payload = torch.empty((rows, k // 2), dtype=torch.uint8, device=device)
    region = torch.zeros(align(rows, 128) * skp, dtype=torch.uint8, device=device)
    for r0 in range(0, rows, chunk_rows):       # chunk_rows is a multiple of 128: whole scale atoms per chunk
        n = min(rows, r0 + chunk_rows) - r0
        x = torch.randn((n, k), device=device, generator=g)
        if sigma != 1.0:
            x *= sigma
        x = x.to(torch.bfloat16)
        m_pad = align(n, 128)
        seq = torch.tensor([n], dtype=torch.int32, device=device)
        cu = torch.tensor([0, n], dtype=torch.int32, device=device)
        ops.quantize_expert(x, seq, cu, scale_m_pad=m_pad, output=payload[r0:r0 + n],
                            output_scale=region[r0 * skp:(r0 + m_pad) * skp].view(1, -1))
    return payload, region


def quantized_expert_weights(experts: int, rows: int, k: int, seed: int, device, sigma: float, chunk: int = 4):
    """[experts, rows, k] seeded N(0, sigma^2) weights -> NVFP4 (ops.pack_weights), a few experts at a time."""
    import sm120_nvfp4_b200 as ops
    g = torch.Generator(device=device).manual_seed(seed)
    payload = torch.empty((experts, rows, k // 2), dtype=torch.uint8, device=device)
    scales = torch.empty((experts, align(rows, 128) * scale_k_padded(k)), dtype=torch.uint8, device=device)
    for e0 in range(0, experts, chunk):
        n = min(experts, e0 + chunk) - e0
        w = (torch.randn((n, rows, k), device=device, generator=g) * sigma).to(torch.bfloat16)
        p, s = ops.pack_weights(w)
        payload[e0:e0 + n] = p
        scales[e0:e0 + n] = s
    return payload, scales


# ------------------------------------------------------------------------ distributed


def dist_setup():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        dist.init_process_group("nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", local_rank))
    return world, rank, local_rank


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def max_over_ranks(value: float, world: int, device) -> float:
    if world == 1:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_steps(fn, steps: int, warmup: int, world: int, device, flush):
    """W untimed steps, then K steps timed one by one with CUDA events on the current stream (an L2
    flush - a write of a buffer larger than L2 - sits between steps, outside the events), bracketed
    by a barrier + synchronize on both sides. Returns (mean ms per step as the max over ranks, the
    per-step list of this rank)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    barrier(world)
    torch.cuda.synchronize()
    per_step = []
    for _ in range(steps):
        if flush is not None:
            flush.zero_()
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        per_step.append(start.elapsed_time(end))
    torch.cuda.synchronize()
    barrier(world)
    torch.cuda.synchronize()
    return max_over_ranks(float(np.mean(per_step)), world, device), per_step


def percentiles(per_step_ms):
    a = np.asarray(per_step_ms, dtype=np.float64)
    return {"p50_ms": float(np.percentile(a, 50)), "p95_ms": float(np.percentile(a, 95))}


# ------------------------------------------------------------------------ GEMM workloads


def gemm_config(name, m, n, k, world):
    return {"workload": name, "m": m, "n": n, "k": k, "n_per_rank": n // world, "l2": L2_NOTE}


def gemm_shape(workload: str, world: int):
    if workload == "gemm8192":
        return "gemm_m8192_n8192_k8192", 8192, 8192 * world, 8192, "weak"
    if workload == "gemm4096":
        return "gemm_m4096_n4096_k8192", 4096, 4096 * world, 8192, "weak"
    if workload == "gemm_m16":
        return "gemm_m16_n4096_k8192", 16, 4096 * world, 8192, "weak"
    return "gemm_nsharded_m16384_n28672_k8192", 16384, 28672, 8192, "strong"


class GemmWorkload:
    """One dense NVFP4 GEMM through the default dispatcher (b200_nvfp4_gemm_auto)."""

    def __init__(self, m, n_total, k, world, rank, device, name, seed=0xB2000500):
        from sm120_nvfp4_b200 import _lib
        self.L = _lib.lib()
        self.m, self.k, self.n_total = m, k, n_total
        self.n = n_total // world          # this rank's column block of B / C
        self.name = name
        self.device = device
        self.a, self.sfa = quantized_normal(m, k, seed, device)                       # A replicated
        self.b, self.sfb = quantized_normal(self.n, k, seed + 0x10 + rank, device)     # B shard
        self.c = torch.empty((m, self.n), dtype=torch.float16, device=device)
        ws_bytes = self.L.b200_nvfp4_gemm_workspace_bytes(m, self.n, k)
        self.ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
        self.ws_bytes = ws_bytes
        self.path = self.L.b200_nvfp4_gemm_path_string(self.L.b200_nvfp4_gemm_path(m, self.n, k)).decode()
        self.flops_total = 2.0 * m * n_total * k
        self.flops_rank = 2.0 * m * self.n * k
        self.bytes_rank = m * k / 2 + self.n * k / 2 + self.sfa.numel() + self.sfb.numel() + 2 * m * self.n
        self.host = None

    def step(self):
        st = torch.cuda.current_stream().cuda_stream
        status = self.L.b200_nvfp4_gemm_auto(self.m, self.n, self.k, self.a.data_ptr(), self.b.data_ptr(),
                                             self.sfa.data_ptr(), self.sfb.data_ptr(), self.c.data_ptr(),
                                             self.ws.data_ptr(), self.ws_bytes, st)
        if status != 0:
            raise RuntimeError(f"gemm failed with status {status}")

    def prepare_e2e(self):
        self.host = {name: torch.empty(t.shape, dtype=t.dtype).pin_memory().copy_(t.cpu())
                     for name, t in (("a", self.a), ("b", self.b), ("sfa", self.sfa), ("sfb", self.sfb))}
        self.host_c = torch.empty(self.c.shape, dtype=self.c.dtype).pin_memory()
        self.h2d = sum(t.numel() * t.element_size() for t in self.host.values())
        self.d2h = self.host_c.numel() * self.host_c.element_size()

    def step_e2e(self):
        # the library's host-memory entry point: operands and result in page-locked host memory, the
        # device buffers are its scratch; chunked copies both ways overlap with the blocks' GEMMs
        st = torch.cuda.current_stream().cuda_stream
        h = self.host
        status = self.L.b200_nvfp4_gemm_host(self.m, self.n, self.k, h["a"].data_ptr(), h["b"].data_ptr(),
                                             h["sfa"].data_ptr(), h["sfb"].data_ptr(), self.host_c.data_ptr(),
                                             self.a.data_ptr(), self.b.data_ptr(), self.sfa.data_ptr(),
                                             self.sfb.data_ptr(), self.c.data_ptr(), 0, 0, st)
        if status != 0:
            raise RuntimeError(f"host-memory gemm failed with status {status}")

    def metric(self, ms):
        return self.flops_total / (ms * 1e-3) / 1e12


def gemm_roofline(flops, nbytes, mean_ms, peaks):
    """Both fractions of a GEMM launch: tensor (4 x the measured cuBLAS bf16 burst; no FP4 figure is
    measured on this pool and FP4 : BF16 is nominally 4) and HBM (measured copy bandwidth)."""
    sec = mean_ms * 1e-3
    tf, gbs = flops / sec / 1e12, nbytes / sec / 1e9
    fp4_peak = 4.0 * peaks["bf16_tflops"]
    return {"tflops": tf, "algorithmic_gbs": gbs, "frac_tensor": tf / fp4_peak, "frac_hbm": gbs / peaks["hbm_gbs"],
            "frac_tensor_of_nominal_9pf": tf / NOMINAL_FP4_TFLOPS}


def run_gemm(args, world, rank, device, peaks):
    from sm120_nvfp4_b200 import _lib
    name, m, n_total, k, scaling = gemm_shape(args.workload, world)
    wl = GemmWorkload(m, n_total, k, world, rank, device, name)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    wl.step()
    torch.cuda.synchronize()
    launches0 = _lib.launch_count()
    wl.step()
    launches_per_step = _lib.launch_count() - launches0
    sampler = ClockSampler(torch.cuda.current_device()).start()
    t_begin = time.time()
    ms, per_step = time_steps(wl.step, args.steps, args.warmup, world, device, flush)
    clocks = sampler.stop((t_begin, time.time()))
    value = wl.metric(ms)

    wl.prepare_e2e()
    e2e_steps = min(args.steps, 300)
    ms_e2e, _ = time_steps(wl.step_e2e, e2e_steps, 3, world, device, None)
    e2e_value = wl.metric(ms_e2e)

    fp4_peak = 4.0 * peaks["bf16_tflops"]
    mean_rank = float(np.mean(per_step))
    achieved = wl.flops_rank / (mean_rank * 1e-3) / 1e12
    hbm_bound = wl.flops_rank / wl.bytes_rank < fp4_peak * 1e12 / (peaks["hbm_gbs"] * 1e9)
    # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload, from
    # the ncu captures summarised under profiles/ (time-and-DRAM summary of the 8192^3 case, full capture
    # of the 4096 x 4096 x 8192 case, launch list of the sweep); not captured for the sharded workload
    ncu_traffic = {"gemm8192": 262.8e6, "gemm4096": 43.7e6, "gemm_m16": 19.3e6}.get(args.workload) if world == 1 else None
    if hbm_bound:
        roof = {"bound": "hbm", "achieved": wl.bytes_rank / (mean_rank * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "peak_source": f"{peaks['source']} copy bandwidth"}
    else:
        roof = {"bound": "tensor", "achieved": achieved, "peak": fp4_peak, "unit": "TFLOP/s",
                "peak_source": f"4 x {peaks['source']} cuBLAS bf16 burst ({peaks['bf16_tflops']:.0f} TF/s): "
                               "no FP4 figure is measured on this pool; FP4 : BF16 nominal ratio is 4",
                "frac_of_nominal_9pf": achieved / NOMINAL_FP4_TFLOPS}
    roof.update({"frac": roof["achieved"] / roof["peak"], "traffic": ncu_traffic,
                 "algorithmic_bytes": wl.bytes_rank, "kernel": "nvfp4_gemm_kernel", "path": wl.path})
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, **percentiles(per_step), "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None,
        "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate, fp16 out)",
        "data": "synthetic: seeded N(0,1) (bf16-rounded) quantised to NVFP4 by the library's row quantiser",
        "config": gemm_config(wl.name, wl.m, wl.n_total, wl.k, world),
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                "ms_per_step": ms_e2e, "steps": e2e_steps,
                "copy_gbs_per_gpu": (wl.h2d + wl.d2h) / (ms_e2e * 1e-3) / 1e9,
                "note": "copy-bound: every rank uploads A and its shard of B and downloads its block of C "
                        "over its own host link (the ranks of one box share the host's memory bandwidth)"},
        "gpu_launches": int(launches_per_step * args.steps),
        "clocks": clocks,
        "roofline": roof,
    }
    return line, wl


def sustained_gemm(wl, peaks, seconds: float = 2.0):
    """The same GEMM launched back to back (no flush, no per-step events) for at least `seconds`:
    the power-limited reading, with the SM clock sampled meanwhile."""
    wl.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(20):
        wl.step()
    torch.cuda.synchronize()
    per = (time.perf_counter() - t0) / 20
    iters = int(max(50, seconds / max(per, 1e-6)))
    sampler = ClockSampler(torch.cuda.current_device()).start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.time()
    start.record()
    for _ in range(iters):
        wl.step()
    end.record()
    end.synchronize()
    clocks = sampler.stop((t_begin + 0.3, time.time()))     # skip the ramp at the start of the run
    ms = start.elapsed_time(end) / iters
    tf = wl.flops_rank / (ms * 1e-3) / 1e12
    peak = 4.0 * peaks["bf16_tflops_sustained"]
    return {"tflops": tf, "ms_per_launch": ms, "launches": iters, "seconds": start.elapsed_time(end) / 1e3,
            "frac_of_4x_bf16_sustained": tf / peak, "peak": peak, "frac_of_nominal_9pf": tf / NOMINAL_FP4_TFLOPS,
            "clocks": clocks, "l2": "no flush: launches back to back (operands 72 MB, output 134 MB, L2 126 MB)"}


class GroupedWorkload:
    """Grouped GEMM of 8 experts with weight [4096, 8192] each over 2048 rows split by a seeded
    multinomial with Dirichlet(0.5) proportions (an expert may get no row), per-expert alpha ~ U(0.5, 2)."""

    def __init__(self, device, experts=8, total_rows=2048, n=4096, k=8192, seed=0xB2000300):
        import sm120_nvfp4_b200 as ops
        from sm120_nvfp4_b200 import _lib
        self.L = _lib.lib()
        rng = np.random.default_rng(seed)
        counts = rng.multinomial(total_rows, rng.dirichlet([0.5] * experts)).astype(np.int32)
        self.counts = counts.tolist()
        cu = np.concatenate(([0], np.cumsum(counts))).astype(np.int32)
        self.e, self.m, self.n, self.k = experts, total_rows, n, k
        self.m_pad = max(128, align(int(counts.max()), 128))
        self.seq = torch.from_numpy(counts).to(device)
        self.cu = torch.from_numpy(cu).to(device)
        g = torch.Generator(device=device).manual_seed(seed + 1)
        x = torch.randn((total_rows, k), device=device, generator=g).to(torch.bfloat16)
        self.x, self.xs = ops.quantize_expert(x, self.seq, self.cu, scale_m_pad=self.m_pad)
        self.w, self.ws = quantized_expert_weights(experts, n, k, seed + 2, device, 1.0, chunk=2)
        self.alpha = torch.from_numpy(rng.uniform(0.5, 2.0, experts).astype(np.float32)).to(device)
        self.y = torch.empty((total_rows, n), dtype=torch.float16, device=device)
        self.flops = 2.0 * total_rows * n * k
        self.bytes = (total_rows * k / 2 + experts * n * k / 2 + total_rows * scale_k_padded(k) +
                      experts * n * scale_k_padded(k) + 2 * total_rows * n)

    def step(self):
        st = torch.cuda.current_stream().cuda_stream
        status = self.L.b200_nvfp4_grouped_gemm(self.y.data_ptr(), self.x.data_ptr(), self.w.data_ptr(),
                                                self.seq.data_ptr(), self.cu.data_ptr(), self.xs.data_ptr(),
                                                self.ws.data_ptr(), None, None, None, self.e, self.m, self.n, self.k,
                                                self.m_pad, self.m // self.e, 1, self.alpha.data_ptr(), st)
        if status != 0:
            raise RuntimeError(f"grouped gemm failed with status {status}")


def sweep_entry(name, step, flops, nbytes, device, peaks, flush, iters, extra):
    from sm120_nvfp4_b200 import _lib
    step()
    torch.cuda.synchronize()
    l0 = _lib.launch_count()
    step()
    launches = _lib.launch_count() - l0
    ms, per_step = time_steps(step, iters, 10, 1, device, flush)
    pc = percentiles(per_step)
    # second reading, the reference's own method (benchmarks/benchmark_gemm_vs_cublaslt.cu:210-228): the
    # calls back to back between one pair of events, no flush - what a call costs inside a pipeline of
    # calls, operands that fit L2 (126 MB) staying there
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        step()
    end.record()
    end.synchronize()
    b2b_us = start.elapsed_time(end) / iters * 1e3
    entry = {"workload": name, "us_mean": ms * 1e3, "us_p50": pc["p50_ms"] * 1e3, "us_p95": pc["p95_ms"] * 1e3,
             "us_back_to_back": b2b_us, "calls": iters, "launches_per_call": int(launches),
             **gemm_roofline(flops, nbytes, ms, peaks), "algorithmic_bytes": nbytes}
    entry["bound"] = "hbm" if entry["frac_hbm"] > entry["frac_tensor"] else "tensor"
    entry.update(extra)
    return entry


def run_sweep(args, device, peaks, which=("m16", "m128", "m256", "m1024", "m4096", "grouped_c3")):
    """Per-call timing (CUDA events around every call, L2 flushed between calls) of the remaining
    dense configurations and the grouped GEMM; a CPU-oracle rate for each on a bounded sample."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    iters = max(20, min(args.steps, 200))
    out = []
    # what the per-call protocol itself costs: the same event pair around a 4-byte fill
    tiny = torch.zeros(1, dtype=torch.int32, device=device)
    _, floor = time_steps(lambda: tiny.fill_(1), iters, 10, 1, device, flush)
    out.append({"workload": "timing_floor_4_byte_fill", "us_mean": float(np.mean(floor)) * 1e3,
                "us_p50": percentiles(floor)["p50_ms"] * 1e3, "us_p95": percentiles(floor)["p95_ms"] * 1e3,
                "note": "per-call CUDA events around a trivial kernel after the L2 flush: the part of every us_p50 "
                        "below that is not the measured kernel"})
    for m in (16, 128, 256, 1024, 4096):
        if f"m{m}" not in which:
            continue
        wl = GemmWorkload(m, 4096, 8192, 1, 0, device, f"gemm_m{m}_n4096_k8192", seed=0xB2000100 + m)
        tf, dt, cores = cpu_gemm_sample(m, 4096, 8192, min(m, 64), 2048)
        out.append(sweep_entry(wl.name, wl.step, wl.flops_rank, wl.bytes_rank, device, peaks, flush, iters,
                               {"path": wl.path, "cpu_tflops": tf, "cpu_cores": cores,
                                "cpu_sample": f"{min(m, 64)} rows x 2048 columns of the problem"}))
        del wl
    if "grouped_c3" in which:
        gw = GroupedWorkload(device)
        tf, dt, cores = cpu_gemm_sample(2048, 4096, 8192, 64, 2048)
        out.append(sweep_entry("grouped_e8_rows2048_n4096_k8192_dirichlet0.5", gw.step, gw.flops, gw.bytes, device,
                               peaks, flush, iters,
                               {"rows_per_expert": gw.counts, "cpu_tflops": tf, "cpu_cores": cores,
                                "cpu_sample": "64 rows x 2048 columns of one expert's product"}))
        del gw
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------- MoE workload


class MoeWeights:
    """This rank's experts of the DeepSeek-V3-shaped layer: NVFP4 weights from seeded N(0, 0.02^2)."""

    def __init__(self, world, rank, device, experts=256, hidden=7168, inter=2048, topk=8):
        self.e, self.h, self.i, self.k = experts, hidden, inter, topk
        self.world, self.rank, self.device = world, rank, device
        self.e_local = experts // world
        self.gw, self.gws = quantized_expert_weights(self.e_local, 2 * inter, hidden, 0xB2000400 + 2 * rank, device, 0.02)
        self.dw, self.dws = quantized_expert_weights(self.e_local, hidden, inter, 0xB2000401 + 2 * rank, device, 0.02)


class MoeWorkload:
    """One layer call on `tokens` tokens of this rank: router step, activation quantisation, routed
    experts (expert-parallel exchange when world > 1), combine to BF16."""

    def __init__(self, weights: MoeWeights, tokens: int):
        import sm120_nvfp4_b200 as ops
        from sm120_nvfp4_b200.ep import ExpertParallelMoE
        self.ops, self.wt = ops, weights
        w = weights
        self.t, self.world, self.rank, self.device = tokens, w.world, w.rank, w.device
        g = torch.Generator(device=w.device).manual_seed(0xB2000480 + w.rank + 64 * tokens)
        self.x = torch.randn((tokens, w.h), device=w.device, generator=g).to(torch.bfloat16)
        # router logits; the router step itself (sigmoid, top-k, renormalised weights) runs inside
        # every timed step, in this library's kernel
        self.logits = torch.randn((tokens, w.e), device=w.device, generator=g)
        self.seq1 = torch.tensor([tokens], dtype=torch.int32, device=w.device)
        self.cu1 = torch.tensor([0, tokens], dtype=torch.int32, device=w.device)
        self.in_pad = align(tokens, 128)
        # transport of the expert-parallel exchange: "p2p" = this library's kernels store into the
        # peers' buffers over NVLink, "nccl" = all_to_all_single
        self.transport = os.environ.get("B200_NVFP4_EP_TRANSPORT", "p2p") if w.world > 1 else "none"
        # ordering of the two hand-offs of the p2p transport: "flags" = per-rank ready words that the
        # consuming kernels wait for, "barrier" = two full cross-GPU barriers per layer
        self.handoff = os.environ.get("B200_NVFP4_EP_HANDOFF", "flags")
        # down projection in this many column blocks, the return stores of a block beside the next block
        self.return_blocks = int(os.environ.get("B200_NVFP4_EP_RETURN_BLOCKS", "0"))    # 0 = the layer's own choice
        self.layer = None
        self.events = None
        if w.world > 1:
            import torch.distributed as dist
            layer, err = None, None
            try:
                layer = ExpertParallelMoE(w.gw, w.gws, w.dw, w.dws, w.e, transport=self.transport,
                                          max_tokens=tokens, num_topk=w.k, handoff=self.handoff,
                                          return_blocks=self.return_blocks)
            except Exception as exc:   # e.g. no symmetric memory on this box
                if self.transport != "p2p":
                    raise
                err = f"{type(exc).__name__}: {exc}"
            # every rank must use the same transport: agree on the outcome
            ok = torch.tensor([0 if layer is None else 1], dtype=torch.int32, device=w.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                if w.rank == 0:
                    print(f"[bench] p2p transport unavailable on some rank ({err}); using nccl", file=sys.stderr)
                self.transport = "nccl"
                layer = ExpertParallelMoE(w.gw, w.gws, w.dw, w.dws, w.e)
            self.layer = layer
        self.out = None
        a = tokens * w.k
        self.flops_rank = 6.0 * a * w.h * w.i      # this rank's share when routing is balanced
        w_bytes = w.e_local * (2 * w.i * w.h // 2 + w.h * w.i // 2)
        sf_bytes = w.e_local * (2 * w.i * w.h // 16 + w.h * w.i // 16)
        act = (tokens * w.h * 2 + a * (w.h // 2 + w.h // 16) * 2          # quantise + gather
               + a * (w.h // 2 + w.h // 16) + a * 2 * w.i * 2              # gate/up GEMM in/out
               + a * (4 * w.i + w.i // 2 + w.i // 16)                      # SiLU*up + quant
               + a * (w.i // 2 + w.i // 16) + a * w.h * 2                  # down GEMM in/out
               + tokens * (w.k * 2 * w.h + 2 * w.h))                       # combine
        self.bytes_rank = w_bytes + sf_bytes + act

    def step(self):
        w = self.wt
        ev = self.events
        if ev is not None:
            ev.append([])
        ids, wts = self.ops.router_topk(self.logits, w.k)
        if self.world == 1:
            packed, scales = self.ops.quantize_expert(self.x, self.seq1, self.cu1, scale_m_pad=self.in_pad)
            self.out = self.ops.fused_moe(packed, scales.flatten(), w.gw, w.gws, w.dw, w.dws, ids, wts)
        else:
            self.out = self.layer.forward(self.x, ids, wts, out_bf16=True,
                                          phase_events=ev[-1] if ev is not None else None)

    def prepare_e2e(self):
        self.hx = torch.empty(self.x.shape, dtype=self.x.dtype).pin_memory().copy_(self.x.cpu())
        self.hlogits = torch.empty(self.logits.shape, dtype=self.logits.dtype).pin_memory().copy_(self.logits.cpu())
        self.step()
        self.hout = torch.empty(self.out.shape, dtype=self.out.dtype).pin_memory()
        self.h2d = sum(t.numel() * t.element_size() for t in (self.hx, self.hlogits))
        self.d2h = self.hout.numel() * self.hout.element_size()

    def step_e2e(self):
        self.x.copy_(self.hx, non_blocking=True)
        self.logits.copy_(self.hlogits, non_blocking=True)
        self.step()
        self.hout.copy_(self.out, non_blocking=True)


def phase_means(step_events, step_starts):
    """Mean duration of every phase over the timed steps: events are recorded after each phase on
    the timing stream; a phase lasts from the previous event (the step's start event for the first)."""
    names, sums = [], {}
    for start, evs in zip(step_starts, step_events):
        prev = start
        for name, ev in evs:
            if name == "start":       # router step sits between the step's start and the layer's start
                name = "router"
            dt = prev.elapsed_time(ev)
            if name not in sums:
                names.append(name)
                sums[name] = 0.0
            sums[name] += dt
            prev = ev
    n = max(1, len(step_events))
    return {name: sums[name] / n for name in names}


def moe_reading(weights: MoeWeights, tokens_per_rank: int, label: str, steps: int, warmup: int, peaks,
                with_e2e: bool = True):
    """One reading of the MoE layer: tokens/s over all ranks (max-over-ranks time), P50 / P95, the
    phases of the slowest rank, roofline, e2e."""
    from sm120_nvfp4_b200 import _lib
    world, rank, device = weights.world, weights.rank, weights.device
    wl = MoeWorkload(weights, tokens_per_rank)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    wl.step()
    torch.cuda.synchronize()
    launches0 = _lib.launch_count()
    wl.step()
    launches_per_step = _lib.launch_count() - launches0
    # the sampler starts (and waits for its first sample) before the warm-up: started after the
    # barrier it would let the ranks drift apart again by the start-up time of their samplers
    sampler = ClockSampler(torch.cuda.current_device()).start()
    for _ in range(warmup):
        wl.step()
    torch.cuda.synchronize()
    barrier(world)
    torch.cuda.synchronize()
    t_begin = time.time()
    per_step, starts = [], []
    wl.events = [] if (world > 1 and wl.transport == "p2p") else None
    for _ in range(steps):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        wl.step()
        end.record()
        end.synchronize()
        per_step.append(start.elapsed_time(end))
        starts.append(start)
    torch.cuda.synchronize()
    barrier(world)
    torch.cuda.synchronize()
    clocks = sampler.stop((t_begin, time.time()))
    mean_rank = float(np.mean(per_step))
    ms = max_over_ranks(mean_rank, world, device)
    tokens_total = tokens_per_rank * world
    reading = {"label": label, "tokens_per_rank": tokens_per_rank, "tokens_total": tokens_total,
               "tokens_per_s": tokens_total / (ms * 1e-3), "ms_per_step": ms, **percentiles(per_step),
               "per_step_ms_this_rank": [round(v, 4) for v in per_step],
               "steps": steps, "warmup": warmup, "transport": wl.transport, "handoff": wl.handoff if wl.transport == "p2p" else None,
               "return_blocks": wl.layer.return_blocks if wl.transport == "p2p" else None, "experts_per_rank": weights.e_local,
               "gpu_launches_per_step": int(launches_per_step), "clocks": clocks}
    if wl.events is not None:
        ph = phase_means(wl.events, starts)
        wl.events = None
        names = list(ph)
        if world > 1:
            import torch.distributed as dist
            mine = torch.tensor([mean_rank] + [ph[n] for n in names], dtype=torch.float64, device=device)
            allv = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(allv, mine)
            slow = int(np.argmax([float(v[0]) for v in allv]))
            reading["phases_ms"] = {n: float(allv[slow][1 + i]) for i, n in enumerate(names)}
            reading["phases_rank"] = slow
            reading["phases_sum_ms"] = float(sum(reading["phases_ms"].values()))
            reading["phases_note"] = ("means over the timed steps on the slowest rank; CUDA events after each phase "
                                      "on the timing stream, so they add up to that rank's step time")
    flops_time = wl.flops_rank / (mean_rank * 1e-3) / 1e12
    if world == 1:
        achieved = wl.bytes_rank / (mean_rank * 1e-3) / 1e9
        reading["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                               "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                               "algorithmic_bytes": wl.bytes_rank,
                               "kernel": "whole layer (two grouped nvfp4_gemm_kernel launches dominate)",
                               "peak_source": f"{peaks['source']} copy bandwidth"}
    else:
        peak = 4.0 * peaks["bf16_tflops_sustained"]
        reading["roofline"] = {"bound": "tensor", "achieved": flops_time, "peak": peak, "unit": "TFLOP/s",
                               "frac": flops_time / peak, "traffic": None,
                               "kernel": "whole layer incl. the exchange (two grouped nvfp4_gemm_kernel launches dominate)",
                               "peak_source": f"4 x {peaks['source']} cuBLAS bf16 sustained"}
    reading["tflops_per_rank"] = flops_time
    if with_e2e:
        wl.prepare_e2e()
        ms_e2e, _ = time_steps(wl.step_e2e, min(steps, 10), 3, world, device, None)
        reading["e2e"] = {"value": tokens_total / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": wl.h2d,
                          "d2h_bytes_per_step": wl.d2h, "ms_per_step": ms_e2e}
    del wl
    torch.cuda.empty_cache()
    return reading


def moe_stage_times(weights: MoeWeights, tokens: int, iters: int, peaks):
    """The one-GPU layer stage by stage through the C ABI (the calls b200_nvfp4_fused_moe makes), a CUDA
    event after every stage - what the reference's benchmarks/benchmark_moe_ops.py:79-109 times per
    operator. Per stage: mean microseconds, algorithmic bytes, GB/s against the measured copy bandwidth,
    and for the two grouped GEMMs TFLOP/s. An L2 flush precedes every pass, not every stage: the stages
    see the cache state the layer leaves them."""
    import sm120_nvfp4_b200 as ops
    from sm120_nvfp4_b200 import _lib
    from sm120_nvfp4_b200.ops import scale_k_padded
    L = _lib.lib()
    w, dev = weights, weights.device
    t, h, inter, k, e = tokens, weights.h, weights.i, weights.k, weights.e_local
    a = t * k
    in_pad = m_pad = align(t, 128)
    g = torch.Generator(device=dev).manual_seed(0xB2000490)
    x = torch.randn((t, h), device=dev, generator=g).to(torch.bfloat16)
    logits = torch.randn((t, weights.e), device=dev, generator=g)
    seq1 = torch.tensor([t], dtype=torch.int32, device=dev)
    cu1 = torch.tensor([0, t], dtype=torch.int32, device=dev)
    u8, i32 = dict(dtype=torch.uint8, device=dev), dict(dtype=torch.int32, device=dev)
    gin, gin_s = torch.empty((a, h // 2), **u8), torch.empty((e, m_pad * scale_k_padded(h)), **u8)
    din, din_s = torch.empty((a, inter // 2), **u8), torch.empty((e, m_pad * scale_k_padded(inter)), **u8)
    dout = torch.empty((a, h), dtype=torch.float16, device=dev)
    pos, seq, cu = torch.empty((t, k), **i32), torch.empty(e, **i32), torch.empty(e + 1, **i32)
    out = torch.empty((t, h), dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    avg = max(1, a // e)
    state = {}

    def stages():
        yield "router_topk", lambda: state.update(zip(("ids", "wts"), ops.router_topk(logits, k)))
        yield "quantize_tokens", lambda: state.update(zip(("xq", "xs"), ops.quantize_expert(x, seq1, cu1, scale_m_pad=in_pad)))
        yield "count_and_gather", lambda: _lib.check(L.b200_nvfp4_moe_count_and_gather(
            gin.data_ptr(), gin_s.data_ptr(), state["xq"].data_ptr(), state["xs"].data_ptr(), state["ids"].data_ptr(),
            pos.data_ptr(), seq.data_ptr(), cu.data_ptr(), t, h, k, e, 0, in_pad, m_pad, 0, stream), "count_and_gather")
        yield "gate_up_gemm_silu_quant", lambda: _lib.check(L.b200_nvfp4_grouped_gemm_swiglu_quant(
            din.data_ptr(), din_s.data_ptr(), gin.data_ptr(), w.gw.data_ptr(), seq.data_ptr(), cu.data_ptr(),
            gin_s.data_ptr(), w.gws.data_ptr(), None, None, e, a, inter, h, m_pad, m_pad, avg, stream), "gate/up")
        yield "down_gemm", lambda: _lib.check(L.b200_nvfp4_grouped_gemm(
            dout.data_ptr(), din.data_ptr(), w.dw.data_ptr(), seq.data_ptr(), cu.data_ptr(), din_s.data_ptr(),
            w.dws.data_ptr(), None, None, None, e, a, h, inter, m_pad, avg, 1, None, stream), "down")
        yield "reduce", lambda: _lib.check(L.b200_nvfp4_moe_reduce(
            out.data_ptr(), dout.data_ptr(), pos.data_ptr(), state["wts"].data_ptr(), None, t, h, k, 1, stream), "reduce")

    sf = lambda rows, kk: rows * (kk // 16)
    algorithmic = {
        "router_topk": 4 * t * weights.e + 8 * t * k,
        "quantize_tokens": t * (2 * h + h // 2 + h // 16),
        "count_and_gather": 2 * a * (h // 2 + h // 16) + 8 * a,
        "gate_up_gemm_silu_quant": e * 2 * inter * h // 2 + sf(e * 2 * inter, h) + a * (h // 2 + h // 16) + a * (inter // 2 + inter // 16),
        "down_gemm": e * h * inter // 2 + sf(e * h, inter) + a * (inter // 2 + inter // 16) + a * 2 * h,
        "reduce": t * (k * 2 * h + 2 * h),
    }
    flops = {"gate_up_gemm_silu_quant": 2.0 * a * 2 * inter * h, "down_gemm": 2.0 * a * h * inter}
    names = [n for n, _ in stages()]
    sums = dict.fromkeys(names, 0.0)
    for it in range(iters + 2):
        flush.zero_()
        evs = [torch.cuda.Event(enable_timing=True)]
        evs[0].record()
        for _, call in stages():
            call()
            evs.append(torch.cuda.Event(enable_timing=True))
            evs[-1].record()
        evs[-1].synchronize()
        if it >= 2:                                   # two warm-up passes
            for i, n in enumerate(names):
                sums[n] += evs[i].elapsed_time(evs[i + 1])
    result, total = [], 0.0
    for n in names:
        us = sums[n] / iters * 1e3
        total += us
        entry = {"stage": n, "us": us, "algorithmic_bytes": algorithmic[n], "gbs": algorithmic[n] / (us * 1e-6) / 1e9,
                 "frac_of_measured_hbm": algorithmic[n] / (us * 1e-6) / 1e9 / peaks["hbm_gbs"]}
        if n in flops:
            entry["tflops"] = flops[n] / (us * 1e-6) / 1e12
        result.append(entry)
    return {"stages": result, "sum_us": total, "iters": iters,
            "note": "C-ABI calls of the fused layer issued one by one with a CUDA event after each; one L2 flush per pass"}


def moe_block(world, rank, device, peaks, steps: int, warmup: int, experts: int = 256):
    weights = MoeWeights(world, rank, device, experts=experts)
    block = {"config": {"workload": "fused_moe_deepseek_v3_shape", "hidden": weights.h, "intermediate": weights.i,
                        "experts": weights.e, "topk": weights.k, "parallelism": f"ep{world}" if world > 1 else "single",
                        "weights": "seeded N(0, 0.02^2) quantised to NVFP4", "l2": L2_NOTE}}
    if world == 1:
        block["single"] = moe_reading(weights, 4096, "T=4096 on one GPU", steps, warmup, peaks)
        block["tokens_per_s"] = block["single"]["tokens_per_s"]
        block["stage_times"] = moe_stage_times(weights, 4096, min(steps, 20), peaks)
    else:
        block["weak"] = moe_reading(weights, 4096, f"weak scaling: T=4096 per rank, {4096 * world} in total",
                                    steps, warmup, peaks)
        block["strong"] = moe_reading(weights, 4096 // world, f"strong scaling: T=4096 in total, {4096 // world} per rank",
                                      steps, warmup, peaks, with_e2e=False)
        block["tokens_per_s"] = block["weak"]["tokens_per_s"]
    return block


def run_moe(args, world, rank, device, peaks):
    steps, warmup = min(args.steps, 50), max(3, min(args.warmup, 5))
    block = moe_block(world, rank, device, peaks, steps, warmup, args.moe_experts)
    main = block["single"] if world == 1 else block["weak"]
    line = {
        "metric": METRIC, "value": main["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": main["ms_per_step"], "p50_ms": main["p50_ms"], "p95_ms": main["p95_ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate), bf16 activations", "data": "synthetic",
        "config": {**block["config"], "tokens_per_rank": 4096, "exchange": main["transport"]},
        "e2e": main.get("e2e"), "gpu_launches": int(main["gpu_launches_per_step"] * steps),
        "clocks": main["clocks"], "roofline": main["roofline"], "moe": block,
    }
    return line


# ------------------------------------------------------------------------ CPU arm


def cpu_gemm_sample(m, n, k, rows, cols, seed=0xB2000900):
    """Times the CPU oracle on `rows` x `cols` outputs of an M x N x K problem (all host threads;
    the oracle's run time does not depend on the operand values). Returns (tflops, seconds, cores)."""
    import oracle
    cores = oracle.set_threads(os.cpu_count() or 1)
    rng = np.random.default_rng(seed)
    a = rng.integers(0, 256, (rows, k // 2), dtype=np.uint8)
    b = rng.integers(0, 256, (cols, k // 2), dtype=np.uint8)
    sfa = rng.integers(0x2c, 0x36, oracle.scale_region_bytes(rows, k), dtype=np.uint8)
    sfb = rng.integers(0x2c, 0x36, oracle.scale_region_bytes(cols, k), dtype=np.uint8)
    oracle.gemm_sampled(a[:8], b[:64], sfa, sfb, np.arange(8, dtype=np.int32), np.arange(64, dtype=np.int32))
    t0 = time.perf_counter()
    oracle.gemm_sampled(a, b, sfa, sfb, np.arange(rows, dtype=np.int32), np.arange(cols, dtype=np.int32))
    dt = time.perf_counter() - t0
    return 2.0 * rows * cols * k / dt / 1e12, dt, cores


def run_reference(args, world, rank):
    """The reference's own CPU implementation of the path = the CPU oracle (the reference's kernels
    are SM120-only and its CPU reference GEMM lives inside a CUDA test main(), so the restatement in
    oracle/ is what can run). A step is a bounded sample of the workload - 64 rows x 8192 columns of
    the product - on all host cores; `value` extrapolates its rate to the whole problem,
    `ms_per_step` is the measured time of one sample."""
    if rank != 0:
        return None
    name, m, n, k, scaling = gemm_shape(args.workload if args.workload in ("gemm8192", "gemm4096", "gemm_m16",
                                                                           "gemm_nshard") else
                                        ("gemm8192" if world == 1 else "gemm_nshard"), world)
    rows, cols = min(64, m), min(8192, n)
    per_tf, per_ms = [], []
    cores = 1
    for i in range(args.warmup + args.steps):
        tf, dt, cores = cpu_gemm_sample(m, n, k, rows, cols)
        if i >= args.warmup:
            per_tf.append(tf)
            per_ms.append(dt * 1e3)
    value = float(np.mean(per_tf))
    sample = (f"{rows} rows x {cols} columns of the {m}x{n}x{k} product per step "
              f"({2.0 * rows * cols * k / 1e9:.1f} GFLOP of {2.0 * m * n * k / 1e9:.0f}); the whole problem at this rate "
              f"would take {2.0 * m * n * k / (value * 1e12):.1f} s")
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean(per_ms)), "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None,
        "dtype": "nvfp4 (e2m1 x ue4m3, exact block sums, fp16 out)", "data": "synthetic",
        "config": gemm_config(name, m, n, k, world),
        "note": "CPU oracle on the host cores; `config.l2` describes the GPU arm's timing",
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# ------------------------------------------------------------------------------ main


def guarded(what, fn):
    """Extras must not take the headline down with them: a failure is recorded in the line."""
    try:
        return fn()
    except Exception as exc:      # noqa: BLE001
        return {"error": f"{what}: {type(exc).__name__}: {exc}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None, "gemm8192", "gemm4096", "gemm_nshard", "moe",
                                                         "gemm_m16", "gemm_sweep", "grouped_c3"])
    ap.add_argument("--moe-experts", type=int, default=256,
                    help="experts of the MoE workload (default 256; 32 with --gpus 1 is the per-rank shape of 8-way "
                         "expert parallelism, small enough for profiler captures)")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline workload (no sweep / moe / sustained objects)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    env_world = int(os.environ.get("WORLD_SIZE", "1"))
    default_run = args.workload is None
    if args.workload is None:
        args.workload = "gemm8192" if max(args.gpus, env_world) == 1 else "gemm_nshard"

    if args.impl == "reference":
        rank = int(os.environ.get("RANK", "0"))
        line = run_reference(args, max(args.gpus, env_world), rank)
        if line is not None:
            print(json.dumps(line), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    world, rank, local_rank = dist_setup()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    peaks = load_peaks()
    extras = default_run and not args.no_extras
    if args.workload == "moe":
        line = run_moe(args, world, rank, device, peaks)
    elif args.workload in ("gemm_sweep", "grouped_c3"):
        if world != 1:
            raise SystemExit("the sweep workloads run on one GPU")
        which = ("grouped_c3",) if args.workload == "grouped_c3" else ("m16", "m128", "m256", "m1024", "m4096")
        sweep = run_sweep(args, device, peaks, which)
        first = sweep[1]
        line = {"metric": METRIC, "value": first["tflops"], "unit": "TFLOP/s", "n_gpus": 1, "steps": first["calls"],
                "warmup": 10, "ms_per_step": first["us_mean"] / 1e3, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate, fp16 out)", "data": "synthetic",
                "config": {"workload": first["workload"], "l2": L2_NOTE}, "sweep": sweep}
    else:
        line, wl = run_gemm(args, world, rank, device, peaks)
        if extras and world == 1:
            line["sustained"] = guarded("sustained", lambda: sustained_gemm(wl, peaks))
        del wl
        torch.cuda.empty_cache()
        if extras and world == 1:
            sweep = guarded("sweep", lambda: run_sweep(args, device, peaks))
            line["sweep"] = sweep
        if extras:
            line["moe"] = guarded("moe", lambda: moe_block(world, rank, device, peaks, 20, 3))
    # A bounded wait inside a kernel that gave up makes the launch finish (late) with wrong results:
    # a number measured over such a launch is not a measurement.
    from sm120_nvfp4_b200 import _lib
    err = _lib.device_error()
    if world > 1:
        import torch.distributed as dist
        worst = torch.tensor([err], dtype=torch.int64, device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        err = int(worst.item())
    if err:
        raise SystemExit(f"a kernel reported a timed-out wait (device error word {err}: code {err & 255}, "
                         f"block or rank {err >> 8}); no result printed")
    if rank == 0 and world == 1 and "cpu_baseline" not in line and args.workload.startswith("gemm") and \
            "m" in line["config"]:
        c = line["config"]
        tf, dt, cores = cpu_gemm_sample(c["m"], c["n"], c["k"], min(c["m"], 4096), min(c["n"], 8192))
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                "sample": f"{min(c['m'], 4096)} rows x {min(c['n'], 8192)} columns of the problem, "
                                          f"{dt:.1f} s of CPU oracle time"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
