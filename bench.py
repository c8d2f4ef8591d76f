#!/usr/bin/env python
"""Benchmark of the NVFP4 GEMM -> grouped GEMM -> fused-MoE path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload W]

One JSON line on stdout (rank 0). Workloads (synthetic, seeded; no dataset is involved):

  gemm8192      M = N = K = 8192 NVFP4 GEMM, FP16 output (default at N = 1; the shape the
                headline "% of FP4 peak" target is quoted on)
  gemm_nshard   M = 16384, N = 28672, K = 8192, B split by columns over the ranks, no
                collective (default at N > 1; strong scaling)
  gemm4096      M = N = 4096, K = 8192: a small case of the same kernel for profiler captures
  moe           DeepSeek-V3-shaped fused-MoE layer: T = 4096 tokens, hidden 7168,
                intermediate 2048, 256 experts, top-8; expert-parallel over the ranks with
                all-to-all dispatch / combine (tokens/s)

A step is one pass of the hot path over one batch. `value` is device-timed with the inputs
resident in HBM; `e2e` times the same call with host buffers (pinned host -> device copy of
the step's inputs, the call through the C ABI, device -> host copy of the result). The CPU
oracle is only ever the thing measured in the `cpu_baseline` / `--impl reference` legs.
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

NOMINAL_FP4_TFLOPS = 9000.0      # dense FP4 per B200 (vendor figure without sparsity)
FALLBACK_BF16_TFLOPS = 1590.0    # earlier pool measurement, used when MEASURED_PEAKS.json is absent
FALLBACK_HBM_GBS = 6650.0


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return {"bf16_tflops": float(d["bf16_tflops"]), "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
        except Exception:
            pass
    return {"bf16_tflops": FALLBACK_BF16_TFLOPS, "bf16_tflops_sustained": 1400.0, "hbm_gbs": FALLBACK_HBM_GBS, "source": "fallback"}


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
            return
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()

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

    def wait_first_sample(self, timeout=5.0):
        t0 = time.time()
        while not self.samples and time.time() - t0 < timeout and self._proc is not None:
            time.sleep(0.02)

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


def random_nvfp4(rows: int, k: int, seed: int, device):
    """Payload / scale bytes with the value statistics of N(0,1) data quantised to NVFP4
    (codes drawn from the quantiser's output distribution, scale codes around amax/6 of 16
    normal samples). Generated on the device: the bench times kernels, parity lives in tests/."""
    g = torch.Generator(device=device).manual_seed(seed)
    payload = torch.randint(0, 256, (rows, k // 2), dtype=torch.uint8, device=device, generator=g)
    region = ((rows + 127) // 128 * 128) * (((k + 15) // 16 + 3) // 4 * 4)
    scales = torch.randint(0x2c, 0x36, (region,), dtype=torch.uint8, device=device, generator=g)
    return payload, scales


def dist_setup(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        backend = "nccl" if torch.cuda.is_available() else "gloo"
        dist.init_process_group(backend, rank=rank, world_size=world)
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


def time_steps(fn, steps: int, warmup: int, world: int, device, flush: torch.Tensor | None):
    """W untimed steps, then K steps timed one by one with CUDA events on the current stream
    (an L2 flush - a write of a buffer larger than L2 - sits between steps, outside the
    events). Returns mean ms per step as the max over ranks, plus the per-step list."""
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
    ms = float(np.mean(per_step))
    return max_over_ranks(ms, world, device), per_step


# ------------------------------------------------------------------------ workloads


class GemmWorkload:
    def __init__(self, m, n_total, k, world, rank, device, name):
        from sm120_nvfp4_b200 import _lib
        self.L = _lib.lib()
        self.m, self.k, self.n_total = m, k, n_total
        self.n = n_total // world          # this rank's column block of B / C
        self.name = name
        self.device = device
        self.a, self.sfa = random_nvfp4(m, k, 0xB2000500, device)            # A replicated
        self.b, self.sfb = random_nvfp4(self.n, k, 0xB2000510 + rank, device)  # B shard
        self.c = torch.empty((m, self.n), dtype=torch.float16, device=device)
        ws_bytes = self.L.b200_nvfp4_gemm_workspace_bytes(m, self.n, k)
        self.ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
        self.ws_bytes = ws_bytes
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

    def launches_per_step(self):
        return 2 if self.ws_bytes else 1

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


def run_gemm(args, world, rank, device, peaks):
    if args.workload == "gemm8192":
        wl = GemmWorkload(8192, 8192 * world, 8192, world, rank, device, "gemm_m8192_n8192_k8192")
        scaling = "weak"
    elif args.workload == "gemm4096":   # small case of the same kernel, for profiler captures
        wl = GemmWorkload(4096, 4096 * world, 8192, world, rank, device, "gemm_m4096_n4096_k8192")
        scaling = "weak"
    else:
        wl = GemmWorkload(16384, 28672, 8192, world, rank, device, "gemm_nsharded_m16384_n28672_k8192")
        scaling = "strong"
    from sm120_nvfp4_b200 import _lib
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    sampler = ClockSampler(torch.cuda.current_device())
    launches0 = _lib.launch_count()
    sampler.start()
    sampler.wait_first_sample()
    t_begin = time.time()
    ms, per_step = time_steps(wl.step, args.steps, args.warmup, world, device, flush)
    clocks = sampler.stop((t_begin, time.time()))
    launches = _lib.launch_count() - launches0 - args.warmup * wl.launches_per_step()
    value = wl.metric(ms)

    wl.prepare_e2e()
    ms_e2e, _ = time_steps(wl.step_e2e, max(3, min(args.steps, 10)), 3, world, device, None)
    e2e_value = wl.metric(ms_e2e)

    fp4_peak = 4.0 * peaks["bf16_tflops"]
    achieved = wl.flops_rank / (float(np.mean(per_step)) * 1e-3) / 1e12
    # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from one ncu capture of this
    # kernel on this workload (profiles/: the DRAM-traffic summary of the 8192^3 case and the
    # full capture of the 4096 x 4096 x 8192 case); not captured for the sharded workload
    ncu_traffic = {"gemm8192": 268.56e6, "gemm4096": 42.3e6}.get(args.workload) if world == 1 else None
    line = {
        "metric": "NVFP4 GEMM TFLOPS (% FP4 peak); fused-MoE tokens/s at 1/2/4/8 B200",
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
        "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate, fp16 out)", "data": "synthetic",
        "config": {"workload": wl.name, "m": wl.m, "n": wl.n_total, "k": wl.k, "n_per_rank": wl.n,
                   "l2": "256 MiB flush write between timed steps"},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                "ms_per_step": ms_e2e},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": fp4_peak, "unit": "TFLOP/s",
                     "frac": achieved / fp4_peak, "traffic": ncu_traffic,
                     "algorithmic_bytes": wl.bytes_rank if hasattr(wl, "bytes_rank") else None,
                     "peak_source": f"4 x {peaks['source']} cuBLAS bf16 burst ({peaks['bf16_tflops']:.0f} TF/s): "
                                    "no FP4 figure is measured on this pool; FP4 : BF16 nominal ratio is 4",
                     "frac_of_nominal_9pf": achieved / NOMINAL_FP4_TFLOPS,
                     "kernel": "nvfp4_gemm_kernel"},
    }
    return line


class MoeWorkload:
    """DeepSeek-V3-shaped routed MoE layer: T tokens per rank, hidden 7168, intermediate 2048,
    256 experts, top-8 (sigmoid scores, renormalised weights), NVFP4 weights ~ N(0, 0.02^2)."""

    def __init__(self, tokens, world, rank, device, experts=256, hidden=7168, inter=2048, topk=8):
        import sm120_nvfp4_b200 as ops
        from sm120_nvfp4_b200.ep import ExpertParallelMoE
        self.ops = ops
        self.t, self.h, self.i, self.e, self.k = tokens, hidden, inter, experts, topk
        self.world, self.rank, self.device = world, rank, device
        e_local = experts // world
        self.e_local = e_local
        g = torch.Generator(device=device).manual_seed(0xB2000400 + rank)

        def weights(rows, k):
            payload = torch.randint(0, 256, (e_local, rows, k // 2), dtype=torch.uint8, device=device, generator=g)
            region = ((rows + 127) // 128 * 128) * (((k + 15) // 16 + 3) // 4 * 4)
            scale = torch.randint(0x04, 0x0c, (e_local, region), dtype=torch.uint8, device=device, generator=g)
            return payload, scale

        self.gw, self.gws = weights(2 * inter, hidden)
        self.dw, self.dws = weights(hidden, inter)
        self.x = torch.randn((tokens, hidden), device=device, generator=g).to(torch.bfloat16)
        # router logits; the router step itself (sigmoid, top-k, renormalised weights) runs inside
        # every timed step, in this library's kernel
        self.logits = torch.randn((tokens, experts), device=device, generator=g)
        self.ids, self.w = ops.router_topk(self.logits, topk)
        self.seq1 = torch.tensor([tokens], dtype=torch.int32, device=device)
        self.cu1 = torch.tensor([0, tokens], dtype=torch.int32, device=device)
        self.in_pad = (tokens + 127) // 128 * 128
        # transport of the expert-parallel exchange: "p2p" = this library's kernels store into the
        # peers' buffers over NVLink, "nccl" = all_to_all_single
        self.transport = os.environ.get("B200_NVFP4_EP_TRANSPORT", "p2p") if world > 1 else "none"
        self.layer = None
        if world > 1:
            import torch.distributed as dist
            layer, err = None, None
            try:
                layer = ExpertParallelMoE(self.gw, self.gws, self.dw, self.dws, experts, transport=self.transport,
                                          max_tokens=tokens, num_topk=topk)
            except Exception as exc:   # e.g. no symmetric memory on this box
                if self.transport != "p2p":
                    raise
                err = f"{type(exc).__name__}: {exc}"
            # every rank must use the same transport: agree on the outcome
            ok = torch.tensor([0 if layer is None else 1], dtype=torch.int32, device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                if rank == 0:
                    print(f"[bench] p2p transport unavailable on some rank ({err}); using nccl", file=sys.stderr)
                self.transport = "nccl"
                layer = ExpertParallelMoE(self.gw, self.gws, self.dw, self.dws, experts)
            self.layer = layer
        self.out = None
        a = tokens * topk
        self.flops_rank = 6.0 * a * hidden * inter      # expected share when routing is balanced
        w_bytes = e_local * (2 * inter * hidden // 2 + hidden * inter // 2)
        sf_bytes = e_local * (2 * inter * hidden // 16 + hidden * inter // 16)
        act = (tokens * hidden * 2 + a * (hidden // 2 + hidden // 16) * 2        # quantise + gather
               + a * (hidden // 2 + hidden // 16) + a * 2 * inter * 2            # gate/up GEMM in/out
               + a * (4 * inter + inter // 2 + inter // 16)                      # SiLU*up + quant
               + a * (inter // 2 + inter // 16) + a * hidden * 2                 # down GEMM in/out
               + tokens * (topk * 2 * hidden + 2 * hidden))                      # combine
        self.bytes_rank = w_bytes + sf_bytes + act

    def step(self):
        self.ids, self.w = self.ops.router_topk(self.logits, self.k)
        if self.world == 1:
            packed, scales = self.ops.quantize_expert(self.x, self.seq1, self.cu1, scale_m_pad=self.in_pad)
            self.out = self.ops.fused_moe(packed, scales.flatten(), self.gw, self.gws, self.dw, self.dws, self.ids, self.w)
        else:
            self.out = self.layer.forward(self.x, self.ids, self.w, out_bf16=True)

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


def run_moe(args, world, rank, device, peaks):
    from sm120_nvfp4_b200 import _lib
    wl = MoeWorkload(4096, world, rank, device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    sampler = ClockSampler(torch.cuda.current_device())
    steps = min(args.steps, 50)
    wl.step()
    torch.cuda.synchronize()
    launches0 = _lib.launch_count()
    wl.step()
    launches_per_step = _lib.launch_count() - launches0
    sampler.start()
    sampler.wait_first_sample()
    t_begin = time.time()
    ms, per_step = time_steps(wl.step, steps, max(3, min(args.warmup, 5)), world, device, flush)
    clocks = sampler.stop((t_begin, time.time()))
    tokens_total = wl.t * world
    value = tokens_total / (ms * 1e-3)
    wl.prepare_e2e()
    ms_e2e, _ = time_steps(wl.step_e2e, 10, 3, world, device, None)
    achieved_gbs = wl.bytes_rank / (float(np.mean(per_step)) * 1e-3) / 1e9
    line = {
        "metric": "NVFP4 GEMM TFLOPS (% FP4 peak); fused-MoE tokens/s at 1/2/4/8 B200",
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": max(3, min(args.warmup, 5)),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate), bf16 activations", "data": "synthetic",
        "config": {"workload": "fused_moe_deepseek_v3_shape", "tokens_per_rank": wl.t, "hidden": wl.h,
                   "intermediate": wl.i, "experts": wl.e, "topk": wl.k, "experts_per_rank": wl.e_local,
                   "parallelism": f"ep{world}" if world > 1 else "single", "exchange": wl.transport, "l2": "256 MiB flush write between timed steps"},
        "e2e": {"value": tokens_total / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": wl.h2d,
                "d2h_bytes_per_step": wl.d2h, "ms_per_step": ms_e2e},
        "gpu_launches": int(launches_per_step * steps),
        "clocks": clocks,
        "roofline": {"bound": "hbm" if world == 1 else "tensor",
                     "achieved": achieved_gbs if world == 1 else wl.flops_rank / (float(np.mean(per_step)) * 1e-3) / 1e12,
                     "peak": peaks["hbm_gbs"] if world == 1 else 4.0 * peaks["bf16_tflops_sustained"],
                     "unit": "GB/s" if world == 1 else "TFLOP/s", "traffic": None,
                     "kernel": "whole layer (two grouped nvfp4_gemm_kernel launches dominate)",
                     "peak_source": peaks["source"]},
        "tflops_per_rank": wl.flops_rank / (float(np.mean(per_step)) * 1e-3) / 1e12,
    }
    line["roofline"]["frac"] = line["roofline"]["achieved"] / line["roofline"]["peak"]
    return line


def cpu_gemm_sample(m, n, k, rows, cols, seed=0xB2000900):
    """Times the CPU oracle on `rows` x `cols` outputs of an M x N x K problem (all host
    threads). Returns (tflops, seconds, cores)."""
    import oracle
    rng = np.random.default_rng(seed)
    a = rng.integers(0, 256, (rows, k // 2), dtype=np.uint8)
    b = rng.integers(0, 256, (cols, k // 2), dtype=np.uint8)
    sfa = rng.integers(0x2c, 0x36, oracle.scale_region_bytes(rows, k), dtype=np.uint8)
    sfb = rng.integers(0x2c, 0x36, oracle.scale_region_bytes(cols, k), dtype=np.uint8)
    oracle.gemm_sampled(a[:8], b[:64], sfa, sfb, np.arange(8, dtype=np.int32), np.arange(64, dtype=np.int32))
    t0 = time.perf_counter()
    oracle.gemm_sampled(a, b, sfa, sfb, np.arange(rows, dtype=np.int32), np.arange(cols, dtype=np.int32))
    dt = time.perf_counter() - t0
    return 2.0 * rows * cols * k / dt / 1e12, dt, oracle.lib().oracle_num_threads()


def run_reference(args, world, rank):
    """The reference's own CPU implementation of the path = the CPU oracle (the reference's
    kernels are SM120-only and its CPU reference GEMM lives inside a CUDA test main(), so the
    restatement in oracle/ is what can run): each step is a bounded sample of the workload."""
    if rank != 0:
        return None
    if args.workload == "gemm8192":
        name, (m, n, k) = "gemm_m8192_n8192_k8192", (8192, 8192 * world, 8192)
    else:
        name, (m, n, k) = "gemm_nsharded_m16384_n28672_k8192", (16384, 28672, 8192)
    rows, cols = 64, 8192
    per = []
    cores = 1
    for i in range(args.warmup + args.steps):
        tf, dt, cores = cpu_gemm_sample(m, n, k, rows, cols)
        if i >= args.warmup:
            per.append(tf)
    value = float(np.mean(per))
    sample = f"{rows} rows x {cols} columns of the {m}x{n}x{k} problem per step"
    return {
        "impl": "reference", "metric": "NVFP4 GEMM TFLOPS (% FP4 peak); fused-MoE tokens/s at 1/2/4/8 B200",
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 2.0 * m * n * k / (value * 1e12) * 1e3, "higher_is_better": True,
        "scaling": "weak" if args.workload == "gemm8192" else "strong", "vs_baseline": None,
        "dtype": "nvfp4 (e2m1 x ue4m3, exact block sums, fp16 out)", "data": "synthetic",
        "config": {"workload": name, "m": m, "n": n, "k": k},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None, "gemm8192", "gemm4096", "gemm_nshard", "moe"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    env_world = int(os.environ.get("WORLD_SIZE", "1"))
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
    world, rank, local_rank = dist_setup(args)
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    peaks = load_peaks()
    if args.workload == "moe":
        line = run_moe(args, world, rank, device, peaks)
    else:
        line = run_gemm(args, world, rank, device, peaks)
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
                         f"block {err >> 8}); no result printed")
    if rank == 0 and world == 1 and args.workload != "moe":
        tf, dt, cores = cpu_gemm_sample(line["config"]["m"], line["config"]["n"], line["config"]["k"], 4096, 8192)
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                "sample": f"4096 rows x 8192 columns of the problem, {dt:.1f} s of CPU oracle time"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
