#!/usr/bin/env python
"""Benchmark of the hot path: sky-1 decoder block forward + backward, tokens/s.

Workload (benchmark configuration 4): hidden 2048, 16 heads x 128, RoPE, pre-RMSNorm, SwiGLU FFN 5632,
batch 8 x seq 2048 per GPU, weights ~ N(0, 0.02) bf16, tokens uniform over a 32768-token vocabulary,
seed 3.  One step = token embedding lookup -> block forward -> block backward (weight gradients
accumulated in f32) for one batch; at N > 1 every rank runs its own batch (weak scaling, data
parallel) and the weight gradients are all-reduced with NCCL in five slices of one flat f32 bucket,
each slice as soon as the backward has completed it (an event per gradient group), on a second
stream; the last slice drains under the next step's forward.

Printed line (rank 0): `value` = tokens/s with inputs resident in HBM, timed with CUDA events over
exactly K steps, max over ranks; `e2e` = the same through the public API with the step's token ids
copied from pinned host memory and the step's result (the gradient of the first norm gain, 8 KiB)
read back every step; `roofline` = the GEMM kernel (the dominant one) timed per launch by the
library's event profiler in a separate pass over the same steps (the timed passes run without
it); `cpu_baseline` = the CPU oracle of the same block on a bounded sample.  The same line carries,
under `kernels` (and as flat `k_*` scalars in `config`), every kernel-level target at its stated
shape -- GEMM 8192^3, RMSNorm forward / backward on [16384, 2048], causal attention forward /
backward at B 8, H 16, S 2048 -- next to the library stand-ins for the reference's own route
(torch.matmul = cuBLASLt, torch SDPA), and under `lm_step` a short run of the 24-layer training
step (configuration 5).  `--impl reference` times only the CPU path (the reference has no other
host implementation of these operators and cannot be built here).

`--kernel NAME` times one kernel alone (a CUDA graph of `--steps` back-to-back calls, best of three
replays): gemm (`--m --n --k --layout --accumulate`), norm_fwd / norm_bwd (`--rows --cols --residual
--variant`), attn_fwd / attn_bwd (`--batch --seq --heads`, `--variant` 1 = one short-lived CTA per
block, 2 = one CTA per SM; `--fused-qkv` = operands as views of one [B, S, 3H, 128] buffer; attn_bwd
`--rope` = with the inverse rotary rotation in the store epilogues), gemm_mx, norm_fwd_mx.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

VOCAB = 32768
SEED = 3
METRIC = "sky1_block_fwd_bwd_tokens_per_s"


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"bf16": float(d["bf16_tflops_sustained"]), "bf16_burst": float(d["bf16_tflops"]),
                "hbm": float(d["hbm_gbs"]), "source": "measured"}
    return {"bf16": 1400.0, "bf16_burst": 1590.0, "hbm": 6650.0, "source": "fallback"}


# ------------------------------------------------------------------ CPU baseline (oracle)
def cpu_block_tokens_per_s(seqlen: int, repeats: int = 1):
    """Times the float64 CPU restatement of the block (oracle/block_ref.py), forward + backward,
    on batch 1 x `seqlen` tokens at the full model dimensions. Returns (tokens/s, threads)."""
    import torch

    from oracle import block_ref

    cfg = dict(heads=16, kv_heads=16, head_dim=128, eps=1e-6)
    gen = torch.Generator().manual_seed(SEED)
    shapes = {"norm1": (2048,), "wqkv": (2048, 6144), "wo": (2048, 2048), "norm2": (2048,),
              "wup": (2048, 5632), "wgate": (2048, 5632), "wdown": (5632, 2048)}
    w = {n: (torch.ones(s) if n.startswith("norm") else torch.randn(s, generator=gen) * 0.02)
         .to(torch.bfloat16) for n, s in shapes.items()}
    x = torch.randn(1, seqlen, 2048, generator=gen).to(torch.bfloat16)
    dy = torch.randn(1, seqlen, 2048, generator=gen).to(torch.bfloat16)
    table = block_ref.rope_table(seqlen, 128)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        block_ref.block_forward_backward(x, w, dy, cfg, table)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return seqlen / best, torch.get_num_threads()


WORKLOAD = ("sky-1 block fwd+bwd (config 4): hidden 2048, 16x128 heads, RoPE, pre-RMSNorm, SwiGLU 5632, "
            "batch 8 x seq 2048 per GPU, seed 3")
L2_NOTE = "per-step working set (~1 GB of activations) exceeds the 126 MB L2"


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    # torchrun pins every rank to one OpenMP thread; the CPU arm uses all host cores it can get.
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    seqlen = 512
    for _ in range(args.warmup):
        cpu_block_tokens_per_s(seqlen)
    t0 = time.perf_counter()
    threads = 1
    for _ in range(args.steps):
        _, threads = cpu_block_tokens_per_s(seqlen)
    dt = time.perf_counter() - t0
    value = args.steps * seqlen / dt
    sample = f"batch 1 x seq {seqlen} of the block at full width, float64, per step"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": f"dp{args.gpus}", "l2": L2_NOTE},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------ clocks sampler
def init_nccl(dist, dev, max_ctas: int) -> None:
    """One NCCL communicator per rank.  `max_ctas` > 0 bounds the CTAs NCCL's kernels may take
    (ncclConfig_t.maxCTAs): the all-reduces run next to persistent GEMMs that are scheduled for
    the whole machine, and every SM NCCL holds delays the GEMM CTAs that would run there."""
    opts = None
    if max_ctas > 0:
        opts = dist.ProcessGroupNCCL.Options()
        opts.config.max_ctas = max_ctas
        opts.config.min_ctas = 1
    dist.init_process_group("nccl", device_id=dev, pg_options=opts)


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.samples = []
        self.proc = None
        self.t_begin = None  # samples read before mark() are dropped
        self.nvml = None
        # NVML read-only queries from a thread (a sample every few ms); nvidia-smi as a fallback
        # (it manages two or three samples in a 100 ms region).
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.stop_flag = False
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    @staticmethod
    def _physical_index(index: int) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if index < len(ids) and ids[index].isdigit():
                return int(ids[index])
        return index

    def _poll(self):
        n = self.nvml
        bits = (("hw_slowdown", n.nvmlClocksEventReasonHwSlowdown if hasattr(n, "nvmlClocksEventReasonHwSlowdown")
                 else n.nvmlClocksThrottleReasonHwSlowdown),
                ("hw_thermal_slowdown", getattr(n, "nvmlClocksEventReasonHwThermalSlowdown",
                                                getattr(n, "nvmlClocksThrottleReasonHwThermalSlowdown", 0))),
                ("sw_thermal_slowdown", getattr(n, "nvmlClocksEventReasonSwThermalSlowdown",
                                                getattr(n, "nvmlClocksThrottleReasonSwThermalSlowdown", 0))),
                ("sw_power_cap", getattr(n, "nvmlClocksEventReasonSwPowerCap",
                                         getattr(n, "nvmlClocksThrottleReasonSwPowerCap", 0))))
        reasons_fn = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons",
                             getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons", None))
        while not self.stop_flag:
            try:
                sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                mask = reasons_fn(self.handle) if reasons_fn else 0
            except Exception:
                break
            if self.t_begin is not None:
                self.samples.append([str(sm), str(self.max_sm)] +
                                    ["Active" if mask & bit else "Not Active" for _, bit in bits])
            time.sleep(0.002)

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit() and self.t_begin is not None:
                self.samples.append(parts)

    def mark(self):
        """Start of the timed region: keep samples from here on."""
        self.t_begin = time.time()

    def stop(self) -> dict:
        if self.nvml is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
        elif self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        else:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [int(s[0]) for s in self.samples]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": int(self.samples[0][1]),
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------ our arm
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    import cleanlm_b200 as cdl

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        init_nccl(dist, dev, args.nccl_max_ctas)
    L = cdl._lib
    L.check(L.lib.cdl_b200_device_ok(local))

    cfg = cdl.sky1.Sky1Config()  # config 4
    T = cfg.tokens
    params = cdl.sky1.init_params(cfg, seed=SEED)
    # One flat f32 gradient bucket, FFN gradients first (they are final first in the backward).
    order = ("wdown", "wup", "wgate", "norm2", "wo", "wqkv", "norm1")
    shapes = cfg.param_shapes()
    sizes = {n: int(torch.Size(shapes[n]).numel()) for n in order}
    bucket = torch.zeros(sum(sizes.values()), dtype=torch.float32, device=dev)
    grads, off = {}, 0
    for n in order:
        grads[n] = bucket[off:off + sizes[n]].view(shapes[n])
        off += sizes[n]
    blk = cdl.sky1.Sky1Block(cfg, params, device=dev, grads=grads)
    # One slice of the bucket per group of gradients the backward completes together, in the
    # backward's order: each slice's all-reduce starts as soon as its weight gradients are done.
    slices, off = [], 0
    for group in blk.GRAD_GROUPS:
        n = sum(sizes[g] for g in group)
        slices.append((off, off + n))
        off += n
    assert off == bucket.numel() and [g for grp in blk.GRAD_GROUPS for g in grp] == list(order)

    gen = torch.Generator().manual_seed(SEED + 1000 * rank)
    emb = (torch.randn(VOCAB, cfg.hidden, generator=gen) * 0.02).to(torch.bfloat16).to(dev)
    dy = torch.randn(T, cfg.hidden, generator=gen).to(torch.bfloat16).to(dev)
    n_host = args.warmup + args.steps
    tokens_host = torch.randint(0, VOCAB, (n_host, T), generator=gen, dtype=torch.int32).pin_memory()
    tokens_dev = torch.empty(T, dtype=torch.int32, device=dev)
    x = torch.empty(T, cfg.hidden, dtype=torch.bfloat16, device=dev)
    out = torch.empty_like(x)
    dx = torch.empty_like(x)
    result_host = torch.empty(cfg.hidden, dtype=torch.float32).pin_memory()

    main = torch.cuda.Stream(device=dev)
    comm = torch.cuda.Stream(device=dev)
    group_done = [torch.cuda.Event() for _ in slices]
    reduced = torch.cuda.Event()

    def embed():
        tt, te, tx = L.tensor_arg(tokens_dev), L.tensor_arg(emb), L.tensor_arg(x)
        L.check(L.lib.cdl_b200_embedding_fwd(L.ref(tt), L.ref(te), L.ref(tx),
                                             torch.cuda.current_stream().cuda_stream))

    def fwd_bwd():
        blk.forward(x, out)
        if world == 1:
            bucket.zero_()
            blk.backward(dy, dx)
            return
        # The previous step's all-reduce must have drained before gradients are touched again.
        torch.cuda.current_stream().wait_event(reduced)
        bucket.zero_()
        blk.backward(dy, dx, events=group_done)
        with torch.cuda.stream(comm):
            for ev, (lo, hi) in zip(group_done, slices):
                comm.wait_event(ev)
                dist.all_reduce(bucket[lo:hi])
            reduced.record()

    def step_resident():
        embed()
        fwd_bwd()

    def step_e2e(i: int):
        tokens_dev.copy_(tokens_host[i], non_blocking=True)
        embed()
        fwd_bwd()
        if world > 1:
            torch.cuda.current_stream().wait_event(reduced)
        result_host.copy_(grads["norm1"], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(step_fn, indexed: bool):
        """W warm-up steps, then exactly K steps between a barrier + synchronize on both sides,
        CUDA events on the launching stream; returns the max over ranks of the elapsed ms."""
        for i in range(args.warmup):
            step_fn(i) if indexed else step_fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(args.steps):
            step_fn(args.warmup + i) if indexed else step_fn()
        if world > 1:
            torch.cuda.current_stream().wait_event(reduced)
        b.record()
        barrier()
        return max_over_ranks(a.elapsed_time(b))

    with torch.cuda.stream(main):
        reduced.record()
        tokens_dev.copy_(tokens_host[0])
        # ---- device-resident number (no per-launch profiling inside the timed region)
        sampler = ClockSampler(local) if rank == 0 else None
        for _ in range(args.warmup):
            step_resident()
        barrier()
        if sampler:
            sampler.mark()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step_resident()
        if world > 1:
            torch.cuda.current_stream().wait_event(reduced)
        e1.record()
        barrier()
        clocks = sampler.stop() if sampler else None
        ms_resident = max_over_ranks(e0.elapsed_time(e1))

        # ---- end to end: host token ids in, result read back, every step
        ms_e2e = timed(step_e2e, indexed=True)

        # ---- the same steps once more with the library's per-launch event pairs: per-kernel times
        barrier()
        L.profile_start(64 * args.steps + 64)
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        for _ in range(args.steps):
            step_resident()
        if world > 1:
            torch.cuda.current_stream().wait_event(reduced)
        p1.record()
        barrier()
        records = L.profile_stop(64 * args.steps + 64)
        ms_profiled = p0.elapsed_time(p1)
    status = L.device_status()
    if status != 0:
        raise RuntimeError(f"a kernel reported status {status} (bounded wait ran out)")

    # ---- every kernel-level target at its stated shape + the library stand-ins (rank 0)
    kernels = None
    if rank == 0 and not args.no_kernels:
        time.sleep(2.0)  # let the clocks recover from the block loops (see kernel_targets)
        kernels = kernel_targets(torch, cdl, dev)
    barrier()
    # ---- configuration 5: a short run of the 24-layer training step on all ranks
    lm = None
    if not args.no_lm:
        lm = lm_short_run(torch, dist, cdl, dev, world, rank, barrier, max_over_ranks)
    barrier()

    if rank == 0:
        peaks = measured_peaks()
        by_kind = {}
        for kind, ms, work in records:
            k = by_kind.setdefault(kind, [0, 0.0, 0.0])
            k[0] += 1
            k[1] += ms
            k[2] += work
        gemm = by_kind.get("gemm", [0, 0.0, 0.0])
        achieved = gemm[2] / (gemm[1] * 1e-3) / 1e12 if gemm[1] > 0 else None
        kernel_ms = {k: round(v[1] / args.steps, 4) for k, v in by_kind.items()}
        # kernels launched per step: 15 GEMM (SwiGLU fused into two of them, RoPE into the QKV
        # projection), 4 norm fwd, 2 x 2 norm bwd, 1 attn fwd, 3 attn bwd (the inverse RoPE in
        # their store epilogues), 1 embedding
        launches_per_step = 15 + 4 + 4 + 1 + 3 + 1
        # DRAM traffic of the average GEMM launch.  The block's shapes are too large to capture
        # under Nsight Compute, so: the minimum bytes of each of the 15 GEMMs (operands read once,
        # outputs written once, accumulated outputs read and written, fused-epilogue operands
        # included) times the measured-to-minimum ratio of the committed capture of the same
        # KIND of launch -- forward / dgrad shapes: profiles/gemm_bf16_pair_8192x8192x2048.md;
        # weight-gradient shapes: profiles/gemm_bf16_pair_wgrad_2048x5632x16384.md.
        Hd, QKV, F = cfg.hidden, cfg.qkv_dim, cfg.ffn
        plain_bytes = [
            2 * (T * Hd + Hd * QKV + T * QKV),              # qkv
            2 * (T * Hd + Hd * Hd + 2 * T * Hd),            # o + residual
            2 * (T * Hd + Hd * F + T * F),                  # up
            2 * (T * Hd + Hd * F + 3 * T * F),              # gate (+ up in, act out)
            2 * (T * F + F * Hd + 2 * T * Hd),              # down + residual
            2 * (T * Hd + F * Hd + 4 * T * F),              # d_act fused: gate, up in; d_up, d_gate out
            2 * (T * F + Hd * F + T * Hd),                  # dh2
            2 * (T * F + Hd * F + 2 * T * Hd),              # dh2 += (C read)
            2 * (T * Hd + Hd * Hd + T * Hd),                # d_attn
            2 * (T * QKV + Hd * QKV + T * Hd),              # dh1
        ]
        wgrad_bytes = [
            2 * (T * F + T * Hd) + 8 * F * Hd,              # dW down (f32 read + write)
            2 * (T * Hd + T * F) + 8 * Hd * F,              # dW up
            2 * (T * Hd + T * F) + 8 * Hd * F,              # dW gate
            2 * (T * Hd + T * Hd) + 8 * Hd * Hd,            # dW o
            2 * (T * Hd + T * QKV) + 8 * Hd * QKV,          # dW qkv
        ]
        gemm_traffic = (sum(plain_bytes) * TRAFFIC_RATIO_PLAIN + sum(wgrad_bytes) * TRAFFIC_RATIO_WGRAD) / 15
        # Which cuBLAS figure bounds the kernel: the burst one unless the clocks sampled during the
        # timed region had settled well below the maximum (a seconds-long, power-capped region).
        sm, sm_max = (clocks or {}).get("sm_mhz"), (clocks or {}).get("sm_max_mhz")
        settled = bool(sm and sm_max and sm < 0.9 * sm_max)
        peak = peaks["bf16"] if settled else peaks["bf16_burst"]
        # CPU baseline on rank 0 at N = 1 only (torchrun pins ranks to one OpenMP thread).
        cpu_value, cpu_threads = cpu_block_tokens_per_s(512, repeats=2) if world == 1 else (None, None)
        config = {"workload": WORKLOAD, "parallelism": f"dp{world}", "l2": L2_NOTE,
                  "tflops_per_gpu": cfg.flops_fwd_bwd() * args.steps / (ms_resident * 1e-3) / 1e12,
                  "ms_per_step_with_event_profiler": ms_profiled / args.steps,
                  "kernel_ms_per_step": kernel_ms}
        for kname, ms in kernel_ms.items():
            config[f"ms_{kname}"] = ms
        if kernels:
            for name, rec in kernels.items():
                for key in ("ms", "achieved", "frac"):
                    if key in rec:
                        config[f"k_{name}_{key}"] = rec[key]
        if lm:
            for key, val in lm.items():
                config[f"lm_{key}"] = val
        line = {
            "metric": METRIC, "value": args.steps * T * world / (ms_resident * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_resident / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config,
            "e2e": {"value": args.steps * T * world / (ms_e2e * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": T * 4, "d2h_bytes_per_step": cfg.hidden * 4,
                    "ms_per_step": ms_e2e / args.steps},
            # resident, end-to-end and profiled passes, warm-up included
            "gpu_launches": launches_per_step * (args.steps + args.warmup) * 2 + launches_per_step * args.steps,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": (achieved / peak) if achieved else None,
                         "frac_of_burst": (achieved / peaks["bf16_burst"]) if achieved else None,
                         "frac_of_sustained": (achieved / peaks["bf16"]) if achieved else None,
                         "traffic": gemm_traffic, "traffic_unit": "bytes per launch (mean of the 15 GEMMs)",
                         "traffic_source": f"minimum bytes x {TRAFFIC_RATIO_PLAIN} (forward / dgrad shapes, "
                                           f"profiles/gemm_bf16_pair_8192x8192x2048.md) and x {TRAFFIC_RATIO_WGRAD} "
                                           "(weight-gradient shapes, profiles/gemm_bf16_pair_wgrad_2048x5632x16384.md)",
                         "kernel": "gemm_bf16_pair_kernel", "launches": gemm[0],
                         "timed": "per-launch CUDA events in a separate pass over the same steps",
                         "peak_source": peaks["source"] + (" sustained" if settled else " burst") +
                                        " cuBLAS bf16 (chosen by the SM clock sampled in the timed region)"},
            "cpu_baseline": None if cpu_value is None else {
                "value": cpu_value, "unit": "tokens/s", "cores": cpu_threads, "kind": "port",
                "sample": "batch 1 x seq 512 of the same block, float64 oracle, best of 2 passes"},
            "kernels": kernels,
            "lm_step": lm,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes measured with Nsight Compute over the minimum bytes, per kind of GEMM launch (see the
# two profiles named where these are used).
TRAFFIC_RATIO_PLAIN = 1.10
TRAFFIC_RATIO_WGRAD = 1.86


def graph_time_ms(torch, fns, steps: int, replays: int = 3) -> float:
    """`steps` launches (round-robin over fns) captured into one CUDA graph and replayed back to
    back; best of `replays` replays, per launch."""
    for i in range(max(3, len(fns))):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(steps):
            fns[i % len(fns)]()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = None
    for _ in range(replays):
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        best = ms if best is None else min(best, ms)
    return best


def eager_time_ms(torch, fn, steps: int) -> float:
    """Plain launches timed with one CUDA event pair around `steps` of them (library routines that
    cannot be captured into a graph, e.g. an autograd backward)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def kernel_targets(torch, cdl, dev) -> dict:
    """Times every kernel-level target at its stated shape (back-to-back launches from a CUDA
    graph, inputs rotated where one launch's data would fit in L2) and the library routines the
    reference itself would call for the same operator: torch.matmul (cuBLASLt, what
    crates/cleandl/src/execgraph/ops/matmul.rs:1160-1182 runs) and torch's fused attention."""
    import torch.nn.functional as Fnn

    peaks = measured_peaks()
    gen = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=gen).to(torch.bfloat16)
    out = {}

    def rec(name, ms, work, unit, peak, note=None):
        ach = work / (ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9)
        r = {"ms": round(ms, 5), "achieved": round(ach, 2), "unit": unit, "frac": round(ach / peak, 4),
             "peak": peak}
        if note:
            r["note"] = note
        out[name] = r

    burst, hbm = peaks["bf16_burst"], peaks["hbm"]
    # The memory-bound and attention kernels run first and the GEMMs last, with short pauses in
    # between: seconds of dense GEMMs leave the chip at the power cap with reduced clocks, which the
    # 25-200 us kernels measured right after them would inherit.
    time.sleep(1.0)
    # ---- RMSNorm forward / backward on x[16384, 2048]
    rows, cols = 16384, 2048
    nbuf = 3  # 3 x 67 MB per tensor: successive launches do not find their input in L2
    xs = [rnd(rows, cols) for _ in range(nbuf)]
    dys = [rnd(rows, cols) for _ in range(nbuf)]
    ress = [rnd(rows, cols) for _ in range(nbuf)]
    w = (1 + 0.02 * torch.randn(cols, device=dev, generator=gen)).to(torch.bfloat16)
    o = cdl.ops.NormFwdOpts(scale=w, save_stats=True)
    ys = [torch.empty_like(x) for x in xs]
    r_inv = cdl.ops.norm_fwd(xs[0], o).r_inv
    L = cdl._lib

    def norm_fwd_into(x, y):
        tx, ts, ty, tr = (L.tensor_arg(t) for t in (x, w, y, r_inv))
        L.check(L.lib.cdl_b200_rmsnorm_fwd(L.ref(tx), L.ref(ts), None, 1e-6, L.ref(ty), L.ref(tr),
                                           torch.cuda.current_stream().cuda_stream))

    rec("rmsnorm_fwd", graph_time_ms(torch, [(lambda x=x, y=y: norm_fwd_into(x, y)) for x, y in zip(xs, ys)], 30),
        4.0 * rows * cols + 2 * cols + 4 * rows, "GB/s", hbm)
    ds = torch.zeros(cols, device=dev)
    scr = torch.empty(cdl.ops.norm_bwd_scratch_bytes(rows, cols), dtype=torch.uint8, device=dev)
    rec("rmsnorm_bwd", graph_time_ms(torch, [(lambda x=x, dy=dy, y=y: cdl.ops.norm_bwd(x, dy, w, r_inv, ds, scratch=scr, dx=y))
                                             for x, dy, y in zip(xs, dys, ys)], 30),
        6.0 * rows * cols + 6 * cols + 4 * rows, "GB/s", hbm)
    rec("rmsnorm_bwd_residual",
        graph_time_ms(torch, [(lambda x=x, dy=dy, rs=rs, y=y: cdl.ops.norm_bwd(x, dy, w, r_inv, ds, scratch=scr,
                                                                             residual_dy=rs, dx=y))
                              for x, dy, rs, y in zip(xs, dys, ress, ys)], 30),
        8.0 * rows * cols + 6 * cols + 4 * rows, "GB/s", hbm, "the form the block uses")
    del xs, dys, ress, ys
    # ---- causal attention forward / backward, B 8, H 16, S 2048, D 128
    bsz, s_, h = 8, 2048, 16
    q, kx, v, do = (rnd(bsz, s_, h, 128) for _ in range(4))
    fwd = cdl.ops.attention_fwd(q, kx, v)
    f_fwd = 4.0 * bsz * h * s_ * s_ * 128 / 2
    rec("attn_fwd", graph_time_ms(torch, [lambda: cdl.ops.attention_fwd(q, kx, v, out=fwd.out)], 20), f_fwd,
        "TFLOP/s", burst)
    scr = torch.empty(cdl.ops.attention_bwd_scratch_bytes(q, kx), dtype=torch.uint8, device=dev)
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    rec("attn_bwd", graph_time_ms(torch, [lambda: cdl.ops.attention_bwd(q, kx, v, fwd.out, do, fwd.lse, scratch=scr,
                                                                        dq=dq, dk=dk, dv=dv)], 20),
        2.5 * f_fwd, "TFLOP/s", burst, "2.5 x forward FLOP convention; three launches")
    try:
        qt, kt, vt = (t.transpose(1, 2).detach().requires_grad_(True) for t in (q, kx, v))
        dot = do.transpose(1, 2)
        ms_f = eager_time_ms(torch, lambda: Fnn.scaled_dot_product_attention(qt, kt, vt, is_causal=True), 20)
        rec("attn_fwd_torch_sdpa", ms_f, f_fwd, "TFLOP/s", burst, "library stand-in: torch SDPA")
        o_ref = Fnn.scaled_dot_product_attention(qt, kt, vt, is_causal=True)
        ms_b = eager_time_ms(
            torch, lambda: torch.autograd.grad(o_ref, (qt, kt, vt), dot, retain_graph=True), 20)
        rec("attn_bwd_torch_sdpa", ms_b, 2.5 * f_fwd, "TFLOP/s", burst, "library stand-in: torch SDPA backward")
    except Exception as exc:  # a stand-in that cannot run is reported, not fatal
        out["attn_torch_sdpa"] = {"unavailable": str(exc)[:200]}
    time.sleep(1.0)
    # ---- GEMM 8192^3 and the block's five forward shapes: ours and cuBLASLt through torch.matmul
    shapes = {"gemm_8192": (8192, 8192, 8192), "gemm_qkv": (16384, 6144, 2048), "gemm_o": (16384, 2048, 2048),
              "gemm_up": (16384, 5632, 2048), "gemm_down": (16384, 2048, 5632)}
    for name, (m, n, k) in shapes.items():
        a, b = rnd(m, k), rnd(k, n)
        d = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        steps = 10 if name == "gemm_8192" else 20
        rec(name, graph_time_ms(torch, [lambda: cdl.ops.matmul(a, b, out=d)], steps), 2.0 * m * n * k,
            "TFLOP/s", burst)
        rec(name + "_cublaslt", graph_time_ms(torch, [lambda: torch.matmul(a, b, out=d)], steps),
            2.0 * m * n * k, "TFLOP/s", burst, "library stand-in: torch.matmul")
        del a, b, d
    # weight-gradient form of the widest weight: D (f32) += A^T B
    m, n, k = 2048, 5632, 16384
    a, b = rnd(k, m), rnd(k, n)
    d = torch.zeros(m, n, device=dev, dtype=torch.float32)
    wopts = cdl.ops.MatmulOpts(out=torch.float32, c=d, beta=1.0)
    rec("gemm_wgrad_up", graph_time_ms(torch, [lambda: cdl.ops.matmul(a.T, b, wopts, out=d)], 20),
        2.0 * m * n * k, "TFLOP/s", burst)
    dbf = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
    rec("gemm_wgrad_up_cublaslt", graph_time_ms(torch, [lambda: torch.matmul(a.T, b, out=dbf)], 20),
        2.0 * m * n * k, "TFLOP/s", burst, "library stand-in: torch.matmul (bf16 out, no f32 accumulate)")
    del a, b, d, dbf
    torch.cuda.synchronize()
    assert L.device_status() == 0
    return out


def lm_short_run(torch, dist, cdl, dev, world, rank, barrier, max_over_ranks, warmup=2, steps=3):
    """Configuration 5 inside the default run: the 24-layer LM, global batch 64 x 2048 uniform
    random tokens split over the ranks (strong scaling), microbatches of 8 x 2048, AdamW; 2 warm-up
    and 3 timed optimizer steps with the token ids copied from pinned host memory and the loss read
    back every step."""
    blk = cdl.sky1.Sky1Config()
    cfg = cdl.sky1.Sky1LMConfig(block=blk, layers=24, vocab=VOCAB)
    model = cdl.sky1.Sky1LM(cfg, seed=4, device=dev, init_on_device=True)
    seqs_per_rank = max(1, 64 // world)
    mb = max(1, seqs_per_rank // blk.batch)
    global_tokens = mb * blk.tokens * world
    gen = torch.Generator().manual_seed(4 + 1000 * rank)
    n = warmup + steps
    data = torch.randint(0, VOCAB, (n, mb, blk.batch, blk.seqlen + 1), generator=gen, dtype=torch.int32)
    tok = data[..., :-1].reshape(n, mb, -1).contiguous().pin_memory()
    tgt = data[..., 1:].reshape(n, mb, -1).contiguous().pin_memory()
    d_tok = torch.empty(mb, blk.tokens, dtype=torch.int32, device=dev)
    d_tgt = torch.empty_like(d_tok)
    losses = []

    def step(i):
        d_tok.copy_(tok[i], non_blocking=True)
        d_tgt.copy_(tgt[i], non_blocking=True)
        loss = model.train_step(d_tok, d_tgt, global_tokens=global_tokens)
        if world > 1:
            dist.all_reduce(loss)
        losses.append(loss.item())

    for i in range(warmup):
        step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(warmup + i)
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1))
    assert cdl._lib.device_status() == 0
    flops = (cfg.layers * blk.flops_fwd_bwd() + 3 * 2.0 * blk.tokens * blk.hidden * VOCAB) * mb
    del model
    torch.cuda.empty_cache()
    return {"tokens_per_s": steps * global_tokens / (ms * 1e-3), "ms_per_step": ms / steps,
            "tflops_per_gpu": flops * steps / (ms * 1e-3) / 1e12, "loss_first": losses[0],
            "loss_last": losses[-1], "steps": steps, "warmup": warmup, "microbatches_per_rank": mb,
            "scaling": "strong", "params": cfg.param_count()}


# ------------------------------------------------------------------ single-kernel mode
def run_kernel(args) -> None:
    """Times one operator alone (CUDA events, warm-up, buffers rotated so that every iteration
    reads data that is not in L2) and prints its achieved rate against the measured roofline.
    Also the small case the Nsight Compute captures under profiles/ are taken on."""
    import torch

    import cleanlm_b200 as cdl

    torch.cuda.set_device(0)
    dev = "cuda"
    L = cdl._lib
    peaks = measured_peaks()
    gen = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=gen).to(torch.bfloat16)
    k = args.kernel
    if k == "gemm":
        m, n, kk = args.m, args.n, args.k
        a = rnd(kk, m).T if args.layout[0] == "t" else rnd(m, kk)
        b = rnd(n, kk).T if args.layout[1] == "t" else rnd(kk, n)
        out_dtype = torch.float32 if args.accumulate else torch.bfloat16
        d = torch.zeros(m, n, device=dev, dtype=out_dtype)
        opts = cdl.ops.MatmulOpts(out=out_dtype, c=d if args.accumulate else None,
                                  beta=1.0 if args.accumulate else 0.0)
        fns = [lambda: cdl.ops.matmul(a, b, opts, out=d)]
        work, unit, peak = 2.0 * m * n * kk, "TFLOP/s", peaks["bf16_burst"]
        desc = f"gemm {m}x{n}x{kk} layout {args.layout}" + (" f32 accumulate" if args.accumulate else "")
    elif k in ("norm_fwd", "norm_bwd"):
        rows, cols = args.rows, args.cols
        nbuf = max(2, int(300e6 // (rows * cols * 2)) + 1)
        xs = [rnd(rows, cols) for _ in range(nbuf)]
        w = (1 + 0.02 * torch.randn(cols, device=dev, generator=gen)).to(torch.bfloat16)
        if k == "norm_fwd":
            o = cdl.ops.NormFwdOpts(scale=w, save_stats=True, variant=args.variant)
            fns = [(lambda x=x: cdl.ops.norm_fwd(x, o)) for x in xs]
            work = 4.0 * rows * cols + 2 * cols + 4 * rows
        else:
            dys = [rnd(rows, cols) for _ in range(nbuf)]
            r_inv = cdl.ops.norm_fwd(xs[0], cdl.ops.NormFwdOpts(scale=w, save_stats=True)).r_inv
            ds = torch.zeros(cols, device=dev)
            scr = torch.empty(cdl.ops.norm_bwd_scratch_bytes(rows, cols), dtype=torch.uint8, device=dev)
            ress = [rnd(rows, cols) for _ in range(nbuf)] if args.residual else [None] * nbuf
            fns = [(lambda x=x, dy=dy, rs=rs: cdl.ops.norm_bwd(x, dy, w, r_inv, ds, scratch=scr, residual_dy=rs,
                                                                  variant=args.variant))
                   for x, dy, rs in zip(xs, dys, ress)]
            work = (8.0 if args.residual else 6.0) * rows * cols + 6 * cols + 4 * rows
        unit, peak = "GB/s", peaks["hbm"]
        desc = (f"{k} x[{rows},{cols}] bf16" + (" + residual gradient" if k == "norm_bwd" and args.residual else "")
                + (f" variant {args.variant}" if args.variant else ""))
    elif k == "gemm_mx":
        # D[m, n] = A[m, k] . B[k, n] with MXFP8 operands (quantised once, outside the timing)
        m, n, kk = args.m, args.n, args.k
        if args.mx_format == "nvfp4":
            qa, _ = cdl.mx.quantize(rnd(m, kk), rowwise=True, fmt=cdl.mx.NVFP4)
            qb = cdl.mx.quantize(rnd(n, kk), rowwise=True, fmt=cdl.mx.NVFP4)[0].transposed()
        else:
            qa, _ = cdl.mx.quantize(rnd(m, kk), rowwise=True)
            _, qb = cdl.mx.quantize(rnd(kk, n), rowwise=False, colwise=True)
        d = torch.zeros(m, n, device=dev, dtype=torch.bfloat16)
        fns = [lambda: cdl.mx.matmul_mx(qa, qb, out=d)]
        work, unit, peak = 2.0 * m * n * kk, "TFLOP/s", peaks["bf16_burst"]
        desc = f"gemm_mx ({args.mx_format.upper()} operands, bf16 out) {m}x{n}x{kk}"
    elif k == "norm_fwd_mx":
        rows, cols = args.rows, args.cols
        nbuf = max(2, int(300e6 // (rows * cols * 2)) + 1)
        xs = [rnd(rows, cols) for _ in range(nbuf)]
        w = (1 + 0.02 * torch.randn(cols, device=dev, generator=gen)).to(torch.bfloat16)
        fmt = cdl.mx.NVFP4 if args.mx_format == "nvfp4" else cdl.mx.MXFP8
        outs = [cdl.mx.norm_fwd_mx(x, w, colwise=args.colwise, save_stats=True, fmt=fmt) for x in xs]
        fns = [(lambda x=x, o=o: cdl.mx.norm_fwd_mx(x, w, colwise=args.colwise, save_stats=True, out=o,
                                                    fmt=fmt))
               for x, o in zip(xs, outs)]
        n_out = 2 if args.colwise else 1
        per_elem = (0.5 + 1 / 16) if args.mx_format == "nvfp4" else (1 + 1 / 32)
        work = 2.0 * rows * cols + n_out * rows * cols * per_elem + 2 * cols + 4 * rows
        unit, peak = "GB/s", peaks["hbm"]
        desc = f"norm_fwd_mx x[{rows},{cols}] bf16 -> {args.mx_format.upper()} rowwise" + (
            " + colwise" if args.colwise else "")
    else:
        bsz, s_, h = args.batch, args.seq, args.heads
        if args.fused_qkv:  # q, k, v (and their gradients) as views of one [B, S, 3H, 128] buffer, the block's layout
            qkv, dqkv = rnd(bsz, s_, 3 * h, 128), rnd(bsz, s_, 3 * h, 128)
            q, kx, v = qkv[:, :, :h], qkv[:, :, h:2 * h], qkv[:, :, 2 * h:]
            dq, dk, dv = dqkv[:, :, :h], dqkv[:, :, h:2 * h], dqkv[:, :, 2 * h:]
            do = rnd(bsz, s_, h, 128)
        else:
            q, kx, v, do = (rnd(bsz, s_, h, 128) for _ in range(4))
            dq, dk, dv = (torch.empty_like(q) for _ in range(3))
        aopts = cdl.ops.AttentionOpts(variant=args.variant)
        fwd = cdl.ops.attention_fwd(q, kx, v, aopts)
        if k == "attn_fwd":
            fns = [lambda: cdl.ops.attention_fwd(q, kx, v, aopts, out=fwd.out)]
            work = 4.0 * bsz * h * s_ * s_ * 128 / 2
        else:
            scr = torch.empty(cdl.ops.attention_bwd_scratch_bytes(q, kx), dtype=torch.uint8, device=dev)
            table = None
            if args.rope:  # the inverse rotary rotation of dQ / dK inside the store epilogues
                inv = 1.0 / (10000.0 ** (torch.arange(0, 64, dtype=torch.float64) / 64))
                ang = torch.arange(s_, dtype=torch.float64)[:, None] * inv[None]
                table = torch.cat([ang.cos(), ang.sin()], 1).float().to(dev).contiguous()
            fns = [lambda: cdl.ops.attention_bwd(q, kx, v, fwd.out, do, fwd.lse, aopts, scratch=scr,
                                                 dq=dq, dk=dk, dv=dv, rope_table=table)]
            work = 10.0 * bsz * h * s_ * s_ * 128 / 2
        unit, peak = "TFLOP/s", peaks["bf16_burst"]
        desc = (f"{k} causal B={bsz} H={h} S={s_} D=128" + (f" variant {args.variant}" if args.variant else "")
                + (" fused-qkv views" if args.fused_qkv else "") + (" + inverse RoPE" if args.rope and k == "attn_bwd" else ""))
    for i in range(args.warmup):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    # The `steps` launches are captured into one CUDA graph and replayed, so that they run back to
    # back on the device: through Python a launch costs more host time than a 25-100 us kernel
    # runs, and an event pair around every single launch adds several microseconds to each.
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(args.steps):
            fns[i % len(fns)]()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = []
    for _ in range(3):
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        reps.append(e0.elapsed_time(e1) / args.steps)
    ms = min(reps)
    # Per-launch CUDA events recorded by the library around its own kernels, for comparison.
    L.profile_start(4 * args.steps + 16)
    for i in range(args.steps):
        fns[i % len(fns)]()
    kind = {"gemm": "gemm", "norm_fwd": "norm_fwd", "norm_bwd": "norm_bwd", "attn_fwd": "attn_fwd",
            "attn_bwd": "attn_bwd", "gemm_mx": "gemm", "norm_fwd_mx": "norm_fwd"}[k]
    times = [ms_ for kd, ms_, _ in L.profile_stop(4 * args.steps + 16) if kd == kind]
    ms_events = sum(times) / len(times)
    assert L.device_status() == 0
    achieved = work / (ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9)
    print(json.dumps({"kernel": k, "case": desc, "ms": ms, "ms_per_launch_events": ms_events,
                      "timing": "CUDA graph of `steps` back-to-back launches, best of 3 replays",
                      "achieved": achieved, "unit": unit,
                      "peak": peak, "frac": achieved / peak,
                      "peak_source": peaks["source"] + (" burst cuBLAS bf16" if unit == "TFLOP/s"
                                                        else " copy bandwidth"),
                      "steps": args.steps, "warmup": args.warmup}))


# ------------------------------------------------------------------ block with MXFP8 products
def run_block_mx(args) -> None:
    """The block of benchmark configuration 4 with every matrix product on MXFP8 operands
    (clean-lm_b200/sky1_mx.py), one GPU, inputs resident.  Not the headline metric: the numerics are
    those of MXFP8; the line exists to measure the block-scaled operators end to end."""
    import torch

    import cleanlm_b200 as cdl

    torch.cuda.set_device(0)
    cfg = cdl.sky1.Sky1Config()
    blk = cdl.sky1_mx.Sky1BlockMX(cfg, cdl.sky1.init_params(cfg, 3))
    gen = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(cfg.tokens, cfg.hidden, device="cuda", generator=gen).to(torch.bfloat16)
    dy = torch.randn(cfg.tokens, cfg.hidden, device="cuda", generator=gen).to(torch.bfloat16)
    out, dx = torch.empty_like(x), torch.empty_like(x)

    def step():
        blk.forward(x, out)
        blk.zero_grads()
        blk.backward(dy, dx)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cdl._lib.profile_start(128 * args.steps + 64)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    records = cdl._lib.profile_stop(128 * args.steps + 64)
    ms = e0.elapsed_time(e1) / args.steps
    by_kind = {}
    for kind, t, _ in records:
        by_kind[kind] = by_kind.get(kind, 0.0) + t
    assert cdl._lib.device_status() == 0
    print(json.dumps({
        "metric": "sky1_block_mxfp8_fwd_bwd_tokens_per_s", "value": cfg.tokens / (ms * 1e-3),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms, "higher_is_better": True, "dtype": "mxfp8 products, bf16 elsewhere",
        "data": "synthetic",
        "config": {"workload": "sky-1 block fwd+bwd (config 4) with MXFP8 matrix products; weights "
                               "quantised once outside the timed region",
                   "kernel_ms_per_step": {k: round(v / args.steps, 4) for k, v in by_kind.items()}}}))


# ------------------------------------------------------------------ full LM step (config 5)
def run_lm(args) -> None:
    """24-layer sky-1-style LM training step (benchmark configuration 5): global batch 64 x 2048
    uniform-random tokens split over the ranks, microbatches of 8 x 2048 with gradient
    accumulation, per-layer all-reduce overlapped with the backward, AdamW.  Prints one JSON
    line with tokens/s (device-timed, max over ranks) and the last loss."""
    import torch
    import torch.distributed as dist

    import cleanlm_b200 as cdl

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        init_nccl(dist, dev, args.nccl_max_ctas)
    blk = cdl.sky1.Sky1Config()
    cfg = cdl.sky1.Sky1LMConfig(block=blk, layers=args.layers, vocab=VOCAB)
    model = cdl.sky1.Sky1LM(cfg, seed=4, device=dev)
    seqs_per_rank = max(1, 64 // world)
    mb = max(1, seqs_per_rank // blk.batch)
    global_tokens = mb * blk.tokens * world
    gen = torch.Generator().manual_seed(4 + 1000 * rank)
    n = args.warmup + args.steps
    data = torch.randint(0, VOCAB, (n, mb, blk.batch, blk.seqlen + 1), generator=gen, dtype=torch.int32)
    tok = data[..., :-1].reshape(n, mb, -1).contiguous().pin_memory()
    tgt = data[..., 1:].reshape(n, mb, -1).contiguous().pin_memory()
    d_tok = torch.empty(mb, blk.tokens, dtype=torch.int32, device=dev)
    d_tgt = torch.empty_like(d_tok)
    losses = []

    def step(i):
        d_tok.copy_(tok[i], non_blocking=True)
        d_tgt.copy_(tgt[i], non_blocking=True)
        loss = model.train_step(d_tok, d_tgt, global_tokens=global_tokens)
        if world > 1:
            dist.all_reduce(loss)
        losses.append(loss.item())  # the step's result is read back every step

    for i in range(args.warmup):
        step(i)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(args.warmup + i)
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    assert cdl._lib.device_status() == 0
    if rank == 0:
        flops = (cfg.layers * blk.flops_fwd_bwd() + 3 * 2.0 * blk.tokens * blk.hidden * VOCAB) * mb
        print(json.dumps({
            "metric": "sky1_lm_train_tokens_per_s", "value": args.steps * global_tokens / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"sky-1 LM training step (config 5): {cfg.layers} layers, vocab {VOCAB}, "
                                   f"global batch 64 x 2048, AdamW lr 3e-4 betas (0.9, 0.95) wd 0.1",
                       "parallelism": f"dp{world}", "microbatches_per_rank": mb,
                       "params": cfg.param_count(),
                       "tflops_per_gpu": flops * args.steps / (ms * 1e-3) / 1e12},
            "loss_first": losses[0], "loss_last": losses[-1]}))
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernel", default=None,
                    choices=["gemm", "norm_fwd", "norm_bwd", "attn_fwd", "attn_bwd", "gemm_mx", "norm_fwd_mx"],
                    help="time one operator alone instead of the block")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--layout", default="nn", choices=["nn", "nt", "tn", "tt"],
                    help="gemm: n = row-major operand, t = transposed view (A then B)")
    ap.add_argument("--accumulate", action="store_true", help="gemm: D (f32) += A.B, the wgrad form")
    ap.add_argument("--residual", action="store_true",
                    help="norm_bwd: add a residual gradient into dx (the form the block uses)")
    ap.add_argument("--mx-format", default="mxfp8", choices=["mxfp8", "nvfp4"],
                    help="gemm_mx / norm_fwd_mx: the block-scaled format")
    ap.add_argument("--colwise", action="store_true",
                    help="norm_fwd_mx: also produce the colwise (transposed-block) output")
    ap.add_argument("--variant", type=int, default=0,
                    help="attn_fwd / attn_bwd: cdl_attn_desc.variant (0 default, 1 one-shot kernels, 2 persistent kernels); "
                         "norm_fwd / norm_bwd: cdl_norm_options.variant")
    ap.add_argument("--rope", action="store_true",
                    help="attn_bwd: with the inverse rotary rotation in the store epilogues (cdl_b200_attn_bwd_rope)")
    ap.add_argument("--fused-qkv", action="store_true",
                    help="attn_fwd / attn_bwd: q, k, v and dq, dk, dv are views of one [B, S, 3H, 128] buffer")
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--cols", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--workload", default="block", choices=["block", "lm", "block_mx"],
                    help="block = benchmark configuration 4 (the headline metric); lm = the 24-layer "
                         "training step; block_mx = the block with MXFP8 matrix products (one GPU)")
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--nccl-max-ctas", type=int, default=0,
                    help="N > 1: upper bound on the CTAs of NCCL's kernels (0: NCCL's default)")
    ap.add_argument("--no-kernels", action="store_true",
                    help="block workload: skip the per-kernel targets and library stand-ins")
    ap.add_argument("--no-lm", action="store_true",
                    help="block workload: skip the short run of the 24-layer training step")
    args = ap.parse_args()
    if args.workload == "lm":
        run_lm(args)
        return
    if args.workload == "block_mx":
        run_block_mx(args)
        return
    if args.kernel:
        args.warmup = max(args.warmup, 3)
        run_kernel(args)
        return
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
