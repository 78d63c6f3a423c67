#!/usr/bin/env python
"""Benchmark of the dequantize-GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--m M] [--allgather]

Workload (``config.workload``): the Llama-70B-MLP-shaped W4A16 GEMM with group
zeros -- N = 28672, K = 8192, uint4 weights two per byte, group 128, bf16 scales
U[0.005, 0.02] and bf16 zeros U[6, 10], A bf16 ~ N(0,1), fp32 accumulate, bf16 out
-- at M = 4096 tokens (the tensor-bound end of the configuration's M sweep). A step
is one GEMM over one batch of synthetic activations. ``value`` is TFLOPS
(2 M N K / time) with everything resident in HBM; ``sweep`` holds the other M of the
configuration (GB/s against the HBM roofline for M <= 16, TFLOPS otherwise) and
``configs`` the other benchmark configurations (W4A16 16x1024x1024, MXFP4, BitNet
int8 x int2, the single-GPU MoE layer). Those entries are timed with inputs larger than
L2: several packed copies of the weight (together well over the 126 MB L2) are used
round-robin, the way consecutive layers of a model stream different weights, and the
time is that of the whole back-to-back loop divided by the calls. (A 256 MB zero-fill
before every call, the reference's do_bench recipe, leaves the L2 full of dirty lines
whose write-back the timed kernel then pays for: about 4 us on a 40 us kernel.) ``e2e``
is the same GEMM through the public kernel-factory call with the activations coming
from pinned host memory and the result going back to it inside the timed region
(weights stay resident: they are model parameters, packed once); ``e2e_small`` repeats
that for 1 and 16 tokens.

With ``--gpus N`` (launched under torchrun, one rank per GPU) the weight is
column-sharded over the ranks (``tilelang_b200.parallel``); the total work is
fixed ("strong" scaling), C stays column-sharded as a row-parallel consumer takes
it, and ``--allgather`` adds the all-gather of C to every step.

``--impl reference`` times the reference's own CPU path for this GEMM -- its torch
``ref_program`` (dequantise, fp32 matmul, cast), restated in ``oracle/`` -- on all
host threads, on a bounded slice of the weight rows per step.
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

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_FULL, K_FULL, GROUP = 28672, 8192, 128
SWEEP_M = (1, 16, 128, 1024, 4096)
METRIC = "dequant-GEMM TFLOPS (M>=128) & HBM GB/s (M<=16) per B200, % of roofline"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def algorithmic_bytes(M, N, K, group):
    # one read of every input and one write of the output, packed sizes
    return M * K * 2 + N * K // 2 + 2 * N * (K // group) * 2 + M * N * 2


def make_inputs(M, N, K, group, device, seed=0):
    """Seeded synthetic stand-ins for real checkpoint tensors (one generator per tensor)."""
    def gen(i):
        g = torch.Generator(device="cpu")
        g.manual_seed(seed + i)
        return g
    A = torch.randn(M, K, generator=gen(0), dtype=torch.float32).to(torch.bfloat16)
    qB = torch.randint(0, 256, (N, K // 2), generator=gen(1), dtype=torch.uint8)          # two uniform uint4 per byte
    s = (torch.rand(N, K // group, generator=gen(2)) * 0.015 + 0.005).to(torch.bfloat16)
    z = (torch.rand(N, K // group, generator=gen(3)) * 4.0 + 6.0).to(torch.bfloat16)
    return A, qB, s, z


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
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

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


EXTRAS_LIMIT_S = 300


class LineGuard:
    """Owns the one JSON line of a multi-rank run while optional measurements are still running.

    ``emit`` prints a line once. If nothing has been emitted ``limit_s`` seconds after
    construction, the timer prints ``fallback`` (the line measured so far, on the rank that
    holds one) with ``missing`` merged in, and ends the process with exit code 0 on every rank:
    a rank that waits in a collective for a peer that gave up would otherwise wait for the
    process group's own timeout, far beyond the run's budget, and the run would report nothing."""

    def __init__(self, limit_s, fallback, missing):
        self._lock = threading.Lock()
        self._emitted = False
        self._fallback, self._missing = fallback, missing
        self._timer = threading.Timer(limit_s, self._expire)
        self._timer.daemon = True
        self._timer.start()

    def emit(self, line):
        with self._lock:
            if self._emitted:
                return False
            self._emitted = True
            sys.stdout.write(json.dumps(line) + "\n")
            sys.stdout.flush()
            return True

    def _expire(self):
        if self._fallback is not None:
            late = dict(self._fallback)
            late.update(self._missing)
            self.emit(late)
        sys.stdout.flush()
        os._exit(0)


def time_rotating(call, n_variants, rounds=6):
    """Milliseconds per call of ``call(i)``, i cycling over ``n_variants`` input sets that
    together exceed the L2, timed as one back-to-back loop (CUDA events on the launching
    stream). A device-side sleep sized from the measured host time per call lets the host
    enqueue the whole loop first, so that a kernel shorter than the host's launch path is not
    timed at the host's pace."""
    t0 = time.perf_counter()
    for i in range(n_variants):
        call(i)
    host_s = (time.perf_counter() - t0) / n_variants          # host time to enqueue one call
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # the device idles until the host has enqueued the whole loop (about 2 cycles per ns)
    torch.cuda._sleep(int(2.5e9 * host_s * rounds * n_variants) + 2_000_000)
    e0.record()
    for _ in range(rounds):
        for i in range(n_variants):
            call(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (rounds * n_variants)


def time_graph(call, n_variants, rounds=20):
    """Milliseconds per call for kernels shorter than the host's launch path: the whole loop
    (``rounds`` passes over ``n_variants`` input sets that together exceed the L2) is captured in
    one CUDA graph and replayed, so the device never waits for the host; CUDA events around the
    second replay."""
    for i in range(n_variants):
        call(i)                      # warm-up outside the capture: workspaces, tensor maps
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(rounds):
                for i in range(n_variants):
                    call(i)
    torch.cuda.synchronize()
    graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (rounds * n_variants)


CPU_SAMPLE_ROWS = 4096      # weight rows of the bounded CPU sample (of N_FULL)


def cpu_reference_run(M, threads, steps, warmup):
    """The reference's CPU path (torch ref_program restated in oracle/) on the first
    CPU_SAMPLE_ROWS weight rows of the seeded benchmark weight: dequantise to bf16, fp32 matmul,
    cast -- dequantisation included. ``warmup`` untimed evaluations, then the mean over
    ``steps`` timed ones. Both the ``cpu_baseline`` of the CUDA arm and ``--impl reference``
    use this one protocol, so their numbers agree up to run-to-run noise."""
    from oracle import ref_programs as R
    torch.set_num_threads(threads)
    A, qB, s, z = make_inputs(M, CPU_SAMPLE_ROWS, K_FULL, GROUP, "cpu", 0)
    secs = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        R.ref_w4a16(A, qB, s, z, GROUP, torch.bfloat16)
        if i >= warmup:
            secs.append(time.perf_counter() - t0)
    mean = statistics.mean(secs)
    sample = (f"weight rows [0, {CPU_SAMPLE_ROWS}) of {N_FULL}, M={M}, K={K_FULL}, mean of {steps} evaluations "
              f"after {warmup} untimed, {mean:.3f} s each, dequantisation included")
    return 2.0 * M * CPU_SAMPLE_ROWS * K_FULL / mean / 1e12, mean, sample


def run_reference(args, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    M = args.m
    value, mean, sample = cpu_reference_run(M, threads, args.steps, args.warmup)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * mean,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(M, args.gpus, args.allgather),
        "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(M, gpus, allgather):
    return {"workload": f"W4A16 dequant-GEMM with group zeros, Llama-70B-MLP shape: M={M}, N={N_FULL}, K={K_FULL}, "
                        f"group_size={GROUP}, bf16 activations/scales/zeros, fp32 accumulate, bf16 out",
            "M": M, "N": N_FULL, "K": K_FULL, "group_size": GROUP,
            "parallelism": "single GPU" if gpus == 1 else f"column-parallel over N, {gpus} ranks, "
                           + ("all-gather of C per step" if allgather else "C left column-sharded (no collective)"),
            "l2": "working set (A + packed W + C = 0.43 GB at M=4096) exceeds the 126 MB L2; sweep and configs entries "
                  "use inputs larger than L2 (several packed weight copies, round-robin)"}


# DRAM traffic of the dominant kernel per launch, from one ncu --set full capture of this
# command at the given M (dram__bytes_read.sum + dram__bytes_write.sum): M = 4096
# 664,374,784 + 244,163,584 (algorithmic 426,770,432); M = 16 125,729,280 + 4,781,056 and
# M = 1 124,979,200 + 4,661,760 (algorithmic 125,960,192 / 125,656,066: the weight is read once,
# the writes are stream-K partial tiles).
TRAFFIC = {4096: 908538368, 16: 130510336, 1: 129640960}


def load_traffic_note(M):
    if M not in TRAFFIC:
        return {}
    return {"dram_bytes_per_launch": TRAFFIC[M],
            "source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, one launch of the same command"}


def other_configs(dev, peaks):
    """The other benchmark configurations on one GPU, each timed with weight copies used
    round-robin (inputs larger than L2) and quoted against its roofline: algorithmic bytes over
    time for the memory-bound shapes, 2 M N K over time for the rest. The int8 and fp4 figures are
    quoted against the issue-rate ceiling of their tcgen05.mma kind measured in the same run."""
    from tilelang_b200 import kernels, moe, ops, quantize
    out = {}
    hbm, bf16 = peaks["hbm_gbs"], peaks["bf16_tflops"]
    # tensor-pipe ceilings measured here: back-to-back tcgen05.mma from shared memory, one CTA per SM
    issue = {k: ops.tensor_peak(k, mmas=32768, repeats=8) / 1e12 for k in ("bf16", "int8", "mxfp4")}
    nominal = {"int8": 4500.0, "mxfp4": 9000.0}        # dense, per GPU
    out["tensor_issue_peaks"] = {
        "bf16_tflops": issue["bf16"], "int8_tops": issue["int8"], "mxfp4_tflops": issue["mxfp4"],
        "method": "b200dq_tensor_peak: 32768 back-to-back tcgen05.mma 128x256x(32 B of K) per SM, best of 8; "
                  "an issue-rate ceiling (low-entropy operands, a few ms) that moves with the GPU's power state: "
                  "2200 / 4530 / 8800 on a cool GPU, lower right after a long sweep; nominal dense figures are "
                  "2250 / 4500 / 9000"}

    def gen(seed):
        g = torch.Generator()
        g.manual_seed(seed)
        return g

    # C1: W4A16 16 x 1024 x 1024, fp16, zero-point 8 (fits L2 many times over: latency-bound)
    M, N, K = 16, 1024, 1024
    a = torch.randn(M, K, generator=gen(0)).to(torch.float16).to(dev)
    packs = []
    for i in range(8):
        q = torch.randint(0, 256, (N, K // 2), generator=gen(10 + i), dtype=torch.uint8).to(dev)
        sc = (torch.rand(N, K // 128, generator=gen(20 + i)) * 0.015 + 0.005).to(torch.float16).to(dev)
        packs.append(ops.pack_w4a16(q, sc, None, N, K, 128, torch.float16))
    c = torch.empty(M, N, dtype=torch.float16, device=dev)
    ms = time_rotating(lambda i: ops.gemm(a, packs[i], out=c), len(packs), rounds=20)
    ms_graph = time_graph(lambda i: ops.gemm(a, packs[i], out=c), len(packs))
    by = M * K * 2 + N * K // 2 + N * (K // 128) * 2 + M * N * 2
    out["C1 W4A16 16x1024x1024 fp16"] = {"us": ms * 1e3, "us_in_a_cuda_graph": ms_graph * 1e3, "gbs": by / ms_graph / 1e6,
                                         "bound": "launch latency (606 KB of work)",
                                         "frac_of_measured_hbm": by / ms_graph / 1e6 / hbm}

    # C3: MXFP4, N = 14336, K = 4096
    N, K = 14336, 4096
    packs = []
    for i in range(5):
        q = torch.randint(0, 256, (N, K // 2), generator=gen(30 + i), dtype=torch.uint8).to(dev)
        e = (torch.randint(-8, 1, (N, K // 32), generator=gen(40 + i)) + 127).to(torch.uint8).to(dev)
        packs.append(ops.pack_mxfp4(q, e, N, K))
    for M in (1, 32, 512, 8192):
        a = torch.randn(M, K, generator=gen(50 + M)).to(torch.bfloat16).to(dev)
        c = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        ms = time_rotating(lambda i: ops.gemm(a, packs[i], out=c), len(packs))
        by = M * K * 2 + N * K // 2 + N * (K // 32) + M * N * 2
        tf = 2.0 * M * N * K / ms / 1e9
        entry = {"us": ms * 1e3, "tflops": tf, "gbs": by / ms / 1e6, "path": "bf16 kind::f16 with in-register e2m1 decode"}
        if M <= 32:
            entry.update(bound="hbm", frac_of_measured_hbm=by / ms / 1e6 / hbm)
        else:
            entry.update(bound="tensor", frac_of_measured_bf16=tf / bf16)
        out[f"C3 MXFP4 N=14336 K=4096 M={M}"] = entry
    del packs
    # the same shape on the block-scaled fp4 instruction, activation re-quantised on the device
    ws = []
    for i in range(5):
        q = torch.randint(0, 256, (N, K // 2), generator=gen(30 + i), dtype=torch.uint8).to(dev)
        e = (torch.randint(-8, 1, (N, K // 32), generator=gen(40 + i)) + 127).to(torch.uint8)
        ws.append((q, ops.block_mxfp4_scales(e).to(dev)))
    for M in (512, 8192):
        a = torch.randn(M, K, generator=gen(50 + M)).to(torch.bfloat16).to(dev)
        c = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        a_codes, a_sf = ops.quant_mxfp4(a, blocked_scales=True)
        ms_gemm = time_rotating(lambda i: ops.gemm_mxfp4_native(a_codes, a_sf, ws[i][0], ws[i][1], out=c), len(ws))

        def both(i):
            ac, sf = ops.quant_mxfp4(a, blocked_scales=True)
            ops.gemm_mxfp4_native(ac, sf, ws[i][0], ws[i][1], out=c)

        ms_both = time_rotating(both, len(ws))
        tf = 2.0 * M * N * K / ms_gemm / 1e9
        out[f"C3 MXFP4 native N=14336 K=4096 M={M}"] = {
            "us": ms_gemm * 1e3, "tflops": tf, "us_with_activation_quantiser": ms_both * 1e3,
            "tflops_with_activation_quantiser": 2.0 * M * N * K / ms_both / 1e9,
            "path": "tcgen05.mma kind::mxf4.block_scale, both operands e2m1 + e8m0 per 32", "bound": "tensor (fp4)",
            "frac_of_measured_mxfp4_issue_peak": tf / issue["mxfp4"], "frac_of_nominal_fp4": tf / nominal["mxfp4"],
            "speedup_over_dequantising_path":
                out[f"C3 MXFP4 N=14336 K=4096 M={M}"]["us"] / (ms_both * 1e3)}
    del ws

    # C4: BitNet int8 x int2
    for (N, K) in ((3200, 3200), (8640, 3200), (3200, 8640)):
        packs = []
        for i in range(12):
            codes = torch.randint(0, 256, (N, K // 4), generator=gen(60 + i), dtype=torch.uint8).to(dev)
            packs.append(ops.pack_int2(codes, N, K, code_offset=2))
        for M in (1, 64, 2048):
            a = torch.randint(-127, 128, (M, K), generator=gen(70 + M), dtype=torch.int8).to(dev)
            c = torch.empty(M, N, dtype=torch.int32, device=dev)
            ms = time_rotating(lambda i: ops.gemm(a, packs[i], out=c), len(packs))
            by = M * K + N * K // 4 + M * N * 4
            entry = {"us": ms * 1e3}
            if M <= 64:
                # shorter than the host's launch path: the same loop replayed from a CUDA graph
                ms = time_graph(lambda i: ops.gemm(a, packs[i], out=c), len(packs), rounds=5)
                entry["us_in_a_cuda_graph"] = ms * 1e3
            tops = 2.0 * M * N * K / ms / 1e9
            entry.update(tops=tops, gbs=by / ms / 1e6)
            if M <= 64:
                entry.update(bound="hbm / launch latency", frac_of_measured_hbm=by / ms / 1e6 / hbm)
            else:
                entry.update(bound="tensor (int8)", frac_of_measured_int8_issue_peak=tops / issue["int8"],
                             frac_of_nominal_int8=tops / nominal["int8"])
            out[f"C4 BitNet N={N} K={K} M={M}"] = entry
        del packs

    # C5: the MoE layer on one GPU (64 experts, 16384 tokens, top-6)
    cfg = MOE
    E, H, F, g = cfg["experts"], cfg["hidden"], cfg["ffn"], cfg["group"]

    def pack_experts(n, k, seed):
        packs = []
        for e in range(E):
            ge = gen(seed * 1000 + e)
            q = torch.randint(0, 256, (n, k // 2), generator=ge, dtype=torch.uint8).to(dev)
            sc = (torch.rand(n, k // g, generator=ge) * 0.015 + 0.005).to(torch.bfloat16).to(dev)
            packs.append(ops.pack_w4a16(q, sc, None, n, k, g, torch.bfloat16))
        return ops.stack_packed(packs)

    mlp = moe.make_gpu_expert_mlp(pack_experts(2 * F, H, 1), pack_experts(H, F, 2))
    x = torch.randn(cfg["tokens"], H, generator=gen(77)).to(torch.bfloat16).to(dev)
    logits = torch.randn(cfg["tokens"], E, generator=gen(78)).to(dev)
    ms = time_rotating(lambda i: moe.moe_forward(x, logits, cfg["top_k"], E, mlp), 1, rounds=10)
    fl = 2.0 * cfg["tokens"] * cfg["top_k"] * (2 * F * H + H * F)
    out["C5 MoE layer 64 experts top-6 16384 tokens"] = {
        "ms": ms, "tflops": fl / ms / 1e9, "bound": "tensor", "frac_of_measured_bf16": fl / ms / 1e9 / bf16,
        "note": "route + gather + W1 grouped GEMM + silu*up + W2 grouped GEMM + weighted combine; weights 285 MB"}
    ops.check_status(dev)
    return out


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from tilelang_b200 import ops, kernels
    from tilelang_b200.parallel import plan_column_shards

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    peaks = measured_peaks()
    M = args.m

    shard = plan_column_shards(N_FULL, world)[rank]
    n_local = shard.size
    A_h, qB_h, s_h, z_h = make_inputs(M, N_FULL, K_FULL, GROUP, "cpu")
    rows = slice(shard.start, shard.stop)
    qB, s, z = qB_h[rows].to(dev), s_h[rows].contiguous().to(dev), z_h[rows].contiguous().to(dev)
    A = A_h.to(dev)
    pw = ops.pack_w4a16(qB, s, z, n_local, K_FULL, GROUP, torch.bfloat16)
    C = torch.empty(M, n_local, dtype=torch.bfloat16, device=dev)
    C_full = torch.empty(world * M, n_local, dtype=torch.bfloat16, device=dev) if (args.allgather and world > 1) else None
    torch.cuda.synchronize()

    def step():
        ops.gemm(A, pw, out=C)
        if C_full is not None:
            dist.all_gather_into_tensor(C_full, C)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    launches_per_step = 1 if M <= 16 else 2      # the GEMM and, for the tcgen05 kernel, the stream-K fix-up pass
    with ClockSampler(local_rank) as clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
        ms_total = e0.elapsed_time(e1)
        time.sleep(0.25)
    ops.check_status(dev)
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    flops = 2.0 * M * N_FULL * K_FULL
    value = flops / (ms_step * 1e-3) / 1e12

    # ---- end to end through the public factory call, host buffers -------------------
    kernel = kernels.matmul(M, n_local, K_FULL, "bfloat16", "bfloat16", "float32", num_bits=4, group_size=GROUP,
                            with_zeros=True)
    kernel.pack(qB, s, z)
    A_pin = A_h.pin_memory()
    C_pin = torch.empty(M, n_local, dtype=torch.bfloat16).pin_memory()
    A_dev = [torch.empty_like(A) for _ in range(2)]
    copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    compute = torch.cuda.current_stream(dev)

    def e2e_steps(n):
        """H2D of the activations, GEMM, D2H of the result; the copies of neighbouring
        steps overlap the GEMM on their own streams (two activation buffers)."""
        buf_free = [None, None]           # event: last GEMM that read each activation buffer
        prev_out, prev_done = None, None
        for i in range(n):
            b = i % 2
            with torch.cuda.stream(copy_in):
                if buf_free[b] is not None:
                    copy_in.wait_event(buf_free[b])
                A_dev[b].copy_(A_pin, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(copy_in)
            compute.wait_event(ready)
            out = kernel(A_dev[b], qB, s, z)
            done = torch.cuda.Event()
            done.record(compute)
            buf_free[b] = done
            if prev_out is not None:
                with torch.cuda.stream(copy_out):
                    copy_out.wait_event(prev_done)
                    C_pin.copy_(prev_out, non_blocking=True)
                    prev_out.record_stream(copy_out)
            prev_out, prev_done = out, done
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(prev_done)
            C_pin.copy_(prev_out, non_blocking=True)
            prev_out.record_stream(copy_out)
        copy_out.synchronize()
        return float(C_pin[0, 0])         # the host reads the result

    e2e_steps(2)
    barrier()
    t0 = time.perf_counter()
    e2e_steps(args.steps)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = flops * args.steps / t.item() / 1e12

    def line(sweep, configs, e2e_small, cpu):
        """The JSON line of this run from what has been measured so far."""
        traffic = load_traffic_note(M)
        if M <= 16:
            # decode shapes: the small-M kernel streams every weight byte once, HBM-bound
            gbs = algorithmic_bytes(M, N_FULL // world, K_FULL, GROUP) / ms_step / 1e6
            roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": gbs / peaks["hbm_gbs"], "traffic": traffic.get("dram_bytes_per_launch"),
                        "peak_source": f"{peaks['source']} copy bandwidth",
                        "frac_of_nominal_8tbs": gbs / 8000.0,
                        "kernel": f"skinny_dequant_gemm_kernel<{1 if M <= 8 else 2}, U4_SZ, BF16>; "
                                  "duration = step time (one launch: cut tiles are finished inside the kernel)",
                        "traffic_source": traffic.get("source")}
        else:
            tile = 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256
            roofline = {"bound": "tensor", "achieved": value / world, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                        "frac": value / world / peaks["bf16_tflops"], "traffic": traffic.get("dram_bytes_per_launch"),
                        "peak_source": f"{peaks['source']} burst bf16 (sustained {peaks['bf16_tflops_sustained']})",
                        "frac_of_sustained": value / world / peaks["bf16_tflops_sustained"],
                        "kernel": f"umma_dequant_gemm_kernel<{tile}, U4_SZ, BF16>; duration = step time (GEMM + fix-up pass)",
                        "traffic_source": traffic.get("source")}
        return {
            "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(M, world, args.allgather),
            "roofline": roofline,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "TFLOPS", "h2d_bytes_per_step": M * K_FULL * 2 * world,
                    "d2h_bytes_per_step": M * N_FULL * 2,
                    "note": "activations from pinned host memory and result back to it every step; packed weights resident"},
            "gpu_launches": launches_per_step * args.steps * world,
            "clocks": clocks.summary(),
            "sweep": sweep,
            "configs": configs,
            "e2e_small": e2e_small,
        }

    # ---- what the other ranks take part in: the gather of C and the expert-parallel layer ----
    if world > 1:
        # The headline is already measured: a collective that never returns must not lose it.
        guard = LineGuard(EXTRAS_LIMIT_S, line({}, {}, {}, None) if rank == 0 else None,
                          {"with_allgather": {"unavailable": f"the multi-GPU measurements did not return in {EXTRAS_LIMIT_S} s"}})
        try:
            multi = multi_gpu_extras(args, rank, world, local_rank, A, pw, n_local, ms_step)
        except Exception as e:      # the headline stands; a rank left waiting for this one is ended by the guard
            multi = {"with_allgather": {"unavailable": f"{type(e).__name__}: {e}"[:300]}}
        if rank == 0:
            out = line({}, {}, {}, None)
            out.update(multi)
            guard.emit(out)
        return

    # ---- the rest of the configuration's M sweep, single GPU numbers -----------------
    sweep, configs, e2e_small = {}, {}, {}
    if world == 1 and not args.no_sweep:
        copies = [pw] + [ops.pack_w4a16(qB, s, z, n_local, K_FULL, GROUP, torch.bfloat16) for _ in range(3)]
        for m in SWEEP_M:
            a = torch.randn(m, K_FULL, device=dev).to(torch.bfloat16)
            c = torch.empty(m, N_FULL, dtype=torch.bfloat16, device=dev)
            ms = time_rotating(lambda i: ops.gemm(a, copies[i], out=c), len(copies))
            fl, by = 2.0 * m * N_FULL * K_FULL, algorithmic_bytes(m, N_FULL, K_FULL, GROUP)
            entry = {"ms": ms, "tflops": fl / ms / 1e9, "gbs": by / ms / 1e6}
            if m <= 16:
                entry.update(bound="hbm", frac_of_measured_hbm=entry["gbs"] / peaks["hbm_gbs"],
                             frac_of_nominal_8tbs=entry["gbs"] / 8000.0)
            else:
                entry.update(bound="tensor", frac_of_measured_bf16=entry["tflops"] / peaks["bf16_tflops"])
            sweep[f"M={m}"] = entry
        del copies
        ops.check_status(dev)
        configs = other_configs(dev, peaks)
        # decode shapes end to end: pinned host activations in, pinned host result out, every call
        for m in (1, 16):
            km = kernels.matmul(m, n_local, K_FULL, "bfloat16", "bfloat16", "float32", num_bits=4, group_size=GROUP,
                                with_zeros=True)
            km.pack(qB, s, z)
            a_pin = torch.randn(m, K_FULL).to(torch.bfloat16).pin_memory()
            c_pin = torch.empty(m, n_local, dtype=torch.bfloat16).pin_memory()
            a_dev = torch.empty(m, K_FULL, dtype=torch.bfloat16, device=dev)

            def one():
                a_dev.copy_(a_pin, non_blocking=True)
                c_pin.copy_(km(a_dev, qB, s, z), non_blocking=True)
                torch.cuda.current_stream(dev).synchronize()
                return float(c_pin[0, 0])

            for _ in range(5):
                one()
            t0 = time.perf_counter()
            n = 200
            for _ in range(n):
                one()
            us = (time.perf_counter() - t0) / n * 1e6
            # the same step (copy in, GEMM, copy out) as one CUDA graph launch per call
            replay, _ = km.capture(a_dev, qB, s, z, before=lambda: a_dev.copy_(a_pin, non_blocking=True),
                                   after=lambda o: c_pin.copy_(o, non_blocking=True))

            def one_graph():
                replay()
                torch.cuda.current_stream(dev).synchronize()
                return float(c_pin[0, 0])

            for _ in range(5):
                one_graph()
            t0 = time.perf_counter()
            for _ in range(n):
                one_graph()
            us_graph = (time.perf_counter() - t0) / n * 1e6
            e2e_small[f"M={m}"] = {"us_per_call": us, "us_per_call_cuda_graph": us_graph,
                                   "gbs": algorithmic_bytes(m, N_FULL, K_FULL, GROUP) / us / 1e3,
                                   "h2d_bytes": m * K_FULL * 2, "d2h_bytes": m * n_local * 2,
                                   "note": "one synchronous call at a time: host launch path and copies included"}

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        v, _, sample = cpu_reference_run(M, threads, steps=5, warmup=1)
        cpu = {"value": v, "unit": "TFLOPS", "cores": threads, "kind": "port", "sample": sample}

    print(json.dumps(line(sweep, configs, e2e_small, cpu)))


def multi_gpu_extras(args, rank, world, local_rank, A, pw, n_local, ms_plain):
    """The collectives of the sharded path, measured on the same shards as the headline step.

    ``with_allgather``: the column-parallel GEMM followed by the all-gather of C that a
    replicated consumer needs, (a) one gather after the GEMM and (b) the GEMM cut into token
    chunks whose gathers run on NCCL's stream under the next chunk's GEMM. The gathered tensor
    is (world, M, N / world): rank-major column blocks.
    ``moe_ep``: the expert-parallel MoE layer (two all-to-alls per step) with its efficiency
    against the same layer on one GPU, both measured in this run."""
    import torch.distributed as dist
    from tilelang_b200 import ops

    dev = torch.device("cuda", local_rank)
    M = A.shape[0]
    flops = 2.0 * M * N_FULL * K_FULL
    steps = args.steps

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    C = torch.empty(M, n_local, dtype=torch.bfloat16, device=dev)
    C_full = torch.empty(world, M, n_local, dtype=torch.bfloat16, device=dev)

    def serial():
        ops.gemm(A, pw, out=C)
        dist.all_gather_into_tensor(C_full.view(world * M, n_local), C)

    chunks = 4 if M >= 1024 else 1
    mc = M // chunks
    C_parts = [torch.empty(mc, n_local, dtype=torch.bfloat16, device=dev) for _ in range(chunks)]
    G_parts = [torch.empty(world * mc, n_local, dtype=torch.bfloat16, device=dev) for _ in range(chunks)]

    sms = torch.cuda.get_device_properties(dev).multi_processor_count

    def overlapped(spare):
        # The GEMM is persistent, one CTA per SM: NCCL's kernel only runs beside it if some SMs
        # are left free, so the chunk GEMMs are capped at sms - spare CTAs.
        works = []
        for i in range(chunks):
            ops.gemm(A[i * mc:(i + 1) * mc], pw, out=C_parts[i], max_ctas=sms - spare)
            works.append(dist.all_gather_into_tensor(G_parts[i], C_parts[i], async_op=True))
        for w in works:
            w.wait()

    # the gather done by the GEMM's own epilogue: peer stores over NVLink, then a barrier
    from tilelang_b200.parallel import PeerGatheredOutput
    peer_out = PeerGatheredOutput(M, n_local, torch.bfloat16, dev)

    def fused():
        peer_out.gemm(A, pw)
        peer_out.wait()

    ms_fused = timed(fused)
    del peer_out
    ms_serial = timed(serial)
    ms_overlap = {}
    if chunks > 1:
        for spare in (0, 8, 16, 32):
            ms_overlap[f"spare_sms_{spare}"] = timed(lambda: overlapped(spare))
    ops.check_status(dev)
    del C_full, G_parts, C_parts
    best = min([ms_serial, ms_fused] + list(ms_overlap.values()))
    gathered = (world - 1) * M * n_local * 2
    out = {"with_allgather": {
        "value": flops / best / 1e9, "unit": "TFLOPS", "ms_per_step": best,
        "ms_peer_stores_from_the_epilogue": ms_fused,
        "ms_gemm_then_gather": ms_serial, "ms_chunked_overlap": ms_overlap, "token_chunks": chunks,
        "ms_without_collective": ms_plain, "bytes_received_per_rank": gathered,
        "gather_gbs_per_rank_if_exposed": gathered / max(ms_serial - ms_plain, 1e-6) / 1e6,
        "nvlink_floor_ms": gathered / 770e6,
        "note": "peer stores = the GEMM epilogue writes every tile to all ranks' gathered buffers (symmetric memory), "
                "then one barrier; the others use all_gather_into_tensor over NCCL: after the GEMM, or per token chunk "
                "under the next chunk's GEMM with `spare` SMs left to NCCL's kernel. nvlink_floor_ms = bytes sent per "
                "rank over the 770 GB/s measured per direction"}}

    try:
        ms_step, ms_gemm, ms_single = moe_measure(max(5, steps // 3), 3, rank, world, local_rank, compare_single=True)
    except RuntimeError as e:           # raised on every rank together (see moe_measure: healthy())
        out["moe_ep"] = {"unavailable": str(e)[:200]}
        return out
    fl = moe_flops()
    out["moe_ep"] = {
        "value": fl / ms_step / 1e9, "unit": "TFLOPS", "ms_per_step": ms_step, "ms_grouped_gemms_only": ms_gemm,
        "ms_routing_and_all_to_all": ms_step - ms_gemm, "ms_same_layer_one_gpu": ms_single,
        "efficiency_vs_one_gpu": ms_single / (world * ms_step) if ms_step > 0 else None,
        "config": "64 experts over the ranks, 16384 tokens, top-6; two all_to_all_single per step; every grouped GEMM "
                  "here, the one-GPU layer included, on 256-token tiles (--workload moe measures the one-GPU layer on "
                  "the tile it picks itself)"}
    return out


# ---- secondary workload: the grouped W4A16 MoE layer, expert-parallel ------------------
MOE = dict(experts=64, top_k=6, tokens=16384, hidden=2048, ffn=1408, group=128)


def moe_measure(steps, warmup, rank, world, local_rank, compare_single=False):
    """64 experts of W1 (2*1408, 2048) and W2 (2048, 1408), uint4 g=128, 16384 tokens, top-6.
    Experts are split over the ranks, every rank starts with tokens/world tokens; one step
    is route + dispatch all-to-all + two grouped GEMMs with silu_mul between + combine
    all-to-all + weighted sum. Strong scaling: the token count is the whole job's. Returns
    (on every rank) step time, grouped-GEMM time and, with ``compare_single``, the time of the
    whole layer on one GPU measured on this rank (max over ranks), all in ms."""
    import torch.distributed as dist
    from tilelang_b200 import moe, ops

    dev = torch.device("cuda", local_rank)
    c = MOE
    E, H, F, g = c["experts"], c["hidden"], c["ffn"], c["group"]

    def pack_experts(n, k, seed, which):
        packs = []
        for e in which:
            gen = torch.Generator().manual_seed(seed * 1000 + e)
            q = torch.randint(0, 256, (n, k // 2), generator=gen, dtype=torch.uint8).to(dev)
            sc = (torch.rand(n, k // g, generator=gen) * 0.015 + 0.005).to(torch.bfloat16).to(dev)
            z = torch.full((n, k // g), 8.0, dtype=torch.bfloat16, device=dev)
            packs.append(ops.pack_w4a16(q, sc, z, n, k, g, torch.bfloat16))
        return ops.stack_packed(packs)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    class DeviceFault(RuntimeError):
        pass

    def healthy():
        """False on every rank as soon as any rank's status word reports a wait that gave up: a
        measurement on a faulted pipeline would crawl from one 2-second limit to the next."""
        ok = 1
        try:
            ops.check_status(dev)
        except Exception:
            ok = 0
        flag = torch.tensor([ok], dtype=torch.int32, device=dev)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return int(flag.item()) == 1

    def timed(fn):
        fn()
        if not healthy():
            raise DeviceFault("a bounded wait gave up in the first call")
        for _ in range(max(warmup, 3) - 1):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return e0.elapsed_time(e1) / steps

    mine = moe.expert_ranges(E, world)[rank]
    # expert-parallel runs keep the 256-token tile for every grouped GEMM of the measurement (a rank's
    # share of the rows is too small for the whole-tile schedule of the 128-token tile)
    tile = None if world == 1 else 256
    mlp = moe.make_gpu_expert_mlp(pack_experts(2 * F, H, 1, mine), pack_experts(H, F, 2, mine), token_tile=tile)
    t_local = c["tokens"] // world
    gen = torch.Generator().manual_seed(77 + rank)
    x = torch.randn(t_local, H, generator=gen).to(torch.bfloat16).to(dev)
    logits = torch.randn(t_local, E, generator=gen).to(dev)
    if world == 1:
        ms_step = timed(lambda: moe.moe_forward(x, logits, c["top_k"], E, mlp))
    else:
        ms_step = timed(lambda: moe.moe_forward_ep(x, logits, c["top_k"], E, mlp))
    if not healthy():
        raise DeviceFault("a bounded wait gave up during the layer's timed steps")

    # the two grouped GEMMs alone, on this rank's share of evenly routed rows
    rows = c["tokens"] * c["top_k"] // world
    counts = [rows // len(mine)] * len(mine)
    xs = torch.randn(sum(counts), H, device=dev).to(torch.bfloat16)
    ms_gemm = timed(lambda: mlp(xs, counts))
    ms_single = 0.0
    if compare_single and world > 1:
        del mlp
        full = moe.make_gpu_expert_mlp(pack_experts(2 * F, H, 1, range(E)), pack_experts(H, F, 2, range(E)), token_tile=tile)
        xf = torch.randn(c["tokens"], H, generator=gen).to(torch.bfloat16).to(dev)
        lf = torch.randn(c["tokens"], E, generator=gen).to(dev)
        ms_single = timed(lambda: moe.moe_forward(xf, lf, c["top_k"], E, full))
    if not healthy():
        raise DeviceFault("a bounded wait gave up during the grouped-GEMM or single-GPU steps")
    t = torch.tensor([ms_step, ms_gemm, ms_single], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t[0].item(), t[1].item(), t[2].item()


def moe_flops():
    c = MOE
    return 2.0 * c["tokens"] * c["top_k"] * (2 * c["ffn"] * c["hidden"] + c["hidden"] * c["ffn"])


def run_moe(args, rank, world, local_rank):
    torch.cuda.set_device(local_rank)
    with ClockSampler(local_rank) as clocks:
        ms_step, ms_gemm, _ = moe_measure(args.steps, args.warmup, rank, world, local_rank)
        time.sleep(0.25)
    if rank != 0:
        return
    flops = moe_flops()
    peaks = measured_peaks()
    print(json.dumps({
        "metric": "moe_w4a16_layer_tflops", "value": flops / ms_step / 1e9, "unit": "TFLOPS", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "MoE W4A16: 64 experts, W1 2816x2048, W2 2048x1408, uint4 g=128, 16384 tokens, top-6",
                   "parallelism": f"ep{world}", "l2": "working set (weights 348 MB + rows) exceeds L2"},
        "grouped_gemms_only": {"ms": ms_gemm, "tflops": flops / ms_gemm / 1e9,
                               "frac_of_measured_bf16": flops / ms_gemm / 1e9 / world / peaks["bf16_tflops"],
                               "note": "W1 grouped GEMM + silu_mul + W2 grouped GEMM on evenly routed rows"},
        "gpu_launches": 5 * args.steps * world, "clocks": clocks.summary(),
    }))


def run_mxfp4(args, local_rank):
    """Secondary workload: the MXFP4 shape (N = 14336, K = 4096) on the block-scaled fp4
    instruction, activation quantiser included, at ``--m`` tokens. One GPU."""
    from tilelang_b200 import ops
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    N, K, M = 14336, 4096, args.m
    gen = torch.Generator().manual_seed(5)
    ws = []
    for _ in range(5):
        q = torch.randint(0, 256, (N, K // 2), generator=gen, dtype=torch.uint8).to(dev)
        e = (torch.randint(-8, 1, (N, K // 32), generator=gen) + 127).to(torch.uint8)
        ws.append((q, ops.block_mxfp4_scales(e).to(dev)))
    a = torch.randn(M, K, generator=gen).to(torch.bfloat16).to(dev)
    c = torch.empty(M, N, dtype=torch.bfloat16, device=dev)

    def step(i):
        codes, sf = ops.quant_mxfp4(a, blocked_scales=True)
        ops.gemm_mxfp4_native(codes, sf, ws[i][0], ws[i][1], out=c)

    for i in range(max(args.warmup, 3)):
        step(i % len(ws))
    with ClockSampler(local_rank) as clocks:
        ms = time_rotating(step, len(ws), rounds=max(1, args.steps // len(ws)))
        time.sleep(0.25)
    ops.check_status(dev)
    peak = ops.tensor_peak("mxfp4") / 1e12
    tf = 2.0 * M * N * K / ms / 1e9
    print(json.dumps({
        "metric": "mxfp4_native_tflops", "value": tf, "unit": "TFLOPS", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp4 (e2m1 x e2m1, e8m0 scales per 32, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"MXFP4 native: M={M}, N={N}, K={K}, bf16 activations quantised to MXFP4 in the step",
                   "l2": "five weight copies round-robin (inputs larger than L2)"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                     "peak_source": "b200dq_tensor_peak(mxfp4) in this run", "traffic": None},
        "gpu_launches": 2 * args.steps, "clocks": clocks.summary()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="dense", choices=["dense", "moe", "mxfp4"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--allgather", action="store_true")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))
    try:
        if args.workload == "mxfp4":
            if rank == 0:
                run_mxfp4(args, local_rank)
        else:
            (run_moe if args.workload == "moe" else run_ours)(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
