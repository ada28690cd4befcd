#!/usr/bin/env python
"""Benchmark of the axiom matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline (one JSON line on stdout): fp32-accurate GEMM, M=N=K=8192 per GPU
(rows sharded across GPUs, weights replicated, no data-path collective: weak
scaling), in TFLOP/s through the C ABI (operand split pre-pass + tcgen05
kernel, both inside the timed step).  `extra` carries the other metrics of
the suite on the same box: int8 TOPS at 16384^3, the bs=1 / 8 / 32 skinny-M
route in GB/s of weight traffic, the 1024^3 dense+ReLU, the 512x4096x4096
quantised GEMM and causal attention, each with its own roofline fraction.

`--impl reference` times the reference's own CPU path (the compiled axiom
library under oracle/_ref, OpenMP over the box's host cores) on a bounded
sample of the same workload and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

GEMM_N = 8192
FLOP_HEADLINE = 2.0 * GEMM_N ** 3


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- reference arm

def cpu_reference_gemm(steps, warmup, autotune=True):
    """axiom's own OpenMP/AVX2 GEMM (ax_compute_gemm) on a row slice of the 8192^3 problem."""
    import numpy as np
    from oracle_lib import Oracle, Reference
    if not Reference.available():
        return None
    ref = Reference(autotune=autotune)   # tuning happens here, outside the timing
    o = Oracle()
    rows = 1024
    A = o.uniform((rows, GEMM_N), 7)
    B = o.uniform((GEMM_N, GEMM_N), 13)
    for _ in range(max(1, warmup)):
        ref.gemm(A, B)
    times = []
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        ref.gemm(A, B)
        times.append(time.perf_counter() - t0)
    flop = 2.0 * rows * GEMM_N * GEMM_N
    t = sum(times) / len(times)
    return {"value": flop / t / 1e12, "unit": "TFLOP/s", "cores": ref.num_threads(), "kind": "reference",
            "sample": f"ax_compute_gemm on a {rows}x{GEMM_N}x{GEMM_N} row slice of the 8192^3 problem "
                      f"(includes the shim's operand copies), mean of {len(times)} runs, host has {os.cpu_count()} cpus",
            "ms_per_step": t * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = min(args.steps, 5)
    cb = cpu_reference_gemm(steps, min(args.warmup, 2))
    if cb is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libaxiom_ref.so was not built"}))
        return
    line = {
        "impl": "reference", "metric": "gemm_fp32_tflops", "value": cb["value"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 2), "ms_per_step": cb["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "fp32 GEMM M=N=K=8192 per GPU (reference: 1024-row slice on host cores)"},
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- our arm

def timed(torch, dist, world, fn, steps, warmup):
    """W warm-ups, then exactly `steps` calls between barrier+synchronize pairs; max over ranks, ms."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = float(t.item())
    return ms


def run_ours(args):
    import torch
    import torch.distributed as dist
    from axiom_b200.engine import get_engine

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    eng = get_engine(local)
    peaks = measured_peaks()
    K, W = args.steps, max(args.warmup, 3)
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)

    def uniform(shape):
        return torch.rand(shape, device="cuda", generator=gen) * 2 - 1

    # ---------------- headline: fp32-accurate GEMM 8192^3 per GPU (3xTF32)
    A, B = uniform((GEMM_N, GEMM_N)), uniform((GEMM_N, GEMM_N))
    Cout = torch.empty((GEMM_N, GEMM_N), device="cuda")
    step = lambda: eng.gemm(A, B, Cout)
    for _ in range(W):
        step()
    eng.set_profiling(True)
    try:
        gpu_id = "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
    except Exception:
        gpu_id = str(local)
    sampler = ClockSampler(gpu_id)
    if rank == 0:
        sampler.start()
    eng.launch_count(reset=True)
    ms = timed(torch, dist, world, step, K, 0)
    launches = eng.launch_count()
    clocks = sampler.stop() if rank == 0 else None
    calls, pre_ms, core_ms = eng.timing_summary()
    eng.set_profiling(False)
    ms_per_step = ms / K
    value = world * FLOP_HEADLINE / (ms_per_step * 1e-3) / 1e12
    core_avg_ms = core_ms / max(calls, 1)
    tf32_split_peak = peaks["bf16_tflops"] / 2.0 / 3.0   # TF32 issues at half the bf16 rate; 3 products per result
    achieved = FLOP_HEADLINE / (core_avg_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": achieved, "peak": tf32_split_peak, "unit": "TFLOP/s",
                "frac": achieved / tf32_split_peak,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload
                # (profiles/gemm_tc_pair_tf32_8192.md); algorithmic bytes are 1.34e9 (4 operand planes + C)
                "traffic": 5.64e9, "algorithmic_bytes": 1.34e9,
                "kernel": "gemm_tc_pair_kernel<tf32,SW64,3 products> (CTA pairs, 256x256 tiles)", "kernel_ms": core_avg_ms,
                "prepass_ms": pre_ms / max(calls, 1),
                "peak_source": f"{peaks['source']} bf16 burst {peaks['bf16_tflops']} TFLOP/s / 2 (tf32 rate) / 3 (products)"}

    # ---------------- end to end: pinned host operands in, result out, every step
    e2e = None
    hA = torch.empty((GEMM_N, GEMM_N), pin_memory=True).copy_(A.cpu())
    hB = torch.empty((GEMM_N, GEMM_N), pin_memory=True).copy_(B.cpu())
    hC = torch.empty((GEMM_N, GEMM_N), pin_memory=True)
    nbytes = GEMM_N * GEMM_N * 4

    def e2e_step():
        eng.memcpy_h2d(A, hA.data_ptr(), nbytes)
        eng.memcpy_h2d(B, hB.data_ptr(), nbytes)
        eng.gemm(A, B, Cout)
        eng.memcpy_d2h(hC.data_ptr(), Cout, nbytes)

    def e2e_pipelined():
        eng.gemm_host(hA, hB, hC)   # the host-operand entry: chunked uploads overlap the GEMM and the download

    e2e_steps = max(1, min(K, 8))
    ms_serial = timed(torch, dist, world, e2e_step, e2e_steps, 1)
    ms_e2e = timed(torch, dist, world, e2e_pipelined, e2e_steps, 1)
    e2e = {"value": world * FLOP_HEADLINE / (ms_e2e / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": 2 * nbytes, "d2h_bytes_per_step": nbytes, "ms_per_step": ms_e2e / e2e_steps,
           "steps": e2e_steps, "api": "axb_gemm_host (pinned host A, B in, C out; transfers overlapped with the GEMM)",
           "serial_value": world * FLOP_HEADLINE / (ms_serial / e2e_steps * 1e-3) / 1e12,
           "serial_ms_per_step": ms_serial / e2e_steps,
           "serial_api": "axb_memcpy_h2d x2 + axb_gemm + axb_memcpy_d2h, one after the other (the vtable's order)"}
    del hA, hB, hC

    extra = []
    if not args.headline_only:
        extra = extras(torch, dist, world, eng, peaks, uniform, A, B, Cout, K)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cb = cpu_reference_gemm(3, 1)
        if cb:
            cpu_baseline = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}

    err = eng.device_error()
    if rank == 0:
        line = {
            "metric": "gemm_fp32_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "fp32-accurate GEMM C=A.B, M=N=K=8192 per GPU, U[-1,1], rows sharded across GPUs "
                                   "(weights replicated, no collective)", "fp32_mode": "3xtf32",
                       "l2": "inputs (512 MiB fp32 + 1 GiB operand planes) larger than L2", "parallelism": f"m-shard x{world}"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": launches,
            "clocks": clocks, "device_error": err, "extra": extra,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def graph_time(eng, fn, calls=64, replays=4):
    """Mean device time of one call of `fn`, from a CUDA graph of `calls` calls replayed on a side stream.
    A ~10 us kernel is launch-bound when driven call by call from Python; the graph shows the kernel's own
    duration.  Returns None when capture is not possible (the measurement then falls back to event timing)."""
    import torch
    ms = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        eng.set_stream(side.cuda_stream)
        with torch.cuda.stream(side):
            fn()
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(calls):
                    fn()
            for _ in range(3):
                g.replay()
            side.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            for _ in range(replays):
                g.replay()
            e1.record(side)
            side.synchronize()
            ms = e0.elapsed_time(e1) / (replays * calls)
    except Exception as exc:  # capture is an optimisation of the measurement, not of the product
        sys.stderr.write(f"bench: graph timing unavailable ({exc})\n")
    finally:
        eng.set_stream(0)
        torch.cuda.synchronize()
    return ms


def extras(torch, dist, world, eng, peaks, uniform, A, B, Cout, K):
    """The other metrics of the suite; each entry: workload, value, unit, ms, roofline fraction."""
    out = []
    hbm = peaks["hbm_gbs"]
    bf16 = peaks["bf16_tflops"]

    def core_time(fn, steps, warmup=3):
        for _ in range(warmup):
            fn()
        eng.set_profiling(True)
        ms = timed(torch, dist, world, fn, steps, 0)
        calls, pre, core = eng.timing_summary()
        eng.set_profiling(False)
        return ms / steps, core / max(calls, 1), pre / max(calls, 1)

    # fp32 GEMM 8192^3 in the two faster modes
    for mode, peak, note in (("bf16x3", bf16 / 3.0, "bf16 burst / 3 products"), ("bf16", bf16, "bf16 burst")):
        eng.set_fp32_mode(mode)
        step_ms, core_ms, pre_ms = core_time(lambda: eng.gemm(A, B, Cout), max(3, K // 2))
        eng.set_fp32_mode("3xtf32")
        tf = FLOP_HEADLINE / (core_ms * 1e-3) / 1e12
        out.append({"workload": f"fp32 GEMM 8192^3, mode {mode}", "value": world * FLOP_HEADLINE / (step_ms * 1e-3) / 1e12,
                    "unit": "TFLOP/s", "ms_per_step": step_ms, "kernel_ms": core_ms, "prepass_ms": pre_ms,
                    "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "frac": tf / peak, "peak_source": note}})

    # int8 GEMM 16384^3 -> requantised int8 (benchmark config 5b)
    n8 = 16384
    a8 = torch.randint(-127, 128, (n8, n8), device="cuda", dtype=torch.int8)
    b8 = torch.randint(-127, 128, (n8, n8), device="cuda", dtype=torch.int8)
    bs = torch.rand((n8,), device="cuda") * 0.019 + 0.001
    q8 = torch.empty((n8, n8), device="cuda", dtype=torch.int8)
    ops = 2.0 * n8 ** 3
    step_ms, core_ms, pre_ms = core_time(lambda: eng.qgemm_w8a8(a8, 0.02, b8, bs, 40.0, q8, None), max(3, K // 2), 2)
    tops = ops / (core_ms * 1e-3) / 1e12
    out.append({"workload": "int8 GEMM 16384^3, s32 accumulate, requantised int8 out", "value": world * ops / (step_ms * 1e-3) / 1e12,
                "unit": "TOPS", "ms_per_step": step_ms, "kernel_ms": core_ms,
                "roofline": {"bound": "tensor", "achieved": tops, "peak": 2 * bf16, "frac": tops / (2 * bf16),
                             "peak_source": "2 x measured bf16 burst (int8 issues at twice the bf16 rate)"}})
    del a8, b8, q8

    # skinny-M route: x[M,4096].W[4096,4096] + bias -> GELU (benchmark config 2); 8 rotating weight
    # buffers (512 MiB > L2) so every step streams W from HBM
    n = 4096
    Ws = [torch.randn((n, n), device="cuda") / 64 for _ in range(8)]
    bias = uniform((n,))
    for M in (1, 8, 32):
        x = torch.randn((M, n), device="cuda")
        y = torch.empty((M, n), device="cuda")
        state = {"i": 0}

        def sk():
            eng.gemm_bias_act(x, Ws[state["i"] % 8], bias, y, M, n, n, act="gelu")
            state["i"] += 1
        step_ms, core_ms, _ = core_time(sk, 64, 8)
        nbytes = n * n * 4 + 2 * M * n * 4 + n * 4
        graph_ms = graph_time(eng, sk)
        kern_ms = graph_ms if graph_ms else core_ms
        gbs = nbytes / (kern_ms * 1e-3) / 1e9
        out.append({"workload": f"skinny-M dense+bias+GELU, x[{M}x4096].W[4096x4096]", "value": nbytes / (step_ms * 1e-3) / 1e9,
                    "unit": "GB/s", "ms_per_step": step_ms, "kernel_ms": kern_ms, "kernel_ms_eager_events": core_ms,
                    "timing": "kernel_ms: mean over a replayed CUDA graph of 64 calls; value/ms_per_step: eager calls from Python",
                    "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "frac": gbs / hbm,
                                 "peak_source": f"{peaks['source']} HBM copy bandwidth"}})
    del Ws

    # dense + bias + ReLU 1024^3 (benchmark config 1)
    a1, b1, bias1 = uniform((1024, 1024)), uniform((1024, 1024)), uniform((1024,))
    c1 = torch.empty((1024, 1024), device="cuda")
    step_ms, core_ms, pre_ms = core_time(lambda: eng.gemm_relu(a1, b1, bias1, c1), 50, 5)
    out.append({"workload": "fp32 GEMM+bias+ReLU 1024^3 (3xTF32)", "value": 2.0 * 1024 ** 3 / (step_ms * 1e-3) / 1e12,
                "unit": "TFLOP/s", "ms_per_step": step_ms, "kernel_ms": core_ms, "prepass_ms": pre_ms})

    # quantised GEMM 512x4096x4096 (benchmark config 3): W8A8 and the reference's W8A32
    a3 = torch.randint(-127, 128, (512, 4096), device="cuda", dtype=torch.int8)
    b3 = torch.randint(-127, 128, (4096, 4096), device="cuda", dtype=torch.int8)
    s3 = torch.rand((4096,), device="cuda") * 0.019 + 0.001
    q3 = torch.empty((512, 4096), device="cuda", dtype=torch.int8)
    step_ms, core_ms, _ = core_time(lambda: eng.qgemm_w8a8(a3, 0.02, b3, s3, 20.0, q3, None), 50, 5)
    out.append({"workload": "int8 W8A8 GEMM 512x4096x4096 -> int8", "value": 2.0 * 512 * 4096 * 4096 / (step_ms * 1e-3) / 1e12,
                "unit": "TOPS", "ms_per_step": step_ms, "kernel_ms": core_ms})
    af = uniform((512, 4096))
    of = torch.empty((512, 4096), device="cuda")
    step_ms, core_ms, pre_ms = core_time(lambda: eng.qgemm_w8a32(af, b3, s3, of), 30, 3)
    out.append({"workload": "W8A32 GEMM 512x4096x4096 (fp32 activations, int8 weights)",
                "value": 2.0 * 512 * 4096 * 4096 / (step_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": step_ms,
                "kernel_ms": core_ms, "prepass_ms": pre_ms})

    # W8A32 at bs=1: the case the reference's quantised path exists for (int8 weights streamed once);
    # rotating weight buffers of 256 MiB in total (> L2) so every call streams from HBM
    # bs = 8 and 32 (batched decode) take the integer tensor-core kernel: activations as int8 digit planes
    for nq, bs in ((4096, 1), (16384, 1), (16384, 8), (16384, 32)):
        try:
            nbuf = 256 * 2 ** 20 // (nq * 4096)
            w8 = [torch.randint(-127, 128, (nq, 4096), device="cuda", dtype=torch.int8) for _ in range(nbuf)]
            sq = torch.rand((nq,), device="cuda") * 0.019 + 0.001
            x1, o1 = uniform((bs, 4096)), torch.empty((bs, nq), device="cuda")
            st8 = {"i": 0}

            def qv():
                eng.qgemm_w8a32(x1, w8[st8["i"] % nbuf], sq, o1)
                st8["i"] += 1
            step_ms, core_ms, _ = core_time(qv, 64, 8)
            kern_ms = graph_time(eng, qv) or core_ms
            nb = nq * 4096 + bs * 4096 * 4 + (1 + bs) * nq * 4
            out.append({"workload": f"W8A32 GEMV bs={bs}, int8 W[{nq}x4096] ({nbuf} rotating weight buffers)",
                        "value": nb / (step_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": step_ms, "kernel_ms": kern_ms,
                        "kernel_ms_eager_events": core_ms,
                        "timing": "kernel_ms: mean over a replayed CUDA graph of 64 calls; value/ms_per_step: eager calls from Python",
                        "roofline": {"bound": "hbm", "achieved": nb / (kern_ms * 1e-3) / 1e9, "peak": hbm,
                                     "frac": nb / (kern_ms * 1e-3) / 1e9 / hbm, "peak_source": f"{peaks['source']} HBM copy bandwidth"}})
            del w8
        except Exception as exc:
            out.append({"workload": f"W8A32 GEMV bs={bs} N={nq}", "error": repr(exc)})

    # causal attention B=8,H=16,S=1024,dk=64 (benchmark config 4); FLOPs by the reference's 4*BH*S^2*dk convention
    BH, S, dk = 128, 1024, 64
    Q, Kt, V = (torch.randn((BH, S, dk), device="cuda") for _ in range(3))
    O = torch.empty((BH, S, dk), device="cuda")
    L = torch.empty((BH, S), device="cuda")
    step_ms, core_ms, _ = core_time(lambda: eng.sdpa_fwd(Q, Kt, V, O, L, 0.125, True), 20, 3)
    # tensor work actually issued: 128-row query tiles x 128-key blocks at or below the diagonal, two contractions
    tiles = S // 128
    done = 2 * 2.0 * BH * (tiles * (tiles + 1) // 2) * 128 * 128 * dk
    tf = done / (core_ms * 1e-3) / 1e12
    out.append({"workload": "causal SDPA fwd BH=128 S=1024 dk=64 (fp32 in/out, 3xTF32 on the tensor cores)",
                "value": 4.0 * BH * S * S * dk / (step_ms * 1e-3) / 1e12,
                "unit": "TFLOP/s (4*BH*S^2*dk convention; causal does half)", "ms_per_step": step_ms, "kernel_ms": core_ms,
                "roofline": {"bound": "tensor", "achieved": tf, "peak": bf16 / 6, "frac": tf / (bf16 / 6), "unit": "TFLOP/s",
                             "peak_source": "measured bf16 burst / 2 (tf32 rate) / 3 (products)",
                             "note": "achieved counts the useful FLOP of the key blocks the kernel visits (diagonal blocks whole)"}})
    # convolution as GEMM: a ResNet 3x3 layer on one sample (C_in = C_out = 256, 56x56, pad 1): weight [256 x 2304]
    try:
        wc, xc = torch.randn((256, 2304), device="cuda") / 48, uniform((256, 56, 56))
        oc = torch.empty((256, 56 * 56), device="cuda")
        step_ms, core_ms, pre_ms = core_time(lambda: eng.conv_gemm(wc, xc, 3, 3, 1, 1, 1, 1, oc), 20, 3)
        out.append({"workload": "conv 3x3 pad 1 as GEMM, one sample [256,56,56] -> [256,56,56] (implicit im2col into the operand planes)",
                    "value": 2.0 * 256 * 2304 * 3136 / (step_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": step_ms,
                    "kernel_ms": core_ms, "prepass_ms": pre_ms})
    except Exception as exc:
        out.append({"workload": "conv 3x3 as GEMM", "error": repr(exc)})

    # attention backward at config 4 (fp32 FMA kernels; recomputes the scores, no S x S buffer)
    try:
        dOt = torch.randn((BH, S, dk), device="cuda")
        gq, gk, gv = (torch.empty((BH, S, dk), device="cuda") for _ in range(3))
        step_ms, core_ms, _ = core_time(lambda: eng.sdpa_bwd(Q, Kt, V, O, dOt, L, gq, gk, gv, 0.125, True), 10, 2)
        out.append({"workload": "causal SDPA bwd BH=128 S=1024 dk=64 (fp32 FMA, dQ and dK/dV kernels)",
                    "value": 2.5 * 4.0 * BH * S * S * dk / (step_ms * 1e-3) / 1e12,
                    "unit": "TFLOP/s (2.5 x the forward's 4*BH*S^2*dk convention; causal does half)", "ms_per_step": step_ms,
                    "kernel_ms": core_ms})
    except Exception as exc:
        out.append({"workload": "causal SDPA bwd", "error": repr(exc)})

    # fused QKV projection into the head-major layout: B=8, S=1024, D=1024 (H=16, dk=64, the config-4 heads)
    try:
        Bq, Sq, Hq = 8, 1024, 16
        Dq = Hq * dk
        Xq, Wq, bq = uniform((Bq * Sq, Dq)), torch.randn((Dq, 3 * Dq), device="cuda") / 32, uniform((3 * Dq,))
        heads = [torch.empty((Bq * Hq, Sq, dk), device="cuda") for _ in range(3)]
        step_ms, core_ms, pre_ms = core_time(lambda: eng.qkv_head_gemm(Xq, Wq, bq, Bq, Sq, Hq, dk, *heads), 20, 3)
        fl = 2.0 * Bq * Sq * Dq * 3 * Dq
        out.append({"workload": "QKV projection + head-major split, X[8192x1024].Wqkv[1024x3072]+b -> Qh,Kh,Vh [128,1024,64] (one launch)",
                    "value": fl / (step_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": step_ms, "kernel_ms": core_ms,
                    "prepass_ms": pre_ms})
    except Exception as exc:
        out.append({"workload": "QKV projection + head-major split", "error": repr(exc)})

    # single-token decode against a KV cache: config-4 heads (BH=128, dk=64), 4096 cached tokens = 268 MB of K and V
    try:
        kc, vc = (torch.randn((BH, 4096, dk), device="cuda") for _ in range(2))
        qn, on = torch.randn((BH, dk), device="cuda"), torch.empty((BH, dk), device="cuda")
        kv = lambda: eng.kv_cache_attend(kc, vc, qn, on, 4096, 0.125)
        step_ms, core_ms, _ = core_time(kv, 32, 4)
        kern_ms = graph_time(eng, kv, calls=16) or core_ms
        nb = 2.0 * BH * 4096 * dk * 4
        out.append({"workload": "KV-cache attention, 1 new token, BH=128, 4096 cached tokens, dk=64 (K+V = 268 MB > L2)",
                    "value": nb / (step_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": step_ms, "kernel_ms": kern_ms,
                    "kernel_ms_eager_events": core_ms,
                    "roofline": {"bound": "hbm", "achieved": nb / (kern_ms * 1e-3) / 1e9, "peak": hbm,
                                 "frac": nb / (kern_ms * 1e-3) / 1e9 / hbm, "peak_source": f"{peaks['source']} HBM copy bandwidth"}})
        del kc, vc
    except Exception as exc:
        out.append({"workload": "KV-cache attention", "error": repr(exc)})
    # the fp32-FMA kernel that serves head dims above 64, on its own largest case
    Q2, K2, V2 = (torch.randn((64, 1024, 128), device="cuda") for _ in range(3))
    O2 = torch.empty((64, 1024, 128), device="cuda")
    step_ms, core_ms, _ = core_time(lambda: eng.sdpa_fwd(Q2, K2, V2, O2, None, 0.0884, True), 10, 3)
    out.append({"workload": "causal SDPA fwd BH=64 S=1024 dk=128 (fp32 FMA kernel)", "value": 4.0 * 64 * S * S * 128 / (step_ms * 1e-3) / 1e12,
                "unit": "TFLOP/s (4*BH*S^2*dk convention; causal does half)", "ms_per_step": step_ms, "kernel_ms": core_ms})
    del Q, Kt, V, O, L, Q2, K2, V2, O2

    # LAST, because it runs for seconds at the power cap and leaves the clocks low for whatever follows:
    # 3-layer MLP 8192 -> 16384 -> 16384 -> 8192 at batch 16384, bias + GELU fused (benchmark config 5c):
    # rows of the batch sharded over the ranks (no collective), and, with more than one rank, output
    # columns sharded with one all-gather per layer.  Fixed total batch: strong scaling for this line.
    try:
        out.extend(mlp_extras(torch, dist, world, eng, K))
    except Exception as exc:
        out.append({"workload": "3-layer MLP batch 16384", "error": repr(exc)})
    return out


def run_profile_case(args):
    """A short, small run of one route for capture under a profiler: 1 warm-up + 2 calls, then exit.
    Not a benchmark: prints nothing that should be read as a measurement."""
    import torch
    from axiom_b200.engine import get_engine
    torch.cuda.set_device(0)
    eng = get_engine(0)
    n = args.size
    case = args.profile_case
    if case.startswith("gemm_fp32"):
        mode = case.split(":")[1] if ":" in case else "3xtf32"
        eng.set_fp32_mode(mode)
        A, B = torch.rand((n, n), device="cuda") * 2 - 1, torch.rand((n, n), device="cuda") * 2 - 1
        C = torch.empty((n, n), device="cuda")
        fn = lambda: eng.gemm(A, B, C)
    elif case == "gemm_int8":
        a = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
        b = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
        bs = torch.rand((n,), device="cuda") * 0.019 + 0.001
        q = torch.empty((n, n), device="cuda", dtype=torch.int8)
        fn = lambda: eng.qgemm_w8a8(a, 0.02, b, bs, 40.0, q, None)
    elif case.startswith("skinny"):
        M = int(case.split(":")[1]) if ":" in case else 1
        Ws = [torch.randn((4096, 4096), device="cuda") / 64 for _ in range(4)]
        x, bias, y = torch.randn((M, 4096), device="cuda"), torch.rand((4096,), device="cuda"), torch.empty((M, 4096), device="cuda")
        state = {"i": 0}

        def fn():
            eng.gemm_bias_act(x, Ws[state["i"] % 4], bias, y, M, 4096, 4096, act="gelu")
            state["i"] += 1
    elif case == "qgemv":
        # the fp32-FMA GEMV itself: at this size a single row would otherwise take the integer tensor-core kernel
        os.environ["AX_B200_QSKINNY_TC_MIN"] = "65"
        Wq = [torch.randint(-127, 128, (16384, 4096), device="cuda", dtype=torch.int8) for _ in range(4)]
        sc = torch.rand((16384,), device="cuda") * 0.019 + 0.001
        xq, oq = torch.randn((1, 4096), device="cuda"), torch.empty((1, 16384), device="cuda")
        state = {"i": 0}

        def fn():
            eng.qgemm_w8a32(xq, Wq[state["i"] % 4], sc, oq)
            state["i"] += 1
    elif case == "qskinny":
        Wq = [torch.randint(-127, 128, (16384, 4096), device="cuda", dtype=torch.int8) for _ in range(4)]
        sc = torch.rand((16384,), device="cuda") * 0.019 + 0.001
        xq, oq = torch.randn((8, 4096), device="cuda"), torch.empty((8, 16384), device="cuda")
        state = {"i": 0}

        def fn():
            eng.qgemm_w8a32(xq, Wq[state["i"] % 4], sc, oq)
            state["i"] += 1
    elif case == "kv":
        kc, vc = (torch.randn((128, 4096, 64), device="cuda") for _ in range(2))
        qn, on = torch.randn((128, 64), device="cuda"), torch.empty((128, 64), device="cuda")
        fn = lambda: eng.kv_cache_attend(kc, vc, qn, on, 4096, 0.125)
    elif case == "sdpa":
        Q, K, V = (torch.randn((128, 1024, 64), device="cuda") for _ in range(3))
        O, L = torch.empty((128, 1024, 64), device="cuda"), torch.empty((128, 1024), device="cuda")
        fn = lambda: eng.sdpa_fwd(Q, K, V, O, L, 0.125, True)
    else:
        raise SystemExit(f"unknown profile case {case}")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    assert eng.device_error() == 0
    print(json.dumps({"profile_case": case, "size": n, "calls": 3, "note": "not a measurement"}))


def mlp_extras(torch, dist, world, eng, K):
    from axiom_b200.multi_gpu import ColumnShardedMLP, RowShardedMLP, shard_bounds
    rank = dist.get_rank() if world > 1 else 0
    dims = [8192, 16384, 16384, 8192]
    batch = 16384
    flop = 2.0 * batch * sum(dims[i] * dims[i + 1] for i in range(3))
    gen = torch.Generator(device="cuda").manual_seed(99)          # same weights on every rank
    Ws = [torch.randn((dims[i], dims[i + 1]), device="cuda", generator=gen) / (dims[i] ** 0.5) for i in range(3)]
    bs = [torch.rand((dims[i + 1],), device="cuda", generator=gen) * 2 - 1 for i in range(3)]
    x = torch.rand((batch, dims[0]), device="cuda", generator=gen) * 2 - 1
    new_empty = lambda shape: torch.empty(shape, device="cuda", dtype=torch.float32)
    steps = max(2, min(K, 3))
    res = []
    r0, r1 = shard_bounds(batch, world, rank)
    rows = RowShardedMLP(eng, Ws, bs, act="gelu")
    xr = x[r0:r1].contiguous()
    ms = timed(torch, dist, world, lambda: rows.forward(xr, new_empty), steps, 1) / steps
    res.append({"workload": f"3-layer MLP 8192-16384-16384-8192, batch 16384, rows sharded x{world} (no collective)",
                "value": flop / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "kernel_ms": ms, "scaling": "strong"})
    if world > 1:
        slabs, bias_slabs = [], []
        for W, b in zip(Ws, bs):
            c0, c1 = shard_bounds(W.shape[1], world, rank)
            slabs.append(W[:, c0:c1].contiguous())
            bias_slabs.append(b[c0:c1].contiguous())
        del Ws
        torch.cuda.empty_cache()
        ag = lambda dst, src: dist.all_gather_into_tensor(dst.view(-1, dst.shape[-1]), src)
        cols = ColumnShardedMLP(eng, slabs, bias_slabs, world, rank, ag, act="gelu")
        ms = timed(torch, dist, world, lambda: cols.forward(x, new_empty), steps, 1) / steps
        fused = None
        try:
            from axiom_b200.multi_gpu import PeerScatterColumnMLP
            fused = PeerScatterColumnMLP(eng, slabs, bias_slabs, world, rank, batch, dist, act="gelu")
            ms_f = timed(torch, dist, world, lambda: fused.forward(x, new_empty), steps, 1) / steps
            # the two data paths must agree bit for bit (same kernels, same operands; only the route of the slabs differs)
            y_ref = cols.forward(x, new_empty)
            out_ptr, n_last = fused.forward(x, new_empty)
            y_fused = torch.empty_like(y_ref)
            eng._check(eng.lib.axb_memcpy_d2d(ctypes.c_void_p(y_fused.data_ptr()), ctypes.c_void_p(out_ptr), y_ref.numel() * 4))
            torch.cuda.synchronize()
            fused_equal = bool(torch.equal(y_fused, y_ref))
            res.append({"workload": f"3-layer MLP, batch 16384, output columns sharded x{world}, gather fused into the GEMM "
                                    "epilogue as peer stores over NVLink (one 4-byte all-reduce per layer to order reads)",
                        "value": flop / (ms_f * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_f, "kernel_ms": ms_f,
                        "scaling": "strong", "bit_identical_to_nccl_path": fused_equal})
        except Exception as exc:
            res.append({"workload": "3-layer MLP, peer-store gather", "error": repr(exc)})
        finally:
            if fused is not None:
                fused.close()
        res.append({"workload": f"3-layer MLP, batch 16384, output columns sharded x{world}, NCCL all-gather per layer",
                    "value": flop / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "kernel_ms": ms,
                    "scaling": "strong", "allgather_bytes_per_rank_per_layer": [batch * d // world * 4 for d in dims[1:]]})
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--headline-only", action="store_true", help="skip the extra workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--profile-case", default=None,
                    help="gemm_fp32[:mode] | gemm_int8 | skinny[:M] | sdpa — 3 calls of one route on a small case, for ncu")
    ap.add_argument("--size", type=int, default=4096, help="matrix size of --profile-case")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
