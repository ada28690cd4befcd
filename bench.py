#!/usr/bin/env python
"""Benchmark of the axiom matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--only NAME[,NAME...]]

Headline (ONE JSON line on stdout): fp32-accurate GEMM, M=N=K=8192 per GPU
(rows sharded across GPUs, weights replicated, no data-path collective: weak
scaling), in TFLOP/s through the C ABI (operand split pre-pass + tcgen05
kernel, both inside the timed step).  The other metrics of the suite on the same
box — int8 TOPS at 16384^3, the bs=1 / 8 / 32 skinny-M route in GB/s, the 1024^3
dense+ReLU, the 512x4096x4096 quantised GEMMs, causal attention forward and
backward, the 3-layer MLP — ride inside the line as compact records
(`roofline.suite`, CPU baselines under `cpu_baseline.per_config`); their full
records go to stderr as one JSON line.  Every timed output is checked against
the CPU oracle on sampled rows (`parity_checked`).

`--only` runs the named suite workloads alone (no headline line): the form the
profiling captures under profiles/ use.

`--impl reference` times the reference's own CPU path (the compiled axiom
library under oracle/_ref, OpenMP over the box's host cores) on the same
configuration and prints the same line with "impl": "reference".
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
SEED = 1234


def headline_config(world):
    """The workload both arms are timed on (BASELINE config 5a); identical in both JSON lines."""
    return {"workload": "fp32-accurate GEMM C=A.B, M=N=K=8192 per GPU, U[-1,1] seeded, rows sharded across GPUs "
                        "(weights replicated, no collective)",
            "arithmetic": "fp32 in, fp32 out, normalised error <= 1e-5 (GPU arm: 3xTF32 on the tensor cores; reference arm: "
                          "fp32 FMA on the host cores)",
            "l2": "inputs (512 MiB fp32, 1 GiB of operand planes) larger than L2", "parallelism": f"m-shard x{world}"}


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


def med_min(xs):
    return (statistics.median(xs), min(xs)) if xs else (None, None)


# --------------------------------------------------------------------------- CPU legs (the reference's own code)

def host_threads_for_reference():
    """The reference picks its own thread count (ax_autotune_threads) when OMP_NUM_THREADS is unset; a launcher's
    OMP_NUM_THREADS=1 (torchrun exports it) would pin it to one core.  Must run before libgomp is loaded."""
    os.environ.pop("OMP_NUM_THREADS", None)
    return len(os.sched_getaffinity(0))


def load_reference(autotune=True):
    from oracle_lib import Oracle, Reference
    if not Reference.available():
        return None, None
    return Reference(autotune=autotune), Oracle()   # the reference's tuning happens here, outside every timing


def cpu_headline(ref, o, steps, warmup, budget_s=200.0):
    """ax_compute_gemm on the 8192^3 problem: operands built once, only the call timed.  The whole problem when
    warmup + steps runs fit the budget, otherwise the largest whole-row slice of A that does (stated in `sample`)."""
    import numpy as np
    A = o.uniform((GEMM_N, GEMM_N), 7)
    B = o.uniform((GEMM_N, GEMM_N), 13)
    out = np.empty((GEMM_N, GEMM_N), np.float32)
    probe = ref.time_gemm(A, B, out, 0, 1)[0]          # first call: also the first warm-up
    rows = GEMM_N
    runs_left = max(warmup - 1, 0) + steps
    if probe * runs_left > budget_s:
        rows = max(256, int(GEMM_N * budget_s / (probe * runs_left)) // 256 * 256)
    secs = ref.time_gemm(A[:rows], B, out[:rows], max(warmup - 1, 0), steps)
    flop = 2.0 * rows * GEMM_N * GEMM_N
    med, mn = med_min(secs)
    mean = sum(secs) / len(secs)
    what = "the whole 8192^3 problem" if rows == GEMM_N else f"a {rows}-row slice of A against the whole B (time budget)"
    return {"value": flop / mean / 1e12, "unit": "TFLOP/s", "cores": ref.num_threads(), "kind": "reference",
            "sample": f"axiom ax_compute_gemm (cpu_opt, OpenMP, autotuned outside the timing) on {what}; operands built once, "
                      f"only the call timed; mean of {len(secs)} runs after {warmup} warm-ups; host offers {len(os.sched_getaffinity(0))} cpus",
            "ms_per_step": mean * 1e3, "ms_median": med * 1e3, "ms_min": mn * 1e3, "rows": rows}


def cpu_per_config(ref, o, iters=3):
    """The reference's CPU entry point of each of the other benchmark configurations, same shapes as the GPU lines."""
    import numpy as np
    res = []

    def add(name, entry, secs, work, unit):
        med, mn = med_min(secs)
        res.append({"config": name, "entry": entry, "ms_median": med * 1e3, "ms_min": mn * 1e3,
                    "value": work / med / (1e12 if unit != "GB/s" else 1e9), "unit": unit})

    a, b, bias = o.uniform((1024, 1024), 7), o.uniform((1024, 1024), 13), o.uniform((1024,), 29)
    add("C1 1024^3 +bias+ReLU", "ax_matmul_bias_relu", ref.time_matmul_bias_relu(a, b, bias, np.empty((1024, 1024), np.float32), 2, iters + 2),
        2.0 * 1024 ** 3, "TFLOP/s")
    W, b2 = o.normal((4096, 4096), 13, sigma=1 / 64), o.uniform((4096,), 29)
    for M in (1, 32):
        x = o.normal((M, 4096), 31)
        add(f"C2 x[{M}x4096].W+bias->GELU", "ax_compute_gemm + column bias + ax_gelu",
            ref.time_dense_gelu(x, W, b2, np.empty((M, 4096), np.float32), 2, iters + 2), 4096 * 4096 * 4.0, "GB/s")
    a3 = o.uniform((512, 4096), 7)
    q, s = o.quantize_rows(o.uniform((4096, 4096), 13))
    add("C3 W8A32 512x4096x4096", "ax_qgemm_w8a32", ref.time_qgemm_w8a32(a3, q, s, np.empty((512, 4096), np.float32), 1, iters),
        2.0 * 512 * 4096 * 4096, "TFLOP/s")
    x1 = o.uniform((1, 4096), 31)
    add("W8A32 GEMV bs=1 4096x4096", "ax_qgemm_w8a32", ref.time_qgemm_w8a32(x1, q, s, np.empty((1, 4096), np.float32), 2, iters + 2),
        4096 * 4096 * 1.0, "GB/s")
    Q, K, V = (o.normal((128, 1024, 64), sd) for sd in (41, 43, 47))
    add("C4 causal SDPA BH=128 S=1024 dk=64", "ax_fused_attention_fwd_causal",
        ref.time_sdpa_causal(Q, K, V, np.empty_like(Q), np.empty((128, 1024), np.float32), 0.125, 1, iters),
        4.0 * 128 * 1024 * 1024 * 64, "TFLOP/s")
    return res


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    host_threads_for_reference()
    ref, o = load_reference(autotune=True)
    if ref is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libaxiom_ref.so was not built"}))
        return
    K, W = max(args.steps, 1), max(args.warmup, 1)
    cb = cpu_headline(ref, o, K, W)
    line = {
        "impl": "reference", "metric": "gemm_fp32_tflops", "value": cb["value"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_step"],
        "ms_median": cb["ms_median"], "ms_min": cb["ms_min"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(args.gpus),
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- our arm

class Ctx:
    """What every suite workload needs: torch, the engine, the process group, the peaks and the CPU oracle."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        from axiom_b200.engine import get_engine
        from oracle_lib import Oracle
        self.torch, self.dist = torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
        self.eng = get_engine(self.local)
        self.peaks = measured_peaks()
        self.K, self.W = max(args.steps, 1), max(args.warmup, 3)
        # --steps below 5: a short pass for captures under a profiler (few launches, no graph replays)
        self.short = args.steps < 5
        self.oracle = Oracle()
        self.gen = torch.Generator(device="cuda").manual_seed(SEED + self.rank)

    def uniform(self, shape):
        return self.torch.rand(shape, device="cuda", generator=self.gen) * 2 - 1

    def normal(self, shape, sigma=1.0):
        return self.torch.randn(shape, device="cuda", generator=self.gen) * sigma

    def int8(self, shape):
        return self.torch.randint(-127, 128, shape, device="cuda", dtype=self.torch.int8, generator=self.gen)

    def timed(self, fn, steps, warmup):
        """W warm-ups, then exactly `steps` calls between barrier+synchronize pairs, one CUDA event per call boundary.
        Returns (total ms as the max over ranks, per-step ms list of this rank)."""
        torch, dist = self.torch, self.dist
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        ev[0].record()
        for i in range(steps):
            fn()
            ev[i + 1].record()
        torch.cuda.synchronize()
        ms = ev[0].elapsed_time(ev[steps])
        per = [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]
        if self.world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.barrier()
            ms = float(t.item())
        return ms, per

    def core_time(self, fn, steps, warmup=3):
        """Step time and, from the engine's own events around each call's pre-pass and main kernel, their medians."""
        eng = self.eng
        if self.short:
            steps, warmup = 2, 1
        for _ in range(warmup):
            fn()
        eng.set_profiling(True)
        ms, per = self.timed(fn, steps, 0)
        pre, core = eng.timing_samples()
        eng.set_profiling(False)
        step_med, step_min = med_min(per)
        # a call with several main kernels records one window per kernel-carrying sub-call: fold to per-step sums
        per_call = max(1, len(core) // steps) if len(core) >= steps else 1
        if per_call > 1 and len(core) % steps == 0:
            core = [sum(core[i * per_call:(i + 1) * per_call]) for i in range(steps)]
            pre = [sum(pre[i * per_call:(i + 1) * per_call]) for i in range(steps)]
        k_med, k_min = med_min(core)
        p_med, _ = med_min(pre)
        return {"ms_per_step": ms / steps, "ms_median": step_med, "ms_min": step_min, "kernel_ms": k_med,
                "kernel_ms_min": k_min, "prepass_ms": p_med}

    def graph_time(self, fn, calls=64, replays=4):
        """Mean device time of one call of `fn`, from a CUDA graph of `calls` calls replayed on a side stream.
        A ~10 us kernel is launch-bound when driven call by call from Python; the graph shows the kernel's own
        duration.  Returns None when capture is not possible (the measurement then falls back to event timing)."""
        torch, eng = self.torch, self.eng
        ms = None
        if self.short:
            return None
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
                samples = []
                for _ in range(replays):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(side)
                    g.replay()
                    e1.record(side)
                    side.synchronize()
                    samples.append(e0.elapsed_time(e1) / calls)
                ms = statistics.median(samples)
        except Exception as exc:  # capture is an optimisation of the measurement, not of the product
            sys.stderr.write(f"bench: graph timing unavailable ({exc})\n")
        finally:
            eng.set_stream(0)
            torch.cuda.synchronize()
        return ms


def host(t):
    return t.detach().cpu().numpy()


def nerr(x, ref):
    from oracle_lib import nerr as _n
    return _n(x, ref)


def sample_rows(n, count=4):
    return sorted({0, n - 1, *[(n * (2 * i + 1)) // (2 * count) for i in range(count)]})


def check_gemm_rows(ctx, A, B, C, tol, rows=None):
    """Sampled rows of C = A.B against the double-precision oracle; returns (ok, normalised error)."""
    import numpy as np
    rows = rows or sample_rows(A.shape[0])
    Ah = np.ascontiguousarray(host(A[rows]))
    want = ctx.oracle.gemm_f64(Ah, np.ascontiguousarray(host(B)))
    e = nerr(host(C[rows]), want)
    return bool(e <= tol), e


def headline(ctx, args):
    torch, eng = ctx.torch, ctx.eng
    peaks, K, W = ctx.peaks, ctx.K, ctx.W
    A, B = ctx.uniform((GEMM_N, GEMM_N)), ctx.uniform((GEMM_N, GEMM_N))
    Cout = torch.empty((GEMM_N, GEMM_N), device="cuda")
    step = lambda: eng.gemm(A, B, Cout)
    for _ in range(W):
        step()
    eng.set_profiling(True)
    try:
        gpu_id = "GPU-" + str(torch.cuda.get_device_properties(ctx.local).uuid)
    except Exception:
        gpu_id = str(ctx.local)
    sampler = ClockSampler(gpu_id)
    if ctx.rank == 0:
        sampler.start()
    eng.launch_count(reset=True)
    ms, per = ctx.timed(step, K, 0)
    launches = eng.launch_count()
    clocks = sampler.stop() if ctx.rank == 0 else None
    pre, core = eng.timing_samples()
    eng.set_profiling(False)
    ms_per_step = ms / K
    value = ctx.world * FLOP_HEADLINE / (ms_per_step * 1e-3) / 1e12
    core_avg_ms = sum(core) / max(len(core), 1)
    k_med, k_min = med_min(core)
    step_med, step_min = med_min(per)
    tf32_split_peak = peaks["bf16_tflops"] / 2.0 / 3.0   # TF32 issues at half the bf16 rate; 3 products per result
    achieved = FLOP_HEADLINE / (core_avg_ms * 1e-3) / 1e12
    ok, e = check_gemm_rows(ctx, A, B, Cout, 1e-5)
    roofline = {"bound": "tensor", "achieved": achieved, "peak": tf32_split_peak, "unit": "TFLOP/s",
                "frac": achieved / tf32_split_peak,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload, from the
                # ncu capture summarised for this kernel; algorithmic bytes: 4 operand planes + C
                "traffic": 6.65e9, "algorithmic_bytes": 1.34e9,
                "kernel": "gemm_tc_pair_kernel<tf32, 3 products> (CTA pairs, 256x256 tiles)", "kernel_ms": core_avg_ms,
                "kernel_ms_median": k_med, "kernel_ms_min": k_min, "prepass_ms": sum(pre) / max(len(pre), 1),
                "peak_source": f"{peaks['source']} bf16 burst {peaks['bf16_tflops']} TFLOP/s / 2 (tf32 rate) / 3 (products)"}

    # ---------------- end to end: pinned host operands in, result out, every step
    hA = torch.empty((GEMM_N, GEMM_N), pin_memory=True).copy_(A.cpu())
    hB = torch.empty((GEMM_N, GEMM_N), pin_memory=True).copy_(B.cpu())
    hC = torch.empty((GEMM_N, GEMM_N), pin_memory=True)
    nbytes = GEMM_N * GEMM_N * 4

    def e2e_serial():
        eng.memcpy_h2d(A, hA.data_ptr(), nbytes)
        eng.memcpy_h2d(B, hB.data_ptr(), nbytes)
        eng.gemm(A, B, Cout)
        eng.memcpy_d2h(hC.data_ptr(), Cout, nbytes)

    def e2e_pipelined():
        eng.gemm_host(hA, hB, hC)   # the host-operand entry: chunked uploads overlap the GEMM and the download

    # the host-side ceiling of this step: a plain pinned upload of one operand on every rank at the same time (the ranks
    # of one box share the host's memory and PCIe root ports), max over ranks
    ms_up, _ = ctx.timed(lambda: eng.memcpy_h2d(A, hA.data_ptr(), nbytes), 3, 1)
    h2d_gbs = nbytes / (ms_up / 3 * 1e-3) / 1e9

    e2e_steps = max(1, min(K, 8))
    ms_serial, _ = ctx.timed(e2e_serial, e2e_steps, 1)
    ms_e2e, per_e2e = ctx.timed(e2e_pipelined, e2e_steps, 1)
    rows = sample_rows(GEMM_N)
    e2e_same = bool(torch.equal(hC[rows], Cout[rows].cpu()))
    e2e_med, e2e_min = med_min(per_e2e)
    e2e = {"value": ctx.world * FLOP_HEADLINE / (ms_e2e / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": 2 * nbytes, "d2h_bytes_per_step": nbytes, "ms_per_step": ms_e2e / e2e_steps,
           "ms_median": e2e_med, "ms_min": e2e_min,
           "steps": e2e_steps, "api": "axb_gemm_host (pinned host A, B in, C out; transfers overlapped with the GEMM)",
           "parity_checked": e2e_same, "parity": "sampled rows bit-identical to the device-resident call",
           "serial_value": ctx.world * FLOP_HEADLINE / (ms_serial / e2e_steps * 1e-3) / 1e12,
           "serial_ms_per_step": ms_serial / e2e_steps,
           "serial_api": "axb_memcpy_h2d x2 + axb_gemm + axb_memcpy_d2h, one after the other (the vtable's order)",
           # what the host delivers: pinned H2D rate per GPU with all ranks uploading at once (slowest rank), and the
           # step time that rate alone allows (the step uploads 2 operands)
           "h2d_gbs_per_gpu_all_ranks_at_once": h2d_gbs, "h2d_gbs_aggregate": h2d_gbs * ctx.world,
           "upload_floor_ms": 2 * nbytes / (h2d_gbs * 1e9) * 1e3}
    del hA, hB, hC
    line = {
        "metric": "gemm_fp32_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": ctx.world, "steps": K, "warmup": W,
        "ms_per_step": ms_per_step, "ms_median": step_med, "ms_min": step_min, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(ctx.world),
        "roofline": roofline, "cpu_baseline": None, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        "parity_checked": ok, "parity": {"check": "sampled rows vs the float64 oracle", "nerr": e, "tol": 1e-5},
    }
    return line, (A, B, Cout)


# --------------------------------------------------------------------------- suite workloads

def hbm_roof(ctx, nbytes, kern_ms):
    hbm = ctx.peaks["hbm_gbs"]
    gbs = nbytes / (kern_ms * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": gbs, "peak": hbm, "frac": gbs / hbm, "unit": "GB/s",
            "peak_source": f"{ctx.peaks['source']} HBM copy bandwidth"}


def tensor_roof(achieved, peak, src):
    return {"bound": "tensor", "achieved": achieved, "peak": peak, "frac": achieved / peak, "unit": "TFLOP/s", "peak_source": src}


def w_gemm_modes(ctx, shared):
    """fp32 GEMM 8192^3 in the two faster modes (same operands as the headline)."""
    eng, bf16 = ctx.eng, ctx.peaks["bf16_tflops"]
    if shared is None:
        A, B = ctx.uniform((GEMM_N, GEMM_N)), ctx.uniform((GEMM_N, GEMM_N))
        Cout = ctx.torch.empty((GEMM_N, GEMM_N), device="cuda")
    else:
        A, B, Cout = shared
    out = []
    for mode, peak, note, tol in (("bf16x3", bf16 / 3.0, "bf16 burst / 3 products", 1e-5), ("bf16", bf16, "bf16 burst", 5e-3)):
        eng.set_fp32_mode(mode)
        t = ctx.core_time(lambda: eng.gemm(A, B, Cout), max(3, ctx.K // 2))
        ok, e = check_gemm_rows(ctx, A, B, Cout, tol)
        eng.set_fp32_mode("3xtf32")
        tf = FLOP_HEADLINE / (t["kernel_ms"] * 1e-3) / 1e12
        out.append(dict(t, name=f"gemm8192_{mode}", workload=f"fp32 GEMM 8192^3, mode {mode}",
                        value=ctx.world * FLOP_HEADLINE / (t["ms_per_step"] * 1e-3) / 1e12, unit="TFLOP/s",
                        roofline=tensor_roof(tf, peak, note), parity_checked=ok, parity_nerr=e))
    return out


def w_int8_16384(ctx, shared):
    """int8 GEMM 16384^3 -> requantised int8 (benchmark config 5b); sampled rows bit-exact against the oracle."""
    import numpy as np
    torch, eng, bf16 = ctx.torch, ctx.eng, ctx.peaks["bf16_tflops"]
    n8 = 16384
    a8, b8 = ctx.int8((n8, n8)), ctx.int8((n8, n8))
    bs = torch.rand((n8,), device="cuda", generator=ctx.gen) * 0.019 + 0.001
    q8 = torch.empty((n8, n8), device="cuda", dtype=torch.int8)
    ops = 2.0 * n8 ** 3
    t = ctx.core_time(lambda: eng.qgemm_w8a8(a8, 0.02, b8, bs, 40.0, q8, None), max(3, ctx.K // 2), 2)
    rows = sample_rows(n8, 2)
    _, q_ref = ctx.oracle.qgemm_w8a8(np.ascontiguousarray(host(a8[rows])), 0.02, host(b8), host(bs), 40.0)
    ok = bool(np.array_equal(host(q8[rows]), q_ref))
    tops = ops / (t["kernel_ms"] * 1e-3) / 1e12
    return [dict(t, name="int8_16384", workload="int8 GEMM 16384^3, s32 accumulate, requantised int8 out",
                 value=ctx.world * ops / (t["ms_per_step"] * 1e-3) / 1e12, unit="TOPS",
                 roofline=dict(tensor_roof(tops, 2 * bf16, "2 x measured bf16 burst (int8 issues at twice the bf16 rate)"), unit="TOPS",
                               frac_of_nominal_4500=tops / 4500.0),
                 parity_checked=ok, parity="sampled rows of the int8 output bit-exact vs the oracle")]


def w_skinny(ctx, shared):
    """skinny-M route: x[M,4096].W[4096,4096] + bias -> GELU (benchmark config 2); 8 rotating weight buffers
    (512 MiB > L2) so every step streams W from HBM."""
    torch, eng = ctx.torch, ctx.eng
    n = 4096
    Ws = [ctx.normal((n, n), 1 / 64) for _ in range(8)]
    bias = ctx.uniform((n,))
    out = []
    for M in (1, 8, 32):
        x = ctx.normal((M, n))
        y = torch.empty((M, n), device="cuda")
        state = {"i": 0}

        def sk():
            eng.gemm_bias_act(x, Ws[state["i"] % 8], bias, y, M, n, n, act="gelu")
            state["i"] += 1
        t = ctx.core_time(sk, 64, 8)
        nbytes = n * n * 4 + 2 * M * n * 4 + n * 4
        graph_ms = ctx.graph_time(sk)
        kern_ms = graph_ms if graph_ms else t["kernel_ms"]
        state["i"] = 0
        sk()
        want = ctx.oracle.bias_act(ctx.oracle.gemm_f64(host(x), host(Ws[0])).astype("float32"), host(bias), "gelu")
        e = nerr(host(y), want)
        out.append(dict(t, name=f"skinny_m{M}", workload=f"skinny-M dense+bias+GELU, x[{M}x4096].W[4096x4096]",
                        value=nbytes / (t["ms_per_step"] * 1e-3) / 1e9, unit="GB/s", kernel_ms=kern_ms,
                        kernel_ms_eager_events=t["kernel_ms"],
                        timing="kernel_ms: median over replays of a CUDA graph of 64 calls; value/ms_per_step: eager calls from Python",
                        roofline=dict(hbm_roof(ctx, nbytes, kern_ms), frac_of_nominal_8000=nbytes / (kern_ms * 1e-3) / 1e9 / 8000.0),
                        parity_checked=bool(e <= 1e-5), parity_nerr=e))
    return out


def w_c1(ctx, shared):
    """dense + bias + ReLU 1024^3 (benchmark config 1)"""
    import numpy as np
    torch, eng = ctx.torch, ctx.eng
    a1, b1, bias1 = ctx.uniform((1024, 1024)), ctx.uniform((1024, 1024)), ctx.uniform((1024,))
    c1 = torch.empty((1024, 1024), device="cuda")
    fn = lambda: eng.gemm_relu(a1, b1, bias1, c1)
    t = ctx.core_time(fn, 50, 5)
    g_ms = ctx.graph_time(fn, calls=32)
    rows = sample_rows(1024, 8)
    want = np.maximum(ctx.oracle.gemm_f64(np.ascontiguousarray(host(a1[rows])), host(b1)) + host(bias1).astype(np.float64), 0)
    e = nerr(host(c1[rows]), want)
    fl = 2.0 * 1024 ** 3
    peak = ctx.peaks["bf16_tflops"] / 6
    step = g_ms or t["ms_per_step"]
    out = [dict(t, name="c1_1024", workload="fp32 GEMM+bias+ReLU 1024^3 (3xTF32)", value=fl / (t["ms_per_step"] * 1e-3) / 1e12,
                unit="TFLOP/s", graph_ms_per_call=g_ms,
                roofline=tensor_roof(fl / (step * 1e-3) / 1e12, peak, "measured bf16 burst / 2 / 3; whole call (pre-pass included) from a replayed graph"),
                parity_checked=bool(e <= 1e-5), parity_nerr=e)]
    # the same layer with its weight prepared once, as a dense layer would hold it
    w = eng.weight_prepare(b1)
    try:
        fn2 = lambda: eng.gemm_prepared(a1, w, bias1, c1, 1024, act="relu")
        t2 = ctx.core_time(fn2, 50, 5)
        g2 = ctx.graph_time(fn2, calls=32)
        e2 = nerr(host(c1[rows]), want)
        out.append(dict(t2, name="c1_1024_prepared", workload="fp32 GEMM+bias+ReLU 1024^3, weight prepared once (axb_weight_prepare)",
                        value=fl / (t2["ms_per_step"] * 1e-3) / 1e12, unit="TFLOP/s", graph_ms_per_call=g2,
                        roofline=tensor_roof(fl / ((g2 or t2["ms_per_step"]) * 1e-3) / 1e12, peak, "measured bf16 burst / 2 / 3; whole call from a replayed graph"),
                        parity_checked=bool(e2 <= 1e-5), parity_nerr=e2))
    finally:
        eng.weight_release(w)
    return out


def w_c3(ctx, shared):
    """quantised GEMM 512x4096x4096 (benchmark config 3): W8A8 and the reference's W8A32"""
    import numpy as np
    torch, eng, bf16 = ctx.torch, ctx.eng, ctx.peaks["bf16_tflops"]
    a3, b3 = ctx.int8((512, 4096)), ctx.int8((4096, 4096))
    s3 = torch.rand((4096,), device="cuda", generator=ctx.gen) * 0.019 + 0.001
    q3 = torch.empty((512, 4096), device="cuda", dtype=torch.int8)
    fn = lambda: eng.qgemm_w8a8(a3, 0.02, b3, s3, 20.0, q3, None)
    t = ctx.core_time(fn, 50, 5)
    g_ms = ctx.graph_time(fn, calls=32)
    rows = sample_rows(512, 8)
    _, q_ref = ctx.oracle.qgemm_w8a8(np.ascontiguousarray(host(a3[rows])), 0.02, host(b3), host(s3), 20.0)
    ok = bool(np.array_equal(host(q3[rows]), q_ref))
    ops = 2.0 * 512 * 4096 * 4096
    tops = ops / (t["kernel_ms"] * 1e-3) / 1e12
    out = [dict(t, name="c3_w8a8", workload="int8 W8A8 GEMM 512x4096x4096 -> int8", value=ops / (t["ms_per_step"] * 1e-3) / 1e12,
                unit="TOPS", graph_ms_per_call=g_ms, roofline=dict(tensor_roof(tops, 2 * bf16, "2 x measured bf16 burst"), unit="TOPS"),
                parity_checked=ok, parity="sampled rows bit-exact vs the oracle")]
    af = ctx.uniform((512, 4096))
    of = torch.empty((512, 4096), device="cuda")
    t = ctx.core_time(lambda: eng.qgemm_w8a32(af, b3, s3, of), 30, 3)
    want = ctx.oracle.qgemm_w8a32_f64(np.ascontiguousarray(host(af[rows])), host(b3), host(s3))
    e = nerr(host(of[rows]), want)
    out.append(dict(t, name="c3_w8a32", workload="W8A32 GEMM 512x4096x4096 (fp32 activations, int8 weights)",
                    value=ops / (t["ms_per_step"] * 1e-3) / 1e12, unit="TFLOP/s", parity_checked=bool(e <= 1e-5), parity_nerr=e))
    return out


def w_qgemv(ctx, shared):
    """W8A32 at bs=1 (the case the reference's quantised path exists for: int8 weights streamed once) and bs=8/32;
    rotating weight buffers of 256 MiB in total (> L2) so every call streams from HBM."""
    import numpy as np
    torch, eng = ctx.torch, ctx.eng
    out = []
    for nq, bs in ((4096, 1), (16384, 1), (16384, 8), (16384, 32)):
        nbuf = 256 * 2 ** 20 // (nq * 4096)
        w8 = [ctx.int8((nq, 4096)) for _ in range(nbuf)]
        sq = torch.rand((nq,), device="cuda", generator=ctx.gen) * 0.019 + 0.001
        x1, o1 = ctx.uniform((bs, 4096)), torch.empty((bs, nq), device="cuda")
        st8 = {"i": 0}

        def qv():
            eng.qgemm_w8a32(x1, w8[st8["i"] % nbuf], sq, o1)
            st8["i"] += 1
        t = ctx.core_time(qv, 64, 8)
        kern_ms = ctx.graph_time(qv) or t["kernel_ms"]
        st8["i"] = 0
        qv()
        e = nerr(host(o1), ctx.oracle.qgemm_w8a32_f64(host(x1), host(w8[0]), host(sq)))
        nb = nq * 4096 + bs * 4096 * 4 + (1 + bs) * nq * 4
        out.append(dict(t, name=f"qgemv_n{nq}_bs{bs}", workload=f"W8A32 GEMV bs={bs}, int8 W[{nq}x4096] ({nbuf} rotating weight buffers)",
                        value=nb / (t["ms_per_step"] * 1e-3) / 1e9, unit="GB/s", kernel_ms=kern_ms, kernel_ms_eager_events=t["kernel_ms"],
                        timing="kernel_ms: median over replays of a CUDA graph of 64 calls; value/ms_per_step: eager calls from Python",
                        roofline=hbm_roof(ctx, nb, kern_ms), parity_checked=bool(e <= 1e-5), parity_nerr=e))
        del w8
    return out


def w_attention(ctx, shared):
    """causal attention B=8,H=16,S=1024,dk=64 (benchmark config 4), forward and backward, the QKV projection that feeds
    it, single-token decode against a KV cache, and the FMA kernel that serves head dims above 64."""
    import numpy as np
    torch, eng, bf16 = ctx.torch, ctx.eng, ctx.peaks["bf16_tflops"]
    out = []
    BH, S, dk = 128, 1024, 64
    Q, Kt, V = (ctx.normal((BH, S, dk)) for _ in range(3))
    O = torch.empty((BH, S, dk), device="cuda")
    L = torch.empty((BH, S), device="cuda")
    t = ctx.core_time(lambda: eng.sdpa_fwd(Q, Kt, V, O, L, 0.125, True), 20, 3)
    heads = [0, 77, BH - 1]
    O64, L64 = ctx.oracle.sdpa_fwd_f64(*(np.ascontiguousarray(host(x[heads])) for x in (Q, Kt, V)), 0.125, 1)
    e = float(np.abs(host(O[heads]) - O64).max())
    # tensor work actually issued: 128-row query tiles x 128-key blocks at or below the diagonal, two contractions
    tiles = S // 128
    done = 2 * 2.0 * BH * (tiles * (tiles + 1) // 2) * 128 * 128 * dk
    tf = done / (t["kernel_ms"] * 1e-3) / 1e12
    out.append(dict(t, name="sdpa_fwd_c4", workload="causal SDPA fwd BH=128 S=1024 dk=64 (fp32 in/out, 3xTF32 on the tensor cores)",
                    value=4.0 * BH * S * S * dk / (t["ms_per_step"] * 1e-3) / 1e12,
                    unit="TFLOP/s (4*BH*S^2*dk convention; causal does half)",
                    roofline=dict(tensor_roof(tf, bf16 / 6, "measured bf16 burst / 2 (tf32 rate) / 3 (products)"),
                                  note="achieved counts the useful FLOP of the key blocks the kernel visits (diagonal blocks whole)"),
                    parity_checked=bool(e < 1e-5), parity_maxabs=e))
    dOt = ctx.normal((BH, S, dk))
    gq, gk, gv = (torch.empty((BH, S, dk), device="cuda") for _ in range(3))
    t = ctx.core_time(lambda: eng.sdpa_bwd(Q, Kt, V, O, dOt, L, gq, gk, gv, 0.125, True), 10, 2)
    hq, hk, hv, ho, hd = (np.ascontiguousarray(host(x[heads])) for x in (Q, Kt, V, O, dOt))
    want = ctx.oracle.sdpa_bwd_f64(hq, hk, hv, ho, hd, 0.125, 1)
    e = max(nerr(host(g[heads]), w) for g, w in zip((gq, gk, gv), want))
    done_b = 5 * 2.0 * BH * (tiles * (tiles + 1) // 2) * 128 * 128 * dk
    out.append(dict(t, name="sdpa_bwd_c4", workload="causal SDPA bwd BH=128 S=1024 dk=64 (scores recomputed, no S x S buffer)",
                    value=2.5 * 4.0 * BH * S * S * dk / (t["ms_per_step"] * 1e-3) / 1e12,
                    unit="TFLOP/s (2.5 x the forward's 4*BH*S^2*dk convention; causal does half)",
                    roofline=tensor_roof(done_b / (t["kernel_ms"] * 1e-3) / 1e12, bf16 / 6, "measured bf16 burst / 2 / 3"),
                    parity_checked=bool(e <= 1e-5), parity_nerr=e))
    # fused QKV projection into the head-major layout: B=8, S=1024, D=1024 (H=16, dk=64, the config-4 heads)
    Bq, Sq, Hq = 8, 1024, 16
    Dq = Hq * dk
    Xq, Wq, bq = ctx.uniform((Bq * Sq, Dq)), ctx.normal((Dq, 3 * Dq), 1 / 32), ctx.uniform((3 * Dq,))
    hd3 = [torch.empty((Bq * Hq, Sq, dk), device="cuda") for _ in range(3)]
    t = ctx.core_time(lambda: eng.qkv_head_gemm(Xq, Wq, bq, Bq, Sq, Hq, dk, *hd3), 20, 3)
    rows = sample_rows(Bq * Sq, 2)
    want = ctx.oracle.gemm_f64(np.ascontiguousarray(host(Xq[rows])), host(Wq)) + host(bq).astype(np.float64)
    got = np.stack([np.concatenate([host(h)[(r // Sq) * Hq:(r // Sq + 1) * Hq, r % Sq, :].reshape(-1) for h in hd3]) for r in rows])
    e = nerr(got, want)
    fl = 2.0 * Bq * Sq * Dq * 3 * Dq
    out.append(dict(t, name="qkv_proj", workload="QKV projection + head-major split, X[8192x1024].Wqkv[1024x3072]+b -> Qh,Kh,Vh [128,1024,64] (one launch)",
                    value=fl / (t["ms_per_step"] * 1e-3) / 1e12, unit="TFLOP/s",
                    roofline=tensor_roof(fl / (t["kernel_ms"] * 1e-3) / 1e12, bf16 / 6, "measured bf16 burst / 2 / 3"),
                    parity_checked=bool(e <= 1e-5), parity_nerr=e))
    # the layer's backward GEMMs on the same shapes: the fused projection's weight gradients accumulated into the three
    # [D, D] gradients (x^T . dQKV with beta = 1: the epilogue leaves as TMA reduce-adds), and dattn = dout . Wo^T stored
    # head-major
    dQKV = ctx.normal((Bq * Sq, 3 * Dq), 0.5)
    g0 = [ctx.uniform((Dq, Dq)) for _ in range(3)]
    grads = [g.clone() for g in g0]
    calls = [0]

    def dw():
        calls[0] += 1
        eng.dwqkv_split_acc(Xq, dQKV, *grads)
    t = ctx.core_time(dw, 10, 2)
    rows = sample_rows(Dq, 2)
    prod = ctx.oracle.gemm_f64(np.ascontiguousarray(host(Xq).T[rows]), host(dQKV))            # rows of x^T . dQKV
    e = max(nerr(host(grads[i][rows]), host(g0[i][rows]).astype(np.float64) + calls[0] * prod[:, i * Dq:(i + 1) * Dq]) for i in range(3))
    out.append(dict(t, name="dwqkv_acc", workload="dWq,dWk,dWv [1024x1024] += X[8192x1024]^T . dQKV[8192x3072] column blocks (one launch, "
                    "accumulating epilogue)", value=fl / (t["ms_per_step"] * 1e-3) / 1e12, unit="TFLOP/s",
                    roofline=tensor_roof(fl / (t["kernel_ms"] * 1e-3) / 1e12, bf16 / 6, "measured bf16 burst / 2 / 3"),
                    parity_checked=bool(e <= 1e-5), parity_nerr=e, parity="sampled rows after every timed call against float64"))
    del Xq, Wq, hd3, gq, gk, gv, dOt, dQKV, grads, g0
    # single-token decode against a KV cache: config-4 heads, 4096 cached tokens = 268 MB of K and V
    kc, vc = (ctx.normal((BH, 4096, dk)) for _ in range(2))
    qn, on = ctx.normal((BH, dk)), torch.empty((BH, dk), device="cuda")
    kv = lambda: eng.kv_cache_attend(kc, vc, qn, on, 4096, 0.125)
    t = ctx.core_time(kv, 32, 4)
    kern_ms = ctx.graph_time(kv, calls=16) or t["kernel_ms"]
    want = ctx.oracle.kv_cache_attend_f64(np.ascontiguousarray(host(kc[heads])), np.ascontiguousarray(host(vc[heads])),
                                          np.ascontiguousarray(host(qn[heads])), 4096, 0.125)
    e = float(np.abs(host(on[heads]) - want).max())
    nb = 2.0 * BH * 4096 * dk * 4
    out.append(dict(t, name="kv_attend", workload="KV-cache attention, 1 new token, BH=128, 4096 cached tokens, dk=64 (K+V = 268 MB > L2)",
                    value=nb / (t["ms_per_step"] * 1e-3) / 1e9, unit="GB/s", kernel_ms=kern_ms, kernel_ms_eager_events=t["kernel_ms"],
                    roofline=hbm_roof(ctx, nb, kern_ms), parity_checked=bool(e < 1e-5), parity_maxabs=e))
    del kc, vc
    Q2, K2, V2 = (ctx.normal((64, 1024, 128)) for _ in range(3))
    O2 = torch.empty((64, 1024, 128), device="cuda")
    t = ctx.core_time(lambda: eng.sdpa_fwd(Q2, K2, V2, O2, None, 0.0884, True), 10, 3)
    O64, _ = ctx.oracle.sdpa_fwd_f64(*(np.ascontiguousarray(host(x[:2])) for x in (Q2, K2, V2)), 0.0884, 1)
    e = float(np.abs(host(O2[:2]) - O64).max())
    out.append(dict(t, name="sdpa_fwd_dk128", workload="causal SDPA fwd BH=64 S=1024 dk=128 (fp32 FMA kernel)",
                    value=4.0 * 64 * S * S * 128 / (t["ms_per_step"] * 1e-3) / 1e12,
                    unit="TFLOP/s (4*BH*S^2*dk convention; causal does half)", parity_checked=bool(e < 1e-5), parity_maxabs=e))
    return out


def w_conv(ctx, shared):
    """convolution as GEMM: a ResNet 3x3 layer on one sample (C_in = C_out = 256, 56x56, pad 1): weight [256 x 2304]"""
    import numpy as np
    torch, eng = ctx.torch, ctx.eng
    wc, xc = ctx.normal((256, 2304), 1 / 48), ctx.uniform((256, 56, 56))
    oc = torch.empty((256, 56 * 56), device="cuda")
    t = ctx.core_time(lambda: eng.conv_gemm(wc, xc, 3, 3, 1, 1, 1, 1, oc), 20, 3)
    want = ctx.oracle.conv_gemm(host(wc), host(xc), 3, 3, 1, 1, 1, 1)
    e = nerr(host(oc), want)
    res = [dict(t, name="conv3x3", workload="conv 3x3 pad 1 as an implicit GEMM, one sample [256,56,56] -> [256,56,56] (shifted TMA windows of the channel-innermost image; no patch matrix)",
                value=2.0 * 256 * 2304 * 3136 / (t["ms_per_step"] * 1e-3) / 1e12, unit="TFLOP/s",
                parity_checked=bool(e <= 2e-5), parity_nerr=e, parity="whole output vs the fp32 oracle (tolerance of two fp32 summation orders)")]
    # the same layer over a batch of 16 samples: one implicit GEMM whose columns are the pixels of all samples
    nb = 16
    xb = ctx.uniform((nb, 256, 56, 56))
    ob = torch.empty((nb, 256, 56 * 56), device="cuda")
    tb = ctx.core_time(lambda: eng.conv_gemm_batched(wc, xb, 3, 3, 1, 1, 1, 1, ob), 20, 3)
    probe = [0, nb - 1]
    eb = max(nerr(host(ob[i]), ctx.oracle.conv_gemm(host(wc), host(xb[i]), 3, 3, 1, 1, 1, 1)) for i in probe)
    peak = ctx.peaks["bf16_tflops"] / 6.0
    val = 2.0 * nb * 256 * 2304 * 3136 / (tb["ms_per_step"] * 1e-3) / 1e12
    kern = 2.0 * nb * 256 * 2304 * 3136 / (tb["kernel_ms"] * 1e-3) / 1e12 if tb.get("kernel_ms") else None
    res.append(dict(tb, name="conv3x3_batch16", workload="the same layer on 16 samples through axb_conv_gemm_batched (one implicit GEMM, [256 x 2304] . [2304 x 50176])",
                    value=val, unit="TFLOP/s",
                    roofline={"bound": "tensor", "achieved": kern, "peak": peak, "frac": (kern / peak) if kern else None, "unit": "TFLOP/s",
                              "peak_source": "measured bf16 burst / 2 / 3"},
                    parity_checked=bool(eb <= 2e-5), parity_nerr=eb, parity="first and last sample vs the fp32 oracle"))
    return res


def w_mlp(ctx, shared):
    """3-layer MLP 8192 -> 16384 -> 16384 -> 8192 at batch 16384, bias + GELU fused (benchmark config 5c): rows of the
    batch sharded over the ranks (no collective), and, with more than one rank, output columns sharded with one gather
    per layer.  Fixed total batch: strong scaling for these lines.  Runs last: seconds at the power cap."""
    import numpy as np
    from axiom_b200.multi_gpu import ColumnShardedMLP, RowShardedMLP, gathered_to_full, shard_bounds
    torch, dist, eng, world, rank = ctx.torch, ctx.dist, ctx.eng, ctx.world, ctx.rank
    dims = [8192, 16384, 16384, 8192]
    batch = 16384
    flop = 2.0 * batch * sum(dims[i] * dims[i + 1] for i in range(3))
    gen = torch.Generator(device="cuda").manual_seed(99)          # same weights on every rank
    Ws = [torch.randn((dims[i], dims[i + 1]), device="cuda", generator=gen) / (dims[i] ** 0.5) for i in range(3)]
    bs = [torch.rand((dims[i + 1],), device="cuda", generator=gen) * 2 - 1 for i in range(3)]
    x = torch.rand((batch, dims[0]), device="cuda", generator=gen) * 2 - 1
    new_empty = lambda shape: torch.empty(shape, device="cuda", dtype=torch.float32)
    steps = max(2, min(ctx.K, 3))
    r0, r1 = shard_bounds(batch, world, rank)
    # the oracle's answer for two rows this rank owns and two it may not: float64 through all three layers
    probe = sorted({r0, r1 - 1, (rank * 7919) % batch})
    h = host(x[probe]).astype(np.float64)
    for Wl, bl in zip(Ws, bs):
        # fp32 activations between the layers, as on the device; sums in float64
        z = ctx.oracle.gemm_f64(np.ascontiguousarray(h.astype(np.float32)), host(Wl)) + host(bl).astype(np.float64)
        h = 0.5 * z * (1.0 + np.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
    want = h

    def all_ranks(ok):
        if world == 1:
            return bool(ok)
        t = torch.tensor([1.0 if ok else 0.0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item() > 0.5)

    res = []
    xr = x[r0:r1].contiguous()
    mine = [i for i, r in enumerate(probe) if r0 <= r < r1]
    for prepared in (True, False):
        rows = RowShardedMLP(eng, Ws, bs, act="gelu", prepare=prepared)
        ms, per = ctx.timed(lambda: rows.forward(xr, new_empty), steps, 1)
        ms /= steps
        y = rows.forward(xr, new_empty)
        e = nerr(host(y[[probe[i] - r0 for i in mine]]), want[mine])
        how = ("weights prepared once (axb_weight_prepare: only activations are split per step)" if prepared
               else "plain axb_gemm_bias_act (weights split every step)")
        res.append({"name": "mlp_rows" if prepared else "mlp_rows_unprepared",
                    "workload": f"3-layer MLP 8192-16384-16384-8192, batch 16384, rows sharded x{world} (no collective), {how}",
                    "value": flop / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "ms_median": statistics.median(per),
                    "ms_min": min(per), "scaling": "strong", "parity_checked": all_ranks(e <= 1e-5), "parity_nerr": e,
                    "parity": "sampled rows on every rank vs a float64 forward"})
        rows.close()
        del y, rows
        torch.cuda.empty_cache()
    if world > 1:
        slabs, bias_slabs = [], []
        for Wl, b in zip(Ws, bs):
            c0, c1 = shard_bounds(Wl.shape[1], world, rank)
            slabs.append(Wl[:, c0:c1].contiguous())
            bias_slabs.append(b[c0:c1].contiguous())
        del Ws
        torch.cuda.empty_cache()
        ag = lambda dst, src: dist.all_gather_into_tensor(dst.view(-1, dst.shape[-1]), src)
        # the column variants keep their slabs' operand planes too, like the prepared row variant they are compared with
        cols = ColumnShardedMLP(eng, slabs, bias_slabs, world, rank, ag, act="gelu", prepare=True)
        ms, per = ctx.timed(lambda: cols.forward(x, new_empty), steps, 1)
        ms /= steps
        y_ref = cols.forward(x, new_empty)
        e_cols = nerr(host(gathered_to_full(y_ref[:, probe, :])), want)
        fused = None
        try:
            from axiom_b200.multi_gpu import PeerScatterColumnMLP
            fused = PeerScatterColumnMLP(eng, slabs, bias_slabs, world, rank, batch, dist, act="gelu", prepare=True)
            ms_f, per_f = ctx.timed(lambda: fused.forward(x, new_empty), steps, 1)
            ms_f /= steps
            out_ptr, n_last = fused.forward(x, new_empty)
            y_fused = torch.empty_like(y_ref)
            eng._check(eng.lib.axb_memcpy_d2d(ctypes.c_void_p(y_fused.data_ptr()), ctypes.c_void_p(out_ptr), y_ref.numel() * 4))
            torch.cuda.synchronize()
            e_f = nerr(host(gathered_to_full(y_fused[:, probe, :])), want)
            res.append({"name": "mlp_cols_peer", "workload": f"3-layer MLP, batch 16384, output columns sharded x{world} (slabs prepared once), gather fused "
                        "into the GEMM epilogue as peer stores over NVLink", "value": flop / (ms_f * 1e-3) / 1e12, "unit": "TFLOP/s",
                        "ms_per_step": ms_f, "ms_median": statistics.median(per_f), "ms_min": min(per_f), "scaling": "strong",
                        "bit_identical_to_nccl_path": all_ranks(torch.equal(y_fused, y_ref)),
                        "parity_checked": all_ranks(e_f <= 1e-5), "parity_nerr": e_f})
        except Exception as exc:
            res.append({"name": "mlp_cols_peer", "workload": "3-layer MLP, peer-store gather", "error": repr(exc)})
        finally:
            if fused is not None:
                fused.close()
        res.append({"name": "mlp_cols_nccl", "workload": f"3-layer MLP, batch 16384, output columns sharded x{world} (slabs prepared once), NCCL all-gather per layer",
                    "value": flop / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "ms_median": statistics.median(per),
                    "ms_min": min(per), "scaling": "strong", "parity_checked": all_ranks(e_cols <= 1e-5), "parity_nerr": e_cols,
                    "allgather_bytes_per_rank_per_layer": [batch * d // world * 4 for d in dims[1:]]})
        cols.close()
    return res


SUITE = [("gemm_modes", w_gemm_modes), ("int8_16384", w_int8_16384), ("skinny", w_skinny), ("c1", w_c1), ("c3", w_c3),
         ("qgemv", w_qgemv), ("attention", w_attention), ("conv", w_conv), ("mlp", w_mlp)]


def run_suite(ctx, names, shared):
    out = []
    for name, fn in SUITE:
        if names is not None and name not in names:
            continue
        try:
            out.extend(fn(ctx, shared))
        except Exception as exc:
            out.append({"name": name, "workload": (fn.__doc__ or name).strip().split("\n")[0], "error": repr(exc)})
        ctx.torch.cuda.empty_cache()
    return out


def compact(entry):
    """The few numbers of a suite record that belong in the headline line."""
    keep = {k: entry.get(k) for k in ("name", "value", "unit", "ms_per_step", "ms_median", "ms_min", "kernel_ms", "kernel_ms_min",
                                      "graph_ms_per_call", "parity_checked", "scaling", "error") if entry.get(k) is not None}
    if "unit" in keep:
        keep["unit"] = keep["unit"].split(" (")[0]
    r = entry.get("roofline")
    if r:
        keep.update(bound=r["bound"], achieved=r["achieved"], peak=r["peak"], frac=r["frac"])
    return keep


def run_ours(args):
    ctx = Ctx(args)
    only = [s for s in args.only.split(",") if s] if args.only else None
    if only is not None:
        unknown = [s for s in only if s not in dict(SUITE)]
        if unknown:
            raise SystemExit(f"--only: unknown workload(s) {unknown}; known: {[n for n, _ in SUITE]}")
        extra = run_suite(ctx, only, None)
        err = ctx.eng.device_error()
        if ctx.rank == 0:
            print(json.dumps({"only": only, "device_error": err, "suite": extra}))
        if ctx.world > 1:
            ctx.dist.destroy_process_group()
        return
    line, shared = headline(ctx, args)
    extra = [] if args.headline_only else run_suite(ctx, None, shared)
    del shared
    if ctx.rank == 0 and ctx.world == 1 and not args.no_cpu:
        host_threads_for_reference()
        ref, o = load_reference(autotune=True)
        if ref is not None:
            cb = cpu_headline(ref, o, 3, 1)
            line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
            if not args.headline_only:
                line["cpu_baseline"]["per_config"] = cpu_per_config(ref, o)
    err = ctx.eng.device_error()
    if ctx.rank == 0:
        line["roofline"]["suite"] = [compact(e) for e in extra]
        line["parity_checked"] = bool(line["parity_checked"] and all(e.get("parity_checked", False) for e in extra if "error" not in e))
        line["device_error"] = err
        sys.stderr.write(json.dumps({"suite": extra}) + "\n")
        print(json.dumps(line))
    if ctx.world > 1:
        ctx.dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--headline-only", action="store_true", help="skip the suite workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--only", default=None, help="comma-separated suite workloads to run alone: " + ",".join(n for n, _ in SUITE))
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
