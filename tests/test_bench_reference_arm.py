"""The reference arm of bench.py runs on the host cores alone: its JSON line must carry the contract's keys and the
same metric, unit and workload description as the GPU arm (the two lines are compared key by key downstream)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_line(reference):
    """`reference` (the compiled axiom library) is the arm's only dependency; skipped where it cannot be built."""
    env = dict(os.environ, OMP_NUM_THREADS="1")          # inherited from a launcher: the arm must override it
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, env=env, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    sys.path.insert(0, ROOT)
    import bench
    assert line["impl"] == "reference"
    assert line["metric"] == "gemm_fp32_tflops" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["config"] == bench.headline_config(1)            # the same workload as the GPU arm, word for word
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["warmup"] == 1
    assert line["value"] > 0 and abs(line["value"] - bench.FLOP_HEADLINE / (line["ms_per_step"] * 1e-3) / 1e12) < 1e-6 * line["value"]
    cb = line["cpu_baseline"]
    assert cb["kind"] == "reference" and cb["value"] == line["value"]
    assert cb["cores"] == len(os.sched_getaffinity(0)) and cb["cores"] >= 1        # not the inherited single thread
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["vs_baseline"] is None
