"""The GPU arm of bench.py: one JSON line with the keys the measurement contract names, consistent with each other."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_headline_line(engine):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--headline-only", "--no-cpu", "--steps", "3", "--warmup", "3"],
                         capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    sys.path.insert(0, ROOT)
    import bench
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "roofline", "cpu_baseline", "e2e", "gpu_launches", "clocks"):
        assert key in line, key
    assert line["metric"] == "gemm_fp32_tflops" and line["unit"] == "TFLOP/s" and line["dtype"] == "f32" and line["data"] == "synthetic"
    assert line["config"] == bench.headline_config(1) and line["n_gpus"] == 1 and line["steps"] == 3 and line["warmup"] == 3
    assert abs(line["value"] - bench.FLOP_HEADLINE / (line["ms_per_step"] * 1e-3) / 1e12) < 1e-6 * line["value"]
    r = line["roofline"]
    assert r["bound"] == "tensor" and r["unit"] == "TFLOP/s" and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    assert r["kernel_ms"] < line["ms_per_step"]                 # the kernel is a part of the step
    assert r["traffic"] > r["algorithmic_bytes"] > 0
    e = line["e2e"]
    assert e["h2d_bytes_per_step"] == 2 * 8192 * 8192 * 4 and e["d2h_bytes_per_step"] == 8192 * 8192 * 4
    assert 0 < e["value"] < line["value"] and e["parity_checked"] is True      # copies inside the timed region cost time
    assert line["gpu_launches"] >= 2 * line["steps"]            # pre-pass + tcgen05 kernel per step
    assert line["parity_checked"] is True and line["device_error"] == 0
    c = line["clocks"]
    assert c["sm_max_mhz"] >= c["sm_mhz"] > 0 and isinstance(c["reasons"], list)
