"""The benchmark's reference arm runs on host cores only: its JSON line is checked here without a GPU."""
from __future__ import annotations

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                          "--cpu-rows", "64"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["metric"] == "w8a8_linear_tops" and d["unit"] == "TOPS" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and "sample" in d["cpu_baseline"]
    assert d["e2e"] == {"value": d["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"]


def test_ours_without_a_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        return
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "0"], capture_output=True,
                         text=True, timeout=600, cwd=ROOT)
    assert out.returncode != 0 and "no CPU fallback" in (out.stderr + out.stdout)


def test_reference_arm_does_not_map_the_cuda_library():
    """The CPU arm takes shapes and seeded inputs from workloads.py by file path; the product's shared library stays out
    of its process."""
    code = ("import sys; sys.path.insert(0, %r); import bench; wl = bench.load_workloads(); assert wl.config(1)[0].N == 12288; "
            "assert 'libb200_qlinear' not in open('/proc/self/maps').read(); assert 'cbr_b200' not in sys.modules" % ROOT)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]


def test_both_arms_print_the_same_config():
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    assert b.CONFIG["workload"] == b.WORKLOAD and b.CONFIG["tokens_per_gpu"] == 4352
    # the roofline's traffic comes from the committed ncu summary of the kernel form the step runs
    assert b.profiled_dram_bytes(False) == 97.6e6 + 74.4e6
    assert b.profiled_dram_bytes(True) == 97.7e6 + 75.6e6
