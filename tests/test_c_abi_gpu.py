"""The C ABI used from plain C: tests/c_abi/abi_smoke.c is compiled with gcc against include/gpu_kernels.h, linked with
libb200_qlinear.so and the CUDA runtime, and run as a process of its own (no Python, no torch on its path)."""
from __future__ import annotations

import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def test_plain_c_host_program(pkg, dev, tmp_path):
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    gcc = shutil.which("gcc")
    if gcc is None or not os.path.exists(os.path.join(cuda, "include", "cuda_runtime_api.h")):
        pytest.skip("no gcc or CUDA headers")
    libdir = os.path.join(ROOT, "comfyui-backend-but-rust_b200")
    exe = str(tmp_path / "abi_smoke")
    subprocess.check_call([gcc, "-O1", "-std=c11", os.path.join(ROOT, "tests", "c_abi", "abi_smoke.c"), "-I", os.path.join(ROOT, "include"),
                           "-I", os.path.join(cuda, "include"), "-L", libdir, "-lb200_qlinear", "-L", os.path.join(cuda, "lib64"),
                           "-lcudart", "-lm", "-Wl,-rpath," + libdir, "-Wl,-rpath," + os.path.join(cuda, "lib64"), "-o", exe])
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "abi smoke ok" in out.stdout
