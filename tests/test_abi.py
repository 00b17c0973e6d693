"""CPU tests of the drop-in boundary: the library loads, exports every symbol the header declares with no extras
missing, and rejects bad arguments with the reference's codes before touching a device."""
from __future__ import annotations

import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "gpu_kernels.h")


def _declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(?:int|void)\s+(gpu_\w+)\s*\(", text)))


def test_header_declares_the_reference_symbols_of_the_path():
    names = _declared()
    for must in ("gpu_quant_rows", "gpu_rotate_rows_f32", "gpu_sd_quant_rows", "gpu_int8_gemm", "gpu_int8_gemm_residual",
                 "gpu_w6_decode", "gpu_convrot_requant", "gpu_convrot_dequant", "gpu_dequant_i8", "gpu_embed_dequant",
                 "gpu_wddm_budget"):
        assert must in names, must


def test_library_exports_every_declared_symbol(pkg):
    lib = C.CDLL(pkg.ffi.LIB_PATH)
    for name in _declared():
        assert hasattr(lib, name), f"{name} declared in include/gpu_kernels.h but not exported"
    assert set(pkg.ffi.SIGNATURES) == set(_declared()), "ffi.py and the header list the same entry points"


def test_dynamic_symbols_are_exactly_the_header(pkg):
    """Nothing but the declared entry points leaves the shared library, and the static archive (the form a host that
    links statically takes, under a name that cannot collide with the reference's own `gpu_kernels`) defines the same
    entry points and otherwise only names inside the library's own namespace."""
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", pkg.ffi.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = sorted(ln.split()[2] for ln in out.splitlines() if len(ln.split()) == 3 and ln.split()[1] in "TDB")
    assert exported == _declared(), set(exported) ^ set(_declared())
    archive = os.path.join(os.path.dirname(pkg.ffi.LIB_PATH), "libb200_qlinear.a")
    assert os.path.exists(archive)
    out = subprocess.run(["nm", "-g", "--defined-only", archive], capture_output=True, text=True, check=True).stdout
    glob = {ln.split()[2] for ln in out.splitlines() if len(ln.split()) == 3 and ln.split()[1] == "T"}
    assert set(_declared()) <= glob
    # what else the objects define is either in the library's namespace or carries nvcc's per-file unique prefix
    stray = {n for n in glob - set(_declared()) if not (n.startswith("_ZN5b200q") or "_GLOBAL__N_" in n or n.startswith("__cudaRegister")
                                                        or n.startswith("__sti") or "__nv_" in n)}
    assert not stray, stray


def test_argument_errors_need_no_device(pkg):
    lib = pkg.lib
    # K % 256 != 0 -> -1 (reference: csrc/kernels.cu:275)
    assert lib.gpu_quant_rows(2, 0, 0, 0, 0, 0, 0, 0, 0.0, 0, 0, 0, 0, 4, 300, 0, 0) == -1
    assert lib.gpu_rotate_rows_f32(0, 0, 0, 0, 0, 0.0, 0, 4, 100, 0) == -1
    # rotate not in {0, 64, 256}, or not dividing K -> -1 (csrc/sd.cu:600)
    assert lib.gpu_sd_quant_rows(0, 0, 0, 0, 4, 640, 128, 0) == -1
    assert lib.gpu_sd_quant_rows(0, 0, 0, 0, 4, 640, 256, 0) == -1
    # K % 32 or G % 16 -> -1 (csrc/h3.cu:41)
    assert lib.gpu_w6_decode(0, 0, 0, 4, 48, 32, 0) == -1
    assert lib.gpu_w6_decode(0, 0, 0, 4, 64, 8, 0) == -1
    assert lib.gpu_convrot_requant(0, 0, 0, 0, 4, 100, 0, 0) == -1
    assert lib.gpu_dequant_i8(0, 0, 0, 4, 6, 0) == -1
    assert lib.gpu_embed_dequant(0, 0, 0, 4, 256, 0, 0) == -1
    # GEMM: empty problems succeed without work (csrc/vendor/cutlass_gemm_int8.cu:377); the residual form declines
    # K == 0 and missing rscale / resid (:353-357)
    assert lib.gpu_int8_gemm(0, 0, 0, 0, 0, 0, 0, 16, 16, 2, 0) == 0
    assert lib.gpu_int8_gemm(0, 0, 0, 0, 0, 0, 16, 16, 0, 2, 0) == 0
    assert lib.gpu_int8_gemm_residual(0, 0, 0, 0, 0, 0, 0, 0, 16, 16, 0, 2, 0) == -201
    assert lib.gpu_int8_gemm_residual(0, 0, 0, 0, 0, 0, 0, 0, 16, 16, 16, 2, 0) == -201
    assert lib.gpu_int8_gemm(0, 0, 0, 0, 0, 0, 16, 16, 16, 7, 0) == -200
    assert lib.gpu_int8_gemm_act(0, 0, 0, 0, 0, 0, 16, 16, 16, 2, 9, 0) == -204


def test_wddm_budget_stub(pkg):
    b, u = C.c_uint64(5), C.c_uint64(5)
    assert pkg.lib.gpu_wddm_budget(C.byref(b), C.byref(u)) != 0
    assert b.value == 0 and u.value == 0


def test_ok_maps_codes_like_the_reference(pkg):
    pkg.ok(0, "x")
    with pytest.raises(pkg.GpuKernelError, match="failed with code -1"):
        pkg.ok(-1, "gpu_quant_rows")
    with pytest.raises(pkg.GpuKernelError, match="CUDA error 700"):
        pkg.ok(700, "gpu_int8_gemm")


def test_workload_configs(pkg):
    import importlib
    wl = importlib.import_module("cbr_b200.workloads")
    up, down = wl.config(1)
    assert (up.M, up.K, up.N) == (4352, 3072, 12288) and (down.K, down.N) == (12288, 3072)
    assert abs(up.ops - 328.6e9) < 0.1e9
    assert len(wl.config(3)) == 12 and all(s.K % s.rotate == 0 for s in wl.config(3))
    block = wl.config(4)
    assert abs(sum(s.ops for s in block) - 3827e9) < 2e9
