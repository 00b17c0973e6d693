"""Builds libb200_qlinear.so (the C-ABI library) and libb200_qlinear.a (the same objects as a static archive, for hosts
that link statically) from csrc/*.cu with nvcc, for sm_100a only. The name differs on purpose from the reference's own
static library `gpu_kernels`, which keeps supplying every symbol this library does not replace.

The GEMM uses tcgen05.mma kind::i8, which exists on sm_100a and not on sm_103a or sm_120: no other -gencode
may be added. No fast-math: the rounding points of the quantizer and of the epilogue are part of the contract.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libb200_qlinear.so")
ARCHIVE = os.path.join(HERE, "libb200_qlinear.a")
UNITS = ["quant_rows", "gemm_i8", "gemm_skinny", "weight_pack"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
         "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I" + CSRC, "-I" + os.path.join(os.path.dirname(HERE), "include")]


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".inl"))]
    headers.append(os.path.abspath(__file__))

    def compile_unit(u: str) -> str:
        src, obj = os.path.join(CSRC, u + ".cu"), os.path.join(OBJ, u + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [NVCC, "-c", src, "-o", obj] + FLAGS + (["-Xptxas", "-v"] if verbose else [])
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {u}.cu")
        return obj

    with ThreadPoolExecutor(max_workers=len(UNITS)) as ex:
        objs = list(ex.map(compile_unit, UNITS))
    if force or _stale(LIB, objs):
        subprocess.check_call([NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"])
    if force or _stale(ARCHIVE, objs):
        if os.path.exists(ARCHIVE):
            os.remove(ARCHIVE)
        subprocess.check_call(["ar", "rcs", ARCHIVE] + objs)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
