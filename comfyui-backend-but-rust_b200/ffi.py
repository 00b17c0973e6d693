"""ctypes declarations of the C ABI in ``include/gpu_kernels.h`` -- the Python twin of the reference's
``src/ffi.rs`` for the quantized-linear path: same names, same argument order, raw device pointers and a raw
``cudaStream_t``; ``ok()`` maps return codes to errors the way ``src/ffi.rs:336-344`` does.

The library is loaded from this directory and nowhere else. If it is missing, importing fails: there is no
fallback path.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200_qlinear.so")

DT_F32, DT_F16, DT_BF16 = 0, 1, 2
(PRO_PLAIN, PRO_RMS, PRO_GATE, PRO_SWIGLU, PRO_LAYERNORM, PRO_SILU, PRO_GELU, PRO_ADALN, PRO_SITU, PRO_LN_MOD,
 PRO_LN_AFFINE, PRO_GELU_TANH, PRO_LN_AFFINE_SILU, PRO_SITU_FAST) = range(14)
ACT_NONE, ACT_GELU_TANH, ACT_SILU, ACT_GELU_ERF = range(4)

P = C.c_void_p
i32, i64, u64, f32 = C.c_int, C.c_int64, C.c_uint64, C.c_float

# name -> argument types (all return int unless noted), in the order of include/gpu_kernels.h
SIGNATURES = {
    "gpu_quant_rows": [i32, i32, P, i64, P, i64, i64, P, f32, P, P, P, P, i32, i32, i32, P],
    "gpu_quant_rows_b": [i32, i32, P, i64, P, P, f32, P, P, P, P, i32, i32, i32, P],
    "gpu_rotate_rows_f32": [i32, P, i64, i64, P, f32, P, i32, i32, P],
    "gpu_sd_quant_rows": [P, i64, P, P, i32, i32, i32, P],
    "gpu_sd_ln_quant_rows": [P, i64, P, P, f32, P, P, i32, i32, i32, P],
    "gpu_sd_geglu_quant_rows": [P, P, P, i32, i32, i32, P],
    "gpu_sd_unpad_quant_rows": [P, P, P, i32, i32, i32, i32, i32, P],
    "gpu_sd_group_norm_quant_rows": [P, P, P, P, i32, i64, i32, i32, f32, P, P, i32, P],
    "gpu_int8_gemm": [P, P, P, P, P, P, i64, i64, i64, i32, P],
    "gpu_int8_gemm_residual": [P, P, P, P, P, P, P, P, i64, i64, i64, i32, P],
    "gpu_int8_gemm_act": [P, P, P, P, P, P, i64, i64, i64, i32, i32, P],
    "gpu_int8_gemm_act_rot": [P, P, P, P, P, P, P, i64, i64, i64, i32, P],
    "gpu_quant_rows_rotated": [P, P, P, P, i32, i32, P],
    "gpu_int8_gemm_noalloc": [P, P, P, P, P, P, i64, i64, i64, i32, P],
    "gpu_int8_gemm_acc_i32": [P, P, P, i64, i64, i64, P],
    "gpu_w6a8_gemm": [P, P, P, P, P, P, P, i64, i64, i64, i32, i32, P],
    "gpu_w6a8_gemm_residual": [P, P, P, P, P, P, P, P, P, i64, i64, i64, i32, i32, P],
    "gpu_w6a8_gemm_act": [P, P, P, P, P, P, P, i64, i64, i64, i32, i32, i32, P],
    "gpu_w6a8_gemm_acc_i32": [P, P, P, P, i64, i64, i64, i32, P],
    "gpu_quant_rows_amax": [i32, i32, P, i64, P, i64, i64, P, i32, i32, i32, P],
    "gpu_quant_rows_scaled": [i32, i32, P, i64, P, i64, i64, P, P, P, i32, i32, i32, P],
    "gpu_int8_epilogue": [P, P, P, P, P, P, P, i64, i64, i32, i32, P],
    "gpu_wo8_linear": [i32, P, i64, i64, P, f32, P, P, P, f32, P, P, i32, i32, i32, P],
    "gpu_bias_residual_add": [P, P, P, P, i64, i64, i64, i64, i32, P],
    "gpu_int8_gemm_set_cluster_limit": [i32],
    "gpu_w6_decode": [P, P, P, i64, i32, i32, P],
    "gpu_w6_requant": [P, P, P, P, i64, i32, u64, P],
    "gpu_convrot_requant": [i32, P, P, P, i64, i32, u64, P],
    "gpu_convrot_dequant": [i32, P, P, P, i64, i32, P],
    "gpu_dequant_i8": [P, P, P, i64, i64, P],
    "gpu_embed_dequant": [P, P, P, i32, i32, i32, P],
    "gpu_wddm_budget": [C.POINTER(u64), C.POINTER(u64)],
    "gpu_kernels_status": [C.POINTER(i32)],
}
_VOID = set()


def load(path: str = LIB_PATH) -> C.CDLL:
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: build it with `python comfyui-backend-but-rust_b200/build.py` "
                          "(there is no CPU or library fallback for this path)")
    lib = C.CDLL(path)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = the library does not export a declared symbol
        fn.argtypes = args
        fn.restype = None if name in _VOID else i32
    return lib


class GpuKernelError(RuntimeError):
    pass


def ok(code: int, what: str) -> None:
    """Turn a launcher return code into an error naming the call (src/ffi.rs:336-344)."""
    if code == 0:
        return
    if code > 0:
        raise GpuKernelError(f"{what} failed: CUDA error {code}")
    raise GpuKernelError(f"{what} failed with code {code}")
