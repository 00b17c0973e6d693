"""B200 (sm_100a) quantized-linear kernels behind the C ABI of BetaDoggo/comfyui-backend-but-rust.

``ffi``     raw ctypes bindings of libb200_qlinear.so (the drop-in boundary, mirrors the reference's src/ffi.rs)
``linear``  host-side helpers over torch device tensors: the call sequences the reference's model code issues
            (quantize rows -> int8 GEMM with fused epilogue), weight packing at load, tensor-parallel linears
"""
from . import ffi  # noqa: F401
from .ffi import load, ok, GpuKernelError  # noqa: F401

lib = load()

from . import linear  # noqa: E402,F401
