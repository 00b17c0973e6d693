"""ctypes binding of ``oracle/_ref/libref.so``: the reference's own CUDA kernels for the path, compiled for sm_100a
from the reference tree by ``oracle/build_ref.sh``.

TEST INFRASTRUCTURE ONLY (GPU tests and profiling of the incumbent). Takes torch CUDA tensors; call signatures are
the reference's (csrc/kernels.cu:271, csrc/sd.cu:599, csrc/h3.cu:40, csrc/kernels.cu:1393-1420,
csrc/vendor/cutlass_gemm_int8.cu:343-388).
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libref.so")
_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(LIB_PATH)
        _lib.launch_cutlass_int8_dequant.restype = C.c_bool
        _lib.launch_cutlass_int8_dequant_residual.restype = C.c_bool
    return _lib


def _p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _st():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def quant_rows(x, prologue=0, rotate=0, *, K=None, g=None, up_offset=0, q=None, scales=None, norm_w=None, norm_b=None,
               eps=0.0, mod_scale=None, mod_shift=None):
    """The reference's gpu_quant_rows (gpu_quant_rows_b when norm_b is given), csrc/kernels.cu:271-314."""
    M = x.shape[0]
    K = K if K is not None else x.shape[1]
    q = q if q is not None else torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = scales if scales is not None else torch.empty((M,), dtype=torch.float32, device=x.device)
    if norm_b is not None:
        rc = lib().gpu_quant_rows_b(C.c_int(_DT[x.dtype]), C.c_int(prologue), _p(x), C.c_int64(x.stride(0)), _p(norm_w),
                                    _p(norm_b), C.c_float(eps), _p(mod_scale), _p(mod_shift), _p(q), _p(s), C.c_int(M),
                                    C.c_int(K), C.c_int(rotate), _st())
    else:
        rc = lib().gpu_quant_rows(C.c_int(_DT[x.dtype]), C.c_int(prologue), _p(x), C.c_int64(x.stride(0)), _p(g),
                                  C.c_int64(g.stride(0) if g is not None else 0), C.c_int64(up_offset), _p(norm_w),
                                  C.c_float(eps), _p(mod_scale), _p(mod_shift), _p(q), _p(s), C.c_int(M), C.c_int(K),
                                  C.c_int(rotate), _st())
    assert rc == 0, rc
    return q, s


def rotate_rows_f32(x, prologue=0, *, K=None, up_offset=0, norm_w=None, eps=0.0):
    """The reference's gpu_rotate_rows_f32 (csrc/kernels.cu:316-327): f32 rows in, rotated f32 rows out."""
    M = x.shape[0]
    K = K if K is not None else x.shape[1]
    out = torch.empty((M, K), dtype=torch.float32, device=x.device)
    rc = lib().gpu_rotate_rows_f32(C.c_int(prologue), _p(x), C.c_int64(x.stride(0)), C.c_int64(up_offset), _p(norm_w),
                                   C.c_float(eps), _p(out), C.c_int(M), C.c_int(K), _st())
    assert rc == 0, rc
    return out


def sd_quant_rows(x, rotate=0):
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    rc = lib().gpu_sd_quant_rows(_p(x), C.c_int64(x.stride(0)), _p(q), _p(s), C.c_int(M), C.c_int(K), C.c_int(rotate), _st())
    assert rc == 0, rc
    return q, s


def sd_src_quant_rows(mode, x, rotate=0, *, w=None, b=None, eps=0.0, d=0):
    """The reference's fused-source SD quantizers (csrc/sd.cu:690-708); mode 'ln', 'geglu' or 'unpad'."""
    M = x.shape[0]
    K = {"ln": lambda: x.shape[1], "geglu": lambda: x.shape[1] // 2, "unpad": lambda: x.shape[1] * d}[mode]()
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    if mode == "ln":
        rc = lib().gpu_sd_ln_quant_rows(_p(x), C.c_int64(x.stride(0)), _p(w), _p(b), C.c_float(eps), _p(q), _p(s), C.c_int(M),
                                        C.c_int(K), C.c_int(rotate), _st())
    elif mode == "geglu":
        rc = lib().gpu_sd_geglu_quant_rows(_p(x), _p(q), _p(s), C.c_int(M), C.c_int(K), C.c_int(rotate), _st())
    else:
        rc = lib().gpu_sd_unpad_quant_rows(_p(x), _p(q), _p(s), C.c_int(M), C.c_int(x.shape[1]), C.c_int(d), C.c_int(x.shape[2]),
                                           C.c_int(rotate), _st())
    assert rc == 0, rc
    return q, s


def sd_group_norm_quant_rows(x, w, b, groups, eps, rotate=0):
    """The reference's gpu_sd_group_norm_quant_rows (csrc/sd.cu:710-724); x [N, P, C] half."""
    N, P, Cc = x.shape
    q = torch.empty((N * P, Cc), dtype=torch.int8, device=x.device)
    s = torch.empty((N * P,), dtype=torch.float32, device=x.device)
    sums = torch.empty((N * groups * 2 + 2,), dtype=torch.float64, device=x.device)
    rc = lib().gpu_sd_group_norm_quant_rows(_p(x), _p(w), _p(b), _p(sums), C.c_int(N), C.c_int64(P), C.c_int(Cc), C.c_int(groups),
                                            C.c_float(eps), _p(q), _p(s), C.c_int(rotate), _st())
    assert rc == 0, rc
    return q, s


def convrot_requant(x, seed=0):
    N, K = x.shape
    q = torch.empty((N, K), dtype=torch.int8, device=x.device)
    s = torch.empty((N,), dtype=torch.float32, device=x.device)
    rc = lib().gpu_convrot_requant(C.c_int(_DT[x.dtype]), _p(x), _p(q), _p(s), C.c_int64(N), C.c_int(K), C.c_uint64(seed), _st())
    assert rc == 0, rc
    return q, s


def convrot_dequant(q, s, dtype=torch.float32):
    N, K = q.shape
    out = torch.empty((N, K), dtype=dtype, device=q.device)
    rc = lib().gpu_convrot_dequant(C.c_int(_DT[dtype]), _p(q), _p(s), _p(out), C.c_int64(N), C.c_int(K), _st())
    assert rc == 0, rc
    return out


def w6_decode(packed, s_rel, K, G=32):
    N = packed.shape[0]
    out = torch.empty((N, K), dtype=torch.int8, device=packed.device)
    rc = lib().gpu_w6_decode(_p(packed), _p(s_rel), _p(out), C.c_int64(N), C.c_int(K), C.c_int(G), _st())
    assert rc == 0, rc
    return out


def w6_requant(w, seed=1):
    """bf16 [N,K] -> (packed u8 [N,3K/4], s_rel u8 [N,K/32], s_channel f32 [N]); always stochastic in the reference."""
    N, K = w.shape
    packed = torch.empty((N, K * 3 // 4), dtype=torch.uint8, device=w.device)
    s_rel = torch.empty((N, K // 32), dtype=torch.uint8, device=w.device)
    s_ch = torch.empty((N,), dtype=torch.float32, device=w.device)
    rc = lib().gpu_w6_requant(_p(w), _p(packed), _p(s_rel), _p(s_ch), C.c_int64(N), C.c_int(K), C.c_uint64(seed), _st())
    assert rc == 0, rc
    return packed, s_rel, s_ch


def int8_gemm(A, W, xs, ws, bias=None, *, out_dtype=torch.bfloat16, rscale=None, resid=None, out=None):
    M, K = A.shape
    N = W.shape[0]
    D = out if out is not None else torch.empty((M, N), dtype=out_dtype, device=A.device)
    if resid is not None:
        good = lib().launch_cutlass_int8_dequant_residual(_p(A), _p(W), _p(xs), _p(ws), _p(bias), _p(rscale), _p(resid),
                                                          _p(D), C.c_int64(M), C.c_int64(N), C.c_int64(K),
                                                          C.c_int(_DT[D.dtype]), _st())
    else:
        good = lib().launch_cutlass_int8_dequant(_p(A), _p(W), _p(xs), _p(ws), _p(bias), _p(D), C.c_int64(M), C.c_int64(N),
                                                 C.c_int64(K), C.c_int(_DT[D.dtype]), _st())
    assert good, "reference CUTLASS launcher declined"
    return D


def selected_config(M, N, K) -> int:
    return lib().cutlass_int8_selected_config(C.c_int64(M), C.c_int64(N), C.c_int64(K))
