"""ctypes binding of the CPU oracle (``liboracle.so``, built from ``oracle.cpp`` by ``make -C oracle``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` -- never by the product package.

All arguments are CPU ``torch`` tensors (contiguous unless a stride is passed); dtype codes follow the
reference (0 f32, 1 f16, 2 bf16; ``src/ffi.rs:11-13``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

DT_F32, DT_F16, DT_BF16 = 0, 1, 2
PRO_PLAIN, PRO_RMS, PRO_GATE, PRO_SWIGLU, PRO_LAYERNORM, PRO_SILU, PRO_GELU, PRO_ADALN = range(8)
PRO_SITU, PRO_LN_MOD, PRO_LN_AFFINE = 8, 9, 10
PRO_GELU_TANH = 11
PRO_SITU_FAST = 13
_DT = {torch.float32: DT_F32, torch.float16: DT_F16, torch.bfloat16: DT_BF16}
_TORCH = {v: k for k, v in _DT.items()}


def build(force: bool = False) -> str:
    """Compile liboracle.so if it is missing or older than its source."""
    src = os.path.join(_HERE, "oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _chk(t, *dtypes):
    assert t.device.type == "cpu" and t.is_contiguous(), "oracle takes contiguous CPU tensors"
    if dtypes:
        assert t.dtype in dtypes, (t.dtype, dtypes)
    return t


def num_threads() -> int:
    return lib().orc_num_threads()


def use_all_cores() -> int:
    """Use every host core the process may run on, whatever OMP_NUM_THREADS says; returns the thread count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_threads(C.c_int(n))
    return num_threads()


def fht_rows(x: torch.Tensor, group: int = 256) -> torch.Tensor:
    """Rotated copy of f32 rows (groups of 256 or 64 along the last dim)."""
    y = _chk(x.clone(), torch.float32)
    K = y.shape[-1]
    assert K % group == 0
    lib().orc_fht_rows(_p(y), C.c_int64(y.numel() // K), C.c_int(K), C.c_int(group))
    return y


def quant_rows(x, prologue=PRO_PLAIN, rotate=0, *, K=None, x_stride=None, g=None, g_stride=0, up_offset=0,
               norm_w=None, eps=0.0, mod_scale=None, mod_shift=None, out_f=False, contract=1, norm_b=None):
    """gpu_quant_rows on host cores. Returns (q int8 [M,K], scales f32 [M]) or the rotated f32 rows."""
    _chk(x, torch.bfloat16, torch.float32)
    M = x.shape[0]
    K = K if K is not None else x.shape[1]
    x_stride = x_stride if x_stride is not None else x.stride(0)
    q = torch.empty((M, K), dtype=torch.int8)
    s = torch.empty((M,), dtype=torch.float32)
    o = torch.empty((M, K), dtype=torch.float32) if out_f else None
    rc = lib().orc_quant_rows(C.c_int(_DT[x.dtype]), C.c_int(prologue), _p(x), C.c_int64(x_stride), _p(g),
                              C.c_int64(g_stride), C.c_int64(up_offset), _p(norm_w), C.c_float(eps), _p(mod_scale),
                              _p(mod_shift), _p(q), _p(s), C.c_int(M), C.c_int(K), C.c_int(rotate), _p(o),
                              C.c_int(contract), _p(norm_b))
    if rc:
        raise RuntimeError(f"orc_quant_rows failed with code {rc}")
    return o if out_f else (q, s)


def sd_quant_rows(x, rotate=0):
    _chk(x, torch.float16)
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8)
    s = torch.empty((M,), dtype=torch.float32)
    rc = lib().orc_sd_quant_rows(_p(x), C.c_int64(x.stride(0)), _p(q), _p(s), C.c_int(M), C.c_int(K), C.c_int(rotate))
    if rc:
        raise RuntimeError(f"orc_sd_quant_rows failed with code {rc}")
    return q, s


def sd_src_quant_rows(mode, x, rotate=0, *, w=None, b=None, eps=0.0, d=0):
    """gpu_sd_{ln,geglu,unpad}_quant_rows on host cores; mode 'ln' (x [M,K] half), 'geglu' (x [M,2K]), 'unpad' (x [M,H,dp])."""
    _chk(x, torch.float16)
    M = x.shape[0]
    code = {"ln": 1, "geglu": 2, "unpad": 3}[mode]
    K = x.shape[1] if code == 1 else x.shape[1] // 2 if code == 2 else x.shape[1] * d
    heads, dp = (x.shape[1], x.shape[2]) if code == 3 else (0, 0)
    q = torch.empty((M, K), dtype=torch.int8)
    s = torch.empty((M,), dtype=torch.float32)
    rc = lib().orc_sd_src_quant_rows(C.c_int(code), _p(x), C.c_int64(x.stride(0)), _p(w), _p(b), C.c_float(eps), C.c_int(heads),
                                     C.c_int(d), C.c_int(dp), _p(q), _p(s), C.c_int(M), C.c_int(K), C.c_int(rotate))
    if rc:
        raise RuntimeError(f"orc_sd_src_quant_rows failed with code {rc}")
    return q, s


def sd_group_norm_quant_rows(x, w, b, groups, eps, rotate=0):
    """gpu_sd_group_norm_quant_rows on host cores: x [N, P, C] half -> (codes [N * P, C], scales [N * P])."""
    _chk(x, torch.float16)
    N, P, Cc = x.shape
    q = torch.empty((N * P, Cc), dtype=torch.int8)
    s = torch.empty((N * P,), dtype=torch.float32)
    rc = lib().orc_sd_gn_quant_rows(_p(x), _p(_chk(w, torch.float32)), _p(_chk(b, torch.float32)), C.c_int(N), C.c_int64(P),
                                    C.c_int(Cc), C.c_int(groups), C.c_float(eps), _p(q), _p(s), C.c_int(rotate))
    if rc:
        raise RuntimeError(f"orc_sd_gn_quant_rows failed with code {rc}")
    return q, s


def convrot_requant(x, seed=0):
    _chk(x, torch.float32, torch.bfloat16)
    N, K = x.shape
    q = torch.empty((N, K), dtype=torch.int8)
    s = torch.empty((N,), dtype=torch.float32)
    rc = lib().orc_convrot_requant(C.c_int(_DT[x.dtype]), _p(x), _p(q), _p(s), C.c_int64(N), C.c_int(K),
                                   C.c_uint64(seed))
    if rc:
        raise RuntimeError(f"orc_convrot_requant failed with code {rc}")
    return q, s


def convrot_dequant(q, s, dtype=torch.float32):
    _chk(q, torch.int8), _chk(s, torch.float32)
    N, K = q.shape
    out = torch.empty((N, K), dtype=dtype)
    rc = lib().orc_convrot_dequant(C.c_int(_DT[dtype]), _p(q), _p(s), _p(out), C.c_int64(N), C.c_int(K))
    if rc:
        raise RuntimeError(f"orc_convrot_dequant failed with code {rc}")
    return out


def dequant_i8(q, s):
    N, K = q.shape
    out = torch.empty((N, K), dtype=torch.float32)
    rc = lib().orc_dequant_i8(_p(_chk(q, torch.int8)), _p(_chk(s, torch.float32)), _p(out), C.c_int64(N), C.c_int64(K))
    if rc:
        raise RuntimeError(f"orc_dequant_i8 failed with code {rc}")
    return out


def embed_dequant(q, s, rotate=1):
    M, K = q.shape
    out = torch.empty((M, K), dtype=torch.float32)
    rc = lib().orc_embed_dequant(_p(_chk(q, torch.int8)), _p(_chk(s, torch.float32)), _p(out), C.c_int(M), C.c_int(K),
                                 C.c_int(rotate))
    if rc:
        raise RuntimeError(f"orc_embed_dequant failed with code {rc}")
    return out


def w6_decode(packed, s_rel, K, G=32):
    """packed u8 [N, 3K/4], s_rel u8 (e4m3 bits) [N, K/G] -> int8 [N, K]."""
    _chk(packed, torch.uint8), _chk(s_rel, torch.uint8)
    N = packed.shape[0]
    out = torch.empty((N, K), dtype=torch.int8)
    rc = lib().orc_w6_decode(_p(packed), _p(s_rel), _p(out), C.c_int64(N), C.c_int(K), C.c_int(G))
    if rc:
        raise RuntimeError(f"orc_w6_decode failed with code {rc}")
    return out


def w6_requant(w: torch.Tensor, seed: int = 1):
    """gpu_w6_requant on host cores: bf16 [N, K] -> (packed u8 [N, 3K/4], s_rel u8 [N, K/32], s_channel f32 [N])."""
    _chk(w, torch.bfloat16)
    N, K = w.shape
    packed = torch.empty((N, K * 3 // 4), dtype=torch.uint8)
    s_rel = torch.empty((N, K // 32), dtype=torch.uint8)
    s_ch = torch.empty((N,), dtype=torch.float32)
    rc = lib().orc_w6_requant(_p(w), _p(packed), _p(s_rel), _p(s_ch), C.c_int64(N), C.c_int(K), C.c_uint64(seed))
    if rc:
        raise RuntimeError(f"orc_w6_requant failed with code {rc}")
    return packed, s_rel, s_ch


def w6_pack_codes(codes: torch.Tensor) -> torch.Tensor:
    """6-bit codes u8 [N,K] (1..63) -> the reference's two-plane row layout u8 [N, 3K/4]
    (nibble plane then 2-bit plane; csrc/vendor/w6a8_requant.cu:128-151)."""
    N, K = codes.shape
    c = codes.to(torch.int32)
    lo = (c[:, 0::2] & 15) | ((c[:, 1::2] & 15) << 4)
    t = (c >> 4) & 3
    hi = t[:, 0::4] | (t[:, 1::4] << 2) | (t[:, 2::4] << 4) | (t[:, 3::4] << 6)
    return torch.cat([lo, hi], dim=1).to(torch.uint8).contiguous()


def int8_gemm_acc(A, W):
    _chk(A, torch.int8), _chk(W, torch.int8)
    M, K = A.shape
    N = W.shape[0]
    acc = torch.empty((M, N), dtype=torch.int32)
    lib().orc_int8_gemm_acc(_p(A), _p(W), _p(acc), C.c_int64(M), C.c_int64(N), C.c_int64(K))
    return acc


def epilogue(acc, xs, ws, bias=None, rscale=None, resid=None, out_dtype=torch.bfloat16, act=0, contract=0):
    _chk(acc, torch.int32)
    M, N = acc.shape
    D = torch.empty((M, N), dtype=out_dtype)
    rc = lib().orc_epilogue(_p(acc), _p(_chk(xs, torch.float32)), _p(_chk(ws, torch.float32)), _p(bias), _p(rscale),
                            _p(resid), _p(D), C.c_int64(M), C.c_int64(N), C.c_int(_DT[out_dtype]), C.c_int(act),
                            C.c_int(contract))
    if rc:
        raise RuntimeError(f"orc_epilogue failed with code {rc}")
    return D


def int8_gemm(A, W, xs, ws, bias=None, rscale=None, resid=None, out_dtype=torch.bfloat16, act=0, contract=0):
    """The whole quantized linear on host cores (the timed CPU baseline)."""
    M, K = A.shape
    N = W.shape[0]
    D = torch.empty((M, N), dtype=out_dtype)
    rc = lib().orc_int8_gemm(_p(_chk(A, torch.int8)), _p(_chk(W, torch.int8)), _p(xs), _p(ws), _p(bias), _p(rscale),
                             _p(resid), _p(D), C.c_int64(M), C.c_int64(N), C.c_int64(K), C.c_int(_DT[out_dtype]),
                             C.c_int(act), C.c_int(contract))
    if rc:
        raise RuntimeError(f"orc_int8_gemm failed with code {rc}")
    return D
