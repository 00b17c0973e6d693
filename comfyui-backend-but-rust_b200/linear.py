"""Host side of the quantized linear over torch CUDA tensors.

Mirrors how the reference's model code drives the path (e.g. src/qwen21.rs:365-418, src/dit.rs:539-614,
src/unet.rs:359-457): ``gpu_quant_rows`` produces the int8 A operand and per-row scales, ``gpu_int8_gemm`` /
``gpu_int8_gemm_residual`` consume them together with an int8 weight and per-channel scales. torch supplies device
memory and the stream only; every computation is one of the library's kernels.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import ffi
from .ffi import ok

_DT = {torch.float32: ffi.DT_F32, torch.float16: ffi.DT_F16, torch.bfloat16: ffi.DT_BF16}


def _lib():
    from . import lib
    return lib


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _cuda(t: torch.Tensor) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError("this path runs on CUDA tensors only")
    return t


def quant_rows(x: torch.Tensor, prologue: int = ffi.PRO_PLAIN, rotate: int = 0, *, K: Optional[int] = None,
               g: Optional[torch.Tensor] = None, up_offset: int = 0, q: Optional[torch.Tensor] = None,
               scales: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
               norm_b: Optional[torch.Tensor] = None, eps: float = 0.0, mod_scale: Optional[torch.Tensor] = None,
               mod_shift: Optional[torch.Tensor] = None):
    """gpu_quant_rows (gpu_quant_rows_b when a LayerNorm bias is given): x [M, >=K] bf16/f32 -> (q int8 [M, K],
    scales f32 [M]). norm_w / norm_b f32 [K]; mod_scale / mod_shift [K] in x's dtype."""
    _cuda(x)
    M = x.shape[0]
    K = K if K is not None else x.shape[1]
    q = q if q is not None else torch.empty((M, K), dtype=torch.int8, device=x.device)
    scales = scales if scales is not None else torch.empty((M,), dtype=torch.float32, device=x.device)
    if norm_b is not None:
        ok(_lib().gpu_quant_rows_b(_DT[x.dtype], prologue, _ptr(x), x.stride(0), _ptr(norm_w), _ptr(norm_b), eps,
                                   _ptr(mod_scale), _ptr(mod_shift), _ptr(q), _ptr(scales), M, K, rotate, _stream()),
           "gpu_quant_rows_b")
        return q, scales
    ok(_lib().gpu_quant_rows(_DT[x.dtype], prologue, _ptr(x), x.stride(0), _ptr(g), g.stride(0) if g is not None else 0,
                             up_offset, _ptr(norm_w), eps, _ptr(mod_scale), _ptr(mod_shift), _ptr(q), _ptr(scales), M, K,
                             rotate, _stream()), "gpu_quant_rows")
    return q, scales


def quant_rows_amax(x: torch.Tensor, prologue: int = ffi.PRO_PLAIN, rotate: int = 0, *, K: Optional[int] = None,
                    g: Optional[torch.Tensor] = None, up_offset: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """gpu_quant_rows_amax: row maxima after prologue and rotation, f32 [M]."""
    _cuda(x)
    M = x.shape[0]
    K = K if K is not None else x.shape[1]
    amax = out if out is not None else torch.empty((M,), dtype=torch.float32, device=x.device)
    ok(_lib().gpu_quant_rows_amax(_DT[x.dtype], prologue, _ptr(x), x.stride(0), _ptr(g), g.stride(0) if g is not None else 0,
                                  up_offset, _ptr(amax), M, K, rotate, _stream()), "gpu_quant_rows_amax")
    return amax


def quant_rows_scaled(x: torch.Tensor, amax: torch.Tensor, prologue: int = ffi.PRO_PLAIN, rotate: int = 0, *,
                      K: Optional[int] = None, g: Optional[torch.Tensor] = None, up_offset: int = 0,
                      q: Optional[torch.Tensor] = None, scales: Optional[torch.Tensor] = None):
    """gpu_quant_rows_scaled: quantize with given row maxima -> (q int8 [M, K], scales f32 [M])."""
    _cuda(x)
    M = x.shape[0]
    K = K if K is not None else x.shape[1]
    q = q if q is not None else torch.empty((M, K), dtype=torch.int8, device=x.device)
    scales = scales if scales is not None else torch.empty((M,), dtype=torch.float32, device=x.device)
    ok(_lib().gpu_quant_rows_scaled(_DT[x.dtype], prologue, _ptr(x), x.stride(0), _ptr(g),
                                    g.stride(0) if g is not None else 0, up_offset, _ptr(amax), _ptr(q), _ptr(scales), M, K,
                                    rotate, _stream()), "gpu_quant_rows_scaled")
    return q, scales


def int8_epilogue(acc, xs, ws, bias=None, *, out_dtype=torch.bfloat16, act: int = 0, rscale=None, resid=None, out=None):
    """gpu_int8_epilogue: the dequant epilogue over int32 accumulators [M, N] in global memory."""
    M, N = acc.shape
    D = out if out is not None else torch.empty((M, N), dtype=out_dtype, device=acc.device)
    ok(_lib().gpu_int8_epilogue(_ptr(acc), _ptr(xs), _ptr(ws), _ptr(bias), _ptr(rscale), _ptr(resid), _ptr(D), M, N,
                                _DT[D.dtype], act, _stream()), "gpu_int8_epilogue")
    return D


def bias_residual_add(y, bias=None, resid=None, *, out=None, n0: int = 0):
    """gpu_bias_residual_add: out[:, n0:n0+Nc] = y + bias[n0:n0+Nc] + resid[:, n0:n0+Nc]; y [M, Nc] contiguous, resid / out
    [M, ld] (out defaults to a new [M, Nc] tensor when neither is given a wider one)."""
    M, Nc = y.shape
    D = out if out is not None else torch.empty((M, Nc), dtype=y.dtype, device=y.device)
    ok(_lib().gpu_bias_residual_add(_ptr(y), _ptr(bias), _ptr(resid), _ptr(D), M, Nc, D.stride(0), n0, _DT[y.dtype], _stream()),
       "gpu_bias_residual_add")
    return D


def set_gemm_cluster_limit(clusters: int) -> int:
    """gpu_int8_gemm_set_cluster_limit: GEMM launches that follow occupy at most this many CTA pairs (0 = all)."""
    return _lib().gpu_int8_gemm_set_cluster_limit(clusters)


def rotate_rows_f32(x: torch.Tensor, prologue: int = ffi.PRO_PLAIN, *, K: Optional[int] = None, up_offset: int = 0,
                    norm_w: Optional[torch.Tensor] = None, eps: float = 0.0):
    _cuda(x)
    M = x.shape[0]
    K = K if K is not None else x.shape[1]
    out = torch.empty((M, K), dtype=torch.float32, device=x.device)
    ok(_lib().gpu_rotate_rows_f32(prologue, _ptr(x), x.stride(0), up_offset, _ptr(norm_w), eps, _ptr(out), M, K, _stream()),
       "gpu_rotate_rows_f32")
    return out


def wo8_linear(x: torch.Tensor, Wq: torch.Tensor, ws: torch.Tensor, prologue: int = ffi.PRO_PLAIN, *, K: Optional[int] = None,
               up_offset: int = 0, norm_w: Optional[torch.Tensor] = None, eps: float = 0.0, out: Optional[torch.Tensor] = None,
               beta: float = 0.0, scratch: Optional[tuple] = None):
    """gpu_wo8_linear: the text encoders' weight-only int8 linear, out = beta * out + R256(prologue(x)) @ (Wq * ws)^T in f32.
    `scratch` = (a_scratch >= 4 M K bytes, w_scratch >= 2 N K bytes), allocated here when not given."""
    _cuda(x)
    M = x.shape[0]
    K = K if K is not None else x.shape[1]
    N = Wq.shape[0]
    out = out if out is not None else torch.empty((M, N), dtype=torch.float32, device=x.device)
    a_s, w_s = scratch if scratch is not None else (torch.empty(4 * M * K, dtype=torch.uint8, device=x.device),
                                                    torch.empty(2 * N * K, dtype=torch.uint8, device=x.device))
    ok(_lib().gpu_wo8_linear(prologue, _ptr(x), x.stride(0), up_offset, _ptr(norm_w), eps, _ptr(Wq), _ptr(ws), _ptr(out), beta,
                             _ptr(a_s), _ptr(w_s), M, N, K, _stream()), "gpu_wo8_linear")
    return out


def sd_quant_rows(x: torch.Tensor, rotate: int = 0):
    """gpu_sd_quant_rows: fp16 rows (activations, or weights at load) -> (q int8, scales f32)."""
    _cuda(x)
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    ok(_lib().gpu_sd_quant_rows(_ptr(x), x.stride(0), _ptr(q), _ptr(s), M, K, rotate, _stream()), "gpu_sd_quant_rows")
    return q, s


def sd_ln_quant_rows(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float, rotate: int = 0):
    """gpu_sd_ln_quant_rows: LayerNorm (f32 weight, bias) of half rows, then the fp16 quantizer."""
    _cuda(x)
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    ok(_lib().gpu_sd_ln_quant_rows(_ptr(x), x.stride(0), _ptr(w), _ptr(b), eps, _ptr(q), _ptr(s), M, K, rotate, _stream()),
       "gpu_sd_ln_quant_rows")
    return q, s


def sd_geglu_quant_rows(x: torch.Tensor, rotate: int = 0):
    """gpu_sd_geglu_quant_rows: x [M, 2 I] half (value, gate) -> codes of value * gelu(gate) [M, I]."""
    _cuda(x)
    M, I = x.shape[0], x.shape[1] // 2
    q = torch.empty((M, I), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    ok(_lib().gpu_sd_geglu_quant_rows(_ptr(x), _ptr(q), _ptr(s), M, I, rotate, _stream()), "gpu_sd_geglu_quant_rows")
    return q, s


def sd_group_norm_quant_rows(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, groups: int, eps: float, rotate: int = 0):
    """gpu_sd_group_norm_quant_rows: x [N, P, C] half -> GroupNorm (f32 weight, bias; no SiLU) -> codes [N * P, C]."""
    _cuda(x)
    N, P, C = x.shape
    q = torch.empty((N * P, C), dtype=torch.int8, device=x.device)
    s = torch.empty((N * P,), dtype=torch.float32, device=x.device)
    sums = torch.empty((N * groups * 2 + 2,), dtype=torch.float64, device=x.device)
    ok(_lib().gpu_sd_group_norm_quant_rows(_ptr(x), _ptr(w), _ptr(b), _ptr(sums), N, P, C, groups, eps, _ptr(q), _ptr(s), rotate,
                                           _stream()), "gpu_sd_group_norm_quant_rows")
    return q, s


def sd_unpad_quant_rows(x: torch.Tensor, d: int, rotate: int = 0):
    """gpu_sd_unpad_quant_rows: x [M, H, dp] half -> codes of the first d values of every head, [M, H * d]."""
    _cuda(x)
    M, H, dp = x.shape
    q = torch.empty((M, H * d), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    ok(_lib().gpu_sd_unpad_quant_rows(_ptr(x), _ptr(q), _ptr(s), M, H, d, dp, rotate, _stream()), "gpu_sd_unpad_quant_rows")
    return q, s


def convrot_requant(x: torch.Tensor, seed: int = 0):
    _cuda(x)
    N, K = x.shape
    q = torch.empty((N, K), dtype=torch.int8, device=x.device)
    s = torch.empty((N,), dtype=torch.float32, device=x.device)
    ok(_lib().gpu_convrot_requant(_DT[x.dtype], _ptr(x), _ptr(q), _ptr(s), N, K, seed, _stream()), "gpu_convrot_requant")
    return q, s


def convrot_dequant(q: torch.Tensor, s: torch.Tensor, dtype=torch.float32):
    N, K = q.shape
    out = torch.empty((N, K), dtype=dtype, device=q.device)
    ok(_lib().gpu_convrot_dequant(_DT[dtype], _ptr(q), _ptr(s), _ptr(out), N, K, _stream()), "gpu_convrot_dequant")
    return out


def dequant_i8(q: torch.Tensor, s: torch.Tensor):
    N, K = q.shape
    out = torch.empty((N, K), dtype=torch.float32, device=q.device)
    ok(_lib().gpu_dequant_i8(_ptr(q), _ptr(s), _ptr(out), N, K, _stream()), "gpu_dequant_i8")
    return out


def embed_dequant(q: torch.Tensor, s: torch.Tensor, rotate: int = 1):
    M, K = q.shape
    out = torch.empty((M, K), dtype=torch.float32, device=q.device)
    ok(_lib().gpu_embed_dequant(_ptr(q), _ptr(s), _ptr(out), M, K, rotate, _stream()), "gpu_embed_dequant")
    return out


def w6_decode(packed: torch.Tensor, s_rel: torch.Tensor, K: int, G: int = 32):
    N = packed.shape[0]
    out = torch.empty((N, K), dtype=torch.int8, device=packed.device)
    ok(_lib().gpu_w6_decode(_ptr(packed), _ptr(s_rel), _ptr(out), N, K, G, _stream()), "gpu_w6_decode")
    return out


def w6_requant(w: torch.Tensor, seed: int = 1):
    """gpu_w6_requant: bf16 [N, K] -> (packed u8 [N, 3K/4], s_rel u8 [N, K/32], s_channel f32 [N])."""
    _cuda(w)
    N, K = w.shape
    packed = torch.empty((N, K * 3 // 4), dtype=torch.uint8, device=w.device)
    s_rel = torch.empty((N, K // 32), dtype=torch.uint8, device=w.device)
    s_ch = torch.empty((N,), dtype=torch.float32, device=w.device)
    ok(_lib().gpu_w6_requant(_ptr(w), _ptr(packed), _ptr(s_rel), _ptr(s_ch), N, K, seed, _stream()), "gpu_w6_requant")
    return packed, s_rel, s_ch


def int8_gemm(A, W, xs, ws, bias=None, *, out_dtype=torch.bfloat16, act: int = 0, rscale=None, resid=None, out=None):
    """gpu_int8_gemm / gpu_int8_gemm_act / gpu_int8_gemm_residual, chosen by the arguments given."""
    _cuda(A)
    M, K = A.shape
    N = W.shape[0]
    D = out if out is not None else torch.empty((M, N), dtype=out_dtype, device=A.device)
    lib = _lib()
    if resid is not None:
        ok(lib.gpu_int8_gemm_residual(_ptr(A), _ptr(W), _ptr(xs), _ptr(ws), _ptr(bias), _ptr(rscale), _ptr(resid), _ptr(D),
                                      M, N, K, _DT[D.dtype], _stream()), "gpu_int8_gemm_residual")
    elif act:
        ok(lib.gpu_int8_gemm_act(_ptr(A), _ptr(W), _ptr(xs), _ptr(ws), _ptr(bias), _ptr(D), M, N, K, _DT[D.dtype], act,
                                 _stream()), "gpu_int8_gemm_act")
    else:
        ok(lib.gpu_int8_gemm(_ptr(A), _ptr(W), _ptr(xs), _ptr(ws), _ptr(bias), _ptr(D), M, N, K, _DT[D.dtype], _stream()),
           "gpu_int8_gemm")
    return D


def int8_gemm_act_rot(A, W, xs, ws, bias=None, *, act: int = 1, out=None, amax_part=None):
    """gpu_int8_gemm_act_rot: bf16(R256(act(linear output))) [M, N] and the partial row maxima [N / 64, M] that
    quant_rows_rotated turns into codes and scales."""
    _cuda(A)
    M, K = A.shape
    N = W.shape[0]
    D = out if out is not None else torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    parts = amax_part if amax_part is not None else torch.empty((N // 64, M), dtype=torch.float32, device=A.device)
    ok(_lib().gpu_int8_gemm_act_rot(_ptr(A), _ptr(W), _ptr(xs), _ptr(ws), _ptr(bias), _ptr(D), _ptr(parts), M, N, K, act,
                                    _stream()), "gpu_int8_gemm_act_rot")
    return D, parts


def quant_rows_rotated(xr, amax_part, *, q=None, scales=None):
    """gpu_quant_rows_rotated: the quantizer's second pass on rows a rotating GEMM epilogue left."""
    _cuda(xr)
    M, K = xr.shape
    q = q if q is not None else torch.empty((M, K), dtype=torch.int8, device=xr.device)
    scales = scales if scales is not None else torch.empty((M,), dtype=torch.float32, device=xr.device)
    ok(_lib().gpu_quant_rows_rotated(_ptr(xr), _ptr(amax_part), _ptr(q), _ptr(scales), M, K, _stream()),
       "gpu_quant_rows_rotated")
    return q, scales


def int8_gemm_acc_i32(A, W, out=None):
    M, K = A.shape
    N = W.shape[0]
    D = out if out is not None else torch.empty((M, N), dtype=torch.int32, device=A.device)
    ok(_lib().gpu_int8_gemm_acc_i32(_ptr(A), _ptr(W), _ptr(D), M, N, K, _stream()), "gpu_int8_gemm_acc_i32")
    return D


def w6a8_gemm(A, packed, s_rel, xs, s_channel, bias=None, *, out_dtype=torch.bfloat16, act: int = 0, rscale=None, resid=None,
              out=None, G: int = 32):
    """gpu_w6a8_gemm / gpu_w6a8_gemm_act / gpu_w6a8_gemm_residual: the W6A8 linear from the packed weight [N, 3K/4] and
    e4m3 scales [N, K/G]."""
    _cuda(A)
    M, K = A.shape
    N = packed.shape[0]
    D = out if out is not None else torch.empty((M, N), dtype=out_dtype, device=A.device)
    lib = _lib()
    if resid is not None:
        ok(lib.gpu_w6a8_gemm_residual(_ptr(A), _ptr(packed), _ptr(s_rel), _ptr(xs), _ptr(s_channel), _ptr(bias), _ptr(rscale),
                                      _ptr(resid), _ptr(D), M, N, K, G, _DT[D.dtype], _stream()), "gpu_w6a8_gemm_residual")
    elif act:
        ok(lib.gpu_w6a8_gemm_act(_ptr(A), _ptr(packed), _ptr(s_rel), _ptr(xs), _ptr(s_channel), _ptr(bias), _ptr(D), M, N, K, G,
                                 _DT[D.dtype], act, _stream()), "gpu_w6a8_gemm_act")
    else:
        ok(lib.gpu_w6a8_gemm(_ptr(A), _ptr(packed), _ptr(s_rel), _ptr(xs), _ptr(s_channel), _ptr(bias), _ptr(D), M, N, K, G,
                             _DT[D.dtype], _stream()), "gpu_w6a8_gemm")
    return D


def w6a8_gemm_acc_i32(A, packed, s_rel, G: int = 32):
    M, K = A.shape
    N = packed.shape[0]
    D = torch.empty((M, N), dtype=torch.int32, device=A.device)
    ok(_lib().gpu_w6a8_gemm_acc_i32(_ptr(A), _ptr(packed), _ptr(s_rel), _ptr(D), M, N, K, G, _stream()), "gpu_w6a8_gemm_acc_i32")
    return D


def kernel_status() -> int:
    """Device status word (0 = every kernel completed its waits); synchronises the device and clears the word."""
    import ctypes as C
    v = C.c_int(0)
    ok(_lib().gpu_kernels_status(C.byref(v)), "gpu_kernels_status")
    return v.value


@dataclass
class QuantLinear:
    """An int8 linear as the reference's DiT blocks hold it: weight int8 [N, K] (already rotated when `rotate`),
    per-output-channel scales f32 [N], optional bias in the activation dtype."""
    weight: torch.Tensor
    scale: torch.Tensor
    bias: Optional[torch.Tensor] = None
    rotate: int = 0

    @staticmethod
    def from_float(w: torch.Tensor, bias=None, rotate: int = 0) -> "QuantLinear":
        """Quantize-at-load: fp16 weights through gpu_sd_quant_rows (src/unet.rs:367-383), f32/bf16 weights through
        gpu_convrot_requant with seed 0 (src/moss.rs:88-94; always R256)."""
        if w.dtype == torch.float16:
            q, s = sd_quant_rows(w.contiguous(), rotate)
        else:
            if rotate not in (1, 256):
                raise ValueError("f32/bf16 weights are packed by gpu_convrot_requant, which always rotates (R256)")
            q, s = convrot_requant(w.contiguous(), 0)
        return QuantLinear(q, s, bias, rotate)

    def forward(self, x: torch.Tensor, *, prologue: int = ffi.PRO_PLAIN, act: int = 0, rscale=None, resid=None,
                out=None) -> torch.Tensor:
        if x.dtype == torch.float16:
            a8, xs = sd_quant_rows(x, self.rotate)
        else:
            a8, xs = quant_rows(x, prologue, 1 if self.rotate else 0)
        return int8_gemm(a8, self.weight, xs, self.scale, self.bias, out_dtype=x.dtype, act=act, rscale=rscale,
                         resid=resid, out=out)
