"""CPU stand-in for the product's `linear` module, built on the oracle, so that host-side logic (tensor-parallel
sharding and its collectives) can be tested without a GPU. Same call names and argument meaning as
comfyui-backend-but-rust_b200/linear.py."""
from __future__ import annotations

import torch

from oracle import oracle as O


def quant_rows(x, prologue=0, rotate=0, **kw):
    return O.quant_rows(x.contiguous(), prologue, rotate, **kw)


def quant_rows_amax(x, prologue=0, rotate=0, **kw):
    v = O.quant_rows(x.contiguous(), prologue, rotate, out_f=True)
    return v.abs().amax(1)


def quant_rows_scaled(x, amax, prologue=0, rotate=0, **kw):
    """q = clamp(rint(bf(bf(v) / bf(scale)))) with scale from the given maxima (csrc/kernels.cu:241-255)."""
    assert x.dtype == torch.bfloat16
    v = O.quant_rows(x.contiguous(), prologue, rotate, out_f=True)
    scale = torch.clamp(torch.clamp(amax, max=3.38953139e38) * torch.tensor(1 / 127, dtype=torch.float32), min=1e-30)
    st = scale.bfloat16()
    q = torch.clamp(torch.round((v.bfloat16() / st[:, None]).float()), -128, 127).to(torch.int8)
    return q, scale


def int8_gemm(A, W, xs, ws, bias=None, *, out_dtype=torch.bfloat16, act=0, rscale=None, resid=None, out=None):
    return O.int8_gemm(A.contiguous(), W.contiguous(), xs.contiguous(), ws.contiguous(), bias, rscale, resid, out_dtype, act, 3)


def int8_gemm_acc_i32(A, W, out=None):
    return O.int8_gemm_acc(A.contiguous(), W.contiguous())


def int8_epilogue(acc, xs, ws, bias=None, *, out_dtype=torch.bfloat16, act=0, rscale=None, resid=None, out=None):
    return O.epilogue(acc.contiguous(), xs.contiguous(), ws.contiguous(), bias, rscale, resid.contiguous() if resid is not None else None,
                      out_dtype, act, 3)


def bias_residual_add(y, bias=None, resid=None, *, out=None, n0=0):
    """out[:, n0:n0+Nc] = T(T(y + bias) + resid) like gpu_bias_residual_add."""
    Nc = y.shape[1]
    v = y.float()
    if bias is not None:
        v = (v + bias[n0:n0 + Nc].float()).to(y.dtype).float()
    if resid is not None:
        v = v + resid[:, n0:n0 + Nc].float()
    v = v.to(y.dtype)
    if out is None:
        return v
    out[:, n0:n0 + Nc] = v
    return out


def set_gemm_cluster_limit(clusters):
    return 0


def convrot_requant(w, seed=0):
    return O.convrot_requant(w.contiguous(), seed)
