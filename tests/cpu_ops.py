"""CPU stand-in for the product's `linear` module, built on the oracle, so that host-side logic (tensor-parallel
sharding and its collectives) can be tested without a GPU. Same call names and argument meaning as
comfyui-backend-but-rust_b200/linear.py."""
from __future__ import annotations

import torch

from oracle import oracle as O


def quant_rows(x, prologue=0, rotate=0, **kw):
    return O.quant_rows(x.contiguous(), prologue, rotate, **kw)


def quant_rows_amax(x, prologue=0, rotate=0):
    v = O.quant_rows(x.contiguous(), prologue, rotate, out_f=True)
    return v.abs().amax(1)


def quant_rows_scaled(x, amax, prologue=0, rotate=0):
    """q = clamp(rint(bf(bf(v) / bf(scale)))) with scale from the given maxima (csrc/kernels.cu:241-255)."""
    assert x.dtype == torch.bfloat16
    v = O.quant_rows(x.contiguous(), prologue, rotate, out_f=True)
    scale = torch.clamp(torch.clamp(amax, max=3.38953139e38) * torch.tensor(1 / 127, dtype=torch.float32), min=1e-30)
    st = scale.bfloat16()
    q = torch.clamp(torch.round((v.bfloat16() / st[:, None]).float()), -128, 127).to(torch.int8)
    return q, scale


def int8_gemm(A, W, xs, ws, bias=None, *, out_dtype=torch.bfloat16, act=0, rscale=None, resid=None, out=None):
    return O.int8_gemm(A.contiguous(), W.contiguous(), xs.contiguous(), ws.contiguous(), bias, rscale, resid, out_dtype, act, 3)


def int8_gemm_acc_i32(A, W):
    return O.int8_gemm_acc(A.contiguous(), W.contiguous())


def int8_epilogue(acc, xs, ws, bias=None, *, out_dtype=torch.bfloat16, act=0, rscale=None, resid=None, out=None):
    return O.epilogue(acc.contiguous(), xs.contiguous(), ws.contiguous(), bias, rscale, resid.contiguous() if resid is not None else None,
                      out_dtype, act, 3)


def convrot_requant(w, seed=0):
    return O.convrot_requant(w.contiguous(), seed)
