"""The weight-only int8 linear of the text encoders (gpu_wo8_linear) against the reference's three-call flow: rotate the f32
rows (gpu_rotate_rows_f32, bit-identical to the reference's kernel), dequantize the weight (gpu_dequant_i8, likewise), fp32
product. The product here runs on the bf16 tensor cores with the activation split in two bf16 terms, so it is not
bit-identical to an fp32 GEMM (which has no canonical summation order either); the tolerance is stated against the exact
(fp64) product of the same rotated rows and dequantized weights: 1e-5 of the largest output magnitude, and no worse than
three times the error of an fp32 GEMM of the same operands."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
PLAIN, RMS, SWIGLU = 0, 1, 3


@pytest.mark.parametrize("M,N,K,pro", [(77, 1024, 1024, PLAIN), (300, 2560, 2560, RMS), (512, 1536, 4096, SWIGLU), (1, 768, 256, PLAIN)])
def test_against_the_fp32_flow(pkg, dev, M, N, K, pro):
    g = torch.Generator().manual_seed(M + N + K)
    L = pkg.linear
    width = 2 * K if pro == SWIGLU else K
    x = (torch.randn(M, width, generator=g) * 1.5).to(dev)
    x[:, 3] *= 30.0                                                # an outlier channel, as text-encoder states have
    norm_w = (torch.randn(K, generator=g) * 0.1 + 1.0).to(dev) if pro == RMS else None
    w = torch.randn(N, K, generator=g) * 0.03
    Wq, ws = L.convrot_requant(w.to(dev), 0)                       # int8 ConvRot weight + per-channel scale
    kw = dict(K=K, up_offset=K if pro == SWIGLU else 0, norm_w=norm_w, eps=1e-6)
    xr = L.rotate_rows_f32(x, pro, **kw)
    wf = L.dequant_i8(Wq, ws)
    exact = xr.double() @ wf.double().t()
    fp32 = (xr @ wf.t()).double()                                  # what the reference's flow computes (cuBLAS fp32)
    got = L.wo8_linear(x, Wq, ws, pro, **kw)
    scale = exact.abs().max().item()
    err, err32 = (got.double() - exact).abs().max().item(), (fp32 - exact).abs().max().item()
    assert err <= 1e-5 * scale, (err, scale)
    assert err <= max(3 * err32, 2e-6 * scale), (err, err32)
    # beta = 1 accumulates into the residual stream, as the attention-out and MLP-down linears do
    base = torch.randn(M, N, generator=g).to(dev)
    acc = base.clone()
    L.wo8_linear(x, Wq, ws, pro, out=acc, beta=1.0, **kw)
    assert (acc.double() - (base.double() + exact)).abs().max().item() <= 1e-5 * max(scale, base.abs().max().item())
    assert L.kernel_status() == 0


def test_argument_checks(pkg, dev):
    L = pkg.linear
    x = torch.zeros(4, 300, device=dev)
    Wq = torch.zeros(8, 300, dtype=torch.int8, device=dev)
    ws = torch.ones(8, device=dev)
    with pytest.raises(pkg.GpuKernelError, match="-1"):
        L.wo8_linear(x, Wq, ws)                                     # K % 256 != 0
    x = torch.zeros(4, 256, device=dev)
    Wq = torch.zeros(8, 256, dtype=torch.int8, device=dev)
    with pytest.raises(pkg.GpuKernelError, match="-207"):
        L.wo8_linear(x, Wq, ws, beta=0.5)
    with pytest.raises(pkg.GpuKernelError, match="-3"):
        L.wo8_linear(x, Wq, ws, 11)                                 # a prologue gpu_rotate_rows_f32 does not take
