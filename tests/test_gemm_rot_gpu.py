"""The GEMM whose epilogue applies the activation and the R256 rotation (gpu_int8_gemm_act_rot) and the quantizer's second
pass on its rows (gpu_quant_rows_rotated), through the C ABI. The pair must give, bit for bit, the codes and scales of the
reference's arrangement: its GEMM, then its quantizer with the activation prologue and rotate = 1 (src/qwen21.rs:378-417;
csrc/kernels.cu:76-259), run here from the reference's own kernels on the same device buffers. The rotated rows themselves
are checked against this library's f32 rotation of the activation GEMM's output."""
from __future__ import annotations

import pytest
import torch

from conftest import assert_bits_equal

pytestmark = pytest.mark.gpu

PROLOGUE_OF_ACT = {1: 11, 2: 5, 3: 6}     # gelu-tanh, silu, gelu-erf as quantizer prologues (src/ffi.rs:15-29)


def _operands(M, N, K, seed, dev, spread=0.3):
    g = torch.Generator().manual_seed(seed)
    A = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
    W = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8)
    xs = (torch.rand(M, generator=g) * 0.05 + 1e-3) * spread
    ws = torch.rand(N, generator=g) * 1e-3 + 1e-4
    bias = (torch.randn(N, generator=g) * 0.5).bfloat16()
    return A.to(dev), W.to(dev), xs.to(dev), ws.to(dev), bias.to(dev)


def _check(pkg, ref, A, W, xs, ws, bias, act):
    L = pkg.linear
    D, parts = L.int8_gemm_act_rot(A, W, xs, ws, bias, act=act)
    q, s = L.quant_rows_rotated(D, parts)
    y_ref = ref.int8_gemm(A, W, xs, ws, bias, out_dtype=torch.bfloat16)
    q_ref, s_ref = ref.quant_rows(y_ref, PROLOGUE_OF_ACT[act], 1)
    assert_bits_equal(s, s_ref, "scales")
    assert_bits_equal(q, q_ref, "codes")
    assert L.kernel_status() == 0
    return D, parts


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (1, 256, 64), (300, 512, 512), (129, 1024, 272), (1000, 768, 1040),
                                   (2048, 2560, 640)])
@pytest.mark.parametrize("act", [1, 2, 3])
def test_pair_equals_the_reference_gemm_then_quantizer(pkg, ref, dev, M, N, K, act):
    A, W, xs, ws, bias = _operands(M, N, K, 7 * M + N + K + act, dev)
    D, _ = _check(pkg, ref, A, W, xs, ws, bias, act)
    # the rotated rows: this library's f32 rotation of the activation GEMM's output, rounded to bf16
    ya = pkg.linear.int8_gemm(A, W, xs, ws, bias, act=act)
    want = pkg.linear.rotate_rows_f32(ya.float()).bfloat16()
    assert_bits_equal(D, want, "rotated rows")


def test_without_bias_and_with_wide_values(pkg, ref, dev):
    A, W, xs, ws, _ = _operands(520, 512, 256, 5, dev, spread=40.0)     # values far outside the table's shared-memory part
    _check(pkg, ref, A, W, xs, ws, None, 1)
    A, W, xs, ws, _ = _operands(520, 512, 256, 6, dev, spread=1e-4)    # ... and far below it
    _check(pkg, ref, A, W, xs, ws, None, 1)


def test_rows_with_infinities_and_nans_take_the_exact_division(pkg, ref, dev):
    A, W, xs, ws, bias = _operands(300, 768, 256, 9, dev)
    xs[3] = float("inf")          # acc * inf: +-inf, or NaN where acc == 0
    xs[100] = float("nan")
    xs[257] = 3.0e38              # finite values whose rotation overflows
    xs[299] = 0.0                 # a row of bias only
    A[3, :] = 0
    A[3, ::2] = 1
    _check(pkg, ref, A, W, xs, ws, bias, 1)
    # huge but finite values in one half of one tile: below 2^120 the sums run without the halvings, above it with them
    for big in (1.0e36, 2.0e37, 3.0e38):
        b = bias.clone()
        b[600] = big
        b[77] = -big
        _check(pkg, ref, A, W, xs, ws, b, 1)
        _check(pkg, ref, A, W, xs, ws, b, 2)
    bias2 = bias.clone()
    bias2[5] = float("inf")       # one column of every row
    bias2[700] = float("nan")
    _check(pkg, ref, A, W, xs, ws, bias2, 1)


def test_benchmark_up_projection_in_full(pkg, ref, dev):
    import importlib
    wl = importlib.import_module("cbr_b200.workloads")
    sp = wl.config(1)[0]
    x = wl.activations(sp.M, sp.K, 1234, outliers="student").to(dev)
    w = wl.weight(sp.N, sp.K, 2345, 0.02).to(dev)
    bias = wl.bias(sp.N, 3456).to(dev)
    a8, xs = pkg.linear.quant_rows(x, 0, 1)
    wq, ws = pkg.linear.convrot_requant(w, 0)
    _check(pkg, ref, a8, wq, xs, ws, bias, 1)


def test_rejects_what_the_epilogue_cannot_rotate(pkg, dev):
    A, W, xs, ws, bias = _operands(64, 384, 128, 3, dev)            # N is not a whole number of rotation groups
    with pytest.raises(pkg.GpuKernelError, match="-208"):
        pkg.linear.int8_gemm_act_rot(A, W, xs, ws, bias, act=1)
    A, W, xs, ws, bias = _operands(64, 256, 128, 3, dev)
    with pytest.raises(pkg.GpuKernelError, match="-208"):
        pkg.linear.int8_gemm_act_rot(A, W, xs, ws, bias, act=0)
    xr = torch.zeros((4, 384), dtype=torch.bfloat16, device=dev)
    with pytest.raises(pkg.GpuKernelError, match="-1"):
        pkg.linear.quant_rows_rotated(xr, torch.zeros((6, 4), device=dev))
