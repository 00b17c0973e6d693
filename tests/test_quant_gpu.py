"""GPU parity of the activation quantizer (through the C ABI) against the CPU oracle, the committed golden vectors
and, where it is built, the reference's own kernel. int8 codes and fp32 scales are compared bit for bit."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import assert_bits_equal

pytestmark = pytest.mark.gpu
PLAIN, GATE, SWIGLU, SILU, GELU, GELU_TANH = 0, 2, 3, 5, 6, 11


def _x(M, K, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    x[:, torch.randperm(K, generator=g)[: max(1, K // 100)]] *= 20.0
    return x.to(dtype)


@pytest.mark.parametrize("M,K", [(1, 256), (64, 256), (200, 3072), (70, 768), (33, 12288), (9, 13824), (5, 32768)])
@pytest.mark.parametrize("rotate", [0, 1])
def test_plain_bf16_bit_exact(pkg, oracle, dev, M, K, rotate):
    x = _x(M, K, 1000 + K + M)
    q, s = pkg.linear.quant_rows(x.to(dev), PLAIN, rotate)
    qo, so = oracle.quant_rows(x, PLAIN, rotate)
    assert_bits_equal(q, qo, "codes")
    assert_bits_equal(s, so, "scales")


def test_f32_rows_and_row_stride(pkg, oracle, dev):
    x = _x(40, 2048, 7, torch.float32)
    q, s = pkg.linear.quant_rows(x.to(dev), PLAIN, 1, K=1024)           # rows 2048 apart, only 1024 columns used
    qo, so = oracle.quant_rows(x, PLAIN, 1, K=1024)
    assert_bits_equal(q, qo, "codes")
    assert_bits_equal(s, so, "scales")
    rot = pkg.linear.rotate_rows_f32(x[:, :512].contiguous().to(dev))
    assert_bits_equal(rot, oracle.fht_rows(x[:, :512].contiguous()), "gpu_rotate_rows_f32")


def test_special_rows(pkg, oracle, dev):
    x = torch.zeros(4, 512).bfloat16()
    x[1, 5] = float("inf")
    x[2, 300] = float("nan")
    x[3] = 1e-38
    for rot in (0, 1):
        q, s = pkg.linear.quant_rows(x.to(dev), PLAIN, rot)
        qo, so = oracle.quant_rows(x, PLAIN, rot)
        assert_bits_equal(s, so, f"scales rot={rot}")
        # rows holding inf or NaN turn into NaN everywhere once rotated; codes still follow the same clamp rules
        assert_bits_equal(q, qo, f"codes rot={rot}")


@pytest.mark.parametrize("pro", [SILU, GELU, GELU_TANH, SWIGLU, GATE])
def test_activation_prologues_within_one_step_of_the_oracle(pkg, oracle, dev, pro):
    # expf / tanhf / erff differ between CUDA and the host libm in the last ulp: at most one step on <= 0.1 % of codes
    x = _x(96, 2048, 50 + pro)
    gt = _x(96, 1024, 60 + pro)
    kw = dict(K=1024, up_offset=1024) if pro == SWIGLU else dict(K=1024)
    kwo = dict(kw)
    if pro == GATE:
        kw["g"] = gt.to(dev)
        kwo.update(g=gt, g_stride=1024)
    q, s = pkg.linear.quant_rows(x.to(dev), pro, 1, **kw)
    qo, so = oracle.quant_rows(x, pro, 1, **kwo)
    d = (q.cpu().int() - qo.int()).abs()
    assert int(d.max()) <= 1 and float((d != 0).float().mean()) <= 1e-3
    assert torch.allclose(s.cpu(), so, rtol=2e-2)


@pytest.mark.parametrize("pro", [PLAIN, SILU, GELU, GELU_TANH, SWIGLU, GATE])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_bit_exact_against_the_reference_kernel(pkg, ref, dev, pro, dtype):
    x = _x(130, 6144, 70 + pro, dtype).to(dev)
    gt = _x(130, 3072, 80 + pro, dtype).to(dev)
    kw = dict(K=3072)
    if pro == SWIGLU:
        kw["up_offset"] = 3072
    if pro == GATE:
        kw["g"] = gt
    for rot in (0, 1):
        q, s = pkg.linear.quant_rows(x, pro, rot, **kw)
        qr, sr = ref.quant_rows(x, pro, rot, **kw)
        assert_bits_equal(q, qr, f"codes pro={pro} rot={rot}")
        assert_bits_equal(s, sr, f"scales pro={pro} rot={rot}")


def test_golden_vectors(pkg, dev, golden_inputs, golden_reference):
    x = golden_inputs["x_bf16"].to(dev)
    L = pkg.linear
    for rot in (0, 1):
        q, s = L.quant_rows(x[:, :768].contiguous(), PLAIN, rot)
        assert_bits_equal(q, golden_reference[f"quant_plain_rot{rot}_q"], "golden codes")
        assert_bits_equal(s, golden_reference[f"quant_plain_rot{rot}_s"], "golden scales")
    for name, pro in (("silu", SILU), ("gelu", GELU), ("gelu_tanh", GELU_TANH)):
        q, s = L.quant_rows(x[:, :768].contiguous(), pro, 1)
        assert_bits_equal(q, golden_reference[f"quant_{name}_q"], name)
    q, s = L.quant_rows(x, SWIGLU, 1, K=768, up_offset=768)
    assert_bits_equal(q, golden_reference["quant_swiglu_q"], "swiglu")
    q, s = L.quant_rows(golden_inputs["x_f32"].to(dev), PLAIN, 1)
    assert_bits_equal(q, golden_reference["quant_f32_q"], "f32 rows")


def test_full_size_properties(pkg, dev):
    """Benchmark-size rows (M = 4352, K = 12288): properties that need no oracle pass."""
    x = _x(4352, 12288, 99).to(dev)
    q, s = pkg.linear.quant_rows(x, PLAIN, 0)
    amax = x.float().abs().amax(1)
    assert torch.equal(s, torch.clamp(amax * torch.tensor(1 / 127, device=dev), min=1e-30))
    qa = q.int().abs()
    assert int(qa.max()) >= 127 and bool((qa.amax(1) >= 126).all()), "every row uses the full int8 range"
    # the rotation preserves the row norm: dequantized rotated rows keep ||x|| within quantization noise
    q1, s1 = pkg.linear.quant_rows(x, PLAIN, 1)
    n0 = x.float().norm(dim=1)
    n1 = (q1.float() * s1[:, None]).norm(dim=1)
    assert torch.allclose(n0, n1, rtol=2e-2)
    # idempotence of the code grid: quantizing the dequantized codes returns the same codes
    xq = (q.float() * s[:, None].bfloat16().float()).bfloat16()
    q2, _ = pkg.linear.quant_rows(xq, PLAIN, 0)
    assert float((q2 != q).float().mean()) < 1e-3
    assert pkg.linear.kernel_status() == 0


def test_errors(pkg, dev):
    x = torch.zeros(4, 512, device=dev, dtype=torch.bfloat16)
    with pytest.raises(pkg.GpuKernelError, match="-3"):
        pkg.linear.quant_rows(x, 12, 0)         # LN_AFFINE_SILU: no quantizing entry point takes it
    with pytest.raises(pkg.GpuKernelError, match="-2"):
        pkg.linear.quant_rows(torch.zeros(1, 33024, device=dev, dtype=torch.bfloat16), 0, 0)
    q, s = pkg.linear.quant_rows(torch.zeros(0, 512, device=dev, dtype=torch.bfloat16), 0, 0)
    assert q.shape == (0, 512)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_every_row_length_the_reference_accepts(pkg, oracle, dev, dtype):
    """K = 256 n for n = 1 .. 128 (the reference takes every one of them, csrc/kernels.cu:261-268), a few rows each so
    that CTAs hold several rows, rows straddle warps and the last warp of a CTA is partial."""
    g = torch.Generator().manual_seed(4242)
    for n in range(1, 129):
        K, M = 256 * n, 5 if n < 64 else 2
        x = torch.randn(M, K, generator=g)
        x[:, torch.randperm(K, generator=g)[:3]] *= 25.0
        x = x.to(dtype)
        xd = x.to(dev)
        for rotate in (0, 1):
            q, s = pkg.linear.quant_rows(xd, PLAIN, rotate)
            qo, so = oracle.quant_rows(x, PLAIN, rotate)
            assert_bits_equal(s, so, f"scales K={K} rot={rotate}")
            assert_bits_equal(q, qo, f"codes K={K} rot={rotate}")
    assert pkg.linear.kernel_status() == 0


@pytest.mark.parametrize("n", [1, 3, 12, 33, 48, 66, 127])
def test_many_row_blocks_through_the_staging_buffer(pkg, oracle, dev, n):
    """Enough rows that every CTA walks several row blocks (bulk copies into the staging buffer, one block ahead), with a
    row stride larger than K and a ragged last block."""
    K = 256 * n
    M = 3001 if n <= 12 else 701
    g = torch.Generator().manual_seed(n)
    x = torch.randn(M, K + 256, generator=g).bfloat16()
    for rotate in (0, 1):
        q, s = pkg.linear.quant_rows(x.to(dev), PLAIN, rotate, K=K)
        qo, so = oracle.quant_rows(x, PLAIN, rotate, K=K)
        assert_bits_equal(s, so, f"scales rot={rotate}")
        assert_bits_equal(q, qo, f"codes rot={rotate}")
    assert pkg.linear.kernel_status() == 0


@pytest.mark.parametrize("pro", [SILU, GELU, GELU_TANH, SWIGLU, GATE])
def test_tabulated_prologues_bit_exact_against_the_reference_kernel(pkg, ref, dev, pro):
    """Rows of 2^20 elements and more take the one-variable activations from tables (the hot part in shared memory, the
    rest from the whole table). Inputs cover the table's whole domain: zeros, subnormals, tiny and huge magnitudes of both
    signs, infinities and NaN beside ordinary values."""
    M, K = 420, 3072
    g = torch.Generator().manual_seed(90 + pro)
    x = torch.randn(M, 2 * K, generator=g) * 2.0
    special = torch.tensor([0.0, -0.0, 1e-40, -1e-40, 1e-30, -1e-30, 6e-5, -6e-5, 3e-5, 127.0, 128.0, -128.0, 200.0, -200.0,
                            1e30, -1e30, 3.3e38, -3.3e38, float("inf"), float("-inf"), float("nan")])
    idx = torch.randint(0, M * 2 * K, (4000,), generator=g)
    x.view(-1)[idx] = special[torch.randint(0, len(special), (4000,), generator=g)]
    x[7] = 0.0                                  # a whole row outside the shared-memory part
    x[9, :K] = 1e-20
    x = x.bfloat16().to(dev)
    gt = (torch.randn(M, K, generator=g) * 3.0).bfloat16().to(dev)
    kw = dict(K=K)
    if pro == SWIGLU:
        kw["up_offset"] = K
    if pro == GATE:
        kw["g"] = gt
    for rot in (0, 1):
        q, s = pkg.linear.quant_rows(x, pro, rot, **kw)
        qr, sr = ref.quant_rows(x, pro, rot, **kw)
        assert_bits_equal(s, sr, f"scales pro={pro} rot={rot}")
        assert_bits_equal(q, qr, f"codes pro={pro} rot={rot}")
    assert pkg.linear.kernel_status() == 0


def test_every_bf16_value_through_the_tabulated_prologues(pkg, ref, dev):
    """All 65536 bf16 bit patterns, each as a one-hot row (so that its own code is +-127 or 0 and the scale exposes the
    activation's value), through SiLU / GELU / GELU-tanh with the tables in use: scales and codes equal the reference's."""
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    vals = bits.view(torch.bfloat16)
    x = torch.zeros(65536, 256, dtype=torch.bfloat16)
    x[:, 17] = vals
    x = x.to(dev)
    for pro in (SILU, GELU, GELU_TANH):
        q, s = pkg.linear.quant_rows(x, pro, 0)
        qr, sr = ref.quant_rows(x, pro, 0)
        assert_bits_equal(s, sr, f"scales pro={pro}")
        assert_bits_equal(q, qr, f"codes pro={pro}")


def test_misaligned_rows_are_refused(pkg, dev):
    x = torch.zeros(4, 520, device=dev, dtype=torch.bfloat16)
    with pytest.raises(pkg.GpuKernelError, match="-5"):
        pkg.linear.quant_rows(x[:, 4:], PLAIN, 0, K=512)          # rows start 8 bytes off a 16-byte boundary
