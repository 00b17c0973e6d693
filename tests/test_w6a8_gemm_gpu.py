"""GPU parity of the W6A8 linear that reads the packed weight (gpu_w6a8_gemm*): the reference's flow is gpu_w6_decode into
an int8 scratch copy followed by gpu_int8_gemm (src/h3.rs:1208-1216); the fused kernel must give the same int32 accumulators
and the same outputs bit for bit, for every 6-bit code and every e4m3 scale byte (zero, NaN, negative and saturating ones
included)."""
from __future__ import annotations

import pytest
import torch

from conftest import assert_bits_equal

pytestmark = pytest.mark.gpu


def _packed(oracle, N, K, seed, scales="any"):
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(0, 64, (N, K), generator=g, dtype=torch.uint8)
    if scales == "unit":
        s_rel = torch.full((N, K // 32), 0x38, dtype=torch.uint8)
    elif scales == "fitted":       # what the packer emits: e4m3 values in [2^-6, 4.1]
        s_rel = torch.randint(0x08, 0x49, (N, K // 32), generator=g, dtype=torch.uint8)
    else:                          # every byte value, NaN (0x7f, 0xff), zeros, negatives and 448 among them
        s_rel = torch.randint(0, 256, (N, K // 32), generator=g, dtype=torch.uint8)
    return g, oracle.w6_pack_codes(codes), s_rel


SHAPES = [(1, 8, 128), (5, 130, 256), (128, 256, 128), (300, 520, 384), (257, 1000, 1024), (513, 96, 2048), (64, 2080, 640)]


@pytest.mark.parametrize("scales", ["any", "unit", "fitted"])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_accumulators_equal_decode_then_gemm(pkg, oracle, dev, M, N, K, scales):
    g, packed, s_rel = _packed(oracle, N, K, M + N + K, scales)
    A = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
    w8 = oracle.w6_decode(packed, s_rel, K)
    got = pkg.linear.w6a8_gemm_acc_i32(A.to(dev), packed.to(dev), s_rel.to(dev))
    assert_bits_equal(got, oracle.int8_gemm_acc(A, w8), "accumulators")
    assert pkg.linear.kernel_status() == 0


def test_every_code_with_every_scale_byte(pkg, oracle, dev):
    """A one-hot A row picks single weights: 256 scale bytes x 64 codes, each seen as an accumulator of its own."""
    K, N = 128, 256 * 2
    codes = torch.arange(64, dtype=torch.uint8).repeat(N, 2)                  # [N, 128]: code = column % 64
    s_rel = (torch.arange(N, dtype=torch.int32) % 256).to(torch.uint8)[:, None].repeat(1, K // 32)
    packed = oracle.w6_pack_codes(codes)
    A = torch.zeros((128, K), dtype=torch.int8)
    A[torch.arange(128), torch.arange(128)] = 1
    got = pkg.linear.w6a8_gemm_acc_i32(A.to(dev), packed.to(dev), s_rel.to(dev))
    want = oracle.w6_decode(packed, s_rel, K).t().to(torch.int32).contiguous()   # [K, N]
    assert_bits_equal(got, want, "decoded weights")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_outputs_equal_the_two_call_flow(pkg, oracle, dev, dtype):
    M, N, K = 300, 520, 640
    g, packed, s_rel = _packed(oracle, N, K, 5, "fitted")
    A = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
    xs = torch.rand(M, generator=g) * 0.05 + 1e-3
    sc = torch.rand(N, generator=g) * 1e-3 + 1e-4
    bias = (torch.randn(N, generator=g) * 0.5).to(dtype)
    rs = torch.randn(N, generator=g).to(dtype)
    rr = torch.randn(M, N, generator=g).to(dtype)
    d = lambda t: t.to(dev)
    L = pkg.linear
    w8 = L.w6_decode(d(packed), d(s_rel), K)
    acc = oracle.int8_gemm_acc(A, oracle.w6_decode(packed, s_rel, K))
    got = L.w6a8_gemm(d(A), d(packed), d(s_rel), d(xs), d(sc), d(bias), out_dtype=dtype)
    assert_bits_equal(got, L.int8_gemm(d(A), w8, d(xs), d(sc), d(bias), out_dtype=dtype), "plain vs decode + gemm")
    assert_bits_equal(got, oracle.epilogue(acc, xs, sc, bias, out_dtype=dtype, contract=3), "plain vs oracle")
    got = L.w6a8_gemm(d(A), d(packed), d(s_rel), d(xs), d(sc), None, out_dtype=dtype, rscale=d(rs), resid=d(rr))
    assert_bits_equal(got, oracle.epilogue(acc, xs, sc, None, rs, rr, out_dtype=dtype, contract=3), "residual vs oracle")
    assert L.kernel_status() == 0


def test_full_size_layer_matches_decode_then_gemm(pkg, dev):
    """An FFN-up sized W6 layer (hidden 5120 -> 13824 on 2048 tokens): fused against the decoded copy, on the device."""
    from importlib import import_module
    wl = import_module(pkg.__name__ + ".workloads")
    M, N, K = 2048, 13824, 5120
    g = torch.Generator().manual_seed(3)
    w = torch.randn(N, K, generator=g) * 0.02
    packed, s_rel, s_channel = wl.w6_pack(w, True)
    A = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8).to(dev)
    xs = (torch.rand(M, generator=g) * 0.05 + 1e-3).to(dev)
    L = pkg.linear
    packed, s_rel, s_channel = packed.to(dev), s_rel.to(dev), s_channel.to(dev)
    got = L.w6a8_gemm(A, packed, s_rel, xs, s_channel, None)
    want = L.int8_gemm(A, L.w6_decode(packed, s_rel, K), xs, s_channel, None)
    assert_bits_equal(got, want, "full-size layer")
    assert L.kernel_status() == 0


@pytest.mark.parametrize("act", [1, 2, 3])
@pytest.mark.parametrize("M", [96, 1300])
def test_activation_epilogue_equals_the_int8_form(pkg, dev, act, M):
    """gpu_w6a8_gemm_act == gpu_w6_decode + gpu_int8_gemm_act, bit for bit, below and above the output size from which
    the activation comes from the table (1300 x 1024 outputs) and in both tile forms (up to / above 256 rows)."""
    from importlib import import_module
    wl = import_module(pkg.__name__ + ".workloads")
    N, K = 1024, 768
    g = torch.Generator().manual_seed(40 + act)
    packed, s_rel, s_channel = (t.to(dev) for t in wl.w6_pack(torch.randn(N, K, generator=g) * 0.02, True))
    A = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8).to(dev)
    xs = (torch.rand(M, generator=g) * 0.02 + 1e-3).to(dev)
    bias = (torch.randn(N, generator=g) * 0.5).bfloat16().to(dev)
    L = pkg.linear
    got = L.w6a8_gemm(A, packed, s_rel, xs, s_channel, bias, act=act)
    want = L.int8_gemm(A, L.w6_decode(packed, s_rel, K), xs, s_channel, bias, act=act)
    assert_bits_equal(got, want, f"act {act}")
    with pytest.raises(RuntimeError, match="-204"):
        L.w6a8_gemm(A, packed, s_rel, xs, s_channel, bias, act=7)
    assert L.kernel_status() == 0


def test_argument_checks(pkg, dev):
    L = pkg.linear
    A = torch.zeros((8, 192), dtype=torch.int8, device=dev)
    packed = torch.zeros((16, 144), dtype=torch.uint8, device=dev)
    s_rel = torch.zeros((16, 6), dtype=torch.uint8, device=dev)
    with pytest.raises(RuntimeError, match="-202"):
        L.w6a8_gemm_acc_i32(A, packed, s_rel)                      # K = 192 is not a multiple of 128
    A = torch.zeros((8, 256), dtype=torch.int8, device=dev)
    packed = torch.zeros((16, 192), dtype=torch.uint8, device=dev)
    with pytest.raises(RuntimeError, match="-206"):
        L.w6a8_gemm_acc_i32(A, packed, torch.zeros((16, 4), dtype=torch.uint8, device=dev), G=64)
