"""GPU parity of the int8 GEMM and its fused epilogues (through the C ABI). int32 accumulators are bit-exact against
the CPU oracle; outputs are bit-exact against the oracle's fused-multiply-add form and against the reference's own
CUTLASS kernel where it is built. Where a different float form or a host libm is on the other side, the tolerance
is the path's stated one: one ulp of a 16-bit output (half an ulp of bf16 is a relative 4e-3), 1e-5 relative for f32."""
from __future__ import annotations

import pytest
import torch

from conftest import assert_bits_equal, assert_close_out

pytestmark = pytest.mark.gpu


def _operands(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    A = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
    W = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8)
    xs = torch.rand(M, generator=g) * 0.05 + 1e-3
    ws = torch.rand(N, generator=g) * 1e-3 + 1e-4
    return g, A, W, xs, ws


SHAPES = [(1, 8, 16), (1, 256, 256), (17, 40, 48), (127, 129, 144), (128, 256, 128), (129, 257 * 8, 272), (256, 512, 1024),
          (300, 520, 1024), (154, 640, 2048), (513, 1000, 80), (260, 96, 4096), (2048, 640, 640)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_int32_accumulators_bit_exact(pkg, oracle, dev, M, N, K):
    _, A, W, _, _ = _operands(M, N, K, M + N + K)
    acc = pkg.linear.int8_gemm_acc_i32(A.to(dev), W.to(dev))
    assert_bits_equal(acc, oracle.int8_gemm_acc(A, W), "accumulators")
    assert pkg.linear.kernel_status() == 0


def test_extreme_values_do_not_saturate(pkg, dev):
    K = 8192
    A = torch.full((130, K), -128, dtype=torch.int8, device=dev)
    W = torch.full((72, K), -128, dtype=torch.int8, device=dev)
    W[1] = 127
    acc = pkg.linear.int8_gemm_acc_i32(A, W)
    assert int(acc[0, 0]) == 128 * 128 * K and int(acc[5, 1]) == -128 * 127 * K


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(300, 520, 1024), (72, 88, 512), (640, 1284, 256)])
def test_epilogues_against_the_oracle(pkg, oracle, dev, dtype, M, N, K):
    g, A, W, xs, ws = _operands(M, N, K, 11)
    bias = (torch.randn(N, generator=g) * 0.5).to(dtype)
    rs = torch.randn(N, generator=g).to(dtype)
    rr = torch.randn(M, N, generator=g).to(dtype)
    acc = oracle.int8_gemm_acc(A, W)
    d = lambda t: t.to(dev)
    L = pkg.linear
    got = L.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias), out_dtype=dtype)
    want = oracle.epilogue(acc, xs, ws, bias, out_dtype=dtype, contract=3)
    assert_bits_equal(got, want, "plain")
    got = L.int8_gemm(d(A), d(W), d(xs), d(ws), None, out_dtype=dtype)
    assert_bits_equal(got, oracle.epilogue(acc, xs, ws, None, out_dtype=dtype, contract=3), "no bias")
    resid = d(rr).clone()
    got = L.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias), out_dtype=dtype, rscale=d(rs), resid=resid, out=resid)  # D aliases resid
    want = oracle.epilogue(acc, xs, ws, bias, rs, rr, out_dtype=dtype, contract=3)
    assert_bits_equal(got, want, "residual, in place")
    # the unfused float form differs by at most one ulp of the output type
    loose = oracle.epilogue(acc, xs, ws, bias, out_dtype=dtype, contract=0)
    assert_close_out(L.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias), out_dtype=dtype), loose, "unfused form")
    for act in (1, 2, 3):
        got = L.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias), out_dtype=dtype, act=act)
        assert_close_out(got, oracle.epilogue(acc, xs, ws, bias, out_dtype=dtype, act=act, contract=7), f"act {act}", tiny=1e-3)
    assert L.kernel_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_bit_exact_against_the_reference_gemm(pkg, ref, dev, dtype):
    # the last five take the one-CTA-per-tile kernel (small problems; 2048 x 1280 x 1280 by its second rule)
    for (M, N, K) in [(1024, 3072, 768), (8192, 640, 640), (300, 520, 1024), (154, 640, 2048), (2048, 1280, 1280), (128, 128, 128), (17, 40, 144)]:
        g, A, W, xs, ws = _operands(M, N, K, 21)
        A, W, xs, ws = A.to(dev), W.to(dev), xs.to(dev), ws.to(dev)
        bias = (torch.randn(N, generator=g) * 0.5).to(dtype).to(dev)
        rs = torch.randn(N, generator=g).to(dtype).to(dev)
        rr = torch.randn(M, N, generator=g).to(dtype).to(dev)
        assert_bits_equal(pkg.linear.int8_gemm(A, W, xs, ws, bias, out_dtype=dtype),
                          ref.int8_gemm(A, W, xs, ws, bias, out_dtype=dtype), f"plain {M}x{N}x{K}")
        assert_bits_equal(pkg.linear.int8_gemm(A, W, xs, ws, bias, out_dtype=dtype, rscale=rs, resid=rr),
                          ref.int8_gemm(A, W, xs, ws, bias, out_dtype=dtype, rscale=rs, resid=rr), f"residual {M}x{N}x{K}")


@pytest.mark.parametrize("act,pro", [(1, 11), (2, 5), (3, 6)])
def test_activation_epilogue_equals_the_reference_prologue_flow(pkg, ref, dev, act, pro):
    """epilogue-activation then a PLAIN quantizer == the reference's plain GEMM then its quantizer with that prologue."""
    g, A, W, xs, ws = _operands(256, 1024, 1024, 31)
    A, W, xs, ws = A.to(dev), W.to(dev), (xs * 0.3).to(dev), ws.to(dev)
    y = ref.int8_gemm(A, W, xs, ws, None)
    q_ref, s_ref = ref.quant_rows(y, pro, 1)
    ya = pkg.linear.int8_gemm(A, W, xs, ws, None, act=act)
    q, s = pkg.linear.quant_rows(ya, 0, 1)
    assert_bits_equal(q, q_ref, "codes")
    assert_bits_equal(s, s_ref, "scales")


@pytest.mark.parametrize("act", [1, 2, 3])
def test_tabulated_activation_epilogue_equals_the_computed_one(pkg, dev, act):
    """Outputs of 2^20 elements and more take the activation from the bf16 -> bf16 table; smaller ones compute it. The same
    rows must come out of both (row blocks of the large problem, run as problems of their own)."""
    g, A, W, xs, ws = _operands(1536, 1024, 512, 77)
    bias = (torch.randn(1024, generator=g) * 0.5).bfloat16().to(dev)
    A, W, xs, ws = A.to(dev), W.to(dev), (xs * 0.3).to(dev), ws.to(dev)
    big = pkg.linear.int8_gemm(A, W, xs, ws, bias, act=act)                      # 1.5 M outputs: table
    for r0 in (0, 512, 1024):
        part = pkg.linear.int8_gemm(A[r0:r0 + 512].contiguous(), W, xs[r0:r0 + 512].contiguous(), ws, bias, act=act)   # computed
        assert_bits_equal(big[r0:r0 + 512], part, f"rows {r0}..")


def test_golden_vectors(pkg, dev, golden_inputs, golden_reference):
    I = {k: v.to(dev) for k, v in golden_inputs.items()}
    for name, dt in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
        got = pkg.linear.int8_gemm(I["A"], I["W"], I["xs"], I["ws"], I[f"bias_{name}"], out_dtype=dt)
        assert_bits_equal(got, golden_reference[f"gemm_plain_{name}"], f"plain {name}")
        got = pkg.linear.int8_gemm(I["A"], I["W"], I["xs"], I["ws"], None, out_dtype=dt)
        assert_bits_equal(got, golden_reference[f"gemm_nobias_{name}"], f"nobias {name}")
        got = pkg.linear.int8_gemm(I["A"], I["W"], I["xs"], I["ws"], I[f"bias_{name}"], out_dtype=dt,
                                   rscale=I[f"rscale_{name}"], resid=I[f"resid_{name}"])
        assert_bits_equal(got, golden_reference[f"gemm_resid_{name}"], f"resid {name}")


def test_unaligned_output_takes_the_direct_store_path(pkg, oracle, dev):
    g, A, W, xs, ws = _operands(200, 100, 256, 41)      # N * 2 bytes is not a multiple of 16: no TMA store
    acc = oracle.int8_gemm_acc(A, W)
    got = pkg.linear.int8_gemm(A.to(dev), W.to(dev), xs.to(dev), ws.to(dev), None)
    assert_bits_equal(got, oracle.epilogue(acc, xs, ws, None, contract=3), "ragged N")
    # rows that are not a whole number of 8-byte pieces: the reference's "no configuration" code
    with pytest.raises(pkg.GpuKernelError, match="-200"):
        pkg.linear.int8_gemm(A[:, :250].contiguous().to(dev), W[:, :250].contiguous().to(dev), xs.to(dev), ws.to(dev), None)


@pytest.mark.parametrize("M,N,K", [(70, 96, 8), (129, 200, 24), (300, 520, 72), (64, 1000, 264), (513, 136, 1000)])
def test_rows_of_8_byte_pieces(pkg, oracle, ref, dev, M, N, K):
    """K a multiple of 8 but not of 16: the reference serves these with its narrow-alignment tile configurations; here a
    CUDA-core kernel does (TMA needs a 16-byte row pitch). Same bits as the oracle and as the reference's kernel."""
    g, A, W, xs, ws = _operands(M, N, K, 33)
    acc = oracle.int8_gemm_acc(A, W)
    d = lambda t: t.to(dev)
    L = pkg.linear
    assert_bits_equal(L.int8_gemm_acc_i32(d(A), d(W)), acc, "accumulators")
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        bias = (torch.randn(N, generator=g) * 0.5).to(dtype)
        rs = torch.randn(N, generator=g).to(dtype)
        rr = torch.randn(M, N, generator=g).to(dtype)
        got = L.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias), out_dtype=dtype)
        assert_bits_equal(got, oracle.epilogue(acc, xs, ws, bias, out_dtype=dtype, contract=3), f"plain {dtype}")
        resid = d(rr).clone()
        L.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias), out_dtype=dtype, rscale=d(rs), resid=resid, out=resid)
        assert_bits_equal(resid, oracle.epilogue(acc, xs, ws, bias, rs, rr, out_dtype=dtype, contract=3), f"residual {dtype}")
        if N % 8 == 0:      # the reference's kernels write 16-byte output vectors
            assert_bits_equal(got, ref.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias), out_dtype=dtype), f"reference kernel {dtype}")


def test_misaligned_operand_bases(pkg, oracle, dev):
    """A and W that start off a 16-byte boundary (views into larger buffers) take the same CUDA-core kernel."""
    g, A, W, xs, ws = _operands(100, 72, 256, 34)
    bufA = torch.zeros(100 * 256 + 8, dtype=torch.int8, device=dev)
    bufW = torch.zeros(72 * 256 + 8, dtype=torch.int8, device=dev)
    Ad = bufA[8:].view(100, 256); Ad.copy_(A)
    Wd = bufW[8:].view(72, 256); Wd.copy_(W)
    acc = oracle.int8_gemm_acc(A, W)
    assert_bits_equal(pkg.linear.int8_gemm_acc_i32(Ad, Wd), acc, "accumulators")
    assert_bits_equal(pkg.linear.int8_gemm(Ad, Wd, xs.to(dev), ws.to(dev), None), oracle.epilogue(acc, xs, ws, None, contract=3), "bf16 output")


def test_full_size_linearity_and_guard_bands(pkg, dev):
    """Benchmark-size shape (M=4352, K=3072, N=12288): accumulators are linear in A, and nothing is written outside D."""
    M, K, N = 4352, 3072, 12288
    g = torch.Generator(device=dev).manual_seed(5)
    A1 = torch.randint(-64, 64, (M, K), generator=g, dtype=torch.int8, device=dev)
    A2 = torch.randint(-63, 64, (M, K), generator=g, dtype=torch.int8, device=dev)
    W = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8, device=dev)
    L = pkg.linear
    s = L.int8_gemm_acc_i32(A1, W)
    s += L.int8_gemm_acc_i32(A2, W)
    assert torch.equal(s, L.int8_gemm_acc_i32(A1 + A2, W))
    rows = torch.randint(0, M, (64,), device=dev)
    want = (A1[rows].double() @ W.double().T + A2[rows].double() @ W.double().T).to(torch.int32)
    assert torch.equal(s[rows], want), "sampled rows against an fp64 product"
    # canary bands around the output
    pad = 4096
    buf = torch.full((M * N + 2 * pad,), -7.0, dtype=torch.bfloat16, device=dev)
    D = buf[pad:pad + M * N].view(M, N)
    xs = torch.rand(M, device=dev) * 1e-2
    ws = torch.rand(N, device=dev) * 1e-3
    L.int8_gemm(A1, W, xs, ws, None, out=D)
    assert bool((buf[:pad] == -7).all()) and bool((buf[-pad:] == -7).all())
    assert L.kernel_status() == 0


@pytest.mark.parametrize("M", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_few_rows_kernel(pkg, oracle, dev, M, dtype):
    """M <= 8 takes the weight-streaming kernel (adaLN modulation, pooled conditioning): same results, bit for bit."""
    N, K = 1003 if dtype == torch.float32 else 1000, 3072
    g, A, W, xs, ws = _operands(M, N, K, 51 + M)
    bias = (torch.randn(N, generator=g) * 0.5).to(dtype)
    rs = torch.randn(N, generator=g).to(dtype)
    rr = torch.randn(M, N, generator=g).to(dtype)
    acc = oracle.int8_gemm_acc(A, W)
    d = lambda t: t.to(dev)
    L = pkg.linear
    assert_bits_equal(L.int8_gemm_acc_i32(d(A), d(W)), acc, "accumulators")
    assert_bits_equal(L.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias), out_dtype=dtype),
                      oracle.epilogue(acc, xs, ws, bias, out_dtype=dtype, contract=3), "plain")
    assert_bits_equal(L.int8_gemm(d(A), d(W), d(xs), d(ws), None, out_dtype=dtype),
                      oracle.epilogue(acc, xs, ws, None, out_dtype=dtype, contract=3), "no bias")
    resid = d(rr).clone()
    L.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias), out_dtype=dtype, rscale=d(rs), resid=resid, out=resid)
    assert_bits_equal(resid, oracle.epilogue(acc, xs, ws, bias, rs, rr, out_dtype=dtype, contract=3), "residual in place")
    got = L.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias), out_dtype=dtype, act=1)
    assert_close_out(got, oracle.epilogue(acc, xs, ws, bias, out_dtype=dtype, act=1, contract=7), "gelu-tanh", tiny=1e-3)


def test_adaln_shape_matches_the_reference(pkg, ref, dev):
    g, A, W, xs, ws = _operands(1, 18432, 3072, 61)
    A, W, xs, ws = A.to(dev), W.to(dev), xs.to(dev), ws.to(dev)
    bias = torch.randn(18432, generator=g).bfloat16().to(dev)
    assert_bits_equal(pkg.linear.int8_gemm(A, W, xs, ws, bias), ref.int8_gemm(A, W, xs, ws, bias), "adaLN M=1")


@pytest.mark.parametrize("M,N,K", [(256, 512, 8192), (100, 384, 16384), (300, 96, 4096), (1000, 256, 6144)])
def test_k_split_problems(pkg, oracle, dev, M, N, K):
    """Few tiles and a long K: the tiles are cut along K and meet through atomic adds in global scratch. Two launches in
    a row also check that the first leaves the scratch (sums and counters) at zero."""
    g, A, W, xs, ws = _operands(M, N, K, 71)
    bias = (torch.randn(N, generator=g) * 0.5).bfloat16()
    acc = oracle.int8_gemm_acc(A, W)
    want = oracle.epilogue(acc, xs, ws, bias, contract=3)
    d = lambda t: t.to(dev)
    for _ in range(2):
        assert_bits_equal(pkg.linear.int8_gemm_acc_i32(d(A), d(W)), acc, "accumulators")
        assert_bits_equal(pkg.linear.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias)), want, "bf16 output")
    assert pkg.linear.kernel_status() == 0


def test_two_pass_quantizer_and_epilogue_only(pkg, oracle, dev):
    """The entry points of the tensor-parallel row-parallel linear: column halves quantized with the reduced row maxima
    equal the halves of the one-pass codes; the epilogue over summed int32 partials equals the fused one."""
    g = torch.Generator().manual_seed(81)
    x = torch.randn(96, 2048, generator=g).bfloat16().to(dev)
    L = pkg.linear
    q, s = L.quant_rows(x, 11, 1)
    halves = [x[:, :1024].contiguous(), x[:, 1024:].contiguous()]
    amax = torch.stack([L.quant_rows_amax(h, 11, 1) for h in halves]).amax(0)
    for i, h in enumerate(halves):
        qi, si = L.quant_rows_scaled(h, amax, 11, 1)
        assert_bits_equal(qi, q[:, 1024 * i:1024 * (i + 1)].contiguous(), f"codes of half {i}")
        assert_bits_equal(si, s, "scales")
    W = torch.randint(-128, 128, (320, 2048), generator=g, dtype=torch.int8).to(dev)
    ws = (torch.rand(320, generator=g) * 1e-3).to(dev)
    bias = torch.randn(320, generator=g).bfloat16().to(dev)
    rs = torch.randn(320, generator=g).bfloat16().to(dev)
    rr = torch.randn(96, 320, generator=g).bfloat16().to(dev)
    part = sum(L.int8_gemm_acc_i32(q[:, 1024 * i:1024 * (i + 1)].contiguous(), W[:, 1024 * i:1024 * (i + 1)].contiguous()) for i in range(2))
    assert_bits_equal(part, L.int8_gemm_acc_i32(q, W), "int32 partials sum to the whole")
    assert_bits_equal(L.int8_epilogue(part, s, ws, bias), L.int8_gemm(q, W, s, ws, bias), "plain")
    assert_bits_equal(L.int8_epilogue(part, s, ws, bias, rscale=rs, resid=rr), L.int8_gemm(q, W, s, ws, bias, rscale=rs, resid=rr), "residual")
    assert_bits_equal(L.int8_epilogue(part, s, ws, bias, act=1), L.int8_gemm(q, W, s, ws, bias, act=1), "gelu")


@pytest.mark.parametrize("M,N,K", [(2304, 2560, 1024), (4352, 4608, 2048), (2100, 9000, 1280), (5000, 3100, 3072)])
def test_many_rounds_with_a_ragged_last_one(pkg, oracle, dev, M, N, K):
    """More tiles than clusters, a last round that is only partly filled, ragged M and N: accumulators and every output
    form equal the oracle's, twice in a row, and a K-split problem (which uses the global scratch) runs right after."""
    g, A, W, xs, ws = _operands(M, N, K, 91)
    bias = (torch.randn(N, generator=g) * 0.5).bfloat16()
    rr = torch.randn(M, N, generator=g).bfloat16()
    rs = torch.randn(N, generator=g).bfloat16()
    acc = oracle.int8_gemm_acc(A, W)
    d = lambda t: t.to(dev)
    L = pkg.linear
    for _ in range(2):
        assert_bits_equal(L.int8_gemm_acc_i32(d(A), d(W)), acc, "accumulators")
        assert_bits_equal(L.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias)), oracle.epilogue(acc, xs, ws, bias, contract=3), "plain")
    resid = d(rr).clone()
    L.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias), rscale=d(rs), resid=resid, out=resid)
    assert_bits_equal(resid, oracle.epilogue(acc, xs, ws, bias, rs, rr, contract=3), "residual in place")
    got = L.int8_gemm(d(A), d(W), d(xs), d(ws), d(bias.float()), out_dtype=torch.float32)
    assert_bits_equal(got, oracle.epilogue(acc, xs, ws, bias.float(), out_dtype=torch.float32, contract=3), "f32 output")
    g2, A2, W2, xs2, ws2 = _operands(256, 512, 8192, 92)
    assert_bits_equal(L.int8_gemm_acc_i32(d(A2), d(W2)), oracle.int8_gemm_acc(A2, W2), "K-split problem after")
    assert L.kernel_status() == 0


def test_bias_residual_add_and_cluster_limit(pkg, oracle, dev):
    """The two tensor-parallel helpers: the bias + residual tail over reduced partial outputs (whole and by column blocks,
    in place), and GEMM launches restricted to part of the SMs (same results)."""
    g = torch.Generator().manual_seed(101)
    M, N = 130, 512
    L = pkg.linear
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        y = torch.randn(M, N, generator=g).to(dtype)
        bias = torch.randn(N, generator=g).to(dtype)
        resid = torch.randn(M, N, generator=g).to(dtype)
        want = ((y.float() + bias.float()).to(dtype).float() + resid.float()).to(dtype)
        got = L.bias_residual_add(y.to(dev), bias.to(dev), resid.to(dev))
        assert_bits_equal(got, want, f"whole {dtype}")
        out = resid.to(dev).clone()
        for c in range(4):                                   # column blocks of contiguous partial outputs, written in place
            L.bias_residual_add(y[:, 128 * c:128 * (c + 1)].contiguous().to(dev), bias.to(dev), out, out=out, n0=128 * c)
        assert_bits_equal(out, want, f"column blocks in place {dtype}")
        assert_bits_equal(L.bias_residual_add(y.to(dev), None, None), y, "nothing to add")
    g, A, W, xs, ws = _operands(2304, 2560, 1024, 102)
    acc = oracle.int8_gemm_acc(A, W)
    want = oracle.epilogue(acc, xs, ws, None, contract=3)
    d = lambda t: t.to(dev)
    try:
        assert L.set_gemm_cluster_limit(40) == 0
        assert_bits_equal(L.int8_gemm(d(A), d(W), d(xs), d(ws), None), want, "40 CTA pairs")
        assert L.set_gemm_cluster_limit(3) == 40
        assert_bits_equal(L.int8_gemm_acc_i32(d(A), d(W)), acc, "3 CTA pairs")
    finally:
        L.set_gemm_cluster_limit(0)
    assert L.kernel_status() == 0
