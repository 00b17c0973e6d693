"""GPU parity of the quantize-at-load packers, their inverses, the fp16 (SD) row quantizer and the W6 decode."""
from __future__ import annotations

import importlib

import pytest
import torch

from conftest import assert_bits_equal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,rot", [(50, 640, 0), (50, 640, 64), (30, 1280, 256), (20, 2048, 256), (9, 5120, 0), (7, 77, 0),
                                     (12, 320, 64), (3, 10240, 256), (1, 64, 64)])
def test_sd_quant_rows(pkg, oracle, dev, M, K, rot):
    g = torch.Generator().manual_seed(K + rot)
    x = (torch.randn(M, K, generator=g) * 0.02).half()
    x[0, 0] = 3.0                                     # an outlier
    q, s = pkg.linear.sd_quant_rows(x.to(dev), rot)
    qo, so = oracle.sd_quant_rows(x, rot)
    assert_bits_equal(q, qo, "codes")
    assert_bits_equal(s, so, "scales")


@pytest.mark.parametrize("rot", [0, 64, 256])
def test_sd_quant_rows_row_lengths_and_special_values(pkg, ref, dev, rot):
    """Every row length the register kernel takes for this rotation (K = 32 n, 64 n or 256 n up to 16384, longer rows and
    ragged K on the shared-memory kernel), several rows per CTA, with infinities, NaN, zeros, half's largest and smallest
    values sprinkled in: codes and scales equal the reference's kernel."""
    step = {0: 32, 64: 64, 256: 256}[rot]
    g = torch.Generator().manual_seed(rot + 5)
    special = torch.tensor([0.0, 65504.0, -65504.0, 6e-8, -6e-8, 1e-4, float("inf"), float("-inf"), float("nan")]).half()
    for K in list(range(step, 2561, step)) + [5120, 10240, 16384, 16384 + step]:
        M = 37 if K <= 2560 else 5
        x = (torch.randn(M, K + 8, generator=g) * 0.5).half()
        idx = torch.randint(0, M * (K + 8), (M,), generator=g)
        x.view(-1)[idx] = special[torch.randint(0, len(special), (M,), generator=g)]
        x[1] = 0
        xd = x.to(dev)[:, :K]                            # row stride K + 8
        q, s = pkg.linear.sd_quant_rows(xd, rot)
        qr, sr = ref.sd_quant_rows(xd, rot)
        assert_bits_equal(s, sr, f"scales K={K}")
        assert_bits_equal(q, qr, f"codes K={K}")


def test_sd_quant_rows_tiny_scale_and_stride(pkg, oracle, dev):
    x = torch.zeros(3, 256).half()
    x[1] = 6e-8           # scale below half's range: the division stays in float (csrc/sd.cu:592-593)
    x[2, 3] = 65504.0
    q, s = pkg.linear.sd_quant_rows(x.to(dev), 0)
    qo, so = oracle.sd_quant_rows(x, 0)
    assert_bits_equal(q, qo, "codes")
    assert_bits_equal(s, so, "scales")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("seed", [0, 12345, (7 << 32) + 99])
def test_convrot_requant_and_dequant(pkg, oracle, dev, dtype, seed):
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(48, 3072, generator=g) * 0.02).to(dtype)
    q, s = pkg.linear.convrot_requant(w.to(dev), seed)
    qo, so = oracle.convrot_requant(w, seed)
    assert_bits_equal(q, qo, "codes")
    assert_bits_equal(s, so, "scales")
    back = pkg.linear.convrot_dequant(q, s, dtype)
    assert_bits_equal(back, oracle.convrot_dequant(qo, so, dtype), "dequant")
    assert_bits_equal(pkg.linear.dequant_i8(q, s), oracle.dequant_i8(qo, so), "dequant_i8")
    assert_bits_equal(pkg.linear.embed_dequant(q, s), oracle.embed_dequant(qo, so), "embed_dequant")


def test_packers_against_the_reference_kernels(pkg, ref, dev):
    g = torch.Generator().manual_seed(10)
    for K, rot in ((640, 64), (1280, 256), (2560, 0)):
        x = (torch.randn(64, K, generator=g) * 0.02).half().to(dev)
        q, s = pkg.linear.sd_quant_rows(x, rot)
        qr, sr = ref.sd_quant_rows(x, rot)
        assert_bits_equal(q, qr, f"sd codes K={K}")
        assert_bits_equal(s, sr, f"sd scales K={K}")
    for dtype in (torch.float32, torch.bfloat16):
        w = (torch.randn(40, 12288, generator=g) * 0.02).to(dtype).to(dev)
        for seed in (0, 4242):
            q, s = pkg.linear.convrot_requant(w, seed)
            qr, sr = ref.convrot_requant(w, seed)
            assert_bits_equal(q, qr, "requant codes")
            assert_bits_equal(s, sr, "requant scales")
        assert_bits_equal(pkg.linear.convrot_dequant(q, s, dtype), ref.convrot_dequant(q, s, dtype), "dequant")
    # a weight packed by the reference's own W6 packer decodes identically
    w = (torch.randn(32, 2048, generator=g) * 0.015).bfloat16().to(dev)
    packed, s_rel, _ = ref.w6_requant(w, 3)
    assert_bits_equal(pkg.linear.w6_decode(packed, s_rel, 2048), ref.w6_decode(packed, s_rel, 2048), "w6 decode")


def test_w6_decode(pkg, oracle, dev):
    wl = importlib.import_module("cbr_b200.workloads")
    g = torch.Generator().manual_seed(12)
    codes = torch.randint(1, 64, (40, 1024), generator=g).to(torch.uint8)
    packed = oracle.w6_pack_codes(codes)
    s_rel = torch.randint(0x20, 0x50, (40, 32), generator=g).to(torch.uint8)   # e4m3 from 2^-3 to 8: some codes clamp
    got = pkg.linear.w6_decode(packed.to(dev), s_rel.to(dev), 1024)
    assert_bits_equal(got, oracle.w6_decode(packed, s_rel, 1024), "decode")
    w = wl.weight(24, 5120, 2031, 0.015)
    for fitted in (False, True):
        packed, s_rel, _ = wl.w6_pack(w, fitted)
        assert_bits_equal(pkg.linear.w6_decode(packed.to(dev), s_rel.to(dev), 5120), oracle.w6_decode(packed, s_rel, 5120),
                          f"decode fitted={fitted}")


def test_golden_vectors(pkg, dev, golden_inputs, golden_reference):
    import make_golden
    I, L = golden_inputs, pkg.linear
    for rot in (0, 64):
        q, s = L.sd_quant_rows(I["sd_x640"].to(dev), rot)
        assert_bits_equal(q, golden_reference[f"sd640_rot{rot}_q"], "sd codes")
        assert_bits_equal(s, golden_reference[f"sd640_rot{rot}_s"], "sd scales")
    for name in ("w_f32", "w_bf16"):
        for seed in (0, 12345):
            q, s = L.convrot_requant(I[name].to(dev), seed)
            assert_bits_equal(q, golden_reference[f"requant_{name}_seed{seed}_q"], f"requant {name} {seed}")
            assert_bits_equal(s, golden_reference[f"requant_{name}_seed{seed}_s"], f"requant scales {name} {seed}")
    got = L.w6_decode(make_golden.w6_pack_codes(I["w6_codes"]).to(dev), I["w6_srel"].to(dev), 512)
    assert_bits_equal(got, golden_reference["w6_decode"], "w6 decode")


def test_quantize_at_load_full_size_round_trip(pkg, dev):
    """A benchmark-size weight (12288 x 3072): requant -> dequant returns the weight within half a step per rotated
    coordinate, and packing the dequantized weight again reproduces the codes (idempotence)."""
    wl = importlib.import_module("cbr_b200.workloads")
    w = wl.weight(12288, 3072, 2011).to(dev)
    q, s = pkg.linear.convrot_requant(w, 0)
    back = pkg.linear.convrot_dequant(q, s, torch.float32)
    err = (pkg.linear.rotate_rows_f32(back) - pkg.linear.rotate_rows_f32(w)).abs()
    assert bool((err <= 0.5001 * s[:, None] + 1e-7).all())
    q2, s2 = pkg.linear.convrot_requant(back, 0)
    assert float((q2 != q).float().mean()) < 1e-4 and torch.allclose(s2, s, rtol=1e-5)


# ---- fp16 quantizer with a fused source stage (gpu_sd_{ln,geglu,unpad}_quant_rows) -------------------------------------
def _sd_src_case(mode, M, K, seed):
    g = torch.Generator().manual_seed(seed)
    if mode == "ln":
        x = (torch.randn(M, K, generator=g) * 2.0 + 0.5).half()
        return x, dict(w=torch.randn(K, generator=g) * 0.2 + 1.0, b=torch.randn(K, generator=g) * 0.1, eps=1e-5)
    if mode == "geglu":
        return (torch.randn(M, 2 * K, generator=g) * 1.5).half(), {}
    d = 64
    return torch.randn(M, K // d, d + 8, generator=g).half(), dict(d=d)


def _sd_src_run(L, mode, x, rotate, kw):
    if mode == "ln":
        return L.sd_ln_quant_rows(x, kw["w"], kw["b"], kw["eps"], rotate)
    if mode == "geglu":
        return L.sd_geglu_quant_rows(x, rotate)
    return L.sd_unpad_quant_rows(x, kw["d"], rotate)


@pytest.mark.parametrize("mode", ["ln", "geglu", "unpad"])
@pytest.mark.parametrize("M,K,rotate", [(9, 320, 64), (40, 640, 0), (33, 1280, 256), (12, 2560, 64), (3, 5120, 256)])
def test_sd_fused_source_quantizers(pkg, oracle, dev, mode, M, K, rotate):
    """Bit-exact against the reference's kernels where they are built; against the oracle exactly for the gather, within
    one step on a small fraction of codes where erff (GEGLU) or rsqrt (LayerNorm) differ between host and GPU."""
    x, kw = _sd_src_case(mode, M, K, 11 + K + M)
    dkw = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in kw.items()}
    q, s = _sd_src_run(pkg.linear, mode, x.to(dev), rotate, dkw)
    qo, so = oracle.sd_src_quant_rows(mode, x, rotate, **kw)
    if mode == "unpad":
        assert_bits_equal(q, qo, "codes"), assert_bits_equal(s, so, "scales")
    else:
        dlt = (q.cpu().int() - qo.int()).abs()
        assert int(dlt.max()) <= 1 and float((dlt != 0).float().mean()) <= 2e-3
        assert torch.allclose(s.cpu(), so, rtol=2e-3)
    from oracle import ref as R
    if R.available():
        qr, sr = R.sd_src_quant_rows(mode, x.to(dev), rotate, **dkw)
        assert_bits_equal(s, sr, "scales vs the reference kernel")
        assert_bits_equal(q, qr, "codes vs the reference kernel")


def test_sd_geglu_equals_the_two_kernel_flow(pkg, dev):
    """The fused form against value * gelu(gate) materialised in half and quantized by gpu_sd_quant_rows (full-size row)."""
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(512, 2 * 5120, generator=g) * 1.5).half().to(dev)
    q, s = pkg.linear.sd_geglu_quant_rows(x, 64)
    val = (x[:, :5120].float() * torch.nn.functional.gelu(x[:, 5120:].float()).half().float()).half()
    q2, s2 = pkg.linear.sd_quant_rows(val, 64)
    dlt = (q.int() - q2.int()).abs()      # torch's erf against CUDA's erff: last-ulp differences of the gate
    assert int(dlt.max()) <= 1 and float((dlt != 0).float().mean()) <= 2e-3


# ---- W6A8 packer (gpu_w6_requant) ------------------------------------------------------------------------------------
@pytest.mark.parametrize("N,K,seed", [(3, 256, 1), (20, 768, 3), (9, 5120, 0xDEADBEEF12345), (5, 13824, 7)])
def test_w6_requant_bit_exact(pkg, oracle, dev, N, K, seed):
    """Packed codes, e4m3 group scales and channel scales against the CPU oracle and, where built, the reference's kernel
    (every step is IEEE arithmetic in a fixed order, so all three agree bit for bit); decoding gives back the weight."""
    g = torch.Generator().manual_seed(N + K)
    w = (torch.randn(N, K, generator=g) * 0.02)
    w[:, ::97] *= 6.0                                        # a few outliers per row
    w = w.bfloat16()
    packed, s_rel, s_ch = pkg.linear.w6_requant(w.to(dev), seed)
    po, so, co = oracle.w6_requant(w, seed)
    assert_bits_equal(s_ch, co, "s_channel"), assert_bits_equal(s_rel, so, "s_rel"), assert_bits_equal(packed, po, "packed")
    from oracle import ref as R
    if R.available():
        pr, sr, cr = R.w6_requant(w.to(dev), seed)
        assert_bits_equal(s_ch, cr, "s_channel vs reference"), assert_bits_equal(s_rel, sr, "s_rel vs reference")
        assert_bits_equal(packed, pr, "packed vs reference")
    # round trip: decode to int8, undo the rotation, compare with the weight (6-bit steps: a few per cent of the row maximum)
    w8 = pkg.linear.w6_decode(packed, s_rel, K)
    back = pkg.linear.convrot_dequant(w8, s_ch, torch.float32).cpu()
    err = (back - w.float()).abs().amax(1) / w.float().abs().amax(1)
    assert float(err.max()) < 0.08, float(err.max())


def test_w6_requant_feeds_the_fused_gemm(pkg, dev):
    """Packer -> fused W6A8 GEMM equals packer -> decode -> int8 GEMM."""
    g = torch.Generator().manual_seed(4)
    w = (torch.randn(384, 1024, generator=g) * 0.02).bfloat16().to(dev)
    packed, s_rel, s_ch = pkg.linear.w6_requant(w, 11)
    A = torch.randint(-128, 128, (200, 1024), generator=g, dtype=torch.int8).to(dev)
    xs = (torch.rand(200, generator=g) * 0.05 + 1e-3).to(dev)
    got = pkg.linear.w6a8_gemm(A, packed, s_rel, xs, s_ch, None)
    want = pkg.linear.int8_gemm(A, pkg.linear.w6_decode(packed, s_rel, 1024), xs, s_ch, None)
    assert_bits_equal(got, want, "fused vs decoded")


@pytest.mark.parametrize("N,P,C,G,rotate", [(1, 64, 320, 32, 64), (2, 1024, 640, 32, 64), (1, 4096, 320, 32, 0), (2, 256, 1280, 32, 256)])
def test_sd_group_norm_quantizer(pkg, oracle, dev, N, P, C, G, rotate):
    """GroupNorm fused into the fp16 quantizer: bit-exact against the reference's pair of kernels where built; against the
    oracle the group statistics agree exactly (same float partial sums, double accumulation), so codes and scales do too."""
    g = torch.Generator().manual_seed(N + P + C)
    x = (torch.randn(N, P, C, generator=g) * 1.5 + 0.25).half()
    w = torch.randn(C, generator=g) * 0.2 + 1.0
    b = torch.randn(C, generator=g) * 0.1
    q, s = pkg.linear.sd_group_norm_quant_rows(x.to(dev), w.to(dev), b.to(dev), G, 1e-5, rotate)
    qo, so = oracle.sd_group_norm_quant_rows(x, w, b, G, 1e-5, rotate)
    assert_bits_equal(s, so, "scales vs oracle"), assert_bits_equal(q, qo, "codes vs oracle")
    from oracle import ref as R
    if R.available():
        qr, sr = R.sd_group_norm_quant_rows(x.to(dev), w.to(dev), b.to(dev), G, 1e-5, rotate)
        assert_bits_equal(s, sr, "scales vs the reference kernels"), assert_bits_equal(q, qr, "codes vs the reference kernels")


def test_argument_checks_of_the_packers_and_fused_quantizers(pkg, dev):
    L = pkg.linear
    with pytest.raises(RuntimeError, match="-1"):
        L.w6_requant(torch.zeros((4, 384), dtype=torch.bfloat16, device=dev))                  # K % 256
    x = torch.zeros((4, 640), dtype=torch.float16, device=dev)
    w = torch.ones(640, device=dev)
    with pytest.raises(RuntimeError, match="-1"):
        L.sd_ln_quant_rows(x, w, w, 1e-5, 256)                                                 # 640 % 256
    with pytest.raises(RuntimeError, match="-1"):
        L.sd_geglu_quant_rows(x, 128)                                                          # rotate must be 0, 64 or 256
    with pytest.raises(RuntimeError, match="-1"):
        L.sd_group_norm_quant_rows(x.view(1, 4, 640), w, w, 48, 1e-5, 0)                       # 640 % 48
    q, s = L.sd_unpad_quant_rows(torch.zeros((0, 10, 72), dtype=torch.float16, device=dev), 64, 64)   # no rows: nothing to do
    assert q.shape == (0, 640)
