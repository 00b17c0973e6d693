"""GPU parity of the quantizer's normalising prologues (RMS, LAYERNORM, ADALN, LN_MOD, LN_AFFINE) and of the SITU
activation, through the C ABI.

Against the reference's own kernel (where built) the codes and scales must be bit-identical: the row sums are added in
the reference's order and the same rsqrt / expf / expm1f instructions run on the same GPU. Against the CPU oracle the
sums are the same too, but its 1/sqrtf and host libm differ from the GPU's rsqrt.approx (2 ulp) and libm in the last
bits: at most one int8 step on a small fraction of codes, scales within 2^-20 relative."""
from __future__ import annotations

import pytest
import torch

from conftest import assert_bits_equal

pytestmark = pytest.mark.gpu
RMS, LAYERNORM, ADALN, SITU, LN_MOD, LN_AFFINE, SITU_FAST = 1, 4, 7, 8, 9, 10, 13


def _case(M, K, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g) * 1.7 + 0.3
    x[:, torch.randperm(K, generator=g)[: max(1, K // 100)]] *= 15.0
    return dict(x=x.to(dtype), norm_w=(torch.randn(K, generator=g) * 0.2 + 1.0), norm_b=torch.randn(K, generator=g) * 0.1,
                mod_scale=(torch.randn(K, generator=g) * 0.3).to(dtype), mod_shift=(torch.randn(K, generator=g) * 0.5).to(dtype))


def _kwargs(pro, c, variant):
    kw = dict(eps=1e-6)
    if pro in (RMS, LAYERNORM):
        if variant & 1:
            kw["norm_w"] = c["norm_w"]
        if variant & 2:
            kw.update(mod_scale=c["mod_scale"], mod_shift=c["mod_shift"])
    elif pro == ADALN:
        kw.update(mod_scale=c["mod_scale"], mod_shift=c["mod_shift"])
    elif pro == LN_MOD:
        if variant & 2:
            kw.update(mod_scale=c["mod_scale"], mod_shift=c["mod_shift"])
    elif pro == LN_AFFINE:
        kw.update(norm_w=c["norm_w"], norm_b=c["norm_b"])
    return kw


def _to(dev, kw):
    return {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in kw.items()}


CASES = [(RMS, 0), (RMS, 1), (RMS, 2), (RMS, 3), (LAYERNORM, 0), (LAYERNORM, 1), (LAYERNORM, 2), (LAYERNORM, 3), (ADALN, 0), (LN_MOD, 0), (LN_MOD, 2), (LN_AFFINE, 0)]
# K / 256 groups: 1 (one reference warp), 5 and 12 (ragged last round), 16, 20 (five warps), 128 (the 32-warp limit)
SHAPES = [(7, 256), (33, 1280), (130, 3072), (64, 4096), (40, 5120), (3, 32768)]


@pytest.mark.parametrize("pro,variant", CASES)
@pytest.mark.parametrize("M,K", SHAPES)
def test_norm_prologues_bit_exact_against_the_reference_kernel(pkg, ref, dev, pro, variant, M, K):
    for dtype in ([torch.bfloat16] if pro == LN_AFFINE else [torch.bfloat16, torch.float32]):
        c = _case(M, K, 31 * pro + variant + K, dtype)
        kw = _to(dev, _kwargs(pro, c, variant))
        for rotate in (0, 1):
            q, s = pkg.linear.quant_rows(c["x"].to(dev), pro, rotate, **kw)
            qr, sr = ref.quant_rows(c["x"].to(dev), pro, rotate, **kw)
            assert_bits_equal(s, sr, f"scales {dtype} rot={rotate}")
            assert_bits_equal(q, qr, f"codes {dtype} rot={rotate}")


@pytest.mark.parametrize("pro,variant", CASES)
def test_norm_prologues_against_the_oracle(pkg, oracle, dev, pro, variant):
    M, K = 48, 3072
    c = _case(M, K, 77 + pro + variant)
    kw = _kwargs(pro, c, variant)
    q, s = pkg.linear.quant_rows(c["x"].to(dev), pro, 1, **_to(dev, kw))
    qo, so = oracle.quant_rows(c["x"], pro, 1, **kw)
    d = (q.cpu().int() - qo.int()).abs()
    assert int(d.max()) <= 1 and float((d != 0).float().mean()) <= 2e-3, (int(d.max()), float((d != 0).float().mean()))
    assert torch.allclose(s.cpu(), so, rtol=2e-2)     # one bf16 step of a normalised value can move the row maximum


@pytest.mark.parametrize("pro", [SITU, SITU_FAST])
def test_situ_against_reference_and_oracle(pkg, oracle, dev, pro, request):
    M, K = 70, 2048
    g = torch.Generator().manual_seed(5 + pro)
    x = (torch.randn(M, 2 * K, generator=g) * 3.0).bfloat16()
    q, s = pkg.linear.quant_rows(x.to(dev), pro, 1, K=K, up_offset=K)
    qo, so = oracle.quant_rows(x, pro, 1, K=K, up_offset=K)
    d = (q.cpu().int() - qo.int()).abs()
    lim = 1 if pro == SITU else 2                      # the fast form's hardware tanh / exp: about 2^-11 relative
    assert int(d.max()) <= lim and float((d != 0).float().mean()) <= (2e-3 if pro == SITU else 0.2)
    assert torch.allclose(s.cpu(), so, rtol=2e-2 if pro == SITU else 5e-2)
    from oracle import ref as R
    if R.available():
        qr, sr = R.quant_rows(x.to(dev), pro, 1, K=K, up_offset=K)
        assert_bits_equal(s, sr, "scales vs reference kernel")
        assert_bits_equal(q, qr, "codes vs reference kernel")


def test_golden_vectors(pkg, dev, golden_inputs, golden_reference):
    """Outputs of the reference's kernels on a B200, committed: the same bits must come out here."""
    import make_golden
    x = golden_inputs["x_bf16"].to(dev)
    for name, (pro, K, kw) in make_golden.norm_cases(golden_inputs, lambda t: t.to(dev)).items():
        rows = x if (K == 1536 or pro == "situ") else x[:, :768].contiguous()
        q, s = pkg.linear.quant_rows(rows, make_golden.PRO[pro], 1, K=K, **kw)
        assert_bits_equal(s, golden_reference[f"{name}_s"], f"{name} scales")
        assert_bits_equal(q, golden_reference[f"{name}_q"], f"{name} codes")


def test_rotate_rows_f32_rms_against_reference(pkg, ref, dev):
    c = _case(21, 2048, 9, torch.float32)
    got = pkg.linear.rotate_rows_f32(c["x"].to(dev), RMS, norm_w=c["norm_w"].to(dev), eps=1e-6)
    want = ref.rotate_rows_f32(c["x"].to(dev), RMS, norm_w=c["norm_w"].to(dev), eps=1e-6)
    assert_bits_equal(got, want, "rotated rows")


def test_error_codes(pkg, dev):
    x = torch.zeros((4, 512), dtype=torch.bfloat16, device=dev)
    w = torch.ones(512, device=dev)
    with pytest.raises(RuntimeError, match="-3"):
        pkg.linear.quant_rows(x, ADALN, 1)                      # ADALN without its modulation vectors
    with pytest.raises(RuntimeError, match="-3"):
        pkg.linear.quant_rows(x, LN_AFFINE, 1, norm_w=w)        # LN_AFFINE needs the bias: gpu_quant_rows_b
    with pytest.raises(RuntimeError, match="-3"):
        pkg.linear.quant_rows(x, RMS, 1, norm_w=w, norm_b=w)    # gpu_quant_rows_b takes LN_MOD and LN_AFFINE only
    with pytest.raises(RuntimeError, match="-4"):
        pkg.linear.quant_rows(x.float(), LN_AFFINE, 1, norm_w=w, norm_b=w)


@pytest.mark.parametrize("pro,variant", [(RMS, 2), (RMS, 3), (LAYERNORM, 3)])
def test_f32_rows_with_modulation_for_every_row_length(pkg, ref, dev, pro, variant):
    """f32 rows with modulation: where nothing rounds between a * n and + shift the reference's build decides whether the
    two fuse, and for RMS it depends on which of the four groups of a reference warp an element belongs to. Every
    K = 256 n, n = 1 .. 128, against the reference's kernel."""
    for n in range(1, 129):
        K, M = 256 * n, 3 if n < 64 else 2
        c = _case(M, K, 1000 + n, torch.float32)
        kw = _to(dev, _kwargs(pro, c, variant))
        for rotate in (0, 1):
            q, s = pkg.linear.quant_rows(c["x"].to(dev), pro, rotate, **kw)
            qr, sr = ref.quant_rows(c["x"].to(dev), pro, rotate, **kw)
            assert_bits_equal(s, sr, f"scales K={K} rot={rotate}")
            assert_bits_equal(q, qr, f"codes K={K} rot={rotate}")


@pytest.mark.parametrize("pro,variant", [(RMS, 3), (LN_MOD, 2), (ADALN, 0), (LN_AFFINE, 0)])
def test_bf16_norm_prologues_for_every_row_length(pkg, ref, dev, pro, variant):
    for n in list(range(1, 40)) + [47, 54, 64, 66, 97, 128]:
        K, M = 256 * n, 3
        c = _case(M, K, 2000 + n)
        kw = _to(dev, _kwargs(pro, c, variant))
        q, s = pkg.linear.quant_rows(c["x"].to(dev), pro, 1, **kw)
        qr, sr = ref.quant_rows(c["x"].to(dev), pro, 1, **kw)
        assert_bits_equal(s, sr, f"scales K={K}")
        assert_bits_equal(q, qr, f"codes K={K}")
