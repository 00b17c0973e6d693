"""CPU tests of the oracle itself: closed forms, round trips, and the committed golden vectors
(oracle.npz produced by the oracle, reference.npz produced by the reference's own CUDA kernels on a B200)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import as_np, assert_bits_equal

H4 = torch.tensor([[1, 1, 1, -1], [1, 1, -1, 1], [1, -1, 1, 1], [-1, 1, 1, 1]], dtype=torch.float64)


def _hadamard(stages: int) -> torch.Tensor:
    H = H4
    for _ in range(stages - 1):
        H = torch.kron(H, H4)
    return H / (2.0 ** stages)


@pytest.mark.parametrize("group,stages", [(256, 4), (64, 3)])
def test_rotation_is_the_kron_of_regular_hadamard_blocks(oracle, group, stages):
    # the matrix the reference's tools/te_q.py builds explicitly: kron(H4r, ..., H4r) / 2^stages
    x = torch.randint(-8, 9, (5, 2 * group)).float()   # small integers: every partial sum is exact
    y = oracle.fht_rows(x, group)
    want = (x.double().view(5, 2, group) @ _hadamard(stages).T).view(5, 2 * group)
    assert torch.equal(y.double(), want)
    assert torch.equal(oracle.fht_rows(y, group), x), "the rotation is its own inverse"


def test_quant_rows_matches_a_torch_restatement(oracle):
    torch.manual_seed(0)
    x = torch.randn(32, 3072).bfloat16()
    q, s = oracle.quant_rows(x, rotate=0)
    amax = x.float().abs().amax(1)
    scale = torch.clamp(amax * torch.tensor(1 / 127, dtype=torch.float32), min=1e-30)
    st = scale.bfloat16()
    want = torch.clamp(torch.round(x / st[:, None]), -128, 127).to(torch.int8)   # bf16 division, rounded to bf16
    assert torch.equal(s, scale) and torch.equal(q, want)


def test_quant_rows_edge_rows(oracle):
    x = torch.zeros(3, 256).bfloat16()
    x[1, 7] = float("inf")
    x[2, 9] = float("nan")
    q, s = oracle.quant_rows(x, rotate=0)
    assert s[0].item() == pytest.approx(1e-30) and int(q[0].abs().max()) == 0      # all-zero row: floor scale
    assert q[1, 7].item() == 127 and np.isfinite(s[1].item())                      # infinity caps at the bf16 max
    assert q[2, 9].item() == -128                                                  # NaN takes the fmaxf(lo, NaN) way


def test_error_codes(oracle):
    x = torch.zeros(2, 300).bfloat16()
    with pytest.raises(RuntimeError, match="-1"):
        oracle.quant_rows(x)                       # K % 256
    with pytest.raises(RuntimeError, match="-3"):
        oracle.quant_rows(torch.zeros(2, 256).bfloat16(), prologue=12)   # LN_AFFINE_SILU: not reachable through gpu_quant_rows
    with pytest.raises(RuntimeError, match="-1"):
        oracle.sd_quant_rows(torch.zeros(2, 100).half(), rotate=64)


def test_w6_pack_decode_round_trip(oracle, pkg):
    import importlib
    wl = importlib.import_module("cbr_b200.workloads")
    w = wl.weight(12, 512, 5, 0.015)
    packed, s_rel, s_ch = wl.w6_pack(w, fitted_groups=False)
    dec = oracle.w6_decode(packed, s_rel, 512)
    level = torch.clamp(torch.round(w / s_ch[:, None]), -31, 31).to(torch.int8)
    assert torch.equal(dec, level), "s_rel = 1.0 decodes to the 6-bit levels themselves"
    packed, s_rel, s_ch = wl.w6_pack(w, fitted_groups=True)
    dec = oracle.w6_decode(packed, s_rel, 512)
    assert (dec.float() * s_ch[:, None] - w).abs().max() < 0.06 * w.abs().max()
    # pack -> unpack of raw codes
    codes = torch.randint(1, 64, (4, 64)).to(torch.uint8)
    one = torch.full((4, 2), 0x38, dtype=torch.uint8)
    assert torch.equal(oracle.w6_decode(oracle.w6_pack_codes(codes), one, 64), (codes.int() - 32).to(torch.int8))


def test_int8_gemm_accumulators_and_linearity(oracle):
    g = torch.Generator().manual_seed(3)
    A = torch.randint(-128, 128, (37, 384), generator=g, dtype=torch.int8)
    B = torch.randint(-128, 128, (37, 384), generator=g, dtype=torch.int8) // 2
    W = torch.randint(-128, 128, (53, 384), generator=g, dtype=torch.int8)
    acc = oracle.int8_gemm_acc(A, W)
    assert torch.equal(acc, (A.double() @ W.double().T).to(torch.int32))
    A2 = (A // 2)
    assert torch.equal(oracle.int8_gemm_acc(A2, W) + oracle.int8_gemm_acc(B, W),
                       oracle.int8_gemm_acc((A2 + B).to(torch.int8), W)), "accumulation is linear in A"
    worst = oracle.int8_gemm_acc(torch.full((1, 32768), -128, dtype=torch.int8), torch.full((1, 32768), -128, dtype=torch.int8))
    assert worst.item() == 128 * 128 * 32768, "largest K the quantizer allows stays inside int32"


def test_convrot_requant_dequant_round_trip(oracle):
    w = torch.randn(6, 512) * 0.02
    q, s = oracle.convrot_requant(w, 0)
    back = oracle.convrot_dequant(q, s)
    assert (back - w).abs().max() <= 0.51 * s.max() * 16, "rotation spreads at most half a step per coordinate"
    q2, _ = oracle.convrot_requant(w, 777)
    assert int((q2.int() - q.int()).abs().max()) <= 1, "stochastic rounding moves a code by at most one step"


def test_oracle_reproduces_its_golden_file(oracle, golden_inputs, golden_oracle):
    import make_golden
    out = make_golden.run_cases(golden_inputs, make_golden.OracleBackend(), "cpu")
    assert set(out) == set(golden_oracle.files)
    for k, v in out.items():
        assert_bits_equal(v, golden_oracle[k], k)


# prologues that call expf/tanhf/erff: the host libm may differ from CUDA's in the last ulp, which can move a code by one
# normalising prologues: rsqrt.approx on the GPU against 1/sqrtf here (2 ulp), with the same effect
_LIBM = ("quant_silu", "quant_gelu", "quant_gelu_tanh", "quant_swiglu", "quant_gate", "quant_rms", "quant_layernorm",
         "quant_adaln", "quant_ln_", "quant_situ")


def test_oracle_matches_the_reference_run_on_b200(golden_oracle, golden_reference):
    """The pin: every output of the reference's own kernels on a B200 equals the CPU oracle's, bit for bit, except
    where a transcendental of the host libm is involved (at most one int8 step on at most 0.1 % of the codes)."""
    assert set(golden_reference.files) == set(golden_oracle.files)
    for k in golden_reference.files:
        r, o = golden_reference[k], golden_oracle[k]
        assert r.shape == o.shape, k
        if k.startswith(_LIBM):
            if k.endswith("_q"):
                d = np.abs(r.astype(np.int32) - o.astype(np.int32))
                assert d.max() <= 1 and (d != 0).mean() <= 2e-3, (k, int(d.max()), float((d != 0).mean()))
            else:
                assert np.allclose(r, o, rtol=2e-2), k      # a scale moves with the row maximum's bf16 step
        else:
            assert np.array_equal(r.view(np.uint8), o.view(np.uint8)), f"{k}: {(r != o).sum()} of {r.size} differ"
