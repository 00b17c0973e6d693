"""Every linear of the five benchmark configurations at its full size, these kernels against the reference's own CUDA
kernels (oracle/_ref/libref.so, built from the reference tree) on the same device buffers and the same seeded inputs.

Per linear: the activation quantizer's codes and scales, the packed / quantized weight, the GEMM output with bias
(and the residual form where the configuration has one) must be bit-identical; the int32 accumulators are checked
against an integer product (torch._int_mm, a library routine used here as a checker only); where the configuration has
a GELU epilogue, "activation epilogue then PLAIN quantizer" and "activation + rotation epilogue then the quantizer's second
pass" must both give the codes of the reference's "plain GEMM then GELU-tanh prologue quantizer". W6A8 linears are compared with the reference's decode followed by its int8 GEMM.
The first configuration additionally runs against the CPU oracle in full."""
from __future__ import annotations

import pytest
import torch

from conftest import assert_bits_equal

pytestmark = pytest.mark.gpu


def _specs(pkg):
    import importlib
    wl = importlib.import_module("cbr_b200.workloads")
    out = []
    for ci in range(5):
        for sp in wl.config(ci) + (wl.config(2, 6144) if ci == 2 else []):
            out.append((ci, sp))
    return wl, out


def _ids():
    # the names are fixed by workloads.config; listed here so that collection needs no package import
    names = ["c0-w8a8-4096"]
    names += [f"c1-{n}-4352" for n in ("mlp_up", "mlp_down")]
    names += [f"c2-{n}-{m}" for m in (2048, 6144) for n in ("qkv", "out", "ffn_up", "ffn_down")]
    names += [f"c3-{n}" for n in ("sa_qkv_640", "sa_out_640", "sa_qkv_1280", "sa_out_1280", "ca_q_640", "ca_q_1280", "ca_kv_640",
                                  "ca_kv_1280", "geglu_640", "geglu_1280", "ff2_640", "ff2_1280")]
    names += [f"c4-{n}" for n in ("qkv", "attn_out", "mlp_up", "mlp_down", "adaln")]
    return names


IDS = _ids()


def _int_product(A, W):
    """Exact int32 product on the device: torch._int_mm where its shape rules allow, else an fp64 product by row blocks."""
    M, K = A.shape
    N = W.shape[0]
    if M > 16 and K % 8 == 0 and N % 8 == 0:
        try:
            return torch._int_mm(A, W.t())
        except RuntimeError:
            pass
    Wd = W.double().t()
    return torch.cat([(A[r:r + 2048].double() @ Wd).to(torch.int32) for r in range(0, M, 2048)])


@pytest.mark.parametrize("index", range(len(IDS)), ids=IDS)
def test_linear_bit_exact_against_the_reference_kernels(pkg, ref, dev, index):
    wl, specs = _specs(pkg)
    assert len(specs) == len(IDS)
    ci, sp = specs[index]
    L = pkg.linear
    M, K, N, dt = sp.M, sp.K, sp.N, sp.act_dtype
    seed = 100 * ci + index
    x = wl.activations(M, K, 1000 + seed, outliers="student" if ci in (1,) else ("none" if ci in (2, 3) else "x20"), dtype=dt).to(dev)
    bias = wl.bias(N, 3000 + seed, dtype=dt).to(dev)

    # ---- activation side
    if dt == torch.float16:
        a8, xs = L.sd_quant_rows(x, sp.rotate)
        a8r, xsr = ref.sd_quant_rows(x, sp.rotate)
    else:
        a8, xs = L.quant_rows(x, 0, 1 if sp.rotate else 0)
        a8r, xsr = ref.quant_rows(x, 0, 1 if sp.rotate else 0)
    assert_bits_equal(xs, xsr, "activation scales")
    assert_bits_equal(a8, a8r, "activation codes")

    # ---- weight side
    if sp.weight_format == "w6":
        w = wl.weight(N, K, 2000 + seed, 0.015)
        packed, s_rel, s_ch = (t.to(dev) for t in wl.w6_pack(w, fitted_groups=(index % 2 == 0)))
        wq_ref = ref.w6_decode(packed, s_rel, K)
        assert_bits_equal(L.w6_decode(packed, s_rel, K), wq_ref, "decoded W6 weight")
        wq, ws = wq_ref, s_ch
    elif dt == torch.float16:
        w = wl.weight(N, K, 2000 + seed, 0.02, dtype=torch.float16).to(dev)
        wq, ws = L.sd_quant_rows(w, sp.rotate)                       # quantize-at-load, src/unet.rs:367-383
        wqr, wsr = ref.sd_quant_rows(w, sp.rotate)
        assert_bits_equal(wq, wqr, "weight codes")
        assert_bits_equal(ws, wsr, "weight scales")
    elif sp.rotate:
        w = wl.weight(N, K, 2000 + seed, 0.02).to(dev)
        wq, ws = L.convrot_requant(w, 0)
        wqr, wsr = ref.convrot_requant(w, 0)
        assert_bits_equal(wq, wqr, "weight codes")
        assert_bits_equal(ws, wsr, "weight scales")
    else:                                                             # configuration 0: fp16 weights, no rotation
        w = wl.weight(N, K, 2000 + seed, 0.02, dtype=torch.float16).to(dev)
        wq, ws = L.sd_quant_rows(w, 0)
        wqr, wsr = ref.sd_quant_rows(w, 0)
        assert_bits_equal(wq, wqr, "weight codes")
        assert_bits_equal(ws, wsr, "weight scales")

    # ---- int32 accumulators
    acc = L.int8_gemm_acc_i32(a8, wq)
    want = _int_product(a8, wq)
    assert torch.equal(acc, want), "int32 accumulators"
    del want

    # ---- fused epilogues
    y_ref = ref.int8_gemm(a8, wq, xs, ws, bias, out_dtype=dt)
    y = L.int8_gemm(a8, wq, xs, ws, bias, out_dtype=dt)
    assert_bits_equal(y, y_ref, "GEMM + bias")
    if sp.weight_format == "w6":
        assert torch.equal(L.w6a8_gemm_acc_i32(a8, packed, s_rel), acc), "W6A8 accumulators from the packed weight"
        assert_bits_equal(L.w6a8_gemm(a8, packed, s_rel, xs, ws, bias, out_dtype=dt), y_ref, "W6A8 GEMM from the packed weight")
    del acc
    if sp.epilogue == "residual":
        resid = wl.activations(M, N, 4000 + seed, outliers="none", dtype=dt).to(dev)
        ones = torch.ones(N, dtype=dt, device=dev)
        want = ref.int8_gemm(a8, wq, xs, ws, bias, out_dtype=dt, rscale=ones, resid=resid)
        got = resid.clone()
        L.int8_gemm(a8, wq, xs, ws, bias, out_dtype=dt, rscale=ones, resid=got, out=got)     # in place, as every caller does
        assert_bits_equal(got, want, "residual form, D aliasing resid")
    if sp.epilogue == "gelu_tanh" and dt == torch.bfloat16:
        ya = L.int8_gemm(a8, wq, xs, ws, bias, out_dtype=dt, act=1)
        q2, s2 = L.quant_rows(ya, 0, 1 if sp.rotate else 0)
        q2r, s2r = ref.quant_rows(y_ref, 11, 1 if sp.rotate else 0)
        assert_bits_equal(s2, s2r, "scales after the GELU epilogue")
        assert_bits_equal(q2, q2r, "codes after the GELU epilogue")
        if sp.weight_format == "w6":
            assert_bits_equal(L.w6a8_gemm(a8, packed, s_rel, xs, ws, bias, out_dtype=dt, act=1), ya, "W6A8 GEMM with the GELU epilogue")
        if sp.rotate and N % 256 == 0:
            # activation and rotation in the GEMM's epilogue, the quantizer's second pass after it
            rows, parts = L.int8_gemm_act_rot(a8, wq, xs, ws, bias, act=1)
            q4, s4 = L.quant_rows_rotated(rows, parts)
            assert_bits_equal(s4, s2r, "scales after the rotating epilogue")
            assert_bits_equal(q4, q2r, "codes after the rotating epilogue")
            del rows, parts, q4
        q3, s3 = L.quant_rows(y, 11, 1 if sp.rotate else 0)                                    # and the prologue form itself
        assert_bits_equal(q3, q2r, "codes of the GELU-tanh prologue")
        assert_bits_equal(s3, s2r, "scales of the GELU-tanh prologue")
    assert L.kernel_status() == 0


def test_first_configuration_against_the_cpu_oracle(pkg, oracle, dev):
    """Single W8A8 linear 4096 x 3072 x 3072 in full: quantizer, fp16 weight packer, accumulators and bf16 output."""
    import importlib
    wl = importlib.import_module("cbr_b200.workloads")
    sp = wl.config(0)[0]
    x = wl.activations(sp.M, sp.K, 1001)
    w = wl.weight(sp.N, sp.K, 2001, 0.02, dtype=torch.float16)
    bias = wl.bias(sp.N, 3001)
    L = pkg.linear
    a8, xs = L.quant_rows(x.to(dev), 0, 0)
    wq, ws = L.sd_quant_rows(w.to(dev), 0)
    a8o, xso = oracle.quant_rows(x, 0, 0)
    wqo, wso = oracle.sd_quant_rows(w, 0)
    assert_bits_equal(a8, a8o, "activation codes")
    assert_bits_equal(xs, xso, "activation scales")
    assert_bits_equal(wq, wqo, "weight codes")
    assert_bits_equal(ws, wso, "weight scales")
    acco = oracle.int8_gemm_acc(a8o, wqo)
    assert_bits_equal(L.int8_gemm_acc_i32(a8, wq), acco, "accumulators")
    assert_bits_equal(L.int8_gemm(a8, wq, xs, ws, bias.to(dev)), oracle.epilogue(acco, xso, wso, bias, contract=3), "bf16 output")
