"""Generates the golden fixtures of the parity tests.

    python tests/golden/make_golden.py inputs                  # seeded inputs            -> tests/golden/inputs.npz
    python tests/golden/make_golden.py oracle                  # CPU oracle outputs       -> tests/golden/oracle.npz
    python tests/golden/make_golden.py reference OUT.npz       # the reference's own CUDA kernels (oracle/_ref/libref.so,
                                                               # built by oracle/build_ref.sh) run on a B200

The committed ``reference.npz`` was produced by the third form on a B200 and is what pins the CPU oracle: the
reference's own tests hold no vector for this path, so outputs of the reference itself are the anchor.
All three read the same ``inputs.npz``. 16-bit floats are stored as their uint16 bit patterns.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

BITS = {torch.bfloat16: torch.int16, torch.float16: torch.int16}
PRO = {"plain": 0, "rms": 1, "gate": 2, "swiglu": 3, "layernorm": 4, "silu": 5, "gelu": 6, "adaln": 7, "situ": 8, "ln_mod": 9,
       "ln_affine": 10, "gelu_tanh": 11}
EPS = 1e-6


def norm_cases(I: dict, mv) -> dict:
    """name -> (prologue, K, keyword arguments) of the normalising / SITU quantizer cases; rows are x_bf16[:, :K]."""
    w, b, ms, sh = mv(I["norm_w_f32"]), mv(I["norm_b_f32"]), mv(I["mod_scale_bf16"]), mv(I["mod_shift_bf16"])
    c = lambda t, K: t[:K].contiguous()
    return {
        "quant_rms_w": ("rms", 768, dict(norm_w=c(w, 768), eps=EPS)),
        "quant_rms_w_mod_k1536": ("rms", 1536, dict(norm_w=w, mod_scale=ms, mod_shift=sh, eps=EPS)),
        "quant_layernorm_w_mod": ("layernorm", 768, dict(norm_w=c(w, 768), mod_scale=c(ms, 768), mod_shift=c(sh, 768), eps=EPS)),
        "quant_layernorm_k1536": ("layernorm", 1536, dict(eps=EPS)),
        "quant_adaln": ("adaln", 768, dict(mod_scale=c(ms, 768), mod_shift=c(sh, 768), eps=EPS)),
        "quant_ln_mod_k1536": ("ln_mod", 1536, dict(mod_scale=ms, mod_shift=sh, eps=EPS)),
        "quant_ln_affine": ("ln_affine", 768, dict(norm_w=c(w, 768), norm_b=c(b, 768), eps=EPS)),
        "quant_situ": ("situ", 768, dict(up_offset=768)),
    }


def to_np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype in BITS:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def from_np(a: np.ndarray, dtype=None) -> torch.Tensor:
    if dtype in BITS:
        return torch.from_numpy(a.view(np.int16).copy()).view(dtype)
    return torch.from_numpy(a.copy())


def make_inputs() -> dict:
    g = torch.Generator().manual_seed(20240607)
    d = {}
    x = torch.randn(16, 1536, generator=g)
    x[:, torch.randperm(1536, generator=g)[:15]] *= 20.0
    d["x_bf16"] = x.bfloat16()                       # quantizer rows; SWIGLU reads [gate | up] halves of 768
    d["gate_bf16"] = torch.randn(16, 768, generator=g).bfloat16()
    d["x_f32"] = torch.randn(8, 512, generator=g) * 3.0
    d["sd_x640"] = (torch.randn(12, 640, generator=g)).half()
    d["sd_x1280"] = (torch.randn(6, 1280, generator=g) * 0.02).half()
    d["w_f32"] = torch.randn(10, 768, generator=g) * 0.02
    d["w_bf16"] = (torch.randn(10, 768, generator=g) * 0.02).bfloat16()
    d["w6_codes"] = torch.randint(1, 64, (10, 512), generator=g).to(torch.uint8)
    d["w6_srel"] = torch.randint(0x28, 0x40, (10, 16), generator=g).to(torch.uint8)
    d["A"] = torch.randint(-128, 128, (72, 512), generator=g, dtype=torch.int8)
    d["W"] = torch.randint(-128, 128, (88, 512), generator=g, dtype=torch.int8)
    d["xs"] = torch.rand(72, generator=g) * 0.05 + 1e-3
    d["ws"] = torch.rand(88, generator=g) * 1e-3 + 1e-4
    for name, dt in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
        d[f"bias_{name}"] = (torch.randn(88, generator=g) * 0.5).to(dt)
        d[f"rscale_{name}"] = torch.randn(88, generator=g).to(dt)
        d[f"resid_{name}"] = torch.randn(72, 88, generator=g).to(dt)
    # per-column vectors of the normalising prologues (drawn last: everything above keeps its values)
    d["norm_w_f32"] = torch.randn(1536, generator=g) * 0.2 + 1.0
    d["norm_b_f32"] = torch.randn(1536, generator=g) * 0.1
    d["mod_scale_bf16"] = (torch.randn(1536, generator=g) * 0.3).bfloat16()
    d["mod_shift_bf16"] = (torch.randn(1536, generator=g) * 0.5).bfloat16()
    return d


DTYPES = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def load_inputs() -> dict:
    z = np.load(os.path.join(HERE, "inputs.npz"))
    out = {}
    for k in z.files:
        dt = None
        if z[k].dtype == np.uint16:
            dt = torch.bfloat16 if k.endswith("bf16") else torch.float16
        out[k] = from_np(z[k], dt)
    return out


def w6_pack_codes(codes: torch.Tensor) -> torch.Tensor:
    c = codes.to(torch.int32)
    lo = (c[:, 0::2] & 15) | ((c[:, 1::2] & 15) << 4)
    t = (c >> 4) & 3
    hi = t[:, 0::4] | (t[:, 1::4] << 2) | (t[:, 2::4] << 4) | (t[:, 3::4] << 6)
    return torch.cat([lo, hi], dim=1).to(torch.uint8).contiguous()


def run_cases(I: dict, B, dev: str) -> dict:
    """B: backend with quant_rows / sd_quant_rows / convrot_requant / convrot_dequant / w6_decode / int8_gemm."""
    out = {}
    mv = (lambda t: t.to(dev)) if dev != "cpu" else (lambda t: t)
    x = mv(I["x_bf16"])
    for rot in (0, 1):
        q, s = B.quant_rows(x[:, :768].contiguous(), PRO["plain"], rot)
        out[f"quant_plain_rot{rot}_q"], out[f"quant_plain_rot{rot}_s"] = q, s
    for pro in ("silu", "gelu", "gelu_tanh"):
        q, s = B.quant_rows(x[:, :768].contiguous(), PRO[pro], 1)
        out[f"quant_{pro}_q"], out[f"quant_{pro}_s"] = q, s
    q, s = B.quant_rows(x, PRO["swiglu"], 1, K=768, up_offset=768)
    out["quant_swiglu_q"], out["quant_swiglu_s"] = q, s
    q, s = B.quant_rows(x[:, :768].contiguous(), PRO["gate"], 0, g=mv(I["gate_bf16"]))
    out["quant_gate_q"], out["quant_gate_s"] = q, s
    q, s = B.quant_rows(mv(I["x_f32"]), PRO["plain"], 1)
    out["quant_f32_q"], out["quant_f32_s"] = q, s
    for name, (pro, K, kw) in norm_cases(I, mv).items():
        rows = x if (K == 1536 or pro == "situ") else x[:, :768].contiguous()
        q, s = B.quant_rows(rows, PRO[pro], 1, K=K, **kw)
        out[f"{name}_q"], out[f"{name}_s"] = q, s
    for rot in (0, 64):
        q, s = B.sd_quant_rows(mv(I["sd_x640"]), rot)
        out[f"sd640_rot{rot}_q"], out[f"sd640_rot{rot}_s"] = q, s
    q, s = B.sd_quant_rows(mv(I["sd_x1280"]), 256)
    out["sd1280_rot256_q"], out["sd1280_rot256_s"] = q, s
    for name in ("w_f32", "w_bf16"):
        for seed in (0, 12345):
            q, s = B.convrot_requant(mv(I[name]), seed)
            out[f"requant_{name}_seed{seed}_q"], out[f"requant_{name}_seed{seed}_s"] = q, s
            if seed == 0:
                out[f"dequant_{name}"] = B.convrot_dequant(q, s, I[name].dtype)
    out["w6_decode"] = B.w6_decode(mv(w6_pack_codes(I["w6_codes"])), mv(I["w6_srel"]), 512)
    out["w6_requant_packed"], out["w6_requant_srel"], out["w6_requant_schannel"] = B.w6_requant(mv(I["w_bf16"]), 3)
    A, W, xs, ws = mv(I["A"]), mv(I["W"]), mv(I["xs"]), mv(I["ws"])
    for name, dt in DTYPES.items():
        b, rs, rr = mv(I[f"bias_{name}"]), mv(I[f"rscale_{name}"]), mv(I[f"resid_{name}"])
        out[f"gemm_plain_{name}"] = B.int8_gemm(A, W, xs, ws, b, out_dtype=dt)
        out[f"gemm_nobias_{name}"] = B.int8_gemm(A, W, xs, ws, None, out_dtype=dt)
        out[f"gemm_resid_{name}"] = B.int8_gemm(A, W, xs, ws, b, out_dtype=dt, rscale=rs, resid=rr)
    return out


class OracleBackend:
    def __init__(self):
        from oracle import oracle as O
        self.O = O

    def quant_rows(self, x, pro, rot, K=None, up_offset=0, g=None, **norm):
        return self.O.quant_rows(x, pro, rot, K=K, up_offset=up_offset, g=g, g_stride=g.stride(0) if g is not None else 0, **norm)

    def sd_quant_rows(self, x, rot):
        return self.O.sd_quant_rows(x, rot)

    def convrot_requant(self, x, seed):
        return self.O.convrot_requant(x, seed)

    def convrot_dequant(self, q, s, dt):
        return self.O.convrot_dequant(q, s, dt)

    def w6_decode(self, p, s, K):
        return self.O.w6_decode(p, s, K)

    def w6_requant(self, w, seed):
        return self.O.w6_requant(w, seed)

    def int8_gemm(self, A, W, xs, ws, bias, out_dtype, rscale=None, resid=None):
        # both multiply-adds of the epilogue fused: the form the reference binary has (contract = 3)
        return self.O.int8_gemm(A, W, xs, ws, bias, rscale, resid, out_dtype, 0, 3)


def save(path: str, d: dict) -> None:
    np.savez_compressed(path, **{k: to_np(v) for k, v in d.items()})
    print(f"wrote {path}: {len(d)} arrays, {os.path.getsize(path) / 1024:.0f} KiB")


def main() -> None:
    what = sys.argv[1]
    if what == "inputs":
        save(os.path.join(HERE, "inputs.npz"), make_inputs())
    elif what == "oracle":
        save(os.path.join(HERE, "oracle.npz"), run_cases(load_inputs(), OracleBackend(), "cpu"))
    elif what == "reference":
        from oracle import ref as R
        out = run_cases(load_inputs(), R, "cuda:0")
        torch.cuda.synchronize()
        save(sys.argv[2], out)
    else:
        raise SystemExit(__doc__)


if __name__ == "__main__":
    main()
