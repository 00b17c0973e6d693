"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The reference is measured on real checkpoints (Qwen-Image, Wan-style video DiT, SDXL); none is available offline,
so tensors of the same shapes and distributions stand in for them. Everything is generated on the CPU from a
``torch.Generator`` with a fixed seed per tensor, so every implementation (these kernels, the CPU oracle, the
reference's kernels) receives identical bytes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def activations(M: int, K: int, seed: int, *, outliers: str = "x20", dtype=torch.bfloat16) -> torch.Tensor:
    """[M, K] ~ N(0,1); ``x20``: 1 % of the K channels scaled by 20; ``student``: per-channel scale |t(nu=3)| clipped
    to [0.2, 50] (heavy-tailed outlier channels); ``none``: plain normal."""
    g = _gen(seed)
    x = torch.randn(M, K, generator=g)
    if outliers == "x20":
        cols = torch.randperm(K, generator=g)[: max(1, K // 100)]
        x[:, cols] *= 20.0
    elif outliers == "student":
        z = torch.randn(K, generator=g)
        chi = (torch.randn(3, K, generator=g) ** 2).sum(0) / 3.0
        x *= (z / chi.sqrt()).abs().clamp(0.2, 50.0)[None, :]
    return x.to(dtype)


def weight(N: int, K: int, seed: int, std: float = 0.02, dtype=torch.float32) -> torch.Tensor:
    return (torch.randn(N, K, generator=_gen(seed)) * std).to(dtype)


def bias(N: int, seed: int, std: float = 0.01, dtype=torch.bfloat16) -> torch.Tensor:
    return (torch.randn(N, generator=_gen(seed)) * std).to(dtype)


def w6_pack(w: torch.Tensor, fitted_groups: bool = False):
    """Symmetric 6-bit weights in the reference's W6A8 storage (csrc/vendor/w6a8_requant.cu:128-151, csrc/h3.cu:8-37):
    codes = level + 32 with level in [-31, 31], two-plane packed rows, one e4m3 ``s_rel`` per 32 columns and one f32
    ``s_channel`` per row. ``fitted_groups=False`` realises plain per-output-channel scaling (s_rel = 1.0 exactly);
    ``True`` gives each group its own e4m3 scale relative to the row (values in [0.25, 1])."""
    N, K = w.shape
    wf = w.float()
    if not fitted_groups:
        # the GEMM sees clamp(rint(level * 1.0)) = level; the dequantized weight is level * s_channel
        s_channel = (wf.abs().amax(1) / 31.0).clamp_min(1e-8)
        level = torch.clamp(torch.round(wf / s_channel[:, None]), -31, 31)
        s_rel = torch.full((N, K // 32), 0x38, dtype=torch.uint8)  # e4m3 1.0
    else:
        # the GEMM sees rint(level * s_rel) on the +-127 grid; the dequantized weight is that times s_channel
        g = wf.view(N, K // 32, 32)
        gmax = g.abs().amax(2)
        rmax = gmax.amax(1, keepdim=True).clamp_min(1e-30)
        s_channel = (rmax[:, 0] / 127.0).clamp_min(1e-8)
        rel8 = ((gmax / rmax) * (127.0 / 31.0)).clamp_min(2.0 ** -6).to(torch.float8_e4m3fn)
        s_rel = rel8.view(torch.uint8)
        level = torch.clamp(torch.round(g / (s_channel[:, None, None] * rel8.float()[:, :, None])), -31, 31).view(N, K)
    codes = (level + 32).to(torch.uint8)
    c = codes.to(torch.int32)
    lo = (c[:, 0::2] & 15) | ((c[:, 1::2] & 15) << 4)
    t = (c >> 4) & 3
    hi = t[:, 0::4] | (t[:, 1::4] << 2) | (t[:, 2::4] << 4) | (t[:, 3::4] << 6)
    packed = torch.cat([lo, hi], dim=1).to(torch.uint8).contiguous()
    return packed, s_rel.contiguous(), s_channel.float().contiguous()


@dataclass
class LinearSpec:
    name: str
    M: int
    K: int
    N: int
    epilogue: str = "plain"          # plain | gelu_tanh | residual
    rotate: int = 0                  # 0, 64 or 256 (activation side and weight side agree)
    act_dtype: torch.dtype = torch.bfloat16
    weight_format: str = "int8"      # int8 | w6
    bias: bool = True

    @property
    def ops(self) -> float:
        return 2.0 * self.M * self.N * self.K


def config(idx: int, M: Optional[int] = None) -> List[LinearSpec]:
    """The linears of benchmark configuration ``idx`` (0-4, in the order the benchmark definition lists them)."""
    if idx == 0:   # single W8A8 linear, outliers x20, fp16 weights quantized per output channel
        return [LinearSpec("w8a8", M or 4096, 3072, 3072, "plain", 0)]
    if idx == 1:   # ConvRot int8 MMDiT MLP pair, Qwen-Image-shaped block at 1024x1024
        m = M or 4352
        return [LinearSpec("mlp_up", m, 3072, 12288, "gelu_tanh", 256), LinearSpec("mlp_down", m, 12288, 3072, "residual", 256)]
    if idx == 2:   # W6A8 video-DiT linears (hidden 5120, FFN 13824)
        m = M or 2048
        return [LinearSpec("qkv", m, 5120, 15360, "plain", 0, weight_format="w6"),
                LinearSpec("out", m, 5120, 5120, "plain", 0, weight_format="w6"),
                LinearSpec("ffn_up", m, 5120, 13824, "gelu_tanh", 0, weight_format="w6"),
                LinearSpec("ffn_down", m, 13824, 5120, "plain", 0, weight_format="w6")]
    if idx == 3:   # SDXL UNet int8 linears at 1024x1024, CFG batch 2, fp16 activations
        h = torch.float16
        shapes = [("sa_qkv_640", 8192, 640, 1920), ("sa_out_640", 8192, 640, 640), ("sa_qkv_1280", 2048, 1280, 3840),
                  ("sa_out_1280", 2048, 1280, 1280), ("ca_q_640", 8192, 640, 640), ("ca_q_1280", 2048, 1280, 1280),
                  ("ca_kv_640", 154, 2048, 640), ("ca_kv_1280", 154, 2048, 1280), ("geglu_640", 8192, 640, 5120),
                  ("geglu_1280", 2048, 1280, 10240), ("ff2_640", 8192, 2560, 640), ("ff2_1280", 2048, 5120, 1280)]
        return [LinearSpec(n, m, k, nn, "plain", 256 if k % 256 == 0 else 64, act_dtype=h) for n, m, k, nn in shapes]
    if idx == 4:   # one block of the 60-block Qwen-Image-shaped MMDiT stack at 2048x2048
        m = M or 16896
        return [LinearSpec("qkv", m, 3072, 9216, "plain", 256), LinearSpec("attn_out", m, 3072, 3072, "residual", 256),
                LinearSpec("mlp_up", m, 3072, 12288, "gelu_tanh", 256), LinearSpec("mlp_down", m, 12288, 3072, "residual", 256),
                LinearSpec("adaln", 1, 3072, 18432, "plain", 256)]
    raise ValueError(idx)
