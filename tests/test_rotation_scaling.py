"""The rotating GEMM epilogue runs the R256 butterflies without the reference's per-stage halvings and scales once (by
1/16 after the third stage, the last stage then adding values that are already half the reference's). This is exact as
long as nothing overflows and no subnormal is rounded: rounding to nearest commutes with a scaling by a power of two, and
sums of bf16 values are multiples of 2^-133, so every subnormal intermediate is representable. The test restates both
forms in IEEE single precision (numpy, no contraction) and compares them bit for bit on bf16 inputs drawn from every
magnitude below the kernel's switch-over point (2^120), subnormal inputs, signed zeros and heavy cancellation included.
Reference order of the butterfly: csrc/common.cuh:99-126."""
from __future__ import annotations

import numpy as np

F = np.float32


def _butterfly(x0, x1, x2, x3, halve: bool):
    s, d = x0 + x1, x0 - x1
    r0, r1, r2, r3 = (s + x2) - x3, (s - x2) + x3, (d + x2) + x3, (x2 - d) + x3
    if halve:
        h = F(0.5)
        return h * r0, h * r1, h * r2, h * r3
    return r0, r1, r2, r3


def _stage(v: np.ndarray, stride: int, halve: bool) -> np.ndarray:
    """One radix-4 stage over the last axis (256 values): elements i, i+s, i+2s, i+3s inside blocks of 4s."""
    rows = v.shape[0]
    w = v.reshape(rows, 256 // (4 * stride), 4, stride)
    out = np.stack(_butterfly(w[:, :, 0], w[:, :, 1], w[:, :, 2], w[:, :, 3], halve), axis=2)
    return out.reshape(rows, 256)


def _reference(v):
    for s in (1, 4, 16, 64):
        v = _stage(v, s, True)
    return v


def _epilogue(v):
    for s in (1, 4, 16):
        v = _stage(v, s, False)
    v = v * F(0.0625)            # half the reference's values after three stages
    return _stage(v, 64, False)


def _bf16_values(rng, rows, lo_exp, hi_exp):
    """Random bf16 values (as float32) with exponents in [lo_exp, hi_exp], random signs, some zeros."""
    e = rng.integers(lo_exp, hi_exp + 1, size=(rows, 256))
    m = rng.integers(0, 128, size=(rows, 256))
    sign = rng.integers(0, 2, size=(rows, 256)).astype(np.uint32) << 31
    bits = sign | ((e + 127).astype(np.uint32) << 23) | (m.astype(np.uint32) << 16)
    x = bits.view(np.float32).copy()
    x[rng.random((rows, 256)) < 0.02] = 0.0
    return x


def test_one_scaling_equals_four_halvings_bit_for_bit():
    rng = np.random.default_rng(3)
    cases = [
        _bf16_values(rng, 400, -8, 4),          # activations
        _bf16_values(rng, 400, -126, -100),     # next to the subnormal range: intermediates become subnormal
        _bf16_values(rng, 400, 100, 119),       # just below the switch-over point: no overflow yet
        _bf16_values(rng, 400, -126, 119),      # everything at once: heavy cancellation between magnitudes
    ]
    sub = (rng.integers(0, 128, size=(200, 256)).astype(np.uint32) << 16).view(np.float32)      # bf16 subnormals
    cases.append(sub.copy())
    same = np.tile(_bf16_values(rng, 100, -3, 3)[:, :1], (1, 256))                               # exact cancellation to +-0
    cases.append(same)
    for x in cases:
        with np.errstate(over="raise", invalid="raise"):
            a, b = _reference(x), _epilogue(x)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_the_switch_over_point_is_needed():
    """Above 2^120 the unhalved sums can overflow where the reference's do not: the kernel switches to the halved form there."""
    x = np.full((1, 256), F(2.0) ** 125, dtype=np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        a, b = _reference(x), _epilogue(x)
    assert np.isfinite(a).all() and not np.isfinite(b).all()
