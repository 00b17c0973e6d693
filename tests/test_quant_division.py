"""The bf16 quantizer divides by the (bf16-rounded) scale with one multiplication by the correctly rounded reciprocal.
That is exact for its purpose: bf16(a * rcp(st)) == bf16(a / st) for every pair of bf16 values, because the exact quotient
of two 8-bit significands can never sit on (or within 2^-17 of) a bf16 rounding boundary. Scaling either operand by a
power of two scales the quotient exactly, so enumerating the 128 x 128 significands over a span of exponents that covers
quotients from far below one code step to beyond the int8 range proves it for all inputs the kernel can see."""
from __future__ import annotations

import numpy as np
import torch


def _bf16(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).bfloat16().float().numpy()


def test_reciprocal_multiply_rounds_like_the_division_for_every_significand_pair():
    A = np.arange(128, 256, dtype=np.float32)[:, None]      # significands of the value, 1.0000000b .. 1.1111111b
    S = np.arange(128, 256, dtype=np.float32)[None, :]      # significands of the scale
    rcp = (np.float32(1.0) / S).astype(np.float32)           # what __frcp_rn returns: the correctly rounded reciprocal
    for e in range(-14, 10):                                 # quotients from 2^-15 to 2^10
        a = (A * np.float32(2.0 ** e)).astype(np.float32)
        fast = _bf16((a * rcp).astype(np.float32))
        ieee = _bf16((a / S).astype(np.float32))
        assert np.array_equal(fast, ieee), e
        # and the codes that follow: round half to even, clamp to int8
        assert np.array_equal(np.clip(np.rint(fast), -128, 127), np.clip(np.rint(ieee), -128, 127))


def test_no_quotient_sits_on_a_rounding_boundary():
    """The argument itself: A * 2^n == S * M has no solution with A, S < 256 and M odd in (256, 512)."""
    A = np.arange(1, 256, dtype=np.int64)
    odd_part = A.copy()
    while ((odd_part & 1) == 0).any():
        odd_part = np.where((odd_part & 1) == 0, odd_part >> 1, odd_part)
    assert odd_part.max() < 256          # odd part of the left side
    # odd part of the right side is odd(S) * M >= 257: the two can never be equal
    assert 1 * 257 > odd_part.max()


def test_half_division_by_refined_reciprocal_for_every_significand_pair():
    """The fp16 quantizer's division: q0 = a * rcp(st), t = fma(fma(-q0, st, a), rcp, q0), then half(t). For every pair of
    11-bit significands (and exponents covering quotients from 2^-12 to 2^9) half(t) equals half(a / st)."""
    A = np.arange(1024, 2048, dtype=np.float64)[:, None]
    S = np.arange(1024, 2048, dtype=np.float64)[None, :]
    rcp = (np.float32(1.0) / S.astype(np.float32)).astype(np.float32).astype(np.float64)
    for e in range(-12, 10):
        a = A * 2.0 ** e
        q0 = (a.astype(np.float32) * rcp.astype(np.float32)).astype(np.float32).astype(np.float64)
        r = (a - q0 * S).astype(np.float32).astype(np.float64)          # fma(-q0, st, a): the difference is exact in double
        t = (q0 + r * rcp).astype(np.float32)                           # fma(r, rcp, q0)
        ieee = (a.astype(np.float32) / S.astype(np.float32)).astype(np.float32)
        assert np.array_equal(t.astype(np.float16), ieee.astype(np.float16)), e
        assert np.array_equal(ieee.astype(np.float16), (a / S).astype(np.float16)), e
