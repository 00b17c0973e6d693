"""Shared fixtures. GPU tests carry @pytest.mark.gpu and call the kernels through the C ABI; everything else runs on CPU."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def pkg():
    """The product package; importing it loads libb200_qlinear.so and fails loudly if it is missing."""
    from __graft_entry__ import load_package
    return load_package()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CUDA kernels built for sm_100a (oracle/_ref/libref.so); tests skip where it is absent."""
    from oracle import ref as R
    if not R.available():
        pytest.skip("oracle/_ref/libref.so not built (needs the reference tree: oracle/build_ref.sh)")
    return R


@pytest.fixture(scope="session")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


def _load_npz(name):
    path = os.path.join(GOLDEN, name)
    if not os.path.exists(path):
        return None
    return np.load(path)


@pytest.fixture(scope="session")
def golden_inputs():
    sys.path.insert(0, GOLDEN)
    import make_golden
    return make_golden.load_inputs()


@pytest.fixture(scope="session")
def golden_oracle():
    return _load_npz("oracle.npz")


@pytest.fixture(scope="session")
def golden_reference():
    z = _load_npz("reference.npz")
    if z is None:
        pytest.skip("tests/golden/reference.npz not present")
    return z


def as_np(t: torch.Tensor) -> np.ndarray:
    """Bit-level numpy view of a tensor (16-bit floats as uint16)."""
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def assert_bits_equal(a: torch.Tensor, b, what: str = ""):
    an = as_np(a)
    bn = b if isinstance(b, np.ndarray) else as_np(b)
    assert an.shape == bn.shape, (what, an.shape, bn.shape)
    if an.dtype != bn.dtype:
        bn = bn.view(an.dtype) if an.itemsize == bn.itemsize else bn.astype(an.dtype)
    bad = int((an != bn).sum())
    assert bad == 0, f"{what}: {bad}/{an.size} elements differ"


def max_ulp_diff(a: torch.Tensor, b: torch.Tensor) -> int:
    """Largest distance, in units in the last place of their (shared, 16-bit) type, between two finite tensors."""
    assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16)
    def key(t):
        i = t.detach().cpu().contiguous().view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7FFF), i)      # sign-magnitude -> monotone integer
    return int((key(a) - key(b)).abs().max())


def assert_close_out(got: torch.Tensor, want: torch.Tensor, what: str = "", tiny: float = 0.0):
    """The tolerance of this path: one ulp of a 16-bit output type; 1e-5 of max(|value|, 1) for f32 outputs
    (the terms being summed can be larger than the sum). Elements whose
    expected magnitude is below `tiny` (activations that cancel to almost zero) are held to an absolute 1e-6."""
    g, w = got.detach().cpu(), want.detach().cpu()
    small = w.float().abs() < tiny
    if bool(small.any()):
        assert float((g.float() - w.float()).abs()[small].max()) <= 1e-6, what
        g, w = torch.where(small, w, g), w
    if got.dtype == torch.float32:
        rel = ((g - w).abs() / w.abs().clamp_min(1.0)).max().item()
        assert rel <= 1e-5, (what, rel)
    else:
        d = max_ulp_diff(g, w)
        assert d <= 1, f"{what}: {d} ulp apart"
