"""The library's calls are plain stream-ordered launches, so a block's sequence of quantizer and GEMM calls can be
captured into a CUDA graph (as the reference's engine does with its own kernels) and replayed: same bits as the eager
calls. Everything the library creates lazily (activation tables, the K-split workspace) is created by the warm-up call
before the capture starts."""
from __future__ import annotations

import pytest
import torch

from conftest import assert_bits_equal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M", [1, 77, 1024])
def test_block_sequence_replays_bit_identically(pkg, dev, M):
    L = pkg.linear
    g = torch.Generator().manual_seed(M)
    F, H = 1024, 4096
    x = torch.randn(M, F, generator=g).bfloat16().to(dev)
    w1, s1 = L.convrot_requant((torch.randn(H, F, generator=g) * 0.02).to(dev), 0)
    w2, s2 = L.convrot_requant((torch.randn(F, H, generator=g) * 0.02).to(dev), 0)
    b1 = (torch.randn(H, generator=g) * 0.1).bfloat16().to(dev)
    ones = torch.ones(F, dtype=torch.bfloat16, device=dev)
    a1 = torch.empty((M, F), dtype=torch.int8, device=dev); xs1 = torch.empty(M, device=dev)
    h = torch.empty((M, H), dtype=torch.bfloat16, device=dev)
    a2 = torch.empty((M, H), dtype=torch.int8, device=dev); xs2 = torch.empty(M, device=dev)
    out = torch.empty((M, F), dtype=torch.bfloat16, device=dev)

    def block():
        L.quant_rows(x, 0, 1, q=a1, scales=xs1)
        L.int8_gemm(a1, w1, xs1, s1, b1, out=h)
        L.quant_rows(h, 11, 1, q=a2, scales=xs2)                 # GELU-tanh prologue
        L.int8_gemm(a2, w2, xs2, s2, None, rscale=ones, resid=x, out=out)

    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        block()                                                  # warm-up on the capture stream: lazy set-up happens here
        side.synchronize()
        eager = out.clone()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            block()
        out.zero_()
        graph.replay()
        side.synchronize()
        assert_bits_equal(out, eager, "replayed block")
        x.copy_((torch.randn(M, F, generator=g) * 2).bfloat16())   # new input, same graph
        graph.replay()
        side.synchronize()
        replayed = out.clone()
        block()
        side.synchronize()
        assert_bits_equal(replayed, out, "replay on new data")
    assert L.kernel_status() == 0
