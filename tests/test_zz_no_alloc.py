"""gpu_int8_gemm_noalloc: the GEMM variant for hosts that cannot allocate device memory while they run (for instance an
engine that has already handed the whole card to its own budgeted allocator). Its K-split scratch is a fixed array
inside the library, so the only thing to prove is that it computes what gpu_int8_gemm computes -- also on a second
call, which finds the array as the first one left it. Collected last on purpose (file name), so a failure here cannot
hide the result of any other test; it needs nothing the other tests set up."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
DT_BF16, DT_F32 = 2, 0


def _call(fn, A, W, xs, ws, bias, D, out_dt):
    M, K = A.shape
    N = W.shape[0]
    return fn(A.data_ptr(), W.data_ptr(), xs.data_ptr(), ws.data_ptr(), bias.data_ptr() if bias is not None else 0, D.data_ptr(),
              M, N, K, out_dt, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("M,N,K,dtype,code", [(256, 512, 8192, torch.bfloat16, DT_BF16), (200, 300, 4096, torch.float32, DT_F32),
                                              (130, 1000, 2048, torch.bfloat16, DT_BF16),
                                              (256, 2048, 8192, torch.bfloat16, DT_BF16),      # 8 tiles once the width is 256
                                              (1024, 1024, 1024, torch.bfloat16, DT_BF16)])    # the full 16 tiles of 256 x 256
def test_matches_the_allocating_entry_point_twice_in_a_row(pkg, dev, M, N, K, dtype, code):
    g = torch.Generator().manual_seed(M + N + K)
    A = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8).to(dev)
    W = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8).to(dev)
    xs = (torch.rand(M, generator=g) * 0.05 + 1e-3).to(dev)
    ws = (torch.rand(N, generator=g) * 1e-3 + 1e-4).to(dev)
    bias = (torch.randn(N, generator=g) * 0.5).to(dtype).to(dev)
    want = torch.empty((M, N), dtype=dtype, device=dev)
    assert _call(pkg.lib.gpu_int8_gemm, A, W, xs, ws, bias, want, code) == 0
    for attempt in range(2):            # the second call starts from whatever the first left in the static array
        got = torch.full((M, N), float("nan"), dtype=dtype, device=dev)
        assert _call(pkg.lib.gpu_int8_gemm_noalloc, A, W, xs, ws, bias, got, code) == 0
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                           want.view(torch.int16 if dtype == torch.bfloat16 else torch.int32)), f"call {attempt + 1} differs"
    # a different problem right after reuses the same array
    A2 = torch.randint(-128, 128, (64, K), generator=g, dtype=torch.int8).to(dev)
    want2 = torch.empty((64, N), dtype=dtype, device=dev)
    got2 = torch.empty((64, N), dtype=dtype, device=dev)
    assert _call(pkg.lib.gpu_int8_gemm, A2, W, xs[:64].contiguous(), ws, bias, want2, code) == 0
    assert _call(pkg.lib.gpu_int8_gemm_noalloc, A2, W, xs[:64].contiguous(), ws, bias, got2, code) == 0
    torch.cuda.synchronize()
    assert torch.equal(got2.float(), want2.float())
    assert pkg.linear.kernel_status() == 0


def test_rejects_what_the_static_array_cannot_hold(pkg, dev):
    M, N, K = 4096, 4096, 256        # 256 tiles: far beyond the 16 the array has room for
    A = torch.zeros((M, K), dtype=torch.int8, device=dev)
    W = torch.zeros((N, K), dtype=torch.int8, device=dev)
    xs = torch.ones(M, device=dev)
    ws = torch.ones(N, device=dev)
    D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    assert _call(pkg.lib.gpu_int8_gemm_noalloc, A, W, xs, ws, None, D, DT_BF16) == -205
    # 17 tiles at the widest tile: one beyond the array
    W17 = torch.zeros((17 * 256, K), dtype=torch.int8, device=dev)
    assert _call(pkg.lib.gpu_int8_gemm_noalloc, A[:256], W17, xs, torch.ones(17 * 256, device=dev), None,
                 torch.empty((256, 17 * 256), dtype=torch.bfloat16, device=dev), DT_BF16) == -205
    # K not a multiple of 16: refused before anything else is looked at
    A8 = torch.zeros((64, 8), dtype=torch.int8, device=dev)
    assert _call(pkg.lib.gpu_int8_gemm_noalloc, A8, A8, xs, ws, None, D, DT_BF16) == -202


def test_second_call_allocates_no_device_memory(pkg, dev):
    """After one warm-up call per output type (module load and kernel set-up are the runtime's), further calls leave the
    free device memory as it is."""
    M, N, K = 256, 512, 4096
    A = torch.ones((M, K), dtype=torch.int8, device=dev)
    W = torch.ones((N, K), dtype=torch.int8, device=dev)
    xs = torch.ones(M, device=dev)
    ws = torch.ones(N, device=dev)
    D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    assert _call(pkg.lib.gpu_int8_gemm_noalloc, A, W, xs, ws, None, D, DT_BF16) == 0
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert _call(pkg.lib.gpu_int8_gemm_noalloc, A, W, xs, ws, None, D, DT_BF16) == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    assert bool((D.float() == K).all())
