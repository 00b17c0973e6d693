"""Two-GPU (NCCL) test of the tensor-parallel pair: exact mode equals the single-GPU result bit for bit, fast mode stays
within quantization noise. Skipped on boxes with one GPU; the sharding logic itself is covered on CPU with gloo."""
from __future__ import annotations

import importlib
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _inputs(dev):
    g = torch.Generator().manual_seed(17)
    F, H, M = 1024, 4096, 1024
    w1 = (torch.randn(H, F, generator=g) * 0.02).to(dev)
    w2 = (torch.randn(F, H, generator=g) * 0.02).to(dev)
    b1 = (torch.randn(H, generator=g) * 0.01).bfloat16().to(dev)
    b2 = (torch.randn(F, generator=g) * 0.01).bfloat16().to(dev)
    x = torch.randn(M, F, generator=g).bfloat16().to(dev)
    return w1, b1, w2, b2, x


def _run(rank, world, exact, dev):
    from __graft_entry__ import load_package
    pkg = load_package()
    tp = importlib.import_module("cbr_b200.tensor_parallel")
    L = pkg.linear
    w1, b1, w2, b2, x = _inputs(dev)
    w1q, s1 = L.convrot_requant(w1)
    w2q, s2 = L.convrot_requant(w2)
    pair = tp.TPPair(L, tp.Comm(), tp.shard_pair(w1q, s1, b1, w2q, s2, b2, rank, world), rotate=1, act_prologue=11, exact=exact)
    rows = x.shape[0] // world
    out = pair.forward(x[rank * rows:(rank + 1) * rows].contiguous())
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    return out


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    for exact in (True, False):
        torch.save(_run(rank, world, exact, dev).cpu(), os.path.join(out_dir, f"out_{int(exact)}_{rank}.pt"))
    dist.barrier(device_ids=[rank])
    dist.destroy_process_group()


def test_pair_on_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = 29700 + os.getpid() % 200
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    sys.path.insert(0, ROOT)
    torch.cuda.set_device(0)
    want = _run(0, 1, True, torch.device("cuda:0")).cpu()
    exact = torch.cat([torch.load(tmp_path / f"out_1_{r}.pt") for r in range(2)])
    fast = torch.cat([torch.load(tmp_path / f"out_0_{r}.pt") for r in range(2)])
    assert torch.equal(exact.view(torch.int16), want.view(torch.int16)), "exact mode: bit-identical to one GPU"
    assert (fast.float() - want.float()).abs().max().item() < 0.05 * want.float().abs().max().item()


def test_the_three_arrangements_of_the_mlp_pair_agree_bit_for_bit():
    """One GPU: the pair with GELU-tanh and the rotation in the first GEMM's epilogue, with the GELU in the epilogue and the
    whole quantizer after it, and with the GELU in the quantizer's prologue (the reference's arrangement,
    src/qwen21.rs:378-417) must write the same output."""
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    pkg = load_package()
    tp = importlib.import_module("cbr_b200.tensor_parallel")
    L = pkg.linear
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    w1, b1, w2, b2, x = _inputs(dev)
    w1q, s1 = L.convrot_requant(w1)
    w2q, s2 = L.convrot_requant(w2)
    comm = tp.Comm()                      # no process group: world size 1
    outs = {}
    for form in ("rot", "epilogue", "prologue"):
        pair = tp.TPPair(L, comm, tp.shard_pair(w1q, s1, b1, w2q, s2, b2, 0, 1), rotate=1, act_prologue=11, act_form=form)
        outs[form] = pair.forward(x).clone()
    torch.cuda.synchronize()
    assert L.kernel_status() == 0
    assert torch.equal(outs["rot"].view(torch.int16), outs["prologue"].view(torch.int16))
    assert torch.equal(outs["epilogue"].view(torch.int16), outs["prologue"].view(torch.int16))
