"""World-size-2 (gloo, CPU) tests of the tensor-parallel sharding logic, with the oracle standing in for the kernels."""
from __future__ import annotations

import importlib
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _weights():
    g = torch.Generator().manual_seed(5)
    F, H = 512, 768          # three rotation groups of hidden columns: ranks take one and two
    w1 = torch.randn(H, F, generator=g) * 0.02
    w2 = torch.randn(F, H, generator=g) * 0.02
    b1 = (torch.randn(H, generator=g) * 0.01).bfloat16()
    b2 = (torch.randn(F, generator=g) * 0.01).bfloat16()
    x = torch.randn(64, F, generator=g).bfloat16()
    return F, H, w1, b1, w2, b2, x


def _worker(rank, world, port, exact, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from __graft_entry__ import load_package
    load_package()
    tp = importlib.import_module("cbr_b200.tensor_parallel")
    import cpu_ops
    F, H, w1, b1, w2, b2, x = _weights()
    w1q, s1 = cpu_ops.convrot_requant(w1)
    w2q, s2 = cpu_ops.convrot_requant(w2)
    comm = tp.Comm()
    shard = tp.shard_pair(w1q, s1, b1, w2q, s2, b2, rank, world)
    pair = tp.TPPair(cpu_ops, comm, shard, rotate=1, act_prologue=11, exact=exact)
    rows = x.shape[0] // world
    out = pair.forward(x[rank * rows:(rank + 1) * rows].contiguous())
    torch.save(out, os.path.join(out_dir, f"out_{int(exact)}_{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _single_device():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from __graft_entry__ import load_package
    load_package()
    tp = importlib.import_module("cbr_b200.tensor_parallel")
    import cpu_ops
    F, H, w1, b1, w2, b2, x = _weights()
    w1q, s1 = cpu_ops.convrot_requant(w1)
    w2q, s2 = cpu_ops.convrot_requant(w2)
    pair = tp.TPPair(cpu_ops, tp.Comm(), tp.shard_pair(w1q, s1, b1, w2q, s2, b2, 0, 1), rotate=1, act_prologue=11, exact=True)
    return pair.forward(x)


@pytest.mark.parametrize("exact", [True, False])
def test_column_row_pair_on_two_ranks(tmp_path, exact):
    port = 29600 + (os.getpid() % 200) + (1 if exact else 0)
    mp.spawn(_worker, args=(2, port, exact, str(tmp_path)), nprocs=2, join=True)
    got = torch.cat([torch.load(tmp_path / f"out_{int(exact)}_{r}.pt") for r in range(2)])
    want = _single_device()
    if exact:
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), "exact mode equals the single-device result bit for bit"
    else:
        err = (got.float() - want.float()).abs().max().item()
        assert err < 0.05 * want.float().abs().max().item(), err


def test_qkv_sharding_keeps_heads_together(pkg):
    tp = importlib.import_module("cbr_b200.tensor_parallel")
    F = 512
    w1 = torch.arange(3 * F).to(torch.int8).view(-1, 1).repeat(1, 256)       # row index mod 256 as the code
    s1 = torch.arange(3 * F, dtype=torch.float32)
    w2 = torch.zeros(64, F, dtype=torch.int8)
    sh = tp.shard_pair(w1, s1, None, w2, torch.ones(64), None, 1, 2, hidden_of=(0, F))
    assert sh.w1.shape == (3 * F // 2, 256) and sh.w2.shape == (64, F // 2)
    assert sh.s1.tolist() == list(range(256, 512)) + list(range(768, 1024)) + list(range(1280, 1536))
    with pytest.raises(AssertionError):
        tp.shard_pair(w1, s1, None, w2, torch.ones(64), None, 0, 4, hidden_of=(0, F))   # 128-wide K slices split a rotation group
