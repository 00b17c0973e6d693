"""Column / row tensor parallelism of the quantized linears across the GPUs of one box (new: the reference is
single-device, src/cuda.rs:88-97).

Activations between linears are sharded by tokens (rows). A (column-parallel, row-parallel) pair of linears --
QKV -> attention-out, MLP-up -> MLP-down -- runs as

    local rows --quantize--> int8 + scales --all-gather--> every rank holds all rows (1 byte per element on the wire)
    column-parallel GEMM with this rank's output channels (a row slice of W [N, K])
    [activation] quantize this rank's K slice of the hidden rows
    row-parallel GEMM with this rank's K slice of W (a column slice), giving partial sums for all rows
    --reduce-scatter--> this rank's rows, + bias + residual

Two ways to run the row-parallel half:
  exact  the per-token scale must come from the whole hidden row, so ranks all-reduce(max) their row maxima and quantize
         with the result (gpu_quant_rows_amax / gpu_quant_rows_scaled); int32 partial accumulators are reduce-scattered
         (integer sums are order-independent) and one epilogue runs on the sums (gpu_int8_epilogue). Codes, accumulators
         and outputs equal the single-device result bit for bit. Twice the bytes on the wire (4 B per element).
  fast   every rank quantizes its K slice with its own row scale and reduce-scatters dequantized bf16 partial outputs;
         bias and residual are added after the reduction. Not bit-identical (finer-grained scales, bf16 partial sums).

`ops` supplies the kernels (the product's `linear` module on GPUs; a CPU stand-in in the tests) and `comm` the three
collectives (torch.distributed: NCCL on GPUs, gloo in the tests), so the sharding logic itself runs anywhere.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import List, Optional

import torch

PRO_PLAIN, PRO_GELU_TANH = 0, 11


class Comm:
    """The collectives the path needs, over a torch.distributed process group (or none: world size 1)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist if (dist.is_available() and dist.is_initialized()) else None
        self.group = group
        self.world = self.dist.get_world_size(group) if self.dist else 1
        self.rank = self.dist.get_rank(group) if self.dist else 0

    def all_gather_rows(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t
        out = torch.empty((t.shape[0] * self.world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        self.dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out

    def reduce_scatter_rows(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t
        out = torch.empty((t.shape[0] // self.world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        if t.device.type == "cpu":   # gloo has no reduce-scatter (nor bf16 sums): all-reduce and keep this rank's rows
            full = t.float() if t.dtype == torch.bfloat16 else t.clone()
            self.dist.all_reduce(full, group=self.group)
            rows = t.shape[0] // self.world
            return full[self.rank * rows:(self.rank + 1) * rows].to(t.dtype).contiguous()
        self.dist.reduce_scatter_tensor(out, t.contiguous(), group=self.group)
        return out

    def all_reduce_max(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX, group=self.group)
        return t


@dataclass
class PairWeights:
    """This rank's shard of a (column-parallel, row-parallel) pair: W1 rows [n0:n1) with their scales and bias, W2
    columns [n0:n1) (contiguous copy) with the full per-channel scales and bias."""
    w1: torch.Tensor
    s1: torch.Tensor
    b1: Optional[torch.Tensor]
    w2: torch.Tensor
    s2: torch.Tensor
    b2: Optional[torch.Tensor]


def shard_pair(w1q, s1, b1, w2q, s2, b2, rank: int, world: int, hidden_of=None) -> PairWeights:
    """Slices already-quantized weights. w1q [N1, K1], w2q [N2, K2] with K2 == N1 (or K2 == N1 / 3 for a QKV whose V
    third feeds the second linear: pass hidden_of = (offset, length) of that part inside N1)."""
    n1 = w1q.shape[0]
    off, length = hidden_of if hidden_of else (0, n1)
    groups = length // 256
    assert length == w2q.shape[1] and length % 256 == 0 and groups >= world, "K slices must hold whole 256-wide rotation groups"
    # whole rotation groups per rank, as even as they divide (3072 hidden columns over 8 ranks: 1 or 2 groups each)
    c0, c1 = 256 * (rank * groups // world), 256 * ((rank + 1) * groups // world)
    if hidden_of:   # QKV: keep q, k, v rows of this rank's heads together: [q_r | k_r | v_r]
        parts = [slice(p * length + c0, p * length + c1) for p in range(n1 // length)]
        idx = torch.cat([torch.arange(s.start, s.stop) for s in parts]).to(w1q.device)
        w1 = w1q.index_select(0, idx).contiguous()
        s1r = s1.index_select(0, idx).contiguous()
        b1r = b1.index_select(0, idx).contiguous() if b1 is not None else None
    else:
        sl = slice(c0, c1)
        w1, s1r, b1r = w1q[sl].contiguous(), s1[sl].contiguous(), (b1[sl].contiguous() if b1 is not None else None)
    w2 = w2q[:, c0:c1].contiguous()
    return PairWeights(w1, s1r, b1r, w2, s2, b2)


class TPPair:
    """One (column-parallel, row-parallel) pair with a residual around it: out = x + W2 act(W1 x)."""

    def __init__(self, ops, comm: Comm, weights: PairWeights, *, rotate: int = 1, act_prologue: int = PRO_PLAIN,
                 hidden_cols: Optional[slice] = None, exact: bool = False):
        self.ops, self.comm, self.w = ops, comm, weights
        self.rotate, self.pro, self.hidden_cols, self.exact = rotate, act_prologue, hidden_cols, exact
        self.ones = None

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        ops, comm, w = self.ops, self.comm, self.w
        a8, xs = ops.quant_rows(x_local, PRO_PLAIN, self.rotate)
        a8, xs = comm.all_gather_rows(a8), comm.all_gather_rows(xs)
        h = ops.int8_gemm(a8, w.w1, xs, w.s1, w.b1, out_dtype=x_local.dtype)             # [M, N1 / P]
        if self.hidden_cols is not None:
            h = h[:, self.hidden_cols].contiguous()
        if self.ones is None:
            self.ones = torch.ones(w.w2.shape[0], dtype=x_local.dtype, device=x_local.device)
        rows = x_local.shape[0]
        if self.exact:
            amax = comm.all_reduce_max(ops.quant_rows_amax(h, self.pro, self.rotate))
            a2, xs2 = ops.quant_rows_scaled(h, amax, self.pro, self.rotate)
            acc = comm.reduce_scatter_rows(ops.int8_gemm_acc_i32(a2, w.w2))                # int32 [M / P, N2]
            xs2_local = xs2[comm.rank * rows:(comm.rank + 1) * rows].contiguous()
            return ops.int8_epilogue(acc, xs2_local, w.s2, w.b2, out_dtype=x_local.dtype, rscale=self.ones, resid=x_local)
        a2, xs2 = ops.quant_rows(h, self.pro, self.rotate)
        part = ops.int8_gemm(a2, w.w2, xs2, w.s2, None, out_dtype=x_local.dtype)          # partial sums, all rows
        y = comm.reduce_scatter_rows(part)
        if w.b2 is not None:
            y = y + w.b2
        return y + x_local


class TPBlock:
    """The linears of one MMDiT block: joint QKV -> (attention taken as identity on V) -> out, and MLP up -> down."""

    def __init__(self, ops, comm: Comm, attn: PairWeights, mlp: PairWeights, exact: bool = False):
        v_cols = attn.w2.shape[1]
        self.attn = TPPair(ops, comm, attn, rotate=1, act_prologue=PRO_PLAIN, hidden_cols=slice(2 * v_cols, 3 * v_cols), exact=exact)
        self.mlp = TPPair(ops, comm, mlp, rotate=1, act_prologue=PRO_GELU_TANH, exact=exact)

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        return self.mlp.forward(self.attn.forward(x_local))


# ---- benchmark leg: `bench.py --mode tp` ----------------------------------------------------------------------------
def bench_main(args, rank, world, local, metric, unit):
    """The 60-block Qwen-Image-shaped MMDiT linear stack at 2048x2048 (M = 16896 tokens, hidden 3072) under column/row
    tensor parallelism: tokens sharded between blocks, int8 all-gather before the column-parallel linears,
    reduce-scatter after the row-parallel ones. Random int8 weights per block (generated on the device)."""
    import os
    import torch.distributed as dist
    from . import linear as ops

    dev = torch.device("cuda", local)
    comm = Comm()
    blocks = int(os.environ.get("BENCH_TP_BLOCKS", "60"))
    exact = os.environ.get("BENCH_TP_EXACT", "0") == "1"
    M, F, MLP = 16896, 3072, 12288
    assert M % world == 0 and F // 256 >= world
    g = torch.Generator(device=dev).manual_seed(1234)          # same seed on every rank: identical full weights, then sliced

    def qweight(n, k):
        return (torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8, device=dev),
                torch.rand(n, generator=g, device=dev) * 2e-4 + 1e-5,
                (torch.randn(n, generator=g, device=dev) * 0.01).bfloat16())

    stack: List[TPBlock] = []
    for _ in range(blocks):
        wqkv, sqkv, bqkv = qweight(3 * F, F)
        wo, so, bo = qweight(F, F)
        wu, su, bu = qweight(MLP, F)
        wd, sd, bd = qweight(F, MLP)
        attn = shard_pair(wqkv, sqkv, bqkv, wo, so, bo, rank, world, hidden_of=(0, F))
        mlp = shard_pair(wu, su, bu, wd, sd, bd, rank, world)
        stack.append(TPBlock(ops, comm, attn, mlp, exact))
        del wqkv, wo, wu, wd
    rows = M // world
    x = torch.randn(rows, F, generator=torch.Generator(device=dev).manual_seed(99 + rank), device=dev).bfloat16()

    # Micro-batches (BENCH_TP_MICRO, default 1 = off): the rank's rows split into independent parts, each on its own stream
    # and walked through the stack block by block in turn, so that the collectives of one part could overlap the kernels of
    # the other. Measured on two GPUs it does not pay: the persistent GEMM holds every SM, NCCL's kernels wait for it, and
    # the halved GEMMs are less efficient (fast mode 105 against 99.6 ms per stack, exact 141 against 125).
    micro = int(os.environ.get("BENCH_TP_MICRO", "1"))
    assert rows % micro == 0
    parts = [x[i * (rows // micro):(i + 1) * (rows // micro)].contiguous() for i in range(micro)]
    streams = [torch.cuda.Stream(dev) for _ in range(micro)]

    def step():
        cur = torch.cuda.current_stream()
        hs = list(parts)
        for s in streams:
            s.wait_stream(cur)
        for b in stack:
            for i, s in enumerate(streams):
                with torch.cuda.stream(s):
                    hs[i] = b.forward(hs[i])
        for s in streams:
            cur.wait_stream(s)
        return hs

    for _ in range(max(1, args.warmup)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier(device_ids=[local])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ops_per_block = 2.0 * M * (3 * F * F + F * F + MLP * F + F * MLP)
    value = ops_per_block * blocks * args.steps / (ms * 1e-3) / 1e12
    if rank == 0:
        print(json.dumps({"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                          "config": {"workload": f"mmdit_linear_stack_{blocks}blocks_M16896_hidden3072", "parallelism": f"tp{world}",
                                     "mode": "exact (int32 reduce-scatter)" if exact else "fast (bf16 reduce-scatter)",
                                     "micro_batches": micro,
                                     "dit_block_gemm_ms": ms / args.steps / blocks},
                          "gpu_launches": args.steps * blocks * (10 if exact else 8), "kernel_status": ops.kernel_status()}), flush=True)
    if world > 1:
        dist.destroy_process_group()
