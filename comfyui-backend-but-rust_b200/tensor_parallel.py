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

    def all_gather_rows(self, t: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.world == 1:
            return t
        if out is None:
            out = torch.empty((t.shape[0] * self.world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        self.dist.all_gather_into_tensor(out, t, group=self.group)
        return out

    def reduce_scatter_rows(self, t: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.world == 1:
            return t
        if t.device.type == "cpu":   # gloo has no reduce-scatter (nor bf16 sums): all-reduce and keep this rank's rows
            full = t.float() if t.dtype == torch.bfloat16 else t.clone()
            self.dist.all_reduce(full, group=self.group)
            rows = t.shape[0] // self.world
            return full[self.rank * rows:(self.rank + 1) * rows].to(t.dtype).contiguous()
        if out is None:
            out = torch.empty((t.shape[0] // self.world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        self.dist.reduce_scatter_tensor(out, t, group=self.group)
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


_ACT_OF_PROLOGUE = {PRO_GELU_TANH: 1, 5: 2, 6: 3}     # quantizer prologues that are activations -> the GEMM epilogue's codes


class TPPair:
    """One (column-parallel, row-parallel) pair with a residual around it: out = x + W2 act(W1 x).

    Every step is one of the library's kernels or a collective: no eager tensor arithmetic, no copies (the V part of a
    QKV output is read in place through its row stride), and on CUDA every intermediate lives in buffers allocated once
    (`bufs`, shared by the pairs of a stack), so that a pass allocates nothing and can be captured in a CUDA graph.

    `chunks` > 1 (fast mode, CUDA): the row-parallel GEMM runs as that many column blocks of the output; the
    reduce-scatter of block i runs on `comm_stream` while the GEMM of block i + 1 runs on the compute stream (the caller
    limits the GEMM's share of the SMs with gpu_int8_gemm_set_cluster_limit so that the collective's kernels find room)."""

    def __init__(self, ops, comm: Comm, weights: PairWeights, *, rotate: int = 1, act_prologue: int = PRO_PLAIN,
                 hidden_cols: Optional[slice] = None, exact: bool = False, bufs: Optional[dict] = None, chunks: int = 1,
                 comm_stream=None, act_form: str = "rot"):
        # act_form: where the activation of an MLP pair runs. "rot": with the rotation in the first GEMM's epilogue;
        # "epilogue": in the epilogue, the whole quantizer after it; "prologue": in the quantizer (the reference's arrangement)
        self.act_form = act_form
        self.ops, self.comm, self.w = ops, comm, weights
        self.rotate, self.pro, self.hidden_cols, self.exact = rotate, act_prologue, hidden_cols, exact
        self.bufs = bufs if bufs is not None else {}
        self.chunks, self.comm_stream = chunks, comm_stream
        self.ones = None

    def _buf(self, name, shape, dtype, like):
        """A persistent buffer on CUDA (keyed by name and shape, shared across pairs); None on CPU (the stand-in allocates)."""
        if like.device.type != "cuda":
            return None
        key = (name, tuple(shape), dtype)
        t = self.bufs.get(key)
        if t is None:
            t = self.bufs[key] = torch.empty(tuple(shape), dtype=dtype, device=like.device)
        return t

    def forward(self, x_local: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        ops, comm, w = self.ops, self.comm, self.w
        rows, F = x_local.shape
        M, dt, P = rows * comm.world, x_local.dtype, comm.world
        kw = {}
        if x_local.device.type == "cuda":
            kw = dict(q=self._buf("a8_local", (rows, F), torch.int8, x_local), scales=self._buf("xs_local", (rows,), torch.float32, x_local))
        a8, xs = ops.quant_rows(x_local, PRO_PLAIN, self.rotate, **kw)
        a8 = comm.all_gather_rows(a8, self._buf("a8", (M, F), torch.int8, x_local) if P > 1 else None)
        xs = comm.all_gather_rows(xs, self._buf("xs", (M,), torch.float32, x_local) if P > 1 else None)
        n1 = w.w1.shape[0]
        cuda = x_local.device.type == "cuda"
        # Activation and rotation in the column-parallel GEMM's epilogue, the quantizer's second pass after it (same codes
        # and scales as the plain GEMM followed by the quantizer with that prologue). Not in exact mode, whose row maxima
        # are reduced across the ranks between the quantizer's two passes.
        act = _ACT_OF_PROLOGUE.get(self.pro, 0)
        fused = (cuda and act and self.rotate and not self.exact and self.hidden_cols is None and dt == torch.bfloat16
                 and n1 % 256 == 0 and F % 16 == 0 and hasattr(ops, "int8_gemm_act_rot") and self.act_form == "rot")
        in_epilogue = cuda and act and not fused and not self.exact and self.hidden_cols is None and self.act_form == "epilogue"
        if fused:
            h, parts = ops.int8_gemm_act_rot(a8, w.w1, xs, w.s1, w.b1, act=act, out=self._buf("h", (M, n1), dt, x_local),
                                             amax_part=self._buf("parts", (n1 // 64, M), torch.float32, x_local))
        elif in_epilogue:
            h = ops.int8_gemm(a8, w.w1, xs, w.s1, w.b1, out_dtype=dt, act=act, out=self._buf("h", (M, n1), dt, x_local))
        else:
            h = ops.int8_gemm(a8, w.w1, xs, w.s1, w.b1, out_dtype=dt, out=self._buf("h", (M, n1), dt, x_local))   # [M, N1 / P]
        if self.hidden_cols is not None:
            h = h[:, self.hidden_cols]            # a view: the quantizers take the row stride
        kh, n2 = h.shape[1], w.w2.shape[0]
        if self.ones is None:
            self.ones = torch.ones(n2, dtype=dt, device=x_local.device)
        if out is None:
            out = self._buf("out_" + ("a" if self.hidden_cols is not None else "m"), (rows, n2), dt, x_local)
        if self.exact:
            amax = comm.all_reduce_max(ops.quant_rows_amax(h, self.pro, self.rotate, **(dict(out=self._buf("amax", (M,), torch.float32, x_local)) if cuda else {})))
            qkw = dict(q=self._buf("a2", (M, kh), torch.int8, x_local), scales=self._buf("xs2", (M,), torch.float32, x_local)) if cuda else {}
            a2, xs2 = ops.quant_rows_scaled(h, amax, self.pro, self.rotate, **qkw)
            acc = ops.int8_gemm_acc_i32(a2, w.w2, out=self._buf("acc", (M, n2), torch.int32, x_local))
            acc = comm.reduce_scatter_rows(acc, self._buf("acc_local", (rows, n2), torch.int32, x_local) if P > 1 else None)  # int32 [M / P, N2]
            xs2_local = xs2[comm.rank * rows:(comm.rank + 1) * rows]
            return ops.int8_epilogue(acc, xs2_local, w.s2, w.b2, out_dtype=dt, rscale=self.ones, resid=x_local, out=out)
        qkw = dict(q=self._buf("a2", (M, kh), torch.int8, x_local), scales=self._buf("xs2", (M,), torch.float32, x_local)) if cuda else {}
        if fused:
            a2, xs2 = ops.quant_rows_rotated(h, parts, **qkw)
        else:
            a2, xs2 = ops.quant_rows(h, PRO_PLAIN if in_epilogue else self.pro, self.rotate, **qkw)
        C = self.chunks if (cuda and P > 1 and self.comm_stream is not None and n2 % (8 * self.chunks) == 0) else 1
        if C == 1:
            part = ops.int8_gemm(a2, w.w2, xs2, w.s2, None, out_dtype=dt, out=self._buf("part", (M, n2), dt, x_local))   # partial sums, all rows
            y = comm.reduce_scatter_rows(part, self._buf("y", (rows, n2), dt, x_local) if P > 1 else None)
            return ops.bias_residual_add(y, w.b2, x_local, out=out)
        # column blocks of the row-parallel GEMM, each reduce-scattered on the communication stream while the next one runs
        nc = n2 // C
        cur = torch.cuda.current_stream()
        ys, done = [], []
        for c in range(C):
            part = ops.int8_gemm(a2, w.w2[c * nc:(c + 1) * nc], xs2, w.s2[c * nc:(c + 1) * nc], None, out_dtype=dt,
                                 out=self._buf(f"part{c}", (M, nc), dt, x_local))
            ready = torch.cuda.Event()
            ready.record(cur)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                ys.append(comm.reduce_scatter_rows(part, self._buf(f"y{c}", (rows, nc), dt, x_local)))
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
                done.append(ev)
        for c in range(C):
            cur.wait_event(done[c])
            ops.bias_residual_add(ys[c], w.b2, x_local, out=out, n0=c * nc)
        return out


class TPBlock:
    """The linears of one MMDiT block: joint QKV -> (attention taken as identity on V) -> out, and MLP up -> down, plus
    the adaLN modulation linear (M = 1, hidden -> 6 x hidden, weight-streaming; column-parallel with no exchange: every
    rank computes its slice of the modulation vector, which the block's own ranks would consume)."""

    def __init__(self, ops, comm: Comm, attn: PairWeights, mlp: PairWeights, exact: bool = False, bufs: Optional[dict] = None,
                 chunks: int = 1, comm_stream=None, adaln=None, act_form: str = "rot"):
        v_cols = attn.w2.shape[1]
        self.ops, self.adaln = ops, adaln
        self.bufs = bufs if bufs is not None else {}
        common = dict(exact=exact, bufs=self.bufs, chunks=chunks, comm_stream=comm_stream)
        self.attn = TPPair(ops, comm, attn, rotate=1, act_prologue=PRO_PLAIN, hidden_cols=slice(2 * v_cols, 3 * v_cols), **common)
        self.mlp = TPPair(ops, comm, mlp, rotate=1, act_prologue=PRO_GELU_TANH, act_form=act_form, **common)

    def forward(self, x_local: torch.Tensor, cond: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.adaln is not None and cond is not None:
            wq, ws, b = self.adaln
            key = ("mod", tuple(wq.shape))
            c8 = self.bufs.get(key)
            if c8 is None:
                c8 = self.bufs[key] = (torch.empty((1, wq.shape[1]), dtype=torch.int8, device=cond.device),
                                       torch.empty((1,), dtype=torch.float32, device=cond.device),
                                       torch.empty((1, wq.shape[0]), dtype=cond.dtype, device=cond.device))
            q, sc = self.ops.quant_rows(cond, 5, 1, q=c8[0], scales=c8[1])          # SiLU prologue, as the DiTs' modulation does
            self.ops.int8_gemm(q, wq, sc, ws, b, out_dtype=cond.dtype, out=c8[2])
        # two output buffers alternate so that a pair never writes the rows it still reads as its residual
        mid = self.attn.forward(x_local)
        return self.mlp.forward(mid)


# ---- benchmark legs ---------------------------------------------------------------------------------------------------
STACK_M, STACK_F, STACK_MLP = 16896, 3072, 12288          # the Qwen-Image-shaped MMDiT stack at 2048 x 2048
PEER_GBS = 770.0                                          # measured peer-copy bandwidth per direction per GPU on this pool


def stack_ops_per_block(M: int = STACK_M) -> float:
    F, MLP = STACK_F, STACK_MLP
    return 2.0 * M * (3 * F * F + F * F + MLP * F + F * MLP) + 2.0 * 6 * F * F      # four linears + adaLN (M = 1)


def link_model_ms(world: int, exact: bool, M: int = STACK_M) -> float:
    """Time per block the NVLink transfers alone need at the measured peer bandwidth: per pair, every rank receives the
    other ranks' int8 rows (+ scales) and sends (world - 1) / world of its partial outputs (bf16, or int32 in exact mode)."""
    if world == 1:
        return 0.0
    f = (world - 1) / world
    per_pair = f * M * (STACK_F + 4) + f * M * STACK_F * (4 if exact else 2) + (f * M * 4 if exact else 0)
    return 2 * per_pair / (PEER_GBS * 1e9) * 1e3


def run_stack(mode: str, rank: int, world: int, local: int, *, blocks: int = 60, steps: int = 3, warmup: int = 1,
              chunks: int = 3, gemm_clusters: int = 0, graph: bool = True, act_form: str = "rot") -> dict:
    """One of the three ways to run the 60-block linear stack (QKV, attention-out, MLP up / down with GELU-tanh, adaLN) on
    `world` GPUs, timed with CUDA events (maximum over ranks):
      token     tokens sharded over the ranks, weights replicated, no data-path collective
      tp_fast   column / row tensor parallelism, bf16 partial outputs reduce-scattered (overlapped in column blocks)
      tp_exact  the same with int32 accumulators reduce-scattered: bit-identical to one GPU
    Random int8 weights per block, generated on the device from one seed on every rank."""
    import torch.distributed as dist
    from . import linear as ops

    dev = torch.device("cuda", local)
    tp = mode != "token"
    exact = mode == "tp_exact"
    comm = Comm() if tp else Comm.__new__(Comm)
    if not tp:
        comm.dist, comm.group, comm.world, comm.rank = None, None, 1, 0
    M, F, MLP = STACK_M, STACK_F, STACK_MLP
    assert M % world == 0 and F // 256 >= world
    g = torch.Generator(device=dev).manual_seed(1234)          # same seed on every rank: identical full weights, then sliced

    def qweight(n, k):
        return (torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8, device=dev),
                torch.rand(n, generator=g, device=dev) * 2e-4 + 1e-5,
                (torch.randn(n, generator=g, device=dev) * 0.01).bfloat16())

    bufs: dict = {}
    comm_stream = torch.cuda.Stream(dev) if (tp and world > 1 and not exact and chunks > 1) else None
    stack: List[TPBlock] = []
    for _ in range(blocks):
        wqkv, sqkv, bqkv = qweight(3 * F, F)
        wo, so, bo = qweight(F, F)
        wu, su, bu = qweight(MLP, F)
        wd, sd, bd = qweight(F, MLP)
        wa, sa, ba = qweight(6 * F, F)
        r, w = (rank, world) if tp else (0, 1)
        attn = shard_pair(wqkv, sqkv, bqkv, wo, so, bo, r, w, hidden_of=(0, F))
        mlp = shard_pair(wu, su, bu, wd, sd, bd, r, w)
        n_mod = 6 * F // w                                       # the modulation vector's slice of this rank
        adaln = (wa[r * n_mod:(r + 1) * n_mod].contiguous(), sa[r * n_mod:(r + 1) * n_mod].contiguous(), ba[r * n_mod:(r + 1) * n_mod].contiguous())
        stack.append(TPBlock(ops, comm, attn, mlp, exact, bufs=bufs, chunks=chunks, comm_stream=comm_stream, adaln=adaln,
                             act_form=act_form))
        del wqkv, wo, wu, wd, wa
    rows = M // world
    x = torch.randn(rows, F, generator=torch.Generator(device=dev).manual_seed(99 + rank), device=dev).bfloat16()
    cond = torch.randn(1, F, generator=torch.Generator(device=dev).manual_seed(7), device=dev).bfloat16()
    if comm_stream is not None and gemm_clusters > 0:
        ops.set_gemm_cluster_limit(gemm_clusters)

    def one_pass():
        h = x
        for b in stack:
            h = b.forward(h, cond)
        return h

    one_pass()                                                  # lazy set-up (tables, scratch, buffers) before any capture
    torch.cuda.synchronize()
    run, graphed = one_pass, False
    if graph and (world == 1 or not tp):                        # no collective inside: the whole pass replays as one CUDA graph
        try:
            side = torch.cuda.Stream(dev)
            with torch.cuda.stream(side):
                cg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(cg, stream=side):
                    one_pass()
            torch.cuda.synchronize()
            run, graphed = cg.replay, True
        except Exception:                                       # capture is an optimisation only
            torch.cuda.synchronize()
            run, graphed = one_pass, False
    for _ in range(warmup):
        run()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier(device_ids=[local])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ops.set_gemm_cluster_limit(0)
    status = ops.kernel_status()
    del stack, bufs
    torch.cuda.empty_cache()
    tops = stack_ops_per_block() * blocks / (ms * 1e-3) / 1e12
    launches = blocks * ((12 if exact else 10 + (2 * (chunks - 1) if comm_stream is not None else 0)) + 2)
    return {"mode": mode, "blocks": blocks, "stack_ms": ms, "dit_block_gemm_ms": ms / blocks, "tops": tops, "cuda_graph": graphed,
            "link_model_ms_per_block": link_model_ms(world if tp else 1, exact), "launches_per_pass": launches,
            "kernel_status": status}


def bench_main(args, rank, world, local, metric, unit):
    """`bench.py --mode tp`: the stack under tensor parallelism alone (BENCH_TP_EXACT=1 for the exact mode), one JSON line."""
    import os
    import torch.distributed as dist
    mode = "tp_exact" if os.environ.get("BENCH_TP_EXACT", "0") == "1" else "tp_fast"
    r = run_stack(mode, rank, world, local, blocks=int(os.environ.get("BENCH_TP_BLOCKS", "60")), steps=args.steps,
                  warmup=max(1, args.warmup), chunks=int(os.environ.get("BENCH_TP_CHUNKS", "3")),
                  gemm_clusters=int(os.environ.get("BENCH_TP_CLUSTERS", "66")))
    if rank == 0:
        print(json.dumps({"metric": metric, "value": r["tops"], "unit": unit, "n_gpus": world, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": r["stack_ms"], "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                          "config": {"workload": f"mmdit_linear_stack_{r['blocks']}blocks_M16896_hidden3072", "parallelism": f"tp{world}",
                                     **{k: r[k] for k in ("mode", "dit_block_gemm_ms", "link_model_ms_per_block", "cuda_graph")}},
                          "gpu_launches": args.steps * r["launches_per_pass"], "kernel_status": r["kernel_status"]}), flush=True)
    if world > 1:
        dist.destroy_process_group()
