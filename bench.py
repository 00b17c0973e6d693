#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-gpu] [--mode replicas|tp]

One step = one pass of the path over one batch of the ConvRot int8 MMDiT MLP pair (Qwen-Image-shaped block at
1024x1024: M = 4352 tokens, 3072 -> 12288 with GELU-tanh, 12288 -> 3072 with the residual add):
    quantize rows (rotate) -> int8 GEMM whose epilogue applies GELU-tanh and the next quantizer's rotation -> the
    quantizer's second pass (row maximum, scale, codes) -> int8 GEMM + residual epilogue
(--act-epilogue: GELU in the epilogue, the whole quantizer after it; --unfused-gelu: the reference's arrangement, plain
epilogue and the GELU in the next quantizer's prologue; all three give the same bits)
Inputs are seeded synthetic tensors with the block's shapes and distributions (no checkpoint is available offline).

Prints ONE JSON line. `value` is whole-job tera-ops/s (2*M*N*K per linear) with inputs resident in HBM; `e2e` is the
same metric through the host-facing call with the activations copied from pinned host memory and the result copied
back inside the timed region; `roofline` describes the dominant kernel (the up-projection GEMM) against the tensor
peak; `cpu_baseline` is the CPU oracle timed on a bounded row sample of the same workload.

--impl reference times that CPU restatement of the reference's arithmetic on the host cores (the reference has no
CPU implementation of this path; its own code is CUDA). --impl reference-gpu times the reference's own CUDA kernels,
compiled unmodified for sm_100a (oracle/_ref/libref.so), on the same GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CHAIN_BLOCKS = 60       # blocks between one host-to-device and one device-to-host copy in the chained end-to-end leg
SETTLE_S = 1.2          # untimed back-to-back load before the timed steps (see main)
METRIC = "w8a8_linear_tops"
UNIT = "TOPS"
WORKLOAD = "convrot_int8_mmdit_mlp_pair_M4352_K3072_N12288"
INT8_NOMINAL_TOPS = 4500.0
# the same `config` in both arms: what is computed, not how
CONFIG = {"workload": WORKLOAD, "step": "quant(R256) -> gemm -> gelu -> quant(R256) -> gemm+residual", "tokens_per_gpu": 4352}


# --mode kernel: one kernel of the step alone, on the step's own buffers (what profiles/ summarises)
KERNELS = {
    "quant_rot": lambda b, I: I.quant_rows(b.h, 0, 1, q=b.a2, scales=b.xs2),             # M=4352 K=12288, PLAIN + R256
    "quant_gelu": lambda b, I: I.quant_rows(b.h, 11, 1, q=b.a2, scales=b.xs2),           # the same with the GELU-tanh prologue
    "quant_in": lambda b, I: I.quant_rows(b.x, 0, 1, q=b.a1, scales=b.xs1),              # M=4352 K=3072
    "gemm_up": lambda b, I: I.int8_gemm(b.a1, b.w1, b.xs1, b.s1, b.b1, out=b.h),         # M=4352 K=3072 N=12288
    "gemm_up_act": lambda b, I: I.int8_gemm(b.a1, b.w1, b.xs1, b.s1, b.b1, act=1, out=b.h),
    # the activation and the rotation in the epilogue, and the quantizer pass that is left after it
    "gemm_up_rot": lambda b, I: I.int8_gemm_act_rot(b.a1, b.w1, b.xs1, b.s1, b.b1, act=1, out=b.h, amax_part=b.parts),
    "quant_rotated": lambda b, I: I.quant_rows_rotated(b.h, b.parts, q=b.a2, scales=b.xs2),
    "gemm_down": lambda b, I: I.int8_gemm(b.a2, b.w2, b.xs2, b.s2, b.b2, rscale=b.ones, resid=b.x, out=b.out),
    "gemm_down_plain": lambda b, I: I.int8_gemm(b.a2, b.w2, b.xs2, b.s2, b.b2, out=b.out),      # the same without the residual
    # the up-projection with its weight in W6 storage (fitted group scales / s_rel = 1), unpacked inside the GEMM
    "w6a8_up": lambda b, I: I.w6a8_gemm(b.a1, b.w6[0], b.w6[1], b.xs1, b.w6[2], b.b1, out=b.h),
    "w6a8_up_unit": lambda b, I: I.w6a8_gemm(b.a1, b.w6u[0], b.w6u[1], b.xs1, b.w6u[2], b.b1, out=b.h),
}


# Kernels outside the step, HBM-bound: set-up (returns the algorithmic bytes of one launch) and the launch itself.
def _setup_hbm(name, b, torch, dev, wl, I):
    g = torch.Generator(device=dev).manual_seed(11)
    rnd = lambda *shape: torch.randn(*shape, generator=g, device=dev)
    if name in ("pack_f32", "pack_bf16"):                        # quantize-at-load of an MLP-up weight (gpu_convrot_requant, seed 0)
        N, K, esz = 12288, 3072, 4 if name == "pack_f32" else 2
        b.hw = (rnd(N, K) * 0.02).to(torch.float32 if esz == 4 else torch.bfloat16)
        return esz * N * K + N * K + 4 * N
    if name == "sd_quant":                                       # fp16 rows, R256: activations at run time, weights at load
        M, K = 32768, 2560
        b.hx = rnd(M, K).half()
        return 3 * M * K + 4 * M
    if name == "w6_requant":                                     # the W6 packer (bf16 weight -> two-plane 6-bit + e4m3 group scales)
        N, K = 13824, 5120
        b.hw = (rnd(N, K) * 0.015).bfloat16()
        return 2 * N * K + N * K * 3 // 4 + N * K // 32 + 4 * N
    if name == "w6_decode":
        N, K = 13824, 5120
        b.h6 = I.w6_requant((rnd(N, K) * 0.015).bfloat16(), 1)
        return N * K * 3 // 4 + N * K // 32 + N * K
    if name == "adaln":                                          # few-rows weight-streaming GEMM: M = 1, 3072 -> 18432
        N, K = 18432, 3072
        b.ha = torch.randint(-128, 128, (1, K), generator=g, dtype=torch.int8, device=dev)
        b.hw = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8, device=dev)
        b.hs = (torch.rand(1, generator=g, device=dev) * 0.01, torch.rand(N, generator=g, device=dev) * 1e-3, rnd(N).bfloat16())
        b.hd = torch.empty((1, N), dtype=torch.bfloat16, device=dev)
        return N * K + K + 4 + 4 * N + 2 * N + 2 * N
    if name in ("wo8_linear", "wo8_fp32_flow"):                  # a text-encoder MLP-up linear: 512 tokens, 2560 -> 19456
        M, K, N = 512, 2560, 19456
        b.tx = rnd(M, K)
        b.tw = I.convrot_requant(rnd(N, K) * 0.03, 0)
        b.tout = torch.empty((M, N), dtype=torch.float32, device=dev)
        b.tscr = (torch.empty(4 * M * K, dtype=torch.uint8, device=dev), torch.empty(2 * N * K, dtype=torch.uint8, device=dev))
        return None
    raise KeyError(name)


def _fp32_flow(b, I):
    """The reference's arrangement of the weight-only linear: rotate, dequantize the whole weight to f32, fp32 GEMM (a library
    GEMM stands in for its cuBLASLt call: a baseline beside gpu_wo8_linear, not part of the product path)."""
    import torch
    torch.matmul(I.rotate_rows_f32(b.tx), I.dequant_i8(*b.tw).t(), out=b.tout)


HBM_KERNELS = {
    "wo8_linear": lambda b, I: I.wo8_linear(b.tx, b.tw[0], b.tw[1], out=b.tout, scratch=b.tscr),
    "wo8_fp32_flow": _fp32_flow,
    "pack_f32": lambda b, I: I.convrot_requant(b.hw, 0),
    "pack_bf16": lambda b, I: I.convrot_requant(b.hw, 0),
    "sd_quant": lambda b, I: I.sd_quant_rows(b.hx, 256),
    "w6_requant": lambda b, I: I.w6_requant(b.hw, 1),
    "w6_decode": lambda b, I: I.w6_decode(b.h6[0], b.h6[1], 5120),
    "adaln": lambda b, I: I.int8_gemm(b.ha, b.hw, b.hs[0], b.hs[1], b.hs[2], out=b.hd),
}
QUANT_BYTES = {"quant_rot": 3 * 4352 * 12288, "quant_gelu": 3 * 4352 * 12288, "quant_in": 3 * 4352 * 3072,
               "quant_rotated": 3 * 4352 * 12288 + 4 * 4352 * (12288 // 64)}      # rows in, codes out, partial maxima in


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--mode", default="replicas", choices=["replicas", "tp", "kernel", "shapes"])
    ap.add_argument("--kernel", default="gemm_up", choices=sorted(list(KERNELS) + list(HBM_KERNELS)),
                    help="--mode kernel: the one kernel to launch --steps times (the command ncu captures are taken from)")
    ap.add_argument("--cpu-rows", type=int, default=4352, help="rows of the batch the CPU baseline computes")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--unfused-gelu", action="store_true",
                    help="the reference's arrangement: plain GEMM epilogue, GELU-tanh in the next quantizer's prologue")
    ap.add_argument("--act-epilogue", action="store_true",
                    help="GELU-tanh in the up-projection's epilogue but the rotation in the quantizer (gpu_int8_gemm_act, then "
                         "gpu_quant_rows) instead of both in the epilogue (gpu_int8_gemm_act_rot, then gpu_quant_rows_rotated)")
    ap.add_argument("--gemm-clusters", type=int, default=0,
                    help="upper bound on the CTA pairs a GEMM launch occupies (gpu_int8_gemm_set_cluster_limit; 0 = the library's choice)")
    ap.add_argument("--no-stack", action="store_true", help="skip the 60-block stack record")
    ap.add_argument("--settle-s", type=float, default=SETTLE_S, help="seconds of untimed back-to-back load before the timed steps")
    ap.add_argument("--stack-blocks", type=int, default=60)
    return ap.parse_args()


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ---- workload -----------------------------------------------------------------------------------------------------
def host_inputs(wl, seed_base: int):
    """Seeded host tensors of the MLP pair: activations, fp32 weights, biases."""
    up, down = wl.config(1)
    x = wl.activations(up.M, up.K, 1002 + seed_base, outliers="student")
    w1 = wl.weight(up.N, up.K, 2021, 0.02)
    w2 = wl.weight(down.N, down.K, 2022, 0.02)
    b1 = wl.bias(up.N, 3021)
    b2 = wl.bias(down.N, 3022)
    return up, down, x, w1, w2, b1, b2


class Block:
    """Device state of one MLP pair and the four kernel launches of a step, through `impl` (the product's
    host layer, or the binding of the reference's CUDA kernels: both expose the same calls)."""

    def __init__(self, impl, torch, dev, up, down, x, w1, w2, b1, b2, fused_gelu: bool, rot_epilogue: bool = False):
        self.impl, self.torch, self.fused_gelu, self.rot_epilogue = impl, torch, fused_gelu, rot_epilogue
        self.up, self.down = up, down
        self.x = x.to(dev)
        # quantize-at-load: f32 weights -> R256 -> int8 + per-channel scale (seed 0 = nearest)
        self.w1, self.s1 = impl.convrot_requant(w1.to(dev), 0)
        self.w2, self.s2 = impl.convrot_requant(w2.to(dev), 0)
        self.b1, self.b2 = b1.to(dev), b2.to(dev)
        self.ones = torch.ones(down.N, dtype=torch.bfloat16, device=dev)          # rscale of the residual form
        # ... and the gate of the chained leg: an ungated branch added 60 times over drives the residual stream out of the
        # input's distribution (the models gate the branch by their modulation vector: rscale of src/qwen21.rs:416)
        self.gate = torch.full((down.N,), 0.125, dtype=torch.bfloat16, device=dev)
        M = up.M
        self.a1 = torch.empty((M, up.K), dtype=torch.int8, device=dev)
        self.xs1 = torch.empty((M,), dtype=torch.float32, device=dev)
        self.h = torch.empty((M, up.N), dtype=torch.bfloat16, device=dev)
        self.parts = torch.empty((up.N // 64, M), dtype=torch.float32, device=dev)
        self.a2 = torch.empty((M, down.K), dtype=torch.int8, device=dev)
        self.xs2 = torch.empty((M,), dtype=torch.float32, device=dev)
        self.out = torch.empty((M, down.N), dtype=torch.bfloat16, device=dev)
        self.launches_per_step = 4

    def step(self, x=None, out=None, rscale=None):
        I = self.impl
        x = self.x if x is None else x
        out = self.out if out is None else out
        rscale = self.ones if rscale is None else rscale
        I.quant_rows(x, 0, 1, q=self.a1, scales=self.xs1)
        if self.rot_epilogue:
            I.int8_gemm_act_rot(self.a1, self.w1, self.xs1, self.s1, self.b1, act=1, out=self.h, amax_part=self.parts)
            I.quant_rows_rotated(self.h, self.parts, q=self.a2, scales=self.xs2)
        elif self.fused_gelu:
            I.int8_gemm(self.a1, self.w1, self.xs1, self.s1, self.b1, act=1, out=self.h)
            I.quant_rows(self.h, 0, 1, q=self.a2, scales=self.xs2)
        else:   # the reference's arrangement: plain epilogue, GELU in the next quantizer's prologue
            I.int8_gemm(self.a1, self.w1, self.xs1, self.s1, self.b1, out=self.h)
            I.quant_rows(self.h, 11, 1, q=self.a2, scales=self.xs2)
        I.int8_gemm(self.a2, self.w2, self.xs2, self.s2, self.b2, rscale=rscale, resid=x, out=out)

    def ops(self) -> float:
        return self.up.ops + self.down.ops


class RefImpl:
    """The reference's CUDA kernels behind the call names Block uses (no activation epilogue exists there)."""

    def __init__(self, R):
        self.R = R

    def convrot_requant(self, w, seed):
        return self.R.convrot_requant(w, seed)

    def quant_rows(self, x, pro, rot, q=None, scales=None):
        self.R.quant_rows(x, pro, rot, q=q, scales=scales)

    def sd_quant_rows(self, x, rot):
        return self.R.sd_quant_rows(x, rot)

    def int8_gemm(self, A, W, xs, ws, bias, act=0, rscale=None, resid=None, out=None):
        assert act == 0
        return self.R.int8_gemm(A, W, xs, ws, bias, rscale=rscale, resid=resid, out=out)


def run_shapes(torch, wl, impl, dev, tag):
    """--mode shapes: every linear of the five benchmark configurations alone (GEMM with bias in the configuration's
    activation dtype, and the quantizer that feeds it), one JSON line each. Operands smaller than the L2 are timed one
    launch at a time with a 256 MB buffer read in between (a read leaves clean lines behind; after a written buffer the
    timed kernel also pays for the write-back of the dirty lines it evicts)."""
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    sink = torch.zeros((), device=dev)

    def timed(fn, small, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if not small:
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / iters * 1e3
        tot = 0.0
        for _ in range(iters):
            sink.copy_(flush.sum())
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        return tot / iters * 1e3

    for ci in range(5):
        specs = wl.config(ci) + (wl.config(2, 6144) if ci == 2 else [])
        for sp in specs:
            M, K, N, dt = sp.M, sp.K, sp.N, sp.act_dtype
            A = torch.randint(-128, 128, (M, K), dtype=torch.int8, device=dev)
            W = torch.randint(-128, 128, (N, K), dtype=torch.int8, device=dev)
            xs, ws = torch.rand(M, device=dev) * 0.01, torch.rand(N, device=dev) * 0.001
            bias, D = torch.randn(N, device=dev).to(dt), torch.empty(M, N, dtype=dt, device=dev)
            small = (M * K + N * K + M * N * D.element_size()) < 126e6
            us = timed(lambda: impl.int8_gemm(A, W, xs, ws, bias, out=D), small)
            line = {"impl": tag, "cfg": ci, "linear": sp.name, "M": M, "K": K, "N": N, "out": str(dt).split(".")[-1],
                    "gemm_us": us, "tops": 2.0 * M * N * K / us / 1e6, "frac_of_4500": 2.0 * M * N * K / us / 1e6 / INT8_NOMINAL_TOPS,
                    "gemm_gbs": (M * K + N * K + M * N * D.element_size()) / us / 1e3, "l2_flushed": small}
            if K % 256 == 0 and dt == torch.bfloat16 and M > 1:
                X = torch.randn(M, K, device=dev).to(dt)
                Q, S = torch.empty(M, K, dtype=torch.int8, device=dev), torch.empty(M, device=dev)
                qus = timed(lambda: impl.quant_rows(X, 0, 1 if sp.rotate else 0, q=Q, scales=S), small)
                line.update(quant_us=qus, quant_gbs=3.0 * M * K / qus / 1e3)
            elif dt == torch.float16:
                X = torch.randn(M, K, device=dev).half()
                qus = timed(lambda: impl.sd_quant_rows(X, sp.rotate), small)
                line.update(quant_us=qus, quant_gbs=3.0 * M * K / qus / 1e3)
            print(json.dumps(line), flush=True)
            del A, W, D


def time_steps(torch, fn, steps: int, warmup: int, barrier=None):
    """W warm-up steps, then exactly `steps` timed with CUDA events on the current stream; returns milliseconds."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return e0.elapsed_time(e1)


def cpu_baseline(wl, rows: int):
    """The CPU oracle on the first `rows` rows of the batch (weights quantized once, outside the timed part)."""
    import torch
    from oracle import oracle as O
    O.use_all_cores()
    up, down, x, w1, w2, b1, b2 = host_inputs(wl, 0)
    rows = min(rows, up.M)
    xr = x[:rows].contiguous()
    wq1, s1 = O.convrot_requant(w1, 0)
    wq2, s2 = O.convrot_requant(w2, 0)
    ones = torch.ones(down.N, dtype=torch.bfloat16)
    t0 = time.perf_counter()
    a1, xs1 = O.quant_rows(xr, O.PRO_PLAIN, 1)
    h = O.int8_gemm(a1, wq1, xs1, s1, b1, act=1, contract=7)
    a2, xs2 = O.quant_rows(h, O.PRO_PLAIN, 1)
    O.int8_gemm(a2, wq2, xs2, s2, b2, ones, xr, contract=3)
    dt = time.perf_counter() - t0
    ops = 2.0 * rows * (up.N * up.K + down.N * down.K)
    return {"value": ops / dt / 1e12, "unit": UNIT, "cores": O.num_threads(), "kind": "port",
            "sample": f"first {rows} of {up.M} rows of the batch, both linears with their quantizers and epilogues, "
                      f"{dt:.1f} s on the host cores (weights packed beforehand)"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("bf16_tflops"), d.get("bf16_tflops_sustained"), d.get("hbm_gbs"), "measured"
    return 1590.0, 1400.0, 6650.0, "fallback"


def load_workloads():
    """workloads.py by file path: the CPU arm needs the shapes and seeded inputs, not the CUDA library the package loads."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("cbr_b200_workloads", os.path.join(ROOT, "comfyui-backend-but-rust_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod            # dataclasses look their module up by name
    spec.loader.exec_module(mod)
    return mod


def run_reference_cpu(args, rank):
    """The reference arm: the CPU restatement of the reference's arithmetic on the host cores, rank 0 only."""
    if rank != 0:
        return
    wl = load_workloads()
    vals, base = [], None
    for i in range(max(1, min(args.steps, 3))):       # each step is seconds of CPU work: at most three are timed
        base = cpu_baseline(wl, args.cpu_rows)
        vals.append(base["value"])
    v = sum(vals) / len(vals)
    base["value"] = v
    up, down = wl.config(1)
    ms = 2.0 * args.cpu_rows * (up.N * up.K + down.N * down.K) / (v * 1e12) * 1e3
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": len(vals),
                      "warmup": 0, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "int8", "data": "synthetic", "config": dict(CONFIG), "rows_per_step": args.cpu_rows,
                      "cpu_baseline": base,
                      "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)


def profiled_dram_bytes(rotating: bool = False):
    """DRAM bytes (read + write) of one launch of the dominant kernel, from the record line of the committed ncu summary
    of the kernel form the step runs ("dram_bytes_per_launch: <read> + <write>" in profiles/gemm_i8_pair_mlp_up.md or
    profiles/gemm_i8_pair_rotating_epilogue_mlp_up.md); None when the summary is absent."""
    import re
    name = "gemm_i8_pair_rotating_epilogue_mlp_up.md" if rotating else "gemm_i8_pair_mlp_up.md"
    try:
        text = open(os.path.join(ROOT, "profiles", name)).read()
    except OSError:
        return None
    m = re.search(r"dram_bytes_per_launch:\s*([0-9.eE+]+)\s*\+\s*([0-9.eE+]+)", text)
    return float(m.group(1)) + float(m.group(2)) if m else None


def main():
    args = parse_args()
    rank, world, local = dist_env()
    if args.impl == "reference":
        run_reference_cpu(args, rank)
        return
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    import importlib
    wl = importlib.import_module("cbr_b200.workloads")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the path has no CPU fallback (use --impl reference for the CPU oracle)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    barrier = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        barrier = lambda: dist.barrier(device_ids=[local])
    if args.mode == "tp":
        tp = importlib.import_module("cbr_b200.tensor_parallel")
        tp.bench_main(args, rank, world, local, METRIC, UNIT)
        return

    if args.impl == "reference-gpu":
        from oracle import ref as R
        if not R.available():
            if rank == 0:
                print(json.dumps({"impl": "reference-gpu", "unavailable": "oracle/_ref/libref.so is not built"}))
            return
        impl, fused = RefImpl(R), False
    else:
        impl, fused = pkg.linear, not args.unfused_gelu

    if args.mode == "shapes":
        if rank == 0:
            run_shapes(torch, wl, impl, dev, args.impl)
        return

    # token-sharded replicas: every rank owns one batch of the block (weights replicated), no data-path collective
    up, down, x, w1, w2, b1, b2 = host_inputs(wl, rank)
    rot = fused and not args.act_epilogue and args.impl != "reference-gpu"
    if args.gemm_clusters and args.impl != "reference-gpu":
        pkg.linear.set_gemm_cluster_limit(args.gemm_clusters)
    blk = Block(impl, torch, dev, up, down, x, w1, w2, b1, b2, fused, rot)
    if args.mode == "kernel":
        # the rotated rows and their partial maxima in h / parts for the second pass; the GELU output for the others
        blk.rot_epilogue = args.kernel == "quant_rotated"
        blk.step()                                   # fills every buffer the single kernels read
        if args.kernel.startswith("w6a8"):
            blk.w6 = tuple(t.to(dev) for t in wl.w6_pack(w1, True))
            blk.w6u = tuple(t.to(dev) for t in wl.w6_pack(w1, False))
        nbytes = QUANT_BYTES.get(args.kernel)
        if args.kernel in HBM_KERNELS:
            nbytes = _setup_hbm(args.kernel, blk, torch, dev, wl, impl)
            fn = HBM_KERNELS[args.kernel]
        else:
            fn = KERNELS[args.kernel]
        out = {"kernel": args.kernel, "launches": args.steps}
        if nbytes is not None and nbytes < 200e6:
            # operands that would stay in the 126 MB L2 between launches: one launch at a time, a 256 MB buffer read in between
            flush = torch.zeros(64 * 1024 * 1024, device=dev)
            sink = torch.zeros((), device=dev)
            for _ in range(args.warmup):
                fn(blk, impl)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            tot = 0.0
            for _ in range(args.steps):
                sink.copy_(flush.sum())
                e0.record(); fn(blk, impl); e1.record()
                torch.cuda.synchronize()
                tot += e0.elapsed_time(e1)
            k_ms = tot / args.steps
            out["l2"] = "flushed by a 256 MB read before every launch"
        else:
            k_ms = time_steps(torch, lambda: fn(blk, impl), args.steps, args.warmup) / args.steps
        out["us_per_launch"] = k_ms * 1e3
        if nbytes is not None:
            _, _, hbm, src = measured_peaks()
            out.update(algorithmic_bytes=nbytes, gbs=nbytes / (k_ms * 1e-3) / 1e9, frac_of_hbm=nbytes / (k_ms * 1e-3) / 1e9 / hbm,
                       hbm_peak_gbs=hbm, peak_source=src)
        out["kernel_status"] = pkg.linear.kernel_status()
        print(json.dumps(out), flush=True)
        return
    # A 1 kW part reaches its power-capped clock only after about a second of load, and a few dozen steps last milliseconds:
    # the warm-up therefore continues, untimed, until the step has run back to back for SETTLE_S seconds, and the K timed
    # steps follow without a pause, so that `value` is the sustained figure and the clock samples describe the same state.
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        blk.step()
    torch.cuda.synchronize()
    t_settle, settle_steps = time.perf_counter(), 0
    while time.perf_counter() - t_settle < args.settle_s:
        for _ in range(100):
            blk.step()
        torch.cuda.synchronize()
        settle_steps += 100
    ms = time_steps(torch, blk.step, args.steps, 0, barrier)
    tail_n = max(args.steps, 300) if args.settle_s > 0 else args.steps
    tail_ms = time_steps(torch, blk.step, tail_n, 0)                      # keeps the load up while the sampler takes its last samples
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        clocks["source"] = (f"sampled over {settle_steps} untimed settling steps ({args.settle_s} s), the {args.steps} timed steps "
                            f"and {tail_n} more steps right after them ({tail_ms / tail_n:.4f} ms per step)")
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = blk.ops() * world * args.steps / (ms * 1e-3) / 1e12

    # end to end: activations from pinned host memory, result back to pinned host memory, every step
    x_host = x.pin_memory()
    out_host = torch.empty((up.M, down.N), dtype=torch.bfloat16).pin_memory()

    def e2e_run(n):
        """n steps from host buffers to host buffers, each with its own H2D copy of the activations and D2H copy of the
        result, pipelined as a serving loop would: copy-in, compute and copy-out streams over two device buffer sets, so
        the copy of step i+1 and the read-back of step i-1 overlap the kernels of step i. Returns milliseconds."""
        s_in, s_comp, s_out = (torch.cuda.Stream(dev) for _ in range(3))
        xd = [torch.empty_like(blk.x) for _ in range(2)]
        od = [torch.empty_like(blk.out) for _ in range(2)]
        oh = [out_host, torch.empty_like(out_host).pin_memory()]
        h2d = [torch.cuda.Event() for _ in range(n)]
        comp = [torch.cuda.Event() for _ in range(n)]
        d2h = [torch.cuda.Event() for _ in range(n)]
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record(s_in)
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(comp[i - 2])          # the kernels of step i-2 have read this input buffer
                xd[b].copy_(x_host, non_blocking=True)
                h2d[i].record(s_in)
            with torch.cuda.stream(s_comp):
                s_comp.wait_event(h2d[i])
                if i >= 2:
                    s_comp.wait_event(d2h[i - 2])         # the result of step i-2 has left this output buffer
                blk.step(xd[b], od[b])
                comp[i].record(s_comp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp[i])
                oh[b].copy_(od[b], non_blocking=True)
                d2h[i].record(s_out)
        t1.record(s_out)
        torch.cuda.synchronize()
        return t0.elapsed_time(t1)

    e2e_run(min(args.warmup, 3) + 2)
    if barrier:
        barrier()
    e2e_ms = e2e_run(args.steps)
    if barrier:
        barrier()
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = blk.ops() * world * args.steps / (e2e_ms * 1e-3) / 1e12
    # The same path as the product drives it: a chain of CHAIN_BLOCKS blocks between one copy in and one copy out
    # (the reference uploads a step's input once and downloads once at its end, src/h3.rs:1361-1364). The blocks share
    # this block's weights; every block still runs its four kernels on the previous block's output, its MLP branch gated by
    # 1/8 so that the residual stream stays in the input's distribution over the 60 blocks.
    def chain_run(n):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        xa, xb = torch.empty_like(blk.x), torch.empty_like(blk.out)
        torch.cuda.synchronize()
        t0.record()
        for _ in range(n):
            xa.copy_(x_host, non_blocking=True)
            cur, nxt = xa, xb
            for _b in range(CHAIN_BLOCKS):
                blk.step(cur, nxt, blk.gate)
                cur, nxt = nxt, cur
            out_host.copy_(cur, non_blocking=True)
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1)

    chain_run(1)
    if barrier:
        barrier()
    chain_n = max(1, min(args.steps, 5))
    chain_ms = chain_run(chain_n)
    if world > 1:
        t = torch.tensor([chain_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        chain_ms = float(t.item())
    chain_value = blk.ops() * CHAIN_BLOCKS * world * chain_n / (chain_ms * 1e-3) / 1e12
    status = pkg.linear.kernel_status()

    # The 60-block stack of the scaling configuration (M = 16896 tokens at 2048 x 2048, adaLN linear included) on these N
    # GPUs: token-sharded, and under column / row tensor parallelism in both modes. Every rank takes part.
    dit_stack = None
    if args.impl == "ours" and not args.no_stack:
        tp = importlib.import_module("cbr_b200.tensor_parallel")
        dit_stack = {"workload": "mmdit_linear_stack_60blocks_M16896_hidden3072 (QKV, attention-out, MLP up/down, adaLN)",
                     "peer_gbs_assumed": tp.PEER_GBS, "runs": []}
        modes = ["token"] + (["tp_fast", "tp_exact"] if world > 1 and 12 % world == 0 else [])
        for mode in modes:
            dit_stack["runs"].append(tp.run_stack(mode, rank, world, local, blocks=args.stack_blocks, steps=2, warmup=1,
                                                  gemm_clusters=66))

    if rank != 0:
        return
    # roofline of the dominant kernel: the up-projection GEMM alone, as the step runs it, CUDA events over back-to-back launches
    blk.step()                                   # the timed step's own operands again (the chained leg left its last block's)
    def gemm_up():
        if rot:
            impl.int8_gemm_act_rot(blk.a1, blk.w1, blk.xs1, blk.s1, blk.b1, act=1, out=blk.h, amax_part=blk.parts)
        else:
            impl.int8_gemm(blk.a1, blk.w1, blk.xs1, blk.s1, blk.b1, act=1 if fused else 0, out=blk.h)
    k_ms = time_steps(torch, gemm_up, 20, 3) / 20
    plain_ms = time_steps(torch, lambda: impl.int8_gemm(blk.a1, blk.w1, blk.xs1, blk.s1, blk.b1, out=blk.h), 20, 3) / 20
    act_ms = time_steps(torch, lambda: impl.int8_gemm(blk.a1, blk.w1, blk.xs1, blk.s1, blk.b1, act=1, out=blk.h), 20, 3) / 20 if fused else None
    bf16_burst, bf16_sust, hbm, src = measured_peaks()
    achieved = up.ops / (k_ms * 1e-3) / 1e12
    peak = 2.0 * bf16_burst                      # dense int8 runs at twice the dense bf16 rate on this part
    form = ("GELU-tanh and the next quantizer's R256 rotation in the epilogue, as in the step: the epilogue's table look-ups "
            "and the tile loads share the SM's shared-memory bandwidth, so this kernel is slower than the plain one and the "
            "quantizer after it 2.3x faster)" if rot else "GELU-tanh epilogue as in the step)" if fused else "plain epilogue)")
    sub = lambda t: {"us_per_launch": t * 1e3, "achieved": up.ops / (t * 1e-3) / 1e12, "frac": up.ops / (t * 1e-3) / 1e12 / peak}
    roofline = {"bound": "tensor", "kernel": "gemm_i8_pair_kernel (mlp_up, M=4352 K=3072 N=12288, " + form, "achieved": achieved,
                "peak": peak, "unit": "TOPS", "frac": achieved / peak,
                "peak_source": f"2 x {src} dense bf16 burst ({bf16_burst} TFLOP/s); no int8 figure is measured on this pool",
                "frac_of_nominal_4500": achieved / INT8_NOMINAL_TOPS, "us_per_launch": k_ms * 1e3,
                "traffic": profiled_dram_bytes(rot),
                "plain_epilogue": sub(plain_ms)}
    if act_ms is not None:
        roofline["act_epilogue"] = sub(act_ms)
    if clocks and clocks.get("sm_mhz"):
        # time x the SM clock sampled under the sustained load: separates the kernel from the power-capped clock (the
        # roofline launches run in short bursts, so their own clock lies between this one and the maximum)
        roofline["kcycles_at_sampled_clock"] = {"sm_mhz": clocks["sm_mhz"], "as_in_step": k_ms * clocks["sm_mhz"],
                                                "plain_epilogue": plain_ms * clocks["sm_mhz"]}
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
            "data": "synthetic",
            "config": dict(CONFIG),
            "run": {"sharding": "tokens (replicated weights), no data-path collective", "fused_gelu_epilogue": fused, "rotating_epilogue": rot,
                    "l2": "working set per step ~300 MB exceeds the 126 MB L2",
                    "settle": f"{settle_steps} untimed steps ({args.settle_s} s) directly before the timed ones: value is the power-capped, sustained rate"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 2,
                    "pipelining": "every step copies its own input and output; copies of neighbouring steps overlap its kernels "
                                  "(three streams, two device buffer sets)",
                    "chain": {"value": chain_value, "unit": UNIT, "blocks_per_copy": CHAIN_BLOCKS, "ms_per_chain": chain_ms / chain_n,
                              "h2d_bytes_per_chain": x_host.numel() * 2, "d2h_bytes_per_chain": out_host.numel() * 2,
                              "what": "one copy in, 60 blocks back to back, one copy out: how the reference's engine drives the path"}},
            "gpu_launches": blk.launches_per_step * args.steps, "kernel_status": status, "roofline": roofline,
            "frac_of_nominal_int8_peak": value / world / INT8_NOMINAL_TOPS}
    if dit_stack is not None:
        line["dit_stack"] = dit_stack
    if args.impl == "reference-gpu":
        line["impl"] = "reference-gpu"
    else:
        # the incumbent on the same GPU: the reference's own CUDA kernels (CUTLASS 2.x mma.sync GEMM, its quantizer),
        # compiled unmodified for sm_100a, driving the same four launches on the same buffers
        try:
            from oracle import ref as R
            if R.available():
                inc = Block(RefImpl(R), torch, dev, up, down, x, w1, w2, b1, b2, False)
                inc_ms = time_steps(torch, inc.step, 20, 3) / 20
                line["incumbent"] = {"impl": "reference CUDA kernels compiled for sm_100a (oracle/_ref/libref.so)", "ms_per_step": inc_ms,
                                     "value": inc.ops() / (inc_ms * 1e-3) / 1e12, "unit": UNIT}
            else:
                line["incumbent"] = {"unavailable": "oracle/_ref/libref.so is not built"}
        except Exception as e:                                   # the checker's absence must not cost the bench line
            line["incumbent"] = {"unavailable": repr(e)[:200]}
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(wl, args.cpu_rows)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
