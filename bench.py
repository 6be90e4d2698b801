#!/usr/bin/env python
"""Benchmark of the prefill hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--format q4_0|mlx_4bit|...] [--m M]

One *step* is one pass of the hot path over one batch of synthetic input: the 8B-shape projection
Y[2048, 4096] = X[2048, 4096] . dequant(W[4096, 4096])^T with Q4_0 weights (the configuration the
headline metric is quoted on).  Inputs have the shapes and value distributions the benchmark
contract names (X ~ N(0,1) fp16; Q4_0 scale ~ U(0.005, 0.02), nibbles uniform) and are generated
from a fixed seed -- there is no dataset behind this benchmark.

Order of work follows the reference's router bench (bench_universal_router.mm:840-1018): verify, then
time.  Before a configuration is timed, sampled token rows of its output are compared with the CPU
verifier's double-precision gold and the result goes into the line as `parity`.

Timed region: K steps enqueued back to back on the library's stream, CUDA events on that stream,
a barrier and a device synchronise on both sides, the maximum over ranks; this is repeated for
BLOCKS blocks of K steps and the median block is reported (all block times are in the line).  Every
step uses the next of a ring of disjoint (X, W, Y) sets larger than the 126 MB L2, so no step finds
its operands in cache.  With N > 1 (launched by torchrun, one rank per GPU) every rank runs the
headline projection on its own token batch with replicated weights: data parallel, no data-path
collective, weak scaling; `value` is the aggregate over ranks.  What does shard is reported beside
it: `c4`, the ternary K=4096 -> N=14336 projection with its output columns split over the ranks (no
collective), and `layer`, the tensor-parallel 8B decoder layer (both strong scaling).

The printed JSON line also carries: `roofline` (achieved TFLOP/s of the GEMM kernel against the
measured dense-tensor peak), `sweep` (one device-timed row per benchmark configuration that fits
one GPU, each with its roofline fraction and parity), `e2e` (the same projection through the C ABI
with pinned host buffers: X copied to the device and Y copied back inside every timed step, weights
resident), `cpu_baseline` (the CPU verifier timed on the host cores on a bounded slab of the same
workload) and `clocks` (SM clock and throttle reasons sampled with nvidia-smi while the kernels run).

`--impl reference` times the reference's own CPU implementation of the path (its double-precision
verifier: oracle/_ref when it was built from the reference sources, else the restatement in oracle/)
on all host cores, on a bounded row slab of the same workload per step.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M, K, N = 2048, 4096, 4096
FLOPS_PER_STEP = 2.0 * M * N * K
BLOCKS = 5
FORMATS = {"q4_0": 0, "mlx_4bit": 1, "q4_k": 2, "ternary_1_58": 3, "var_rate_affine": 4, "exl3": 5, "prism_q2_0": 7,
           "mlx_4bit_g64": 100, "ternary_row": 101, "mlx_4bit_planar": 102}
FMT_NAME = {v: k for k, v in FORMATS.items()}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, only for the (format, M) pairs that have a committed
# ncu summary (K = N = 4096); every other row reports traffic null
NCU_TRAFFIC = {("q4_0", 2048): (26.3e6, "profiles/qgemm_q4_0_m2048.md"), ("q4_0", 33): (9.78e6, "profiles/qgemm_small_q4_0_m33.md"),
               ("var_rate_affine", 2048): (27.4e6, "profiles/qgemm_var_rate_m2048.md")}
LAYER = dict(M=2048, K=4096, H=32, Hkv=8, D=128, F=14336)
TOL = 1.0 / 128.0


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), float(d["hbm_gbs"]), "measured"
    return 1590.0, 1400.0, 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi sampling in the background while kernels run."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,utilization.gpu,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        rows = [[c.strip() for c in line.split(",")] for line in out.strip().splitlines() if line.count(",") >= 9]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}

        def num(s):
            try:
                return float(s)
            except ValueError:
                return 0.0
        busy = [r for r in rows if num(r[4]) >= 50.0] or rows
        reasons = set()
        for r in busy:
            for name, col in (("hw_slowdown", 6), ("hw_thermal_slowdown", 7), ("sw_thermal_slowdown", 8), ("sw_power_cap", 9)):
                if r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(num(r[1]) for r in busy), "sm_max_mhz": max(num(r[2]) for r in rows),
                "power_w_max": max(num(r[3]) for r in busy), "samples_under_load": len(busy), "samples": len(rows),
                "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------
# CPU legs (the only places that execute oracle/): the timed CPU baseline, and the parity checks
# that precede every timed configuration (oracle as the checker)
# ---------------------------------------------------------------------------------------------
def cpu_threads() -> int:
    """All host cores for the CPU verifier, whatever OMP_NUM_THREADS the launcher exported; returns the OpenMP team
    size the verifier really runs with."""
    import oracle as o
    return o.set_num_threads(0)


def cpu_slab(fmt: int, rows: int, use_ref: bool):
    import oracle as o
    X, W = o.baseline_inputs(fmt, rows, K, N, 1234)
    fn = (lambda: o.ref_gemm(fmt, X, W, N)) if use_ref else (lambda: o.gemm(fmt, X, W, N))
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0


def cpu_baseline(fmt: int, budget_s: float = 12.0) -> dict:
    import oracle as o
    cores = cpu_threads()
    use_ref = o.ref_lib() is not None and fmt in (0, 1, 2, 3, 4, 5)
    t = cpu_slab(fmt, 64, use_ref)                      # calibrate on 64 token rows (enough rows to keep every thread busy)
    rows = int(max(4, min(M, 64 * budget_s / max(t, 1e-3))))
    rows -= rows % 4
    t = cpu_slab(fmt, rows, use_ref)
    return {"value": 2.0 * rows * N * K / t / 1e12, "unit": "TFLOP/s", "cores": cores,
            "kind": "reference" if use_ref else "port",
            "sample": f"{rows} of {M} token rows x all {N} outputs, K={K}, double-precision verifier, {t:.2f} s, {cores} OpenMP threads"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle as o
    cores = cpu_threads()
    fmt = FORMATS[args.format]
    use_ref = o.ref_lib() is not None and fmt in (0, 1, 2, 3, 4, 5)
    t = cpu_slab(fmt, 4, use_ref)
    per_step_budget = max(0.2, min(8.0, 120.0 / max(1, args.steps + args.warmup)))
    rows = int(max(4, min(M, 4 * per_step_budget / max(t, 1e-3))))
    rows -= rows % 4
    for _ in range(args.warmup):
        cpu_slab(fmt, rows, use_ref)
    times = [cpu_slab(fmt, rows, use_ref) for _ in range(args.steps)]
    total = sum(times)
    flops = 2.0 * rows * N * K
    val = flops * args.steps / total / 1e12
    line = {"impl": "reference", "metric": f"W4 prefill projection throughput (8B shape, M={M})", "value": val, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic (seeded)",
            "config": {"workload": f"{args.format} projection K={K} N={N}, {rows}-row slab of M={M} per step", "format": args.format},
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "reference" if use_ref else "port",
                             "sample": f"each step: {rows} of {M} token rows x all {N} outputs, {cores} OpenMP threads "
                                       "(rank 0 only; the thread count is set explicitly, not taken from OMP_NUM_THREADS)"},
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def parity_of(Y: np.ndarray, gold64: np.ndarray, rows) -> dict:
    """Difference of fp16 outputs from the double-precision gold on the sampled rows: the largest, how many are over
    1/128 (the reference's tier-1 tolerance), and how many of those are also over one fp16 ulp of the gold."""
    d = np.abs(Y.astype(np.float64) - gold64)
    ulp = np.spacing(np.abs(gold64).astype(np.float16)).astype(np.float64)
    rms = float(np.sqrt(np.mean(gold64 ** 2)))
    return {"max_abs": float(d.max()), "over_1_128": int((d > TOL).sum()), "over_1_128_and_1ulp": int((d > np.maximum(TOL, ulp)).sum()),
            "outputs": int(d.size), "rows": [int(r) for r in rows], "gold_rms": rms,
            "ok": bool(np.all(np.isfinite(Y.astype(np.float32))) and np.all(d <= np.maximum(np.maximum(TOL, ulp), 2.0 ** -9 * rms)))}


# ---------------------------------------------------------------------------------------------
# synthetic inputs
# ---------------------------------------------------------------------------------------------
def synth_q4_0(n_rows: int, k: int, device, gen, scale_lo=0.005, scale_hi=0.02):
    """Random-init Q4_0 matrix generated on the device: uniform nibbles, fp16 scale ~ U(lo, hi)."""
    import torch
    nb = n_rows * (k // 32)
    blocks = torch.randint(0, 256, (nb, 18), dtype=torch.uint8, device=device, generator=gen)
    d = (torch.rand(nb, device=device, generator=gen) * (scale_hi - scale_lo) + scale_lo).to(torch.float16)
    blocks[:, 0:2] = d.view(torch.uint8).reshape(nb, 2)
    return blocks.reshape(-1)


def synth_w(fmt: int, k: int, n: int, rng) -> np.ndarray:
    """Seeded packed weights [n][k/blk] with the benchmark's value distributions.
    Q4_0: d ~ U(0.005, 0.02), uniform nibbles.  MLX: s ~ U(0.005, 0.02), b = -8s + U(-0.01, 0.01).  Q4_K: d ~ U(2e-4, 2e-3),
    dmin ~ U(1e-4, 1e-3), 6-bit sub-scales/minimums uniform.  Ternary: codes with p = (0.25, 0.5, 0.25), d ~ U(0.01, 0.05) per
    block, or per row for the planar layout.  Variable-rate / codebook: uniform payload bytes, header scales in the reference
    generator's ranges, bit depths 3,3,4,4,4,4,5,5 and the three permutations in turn.  Prism: uniform 2-bit codes."""
    def f16(a):
        return np.asarray(a, dtype=np.float16).view(np.uint8).reshape(-1, 2)
    if fmt == 0:
        nb = n * k // 32
        W = rng.integers(0, 256, (nb, 18), dtype=np.uint8)
        W[:, 0:2] = f16(rng.uniform(0.005, 0.02, nb))
    elif fmt == 1:
        nb = n * k // 32
        W = rng.integers(0, 256, (nb, 20), dtype=np.uint8)
        sc = rng.uniform(0.005, 0.02, nb)
        W[:, 0:2] = f16(sc)
        W[:, 2:4] = f16(-8.0 * sc + rng.uniform(-0.01, 0.01, nb))
    elif fmt == 2:
        nb = n * k // 256
        W = rng.integers(0, 256, (nb, 144), dtype=np.uint8)
        W[:, 0:2] = f16(rng.uniform(2e-4, 2e-3, nb))
        W[:, 2:4] = f16(rng.uniform(1e-4, 1e-3, nb))
    elif fmt == 3:
        nb = n * k // 32
        codes = rng.choice(np.array([0, 1, 2], dtype=np.uint32), size=(nb, 2, 16), p=[0.25, 0.5, 0.25])
        words = (codes << (2 * np.arange(16, dtype=np.uint32))).sum(axis=2, dtype=np.uint32)
        W = np.zeros((nb, 12), dtype=np.uint8)
        W[:, 0:2] = f16(rng.uniform(0.01, 0.05, nb))
        W[:, 4:12] = words.view(np.uint8).reshape(nb, 8)
    elif fmt == 4:
        nb = n * k // 256
        W = rng.integers(0, 256, (nb, 160), dtype=np.uint8)
        W[:, 0:2] = f16(rng.uniform(4e-4, 4e-3, nb))
        W[:, 2:4] = f16(rng.uniform(-0.005, 0.01, nb))
        W[:, 20:28] = np.array([(s % 3) << 3 | b for s, b in enumerate((3, 3, 4, 4, 4, 4, 5, 5))], dtype=np.uint8)
    elif fmt == 7:
        nb = n * k // 128
        W = rng.integers(0, 256, (nb, 34), dtype=np.uint8)
        W[:, 0:2] = f16(rng.uniform(0.01, 0.05, nb))
    elif fmt == 100:     # planar MLX group 64: [n][k/8] u32 nibbles, then fp16 scales [n][k/64], then fp16 biases
        sc = rng.uniform(0.005, 0.02, n * k // 64)
        W = np.concatenate([rng.integers(0, 256, n * k // 2, dtype=np.uint8), f16(sc).reshape(-1),
                            f16(-8.0 * sc + rng.uniform(-0.01, 0.01, sc.size)).reshape(-1)])
    elif fmt == 102:     # the reference's planar MLX group 32: 16 nibble bytes per block, then fp16 scales, then fp16 biases
        sc = rng.uniform(0.005, 0.02, n * k // 32)       # (n * k / 32 blocks; the planes are 16-byte multiples whenever k % 256 == 0)
        W = np.concatenate([rng.integers(0, 256, n * k // 2, dtype=np.uint8), f16(sc).reshape(-1),
                            f16(-8.0 * sc + rng.uniform(-0.01, 0.01, sc.size)).reshape(-1)])
    elif fmt == 101:     # planar ternary: [n][k/16] u32 of 2-bit codes, then one fp16 absmean scale per row
        codes = rng.choice(np.array([0, 1, 2], dtype=np.uint32), size=(n * k // 16, 16), p=[0.25, 0.5, 0.25])
        words = (codes << (2 * np.arange(16, dtype=np.uint32))).sum(axis=1, dtype=np.uint32)
        W = np.concatenate([words.view(np.uint8), f16(rng.uniform(0.01, 0.05, n)).reshape(-1)])
    else:
        nb = n * k // 256
        W = rng.integers(0, 256, (nb, 144), dtype=np.uint8)
        W[:, 0:2] = f16(rng.uniform(3e-4, 3e-3, nb))
        W[:, 2:4] = f16(rng.uniform(-0.004, 0.008, nb))
        W[:, 20:36] = rng.integers(-8, 8, (nb, 16)).astype(np.int8).view(np.uint8)
    return np.ascontiguousarray(W).reshape(-1)


def plane_cuts(fmt: int, k: int, n: int) -> list:
    """Byte offsets where the second and later planes of a planar layout start (empty for block layouts)."""
    return {100: [n * k // 2, n * k // 2 + n * k // 32], 101: [n * k // 4]}.get(fmt, [])


def roll_rows(Wh: np.ndarray, i: int, cuts: list, n: int) -> np.ndarray:
    """A different weight matrix for ring slot i: the rows of the packed matrix rotated by i.  Planar layouts are
    several [n][x] planes back to back (`cuts` = where they start); every plane is rotated alike, so a row keeps
    its own scales."""
    return np.concatenate([np.roll(pl.reshape(n, -1), i, axis=0).reshape(-1) for pl in np.split(Wh, cuts)])


# ---------------------------------------------------------------------------------------------
# one projection configuration: ring of operand sets, parity, timing
# ---------------------------------------------------------------------------------------------
class ProjCase:
    """Y = X . W^T (or the fused gate/up SwiGLU when `swiglu`) for one (format, m, k, n): a ring of disjoint operand
    sets larger than L2 on the device, one parity check of ring slot 0 against the CPU verifier, and a timer."""

    def __init__(self, br, fmt: int, m: int, k: int, n: int, seed: int, swiglu: bool = False, min_ring_bytes: float = 300e6,
                 shard=None):
        import torch
        self.br, self.fmt, self.m, self.k, self.n, self.swiglu = br, fmt, m, k, n, swiglu
        rng = np.random.default_rng(seed)
        self.Xh = rng.standard_normal((m, k), dtype=np.float32).astype(np.float16)
        if swiglu:
            self.Xh = (self.Xh.astype(np.float32) * 0.25).astype(np.float16)      # keeps silu(g) * u inside the fp16 range
        n_full = n if shard is None else n * shard[1]
        Wfull = [synth_w(fmt, k, n_full, rng) for _ in range(2 if swiglu else 1)]
        if shard is not None:       # this rank's output columns of the whole matrix: whole rows of every plane
            from m4_prefill_engine_b200.layer import shard_rows_any
            Wfull = [shard_rows_any(w, fmt, k, n_full, shard[0], shard[1]) for w in Wfull]
        self.Wh = Wfull
        self.w_bytes = sum(int(w.size) for w in self.Wh)
        self.algo_bytes = self.w_bytes + m * k * 2 + m * n * 2
        self.flops = (4.0 * m * k * n + 4.0 * m * n) if swiglu else 2.0 * m * n * k
        self.ring = int(max(2, min(32, math.ceil(min_ring_bytes / self.algo_bytes))))
        dev = torch.device("cuda")
        cuts = plane_cuts(fmt, k, n)
        gen = torch.Generator(device=dev); gen.manual_seed(seed + 1)
        self.Xs, self.Ws, self.Ys = [], [], []
        for i in range(self.ring):
            self.Xs.append(torch.from_numpy(self.Xh).to(dev) if i == 0 else
                           (torch.randn(m, k, device=dev, generator=gen) * (0.25 if swiglu else 1.0)).to(torch.float16))
            self.Ws.append([torch.from_numpy(w if i == 0 else roll_rows(w, i, cuts, n)).to(dev) for w in self.Wh])
            self.Ys.append(torch.zeros(m, n, dtype=torch.float16, device=dev))
        L = br.lib
        self.calls = []
        for j in range(self.ring):
            x, y = self.Xs[j].data_ptr(), self.Ys[j].data_ptr()
            w0 = self.Ws[j][0]
            if swiglu:
                self.calls.append((L.b200_bridge_dispatch_swiglu, (x, m * k * 2, w0.data_ptr(), self.Ws[j][1].data_ptr(), w0.numel(), y,
                                                                   m * n * 2, fmt, m, k, n)))
            elif fmt < 6:
                self.calls.append((L.m4_bridge_dispatch_gemm, (x, m * k * 2, w0.data_ptr(), w0.numel(), y, m * n * 2, fmt, m, k, n)))
            else:
                self.calls.append((L.b200_bridge_dispatch_gemm_ex, (x, m * k * 2, w0.data_ptr(), w0.numel(), y, m * n * 2, fmt, m, k, n,
                                                                    0, 0, 0, None, 0)))
        torch.cuda.synchronize()

    def step(self, i: int) -> None:
        fn, a = self.calls[i % self.ring]
        rc = fn(*a)
        if rc != 0:
            raise SystemExit(f"dispatch failed with status {rc} (format {self.fmt}, M={self.m}, K={self.k}, N={self.n})")

    def parity(self, n_rows: int = 12) -> dict:
        """Ring slot 0 through the kernel, sampled token rows (first, last, both sides of the first tile edge, random)
        against the CPU verifier's double-precision gold."""
        import oracle as o
        self.step(0)
        self.br.synchronize()
        rows = sorted(set([0, self.m - 1, min(255, self.m - 1), min(256, self.m - 1)] +
                          [int(r) for r in np.random.default_rng(5).integers(0, self.m, max(0, n_rows - 4))]))
        Y = self.Ys[0][rows].cpu().numpy()
        X = self.Xh[rows]
        if self.swiglu:
            g = o.gemm_f64(self.fmt, X, self.Wh[0], self.n)
            u = o.gemm_f64(self.fmt, X, self.Wh[1], self.n)
            gold = g / (1.0 + np.exp(-g)) * u
            p = parity_of(Y, gold, rows)
            # the activation multiplies two contractions: propagate the per-GEMM criterion through the product
            tg = np.maximum(TOL, 2.0 ** -9 * np.sqrt(np.mean(g ** 2)))
            tu = np.maximum(TOL, 2.0 ** -9 * np.sqrt(np.mean(u ** 2)))
            tol = 1.1 * np.abs(u) * tg + np.abs(g / (1.0 + np.exp(-g))) * tu + np.maximum(TOL, np.spacing(np.abs(gold).astype(np.float16)).astype(np.float64))
            p["ok"] = bool(np.all(np.abs(Y.astype(np.float64) - gold) <= tol))
            return p
        return parity_of(Y, o.gemm_f64(self.fmt, X, self.Wh[0], self.n), rows)

    def time(self, steps: int, warmup: int, blocks: int, dist=None):
        """`blocks` timed blocks of `steps` launches (CUDA events on the library's stream, barrier + synchronise on both
        sides, maximum over ranks per block).  Returns (median ms per step, [ms per step of every block], launches in the
        median-sized block, host microseconds per dispatch)."""
        import torch
        stream = torch.cuda.ExternalStream(self.br.lib.b200_bridge_stream())
        for i in range(warmup):
            self.step(i)
        self.br.synchronize()
        per_block, launches, host_us = [], 0, 0.0
        it = warmup
        for _ in range(blocks):
            if dist:
                dist.barrier()
            torch.cuda.synchronize()
            l0 = self.br.kernel_launches()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            h0 = time.perf_counter()
            for _ in range(steps):
                self.step(it); it += 1
            host_us = (time.perf_counter() - h0) / steps * 1e6
            e1.record(stream)
            self.br.synchronize(); e1.synchronize()
            if dist:
                dist.barrier()
            torch.cuda.synchronize()
            launches = self.br.kernel_launches() - l0
            t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
            if dist:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            per_block.append(float(t.item()) / steps)
        return statistics.median(per_block), per_block, int(launches), host_us

    def free(self) -> None:
        import torch
        self.Xs = self.Ws = self.Ys = self.calls = None
        torch.cuda.empty_cache()


def roofline_of(fmt_name: str, m: int, k: int, n: int, flops: float, algo_bytes: int, ms_step: float, burst, sustained, hbm, src) -> dict:
    """Tensor roofline for the prefill shapes; HBM roofline for the few-token shapes (M <= 256), where the packed
    weights (read once) dominate the algorithmic bytes W + X + Y.  Both fractions are given either way."""
    gbs = algo_bytes / (ms_step * 1e-3) / 1e9
    tfl = flops / (ms_step * 1e-3) / 1e12
    traffic, tsrc = NCU_TRAFFIC.get((fmt_name, m), (None, None)) if (k, n) == (4096, 4096) else (None, None)
    common = {"traffic": traffic, "traffic_source": tsrc, "algorithmic_flops_per_launch": flops, "algorithmic_bytes_per_launch": algo_bytes}
    if m > 256:
        return {"bound": "tensor", "achieved": tfl, "peak": burst, "unit": "TFLOP/s", "frac": tfl / burst,
                "peak_source": f"{src}: dense bf16/fp16 cuBLAS burst (sustained {sustained})",
                # the timed blocks are back-to-back launches under the power cap, the condition the sustained figure was taken in
                "frac_of_sustained": (tfl / sustained) if sustained else None, "hbm_frac": gbs / hbm, **common}
    return {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm,
            "peak_source": f"{src}: device copy bandwidth", "tensor_frac": tfl / burst, **common}


def run_sweep(br, steps: int) -> list:
    """One device-timed row per benchmark configuration that fits one GPU: the 8B projection in Q4_0 and in the MLX
    group-64 layout at M in {33, 128, 129, 2048}; the other router formats at M = 2048; the Q4_K SwiGLU MLP (gate/up
    fused, then down) at M = 2048; the ternary K=4096 -> N=14336 projection at M in {128, 2048}."""
    burst, sustained, hbm, src = peaks()
    cases = []
    for f in ("q4_0", "mlx_4bit_g64"):
        for m in (33, 128, 129, 2048):
            cases.append((f, m, 4096, 4096, False, f"{f} projection M={m} K=N=4096"))
    for f in ("mlx_4bit", "mlx_4bit_planar", "q4_k", "ternary_1_58", "var_rate_affine", "exl3", "ternary_row", "prism_q2_0"):
        cases.append((f, 2048, 4096, 4096, False, f"{f} projection M=2048 K=N=4096"))
    cases.append(("q4_k", 2048, 4096, 14336, True, "q4_k fused gate/up SwiGLU M=2048 K=4096 F=14336"))
    cases.append(("q4_k", 2048, 14336, 4096, False, "q4_k down projection M=2048 K=14336 N=4096"))
    for f in ("ternary_row", "ternary_1_58"):
        for m in (128, 2048):
            cases.append((f, m, 4096, 14336, False, f"{f} projection M={m} K=4096 N=14336"))
    out = []
    for f, m, k, n, sw, what in cases:
        try:
            c = ProjCase(br, FORMATS[f], m, k, n, seed=77 + m, swiglu=sw)
            par = c.parity(8)
            st = steps if m > 256 else max(steps, 50)
            ms, blocks, _, _ = c.time(st, 5, 3)
            row = {"workload": what, "ms": ms, "ms_blocks": blocks, "tflops": c.flops / ms / 1e9, "gbs": c.algo_bytes / ms / 1e6,
                   "ring_sets": c.ring, "parity": par,
                   "roofline": roofline_of(f, m, k, n, c.flops, c.algo_bytes, ms, burst, sustained, hbm, src)}
            c.free()
        except SystemExit as e:           # a format this library does not serve on the device is reported, not hidden
            row = {"workload": what, "error": str(e)}
        out.append(row)
    return out


def run_c4(br, world: int, rank: int, steps: int, dist) -> list:
    """The ternary projection K=4096 -> N=14336 with its output columns split over the ranks (rows of the packed
    matrix; no collective follows it): every rank times its N/world columns, the slowest rank sets the time."""
    import torch
    burst, _, hbm, _ = peaks()
    out = []
    k, n = 4096, 14336
    if n % (world * 128):
        return out
    for f in ("ternary_row", "ternary_1_58"):
        for m in (128, 2048):
            c = ProjCase(br, FORMATS[f], m, k, n // world, seed=500 + m, shard=(rank, world))
            par = c.parity(8)
            worst = torch.tensor([par["max_abs"], 0.0 if par["ok"] else 1.0], device="cuda")
            if dist:
                dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            ms, blocks, _, _ = c.time(steps if m > 256 else max(steps, 50), 5, 3, dist)
            flops = 2.0 * m * n * k
            out.append({"workload": f"{f} projection M={m} K={k} N={n}, output columns split over {world} GPU(s): {n // world} per rank",
                        "parallelism": f"column-split x{world}, no collective", "scaling": "strong", "ms": ms, "ms_blocks": blocks,
                        "tflops": flops / ms / 1e9, "tensor_frac_per_gpu": flops / world / ms / 1e9 / burst,
                        "hbm_frac_per_gpu": c.algo_bytes / ms / 1e6 / hbm,
                        "parity": {"max_abs_over_ranks": float(worst[0].item()), "ok_on_every_rank": bool(worst[1].item() == 0.0),
                                   "rank0": par}})
            c.free()
    return out


# ---------------------------------------------------------------------------------------------
# decoder layer
# ---------------------------------------------------------------------------------------------
def shard_q4_0_device(W, n_rows: int, k: int, rank: int, world: int, by: str):
    """Device-side twin of layer.shard_rows / shard_cols for Q4_0 [n_rows][k/32] blocks of 18 bytes."""
    blocks = W.reshape(n_rows, k // 32, 18)
    if by == "rows":
        r = n_rows // world
        return blocks[rank * r:(rank + 1) * r].contiguous().reshape(-1)
    b = (k // 32) // world
    return blocks[:, rank * b:(rank + 1) * b].contiguous().reshape(-1)


def time_layer(br, pkg, world: int, rank: int, steps: int, warmup: int, collective: str = "peer", check: bool = True):
    """Tensor-parallel decoder layer (Q4_0, RMSNorm, GQA 32/8, RoPE, Q8_0 KV, SwiGLU 14336), M=2048.  Every rank builds
    the same whole-layer weights from one seed and keeps its own shard; before timing, rank 0 compares the first 48
    output rows with the CPU verifier's layer on 48 tokens (a causal layer's first rows depend on the first tokens
    only) and all ranks compare their outputs bit for bit."""
    import torch
    import torch.distributed as dist
    from m4_prefill_engine_b200.layer import PeerExchange, TransformerLayerConfig, TransformerLayerCoordinator, torch_allreduce_hook
    c = LAYER
    if c["Hkv"] % world or c["F"] % world:
        return None
    cfg = TransformerLayerConfig(M=c["M"], K=c["K"], H=c["H"], D=c["D"], N_mlp=c["F"], attn_scale=c["D"] ** -0.5, weight_format=0,
                                 num_kv_heads=c["Hkv"], rms_eps=1e-5, rope_theta=500000.0, kv_q8_0=True, tp_size=world)
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev); gen.manual_seed(100)       # whole-layer weights: the same on every rank
    qd, kd = c["H"] * c["D"], c["Hkv"] * c["D"]
    dims = {"q": (qd, c["K"], "rows"), "k": (kd, c["K"], "rows"), "v": (kd, c["K"], "rows"), "o": (c["K"], qd, "cols"),
            "gate": (c["F"], c["K"], "rows"), "up": (c["F"], c["K"], "rows"), "down": (c["K"], c["F"], "cols")}
    full, w = {}, {}
    for name, (nr, kk, by) in dims.items():
        Wf = synth_q4_0(nr, kk, dev, gen, 0.0003, 0.0033)
        if check and rank == 0:
            full[name] = Wf.cpu().numpy()
        w[name] = shard_q4_0_device(Wf, nr, kk, rank, world, by) if world > 1 else Wf
        del Wf
    gx = torch.Generator(device=dev); gx.manual_seed(7)       # the residual stream is replicated: same seed on every rank
    X = (torch.randn(c["M"], c["K"], device=dev, generator=gx) * 0.35).to(torch.float16)
    Y = torch.zeros_like(X)
    n1 = (1.0 + 0.1 * torch.randn(c["K"], device=dev, generator=gx)).to(torch.float16)
    n2 = (1.0 + 0.1 * torch.randn(c["K"], device=dev, generator=gx)).to(torch.float16)
    layer = TransformerLayerCoordinator(cfg, br)
    layer.set_norm_weights(n1, n2)
    px = None
    if world > 1 and collective == "peer" and (c["M"] // world) % 256 == 0:
        px = PeerExchange.setup(layer)           # reduce-scatter fused into the projection epilogue, over peer memory
    if world > 1 and px is None:                 # shape not supported, or peer mappings not available on this node
        collective = "nccl"
        layer.set_allreduce(torch_allreduce_hook(br))
    stream = torch.cuda.ExternalStream(br.lib.b200_bridge_stream())
    if px is not None:
        Y = px.result_tensor(c["M"], c["K"])     # the output stays in the exchange's result buffer, as between the layers of a model
    args = (X, w["q"], w["k"], w["v"], w["o"], w["gate"], w["up"], w["down"], Y)
    layer.forward(*args)
    br.synchronize()
    if px is not None:
        # a rank that did not hear from its peers within the wait limit has set the error word: every rank then
        # drops the fused exchange together and the caller measures the NCCL path instead
        bad = torch.tensor([1 if br.device_error() != 0 else 0], device=dev)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()):
            layer.close(); px.close()
            return {"error": "peer exchange timed out on the first layer", "device_error": br.device_error()}
    parity = None
    if check:
        same = True
        if world > 1:
            Y0 = Y.clone()
            dist.broadcast(Y0, src=0)
            eq = torch.tensor([1 if torch.equal(Y0, Y) else 0], device=dev)
            dist.all_reduce(eq, op=dist.ReduceOp.MIN)
            same = bool(int(eq.item()))
        if rank == 0:
            import oracle as o
            cpu_threads()
            R = 48
            gold = o.layer(0, X[:R].cpu().numpy(), full["q"], full["k"], full["v"], full["o"], full["gate"], full["up"], full["down"],
                           c["H"], c["Hkv"], c["D"], c["F"], c["D"] ** -0.5, rms_eps=1e-5, norm1=n1.cpu().numpy(), norm2=n2.cpu().numpy(),
                           rope_theta=500000.0, kv_q8=True)
            g64 = gold.astype(np.float64)
            d = np.abs(Y[:R].cpu().numpy().astype(np.float64) - g64)
            # A layer output passes through six fp16 roundings of intermediates, each 2^-11 relative, so the bound scales
            # with the magnitude of the token row: |d| <= max(2/128, 2^-7 * rms(row)).  (Token 0 attends to itself only,
            # its attention output is one un-averaged value row and its outputs are an order of magnitude larger.)
            row_rms = np.sqrt(np.mean(g64 ** 2, axis=1, keepdims=True))
            tol = np.maximum(2 * TOL, 2.0 ** -7 * row_rms)
            worst = int(np.argmax(d.max(axis=1)))
            parity = {"rows": "first 48 of 2048 against the CPU verifier's layer", "max_abs": float(d.max()), "max_abs_row": worst,
                      "rms_of_that_row": float(row_rms[worst, 0]), "max_abs_rows_1_to_47": float(d[1:].max()),
                      "over_1_128": int((d > TOL).sum()), "outputs": int(d.size), "criterion": "max(2/128, 2^-7 * rms(row))",
                      "ok": bool(np.all(d <= tol)), "ranks_bit_identical": same}
        full.clear()
        if world > 1:
            dist.barrier()
    for _ in range(max(3, warmup) - 1):
        layer.forward(*args)
    br.synchronize()
    blocks = []
    for _ in range(3):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            layer.forward(*args)
        e1.record(stream)
        br.synchronize(); e1.synchronize(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        blocks.append(float(t.item()))
    ms = statistics.median(blocks)
    finite = bool(torch.isfinite(Y.float()).all().item())
    kernels = layer.kernels_per_forward()
    timeline = layer.profile_forward(*args) if hasattr(layer, "profile_forward") else None
    dev_err = br.device_error()
    if world > 1:
        dist.barrier()
    layer.close()
    if px is not None:
        px.close()
    flops = 2.0 * c["M"] * c["K"] * (qd + 2 * kd) + 2.0 * c["H"] * c["M"] * (c["M"] + 1) * c["D"] + 2.0 * c["M"] * qd * c["K"] + \
        4.0 * c["M"] * c["K"] * c["F"] + 2.0 * c["M"] * c["F"] * c["K"]
    burst = peaks()[0]
    return {"workload": "Llama-style 8B decoder layer prefill, M=2048, Q4_0, GQA 32/8, D=128, RoPE, Q8_0 KV, SwiGLU 14336",
            "parallelism": f"tp{world}", "scaling": "strong", "ms": ms, "ms_blocks": blocks, "tflops": flops / ms / 1e9,
            "tensor_frac_per_gpu": flops / world / ms / 1e9 / burst, "gflop_per_layer": flops / 1e9,
            "kernels_per_layer": kernels, "finite": finite, "device_error": dev_err, "parity": parity, "timeline_us": timeline,
            "allreduce": None if world == 1 else ("nccl fp32 [M,K] x2" if collective == "nccl" else
                                                  "partial rows scattered to their owner from the projection epilogue over peer memory, "
                                                  "owner adds + residual (+ RMSNorm), fp16 rows written to every rank, x2")}


def time_model(br, pkg, world: int, rank: int, layers: int = 32):
    """End-to-end prefill of an L-layer model (embedding gather, L decoder layers, final RMSNorm, lm_head) through the
    model entry points, where the library has them."""
    try:
        from m4_prefill_engine_b200.model import bench_prefill
    except ImportError:
        return None
    return bench_prefill(br, world, rank, layers)


def run_ours(args) -> None:
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU implementation (use --impl reference for the CPU leg)")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from __graft_entry__ import load_package
    pkg = load_package()
    br = pkg.B200Bridge.get_instance()
    if not br.init():
        raise SystemExit("bridge init failed: " + (br.lib.b200_bridge_last_error_string() or b"").decode())
    fmt = FORMATS[args.format]
    dev = torch.device("cuda")
    warmup = max(3, args.warmup)

    # The timed loop calls the C ABI entry point directly with pre-extracted addresses (what a C host does): the
    # Python wrapper's per-call stream synchronisation and tensor bookkeeping cost about as much host time as one
    # of these kernels runs, and would turn the kernel-only figure into a measurement of the interpreter.
    case = ProjCase(br, fmt, M, K, N, seed=2024 + rank, min_ring_bytes=340e6)
    parity = case.parity(16)                       # verify, then time
    sampler = ClockSampler(local) if rank == 0 else None
    ms_step, ms_blocks, launches, host_us = case.time(args.steps, warmup, 1 if args.quick else BLOCKS, dist)
    # keep the same kernel running long enough for nvidia-smi to see the clocks it runs at (not timed)
    t_end = time.time() + (0.0 if args.quick else 0.6)
    i = 0
    while time.time() < t_end:
        for _ in range(200):
            case.step(i); i += 1
        br.synchronize()
    clocks = sampler.stop() if sampler else None
    dev_err = br.device_error()

    # ---- end to end through the C ABI with pinned host buffers ----
    e2e_s, e2e_serial_s, e2e_steps, e2e_ok, DEPTH = float('nan'), float('nan'), 1, False, 1
    e2e_call = br.dispatch_gemm if fmt < 6 else br.dispatch_gemm_ex     # formats 7/100/101 exist only on the extended entry point
    if not args.quick:
        # DEPTH steps are in flight between two m4_bridge_synchronize calls, each with its own pinned X and Y (a
        # serving loop that batches DEPTH requests per synchronize): the bridge uploads step i+1 while step i computes
        # and downloads.  Every step's X is copied host -> device and every step's Y device -> host inside the timed
        # region.  `serial` repeats the measurement with a synchronize after every dispatch.
        DEPTH = 8
        Xh, Wh = case.Xh, case.Wh[0]
        Xp = [torch.from_numpy(Xh if i == 0 else Xh.copy()).pin_memory() for i in range(DEPTH)]
        Yp = [torch.zeros(M, N, dtype=torch.float16).pin_memory() for _ in range(DEPTH)]
        Wp = torch.from_numpy(Wh).pin_memory()
        assert br.register_weights(Wp) == 0
        e2e_steps = max(DEPTH, min(args.steps, 48) // DEPTH * DEPTH)
        for i in range(DEPTH):
            e2e_call(Xp[i], Wp, Yp[i], fmt, M, K, N)
        br.synchronize()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            e2e_call(Xp[i % DEPTH], Wp, Yp[i % DEPTH], fmt, M, K, N)
            if i % DEPTH == DEPTH - 1:
                br.synchronize()                  # the results of these DEPTH steps are on the host
        e2e_s = time.perf_counter() - t0
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            e2e_call(Xp[i % DEPTH], Wp, Yp[i % DEPTH], fmt, M, K, N)
            br.synchronize()
        e2e_serial_s = time.perf_counter() - t0
        te = torch.tensor([e2e_s], device=dev)
        if dist:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_s = float(te.item())
        # the host result of the first buffer is the device result of ring slot 0, bit for bit (same X, same W)
        e2e_ok = all(bool(torch.isfinite(y.float()).all().item()) and float(y.float().abs().max()) > 0 for y in Yp) and \
            bool(torch.equal(Yp[0], case.Ys[0].cpu()))
        br.lib.b200_bridge_unregister_weights(Wp.data_ptr())
    algo_bytes, w_bytes = case.algo_bytes, case.w_bytes
    ring_sets = case.ring
    case.free()

    sweep = run_sweep(br, min(args.steps, 30)) if (world == 1 and not args.quick and not args.no_sweep) else None
    c4 = run_c4(br, world, rank, min(args.steps, 30), dist) if not (args.quick or args.no_sweep) else None

    layer_steps = max(3, min(args.steps, 20))
    layer = time_layer(br, pkg, world, rank, layer_steps, 3) if not args.no_layer else None
    if layer is not None and world > 1:          # the same layer with NCCL all-reduces, for comparison (or as the fallback)
        nccl = time_layer(br, pkg, world, rank, layer_steps, 3, collective="nccl", check=False)
        if "error" in layer:
            nccl["peer_exchange_error"] = layer["error"]
            layer = nccl
        elif nccl is not None:
            layer["nccl_allreduce_ms"] = nccl["ms"]
    model = time_model(br, pkg, world, rank) if not (args.no_layer or args.no_model) else None

    if rank == 0:
        burst, sustained, hbm, src = peaks()
        achieved = FLOPS_PER_STEP / (ms_step * 1e-3) / 1e12
        line = {
            "metric": f"W4 prefill projection throughput (8B shape, M={M})", "value": world * achieved, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic (seeded)",
            "config": {"workload": f"{args.format} dequant-fused projection Y[{M},{N}] = X[{M},{K}] . W^T, 8B shape",
                       "format": args.format, "M": M, "K": K, "N": N, "parallelism": f"dp{world} (replicated weights, own token batch per rank)",
                       "cache": f"ring of {ring_sets} disjoint (X, W, Y) sets = {ring_sets * algo_bytes / 1e6:.0f} MB > 126 MB L2",
                       "timing": f"median of {len(ms_blocks)} blocks of {args.steps} steps, each block between CUDA events, max over ranks"},
            "ms_per_step_blocks": ms_blocks, "parity": parity,
            "roofline": roofline_of(args.format, M, K, N, FLOPS_PER_STEP, algo_bytes, ms_step, burst, sustained, hbm, src),
            "e2e": None if args.quick else {
                "value": world * FLOPS_PER_STEP / (e2e_s / e2e_steps) / 1e12, "unit": "TFLOP/s", "ms_per_step": 1e3 * e2e_s / e2e_steps,
                "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2, "steps": e2e_steps, "steps_per_synchronize": DEPTH,
                "serial": {"value": world * FLOPS_PER_STEP / (e2e_serial_s / e2e_steps) / 1e12, "ms_per_step": 1e3 * e2e_serial_s / e2e_steps,
                           "note": "m4_bridge_synchronize after every dispatch"},
                "note": "pinned host X in, host Y out through m4_bridge_dispatch_gemm; steps_per_synchronize dispatches, then m4_bridge_synchronize; weights registered (resident)",
                "finite_nonzero_and_equal_to_device_result": e2e_ok},
            "gpu_launches": int(launches), "host_us_per_dispatch": round(host_us, 2), "device_error": dev_err, "clocks": clocks,
            "sweep": sweep, "c4": c4, "layer": layer, "model": model,
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(fmt)
        print(json.dumps(line), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--format", choices=sorted(FORMATS), default="q4_0")
    ap.add_argument("--no-layer", action="store_true", help="skip the decoder-layer and model timing")
    ap.add_argument("--no-model", action="store_true", help="skip the multi-layer model timing")
    ap.add_argument("--no-sweep", action="store_true", help="skip the per-configuration sweep and the column-split ternary rows")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--m", type=int, default=2048, help="token rows of the projection (33/128/129: the small-M shapes)")
    ap.add_argument("--quick", action="store_true",
                    help="one timed block of the projection only (no clock-sampling loop, sweep, end-to-end, layer or CPU legs): for profiler runs")
    args = ap.parse_args()
    global M, FLOPS_PER_STEP
    M = args.m
    FLOPS_PER_STEP = 2.0 * M * N * K
    if args.quick:
        args.no_layer = args.no_cpu = True
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
