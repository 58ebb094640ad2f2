#!/usr/bin/env python
"""Benchmark of the tensor hot path on B200: one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload rows|gemm|attn|mlp|matmul_f32]
    python bench.py --impl reference ...      # the CPU restatement of the reference's lowering, host cores

Workloads (seeded synthetic inputs of the stated shapes and distributions):
  rows        X[16384,8192] f32 -> bf16, one step = row softmax + row RMSNorm (two kernels)       HBM GB/s
  gemm        bf16 8192^3, A row-major, B stored [N,K], f32 accumulation, bf16 C                   TFLOP/s
  attn        causal attention forward, batch*heads = 128, seq 4096, head_dim 128, bf16            TFLOP/s
  mlp         (silu(X W1) * (X W3)) W2, X[8192,4096], W1/W3[4096,14336], W2[14336,4096], bf16      TFLOP/s
  matmul_f32  f32 256^3 (the reference's CPU-runnable case)                                        TFLOP/s
Under torchrun every rank runs the same per-GPU workload on its own shard (row blocks, B column slabs, heads):
weak scaling, no collective on the data path; the time is the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="rows", choices=["rows", "gemm", "attn", "mlp", "mlp_tp", "matmul_f32"])
    ap.add_argument("--tp-gather", default="auto", choices=["auto", "fused", "nccl"],
                    help="mlp_tp: all-gather of H fused into the GEMM epilogue (peer stores) or a separate NCCL all-gather")
    ap.add_argument("--no-extras", action="store_true", help="skip the short runs of the other workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (for profiler runs)")
    ap.add_argument("--gather", action="store_true",
                    help="gemm / attn under torchrun: all-gather every rank's output shard inside the timed step (NCCL)")
    return ap.parse_args()


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm": float(p["hbm_gbs"]), "tensor": float(p["bf16_tflops"]),
                "tensor_sustained": float(p["bf16_tflops_sustained"]), "source": "measured"}
    except Exception:
        return {"hbm": 6650.0, "tensor": 1590.0, "tensor_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.samples, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def stop(self, t0, t1):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.samples:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clk, mxc = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            mx = mxc
            if t0 - 0.05 <= t <= t1 + 0.05:
                sm.append(clk)
                for n, v in zip(names, parts[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        if not sm:  # region shorter than one sampling period: take what there is
            for _, line in self.samples:
                try:
                    sm.append(float(line.split(",")[0]))
                except ValueError:
                    pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ workloads
class Workload:
    name = ""
    metric = ""
    unit = ""
    dtype = ""
    bound = "hbm"
    kernel = ""
    launches_per_step = 1
    traffic = None  # dram bytes (read + write) of one launch of the dominant kernel, from the ncu capture in profiles/

    def __init__(self, torch, T, H, rank, world):
        self.torch, self.T, self.H, self.rank, self.world = torch, T, H, rank, world

    gather = False
    gathered = None

    def all_gather(self, local):
        """All-gather the ranks' output shards into one [world, ...] tensor on every rank (NCCL over NVLink)."""
        import torch.distributed as dist
        if self.gathered is None:
            self.gathered = self.torch.empty((self.world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(self.gathered, local)

    def gen(self, seed):
        g = self.torch.Generator(device="cuda")
        g.manual_seed(seed + 1000 * self.rank)
        return g


class Rows(Workload):
    name, metric, unit, dtype, bound = "row softmax + RMSNorm f32 X[16384,8192] -> bf16", "HBM GB/s (row softmax+RMSNorm)", "GB/s", "f32", "hbm"
    kernel, launches_per_step = "rows_in_regs_kernel<softmax>", 2
    traffic = 536886016 + 229935360   # profiles/rows_softmax_rmsnorm_c2.md
    R, Cc = 16384, 8192

    def setup(self):
        t = self.torch
        g = self.gen(1235)
        self.x = t.randn((self.R, self.Cc), generator=g, device="cuda", dtype=t.float32)
        self.gamma = t.rand((self.Cc,), generator=g, device="cuda", dtype=t.float32) + 0.5
        self.y1 = self.y2 = None
        self.units = 2 * (self.R * self.Cc * 6) + self.Cc * 4      # algorithmic bytes per step (read f32 + write bf16, twice)
        self.dom_units = self.R * self.Cc * 6                      # the softmax launch
        self.config = {"workload": self.name, "rows_per_gpu": self.R, "cols": self.Cc, "eps": 1e-6,
                       "l2": "input (512 MiB) larger than L2", "sharding": "row blocks, one per GPU"}

    def step(self, ev=None):
        if ev:
            ev[0].record()
        self.y1 = self.T.softmax(1, self.x, out_dtype=self.torch.bfloat16)
        if ev:
            ev[1].record()
        self.y2 = self.T.rmsnorm(self.x, self.gamma, 1e-6, out_dtype=self.torch.bfloat16)

    def e2e_setup(self):
        t = self.torch
        self.hx = self.x.cpu().pin_memory()
        self.hg = self.gamma.cpu().pin_memory()
        self.hy1 = t.empty((self.R, self.Cc), dtype=t.bfloat16).pin_memory()
        self.hy2 = t.empty((self.R, self.Cc), dtype=t.bfloat16).pin_memory()
        self.h2d = self.R * self.Cc * 4 + self.Cc * 4     # x is uploaded once for both results
        self.d2h = 2 * self.R * self.Cc * 2

    def e2e_step(self):
        self.H.softmax_and_rmsnorm(self.hx, self.hg, 1e-6, out_softmax=self.hy1, out_rmsnorm=self.hy2)
        return float(self.hy2[0, 0])

    @staticmethod
    def cpu_sample(mo, np, rows=2048):
        rng = np.random.default_rng(1235)
        x = rng.standard_normal((rows, 8192), dtype=np.float32)
        gamma = rng.uniform(0.5, 1.5, 8192).astype(np.float32)
        t0 = time.perf_counter()
        y = mo.to_bf16(mo.softmax_rows(x))
        z = mo.to_bf16(mo.rmsnorm_rows(x, gamma, 1e-6))
        dt = time.perf_counter() - t0
        units = 2 * rows * 8192 * 6 + 8192 * 4
        return units / dt / 1e9, f"{rows} of 16384 rows x 8192, softmax + RMSNorm, f32 -> bf16, one pass", float(y[0, 0]) + float(z[0, 0])


class Gemm(Workload):
    name, metric, unit, dtype, bound = "matmul bf16 M=N=K=8192, A row-major, B stored [N,K], f32 accumulate", "TFLOP/s (bf16 GEMM 8192^3)", "TFLOP/s", "bf16", "tensor"
    kernel = "gemm_tc2_kernel"
    traffic = 1115728000 + 127246592  # profiles/gemm_tc2_bf16_8192_c3.md
    n = 8192

    def setup(self):
        t = self.torch
        g = self.gen(1236)
        self.a = (t.randn((self.n, self.n), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        self.b = (t.randn((self.n, self.n), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        self.units = self.dom_units = 2 * self.n ** 3
        self.config = {"workload": self.name, "l2": "A+B (256 MiB) larger than L2",
                       "sharding": "B column slabs, one 8192-column slab per GPU"}

    def step(self, ev=None):
        if ev:
            ev[0].record()
        self.c = self.T.product_2d(self.a, self.T.transpose_2d(self.b))
        if ev:
            ev[1].record()
        if self.gather and self.world > 1:
            self.all_gather(self.c)

    def e2e_setup(self):
        self.ha, self.hb = self.a.cpu().pin_memory(), self.b.cpu().pin_memory()
        self.hc = self.torch.empty((self.n, self.n), dtype=self.torch.bfloat16).pin_memory()
        self.h2d, self.d2h = 2 * self.n * self.n * 2, self.n * self.n * 2

    def e2e_step(self):
        self.H.product_2d(self.ha, self.T.transpose_2d(self.hb), out=self.hc)
        return float(self.hc[0, 0])

    @staticmethod
    def cpu_sample(mo, np, rows=8, k=8192):
        rng = np.random.default_rng(1236)
        a = mo.to_bf16((rng.standard_normal((rows, k)) * 0.02).astype(np.float32))
        b = mo.to_bf16((rng.standard_normal((8192, k)) * 0.02).astype(np.float32))
        t0 = time.perf_counter()
        c = mo.gemm(a, b, b_nk=True, bf16=True)
        dt = time.perf_counter() - t0
        return 2 * rows * 8192 * k / dt / 1e12, f"{rows} of 8192 output rows (N=K=8192), f32 accumulate ascending k", float(c[0, 0])


class Attn(Workload):
    name, metric, unit, dtype, bound = "causal attention fwd bf16 batch*heads=128 seq=4096 head_dim=128", "TFLOP/s (causal attention fwd)", "TFLOP/s", "bf16", "tensor"
    kernel = "attn_tc_persistent_kernel"
    traffic = 402723328 + 113826816   # profiles/attn_tc_causal_c4.md
    BH, S, D = 128, 4096, 128

    def setup(self):
        t = self.torch
        g = self.gen(1237)
        self.q, self.k, self.v = (t.randn((self.BH, self.S, self.D), generator=g, device="cuda").to(t.bfloat16) for _ in range(3))
        self.units = self.dom_units = 4 * self.BH * self.S * self.S * self.D // 2   # causal convention
        self.config = {"workload": self.name, "flop_count": "4*B*H*S^2*D/2 (causal)", "l2": "Q,K,V (384 MiB) larger than L2",
                       "sharding": "128 heads per GPU"}

    def step(self, ev=None):
        if ev:
            ev[0].record()
        self.o = self.T.attention(self.q, self.k, self.v, scale=1.0 / self.D ** 0.5, causal=True)
        if ev:
            ev[1].record()
        if self.gather and self.world > 1:
            self.all_gather(self.o)

    def e2e_setup(self):
        self.hq, self.hk, self.hv = (x.cpu().pin_memory() for x in (self.q, self.k, self.v))
        self.ho = self.torch.empty_like(self.hq).pin_memory()
        self.h2d, self.d2h = 3 * self.BH * self.S * self.D * 2, self.BH * self.S * self.D * 2

    def e2e_step(self):
        self.H.attention(self.hq, self.hk, self.hv, scale=1.0 / self.D ** 0.5, causal=True, out=self.ho)
        return float(self.ho[0, 0, 0])

    @staticmethod
    def cpu_sample(mo, np, s=1024):
        rng = np.random.default_rng(1237)
        q, k, v = (mo.to_bf16(rng.standard_normal((1, s, 128)).astype(np.float32)) for _ in range(3))
        t0 = time.perf_counter()
        o = mo.attention(q, k, v, scale=1 / 128 ** 0.5, causal=True, bf16=True, truth=False)
        dt = time.perf_counter() - t0
        return 4 * s * s * 128 / 2 / dt / 1e12, f"1 head at seq {s} (of 128 heads at 4096), unfused f32 chain with the score matrix", float(o[0, 0, 0])


class Mlp(Workload):
    name, metric, unit, dtype, bound = "MLP block bf16 X[8192,4096] W1/W3[4096,14336] SiLU-gate W2[14336,4096]", "TFLOP/s (gated MLP block)", "TFLOP/s", "bf16", "tensor"
    kernel, launches_per_step = "gemm_tc2_kernel<gated> + gemm_tc2_kernel (the two launches of one mimk_mlp_gated call)", 2
    M, K, F = 8192, 4096, 14336

    def setup(self):
        t = self.torch
        g = self.gen(1238)
        self.x = t.randn((self.M, self.K), generator=g, device="cuda").to(t.bfloat16)
        self.w1 = (t.randn((self.K, self.F), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        self.w3 = (t.randn((self.K, self.F), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        self.w2 = (t.randn((self.F, self.K), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        self.h = t.empty((self.M, self.F), device="cuda", dtype=t.bfloat16)
        self.units = 3 * 2 * self.M * self.K * self.F
        self.dom_units = self.units   # the events bracket the whole call (both launches)
        self.config = {"workload": self.name, "l2": "weights (336 MiB) larger than L2", "sharding": "replica per GPU"}

    def step(self, ev=None):
        if ev:
            ev[0].record()
        self.y = self.T.mlp_gated(self.x, self.w1, self.w3, self.w2, h=self.h)
        if ev:
            ev[1].record()

    def e2e_setup(self):
        self.hx, self.hw1, self.hw3, self.hw2 = (x.cpu().pin_memory() for x in (self.x, self.w1, self.w3, self.w2))
        self.hy = self.torch.empty((self.M, self.K), dtype=self.torch.bfloat16).pin_memory()
        self.h2d = (self.M * self.K + 3 * self.K * self.F) * 2
        self.d2h = self.M * self.K * 2

    def e2e_step(self):
        self.H.mlp_gated(self.hx, self.hw1, self.hw3, self.hw2, out=self.hy)
        return float(self.hy[0, 0])

    @staticmethod
    def cpu_sample(mo, np, rows=2):
        rng = np.random.default_rng(1238)
        x = mo.to_bf16(rng.standard_normal((rows, 4096)).astype(np.float32))
        w1, w3 = (mo.to_bf16((rng.standard_normal((4096, 14336)) * 0.02).astype(np.float32)) for _ in range(2))
        w2 = mo.to_bf16((rng.standard_normal((14336, 4096)) * 0.02).astype(np.float32))
        t0 = time.perf_counter()
        y = mo.mlp_gated_truth(x, w1, w3, w2)
        dt = time.perf_counter() - t0
        return 6 * rows * 4096 * 14336 / dt / 1e12, f"{rows} of 8192 rows through the full block", float(y[0, 0])


class MlpTP(Workload):
    """The C5 block split over the ranks (tensor parallel, STRONG scaling): rank g owns columns [g F/G, (g+1) F/G) of W1
    and W3 and columns [g N/G, (g+1) N/G) of W2; H is all-gathered between the two stages."""
    name, metric, unit, dtype, bound = "MLP block bf16 X[8192,4096] W1/W3[4096,14336] W2[14336,4096], tensor parallel", "TFLOP/s (gated MLP block, tensor parallel)", "TFLOP/s", "bf16", "tensor"
    kernel, launches_per_step = "gemm_tc2_kernel<gated> (+ fused all-gather) + gemm_tc2_kernel", 2
    scaling = "strong"
    M, K, F = 8192, 4096, 14336
    mode = "fused"

    def setup(self):
        t = self.torch
        from mimir_b200 import shard
        self.shard = shard
        g = t.Generator(device="cuda")
        g.manual_seed(1238)                       # the same global weights on every rank; each keeps its slab
        W = self.world
        self.fl, self.nl = self.F // W, self.K // W
        self.x = t.randn((self.M, self.K), generator=g, device="cuda").to(t.bfloat16)
        w1 = (t.randn((self.K, self.F), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        self.w1 = w1[:, self.rank * self.fl:(self.rank + 1) * self.fl].contiguous()
        w1 = (t.randn((self.K, self.F), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        self.w3 = w1[:, self.rank * self.fl:(self.rank + 1) * self.fl].contiguous()
        w1 = (t.randn((self.F, self.K), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        self.w2 = w1[:, self.rank * self.nl:(self.rank + 1) * self.nl].contiguous()
        del w1
        t.cuda.empty_cache()
        if self.mode == "auto":
            self.mode = "fused"
        self.yg = None
        if W > 1 and self.mode == "fused":
            self.h = shard.GatheredMatrix(self.M, self.F)
            if getattr(self, "gather", False):     # --gather: the whole Y on every rank, gathered in stage 2's epilogue
                self.yg = shard.GatheredMatrix(self.M, self.K)
        else:
            self.h_local = t.empty((self.M, self.fl), device="cuda", dtype=t.bfloat16)
        self.units = 3 * 2 * self.M * self.K * self.F // W     # per-rank share: the driver multiplies by world
        self.dom_units = self.units
        self.config = {"workload": self.name, "l2": "weights larger than L2", "tp_gather": self.mode if W > 1 else "n/a",
                       "sharding": "W1/W3 column slabs, H all-gathered, W2 column slabs (outputs stay sharded)"}

    def step(self, ev=None):
        if ev:
            ev[0].record()
        if self.world == 1:
            self.y = self.T.mlp_gated(self.x, self.w1, self.w3, self.w2, h=self.h_local)
        elif self.mode == "fused":
            self.y = self.shard.tp_mlp_gated(self.x, self.w1, self.w3, self.w2, self.h, gather="fused", y=self.yg)
        else:
            # stage 1 into a local slab (gated contraction with the W2-free path: H slab only), NCCL all-gather, stage 2
            self.shard.gemm_gather_local(self.x, self.w1, self.w3, self.h_local)
            h_full = self.shard.gather_columns(self.h_local, self.F)
            self.y = self.T.product_2d(h_full, self.w2)
            if getattr(self, "gather", False):
                self.y = self.shard.gather_columns(self.y, self.K)
        if ev:
            ev[1].record()

    def e2e_setup(self):
        self.h2d = self.d2h = 0

    def e2e_step(self):
        return 0.0

    @staticmethod
    def cpu_sample(mo, np, rows=2):
        return Mlp.cpu_sample(mo, np, rows)


class MatmulF32(Workload):
    name, metric, unit, dtype, bound = "matmul f32 256^3", "TFLOP/s (f32 matmul 256^3)", "TFLOP/s", "f32", "tensor"
    kernel = "split_kernel x2 + gemm_f32_tc_kernel (3xTF32)"
    launches_per_step = 3

    def setup(self):
        t = self.torch
        g = self.gen(1234)
        self.a = t.rand((256, 256), generator=g, device="cuda") * 2 - 1
        self.b = t.rand((256, 256), generator=g, device="cuda") * 2 - 1
        self.flush = t.empty(160 << 20, dtype=t.uint8, device="cuda")
        self.units = self.dom_units = 2 * 256 ** 3
        self.config = {"workload": self.name, "l2": "160 MiB buffer written between steps"}

    def step(self, ev=None):
        self.flush.zero_()
        if ev:
            ev[0].record()
        self.c = self.T.product_2d(self.a, self.b)
        if ev:
            ev[1].record()

    def e2e_setup(self):
        self.ha, self.hb = self.a.cpu().pin_memory(), self.b.cpu().pin_memory()
        self.hc = self.torch.empty((256, 256)).pin_memory()
        self.h2d, self.d2h = 2 * 256 * 256 * 4, 256 * 256 * 4

    def e2e_step(self):
        self.H.product_2d(self.ha, self.hb, out=self.hc)
        return float(self.hc[0, 0])

    @staticmethod
    def cpu_sample(mo, np):
        rng = np.random.default_rng(1234)
        a, b = (rng.uniform(-1, 1, (256, 256)).astype(np.float32) for _ in range(2))
        t0 = time.perf_counter()
        reps = 20
        for _ in range(reps):
            c = mo.gemm(a, b)
        dt = (time.perf_counter() - t0) / reps
        return 2 * 256 ** 3 / dt / 1e12, "full 256^3, mean of 20 passes", float(c[0, 0])


WORKLOADS = {"rows": Rows, "gemm": Gemm, "attn": Attn, "mlp": Mlp, "mlp_tp": MlpTP, "matmul_f32": MatmulF32}


# ------------------------------------------------------------------------------------------------ arms
def run_reference(args):
    """The reference's lowering, restated for the CPU (oracle/), on this box's host cores. The emitted code of the
    reference is single-threaded (no OpenMP or threads anywhere in its output), so one core is all it can use."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np

    import oracle as mo
    mo.build()
    W = WORKLOADS[args.workload]
    warm = min(args.warmup, 3)
    for _ in range(warm):
        W.cpu_sample(mo, np)
    vals, sample = [], ""
    t0 = time.perf_counter()
    for _ in range(max(1, args.steps)):
        v, sample, _ = W.cpu_sample(mo, np)
        vals.append(v)
        if time.perf_counter() - t0 > 150:
            break
    ms_per_step = (time.perf_counter() - t0) * 1e3 / len(vals)   # one step = one pass over the bounded sample
    val = statistics.mean(vals)
    unit = W.unit
    line = {"impl": "reference", "metric": W.metric, "value": val, "unit": unit, "n_gpus": args.gpus,
            "steps": len(vals), "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": W.dtype, "data": "synthetic",
            "config": {"workload": W.name},
            "cpu_baseline": {"value": val, "unit": unit, "cores": 1, "kind": "port", "sample": sample,
                             "host_cores": os.cpu_count()},
            "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def timed_region(torch, dist, world, fn, steps):
    """barrier + synchronize, `steps` calls of fn timed with CUDA events on the current stream, max over ranks (ms)."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, t0, t1


def run_ours(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the kernels have no CPU path")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import __graft_entry__ as entry
    if rank == 0:
        entry.build()
    if world > 1:
        dist.barrier()
    from mimir_b200 import host as H
    from mimir_b200 import tensor as T

    pk = peaks()
    w = WORKLOADS[args.workload](torch, T, H, rank, world)
    w.gather = bool(args.gather)
    if args.workload == "mlp_tp":
        w.mode = args.tp_gather
        args.no_e2e = True     # the tensor-parallel block has no single-host-buffer form
    w.setup()
    if args.gather:
        w.config["gather"] = "outputs all-gathered over NCCL inside the step" if world > 1 else "n/a at one GPU"
    # clocks are sampled every 20 ms from the first warm-up step to the end of the timed region: the timed region
    # alone (a few ms) is shorter than one nvidia-smi sampling period
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    t_warm = time.perf_counter()
    for _ in range(max(args.warmup, 3)):
        w.step()
    T.device_status()

    K = args.steps
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    ms, t0, t1 = timed_region(torch, dist, world, lambda i: w.step(evs[i]), K)
    clocks = sampler.stop(t_warm, t1) if sampler else None
    if clocks is not None:
        clocks["window"] = "warm-up + timed steps, 20 ms period"
    T.device_status()
    dom_ms = statistics.mean(a.elapsed_time(b) for a, b in evs)
    value = w.units * K * world / (ms * 1e-3) / (1e9 if w.unit == "GB/s" else 1e12)
    achieved = w.dom_units / (dom_ms * 1e-3) / (1e9 if w.bound == "hbm" else 1e12)
    peak = pk["hbm"] if w.bound == "hbm" else pk["tensor"]

    # end to end through the host-buffer entry points: pinned host inputs in, host result out, every step
    e2e = None
    if not args.no_e2e:
        w.e2e_setup()
        w.e2e_step()
        e2e_steps = max(1, min(K, 5))
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        te = time.perf_counter()
        sink = 0.0
        for _ in range(e2e_steps):
            sink += w.e2e_step()
        e2e_s = time.perf_counter() - te
        if world > 1:
            t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = float(t.item())
        e2e_val = w.units * e2e_steps * world / e2e_s / (1e9 if w.unit == "GB/s" else 1e12)
        e2e = {"value": e2e_val, "unit": w.unit, "h2d_bytes_per_step": w.h2d, "d2h_bytes_per_step": w.d2h,
               "steps": e2e_steps, "ms_per_step": e2e_s / e2e_steps * 1e3, "sink": sink}

    line = {"metric": w.metric, "value": value, "unit": w.unit, "n_gpus": world, "steps": K, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": getattr(w, "scaling", "weak"), "vs_baseline": None, "dtype": w.dtype,
            "data": "synthetic", "config": w.config, "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": K * w.launches_per_step,
            "roofline": {"bound": w.bound, "kernel": w.kernel, "achieved": achieved, "peak": peak,
                         "unit": "GB/s" if w.bound == "hbm" else "TFLOP/s", "frac": achieved / peak,
                         "peak_source": pk["source"], "avg_launch_ms": dom_ms, "traffic": w.traffic}}

    if rank == 0 and world == 1 and not args.no_cpu:
        import numpy as np

        import oracle as mo
        mo.build()
        v, sample, _ = type(w).cpu_sample(mo, np)
        line["cpu_baseline"] = {"value": v, "unit": w.unit, "cores": 1, "kind": "port", "sample": sample,
                                "host_cores": os.cpu_count()}

    if world == 1 and not args.no_extras:
        extras = {}
        for name, cls in WORKLOADS.items():
            if name == args.workload or name in ("matmul_f32", "mlp_tp"):
                continue
            w = None
            torch.cuda.empty_cache()
            w = cls(torch, T, H, rank, world)
            try:
                w.setup()
                for _ in range(3):
                    w.step()
                T.device_status()
                n = 5
                xms, _, _ = timed_region(torch, dist, world, lambda i: w.step(), n)
                T.device_status()
                v = w.units * n / (xms * 1e-3) / (1e9 if w.unit == "GB/s" else 1e12)
                pkx = pk["hbm"] if w.bound == "hbm" else pk["tensor"]
                extras[name] = {"value": v, "unit": w.unit, "ms_per_step": xms / n, "frac_of_peak": v / pkx}
            except Exception as e:  # an extra never sinks the headline
                extras[name] = {"error": str(e)[:200]}
        line["extras"] = extras

    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
