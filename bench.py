#!/usr/bin/env python
"""Benchmark of the tensor hot path on B200: one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload attn|rows|gemm|mlp|mlp_tp|matmul_f32]
    torchrun ... bench.py --gpus N ...        # one rank per GPU
    python bench.py --impl reference ...      # the CPU restatement of the reference's lowering, host cores

Workloads (seeded synthetic inputs of the stated shapes and distributions):
  attn        causal attention forward, batch 4 x 32 heads, seq 4096, head_dim 128, bf16 (the default)     TFLOP/s
  rows        X[16384,8192] f32 -> bf16, one step = row softmax + row RMSNorm (two kernels)               HBM GB/s
  gemm        bf16 8192^3, A row-major, B stored [N,K], f32 accumulation, bf16 C                           TFLOP/s
  mlp         (silu(X W1) * (X W3)) W2, X[8192,4096], W1/W3[4096,14336], W2[14336,4096], bf16              TFLOP/s
  mlp_tp      the same block tensor-parallel: W1/W3/W2 column slabs per rank, H all-gathered               TFLOP/s
  matmul_f32  f32 256^3 (the reference's CPU-runnable case)                                                TFLOP/s
Under torchrun the STATED problem is divided over the ranks (strong scaling): attention by batch x head, the
contraction by columns of B, the MLP by columns of W1 / W3 / W2; no collective on the data path except where the line
says so (`gather`). The time of a region is the max over ranks of its CUDA-event time; `value` is the whole job's
units over that time. Before anything is timed every rank checks its own shard against the CPU oracle (`parity`).
The default line carries the other workloads as full sub-records under `extras`.
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

L2_BYTES = 126 << 20


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="attn", choices=list(WORKLOADS))
    ap.add_argument("--tp-gather", default="fused", choices=["fused", "nccl", "rows", "rows_fused"],
                    help="mlp_tp: all-gather of H fused into the GEMM epilogue (peer stores) or a separate NCCL all-gather")
    ap.add_argument("--weak", action="store_true", help="under torchrun: every rank runs the whole stated problem")
    ap.add_argument("--no-extras", action="store_true", help="skip the sub-records of the other workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (for profiler runs)")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check before the timed region")
    ap.add_argument("--gather", action="store_true",
                    help="gemm / attn / mlp_tp under torchrun: all-gather every rank's output shard inside the timed step")
    return ap.parse_args()


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm": float(p["hbm_gbs"]), "tensor": float(p["bf16_tflops"]),
                "tensor_sustained": float(p["bf16_tflops_sustained"]), "source": "measured"}
    except Exception:
        return {"hbm": 6650.0, "tensor": 1590.0, "tensor_sustained": 1400.0, "source": "fallback"}


def dram_traffic_table():
    """DRAM bytes (read + write) per launch of each kernel, from the ncu captures summarised under profiles/: lines
    `kernel-key  bytes  units-of-the-captured-launch  summary-file` of profiles/dram_traffic.txt. A record's `traffic`
    is the captured figure scaled by the units its own launch processes (traffic of these kernels grows in proportion
    to the units: every operand byte is read from DRAM a fixed number of times per tile)."""
    table = {}
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.txt")) as f:
            for line in f:
                line = line.split("#")[0].strip()
                if not line:
                    continue
                key, nbytes, units, src = line.split()[:4]
                table[key] = (float(nbytes), float(units), src)
    except OSError:
        pass
    return table


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
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def window(self, t0, t1):
        """Median SM clock and the throttle reasons seen between two perf_counter stamps."""
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in list(self.samples):
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
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "window": "warm-up + timed steps, 20 ms period"}

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass


# ------------------------------------------------------------------------------------------------ workloads
def _split(n, rank, world):
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


class Workload:
    key = metric = unit = dtype = kernel = name = ""
    bound = "tensor"
    launches_per_step = 1
    scaling = "strong"
    tol = 2e-2

    def __init__(self, env, world=None, rank=None, weak=False, gather=False):
        self.env = env
        self.torch, self.T, self.H = env.torch, env.T, env.H
        self.world = env.world if world is None else world
        self.rank = env.rank if rank is None else rank
        self.weak, self.gather = weak, gather
        if weak:
            self.scaling = "weak"

    def gen(self, seed):
        g = self.torch.Generator(device="cuda")
        g.manual_seed(seed)
        return g

    def free(self):
        for k in list(self.__dict__):
            if k not in ("env", "torch", "T", "H", "world", "rank", "weak", "gather", "scaling", "units", "dom_units",
                         "traffic_units", "h2d", "d2h"):
                self.__dict__.pop(k)
        self.torch.cuda.empty_cache()


def bits_np(np, torch, t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


class Attn(Workload):
    key = "attn"
    name = "causal attention fwd bf16 batch=4 heads=32 seq=4096 head_dim=128 (config C4)"
    metric, unit, dtype, bound = "TFLOP/s (causal attention fwd)", "TFLOP/s", "bf16", "tensor"
    kernel = "attn_tc_persistent_kernel<128,208,88>"
    BH, S, D = 128, 4096, 128

    @classmethod
    def config(cls, world, weak=False, gather=False):
        nh = cls.BH if weak else cls.BH // world
        return {"workload": cls.name, "flop_count": "4*B*H*S^2*D/2 (causal)", "scale": "1/sqrt(128)",
                "heads_per_gpu": nh, "sharding": ("every GPU runs all 128 batch x head" if weak else
                                                  f"batch x head, {nh} contiguous heads per GPU, outputs stay sharded"),
                "l2": "rotating input sets of >= 384 MiB in total (larger than the 126 MB L2)",
                "gather": "O all-gathered over NCCL inside the step" if gather and world > 1 else "none"}

    def setup(self):
        t = self.torch
        self.lo, self.hi = (0, self.BH) if self.weak else _split(self.BH, self.rank, self.world)
        nh = self.hi - self.lo
        set_bytes = 3 * nh * self.S * self.D * 2
        self.nsets = max(1, -(-(384 << 20) // set_bytes))
        self.sets = []
        for i in range(self.nsets):
            # set 0 is the stated problem: all 128 heads from seed 1237, this rank keeps its own; further sets only rotate
            g = self.gen(1237 + 7919 * i)
            full = [t.randn((self.BH, self.S, self.D), generator=g, device="cuda").to(t.bfloat16) for _ in range(3)]
            self.sets.append(tuple(x[self.lo:self.hi].contiguous() for x in full))
            del full
        self.o = None
        self.units = self.dom_units = self.traffic_units = 4 * nh * self.S * self.S * self.D // 2   # causal convention
        self.i = 0

    def step(self, ev=None):
        q, k, v = self.sets[self.i % self.nsets]
        self.i += 1
        if ev:
            ev[0].record()
        self.o = self.T.attention(q, k, v, scale=1.0 / self.D ** 0.5, causal=True)
        if ev:
            ev[1].record()
        if self.gather and self.world > 1:
            self.env.all_gather(self, self.o)

    def parity(self, mo, np):
        q, k, v = self.sets[0]
        o = self.T.attention(q, k, v, scale=1.0 / self.D ** 0.5, causal=True)
        self.T.device_status()
        nh = self.hi - self.lo
        heads = sorted({(5 * self.rank + 3) % nh, nh - 1} if self.world == 1 else {(5 * self.rank + 3) % nh})
        b = lambda x: bits_np(np, self.torch, x)
        want = mo.attention(b(q), b(k), b(v), scale=1.0 / self.D ** 0.5, causal=True, bf16=True, heads=heads)
        return mo.normalised_error(o[heads].float().cpu().numpy(), want), len(heads) * self.S * self.D

    def e2e_setup(self):
        q, k, v = self.sets[0]
        self.hq, self.hk, self.hv = (x.cpu().pin_memory() for x in (q, k, v))
        self.ho = self.torch.empty_like(self.hq).pin_memory()
        n = (self.hi - self.lo) * self.S * self.D * 2
        self.h2d, self.d2h = 3 * n, n

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
        return 4 * s * s * 128 / 2 / dt / 1e12, (f"1 head at seq {s} (of 128 heads at 4096), the reference's unfused f32 "
                                                 "chain with the score matrix"), float(o[0, 0, 0])


class Rows(Workload):
    key = "rows"
    name = "row softmax + RMSNorm f32 X[16384,8192] -> bf16 (config C2)"
    metric, unit, dtype, bound = "HBM GB/s (row softmax+RMSNorm)", "GB/s", "f32", "hbm"
    kernel, launches_per_step = "rows_in_regs_kernel<0,256,8,float,__nv_bfloat16>", 2
    R, Cc = 16384, 8192
    tol = 2e-2

    @classmethod
    def config(cls, world, weak=False, gather=False):
        nr = cls.R if weak else cls.R // world
        return {"workload": cls.name, "rows_per_gpu": nr, "cols": cls.Cc, "eps": 1e-6,
                "l2": "rotating inputs of >= 512 MiB in total (larger than the 126 MB L2)",
                "sharding": "row blocks, one per GPU" if world > 1 else "one GPU"}

    def setup(self):
        t = self.torch
        self.lo, self.hi = (0, self.R) if self.weak else _split(self.R, self.rank, self.world)
        nr = self.hi - self.lo
        g = self.gen(1235)
        self.nsets = max(1, -(-(512 << 20) // (nr * self.Cc * 4)))
        full = t.randn((self.R, self.Cc), generator=g, device="cuda", dtype=t.float32)
        self.xs = [full[self.lo:self.hi].contiguous() if (self.lo, self.hi) != (0, self.R) else full]
        for i in range(1, self.nsets):
            self.xs.append(t.randn((nr, self.Cc), generator=g, device="cuda", dtype=t.float32))
        self.gamma = t.rand((self.Cc,), generator=self.gen(2235), device="cuda", dtype=t.float32) + 0.5
        self.units = 2 * (nr * self.Cc * 6) + self.Cc * 4      # algorithmic bytes per step (read f32 + write bf16, twice)
        self.dom_units = self.traffic_units = nr * self.Cc * 6  # the softmax launch
        self.i = 0

    def step(self, ev=None):
        x = self.xs[self.i % self.nsets]
        self.i += 1
        if ev:
            ev[0].record()
        self.y1 = self.T.softmax(1, x, out_dtype=self.torch.bfloat16)
        if ev:
            ev[1].record()
        self.y2 = self.T.rmsnorm(x, self.gamma, 1e-6, out_dtype=self.torch.bfloat16)

    def parity(self, mo, np):
        x = self.xs[0]
        y1 = self.T.softmax(1, x, out_dtype=self.torch.bfloat16)
        y2 = self.T.rmsnorm(x, self.gamma, 1e-6, out_dtype=self.torch.bfloat16)
        rows = [0, (x.shape[0] // 2) + 1, x.shape[0] - 1]
        xs = x[rows].cpu().numpy()
        e1 = mo.normalised_error(y1[rows].float().cpu().numpy(), mo.softmax_rows(xs, truth=True))
        e2 = mo.normalised_error(y2[rows].float().cpu().numpy(), mo.rmsnorm_rows(xs, self.gamma.cpu().numpy(), 1e-6, truth=True))
        return max(e1, e2), 2 * len(rows) * self.Cc

    def e2e_setup(self):
        t = self.torch
        nr = self.hi - self.lo
        self.hx = self.xs[0].cpu().pin_memory()
        self.hg = self.gamma.cpu().pin_memory()
        self.hy1 = t.empty((nr, self.Cc), dtype=t.bfloat16).pin_memory()
        self.hy2 = t.empty((nr, self.Cc), dtype=t.bfloat16).pin_memory()
        self.h2d = nr * self.Cc * 4 + self.Cc * 4     # x is uploaded once for both results
        self.d2h = 2 * nr * self.Cc * 2

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
    key = "gemm"
    name = "matmul bf16 M=N=K=8192, A row-major, B stored [N,K], f32 accumulate (config C3)"
    metric, unit, dtype, bound = "TFLOP/s (bf16 GEMM 8192^3)", "TFLOP/s", "bf16", "tensor"
    kernel = "gemm_tc2_kernel<256,0,0,__nv_bfloat16>"
    n = 8192

    @classmethod
    def config(cls, world, weak=False, gather=False):
        nc = cls.n if weak else cls.n // world
        return {"workload": cls.name, "columns_per_gpu": nc, "l2": "A (128 MiB) + B slab stream through the 126 MB L2",
                "sharding": "A replicated, B column slabs (rows of the stored [N,K] tensor)" if world > 1 else "one GPU",
                "gather": ("C column slabs all-gathered over NCCL inside the step" if gather and world > 1 else "none")}

    def setup(self):
        t = self.torch
        g = self.gen(1236)
        self.lo, self.hi = (0, self.n) if self.weak else _split(self.n, self.rank, self.world)
        self.a = (t.randn((self.n, self.n), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        b = (t.randn((self.n, self.n), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        self.b = b[self.lo:self.hi].contiguous() if (self.lo, self.hi) != (0, self.n) else b
        del b
        self.units = self.dom_units = self.traffic_units = 2 * self.n * self.n * (self.hi - self.lo)
        self.full = None

    def step(self, ev=None):
        if ev:
            ev[0].record()
        self.c = self.T.product_2d(self.a, self.T.transpose_2d(self.b))
        if ev:
            ev[1].record()
        if self.gather and self.world > 1:
            self.full = self.env.all_gather_columns(self, self.c)

    def parity(self, mo, np):
        self.step()
        self.T.device_status()
        rows = [0, 4097, self.n - 1]
        b = lambda x: bits_np(np, self.torch, x)
        want = mo.gemm_truth(b(self.a), b(self.b), b_nk=True, bf16=True, rows=rows)
        err = mo.normalised_error(self.c[rows].float().cpu().numpy(), want)
        checked = want.size
        if self.gather and self.world > 1:
            # the gathered matrix holds every rank's slab: compare this rank's view of ALL columns with the oracle's
            g = self.gen(1236)
            t = self.torch
            t.randn((self.n, self.n), generator=g, device="cuda")
            bfull = (t.randn((self.n, self.n), generator=g, device="cuda") * 0.02).to(t.bfloat16)
            want = mo.gemm_truth(b(self.a), b(bfull), b_nk=True, bf16=True, rows=rows[:2])
            err = max(err, mo.normalised_error(self.full[rows[:2]].float().cpu().numpy(), want))
            checked += want.size
        return err, checked

    def e2e_setup(self):
        self.ha, self.hb = self.a.cpu().pin_memory(), self.b.cpu().pin_memory()
        nc = self.hi - self.lo
        self.hc = self.torch.empty((self.n, nc), dtype=self.torch.bfloat16).pin_memory()
        self.h2d, self.d2h = (self.n + nc) * self.n * 2, self.n * nc * 2

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


class Mlp(Workload):
    key = "mlp"
    name = "MLP block bf16 X[8192,4096] W1/W3[4096,14336] SiLU-gate W2[14336,4096] (config C5)"
    metric, unit, dtype, bound = "TFLOP/s (gated MLP block)", "TFLOP/s", "bf16", "tensor"
    kernel, launches_per_step = "gemm_tc2_kernel<128,1,1,__nv_bfloat16>+gemm_tc2_kernel<256,1,0,__nv_bfloat16>", 2
    M, K, F = 8192, 4096, 14336
    scaling = "weak"      # one GPU's block; the tensor-parallel form is mlp_tp

    @classmethod
    def config(cls, world, weak=False, gather=False):
        return {"workload": cls.name, "l2": "weights (336 MiB) larger than the 126 MB L2",
                "sharding": "replica per GPU" if world > 1 else "one GPU"}

    def weights(self):
        t = self.torch
        g = self.gen(1238)                       # the same global tensors on every rank
        x = t.randn((self.M, self.K), generator=g, device="cuda").to(t.bfloat16)
        w1 = (t.randn((self.K, self.F), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        w3 = (t.randn((self.K, self.F), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        w2 = (t.randn((self.F, self.K), generator=g, device="cuda") * 0.02).to(t.bfloat16)
        return x, w1, w3, w2

    def setup(self):
        t = self.torch
        self.x, self.w1, self.w3, self.w2 = self.weights()
        self.h = t.empty((self.M, self.F), device="cuda", dtype=t.bfloat16)
        self.units = self.dom_units = self.traffic_units = 3 * 2 * self.M * self.K * self.F   # events bracket both launches

    def step(self, ev=None):
        if ev:
            ev[0].record()
        self.y = self.T.mlp_gated(self.x, self.w1, self.w3, self.w2, h=self.h)
        if ev:
            ev[1].record()

    def parity(self, mo, np):
        self.step()
        self.T.device_status()
        rows = [1, self.M - 1]
        b = lambda x: bits_np(np, self.torch, x)
        want = mo.mlp_gated_truth(b(self.x[rows]), b(self.w1), b(self.w3), b(self.w2))
        return mo.normalised_error(self.y[rows].float().cpu().numpy(), want), want.size

    def e2e_setup(self):
        self.hx, self.hw1, self.hw3, self.hw2 = (x.cpu().pin_memory() for x in (self.x, self.w1, self.w3, self.w2))
        self.hy = self.torch.empty((self.M, self.K), dtype=self.torch.bfloat16).pin_memory()
        self.h2d = (self.M * self.K + 3 * self.K * self.F) * 2
        self.d2h = self.M * self.K * 2

    def e2e_step(self):
        self.H.mlp_gated(self.hx, self.hw1, self.hw3, self.hw2, out=self.hy)
        return float(self.hy[0, 0])

    @staticmethod
    def cpu_sample(mo, np, rows=4):
        rng = np.random.default_rng(1238)
        x = mo.to_bf16(rng.standard_normal((rows, 4096)).astype(np.float32))
        w1, w3 = (mo.to_bf16((rng.standard_normal((4096, 14336)) * 0.02).astype(np.float32)) for _ in range(2))
        w2 = mo.to_bf16((rng.standard_normal((14336, 4096)) * 0.02).astype(np.float32))
        t0 = time.perf_counter()
        # the block as the reference lowers it: two f32-accumulating contractions, the gate, the third contraction
        g, u = mo.gemm(x, w1, bf16=True), mo.gemm(x, w3, bf16=True)
        h = mo.to_bf16((g / (1.0 + np.exp(-g)) * u).astype(np.float32))
        y = mo.gemm(h, w2, bf16=True)
        dt = time.perf_counter() - t0
        return 6 * rows * 4096 * 14336 / dt / 1e12, f"{rows} of 8192 rows through the full block, f32 accumulate ascending k", float(y[0, 0])


class MlpTP(Mlp):  # noqa: D101
    """The C5 block split over the ranks (tensor parallel, strong scaling): rank g owns columns [g F/G, (g+1) F/G) of W1
    and W3 and columns [g N/G, (g+1) N/G) of W2; H is all-gathered between the two stages."""
    key = "mlp_tp"
    name = "MLP block bf16 X[8192,4096] W1/W3[4096,14336] W2[14336,4096], tensor parallel (config C5)"
    metric = "TFLOP/s (gated MLP block, tensor parallel)"
    # the second contraction runs on the paired-SM kernel or, with few tiles per rank, on the one-CTA kernel: no single
    # captured launch stands for it, so this record carries no DRAM traffic figure
    kernel = "gemm_tc2_kernel<128,1,1,__nv_bfloat16>+gemm_tc2_kernel|gemm_tc_kernel<256,1,0,__nv_bfloat16>"
    scaling = "strong"
    mode = "fused"

    @classmethod
    def config(cls, world, weak=False, gather=False, mode="fused"):
        return {"workload": cls.name, "l2": "weights and H larger than the 126 MB L2",
                "tp_gather": (mode + {"fused": " (H slabs stored into every rank's H from the contraction's epilogue over NVLink)",
                                      "nccl": " (separate NCCL all-gather of the H slabs)",
                                      "rows": " (no gather of H: f32 partials of Y reduce-scattered over NCCL)",
                                      "rows_fused": " (no gather of H: f32 partials of Y added into the owners' row blocks from the "
                                                    "second contraction's epilogue, bulk reductions over NVLink)"}[mode]) if world > 1 else "n/a",
                "sharding": ("W1/W3 column slabs, W2 ROW slabs, Y row blocks after the reduce-scatter" if mode.startswith("rows") and world > 1 else
                             "W1/W3 column slabs, H all-gathered, W2 column slabs" +
                             (", Y all-gathered too" if gather and world > 1 else " (Y stays sharded)"))}

    def setup(self):
        t = self.torch
        from mimir_b200 import shard
        self.shard = shard
        W = self.world
        self.fl, self.nl = self.F // W, self.K // W
        x, w1, w3, w2 = self.weights()
        r = self.rank
        self.x = x
        self.w1 = w1[:, r * self.fl:(r + 1) * self.fl].contiguous()
        self.w3 = w3[:, r * self.fl:(r + 1) * self.fl].contiguous()
        self.w2 = (w2[r * self.fl:(r + 1) * self.fl, :] if self.mode.startswith("rows") and W > 1 else w2[:, r * self.nl:(r + 1) * self.nl]).contiguous()
        del w1, w3, w2
        t.cuda.empty_cache()
        self.yg = self.hg = None
        if W > 1 and self.mode == "fused":
            self.hg = shard.GatheredMatrix(self.M, self.F)
            if self.gather:
                self.yg = shard.GatheredMatrix(self.M, self.K)
        else:
            self.h_local = t.empty((self.M, self.fl), device="cuda", dtype=t.bfloat16)
            if W > 1 and self.mode == "rows":
                self.y_partial = t.empty((self.M, self.K), device="cuda", dtype=t.float32)
            if W > 1 and self.mode == "rows_fused":
                self.acc = shard.GatheredMatrix(self.M // W, self.K, dtype=t.float32)
        self.units = self.dom_units = self.traffic_units = 3 * 2 * self.M * self.K * self.F // W     # this rank's share

    def step(self, ev=None):
        if ev:
            ev[0].record()
        if self.world == 1:
            self.y = self.T.mlp_gated(self.x, self.w1, self.w3, self.w2, h=self.h_local)
        elif self.mode == "fused":
            self.y = self.shard.tp_mlp_gated(self.x, self.w1, self.w3, self.w2, self.hg, gather="fused", y=self.yg)
        elif self.mode == "rows":
            self.y = self.shard.tp_mlp_gated_rows(self.x, self.w1, self.w3, self.w2, self.h_local, self.y_partial)
        elif self.mode == "rows_fused":
            self.y = self.shard.tp_mlp_gated_rows_fused(self.x, self.w1, self.w3, self.w2, self.h_local, self.acc)
        else:
            self.y = self.shard.tp_mlp_gated_nccl(self.x, self.w1, self.w3, self.w2, self.h_local, gather_y=self.gather)
        if ev:
            ev[1].record()

    def parity(self, mo, np):
        t = self.torch
        self.step()
        self.T.device_status()
        t.cuda.synchronize()
        x, w1, w3, w2 = self.weights()
        rows = [1, self.M - 1]
        b = lambda v: bits_np(np, t, v)
        if self.mode.startswith("rows") and self.world > 1:  # this rank holds rows [r M/W, (r+1) M/W) of the whole Y
            per = self.M // self.world
            mine = [1, per - 1]
            rows = [self.rank * per + i for i in mine]
            want = mo.mlp_gated_truth(b(x[rows]), b(w1), b(w3), b(w2))
            got = self.y[mine]
        else:
            want = mo.mlp_gated_truth(b(x[rows]), b(w1), b(w3), b(w2))
            if not (self.gather and self.world > 1):
                want = want[:, self.rank * self.nl:(self.rank + 1) * self.nl]
            got = self.y[rows]
        err = mo.normalised_error(got.float().cpu().numpy(), want)
        checked = want.size
        if self.world > 1 and self.mode == "fused":
            # the gathered H on this rank against the one-GPU product of the whole operands: the same bits, whoever wrote them
            h1 = t.empty((self.M, self.F), device="cuda", dtype=t.bfloat16)
            self.T.mlp_gated(x, w1, w3, w2, h=h1)
            same = bool(t.equal(self.hg.local, h1))
            self.hg.barrier()
            if not same:
                err = float("inf")
            checked += h1.numel()
        return err, checked

    def e2e_setup(self):
        self.h2d = self.d2h = 0

    def e2e_step(self):
        return 0.0


class MatmulF32(Workload):
    key = "matmul_f32"
    name = "matmul f32 256^3 (config C1)"
    metric, unit, dtype, bound = "TFLOP/s (f32 matmul 256^3)", "TFLOP/s", "f32", "tensor"
    kernel = "gemm_simt_small_kernel<0>"
    launches_per_step = 1
    scaling = "weak"
    tol = 1e-5

    @classmethod
    def config(cls, world, weak=False, gather=False):
        return {"workload": cls.name, "l2": "160 MiB buffer written between steps", "sharding": "replicas only"}

    def setup(self):
        t = self.torch
        g = self.gen(1234)
        self.a = t.rand((256, 256), generator=g, device="cuda") * 2 - 1
        self.b = t.rand((256, 256), generator=g, device="cuda") * 2 - 1
        self.flush = t.empty(160 << 20, dtype=t.uint8, device="cuda")
        self.units = self.dom_units = self.traffic_units = 2 * 256 ** 3

    def step(self, ev=None):
        self.flush.zero_()
        if ev:
            ev[0].record()
        self.c = self.T.product_2d(self.a, self.b)
        if ev:
            ev[1].record()

    def parity(self, mo, np):
        self.step()
        want = mo.gemm_truth(self.a.cpu().numpy(), self.b.cpu().numpy())
        return mo.normalised_error(self.c.double().cpu().numpy(), want), want.size

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


WORKLOADS = {"attn": Attn, "rows": Rows, "gemm": Gemm, "mlp": Mlp, "mlp_tp": MlpTP, "matmul_f32": MatmulF32}


# ------------------------------------------------------------------------------------------------ CPU baseline
def cpu_baseline(W, budget_s, warmup=1, steps=None):
    """The oracle's as-lowered loops on ONE host core (the reference emits single-threaded code: no OpenMP, no threads
    anywhere in its output), built the way its own CPU lowering is: -O3 -march=native with contraction, and the same with
    fast-math flags (its math.mode.fast). Both are timed; `value` is the faster one. Returns (record, per-step list)."""
    import numpy as np

    import oracle as mo
    mo.build()
    out = {"unit": W.unit, "cores": 1, "kind": "port", "host_cores": os.cpu_count(), "flags": {}}
    best, best_vals, best_wall = None, [], 0.0
    for variant, flags in mo.TIMED_FLAGS.items():
        with mo.timed_build(variant):
            for _ in range(warmup):
                W.cpu_sample(mo, np)
            vals, t0 = [], time.perf_counter()
            while True:
                v, sample, _ = W.cpu_sample(mo, np)
                vals.append(v)
                if (steps is not None and len(vals) >= steps) or (steps is None and time.perf_counter() - t0 > budget_s / 2):
                    break
                if time.perf_counter() - t0 > 150:
                    break
            wall = (time.perf_counter() - t0) / len(vals)
        out["flags"][flags] = statistics.mean(vals)
        out["sample"] = sample
        if best is None or statistics.mean(vals) > best:
            best, best_vals, best_wall, out["built_with"] = statistics.mean(vals), vals, wall, flags
    out["value"] = best
    out["ms_per_pass"] = best_wall * 1e3
    return out, best_vals


def run_reference(args):
    """The reference's lowering, restated for the CPU (oracle/), timed on this box's host cores: each step is one pass
    over a bounded sample of the same workload (stated in `config.sample`). Rank 0 alone runs it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    W = WORKLOADS[args.workload]
    rec, vals = cpu_baseline(W, 0, warmup=max(0, args.warmup), steps=max(1, args.steps))
    config = dict(_config(W, args, args.gpus))
    config["sample"] = rec["sample"]
    ms_per_step = rec["ms_per_pass"]          # one step = one pass over the bounded sample (inputs generated inside)
    line = {"impl": "reference", "metric": W.metric, "value": rec["value"], "unit": W.unit, "n_gpus": args.gpus,
            "steps": len(vals), "warmup": max(0, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak" if args.weak else W.scaling, "vs_baseline": None, "dtype": W.dtype, "data": "synthetic",
            "config": config, "cpu_baseline": rec,
            "e2e": {"value": rec["value"], "unit": W.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def _config(W, args, world, **kw):
    if W is MlpTP:
        return W.config(world, weak=args.weak, gather=args.gather, mode=kw.get("mode", args.tp_gather))
    return W.config(world, weak=args.weak, gather=args.gather)


# ------------------------------------------------------------------------------------------------ GPU arm
class Env:
    """What every workload needs: torch, the library's two Python faces, the process group, and the collectives the
    `gather` variants use (NCCL over NVLink)."""

    def __init__(self):
        import torch
        self.torch = torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; the kernels have no CPU path")
        torch.cuda.set_device(self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.dist = dist
        import __graft_entry__ as entry
        if self.rank == 0:
            entry.build()
        self.barrier()
        from mimir_b200 import host as H
        from mimir_b200 import tensor as T
        self.T, self.H = T, H
        self.gathered = {}

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def max_over_ranks(self, v):
        if not self.dist:
            return v
        t = self.torch.tensor([v], device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, v):
        if not self.dist:
            return v
        t = self.torch.tensor([v], device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def all_gather(self, w, local):
        """All-gather the ranks' output shards (leading axis) into one tensor on every rank."""
        key = (id(w), "rows")
        if key not in self.gathered:
            self.gathered[key] = self.torch.empty((self.world * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype,
                                                  device=local.device)
        self.dist.all_gather_into_tensor(self.gathered[key], local)
        return self.gathered[key]

    def all_gather_columns(self, w, local):
        """All-gather column slabs into the full row-major matrix on every rank."""
        from mimir_b200 import shard
        return shard.gather_columns(local, local.shape[1] * self.world)


def timed_region(env, fn, steps):
    """barrier + synchronize, `steps` calls of fn timed with CUDA events on the current stream, max over ranks (ms)."""
    torch = env.torch
    env.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    env.barrier()
    return env.max_over_ranks(e0.elapsed_time(e1)), t0, t1


def measure(env, w, args, pk, traffic, sampler, *, e2e=True, cpu=True, config=None):
    """One full record of a workload: parity against the oracle, the device-timed region, the roofline of its dominant
    launch, the end-to-end leg through host buffers, the CPU baseline (rank 0 of a one-GPU run)."""
    torch, T = env.torch, env.T
    K, warm = args.steps, max(args.warmup, 3)
    w.setup()
    rec = {"metric": w.metric, "unit": w.unit, "dtype": w.dtype, "scaling": w.scaling, "config": config}

    if not args.no_parity:
        import numpy as np

        import oracle as mo
        mo.build()
        err, checked = w.parity(mo, np)
        err = env.max_over_ranks(err if err == err else float("inf"))
        rec["parity"] = {"max_err": err, "tolerance": w.tol, "checked": int(env.sum_over_ranks(checked)),
                         "ok": bool(err <= w.tol), "against": "CPU oracle (f64), normalised max error; every rank checks its own shard"}
        if not rec["parity"]["ok"]:
            raise SystemExit(f"bench.py: parity failed for {w.key}: {rec['parity']}")

    t_warm = time.perf_counter()
    for _ in range(warm):
        w.step()
    T.device_status()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    ms, t0, t1 = timed_region(env, lambda i: w.step(evs[i]), K)
    T.device_status()
    if sampler:
        time.sleep(0.06)
        rec["clocks"] = sampler.window(t_warm, t1)
    div = 1e9 if w.unit == "GB/s" else 1e12
    total_units = env.sum_over_ranks(w.units)
    dom_ms = env.max_over_ranks(statistics.mean(a.elapsed_time(b) for a, b in evs))
    peak = pk["hbm"] if w.bound == "hbm" else pk["tensor"]
    achieved = w.dom_units / (dom_ms * 1e-3) / (1e9 if w.bound == "hbm" else 1e12)
    # DRAM bytes of the launches the events bracket: every kernel of `w.kernel` must have a captured figure; the captured
    # launches together did `cap_units` of work, this rank's launches do `w.traffic_units`
    tr, parts = None, w.kernel.split("+")
    if all(part in traffic for part in parts):
        nbytes = sum(traffic[part][0] for part in parts)
        cap_units = sum(traffic[part][1] for part in parts)
        tr = {"bytes": nbytes * w.traffic_units / cap_units, "source": sorted({f"profiles/{traffic[part][2]}" for part in parts}),
              "scaled_by_units": w.traffic_units / cap_units}
    rec.update({"value": total_units * K / (ms * 1e-3) / div, "ms_per_step": ms / K, "steps": K, "warmup": warm,
                "gpu_launches": K * w.launches_per_step,
                "roofline": {"bound": w.bound, "kernel": w.kernel, "achieved": achieved, "peak": peak,
                             "unit": "GB/s" if w.bound == "hbm" else "TFLOP/s", "frac": achieved / peak,
                             "peak_source": pk["source"] + (" (cuBLAS bf16 burst)" if w.bound == "tensor" else " (copy)"),
                             "avg_launch_ms": dom_ms, "per": "GPU (slowest rank's mean launch)",
                             "traffic": tr["bytes"] if tr else None, "traffic_source": tr}})

    # end to end through the host-buffer entry points: pinned host inputs in, host result out, every step
    if e2e and not args.no_e2e:
        w.e2e_setup()
        if w.h2d:
            w.e2e_step()
            w.e2e_step()
            n = max(3, min(K, 10))
            env.barrier()
            torch.cuda.synchronize()
            te = time.perf_counter()
            sink = 0.0
            for _ in range(n):
                sink += w.e2e_step()
            s = env.max_over_ranks(time.perf_counter() - te)
            rec["e2e"] = {"value": total_units * n / s / div, "unit": w.unit,
                          "h2d_bytes_per_step": int(env.sum_over_ranks(w.h2d)), "d2h_bytes_per_step": int(env.sum_over_ranks(w.d2h)),
                          "steps": n, "ms_per_step": s / n * 1e3, "sink": sink,
                          "path": "mimir_b200.host (pinned host tensors -> mimk_host_* -> host result), wall clock, max over ranks"}
    if cpu and env.rank == 0 and env.world == 1 and not args.no_cpu:
        rec["cpu_baseline"], _ = cpu_baseline(type(w), 12.0)
    w.free()
    return rec


def run_ours(args):
    env = Env()
    pk, traffic = peaks(), dram_traffic_table()
    sampler = ClockSampler(env.local).start() if env.rank == 0 else None
    if sampler:
        time.sleep(0.3)
    W = WORKLOADS[args.workload]
    w = W(env, weak=args.weak, gather=args.gather)
    if W is MlpTP:
        w.mode = args.tp_gather
    line = measure(env, w, args, pk, traffic, sampler, config=_config(W, args, env.world))
    line = {"metric": line.pop("metric"), "value": line.pop("value"), "unit": line.pop("unit"), "n_gpus": env.world,
            "steps": line.pop("steps"), "warmup": line.pop("warmup"), "ms_per_step": line.pop("ms_per_step"),
            "higher_is_better": True, "scaling": line.pop("scaling"), "vs_baseline": None, "dtype": line.pop("dtype"),
            "data": "synthetic", **line}
    if "e2e" not in line:
        line["e2e"] = None

    if not args.no_extras:
        extras = {}
        plan = []
        if env.world == 1:
            plan = [("rows", Rows, {}), ("gemm", Gemm, {}), ("mlp", Mlp, {})]
        else:
            plan = [("attn_weak", Attn, {"weak": True}),
                    ("gemm_cols", Gemm, {}), ("gemm_cols_gather", Gemm, {"gather": True}),
                    ("mlp_tp_fused", MlpTP, {"mode": "fused"}), ("mlp_tp_nccl", MlpTP, {"mode": "nccl"}),
                    ("mlp_tp_rows", MlpTP, {"mode": "rows"}), ("mlp_tp_rows_fused", MlpTP, {"mode": "rows_fused"})]
        plan = [p for p in plan if not (p[1] is W and not p[2])]
        for name, cls, kw in plan:
            env.torch.cuda.empty_cache()
            sub = argparse.Namespace(**vars(args))
            sub.weak, sub.gather = kw.get("weak", False), kw.get("gather", False)
            x = cls(env, weak=sub.weak, gather=sub.gather)
            if cls is MlpTP:
                x.mode = kw["mode"]
            try:
                extras[name] = measure(env, x, sub, pk, traffic, sampler, e2e=env.world == 1, cpu=True,
                                       config=_config(cls, sub, env.world, **kw))
            except SystemExit:
                raise
            except Exception as e:  # an extra never sinks the headline
                extras[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
                env.barrier()
        line["extras"] = extras
        line["gpu_launches"] += sum(v.get("gpu_launches", 0) for v in extras.values())
        line["gpu_launches_note"] = "headline's timed region + the extras' timed regions"

    if sampler:
        sampler.stop()
    if env.rank == 0:
        print(json.dumps(line), flush=True)
    if env.dist:
        env.barrier()
        env.dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
