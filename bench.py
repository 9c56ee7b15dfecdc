#!/usr/bin/env python
"""Benchmark of the quantized-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Prints ONE JSON line (rank 0).  A "step" is one pass of the headline workload over its synthetic input:
the operator call(s) through the C ABI with inputs resident in HBM (``value``), and the same call with
pinned-host inputs and a device->host read of the result inside the timed region (``e2e``).  The other
benchmark configurations are measured in the same run and reported under ``workloads``.  Timing is by CUDA
events on the launching stream; buffers rotate over a set larger than L2 so every step reads DRAM.
``--impl reference`` times the CPU restatement of the reference operators (oracle/, all host threads) on a
bounded sample of the same workload; the reference's own CPU-debug build needs the closed tikicpulib and
cannot be produced here.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
SEED = 20251125


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# Synthetic inputs (numpy, seeded): the five benchmark configurations.
# ------------------------------------------------------------------------------------------------
def f32_to_bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def gen_quant_cfg1(rows=256, cols=4096):
    rng = np.random.default_rng(SEED + 1)
    return {"x": rng.standard_normal((rows, cols), dtype=np.float32).astype(np.float16)}


def gen_antiquant_cfg2(K=4096, N=11008):
    rng = np.random.default_rng(SEED + 2)
    return {"w": rng.integers(-127, 128, (K, N), dtype=np.int8),
            "scale": f32_to_bf16_bits(rng.uniform(0.001, 0.02, N).astype(np.float32)),
            "offset": f32_to_bf16_bits(rng.uniform(-4, 4, N).astype(np.float32))}


def gen_dequant_cfg3(M=2048, N=4096):
    rng = np.random.default_rng(SEED + 3)
    return {"acc": rng.integers(-2 ** 20, 2 ** 20 + 1, (M, N)).astype(np.int32),
            "sch": rng.uniform(1e-5, 1e-3, N).astype(np.float32), "stok": rng.uniform(0.5, 2.0, M).astype(np.float32)}


def gen_w8a8_cfg4(M=4096, N=4096, K=4096):
    rng = np.random.default_rng(SEED + 4)
    return {"A": np.clip(np.rint(rng.normal(0, 30, (M, K))), -127, 127).astype(np.int8),
            "B": rng.integers(-127, 128, (N, K), dtype=np.int8),
            "sA": rng.uniform(0.005, 0.02, M).astype(np.float32), "sB": rng.uniform(0.001, 0.01, N).astype(np.float32),
            "bias": f32_to_bf16_bits(rng.normal(0, 0.1, N).astype(np.float32))}


def gen_mxfp4_cfg5(G=16, total=16384, K=7168, N=2048):
    rng = np.random.default_rng(SEED + 5)
    groups = rng.multinomial(total, np.full(G, 1.0 / G)).astype(np.int64)
    return {"groups": groups,
            "A": rng.integers(0, 256, (total, K // 2), dtype=np.uint8),          # all 16 E2M1 codes, two per byte
            "sA": (127 + rng.integers(-4, 5, (total, K // 32))).astype(np.uint8),
            "B": rng.integers(0, 256, (G, N, K // 2), dtype=np.uint8),
            "sB": (127 + rng.integers(-4, 5, (G, N, K // 32))).astype(np.uint8)}


# ------------------------------------------------------------------------------------------------
# Workloads.  Each owns `nsets` rotating device buffer sets and knows its algorithmic bytes.
# ------------------------------------------------------------------------------------------------
class Workload:
    name = ""
    unit = "GB/s"
    bound = "hbm"
    dtype = ""
    launches_per_step = 1

    def work_per_step(self):  # algorithmic bytes (hbm) or ops (tensor)
        raise NotImplementedError

    def nsets_for(self, bytes_per_set):
        return max(2, int(np.ceil(2.0 * L2_BYTES / bytes_per_set)) + 1)


class AntiQuantCfg2(Workload):
    name = "AscendAntiQuant per-channel int8[4096,11008] -> bf16 (config 2)"
    dtype = "f32"
    key = "antiquant_cfg2"

    def __init__(self, torch, ops, dev):
        self.torch, self.ops = torch, ops
        self.K, self.N = 4096, 11008
        h = gen_antiquant_cfg2(self.K, self.N)
        self.host = h
        per_set = self.K * self.N * 3
        self.nsets = self.nsets_for(per_set)
        self.w = [torch.from_numpy(h["w"]).to(dev) for _ in range(self.nsets)]
        self.out = [torch.empty((self.K, self.N), dtype=torch.bfloat16, device=dev) for _ in range(self.nsets)]
        self.scale = torch.from_numpy(h["scale"].view(np.int16)).to(dev).view(torch.bfloat16)
        self.offset = torch.from_numpy(h["offset"].view(np.int16)).to(dev).view(torch.bfloat16)
        self.para = ops.AscendAntiQuantParam(self.K, self.N)
        # e2e: pinned host input and output
        self.h_in = torch.from_numpy(h["w"]).pin_memory()
        self.h_out = torch.empty((self.K, self.N), dtype=torch.bfloat16).pin_memory()

    def work_per_step(self):
        return self.K * self.N * 3 + 2 * self.N * 2

    def step(self, i):
        s = i % self.nsets
        self.ops.AscendAntiQuant(self.out[s], self.w[s], self.offset, self.scale, self.para)

    def e2e_step(self, i):
        s = i % self.nsets
        self.w[s].copy_(self.h_in, non_blocking=True)
        self.ops.AscendAntiQuant(self.out[s], self.w[s], self.offset, self.scale, self.para)
        self.h_out.copy_(self.out[s], non_blocking=True)

    def e2e_bytes(self):
        return self.K * self.N, self.K * self.N * 2

    def cpu_sample(self, O):
        rows = 512
        w = np.ascontiguousarray(self.host["w"][:rows])
        t0 = time.perf_counter()
        O.ascend_antiquant(w, O.I8, O.BF16, policy=O.PER_CHANNEL, m=rows, n=self.N, scale=self.host["scale"],
                           offset=self.host["offset"], scaleT=O.BF16)
        dt = time.perf_counter() - t0
        return rows * self.N * 3 / dt / 1e9, f"{rows} of {self.K} rows"

    def check(self, O):
        rows = 64
        want = O.ascend_antiquant(np.ascontiguousarray(self.host["w"][:rows]), O.I8, O.BF16, policy=O.PER_CHANNEL, m=rows,
                                  n=self.N, scale=self.host["scale"], offset=self.host["offset"], scaleT=O.BF16)
        got = self.out[0][:rows].view(self.torch.int16).cpu().numpy().view(np.uint16)
        return bool(np.array_equal(got, want))


class DequantCfg3(Workload):
    name = "AscendDequant per-channel x per-token int32[2048,4096] -> bf16 (config 3)"
    dtype = "f32"
    key = "dequant_cfg3"

    def __init__(self, torch, ops, dev):
        self.torch, self.ops = torch, ops
        self.M, self.N = 2048, 4096
        h = gen_dequant_cfg3(self.M, self.N)
        self.host = h
        self.nsets = self.nsets_for(self.M * self.N * 6)
        self.acc = [torch.from_numpy(h["acc"]).to(dev) for _ in range(self.nsets)]
        self.out = [torch.empty((self.M, self.N), dtype=torch.bfloat16, device=dev) for _ in range(self.nsets)]
        self.sch = torch.from_numpy(h["sch"]).to(dev)
        self.stok = torch.from_numpy(h["stok"]).to(dev)
        self.params = ops.DequantParams(self.M, self.N, self.N)
        self.h_in = torch.from_numpy(h["acc"]).pin_memory()
        self.h_out = torch.empty((self.M, self.N), dtype=torch.bfloat16).pin_memory()

    def work_per_step(self):
        return self.M * self.N * 6 + self.N * 4 + self.M * 4

    def step(self, i):
        s = i % self.nsets
        self.ops.AscendDequant(self.out[s], self.acc[s], self.sch, self.params, tokScale=self.stok)

    def e2e_step(self, i):
        s = i % self.nsets
        self.acc[s].copy_(self.h_in, non_blocking=True)
        self.ops.AscendDequant(self.out[s], self.acc[s], self.sch, self.params, tokScale=self.stok)
        self.h_out.copy_(self.out[s], non_blocking=True)

    def e2e_bytes(self):
        return self.M * self.N * 4, self.M * self.N * 2

    def cpu_sample(self, O):
        rows = 512
        acc = np.ascontiguousarray(self.host["acc"][:rows])
        t0 = time.perf_counter()
        O.ascend_dequant(acc, O.I32, O.BF16, policy=O.PER_CHANNEL, m=rows, n=self.N, calCount=self.N,
                         scale=self.host["sch"], tokScale=self.host["stok"][:rows].copy(), scaleT=O.F32)
        dt = time.perf_counter() - t0
        return rows * self.N * 6 / dt / 1e9, f"{rows} of {self.M} rows"

    def check(self, O):
        rows = 64
        want = O.ascend_dequant(np.ascontiguousarray(self.host["acc"][:rows]), O.I32, O.BF16, policy=O.PER_CHANNEL, m=rows,
                                n=self.N, calCount=self.N, scale=self.host["sch"],
                                tokScale=self.host["stok"][:rows].copy(), scaleT=O.F32)
        got = self.out[0][:rows].view(self.torch.int16).cpu().numpy().view(np.uint16)
        return bool(np.array_equal(got, want))


class QuantScaled(Workload):
    """Config 1's operator (per-tensor fp16 -> int8, scale 64) on fp16 [16384, 8192]: config 1 itself is 3 MiB,
    which no kernel can stream from DRAM at a meaningful rate; its latency is reported separately."""
    name = "AscendQuant per-tensor fp16[16384,8192] -> int8 (config 1 operator, DRAM-sized)"
    dtype = "f16"
    key = "quant_scaled"

    def __init__(self, torch, ops, dev, rows=16384, cols=8192):
        self.torch, self.ops = torch, ops
        self.rows, self.cols = rows, cols
        h = gen_quant_cfg1(rows, cols)
        self.host = h
        self.nsets = self.nsets_for(rows * cols * 3)
        self.x = [torch.from_numpy(h["x"]).to(dev) for _ in range(self.nsets)]
        self.out = [torch.empty((rows, cols), dtype=torch.int8, device=dev) for _ in range(self.nsets)]
        self.h_in = torch.from_numpy(h["x"]).pin_memory()
        self.h_out = torch.empty((rows, cols), dtype=torch.int8).pin_memory()

    def work_per_step(self):
        return self.rows * self.cols * 3

    def step(self, i):
        s = i % self.nsets
        self.ops.AscendQuant(self.out[s], self.x[s], 64.0, 0.0, self.rows * self.cols)

    def e2e_step(self, i):
        s = i % self.nsets
        self.x[s].copy_(self.h_in, non_blocking=True)
        self.ops.AscendQuant(self.out[s], self.x[s], 64.0, 0.0, self.rows * self.cols)
        self.h_out.copy_(self.out[s], non_blocking=True)

    def e2e_bytes(self):
        return self.rows * self.cols * 2, self.rows * self.cols

    def cpu_sample(self, O):
        rows = 1024
        x = np.ascontiguousarray(self.host["x"][:rows])
        t0 = time.perf_counter()
        O.ascend_quant(x, O.F16, policy=O.PER_TENSOR, scaleScalar=64.0, offsetScalar=0.0)
        dt = time.perf_counter() - t0
        return rows * self.cols * 3 / dt / 1e9, f"{rows} of {self.rows} rows"

    def check(self, O):
        rows = 64
        want = O.ascend_quant(np.ascontiguousarray(self.host["x"][:rows]), O.F16, policy=O.PER_TENSOR, scaleScalar=64.0,
                              offsetScalar=0.0)
        return bool(np.array_equal(self.out[0][:rows].cpu().numpy(), want))


class W8A8Cfg4(Workload):
    """Config 4.  With `world` > 1 the weight matrix B (and sB, bias) is column-sharded over the ranks: each rank
    computes C[:, shard] and an NCCL all-gather reassembles the output on every rank (strong scaling)."""
    name = "W8A8 int8 matmul M=N=K=4096 + per-token x per-channel dequant + bias -> bf16 (config 4)"
    sharding_note = "B column-sharded over N"
    dtype = "int8"
    unit = "TOPS"
    bound = "tensor"
    key = "w8a8_cfg4"

    def __init__(self, torch, ops, dev, dist=None, world=1, rank=0):
        self.torch, self.ops, self.dist, self.world, self.rank = torch, ops, dist, world, rank
        self.M = self.N = self.K = 4096
        h = gen_w8a8_cfg4(self.M, self.N, self.K)
        self.host = h
        self.nl = self.N // world
        n0 = rank * self.nl
        per_set = self.M * self.K + self.nl * self.K + self.M * self.nl * 2
        self.nsets = self.nsets_for(per_set)
        bf = lambda a: torch.from_numpy(a.view(np.int16).copy()).to(dev).view(torch.bfloat16)  # noqa: E731
        self.A = [torch.from_numpy(h["A"]).to(dev) for _ in range(self.nsets)]
        self.B = [torch.from_numpy(np.ascontiguousarray(h["B"][n0:n0 + self.nl])).to(dev) for _ in range(self.nsets)]
        self.C = [torch.empty((self.M, self.nl), dtype=torch.bfloat16, device=dev) for _ in range(self.nsets)]
        self.sA = torch.from_numpy(h["sA"]).to(dev)
        self.sB = torch.from_numpy(h["sB"][n0:n0 + self.nl].copy()).to(dev)
        self.bias = bf(h["bias"][n0:n0 + self.nl])
        self.gathered = torch.empty((world * self.M, self.nl), dtype=torch.bfloat16, device=dev) if world > 1 else None
        self.h_A = torch.from_numpy(h["A"]).pin_memory()
        self.h_sA = torch.from_numpy(h["sA"]).pin_memory()
        self.h_C = torch.empty((self.M, self.N), dtype=torch.bfloat16).pin_memory()
        self.launches_per_step = 1
        # Fused reassembly: every rank's epilogue stores its column block into every rank's [M, N] matrix over NVLink
        # (peer-mapped symmetric memory); a device-side barrier ends the step.  Falls back to an NCCL all-gather.
        self.fused = None
        self.mc = None
        if world > 1:
            try:
                import torch.distributed._symmetric_memory as symm
                self.full, self.hdl = [], []
                for _ in range(2):
                    t = symm.empty((self.M, self.N), dtype=torch.bfloat16, device=dev)
                    self.hdl.append(symm.rendezvous(t, dist.group.WORLD))
                    self.full.append(t)
                self.fused = True
                # ASCQ_BENCH_REASSEMBLY=multicast: one multimem store per piece through NVSwitch multicast instead of one
                # store per peer (measured slower at two ranks, where the local copy then crosses NVLink too)
                mc = [int(getattr(h, "multicast_ptr", 0) or 0) for h in self.hdl]
                self.mc = mc if all(mc) and os.environ.get("ASCQ_BENCH_REASSEMBLY", "peer") == "multicast" else None
            except Exception as e:  # noqa: BLE001
                self.fused = False
                self.fused_error = repr(e)[:200]

    def work_per_step(self):
        return 2 * self.M * self.N * self.K  # whole job (all ranks together)

    def step(self, i):
        s = i % self.nsets
        if self.world == 1:
            self.ops.MatmulW8A8(self.C[s], self.A[s], self.B[s], self.sA, self.sB, self.bias)
        elif self.fused:
            f = i % 2
            if self.mc:
                self.ops.MatmulW8A8Multicast(self.mc[f], self.rank * self.nl, self.N, self.A[s], self.B[s], self.sA, self.sB,
                                             self.bias)
            else:
                self.ops.MatmulW8A8Scatter(self.hdl[f].buffer_ptrs, self.rank + 1, self.rank * self.nl, self.N, self.A[s],
                                           self.B[s], self.sA, self.sB, self.bias)
            self.hdl[f].barrier(channel=0)
        else:
            self.nccl_step(i)

    def nccl_step(self, i):
        s = i % self.nsets
        self.ops.MatmulW8A8(self.C[s], self.A[s], self.B[s], self.sA, self.sB, self.bias)
        self.dist.all_gather_into_tensor(self.gathered, self.C[s])

    def gemm_only_step(self, i):
        s = i % self.nsets
        self.ops.MatmulW8A8(self.C[s], self.A[s], self.B[s], self.sA, self.sB, self.bias)

    def e2e_step(self, i):
        s = i % self.nsets
        self.A[s].copy_(self.h_A, non_blocking=True)     # this step's activations and their scales
        self.sA.copy_(self.h_sA, non_blocking=True)
        self.step(i)
        if self.world == 1:
            self.h_C.copy_(self.C[s], non_blocking=True)
        elif self.fused:
            self.h_C.copy_(self.full[i % 2], non_blocking=True)
        else:
            self.h_C.view(self.world * self.M, self.nl).copy_(self.gathered, non_blocking=True)

    def e2e_bytes(self):
        return self.M * self.K + self.M * 4, self.M * self.N * 2

    def cpu_sample(self, O):
        rows = 64
        A = np.ascontiguousarray(self.host["A"][:rows])
        t0 = time.perf_counter()
        O.matmul_w8a8(A, self.host["B"], self.host["sA"][:rows].copy(), self.host["sB"], self.host["bias"])
        dt = time.perf_counter() - t0
        return 2 * rows * self.N * self.K / dt / 1e12, f"{rows} of {self.M} rows of A"

    def check(self, O):
        rows = 16
        n0 = self.rank * self.nl
        want = O.matmul_w8a8(np.ascontiguousarray(self.host["A"][:rows]), np.ascontiguousarray(self.host["B"][n0:n0 + self.nl]),
                             self.host["sA"][:rows].copy(), self.host["sB"][n0:n0 + self.nl].copy(),
                             self.host["bias"][n0:n0 + self.nl].copy())
        self.gemm_only_step(0)
        got = self.C[0][:rows].view(self.torch.int16).cpu().numpy().view(np.uint16)
        self.ops.MatmulStatus()
        ok = bool(np.array_equal(got, want))
        if self.world > 1 and self.fused:
            # the reassembled matrix on this rank: every rank's column block must have arrived with the oracle's bits
            self.step(0)
            self.torch.cuda.synchronize()
            self.hdl[0].barrier(channel=0)
            self.torch.cuda.synchronize()
            whole = O.matmul_w8a8(np.ascontiguousarray(self.host["A"][:rows]), self.host["B"], self.host["sA"][:rows].copy(),
                                  self.host["sB"], self.host["bias"])
            full = self.full[0][:rows].view(self.torch.int16).cpu().numpy().view(np.uint16)
            ok = ok and bool(np.array_equal(full, whole))
        return ok


class Mxfp4Cfg5(Workload):
    name = "MX-FP4 grouped matmul G=16, 16384 tokens (multinomial), K=7168, N=2048 -> bf16 (config 5)"
    sharding_note = "groups dealt out over the ranks, longest first"
    dtype = "fp4(e2m1)xue8m0, f32 accumulate"
    unit = "TFLOPS"
    bound = "tensor"
    key = "mxfp4_cfg5"

    def __init__(self, torch, ops, dev, dist=None, world=1, rank=0):
        """With `world` > 1 the groups are dealt out over the ranks (longest first); each rank holds the tokens and the
        weights of its groups only and computes their output rows; the full [tokens, N] output is reassembled on every
        rank inside the step (strong scaling)."""
        from asc_devkit_b200 import sharding
        self.torch, self.ops, self.dist, self.world, self.rank = torch, ops, dist, world, rank
        self.G, self.total, self.K, self.N = 16, 16384, 7168, 2048
        h = gen_mxfp4_cfg5(self.G, self.total, self.K, self.N)
        self.all_groups = [int(v) for v in h["groups"]]
        starts = np.concatenate([[0], np.cumsum(self.all_groups)]).astype(np.int64)
        self.plan = sharding.assign_groups_lpt(self.all_groups, world)
        mine = self.plan.groups_of[rank]
        rows = np.concatenate([np.arange(starts[g], starts[g + 1]) for g in mine]) if mine else np.zeros(0, np.int64)
        if world > 1:   # this rank's share, its groups back to back
            h = dict(h, A=np.ascontiguousarray(h["A"][rows]), sA=np.ascontiguousarray(h["sA"][rows]),
                     B=np.ascontiguousarray(h["B"][mine]), sB=np.ascontiguousarray(h["sB"][mine]))
        self.host = h
        self.groups = [self.all_groups[g] for g in mine]
        self.out_row_start = [int(starts[g]) for g in mine]
        self.local_rows = int(sum(self.groups))
        per_set = h["A"].nbytes + h["sA"].nbytes + h["B"].nbytes + h["sB"].nbytes + self.local_rows * self.N * 2
        self.nsets = self.nsets_for(per_set)
        t = lambda a: torch.from_numpy(a).to(dev)  # noqa: E731
        self.A = [t(h["A"]) for _ in range(self.nsets)]
        self.sA = [t(h["sA"]) for _ in range(self.nsets)]
        self.B = [t(h["B"]) for _ in range(self.nsets)]
        self.sB = [t(h["sB"]) for _ in range(self.nsets)]
        self.C = [torch.empty((max(self.local_rows, 1), self.N), dtype=torch.bfloat16, device=dev) for _ in range(self.nsets)]
        self.ws = torch.empty(max(256, ops.GroupMatmulMxfp4Workspace(self.local_rows, max(len(mine), 1), self.K, self.N)),
                              dtype=torch.uint8, device=dev)
        self.fused = None
        if world > 1:
            self.padded = torch.zeros((self.plan.max_rows, self.N), dtype=torch.bfloat16, device=dev)
            self.gathered = torch.empty((world * self.plan.max_rows, self.N), dtype=torch.bfloat16, device=dev)
            try:
                import torch.distributed._symmetric_memory as symm
                self.full, self.hdl = [], []
                for _ in range(2):
                    tt = symm.empty((self.total, self.N), dtype=torch.bfloat16, device=dev)
                    self.hdl.append(symm.rendezvous(tt, dist.group.WORLD))
                    self.full.append(tt)
                self.fused = True
            except Exception as e:  # noqa: BLE001
                self.fused = False
                self.fused_error = repr(e)[:200]
        self.h_A = torch.from_numpy(h["A"]).pin_memory()
        self.h_sA = torch.from_numpy(h["sA"]).pin_memory()
        self.h_C = torch.empty((self.total, self.N), dtype=torch.bfloat16).pin_memory()
        self.launches_per_step = 2  # one scale-repack launch + the matmul

    def work_per_step(self):
        return 2 * self.total * self.N * self.K   # whole job (all ranks together)

    def step(self, i):
        s = i % self.nsets
        if self.world == 1:
            self.ops.GroupMatmulMxfp4(self.C[s], self.A[s], self.sA[s], self.B[s], self.sB[s], self.groups, self.K, self.N,
                                      workspace=self.ws)
        elif self.fused:
            f = i % 2
            if self.groups:
                self.ops.GroupMatmulMxfp4Scatter(self.hdl[f].buffer_ptrs, self.rank + 1, self.out_row_start, self.A[s], self.sA[s],
                                                 self.B[s], self.sB[s], self.groups, self.K, self.N, workspace=self.ws)
            self.hdl[f].barrier(channel=0)
        else:
            self.nccl_step(i)

    def gemm_only_step(self, i):
        s = i % self.nsets
        if self.groups:
            self.ops.GroupMatmulMxfp4(self.C[s], self.A[s], self.sA[s], self.B[s], self.sB[s], self.groups, self.K, self.N,
                                      workspace=self.ws)

    def prepacked_step(self, i):
        """Static weights: their scales were brought into the kernel's order once, outside the step."""
        s = i % self.nsets
        if not hasattr(self, "sB_packed"):
            self.sB_packed = [self.ops.GroupMatmulMxfp4PackScaleB(self.sB[j], self.K, self.N) for j in range(self.nsets)]
        self.ops.GroupMatmulMxfp4Prepacked(self.C[s], self.A[s], self.sA[s], self.B[s], self.sB_packed[s], self.groups, self.K,
                                           self.N, workspace=self.ws)

    def nccl_step(self, i):
        """The unfused variant: local matmul, rows padded to the largest share, NCCL all-gather (the ragged blocks
        still have to be put in order by the consumer)."""
        s = i % self.nsets
        self.gemm_only_step(i)
        self.padded[:self.local_rows].copy_(self.C[s][:self.local_rows])
        self.dist.all_gather_into_tensor(self.gathered, self.padded)

    def e2e_step(self, i):
        s = i % self.nsets
        self.A[s].copy_(self.h_A, non_blocking=True)      # this step's tokens and their scales; expert weights stay resident
        self.sA[s].copy_(self.h_sA, non_blocking=True)
        self.step(i)
        if self.world == 1:
            self.h_C.copy_(self.C[s], non_blocking=True)
        elif self.fused:
            self.h_C.copy_(self.full[i % 2], non_blocking=True)
        else:
            if not hasattr(self, "h_gathered"):
                self.h_gathered = self.torch.empty(self.gathered.shape, dtype=self.torch.bfloat16).pin_memory()
            self.h_gathered.copy_(self.gathered, non_blocking=True)

    def e2e_bytes(self):
        return self.host["A"].nbytes + self.host["sA"].nbytes, self.total * self.N * 2

    def cpu_sample(self, O):
        rows = 16
        h = self.host
        t0 = time.perf_counter()
        O.group_matmul_mxfp4(np.ascontiguousarray(h["A"][:rows]), np.ascontiguousarray(h["sA"][:rows]),
                             np.ascontiguousarray(h["B"][:1]), np.ascontiguousarray(h["sB"][:1]), np.array([rows], np.int64),
                             self.K, self.N)
        dt = time.perf_counter() - t0
        return 2 * rows * self.N * self.K / dt / 1e12, f"{rows} of {self.total} rows (group 0)"

    def check(self, O):
        rows = 8
        h = self.host
        _, want = O.group_matmul_mxfp4(np.ascontiguousarray(h["A"][:rows]), np.ascontiguousarray(h["sA"][:rows]),
                                       np.ascontiguousarray(h["B"][:1]), np.ascontiguousarray(h["sB"][:1]),
                                       np.array([rows], np.int64), self.K, self.N, want_f32=True)
        self.gemm_only_step(0)
        got = self.C[0][:rows].float().cpu().numpy()
        self.ops.MatmulStatus()
        ok = bool(np.all(np.abs(got - want) <= 1e-2 * np.abs(want) + 1e-3 * np.abs(want).max()))
        if self.world > 1 and self.fused:   # the reassembled matrix holds the same bits at this group's rows, on every rank
            self.step(0)
            self.torch.cuda.synchronize()
            r0 = self.out_row_start[0]
            ok = ok and bool(self.torch.equal(self.full[0][r0:r0 + rows], self.C[0][:rows]))
        return ok


WORKLOADS = {"w8a8_cfg4": W8A8Cfg4, "mxfp4_cfg5": Mxfp4Cfg5, "antiquant_cfg2": AntiQuantCfg2, "dequant_cfg3": DequantCfg3,
             "quant_scaled": QuantScaled}
HEADLINE = "w8a8_cfg4"
# DRAM bytes read + written by the dominant kernel of one step at full size on one GPU, from the ncu captures
# summarised in profiles/<workload>_ncu_counters.md (outputs that stay in the 126 MB L2 do not show up as DRAM writes).
TRAFFIC_BYTES = {"w8a8_cfg4": 35.2e6, "mxfp4_cfg5": 234.4e6, "antiquant_cfg2": 78.6e6, "dequant_cfg3": 33.6e6,
                 "quant_scaled": 365.3e6}


# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi in the background for the length of the timed region (read-only queries)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap,utilization.gpu")

    def __init__(self, gpu_index):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(gpu_index)], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        # nvidia-smi needs a moment to start: wait for its first line so the timed region is covered
        t0 = time.time()
        while self.proc is not None and time.time() - t0 < 3.0 and os.path.getsize(self.tmp.name) == 0:
            time.sleep(0.02)

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.tmp.flush()
        self.tmp.seek(0)
        sm, mx, reasons, busy = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.tmp.read().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            try:
                busy.append(float(f[9]) >= 50.0)
            except (ValueError, IndexError):
                busy.append(False)
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        self.tmp.close()
        os.unlink(self.tmp.name)
        if sm:
            loaded = [v for v, b in zip(sm, busy) if b] or sm   # median over the samples taken under load
            out.update(sm_mhz=float(np.median(loaded)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons),
                       samples=len(sm), samples_under_load=int(sum(busy)))
        return out


def time_steps(torch, fn, steps, warmup, dist=None):
    """W untimed + K timed calls of fn(i); CUDA events on the current stream; returns seconds (max over ranks)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / 1e3
    if dist is not None:
        t = torch.tensor([sec], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    return sec


def time_graph(torch, fn, steps, warmup):
    """The same W + K calls, with the K timed ones captured once into a CUDA graph and replayed: the host's launch
    cost (Python, ctypes) is then outside the timed region.  Returns seconds for K steps, or None if capture fails."""
    try:
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(steps):
                fn(warmup + i)
        g.replay()                      # untimed: uploads the graph
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 1e3
    except Exception as e:  # noqa: BLE001
        print(f"bench: CUDA graph capture unavailable ({e!r}); timing eager launches", file=sys.stderr)
        torch.cuda.synchronize()
        return None


def run_ours(args):
    import torch
    from asc_devkit_b200 import _lib, ops
    _lib.lib()  # fail loudly if the CUDA library is missing

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        torch.cuda.set_device(local)
        dist_mod.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
        dist = dist_mod
    else:
        torch.cuda.set_device(0)
    dev = torch.device(f"cuda:{local}")
    peaks = measured_peaks()
    names = [args.workload] if args.workload != "all" else list(WORKLOADS)
    if HEADLINE not in names:
        names = [HEADLINE] + names if args.workload == "all" else names
    results = {}
    head = None
    sampler = ClockSampler(local) if rank == 0 else None   # runs across every timed region of this process
    for nm in names:
        sharded = nm in ("w8a8_cfg4", "mxfp4_cfg5")
        wl = WORKLOADS[nm](torch, ops, dev, dist, world, rank) if sharded else WORKLOADS[nm](torch, ops, dev)
        is_head = nm == (args.workload if args.workload != "all" else HEADLINE)
        sec = time_steps(torch, wl.step, args.steps, args.warmup, dist)
        eager_per = sec / args.steps
        launch = "one host call per step"
        if world == 1:
            gsec_graph = time_graph(torch, wl.step, args.steps, args.warmup)
            if gsec_graph is not None and gsec_graph < sec:
                sec, launch = gsec_graph, "the K steps replayed from one CUDA graph"
        per = sec / args.steps
        work = wl.work_per_step()
        if sharded:
            achieved = work / per / 1e12          # T(FL)OPS of the whole job (strong scaling: work is split over ranks)
            total_value = achieved
            gsec = time_steps(torch, wl.gemm_only_step, args.steps, args.warmup, dist)
            if world == 1:
                gsec = min(gsec, sec)
            # the slowest rank's matmul alone, as a rate per GPU (group shares are not exactly equal)
            kern = work / world / (gsec / args.steps) / 1e12
            int8 = nm == "w8a8_cfg4"
            peak = (2.0 if int8 else 4.0) * peaks["bf16_tflops"]
            extra = {}
            if world > 1:
                extra["reassembly"] = (("fused epilogue multimem stores through NVSwitch multicast + symmetric-memory barrier"
                                        if getattr(wl, "mc", None) else "fused epilogue peer stores + symmetric-memory barrier") if wl.fused
                                       else "NCCL all-gather (symmetric memory unavailable: %s)" % getattr(wl, "fused_error", ""))
                nsec = time_steps(torch, wl.nccl_step, args.steps, args.warmup, dist)
                extra["nccl_allgather_variant"] = work / (nsec / args.steps) / 1e12
            roof = {"bound": "tensor", "achieved": kern, "peak": peak, "unit": wl.unit, "frac": kern / peak, "traffic": None,
                    "peak_source": ("2 x %s dense bf16 cuBLAS burst (int8 runs at twice the bf16 rate; nominal 4500)" if int8 else
                                    "4 x %s dense bf16 cuBLAS burst (FP4 runs at four times the bf16 rate; nominal 9000)")
                                   % peaks["source"], "kernel_ms": gsec / args.steps * 1e3}
        elif wl.bound == "tensor":
            raise AssertionError("every tensor-bound workload shards")
        else:
            achieved = work / per / 1e9           # GB/s (each rank does the full workload: replicas)
            total_value = achieved * world
            roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"]}
        if world == 1:
            roof["traffic"] = TRAFFIC_BYTES.get(nm)
        e2e_sec = time_steps(torch, wl.e2e_step, max(2, args.steps // 4), 2, dist)
        e2e_per = e2e_sec / max(2, args.steps // 4)
        h2d, d2h = wl.e2e_bytes()
        e2e_value = (work / e2e_per / 1e12 if sharded else
                     work / e2e_per / 1e12 * world if wl.bound == "tensor" else work / e2e_per / 1e9 * world)
        rec = {"name": wl.name, "value": total_value, "unit": wl.unit, "ms_per_step": per * 1e3,
               "roofline": roof,
               "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
               "scaling": "strong" if sharded else "weak",
               "nsets": wl.nsets, "launches_per_step": wl.launches_per_step, "launch": launch,
               "ms_per_step_host_launched": eager_per * 1e3}
        if sharded and world > 1:
            rec.update(extra)
        if world == 1 and hasattr(wl, "prepacked_step"):
            psec = time_steps(torch, wl.prepacked_step, args.steps, args.warmup, None)
            gp = time_graph(torch, wl.prepacked_step, args.steps, args.warmup)
            psec = min(psec, gp) if gp is not None else psec
            rec["with_prepacked_weight_scales"] = {"value": work / (psec / args.steps) / 1e12, "unit": wl.unit,
                                                   "ms_per_step": psec / args.steps * 1e3}
        if rank == 0 or (sharded and world > 1):
            from oracle import oracle as O
            ok = wl.check(O)      # every rank takes part when the check runs a sharded step
            if rank == 0:
                rec["parity_vs_oracle"] = ok
        if rank == 0:
            if world == 1:
                v, sample = wl.cpu_sample(O)
                rec["cpu_baseline"] = {"value": v, "unit": wl.unit, "cores": O.num_threads(), "kind": "port",
                                       "sample": sample}
        results[nm] = rec
        if is_head:
            head = (wl, rec)
        del wl
        torch.cuda.empty_cache()
    clocks = sampler.stop() if sampler else None
    if rank == 0:
        wl, rec = head
        line = {"metric": "W8A8/MXFP4 GEMM TOPS at 1/2/4/8 B200; quant/dequant GB/s vs HBM peak",
                "value": rec["value"], "unit": rec["unit"], "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": rec["scaling"], "vs_baseline": None,
                "dtype": wl.dtype, "data": "synthetic",
                "config": {"workload": rec["name"], "timing": "buffers rotate over a set larger than L2 (126 MB)",
                           "launch": rec["launch"],
                           "sharding": ((wl.sharding_note + "; C reassembled inside the step: ") + rec.get("reassembly", "single GPU")
                                        if rec["scaling"] == "strong"
                                        else "replicas only (elementwise operators do not shard)")},
                "roofline": rec["roofline"], "e2e": rec["e2e"], "gpu_launches": args.steps * rec["launches_per_step"],
                "clocks": clocks, "workloads": results}
        if "cpu_baseline" in rec:
            line["cpu_baseline"] = rec["cpu_baseline"]
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def run_extras(args):
    """`--workload extras`: the operators of the path that are not among the five benchmark configurations, each timed
    the same way (K steps replayed from one CUDA graph, CUDA events, inputs rotated over more than the L2 size where
    one set is smaller) and reported in one JSON line.  Single GPU."""
    import ctypes as C
    import numpy as np
    import torch
    from asc_devkit_b200 import _lib as L, ops
    L.lib()
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    steps, warm = min(args.steps, 40), max(args.warmup, 3)
    out = {}

    def add(name, fn, work, unit):
        sec = time_graph(torch, fn, steps, warm)
        if sec is None:
            sec = time_steps(torch, fn, steps, warm)
        us = sec / steps * 1e6
        out[name] = {"us": round(us, 1), "rate": round(work / us / 1e6, 2), "unit": unit}  # work per us -> T(unit)/s
        print(f"extras: {name}: {us:.1f} us, {work / us / 1e6:.2f} {unit}", file=sys.stderr)

    # ---- matmuls at 4096^3 (six operand sets: 200 MB of operands) ----
    M = N = K = 4096
    ns = 6
    flop = 2.0 * M * N * K
    A8 = [torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev) for _ in range(ns)]
    B8 = [torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev) for _ in range(ns)]
    bias = torch.randint(-100, 100, (N,), dtype=torch.int32, device=dev)
    qv = torch.from_numpy((np.random.default_rng(0).uniform(1e-4, 1e-3, N).astype(np.float32).view(np.uint32).astype(np.uint64)
                           | np.uint64(1 << 46)).view(np.int64)).to(dev)
    Ch = [torch.empty((M, N), dtype=torch.float16, device=dev) for _ in range(ns)]
    Cb = [torch.empty((M, N), dtype=torch.int8, device=dev) for _ in range(ns)]
    add("int8 matmul + fixpipe quantisation -> fp16 (VDEQF16)", lambda i: ops.MatmulI8Quant(Ch[i % ns], A8[i % ns], B8[i % ns], bias, qv, 1.0), flop, "TOPS")
    add("int8 matmul + requantisation -> int8 (VREQ8)", lambda i: ops.MatmulI8Requant(Cb[i % ns], A8[i % ns], B8[i % ns], bias, qv), flop, "TOPS")
    del A8, Ch
    for dt, nm in ((torch.bfloat16, "bfloat16"), (torch.float16, "half")):
        A = [torch.randn((M, K), device=dev).to(dt) for _ in range(ns)]
        B = [torch.randn((N, K), device=dev).to(dt) for _ in range(ns)]
        Cc = [torch.empty((M, N), dtype=dt, device=dev) for _ in range(ns)]
        add(f"{nm} matmul", lambda i: ops.MatmulF16(Cc[i % ns], A[i % ns], B[i % ns]), flop, "TFLOPS")
        add(f"{nm} matmul, cuBLAS through torch (for comparison)", lambda i: torch.matmul(A[i % ns], B[i % ns].t(), out=Cc[i % ns]), flop, "TFLOPS")
        add(f"{nm} matmul + fixpipe quantisation -> int8 (QF322B8_PRE)",
            lambda i: ops.MatmulF16Quant(Cb[i % ns], A[i % ns], B[i % ns], None, int(np.float32(0.05).view(np.uint32)) | (1 << 46)), flop, "TFLOPS")
        sc = (torch.rand(N, device=dev) * 0.02).to(dt)
        of = torch.randn(N, device=dev).to(dt)
        ws = torch.empty(N * K * 2, dtype=torch.uint8, device=dev)
        B4 = [b[:, : K // 2].contiguous().view(torch.uint8) for b in B8]
        add(f"weight-only-quantised matmul, int8 weights, {nm} activations", lambda i: ops.MatmulW8A16(Cc[i % ns], A[i % ns], B8[i % ns], of, sc, workspace=ws), flop, "TFLOPS")
        add(f"weight-only-quantised matmul, int4 weights, {nm} activations", lambda i: ops.MatmulW4A16(Cc[i % ns], A[i % ns], B4[i % ns], of, sc, workspace=ws), flop, "TFLOPS")
        del A, B, Cc
    del B8, Cb
    # ---- MX matmul with fp8 operands at config 5's shape (uniform groups) ----
    G, K5, N5, sumM = 16, 7168, 2048, 16384
    groups = [sumM // G] * G
    A5 = torch.randint(0, 120, (sumM, K5), dtype=torch.uint8, device=dev)
    B5 = torch.randint(0, 120, (G, N5, K5), dtype=torch.uint8, device=dev)
    sA5 = torch.randint(123, 131, (sumM, K5 // 32), dtype=torch.uint8, device=dev)
    sB5 = torch.randint(123, 131, (G, N5, K5 // 32), dtype=torch.uint8, device=dev)
    C5 = torch.empty((sumM, N5), dtype=torch.bfloat16, device=dev)
    ws5 = torch.empty(int(L.lib().ascq_group_matmul_mxfp8_workspace_size(sumM, G, K5, N5)) + 256, dtype=torch.uint8, device=dev)
    add("MX matmul, fp8 e4m3 operands, config 5's shape", lambda i: ops.GroupMatmulMxfp8(C5, A5, L.DT_FP8_E4M3, sA5, B5, L.DT_FP8_E4M3, sB5, groups, K5, N5, workspace=ws5),
        2.0 * sumM * K5 * N5, "TFLOPS")
    del A5, B5, C5
    # ---- producers and decoders of the MX operands, [16384, 7168] activations / [4096, 11008] weights ----
    m, n = 16384, 7168
    x = torch.randn((m, n), device=dev).bfloat16()
    d4 = torch.empty((m, n // 2), dtype=torch.uint8, device=dev)
    s4 = torch.empty((m, n // 32), dtype=torch.uint8, device=dev)
    add("dynamic MX-FP4 quantiser, bf16 [16384, 7168]", lambda i: ops.DynamicQuantMxfp4(d4, s4, x), x.numel() * 2 + d4.numel() + s4.numel(), "TB/s")
    scb = (torch.rand((m, n // 32), device=dev) + 0.5).bfloat16()
    qp = L.QuantParam(m, n, m * n, 32, 0, 1, 1)
    add("AscendQuant PER_GROUP -> fp4x2, bf16 [16384, 7168]",
        lambda i: L.check(L.lib().ascq_quant(ops._ptr(d4), L.DT_FP4X2_E2M1, ops._ptr(x), L.DT_BF16, ops._ptr(scb), None, L.DT_BF16, 0.0, 0.0,
                                             L.PER_GROUP, C.byref(qp), ops._stream(None))), x.numel() * 2 + scb.numel() * 2 + d4.numel(), "TB/s")
    d8 = torch.empty((m, n), dtype=torch.int8, device=dev)
    so = torch.empty(m, dtype=torch.float32, device=dev)
    add("dynamic per-token quantiser, bf16 [16384, 7168] -> int8", lambda i: ops.DynamicQuantPerToken(d8, so, x), x.numel() * 3, "TB/s")
    rows, cols = 4096, 11008
    src4 = torch.randint(0, 256, (rows, cols // 2), dtype=torch.uint8, device=dev)
    sc4 = torch.randint(120, 135, (rows * (cols // 32),), dtype=torch.uint8, device=dev)
    dst4 = torch.empty((rows, cols), dtype=torch.bfloat16, device=dev)
    add("MX decode fp4x2 [4096, 11008] -> bf16 (groups along the columns)",
        lambda i: ops.AscendAntiQuant(dst4, src4, None, sc4, ops.AscendAntiQuantParam(rows, cols), isTranspose=True, policy=L.PER_GROUP,
                                      hasOffset=False, src_dtype=L.DT_FP4X2_E2M1, scale_dtype=L.DT_E8M0), src4.numel() + sc4.numel() + dst4.numel() * 2, "TB/s")
    # ---- the three elementwise operators under the other policies, [16384, 7168], group size 128 ----
    gs = 128
    for pol, nm, shape, kd in ((L.PER_TOKEN, "PER_TOKEN", (m,), 1), (L.PER_GROUP, "PER_GROUP kDim=1", (m, n // gs), 1), (L.PER_GROUP, "PER_GROUP kDim=0", (m // gs, n), 0)):
        sc = (torch.rand(shape, device=dev) + 0.5).bfloat16()
        of = torch.randn(shape, device=dev).bfloat16()
        p1 = L.QuantParam(m, n, m * n, gs if pol == L.PER_GROUP else 0, 1, kd, 1)
        add(f"AscendQuant bf16 -> int8 {nm}", lambda i: L.check(L.lib().ascq_quant(ops._ptr(d8), L.DT_I8, ops._ptr(x), L.DT_BF16, ops._ptr(sc), ops._ptr(of),
            L.DT_BF16, 0.0, 0.0, pol, C.byref(p1), ops._stream(None))), x.numel() * 3, "TB/s")
        p2 = L.AntiQuantParam(m, n, m * n, gs if pol == L.PER_GROUP else 0, 1, 0, kd)
        yb = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        add(f"AscendAntiQuant int8 -> bf16 {nm}", lambda i: L.check(L.lib().ascq_antiquant(ops._ptr(yb), L.DT_BF16, ops._ptr(d8), L.DT_I8, ops._ptr(of), ops._ptr(sc),
            L.DT_BF16, 0.0, 0.0, pol, C.byref(p2), ops._stream(None))), x.numel() * 3, "TB/s")
    ops.MatmulStatus()
    print(json.dumps({"metric": "operators of the path beside the five benchmark configurations", "n_gpus": 1, "steps": steps, "warmup": warm,
                      "data": "synthetic", "launch": "the K steps replayed from one CUDA graph", "extras": out}))


def run_reference(args):
    """The reference arm: the CPU restatement of the reference operators on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if "TORCHELASTIC_RUN_ID" in os.environ and os.environ.get("OMP_NUM_THREADS") == "1":
        del os.environ["OMP_NUM_THREADS"]   # torchrun's default of one thread per rank; this arm runs alone on all host cores
    from oracle import oracle as O
    nm = args.workload if args.workload != "all" else HEADLINE
    unit = "GB/s"
    if nm == "w8a8_cfg4":
        h = gen_w8a8_cfg4()
        rows = 128
        A = np.ascontiguousarray(h["A"][:rows])
        sA = h["sA"][:rows].copy()

        def step():
            O.matmul_w8a8(A, h["B"], sA, h["sB"], h["bias"])
        work, sample, name, unit = 2 * rows * 4096 * 4096 / 1e3, f"{rows} of 4096 rows of A per step", W8A8Cfg4.name, "TOPS"
    elif nm == "antiquant_cfg2":
        h = gen_antiquant_cfg2()
        rows, N = 1024, 11008
        w = np.ascontiguousarray(h["w"][:rows])

        def step():
            O.ascend_antiquant(w, O.I8, O.BF16, policy=O.PER_CHANNEL, m=rows, n=N, scale=h["scale"], offset=h["offset"],
                               scaleT=O.BF16)
        work, sample, name = rows * N * 3, f"{rows} of 4096 rows per step", AntiQuantCfg2.name
    elif nm == "dequant_cfg3":
        h = gen_dequant_cfg3()
        rows, N = 1024, 4096
        acc = np.ascontiguousarray(h["acc"][:rows])
        tok = h["stok"][:rows].copy()

        def step():
            O.ascend_dequant(acc, O.I32, O.BF16, policy=O.PER_CHANNEL, m=rows, n=N, calCount=N, scale=h["sch"], tokScale=tok,
                             scaleT=O.F32)
        work, sample, name = rows * N * 6, f"{rows} of 2048 rows per step", DequantCfg3.name
    else:
        h = gen_quant_cfg1(1024, 8192)

        def step():
            O.ascend_quant(h["x"], O.F16, policy=O.PER_TENSOR, scaleScalar=64.0, offsetScalar=0.0)
        work, sample, name = 1024 * 8192 * 3, "1024 of 16384 rows per step", QuantScaled.name
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    per = (time.perf_counter() - t0) / args.steps
    v = work / per / 1e9
    print(json.dumps({"impl": "reference", "metric": "W8A8/MXFP4 GEMM TOPS at 1/2/4/8 B200; quant/dequant GB/s vs HBM peak",
                      "value": v, "unit": unit, "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": per * 1e3, "higher_is_better": True, "scaling": "strong" if unit == "TOPS" else "weak",
                      "vs_baseline": None, "dtype": "int8" if unit == "TOPS" else "f32", "data": "synthetic",
                      "config": {"workload": name},
                      "cpu_baseline": {"value": v, "unit": unit, "cores": O.num_threads(), "kind": "port", "sample": sample},
                      "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                      "note": "CPU restatement of the reference operators (oracle/); the reference's own CPU-debug "
                              "build needs the closed tikicpulib"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="all", choices=["all", "extras"] + list(WORKLOADS))
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    # Libraries (NCCL's version banner, for one) write to file descriptor 1; the JSON line must be the only thing on
    # stdout, so everything else is sent to stderr while the run lasts.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(real_stdout, "w")
    if args.impl == "reference":
        if args.workload == "extras":
            args.workload = "all"
        run_reference(args)
    elif args.workload == "extras":
        run_extras(args)
    else:
        run_ours(args)
    sys.stdout.flush()


if __name__ == "__main__":
    main()
