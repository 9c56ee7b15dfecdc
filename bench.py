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

    def e2e_in(self, i):
        self.w[i % self.nsets].copy_(self.h_in, non_blocking=True)

    def e2e_out(self, i):
        self.h_out.copy_(self.out[i % self.nsets], non_blocking=True)

    def e2e_bytes(self):
        return self.K * self.N, self.K * self.N * 2

    def probe_step(self, i):
        """The same bytes in and out through torch's own type-conversion kernel (int8 -> bfloat16, no arithmetic): an
        independent reading of what a 1-byte-in, 2-bytes-out stream of this size reaches on this GPU."""
        s = i % self.nsets
        self.out[s].copy_(self.w[s])

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

    def e2e_in(self, i):
        self.acc[i % self.nsets].copy_(self.h_in, non_blocking=True)

    def e2e_out(self, i):
        self.h_out.copy_(self.out[i % self.nsets], non_blocking=True)

    def e2e_bytes(self):
        return self.M * self.N * 4, self.M * self.N * 2

    def probe_step(self, i):
        """The same bytes through torch's type-conversion kernel (int32 -> bfloat16): see AntiQuantCfg2.probe_step."""
        s = i % self.nsets
        self.out[s].copy_(self.acc[s])

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

    def e2e_in(self, i):
        self.x[i % self.nsets].copy_(self.h_in, non_blocking=True)

    def e2e_out(self, i):
        self.h_out.copy_(self.out[i % self.nsets], non_blocking=True)

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


class ShardedBuffers:
    """Device memory every rank of the box can write: the [rows, cols] bf16 output matrices (two, used alternately) and
    this rank's flag block.  torch's symmetric-memory allocator is used for the allocation and the address exchange
    only; everything that happens per step goes through the library's communicator (ascq_comm)."""

    def __init__(self, torch, ops, dist, dev, rank, world, rows, cols):
        import torch.distributed._symmetric_memory as symm
        self.full, self.hdl = [], []
        for _ in range(2):
            t = symm.empty((rows, cols), dtype=torch.bfloat16, device=dev)
            self.hdl.append(symm.rendezvous(t, dist.group.WORLD))
            self.full.append(t)
        self.flags = symm.empty(ops.Comm.flag_bytes(), dtype=torch.uint8, device=dev)
        self.flags.zero_()
        fh = symm.rendezvous(self.flags, dist.group.WORLD)
        torch.cuda.synchronize()
        dist.barrier()                      # every block is zeroed and mapped before anyone signals
        torch.cuda.synchronize()
        self.comm = ops.Comm(rank, world, [int(p) for p in fh.buffer_ptrs])
        self.ptrs = [[int(p) for p in h.buffer_ptrs] for h in self.hdl]
        self.mc = [int(getattr(h, "multicast_ptr", 0) or 0) for h in self.hdl]


class W8A8Cfg4(Workload):
    """Config 4.  With `world` > 1 the weight matrix B (and sB, bias) is column-sharded over the ranks: each rank
    computes C[:, shard] and its epilogue writes the block into every rank's [M, N] matrix (strong scaling)."""
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
        self.sA_sets = [self.sA.clone() for _ in range(self.nsets)]   # one copy per operand set: the end-to-end pipeline refills them
        self.sB = torch.from_numpy(h["sB"][n0:n0 + self.nl].copy()).to(dev)
        self.bias = bf(h["bias"][n0:n0 + self.nl])
        self.gathered = torch.empty((world * self.M, self.nl), dtype=torch.bfloat16, device=dev) if world > 1 else None
        self.h_A = torch.from_numpy(h["A"]).pin_memory()
        self.h_sA = torch.from_numpy(h["sA"]).pin_memory()
        self.h_C = torch.empty((self.M, self.nl), dtype=torch.bfloat16).pin_memory()   # this rank's block of the result
        self.launches_per_step = 1
        self.variant = "peer"     # "peer": one TMA store per rank; "multicast": multimem stores through NVSwitch
        self.sh = ShardedBuffers(torch, ops, dist, dev, rank, world, self.M, self.N) if world > 1 else None
        if world > 1:   # the whole job on this GPU alone, for the matmul-phase efficiency T1 / (N * T_N)
            self.B_all = torch.from_numpy(h["B"]).to(dev)
            self.sB_all = torch.from_numpy(h["sB"]).to(dev)
            self.bias_all = bf(h["bias"])
            self.C_all = torch.empty((self.M, self.N), dtype=torch.bfloat16, device=dev)

    def variants(self):
        return ["peer"] + (["multicast"] if self.sh is not None and all(self.sh.mc) and self.nl % 64 == 0 else [])

    def work_per_step(self):
        return 2 * self.M * self.N * self.K  # whole job (all ranks together)

    def step(self, i):
        s = i % self.nsets
        if self.world == 1:
            self.ops.MatmulW8A8(self.C[s], self.A[s], self.B[s], self.sA_of(s), self.sB, self.bias)
        else:
            f = i % 2
            self.ops.MatmulW8A8Sharded(self.sh.comm, self.sh.ptrs[f], self.A[s], self.B[s], self.sA_of(s), self.sB, self.bias, N=self.N,
                                       multicast_ptr=self.sh.mc[f] if self.variant == "multicast" else 0)

    def nccl_step(self, i):
        s = i % self.nsets
        self.ops.MatmulW8A8(self.C[s], self.A[s], self.B[s], self.sA, self.sB, self.bias)
        self.dist.all_gather_into_tensor(self.gathered, self.C[s])

    def gemm_only_step(self, i):
        s = i % self.nsets
        self.ops.MatmulW8A8(self.C[s], self.A[s], self.B[s], self.sA, self.sB, self.bias)

    def single_gpu_step(self, i):
        self.ops.MatmulW8A8(self.C_all, self.A[i % self.nsets], self.B_all, self.sA, self.sB_all, self.bias_all)

    def sA_of(self, s):
        return self.sA_sets[s]

    def e2e_in(self, i):
        s = i % self.nsets
        self.A[s].copy_(self.h_A, non_blocking=True)     # this step's activations and their scales
        self.sA_of(s).copy_(self.h_sA, non_blocking=True)

    def e2e_out(self, i):
        if self.world == 1:
            self.h_C.copy_(self.C[i % self.nsets], non_blocking=True)
        else:   # every rank reads back its own column block of the assembled matrix
            n0 = self.rank * self.nl
            self.h_C.copy_(self.sh.full[i % 2][:, n0:n0 + self.nl], non_blocking=True)

    def e2e_bytes(self):
        return self.M * self.K + self.M * 4, self.M * self.nl * 2

    def cpu_sample(self, O):
        rows = 64
        A = np.ascontiguousarray(self.host["A"][:rows])
        t0 = time.perf_counter()
        O.matmul_w8a8(A, self.host["B"], self.host["sA"][:rows].copy(), self.host["sB"], self.host["bias"])
        dt = time.perf_counter() - t0
        return 2 * rows * self.N * self.K / dt / 1e12, f"{rows} of {self.M} rows of A"

    def check(self, O):
        """One full tile row (256 rows) of the result against the oracle; with several ranks also the assembled matrix
        on every rank, under every reassembly variant."""
        rows = 256
        n0 = self.rank * self.nl
        A = np.ascontiguousarray(self.host["A"][:rows])
        sA = self.host["sA"][:rows].copy()
        whole = O.matmul_w8a8(A, self.host["B"], sA, self.host["sB"], self.host["bias"])
        self.gemm_only_step(0)
        got = self.C[0][:rows].view(self.torch.int16).cpu().numpy().view(np.uint16)
        self.ops.MatmulStatus()
        ok = bool(np.array_equal(got, whole[:, n0:n0 + self.nl]))
        if self.world > 1:
            keep = self.variant
            for v in self.variants():
                self.variant = v
                self.sh.full[0].zero_()
                self.torch.cuda.synchronize()
                self.dist.barrier()
                self.step(0)
                self.ops.MatmulStatus()      # synchronises; raises if the wait for the other ranks ran out
                full = self.sh.full[0][:rows].view(self.torch.int16).cpu().numpy().view(np.uint16)
                ok = ok and bool(np.array_equal(full, whole))
                self.dist.barrier()
            self.variant = keep
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
        if world == 1:   # static weights: scales packed once, as at model-load time
            self.sB_packed = [ops.GroupMatmulMxfp4PackScaleB(self.sB[j], self.K, self.N) for j in range(self.nsets)]
        self.sh = None
        if world > 1:
            self.padded = torch.zeros((self.plan.max_rows, self.N), dtype=torch.bfloat16, device=dev)
            self.gathered = torch.empty((world * self.plan.max_rows, self.N), dtype=torch.bfloat16, device=dev)
            self.sh = ShardedBuffers(torch, ops, dist, dev, rank, world, self.total, self.N)
            owner = ops.ShardGroupsLpt(self.all_groups, world)     # the library's partition is the one the data follows
            assert owner == self.plan.owner, "library and host partition differ"
        self.h_A = torch.from_numpy(h["A"]).pin_memory()
        self.h_sA = torch.from_numpy(h["sA"]).pin_memory()
        self.h_C = torch.empty((max(self.local_rows, 1), self.N), dtype=torch.bfloat16).pin_memory()  # this rank's rows
        self.launches_per_step = 2  # one scale-repack launch + the matmul
        self.variant = "peer"

    def variants(self):
        return ["peer"]

    def work_per_step(self):
        return 2 * self.total * self.N * self.K   # whole job (all ranks together)

    def step(self, i):
        s = i % self.nsets
        if self.world == 1:
            # expert weights are static: their scales were brought into the kernel's order once, when the weights were
            # loaded (ascq_group_matmul_mxfp4_pack_scale_b); the step repacks the activations' scales only
            self.prepacked_step(i)
        else:
            self.ops.GroupMatmulMxfp4Sharded(self.sh.comm, self.sh.ptrs[i % 2], self.A[s], self.sA[s], self.B[s], self.sB[s],
                                             self.all_groups, self.K, self.N, self.ws)

    def gemm_only_step(self, i):
        s = i % self.nsets
        if self.world == 1:
            self.prepacked_step(i)
        elif self.groups:
            self.ops.GroupMatmulMxfp4(self.C[s], self.A[s], self.sA[s], self.B[s], self.sB[s], self.groups, self.K, self.N,
                                      workspace=self.ws)

    def raw_scales_step(self, i):
        """Weight scales in the reference's [G, N, K/32] order: repacked inside every step."""
        s = i % self.nsets
        self.ops.GroupMatmulMxfp4(self.C[s], self.A[s], self.sA[s], self.B[s], self.sB[s], self.groups, self.K, self.N,
                                  workspace=self.ws)

    def prepacked_step(self, i):
        """Static weights: their scales were brought into the kernel's order once, outside the step."""
        s = i % self.nsets
        self.ops.GroupMatmulMxfp4Prepacked(self.C[s], self.A[s], self.sA[s], self.B[s], self.sB_packed[s], self.groups, self.K,
                                           self.N, workspace=self.ws)

    def nccl_step(self, i):
        """The unfused variant: local matmul, rows padded to the largest share, NCCL all-gather (the ragged blocks
        still have to be put in order by the consumer)."""
        s = i % self.nsets
        self.gemm_only_step(i)
        self.padded[:self.local_rows].copy_(self.C[s][:self.local_rows])
        self.dist.all_gather_into_tensor(self.gathered, self.padded)

    def e2e_in(self, i):
        s = i % self.nsets
        self.A[s].copy_(self.h_A, non_blocking=True)      # this step's tokens and their scales; expert weights stay resident
        self.sA[s].copy_(self.h_sA, non_blocking=True)

    def e2e_out(self, i):
        if self.world == 1:
            self.h_C.copy_(self.C[i % self.nsets], non_blocking=True)
        else:   # every rank reads back the rows of its own groups from the assembled matrix
            at = 0
            for r0, n in zip(self.out_row_start, self.groups):
                self.h_C[at:at + n].copy_(self.sh.full[i % 2][r0:r0 + n], non_blocking=True)
                at += n

    def e2e_bytes(self):
        return self.host["A"].nbytes + self.host["sA"].nbytes, self.local_rows * self.N * 2

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
        """128 rows (one tile row) of this rank's first group against the oracle, element by element: |got - want| <=
        1e-2 |want| + K 2^-24 sum |a_k b_k| (rtol of the target plus the worst case of an fp32 accumulation).  With several
        ranks the assembled matrix must hold the same bits at those rows, and every rank's matrix must be complete."""
        rows = min(128, self.groups[0]) if self.groups else 0
        h = self.host
        ok = True
        if rows:
            A, sA = np.ascontiguousarray(h["A"][:rows]), np.ascontiguousarray(h["sA"][:rows])
            B, sB = np.ascontiguousarray(h["B"][:1]), np.ascontiguousarray(h["sB"][:1])
            _, want = O.group_matmul_mxfp4(A, sA, B, sB, np.array([rows], np.int64), self.K, self.N, want_f32=True)
            bound = mx_abs_product_sum(O, A, sA, B[0], sB[0], self.K) * (self.K * 2.0 ** -24)
            self.gemm_only_step(0)
            got = self.C[0][:rows].float().cpu().numpy()
            self.ops.MatmulStatus()
            ok = bool(np.all(np.abs(got - want) <= 1e-2 * np.abs(want) + bound))
        if self.world > 1:
            self.sh.full[0].zero_()
            self.torch.cuda.synchronize()
            self.dist.barrier()
            self.step(0)
            self.ops.MatmulStatus()
            if rows:
                r0 = self.out_row_start[0]
                ok = ok and bool(self.torch.equal(self.sh.full[0][r0:r0 + rows], self.C[0][:rows]))
            # every row of the assembled matrix was written by somebody (random operands: a zero row is a missing row)
            ok = ok and bool((self.sh.full[0] != 0).any(dim=1).all().item())
            self.dist.barrier()
        return ok


def mx_abs_product_sum(O, A, sA, Bg, sBg, K):
    """sum_k |a_k b_k| of dequantised MX-FP4 operands, [rows, N] in float64: the scale of the rounding error of an fp32
    accumulation."""
    lut = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], np.float64)

    def dq(codes, sc):
        lo, hi = codes & 0x7, (codes >> 4) & 0x7
        v = np.empty((codes.shape[0], K), np.float64)
        v[:, 0::2], v[:, 1::2] = lut[lo], lut[hi]
        return v * np.repeat(np.exp2(sc.astype(np.float64) - 127.0), 32, axis=1)
    return dq(A, sA) @ dq(Bg, sBg).T


WORKLOADS = {"w8a8_cfg4": W8A8Cfg4, "mxfp4_cfg5": Mxfp4Cfg5, "antiquant_cfg2": AntiQuantCfg2, "dequant_cfg3": DequantCfg3,
             "quant_scaled": QuantScaled}
HEADLINE = "w8a8_cfg4"


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


def _sync_ranks(torch, dist):
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()


def _regions(torch, dist, run_region, first_sec):
    """Repeats a timed region (K steps) R times back to back, R >= 10 and enough for about 50 ms under load, each
    bracketed by CUDA events on the launching stream; returns the R durations in seconds, max over ranks."""
    R = int(min(200, max(10, np.ceil(0.05 / max(first_sec, 1e-6)))))
    if dist is not None:    # every rank must repeat the same number of times
        t = torch.tensor([R], device="cuda", dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        R = int(t.item())
    _sync_ranks(torch, dist)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(R + 1)]
    ev[0].record()
    for r in range(R):
        run_region()
        ev[r + 1].record()
    _sync_ranks(torch, dist)
    secs = torch.tensor([ev[r].elapsed_time(ev[r + 1]) / 1e3 for r in range(R)], device="cuda", dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(secs, op=dist.ReduceOp.MAX)
    return [float(v) for v in secs.cpu()]


class E2EPipeline:
    """The end-to-end step of a workload as a three-stage pipeline over three streams: while the kernel of step i runs on
    the launching stream, the copy engines bring step i + 1's input from pinned host memory and take step i - 1's result
    back (PCIe carries both directions at once).  Every step still copies its own input in and its own result out inside
    the timed region; `drain` makes the launching stream wait for the last result, so a region's end event covers all of
    its copies.  Order kept by events: the input copy into a buffer set waits for the kernel that last read that set;
    a kernel waits for its input and for the previous step's result copy (which also keeps a peer's next-but-one step
    from overwriting an assembled matrix that is still being read out)."""

    def __init__(self, torch, wl):
        self.torch, self.wl = torch, wl
        self.h2d, self.d2h = torch.cuda.Stream(), torch.cuda.Stream()
        self.ev_in = torch.cuda.Event()
        self.ev_done = [torch.cuda.Event() for _ in range(wl.nsets)]
        self.ev_out = torch.cuda.Event()
        self.ev_begin = torch.cuda.Event()

    def begin(self):    # no copy of a region starts before the region does
        cur = self.torch.cuda.current_stream()
        self.ev_begin.record(cur)
        self.h2d.wait_event(self.ev_begin)
        self.d2h.wait_event(self.ev_begin)

    def step(self, i):
        t, wl = self.torch, self.wl
        cur = t.cuda.current_stream()
        s = i % wl.nsets
        self.h2d.wait_event(self.ev_done[s])      # (an event never recorded counts as complete)
        with t.cuda.stream(self.h2d):
            wl.e2e_in(i)
            self.ev_in.record()
        cur.wait_event(self.ev_in)
        cur.wait_event(self.ev_out)
        wl.step(i)
        self.ev_done[s].record(cur)
        self.d2h.wait_event(self.ev_done[s])
        with t.cuda.stream(self.d2h):
            wl.e2e_out(i)
            self.ev_out.record()

    def drain(self):
        self.torch.cuda.current_stream().wait_event(self.ev_out)


def time_steps(torch, fn, steps, warmup, dist=None, repeats=True, before=None, after=None):
    """W untimed calls of fn(i), then regions of K host-launched calls each (see _regions).  Returns the list of region
    durations in seconds (one region when repeats is False).  `before` / `after` run inside every timed region, at its
    start and its end."""
    _sync_ranks(torch, dist)
    for i in range(warmup):
        fn(i)
    if after:
        after()
    _sync_ranks(torch, dist)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if before:
        before()
    for i in range(steps):
        fn(warmup + i)
    if after:
        after()
    e1.record()
    _sync_ranks(torch, dist)
    first = e0.elapsed_time(e1) / 1e3
    if not repeats:
        t = torch.tensor([first], device="cuda", dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(t.item())]

    def region():
        if before:
            before()
        for i in range(steps):
            fn(warmup + i)
        if after:
            after()
    return _regions(torch, dist, region, first)


def time_graph(torch, fn, steps, warmup, dist=None):
    """The same, with the K timed calls captured once into a CUDA graph and each region one replay: the host's launch
    cost (Python, ctypes) is then outside the timed region.  Every rank captures and replays its own graph; the sharded
    kernels keep their step counter on the device, so replays stay in step across the ranks.  Returns the list of region
    durations, or None if capture fails on any rank."""
    ok = 1
    g = None
    try:
        _sync_ranks(torch, dist)
        for i in range(warmup):
            fn(i)
        _sync_ranks(torch, dist)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(steps):
                fn(warmup + i)
    except Exception as e:  # noqa: BLE001
        print(f"bench: CUDA graph capture unavailable ({e!r}); timing host launches", file=sys.stderr)
        ok = 0
    torch.cuda.synchronize()
    if dist is not None:
        t = torch.tensor([ok], device="cuda", dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        ok = int(t.item())
    if not ok:
        return None
    _sync_ranks(torch, dist)
    g.replay()                      # untimed: uploads the graph
    _sync_ranks(torch, dist)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    _sync_ranks(torch, dist)
    return _regions(torch, dist, g.replay, e0.elapsed_time(e1) / 1e3)


def best_of(torch, fn, steps, warmup, dist):
    """Region durations of fn, host-launched and graph-replayed; returns (median seconds per region, stats, how)."""
    host = time_steps(torch, fn, steps, warmup, dist)
    graph = time_graph(torch, fn, steps, warmup, dist)
    pick, how = host, "one host call per step"
    if graph is not None and np.median(graph) < np.median(host):
        pick, how = graph, "the K steps replayed from one CUDA graph"
    stats = {"regions": len(pick), "median_ms_per_step": float(np.median(pick)) / steps * 1e3,
             "min_ms_per_step": float(np.min(pick)) / steps * 1e3, "max_ms_per_step": float(np.max(pick)) / steps * 1e3,
             "host_launched_median_ms_per_step": float(np.median(host)) / steps * 1e3}
    return float(np.median(pick)), stats, how


def profile_traffic(key):
    """DRAM bytes read + written by the dominant kernel of one step, from the ncu summary kept under profiles/ (a line
    `traffic_bytes_per_launch: N`); None when there is no summary for the workload."""
    path = os.path.join(ROOT, "profiles", f"{key}_ncu_counters.md")
    try:
        with open(path) as f:
            for line in f:
                if line.startswith("traffic_bytes_per_launch:"):
                    return float(line.split(":", 1)[1].split()[0])
    except OSError:
        pass
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
    steps = args.steps
    sampler = ClockSampler(local) if rank == 0 else None   # runs across every timed region of this process
    for nm in names:
        sharded = nm in ("w8a8_cfg4", "mxfp4_cfg5")
        wl = WORKLOADS[nm](torch, ops, dev, dist, world, rank) if sharded else WORKLOADS[nm](torch, ops, dev)
        is_head = nm == (args.workload if args.workload != "all" else HEADLINE)
        variants = wl.variants() if sharded and world > 1 else [None]
        tried = {}
        for v in variants:
            if v is not None:
                wl.variant = v
            tried[v] = best_of(torch, wl.step, steps, args.warmup, dist)
        best = min(tried, key=lambda k: tried[k][0])
        if best is not None:
            wl.variant = best
        sec, stats, launch = tried[best]
        per = sec / steps
        work = wl.work_per_step()
        if sharded:
            achieved = work / per / 1e12          # T(FL)OPS of the whole job (strong scaling: work is split over ranks)
            total_value = achieved
            gsec, gstats, _ = best_of(torch, wl.gemm_only_step, steps, args.warmup, dist)
            if world == 1:
                gsec = min(gsec, sec)
            # the slowest rank's matmul alone, as a rate per GPU (group shares are not exactly equal)
            kern = work / world / (gsec / steps) / 1e12
            int8 = nm == "w8a8_cfg4"
            peak = (2.0 if int8 else 4.0) * peaks["bf16_tflops"]
            extra = {}
            if world > 1:
                extra["reassembly"] = {"peer": "epilogue TMA stores into every rank's matrix + arrival flags inside the launch",
                                       "multicast": "epilogue multimem stores through NVSwitch multicast + arrival flags inside the launch"}[best]
                extra["reassembly_variants_ms_per_step"] = {k: tried[k][0] / steps * 1e3 for k in tried}
                nsec = float(np.median(time_steps(torch, wl.nccl_step, steps, args.warmup, dist)))
                extra["nccl_allgather_variant"] = work / (nsec / steps) / 1e12
                out_bytes = (wl.M * wl.nl if int8 else wl.local_rows * wl.N) * 2 * (world - 1)
                extra["nvlink_egress_gbs_per_gpu"] = out_bytes / per / 1e9   # this rank's block to every peer, over the whole step
                if hasattr(wl, "single_gpu_step"):
                    t1, _, _ = best_of(torch, wl.single_gpu_step, steps, args.warmup, None)
                    extra["matmul_phase_efficiency"] = t1 / (world * gsec)   # T1 / (N * T_N), matmul kernels only
                    extra["single_gpu_ms_per_step_on_this_box"] = t1 / steps * 1e3
            ceiling = measured_tensor_ceiling(torch, ops, _lib.DT_I8 if int8 else _lib.DT_FP4X2_E2M1)
            roof = {"bound": "tensor", "achieved": kern, "peak": peak, "unit": wl.unit, "frac": kern / peak, "traffic": None,
                    "peak_source": ("2 x %s dense bf16 cuBLAS burst (int8 runs at twice the bf16 rate; nominal 4500)" if int8 else
                                    "4 x %s dense bf16 cuBLAS burst (FP4 runs at four times the bf16 rate; nominal 9000)")
                                   % peaks["source"], "kernel_ms": gsec / steps * 1e3,
                    # the tensor cores' own rate on this GPU for this operand type, measured in this run: the kernel's MMA
                    # instructions alone, operands in shared memory (ascq_measure_tensor_rate)
                    "measured_mma_only_ceiling": ceiling, "frac_of_measured_ceiling": kern / ceiling if ceiling else None,
                    "frac_of_nominal": kern / (4500.0 if int8 else 9000.0)}
        elif wl.bound == "tensor":
            raise AssertionError("every tensor-bound workload shards")
        else:
            achieved = work / per / 1e9           # GB/s (each rank does the full workload: replicas)
            total_value = achieved * world
            roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"]}
        if world == 1 and hasattr(wl, "probe_step"):
            psec, _, _ = best_of(torch, wl.probe_step, steps, args.warmup, None)
            roof["same_bytes_through_torch_cast_gbs"] = work / (psec / steps) / 1e9
        if world == 1:
            roof["traffic"] = profile_traffic(nm)
            roof["traffic_source"] = f"profiles/{nm}_ncu_counters.md" if roof["traffic"] is not None else None
        e2e_steps = max(4, min(steps, 64))
        pipe = E2EPipeline(torch, wl)
        e2e_sec = float(np.median(time_steps(torch, pipe.step, e2e_steps, 2, dist, before=pipe.begin, after=pipe.drain)))
        e2e_per = e2e_sec / e2e_steps
        h2d, d2h = wl.e2e_bytes()
        e2e_value = (work / e2e_per / 1e12 if sharded else
                     work / e2e_per / 1e12 * world if wl.bound == "tensor" else work / e2e_per / 1e9 * world)
        rec = {"name": wl.name, "value": total_value, "unit": wl.unit, "ms_per_step": per * 1e3,
               "roofline": roof, "timing": stats,
               "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "steps_per_region": e2e_steps,
                       "pipeline": "three streams: the input copy of step i+1 and the result copy of step i-1 overlap the kernel of step i; "
                                   "every region ends with the last result on the host"},
               "scaling": "strong" if sharded else "weak",
               "nsets": wl.nsets, "launches_per_step": wl.launches_per_step, "launch": launch,
               "ms_per_step_host_launched": stats["host_launched_median_ms_per_step"]}
        if sharded and world > 1:
            rec.update(extra)
        if world == 1 and hasattr(wl, "raw_scales_step"):
            psec, _, _ = best_of(torch, wl.raw_scales_step, steps, args.warmup, None)
            rec["weight_scales"] = "packed once at load time (ascq_group_matmul_mxfp4_pack_scale_b)"
            rec["with_weight_scales_repacked_every_step"] = {"value": work / (psec / steps) / 1e12, "unit": wl.unit,
                                                             "ms_per_step": psec / steps * 1e3}
        if rank == 0 or (sharded and world > 1):
            from oracle import oracle as O
            try:
                ok = wl.check(O)      # every rank takes part when the check runs a sharded step
            except ops.AscqError as e:
                ok = False
                rec["check_error"] = str(e)[:200]
            if rank == 0:
                rec["parity_vs_oracle"] = ok
        try:
            ops.MatmulStatus()
        except ops.AscqError as e:
            rec["device_status"] = str(e)[:200]
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
    published = None
    if world == 1 and args.workload == "all":
        published = run_published_shapes(torch, ops, dev, steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    if rank == 0:
        wl, rec = head
        line = {"metric": "W8A8/MXFP4 GEMM TOPS at 1/2/4/8 B200; quant/dequant GB/s vs HBM peak",
                "value": rec["value"], "unit": rec["unit"], "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": rec["scaling"], "vs_baseline": None,
                "dtype": wl.dtype, "data": "synthetic",
                "config": {"workload": rec["name"], "timing": "buffers rotate over a set larger than L2 (126 MB); median of "
                           "%d regions of K steps each" % rec["timing"]["regions"],
                           "launch": rec["launch"],
                           "sharding": ((wl.sharding_note + "; C reassembled inside the step: ") + rec.get("reassembly", "single GPU")
                                        if rec["scaling"] == "strong"
                                        else "replicas only (elementwise operators do not shard)")},
                "roofline": rec["roofline"], "e2e": rec["e2e"], "gpu_launches": args.steps * rec["launches_per_step"],
                "clocks": clocks, "workloads": results}
        if clocks and clocks.get("sm_mhz"):
            line["ms_per_step_x_sm_mhz"] = rec["ms_per_step"] * clocks["sm_mhz"]
        if "cpu_baseline" in rec:
            line["cpu_baseline"] = rec["cpu_baseline"]
        if published is not None:
            line["published_shapes"] = published
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def measured_tensor_ceiling(torch, ops, dtype_code, k_blocks=2048, reps=10):
    """T(FL)OPS of the MMA-only kernel (operands in shared memory, no copies, no epilogue): the measured ceiling of the
    matmul with that operand type on this GPU, at the clock a burst of that length runs at.  Best of `reps`."""
    best = 0.0
    for _ in range(3):
        ops.MeasureTensorRate(dtype_code, k_blocks)
    torch.cuda.synchronize()
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        n = ops.MeasureTensorRate(dtype_code, k_blocks)
        e1.record()
        torch.cuda.synchronize()
        best = max(best, n / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return best


def run_published_shapes(torch, ops, dev, steps, warmup):
    """The two shapes the reference publishes a timing for (on Ascend 950PR, in its sample READMEs), timed here the same
    way as the benchmark configurations; and config 1 at its own size (3 MiB: a latency, not a bandwidth)."""
    out = {}
    # grouped W8A8 + per-channel x per-token dequant + FasterGelu -> fp16, G = 8, M = N = 8192, K = 1024
    G, M, N, K = 8, 8192, 8192, 1024
    groups = [M // G] * G
    ns = 2
    gen = torch.Generator(device=dev).manual_seed(SEED)
    A = [torch.randint(-10, 10, (M, K), dtype=torch.int8, device=dev, generator=gen) for _ in range(ns)]
    B = [torch.randint(-10, 10, (G, N, K), dtype=torch.int8, device=dev, generator=gen) for _ in range(ns)]
    sA = torch.randn(M, device=dev, generator=gen) * 0.01
    sB = torch.randn((G, N), device=dev, generator=gen) * 0.01
    C = [torch.empty((M, N), dtype=torch.float16, device=dev) for _ in range(ns)]
    for act, nm in ((1, "quant_group_matmul G=8 M=N=8192 K=1024, dequant + FasterGelu -> fp16"),
                    (0, "the same without the activation")):
        sec, stats, how = best_of(torch, lambda i: ops.GroupMatmulW8A8(C[i % ns], A[i % ns], B[i % ns], sA, sB, groups, None, act),
                                  steps, warmup, None)
        us = sec / steps * 1e6
        out[nm] = {"us": round(us, 1), "TOPS": round(2.0 * M * N * K / us / 1e6, 1), "launch": how,
                   "reference_published": {"us": 204.129, "TOPS": 673, "hardware": "Ascend 950PR, 32 cores",
                                           "source": "quant_group_matmul_high_performance/README_en.md:394-396"} if act else None}
    r = slice(0, 64)   # parity of the timed call: 64 rows of group 0 against an exact fp32 product
    acc = A[0][r].float() @ B[0][0].float().T
    want = ((acc * sB[0][None, :]) * sA[r][:, None]).half()
    ops.GroupMatmulW8A8(C[0], A[0], B[0], sA, sB, groups, None, 0)
    torch.cuda.synchronize()
    out["quant_group_matmul parity (no activation, 64 rows, bit-exact)"] = bool(torch.equal(C[0][r], want))
    del A, B, C
    torch.cuda.empty_cache()
    # MX-FP4 matmul 8192^3 -> bf16 (one group)
    M = N = K = 8192
    A4 = [torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device=dev, generator=gen) for _ in range(ns)]
    B4 = [torch.randint(0, 256, (1, N, K // 2), dtype=torch.uint8, device=dev, generator=gen) for _ in range(ns)]
    sA4 = [torch.randint(123, 132, (M, K // 32), dtype=torch.uint8, device=dev, generator=gen) for _ in range(ns)]
    sB4 = [torch.randint(123, 132, (1, N, K // 32), dtype=torch.uint8, device=dev, generator=gen) for _ in range(ns)]
    C4 = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _ in range(ns)]
    ws = torch.empty(max(256, ops.GroupMatmulMxfp4Workspace(M, 1, K, N)), dtype=torch.uint8, device=dev)
    sec, stats, how = best_of(torch, lambda i: ops.GroupMatmulMxfp4(C4[i % ns], A4[i % ns], sA4[i % ns], B4[i % ns], sB4[i % ns], [M], K, N,
                                                                   workspace=ws), steps, warmup, None)
    us = sec / steps * 1e6
    out["matmul_mxfp4 M=N=K=8192 -> bf16"] = {"us": round(us, 1), "TFLOPS": round(2.0 * M * N * K / us / 1e6, 1), "launch": how,
                                             "reference_published": {"us": [693.283, 681.056], "TFLOPS": [1586, 1614],
                                                                     "hardware": "Ascend 950PR, 32 cores",
                                                                     "source": "matmul_mxfp4_high_performance/README_en.md:176-177, "
                                                                               "matmul_mxfp4_basic_api_high_performance/README_en.md:405-407"}}
    del A4, B4, C4, sA4, sB4
    torch.cuda.empty_cache()
    # config 1 at its own size: fp16 [256, 4096] -> int8, 3 MiB in all
    rows, cols = 256, 4096
    h = gen_quant_cfg1(rows, cols)
    ns1 = 96   # 96 x 3 MiB = 288 MiB of distinct buffers: every call reads DRAM
    x = [torch.from_numpy(h["x"]).to(dev) for _ in range(ns1)]
    y = [torch.empty((rows, cols), dtype=torch.int8, device=dev) for _ in range(ns1)]
    sec, stats, how = best_of(torch, lambda i: ops.AscendQuant(y[i % ns1], x[i % ns1], 64.0, 0.0, rows * cols), max(steps, 96), warmup, None)
    us = sec / max(steps, 96) * 1e6
    out["AscendQuant per-tensor fp16 [256, 4096] -> int8 (config 1 at its own size)"] = {
        "latency_us": round(us, 2), "GB/s": round(rows * cols * 3 / us / 1e3, 1), "launch": how,
        "note": "3 MiB per call: launch- and latency-bound; the DRAM-sized run of the same operator is quant_scaled"}
    return out


def few_rows_section(torch, ops, dev, add):
    """The matmuls with at most 32 activation rows (a decode step): bound by reading the 8192 x 8192 int8 weight once.  Six
    weight matrices (400 MB) rotate, so every launch reads its weight from HBM; each line is timed beside the form it
    replaces (two launches / the tcgen05 kernel), selected through the environment."""
    Nw = Kw = 8192
    nw = 6
    Bw = [torch.randint(-128, 128, (Nw, Kw), dtype=torch.int8, device=dev) for _ in range(nw)]
    wsw = torch.empty(Nw * Kw * 2, dtype=torch.uint8, device=dev)
    for dt, nm in ((torch.float16, "half"), (torch.bfloat16, "bfloat16")):
        scw = (torch.rand(Nw, device=dev) * 0.02).to(dt)
        ofw = torch.randn(Nw, device=dev).to(dt)
        for Mw in (1, 8, 16, 32):
            Aw = torch.randn((Mw, Kw), device=dev).to(dt)
            Cw = torch.empty((Mw, Nw), dtype=dt, device=dev)
            for form, label in (("small", "weight converted in registers"), ("twostep", "AscendAntiQuant launch, then the matmul")):
                os.environ["ASCQ_W8A16"] = form
                add(f"weight-only-quantised matmul, {Mw} x 8192 {nm} activations, 8192 x 8192 int8 weight, {label}",
                    lambda i: ops.MatmulW8A16(Cw, Aw, Bw[i % nw], ofw, scw, workspace=wsw), float(Nw * Kw), "TB/s of weight bytes")
            os.environ.pop("ASCQ_W8A16", None)
    B4w = [b[:, : Kw // 2].contiguous().view(torch.uint8) for b in Bw]   # the same bytes read as int4b_t pairs
    for dt, nm in ((torch.float16, "half"), (torch.bfloat16, "bfloat16")):
        scw = (torch.rand(Nw, device=dev) * 0.2).to(dt)
        ofw = torch.randn(Nw, device=dev).to(dt)
        for Mw in (1, 16):
            Aw = torch.randn((Mw, Kw), device=dev).to(dt)
            Cw = torch.empty((Mw, Nw), dtype=dt, device=dev)
            for form, label in (("small", "weight converted in registers"), ("twostep", "AscendAntiQuant launch, then the matmul")):
                os.environ["ASCQ_W8A16"] = form
                add(f"weight-only-quantised matmul, {Mw} x 8192 {nm} activations, 8192 x 8192 int4 weight, {label}",
                    lambda i: ops.MatmulW4A16(Cw, Aw, B4w[i % nw], ofw, scw, workspace=wsw), float(Nw * Kw // 2), "TB/s of weight bytes")
            os.environ.pop("ASCQ_W8A16", None)
    del B4w
    sBw = torch.rand(Nw, device=dev) * 0.01
    for Mw in (1, 16):   # (17 to 32 rows against a weight of this size stay on the tcgen05 kernel)
        A8w = torch.randint(-127, 128, (Mw, Kw), dtype=torch.int8, device=dev)
        sAw = torch.rand(Mw, device=dev) * 0.02
        C8w = torch.empty((Mw, Nw), dtype=torch.bfloat16, device=dev)
        for small, label in (("1", "few-row kernel"), ("0", "tcgen05 kernel")):
            os.environ["ASCQ_W8A8_SMALL"] = small
            add(f"W8A8 matmul + dequant, {Mw} x 8192 int8 activations, 8192 x 8192 int8 weight, {label}",
                lambda i: ops.MatmulW8A8(C8w, A8w, Bw[i % nw], sAw, sBw, None), float(Nw * Kw), "TB/s of weight bytes")
        os.environ.pop("ASCQ_W8A8_SMALL", None)
    del Bw, wsw


def run_extras(args):
    """`--workload extras` (`--workload few_rows`: its few-row matmul section alone): the operators of the path that are not among the five benchmark configurations, each timed
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
    few_rows_only = args.workload == "few_rows"

    def add(name, fn, work, unit):
        secs = time_graph(torch, fn, steps, warm)
        if secs is None:
            secs = time_steps(torch, fn, steps, warm)
        us = float(np.median(secs)) / steps * 1e6
        out[name] = {"us": round(us, 1), "rate": round(work / us / 1e6, 2), "unit": unit}  # work per us -> T(unit)/s
        print(f"extras: {name}: {us:.1f} us, {work / us / 1e6:.2f} {unit}", file=sys.stderr)

    if few_rows_only:
        few_rows_section(torch, ops, dev, add)
        ops.MatmulStatus()
        print(json.dumps({"metric": "matmuls with at most 32 activation rows, 8192 x 8192 int8 weight", "n_gpus": 1, "steps": steps, "warmup": warm,
                          "data": "synthetic", "launch": "the K steps replayed from one CUDA graph", "few_rows": out}))
        return
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
    few_rows_section(torch, ops, dev, add)
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
    # ---- what plain fills and copies of the two small configurations' byte counts reach (torch kernels; a yardstick
    # for the write direction of config 2 and for kernels of 10 to 30 us, not part of the library) ----
    del x, d4, s4, d8, dst4, src4
    torch.cuda.empty_cache()
    for nm, nbytes in (("config 2's output, 90 MB", 4096 * 11008 * 2), ("1 GiB", 1 << 30)):
        bufs = [torch.empty(nbytes, dtype=torch.uint8, device=dev) for _ in range(max(2, int(2.5 * L2_BYTES / nbytes) + 1))]
        add(f"torch fill_ of {nm} (write only)", lambda i: bufs[i % len(bufs)].fill_(1), nbytes, "TB/s")
        del bufs
    for nm, nbytes in (("config 2's total, 135 MB (67.6 MB read + 67.6 MB written)", 4096 * 11008 * 3 // 2),):
        src_ = [torch.empty(nbytes, dtype=torch.uint8, device=dev) for _ in range(max(2, int(1.5 * L2_BYTES / nbytes) + 1))]
        dst_ = [torch.empty(nbytes, dtype=torch.uint8, device=dev) for _ in range(len(src_))]
        add(f"torch copy_ of {nm}", lambda i: dst_[i % len(dst_)].copy_(src_[i % len(src_)]), 2 * nbytes, "TB/s")
        del src_, dst_
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
    ap.add_argument("--workload", default="all", choices=["all", "extras", "few_rows"] + list(WORKLOADS))
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    # Libraries (NCCL's version banner, for one) write to file descriptor 1; the JSON line must be the only thing on
    # stdout, so everything else is sent to stderr while the run lasts.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(real_stdout, "w")
    if args.impl == "reference":
        if args.workload in ("extras", "few_rows"):
            args.workload = "all"
        run_reference(args)
    elif args.workload in ("extras", "few_rows"):
        run_extras(args)
    else:
        run_ours(args)
    sys.stdout.flush()


if __name__ == "__main__":
    main()
