"""Multi-rank host logic on CPU: two gloo ranks shard the W8A8 matmul by output columns and the grouped MX-FP4
matmul by groups, compute their shares with the CPU oracle, all-gather, and must reproduce the unsharded result."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from asc_devkit_b200 import sharding
from oracle import oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)  # same data on every rank
        # ---- W8A8, column sharded ----
        M, N, K = 24, 64, 128
        A = rng.integers(-127, 128, (M, K)).astype(np.int8)
        B = rng.integers(-127, 128, (N, K)).astype(np.int8)
        sA = rng.uniform(0.005, 0.02, M).astype(np.float32)
        sB = rng.uniform(0.001, 0.01, N).astype(np.float32)
        bias = O.f32_to_bf16_bits(rng.normal(0, 0.1, N).astype(np.float32))
        n0, nl = sharding.column_shard(N, world, rank)
        local = O.matmul_w8a8(A, np.ascontiguousarray(B[n0:n0 + nl]), sA, sB[n0:n0 + nl].copy(), bias[n0:n0 + nl].copy())
        gathered = sharding.all_gather_blocks(torch.from_numpy(local.view(np.uint8)), world)  # gloo has no 16-bit types
        full = sharding.interleave_column_blocks(gathered).contiguous().numpy().view(np.uint16)
        ok1 = np.array_equal(full, O.matmul_w8a8(A, B, sA, sB, bias))
        # ---- grouped MX-FP4, group sharded ----
        groups = [5, 0, 9, 3, 7]
        Kx, Nx = 128, 16
        total = sum(groups)
        Ax = rng.integers(0, 256, (total, Kx // 2)).astype(np.uint8)
        sAx = (127 + rng.integers(-2, 3, (total, Kx // 32))).astype(np.uint8)
        Bx = rng.integers(0, 256, (len(groups), Nx, Kx // 2)).astype(np.uint8)
        sBx = (127 + rng.integers(-2, 3, (len(groups), Nx, Kx // 32))).astype(np.uint8)
        plan = sharding.assign_groups_lpt(groups, world)
        mine = plan.groups_of[rank]
        rows = sharding.local_row_index(groups, mine).numpy()
        local = O.group_matmul_mxfp4(np.ascontiguousarray(Ax[rows]), np.ascontiguousarray(sAx[rows]),
                                     np.ascontiguousarray(Bx[mine]), np.ascontiguousarray(sBx[mine]),
                                     np.array([groups[g] for g in mine], np.int64), Kx, Nx)
        padded = torch.zeros((plan.max_rows, Nx * 2), dtype=torch.uint8)
        padded[:rows.size] = torch.from_numpy(local.view(np.uint8))
        gathered = sharding.all_gather_blocks(padded, world)
        fullx = sharding.scatter_group_rows(gathered, plan, groups).numpy().view(np.uint16)
        ok2 = np.array_equal(fullx, O.group_matmul_mxfp4(Ax, sAx, Bx, sBx, np.array(groups, np.int64), Kx, Nx))
        ret[rank] = (ok1, ok2, sorted(plan.rows_of))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_reproduces_the_unsharded_result():
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        for r in range(world):
            ok1, ok2, loads = ret[r]
            assert ok1, "column-sharded W8A8 differs from the unsharded result"
            assert ok2, "group-sharded MX-FP4 differs from the unsharded result"
            assert loads == [12, 12]


def test_lpt_balances_uneven_groups():
    plan = sharding.assign_groups_lpt([1000, 10, 990, 20, 500, 480], 2)
    assert sorted(plan.rows_of) == [1500, 1500]
    assert sorted(sum(plan.groups_of, [])) == list(range(6))
    assert sharding.column_shard(4096, 8, 3) == (1536, 512)
