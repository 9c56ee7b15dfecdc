"""The grouped MX-FP4 matmul through the entry point that brings its own scratch memory.

Some programs that embed this library are not allowed to allocate device memory themselves -- a serving
process whose memory pool already owns all of HBM, or a thread that cannot tolerate the device-wide stall of a
cudaMalloc.  ``ascq_group_matmul_mxfp4_noalloc`` serves them from a fixed array inside the library.  Here it is
called through the C ABI, twice in a row with different problems (the second call finds the first one's
leftovers in the shared scratch) and once more with the first problem, and each result must equal, bit for bit,
what the workspace-taking entry point produces.  Oversized problems must be refused with a clear message.

The file name sorts last so that a run that stops at the first failure has already run every other test.
"""
import ctypes as C
import gc

import numpy as np
import pytest
import torch

from asc_devkit_b200 import _lib as L
from asc_devkit_b200 import ops
from tests.gpu_util import DEV

pytestmark = pytest.mark.gpu


def _problem(groups, N, K, seed):
    rng = np.random.default_rng(seed)
    sumM, G = int(sum(groups)), len(groups)
    t = lambda a: torch.from_numpy(a).to(DEV)  # noqa: E731
    return dict(groups=groups, N=N, K=K,
                A=t(rng.integers(0, 256, (sumM, K // 2)).astype(np.uint8)),
                sA=t((127 + rng.integers(-4, 5, (sumM, K // 32))).astype(np.uint8)),
                B=t(rng.integers(0, 256, (G, N, K // 2)).astype(np.uint8)),
                sB=t((127 + rng.integers(-4, 5, (G, N, K // 32))).astype(np.uint8)))


def _with_workspace(p):
    out = torch.zeros((sum(p["groups"]), p["N"]), dtype=torch.bfloat16, device=DEV)
    ops.GroupMatmulMxfp4(out, p["A"], p["sA"], p["B"], p["sB"], p["groups"], p["K"], p["N"])
    ops.MatmulStatus()
    return out


def _no_alloc(p, check_driver_free=True):
    out = torch.zeros((sum(p["groups"]), p["N"]), dtype=torch.bfloat16, device=DEV)
    gl = (C.c_int64 * len(p["groups"]))(*p["groups"])
    gc.collect()  # tensors of earlier tests must not be released half-way through the measurement
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    reserved = torch.cuda.memory_reserved()
    # what the driver itself reports as free on the device: a cudaMalloc inside the library would show here, whereas
    # torch's own counters only see torch's allocator
    free_before = torch.cuda.mem_get_info()[0]
    rc = L.lib().ascq_group_matmul_mxfp4_noalloc(ops._ptr(out), ops._ptr(p["A"]), ops._ptr(p["sA"]), ops._ptr(p["B"]),
                                                 ops._ptr(p["sB"]), gl, len(p["groups"]), p["K"], p["N"],
                                                 ops._stream(None))
    L.check(rc)
    ops.MatmulStatus()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before and torch.cuda.memory_reserved() == reserved
    if check_driver_free:
        assert torch.cuda.mem_get_info()[0] == free_before, "the device's free memory changed during the call"
    return out


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    first = _problem([100, 0, 300, 129], 384, 384, 1)
    second = _problem([128, 40], 256, 1024, 2)
    want_first, want_second = _with_workspace(first), _with_workspace(second)
    # the first call of each kernel variant on a device loads its code, and the very first looks the array's address
    # up: the driver's free-memory figure is compared from the second round on
    assert torch.equal(_no_alloc(first, check_driver_free=False), want_first)
    assert torch.equal(_no_alloc(second, check_driver_free=False), want_second)
    assert torch.equal(_no_alloc(first), want_first)       # scratch still holds the second call's tables
    assert torch.equal(_no_alloc(second), want_second)     # and now the first call's
    assert torch.equal(_no_alloc(first), want_first)       # and now the second call's


def test_more_than_256_groups_build_their_tile_table_in_the_built_in_scratch():
    """With more than 256 groups the row-tile table is built on the host and copied into the scratch."""
    rng = np.random.default_rng(5)
    many = _problem([int(v) for v in rng.choice([0, 1, 3, 17, 130], 300)], 256, 256, 6)
    want = _with_workspace(many)
    assert torch.equal(_no_alloc(many, check_driver_free=False), want)
    assert torch.equal(_no_alloc(many), want)


def test_problems_beyond_the_built_in_scratch_are_refused():
    limit = L.lib().ascq_group_matmul_mxfp4_noalloc_max_scratch()
    assert limit == 16 << 20
    G, K, N = 16, 14336, 2048
    groups = [1024] * G
    assert L.lib().ascq_group_matmul_mxfp4_workspace_size(sum(groups), G, K, N) > limit
    gl = (C.c_int64 * G)(*groups)
    dummy = C.c_void_p(0x1000)  # never dereferenced: the size check comes first
    rc = L.lib().ascq_group_matmul_mxfp4_noalloc(dummy, dummy, dummy, dummy, dummy, gl, G, K, N, None)
    assert rc == L.ERR_INVALID_ARG
    assert b"built-in scratch" in L.lib().ascq_last_error()
