"""The multi-GPU entry points on ONE GPU: the data path of the *_sharded matmuls (TMA stores into every rank's matrix),
the end-of-step flags, and the two ways a bounded wait runs out -- each in a form that returns.

Ranks are emulated by launches that follow each other on one stream, every "peer" matrix and flag block being a local
buffer.  No launch ever waits for another launch: where a rank would wait for a peer, the peer's arrival flag is either
already in place (written by the earlier launch, or by the host) or the test WANTS the wait to run out, with the limit
lowered to about a millisecond, and checks the status the kernel leaves behind.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from asc_devkit_b200 import _lib as L, ops
from oracle import oracle as O
from tests.gpu_util import DEV, assert_bits_equal
from tests.test_gpu_matmul_mxfp4 import abs_product_sums, check_close, make_case as make_mx_case
from tests.test_gpu_matmul_w8a8 import make_case

pytestmark = pytest.mark.gpu

SHORT = 2_000_000  # SM cycles: about a millisecond


def flag_blocks(n):
    """n zeroed flag blocks in one allocation (512 bytes each) and their addresses."""
    fb = ops.Comm.flag_bytes()
    mem = torch.zeros(n * fb, dtype=torch.uint8, device=DEV)
    return mem, [mem.data_ptr() + r * fb for r in range(n)]


def words(mem):
    return mem.view(torch.int32).cpu().numpy().view(np.uint32).reshape(-1, 128)  # [rank][word]


EPOCH_WORD, ARRIVE_STRIDE = 64, 8  # CommFlags: arrive[src][0] at word 8 * src, epoch at word 64


@pytest.fixture
def short_waits():
    ops.SetWaitLimitCycles(SHORT)
    yield
    ops.SetWaitLimitCycles(0)
    try:
        ops.MatmulStatus()  # leave the status words clear for the tests that follow
    except ops.AscqError:
        pass


def dev_case(A, B, sA, sB, bias):
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)  # noqa: E731
    return t(A), t(B), t(sA), t(sB), torch.from_numpy(bias.view(np.int16).copy()).to(DEV).view(torch.bfloat16)


def test_one_rank_communicator_is_the_plain_matmul():
    M, N, K = 300, 256, 256
    A, B, sA, sB, bias = make_case(M, N, K, 3)
    want = O.matmul_w8a8(A, B, sA, sB, bias)
    mem, ptrs = flag_blocks(1)
    comm = ops.Comm(0, 1, ptrs)
    out = torch.full((M, N), -1.0, dtype=torch.bfloat16, device=DEV)
    dA, dB, dsA, dsB, dbias = dev_case(A, B, sA, sB, bias)
    ops.MatmulW8A8Sharded(comm, [out.data_ptr()], dA, dB, dsA, dsB, dbias)
    ops.MatmulStatus()
    assert_bits_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), want, "one rank")
    comm.destroy()


@pytest.mark.parametrize("nranks,M,N,K", [(2, 384, 512, 256), (4, 200, 1024, 128), (8, 129, 1024, 384)])
def test_w8a8_ranks_one_after_the_other_assemble_every_matrix(nranks, M, N, K):
    """Rank r's launch stores its column block into all `nranks` matrices and signals; launched in rank order with the
    flags of the ranks still to come put in place by the host, no launch waits.  Afterwards every matrix is the whole
    result, every block's epoch is 1 and every arrival slot holds 1."""
    A, B, sA, sB, bias = make_case(M, N, K, nranks)
    want = O.matmul_w8a8(A, B, sA, sB, bias)
    mem, ptrs = flag_blocks(nranks)
    # the host stands in for the ranks that launch later: rank r finds the arrivals of ranks > r already there
    w = np.zeros((nranks, 128), np.uint32)
    for r in range(nranks):
        for src in range(r + 1, nranks):
            w[r, ARRIVE_STRIDE * src] = 1
    mem.copy_(torch.from_numpy(w.view(np.uint8).reshape(-1)).to(DEV))
    outs = [torch.full((M, N), -1.0, dtype=torch.bfloat16, device=DEV) for _ in range(nranks)]
    nl = N // nranks
    dA, _, dsA, _, _ = dev_case(A, B, sA, sB, bias)
    for r in range(nranks):
        comm = ops.Comm(r, nranks, ptrs)
        assert ops.ShardColumns(N, nranks, r) == (r * nl, nl)
        _, dB, _, dsB, dbias = dev_case(A, B[r * nl:(r + 1) * nl], sA, sB[r * nl:(r + 1) * nl], bias[r * nl:(r + 1) * nl])
        ops.MatmulW8A8Sharded(comm, [o.data_ptr() for o in outs], dA, dB, dsA, dsB, dbias)
        comm.destroy()
    ops.MatmulStatus()   # no wait ran out
    for r, o in enumerate(outs):
        assert_bits_equal(o.view(torch.int16).cpu().numpy().view(np.uint16), want, f"matrix of rank {r}")
    w = words(mem)
    for r in range(nranks):
        assert w[r, EPOCH_WORD] == 1
        for src in range(nranks):
            if src != r:
                assert w[r, ARRIVE_STRIDE * src] == 1, (r, src)


def test_mxfp4_ranks_one_after_the_other_assemble_every_matrix():
    groups, N, K, nranks = [300, 0, 5, 256, 129, 64], 512, 512, 3
    A, sA, B, sB = make_mx_case(groups, N, K, 77)
    _, want = O.group_matmul_mxfp4(A, sA, B, sB, np.array(groups, np.int64), K, N, want_f32=True)
    owner = ops.ShardGroupsLpt(groups, nranks)
    from asc_devkit_b200 import sharding
    assert owner == sharding.assign_groups_lpt(groups, nranks).owner
    starts = np.concatenate([[0], np.cumsum(groups)])
    mem, ptrs = flag_blocks(nranks)
    w = np.zeros((nranks, 128), np.uint32)
    for r in range(nranks):
        for src in range(r + 1, nranks):
            w[r, ARRIVE_STRIDE * src] = 1
    mem.copy_(torch.from_numpy(w.view(np.uint8).reshape(-1)).to(DEV))
    total = int(sum(groups))
    outs = [torch.full((total, N), -1.0, dtype=torch.bfloat16, device=DEV) for _ in range(nranks)]
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)  # noqa: E731
    for r in range(nranks):
        mine = [g for g in range(len(groups)) if owner[g] == r]
        rows = np.concatenate([np.arange(starts[g], starts[g + 1]) for g in mine]).astype(np.int64)
        comm = ops.Comm(r, nranks, ptrs)
        ws = torch.empty(max(256, ops.GroupMatmulMxfp4Workspace(len(rows), len(mine), K, N)), dtype=torch.uint8, device=DEV)
        ops.GroupMatmulMxfp4Sharded(comm, [o.data_ptr() for o in outs], t(A[rows]), t(sA[rows]), t(B[mine]), t(sB[mine]), groups, K, N, ws)
        comm.destroy()
    ops.MatmulStatus()
    first = outs[0].view(torch.int16).cpu().numpy().view(np.uint16)
    check_close(first, want, "assembled matrix", abs_product_sums(A, sA, B, sB, groups, K), K)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    assert (words(mem)[:, EPOCH_WORD] == 1).all()


def test_a_rank_without_groups_still_signals():
    groups, N, K, nranks = [128, 64], 256, 256, 3   # rank 2 gets nothing
    assert sorted(set(ops.ShardGroupsLpt(groups, nranks))) == [0, 1]
    mem, ptrs = flag_blocks(nranks)
    w = np.zeros((nranks, 128), np.uint32)
    w[2, 0] = w[2, ARRIVE_STRIDE] = 1   # ranks 0 and 1 "have arrived" at rank 2
    mem.copy_(torch.from_numpy(w.view(np.uint8).reshape(-1)).to(DEV))
    comm = ops.Comm(2, nranks, ptrs)
    out = torch.zeros((192, N), dtype=torch.bfloat16, device=DEV)
    dummy = torch.zeros(256, dtype=torch.uint8, device=DEV)
    ops.GroupMatmulMxfp4Sharded(comm, [out.data_ptr()] * nranks, dummy, dummy, dummy, dummy, groups, K, N, dummy)
    ops.MatmulStatus()
    w = words(mem)
    assert w[2, EPOCH_WORD] == 1 and w[0, ARRIVE_STRIDE * 2] == 1 and w[1, ARRIVE_STRIDE * 2] == 1
    comm.destroy()


def test_a_peer_that_never_arrives_ends_in_a_timeout_status(short_waits):
    """Two ranks, the second never launches: rank 0's stores land, its wait for the peer's flag runs out after the
    (lowered) limit, the kernel ends normally and ascq_matmul_status reports ASCQ_ERR_TIMEOUT once."""
    M, N, K = 256, 256, 128
    A, B, sA, sB, bias = make_case(M, N, K, 9)
    want = O.matmul_w8a8(A, B[:128], sA, sB[:128], bias[:128])
    mem, ptrs = flag_blocks(2)
    comm = ops.Comm(0, 2, ptrs)
    outs = [torch.full((M, N), -1.0, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    dA, dB, dsA, dsB, dbias = dev_case(A, B[:128], sA, sB[:128], bias[:128])
    ops.MatmulW8A8Sharded(comm, [o.data_ptr() for o in outs], dA, dB, dsA, dsB, dbias)
    with pytest.raises(ops.AscqError) as e:
        ops.MatmulStatus()
    assert e.value.status == L.ERR_TIMEOUT
    ops.MatmulStatus()   # the status word was cleared
    for o in outs:
        got = o.view(torch.int16).cpu().numpy().view(np.uint16)
        assert_bits_equal(np.ascontiguousarray(got[:, :128]), want, "block of rank 0")
    assert words(mem)[1, 0] == 1   # rank 0 did signal its peer
    # the exchange on its own runs out the same way
    comm.barrier()
    with pytest.raises(ops.AscqError) as e:
        ops.MatmulStatus()
    assert e.value.status == L.ERR_TIMEOUT
    comm.destroy()


@pytest.mark.parametrize("tile", ["narrow", "wide", "pair"])
def test_abort_path_of_the_matmul_kernel_returns_and_the_next_call_is_exact(tile, short_waits, monkeypatch):
    """The producers stop after three k-blocks (test hook): the MMA thread's wait for the fourth runs out, every role
    leaves its loop, tensor memory is released, the status word reports the timeout -- and the kernel after it is
    bit-exact, so nothing was left behind."""
    monkeypatch.setenv("ASCQ_W8A8_TILE", tile)
    M, N, K = 512, 512, 1024
    A, B, sA, sB, bias = make_case(M, N, K, 17)
    want = O.matmul_w8a8(A, B, sA, sB, bias)
    dA, dB, dsA, dsB, dbias = dev_case(A, B, sA, sB, bias)
    out = torch.full((M, N), -1.0, dtype=torch.bfloat16, device=DEV)
    L.check(L.lib().ascq_test_withhold_after(3))
    ops.MatmulW8A8(out, dA, dB, dsA, dsB, dbias)
    with pytest.raises(ops.AscqError) as e:
        ops.MatmulStatus()
    assert e.value.status == L.ERR_TIMEOUT
    ops.MatmulW8A8(out, dA, dB, dsA, dsB, dbias)
    ops.MatmulStatus()
    assert_bits_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), want, f"call after the abort ({tile})")


def test_argument_checks():
    mem, ptrs = flag_blocks(2)
    with pytest.raises(ops.AscqError):
        ops.Comm(2, 2, ptrs)
    with pytest.raises(ops.AscqError):
        ops.Comm(0, 9, (ptrs * 5)[:9])
    h = C.c_void_p()
    bad = (C.c_void_p * 2)(C.c_void_p(ptrs[0] + 4), C.c_void_p(ptrs[1]))
    assert L.lib().ascq_comm_create(C.byref(h), 0, 2, bad) == L.ERR_ALIGNMENT
    with pytest.raises(ops.AscqError):
        ops.ShardColumns(100, 3, 0)
    comm = ops.Comm(0, 2, ptrs)
    A = torch.zeros((64, 64), dtype=torch.int8, device=DEV)
    with pytest.raises(ops.AscqError):   # N / nranks must be a multiple of 8
        ops.MatmulW8A8Sharded(comm, ptrs, A, torch.zeros((4, 64), dtype=torch.int8, device=DEV))
    comm.destroy()
