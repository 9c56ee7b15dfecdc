"""CPU-only checks of the C-ABI library: it loads, exports every function include/ascq.h declares, its host-only
entry points (tmp-size queries, status strings) give the reference's known answers, and argument validation
returns the documented codes before any CUDA work is attempted."""
import ctypes as C
import os
import re

import pytest

from asc_devkit_b200 import _lib as L
from oracle import oracle as O
from tests.test_oracle_golden import tiling_known_answers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(ascq_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    lib = L.lib()
    declared = declared_functions()
    assert len(declared) >= 10
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported by libascq.so"
    assert declared == set(L.SIGNATURES), "ctypes signature table and header disagree"


def test_version_and_status_strings():
    lib = L.lib()
    assert lib.ascq_version() == 1
    assert L.status_string(L.OK) == "ASCQ_OK"
    assert L.status_string(L.ERR_TIMEOUT) == "ASCQ_ERR_TIMEOUT"


def test_tiling_known_answers_through_c_abi():
    from asc_devkit_b200 import ops
    tiling_known_answers(ops.GetAscendQuantMaxMinTmpSize, ops.GetAscendQuantTmpBufferFactorSize,
                         ops.GetAscendDequantMaxMinTmpSize, ops.GetAscendDequantTmpBufferFactorSize,
                         ops.GetAscendAntiQuantMaxMinTmpSize, ops.GetAscendAntiQuantTmpBufferFactorSize)
    # fp4 input: tmp only when transposed (ascend_antiquant_tiling_impl.cpp:31-45)
    assert ops.GetAscendAntiQuantMaxMinTmpSize([64, 512], [64, 16], True, L.DT_FP4X2_E2M1, L.DT_BF16) == (2048, 2048)
    assert ops.GetAscendAntiQuantMaxMinTmpSize([64, 512], [2, 512], False, L.DT_FP4X2_E2M1, L.DT_BF16) == (0, 0)


def test_tiling_host_asserts_become_error_codes():
    from asc_devkit_b200 import ops
    with pytest.raises(L.AscqError) as e:
        ops.GetAscendQuantMaxMinTmpSize([3], 2)       # 6 bytes: not 32B aligned
    assert e.value.status == L.ERR_INVALID_ARG and "32B aligned" in e.value.message
    with pytest.raises(L.AscqError):
        ops.GetAscendQuantMaxMinTmpSize([512], 1)     # unsupported type size
    with pytest.raises(L.AscqError):
        ops.GetAscendDequantMaxMinTmpSize([2, 3, 4], 4)  # rank 3
    with pytest.raises(L.AscqError):
        ops.GetAscendDequantMaxMinTmpSize([32], 2)    # src must be int32


def _call_quant(policy, dstT=L.DT_I8, srcT=L.DT_F16, scale=None, offset=None, scaleT=L.DT_F16, n=32, cal=64,
                gs=0, dst=0x1000, src=0x2000, kdim=1):
    p = L.QuantParam(2, n, cal, gs, 0, kdim, L.CAST_RINT)
    return L.lib().ascq_quant(C.c_void_p(dst), dstT, C.c_void_p(src), srcT, scale, offset, scaleT, 1.0, 0.0, policy,
                              C.byref(p), None)


def test_argument_validation_without_a_device():
    # these return before any CUDA call, so they are testable on a machine without a GPU
    fake = C.c_void_p(0x3000)
    assert _call_quant(L.PER_CHANNEL_PER_GROUP) == L.ERR_UNSUPPORTED
    assert _call_quant(L.PER_TOKEN_PER_GROUP) == L.ERR_UNSUPPORTED
    assert _call_quant(L.PER_TENSOR, srcT=L.DT_I32) == L.ERR_UNSUPPORTED
    assert _call_quant(L.PER_TENSOR, dstT=L.DT_FP8_E4M3) == L.ERR_UNSUPPORTED
    assert _call_quant(L.PER_TENSOR, dst=0) == L.ERR_INVALID_ARG
    assert _call_quant(L.PER_TENSOR, dst=0x2000) == L.ERR_INVALID_ARG               # src == dst
    assert _call_quant(L.PER_CHANNEL, scale=None) == L.ERR_INVALID_ARG              # missing scale tensor
    assert _call_quant(L.PER_CHANNEL, scale=fake, n=48, cal=64) == L.ERR_INVALID_ARG  # calCount % scaleCount
    assert b"integer multiple" in L.lib().ascq_last_error()
    assert _call_quant(L.PER_CHANNEL, scale=fake, n=8, cal=64) == L.ERR_INVALID_ARG   # scaleCount*2 B not 32B aligned
    assert _call_quant(L.PER_GROUP, scale=fake, gs=48) == L.ERR_INVALID_ARG           # groupSize % 32
    assert _call_quant(L.PER_GROUP, scale=fake, gs=32, kdim=2) == L.ERR_INVALID_ARG
    assert _call_quant(L.PER_TOKEN, scale=fake, srcT=L.DT_F16, scaleT=L.DT_BF16) == L.ERR_UNSUPPORTED

    dp = L.DequantParam(4, 30, 30, 0, 1)
    rc = L.lib().ascq_dequant(fake, L.DT_BF16, C.c_void_p(0x4000), L.DT_I32, fake, None, L.DT_F32, 0.0, L.PER_CHANNEL,
                              C.byref(dp), None)
    assert rc == L.ERR_INVALID_ARG and b"divisible by 32" in L.lib().ascq_last_error()
    dp = L.DequantParam(4, 32, 40, 0, 1)
    rc = L.lib().ascq_dequant(fake, L.DT_BF16, C.c_void_p(0x4000), L.DT_I32, fake, None, L.DT_F32, 0.0, L.PER_CHANNEL,
                              C.byref(dp), None)
    assert rc == L.ERR_INVALID_ARG and b"(0, params.n" in L.lib().ascq_last_error()
    dp = L.DequantParam(4, 32, 32, 0, 1)
    rc = L.lib().ascq_dequant(fake, L.DT_F16, C.c_void_p(0x4000), L.DT_I32, fake, None, L.DT_F32, 0.0, L.PER_CHANNEL,
                              C.byref(dp), None)
    assert rc == L.ERR_UNSUPPORTED  # (float scale, half dst) is not a legal legacy pair

    ap = L.AntiQuantParam(64, 48, 0, 0, 1, 1, 1)
    rc = L.lib().ascq_antiquant(fake, L.DT_BF16, C.c_void_p(0x4000), L.DT_I8, fake, fake, L.DT_BF16, 0.0, 0.0,
                                L.PER_CHANNEL, C.byref(ap), None)
    assert rc == L.ERR_INVALID_ARG and b"32B aligned" in L.lib().ascq_last_error()   # transposed K = 48 bytes
    ap = L.AntiQuantParam(64, 64, 0, 0, 1, 0, 1)
    rc = L.lib().ascq_antiquant(fake, L.DT_F32, C.c_void_p(0x4000), L.DT_I8, fake, fake, L.DT_F32, 0.0, 0.0,
                                L.PER_CHANNEL, C.byref(ap), None)
    assert rc == L.ERR_UNSUPPORTED
    rc = L.lib().ascq_antiquant(fake, L.DT_BF16, C.c_void_p(0x4000), L.DT_FP4X2_E2M1, fake, fake, L.DT_E8M0, 0.0, 0.0,
                                L.PER_GROUP, C.byref(ap), None)
    assert rc == L.ERR_UNSUPPORTED   # fp4 never takes an offset


def test_oracle_rejects_the_same_malformed_calls():
    import numpy as np
    x = np.zeros((2, 32), np.float16)
    with pytest.raises(O.OracleError):
        O.ascend_quant(x, O.F16, policy=O.PER_CHANNEL, n=48, calCount=64, scale=np.zeros(48, np.float16))
    with pytest.raises(O.OracleError):
        O.ascend_quant(x, O.F16, policy=O.PER_GROUP, m=2, n=32, scale=np.zeros(2, np.float16), groupSize=48)


def test_partition_of_the_sharded_matmuls_matches_the_host_side_plan():
    """Host-only entry points of the multi-GPU API: the column partition, and the longest-group-first deal, which must be
    the one asc_devkit_b200.sharding uses (the data of a run is laid out by one and consumed by the other)."""
    import numpy as np

    from asc_devkit_b200 import ops, sharding
    assert ops.ShardColumns(4096, 8, 3) == (1536, 512)
    with pytest.raises(L.AscqError):
        ops.ShardColumns(4096, 3, 0)
    rng = np.random.default_rng(0)
    for trial in range(50):
        G = int(rng.integers(1, 40))
        groups = [int(v) for v in rng.integers(0, 300, G)]
        if trial % 5 == 0:
            groups = [groups[0]] * G          # ties everywhere
        for world in (1, 2, 3, 8):
            assert ops.ShardGroupsLpt(groups, world) == sharding.assign_groups_lpt(groups, world).owner, (groups, world)
    with pytest.raises(L.AscqError):
        ops.ShardGroupsLpt([5, -1], 2)


def test_communicator_argument_checks_need_no_gpu():
    blocks = (C.c_void_p * 2)(C.c_void_p(0x1000), C.c_void_p(0x2000))     # never dereferenced on the host
    h = C.c_void_p()
    lib = L.lib()
    assert lib.ascq_comm_flag_bytes() == 512
    assert lib.ascq_comm_create(C.byref(h), 0, 2, blocks) == L.OK and h.value
    r, n = C.c_int(), C.c_int()
    assert lib.ascq_comm_rank(h, C.byref(r), C.byref(n)) == L.OK and (r.value, n.value) == (0, 2)
    assert lib.ascq_comm_destroy(h) == L.OK
    assert lib.ascq_comm_create(C.byref(h), 2, 2, blocks) == L.ERR_INVALID_ARG
    assert lib.ascq_comm_create(C.byref(h), 0, 9, blocks) == L.ERR_INVALID_ARG
    bad = (C.c_void_p * 2)(C.c_void_p(0x1010), C.c_void_p(0x2000))
    assert lib.ascq_comm_create(C.byref(h), 0, 2, bad) == L.ERR_ALIGNMENT
    assert lib.ascq_matmul_w8a8_sharded(None, blocks, None, None, None, None, None, None, 8, 8, 16, None) == L.ERR_INVALID_ARG
    assert lib.ascq_group_matmul_w8a8(None, L.DT_F16, None, None, None, None, None, None, 1, 8, 16, 0, None) == L.ERR_INVALID_ARG
