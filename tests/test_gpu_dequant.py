"""GPU parity of AscendDequant against the CPU oracle.  Bit-exact."""
import ctypes as C

import numpy as np
import pytest
import torch

from asc_devkit_b200 import _lib as L
from asc_devkit_b200 import ops
from oracle import oracle as O
from tests.gpu_util import DEV, TORCH_OF, assert_bits_equal, rand_float, to_dev, to_host

pytestmark = pytest.mark.gpu
CANARY = {O.F16: 0x1234, O.BF16: 0x1234, O.F32: 0x12345678}


def run_dequant(src, srcT, dstT, **kw):
    policy = kw["policy"]
    m, n, cal = kw["m"], kw["n"], kw["calCount"]
    if policy in (O.PER_TENSOR, O.PER_CHANNEL):
        rows, stride = m, O.dequant_dst_stride(n, dstT)
    else:
        rows, stride = cal // n, n
    fill = kw.get("fill", 0)
    d_dst = torch.empty((rows, stride), dtype=TORCH_OF[dstT], device=DEV)
    d_dst.view(torch.int16 if d_dst.element_size() == 2 else torch.int32).fill_(fill)
    scaleT = kw.get("scaleT", O.F32)
    d_scale = to_dev(kw.get("scale"), scaleT)
    d_tok = to_dev(kw.get("tokScale"), O.F32)
    p = L.DequantParam(m, n, cal, kw.get("groupSize", 0), kw.get("kDim", 1))
    rc = L.lib().ascq_dequant(ops._ptr(d_dst), dstT, ops._ptr(to_dev(src, srcT)), srcT, ops._ptr(d_scale),
                              ops._ptr(d_tok), scaleT, kw.get("scaleScalar", 0.0), policy, C.byref(p), ops._stream(None))
    L.check(rc)
    torch.cuda.synchronize()
    return to_host(d_dst, dstT)


def test_cfg3_full_size():
    # benchmark config 3: int32 [2048, 4096] in [-2^20, 2^20], per-channel fp32 x per-token fp32 -> bf16
    rng = np.random.default_rng(20251125 + 3)
    M, N = 2048, 4096
    acc = rng.integers(-2 ** 20, 2 ** 20 + 1, (M, N)).astype(np.int32)
    sch = rng.uniform(1e-5, 1e-3, N).astype(np.float32)
    stok = rng.uniform(0.5, 2.0, M).astype(np.float32)
    kw = dict(policy=O.PER_CHANNEL, m=M, n=N, calCount=N, scale=sch, tokScale=stok, scaleT=O.F32)
    assert_bits_equal(run_dequant(acc, O.I32, O.BF16, **kw), O.ascend_dequant(acc, O.I32, O.BF16, **kw), "cfg3")


def test_sample_golden_through_gpu(golden_dir):
    import os
    g = np.load(os.path.join(golden_dir, "dequant.npz"))
    got = run_dequant(g["input"], O.I32, O.F32, policy=O.PER_CHANNEL, m=128, n=32, calCount=32, scale=g["scale"],
                      scaleT=O.F32)
    assert_bits_equal(got, g["golden"], "dequant sample golden")


# (dst, scale) pairs of tests/api/adv_api/quantization/dequant/test_ascend_dequant.cpp:76-90
LEGACY = [(O.F16, O.U64), (O.BF16, O.BF16), (O.F32, O.BF16), (O.F32, O.F32), (O.BF16, O.F32)]


def make_scale(rng, n, scaleT):
    s = rng.uniform(-3, 3, n).astype(np.float32)
    if scaleT == O.U64:
        garbage = rng.integers(0, 2 ** 32, n, dtype=np.uint64) << np.uint64(32)  # the high word must be ignored
        return s.view(np.uint32).astype(np.uint64) | garbage
    if scaleT == O.BF16:
        return O.f32_to_bf16_bits(s)
    if scaleT == O.F16:
        return s.astype(np.float16)
    return s


@pytest.mark.parametrize("dstT,scaleT", LEGACY)
@pytest.mark.parametrize("m,n,cal", [(1, 16, 16), (4, 8, 8), (7, 40, 24), (5, 5120, 5120), (64, 264, 200)])
def test_per_channel_legacy(dstT, scaleT, m, n, cal):
    rng = np.random.default_rng(m * n + dstT * 10 + scaleT)
    src = rng.integers(-2 ** 27, 2 ** 27, (m, n)).astype(np.int32)  # beyond 2^24: the int->float cast rounds
    kw = dict(policy=O.PER_CHANNEL, m=m, n=n, calCount=cal, scale=make_scale(rng, n + 8, scaleT), scaleT=scaleT,
              fill=CANARY[dstT])
    got = run_dequant(src, O.I32, dstT, **kw)
    want = O.ascend_dequant(src, O.I32, dstT, **kw)
    assert_bits_equal(got, want, "legacy per-channel (pad columns and columns >= calCount keep the canary)")


@pytest.mark.parametrize("dstT,scalar", [(O.BF16, 0.0123), (O.F32, -7.5)])
def test_per_tensor_scalar(dstT, scalar):
    rng = np.random.default_rng(3)
    src = rng.integers(-2 ** 20, 2 ** 20, (33, 72)).astype(np.int32)
    kw = dict(policy=O.PER_TENSOR, m=33, n=72, calCount=72, scaleScalar=scalar, fill=CANARY[dstT])
    assert_bits_equal(run_dequant(src, O.I32, dstT, **kw), O.ascend_dequant(src, O.I32, dstT, **kw), "scalar")


POLICY_PAIRS = [(O.F16, O.F16), (O.BF16, O.BF16), (O.F32, O.F32), (O.F32, O.F16), (O.F32, O.BF16)]  # (scale, dst)


@pytest.mark.parametrize("srcT", [O.I32, O.F32])
@pytest.mark.parametrize("scaleT,dstT", POLICY_PAIRS)
@pytest.mark.parametrize("m,n", [(10, 256), (3, 40)])
def test_per_token(srcT, scaleT, dstT, m, n):
    rng = np.random.default_rng(m + n + srcT + scaleT * 3 + dstT * 5)
    src = rng.integers(-10 ** 6, 10 ** 6, (m, n)).astype(np.int32) if srcT == O.I32 else rand_float(rng, (m, n), O.F32, -1e4, 1e4)
    kw = dict(policy=O.PER_TOKEN, m=m, n=n, calCount=m * n, scale=make_scale(rng, m, scaleT), scaleT=scaleT)
    assert_bits_equal(run_dequant(src, srcT, dstT, **kw), O.ascend_dequant(src, srcT, dstT, **kw), "per-token")


@pytest.mark.parametrize("srcT", [O.I32, O.F32])
@pytest.mark.parametrize("scaleT,dstT", POLICY_PAIRS)
@pytest.mark.parametrize("kDim,groupSize", [(1, 32), (1, 128), (0, 32), (0, 64)])
def test_per_group(srcT, scaleT, dstT, kDim, groupSize):
    m, n = 128, 256
    rng = np.random.default_rng(groupSize + kDim + srcT + scaleT * 3 + dstT * 5)
    src = rng.integers(-10 ** 6, 10 ** 6, (m, n)).astype(np.int32) if srcT == O.I32 else rand_float(rng, (m, n), O.F32, -1e4, 1e4)
    count = m * (n // groupSize) if kDim == 1 else (m // groupSize) * n
    kw = dict(policy=O.PER_GROUP, m=m, n=n, calCount=m * n, scale=make_scale(rng, count, scaleT), scaleT=scaleT,
              groupSize=groupSize, kDim=kDim)
    assert_bits_equal(run_dequant(src, srcT, dstT, **kw), O.ascend_dequant(src, srcT, dstT, **kw), "per-group")


def test_linearity_at_scale():
    # property at a size the oracle is not run on: power-of-two scales commute exactly with the bf16 cast
    M, N = 8192, 8192
    g = torch.Generator(device=DEV).manual_seed(1)
    acc = torch.randint(-2 ** 20, 2 ** 20, (M, N), device=DEV, dtype=torch.int32, generator=g)
    s = torch.rand(N, device=DEV, generator=g) * 1e-3 + 1e-5
    a = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    b = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    ops.AscendDequant(a, acc, s, ops.DequantParams(M, N, N))
    ops.AscendDequant(b, acc, s * 4.0, ops.DequantParams(M, N, N))
    torch.cuda.synchronize()
    assert torch.equal(a.float() * 4.0, b.float())
