"""GPU parity of AscendAntiQuant against the CPU oracle.  Bit-exact."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from asc_devkit_b200 import _lib as L
from asc_devkit_b200 import ops
from oracle import oracle as O
from tests.gpu_util import DEV, TORCH_OF, assert_bits_equal, rand_float, to_dev, to_host

pytestmark = pytest.mark.gpu


def run_antiquant(src, srcT, dstT, **kw):
    m, n = kw["m"], kw["n"]
    total = kw.get("calCount", 0) or m * n
    scaleT = kw.get("scaleT", O.BF16)
    d_dst = torch.zeros((total // n, n), dtype=TORCH_OF[dstT], device=DEV)
    d_src = to_dev(src, srcT)
    d_scale = to_dev(kw.get("scale"), scaleT)
    d_off = to_dev(kw.get("offset"), scaleT)
    p = L.AntiQuantParam(m, n, kw.get("calCount", 0), kw.get("groupSize", 0), int(kw.get("hasOffset", True)),
                         int(kw.get("isTranspose", False)), kw.get("kDim", 1))
    rc = L.lib().ascq_antiquant(ops._ptr(d_dst), dstT, ops._ptr(d_src), srcT, ops._ptr(d_off), ops._ptr(d_scale), scaleT,
                                kw.get("offsetScalar", 0.0), kw.get("scaleScalar", 0.0), kw["policy"], C.byref(p),
                                ops._stream(None))
    L.check(rc)
    torch.cuda.synchronize()
    return to_host(d_dst, dstT)


def both(src, srcT, dstT, what, **kw):
    assert_bits_equal(run_antiquant(src, srcT, dstT, **kw), O.ascend_antiquant(src, srcT, dstT, **kw), what)


def test_cfg2_full_size():
    # benchmark config 2: int8 [4096, 11008], bf16 scale ~ U(0.001, 0.02), bf16 offset ~ U(-4, 4) -> bf16
    rng = np.random.default_rng(20251125 + 2)
    K, N = 4096, 11008
    w = rng.integers(-127, 128, (K, N)).astype(np.int8)
    scale = O.f32_to_bf16_bits(rng.uniform(0.001, 0.02, N).astype(np.float32))
    offset = O.f32_to_bf16_bits(rng.uniform(-4, 4, N).astype(np.float32))
    both(w, O.I8, O.BF16, "cfg2", policy=O.PER_CHANNEL, m=K, n=N, scale=scale, offset=offset, scaleT=O.BF16)


def test_sample_goldens_through_gpu(golden_dir):
    g = np.load(os.path.join(golden_dir, "antiquant_dav2201.npz"))
    got = run_antiquant(g["input_src"], O.I8, O.F16, policy=O.PER_CHANNEL, m=8, n=128,
                        scale=g["input_scale"].reshape(-1), offset=g["input_offset"].reshape(-1), scaleT=O.F16)
    assert_bits_equal(got, g["golden"], "antiquant sample golden (half arithmetic)")
    g = np.load(os.path.join(golden_dir, "antiquant_dav3510.npz"))
    got = run_antiquant(g["input_src"], O.I8, O.F16, policy=O.PER_TOKEN, m=8, n=128, isTranspose=True,
                        scale=g["input_scale"].reshape(-1).astype(np.float32),
                        offset=g["input_offset"].reshape(-1).astype(np.float32), scaleT=O.F32, hasOffset=True)
    assert_bits_equal(got, g["golden"], "antiquant sample golden (fp32 arithmetic)")


@pytest.mark.parametrize("dstT", [O.F16, O.BF16])
@pytest.mark.parametrize("isTranspose", [False, True])
@pytest.mark.parametrize("rows,cols,groups", [(64, 2048, 1), (96, 12288, 1), (64, 256, 4), (8, 128, 1), (33, 80, 1), (32, 96, 2)])
@pytest.mark.parametrize("with_offset", [True, False])
def test_legacy_per_channel(dstT, isTranspose, rows, cols, groups, with_offset):
    # non-transposed: src [K=rows, N=cols], scale [groups, N]; transposed: src [N=rows, K=cols], scale [N, groups]
    K = cols if isTranspose else rows
    if K % groups or (isTranspose and cols % 32):
        pytest.skip("not a legal layout")
    gs = K // groups
    rng = np.random.default_rng(rows * cols + dstT + groups)
    src = rng.integers(-128, 128, (rows, cols)).astype(np.int8)
    count = groups * cols if not isTranspose else rows * groups
    scale = rand_float(rng, (count,), dstT, -2, 2)
    offset = rand_float(rng, (count,), dstT, -8, 8) if with_offset else None
    both(src, O.I8, dstT, "legacy per-channel", policy=O.PER_CHANNEL, m=rows, n=cols, scale=scale, offset=offset,
         scaleT=dstT, isTranspose=isTranspose, groupSize=0 if groups == 1 else gs)


@pytest.mark.parametrize("dstT", [O.F16, O.BF16])
@pytest.mark.parametrize("hasOffset", [True, False])
def test_scalar(dstT, hasOffset):
    rng = np.random.default_rng(11 + dstT)
    src = rng.integers(-128, 128, (37, 100)).astype(np.int8)
    both(src, O.I8, dstT, "scalar", policy=O.PER_TENSOR, m=37, n=100, scaleScalar=0.0371, offsetScalar=-1.33,
         hasOffset=hasOffset)


POLICY_PAIRS = [(O.F16, O.F16), (O.BF16, O.BF16), (O.F32, O.F32), (O.F16, O.F32), (O.BF16, O.F32)]  # (dst, scale)


@pytest.mark.parametrize("dstT,scaleT", POLICY_PAIRS)
@pytest.mark.parametrize("isTranspose", [False, True])
@pytest.mark.parametrize("hasOffset", [True, False])
def test_per_token(dstT, scaleT, isTranspose, hasOffset):
    m, n = 24, 512
    rng = np.random.default_rng(dstT * 7 + scaleT + isTranspose)
    src = rng.integers(-128, 128, (m, n)).astype(np.int8)
    count = n if isTranspose else m
    both(src, O.I8, dstT, "per-token", policy=O.PER_TOKEN, m=m, n=n, scale=rand_float(rng, (count,), scaleT, -2, 2),
         offset=rand_float(rng, (count,), scaleT, -8, 8) if hasOffset else None, scaleT=scaleT, hasOffset=hasOffset,
         isTranspose=isTranspose)


@pytest.mark.parametrize("dstT,scaleT", POLICY_PAIRS)
@pytest.mark.parametrize("isTranspose,kDim", [(False, 1), (False, 0), (True, 1), (True, 0)])
@pytest.mark.parametrize("groupSize", [32, 128])
def test_per_group(dstT, scaleT, isTranspose, kDim, groupSize):
    m, n = 128, 256
    rng = np.random.default_rng(dstT * 7 + scaleT + kDim * 3 + groupSize)
    src = rng.integers(-128, 128, (m, n)).astype(np.int8)
    along_cols = (kDim == 1 and not isTranspose) or (kDim == 0 and isTranspose)
    count = m * (n // groupSize) if along_cols else (m // groupSize) * n
    both(src, O.I8, dstT, "per-group", policy=O.PER_GROUP, m=m, n=n, scale=rand_float(rng, (count,), scaleT, -2, 2),
         offset=rand_float(rng, (count,), scaleT, -8, 8), scaleT=scaleT, hasOffset=True, isTranspose=isTranspose,
         kDim=kDim, groupSize=groupSize)


@pytest.mark.parametrize("dstT", [O.BF16, O.F16])
@pytest.mark.parametrize("isTranspose", [False, True])
@pytest.mark.parametrize("rows,cols", [(64, 256), (32, 96), (128, 7168), (64, 34)])
def test_mx_fp4_decode(dstT, isTranspose, rows, cols):
    kext = cols if isTranspose else rows
    if kext % 32:
        pytest.skip("K must be a multiple of 32")
    rng = np.random.default_rng(rows + cols)
    src = rng.integers(0, 256, (rows, cols // 2)).astype(np.uint8)          # all 16 codes, both nibbles
    nscale = rows * (cols // 32) if isTranspose else (rows // 32) * cols
    scale = (127 + rng.integers(-10, 11, nscale)).astype(np.uint8)
    scale[0] = 0          # 2^-127
    scale[-1] = 254       # 2^127: overflows half, stays finite in bf16
    d_src = torch.from_numpy(src).to(DEV)
    d_scale = torch.from_numpy(scale).to(DEV)
    d_dst = torch.zeros((rows, cols), dtype=TORCH_OF[dstT], device=DEV)
    ops.AscendAntiQuant(d_dst, d_src, None, d_scale, ops.AscendAntiQuantParam(rows, cols), isTranspose=isTranspose,
                        policy=O.PER_GROUP, hasOffset=False, src_dtype=L.DT_FP4X2_E2M1, scale_dtype=L.DT_E8M0)
    torch.cuda.synchronize()
    want = O.ascend_antiquant(src, O.FP4X2_E2M1, dstT, policy=O.PER_GROUP, m=rows, n=cols, scale=scale, scaleT=O.E8M0,
                              hasOffset=False, isTranspose=isTranspose)
    assert_bits_equal(to_host(d_dst, dstT), want, "mx decode")


def test_quant_of_antiquant_round_trip_at_scale():
    # property at full cfg2 size without the oracle: with scale 2^-3 and offset 0 the bf16 result is exact, so
    # re-quantising with scale 8 returns the int8 weights
    K, N = 4096, 11008
    g = torch.Generator(device=DEV).manual_seed(2)
    w = torch.randint(-128, 128, (K, N), device=DEV, dtype=torch.int8, generator=g)
    scale = torch.full((N,), 0.125, dtype=torch.bfloat16, device=DEV)
    offset = torch.zeros(N, dtype=torch.bfloat16, device=DEV)
    deq = torch.empty((K, N), dtype=torch.bfloat16, device=DEV)
    ops.AscendAntiQuant(deq, w, offset, scale, ops.AscendAntiQuantParam(K, N))
    back = torch.empty((K, N), dtype=torch.int8, device=DEV)
    ops.AscendQuant(back, deq, 8.0, 0.0, K * N)
    torch.cuda.synchronize()
    assert torch.equal(back, w)


@pytest.mark.parametrize("dstT", [O.F16, O.BF16])
@pytest.mark.parametrize("isTranspose", [False, True])
def test_int4_source(dstT, isTranspose):
    """int4b_t weights (two signed nibbles per byte, even element in the low nibble) through the legacy per-channel
    operator: ascend_antiquant_impl.h:246-247 casts them to half and runs the same arithmetic."""
    rng = np.random.default_rng(7 + dstT)
    rows, cols = (96, 256) if not isTranspose else (256, 128)   # [K, N] or [N, K]; cols even
    packed = rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8)
    nper = cols if not isTranspose else rows
    scale = rand_float(rng, (nper,), dstT, 0.01, 0.5)
    offset = rand_float(rng, (nper,), dstT, -4, 4)
    want = O.ascend_antiquant(packed, O.I4X2, dstT, policy=O.PER_CHANNEL, m=rows, n=cols, scale=scale, offset=offset,
                              scaleT=dstT, isTranspose=isTranspose)
    d_dst = torch.zeros((rows, cols), dtype=TORCH_OF[dstT], device=DEV)
    ops.AscendAntiQuant(d_dst, torch.from_numpy(packed).to(DEV), to_dev(offset, dstT), to_dev(scale, dstT),
                        ops.AscendAntiQuantParam(rows, cols), isTranspose=isTranspose, src_dtype=L.DT_I4X2)
    assert_bits_equal(to_host(d_dst, dstT), want, "int4 source")
    # the values themselves: nibble n decodes to ((n ^ 8) - 8)
    ones = O.ascend_antiquant(np.arange(256, dtype=np.uint8).reshape(1, 256), O.I4X2, O.F16, policy=O.PER_TENSOR, m=1,
                              n=512, scaleScalar=1.0, offsetScalar=0.0, scaleT=O.F16, hasOffset=True)
    lo = ((np.arange(256) & 15) ^ 8) - 8
    hi = ((np.arange(256) >> 4) ^ 8) - 8
    assert np.array_equal(ones.reshape(256, 2).astype(np.int32), np.stack([lo, hi], 1))
