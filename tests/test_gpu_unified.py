"""GPU parity of the unified interface (Quantize / Dequantize / AntiQuantize: fp32 arithmetic for every policy)
against the CPU oracle, bit for bit, plus the reference's 950-series sample goldens through the GPU."""
import os

import numpy as np
import pytest
import torch

from asc_devkit_b200 import _lib as L
from asc_devkit_b200 import ops
from oracle import oracle as O
from tests.gpu_util import DEV, assert_bits_equal, rand_float, to_dev, to_host

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _scales(rng, shape, dt, lo, hi):
    return rand_float(rng, shape, dt, lo, hi)


@pytest.mark.parametrize("srcT,scaleT", [(O.F16, O.F16), (O.BF16, O.BF16), (O.F32, O.F32), (O.F16, O.F32), (O.BF16, O.F32)])
@pytest.mark.parametrize("policy,kDim", [(O.PER_TENSOR, 1), (O.PER_CHANNEL, 1), (O.PER_TOKEN, 1), (O.PER_GROUP, 1), (O.PER_GROUP, 0)])
@pytest.mark.parametrize("hasOffset,mode", [(True, O.CAST_RINT), (False, O.CAST_FLOOR), (True, O.CAST_ROUND)])
def test_quantize(srcT, scaleT, policy, kDim, hasOffset, mode):
    rng = np.random.default_rng(policy * 100 + kDim * 10 + srcT + scaleT)
    m, n, gs = 96, 256, 64
    src = rand_float(rng, (m, n), srcT, -40, 40)
    kw = dict(policy=policy, m=m, n=n, hasOffset=hasOffset, roundMode=mode, kDim=kDim, scaleT=scaleT)
    if policy == O.PER_TENSOR:
        sc_h = of_h = None
        kw.update(scaleScalar=3.25, offsetScalar=-1.5)
        scale = 3.25
        offset = -1.5
    else:
        shape = {O.PER_CHANNEL: (n,), O.PER_TOKEN: (m,)}.get(policy, (m, n // gs) if kDim == 1 else ((m + gs - 1) // gs, n))
        if policy == O.PER_GROUP:
            kw["groupSize"] = gs
        sc_h = _scales(rng, shape, scaleT, 0.5, 6.0)
        of_h = _scales(rng, shape, scaleT, -4.0, 4.0)
        kw.update(scale=sc_h, offset=of_h if hasOffset else None)
        scale, offset = to_dev(sc_h, scaleT), (to_dev(of_h, scaleT) if hasOffset else None)
    want = O.quantize(src, srcT, **kw)
    dst = torch.full((m, n), 77, dtype=torch.int8, device=DEV)
    ops.Quantize(dst, to_dev(src, srcT), scale, offset, ops.QuantizeParams(m, n, kw.get("groupSize", 0)), policy=policy,
                 hasOffset=hasOffset, roundMode=mode, kDim=kDim)
    assert_bits_equal(dst.cpu().numpy(), want, "Quantize")


@pytest.mark.parametrize("dstT", [O.F16, O.BF16])
@pytest.mark.parametrize("policy", [O.PER_TENSOR, O.PER_CHANNEL, O.PER_TOKEN, O.PER_GROUP])
@pytest.mark.parametrize("hasOffset", [True, False])
def test_antiquantize(dstT, policy, hasOffset):
    rng = np.random.default_rng(policy * 10 + dstT)
    m, n, gs = 64, 512, 32
    src = rng.integers(-128, 128, (m, n), dtype=np.int8)
    kw = dict(policy=policy, m=m, n=n, hasOffset=hasOffset, scaleT=dstT)
    if policy == O.PER_TENSOR:
        kw.update(scaleScalar=0.0123, offsetScalar=-3.7)
        scale, offset = 0.0123, -3.7
    else:
        shape = {O.PER_CHANNEL: (n,), O.PER_TOKEN: (m,), O.PER_GROUP: (m, n // gs)}[policy]
        if policy == O.PER_GROUP:
            kw["groupSize"] = gs
        sc_h = _scales(rng, shape, dstT, 0.001, 0.05)
        of_h = _scales(rng, shape, dstT, -8.0, 8.0)
        kw.update(scale=sc_h, offset=of_h if hasOffset else None)
        scale, offset = to_dev(sc_h, dstT), (to_dev(of_h, dstT) if hasOffset else None)
    want = O.antiquantize(src, O.I8, dstT, **kw)
    dst = torch.zeros((m, n), dtype=torch.float16 if dstT == O.F16 else torch.bfloat16, device=DEV)
    ops.AntiQuantize(dst, torch.from_numpy(src).to(DEV), scale, offset, ops.QuantizeParams(m, n, kw.get("groupSize", 0)),
                     policy=policy, hasOffset=hasOffset)
    assert_bits_equal(to_host(dst, dstT), want, "AntiQuantize")


@pytest.mark.parametrize("policy,dstT,scaleT", [(O.PER_TENSOR, O.BF16, O.F32), (O.PER_CHANNEL, O.BF16, O.F32), (O.PER_CHANNEL, O.F32, O.F32),
                                                (O.PER_TOKEN, O.F16, O.F32), (O.PER_GROUP, O.BF16, O.BF16)])
def test_dequantize(policy, dstT, scaleT):
    rng = np.random.default_rng(policy + dstT)
    m, n, gs = 48, 256, 32
    src = rng.integers(-2**20, 2**20, (m, n), dtype=np.int32)
    kw = dict(policy=policy, m=m, n=n, scaleT=scaleT)
    if policy == O.PER_TENSOR:
        kw.update(scaleScalar=0.00037)
        scale = 0.00037
    else:
        shape = {O.PER_CHANNEL: (n,), O.PER_TOKEN: (m,), O.PER_GROUP: (m, n // gs)}[policy]
        if policy == O.PER_GROUP:
            kw["groupSize"] = gs
        sc_h = _scales(rng, shape, scaleT, 1e-4, 1e-3)
        kw.update(scale=sc_h)
        scale = to_dev(sc_h, scaleT)
    want = O.dequantize(src, O.I32, dstT, **kw)
    tdt = {O.F16: torch.float16, O.BF16: torch.bfloat16, O.F32: torch.float32}[dstT]
    dst = torch.zeros(want.shape, dtype=tdt, device=DEV)
    ops.Dequantize(dst, torch.from_numpy(src).to(DEV), scale, None, ops.QuantizeParams(m, n, kw.get("groupSize", 0)), policy=policy)
    assert_bits_equal(to_host(dst, dstT), want, "Dequantize")


def test_sample_goldens_through_the_gpu():
    """The reference's own 950-series sample vectors (made by its gen_data.py scripts), through the CUDA path."""
    g = np.load(os.path.join(GOLDEN, "quant_dav3510.npz"))
    dst = torch.zeros(1024, dtype=torch.int8, device=DEV)
    ops.Quantize(dst, torch.from_numpy(g["input"]).to(DEV), 2.0, 0.9, ops.QuantizeParams(1, 1024), policy=L.PER_TENSOR, hasOffset=True)
    assert np.array_equal(dst.cpu().numpy(), g["golden"])
    g = np.load(os.path.join(GOLDEN, "antiquant_dav3510.npz"))
    out = torch.zeros((8, 128), dtype=torch.float16, device=DEV)
    ops.AntiQuantize(out, torch.from_numpy(g["input_src"]).to(DEV), torch.from_numpy(g["input_scale"].reshape(-1)).to(DEV),
                     torch.from_numpy(g["input_offset"].reshape(-1)).to(DEV), ops.QuantizeParams(8, 128), policy=L.PER_CHANNEL,
                     hasOffset=True)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), g["golden"].view(np.uint16))
    g = np.load(os.path.join(GOLDEN, "dequant.npz"))
    out = torch.zeros((128, 32), dtype=torch.float32, device=DEV)
    ops.Dequantize(out, torch.from_numpy(g["input"]).to(DEV), torch.from_numpy(g["scale"]).to(DEV), None,
                   ops.QuantizeParams(128, 32), policy=L.PER_CHANNEL)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), g["golden"].view(np.uint32))


def test_rejections_follow_the_reference():
    d = torch.zeros(64, dtype=torch.int8, device=DEV)
    s = torch.zeros(64, dtype=torch.float16, device=DEV)
    sc = torch.ones(64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ops.AscqError) as e:      # (src, scale) must be (T, T) or (T, float): quantize_impl.h:36-55
        ops.Quantize(d, s, sc, None, ops.QuantizeParams(1, 64), policy=L.PER_CHANNEL)
    assert e.value.status == L.ERR_UNSUPPORTED
    with pytest.raises(ops.AscqError) as e:      # "Dequantize do not support offset currently"
        ops.Dequantize(torch.zeros(64, device=DEV), torch.zeros(64, dtype=torch.int32, device=DEV), 1.0, None,
                       ops.QuantizeParams(1, 64), policy=L.PER_TENSOR, hasOffset=True)
    assert e.value.status == L.ERR_UNSUPPORTED
