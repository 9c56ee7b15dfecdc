"""GPU parity of AscendQuant (C ABI -> CUDA) against the CPU oracle.  Bit-exact."""
import numpy as np
import pytest
import torch

from asc_devkit_b200 import _lib as L
from asc_devkit_b200 import ops
from oracle import oracle as O
from tests.gpu_util import DEV, assert_bits_equal, empty_dev, rand_float, to_dev, to_host

pytestmark = pytest.mark.gpu


def run_quant(src, srcT, **kw):
    """Same keyword interface as oracle.ascend_quant, executed by the CUDA library."""
    policy = kw["policy"]
    dstT = kw.get("dstT", O.I8)
    d_src = to_dev(src, srcT)
    if dstT == O.I8:
        d_dst = torch.full(src.shape, 77, dtype=torch.int8, device=DEV)
    else:
        d_dst = torch.zeros(src.size // 2, dtype=torch.uint8, device=DEV)
    scaleT = kw.get("scaleT", O.F16)
    scale = kw.get("scale")
    offset = kw.get("offset")
    cal = kw.get("calCount", src.size)
    p = L.QuantParam(kw.get("m", 0), kw.get("n", 0), cal, kw.get("groupSize", 0), int(kw.get("hasOffset", False)),
                     kw.get("kDim", 1), kw.get("roundMode", O.CAST_RINT))
    import ctypes as C
    d_scale = to_dev(scale, scaleT) if scale is not None else None
    d_off = to_dev(offset, scaleT) if offset is not None else None
    rc = L.lib().ascq_quant(ops._ptr(d_dst), dstT, ops._ptr(d_src), srcT, ops._ptr(d_scale), ops._ptr(d_off), scaleT,
                            kw.get("scaleScalar", 0.0), kw.get("offsetScalar", 0.0), policy, C.byref(p),
                            ops._stream(None))
    L.check(rc)
    torch.cuda.synchronize()
    return d_dst.cpu().numpy()


def test_cfg1_per_tensor_full_size():
    # benchmark config 1: fp16 [256, 4096] ~ N(0,1), scale 64, offset 0
    x = np.random.default_rng(20251125 + 1).standard_normal((256, 4096)).astype(np.float16)
    want = O.ascend_quant(x, O.F16, policy=O.PER_TENSOR, scaleScalar=64.0, offsetScalar=0.0)
    got = run_quant(x, O.F16, policy=O.PER_TENSOR, scaleScalar=64.0, offsetScalar=0.0)
    assert_bits_equal(got, want, "cfg1")
    assert 0.02 < np.mean((got == 127) | (got == -128)) < 0.08


def test_sample_golden_through_gpu(golden_dir):
    import os
    g = np.load(os.path.join(golden_dir, "quant_dav2201.npz"))
    got = run_quant(g["input"], O.F32, policy=O.PER_TENSOR, scaleScalar=2.0, offsetScalar=0.9)
    assert_bits_equal(got, g["golden"], "quant sample golden")


@pytest.mark.parametrize("srcT", [O.F16, O.F32, O.BF16])
@pytest.mark.parametrize("count", [1, 31, 32, 4096, 4097, 8192 + 17, 100003])
def test_per_tensor_ragged_counts(srcT, count):
    rng = np.random.default_rng(count * 7 + srcT)
    x = rand_float(rng, (count,), srcT, -80, 80)
    kw = dict(policy=O.PER_TENSOR, scaleScalar=1.7, offsetScalar=-0.35)
    assert_bits_equal(run_quant(x, srcT, **kw), O.ascend_quant(x, srcT, **kw), f"per-tensor {count}")


def test_per_tensor_calcount_prefix_only():
    rng = np.random.default_rng(5)
    x = rand_float(rng, (10000,), O.F16, -50, 50)
    kw = dict(policy=O.PER_TENSOR, scaleScalar=3.0, offsetScalar=0.5, calCount=4100)
    got = run_quant(x, O.F16, **kw)
    want = O.ascend_quant(x, O.F16, **kw)
    assert_bits_equal(got[:4100], want[:4100], "prefix")
    assert (got[4100:] == 77).all(), "elements beyond calCount must stay untouched"


def test_unaligned_base_pointers():
    rng = np.random.default_rng(6)
    x = rand_float(rng, (5000,), O.F16, -50, 50)
    d_src = to_dev(x, O.F16)[1:]            # 2-byte offset: not 16-byte aligned
    d_dst = torch.zeros(4999 + 3, dtype=torch.int8, device=DEV)[3:]
    ops.AscendQuant(d_dst, d_src, 2.0, 0.25, 4999)
    torch.cuda.synchronize()
    want = O.ascend_quant(np.ascontiguousarray(x[1:]), O.F16, policy=O.PER_TENSOR, scaleScalar=2.0, offsetScalar=0.25)
    assert_bits_equal(d_dst.cpu().numpy(), want, "unaligned")


@pytest.mark.parametrize("srcT", [O.F16, O.F32])
@pytest.mark.parametrize("tensor_offset", [False, True])
@pytest.mark.parametrize("m,n", [(7, 256), (33, 1024), (5, 48), (3, 16)])
def test_per_channel(srcT, tensor_offset, m, n):
    if (n * O.DT_SIZE[srcT]) % 32:
        pytest.skip("scaleCount must be 32-byte aligned")
    rng = np.random.default_rng(m * n + srcT)
    x = rand_float(rng, (m, n), srcT, -30, 30)
    scale = rand_float(rng, (n,), srcT, 0.5, 4.0)
    offset = rand_float(rng, (n,), srcT, -2, 2) if tensor_offset else None
    kw = dict(policy=O.PER_CHANNEL, n=n, calCount=m * n, scale=scale, offset=offset, scaleT=srcT, offsetScalar=0.37)
    assert_bits_equal(run_quant(x, srcT, **kw), O.ascend_quant(x, srcT, **kw), "per-channel")


PAIRS = [(O.F16, O.F16), (O.BF16, O.BF16), (O.F32, O.F32), (O.F16, O.F32), (O.BF16, O.F32)]


@pytest.mark.parametrize("srcT,scaleT", PAIRS)
@pytest.mark.parametrize("hasOffset", [False, True])
@pytest.mark.parametrize("m,n", [(10, 256), (10, 288), (8, 512), (3, 40)])
def test_per_token(srcT, scaleT, hasOffset, m, n):
    # shapes of tests/api/adv_api/quantization/quant/test_ascend_quant_per_token.cpp:146-173 (+ a ragged one)
    rng = np.random.default_rng(m * n + srcT * 10 + scaleT)
    x = rand_float(rng, (m, n), srcT, -20, 20)
    scale = rand_float(rng, (m,), scaleT, 0.5, 8.0)
    offset = rand_float(rng, (m,), scaleT, -3, 3)
    kw = dict(policy=O.PER_TOKEN, m=m, n=n, calCount=m * n, scale=scale, offset=offset if hasOffset else None,
              scaleT=scaleT, hasOffset=hasOffset)
    assert_bits_equal(run_quant(x, srcT, **kw), O.ascend_quant(x, srcT, **kw), "per-token")


@pytest.mark.parametrize("srcT,scaleT", PAIRS)
@pytest.mark.parametrize("kDim", [0, 1])
@pytest.mark.parametrize("groupSize", [32, 64, 128])
def test_per_group(srcT, scaleT, kDim, groupSize):
    m, n = 128, 256
    rng = np.random.default_rng(groupSize + kDim + srcT * 10 + scaleT)
    x = rand_float(rng, (m, n), srcT, -20, 20)
    sshape = (m, n // groupSize) if kDim == 1 else (m // groupSize, n)
    scale = rand_float(rng, sshape, scaleT, 0.5, 8.0)
    offset = rand_float(rng, sshape, scaleT, -3, 3)
    kw = dict(policy=O.PER_GROUP, m=m, n=n, calCount=m * n, scale=scale, offset=offset, scaleT=scaleT, hasOffset=True,
              groupSize=groupSize, kDim=kDim)
    assert_bits_equal(run_quant(x, srcT, **kw), O.ascend_quant(x, srcT, **kw), "per-group")


@pytest.mark.parametrize("roundMode", [O.CAST_NONE, O.CAST_RINT, O.CAST_FLOOR, O.CAST_CEIL, O.CAST_ROUND, O.CAST_TRUNC])
@pytest.mark.parametrize("srcT,scaleT", [(O.F16, O.F16), (O.F32, O.F32), (O.BF16, O.BF16)])
def test_round_modes_on_exact_halves(roundMode, srcT, scaleT):
    # values k + 0.5 hit every tie; scale 1 keeps them exact
    vals = (np.arange(-300, 300, dtype=np.float32) * 0.5).reshape(4, 150)
    vals = np.tile(vals, (1, 2))[:, :288]
    x = vals.astype(np.float16) if srcT == O.F16 else (O.f32_to_bf16_bits(vals) if srcT == O.BF16 else vals)
    one = rand_float(np.random.default_rng(0), (4,), scaleT, 1.0, 1.0)
    kw = dict(policy=O.PER_TOKEN, m=4, n=288, calCount=4 * 288, scale=one, scaleT=scaleT, roundMode=roundMode)
    assert_bits_equal(run_quant(np.ascontiguousarray(x), srcT, **kw), O.ascend_quant(np.ascontiguousarray(x), srcT, **kw),
                      f"round mode {roundMode}")


@pytest.mark.parametrize("srcT,scaleT", [(O.F16, O.F16), (O.BF16, O.BF16), (O.F16, O.F32)])
def test_per_group_to_fp4(srcT, scaleT):
    m, n, gs = 16, 128, 32
    rng = np.random.default_rng(99 + srcT + scaleT)
    x = rand_float(rng, (m, n), srcT, -7, 7)
    scale = rand_float(rng, (m, n // gs), scaleT, 0.5, 2.0)
    kw = dict(policy=O.PER_GROUP, m=m, n=n, calCount=m * n, scale=scale, scaleT=scaleT, groupSize=gs, kDim=1,
              dstT=O.FP4X2_E2M1)
    assert_bits_equal(run_quant(x, srcT, **kw), O.ascend_quant(x, srcT, **kw), "fp4 quant")


@pytest.mark.parametrize("srcT,scaleT", [(O.F16, O.F16), (O.BF16, O.BF16), (O.F16, O.F32), (O.BF16, O.F32), (O.F32, O.F32)])
@pytest.mark.parametrize("kDim", [0, 1])
@pytest.mark.parametrize("m,n", [(64, 256), (96, 1000), (32, 36)])
def test_per_group_to_fp4_shapes_and_specials(srcT, scaleT, kDim, m, n):
    """The vector kernel (n a multiple of 8) and the scalar one (n = 36) against the oracle: groups along either
    axis, values beyond +-6, infinities, a NaN (positive: the sign of a NaN does not survive a multiply on the GPU and is
    not part of the contract), signed zeros."""
    gs = 32
    rng = np.random.default_rng(7 * m + n + 3 * srcT + scaleT + kDim)
    x = rng.uniform(-9, 9, (m, n)).astype(np.float32)
    x[1, 3] = np.inf; x[2, 5] = -np.inf; x[3, 6] = np.nan; x[5, 8] = -0.0; x[6, 9] = 1e30; x[7, 10] = -1e-30
    x[8, :12] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -2.5, -5.0, 6.5]
    with np.errstate(over="ignore", invalid="ignore"):
        xs = x.astype(np.float16) if srcT == O.F16 else (O.f32_to_bf16_bits(x) if srcT == O.BF16 else x)
    shape = (m, (n + gs - 1) // gs) if kDim == 1 else ((m + gs - 1) // gs, n)
    scale = rand_float(rng, shape, scaleT, 0.5, 2.0)
    if kDim == 1:
        scale.reshape(-1)[0] = scale.reshape(-1)[0] * 0 + 1  # keeps row 8's ties on the ties (first group of row 0 only)
    kw = dict(policy=O.PER_GROUP, m=m, n=n, calCount=m * n, scale=scale, scaleT=scaleT, groupSize=gs, kDim=kDim, dstT=O.FP4X2_E2M1)
    got, want = run_quant(xs, srcT, **kw), O.ascend_quant(xs, srcT, **kw)
    bad = np.argwhere(got.reshape(-1) != want.reshape(-1))
    assert bad.size == 0, f"{len(bad)} bytes differ, first at {bad[0]}: got {got.reshape(-1)[bad[0][0]]:#x} want {want.reshape(-1)[bad[0][0]]:#x}"


def test_dynamic_per_token_quant():
    rng = np.random.default_rng(1234)
    for m, n, dt in [(64, 4096, O.F16), (5, 1000, O.F32), (17, 8192, O.BF16), (3, 7, O.F16)]:
        x = rand_float(rng, (m, n), dt, -9, 9)
        if m > 4:
            x[2] = 0  # an all-zero token
        want_q, want_s, want_d = O.dynamic_quant_per_token(x, dt, m, n)
        d_x = to_dev(x, dt)
        d_q = torch.empty((m, n), dtype=torch.int8, device=DEV)
        d_s = torch.empty(m, dtype=torch.float32, device=DEV)
        d_d = torch.empty(m, dtype=torch.float32, device=DEV)
        ops.DynamicQuantPerToken(d_q, d_s, d_x, d_d)
        torch.cuda.synchronize()
        assert_bits_equal(d_s.cpu().numpy(), want_s, "scale")
        assert_bits_equal(d_d.cpu().numpy(), want_d, "dequant scale")
        assert_bits_equal(d_q.cpu().numpy(), want_q, "int8")


def test_quant_is_monotone_at_scale():
    # size-independent property at a size the oracle is not run on: quantisation preserves order
    n = 1 << 24
    x = torch.linspace(-3.0, 3.0, n, device=DEV, dtype=torch.float32).to(torch.float16)
    q = torch.empty(n, dtype=torch.int8, device=DEV)
    ops.AscendQuant(q, x, 64.0, 0.0, n)
    torch.cuda.synchronize()
    d = q[1:].to(torch.int16) - q[:-1].to(torch.int16)
    assert int(d.min()) >= 0 and int(q.min()) == -128 and int(q.max()) == 127


@pytest.mark.parametrize("srcT", [O.F16, O.BF16, O.F32])
@pytest.mark.parametrize("m,n", [(1, 32), (77, 7168), (512, 4096)])
def test_dynamic_quant_mxfp4(srcT, m, n):
    """Activations -> MX-FP4 operands on the GPU, bit for bit against the oracle (codes and scale bytes)."""
    rng = np.random.default_rng(m + n + srcT)
    x = rng.standard_normal((m, n)).astype(np.float32) * np.exp2(rng.integers(-6, 7, (m, n // 32)).repeat(32, axis=1)).astype(np.float32)
    x[0, :32] = 0.0
    if srcT == O.F16:
        xs = x.astype(np.float16)
    elif srcT == O.BF16:
        xs = O.f32_to_bf16_bits(x)
    else:
        xs = x
    want_codes, want_sc = O.dynamic_quant_mxfp4(xs, srcT, m, n)
    dst = torch.zeros((m, n // 2), dtype=torch.uint8, device=DEV)
    sc = torch.zeros((m, n // 32), dtype=torch.uint8, device=DEV)
    ops.DynamicQuantMxfp4(dst, sc, to_dev(xs, srcT))
    assert np.array_equal(sc.cpu().numpy(), want_sc)
    assert np.array_equal(dst.cpu().numpy(), want_codes)


@pytest.mark.parametrize("srcT", [O.F16, O.BF16, O.F32])
def test_dynamic_quant_mxfp4_edge_blocks(srcT):
    """Blocks with NaN / infinity (scale 0xFF, codes 0), the largest and smallest magnitudes of the source type
    (exponent clamps, two-step scaling), signed zeros, and values on the rounding ties of E2M1."""
    rng = np.random.default_rng(17 + srcT)
    m, n = 64, 256
    x = rng.standard_normal((m, n)).astype(np.float32)
    big = {O.F16: 6.0e4, O.BF16: 3.0e38, O.F32: 3.0e38}[srcT]
    tiny = {O.F16: 6.0e-8, O.BF16: 1.0e-38, O.F32: 1.0e-38}[srcT]
    x[0, 5] = np.nan
    x[1, 40] = np.inf
    x[2, 70] = -np.inf
    x[3, :32] = big * rng.uniform(-1, 1, 32)
    x[4, :32] = tiny * rng.uniform(-1, 1, 32)
    x[5, :32] = tiny * 1e-3 * rng.uniform(-1, 1, 32)          # subnormal (float, bfloat16) or zero (half)
    x[6, :32] = -0.0
    x[7, :32] = 0.0
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, 7.99, 0.2499, 0.2501], np.float32)
    for r, sc in enumerate((1.0, 2.0 ** -20, 2.0 ** 30, 2.0 ** -100 if srcT != O.F16 else 2.0 ** -12)):
        row = 8 + r
        x[row, :32] = 0.0
        x[row, 0] = 7.5 * sc                                   # fixes the block's exponent: 2^e = sc
        x[row, 1:1 + len(ties)] = ties * sc
        x[row, 16:16 + len(ties)] = -ties * sc
    if srcT == O.F16:
        with np.errstate(over="ignore"):
            xs = x.astype(np.float16)
    elif srcT == O.BF16:
        xs = O.f32_to_bf16_bits(x)
    else:
        xs = x
    want_codes, want_sc = O.dynamic_quant_mxfp4(xs, srcT, m, n)
    assert want_sc[0, 0] == 0xFF and want_sc[1, 1] == 0xFF and want_sc[2, 2] == 0xFF
    dst = torch.full((m, n // 2), 0x5A, dtype=torch.uint8, device=DEV)
    sc = torch.full((m, n // 32), 0x5A, dtype=torch.uint8, device=DEV)
    ops.DynamicQuantMxfp4(dst, sc, to_dev(xs, srcT))
    assert np.array_equal(sc.cpu().numpy(), want_sc)
    got = dst.cpu().numpy()
    bad = np.argwhere(got != want_codes)
    assert bad.size == 0, f"first difference at {bad[0]}: got {got[tuple(bad[0])]:#x} want {want_codes[tuple(bad[0])]:#x}"


def test_dynamic_quant_mxfp4_feeds_the_grouped_matmul():
    """bf16 activations -> ascq_dynamic_quant_mxfp4 -> ascq_group_matmul_mxfp4 reproduces the oracle run on the same
    quantised operands, and stays close to the unquantised product."""
    rng = np.random.default_rng(3)
    groups, N, K = [96, 160], 256, 512
    M = sum(groups)
    x = O.f32_to_bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    B = rng.integers(0, 256, (2, N, K // 2)).astype(np.uint8)
    sB = (127 + rng.integers(-2, 3, (2, N, K // 32))).astype(np.uint8)
    dA = torch.zeros((M, K // 2), dtype=torch.uint8, device=DEV)
    dsA = torch.zeros((M, K // 32), dtype=torch.uint8, device=DEV)
    ops.DynamicQuantMxfp4(dA, dsA, to_dev(x, O.BF16))
    C = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    ops.GroupMatmulMxfp4(C, dA, dsA, torch.from_numpy(B).to(DEV), torch.from_numpy(sB).to(DEV), groups, K, N)
    ops.MatmulStatus()
    _, want = O.group_matmul_mxfp4(dA.cpu().numpy(), dsA.cpu().numpy(), B, sB, np.array(groups, np.int64), K, N, want_f32=True)
    got = C.float().cpu().numpy()
    assert (np.abs(got - want) <= 1e-2 * np.abs(want) + 1e-3 * np.abs(want).max()).all()
