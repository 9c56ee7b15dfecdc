"""Pins the CPU oracle: conversion helpers against the worked examples of the reference's
precision_conversion.md, operators against the fixtures generated from the reference's example
gen_data.py scripts (tests/golden/make_golden.py), tmp-size formulas against the known answers of
tests/api/adv_api/tiling/test_tiling.cpp:6540-6712.  CPU only."""
import os

import numpy as np
import pytest

from oracle import oracle as O

L = O.lib()
h = lambda x: int(np.float16(x).view(np.uint16))  # noqa: E731


# ---- docs/zh/api/SIMD-API/基础API/数据结构/precision_conversion.md worked examples ----------------
def test_half_to_int8_examples():
    # :242-248  input 2^7 - 0.5
    x = h(127.5)
    assert L.orc_f16_to_i8(x, O.CAST_RINT) == 127     # rounds to 128, saturates
    assert L.orc_f16_to_i8(x, O.CAST_FLOOR) == 127
    assert L.orc_f16_to_i8(x, O.CAST_CEIL) == 127
    assert L.orc_f16_to_i8(x, O.CAST_ROUND) == 127
    assert L.orc_f16_to_i8(x, O.CAST_TRUNC) == 127
    assert L.orc_f16_to_i8(h(-200.0), O.CAST_RINT) == -128
    assert [L.orc_f16_to_i8(h(v), O.CAST_RINT) for v in (0.5, 1.5, 2.5, -0.5, -1.5)] == [0, 2, 2, 0, -2]
    assert [L.orc_f16_to_i8(h(v), O.CAST_ROUND) for v in (0.5, 1.5, 2.5, -0.5, -1.5)] == [1, 2, 3, -1, -2]


def test_float_to_int16_examples():
    # :506-518  input 2^22 + 0.5 saturates in every mode
    for mode in (O.CAST_RINT, O.CAST_FLOOR, O.CAST_CEIL, O.CAST_ROUND, O.CAST_TRUNC):
        assert L.orc_f32_to_i16(2.0 ** 22 + 0.5, mode) == 2 ** 15 - 1
    # half -> int16 example :281-294 (same rounding rules): 2^7 - 0.5
    assert L.orc_f32_to_i16(127.5, O.CAST_RINT) == 128
    assert L.orc_f32_to_i16(127.5, O.CAST_FLOOR) == 127
    assert L.orc_f32_to_i16(127.5, O.CAST_CEIL) == 128
    assert L.orc_f32_to_i16(127.5, O.CAST_ROUND) == 128
    assert L.orc_f32_to_i16(127.5, O.CAST_TRUNC) == 127


def test_int32_to_float_example():
    # :427-440  2^25 + 3 -> 2^25 + 4 under RINT
    assert L.orc_i32_to_f32(2 ** 25 + 3) == float(2 ** 25 + 4)


def test_float_to_half_and_bf16_examples():
    # :520-539  0.5 + 2^-12 -> 0.5 under RINT
    assert L.orc_f32_to_f16_sat(0.5 + 2.0 ** -12) == h(0.5)
    # :541-555  0.5 + 2^-9 + 2^-11 -> 0.5 + 2^-8 under RINT
    got = L.orc_f32_to_bf16_sat(0.5 + 2.0 ** -9 + 2.0 ** -11)
    assert O.bf16_bits_to_f32(np.array([got], np.uint16))[0] == np.float32(0.5 + 2.0 ** -8)
    # overflow saturates (:30)
    assert L.orc_f32_to_f16_sat(1.0e6) == h(65504.0)
    assert L.orc_f32_to_f16_sat(-1.0e6) == h(-65504.0)


def test_bf16_to_e2m1_example():
    # :331-343  input 2.5
    code = {2.0: 4, 3.0: 5}
    assert L.orc_f32_to_e2m1(2.5, O.CAST_RINT) == code[2.0]
    assert L.orc_f32_to_e2m1(2.5, O.CAST_FLOOR) == code[2.0]
    assert L.orc_f32_to_e2m1(2.5, O.CAST_CEIL) == code[3.0]
    assert L.orc_f32_to_e2m1(2.5, O.CAST_ROUND) == code[3.0]
    assert L.orc_f32_to_e2m1(2.5, O.CAST_TRUNC) == code[2.0]
    assert L.orc_f32_to_e2m1(100.0, O.CAST_RINT) == 7 and L.orc_f32_to_e2m1(-100.0, O.CAST_RINT) == 15
    vals = [L.orc_e2m1_to_f32(c) for c in range(16)]
    assert vals == [0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6]


def test_e8m0_special_cases():
    # impl/adv_api/detail/quantization/antiquant/ascend_antiquant_3510_impl.h:71-74
    assert L.orc_e8m0_to_bf16(0x00) == 0x0040
    assert L.orc_e8m0_to_bf16(0xFF) == 0x7FFF
    assert L.orc_e8m0_to_bf16(127) == 0x3F80  # 1.0
    assert O.bf16_bits_to_f32(np.array([L.orc_e8m0_to_bf16(0)], np.uint16))[0] == np.float32(2.0 ** -127)


def test_half_arithmetic_matches_ieee():
    rng = np.random.default_rng(7)
    a = rng.integers(0, 65536, 20000).astype(np.uint16)
    b = rng.integers(0, 65536, 20000).astype(np.uint16)
    with np.errstate(all="ignore"):
        mul = (a.view(np.float16) * b.view(np.float16))
        add = (a.view(np.float16) + b.view(np.float16))
    gm = np.array([L.orc_f16_mul(int(x), int(y)) for x, y in zip(a, b)], np.uint16)
    ga = np.array([L.orc_f16_add(int(x), int(y)) for x, y in zip(a, b)], np.uint16)
    ok = ~np.isnan(mul)
    assert np.array_equal(gm[ok], mul.view(np.uint16)[ok])
    ok = ~np.isnan(add)
    assert np.array_equal(ga[ok], add.view(np.uint16)[ok])


# ---- fixtures generated from the reference's gen_data.py scripts ---------------------------------
def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name + ".npz"))


def test_quant_sample_golden_dav2201(golden_dir):
    # quant.asc: AscendQuant<float>(dst, src, scale=2.0, offset=0.9, 1024); golden computed in fp16
    g = _load(golden_dir, "quant_dav2201")
    out = O.ascend_quant(g["input"], O.F32, policy=O.PER_TENSOR, scaleScalar=2.0, offsetScalar=0.9)
    assert np.array_equal(out, g["golden"])


def test_quant_sample_golden_dav3510(golden_dir):
    # 950-series sample computes in fp32 (Quantize API); the PER_TOKEN float path is the same arithmetic
    g = _load(golden_dir, "quant_dav3510")
    src = g["input"].reshape(1, -1)
    out = O.ascend_quant(src, O.F32, policy=O.PER_TOKEN, m=1, n=src.size, scale=np.array([2.0], np.float32),
                         offset=np.array([0.9], np.float32), scaleT=O.F32, hasOffset=True)
    assert np.array_equal(out.reshape(-1), g["golden"])


def test_dequant_sample_golden(golden_dir):
    # dequant.asc:139  AscendDequant(dst float, src int32, deqScale float, {128, 32, 32})
    g = _load(golden_dir, "dequant")
    out = O.ascend_dequant(g["input"], O.I32, O.F32, policy=O.PER_CHANNEL, m=128, n=32, calCount=32,
                           scale=g["scale"], scaleT=O.F32)
    assert np.array_equal(out.view(np.uint32), g["golden"].view(np.uint32))


def test_antiquant_sample_golden_dav2201(golden_dir):
    # AscendAntiQuant<int8, half, false>: half add, half multiply
    g = _load(golden_dir, "antiquant_dav2201")
    out = O.ascend_antiquant(g["input_src"], O.I8, O.F16, policy=O.PER_CHANNEL, m=8, n=128,
                             scale=g["input_scale"].reshape(-1), offset=g["input_offset"].reshape(-1), scaleT=O.F16)
    assert np.array_equal(out.view(np.uint16), g["golden"].view(np.uint16))


def test_antiquant_sample_golden_dav3510(golden_dir):
    # 950-series golden: fp32 add, fp32 multiply, cast to half == policy path with scaleT=float, dst=half
    g = _load(golden_dir, "antiquant_dav3510")
    out = O.ascend_antiquant(g["input_src"], O.I8, O.F16, policy=O.PER_TOKEN, m=8, n=128, isTranspose=True,
                             scale=g["input_scale"].reshape(-1).astype(np.float32),
                             offset=g["input_offset"].reshape(-1).astype(np.float32), scaleT=O.F32, hasOffset=True)
    assert np.array_equal(out.view(np.uint16), g["golden"].view(np.uint16))


# ---- the unified interface, which the 950-series samples call ---------------------------------------
def test_quantize_sample_golden_dav3510(golden_dir):
    # quant.asc:113-130: Quantize<{PER_TENSOR, hasOffset, CAST_RINT, 1}>(dst, src float, 2.0f, 0.9f, {1, 1024, 0})
    g = _load(golden_dir, "quant_dav3510")
    out = O.quantize(g["input"], O.F32, policy=O.PER_TENSOR, m=1, n=1024, scaleScalar=2.0, offsetScalar=0.9, hasOffset=True)
    assert np.array_equal(out.reshape(-1), g["golden"])


def test_antiquantize_sample_golden_dav3510(golden_dir):
    # antiquant.asc:159-175: AntiQuantize<{PER_CHANNEL, hasOffset}>(dst half, src int8, scale half[128], offset, {8, 128, 0})
    g = _load(golden_dir, "antiquant_dav3510")
    out = O.antiquantize(g["input_src"], O.I8, O.F16, policy=O.PER_CHANNEL, m=8, n=128, scale=g["input_scale"].reshape(-1),
                         offset=g["input_offset"].reshape(-1), scaleT=O.F16, hasOffset=True)
    assert np.array_equal(out.view(np.uint16), g["golden"].view(np.uint16))
    # the fp32 intermediates matter: the half-arithmetic legacy operator gives other bits on the same inputs
    legacy = O.ascend_antiquant(g["input_src"], O.I8, O.F16, policy=O.PER_CHANNEL, m=8, n=128,
                                scale=g["input_scale"].reshape(-1), offset=g["input_offset"].reshape(-1), scaleT=O.F16)
    assert not np.array_equal(legacy.view(np.uint16), g["golden"].view(np.uint16))


def test_dequantize_sample_golden(golden_dir):
    # dequant.asc:142-152: Dequantize<{PER_CHANNEL, false, 1}>(dst float, src int32, scale float[32], offset, {128, 32, 0})
    g = _load(golden_dir, "dequant")
    out = O.dequantize(g["input"], O.I32, O.F32, policy=O.PER_CHANNEL, m=128, n=32, scale=g["scale"], scaleT=O.F32)
    assert np.array_equal(out.view(np.uint32), g["golden"].view(np.uint32))


def test_quantize_equals_policy_operator_where_both_compute_in_fp32():
    rng = np.random.default_rng(9)
    src = rng.normal(0, 3, (16, 64)).astype(np.float16)
    sc = rng.uniform(1, 20, 16).astype(np.float32)
    of = rng.uniform(-3, 3, 16).astype(np.float32)
    for mode in (O.CAST_RINT, O.CAST_FLOOR, O.CAST_CEIL, O.CAST_ROUND, O.CAST_TRUNC):
        a = O.quantize(src, O.F16, policy=O.PER_TOKEN, m=16, n=64, scale=sc, offset=of, scaleT=O.F32, hasOffset=True, roundMode=mode)
        b = O.ascend_quant(src, O.F16, policy=O.PER_TOKEN, m=16, n=64, scale=sc, offset=of, scaleT=O.F32, hasOffset=True, roundMode=mode)
        assert np.array_equal(a, b)


# ---- int8 matmul with the fixpipe quantisation of the result (matmul_quant sample) ---------------------
@pytest.mark.parametrize("name", ["matmul_quant_scalar", "matmul_quant_vector"])
def test_matmul_quant_sample_golden(golden_dir, name):
    # matmul_quant.asc:113-117 SetQuantVector / SetQuantScalar(0.1); golden by the sample's gen_data.py (-m 0 / -m 1);
    # the fixture keeps the first 96 rows of A and of the golden
    g = _load(golden_dir, name)
    qv = g["quant_vector_gm"] if "quant_vector_gm" in g else None
    out = O.matmul_i8_quant(g["x1_gm"], np.ascontiguousarray(g["x2_gm"].T), g["bias_gm"], qv, 0.1)
    assert np.array_equal(out.view(np.uint16), g["golden"].view(np.uint16))


# ---- int8 matmul with the fixpipe requantisation to int8 / uint8 (fixpipe_l0c2gm sample, (V)REQ8) --------
def test_fixpipe_req8_values_golden(golden_dir):
    # fixpipe_l0c2gm/scripts/gen_data_s322s8.py:75-97 (req8_pre) called value by value when the fixture was made:
    # ties, offsets, both result types, the shift mode, scales with a zero exponent field
    g = _load(golden_dir, "fixpipe_req8_values")
    got = np.array([O.req8(d, q) for d, q in zip(g["data"], g["quant_pre"])], np.int16)
    assert np.array_equal(got, g["golden"])


def test_fixpipe_req8_matmul_sample_golden(golden_dir):
    # gen_data_s322s8.py:147-175 with vector parameters, no ReLU, row-major output; B stored [K, N]
    g = _load(golden_dir, "fixpipe_req8_matmul")
    out = O.matmul_i8_requant(g["x1_gm"], np.ascontiguousarray(g["x2_gm"].T), None, g["quant_pre"])
    assert np.array_equal(out.view(np.int8), g["golden"])
    # the scalar form with the same word gives the same matrix
    out2 = O.matmul_i8_requant(g["x1_gm"], np.ascontiguousarray(g["x2_gm"].T), None, None, int(g["quant_pre"][0]))
    assert np.array_equal(out2, out)


def test_fixpipe_qf322b8_values_golden(golden_dir):
    # fixpipe_l0c2gm/scripts/gen_data_f322s8.py:75-97 (qf322b8_pre) called value by value when the fixture was made
    g = _load(golden_dir, "fixpipe_qf322b8_values")
    got = np.array([O.qf322b8(d, q) for d, q in zip(g["data"], g["quant_pre"])], np.int16)
    assert np.array_equal(got, g["golden"])


def test_fixpipe_qf322b8_matmul_sample_golden(golden_dir):
    # gen_data_f322s8.py:136-165: half operands, fp32 matmul by numpy, vector parameters (scale 2, int8), no ReLU.
    # The oracle sums in double and rounds once; numpy sums in fp32, so a value within rounding distance of a tie
    # may come out one step away: at most 1 apart, and almost never.
    g = _load(golden_dir, "fixpipe_qf322b8_matmul")
    out = O.matmul_f16_quant(g["x1_gm"], np.ascontiguousarray(g["x2_gm"].T), O.F16, g["quant_pre"]).view(np.int8)
    diff = np.abs(out.astype(np.int32) - g["golden"].astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3, (diff.max(), (diff != 0).mean())


# ---- MX matmul with fp8 operands (matmul_mx and mmad_mx samples) --------------------------------------
def test_matmul_mx_sample_golden(golden_dir):
    # matmul_mx/scripts/gen_data.py: e5m2 x e5m2, m=32 n=k=128, B stored [K,N], scaleB stored [sk/2, n, 2]
    g = _load(golden_dir, "matmul_mx_e5m2")
    B_nk = np.ascontiguousarray(g["x2_gm"].T)
    sB = np.ascontiguousarray(g["x2_mx_gm"].transpose(1, 0, 2).reshape(128, 4))
    _, out = O.group_matmul_mxfp8(g["x1_gm"], 1, g["x1_mx_gm"], B_nk[None], 1, sB[None], np.array([32]), 128, 128)
    assert np.array_equal(out.view(np.uint32), g["golden"].view(np.uint32))


@pytest.mark.parametrize("scenario,aFmt,bFmt", [(3, 0, 1), (4, 1, 0)])
def test_mmad_mx_sample_golden(golden_dir, scenario, aFmt, bFmt):
    # mmad_mx/scripts/gen_data.py scenario 3 (e4m3 x e5m2, result doubled) and 4 (e5m2 x e4m3, fp32 bias added);
    # m, n, k = 40, 50, 70: K is padded with zero codes to the next multiple of 128, as the scale arrays already are
    g = _load(golden_dir, f"mmad_mx_scenario{scenario}")
    A = np.zeros((40, 128), np.uint8)
    A[:, :70] = g["x1_gm"]
    B = np.zeros((50, 128), np.uint8)
    B[:, :70] = g["x2_gm"]
    _, out = O.group_matmul_mxfp8(A, aFmt, g["x1_scale_gm"], B[None], bFmt, g["x2_scale_gm"][None], np.array([40]), 128, 50)
    want = out * np.float32(2) if scenario == 3 else out + g["bias_gm"]
    assert np.array_equal(want.view(np.uint32), g["golden"].view(np.uint32))


def test_fp8_decode_matches_ml_dtypes():
    ml_dtypes = pytest.importorskip("ml_dtypes")
    codes = np.arange(256, dtype=np.uint8)
    for fmt, dt in ((0, ml_dtypes.float8_e4m3fn), (1, ml_dtypes.float8_e5m2)):
        want = codes.view(dt).astype(np.float64)
        A = codes.reshape(2, 128)
        ones = np.full((2, 4), 127, np.uint8)
        # one-hot B rows pick out every decoded value: B[n] has 1.0 at k = n
        one = {0: 0x38, 1: 0x3C}[fmt]
        B = np.zeros((128, 128), np.uint8)
        B[np.arange(128), np.arange(128)] = one
        _, out = O.group_matmul_mxfp8(A, fmt, ones, B[None], fmt, np.full((1, 128, 4), 127, np.uint8), np.array([2]), 128, 128)
        got = out.reshape(-1).astype(np.float64)
        ok = (got == want) | (np.isnan(got) & np.isnan(want))
        # a NaN operand poisons its whole row of sums: compare only rows without NaN codes exactly, NaN rows as NaN
        for r in range(2):
            rowcodes = want[r * 128:(r + 1) * 128]
            if np.isnan(rowcodes).any():
                assert np.isnan(got[r * 128:(r + 1) * 128]).all()
            else:
                assert ok[r * 128:(r + 1) * 128].all()


# ---- dynamic MX-FP4 block quantiser (build-defined front end) -----------------------------------------
def test_dynamic_quant_mxfp4_matches_an_independent_restatement():
    ml_dtypes = pytest.importorskip("ml_dtypes")
    rng = np.random.default_rng(17)
    m, n = 24, 256
    x = (rng.standard_normal((m, n)) * np.exp2(rng.integers(-12, 12, (m, n // 32)).repeat(32, axis=1))).astype(np.float32)
    x[3, 32:64] = 0.0                                   # an all-zero block
    codes, sc = O.dynamic_quant_mxfp4(x, O.F32, m, n)
    xb = x.reshape(m, n // 32, 32)
    amax = np.abs(xb).max(axis=2)
    e = np.where(amax > 0, np.floor(np.log2(np.where(amax > 0, amax, 1.0))) - 2, 0).astype(np.int64)
    assert np.array_equal(sc.astype(np.int64), e + 127)
    y = (xb.astype(np.float64) * np.exp2(-e)[:, :, None]).astype(np.float32).astype(ml_dtypes.bfloat16).astype(np.float32)
    want = y.astype(ml_dtypes.float4_e2m1fn).view(np.uint8).reshape(m, n) & 0xF       # RINT, saturating at +-6
    got = np.stack([codes & 0xF, codes >> 4], axis=2).reshape(m, n)
    assert np.array_equal(got, want)
    # what the block decodes to stays within 2 * 2^e of the input: amax / 2^e lies in [4, 8), values above 6 saturate
    mags = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6])
    deq = mags[got].reshape(m, n // 32, 32) * np.exp2(e)[:, :, None]
    assert (np.abs(deq - xb) <= np.exp2(e)[:, :, None] * 2.0 + 1e-30).all()


# ---- tests/api/adv_api/tiling/test_tiling.cpp:6540-6712 known answers -----------------------------
TILING_ANTIQUANT = [
    # srcDims, scaleDims, transpose, outT, (max, min), (live, extra)
    ((640, 5120), (1, 5120), False, O.F16, (0, 0), (0, 0)),
    ((640, 5120), (1, 5120), False, O.BF16, (5120 * 2 * 4 + 64 * 640 * 4,) * 2, (0, 5120 * 2 * 4 + 64 * 640 * 4)),
    ((640, 5120), (1,), False, O.BF16, (640 * 5120 * 4, 1024), (1, 0)),
    ((64, 512), (64, 1), True, O.BF16, (80 * 64 * 4, 80 * 64 * 4), (0, 80 * 64 * 4)),
    ((640, 5120), (1,), True, O.BF16, (640 * 5120 * 4, 1024), (1, 0)),
]


def tiling_known_answers(quant_sz, quant_f, deq_sz, deq_f, aq_sz, aq_f):
    assert quant_sz([512], 2) == (2 * 512, 2 * 256)
    assert quant_f() == (2, 0)
    assert deq_sz([10, 32], 4) == (4 * (64 + 32 * 10 + 40), 4 * (64 + 32 + 40))
    assert deq_f([10, 32]) == (1, 104)
    assert deq_sz([320], 4) == (4 * (64 + 320 + 328),) * 2
    assert deq_f([320]) == (2, 72)
    assert deq_f([10, 32, 3]) == (0, 0)
    for src, sc, tr, outT, sizes, factor in TILING_ANTIQUANT:
        assert aq_sz(src, sc, tr, O.I8, outT) == sizes, (src, sc, tr)
        assert aq_f(src, sc, tr, O.I8, outT) == factor, (src, sc, tr)


def test_tiling_known_answers_oracle():
    tiling_known_answers(O.quant_tmp_size, O.quant_factor, O.dequant_tmp_size, O.dequant_factor,
                         O.antiquant_tmp_size, O.antiquant_factor)


# ---- independent numpy / ml_dtypes restatement of the benchmark configurations (reduced sizes) ------
def test_cfg1_per_tensor_fp16_formula():
    x = np.random.default_rng(20251126).standard_normal((64, 4096)).astype(np.float16)
    out = O.ascend_quant(x, O.F16, policy=O.PER_TENSOR, scaleScalar=64.0, offsetScalar=0.0)
    ref = np.clip(np.rint(x.astype(np.float32) * 64.0), -128, 127).astype(np.int8)
    assert np.array_equal(out, ref)
    assert 0.02 < np.mean((out == 127) | (out == -128)) < 0.08  # the clamp is exercised


def test_cfg2_antiquant_bf16_formula():
    ml_dtypes = pytest.importorskip("ml_dtypes")
    rng = np.random.default_rng(20251127)
    K, N = 96, 1024
    w = rng.integers(-127, 128, (K, N)).astype(np.int8)
    scale = rng.uniform(0.001, 0.02, N).astype(np.float32).astype(ml_dtypes.bfloat16)
    offset = rng.uniform(-4, 4, N).astype(np.float32).astype(ml_dtypes.bfloat16)
    ref = ((w.astype(np.float32) + offset.astype(np.float32)) * scale.astype(np.float32)).astype(ml_dtypes.bfloat16)
    out = O.ascend_antiquant(w, O.I8, O.BF16, policy=O.PER_CHANNEL, m=K, n=N, scale=scale.view(np.uint16),
                             offset=offset.view(np.uint16), scaleT=O.BF16)
    assert np.array_equal(out, ref.view(np.uint16))


def test_cfg3_dequant_channel_token_formula():
    ml_dtypes = pytest.importorskip("ml_dtypes")
    rng = np.random.default_rng(20251128)
    M, N = 64, 512
    acc = rng.integers(-2 ** 20, 2 ** 20 + 1, (M, N)).astype(np.int32)
    sch = rng.uniform(1e-5, 1e-3, N).astype(np.float32)
    stok = rng.uniform(0.5, 2.0, M).astype(np.float32)
    ref = ((acc.astype(np.float32) * sch[None, :]) * stok[:, None]).astype(ml_dtypes.bfloat16)
    out = O.ascend_dequant(acc, O.I32, O.BF16, policy=O.PER_CHANNEL, m=M, n=N, calCount=N, scale=sch, tokScale=stok,
                           scaleT=O.F32)
    assert np.array_equal(out, ref.view(np.uint16))


def test_w8a8_matches_numpy():
    ml_dtypes = pytest.importorskip("ml_dtypes")
    rng = np.random.default_rng(20251129)
    M, N, K = 48, 80, 256
    A = np.clip(np.rint(rng.normal(0, 30, (M, K))), -127, 127).astype(np.int8)
    B = rng.integers(-127, 128, (N, K)).astype(np.int8)
    sA = rng.uniform(0.005, 0.02, M).astype(np.float32)
    sB = rng.uniform(0.001, 0.01, N).astype(np.float32)
    bias = rng.normal(0, 0.1, N).astype(np.float32).astype(ml_dtypes.bfloat16)
    C, acc = O.matmul_w8a8(A, B, sA, sB, bias.view(np.uint16), want_acc=True)
    ref_acc = A.astype(np.int64) @ B.astype(np.int64).T
    assert np.array_equal(acc, ref_acc.astype(np.int32))
    ref = (((ref_acc.astype(np.float32) * sB[None, :]) * sA[:, None]) + bias.astype(np.float32)[None, :])
    assert np.array_equal(C, ref.astype(ml_dtypes.bfloat16).view(np.uint16))


def test_mxfp4_matches_reference_golden_formula():
    # the golden of examples/.../matmul_mxfp4_high_performance/scripts/gen_data.py:52-63, restated with ml_dtypes
    ml_dtypes = pytest.importorskip("ml_dtypes")
    rng = np.random.default_rng(20251130)
    M, N, K = 24, 40, 128
    a_codes = rng.integers(0, 16, (M, K)).astype(np.uint8)
    b_codes = rng.integers(0, 16, (N, K)).astype(np.uint8)
    sA = (127 + rng.integers(-4, 5, (M, K // 32))).astype(np.uint8)
    sB = (127 + rng.integers(-4, 5, (N, K // 32))).astype(np.uint8)
    lut = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], np.float64)
    a_full = lut[a_codes] * np.repeat(2.0 ** (sA.astype(np.float64) - 127), 32, axis=1)
    b_full = lut[b_codes] * np.repeat(2.0 ** (sB.astype(np.float64) - 127), 32, axis=1)
    golden = (a_full @ b_full.T).astype(np.float32).astype(ml_dtypes.bfloat16)
    pack = lambda c: (c[:, 0::2] | (c[:, 1::2] << 4)).astype(np.uint8)  # noqa: E731  element 2i in the low nibble
    out = O.group_matmul_mxfp4(pack(a_codes), sA, pack(b_codes)[None], sB[None], np.array([M], np.int64), K, N)
    assert np.array_equal(out, golden.view(np.uint16))


def test_group_matmul_w8a8_vs_reference_sample_golden(golden_dir):
    """The grouped W8A8 sample's own golden (quant_group_matmul_high_performance/scripts/gen_data.py run unmodified; 16
    rows of each of the 8 groups, 128 columns kept).  The sample multiplies the two scales with each other first and
    uses the overflow-safe form of FastGelu, the operator multiplies one after the other (quant_group_matmul_custom.asc:
    433-441) and divides by 1 + exp(-1.702 x): the results agree within one half-precision step, and far inside the
    sample's own acceptance rule (rtol = atol = 1e-3, at most 1e-4 of the elements outside: scripts/verify_result.py)."""
    d = np.load(os.path.join(golden_dir, "quant_group_matmul.npz"))
    B = np.ascontiguousarray(d["weight_gkn"].transpose(0, 2, 1))      # [G, K, N] as the sample draws it -> [G, N, K]
    got, acc = O.group_matmul_w8a8(d["x"], B, d["perTokenScale"], d["scale"], d["groupList"], act=True, want_acc=True)
    gold = d["golden"]
    starts = np.concatenate([[0], np.cumsum(d["groupList"])])
    for g in range(len(d["groupList"])):   # int32 accumulators: exact
        r = slice(int(starts[g]), int(starts[g + 1]))
        assert np.array_equal(acc[r], d["x"][r].astype(np.int32) @ d["weight_gkn"][g].astype(np.int32))
    outside = ~np.isclose(got.astype(np.float32), gold.astype(np.float32), rtol=1e-3, atol=1e-3)
    assert outside.mean() <= 1e-4
    steps = np.abs(got.view(np.int16).astype(np.int32) - gold.view(np.int16).astype(np.int32))
    assert steps.max() <= 1 and (steps != 0).mean() < 1e-3
    # without the activation and with the scales multiplied in the operator's order the result is exact
    plain = O.group_matmul_w8a8(d["x"], B, d["perTokenScale"], d["scale"], d["groupList"], act=False)
    want = np.empty_like(plain)
    for g in range(len(d["groupList"])):
        r = slice(int(starts[g]), int(starts[g + 1]))
        want[r] = ((acc[r].astype(np.float32) * d["scale"][g][None, :]) * d["perTokenScale"][r][:, None]).astype(np.float16)
    assert np.array_equal(plain.view(np.uint16), want.view(np.uint16))
