"""GPU parity of the MX matmul with fp8 operands (tcgen05 kind::mxf8f6f4.block_scale) against the CPU oracle (fp64
accumulation) and against the reference samples' own golden vectors.  The GPU accumulates in fp32: rtol 1e-2 in
general, bit-exact where every partial sum is representable."""
import ctypes
import os

import numpy as np
import pytest
import torch

from asc_devkit_b200 import _lib as L
from asc_devkit_b200 import ops
from oracle import oracle as O
from tests.gpu_util import DEV

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FMT = {0: L.DT_FP8_E4M3, 1: L.DT_FP8_E5M2}
O.lib().orc_fp8_to_f64.restype = ctypes.c_double
O.lib().orc_fp8_to_f64.argtypes = [ctypes.c_uint8, ctypes.c_int]


def finite_codes(fmt):
    c = np.arange(256, dtype=np.uint8)
    if fmt == 0:
        return c[(c & 0x7F) != 0x7F]            # e4m3fn: S.1111.111 is NaN
    return c[(c & 0x7C) != 0x7C]                # e5m2: exponent 11111 is inf / NaN


def make_case(groups, N, K, aFmt, bFmt, seed, exp_span=3, small=False):
    rng = np.random.default_rng(seed)
    sumM, G = int(sum(groups)), len(groups)
    ca, cb = finite_codes(aFmt), finite_codes(bFmt)
    if small:   # magnitudes <= 2 so that fp32 partial sums stay far from overflow and the comparison is about rounding
        ca = ca[np.abs(np.array([O.lib().orc_fp8_to_f64(int(v), aFmt) for v in ca])) <= 2.0]
        cb = cb[np.abs(np.array([O.lib().orc_fp8_to_f64(int(v), bFmt) for v in cb])) <= 2.0]
    A = rng.choice(ca, (sumM, K)).astype(np.uint8)
    B = rng.choice(cb, (G, N, K)).astype(np.uint8)
    sA = (127 + rng.integers(-exp_span, exp_span + 1, (sumM, K // 32))).astype(np.uint8)
    sB = (127 + rng.integers(-exp_span, exp_span + 1, (G, N, K // 32))).astype(np.uint8)
    return A, sA, B, sB


def run(A, aFmt, sA, B, bFmt, sB, groups, K, N, out=torch.float32):
    t = lambda a: torch.from_numpy(a).to(DEV)  # noqa: E731
    C = torch.full((max(int(sum(groups)), 1), N), -1.0, dtype=out, device=DEV)
    ops.GroupMatmulMxfp8(C, t(A), FMT[aFmt], t(sA), t(B), FMT[bFmt], t(sB), groups, K, N)
    ops.MatmulStatus()
    return C[:int(sum(groups))]


@pytest.mark.parametrize("groups,N,K", [([128], 256, 128), ([128], 128, 256), ([100, 0, 300, 129], 384, 384), ([1, 1, 1], 8, 128),
                                        ([257], 1024, 2048)])
@pytest.mark.parametrize("aFmt,bFmt", [(0, 0), (1, 1), (0, 1), (1, 0)])
@pytest.mark.parametrize("tile", ["single", "pair"])
def test_parity(groups, N, K, aFmt, bFmt, tile, monkeypatch):
    monkeypatch.setenv("ASCQ_MXFP4_TILE", tile)
    A, sA, B, sB = make_case(groups, N, K, aFmt, bFmt, sum(groups) + N + K + aFmt * 2 + bFmt, small=True)
    _, want = O.group_matmul_mxfp8(A, aFmt, sA, B, bFmt, sB, np.array(groups, np.int64), K, N)
    got = run(A, aFmt, sA, B, bFmt, sB, groups, K, N).cpu().numpy()
    tol = 1e-2 * np.abs(want) + 1e-3 * np.abs(want).max()
    assert (np.abs(got - want) <= tol).all(), np.abs(got - want).max()
    gotb = run(A, aFmt, sA, B, bFmt, sB, groups, K, N, out=torch.bfloat16).float().cpu().numpy()
    assert (np.abs(gotb - want) <= tol + np.abs(want) / 128).all()


def test_scale_bytes_are_applied_per_32_elements():
    # one-hot A rows (1.0 at k = 32 r) against an all-ones B: the product is exactly sA[r, r] * sB[n, r]
    M, N, K = 64, 256, 2048
    A = np.zeros((M, K), np.uint8)
    A[np.arange(M), 32 * np.arange(M)] = 0x38                    # 1.0 in e4m3
    B = np.full((1, N, K), 0x3C, np.uint8)                        # 1.0 in e5m2
    rng = np.random.default_rng(3)
    sA = (127 + rng.integers(-6, 7, (M, K // 32))).astype(np.uint8)
    sB = (127 + rng.integers(-6, 7, (1, N, K // 32))).astype(np.uint8)
    got = run(A, 0, sA, B, 1, sB, [M], K, N).cpu().numpy().astype(np.float64)
    want = np.exp2(sA[np.arange(M), np.arange(M)].astype(np.float64) - 127)[:, None] * \
        np.exp2(sB[0][:, :M].T.astype(np.float64) - 127)
    assert np.array_equal(got, want)


def test_matmul_mx_sample_golden_through_the_gpu():
    g = np.load(os.path.join(GOLDEN, "matmul_mx_e5m2.npz"))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)  # noqa: E731
    B_nk = torch.empty((128, 128), dtype=torch.int8, device=DEV)
    ops.TransposeI8KnToNk(B_nk, t(g["x2_gm"]).view(torch.int8))              # [K, N] bytes -> [N, K]
    sB = torch.empty((128, 4), dtype=torch.uint8, device=DEV)
    ops.MxRepackScaleB(sB, t(g["x2_mx_gm"]), 4, 128)                          # [sk/2, N, 2] -> [N, sk]
    C = torch.zeros((32, 128), dtype=torch.float32, device=DEV)
    ops.GroupMatmulMxfp8(C, t(g["x1_gm"]), L.DT_FP8_E5M2, t(g["x1_mx_gm"]), B_nk.view(torch.uint8).unsqueeze(0), L.DT_FP8_E5M2,
                         sB.unsqueeze(0), [32], 128, 128)
    ops.MatmulStatus()
    got, want = C.cpu().numpy(), g["golden"]
    assert (np.abs(got - want) <= 1e-3 * np.abs(want) + 1e-4 * np.abs(want).max()).all()


@pytest.mark.parametrize("scenario,aFmt,bFmt", [(3, 0, 1), (4, 1, 0)])
def test_mmad_mx_sample_golden_through_the_gpu(scenario, aFmt, bFmt):
    g = np.load(os.path.join(GOLDEN, f"mmad_mx_scenario{scenario}.npz"))
    A = np.zeros((40, 128), np.uint8)
    A[:, :70] = g["x1_gm"]
    B = np.zeros((1, 50, 128), np.uint8)
    B[0, :, :70] = g["x2_gm"]
    got = run(A, aFmt, g["x1_scale_gm"], B, bFmt, g["x2_scale_gm"][None], [40], 128, 50).cpu().numpy()
    got = got * np.float32(2) if scenario == 3 else got + g["bias_gm"]
    want = g["golden"]
    assert (np.abs(got - want) <= 1e-3 * np.abs(want) + 1e-4 * np.abs(want).max()).all()


def test_invalid_arguments():
    d = torch.zeros(256, dtype=torch.uint8, device=DEV)
    C = torch.zeros((1, 8), dtype=torch.float16, device=DEV)
    with pytest.raises(ops.AscqError):     # fp16 output is not built
        ops.GroupMatmulMxfp8(C, d, L.DT_FP8_E4M3, d, d, L.DT_FP8_E4M3, d, [1], 128, 8)
    C = torch.zeros((1, 8), dtype=torch.float32, device=DEV)
    with pytest.raises(ops.AscqError):     # int8 is not an fp8 type
        ops.GroupMatmulMxfp8(C, d, L.DT_I8, d, d, L.DT_FP8_E4M3, d, [1], 128, 8)
