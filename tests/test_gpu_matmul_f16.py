"""GPU parity of the half / bfloat16 matmul (tcgen05 kind::f16) and of the weight-only-quantised matmul built on it
(int8 weight through AscendAntiQuant, then the matmul) against the CPU oracle.  fp32 accumulation on the GPU, fp64 in the
oracle: rtol 1e-2 in general; the dequantised weight itself must match the oracle bit for bit."""
import numpy as np
import pytest
import torch

from asc_devkit_b200 import ops
from oracle import oracle as O
from tests.gpu_util import DEV, rand_float, to_dev, to_host

pytestmark = pytest.mark.gpu
TDT = {O.F16: torch.float16, O.BF16: torch.bfloat16, O.F32: torch.float32}


def close(got, want):
    tol = 1e-2 * np.abs(want) + 2e-3 * np.abs(want).max()
    assert (np.abs(got.astype(np.float64) - want.astype(np.float64)) <= tol).all(), np.abs(got - want).max()


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (300, 520, 264), (257, 384, 1024), (2048, 1024, 512)])
@pytest.mark.parametrize("abT,cT", [(O.F16, O.F16), (O.F16, O.F32), (O.BF16, O.BF16), (O.BF16, O.F32)])
@pytest.mark.parametrize("tile", ["pair", "wide", "narrow"])
def test_matmul_f16(M, N, K, abT, cT, tile, monkeypatch):
    monkeypatch.setenv("ASCQ_W8A8_TILE", tile)
    rng = np.random.default_rng(M + N + K + abT)
    A = rand_float(rng, (M, K), abT, -1, 1)
    B = rand_float(rng, (N, K), abT, -1, 1)
    _, want = O.matmul_f16(A, B, abT)
    C = torch.full((M, N), -1.0, dtype=TDT[cT], device=DEV)
    ops.MatmulF16(C, to_dev(A, abT), to_dev(B, abT))
    ops.MatmulStatus()
    close(C.float().cpu().numpy(), want)


def test_matmul_f16_exact_on_small_integers():
    # integer-valued operands with small sums: every partial sum is exact in fp32 -> bit-exact against the oracle
    rng = np.random.default_rng(5)
    M, N, K = 256, 512, 256
    A = rng.integers(-4, 5, (M, K)).astype(np.float16)
    B = rng.integers(-4, 5, (N, K)).astype(np.float16)
    want16, _ = O.matmul_f16(A, B, O.F16, O.F16)
    C = torch.zeros((M, N), dtype=torch.float16, device=DEV)
    ops.MatmulF16(C, torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV))
    ops.MatmulStatus()
    assert np.array_equal(C.cpu().numpy().view(np.uint16), want16)


@pytest.mark.parametrize("abT", [O.F16, O.BF16])
@pytest.mark.parametrize("M,N,K", [(192, 640, 512), (256, 256, 64), (1000, 1030, 2080), (4096, 2048, 1024)])
@pytest.mark.parametrize("per_channel,with_offset", [(True, True), (True, False), (False, True)])
def test_w8a16_fused_equals_two_launches(abT, M, N, K, per_channel, with_offset, monkeypatch):
    """The converter warps inside the matmul run the AscendAntiQuant arithmetic on every weight tile; the two-launch form
    writes the same weight to a workspace first.  Same tile shape and MMA order on both sides: the outputs must be the
    same bits (and both within tolerance of the oracle)."""
    rng = np.random.default_rng(M + N + K + abT)
    A = rand_float(rng, (M, K), abT, -1, 1)
    B = rng.integers(-128, 128, (N, K), dtype=np.int8)
    if per_channel:
        sc_h = rand_float(rng, (N,), abT, 0.002, 0.02)
        of_h = rand_float(rng, (N,), abT, -4, 4) if with_offset else None
        scale, offset = to_dev(sc_h, abT), (to_dev(of_h, abT) if with_offset else None)
    else:
        sc_h, of_h = 0.0078125, 1.5
        scale, offset = sc_h, of_h
    dA, dB = to_dev(A, abT), torch.from_numpy(B).to(DEV)
    outs = {}
    for mode in ("fused", "twostep"):
        monkeypatch.setenv("ASCQ_W8A16", mode)
        monkeypatch.setenv("ASCQ_W8A8_TILE", "pair")
        C = torch.full((M, N), -1.0, dtype=torch.float32, device=DEV)
        ops.MatmulW8A16(C, dA, dB, offset, scale)
        ops.MatmulStatus()
        outs[mode] = C.cpu().numpy()
    assert np.array_equal(outs["fused"].view(np.uint32), outs["twostep"].view(np.uint32))
    if per_channel:
        W = O.ascend_antiquant(B, O.I8, abT, policy=O.PER_CHANNEL, m=N, n=K, scale=sc_h, offset=of_h, scaleT=abT, isTranspose=True)
        _, want = O.matmul_f16(A, W, abT)
    else:
        (_, want), _ = O.matmul_w8a16(A, abT, B, of_h, sc_h)
    close(outs["fused"], want)


@pytest.mark.parametrize("abT", [O.F16, O.BF16])
@pytest.mark.parametrize("per_channel", [True, False])
def test_matmul_w8a16(abT, per_channel, monkeypatch):
    monkeypatch.delenv("ASCQ_W8A16", raising=False)   # two launches: the dequantised weight can be read back from the workspace
    rng = np.random.default_rng(11 + abT)
    M, N, K = 192, 640, 512
    A = rand_float(rng, (M, K), abT, -1, 1)
    B = rng.integers(-128, 128, (N, K), dtype=np.int8)
    if per_channel:
        sc_h, of_h = rand_float(rng, (N,), abT, 0.002, 0.02), rand_float(rng, (N,), abT, -4, 4)
        scale, offset = to_dev(sc_h, abT), to_dev(of_h, abT)
    else:
        sc_h, of_h = 0.0078125, 1.5
        scale, offset = sc_h, of_h
    (_, want), W = O.matmul_w8a16(A, abT, B, of_h, sc_h)
    ws = torch.zeros(N * K * 2, dtype=torch.uint8, device=DEV)
    C = torch.zeros((M, N), dtype=torch.float32, device=DEV)
    ops.MatmulW8A16(C, to_dev(A, abT), torch.from_numpy(B).to(DEV), offset, scale, workspace=ws)
    ops.MatmulStatus()
    # the dequantised weight the tensor cores read is AscendAntiQuant's output, bit for bit
    assert np.array_equal(to_host(ws.view(TDT[abT]).view(N, K), abT).view(np.uint16), W.view(np.uint16))
    close(C.cpu().numpy(), want)


@pytest.mark.parametrize("abT", [O.F16, O.BF16])
def test_matmul_w4a16(abT):
    """int4b_t weights: AscendAntiQuant's int4 source, then the same matmul."""
    rng = np.random.default_rng(21 + abT)
    M, N, K = 160, 384, 256
    A = rand_float(rng, (M, K), abT, -1, 1)
    B4 = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    sc_h, of_h = rand_float(rng, (N,), abT, 0.02, 0.2), rand_float(rng, (N,), abT, -2, 2)
    W = O.ascend_antiquant(B4, O.I4X2, abT, policy=O.PER_CHANNEL, m=N, n=K, scale=sc_h, offset=of_h, scaleT=abT, isTranspose=True)
    _, want = O.matmul_f16(A, W, abT)
    ws = torch.zeros(N * K * 2, dtype=torch.uint8, device=DEV)
    C = torch.zeros((M, N), dtype=torch.float32, device=DEV)
    ops.MatmulW4A16(C, to_dev(A, abT), torch.from_numpy(B4).to(DEV), to_dev(of_h, abT), to_dev(sc_h, abT), workspace=ws)
    ops.MatmulStatus()
    assert np.array_equal(to_host(ws.view(TDT[abT]).view(N, K), abT).view(np.uint16), W.view(np.uint16))
    close(C.cpu().numpy(), want)


# ---- fixpipe quantisation of the fp32 result to int8 / uint8 ((V)QF322B8_PRE) --------------------------------------
def _quant_words(rng, n, lo, hi, signed=None):
    s = rng.uniform(lo, hi, n).astype(np.float32) * rng.choice([1.0, 1.0, -1.0], n).astype(np.float32)
    w = s.view(np.uint32).astype(np.uint64)
    w |= np.where(rng.random(n) < 0.5, 0, rng.integers(0, 512, n)).astype(np.uint64) << np.uint64(37)
    sg = rng.integers(0, 2, n) if signed is None else np.full(n, int(signed))
    return w | (sg.astype(np.uint64) << np.uint64(46))


def _one_step_apart(got, want, signed_cols):
    """Byte results agree, or differ by one step where the fp32 sums of the two sides round differently at a tie."""
    g = np.where(signed_cols[None, :], got.view(np.int8).astype(np.int32), got.astype(np.int32))
    w = np.where(signed_cols[None, :], want.view(np.int8).astype(np.int32), want.astype(np.int32))
    diff = np.abs(g - w)
    assert diff.max() <= 1 and (diff != 0).mean() < 2e-3, (diff.max(), (diff != 0).mean())


def test_fixpipe_qf322b8_sample_golden_through_the_gpu():
    """The fixpipe sample's fp32 -> int8 case: half operands, vector parameters, no ReLU."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fixpipe_qf322b8_matmul.npz"))
    C = torch.zeros((128, 256), dtype=torch.int8, device=DEV)
    ops.MatmulF16Quant(C, torch.from_numpy(g["x1_gm"]).to(DEV), torch.from_numpy(np.ascontiguousarray(g["x2_gm"].T)).to(DEV),
                       torch.from_numpy(g["quant_pre"].view(np.int64)).to(DEV))
    ops.MatmulStatus()
    _one_step_apart(C.cpu().numpy().view(np.uint8), g["golden"].view(np.uint8), np.ones(256, bool))


@pytest.mark.parametrize("M,N,K,abT,vector", [(128, 128, 64, O.F16, True), (300, 520, 264, O.BF16, True), (257, 384, 1024, O.F16, False),
                                             (2048, 1024, 512, O.BF16, True)])
@pytest.mark.parametrize("tile", ["pair", "wide", "narrow"])
def test_matmul_f16_quant_matches_oracle(M, N, K, abT, vector, tile, monkeypatch):
    monkeypatch.setenv("ASCQ_W8A8_TILE", tile)
    rng = np.random.default_rng(3 * M + N + K + abT)
    A = rand_float(rng, (M, K), abT, -1, 1)
    B = rand_float(rng, (N, K), abT, -1, 1)
    spread = np.sqrt(K) / 3.0  # standard deviation of a result entry
    qv = _quant_words(rng, N, 20.0 / spread, 120.0 / spread) if vector else None
    qs = int(_quant_words(rng, 1, 60.0 / spread, 61.0 / spread, signed=True)[0])
    want = O.matmul_f16_quant(A, B, abT, qv, qs)
    assert len(np.unique(want)) > 100
    C = torch.full((M, N), 77, dtype=torch.uint8, device=DEV)
    ops.MatmulF16Quant(C, to_dev(A, abT), to_dev(B, abT), torch.from_numpy(qv.view(np.int64)).to(DEV) if vector else None, qs)
    ops.MatmulStatus()
    signed = ((qv >> np.uint64(46)) & np.uint64(1)).astype(bool) if vector else np.ones(N, bool)
    _one_step_apart(C.cpu().numpy(), want, signed)
