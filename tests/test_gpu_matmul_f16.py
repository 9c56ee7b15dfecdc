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
