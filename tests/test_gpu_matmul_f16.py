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
@pytest.mark.parametrize("tile", ["pair", "wide", "narrow", "slim"])
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
@pytest.mark.parametrize("tile", ["pair", "wide", "narrow", "slim"])
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


# ---- at most 32 activation rows: the weight is converted in registers on its way to the tensor cores -------------------

def _w8a16_case(rng, M, N, K, abT, per_channel, with_offset):
    A = rand_float(rng, (M, K), abT, -1, 1)
    B = rng.integers(-128, 128, (N, K), dtype=np.int8)
    if per_channel:
        sc_h = rand_float(rng, (N,), abT, 0.002, 0.02)
        of_h = rand_float(rng, (N,), abT, -4, 4) if with_offset else None
        return A, B, sc_h, of_h, to_dev(sc_h, abT), (to_dev(of_h, abT) if with_offset else None)
    return A, B, 0.0078125, 1.5, 0.0078125, 1.5


@pytest.mark.parametrize("abT,cT", [(O.F16, O.F16), (O.F16, O.F32), (O.BF16, O.BF16), (O.BF16, O.F32)])
@pytest.mark.parametrize("M,N,K", [(1, 512, 256), (4, 64, 128), (7, 516, 384), (8, 4096, 4096), (16, 1000, 1024), (25, 640, 2176), (32, 2048, 1024)])
@pytest.mark.parametrize("per_channel,with_offset", [(True, True), (True, False), (False, True)])
def test_w8a16_few_rows(abT, cT, M, N, K, per_channel, with_offset, monkeypatch):
    """Both forms against the oracle (AscendAntiQuant, then an fp64 matmul), into a pitched output whose guard row and guard
    columns must stay untouched."""
    rng = np.random.default_rng(M + N + K + abT + cT)
    A, B, sc_h, of_h, scale, offset = _w8a16_case(rng, M, N, K, abT, per_channel, with_offset)
    if per_channel:
        W = O.ascend_antiquant(B, O.I8, abT, policy=O.PER_CHANNEL, m=N, n=K, scale=sc_h, offset=of_h, scaleT=abT, isTranspose=True)
        _, want = O.matmul_f16(A, W, abT)
    else:
        (_, want), _ = O.matmul_w8a16(A, abT, B, of_h, sc_h)
    dA, dB = to_dev(A, abT), torch.from_numpy(B).to(DEV)
    outs = {}
    for form in ("small", "twostep"):
        monkeypatch.setenv("ASCQ_W8A16", form)
        C = torch.full((M + 1, N + 8), -1.0, dtype=TDT[cT], device=DEV)   # a pitched output with a guard row and guard columns
        ops.MatmulW8A16(C[:M, :N], dA, dB, offset, scale)
        ops.MatmulStatus()
        full = C.float().cpu().numpy()
        assert (full[M:] == -1.0).all() and (full[:, N:] == -1.0).all(), form
        outs[form] = full[:M, :N]
        close(outs[form], want)


@pytest.mark.parametrize("abT", [O.F16, O.BF16])
@pytest.mark.parametrize("M", [1, 5, 24, 32])
def test_w8a16_few_rows_exact_on_small_integers(abT, M, monkeypatch):
    """Integer activations, scale a power of two, offset 1.5: every product and partial sum is exact in fp32, so the order of
    summation cannot matter and the result must equal the oracle's, and the two-launch form's, bit for bit."""
    rng = np.random.default_rng(70 + M + abT)
    N, K = 768, 512
    A = rng.integers(-4, 5, (M, K)).astype(np.float32)
    A = A.astype(np.float16) if abT == O.F16 else (A.view(np.uint32) >> 16).astype(np.uint16)
    B = rng.integers(-128, 128, (N, K), dtype=np.int8)
    (_, want), _ = O.matmul_w8a16(A, abT, B, 1.5, 0.0078125)
    outs = {}
    for form in ("small", "twostep"):
        monkeypatch.setenv("ASCQ_W8A16", form)
        C = torch.zeros((M, N), dtype=torch.float32, device=DEV)
        ops.MatmulW8A16(C, to_dev(A, abT), torch.from_numpy(B).to(DEV), 1.5, 0.0078125)
        ops.MatmulStatus()
        outs[form] = C.cpu().numpy()
    assert np.array_equal(outs["small"], want.astype(np.float32))
    assert np.array_equal(outs["small"].view(np.uint32), outs["twostep"].view(np.uint32))


def test_w8a16_few_rows_is_the_default_and_leaves_no_weight_behind(monkeypatch):
    """With ASCQ_W8A16 unset, M <= 32 takes the in-register form: the workspace then holds at most fp32 partial sums, not the
    dequantised weight; above 32 rows the two-launch form writes the weight there."""
    monkeypatch.delenv("ASCQ_W8A16", raising=False)
    rng = np.random.default_rng(3)
    N, K = 512, 512
    B = rng.integers(-128, 128, (N, K), dtype=np.int8)
    sc_h, of_h = rand_float(rng, (N,), O.F16, 0.002, 0.02), rand_float(rng, (N,), O.F16, -4, 4)
    W = O.ascend_antiquant(B, O.I8, O.F16, policy=O.PER_CHANNEL, m=N, n=K, scale=sc_h, offset=of_h, scaleT=O.F16, isTranspose=True)
    for M, weight_in_workspace in ((32, False), (33, True)):
        A = rand_float(rng, (M, K), O.F16, -1, 1)
        ws = torch.zeros(N * K * 2, dtype=torch.uint8, device=DEV)
        C = torch.zeros((M, N), dtype=torch.float32, device=DEV)
        ops.MatmulW8A16(C, to_dev(A, O.F16), torch.from_numpy(B).to(DEV), to_dev(of_h, O.F16), to_dev(sc_h, O.F16), workspace=ws)
        ops.MatmulStatus()
        _, want = O.matmul_f16(A, W, O.F16)
        close(C.cpu().numpy(), want)
        same = np.array_equal(ws.view(torch.float16).view(N, K).cpu().numpy().view(np.uint16), W.view(np.uint16))
        assert same == weight_in_workspace, M


@pytest.mark.parametrize("abT", [O.F16, O.BF16])
@pytest.mark.parametrize("with_offset", [True, False])
def test_w8a16_few_rows_reads_the_weight_antiquant_produces(abT, with_offset, monkeypatch):
    """One-hot activation rows copy single weight columns into the fp32 result, so the weight the tensor cores were fed can
    be compared with AscendAntiQuant's output bit for bit -- including, for bfloat16, a row whose scale is so large that
    the product overflows and AscendAntiQuant saturates it."""
    monkeypatch.setenv("ASCQ_W8A16", "small")
    rng = np.random.default_rng(90 + abT + with_offset)
    M, N, K = 32, 528, 384
    B = rng.integers(-128, 128, (N, K), dtype=np.int8)
    sc_h = rand_float(rng, (N,), abT, 0.002, 0.02)
    of_h = rand_float(rng, (N,), abT, -4, 4) if with_offset else None
    if abT == O.BF16:
        # row 17: scale 2^127; with offset 255/256 the weight 1 gives 1.99609375 * 2^127, which is finite in fp32 and rounds to
        # infinity as a bfloat16 -- AscendAntiQuant stores the largest finite bfloat16 there.  The other weights of the row
        # are kept where the fp32 product stays finite.
        sc_h[17] = np.uint16(0x7F00)
        B[17] = rng.integers(-1, 2, K)
        if with_offset:
            of_h[17] = np.uint16(0x3F7F)
    W = O.ascend_antiquant(B, O.I8, abT, policy=O.PER_CHANNEL, m=N, n=K, scale=sc_h, offset=of_h, scaleT=abT, isTranspose=True)
    Wf = W.astype(np.float32) if abT == O.F16 else (W.astype(np.uint32) << 16).view(np.float32)
    assert np.isfinite(Wf).all()
    if abT == O.BF16 and with_offset:
        assert (W[17][B[17] == 1] == 0x7F7F).all() and (B[17] == 1).any()
    cols = rng.choice(K, M, replace=False)
    A = np.zeros((M, K), np.float32)
    A[np.arange(M), cols] = 1.0
    A = A.astype(np.float16) if abT == O.F16 else (A.view(np.uint32) >> 16).astype(np.uint16)
    C = torch.zeros((M, N), dtype=torch.float32, device=DEV)
    ops.MatmulW8A16(C, to_dev(A, abT), torch.from_numpy(B).to(DEV), to_dev(of_h, abT) if with_offset else None, to_dev(sc_h, abT))
    ops.MatmulStatus()
    assert np.array_equal(C.cpu().numpy().view(np.uint32), np.ascontiguousarray(Wf[:, cols].T).view(np.uint32))


# ---- int4b_t weights, at most 32 activation rows --------------------------------------------------------------------------

@pytest.mark.parametrize("abT,cT", [(O.F16, O.F16), (O.BF16, O.BF16), (O.BF16, O.F32)])
@pytest.mark.parametrize("M,N,K", [(1, 512, 256), (7, 516, 384), (8, 4096, 4096), (16, 1000, 1024), (32, 2048, 1024)])
@pytest.mark.parametrize("per_channel,with_offset", [(True, True), (True, False), (False, True)])
def test_w4a16_few_rows(abT, cT, M, N, K, per_channel, with_offset, monkeypatch):
    rng = np.random.default_rng(M + N + K + abT + cT + 5)
    A = rand_float(rng, (M, K), abT, -1, 1)
    B4 = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    if per_channel:
        sc_h = rand_float(rng, (N,), abT, 0.02, 0.2)
        of_h = rand_float(rng, (N,), abT, -2, 2) if with_offset else None
        W = O.ascend_antiquant(B4, O.I4X2, abT, policy=O.PER_CHANNEL, m=N, n=K, scale=sc_h, offset=of_h, scaleT=abT, isTranspose=True)
        scale, offset = to_dev(sc_h, abT), (to_dev(of_h, abT) if with_offset else None)
    else:
        scale, offset = 0.125, 1.5
        W = O.ascend_antiquant(B4, O.I4X2, abT, policy=O.PER_TENSOR, m=N, n=K, scaleScalar=scale, offsetScalar=offset, scaleT=abT,
                               isTranspose=True, hasOffset=True)
    _, want = O.matmul_f16(A, W, abT)
    for form in ("small", "twostep"):
        monkeypatch.setenv("ASCQ_W8A16", form)
        C = torch.full((M + 1, N + 8), -1.0, dtype=TDT[cT], device=DEV)
        ops.MatmulW4A16(C[:M, :N], to_dev(A, abT), torch.from_numpy(B4).to(DEV), offset, scale)
        ops.MatmulStatus()
        full = C.float().cpu().numpy()
        assert (full[M:] == -1.0).all() and (full[:, N:] == -1.0).all(), form
        close(full[:M, :N], want)


@pytest.mark.parametrize("abT", [O.F16, O.BF16])
@pytest.mark.parametrize("with_offset", [True, False])
def test_w4a16_few_rows_reads_the_weight_antiquant_produces(abT, with_offset, monkeypatch):
    """One-hot activation rows copy weight columns into the fp32 result: the int4 weight the tensor cores were fed is
    AscendAntiQuant's output bit for bit, including (bfloat16) a row that takes the saturating path."""
    monkeypatch.setenv("ASCQ_W8A16", "small")
    rng = np.random.default_rng(190 + abT + with_offset)
    M, N, K = 32, 528, 384
    B4 = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    sc_h = rand_float(rng, (N,), abT, 0.02, 0.2)
    of_h = rand_float(rng, (N,), abT, -2, 2) if with_offset else None
    if abT == O.BF16:
        # row 17: scale 2^127 and weights in {-1, 0, 1}; with offset 255/256 the weight 1 gives 1.99609375 * 2^127, finite
        # in fp32 but past the largest bfloat16: AscendAntiQuant stores the largest finite value
        sc_h[17] = np.uint16(0x7F00)
        nib = rng.integers(-1, 2, K) & 0xF
        B4[17] = (nib[0::2] | (nib[1::2] << 4)).astype(np.uint8)
        if with_offset:
            of_h[17] = np.uint16(0x3F7F)
    W = O.ascend_antiquant(B4, O.I4X2, abT, policy=O.PER_CHANNEL, m=N, n=K, scale=sc_h, offset=of_h, scaleT=abT, isTranspose=True)
    Wf = W.astype(np.float32) if abT == O.F16 else (W.astype(np.uint32) << 16).view(np.float32)
    assert np.isfinite(Wf).all()
    if abT == O.BF16 and with_offset:
        assert (W[17] == 0x7F7F).any()
    cols = rng.choice(K, M, replace=False)
    A = np.zeros((M, K), np.float32)
    A[np.arange(M), cols] = 1.0
    A = A.astype(np.float16) if abT == O.F16 else (A.view(np.uint32) >> 16).astype(np.uint16)
    C = torch.zeros((M, N), dtype=torch.float32, device=DEV)
    ops.MatmulW4A16(C, to_dev(A, abT), torch.from_numpy(B4).to(DEV), to_dev(of_h, abT) if with_offset else None, to_dev(sc_h, abT))
    ops.MatmulStatus()
    assert np.array_equal(C.cpu().numpy().view(np.uint32), np.ascontiguousarray(Wf[:, cols].T).view(np.uint32))
