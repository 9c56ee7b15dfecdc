"""GPU parity of the W8A8 matmul: int32 accumulators bit-exact, bf16 epilogue bit-exact (same fp32 operation
order as the oracle), against the CPU oracle and, at full size, against an exact integer reference on the GPU."""
import os

import numpy as np
import pytest
import torch

from asc_devkit_b200 import ops
from oracle import oracle as O
from tests.gpu_util import DEV, assert_bits_equal

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def make_case(M, N, K, seed):
    rng = np.random.default_rng(seed)
    A = np.clip(np.rint(rng.normal(0, 30, (M, K))), -127, 127).astype(np.int8)
    B = rng.integers(-127, 128, (N, K)).astype(np.int8)
    sA = rng.uniform(0.005, 0.02, M).astype(np.float32)
    sB = rng.uniform(0.001, 0.01, N).astype(np.float32)
    bias = O.f32_to_bf16_bits(rng.normal(0, 0.1, N).astype(np.float32))
    return A, B, sA, sB, bias


def run(A, B, sA=None, sB=None, bias=None, ldc=None, want_acc=True):
    M, K = A.shape
    N = B.shape[0]
    ldc = N if ldc is None else ldc
    dC = torch.full((M, ldc), -1.0, dtype=torch.bfloat16, device=DEV)
    dAcc = torch.full((M, N), 123456789, dtype=torch.int32, device=DEV) if want_acc else None
    t = lambda a: None if a is None else torch.from_numpy(a).to(DEV)  # noqa: E731
    dbias = None if bias is None else torch.from_numpy(bias.view(np.int16)).to(DEV).view(torch.bfloat16)
    ops.MatmulW8A8(dC[:, :N] if ldc != N else dC, t(A), t(B), t(sA), t(sB), dbias, dAcc)
    ops.MatmulStatus()
    return dC.view(torch.int16).cpu().numpy().view(np.uint16), (dAcc.cpu().numpy() if want_acc else None)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (128, 128, 256), (256, 512, 512), (384, 256, 1024),
                                   (100, 200, 144), (1, 8, 16), (129, 257, 272), (512, 1024, 4096), (2048, 384, 640)])
def test_parity_small(M, N, K):
    A, B, sA, sB, bias = make_case(M, N, K, M * 31 + N * 7 + K)
    want_C, want_acc = O.matmul_w8a8(A, B, sA, sB, bias, want_acc=True)
    got_C, got_acc = run(A, B, sA, sB, bias)
    assert_bits_equal(got_acc, want_acc, "int32 accumulators")
    assert_bits_equal(got_C, want_C, "bf16 epilogue")


def test_extreme_values_accumulate_exactly():
    # +-127 everywhere: |acc| = K * 16129, the largest magnitude the int32 accumulator sees for this K
    M, N, K = 128, 256, 8192
    A = np.full((M, K), 127, np.int8)
    B = np.full((N, K), -127, np.int8)
    B[::2] = 127
    _, acc = run(A, B)
    want = np.where(np.arange(N) % 2 == 0, K * 16129, -K * 16129).astype(np.int32)
    assert np.array_equal(acc, np.broadcast_to(want, (M, N)))


def test_optional_operands_and_row_stride():
    A, B, sA, sB, bias = make_case(192, 320, 256, 5)
    for kw in (dict(), dict(sA=sA), dict(sB=sB), dict(bias=bias), dict(sA=sA, sB=sB)):
        want = O.matmul_w8a8(A, B, kw.get("sA"), kw.get("sB"), kw.get("bias"))
        got, _ = run(A, B, kw.get("sA"), kw.get("sB"), kw.get("bias"))
        assert_bits_equal(got, want, f"operands {sorted(kw)}")
    # ldc > N: the columns beyond N keep their previous contents
    ldc = 328
    got, _ = run(A, B, sA, sB, bias, ldc=ldc)
    want = O.matmul_w8a8(A, B, sA, sB, bias, ldc=ldc)
    assert_bits_equal(got[:, :320], want[:, :320], "strided C")
    assert (got[:, 320:] == np.array([-1.0], np.float32).view(np.uint32)[0] >> 16).all()


def test_invalid_arguments():
    a = torch.zeros((16, 24), dtype=torch.int8, device=DEV)
    b = torch.zeros((16, 24), dtype=torch.int8, device=DEV)
    c = torch.zeros((16, 16), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ops.AscqError) as e:
        ops.MatmulW8A8(c, a, b)
    assert "multiple of 16" in e.value.message


def test_cfg4_full_size_exact():
    # benchmark config 4 at full size; the integer reference is computed on the GPU in fp64-free exact arithmetic:
    # int8 products summed in float32 blocks of K=256 stay below 2^24 and are therefore exact.
    M = N = K = 4096
    A, B, sA, sB, bias = make_case(M, N, K, 20251125 + 4)
    dA, dB = torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV)
    acc = torch.zeros((M, N), dtype=torch.int32, device=DEV)
    for k0 in range(0, K, 256):
        part = dA[:, k0:k0 + 256].float() @ dB[:, k0:k0 + 256].float().T   # |sum| <= 256*127*127 < 2^24: exact
        acc += part.to(torch.int32)
    got_C, got_acc = run(A, B, sA, sB, bias)
    assert np.array_equal(got_acc, acc.cpu().numpy())
    # epilogue on the exact accumulators with the oracle's scalar order, vectorised in numpy
    f = acc.cpu().numpy().astype(np.float32)
    f = (f * sB[None, :]) * sA[:, None] + O.bf16_bits_to_f32(bias)[None, :]
    assert_bits_equal(got_C, O.f32_to_bf16_bits(f), "cfg4 epilogue")
    # and a row block through the oracle itself
    want_C = O.matmul_w8a8(np.ascontiguousarray(A[:64]), B, sA[:64].copy(), sB, bias)
    assert_bits_equal(got_C[:64], want_C, "cfg4 rows 0..63 vs oracle")


@pytest.mark.parametrize("M,N,K", [(4096, 4096, 128), (2560, 3840, 192), (2304, 4100, 64)])
@pytest.mark.parametrize("split", [True, False])
def test_tail_split_gives_the_same_bits(M, N, K, split, monkeypatch):
    """Pair-shaped launches whose last wave is at most half full cut its tiles into column halves (two work items per
    tile); shapes chosen so that this happens, with ragged edges too.  Exact against an integer reference on the GPU."""
    monkeypatch.setenv("ASCQ_W8A8_TILE", "pair")
    if not split:
        monkeypatch.setenv("ASCQ_W8A8_NOSPLIT", "1")
    A, B, sA, sB, bias = make_case(M, N, K, M + N + K)
    dA, dB = torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV)
    acc = (dA.float() @ dB.float().T).to(torch.int32).cpu().numpy()      # K <= 256: every sum is exact in fp32
    got_C, got_acc = run(A, B, sA, sB, bias)
    assert np.array_equal(got_acc, acc)
    f = (acc.astype(np.float32) * sB[None, :]) * sA[:, None] + O.bf16_bits_to_f32(bias)[None, :]
    assert_bits_equal(got_C, O.f32_to_bf16_bits(f), "tail split")


def test_scatter_writes_the_block_into_every_buffer():
    # three [M, ldc] matrices stand in for this GPU's and two peers' output: the block must land at colOffset in each
    M, N, K, ldc, col = 200, 192, 256, 640, 256
    A, B, sA, sB, bias = make_case(M, N, K, 99)
    want = O.matmul_w8a8(A, B, sA, sB, bias)
    bufs = [torch.full((M, ldc), -1.0, dtype=torch.bfloat16, device=DEV) for _ in range(3)]
    t = lambda a: torch.from_numpy(a).to(DEV)  # noqa: E731
    dbias = torch.from_numpy(bias.view(np.int16)).to(DEV).view(torch.bfloat16)
    ops.MatmulW8A8Scatter([b.data_ptr() for b in bufs], 1, col, ldc, t(A), t(B), t(sA), t(sB), dbias)
    ops.MatmulStatus()
    for b in bufs:
        got = b.view(torch.int16).cpu().numpy().view(np.uint16)
        assert_bits_equal(np.ascontiguousarray(got[:, col:col + N]), want, "scattered block")
        assert (got[:, :col] == 0xBF80).all() and (got[:, col + N:] == 0xBF80).all(), "columns outside the block changed"
    with pytest.raises(ops.AscqError):
        ops.MatmulW8A8Scatter([bufs[0].data_ptr()] * 9, 0, 0, ldc, t(A), t(B))


@pytest.mark.parametrize("M,N,K", [(2048, 512, 128), (4096, 1280, 64), (4000, 2300, 64)])
def test_pair_tiles_into_two_buffers(M, N, K, monkeypatch):
    """A pair-shaped launch that writes two matrices (one TMA store per matrix from the same staged rows): 16 tiles,
    80 tiles and 144 ragged tiles whose last wave is cut into half-tile items and whose width is not a multiple of 8
    (per-thread stores).  Exact against an integer reference on the GPU."""
    monkeypatch.setenv("ASCQ_W8A8_TILE", "pair")
    A, B, sA, sB, bias = make_case(M, N, K, M + N)
    dA, dB = torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV)
    acc = (dA.float() @ dB.float().T).cpu().numpy()      # K <= 256: every sum is exact in fp32
    want = O.f32_to_bf16_bits((acc * sB[None, :]) * sA[:, None] + O.bf16_bits_to_f32(bias)[None, :])
    ldc = (N + 7) // 8 * 8 + 64
    bufs = [torch.full((M, ldc), -1.0, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    dbias = torch.from_numpy(bias.view(np.int16)).to(DEV).view(torch.bfloat16)
    ops.MatmulW8A8Scatter([b.data_ptr() for b in bufs], 1, 64, ldc, dA, dB, torch.from_numpy(sA).to(DEV), torch.from_numpy(sB).to(DEV), dbias)
    ops.MatmulStatus()
    for b in bufs:
        got = b.view(torch.int16).cpu().numpy().view(np.uint16)
        assert_bits_equal(np.ascontiguousarray(got[:, 64:64 + N]), want, "block")
        assert (got[:, :64] == 0xBF80).all() and (got[:, 64 + N:] == 0xBF80).all()


# ---- fixpipe quantisation of the result (SetQuantScalar / SetQuantVector, fp16 output) ----------------------------
@pytest.mark.parametrize("name", ["matmul_quant_scalar", "matmul_quant_vector"])
def test_matmul_quant_sample_golden_through_the_gpu(name):
    """The reference sample's own vectors (its gen_data.py, first 96 rows of A): transpose B once, one call, same bits."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name + ".npz"))
    A = torch.from_numpy(g["x1_gm"]).to(DEV)
    B_kn = torch.from_numpy(g["x2_gm"]).to(DEV)
    B_nk = torch.empty((1024, 1024), dtype=torch.int8, device=DEV)
    ops.TransposeI8KnToNk(B_nk, B_kn)
    assert torch.equal(B_nk, B_kn.t().contiguous())
    qv = torch.from_numpy(g["quant_vector_gm"].view(np.int64)).to(DEV) if "quant_vector_gm" in g else None
    C = torch.zeros((A.shape[0], 1024), dtype=torch.float16, device=DEV)
    ops.MatmulI8Quant(C, A, B_nk, torch.from_numpy(g["bias_gm"]).to(DEV), qv, 0.1)
    ops.MatmulStatus()
    assert_bits_equal(C.cpu().numpy().view(np.uint16), g["golden"].view(np.uint16), name)


@pytest.mark.parametrize("M,N,K,vector", [(128, 128, 128, True), (300, 520, 272, True), (257, 384, 1024, False), (4096, 512, 512, True)])
@pytest.mark.parametrize("tile", ["pair", "wide", "narrow", "slim"])
def test_matmul_quant_matches_oracle(M, N, K, vector, tile, monkeypatch):
    monkeypatch.setenv("ASCQ_W8A8_TILE", tile)
    rng = np.random.default_rng(M + N + K)
    A = rng.integers(-20, 21, (M, K), dtype=np.int8)
    B = rng.integers(-20, 21, (N, K), dtype=np.int8)
    bias = rng.integers(-50, 50, N, dtype=np.int32)
    qv = rng.uniform(0.01, 2.0, N).astype(np.float32).view(np.uint32).astype(np.uint64) if vector else None
    want = O.matmul_i8_quant(A, B, bias, qv, 0.37)
    C = torch.zeros((M, N), dtype=torch.float16, device=DEV)
    ops.MatmulI8Quant(C, torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV), torch.from_numpy(bias).to(DEV),
                      torch.from_numpy(qv.view(np.int64)).to(DEV) if vector else None, 0.37)
    ops.MatmulStatus()
    assert_bits_equal(C.cpu().numpy().view(np.uint16), want.view(np.uint16), f"{M}x{N}x{K}")


# ---- fixpipe requantisation of the result to int8 / uint8 ((V)REQ8) -----------------------------------------------
def _req8_words(rng, n, scale_lo, scale_hi, signed=None, shift=False):
    """Random 64-bit fixpipe parameters: fp32 scale bits, offset in bits 45:37, result type in bit 46, optional shift."""
    s = rng.uniform(scale_lo, scale_hi, n).astype(np.float32) * rng.choice([1.0, 1.0, -1.0], n).astype(np.float32)
    w = s.view(np.uint32).astype(np.uint64)
    w |= np.where(rng.random(n) < 0.5, 0, rng.integers(0, 512, n)).astype(np.uint64) << np.uint64(37)
    sg = rng.integers(0, 2, n) if signed is None else np.full(n, int(signed))
    w |= sg.astype(np.uint64) << np.uint64(46)
    if shift:
        on = (rng.random(n) < 0.5).astype(np.uint64)
        w |= (on << np.uint64(36)) | (rng.integers(0, 9, n).astype(np.uint64) << np.uint64(32))
    return w


def test_fixpipe_req8_sample_golden_through_the_gpu():
    """The fixpipe sample's int32 -> int8 case (vector parameters, no ReLU): same bytes as its generator wrote."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fixpipe_req8_matmul.npz"))
    A = torch.from_numpy(g["x1_gm"]).to(DEV)
    B_nk = torch.from_numpy(np.ascontiguousarray(g["x2_gm"].T)).to(DEV)
    qv = torch.from_numpy(g["quant_pre"].view(np.int64)).to(DEV)
    C = torch.zeros((128, 256), dtype=torch.int8, device=DEV)
    ops.MatmulI8Requant(C, A, B_nk, None, qv)
    ops.MatmulStatus()
    assert np.array_equal(C.cpu().numpy(), g["golden"])


@pytest.mark.parametrize("M,N,K,vector", [(128, 128, 128, True), (300, 520, 272, True), (257, 384, 1024, False), (4096, 512, 512, True)])
@pytest.mark.parametrize("tile", ["pair", "wide", "narrow", "slim"])
def test_matmul_requant_matches_oracle(M, N, K, vector, tile, monkeypatch):
    monkeypatch.setenv("ASCQ_W8A8_TILE", tile)
    rng = np.random.default_rng(7 * M + N + K)
    A = rng.integers(-20, 21, (M, K), dtype=np.int8)
    B = rng.integers(-20, 21, (N, K), dtype=np.int8)
    bias = rng.integers(-500, 500, N, dtype=np.int32)
    spread = 115.0 * np.sqrt(K)  # standard deviation of an accumulator entry
    qv = _req8_words(rng, N, 20.0 / spread, 200.0 / spread, shift=True) if vector else None
    qs = int(_req8_words(rng, 1, 60.0 / spread, 61.0 / spread, signed=False)[0])
    want = O.matmul_i8_requant(A, B, bias, qv, qs)
    assert len(np.unique(want)) > 100, "the case must not saturate everywhere"
    C = torch.full((M, N), 77, dtype=torch.uint8, device=DEV)
    ops.MatmulI8Requant(C, torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV), torch.from_numpy(bias).to(DEV),
                        torch.from_numpy(qv.view(np.int64)).to(DEV) if vector else None, qs)
    ops.MatmulStatus()
    got = C.cpu().numpy()
    bad = np.argwhere(got != want)
    assert bad.size == 0, f"{len(bad)} bytes differ, first at {bad[0]}: got {got[tuple(bad[0])]} want {want[tuple(bad[0])]}"


def test_matmul_requant_into_a_wider_unaligned_matrix():
    """ldc that is not a multiple of 16 takes the byte-by-byte store path; columns beyond N stay untouched."""
    M, N, K, ldc = 150, 200, 128, 213
    rng = np.random.default_rng(5)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-128, 128, (N, K), dtype=np.int8)
    qv = _req8_words(rng, N, 0.0005, 0.005)
    want = O.matmul_i8_requant(A, B, None, qv)
    C = torch.full((M, ldc), 99, dtype=torch.uint8, device=DEV)
    ops.MatmulI8Requant(C, torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV), None, torch.from_numpy(qv.view(np.int64)).to(DEV))
    ops.MatmulStatus()
    got = C.cpu().numpy()
    assert np.array_equal(got[:, :N], want)
    assert (got[:, N:] == 99).all()


def test_block_into_one_wider_matrix_through_the_tma_store_path(monkeypatch):
    """One aligned output matrix takes the TMA-store epilogue; with a column offset and ragged M / N the tensor map must
    clip exactly: the block lands at its columns, everything around it stays untouched, and the per-thread store path
    gives the same bits."""
    M, N, K, ldc, col = 333, 200, 256, 640, 128
    A, B, sA, sB, bias = make_case(M, N, K, 123)
    want = O.matmul_w8a8(A, B, sA, sB, bias)
    t = lambda a: torch.from_numpy(a).to(DEV)  # noqa: E731
    dbias = torch.from_numpy(bias.view(np.int16)).to(DEV).view(torch.bfloat16)
    outs = {}
    for mode in ("tma", "plain"):
        if mode == "plain":
            monkeypatch.setenv("ASCQ_W8A8_STORE", "plain")
        buf = torch.full((M + 5, ldc), -1.0, dtype=torch.bfloat16, device=DEV)
        ops.MatmulW8A8Scatter([buf.data_ptr()], 0, col, ldc, t(A), t(B), t(sA), t(sB), dbias)
        ops.MatmulStatus()
        got = buf.view(torch.int16).cpu().numpy().view(np.uint16)
        assert_bits_equal(np.ascontiguousarray(got[:M, col:col + N]), want, f"block ({mode})")
        assert (got[:M, :col] == 0xBF80).all() and (got[:M, col + N:] == 0xBF80).all() and (got[M:] == 0xBF80).all(), \
            f"elements outside the block changed ({mode})"
        outs[mode] = got
    assert np.array_equal(outs["tma"], outs["plain"])


# ---- grouped W8A8 (per-group weights and channel scales, per-token scales, optional FasterGelu) --------------------
def make_group_case(groups, N, K, seed):
    rng = np.random.default_rng(seed)
    sumM, G = int(sum(groups)), len(groups)
    A = rng.integers(-10, 10, (sumM, K)).astype(np.int8)
    B = rng.integers(-10, 10, (G, N, K)).astype(np.int8)
    sA = rng.normal(0, 0.01, sumM).astype(np.float32)
    sB = rng.normal(0, 0.01, (G, N)).astype(np.float32)
    return A, B, sA, sB


def run_group(A, B, sA, sB, groups, out=torch.float16, act=0, bias=None):
    t = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(DEV)  # noqa: E731
    C = torch.full((max(int(sum(groups)), 1), B.shape[1]), -1.0, dtype=out, device=DEV)
    dbias = None if bias is None else torch.from_numpy(bias.view(np.int16).copy()).to(DEV).view(torch.bfloat16)
    ops.GroupMatmulW8A8(C, t(A), t(B), t(sA), t(sB), groups, dbias, act)
    ops.MatmulStatus()
    return C[:int(sum(groups))].view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("groups,N,K", [([128, 256], 256, 128), ([100, 0, 300, 129, 1], 384, 272), ([1, 1, 1], 8, 16),
                                        ([700, 52], 520, 1024), ([257] * 5, 640, 64)])
@pytest.mark.parametrize("tile", ["narrow", "wide", "pair"])
@pytest.mark.parametrize("out", [torch.float16, torch.bfloat16])
def test_group_matmul_is_bit_exact_without_activation(groups, N, K, tile, out, monkeypatch):
    monkeypatch.setenv("ASCQ_W8A8_TILE", tile)
    A, B, sA, sB = make_group_case(groups, N, K, sum(groups) + N + K)
    bias = O.f32_to_bf16_bits(np.random.default_rng(1).normal(0, 0.1, (len(groups), N)).astype(np.float32)) if K == 272 else None
    want = O.group_matmul_w8a8(A, B, sA, sB, groups, bias_bf16=bias, out=O.F16 if out == torch.float16 else O.BF16)
    got = run_group(A, B, sA, sB, groups, out, 0, bias)
    assert_bits_equal(got, want.view(np.uint16), f"groups {groups} {tile}")


@pytest.mark.parametrize("tile", ["narrow", "pair"])
def test_group_matmul_with_faster_gelu(tile, monkeypatch):
    """The exponential is the CUDA library's, the oracle's is correctly rounded: at most one half-precision step apart,
    on a small fraction of the elements."""
    monkeypatch.setenv("ASCQ_W8A8_TILE", tile)
    groups, N, K = [300, 0, 129, 64], 512, 512
    A, B, sA, sB = make_group_case(groups, N, K, 5)
    sA, sB = sA * 30, sB * 30          # arguments of the activation of order one
    want = O.group_matmul_w8a8(A, B, sA, sB, groups, act=True)
    got = run_group(A, B, sA, sB, groups, torch.float16, 1)
    steps = np.abs(got.view(np.int16).astype(np.int32) - want.view(np.int16).astype(np.int32))
    assert steps.max() <= 1 and (steps != 0).mean() < 0.01, (steps.max(), (steps != 0).mean())


def test_group_matmul_reference_sample_golden_through_the_gpu():
    """The sample's own vectors (its gen_data.py; 16 rows of each of the 8 groups, 128 columns): within one half-precision
    step of the golden and inside the sample's acceptance rule (rtol = atol = 1e-3, at most 1e-4 of the elements outside)."""
    d = np.load(os.path.join(GOLDEN, "quant_group_matmul.npz"))
    G, K, N = d["weight_gkn"].shape
    Bnk = torch.empty((G, N, K), dtype=torch.int8, device=DEV)
    for g in range(G):   # the sample's weight is [K, N] per group: turned once
        ops.TransposeI8KnToNk(Bnk[g], torch.from_numpy(np.ascontiguousarray(d["weight_gkn"][g])).to(DEV))
    groups = [int(v) for v in d["groupList"]]
    C = torch.empty((sum(groups), N), dtype=torch.float16, device=DEV)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)  # noqa: E731
    ops.GroupMatmulW8A8(C, t(d["x"]), Bnk, t(d["perTokenScale"]), t(d["scale"]), groups, None, 1)
    ops.MatmulStatus()
    got, gold = C.cpu().numpy(), d["golden"]
    outside = ~np.isclose(got.astype(np.float32), gold.astype(np.float32), rtol=1e-3, atol=1e-3)
    assert outside.mean() <= 1e-4
    steps = np.abs(got.view(np.int16).astype(np.int32) - gold.view(np.int16).astype(np.int32))
    assert steps.max() <= 1 and (steps != 0).mean() < 2e-3


def test_group_matmul_published_shape_property():
    """G = 8, M = N = 8192, K = 1024 (the shape of the reference's published timing): int32-exact inputs, compared with
    an fp32 torch matmul per group (every sum < 2^24, so that product is exact) -- all 67 M elements, bit for bit."""
    G, M, N, K = 8, 8192, 8192, 1024
    groups = [M // G] * G
    g = torch.Generator(device=DEV).manual_seed(3)
    A = torch.randint(-10, 10, (M, K), dtype=torch.int8, device=DEV, generator=g)
    B = torch.randint(-10, 10, (G, N, K), dtype=torch.int8, device=DEV, generator=g)
    sA = torch.randn(M, device=DEV, generator=g) * 0.01
    sB = torch.randn((G, N), device=DEV, generator=g) * 0.01
    C = torch.empty((M, N), dtype=torch.float16, device=DEV)
    ops.GroupMatmulW8A8(C, A, B, sA, sB, groups)
    ops.MatmulStatus()
    for i in range(G):
        r = slice(i * (M // G), (i + 1) * (M // G))
        acc = A[r].float() @ B[i].float().T
        want = ((acc * sB[i][None, :]) * sA[r][:, None]).half()
        assert torch.equal(C[r], want), f"group {i}"


def test_group_matmul_argument_checks():
    z = torch.zeros((256, 64), dtype=torch.int8, device=DEV)
    c = torch.zeros((256, 64), dtype=torch.float16, device=DEV)
    with pytest.raises(ops.AscqError):
        ops.GroupMatmulW8A8(c, z, z.view(1, 256, 64), None, None, [-1])
    with pytest.raises(ops.AscqError):
        ops.GroupMatmulW8A8(c, z, z.view(1, 256, 64), None, None, [1] * 129)
    with pytest.raises(ops.AscqError):
        ops.GroupMatmulW8A8(c.float(), z, z.view(1, 256, 64), None, None, [256])


def test_results_beyond_the_16_bit_range_saturate_like_the_oracle():
    """Scales large enough that some results overflow bfloat16 / half: the reference's casts saturate finite overflow to
    the largest finite value; the epilogue detects the rare infinity after its branch-free conversion and redoes the
    chunk with the saturating one."""
    M, N, K = 256, 256, 512
    A, B, sA, sB, bias = make_case(M, N, K, 77)
    sA = sA.copy()
    sA[::3] *= np.float32(3e37)          # rows whose results leave the bfloat16 range
    want = O.matmul_w8a8(A, B, sA, sB, bias)
    got, _ = run(A, B, sA, sB, bias, want_acc=False)
    assert_bits_equal(got, want, "bf16 saturation")
    assert (want == 0x7F7F).any() and (want == 0xFF7F).any(), "the case must saturate somewhere"
    # half output (grouped entry point, one group)
    sA2 = np.abs(sA) % np.float32(1.0) + np.float32(0.5)
    sA2[::5] *= np.float32(1e6)
    wanth = O.group_matmul_w8a8(A, B[None], sA2, sB[None], [M])
    goth = run_group(A, B[None], sA2, sB[None], [M])
    assert_bits_equal(goth, wanth.view(np.uint16), "half saturation")
    assert (wanth.view(np.uint16) == 0x7BFF).any() or (wanth.view(np.uint16) == 0xFBFF).any()


# ---- at most 32 activation rows: the kernel that reads the weight once (mma.sync, K shared by a CTA's warps) ---------------

@pytest.mark.parametrize("M", [1, 7, 8, 16, 25, 32, 33])
@pytest.mark.parametrize("N,K", [(16, 512), (520, 640), (4096, 4096), (2300, 8192), (12288, 1024)])
def test_few_rows_kernel_is_bit_exact(M, N, K, monkeypatch):
    """Against the oracle, and against the tcgen05 kernel on the same inputs (ASCQ_W8A8_SMALL=0), into a pitched output
    whose guard columns must stay untouched."""
    A, B, sA, sB, bias = make_case(M, N, K, M * 13 + N + K)
    want = O.matmul_w8a8(A, B, sA, sB, bias)
    outs = {}
    for small in ("1", "0"):
        monkeypatch.setenv("ASCQ_W8A8_SMALL", small)
        got, _ = run(A, B, sA, sB, bias, ldc=N + 8, want_acc=False)
        assert (got[:, N:] == 0xBF80).all(), small
        outs[small] = got[:, :N]
        assert_bits_equal(outs[small], want, f"ASCQ_W8A8_SMALL={small}")


def test_few_rows_kernel_optional_operands_and_extremes(monkeypatch):
    monkeypatch.delenv("ASCQ_W8A8_SMALL", raising=False)
    A, B, sA, sB, bias = make_case(24, 528, 1024, 77)
    for kw in (dict(), dict(sA=sA), dict(sB=sB), dict(bias=bias), dict(sA=sA, sB=sB)):
        want = O.matmul_w8a8(A, B, kw.get("sA"), kw.get("sB"), kw.get("bias"))
        got, _ = run(A, B, kw.get("sA"), kw.get("sB"), kw.get("bias"), want_acc=False)
        assert_bits_equal(got, want, f"operands {sorted(kw)}")
    # +-127 everywhere: the largest accumulator magnitude for this K; unit scales make the bf16 result saturate-free but huge
    M, N, K = 5, 256, 8192
    A = np.full((M, K), 127, np.int8)
    B = np.full((N, K), -127, np.int8)
    B[::2] = 127
    got, _ = run(A, B, want_acc=False)
    assert_bits_equal(got, O.matmul_w8a8(A, B, None, None, None), "extreme values")
    # rows whose results leave the bfloat16 range: finite overflow saturates, infinities stay, as in the oracle
    A, B, sA, sB, bias = make_case(32, 1024, 512, 78)
    sA = sA.copy()
    sA[::3] *= np.float32(3e37)
    want = O.matmul_w8a8(A, B, sA, sB, bias)
    got, _ = run(A, B, sA, sB, bias, want_acc=False)
    assert_bits_equal(got, want, "saturation")
    assert (want == 0x7F7F).any() or (want == 0xFF7F).any(), "the case must saturate somewhere"


def test_read_rate_yardstick_of_the_few_rows_kernels(tmp_path, capsys):
    """Builds and runs tests/cpp/read_pattern_probe.cu: the weight matrix read once with the few-row kernels' work split
    and three request shapes.  The table is printed (run with -s to see it); the check is only that every variant ran
    and reached a rate of the right order."""
    import os
    import shutil
    import subprocess
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = shutil.which("nvcc") or os.path.join(cuda_home, "bin", "nvcc")
    if not os.path.exists(nvcc):
        pytest.skip("nvcc is needed to build the probe")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = tmp_path / "read_pattern_probe"
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-o", str(exe),
                    os.path.join(root, "tests", "cpp", "read_pattern_probe.cu")], check=True, capture_output=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "done" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
    with capsys.disabled():
        print("\n" + r.stdout)
    rates = [float(line.split("us")[1].split("GB/s")[0]) for line in r.stdout.splitlines() if "GB/s" in line]
    assert len(rates) == 18 and min(rates) > 500.0 and all("no error" in line for line in r.stdout.splitlines() if "GB/s" in line), rates


# ---- skinny products on 64-column tiles ----------------------------------------------------------------------------------

@pytest.mark.parametrize("M,N,K", [(33, 128, 128), (100, 520, 1024), (128, 4096, 4096), (200, 1000, 272), (256, 8192, 512),
                                   (700, 300, 640)])
@pytest.mark.parametrize("forced", [True, False])
def test_skinny_products_on_64_column_tiles(M, N, K, forced, monkeypatch):
    """One or two row tiles and fewer 128-column tiles than SMs: the launch takes 64-column tiles (forced here for every
    shape, and chosen by the library itself for the skinny ones).  Accumulators and results are the oracle's bits."""
    if forced:
        monkeypatch.setenv("ASCQ_W8A8_TILE", "slim")
    else:
        monkeypatch.delenv("ASCQ_W8A8_TILE", raising=False)
    A, B, sA, sB, bias = make_case(M, N, K, M + 3 * N + K)
    want_C, want_acc = O.matmul_w8a8(A, B, sA, sB, bias, want_acc=True)
    got_C, got_acc = run(A, B, sA, sB, bias, ldc=N + 8)
    assert_bits_equal(got_acc, want_acc, "int32 accumulators")
    assert_bits_equal(got_C[:, :N], want_C, "bf16 epilogue")
    assert (got_C[:, N:] == 0xBF80).all()
