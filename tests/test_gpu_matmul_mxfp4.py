"""GPU parity of the MX-FP4 grouped matmul against the CPU oracle (fp64 accumulation, the reference's golden
semantics).  The GPU accumulates in fp32, so general inputs are compared element by element with
|got - want| <= 1e-2 |want| + K 2^-24 sum_k |a_k b_k|: the rtol of the target plus the worst case of an fp32
accumulation of K terms in any order (that term matters only where the sum cancels).  Inputs whose partial sums
are exactly representable must match bit for bit."""
import numpy as np
import pytest
import torch

from asc_devkit_b200 import _lib as L
from asc_devkit_b200 import ops
from oracle import oracle as O
from tests.gpu_util import DEV, assert_bits_equal

pytestmark = pytest.mark.gpu


def make_case(groups, N, K, seed, exp_span=4, codes=None):
    rng = np.random.default_rng(seed)
    sumM, G = int(sum(groups)), len(groups)
    if codes is None:
        A = rng.integers(0, 256, (sumM, K // 2)).astype(np.uint8)
        B = rng.integers(0, 256, (G, N, K // 2)).astype(np.uint8)
    else:
        pick = lambda shape: (rng.choice(codes, shape) | (rng.choice(codes, shape) << 4)).astype(np.uint8)  # noqa: E731
        A, B = pick((sumM, K // 2)), pick((G, N, K // 2))
    sA = (127 + rng.integers(-exp_span, exp_span + 1, (sumM, K // 32))).astype(np.uint8)
    sB = (127 + rng.integers(-exp_span, exp_span + 1, (G, N, K // 32))).astype(np.uint8)
    return A, sA, B, sB


def run(A, sA, B, sB, groups, K, N):
    sumM = int(sum(groups))
    t = lambda a: torch.from_numpy(a).to(DEV)  # noqa: E731
    dC = torch.full((max(sumM, 1), N), -1.0, dtype=torch.bfloat16, device=DEV)
    ops.GroupMatmulMxfp4(dC, t(A), t(sA), t(B), t(sB), groups, K, N)
    ops.MatmulStatus()
    return dC.view(torch.int16).cpu().numpy().view(np.uint16)[:sumM]


E2M1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], np.float64)


def dequant(codes, scales, K):
    """[rows, K/2] packed E2M1 + [rows, K/32] E8M0 -> [rows, K] float64 (element 2i in the low nibble)."""
    v = np.empty((codes.shape[0], K), np.float64)
    v[:, 0::2], v[:, 1::2] = E2M1[codes & 0xF], E2M1[codes >> 4]
    return v * np.repeat(np.exp2(scales.astype(np.float64) - 127.0), 32, axis=1)


def abs_product_sums(A, sA, B, sB, groups, K):
    """sum_k |a_k b_k| for every output element, [sumM, N] float64."""
    out, r0 = [], 0
    for g, mg in enumerate(groups):
        if mg:
            out.append(np.abs(dequant(A[r0:r0 + mg], sA[r0:r0 + mg], K)) @ np.abs(dequant(B[g], sB[g], K)).T)
        r0 += mg
    return np.concatenate(out) if out else np.zeros((0, B.shape[1]))


def check_close(got_bits, want_f32, what, abs_sums, K):
    got = O.bf16_bits_to_f32(got_bits).astype(np.float64)
    want = want_f32.astype(np.float64)
    tol = 1e-2 * np.abs(want) + (K * 2.0 ** -24) * abs_sums
    bad = np.abs(got - want) > tol
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside the bound; worst {np.abs(got - want).max()}"


@pytest.mark.parametrize("groups,N,K", [([128], 256, 256), ([128], 128, 128), ([256], 512, 1024), ([64], 256, 512),
                                        ([100, 0, 300, 129], 384, 384), ([1, 1, 1], 8, 128), ([257], 2048, 7168)])
def test_parity(groups, N, K):
    A, sA, B, sB = make_case(groups, N, K, sum(groups) + N + K)
    want_bits, want_f32 = O.group_matmul_mxfp4(A, sA, B, sB, np.array(groups, np.int64), K, N, want_f32=True)
    got = run(A, sA, B, sB, groups, K, N)
    check_close(got, want_f32, f"groups {groups}", abs_product_sums(A, sA, B, sB, groups, K), K)
    ulp = O.bf16_ulp_diff(got, want_bits)
    assert ulp.max_ulp <= 2 or ulp.mismatches < 0.02 * ulp.total, ulp


def test_many_groups_use_the_host_built_tile_table():
    """More than 256 groups: the row-tile table is built on the host and copied (fewer groups build it on the device)."""
    rng = np.random.default_rng(11)
    groups = [int(v) for v in rng.choice([0, 1, 3, 17, 130], 300)]
    N, K = 256, 256
    A, sA, B, sB = make_case(groups, N, K, 12)
    _, want_f32 = O.group_matmul_mxfp4(A, sA, B, sB, np.array(groups, np.int64), K, N, want_f32=True)
    check_close(run(A, sA, B, sB, groups, K, N), want_f32, "300 groups", abs_product_sums(A, sA, B, sB, groups, K), K)


@pytest.mark.parametrize("tile", ["single", "pair"])
def test_both_tile_shapes_give_the_same_bits(tile, monkeypatch):
    groups, N, K = [300, 0, 5, 256, 129], 512, 512
    A, sA, B, sB = make_case(groups, N, K, 21)
    _, want_f32 = O.group_matmul_mxfp4(A, sA, B, sB, np.array(groups, np.int64), K, N, want_f32=True)
    monkeypatch.setenv("ASCQ_MXFP4_TILE", tile)
    check_close(run(A, sA, B, sB, groups, K, N), want_f32, tile, abs_product_sums(A, sA, B, sB, groups, K), K)


def test_prepacked_weight_scales_give_the_same_bits():
    groups, N, K = [300, 0, 129, 64], 512, 1024
    A, sA, B, sB = make_case(groups, N, K, 41)
    want = run(A, sA, B, sB, groups, K, N)
    t = lambda a: torch.from_numpy(a).to(DEV)  # noqa: E731
    packed = ops.GroupMatmulMxfp4PackScaleB(t(sB), K, N)
    C = torch.full((sum(groups), N), -1.0, dtype=torch.bfloat16, device=DEV)
    for _ in range(2):   # the packed buffer is reused across calls
        ops.GroupMatmulMxfp4Prepacked(C, t(A), t(sA), t(B), packed, groups, K, N)
    ops.MatmulStatus()
    assert_bits_equal(C.view(torch.int16).cpu().numpy().view(np.uint16), want, "prepacked")


def test_scatter_writes_every_buffer_at_the_given_rows():
    """The fused reassembly of a group-parallel layout, on one GPU: three output matrices stand for this GPU's and two
    peers'; the groups computed here are placed at their rows of the full output, other rows stay untouched."""
    groups, N, K = [130, 0, 300, 64], 512, 512
    out_row_start = [700, 0, 100, 420]           # where each group lives in the full [1000, N] output
    A, sA, B, sB = make_case(groups, N, K, 31)
    want = run(A, sA, B, sB, groups, K, N)       # plain entry point: groups one after the other
    t = lambda a: torch.from_numpy(a).to(DEV)  # noqa: E731
    bufs = [torch.full((1000, N), -1.0, dtype=torch.bfloat16, device=DEV) for _ in range(3)]
    ops.GroupMatmulMxfp4Scatter([b.data_ptr() for b in bufs], 1, out_row_start, t(A), t(sA), t(B), t(sB), groups, K, N)
    ops.MatmulStatus()
    expect = np.full((1000, N), O.f32_to_bf16_bits(np.array([-1.0], np.float32))[0], np.uint16)
    src = 0
    for g, mg in enumerate(groups):
        expect[out_row_start[g]:out_row_start[g] + mg] = want[src:src + mg]
        src += mg
    for b in bufs:
        assert_bits_equal(b.view(torch.int16).cpu().numpy().view(np.uint16), expect, "scatter buffer")


@pytest.mark.parametrize("groups,N,K", [([128, 200], 256, 512), ([77], 320, 256)])
def test_exact_when_sums_are_representable(groups, N, K):
    # codes {0, +-0.5, +-1, +-2} with unit scales: every partial sum is a small multiple of 0.25 -> exact in fp32
    A, sA, B, sB = make_case(groups, N, K, 7, exp_span=0, codes=np.array([0, 1, 2, 4, 9, 10, 12], np.uint8))
    want = O.group_matmul_mxfp4(A, sA, B, sB, np.array(groups, np.int64), K, N)
    assert_bits_equal(run(A, sA, B, sB, groups, K, N), want, "exact case")


def test_scale_bytes_are_applied_per_32_elements():
    # one-hot operands: A row r has a single 1.0 at k = 32*r, B row n has 1.0 everywhere; the product picks out
    # exactly sA[r, r] * sB[n, r], so every scale byte position is checked individually
    M, N, K = 128, 256, 4096
    A = np.zeros((M, K // 2), np.uint8)
    for r in range(M):
        A[r, (32 * r) // 2] = 2  # code 2 = 1.0 in the low nibble
    B = np.full((1, N, K // 2), 0x22, np.uint8)
    rng = np.random.default_rng(3)
    sA = (127 + rng.integers(-6, 7, (M, K // 32))).astype(np.uint8)
    sB = (127 + rng.integers(-6, 7, (1, N, K // 32))).astype(np.uint8)
    got = O.bf16_bits_to_f32(run(A, sA, B, sB, [M], K, N))
    want = np.exp2(sA[np.arange(M), np.arange(M)].astype(np.float64) - 127)[:, None] * \
        np.exp2(sB[0][:, :M].T.astype(np.float64) - 127)
    assert np.array_equal(got.astype(np.float64), want)


def test_reference_layout_adapters():
    # B [K, N] with pairs along N and scaleB stored [sK/2, N, 2] (examples/.../matmul_mxfp4_high_performance)
    K, N = 256, 64
    rng = np.random.default_rng(11)
    codes = rng.integers(0, 16, (K, N)).astype(np.uint8)
    b_kn = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    b_nk_want = (codes.T[:, 0::2] | (codes.T[:, 1::2] << 4)).astype(np.uint8)
    d = torch.zeros((N, K // 2), dtype=torch.uint8, device=DEV)
    ops.MxRepackBKnToNk(d, torch.from_numpy(b_kn).to(DEV), K, N)
    assert np.array_equal(d.cpu().numpy(), b_nk_want)
    sK = K // 32
    s = rng.integers(100, 150, (sK, N)).astype(np.uint8)
    s_ref = np.ascontiguousarray(s.reshape(sK // 2, 2, N).transpose(0, 2, 1))
    d = torch.zeros((N, sK), dtype=torch.uint8, device=DEV)
    ops.MxRepackScaleB(d, torch.from_numpy(s_ref).to(DEV), sK, N)
    assert np.array_equal(d.cpu().numpy(), s.T)


def test_invalid_arguments():
    z = torch.zeros(1 << 16, dtype=torch.uint8, device=DEV)
    c = torch.zeros((128, 64), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ops.AscqError) as e:
        ops.GroupMatmulMxfp4(c, z, z, z, z, [128], 96, 64)
    assert "multiple of 128" in e.value.message
    with pytest.raises(ops.AscqError):
        ops.GroupMatmulMxfp4(c, z, z, z, z, [128, -1], 128, 64)
    with pytest.raises(ops.AscqError) as e:
        ops.GroupMatmulMxfp4(c, z, z, z, z, [128], 128, 64, workspace=torch.zeros(256, dtype=torch.uint8, device=DEV))
    assert "workspace" in e.value.message


def decode_on_gpu(codes, scales, K):
    """MX decode of [rows, K/2] packed E2M1 with [rows, K/32] E8M0 scales through AscendAntiQuant on the GPU (its bits
    are pinned by the oracle in tests/test_gpu_antiquant.py) -> fp32 [rows, K].  Every product code x 2^e is exact."""
    rows = codes.shape[0]
    out = torch.empty((rows, K), dtype=torch.bfloat16, device=DEV)
    ops.AscendAntiQuant(out, codes, None, scales.reshape(-1), ops.AscendAntiQuantParam(rows, K), isTranspose=True,
                        policy=L.PER_GROUP, hasOffset=False, src_dtype=L.DT_FP4X2_E2M1, scale_dtype=L.DT_E8M0)
    return out.float()


def test_cfg5_full_size():
    """Benchmark config 5 (G=16, 16384 tokens split by a seeded multinomial, K=7168, N=2048), EVERY output element:
    the operands are decoded by the MX decode operator and multiplied group by group with an fp32 torch.matmul -- a
    checker that shares nothing with the kernel under test but the decode, which the oracle pins bit for bit.  The
    bound per element is 1e-2 |want| + 2 K 2^-24 sum |a_k b_k| (both sides accumulate in fp32).  72 rows at the start,
    at a group boundary and at the end are also compared with the oracle itself."""
    G, K, N, total = 16, 7168, 2048, 16384
    rng = np.random.default_rng(20251125 + 5)
    groups = rng.multinomial(total, np.full(G, 1.0 / G)).astype(np.int64)
    A, sA, B, sB = make_case(list(groups), N, K, 20251125 + 5)
    t = lambda a: torch.from_numpy(a).to(DEV)  # noqa: E731
    dA, dsA, dB, dsB = t(A), t(sA), t(B), t(sB)
    C1 = torch.empty((total, N), dtype=torch.bfloat16, device=DEV)
    ops.GroupMatmulMxfp4(C1, dA, dsA, dB, dsB, list(groups), K, N)
    ops.MatmulStatus()
    starts = np.concatenate([[0], np.cumsum(groups)])
    # all 16384 rows against the independent fp32 product
    tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        fA = decode_on_gpu(dA, dsA, K)
        worst = 0.0
        for g in range(G):
            r0, r1 = int(starts[g]), int(starts[g + 1])
            fB = decode_on_gpu(dB[g], dsB[g], K)
            want = fA[r0:r1] @ fB.T
            bound = 1e-2 * want.abs() + (2 * K * 2.0 ** -24) * (fA[r0:r1].abs() @ fB.abs().T)
            err = (C1[r0:r1].float() - want).abs()
            bad = err > bound
            assert not bool(bad.any()), f"group {g}: {int(bad.sum())} of {bad.numel()} elements outside the bound"
            worst = max(worst, float((err / (want.abs() + 1e-30)).median()))
        assert worst < 2.0 ** -8, f"median relative error {worst} is more than a bf16 rounding step"
    finally:
        torch.backends.cuda.matmul.allow_tf32 = tf32
    # rows sampled from the start, a group boundary and the end, against the oracle
    got = C1.view(torch.int16).cpu().numpy().view(np.uint16)
    for g, lo, cnt in [(0, 0, 24), (5, int(groups[5]) - 24, 24), (G - 1, int(groups[G - 1]) - 24, 24)]:
        r0 = int(starts[g]) + lo
        a, sa, b, sb = A[r0:r0 + cnt], sA[r0:r0 + cnt], B[g:g + 1], sB[g:g + 1]
        _, want = O.group_matmul_mxfp4(np.ascontiguousarray(a), np.ascontiguousarray(sa), np.ascontiguousarray(b),
                                       np.ascontiguousarray(sb), np.array([cnt], np.int64), K, N, want_f32=True)
        check_close(got[r0:r0 + cnt], want, f"cfg5 group {g}", abs_product_sums(a, sa, b, sb, [cnt], K), K)
    # size-independent property: raising every A scale exponent by one doubles the result exactly
    C2 = torch.empty_like(C1)
    ops.GroupMatmulMxfp4(C2, dA, dsA + 1, dB, dsB, list(groups), K, N)
    ops.MatmulStatus()
    assert torch.equal(C2.float(), C1.float() * 2.0)
