"""The C++ host mirror of the Matmul object (include/ascq_matmul.hpp): compiles against the C ABI, reports what the
reference asserts as ascq::Error, and on a GPU gives the oracle's results for every operand-type combination it maps.

The driver program tests/cpp/matmul_mirror_main.cpp uses the object the way the reference's samples do
(matmul_quant.asc:105-135); operands travel through files."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from asc_devkit_b200 import _lib as L  # noqa: E402
from oracle import oracle as O  # noqa: E402

CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
GOLDEN = os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="module")
def exe(tmp_path_factory):
    out = tmp_path_factory.mktemp("mm_mirror") / "matmul_mirror_main"
    libdir = os.path.dirname(L.LIB_PATH)
    cmd = ["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA_HOME, "include"),
           os.path.join(ROOT, "tests", "cpp", "matmul_mirror_main.cpp"), "-o", str(out), "-L", libdir, "-lascq",
           "-L", os.path.join(CUDA_HOME, "lib64"), "-lcudart", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{CUDA_HOME}/lib64"]
    subprocess.run(cmd, check=True)
    return str(out)


def run(exe, op, d, dims=None, **files):
    if dims is not None:
        np.array(dims, np.uint32).tofile(d / "dims.bin")
    for name, arr in files.items():
        np.ascontiguousarray(arr).tofile(d / f"{name}.bin")
    r = subprocess.run([exe, op, str(d)], capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, r.stderr + r.stdout
    return r.stdout


def close(got, want, rtol=1e-2):
    tol = rtol * np.abs(want) + 2e-3 * np.abs(want).max()
    assert (np.abs(got.astype(np.float64) - want.astype(np.float64)) <= tol).all(), np.abs(got - want).max()


def test_matmul_mirror_compiles_and_reports_reference_asserts(exe, tmp_path):
    """A quantised output type without SetQuantScalar / SetQuantVector, a [K, N] 16-bit B, GetTensorC with no block."""
    assert "caught=3" in run(exe, "errors", tmp_path)


@pytest.mark.gpu
@pytest.mark.parametrize("name,op", [("matmul_quant_vector", "quant_vector"), ("matmul_quant_scalar", "quant_scalar")])
def test_matmul_quant_sample_through_the_object(exe, tmp_path, name, op):
    """The matmul_quant sample as its kernel writes it: Init(tiling), SetTensorA/B (B stored [K, N]), SetBias,
    SetQuantVector or SetQuantScalar(bits of 0.1f), IterateAll, End -- and the sample's own golden."""
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    A, B_kn = g["x1_gm"], g["x2_gm"]
    files = dict(a=A, b_kn=B_kn, bias=g["bias_gm"])
    if "quant_vector_gm" in g:
        files["quant"] = g["quant_vector_gm"]
    run(exe, op, tmp_path, [A.shape[0], B_kn.shape[1], A.shape[1]], **files)
    got = np.fromfile(tmp_path / "c.bin", np.uint16).reshape(A.shape[0], B_kn.shape[1])
    assert np.array_equal(got, g["golden"].view(np.uint16))


@pytest.mark.gpu
def test_requant_through_iterate_and_get_tensor_c(exe, tmp_path):
    g = np.load(os.path.join(GOLDEN, "fixpipe_req8_matmul.npz"))
    run(exe, "requant_vector", tmp_path, [128, 256, 128], a=g["x1_gm"], b_nk=g["x2_gm"].T, quant=g["quant_pre"])
    assert np.array_equal(np.fromfile(tmp_path / "c.bin", np.int8).reshape(128, 256), g["golden"])


@pytest.mark.gpu
def test_half_matmul_with_quantised_output(exe, tmp_path):
    g = np.load(os.path.join(GOLDEN, "fixpipe_qf322b8_matmul.npz"))
    run(exe, "f16_quant", tmp_path, [128, 256, 128], a=g["x1_gm"], b_nk=g["x2_gm"].T, quant=g["quant_pre"])
    got = np.fromfile(tmp_path / "c.bin", np.int8).reshape(128, 256).astype(np.int32)
    diff = np.abs(got - g["golden"].astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 2e-3


@pytest.mark.gpu
def test_int32_accumulator_output(exe, tmp_path):
    rng = np.random.default_rng(21)
    M, N, K = 200, 320, 192
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-128, 128, (N, K), dtype=np.int8)
    run(exe, "acc_i32", tmp_path, [M, N, K], a=A, b_nk=B)
    want = A.astype(np.int32) @ B.astype(np.int32).T
    assert np.array_equal(np.fromfile(tmp_path / "c.bin", np.int32).reshape(M, N), want)


@pytest.mark.gpu
def test_bfloat16_matmul(exe, tmp_path):
    rng = np.random.default_rng(22)
    M, N, K = 160, 256, 128
    A = O.f32_to_bf16_bits(rng.normal(0, 1, (M, K)).astype(np.float32))
    B = O.f32_to_bf16_bits(rng.normal(0, 1, (N, K)).astype(np.float32))
    run(exe, "bf16", tmp_path, [M, N, K], a=A, b_nk=B)
    _, want = O.matmul_f16(A, B, O.BF16, O.F32)
    close(np.fromfile(tmp_path / "c.bin", np.float32).reshape(M, N), want)


@pytest.mark.gpu
def test_weight_only_quantised_matmul(exe, tmp_path):
    rng = np.random.default_rng(23)
    M, N, K = 96, 256, 128
    A = rng.normal(0, 1, (M, K)).astype(np.float16)
    B_nk = rng.integers(-128, 128, (N, K), dtype=np.int8)
    scale = rng.uniform(0.01, 0.05, N).astype(np.float16)
    offset = rng.uniform(-4, 4, N).astype(np.float16)
    run(exe, "w8a16", tmp_path, [M, N, K], a=A, b_kn=B_nk.T, offset=offset, scale=scale)
    (c16, _), _ = O.matmul_w8a16(A, O.F16, B_nk, offset, scale, O.F16)
    got = np.fromfile(tmp_path / "c.bin", np.float16).reshape(M, N)
    close(got.astype(np.float32), c16.view(np.float16).astype(np.float32))


@pytest.mark.gpu
def test_mx_fp4_matmul_in_the_sample_layouts(exe, tmp_path):
    """B [K, N] with fp4 pairs along N and scaleB [K/64, N, 2], as the matmul_mxfp4 sample stores them."""
    rng = np.random.default_rng(24)
    M, N, K = 150, 128, 256
    ca = rng.integers(0, 16, (M, K)).astype(np.uint8)
    cb = rng.integers(0, 16, (K, N)).astype(np.uint8)
    A = (ca[:, 0::2] | (ca[:, 1::2] << 4)).astype(np.uint8)
    B_kn = (cb[:, 0::2] | (cb[:, 1::2] << 4)).astype(np.uint8)
    B_nk = np.ascontiguousarray((cb.T[:, 0::2] | (cb.T[:, 1::2] << 4)).astype(np.uint8))
    sK = K // 32
    sA = rng.integers(123, 131, (M, sK)).astype(np.uint8)
    sB = rng.integers(123, 131, (sK, N)).astype(np.uint8)
    sB_ref = np.ascontiguousarray(sB.reshape(sK // 2, 2, N).transpose(0, 2, 1))
    run(exe, "mxfp4", tmp_path, [M, N, K], a=A, b_kn=B_kn, sa=sA, sb_ref=sB_ref)
    _, want = O.group_matmul_mxfp4(A, sA, B_nk[None], np.ascontiguousarray(sB.T)[None], np.array([M]), K, N, want_f32=True)
    got = O.bf16_bits_to_f32(np.fromfile(tmp_path / "c.bin", np.uint16).reshape(M, N))
    close(got, want)


@pytest.mark.gpu
def test_mx_fp8_matmul(exe, tmp_path):
    rng = np.random.default_rng(25)
    M, N, K = 64, 128, 256

    def codes(shape, fmt):  # finite fp8 codes only
        c = rng.integers(0, 256, shape).astype(np.uint8)
        if fmt == 0:
            c[(c & 0x7F) == 0x7F] = 0x3C
        else:
            c[(c & 0x7C) == 0x7C] = 0x3C
        return c
    A, B = codes((M, K), 0), codes((N, K), 1)
    sA = rng.integers(120, 130, (M, K // 32)).astype(np.uint8)
    sB = rng.integers(120, 130, (N, K // 32)).astype(np.uint8)
    run(exe, "mxfp8", tmp_path, [M, N, K], a=A, b_nk=B, sa=sA, sb=sB)
    _, want = O.group_matmul_mxfp8(A, 0, sA, B[None], 1, sB[None], np.array([M]), K, N)
    close(np.fromfile(tmp_path / "c.bin", np.float32).reshape(M, N), want, rtol=1e-3)
