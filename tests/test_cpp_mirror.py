"""The C++ host mirror (include/ascq_ascendc.hpp) compiles against the C ABI and, on a GPU, gives the oracle's bits.

The driver program tests/cpp/ascendc_mirror_main.cpp is built with g++ here; operands travel through files."""
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


@pytest.fixture(scope="module")
def mirror_exe(tmp_path_factory):
    out = tmp_path_factory.mktemp("mirror") / "ascendc_mirror_main"
    libdir = os.path.dirname(L.LIB_PATH)
    cmd = ["g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA_HOME, "include"),
           os.path.join(ROOT, "tests", "cpp", "ascendc_mirror_main.cpp"), "-o", str(out), "-L", libdir, "-lascq",
           "-L", os.path.join(CUDA_HOME, "lib64"), "-lcudart", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{CUDA_HOME}/lib64"]
    subprocess.run(cmd, check=True)
    return str(out)


def run(exe, op, d):
    r = subprocess.run([exe, op, str(d)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr + r.stdout
    return r.stdout


def test_mirror_compiles_and_reports_reference_asserts(mirror_exe, tmp_path):
    """scaleCount != offsetCount is an ASCENDC_ASSERT in the reference (ascend_quant.h:252-347); here ascq::Error."""
    assert "status=1" in run(mirror_exe, "bad_args", tmp_path)


@pytest.mark.gpu
def test_mirror_quant_tensor(mirror_exe, tmp_path):
    rng = np.random.default_rng(5)
    n = 5000 * 32
    src = rng.uniform(-70, 70, n).astype(np.float16)
    src.tofile(tmp_path / "src.bin")
    np.array([n], np.uint32).tofile(tmp_path / "dims.bin")
    np.array([2.0, 0.9], np.float32).tofile(tmp_path / "scalars.bin")
    run(mirror_exe, "quant_tensor", tmp_path)
    want = O.ascend_quant(src, O.F16, policy=O.PER_TENSOR, m=1, n=n, scaleScalar=2.0, offsetScalar=0.9, hasOffset=True)
    got = np.fromfile(tmp_path / "dst.bin", np.int8)
    assert np.array_equal(got, want)


@pytest.mark.gpu
def test_mirror_quant_channel(mirror_exe, tmp_path):
    rng = np.random.default_rng(6)
    m, n = 96, 640
    src = rng.uniform(-9, 9, (m, n)).astype(np.float16)
    scale = rng.uniform(0.5, 14, n).astype(np.float16)
    offset = rng.uniform(-3, 3, n).astype(np.float16)
    for a, f in ((src, "src"), (scale, "scale"), (offset, "offset")):
        a.tofile(tmp_path / f"{f}.bin")
    np.array([m * n, n], np.uint32).tofile(tmp_path / "dims.bin")
    run(mirror_exe, "quant_channel", tmp_path)
    want = O.ascend_quant(src, O.F16, policy=O.PER_CHANNEL, m=m, n=n, scale=scale, offset=offset, scaleT=O.F16, hasOffset=True)
    got = np.fromfile(tmp_path / "dst.bin", np.int8).reshape(m, n)
    assert np.array_equal(got, want)


@pytest.mark.gpu
def test_mirror_dequant_channel(mirror_exe, tmp_path):
    rng = np.random.default_rng(7)
    m, n, cal = 40, 72, 70
    stride = O.dequant_dst_stride(n, O.BF16)
    src = rng.integers(-2**20, 2**20, (m, n), dtype=np.int32)
    scale = rng.uniform(1e-4, 1e-2, n).astype(np.float32)
    src.tofile(tmp_path / "src.bin")
    scale.tofile(tmp_path / "scale.bin")
    np.array([m, n, cal, stride], np.uint32).tofile(tmp_path / "dims.bin")
    run(mirror_exe, "dequant_channel", tmp_path)
    want = O.ascend_dequant(src, O.I32, O.BF16, policy=O.PER_CHANNEL, m=m, n=n, calCount=cal, scale=scale)
    got = np.fromfile(tmp_path / "dst.bin", np.uint16).reshape(m, stride)
    assert np.array_equal(got, want.view(np.uint16))


@pytest.mark.gpu
def test_mirror_antiquant_channel(mirror_exe, tmp_path):
    rng = np.random.default_rng(8)
    K, N = 64, 512
    src = rng.integers(-128, 128, (K, N), dtype=np.int8)
    scale = O.f32_to_bf16_bits(rng.uniform(0.01, 2, N).astype(np.float32))
    offset = O.f32_to_bf16_bits(rng.uniform(-8, 8, N).astype(np.float32))
    for a, f in ((src, "src"), (scale, "scale"), (offset, "offset")):
        a.tofile(tmp_path / f"{f}.bin")
    np.array([K, N], np.uint32).tofile(tmp_path / "dims.bin")
    run(mirror_exe, "antiquant_channel", tmp_path)
    want = O.ascend_antiquant(src, O.I8, O.BF16, policy=O.PER_CHANNEL, m=K, n=N, scale=scale, offset=offset, scaleT=O.BF16)
    got = np.fromfile(tmp_path / "dst.bin", np.uint16).reshape(K, N)
    assert np.array_equal(got, want.view(np.uint16))


@pytest.mark.gpu
def test_mirror_unified_quantize_per_token(mirror_exe, tmp_path):
    rng = np.random.default_rng(9)
    m, n = 40, 320
    src = rng.uniform(-9, 9, (m, n)).astype(np.float16)
    scale = rng.uniform(0.5, 14, m).astype(np.float32)
    offset = rng.uniform(-3, 3, m).astype(np.float32)
    for a, f in ((src, "src"), (scale, "scale"), (offset, "offset")):
        a.tofile(tmp_path / f"{f}.bin")
    np.array([m, n], np.uint32).tofile(tmp_path / "dims.bin")
    run(mirror_exe, "quantize_token", tmp_path)
    want = O.quantize(src, O.F16, policy=O.PER_TOKEN, m=m, n=n, scale=scale, offset=offset, scaleT=O.F32, hasOffset=True)
    assert np.array_equal(np.fromfile(tmp_path / "dst.bin", np.int8).reshape(m, n), want)
