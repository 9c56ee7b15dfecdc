"""Two real GPUs, one process per GPU: the sharded W8A8 matmul over CUDA IPC, from Python (tests/multi_gpu_ipc_worker.py)
and from a plain C++ host that sees nothing but include/ascq.h (tests/cpp/sharded_main.cpp).  The GPU tests are skipped
on a box with one GPU; the single-GPU emulation of the same protocol is tests/test_gpu_comm.py, the host-side partition
is covered by the gloo test.  The C++ program is compiled in the CPU suite too, so the header stays consistent."""
import os
import subprocess
import sys
import tempfile

import pytest
import torch

from asc_devkit_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
two_gpus = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")


def run_ranks(argv_of_rank, world):
    procs = [subprocess.Popen(argv_of_rank(r), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()          # this exact child
            o, _ = p.communicate()
        outs.append(o)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed (exit code {p.returncode}):\n{o[-2000:]}"


@pytest.fixture(scope="module")
def sharded_exe(tmp_path_factory):
    out = tmp_path_factory.mktemp("sharded") / "sharded_main"
    libdir = os.path.dirname(L.LIB_PATH)
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA_HOME, "include"),
           os.path.join(ROOT, "tests", "cpp", "sharded_main.cpp"), "-o", str(out), "-L", libdir, "-lascq",
           "-L", os.path.join(CUDA_HOME, "lib64"), "-lcudart", "-lpthread", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{CUDA_HOME}/lib64"]
    subprocess.run(cmd, check=True)
    return str(out)


def test_cpp_host_compiles_against_the_header(sharded_exe):
    """No GPU needed: wrong arguments end with the usage exit code before any CUDA call."""
    assert subprocess.run([sharded_exe]).returncode == 64


@pytest.mark.gpu
@two_gpus
def test_two_python_processes_over_cuda_ipc():
    with tempfile.TemporaryDirectory() as d:
        run_ranks(lambda r: [sys.executable, os.path.join(ROOT, "tests", "multi_gpu_ipc_worker.py"), str(r), "2", d], 2)


@pytest.mark.gpu
@two_gpus
def test_two_cpp_processes_over_cuda_ipc(sharded_exe):
    with tempfile.TemporaryDirectory() as d:
        run_ranks(lambda r: [sharded_exe, str(r), "2", d], 2)


@pytest.mark.gpu
@two_gpus
def test_peer_store_rate_probe(tmp_path, capsys):
    """The link-rate probe behind the multi-GPU bound: stores of config 4's two-rank block (16.8 MB) into the peer's memory
    under a dozen access patterns.  The table is printed (run with -s to see it); the check is only that peer stores work
    and reach a rate of the right order."""
    import shutil
    nvcc = shutil.which("nvcc") or os.path.join(CUDA_HOME, "bin", "nvcc")
    if not os.path.exists(nvcc):
        pytest.skip("nvcc is needed to build the probe")
    exe = tmp_path / "p2p_store_probe"
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-o", str(exe),
                    os.path.join(ROOT, "tests", "cpp", "p2p_store_probe.cu")], check=True, capture_output=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "done" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
    with capsys.disabled():
        print("\n" + r.stdout)
    rates = [float(line.split("us/launch")[1].split("GB/s")[0]) for line in r.stdout.splitlines() if "contiguous" in line and "LOCAL" not in line]
    assert rates and max(rates) > 200.0, rates


@pytest.mark.gpu
@two_gpus
def test_one_process_drives_two_devices():
    """Kernel attributes (opt-in shared memory), the SM count and the built-in scratch address are per device: the same
    process calls the matmuls on device 0, then on device 1, then on device 0 again, and every result is the oracle's."""
    import ctypes as C

    import numpy as np

    from asc_devkit_b200 import ops
    from oracle import oracle as O
    from tests.test_gpu_matmul_mxfp4 import abs_product_sums, check_close, make_case as make_mx_case
    from tests.test_gpu_matmul_w8a8 import make_case

    M, N, K = 384, 512, 512
    A, B, sA, sB, bias = make_case(M, N, K, 11)
    want = O.matmul_w8a8(A, B, sA, sB, bias)
    groups, N4, K4 = [130, 0, 77], 256, 512
    A4, sA4, B4, sB4 = make_mx_case(groups, N4, K4, 12)
    _, want4 = O.group_matmul_mxfp4(A4, sA4, B4, sB4, np.array(groups, np.int64), K4, N4, want_f32=True)
    bound4 = abs_product_sums(A4, sA4, B4, sB4, groups, K4)
    for dev in ("cuda:0", "cuda:1", "cuda:0"):
        with torch.cuda.device(dev):
            t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
            out = torch.full((M, N), -1.0, dtype=torch.bfloat16, device=dev)
            ops.MatmulW8A8(out, t(A), t(B), t(sA), t(sB), torch.from_numpy(bias.view(np.int16).copy()).to(dev).view(torch.bfloat16))
            ops.MatmulStatus()
            assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), want), dev
            # grouped MX-FP4 through the workspace entry point and through the built-in scratch of THIS device
            for no_alloc in (False, True):
                c4 = torch.full((sum(groups), N4), -1.0, dtype=torch.bfloat16, device=dev)
                if no_alloc:
                    gl = (C.c_int64 * len(groups))(*groups)
                    L.check(L.lib().ascq_group_matmul_mxfp4_noalloc(ops._ptr(c4), ops._ptr(dA4), ops._ptr(dsA4), ops._ptr(dB4), ops._ptr(dsB4),
                                                                    gl, len(groups), K4, N4, ops._stream(None)))
                else:
                    dA4, dsA4, dB4, dsB4 = t(A4), t(sA4), t(B4), t(sB4)
                    ops.GroupMatmulMxfp4(c4, dA4, dsA4, dB4, dsB4, groups, K4, N4)
                ops.MatmulStatus()
                check_close(c4.view(torch.int16).cpu().numpy().view(np.uint16), want4, f"{dev} no_alloc={no_alloc}", bound4, K4)
