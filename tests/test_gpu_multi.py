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
