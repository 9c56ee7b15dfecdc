"""Two real GPUs, two processes: the sharded W8A8 matmul over CUDA IPC (the route of a C / C++ host).  Skipped on a
box with one GPU; the single-GPU emulation of the same protocol is tests/test_gpu_comm.py, the host-side partition is
covered by the gloo test."""
import os
import subprocess
import sys
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_over_cuda_ipc():
    world = 2
    with tempfile.TemporaryDirectory() as d:
        procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "multi_gpu_ipc_worker.py"), str(r), str(world), d],
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
        outs = []
        for p in procs:
            try:
                o, _ = p.communicate(timeout=240)
            except subprocess.TimeoutExpired:
                p.kill()          # this exact child
                o, _ = p.communicate()
            outs.append(o)
        for r, (p, o) in enumerate(zip(procs, outs)):
            assert p.returncode == 0, f"rank {r} failed:\n{o[-2000:]}"
