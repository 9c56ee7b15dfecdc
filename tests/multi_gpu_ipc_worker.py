"""One rank of the two-process test of the sharded W8A8 matmul over CUDA IPC (run by tests/test_gpu_multi.py).

    python tests/multi_gpu_ipc_worker.py RANK WORLD DIR

This is the route a plain C / C++ host takes, without torch's symmetric memory: every rank cudaMalloc's its flag
block and its output matrix, exports both with ascq_comm_ipc_export, the handle bytes travel through files in DIR
(the "channel only the host program has"), the peers open them with ascq_comm_ipc_open, and ascq_comm_create gets the
mapped flag blocks.  Then two sharded steps; after each, this rank's matrix must be the oracle's whole result.
Exit code 0 on success.  Host-side waits are bounded (60 s) so that a rank that died cannot hang the other.
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def wait_for(path, limit=60.0):
    t0 = time.time()
    while not os.path.exists(path):
        if time.time() - t0 > limit:
            raise TimeoutError(path)
        time.sleep(0.01)


def publish(d, name, data: bytes):
    tmp = os.path.join(d, name + ".tmp")
    with open(tmp, "wb") as f:
        f.write(data)
    os.rename(tmp, os.path.join(d, name))


def host_barrier(d, tag, rank, world):
    publish(d, f"{tag}.{rank}", b"1")
    for r in range(world):
        wait_for(os.path.join(d, f"{tag}.{r}"))


def main():
    rank, world, d = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    import torch
    from cuda import cudart
    from asc_devkit_b200 import ops
    from oracle import oracle as O

    torch.cuda.set_device(rank)
    dev = f"cuda:{rank}"

    def ck(res):
        assert int(res[0]) == 0, res
        return res[1] if len(res) > 1 else None

    M, N, K = 512, 1024, 512
    rng = np.random.default_rng(42)      # the same inputs on every rank
    A = np.clip(np.rint(rng.normal(0, 30, (M, K))), -127, 127).astype(np.int8)
    B = rng.integers(-127, 128, (N, K)).astype(np.int8)
    sA = rng.uniform(0.005, 0.02, M).astype(np.float32)
    sB = rng.uniform(0.001, 0.01, N).astype(np.float32)
    bias = O.f32_to_bf16_bits(rng.normal(0, 0.1, N).astype(np.float32))
    want = O.matmul_w8a8(A, B, sA, sB, bias)

    fb = ops.Comm.flag_bytes()
    flags = ck(cudart.cudaMalloc(fb))
    out = ck(cudart.cudaMalloc(M * N * 2))
    ck(cudart.cudaMemset(flags, 0, fb))
    ck(cudart.cudaMemset(out, 0xFF, M * N * 2))
    ck(cudart.cudaDeviceSynchronize())

    class Raw:   # just enough of a tensor for ops.IpcExport
        def __init__(self, p):
            self.p = p

        def data_ptr(self):
            return int(self.p)

    publish(d, f"flags.{rank}", ops.IpcExport(Raw(flags)))
    publish(d, f"out.{rank}", ops.IpcExport(Raw(out)))
    flag_ptrs, out_ptrs = [0] * world, [0] * world
    for r in range(world):
        if r == rank:
            flag_ptrs[r], out_ptrs[r] = int(flags), int(out)
            continue
        for nm, table in (("flags", flag_ptrs), ("out", out_ptrs)):
            path = os.path.join(d, f"{nm}.{r}")
            wait_for(path)
            with open(path, "rb") as f:
                table[r] = ops.IpcOpen(f.read())
    host_barrier(d, "mapped", rank, world)      # every block is zeroed and mapped before anyone signals
    comm = ops.Comm(rank, world, flag_ptrs)

    c0, nl = ops.ShardColumns(N, world, rank)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    dA, dB, dsA, dsB = t(A), t(B[c0:c0 + nl]), t(sA), t(sB[c0:c0 + nl])
    dbias = torch.from_numpy(bias[c0:c0 + nl].view(np.int16).copy()).to(dev).view(torch.bfloat16)
    host = np.empty((M, N), np.uint16)
    for step in range(2):
        torch.cuda.synchronize()
        host_barrier(d, f"step{step}", rank, world)
        ops.MatmulW8A8Sharded(comm, out_ptrs, dA, dB, dsA, dsB, dbias, N=N)
        ops.MatmulStatus()                      # synchronises; raises if the wait for the peer ran out
        ck(cudart.cudaMemcpy(host.ctypes.data, out, M * N * 2, cudart.cudaMemcpyKind.cudaMemcpyDeviceToHost))
        if not np.array_equal(host, want):
            bad = np.argwhere(host != want)
            print(f"rank {rank} step {step}: {len(bad)} elements differ, first at {bad[0]}", file=sys.stderr)
            return 1
        host_barrier(d, f"read{step}", rank, world)   # nobody overwrites a matrix its owner is still reading
    comm.destroy()
    print(f"rank {rank}: ok")
    return 0


if __name__ == "__main__":
    sys.exit(main())
