// ascq_comm: the host side of the multi-GPU form of the two matmuls (one process per GPU, the GPUs of one box).
//
// A communicator is this rank's position plus every rank's flag block (comm.cuh) as mapped into this process.  How
// the blocks get mapped is the caller's choice -- CUDA IPC handles (ascq_comm_ipc_export / ascq_comm_ipc_open below),
// or any allocator that yields peer-mapped addresses (symmetric memory) -- because the exchange of a few bytes between
// the processes needs a channel only the host program has (MPI, a TCP store, pipes).
// The partition of the work is here too: column blocks of the W8A8 weight, whole groups of the grouped matmul dealt
// out longest first.  The reference's counterpart is the HCCL kernel client (include/adv_api/hccl/hccl.h:82-100
// AllGather, :304-326 Commit / Wait); nothing of it is reused.
#include <algorithm>
#include <cstring>
#include <new>
#include <numeric>
#include <vector>

#include "ascq_internal.h"
#include "sm100_ptx.cuh"

namespace ascq {
namespace {

__device__ int g_comm_status = 0;

// A launch of its own that only takes part in the end-of-step exchange: for a rank that has no work in a step (fewer
// groups than ranks) and for hosts that want the exchange without a matmul.
__global__ void comm_signal_kernel(const CommArgs c, long long waitCycles)
{
    if (threadIdx.x == 0 && !comm_finish(c, 1u, waitCycles)) atomicExch(&g_comm_status, 2);
}

long long g_waitCycles = ptx::kWaitCycles;  // host copy of the limit (for kernels that take it as an argument)

ascq_status check_comm(const ascq_comm* comm)
{
    if (!comm) return fail(ASCQ_ERR_INVALID_ARG, "the communicator must not be NULL");
    if (comm->nranks < 1 || comm->nranks > kCommMaxRanks || comm->rank < 0 || comm->rank >= comm->nranks)
        return fail(ASCQ_ERR_NCCL, "the communicator is not valid (rank %d of %d)", comm->rank, comm->nranks);
    return ASCQ_OK;
}

}  // namespace

CommArgs comm_args(const ascq_comm* comm)
{
    CommArgs a{};
    if (comm) {
        a.rank = comm->rank;
        a.nranks = comm->nranks;
        for (int r = 0; r < comm->nranks; ++r) a.flags[r] = comm->flags[r];
    }
    return a;
}

ascq_status comm_read_status(cudaStream_t st)
{
    int v = 0, zero = 0;
    ASCQ_CUDA_CHECK(cudaMemcpyFromSymbolAsync(&v, g_comm_status, sizeof(int), 0, cudaMemcpyDeviceToHost, st));
    ASCQ_CUDA_CHECK(cudaStreamSynchronize(st));
    if (v != 0) {
        ASCQ_CUDA_CHECK(cudaMemcpyToSymbolAsync(g_comm_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, st));
        return fail(ASCQ_ERR_TIMEOUT, "the wait for the other ranks at the end of a step expired (status %d)", v);
    }
    return ASCQ_OK;
}

}  // namespace ascq

using namespace ascq;

extern "C" size_t ascq_comm_flag_bytes(void) { return sizeof(CommFlags); }

extern "C" ascq_status ascq_comm_create(ascq_comm** out, int rank, int nranks, void* const* flagBlocks)
{
    if (!out) return fail(ASCQ_ERR_INVALID_ARG, "the result pointer must not be NULL");
    *out = nullptr;
    if (nranks < 1 || nranks > kCommMaxRanks) return fail(ASCQ_ERR_INVALID_ARG, "between 1 and %d ranks are supported", kCommMaxRanks);
    if (rank < 0 || rank >= nranks) return fail(ASCQ_ERR_INVALID_ARG, "rank %d is outside [0, %d)", rank, nranks);
    if (!flagBlocks) return fail(ASCQ_ERR_INVALID_ARG, "the table of flag blocks must not be NULL");
    for (int r = 0; r < nranks; ++r) {
        if (!flagBlocks[r]) return fail(ASCQ_ERR_INVALID_ARG, "flag block %d is NULL", r);
        if (reinterpret_cast<uintptr_t>(flagBlocks[r]) & 127u) return fail(ASCQ_ERR_ALIGNMENT, "flag block %d must be 128-byte aligned", r);
    }
    ascq_comm* c = new (std::nothrow) ascq_comm{};
    if (!c) return fail(ASCQ_ERR_INVALID_ARG, "out of host memory");
    c->rank = rank;
    c->nranks = nranks;
    for (int r = 0; r < nranks; ++r) c->flags[r] = static_cast<CommFlags*>(flagBlocks[r]);
    *out = c;
    return ASCQ_OK;
}

extern "C" ascq_status ascq_comm_destroy(ascq_comm* comm)
{
    delete comm;
    return ASCQ_OK;
}

extern "C" ascq_status ascq_comm_rank(const ascq_comm* comm, int* rank, int* nranks)
{
    const ascq_status rc = check_comm(comm);
    if (rc != ASCQ_OK) return rc;
    if (rank) *rank = comm->rank;
    if (nranks) *nranks = comm->nranks;
    return ASCQ_OK;
}

// ---- CUDA IPC route to peer-mapped memory -----------------------------------------------------------------------
extern "C" size_t ascq_comm_ipc_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

extern "C" ascq_status ascq_comm_ipc_export(void* handleOut, const void* devPtr)
{
    if (!handleOut || !devPtr) return fail(ASCQ_ERR_INVALID_ARG, "the handle and the device pointer must not be NULL");
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(devPtr));
    if (e != cudaSuccess) return fail(ASCQ_ERR_NCCL, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
    memcpy(handleOut, &h, sizeof(h));
    return ASCQ_OK;
}

extern "C" ascq_status ascq_comm_ipc_open(void** devPtrOut, const void* handle)
{
    if (!devPtrOut || !handle) return fail(ASCQ_ERR_INVALID_ARG, "the result pointer and the handle must not be NULL");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(ASCQ_ERR_NCCL, "cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
    *devPtrOut = p;
    return ASCQ_OK;
}

extern "C" ascq_status ascq_comm_ipc_close(void* devPtr)
{
    if (!devPtr) return ASCQ_OK;
    const cudaError_t e = cudaIpcCloseMemHandle(devPtr);
    if (e != cudaSuccess) return fail(ASCQ_ERR_NCCL, "cudaIpcCloseMemHandle failed: %s", cudaGetErrorString(e));
    return ASCQ_OK;
}

// ---- the exchange on its own ---------------------------------------------------------------------------------------
extern "C" ascq_status ascq_comm_barrier(ascq_comm* comm, void* stream)
{
    const ascq_status rc = check_comm(comm);
    if (rc != ASCQ_OK) return rc;
    if (comm->nranks == 1) return ASCQ_OK;
    comm_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(comm_args(comm), g_waitCycles);
    ASCQ_CUDA_CHECK(cudaGetLastError());
    return ASCQ_OK;
}

// ---- partition of the work -----------------------------------------------------------------------------------------
extern "C" ascq_status ascq_shard_columns(int N, int nranks, int rank, int* firstColumn, int* columns)
{
    if (nranks < 1 || rank < 0 || rank >= nranks || N < 0) return fail(ASCQ_ERR_INVALID_ARG, "invalid N / rank / nranks");
    if (N % nranks != 0) return fail(ASCQ_ERR_INVALID_ARG, "N = %d is not divisible by the number of ranks %d", N, nranks);
    const int nl = N / nranks;
    if (firstColumn) *firstColumn = rank * nl;
    if (columns) *columns = nl;
    return ASCQ_OK;
}

// Longest group first onto the rank with the fewest rows so far (ties: the lower group index, the lower rank).
extern "C" ascq_status ascq_shard_groups_lpt(const int64_t* groupList_host, int G, int nranks, int* owner)
{
    if (!groupList_host || !owner || G < 0 || nranks < 1) return fail(ASCQ_ERR_INVALID_ARG, "invalid groupList / owner / G / nranks");
    std::vector<int> order(static_cast<size_t>(G));
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return groupList_host[a] > groupList_host[b]; });
    std::vector<int64_t> load(static_cast<size_t>(nranks), 0);
    for (int g : order) {
        if (groupList_host[g] < 0) return fail(ASCQ_ERR_INVALID_ARG, "groupList[%d] is negative", g);
        int best = 0;
        for (int r = 1; r < nranks; ++r)
            if (load[r] < load[best]) best = r;
        owner[g] = best;
        load[best] += groupList_host[g];
    }
    return ASCQ_OK;
}

// ---- wait limit of every bounded device-side wait ------------------------------------------------------------------
extern "C" ascq_status ascq_set_wait_limit_cycles(long long cycles)
{
    if (cycles <= 0) cycles = ptx::kWaitCycles;
    g_waitCycles = cycles;
    ascq_status rc = w8a8_set_wait_cycles(cycles);
    if (rc != ASCQ_OK) return rc;
    return mxfp4_set_wait_cycles(cycles);
}
