// End-of-step exchange of the sharded matmuls: the device side of ascq_comm.
//
// Every rank (one process per GPU) owns one CommFlags block in memory that all ranks of the box can write
// (peer-mapped).  A sharded matmul stores its part of the result into every rank's output matrix; when the last
// CTA of the launch has finished its stores it advances this rank's epoch, writes the epoch into its slot of every
// peer's block (release, system scope) and waits -- bounded -- until every peer's slot in its OWN block has reached
// the same epoch.  When the kernel ends, every rank's part has therefore landed in this GPU's matrix: no separate
// barrier launch, and nothing is ever loaded from a peer.  The counterpart in the reference is the kernel-side
// AllGather + Commit / Wait of include/adv_api/hccl/hccl.h:82-100, 304-326.
//
// The epoch lives on the device, so the replays of a CUDA graph advance it like fresh launches do.  All ranks must
// issue the same sequence of launches on a communicator.
#ifndef ASCQ_COMM_CUH_
#define ASCQ_COMM_CUH_

#include <cuda_runtime.h>
#include <stdint.h>

namespace ascq {

constexpr int kCommMaxRanks = 8;

struct CommFlags {
    uint32_t arrive[kCommMaxRanks][8];  // arrive[src][0]: last epoch rank `src` has completed; one 32-byte sector per writer
    uint32_t epoch;                     // launches completed on this communicator by the owning rank
    uint32_t ctaDone;                   // CTAs of the running launch that have finished (reset by the last one)
    uint32_t pad[62];
};
static_assert(sizeof(CommFlags) == 512, "the flag block is 512 bytes");

struct CommArgs {
    CommFlags* flags[kCommMaxRanks];  // every rank's block as mapped in this process; flags[rank] is this GPU's own
    int rank, nranks;                 // nranks == 0: no exchange
};

#ifdef __CUDACC__
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Called by ONE thread of every CTA after all threads of the CTA have finished their stores of the launch (a
// __syncthreads() before it; bulk stores waited for with cp.async.bulk.wait_group 0 by the threads that issued them).
// Returns false when the wait for the peers ran out; the caller sets its status word.
__device__ __forceinline__ bool comm_finish(const CommArgs& c, unsigned numCtas, long long waitCycles)
{
    if (c.nranks <= 1) return true;
    CommFlags* mine = c.flags[c.rank];
    __threadfence_system();  // this CTA's stores (observed through the barrier) are ordered before the count
    const unsigned prev = atomicAdd(&mine->ctaDone, 1u);
    if (prev + 1u != numCtas) return true;
    // last CTA of the launch on this GPU
    __threadfence_system();
    mine->ctaDone = 0;
    const uint32_t e = mine->epoch + 1u;
    mine->epoch = e;
    for (int i = 1; i < c.nranks; ++i) {
        int r = c.rank + i;
        if (r >= c.nranks) r -= c.nranks;
        st_release_sys(&c.flags[r]->arrive[c.rank][0], e);
    }
    const long long t0 = clock64();
    for (int i = 1; i < c.nranks; ++i) {
        int r = c.rank + i;
        if (r >= c.nranks) r -= c.nranks;
        const uint32_t* slot = &mine->arrive[r][0];
        uint32_t spins = 0;
        // signed distance, so that the comparison survives the wrap of the 32-bit epoch
        while (static_cast<int32_t>(ld_acquire_sys(slot) - e) < 0) {
            __nanosleep(64);
            if ((++spins & 0x1Fu) == 0 && clock64() - t0 > waitCycles) return false;
        }
    }
    return true;
}
#endif  // __CUDACC__

}  // namespace ascq
#endif  // ASCQ_COMM_CUH_
