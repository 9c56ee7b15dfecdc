// Thin inline-PTX wrappers for the Blackwell (sm_100a) pieces the GEMM kernels use:
// mbarriers with bounded waits, TMA tile loads, tcgen05 MMA / commit / TMEM load, TMEM allocation,
// and the shared-memory / instruction descriptor encodings of tcgen05.mma.
#ifndef ASCQ_SM100_PTX_CUH_
#define ASCQ_SM100_PTX_CUH_

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ascq {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity.  Gives up after the wait limit (SM cycles; about two seconds unless the
// host changed it with ascq_set_wait_limit_cycles) or as soon as *abortFlag (shared memory) is non-zero; on give-up it
// raises *abortFlag -- in both CTAs when the kernel runs as CTA pairs -- and returns false so that every role of the
// CTA leaves its loop instead of spinning for ever.
constexpr long long kWaitCycles = 4000000000LL;  // about two seconds
// One copy per translation unit that includes this header; the host keeps them equal (wait_limit_set in each unit).
static __constant__ long long c_waitCycles = kWaitCycles;

// Raises the abort flag of this CTA and, in a cluster of two, of its partner.  The partner is still resident: no CTA
// of a pair passes the cluster barrier of the teardown before both have left their loops.
__device__ __forceinline__ void raise_abort(volatile int* abortFlag)
{
    *abortFlag = 1;
    uint32_t n, r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n));
    if (n == 2) {
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(const_cast<int*>(abortFlag))), "r"(r ^ 1u));
        asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(1u) : "memory");
    }
}

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abortFlag)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0x3Fu) == 0) {
            if (*abortFlag) return false;
            if (clock64() - t0 > c_waitCycles) {
                raise_abort(abortFlag);
                return false;
            }
        }
    }
    return true;
}

// The same wait for warps that expect to wait long (an epilogue warp waits for a whole tile): between polls the warp
// sleeps, so that it leaves the issue slots and the barrier unit to warps of the same SM that do arithmetic.
__device__ __forceinline__ bool mbar_wait_bounded_sleepy(uint64_t* bar, uint32_t parity, volatile int* abortFlag)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        __nanosleep(128);
        if ((++spins & 0x3Fu) == 0) {
            if (*abortFlag) return false;
            if (clock64() - t0 > c_waitCycles) {
                raise_abort(abortFlag);
                return false;
            }
        }
    }
    return true;
}

// The same wait with acquire semantics at cluster scope: for barriers whose arrivals (from the other CTA of a pair)
// release ordinary shared-memory writes rather than copy-engine bytes.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint64_t* bar, uint32_t parity, volatile int* abortFlag)
{
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait_cluster(bar, parity)) {
        if ((++spins & 0x3Fu) == 0) {
            if (*abortFlag) return false;
            if (clock64() - t0 > c_waitCycles) {
                raise_abort(abortFlag);
                return false;
            }
        }
    }
    return true;
}

// ---- TMA ---------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tile load global -> shared; c0 = innermost coordinate (elements), c1 = row.
__device__ __forceinline__ void tma_load_2d(void* smemDst, const CUtensorMap* m, uint64_t* bar, int c0, int c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smemDst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smemDst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smemDst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
// TMA store of one 2D box from shared memory (bulk async-group completion).  c0 (innermost) times the element size must
// be a multiple of 16 bytes; boxes that reach past the tensor's extents are clipped.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smemSrc, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smemSrc)), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the newest N groups of this thread have finished READING shared memory (the source may be overwritten)
template <int N> __device__ __forceinline__ void bulk_wait_group_read() { asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory"); }
// all groups of this thread have completed (their global writes are done)
__device__ __forceinline__ void bulk_wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void bulk_load(void* smemDst, const void* gsrc, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smemDst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// ---- tcgen05 -----------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Whole-warp calls (.sync.aligned).  ncols: power of two, 32..512.
__device__ __forceinline__ void tmem_alloc(uint32_t* smemResult, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smemResult)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues.
__device__ __forceinline__ void mma_i8(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_mxf4(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate,
                                         uint32_t tmemSfa, uint32_t tmemSfb)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate), "r"(tmemSfa), "r"(tmemSfb)
        : "memory");
}
// half / bfloat16 operands, fp32 accumulator: K = 16 per instruction
__device__ __forceinline__ void mma_f16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_f16_pair(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 8-bit (and 6/4-bit padded) operands with one E8M0 scale per 32 elements: K = 32 per instruction
__device__ __forceinline__ void mma_mxf8(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate,
                                         uint32_t tmemSfa, uint32_t tmemSfb)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate), "r"(tmemSfa), "r"(tmemSfb)
        : "memory");
}
// The mbarrier receives one arrival when every tcgen05 operation issued so far by this thread is done.
__device__ __forceinline__ void tc_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// shared memory -> tensor memory, 32 rows x 128 bits, replicated to the four 32-lane quarters.
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t tmemDst, uint64_t smemDesc)
{
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmemDst), "l"(smemDesc) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread i = lane i of the warp's quarter).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- CTA pairs (cluster of two CTAs driving one tcgen05.mma.cta_group::2) ------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory variable in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t smemAddr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smemAddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// arrive on an mbarrier that may live in the other CTA of the cluster (address from mapa_u32)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t clusterAddr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
// the same without release semantics: for barriers that order nothing but tensor-memory accesses, which tcgen05.wait / fence
// instructions order on their own
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t clusterAddr)
{
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
// TMA tile load whose completion bytes are counted on an mbarrier of either CTA of the pair (no multicast:
// the data lands only in the issuing CTA's shared memory)
__device__ __forceinline__ void tma_load_2d_pair(void* smemDst, const CUtensorMap* m, uint32_t barClusterAddr, int c0, int c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smemDst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(barClusterAddr), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smemResult, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smemResult)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// One MMA over the pair: M = 256 (128 rows of A and of D per CTA), B's N rows split between the two CTAs.
__device__ __forceinline__ void mma_i8_pair(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_mxf4_pair(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate,
                                              uint32_t tmemSfa, uint32_t tmemSfb)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate), "r"(tmemSfa), "r"(tmemSfb)
        : "memory");
}
__device__ __forceinline__ void mma_mxf8_pair(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate,
                                              uint32_t tmemSfa, uint32_t tmemSfb)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate), "r"(tmemSfa), "r"(tmemSfb)
        : "memory");
}
// shared -> tensor memory in both CTAs of the pair (each from its own shared memory, same offsets)
__device__ __forceinline__ void tc_cp_32x128b_warpx4_pair(uint32_t tmemDst, uint64_t smemDesc)
{
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmemDst), "l"(smemDesc) : "memory");
}
// Arrives (once the issued MMAs are done) on the mbarrier at this shared-memory offset in every CTA of `ctaMask`.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar, uint16_t ctaMask)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(ctaMask)
                 : "memory");
}

// ---- descriptors --------------------------------------------------------------------------------
// Shared-memory matrix descriptor of a K-major operand tile whose rows are 128 bytes and 128B-swizzled
// (what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B writes): 8-row groups are 1024 bytes apart.
//   [0,14) start address >> 4, [16,30) leading byte offset >> 4 (unused for swizzled K-major, 1),
//   [32,46) stride byte offset >> 4, [46,48) version = 1, [61,64) layout type (2 = SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smemAddr)
{
    return static_cast<uint64_t>((smemAddr & 0x3FFFFu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Unswizzled K-major descriptor: 8 x 16-byte core matrices, `sbo` bytes between 8-row groups, `lbo` bytes
// between 16-byte column chunks.
__device__ __forceinline__ uint64_t smem_desc_noswizzle(uint32_t smemAddr, uint32_t lbo, uint32_t sbo)
{
    return static_cast<uint64_t>((smemAddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo >> 4) << 16) |
           (static_cast<uint64_t>(sbo >> 4) << 32) | (1ull << 46);
}

// Instruction descriptor of tcgen05.mma (dense): [4,6) D format (1 = f32, 2 = s32), [7,10) A format,
// [10,13) B format, bit 15 / 16 A / B major (0 = K), [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t idesc_i8(uint32_t M, uint32_t N)
{
    return (2u << 4) | (1u << 7) | (1u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);  // int8 x int8 -> int32
}
// One 16-byte store to a multicast address: NVSwitch delivers it to the memory of every GPU bound to the multicast
// object, so an all-gather costs each GPU one copy of its own data on its links instead of one per peer.
__device__ __forceinline__ void multimem_st_v4(void* mcAddr, uint4 v)
{
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mcAddr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// kind::f16: D format 1 = f32; A/B format 0 = half, 1 = bfloat16
__host__ __device__ constexpr uint32_t idesc_f16(uint32_t M, uint32_t N, uint32_t abFmt)
{
    return (1u << 4) | (abFmt << 7) | (abFmt << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}
// Block-scaled descriptor for kind::mxf4: A/B format 1 = E2M1, bit 23 scale format (1 = UE8M0),
// [4,6) B scale-factor id, [29,31) A scale-factor id (which 16-bit half of the 32-bit SF column pair is used).
__host__ __device__ constexpr uint32_t idesc_mxf4(uint32_t M, uint32_t N, uint32_t sfaId, uint32_t sfbId)
{
    return (sfbId << 4) | (1u << 7) | (1u << 10) | ((N >> 3) << 17) | (1u << 23) | ((M >> 4) << 24) | (sfaId << 29);
}

// Block-scaled descriptor for kind::mxf8f6f4: A/B format 0 = E4M3, 1 = E5M2; the scale-factor ids pick one of the
// four bytes of a 32-bit scale column (one byte per 32 elements of K).
__host__ __device__ constexpr uint32_t idesc_mxf8(uint32_t M, uint32_t N, uint32_t aFmt, uint32_t bFmt, uint32_t sfaId, uint32_t sfbId)
{
    return (sfbId << 4) | (aFmt << 7) | (bFmt << 10) | ((N >> 3) << 17) | (1u << 23) | ((M >> 4) << 24) | (sfaId << 29);
}

}  // namespace ptx
}  // namespace ascq
#endif  // ASCQ_SM100_PTX_CUH_
