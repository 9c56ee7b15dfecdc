// ascq_measure_tensor_rate: the rate at which this GPU's tensor cores retire the matmul kernels' own MMA instructions when
// nothing else is in the way -- operands resident in shared memory, no copies, no epilogue.  The benchmark times it with
// CUDA events and uses the result as the measured ceiling of the int8 and MX-FP4 matmuls (a vendor-independent
// denominator: the driver-measured peak of this pool is a bf16 figure).  No counterpart in the reference.
//
// One cluster of two CTAs per SM pair issues `iters` k-blocks of four tcgen05.mma.cta_group::2 each on a 256 x 256 tile
// (kind::i8, K = 32; or kind::mxf4.block_scale, K = 64, unit scales), alternating between two accumulators, exactly as
// the main loops of gemm_w8a8.cu / gemm_mxfp4.cu do.  The wait for the last MMA is bounded.
#include "ascq_internal.h"
#include "sm100_ptx.cuh"
#include "tma_host.h"

namespace ascq {
namespace {
using namespace ptx;

constexpr int kTileBytes = 128 * 128;  // 128 rows x 128 bytes, 128B-swizzled K-major (one k-block of one CTA's operand rows)
constexpr int kSfBytes = 4 * 512;      // scale chunks (A: 2, B: 2 row tiles x ... shared; all 0x7F = 1.0)
constexpr size_t kSmem = 2 * kTileBytes + 2 * kSfBytes + 1024 + 64;

__device__ int g_peak_status = 0;

template <int KIND>  // 0: kind::i8, 1: kind::mxf4
__global__ void __launch_bounds__(128, 1) tensor_rate_kernel(int iters)
{
    extern __shared__ uint8_t raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sf = smem + 2 * kTileBytes;
    uint64_t* doneBar = reinterpret_cast<uint64_t*>(sf + 2 * kSfBytes);
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(doneBar + 1);
    volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemSlot + 1);
    const uint32_t rank = cluster_ctarank();
    const int warp = threadIdx.x >> 5;

    // operand bytes: a fixed pseudo-random pattern (all-zero operands would draw less power than real ones and flatter the clock)
    for (int i = threadIdx.x; i < 2 * kTileBytes / 4; i += blockDim.x) {
        uint32_t v = (i + blockIdx.x * 7919u) * 2654435761u;
        v ^= v >> 15;
        reinterpret_cast<uint32_t*>(smem)[i] = KIND == 1 ? (v & 0x77777777u) : v;  // fp4: any code is finite
    }
    for (int i = threadIdx.x; i < 2 * kSfBytes / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(sf)[i] = 0x7F7F7F7Fu;
    if (threadIdx.x == 0) {
        mbar_init(doneBar, 1);
        *abortFlag = 0;
        fence_barrier_init();
    }
    fence_proxy_async();
    if (warp == 1) {
        tmem_alloc_pair(tmemSlot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    tc_fence_after();
    const uint32_t tmemBase = *tmemSlot;
    bool ok = true;
    if (warp == 1 && rank == 0 && elect_one()) {
        const uint32_t aAddr = smem_u32(smem);
        const uint64_t descA = smem_desc_sw128(aAddr), descB = smem_desc_sw128(aAddr + kTileBytes);
        const uint32_t sfaCol = tmemBase + 256, sfbCol = sfaCol + 8;   // one 256-column accumulator, then the scale columns
        if constexpr (KIND == 1) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                tc_cp_32x128b_warpx4_pair(sfaCol + 4 * q, smem_desc_noswizzle(smem_u32(sf) + q * 512, 0, 128));
#pragma unroll
                for (int t = 0; t < 2; ++t)
                    tc_cp_32x128b_warpx4_pair(sfbCol + q * 8 + 4 * t, smem_desc_noswizzle(smem_u32(sf) + kSfBytes + (t * 2 + q) * 512, 0, 128));
            }
        }
        for (int it = 0; it < iters; ++it) {
            // int8: two 256-column int32 accumulators, alternating; MX-FP4: one (the second half of tensor memory holds the scales)
            const uint32_t tmemD = tmemBase + (KIND == 0 ? (it & 1) * 256 : 0);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if constexpr (KIND == 0) {
                    mma_i8_pair(tmemD, descA + 2 * k, descB + 2 * k, idesc_i8(256, 256), (it > 1 || k > 0) ? 1u : 0u);
                } else {
                    const uint32_t sfId = (k & 1) * 2;
                    mma_mxf4_pair(tmemD, descA + 2 * k, descB + 2 * k, idesc_mxf4(256, 256, sfId, sfId), (it > 0 || k > 0) ? 1u : 0u,
                                  sfaCol + 4 * (k >> 1), sfbCol + (k >> 1) * 8);
                }
            }
        }
        tc_commit_pair(doneBar, 1);   // arrives on the leader's barrier when every MMA above has retired
        ok = mbar_wait_bounded(doneBar, 0, abortFlag);
    }
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    if (*abortFlag && threadIdx.x == 0) atomicExch(&g_peak_status, 1);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmemBase, 512);
    }
    (void)ok;
}

template <int KIND> ascq_status launch_rate(int iters, cudaStream_t st)
{
    static PerDeviceOnce attrSet;
    const int dev = current_device();
    if (!attrSet.done(dev)) {
        ASCQ_CUDA_CHECK(cudaFuncSetAttribute(tensor_rate_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmem)));
        attrSet.mark(dev);
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(sm_count() / 2 * 2), 1, 1);
    cfg.blockDim = dim3(128, 1, 1);
    cfg.dynamicSmemBytes = kSmem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    ASCQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, tensor_rate_kernel<KIND>, iters));
    ASCQ_CUDA_CHECK(cudaGetLastError());
    return ASCQ_OK;
}
}  // namespace
}  // namespace ascq

using namespace ascq;

// Enqueues the MMA-only kernel; *opsPerLaunch receives the operations (2 x multiply-accumulates) the launch performs.
extern "C" ascq_status ascq_measure_tensor_rate(ascq_dtype operandT, int kBlocks, double* opsPerLaunch, void* stream)
{
    if (kBlocks < 1 || kBlocks > (1 << 22)) return fail(ASCQ_ERR_INVALID_ARG, "kBlocks must be between 1 and 2^22");
    if (operandT != ASCQ_DT_I8 && operandT != ASCQ_DT_FP4X2_E2M1) return fail(ASCQ_ERR_UNSUPPORTED, "operand type must be int8 or fp4x2_e2m1");
    const double perMma = 2.0 * 256.0 * 256.0 * (operandT == ASCQ_DT_I8 ? 32.0 : 64.0);
    if (opsPerLaunch) *opsPerLaunch = perMma * 4.0 * kBlocks * (sm_count() / 2);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return operandT == ASCQ_DT_I8 ? launch_rate<0>(kBlocks, st) : launch_rate<1>(kBlocks, st);
}
