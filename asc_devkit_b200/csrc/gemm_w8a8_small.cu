// W8A8 matmul with dequant epilogue for a few activation rows (M <= 32): C[M, N] = dequant(A[M, K] x B[N, K]^T), the same
// result bit for bit as the tcgen05 kernel of gemm_w8a8.cu (integer sums are exact in any order; the epilogue is the same
// float arithmetic: bf16(((float(acc) * sB[n]) * sA[m]) + bias[n]), finite overflow saturating), for the shapes where
// that kernel leaves most of the GPU idle: with one or two row tiles there are N / 256 tiles for 148 SMs, and the product
// is bound by reading the N x K weight bytes once.  Reference semantics as for ascq_matmul_w8a8
// (include/adv_api/matmul/matmul.h:79-398 with the vector dequant epilogue of quant_group_matmul_custom.asc:425-454).
//
// Shape of the kernel.  The weight rows play the M side of mma.sync.m16n8k32 (s8 x s8 -> s32) and the activation rows the
// N side (blocks of 8).  A CTA owns 16 weight rows; its warps take the 128-wide k chunks in turn (chunk i * WARPS + w goes
// to warp w) and add their int32 sums through shared memory at the end, so no partial sum ever leaves the SM.  Lane
// (g, c) = (lane / 4, lane % 4) loads the 32 consecutive weights k0 + 32c .. k0 + 32c + 31 of rows g and g + 8 (one 32-byte
// load each) and the 32 activations at the same k of row g of each block: because a dot product does not care in which
// order k is visited, those registers are used as the fragments of four MMAs directly (MMA j takes bytes 8j .. 8j + 7 of
// every lane), with no shuffle and no staging.  Weight loads run DEPTH steps ahead in a register ring.
#include "ascq_internal.h"
#include "numerics.cuh"
#include "tma_host.h"

#include <algorithm>

static_assert(ascq::kW8A8SmallMaxM <= 32, "the kernel is instantiated for at most four blocks of eight rows");

namespace ascq {
namespace {

constexpr int kChunkK = 128;  // k values one warp consumes per step (4 lanes x 32)
constexpr int kRows = 16;     // weight rows (output columns) per CTA

struct SmallI8Params {
    const int8_t* B;   // [N, K]
    const int8_t* A;   // [M, K]
    const float* sA;   // [M]
    const float* sB;   // [N]
    const __nv_bfloat16* bias;  // [N] or null
    __nv_bfloat16* C;  // [M, ldc], written at column colOffset + n
    int M, N, K, ldc, colOffset;
};

struct Word8 {
    uint32_t w[8];
};
__device__ __forceinline__ Word8 ld_stream32(const void* p)
{
    Word8 v;
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7])
                 : "l"(p));
    return v;
}
__device__ __forceinline__ Word8 ld_cached32(const void* p)
{
    Word8 v;
    asm volatile("ld.global.nc.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7])
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void mma16832(int32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MB: blocks of 8 activation rows (M <= 8 * MB); WARPS: warps per CTA, which share the CTA's k range; DEPTH: weight chunks
// in flight per lane; MINB: CTAs per SM the register budget is set for
template <int MB, int WARPS, int DEPTH, int MINB>
__global__ void __launch_bounds__(32 * WARPS, MINB) w8a8_small_kernel(const SmallI8Params p)
{
    // launched programmatically: the next launch in the stream may be scheduled now and waits here for this one's
    // predecessor, so launch latency overlaps the neighbour's tail
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ int32_t red[WARPS][MB * 4 * 32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    constexpr int kStep = WARPS * kChunkK;  // distance between two chunks of the same warp
    constexpr int kEpi = (MB * 4 * 32 + 32 * WARPS - 1) / (32 * WARPS);  // results one thread finishes
    for (int n0 = blockIdx.x * kRows; n0 < p.N; n0 += gridDim.x * kRows) {
        // weight rows of this lane; a row past N is read as row N - 1 and its sums are dropped
        const int rLo = min(n0 + g, p.N - 1), rHi = min(n0 + g + 8, p.N - 1);
        const int8_t* wLo = p.B + static_cast<size_t>(rLo) * p.K + 32 * c;
        const int8_t* wHi = p.B + static_cast<size_t>(rHi) * p.K + 32 * c;
        const int8_t* x = p.A + 32 * c;
        const int kBeg = warp * kChunkK, kEnd = p.K;

        int32_t acc[MB][4];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mb][i] = 0;
        // the epilogue's operands are requested now, so that their latency is not added at the end: value v of the CTA's
        // 16 x (8 MB) results is accumulator element i of block mb in lane l, i.e. weight row n0 + l / 4 (+ 8 for
        // i >= 2) and activation row mb * 8 + 2 * (l % 4) + (i & 1); thread t finishes values t, t + 32 WARPS, ...
        float eSB[kEpi], eSA[kEpi], eBias[kEpi];
#pragma unroll
        for (int e = 0; e < kEpi; ++e) {
            const int v = threadIdx.x + e * 32 * WARPS;
            const int l = v & 31, i = (v >> 5) & 3, mb = v >> 7;
            const int m = mb * 8 + 2 * (l & 3) + (i & 1), n = n0 + (l >> 2) + ((i >> 1) << 3);
            const bool ok = v < MB * 4 * 32 && m < p.M && n < p.N;
            // a missing scale counts as 1.0, as in the tcgen05 kernel
            eSB[e] = (ok && p.sB) ? __ldg(p.sB + n) : 1.0f;
            eSA[e] = (ok && p.sA) ? __ldg(p.sA + m) : 1.0f;
            eBias[e] = (ok && p.bias) ? __bfloat162float(p.bias[n]) : 0.0f;
        }

        Word8 ringLo[DEPTH], ringHi[DEPTH];
#pragma unroll
        for (int d = 0; d < DEPTH; ++d) {
            const int k = kBeg + d * kStep;
            if (k < kEnd) {
                ringLo[d] = ld_stream32(wLo + k);
                ringHi[d] = ld_stream32(wHi + k);
            }
        }
        for (int kBase = kBeg; kBase < kEnd; kBase += DEPTH * kStep) {
#pragma unroll
            for (int d = 0; d < DEPTH; ++d) {
                const int k0 = kBase + d * kStep;
                if (k0 >= kEnd) break;
                // this step's activations first: they are the loads the arithmetic below waits for
                Word8 xv[MB];
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                    const int m = mb * 8 + g;
                    xv[mb] = Word8{};
                    if (m < p.M) xv[mb] = ld_cached32(x + static_cast<size_t>(m) * p.K + k0);
                }
                const Word8 lo = ringLo[d], hi = ringHi[d];
                const int kNext = k0 + DEPTH * kStep;
                if (kNext < kEnd) {
                    ringLo[d] = ld_stream32(wLo + kNext);
                    ringHi[d] = ld_stream32(wHi + kNext);
                }
#pragma unroll
                for (int mb = 0; mb < MB; ++mb)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        mma16832(acc[mb], lo.w[2 * j], hi.w[2 * j], lo.w[2 * j + 1], hi.w[2 * j + 1], xv[mb].w[2 * j], xv[mb].w[2 * j + 1]);
            }
        }
        // the warps' sums (exact integers: the order does not matter)
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int i = 0; i < 4; ++i) red[warp][(mb * 4 + i) * 32 + lane] = acc[mb][i];
        __syncthreads();
#pragma unroll
        for (int e = 0; e < kEpi; ++e) {
            const int v = threadIdx.x + e * 32 * WARPS;
            if (v >= MB * 4 * 32) break;
            int32_t sum = red[0][v];
#pragma unroll
            for (int w = 1; w < WARPS; ++w) sum += red[w][v];
            const int l = v & 31, i = (v >> 5) & 3, mb = v >> 7;
            const int m = mb * 8 + 2 * (l & 3) + (i & 1), n = n0 + (l >> 2) + ((i >> 1) << 3);
            if (m >= p.M || n >= p.N) continue;
            float f = __fmul_rn(__fmul_rn(__int2float_rn(sum), eSB[e]), eSA[e]);
            if (p.bias != nullptr) f = __fadd_rn(f, eBias[e]);
            p.C[static_cast<size_t>(m) * p.ldc + p.colOffset + n] = f32_to_bf16_sat(f);
        }
        __syncthreads();  // `red` is reused by the next block of rows
    }
}

template <int MB, int WARPS, int DEPTH, int MINB> cudaError_t launch_i8(const SmallI8Params& p, int rowBlocks, cudaStream_t st)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(std::min(rowBlocks, MINB * static_cast<int>(sm_count()))), 1, 1);
    cfg.blockDim = dim3(32 * WARPS, 1, 1);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, w8a8_small_kernel<MB, WARPS, DEPTH, MINB>, p);
}

// CTAs per SM the variants are compiled for (the MINB of the launches below)
int ctas_per_sm(int warps) { return warps == 8 ? 2 : 4; }

}  // namespace

// Whether the few-row kernel should take a plain W8A8 call.  Beside the shape limits: every CTA owns 16 weight rows over
// the whole of K, so the launch is one wave of CTAs when N / 16 fits the resident CTAs.  With two waves it still wins
// (measured at N = 11008 to 16384, K = 4096) for at most 16 rows when the second wave is reasonably full; beyond that the
// tcgen05 kernel is as fast or faster.
bool w8a8_small_applies(int M, int N, int K, const void* A, const void* B)
{
    if (M < 1 || M > kW8A8SmallMaxM || K % kChunkK || K < 4 * kChunkK) return false;
    if ((reinterpret_cast<uintptr_t>(A) & 31u) || (reinterpret_cast<uintptr_t>(B) & 31u)) return false;
    // 17 to 32 rows re-read the activations from L1 so often that a large weight (measured: 8192 x 8192, 21 against 17.7 us)
    // is streamed faster by the tcgen05 kernel on its 64-column tiles; small weights (4096 x 4096: 6.8 against 9.4 us) are not
    if (M > 16 && static_cast<long long>(N) * K > (40ll << 20)) return false;
    const int rowBlocks = (N + kRows - 1) / kRows;
    const int warps = rowBlocks <= 2 * static_cast<int>(sm_count()) ? 8 : 4;
    const int slots = ctas_per_sm(warps) * static_cast<int>(sm_count());
    const int waves = (rowBlocks + slots - 1) / slots;
    return waves == 1 || (M <= 16 && waves == 2 && static_cast<double>(rowBlocks) >= 0.6 * waves * slots);
}

ascq_status w8a8_small(void* C, const int8_t* A, const int8_t* B_nk, const float* sA_m, const float* sB_n, const void* bias_bf16,
                       int M, int N, int K, int ldc, int colOffset, cudaStream_t st)
{
    const SmallI8Params p{B_nk, A, sA_m, sB_n, static_cast<const __nv_bfloat16*>(bias_bf16), static_cast<__nv_bfloat16*>(C), M, N, K, ldc, colOffset};
    const int rowBlocks = (N + kRows - 1) / kRows, mb = (M + 7) / 8;
    const bool wide = rowBlocks <= 2 * static_cast<int>(sm_count());  // few row blocks: eight warps share each one's k range
    cudaError_t e;
    if (wide) {
        if (mb <= 1) e = launch_i8<1, 8, 3, 2>(p, rowBlocks, st);
        else if (mb <= 2) e = launch_i8<2, 8, 3, 2>(p, rowBlocks, st);
        else e = launch_i8<4, 8, 3, 2>(p, rowBlocks, st);
    } else {
        if (mb <= 1) e = launch_i8<1, 4, 3, 4>(p, rowBlocks, st);
        else if (mb <= 2) e = launch_i8<2, 4, 3, 4>(p, rowBlocks, st);
        else e = launch_i8<4, 4, 3, 4>(p, rowBlocks, st);
    }
    ASCQ_CUDA_CHECK(e);
    return ASCQ_OK;
}

}  // namespace ascq
