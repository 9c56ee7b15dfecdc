// ascq_matmul_w8a8: int8 x int8 -> int32 matmul on the 5th-generation tensor cores (tcgen05.mma kind::i8)
// with the per-channel x per-token dequantisation, bias and bf16 cast fused into the epilogue.
//
// Data layout in HBM: A [M,K] int8 row-major, B [N,K] int8 row-major (both K-major), C [M,ldc] bf16.
// One persistent CTA per SM walks output tiles of 128 x BN.  Per k-block of 128 bytes a TMA producer warp
// loads a 128x128 A tile and a BNx128 B tile into a 128B-swizzled shared-memory stage; one thread of the
// MMA warp issues four tcgen05.mma (K = 32 each) accumulating int32 in tensor memory; tcgen05.commit frees
// the stage.  The accumulator is double buffered (2 x BN TMEM columns) so the four epilogue warps drain
// tile i (tcgen05.ld -> fp32 scale, scale, bias -> bf16 -> 64-byte row segments to global) while the
// tensor cores work on tile i+1.
//
// Roofline: dense int8 tensor throughput; 2*M*N*K operations per call.  Algorithmic HBM bytes are
// M*K + N*K + 2*M*N (operands are re-read from L2 across tiles).
//
// Every mbarrier wait is bounded; on expiry the CTA raises an abort flag, all roles leave their loops, the
// TMEM allocation is released and a device status word reports the timeout.
#include <cuda_bf16.h>

#include <atomic>
#include <type_traits>
#include <cstdlib>
#include <cstring>

#include "ascq_internal.h"
#include "numerics.cuh"
#include "elementwise.cuh"
#include "sm100_ptx.cuh"
#include "comm.cuh"
#include "tma_host.h"

namespace ascq {
namespace {

using namespace ptx;

constexpr int kBM = 128;
constexpr int kBK = 128;        // bytes == int8 elements per k-block: one 128B swizzle atom
constexpr int kUmmaK = 32;      // K per tcgen05.mma for 8-bit operands
constexpr int kEpiWarps = 8;    // two warps per TMEM lane quarter, alternating 32-column chunks
constexpr int kMaxPeers = 8;    // output buffers one launch can write (this GPU's and its peers')
constexpr int kStagePitch = 144;  // bytes per staged row: 128 B of bf16 + 16 B pad (conflict-free both ways)
constexpr int kThreads = 64 + 32 * kEpiWarps;  // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2..9: epilogue
// Staging bytes of one epilogue warp: 16 padded rows for the per-thread stores (16 x 144), or a 1024-byte aligned block of
// 2 KiB for TMA stores -- a region of 2.5 KiB that starts at a multiple of 512 bytes holds either, so a warp never
// touches another warp's staging bytes whichever path the tile it works on takes.
constexpr int kWarpStageBytes = 2560;

__device__ int g_w8a8_status = 0;  // 0 ok, 1 = a bounded wait expired

// PAIR: two CTAs of a cluster drive one tcgen05.mma.cta_group::2 on a 256 x BN tile; each CTA loads its 128 rows of A
// and its half (BN/2 rows) of B, so every byte of B is fetched from L2 once per pair instead of once per CTA.
// CONV (weight-only-quantised matmul): the stage also holds this CTA's int8 rows of B (64 bytes per row and k-block);
// four converter warps turn them into the half / bfloat16 tile the MMAs read.
constexpr int kConvWarps = 4;
template <int BN, bool PAIR, bool CONV = false> struct Cfg {
    static constexpr int kBRows = PAIR ? BN / 2 : BN;          // rows of B this CTA loads
    static constexpr int kABytes = kBM * kBK;
    static constexpr int kBBytes = kBRows * kBK;
    static constexpr int kBqBytes = CONV ? kBRows * (kBK / 2) : 0;
    static constexpr int kStageBytes = kABytes + kBBytes + kBqBytes;
    static constexpr int kStages = CONV ? 4 : (192 * 1024) / kStageBytes;  // 4 x 48 KiB, or 6 x 32 KiB; CONV: 4 x 40 KiB
    static constexpr int kThreadsCta = kThreads + (CONV ? 32 * kConvWarps : 0);
    static constexpr int kTmemCols = 2 * BN;  // two accumulators
    static constexpr int kEpiBytes = 2 * 3 * BN * 4;  // per accumulator: sB[BN], bias[BN] (fp32 or int32 bits), aux[BN]
    static constexpr int kOutBytes = kEpiWarps * kWarpStageBytes;  // per epilogue warp: 16 rows x 64 16-bit columns
    static constexpr size_t kSmemBytes =
        static_cast<size_t>(kStages) * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + kEpiBytes + kOutBytes;
};

struct Params {
    __nv_bfloat16* C[kMaxPeers];  // output buffers (own first); every one gets this launch's [M, N] block
    int multicast;  // C[0] is a multicast address: one multimem store reaches every GPU's matrix
    int nPeers, colOffset, firstPeer;  // block goes to columns [colOffset, colOffset + N); stores start at buffer firstPeer
    const float* sA;
    const float* sB;
    const __nv_bfloat16* bias;
    int32_t* accDump;
    int M, N, K, ldc;
    int tilesM, tilesN;
    // Work items: items [0, fullTiles) are whole tiles; from there on two items share one tile, each taking half of
    // its columns (the tail of a pair-shaped launch, so that the last, partly filled wave lasts half as long).
    // (Half items at the head of a launch that ships its tiles to other GPUs were tried and lost: the first results of
    // a launch are late because its operands come from HBM cold, not because the tile is large.)
    int fullTiles, workItems;
    int aBoxShort;  // bytes one load of A delivers less than a whole 128-row box (a matrix of fewer than 16 rows is loaded through a 16-row box)
    int tmaStore;  // 16-bit result, suitably aligned buffers: the epilogue hands its staged rows to TMA stores (one per buffer)
    int narrowBox;  // one output matrix: 32 x 32 boxes (tmapC.cNarrow) instead of 64 columns x 16 rows
    CommArgs comm;      // sharded form: end-of-step exchange with the other ranks (nranks == 0: none)
#ifdef ASCQ_TRACE
    unsigned long long* trace;  // diagnostic builds: 16 time stamps (ns) per CTA, see trace_stamp
#endif
    int stopAfter;      // test hook: the producer stops after this many k-blocks (< 0: never), so that a bounded wait runs out
    // fixpipe-style epilogue (EPI == kEpiFixpipe): C is fp16 = half(acc + biasI32[n]) scaled by quantVec[n] or quantScalar
    const int32_t* biasI32;
    const uint64_t* quantVec;   // low word: fp32 bits, of which the hardware keeps sign, exponent and 10 mantissa bits
    float quantScalar;
    // kEpiRequant: C is int8 / uint8; quantVec[n] or quantBits is the whole 64-bit fixpipe parameter (scale bits 31:13,
    // shift count 35:32, shift enable 36, offset 45:37, signed-result flag 46)
    unsigned long long quantBits;
    // kEpiFloat: operand format (0 = half, 1 = bfloat16) and output type (0 = half, 1 = bfloat16, 2 = float)
    // kEpiDequant: outKind 0 = bfloat16 (ascq_matmul_w8a8), 1 = half; act 1 = FasterGelu before the cast
    uint32_t abFmt;
    int outKind;
    int act;
    // CONV: AscendAntiQuant operands of the int8 weight: per-row (of B_nk) tensors of the operand type, or two scalars
    const void* aqScale;
    const void* aqOffset;
    float aqScaleScalar, aqOffsetScalar;
    int aqHasOffset;
};
// Diagnostic builds (-DASCQ_TRACE) record where the time of a launch goes: slot 0 set-up done, 1 + 2i accumulator of
// the CTA's i-th item ready, 2 + 2i its stores issued (i < 5), 12 all stores performed, 13 CTA done (after the exchange).
#ifdef ASCQ_TRACE
__device__ __forceinline__ void trace_stamp(const Params& p, int slot)
{
    if (p.trace != nullptr && slot < 16) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.trace[blockIdx.x * 16 + slot] = t;
    }
}
#define ASCQ_STAMP(p, slot) trace_stamp(p, slot)
// slots 8..11 (first item of the CTA, first 64-column chunk of warp 2), SM cycles since the accumulator was ready:
// 8 tensor-memory loads done, 9 arithmetic done, 10 staged and handed to the copy engine, 11 end of the item's epilogue
#define ASCQ_CYCLES(p, slot, t0) do { if ((p).trace != nullptr) (p).trace[blockIdx.x * 16 + (slot)] = static_cast<unsigned long long>(clock64() - (t0)); } while (0)
#else
#define ASCQ_STAMP(p, slot) ((void)0)
#define ASCQ_CYCLES(p, slot, t0) ((void)0)
#endif

// Grouped launch (ascq_group_matmul_w8a8): rows of A per group; row tiles never straddle two groups.  G == 0: plain matmul.
constexpr int kMaxGroupsInline = 128;
struct GroupTable {
    int G;
    int rows[kMaxGroupsInline];
};
// Where a row tile lives: first row in A / C, first row that no longer belongs to it, row offset of its group's weights
// in B (and index offset into the per-channel parameters).
struct RowTile {
    int m0, rowEnd, nBase;
};
// 128-row entry `idx` of the row-tile list: groups in order, ceil(rows / stepRows) * (stepRows / 128) entries per group
// (stepRows = 256 when CTA pairs work on 256-row tiles; the second half of a pair's tile may be empty).
__device__ __forceinline__ RowTile group_row_tile(const GroupTable& gt, int N, int stepRows, int idx)
{
    int start = 0;
    const int per = stepRows / 128;
    for (int g = 0; g < gt.G; ++g) {
        const int mg = gt.rows[g];
        const int n = (mg + stepRows - 1) / stepRows * per;
        if (idx < n) {
            const int first = start + idx * 128;
            const int left = mg - idx * 128;
            return RowTile{first, first + (left <= 0 ? 0 : (left < 128 ? left : 128)), g * N};
        }
        idx -= n;
        start += mg;
    }
    return RowTile{start, start, 0};
}

// Work item -> tile, first column inside the tile, columns of the item.
struct Item {
    int tile, nOff, nCols;
};
template <int BN> __device__ __forceinline__ Item decode_item(const Params& p, int w)
{
    if (w < p.fullTiles) return Item{w, 0, BN};
    const int h = w - p.fullTiles;
    return Item{p.fullTiles + (h >> 1), (h & 1) * (BN / 2), BN / 2};
}
// FasterGelu in the reference's operation order (impl/adv_api/detail/activation/gelu/gelu_impl.h:134-166): x * -1.702, exp,
// + 1, x / that, in fp32.  The exponential and the division are the special-function unit's (ex2.approx, rcp.approx: a few
// units in the last place of fp32, far below one step of the 16-bit result); the reference's own Exp is a hardware
// approximation that nothing in its tree specifies bit for bit.
__device__ __forceinline__ float faster_gelu(float x)
{
    const float e = __expf(__fmul_rn(x, -1.702f));
    return __fdividef(x, __fadd_rn(e, 1.0f));
}
constexpr int kEpiDequant = 0;  // bf16(((float(acc) * sB[n]) * sA[m]) + bias[n])
constexpr int kEpiDequantAct = 4;  // the same with an optional FasterGelu and a half or bfloat16 result (grouped matmul)
constexpr int kEpiFixpipe = 1;  // SetQuantScalar / SetQuantVector of the reference's Matmul (DEQF16)
constexpr int kEpiFloat = 2;    // half / bfloat16 operands (kind::f16), fp32 accumulator cast to the output type
constexpr int kEpiRequant = 3;  // SetQuantScalar / SetQuantVector with an int8 / uint8 result ((V)REQ8)
constexpr int kBytePitch = 80;  // bytes per staged row of a byte-typed result: 64 B + 16 B pad

// Converter warps of the weight-only-quantised matmul.  Warp w takes the k-blocks that land in pipeline stage w (there
// are as many stages as converter warps), so four k-blocks are being converted at any time and the fixed costs of a
// hand-over (barrier wake-up, proxy fence, arrive) are paid once per 8192 weights.  Per pass of 8 rows, lane l owns row
// l/4 and the 16-byte segment l%4 of the row's 64 int8 values; the 32 bytes of half / bfloat16 they become go into the
// 128B-swizzled tile the MMAs read (16-byte chunk c of row r lives at chunk c ^ (r % 8)).
template <typename C, int BN, typename CT, typename Dst, bool HAS_OFF>
__device__ __forceinline__ void convert_tiles(const Params& p, uint8_t* smem, float* rowParams, uint64_t* fullQ, uint64_t* convDone,
                                              volatile int* abortFlag, int w, int lane, uint32_t rank, int unit, int numUnits,
                                              int numTiles, int kBlocks)
{
    static_assert(C::kStages == kConvWarps, "one converter warp per pipeline stage");
    float* myScale = rowParams + w * 2 * C::kBRows;  // this warp's copy of the tile's 128 row scales, then 128 offsets
    float* myOffset = myScale + C::kBRows;
    const int seg = lane & 3;
    const int s = w;  // the stage this warp serves
    uint32_t it = 0;
    bool ok = true;
    for (int tile = unit; tile < numTiles && ok; tile += numUnits) {
        const int n0 = (tile / p.tilesM) * BN + static_cast<int>(rank) * C::kBRows;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < C::kBRows / 32; ++i) {
            const int r = i * 32 + lane, n = n0 + r;
            float fs = p.aqScaleScalar, fo = p.aqOffsetScalar;
            if (p.aqScale != nullptr) {
                fs = 0.f;
                fo = 0.f;
                if (n < p.N) {
                    fs = to_f32<Dst>(static_cast<const Dst*>(p.aqScale)[n]);
                    if (HAS_OFF) fo = to_f32<Dst>(static_cast<const Dst*>(p.aqOffset)[n]);
                }
            }
            myScale[r] = fs;
            myOffset[r] = fo;
        }
        __syncwarp();
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
            if (static_cast<int>(it % C::kStages) != s) continue;
            const uint32_t ph = (it / C::kStages) & 1;
            if (!(ok = mbar_wait_bounded(&fullQ[s], ph, abortFlag))) break;
            const uint8_t* bq = smem + s * C::kStageBytes + C::kABytes + C::kBBytes;
            uint8_t* bc = smem + s * C::kStageBytes + C::kABytes;
#pragma unroll 4
            for (int pass = 0; pass < C::kBRows / 8; ++pass) {
                const int r = pass * 8 + (lane >> 2);
                const uint4 raw = *reinterpret_cast<const uint4*>(bq + r * (kBK / 2) + seg * 16);
                const CT sc = Ct<CT>::from_f32(myScale[r]), of = Ct<CT>::from_f32(myOffset[r]);
                uint4 lo, hi;
                antiquant16<CT, Dst, HAS_OFF>(raw, sc, of, lo, hi);
                uint8_t* row = bc + r * kBK;
                *reinterpret_cast<uint4*>(row + (((2 * seg) ^ (r & 7)) << 4)) = lo;
                *reinterpret_cast<uint4*>(row + (((2 * seg + 1) ^ (r & 7)) << 4)) = hi;
            }
            // the tensor cores read shared memory through the async proxy: order these writes before it
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&convDone[s]), 0));  // the leader's barrier
        }
    }
}

// Tensor maps of the output matrices (TMA stores): one per buffer, this GPU's and its peers'.
struct OutMaps {
    CUtensorMap m[kMaxPeers];
    CUtensorMap bHalf;  // B with a box of half the rows: what a CTA loads for a half-tile work item (pair shape)
    CUtensorMap cNarrow;  // output matrix 0 with a 32-column x 32-row box and the 64B swizzle (single-matrix launches)
};


template <int BN, bool PAIR, int EPI, bool CONV = false>
__global__ void __launch_bounds__(Cfg<BN, PAIR, CONV>::kThreadsCta, 1)
w8a8_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
            const __grid_constant__ OutMaps tmapC, const Params p, const __grid_constant__ GroupTable gt)
{
    using C = Cfg<BN, PAIR, CONV>;
    static_assert(!CONV || (PAIR && EPI == kEpiFloat), "the converting variant is built for CTA pairs and kind::f16 only");
    extern __shared__ uint8_t smem_raw[];
    // stage buffers need 1024-byte alignment for the 128B swizzle pattern
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // [stages][output staging, 1024-aligned for swizzled TMA stores][barriers, 256 B][per-column epilogue parameters]
    uint8_t* outStage = smem + C::kStages * C::kStageBytes;  // [kEpiWarps][kWarpStageBytes]
    uint64_t* bars = reinterpret_cast<uint64_t*>(outStage + C::kOutBytes);
    uint64_t* fullBar = bars;                      // [kStages] TMA -> MMA
    uint64_t* emptyBar = bars + C::kStages;        // [kStages] MMA -> TMA
    uint64_t* tmemFull = bars + 2 * C::kStages;    // [2] MMA -> epilogue
    uint64_t* tmemEmpty = tmemFull + 2;            // [2] epilogue -> MMA
    uint32_t* tmemBaseSlot = reinterpret_cast<uint32_t*>(tmemEmpty + 2);
    volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemBaseSlot + 1);
    uint64_t* fullQ = bars + 2 * C::kStages + 5;   // [kStages] CONV: this CTA's int8 rows have landed
    uint64_t* convDone = fullQ + C::kStages;       // [kStages] CONV: converter warps of both CTAs -> MMA (leader's is used)
    float* epiScale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);  // [2][3][BN]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int numTiles = p.workItems;  // loop bound of every role (work items; whole tiles unless the tail is split)
    const int kBlocks = (p.K + kBK - 1) / kBK;
    // work unit = CTA (single) or cluster of two CTAs (PAIR); rank = position inside the pair, rank 0 issues the MMAs
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const int unit = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int numUnits = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    constexpr int kTileM = PAIR ? 2 * kBM : kBM;
    // this CTA's 128 rows of row tile `mt`: a regular grid over M, or the group-aligned list of a grouped launch
    auto row_tile = [&](int mt) -> RowTile {
        if (gt.G == 0) return RowTile{mt * kTileM + static_cast<int>(rank) * kBM, p.M, 0};
        return group_row_tile(gt, p.N, kTileM, mt * (kTileM / kBM) + static_cast<int>(rank));
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(&fullBar[s], 1);
            mbar_init(&emptyBar[s], 1);
            if constexpr (CONV) {
                mbar_init(&fullQ[s], 1);
                mbar_init(&convDone[s], 2);  // one converter warp of each CTA serves the stage
            }
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tmemFull[a], 1);
            mbar_init(&tmemEmpty[a], PAIR ? 2 * kEpiWarps : kEpiWarps);  // one arrival per epilogue warp (of both CTAs)
        }
        *abortFlag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmapA);
        prefetch_tensormap(&tmapB);
        if (p.tmaStore)
            for (int b = 0; b < p.nPeers; ++b) prefetch_tensormap(&tmapC.m[b]);
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            tmem_alloc_pair(tmemBaseSlot, C::kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmemBaseSlot, C::kTmemCols);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) {  // the peer's barriers must be initialised before anything is signalled across the pair
        cluster_arrive();
        cluster_wait();
    }
    tc_fence_after();
    const uint32_t tmemBase = *tmemBaseSlot;
    // Programmatic dependent launch, both ways: the launch after this one may bring its CTAs onto SMs as they become
    // free and run its own set-up there; and everything above ran while the launch before this one was still
    // draining -- nothing below may touch global memory before that launch has completed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 64) ASCQ_STAMP(p, 0);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            uint32_t it = 0;
            bool ok = true;
            for (int w = unit; w < numTiles && ok; w += numUnits) {
                const Item item = decode_item<BN>(p, w);
                const int tile = item.tile;
                const RowTile rt = row_tile(tile % p.tilesM);
                const int m0 = rt.m0;
                // rows of B this CTA loads: its half of the item's columns (of its group's weights)
                const int n0 = rt.nBase + (tile / p.tilesM) * BN + item.nOff + (PAIR ? static_cast<int>(rank) * (item.nCols / 2) : 0);
                for (int kb = 0; kb < kBlocks; ++kb, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    if (p.stopAfter >= 0 && it >= static_cast<uint32_t>(p.stopAfter)) {  // test hook: the consumers' waits run out
                        ok = false;
                        break;
                    }
                    if (!(ok = mbar_wait_bounded(&emptyBar[s], ph ^ 1, abortFlag))) break;
                    uint8_t* sa = smem + s * C::kStageBytes;
                    if constexpr (CONV) {
                        // A of both CTAs on the leader's barrier; this CTA's int8 rows of B on its own barrier, where
                        // its converter warps wait for them
                        if (rank == 0) mbar_arrive_expect_tx(&fullBar[s], 2 * C::kABytes);
                        const uint32_t leaderBar = mapa_u32(smem_u32(&fullBar[s]), 0);
                        tma_load_2d_pair(sa, &tmapA, leaderBar, kb * kBK, m0);
                        mbar_arrive_expect_tx(&fullQ[s], C::kBqBytes);
                        tma_load_2d(sa + C::kABytes + C::kBBytes, &tmapB, &fullQ[s], kb * (kBK / 2), n0);
                    } else if constexpr (PAIR) {
                        // both CTAs' loads are counted on the leader's barrier; the leader announces the bytes of both
                        // (a half-tile item needs, and loads, only half of this CTA's rows of B)
                        const bool half = item.nCols != BN;
                        if (rank == 0) mbar_arrive_expect_tx(&fullBar[s], half ? 2 * (C::kABytes + C::kBBytes / 2) : 2 * C::kStageBytes);
                        const uint32_t leaderBar = mapa_u32(smem_u32(&fullBar[s]), 0);
                        tma_load_2d_pair(sa, &tmapA, leaderBar, kb * kBK, m0);
                        tma_load_2d_pair(sa + C::kABytes, half ? &tmapC.bHalf : &tmapB, leaderBar, kb * kBK, n0);
                    } else {
                        mbar_arrive_expect_tx(&fullBar[s], C::kStageBytes - p.aBoxShort);
                        tma_load_2d(sa, &tmapA, &fullBar[s], kb * kBK, m0);
                        tma_load_2d(sa + C::kABytes, &tmapB, &fullBar[s], kb * kBK, n0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (rank == 0 && elect_one()) {
            const uint32_t idescFull = (EPI == kEpiFloat) ? idesc_f16(kTileM, BN, p.abFmt) : idesc_i8(kTileM, BN);
            const uint32_t idescHalf = (EPI == kEpiFloat) ? idesc_f16(kTileM, BN / 2, p.abFmt) : idesc_i8(kTileM, BN / 2);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int w = unit; w < numTiles && ok; w += numUnits, ++local) {
                const uint32_t idesc = (w < p.fullTiles) ? idescFull : idescHalf;
                const int acc = local & 1;
                const uint32_t accPh = (local >> 1) & 1;
                if (!(ok = mbar_wait_bounded(&tmemEmpty[acc], accPh ^ 1, abortFlag))) break;
                tc_fence_after();
                const uint32_t tmemD = tmemBase + acc * BN;
                for (int kb = 0; kb < kBlocks; ++kb, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    if (!(ok = mbar_wait_bounded(&fullBar[s], ph, abortFlag))) break;
                    if constexpr (CONV) {
                        // half of the converted tile was written by the other CTA's warps (released at cluster scope)
                        if (!(ok = mbar_wait_bounded_cluster(&convDone[s], ph, abortFlag))) break;
                    }
                    tc_fence_after();
                    const uint32_t aAddr = smem_u32(smem + s * C::kStageBytes);
                    const uint64_t descA = smem_desc_sw128(aAddr);
                    const uint64_t descB = smem_desc_sw128(aAddr + C::kABytes);
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k) {
                        // advancing K inside the swizzle atom: +32 bytes on the start address (>> 4 = 2)
                        if constexpr (EPI == kEpiFloat) {
                            if constexpr (PAIR) mma_f16_pair(tmemD, descA + 2 * k, descB + 2 * k, idesc, (kb | k) != 0);
                            else mma_f16(tmemD, descA + 2 * k, descB + 2 * k, idesc, (kb | k) != 0);
                        } else {
                            if constexpr (PAIR) mma_i8_pair(tmemD, descA + 2 * k, descB + 2 * k, idesc, (kb | k) != 0);
                            else mma_i8(tmemD, descA + 2 * k, descB + 2 * k, idesc, (kb | k) != 0);
                        }
                    }
                    // the stage is free (in both CTAs of a pair) once these MMAs have read it
                    if constexpr (PAIR) tc_commit_pair(&emptyBar[s], 3);
                    else tc_commit(&emptyBar[s]);
                }
                if (ok) {
                    if constexpr (PAIR) tc_commit_pair(&tmemFull[acc], 3);
                    else tc_commit(&tmemFull[acc]);
                }
            }
        }
    } else if (CONV && warp >= 2 + kEpiWarps) {
        // ---------------- converter warps: int8 rows of B -> the swizzled half / bfloat16 tile of the stage ----------------
        if constexpr (CONV) {
            // the operand type and the presence of an offset are fixed for the launch: pick the straight-line loop once
            const int t = threadIdx.x - 32 * (2 + kEpiWarps);
            auto run = [&](auto ctTag, auto dstTag, auto offTag) {
                using CT = decltype(ctTag);
                using Dst = decltype(dstTag);
                constexpr bool kOff = decltype(offTag)::value;
                convert_tiles<C, BN, CT, Dst, kOff>(p, smem, epiScale, fullQ, convDone, abortFlag, t >> 5, lane, rank, unit, numUnits, numTiles,
                                                    kBlocks);
            };
            if (p.abFmt == 1) {
                if (p.aqHasOffset) run(float{}, __nv_bfloat16{}, std::true_type{});
                else run(float{}, __nv_bfloat16{}, std::false_type{});
            } else {
                if (p.aqHasOffset) run(__half{}, __half{}, std::true_type{});
                else run(__half{}, __half{}, std::false_type{});
            }
        }
    } else {
        // ---------------- epilogue: warp w reads TMEM lanes 32*(w%4).. (its 32 rows of the tile) ----------------
        const int q = warp & 3;
        const int sub = (warp - 2) >> 2;
        uint8_t* stageW = outStage + (warp - 2) * kWarpStageBytes;
        // the 1024-byte aligned 2 KiB inside the same region: staging rows of the TMA stores (128B-swizzled)
        uint8_t* stageT = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(stageW) + 1023) & ~uintptr_t(1023));
        uint32_t local = 0;
        bool ok = true;
        for (int w = unit; w < numTiles && ok; w += numUnits, ++local) {
            const Item item = decode_item<BN>(p, w);
            const int tile = item.tile;
            const int acc = local & 1;
            const uint32_t accPh = (local >> 1) & 1;
            const RowTile rt = row_tile(tile % p.tilesM);
            const int m0 = rt.m0, rowEnd = rt.rowEnd;   // rows [m0, rowEnd) of C are this CTA's to write
            const int n0 = (tile / p.tilesM) * BN + item.nOff;
            const int m = m0 + q * 32 + lane;
            const float sa = (p.sA != nullptr && m < rowEnd) ? __ldg(p.sA + m) : 1.0f;
            // this tile's per-channel scale and bias, once, into shared memory (fp32): every thread needs all BN of
            // them and reads them back as warp-wide broadcasts.  Fetched before the accumulator is waited for, so that
            // the latency of these loads is hidden; the buffer of this accumulator was last read two tiles ago, and every
            // warp has passed the barrier of the tile in between since.
            float* sBs = epiScale + acc * 3 * BN;
            float* biasS = sBs + BN;
            uint32_t* auxS = reinterpret_cast<uint32_t*>(biasS + BN);
            {
                const int t = threadIdx.x - 64;  // index over the epilogue threads
                for (int j = t; j < BN; j += 32 * kEpiWarps) {
                    const int n = n0 + j;
                    if constexpr (EPI == kEpiFloat || EPI == kEpiRequant) {
                        if (EPI == kEpiFloat && p.outKind != 3) continue;  // only the quantising form has per-column parameters
                        unsigned long long qp = 0;
                        if (n < p.N) qp = p.quantVec != nullptr ? __ldg(reinterpret_cast<const unsigned long long*>(p.quantVec) + n) : p.quantBits;
                        sBs[j] = __uint_as_float(static_cast<uint32_t>(qp) & 0xFFFFE000u);
                        biasS[j] = __int_as_float((p.biasI32 != nullptr && n < p.N) ? __ldg(p.biasI32 + n) : 0);
                        auxS[j] = static_cast<uint32_t>(qp >> 32) & 0x7FFFu;
                    } else if constexpr (EPI == kEpiFixpipe) {
                        const uint32_t bits = (p.quantVec != nullptr && n < p.N)
                                                  ? static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned long long*>(p.quantVec) + n)) & 0xFFFFE000u
                                                  : 0x3F800000u;
                        sBs[j] = __uint_as_float(bits);
                        biasS[j] = __int_as_float((p.biasI32 != nullptr && n < p.N) ? __ldg(p.biasI32 + n) : 0);
                    } else {
                        sBs[j] = (p.sB != nullptr && n < p.N) ? __ldg(p.sB + rt.nBase + n) : 1.0f;
                        biasS[j] = (p.bias != nullptr && n < p.N) ? __bfloat162float(p.bias[rt.nBase + n]) : 0.0f;
                    }
                }
                ok = CONV ? mbar_wait_bounded_sleepy(&tmemFull[acc], accPh, abortFlag) : mbar_wait_bounded(&tmemFull[acc], accPh, abortFlag);
                tc_fence_after();
                // barrier of the epilogue warps only; it also makes the give-up decision uniform, so that no warp is
                // left waiting at it for one that stopped
                uint32_t anyFail;
                asm volatile(
                    "{\n\t.reg .pred pin, pout;\n\t"
                    "setp.ne.u32 pin, %1, 0;\n\t"
                    "bar.red.or.pred pout, 1, %2, pin;\n\t"
                    "selp.u32 %0, 1, 0, pout;\n\t}"
                    : "=r"(anyFail)
                    : "r"(ok ? 0u : 1u), "n"(32 * kEpiWarps)
                    : "memory");
                if (anyFail) {
                    ok = false;
                    break;
                }
                if (threadIdx.x == 64 && local < 4) ASCQ_STAMP(p, 1 + 2 * static_cast<int>(local));
            }
            [[maybe_unused]] const long long tAcc = clock64();
            [[maybe_unused]] const bool stamp = threadIdx.x == 64 && local == 0;
            const bool hasBias = p.bias != nullptr;
            // A row tile of a grouped launch that ends inside its 128 rows must not touch the next group's rows, which a
            // 16-row box would: such tiles take the per-thread stores.  They stage through the same bytes, so the TMA
            // stores of the tile before must have read them.
            const bool tileTma = p.tmaStore && (gt.G == 0 || rowEnd - m0 >= kBM);
            if (p.tmaStore && !tileTma) {
                if (lane == 0) bulk_wait_group_read<0>();
                __syncwarp();
            }
            const uint32_t taddr = tmemBase + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
            const bool haveC = p.C[0] != nullptr;
            bool vecStore = (p.ldc % 8 == 0) && (p.colOffset % 8 == 0);
            for (int pi = 0; pi < p.nPeers; ++pi) vecStore = vecStore && ((reinterpret_cast<uintptr_t>(p.C[pi]) & 15u) == 0);

            // 32 accumulator columns of this thread's row -> 16 packed bf16x2 words
            auto convert32 = [&](const uint32_t(&r)[32], int colInTile, uint32_t* packed) {
                const float4* sb4 = reinterpret_cast<const float4*>(sBs + colInTile);
                const float4* bi4 = reinterpret_cast<const float4*>(biasS + colInTile);
                if constexpr (EPI == kEpiFloat) {
                    // fp32 accumulator -> half or bfloat16 (RINT; half overflows to infinity as IEEE does)
#pragma unroll
                    for (int v = 0; v < 16; ++v) {
                        const float f0 = __uint_as_float(r[2 * v]), f1 = __uint_as_float(r[2 * v + 1]);
                        if (p.outKind == 1) {
                            packed[v] = pack_bf16x2_sat(f0, f1);
                        } else {
                            const __half2 h = __floats2half2_rn(f0, f1);
                            packed[v] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                    }
                    return;
                }
                if constexpr (EPI == kEpiFixpipe) {
                    // matmul_quant/scripts/gen_data.py:26-44: (acc + bias) -> half; scalar mode: half * half(scale);
                    // vector mode: float(half) * scale (19 significant bits kept) -> half
                    const bool vec = p.quantVec != nullptr;
                    const __half hs = __float2half_rn(p.quantScalar);
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const float4 s4 = sb4[v];
                        const float4 b4 = bi4[v];
                        const float sc[4] = {s4.x, s4.y, s4.z, s4.w};
                        const float bi[4] = {b4.x, b4.y, b4.z, b4.w};
                        unsigned short o[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int32_t a = static_cast<int32_t>(r[4 * v + e]) + __float_as_int(bi[e]);
                            const __half h = __int2half_rn(a);
                            const __half res = vec ? __float2half_rn(__fmul_rn(__half2float(h), sc[e])) : __hmul_rn(h, hs);
                            o[e] = __half_as_ushort(res);
                        }
                        packed[2 * v] = static_cast<uint32_t>(o[0]) | (static_cast<uint32_t>(o[1]) << 16);
                        packed[2 * v + 1] = static_cast<uint32_t>(o[2]) | (static_cast<uint32_t>(o[3]) << 16);
                    }
                    return;
                }
                // The dequantisation proper, as straight-line code: which optional steps run (bias, FasterGelu, half or
                // bfloat16 result) is fixed per launch, so each combination is its own instantiation and the loop body has
                // no branch -- a branch per packed pair (the saturation test used to be one) keeps the compiler from
                // overlapping the 32 independent chains and cost two thirds of the arithmetic's time.  Saturation: the
                // packed words are checked for an infinity AFTER the loop (rare: finite overflow of the 16-bit type) and
                // only then redone with the saturating conversion.
                auto dequant = [&](auto biasTag, auto actTag, auto halfTag) {
                    constexpr bool kBias = decltype(biasTag)::value, kAct = decltype(actTag)::value, kHalf = decltype(halfTag)::value;
                    uint32_t inf = 0;
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const float4 s4 = sb4[v];
                        float f0 = __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int32_t>(r[4 * v + 0])), s4.x), sa);
                        float f1 = __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int32_t>(r[4 * v + 1])), s4.y), sa);
                        float f2 = __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int32_t>(r[4 * v + 2])), s4.z), sa);
                        float f3 = __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int32_t>(r[4 * v + 3])), s4.w), sa);
                        if constexpr (kBias) {
                            const float4 b4 = bi4[v];
                            f0 = __fadd_rn(f0, b4.x); f1 = __fadd_rn(f1, b4.y); f2 = __fadd_rn(f2, b4.z); f3 = __fadd_rn(f3, b4.w);
                        }
                        if constexpr (kAct) {
                            f0 = faster_gelu(f0); f1 = faster_gelu(f1); f2 = faster_gelu(f2); f3 = faster_gelu(f3);
                        }
                        uint32_t w0, w1;
                        if constexpr (kHalf) {
                            asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(w0) : "f"(f1), "f"(f0));
                            asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(w1) : "f"(f3), "f"(f2));
                            inf |= ((w0 & 0x7FFF7FFFu) + 0x04000400u) | ((w1 & 0x7FFF7FFFu) + 0x04000400u);  // bit 15 / 31: exponent all ones
                        } else {
                            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w0) : "f"(f1), "f"(f0));
                            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w1) : "f"(f3), "f"(f2));
                            inf |= ((w0 & 0x7FFF7FFFu) + 0x00800080u) | ((w1 & 0x7FFF7FFFu) + 0x00800080u);
                        }
                        packed[2 * v] = w0;
                        packed[2 * v + 1] = w1;
                    }
                    if (__builtin_expect((inf & 0x80008000u) != 0, 0)) {  // an infinity or NaN came out: redo with saturation
#pragma unroll
                        for (int j = 0; j < 16; ++j) {  // (unrolled: a run-time index would move the registers to local memory)
                            float f[2];
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int c = 2 * j + e;
                                float x = __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int32_t>(r[c])), sBs[colInTile + c]), sa);
                                if constexpr (kBias) x = __fadd_rn(x, biasS[colInTile + c]);
                                if constexpr (kAct) x = faster_gelu(x);
                                f[e] = x;
                            }
                            packed[j] = kHalf ? pack_f16x2_sat(f[0], f[1]) : pack_bf16x2_sat(f[0], f[1]);
                        }
                    }
                };
                using T = std::true_type;
                using F = std::false_type;
                if constexpr (EPI == kEpiDequantAct) {
                    const int sel = (hasBias ? 4 : 0) | (p.act ? 2 : 0) | (p.outKind == 1 ? 1 : 0);
                    switch (sel) {
                        case 0: dequant(F{}, F{}, F{}); break;
                        case 1: dequant(F{}, F{}, T{}); break;
                        case 2: dequant(F{}, T{}, F{}); break;
                        case 3: dequant(F{}, T{}, T{}); break;
                        case 4: dequant(T{}, F{}, F{}); break;
                        case 5: dequant(T{}, F{}, T{}); break;
                        case 6: dequant(T{}, T{}, F{}); break;
                        default: dequant(T{}, T{}, T{}); break;
                    }
                } else {
                    if (hasBias) dequant(T{}, F{}, F{});
                    else dequant(F{}, F{}, F{});
                }
            };
            // (V)REQ8, fixpipe_l0c2gm/scripts/gen_data_s322s8.py:75-97: optional arithmetic shift with saturation to int16,
            // float(acc) * scale in fp32, clamp to [-256, 255], RINT, + offset, clamp to the int8 or uint8 range.
            // (V)QF322B8_PRE (fp32 accumulator of a half / bfloat16 matmul, scripts/gen_data_f322s8.py:75-97): the same
            // from the multiplication on.
            // 32 accumulator columns of this thread's row -> 8 words of four result bytes
            auto requant32 = [&](const uint32_t(&r)[32], int colInTile, uint32_t* packed) {
                const float4* sb4 = reinterpret_cast<const float4*>(sBs + colInTile);
                const int4* bi4 = reinterpret_cast<const int4*>(biasS + colInTile);
                const uint4* ax4 = reinterpret_cast<const uint4*>(auxS + colInTile);
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    const float4 s4 = sb4[v];
                    const int4 b4 = bi4[v];
                    const uint4 a4 = ax4[v];
                    const float sc[4] = {s4.x, s4.y, s4.z, s4.w};
                    const int bi[4] = {b4.x, b4.y, b4.z, b4.w};
                    const uint32_t ax[4] = {a4.x, a4.y, a4.z, a4.w};
                    uint32_t word = 0;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float x;
                        if constexpr (EPI == kEpiFloat) {  // fp32 accumulator: the shift fields do not apply
                            x = __uint_as_float(r[4 * v + e]);
                        } else {
                            int32_t a = static_cast<int32_t>(r[4 * v + e] + static_cast<uint32_t>(bi[e]));
                            if (ax[e] & 16u) a = max(-32768, min(32767, a >> (ax[e] & 15u)));
                            x = __int2float_rn(a);
                        }
                        const float f = fminf(fmaxf(__fmul_rn(x, sc[e]), -256.0f), 255.0f);
                        int o = __float2int_rn(f) + static_cast<int>((ax[e] >> 5) & 0x1FFu);
                        o = (ax[e] & 0x4000u) ? max(-128, min(127, o)) : max(0, min(255, o));
                        word |= static_cast<uint32_t>(o & 0xFF) << (8 * e);
                    }
                    packed[v] = word;
                }
            };
            // slow path for ragged edges / unaligned outputs: every thread writes its own row segment
            auto store_direct = [&](const uint32_t* packed, int n) {
                if (m >= rowEnd || n >= p.N) return;
                for (int pi = 0; pi < p.nPeers; ++pi) {
                    __nv_bfloat16* crow = p.C[pi] + static_cast<size_t>(m) * p.ldc + p.colOffset + n;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (n + j < p.N)
                            crow[j] = __ushort_as_bfloat16(static_cast<unsigned short>(packed[j >> 1] >> ((j & 1) * 16)));
                }
            };
#pragma unroll 1
            for (int c2 = sub; c2 < item.nCols / 64; c2 += kEpiWarps / 4) {  // 64 columns = 128 bytes of bf16 per row at a time
                uint32_t r0[32], r1[32];
                tmem_ld_32x32b_x32(taddr + c2 * 64, r0);
                tmem_ld_32x32b_x32(taddr + c2 * 64 + 32, r1);
                tmem_ld_wait();
                if (stamp && c2 == sub) ASCQ_CYCLES(p, 8, tAcc);
                const int n = n0 + c2 * 64;
                if (n >= p.N) continue;  // uniform over the warp
                if (p.accDump != nullptr && m < rowEnd) {
                    int32_t* d = p.accDump + static_cast<size_t>(m) * p.N + n;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (n + j < p.N) d[j] = static_cast<int32_t>(r0[j]);
                        if (n + 32 + j < p.N) d[32 + j] = static_cast<int32_t>(r1[j]);
                    }
                }
                if (!haveC) continue;
                if constexpr (EPI == kEpiFloat) {
                    if (p.outKind == 2) {  // fp32 output: every thread writes its own row
                        if (m < rowEnd) {
                            float* crow = reinterpret_cast<float*>(p.C[0]) + static_cast<size_t>(m) * p.ldc + p.colOffset + n;
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (n + j < p.N) crow[j] = __uint_as_float(r0[j]);
                                if (n + 32 + j < p.N) crow[32 + j] = __uint_as_float(r1[j]);
                            }
                        }
                        continue;
                    }
                }
                if (EPI == kEpiRequant || (EPI == kEpiFloat && p.outKind == 3)) {
                    uint32_t pk[16];
                    requant32(r0, c2 * 64, pk);
                    requant32(r1, c2 * 64 + 32, pk + 8);
                    uint8_t* Cb = reinterpret_cast<uint8_t*>(p.C[0]);
                    const bool vecB = (p.ldc % 16 == 0) && (p.colOffset % 16 == 0) && ((reinterpret_cast<uintptr_t>(Cb) & 15u) == 0);
                    if (vecB && n + 64 <= p.N) {
                        // as below, with 64-byte row segments: every store instruction writes eight of them
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            if ((lane >> 4) == h) {
#pragma unroll
                                for (int v = 0; v < 4; ++v)
                                    *reinterpret_cast<uint4*>(stageW + (lane & 15) * kBytePitch + v * 16) =
                                        make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
                            }
                            __syncwarp();
                            const int piece = lane & 3;
#pragma unroll
                            for (int i = 0; i < 2; ++i) {
                                const int rl = i * 8 + (lane >> 2);
                                const uint4 val = *reinterpret_cast<const uint4*>(stageW + rl * kBytePitch + piece * 16);
                                const int gm = m0 + q * 32 + h * 16 + rl;
                                if (gm < rowEnd)
                                    *reinterpret_cast<uint4*>(Cb + static_cast<size_t>(gm) * p.ldc + p.colOffset + n + piece * 16) = val;
                            }
                            __syncwarp();
                        }
                    } else if (m < rowEnd) {
                        uint8_t* crow = Cb + static_cast<size_t>(m) * p.ldc + p.colOffset + n;
#pragma unroll
                        for (int j = 0; j < 64; ++j)
                            if (n + j < p.N) crow[j] = static_cast<uint8_t>(pk[j >> 2] >> ((j & 3) * 8));
                    }
                    continue;
                }
                uint32_t packed[32];
                if (tileTma && p.narrowBox) {
                    // One output matrix: 32 columns at a time.  Every lane stages its own row's 64 bytes (piece v of row
                    // r at v ^ ((r >> 1) & 3): the 64B swizzle, free of bank conflicts) and the 32 x 32 box leaves as one
                    // TMA store; the wait for the previous store's read of the staging rows comes after the next 32
                    // columns' arithmetic, which hides it.  (Launches that write to peers keep the 128-byte rows below:
                    // longer segments suit the link.)
#pragma unroll
                    for (int sc = 0; sc < 2; ++sc) {
                        if (sc == 0) convert32(r0, c2 * 64, packed);
                        else convert32(r1, c2 * 64 + 32, packed);
                        if (stamp && c2 == sub && sc == 1) ASCQ_CYCLES(p, 9, tAcc);
                        if (lane == 0) bulk_wait_group_read<0>();
                        __syncwarp();
#pragma unroll
                        for (int v = 0; v < 4; ++v)
                            *reinterpret_cast<uint4*>(stageT + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) =
                                make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                        fence_proxy_async();
                        __syncwarp();
                        const int row0 = m0 + q * 32;
                        if (lane == 0 && row0 < rowEnd && n + sc * 32 < p.N) {
                            tma_store_2d(&tmapC.cNarrow, stageT, p.colOffset + n + sc * 32, row0);
                            bulk_commit_group();
                        }
                    }
                    if (stamp && c2 == sub) ASCQ_CYCLES(p, 10, tAcc);
                    continue;
                }
                convert32(r0, c2 * 64, packed);
                convert32(r1, c2 * 64 + 32, packed + 16);
                if (stamp && c2 == sub) ASCQ_CYCLES(p, 9, tAcc);
                if (tileTma) {
                    // Sixteen rows at a time go into this warp's swizzled staging rows (16-byte piece v of row r at
                    // v ^ (r & 7), which also keeps the writes free of bank conflicts) and leave as one TMA store; rows
                    // past M and columns past N are clipped by the tensor map.
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (lane == 0) bulk_wait_group_read<0>();  // the previous store has read the staging rows
                        __syncwarp();
                        if ((lane >> 4) == h) {
                            const int row = lane & 15;
#pragma unroll
                            for (int v = 0; v < 8; ++v)
                                *reinterpret_cast<uint4*>(stageT + row * 128 + ((v ^ (row & 7)) << 4)) =
                                    make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                            fence_proxy_async();
                        }
                        __syncwarp();
                        const int row0 = m0 + q * 32 + h * 16;
                        if (lane == 0 && row0 < rowEnd) {
                            // one store per output matrix (this GPU's and the peers'), all reading the same staged rows
                            for (int pi = 0; pi < p.nPeers; ++pi) {
                                int b = p.firstPeer + pi;
                                if (b >= p.nPeers) b -= p.nPeers;
                                tma_store_2d(&tmapC.m[b], stageT, p.colOffset + n, row0);
                            }
                            bulk_commit_group();
                        }
                    }
                    if (stamp && c2 == sub) ASCQ_CYCLES(p, 10, tAcc);
                } else if (vecStore && n + 64 <= p.N) {
                    // Transpose through this warp's staging rows, sixteen rows at a time, so that every store instruction
                    // writes four complete 128-byte row segments (instead of thirty-two 16-byte pieces): the output leaves
                    // the SM in whole lines, which is what both L2 and NVLink move best.
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if ((lane >> 4) == h) {
#pragma unroll
                            for (int v = 0; v < 8; ++v)
                                *reinterpret_cast<uint4*>(stageW + (lane & 15) * kStagePitch + v * 16) =
                                    make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                        }
                        __syncwarp();
                        const int piece = lane & 7;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int rl = i * 4 + (lane >> 3);
                            const uint4 val = *reinterpret_cast<const uint4*>(stageW + rl * kStagePitch + piece * 16);
                            const int gm = m0 + q * 32 + h * 16 + rl;
                            if (gm < rowEnd) {
                                const size_t off = static_cast<size_t>(gm) * p.ldc + p.colOffset + n + piece * 8;
                                if (p.multicast) {
                                    multimem_st_v4(p.C[0] + off, val);
                                    continue;
                                }
                                for (int pi = 0; pi < p.nPeers; ++pi) {
                                    int b = p.firstPeer + pi;
                                    if (b >= p.nPeers) b -= p.nPeers;
                                    *reinterpret_cast<uint4*>(p.C[b] + off) = val;
                                }
                            }
                        }
                        __syncwarp();
                    }
                } else {
                    store_direct(packed, n);
                    store_direct(packed + 16, n + 32);
                }
            }
            if (threadIdx.x == 64 && local < 4) ASCQ_STAMP(p, 2 + 2 * static_cast<int>(local));
            if (stamp) ASCQ_CYCLES(p, 11, tAcc);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                // the leader's barrier; relaxed: it guards tensor memory only (reads complete: tcgen05.wait::ld), and a
                // release would make this thread wait for its stores of the tile to become visible first
                if constexpr (PAIR) mbar_arrive_cluster_relaxed(mapa_u32(smem_u32(&tmemEmpty[acc]), 0));
                else mbar_arrive(&tmemEmpty[acc]);
            }
        }
        if (lane == 0) {
            // the staging rows must stay valid until the last TMA store has read them; with an exchange at the end of
            // the step the stores must also have been performed before this CTA reports itself done
            if (p.comm.nranks > 1) bulk_wait_group_all();
            else bulk_wait_group_read<0>();
        }
        if (threadIdx.x == 64) ASCQ_STAMP(p, 12);
    }

    // ---------------- teardown ----------------
    __syncthreads();
    if (p.comm.nranks > 1 && threadIdx.x == 0) {
        if (!comm_finish(p.comm, gridDim.x, c_waitCycles)) atomicExch(&g_w8a8_status, 2);
        ASCQ_STAMP(p, 13);
    }
    if constexpr (PAIR) {  // neither CTA may leave (or free tensor memory) while its partner can still touch it
        cluster_arrive();
        cluster_wait();
    }
    if (*abortFlag) {
        if (threadIdx.x == 0) atomicExch(&g_w8a8_status, 1);
        // give bulk copies that may still be in flight time to land before the shared memory is handed back
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        if constexpr (PAIR) tmem_dealloc_pair(tmemBase, C::kTmemCols);
        else tmem_dealloc(tmemBase, C::kTmemCols);
    }
}

// ---- host side -------------------------------------------------------------------------------------
template <int BN, bool PAIR, int EPI = kEpiDequant, bool CONV = false>
ascq_status launch(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& tc, Params p, cudaStream_t st, const GroupTable& gt)
{
    using C = Cfg<BN, PAIR, CONV>;
    static PerDeviceOnce attrSet;  // the attribute is per device: a process may drive several GPUs
    const int dev = current_device();
    if (!attrSet.done(dev)) {
        ASCQ_CUDA_CHECK(cudaFuncSetAttribute(w8a8_kernel<BN, PAIR, EPI, CONV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(C::kSmemBytes)));
        attrSet.mark(dev);
    }
    const bool pdl = getenv("ASCQ_W8A8_NOPDL") == nullptr;
    constexpr int kRowsPerTile = PAIR ? 2 * kBM : kBM;
    p.tilesM = (p.M + kRowsPerTile - 1) / kRowsPerTile;
    if (gt.G > 0) {  // grouped: every group starts a new row tile
        p.tilesM = 0;
        for (int g = 0; g < gt.G; ++g) p.tilesM += (gt.rows[g] + kRowsPerTile - 1) / kRowsPerTile;
    }
    p.tilesN = (p.N + BN - 1) / BN;
    const int tiles = p.tilesM * p.tilesN;
    p.fullTiles = tiles;
    p.workItems = tiles;
    if constexpr (PAIR) {
        const int maxClusters = sm_count() / 2;
        const bool canSplit = !CONV && BN == 256;
        // Tail split: when the last wave of whole tiles would keep at most half of the pairs busy, its tiles are cut
        // into two column halves, so that every pair gets at most one half tile and the wave lasts half as long.
        const int rest = p.fullTiles % maxClusters;
        const bool noSplit = getenv("ASCQ_W8A8_NOSPLIT") != nullptr;
        if (canSplit && p.fullTiles > maxClusters && rest > 0 && 2 * rest <= maxClusters && !noSplit) {
            p.fullTiles -= rest;
            p.workItems += rest;
        } else if (canSplit && 2 * tiles <= maxClusters && !noSplit) {
            // a problem that would leave more than half of the pairs idle: every tile as two half items
            p.fullTiles = 0;
            p.workItems = 2 * tiles;
        }
        const int clusters = p.workItems < maxClusters ? p.workItems : maxClusters;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters), 1, 1);
        cfg.blockDim = dim3(C::kThreadsCta, 1, 1);
        cfg.dynamicSmemBytes = C::kSmemBytes;
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // set-up may overlap the previous launch's tail
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl ? 2 : 1;
        ASCQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, w8a8_kernel<BN, PAIR, EPI, CONV>, ta, tb, tc, p, gt));
    } else {
        const int grid = tiles < sm_count() ? tiles : sm_count();
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
        cfg.blockDim = dim3(C::kThreadsCta, 1, 1);
        cfg.dynamicSmemBytes = C::kSmemBytes;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl ? 1 : 0;
        ASCQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, w8a8_kernel<BN, PAIR, EPI, CONV>, ta, tb, tc, p, gt));
    }
    ASCQ_CUDA_CHECK(cudaGetLastError());
    return ASCQ_OK;
}

}  // namespace
}  // namespace ascq



namespace ascq {
namespace {
struct FixpipeArgs {
    const int32_t* biasI32;
    const uint64_t* quantVec;
    float quantScalar;
    int floatKind;     // 0: int8 operands + fixpipe epilogue; 1: half / bfloat16 operands (kEpiFloat)
    uint32_t abFmt;    // floatKind: 0 = half, 1 = bfloat16
    int outKind;       // floatKind: 0 = half, 1 = bfloat16, 2 = float, 3 = int8 / uint8 through the fixpipe quantisation
    // floatKind with B_nk int8: AscendAntiQuant inside the matmul (converter warps)
    int convert;
    const void* aqScale;
    const void* aqOffset;
    float aqScaleScalar, aqOffsetScalar;
    int aqHasOffset;
    // int8 operands, int8 / uint8 result ((V)REQ8): the whole 64-bit parameter of the scalar form
    int requant;
    unsigned long long quantBits;
};

#ifdef ASCQ_TRACE
unsigned long long* g_trace = nullptr;  // device buffer of 16 x (number of CTAs) stamps, set by ascq_debug_trace
#endif
// Test hook (ascq_test_withhold_after): the next W8A8 launch's producers stop after this many k-blocks.
std::atomic<int> g_stopAfterNext{-1};

ascq_status run_w8a8(void* const* outBufs, int nBufs, int firstBuf, int colOffset, const int8_t* A, const int8_t* B_nk,
                     const float* sA_m, const float* sB_n, const void* bias_bf16, int M, int N, int K, int ldc, int32_t* accDump,
                     cudaStream_t st, const FixpipeArgs* fix = nullptr, bool multicast = false, const ascq_comm* comm = nullptr,
                     const GroupTable* groups = nullptr, int outKind = 0, int act = 0)
{
    // groups: M is the total number of rows, B_nk holds groups->G matrices [N, K] one after the other, sB_n / bias [G, N]
    const int epi = fix ? (fix->floatKind ? kEpiFloat : (fix->requant ? kEpiRequant : kEpiFixpipe))
                        : ((outKind != 0 || act != 0) ? kEpiDequantAct : kEpiDequant);
    const int elemBytes = (epi == kEpiFloat) ? 2 : 1;
    if (!A || !B_nk) return fail(ASCQ_ERR_INVALID_ARG, "A and B must not be NULL");
    if (nBufs < 0 || nBufs > kMaxPeers) return fail(ASCQ_ERR_INVALID_ARG, "between 1 and %d output buffers are supported", kMaxPeers);
    const bool haveC = nBufs > 0 && outBufs != nullptr && outBufs[0] != nullptr;
    if (!haveC && !accDump) return fail(ASCQ_ERR_INVALID_ARG, "one of C and accDump must be given");
    if (M < 0 || N < 0 || K < 0 || colOffset < 0) return fail(ASCQ_ERR_INVALID_ARG, "M, N, K, colOffset must be non-negative");
    if (haveC && ldc < colOffset + N) return fail(ASCQ_ERR_INVALID_ARG, "ldc %d is smaller than colOffset + N = %d", ldc, colOffset + N);
    if (M == 0 || N == 0) return ASCQ_OK;
    if (K == 0) return fail(ASCQ_ERR_INVALID_ARG, "K must be positive");
    if ((K * elemBytes) % 16 != 0) return fail(ASCQ_ERR_ALIGNMENT, "K %d must be a multiple of %d (TMA row pitch of 16 bytes)", K, 16 / elemBytes);
    if (!aligned16(A) || !aligned16(B_nk)) return fail(ASCQ_ERR_ALIGNMENT, "A and B must be 16-byte aligned");

    // Few activation rows: a kernel built for reading the weight once (gemm_w8a8_small.cu; same bits).  A tile shape forced
    // through the environment, or ASCQ_W8A8_SMALL=0, keeps the call on the tcgen05 kernel.
    if (!fix && !groups && !comm && !accDump && haveC && nBufs == 1 && !multicast && outKind == 0 && act == 0 && !getenv("ASCQ_W8A8_TILE") &&
        g_stopAfterNext.load() < 0 && w8a8_small_applies(M, N, K, A, B_nk)) {
        const char* e = getenv("ASCQ_W8A8_SMALL");
        if (!e || strcmp(e, "0") != 0) return w8a8_small(outBufs[0], A, B_nk, sA_m, sB_n, bias_bf16, M, N, K, ldc, colOffset, st);
    }
    Params p{};
    p.nPeers = haveC ? nBufs : 1;
    for (int i = 0; i < p.nPeers; ++i) {
        p.C[i] = haveC ? static_cast<__nv_bfloat16*>(outBufs[i]) : nullptr;
        if (haveC && !p.C[i]) return fail(ASCQ_ERR_INVALID_ARG, "output buffer %d is NULL", i);
    }
    p.multicast = multicast ? 1 : 0;
    p.firstPeer = (p.nPeers > 0) ? ((firstBuf % p.nPeers) + p.nPeers) % p.nPeers : 0;
    p.colOffset = colOffset;
    p.sA = sA_m;
    p.sB = sB_n;
    p.bias = static_cast<const __nv_bfloat16*>(bias_bf16);
    p.accDump = accDump;
    p.M = M; p.N = N; p.K = K * elemBytes; p.ldc = ldc;  // the kernel counts K in bytes of an operand row
    p.stopAfter = g_stopAfterNext.exchange(-1);
#ifdef ASCQ_TRACE
    p.trace = g_trace;
#endif
    p.comm = comm_args(comm);
    p.outKind = outKind;
    p.act = act;
    const GroupTable noGroups{};
    const GroupTable& gt = groups ? *groups : noGroups;
    if (fix) {
        p.abFmt = fix->abFmt;
        p.outKind = fix->outKind;
        p.aqScale = fix->aqScale;
        p.aqOffset = fix->aqOffset;
        p.aqScaleScalar = fix->aqScaleScalar;
        p.aqOffsetScalar = fix->aqOffsetScalar;
        p.aqHasOffset = fix->aqHasOffset;
        p.biasI32 = fix->biasI32;
        p.quantVec = fix->quantVec;
        p.quantScalar = fix->quantScalar;
        p.quantBits = fix->quantBits;
    }

    // Tile shape: the one with the smallest estimated time = waves x time of one wave.  One wave of CTA pairs on
    // 256 x 256 tiles is the unit; single CTAs on 128 x 256 tiles do the same work per SM about a tenth slower
    // (B crosses the L2-to-SM fabric once per CTA instead of once per pair), 128 x 128 tiles do half the work per
    // wave at about four fifths of the rate.  Small problems (a column shard on eight GPUs) so end up on 128 x 128
    // tiles that occupy every SM.  ASCQ_W8A8_TILE=pair|wide|narrow overrides the choice.
    const int units = sm_count();
    int tilesM = (M + kBM - 1) / kBM, tilesM2 = (tilesM + 1) / 2;   // row tiles of 128 and of 256 rows
    if (gt.G > 0) {
        tilesM = tilesM2 = 0;
        for (int g = 0; g < gt.G; ++g) {
            tilesM += (gt.rows[g] + kBM - 1) / kBM;
            tilesM2 += (gt.rows[g] + 2 * kBM - 1) / (2 * kBM);
        }
    }
    const long long tilesPair = static_cast<long long>(tilesM2) * ((N + 255) / 256);
    const long long tiles256 = static_cast<long long>(tilesM) * ((N + 255) / 256);
    const long long tiles128 = static_cast<long long>(tilesM) * ((N + 127) / 128);
    auto waves = [](long long tiles, int n) { return static_cast<double>((tiles + n - 1) / n); };
    const double costPair = waves(tilesPair, units / 2) * 1.0;
    const double costWide = waves(tiles256, units) * 1.11;
    const double costNarrow = waves(tiles128, units) * 0.62;
    int mode = 2;
    if (costWide < costPair && costWide <= costNarrow) mode = 1;
    else if (costNarrow < costPair) mode = 0;
    // A launch that also ships its tiles to other GPUs is bound by the link, not by the tensor cores, and the link sits
    // idle until the first tiles are done: 128 x 128 tiles bring the first results out after half the time and in more,
    // smaller waves (measured: 49.2 against 50.0 us per step on two GPUs, 63.6 against 66.0 on four).
    if ((nBufs > 1 || multicast) && costNarrow <= 1.3 * (costWide < costPair ? costWide : costPair)) mode = 0;
    // A skinny product whose 64-column tiles still fit the SMs in one wave is bound by streaming B: those tiles put twice
    // as many CTAs on that as 128-column ones (mode 3, built for every epilogue of one plain matrix but the grouped one;
    // measured 8192 x 8192, M = 128: 17.7 against 20.9 us; with a second wave it loses).
    const bool slimBuilt = (epi == kEpiDequant || epi == kEpiFixpipe || epi == kEpiRequant || (epi == kEpiFloat && !fix->convert)) && gt.G == 0 &&
                           nBufs <= 1 && !multicast;
    const long long tiles64 = static_cast<long long>(tilesM) * ((N + 63) / 64);
    if (slimBuilt && tiles64 <= units && tiles64 > tiles128) mode = 3;
    if (const char* e = getenv("ASCQ_W8A8_TILE")) {
        if (!strcmp(e, "pair")) mode = 2;
        else if (!strcmp(e, "wide")) mode = 1;
        else if (!strcmp(e, "narrow")) mode = 0;
        else if (!strcmp(e, "slim") && slimBuilt) mode = 3;
    }
    // 16-bit result in one suitably aligned buffer: TMA stores (ASCQ_W8A8_STORE=plain keeps the per-thread stores)
    const bool out16 = epi == kEpiDequant || epi == kEpiDequantAct || epi == kEpiFixpipe || (epi == kEpiFloat && fix->outKind <= 1);
    const char* storeEnv = getenv("ASCQ_W8A8_STORE");
    // (the copy engine clips a box at the matrix edge in whole 16-byte pieces, so the block must end on one)
    p.tmaStore = haveC && out16 && !multicast && ldc % 8 == 0 && colOffset % 8 == 0 && N % 8 == 0 &&
                 !(storeEnv && !strcmp(storeEnv, "plain"));
    for (int i = 0; i < p.nPeers && p.tmaStore; ++i) p.tmaStore = aligned16(outBufs[i]);
    CUtensorMap ta, tb;
    OutMaps tc;
    // A matrix of fewer than 16 rows behind a 128-row box loads at two thirds of the speed (measured: 8192 x 8192 weight,
    // 30 against 20 us, with a step exactly at 16 rows); single-CTA launches then use a 16-row box -- the other rows of
    // the stage keep stale bytes, whose accumulator rows nobody reads.
    const int aBoxRows = (M < 16 && gt.G == 0 && mode != 2 && !(fix && fix->convert)) ? 16 : kBM;
    p.aBoxShort = (kBM - aBoxRows) * kBK;
    ascq_status rc = make_tmap_u8(&ta, A, static_cast<uint64_t>(M), static_cast<uint64_t>(K) * elemBytes, aBoxRows);
    if (rc != ASCQ_OK) return rc;
    const uint64_t rowsB = static_cast<uint64_t>(N) * (gt.G > 0 ? gt.G : 1);
    rc = make_tmap_u8(&tb, B_nk, rowsB, static_cast<uint64_t>(K) * elemBytes, mode == 1 ? 256 : (mode == 3 ? 64 : 128));
    if (rc != ASCQ_OK) return rc;
    for (int i = 0; i < kMaxPeers; ++i) tc.m[i] = ta;  // placeholders; the kernel reads maps [0, nPeers) and only for TMA stores
    tc.bHalf = tb;
    tc.cNarrow = ta;
    p.narrowBox = 0;
    if (p.tmaStore && p.nPeers == 1 && getenv("ASCQ_W8A8_WIDEBOX") == nullptr) {
        rc = make_tmap_out16(&tc.cNarrow, outBufs[0], static_cast<uint64_t>(M), static_cast<uint64_t>(colOffset) + N,
                             static_cast<uint64_t>(ldc), 32, 32, CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc != ASCQ_OK) return rc;
        p.narrowBox = 1;
    }
    if (mode == 2) {  // pair shape: half-tile work items load 64 rows of B per CTA instead of 128
        rc = make_tmap_u8(&tc.bHalf, B_nk, rowsB, static_cast<uint64_t>(K) * elemBytes, 64);
        if (rc != ASCQ_OK) return rc;
    }
    if (p.tmaStore) {
        // one map per output matrix (this GPU's and the peer-mapped ones): the store path only, nothing is loaded through them
        for (int i = 0; i < p.nPeers; ++i) {
            rc = make_tmap_out16(&tc.m[i], outBufs[i], static_cast<uint64_t>(M), static_cast<uint64_t>(colOffset) + N,
                                 static_cast<uint64_t>(ldc), 16);
            if (rc != ASCQ_OK) return rc;
        }
    }
    if (epi == kEpiFloat && fix->convert) {
        // B_nk is the int8 weight: its tile goes through the converter warps (CTA pairs, 256 x 256 tiles only)
        rc = make_tmap_u8_plain(&tb, B_nk, static_cast<uint64_t>(N), static_cast<uint64_t>(K), kBK / 2, 128);
        if (rc != ASCQ_OK) return rc;
        return launch<256, true, kEpiFloat, true>(ta, tb, tc, p, st, gt);
    }
    if (epi == kEpiFloat) {
        if (mode == 3) return launch<64, false, kEpiFloat>(ta, tb, tc, p, st, gt);
        if (mode == 2) return launch<256, true, kEpiFloat>(ta, tb, tc, p, st, gt);
        return mode == 1 ? launch<256, false, kEpiFloat>(ta, tb, tc, p, st, gt) : launch<128, false, kEpiFloat>(ta, tb, tc, p, st, gt);
    }
    if (epi == kEpiRequant) {
        if (mode == 3) return launch<64, false, kEpiRequant>(ta, tb, tc, p, st, gt);
        if (mode == 2) return launch<256, true, kEpiRequant>(ta, tb, tc, p, st, gt);
        return mode == 1 ? launch<256, false, kEpiRequant>(ta, tb, tc, p, st, gt) : launch<128, false, kEpiRequant>(ta, tb, tc, p, st, gt);
    }
    if (epi == kEpiFixpipe) {
        if (mode == 3) return launch<64, false, kEpiFixpipe>(ta, tb, tc, p, st, gt);
        if (mode == 2) return launch<256, true, kEpiFixpipe>(ta, tb, tc, p, st, gt);
        return mode == 1 ? launch<256, false, kEpiFixpipe>(ta, tb, tc, p, st, gt) : launch<128, false, kEpiFixpipe>(ta, tb, tc, p, st, gt);
    }
    if (epi == kEpiDequantAct) {
        if (mode == 2) return launch<256, true, kEpiDequantAct>(ta, tb, tc, p, st, gt);
        return mode == 1 ? launch<256, false, kEpiDequantAct>(ta, tb, tc, p, st, gt) : launch<128, false, kEpiDequantAct>(ta, tb, tc, p, st, gt);
    }
    if (mode == 3) return launch<64, false>(ta, tb, tc, p, st, gt);
    if (mode == 2) return launch<256, true>(ta, tb, tc, p, st, gt);
    return mode == 1 ? launch<256, false>(ta, tb, tc, p, st, gt) : launch<128, false>(ta, tb, tc, p, st, gt);
}
}  // namespace
}  // namespace ascq

using namespace ascq;

extern "C" ascq_status ascq_matmul_w8a8(void* C_bf16, const int8_t* A, const int8_t* B_nk, const float* sA_m,
                                        const float* sB_n, const void* bias_bf16, int M, int N, int K, int ldc,
                                        int32_t* accDump, void* stream)
{
    void* bufs[1] = {C_bf16};
    return run_w8a8(bufs, 1, 0, 0, A, B_nk, sA_m, sB_n, bias_bf16, M, N, K, ldc, accDump, static_cast<cudaStream_t>(stream));
}

// Grouped W8A8 matmul: rows of A belong to groups (experts), every group has its own weight matrix and channel scales.
extern "C" ascq_status ascq_group_matmul_w8a8(void* C, ascq_dtype cT, const int8_t* A, const int8_t* B_gnk, const float* sA_m,
                                              const float* sB_gn, const void* bias_bf16_gn, const int64_t* groupList_host,
                                              int G, int N, int K, int activation, void* stream)
{
    if (!C || !groupList_host) return fail(ASCQ_ERR_INVALID_ARG, "C and groupList must not be NULL");
    if (cT != ASCQ_DT_F16 && cT != ASCQ_DT_BF16) return fail(ASCQ_ERR_UNSUPPORTED, "output must be half or bfloat16_t");
    if (activation != 0 && activation != 1) return fail(ASCQ_ERR_INVALID_ARG, "activation must be 0 (none) or 1 (FasterGelu)");
    if (G <= 0) return fail(ASCQ_ERR_INVALID_ARG, "G must be positive");
    if (G > kMaxGroupsInline) return fail(ASCQ_ERR_UNSUPPORTED, "at most %d groups per call are supported", kMaxGroupsInline);
    GroupTable gt{};
    gt.G = G;
    int64_t sumM = 0;
    for (int g = 0; g < G; ++g) {
        if (groupList_host[g] < 0) return fail(ASCQ_ERR_INVALID_ARG, "groupList[%d] is negative", g);
        sumM += groupList_host[g];
        if (sumM > 0x7FFFFFFF - 512) return fail(ASCQ_ERR_INVALID_ARG, "too many rows for 32-bit row indices");
        gt.rows[g] = static_cast<int>(groupList_host[g]);
    }
    if (static_cast<int64_t>(G) * N > 0x7FFFFFFF) return fail(ASCQ_ERR_INVALID_ARG, "G * N exceeds 32-bit row indices");
    void* bufs[1] = {C};
    return run_w8a8(bufs, 1, 0, 0, A, B_gnk, sA_m, sB_gn, bias_bf16_gn, static_cast<int>(sumM), N, K, N, nullptr,
                    static_cast<cudaStream_t>(stream), nullptr, false, nullptr, &gt, cT == ASCQ_DT_F16 ? 1 : 0, activation);
}

extern "C" ascq_status ascq_matmul_w8a8_scatter(void* const* C_bufs, int nBufs, int firstBuf, int colOffset, int ldc,
                                                const int8_t* A, const int8_t* B_nk, const float* sA_m, const float* sB_n,
                                                const void* bias_bf16, int M, int N, int K, void* stream)
{
    if (!C_bufs || nBufs < 1) return fail(ASCQ_ERR_INVALID_ARG, "at least one output buffer is needed");
    return run_w8a8(C_bufs, nBufs, firstBuf, colOffset, A, B_nk, sA_m, sB_n, bias_bf16, M, N, K, ldc, nullptr,
                    static_cast<cudaStream_t>(stream));
}

// Reads and clears the device status word of the GEMM kernels on the current device (synchronises `stream`).
extern "C" ascq_status ascq_matmul_status(void* stream)
{
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int v = 0, zero = 0;
    ASCQ_CUDA_CHECK(cudaMemcpyFromSymbolAsync(&v, g_w8a8_status, sizeof(int), 0, cudaMemcpyDeviceToHost, st));
    ASCQ_CUDA_CHECK(cudaStreamSynchronize(st));
    if (v != 0) {
        ASCQ_CUDA_CHECK(cudaMemcpyToSymbolAsync(g_w8a8_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, st));
        return fail(ASCQ_ERR_TIMEOUT, "a bounded wait inside the W8A8 matmul kernel expired (status %d)", v);
    }
    const ascq_status rc = mxfp4_read_status(st);
    if (rc != ASCQ_OK) return rc;
    return comm_read_status(st);
}

ascq_status ascq::w8a8_set_wait_cycles(long long cycles)
{
    ASCQ_CUDA_CHECK(cudaMemcpyToSymbol(ptx::c_waitCycles, &cycles, sizeof(cycles)));
    return ASCQ_OK;
}

// Test hook: the producers of the next W8A8-family launch on this process stop after `kBlocks` k-blocks, so that the
// bounded waits of the other roles run out and the kernel leaves through its abort path.
extern "C" ascq_status ascq_test_withhold_after(int kBlocks)
{
    g_stopAfterNext.store(kBlocks < 0 ? -1 : kBlocks);
    return ASCQ_OK;
}

#ifdef ASCQ_TRACE
extern "C" ascq_status ascq_debug_trace(void* deviceBuffer)
{
    g_trace = static_cast<unsigned long long*>(deviceBuffer);
    return ASCQ_OK;
}
#endif

// Column-parallel W8A8 matmul of one rank with the all-gather and the end-of-step exchange inside the launch.
extern "C" ascq_status ascq_matmul_w8a8_sharded(ascq_comm* comm, void* const* C_bufs, void* C_multicast, const int8_t* A,
                                                const int8_t* B_local, const float* sA_m, const float* sB_local,
                                                const void* bias_local, int M, int N, int K, void* stream)
{
    if (!comm) return fail(ASCQ_ERR_INVALID_ARG, "the communicator must not be NULL");
    if (!C_bufs) return fail(ASCQ_ERR_INVALID_ARG, "the table of output matrices must not be NULL");
    int c0 = 0, nl = 0;
    const ascq_status rc = ascq_shard_columns(N, comm->nranks, comm->rank, &c0, &nl);
    if (rc != ASCQ_OK) return rc;
    if (nl % 8 != 0) return fail(ASCQ_ERR_ALIGNMENT, "N / nranks = %d must be a multiple of 8", nl);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (M == 0 || nl == 0) return ascq_comm_barrier(comm, stream);  // nothing to compute, but the other ranks wait for this one
    if (C_multicast) {
        if (nl % 64 != 0 || (reinterpret_cast<uintptr_t>(C_multicast) & 15u))
            return fail(ASCQ_ERR_ALIGNMENT, "multicast output needs N / nranks %% 64 == 0 and a 16-byte aligned base");
        void* bufs[1] = {C_multicast};
        return run_w8a8(bufs, 1, 0, c0, A, B_local, sA_m, sB_local, bias_local, M, nl, K, N, nullptr, st, nullptr, true, comm);
    }
    // stores start at the next rank's matrix and go round, so that the ranks do not all write to the same GPU at once
    return run_w8a8(C_bufs, comm->nranks, comm->rank + 1, c0, A, B_local, sA_m, sB_local, bias_local, M, nl, K, N, nullptr, st,
                    nullptr, false, comm);
}

// ---- int8 matmul with the reference's fixpipe quantisation of the result (fp16 output) ----------------------------
extern "C" ascq_status ascq_matmul_i8_quant(void* C_f16, const int8_t* A, const int8_t* B_nk, const int32_t* bias_i32,
                                            const uint64_t* quantVector, float quantScalar, int M, int N, int K, int ldc,
                                            void* stream)
{
    if (!C_f16) return fail(ASCQ_ERR_INVALID_ARG, "C must not be NULL");
    if (quantVector && (reinterpret_cast<uintptr_t>(quantVector) & 7u))
        return fail(ASCQ_ERR_ALIGNMENT, "quantVector must be 8-byte aligned");
    void* bufs[1] = {C_f16};
    const FixpipeArgs fix{bias_i32, quantVector, quantScalar, 0, 0, 0, 0, nullptr, nullptr, 0.f, 0.f, 0};
    return run_w8a8(bufs, 1, 0, 0, A, B_nk, nullptr, nullptr, nullptr, M, N, K, ldc, nullptr, static_cast<cudaStream_t>(stream), &fix);
}

// ---- int8 matmul with the reference's fixpipe requantisation of the result (int8 / uint8 output) -----------------
extern "C" ascq_status ascq_matmul_i8_requant(void* C_b8, const int8_t* A, const int8_t* B_nk, const int32_t* bias_i32,
                                              const uint64_t* quantVector, uint64_t quantScalar, int M, int N, int K, int ldc,
                                              void* stream)
{
    if (!C_b8) return fail(ASCQ_ERR_INVALID_ARG, "C must not be NULL");
    if (quantVector && (reinterpret_cast<uintptr_t>(quantVector) & 7u))
        return fail(ASCQ_ERR_ALIGNMENT, "quantVector must be 8-byte aligned");
    void* bufs[1] = {C_b8};
    FixpipeArgs fix{};
    fix.biasI32 = bias_i32;
    fix.quantVec = quantVector;
    fix.requant = 1;
    fix.quantBits = quantScalar;
    return run_w8a8(bufs, 1, 0, 0, A, B_nk, nullptr, nullptr, nullptr, M, N, K, ldc, nullptr, static_cast<cudaStream_t>(stream), &fix);
}

// ---- half / bfloat16 matmul and the weight-only-quantised matmul built on it -------------------------------------
extern "C" ascq_status ascq_matmul_f16(void* C, ascq_dtype cT, const void* A, const void* B_nk, ascq_dtype abT, int M, int N,
                                       int K, int ldc, void* stream)
{
    if (!C) return fail(ASCQ_ERR_INVALID_ARG, "C must not be NULL");
    if (abT != ASCQ_DT_F16 && abT != ASCQ_DT_BF16) return fail(ASCQ_ERR_UNSUPPORTED, "operands must be half or bfloat16_t");
    if (cT != ASCQ_DT_F16 && cT != ASCQ_DT_BF16 && cT != ASCQ_DT_F32)
        return fail(ASCQ_ERR_UNSUPPORTED, "output must be half, bfloat16_t or float");
    void* bufs[1] = {C};
    const FixpipeArgs fa{nullptr, nullptr, 0.f, 1, abT == ASCQ_DT_BF16 ? 1u : 0u, cT == ASCQ_DT_F16 ? 0 : (cT == ASCQ_DT_BF16 ? 1 : 2),
                         0, nullptr, nullptr, 0.f, 0.f, 0};
    return run_w8a8(bufs, 1, 0, 0, static_cast<const int8_t*>(A), static_cast<const int8_t*>(B_nk), nullptr, nullptr, nullptr, M, N,
                    K, ldc, nullptr, static_cast<cudaStream_t>(stream), &fa);
}

extern "C" ascq_status ascq_matmul_f16_quant(void* C_b8, const void* A, const void* B_nk, ascq_dtype abT, const uint64_t* quantVector,
                                             uint64_t quantScalar, int M, int N, int K, int ldc, void* stream)
{
    if (!C_b8) return fail(ASCQ_ERR_INVALID_ARG, "C must not be NULL");
    if (abT != ASCQ_DT_F16 && abT != ASCQ_DT_BF16) return fail(ASCQ_ERR_UNSUPPORTED, "operands must be half or bfloat16_t");
    if (quantVector && (reinterpret_cast<uintptr_t>(quantVector) & 7u))
        return fail(ASCQ_ERR_ALIGNMENT, "quantVector must be 8-byte aligned");
    void* bufs[1] = {C_b8};
    FixpipeArgs fa{};
    fa.floatKind = 1;
    fa.abFmt = abT == ASCQ_DT_BF16 ? 1u : 0u;
    fa.outKind = 3;
    fa.quantVec = quantVector;
    fa.quantBits = quantScalar;
    return run_w8a8(bufs, 1, 0, 0, static_cast<const int8_t*>(A), static_cast<const int8_t*>(B_nk), nullptr, nullptr, nullptr, M, N,
                    K, ldc, nullptr, static_cast<cudaStream_t>(stream), &fa);
}

extern "C" size_t ascq_matmul_w8a16_workspace_size(int N, int K)
{
    return (N <= 0 || K <= 0) ? 0 : static_cast<size_t>(N) * K * 2;
}

static ascq_status matmul_wq_a16(ascq_dtype bT, void* C, ascq_dtype cT, const void* A, ascq_dtype aT, const int8_t* B_nk,
                                         const void* offset, const void* scale, float offsetScalar, float scaleScalar,
                                         int M, int N, int K, int ldc, void* workspace, size_t workspaceBytes, void* stream)
{
    if (!B_nk || !workspace) return fail(ASCQ_ERR_INVALID_ARG, "B and workspace must not be NULL");
    if (N <= 0 || K <= 0) return fail(ASCQ_ERR_INVALID_ARG, "N and K must be positive");
    if (workspaceBytes < ascq_matmul_w8a16_workspace_size(N, K))
        return fail(ASCQ_ERR_INVALID_ARG, "workspace of %zu bytes needed, %zu given", ascq_matmul_w8a16_workspace_size(N, K), workspaceBytes);
    if (aT != ASCQ_DT_F16 && aT != ASCQ_DT_BF16) return fail(ASCQ_ERR_UNSUPPORTED, "A must be half or bfloat16_t");
    // Two forms.  Default: two launches (AscendAntiQuant into the workspace, then the half / bfloat16 matmul).
    // ASCQ_W8A16=fused: four converter warps per CTA run AscendAntiQuant on each int8 tile between the TMA stage and the
    // MMA stage, so the dequantised weight never leaves shared memory -- same bits, but measured 2 to 4 times slower:
    // the tile then crosses shared memory three more times (int8 in, 16-bit out, 16-bit into the tensor cores) next to
    // the operand traffic of the MMAs, and a k-block waits for a whole warp's conversion before its MMAs can start.
    // For at most 32 activation rows a third form converts the weight in registers on its way to the tensor cores
    // (gemm_w8a16_small.cu); any value of ASCQ_W8A16 other than "small" switches it off.
    bool fused = false;
    const char* form = getenv("ASCQ_W8A16");
    if (form) fused = bT == ASCQ_DT_I8 && !strcmp(form, "fused") && (K % 32 == 0) && aligned16(B_nk);
    if ((!form || !strcmp(form, "small")) && w8a16_small_applies(M, N, K, A, B_nk, workspace, workspaceBytes)) {
        if (!C || !A) return fail(ASCQ_ERR_INVALID_ARG, "C and A must not be NULL");
        if (cT != ASCQ_DT_F16 && cT != ASCQ_DT_BF16 && cT != ASCQ_DT_F32)
            return fail(ASCQ_ERR_UNSUPPORTED, "output must be half, bfloat16_t or float");
        if (ldc < N) return fail(ASCQ_ERR_INVALID_ARG, "ldc must be at least N");
        float ss = scaleScalar, os = offsetScalar;
        if (!scale) {  // the scalars arrive as aT values
            if (aT == ASCQ_DT_F16) { ss = __half2float(__float2half_rn(ss)); os = __half2float(__float2half_rn(os)); }
            else { ss = __bfloat162float(__float2bfloat16_rn(ss)); os = __bfloat162float(__float2bfloat16_rn(os)); }
        }
        return w8a16_small(C, cT, A, aT, B_nk, bT == ASCQ_DT_I4X2, offset, scale, os, ss, scale ? offset != nullptr : true, M, N, K, ldc, workspace,
                           workspaceBytes, static_cast<cudaStream_t>(stream));
    }
    if (fused) {
        if (!C) return fail(ASCQ_ERR_INVALID_ARG, "C must not be NULL");
        if (cT != ASCQ_DT_F16 && cT != ASCQ_DT_BF16 && cT != ASCQ_DT_F32)
            return fail(ASCQ_ERR_UNSUPPORTED, "output must be half, bfloat16_t or float");
        float ss = scaleScalar, os = offsetScalar;
        if (!scale) {  // the scalars arrive as aT values (include/adv_api/quantization/ascend_antiquant.h:136-205)
            if (aT == ASCQ_DT_F16) { ss = __half2float(__float2half_rn(ss)); os = __half2float(__float2half_rn(os)); }
            else { ss = __bfloat162float(__float2bfloat16_rn(ss)); os = __bfloat162float(__float2bfloat16_rn(os)); }
        }
        void* bufs[1] = {C};
        const FixpipeArgs fa{nullptr, nullptr, 0.f, 1, aT == ASCQ_DT_BF16 ? 1u : 0u, cT == ASCQ_DT_F16 ? 0 : (cT == ASCQ_DT_BF16 ? 1 : 2),
                             1, scale, offset, ss, os, scale ? (offset ? 1 : 0) : 1};
        return run_w8a8(bufs, 1, 0, 0, static_cast<const int8_t*>(A), B_nk, nullptr, nullptr, nullptr, M, N, K, ldc, nullptr,
                        static_cast<cudaStream_t>(stream), &fa);
    }
    // step 1: the weight tile through AscendAntiQuant<int8_t, aT, isTranspose = true> (src [N, K], one scale / offset per
    // row n), as antiquant_processor_using_ub.h:86-137 does before the cube unit sees it
    ascq_antiquant_param ap{static_cast<uint32_t>(N), static_cast<uint32_t>(K), 0, 0, 1, 1, 1};
    ascq_status rc;
    if (scale) {
        ap.hasOffset = offset ? 1 : 0;
        rc = ascq_antiquant(workspace, aT, B_nk, bT, offset, scale, aT, 0.f, 0.f, ASCQ_PER_CHANNEL, &ap, stream);
    } else {
        rc = ascq_antiquant(workspace, aT, B_nk, bT, nullptr, nullptr, aT, offsetScalar, scaleScalar, ASCQ_PER_TENSOR, &ap, stream);
    }
    if (rc != ASCQ_OK) return rc;
    // step 2: half / bfloat16 matmul on the tensor cores
    return ascq_matmul_f16(C, cT, A, workspace, aT, M, N, K, ldc, stream);
}

extern "C" ascq_status ascq_matmul_w8a16(void* C, ascq_dtype cT, const void* A, ascq_dtype aT, const int8_t* B_nk,
                                         const void* offset, const void* scale, float offsetScalar, float scaleScalar,
                                         int M, int N, int K, int ldc, void* workspace, size_t workspaceBytes, void* stream)
{
    return matmul_wq_a16(ASCQ_DT_I8, C, cT, A, aT, B_nk, offset, scale, offsetScalar, scaleScalar, M, N, K, ldc, workspace,
                         workspaceBytes, stream);
}

// int4b_t weights: B_nk holds [N, K/2] bytes, two signed nibbles per byte (even k in the low nibble)
extern "C" ascq_status ascq_matmul_w4a16(void* C, ascq_dtype cT, const void* A, ascq_dtype aT, const uint8_t* B_nk_int4,
                                         const void* offset, const void* scale, float offsetScalar, float scaleScalar,
                                         int M, int N, int K, int ldc, void* workspace, size_t workspaceBytes, void* stream)
{
    return matmul_wq_a16(ASCQ_DT_I4X2, C, cT, A, aT, reinterpret_cast<const int8_t*>(B_nk_int4), offset, scale, offsetScalar,
                         scaleScalar, M, N, K, ldc, workspace, workspaceBytes, stream);
}

// [K, N] row-major int8 (the reference's ND weight, CubeFormat::ND, not transposed) -> [N, K]: one-off weight preparation.
namespace ascq {
namespace {
__global__ void __launch_bounds__(256) transpose_i8_kernel(int8_t* __restrict__ dst, const int8_t* __restrict__ src, int K, int N)
{
    __shared__ int8_t tile[64][65];
    const int k0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    for (int i = threadIdx.x; i < 64 * 64; i += blockDim.x) {
        const int k = k0 + i / 64, n = n0 + i % 64;
        tile[i / 64][i % 64] = (k < K && n < N) ? src[static_cast<size_t>(k) * N + n] : 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 64; i += blockDim.x) {
        const int n = n0 + i / 64, k = k0 + i % 64;
        if (n < N && k < K) dst[static_cast<size_t>(n) * K + k] = tile[i % 64][i / 64];
    }
}
}  // namespace
}  // namespace ascq

extern "C" ascq_status ascq_transpose_i8_kn_to_nk(int8_t* B_nk, const int8_t* B_kn, int K, int N, void* stream)
{
    if (!B_nk || !B_kn) return fail(ASCQ_ERR_INVALID_ARG, "B_nk and B_kn must not be NULL");
    if (K <= 0 || N <= 0) return fail(ASCQ_ERR_INVALID_ARG, "K and N must be positive");
    const dim3 grid((N + 63) / 64, (K + 63) / 64);
    transpose_i8_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(B_nk, B_kn, K, N);
    ASCQ_CUDA_CHECK(cudaGetLastError());
    return ASCQ_OK;
}
