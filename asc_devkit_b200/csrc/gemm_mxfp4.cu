// ascq_group_matmul_mxfp4: grouped matmul on MX-FP4 operands (E2M1 values, one E8M0 scale per 32 K-elements)
// with tcgen05.mma kind::mxf4.block_scale, fp32 accumulation in tensor memory and a bf16 epilogue.
//
// Data layout in HBM (caller): A [sumM, K/2] bytes, sA [sumM, K/32]; B [G, N, K/2] bytes, sB [G, N, K/32]
// (both operands K-major, two E2M1 codes per byte, element 2i in the low nibble); C [sumM, N] bf16.
//
// Scratch (caller-provided workspace):
//   tile table   one entry per 128-row tile of A: first row, valid rows, group
//   packed sA    per A tile and per 256-element k-block, 1 KiB in the order tcgen05.cp wants:
//                two 512-byte chunks (K = 128 elements each), byte (l*16 + c*4 + j) = scale of row 32c+l,
//                k-group j of the chunk
//   packed sB    per (group, 128-row tile of N), same chunk format
// A repack kernel writes the packed scales once per call; the matmul kernel then moves them with one bulk
// copy per operand per k-block and hands them to tensor memory with tcgen05.cp.32x128b.warpx4.
//
// Matmul kernel: persistent CTAs over (A tile, N tile); warp 0 TMA producer, warp 1 MMA issuer, warps 2..5
// epilogue.  Per k-block: A 128x128 B and B BNx128 B tiles (128B swizzle) + scale chunks into one of kStages
// shared-memory stages; four MMAs of K = 64.  Rows of a tile that belong to the next group are computed and
// dropped at the store.
//
// Roofline: dense FP4 tensor throughput; 2*sumM*N*K flops per call.
#include <cuda_bf16.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "ascq_internal.h"
#include "numerics.cuh"
#include "sm100_ptx.cuh"
#include "comm.cuh"
#include "tma_host.h"

namespace ascq {
namespace {

using namespace ptx;

constexpr int kBM = 128;
constexpr int kBKBytes = 128;   // 256 E2M1 elements per k-block row: one 128B swizzle atom
constexpr int kBKElems = 256;
constexpr int kChunkBytes = 512;  // packed scales of 128 rows x 128 K-elements
constexpr int kEpiWarps = 8;   // two per TMEM lane quarter; each drains half of the accumulator columns
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int kStagePitch = 144;  // bytes per staged output row: 128 B of bf16 + 16 B pad (conflict-free both ways)
constexpr int kNarrowPitch = 80;  // the same for 64-byte rows

__device__ int g_mxfp4_status = 0;

struct TileInfo {
    int rowStart;   // first row of the tile in A / C
    int rowsValid;  // rows of this tile that belong to its group
    int group;
    int outRow;     // row of the output matrix the tile's first row is written to
};

// PAIR: two CTAs of a cluster drive one tcgen05.mma.cta_group::2 on a 256 x BN tile.  Each CTA loads its 128 rows
// of A (with their scales), its half of B's rows, and the scales of ALL BN rows of B (every CTA multiplies its
// rows with every column), so B's data crosses the L2-to-SM fabric once per pair.
// SFC: 512-byte scale chunks (128 elements of K each) per k-block row of 128 bytes: 2 for 4-bit, 1 for 8-bit operands.
template <int BN, bool PAIR, int SFC> struct Cfg {
    static constexpr int kAccStages = (BN == 256) ? 1 : 2;
    static constexpr int kBRows = PAIR ? BN / 2 : BN;
    static constexpr int kABytes = kBM * kBKBytes;
    static constexpr int kBBytes = kBRows * kBKBytes;
    static constexpr int kSfaBytes = SFC * kChunkBytes;
    static constexpr int kSfbBytes = (BN / 128) * SFC * kChunkBytes;
    static constexpr int kLoadBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;  // what the copies of one stage bring
    static constexpr int kStageBytes = (kLoadBytes + 1023) / 1024 * 1024;         // swizzled tiles start 1024-byte aligned
    static constexpr int kStages = PAIR ? 5 : ((BN == 256) ? 4 : 6);
    static constexpr int kSfaCols = 4 * SFC;         // 4 columns per chunk
    static constexpr int kSfbCols = SFC * (BN / 32); // N/32 columns per chunk
    static constexpr int kAccCols = kAccStages * BN;
    static constexpr int kTmemCols = 512;
    static constexpr int kWarpStageBytes = 32 * kNarrowPitch > 16 * kStagePitch ? 32 * kNarrowPitch : 16 * kStagePitch;
    static constexpr int kOutBytes = kEpiWarps * kWarpStageBytes;  // per epilogue warp: 16 rows x 128 B or 32 rows x 64 B
    static constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + 1024 + 256 + kOutBytes;
    static_assert(kWarpStageBytes == 2560, "a 1024-aligned block of 2 KiB must fit into every warp's staging region");
    static_assert(kSmemBytes <= 232448, "shared memory budget");
    static_assert(kAccCols + 2 * (kSfaCols + kSfbCols) <= 512, "tensor memory budget (scale columns are double buffered)");
    static_assert(kStageBytes % 1024 == 0, "stages must keep the 1024-byte alignment of the swizzled tiles");
};

constexpr int kMaxPeers = 8;  // output buffers one launch can write (this GPU's and its peers')
struct Params {
    __nv_bfloat16* C[kMaxPeers];  // every buffer gets this launch's rows (at the tiles' outRow)
    int nPeers, firstPeer;        // stores start at buffer firstPeer and go round
    int wideStores;               // 128-byte row segments (peer buffers) instead of 64-byte ones
    int outF32;                   // the output matrices hold fp32 instead of bf16 (8-bit operands only)
    uint32_t aFmt, bFmt;          // 8-bit operands: 0 = E4M3, 1 = E5M2
    const TileInfo* tiles;
    const uint8_t* sfaPacked;
    const uint8_t* sfbPacked;
    int numTilesM, tilesN, N, K, kBlocks, nTilesPerGroup128;  // nTilesPerGroup128 = ceil(N/128)
    int tmaStore;  // bf16 result in aligned matrices: whole 128-row tiles leave through TMA stores (one per matrix)
    int aBoxShort;  // bytes one load of A delivers less than a whole 128-row box (fewer than 16 rows in all: 16-row box)
    CommArgs comm;  // sharded form: end-of-step exchange with the other ranks (nranks == 0: none)
};
// Tensor maps of the output matrices (TMA stores): one per buffer, this GPU's and its peers'.
struct OutMaps {
    CUtensorMap m[kMaxPeers];
};

// ---- scale repack ----------------------------------------------------------------------------------
// One launch rewrites the e8m0 scales of A and of B into the records the matmul copies to tensor memory.
// Block (x, y): x < numTilesA is a 128-row tile of A (rows from the tile table), otherwise a 128-row tile of B
// (group*N + tile128*128); y selects a slab of kSlab 4-byte chunks along K (128 bytes of every row).  The block reads its rows as they lie
// in memory (whole rows, coalesced), turns them in shared memory and writes whole 512-byte chunks: word w of a
// chunk holds the four scale bytes of row 32*(w&3) + (w>>2).  Rows or chunks without data get scale 1.0 (0x7F);
// the operand bytes there are zero.
//
// The same launch builds the row-tile table the matmul reads: with up to kInlineGroups groups the rows per group
// travel as a kernel argument, every A block derives its own entry and the blocks of slab 0 store theirs.  (No
// host-to-device copy is then part of the call.)  With more groups the host builds the table and copies it.
constexpr int kSlab = 32;
constexpr int kInlineGroups = 256;
struct GroupRows {
    int rows[kInlineGroups];      // rows of A per group
    int outStart[kInlineGroups];  // output row of each group's first row
};
// Entry `tile` of the table: groups in order, ceil(rows / stepRows) * (stepRows / 128) entries of 128 rows each per
// group (stepRows = 256 when CTA pairs work on 256-row tiles; the second half of a pair's tile may be empty).
__device__ __forceinline__ TileInfo tile_entry(const GroupRows& gr, int G, int stepRows, int tile)
{
    int start = 0;
    const int per = stepRows / 128;
    for (int g = 0; g < G; ++g) {
        const int mg = gr.rows[g];
        const int n = (mg + stepRows - 1) / stepRows * per;
        if (tile < n) {
            const int left = mg - tile * 128;
            return TileInfo{start + tile * 128, left <= 0 ? 0 : (left < 128 ? left : 128), g, gr.outStart[g] + tile * 128};
        }
        tile -= n;
        start += mg;
    }
    return TileInfo{start, 0, G > 0 ? G - 1 : 0, start};
}

__global__ void __launch_bounds__(256)
repack_sf_kernel(uint8_t* __restrict__ dstA, uint8_t* __restrict__ dstB, const uint8_t* __restrict__ srcA,
                 const uint8_t* __restrict__ srcB, TileInfo* __restrict__ tiles, const __grid_constant__ GroupRows gr, int G,
                 int stepRows, int numTilesA, int kChunks, int kChunksValid, int sfRowBytes, int N, int tilesPerGroup,
                 long long totalRowsA)
{
    __shared__ uint32_t sm[128][kSlab + 1];
    __shared__ TileInfo myTile;
    asm volatile("griddepcontrol.launch_dependents;");  // the matmul's CTAs may start their set-up
    const int slab0 = blockIdx.y * kSlab;
    const int nch = min(kSlab, kChunks - slab0);
    const bool isA = static_cast<int>(blockIdx.x) < numTilesA;
    const int tile = isA ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x) - numTilesA;
    long long rowBase;
    int rowsValid;
    if (isA) {
        if (threadIdx.x == 0) {
            myTile = G > 0 ? tile_entry(gr, G, stepRows, tile) : tiles[tile];
            if (G > 0 && blockIdx.y == 0) tiles[tile] = myTile;
        }
        __syncthreads();
        rowBase = myTile.rowStart;
        const long long left = totalRowsA - rowBase;
        rowsValid = left < 128 ? static_cast<int>(left) : 128;
    } else {
        const int g = tile / tilesPerGroup, t = tile - g * tilesPerGroup;
        rowBase = static_cast<long long>(g) * N + t * 128;
        rowsValid = min(128, N - t * 128);
    }
    const uint8_t* src = isA ? srcA : srcB;
    uint32_t* dst = reinterpret_cast<uint32_t*>(isA ? dstA : dstB) + (static_cast<size_t>(tile) * kChunks + slab0) * (kChunkBytes / 4);
    // 16 bytes per access when rows and slabs are made of whole groups of four chunks
    const bool vec4 = (nch % 4 == 0) && (kChunksValid % 4 == 0) && (sfRowBytes % 16 == 0) &&
                      ((reinterpret_cast<uintptr_t>(src) & 15u) == 0);
    if (vec4) {
        const int nq = nch >> 2;
        for (int idx = threadIdx.x; idx < 128 * nq; idx += blockDim.x) {
            const int r = idx / nq, q = idx - r * nq;
            uint4 v = make_uint4(0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
            if (r < rowsValid && slab0 + 4 * q < kChunksValid)
                v = __ldg(reinterpret_cast<const uint4*>(src + (rowBase + r) * sfRowBytes + (slab0 + 4 * q) * 4));
            sm[r][4 * q] = v.x;
            sm[r][4 * q + 1] = v.y;
            sm[r][4 * q + 2] = v.z;
            sm[r][4 * q + 3] = v.w;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < 32 * nch; idx += blockDim.x) {
            const int ch = idx >> 5, l = idx & 31;  // words 4l .. 4l+3 of the chunk: rows l, 32+l, 64+l, 96+l
            reinterpret_cast<uint4*>(dst)[idx] = make_uint4(sm[l][ch], sm[32 + l][ch], sm[64 + l][ch], sm[96 + l][ch]);
        }
    } else {
        for (int idx = threadIdx.x; idx < 128 * nch; idx += blockDim.x) {
            const int r = idx / nch, ch = idx - r * nch;
            uint32_t v = 0x7F7F7F7Fu;
            if (r < rowsValid && slab0 + ch < kChunksValid)
                v = *reinterpret_cast<const uint32_t*>(src + (rowBase + r) * sfRowBytes + (slab0 + ch) * 4);
            sm[r][ch] = v;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < 128 * nch; idx += blockDim.x) {
            const int ch = idx >> 7, w = idx & 127;
            dst[idx] = sm[(w & 3) * 32 + (w >> 2)][ch];
        }
    }
}

// ---- matmul ----------------------------------------------------------------------------------------
// Tile order.  The CTAs of one wave work on consecutive tile indices, so the order decides what the wave keeps
// in L2.  Columns are cut into bands of kBandN tiles; inside a band the column index runs fastest, then the row
// tile.  A wave then covers (number of CTAs / kBandN) row tiles x kBandN column tiles: a few MB of A and the
// matching slice of B of the one or two groups those rows belong to, and every byte of A and B comes from HBM
// about once.  (Row tile fastest would sweep all of A once per column tile.)
constexpr int kBandN = 8;
__device__ __forceinline__ void tile_coords(int tile, int numTilesM, int tilesN, int& mt, int& nt)
{
    const int perBand = numTilesM * kBandN;
    const int band = tile / perBand;
    const int within = tile - band * perBand;
    const int width = min(kBandN, tilesN - band * kBandN);
    mt = within / width;
    nt = band * kBandN + (within - mt * width);
}

template <int BN, bool PAIR, int SFC>
__global__ void __launch_bounds__(kThreads, 1)
mxfp4_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
             const __grid_constant__ CUtensorMap tmapSfa, const __grid_constant__ CUtensorMap tmapSfb,
             const __grid_constant__ OutMaps tmapC, const __grid_constant__ Params p)
{
    using C = Cfg<BN, PAIR, SFC>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // [stages][output staging, 1024-aligned for swizzled TMA stores][barriers]
    uint8_t* outStage = smem + C::kStages * C::kStageBytes;  // [kEpiWarps][kWarpStageBytes]
    uint64_t* bars = reinterpret_cast<uint64_t*>(outStage + C::kOutBytes);
    uint64_t* fullBar = bars;
    uint64_t* emptyBar = bars + C::kStages;
    uint64_t* tmemFull = bars + 2 * C::kStages;
    uint64_t* tmemEmpty = tmemFull + 2;
    uint32_t* tmemBaseSlot = reinterpret_cast<uint32_t*>(tmemEmpty + 2);
    volatile int* abortFlag = reinterpret_cast<volatile int*>(tmemBaseSlot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int numTiles = p.numTilesM * p.tilesN;
    // work unit = CTA, or cluster of two CTAs (PAIR); rank 0 of a pair issues the MMAs.  In PAIR mode p.numTilesM
    // counts 256-row tiles and the tile table holds two consecutive 128-row entries per tile.
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const int unit = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int numUnits = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    constexpr int kTileM = PAIR ? 2 * kBM : kBM;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(&fullBar[s], 1);
            mbar_init(&emptyBar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tmemFull[a], 1);
            mbar_init(&tmemEmpty[a], PAIR ? 2 * kEpiWarps : kEpiWarps);
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
    if constexpr (PAIR) {  // the partner's barriers must exist before anything is signalled across the pair
        cluster_arrive();
        cluster_wait();
    }
    tc_fence_after();
    const uint32_t tmemBase = *tmemBaseSlot;
    const uint32_t sfCol0 = tmemBase + C::kAccCols;  // two sets of scale columns, alternating per k-block
    // everything below reads what the launch before this one wrote (row-tile table, packed scales)
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        if (elect_one()) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = unit; tile < numTiles && ok; tile += numUnits) {
                int mt, nt;
                tile_coords(tile, p.numTilesM, p.tilesN, mt, nt);
                mt = mt * (PAIR ? 2 : 1) + static_cast<int>(rank);
                const TileInfo ti = p.tiles[mt];
                const int n0 = nt * BN;
                const size_t sfaRec = static_cast<size_t>(mt) * p.kBlocks;  // 1 KiB records: [A tile][k-block]
                const size_t sfbRec = (static_cast<size_t>(ti.group) * p.nTilesPerGroup128 + n0 / 128) * p.kBlocks;
                for (int kb = 0; kb < p.kBlocks; ++kb, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    if (!(ok = mbar_wait_bounded(&emptyBar[s], ph ^ 1, abortFlag))) break;
                    uint8_t* st = smem + s * C::kStageBytes;
                    uint8_t* stSf = st + C::kABytes + C::kBBytes;
                    if constexpr (PAIR) {
                        // all loads of both CTAs are counted on the leader's barrier; the leader announces both shares
                        if (rank == 0) mbar_arrive_expect_tx(&fullBar[s], 2 * C::kLoadBytes);
                        const uint32_t bar = mapa_u32(smem_u32(&fullBar[s]), 0);
                        tma_load_2d_pair(st, &tmapA, bar, kb * kBKBytes, ti.rowStart);
                        tma_load_2d_pair(st + C::kABytes, &tmapB, bar, kb * kBKBytes,
                                         ti.group * p.N + n0 + static_cast<int>(rank) * C::kBRows);
                        tma_load_2d_pair(stSf, &tmapSfa, bar, 0, static_cast<int>(sfaRec + kb));
#pragma unroll
                        for (int t = 0; t < BN / 128; ++t)
                            tma_load_2d_pair(stSf + C::kSfaBytes + t * SFC * kChunkBytes, &tmapSfb, bar, 0,
                                             static_cast<int>(sfbRec + static_cast<size_t>(t) * p.kBlocks + kb));
                    } else {
                        mbar_arrive_expect_tx(&fullBar[s], C::kLoadBytes - p.aBoxShort);
                        tma_load_2d(st, &tmapA, &fullBar[s], kb * kBKBytes, ti.rowStart);
                        tma_load_2d(st + C::kABytes, &tmapB, &fullBar[s], kb * kBKBytes, ti.group * p.N + n0);
                        bulk_load(stSf, p.sfaPacked + (sfaRec + kb) * C::kSfaBytes, C::kSfaBytes, &fullBar[s]);
#pragma unroll
                        for (int t = 0; t < BN / 128; ++t)
                            bulk_load(stSf + C::kSfaBytes + t * SFC * kChunkBytes,
                                      p.sfbPacked + (sfbRec + static_cast<size_t>(t) * p.kBlocks + kb) * SFC * kChunkBytes,
                                      SFC * kChunkBytes, &fullBar[s]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0 && elect_one()) {
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = unit; tile < numTiles && ok; tile += numUnits, ++local) {
                const int acc = local % C::kAccStages;
                const uint32_t accPh = (local / C::kAccStages) & 1;
                if (!(ok = mbar_wait_bounded(&tmemEmpty[acc], accPh ^ 1, abortFlag))) break;
                tc_fence_after();
                const uint32_t tmemD = tmemBase + acc * BN;
                for (int kb = 0; kb < p.kBlocks; ++kb, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    if (!(ok = mbar_wait_bounded(&fullBar[s], ph, abortFlag))) break;
                    tc_fence_after();
                    const uint32_t base = smem_u32(smem + s * C::kStageBytes);
                    const uint32_t sfaSmem = base + C::kABytes + C::kBBytes;
                    const uint32_t sfbSmem = sfaSmem + C::kSfaBytes;
                    // the copy for this k-block must not wait for the previous k-block's MMAs to finish reading theirs
                    const uint32_t sfaCol = sfCol0 + (it & 1) * (C::kSfaCols + C::kSfbCols);
                    const uint32_t sfbCol = sfaCol + C::kSfaCols;
                    // scales: shared -> tensor memory.  Chunk q of A -> columns sfaCol + 4q; chunk q of the
                    // 128-row tile t of B -> columns sfbCol + q*(BN/32) + 4t.
#pragma unroll
                    for (int q = 0; q < SFC; ++q) {
                        const uint64_t da = smem_desc_noswizzle(sfaSmem + q * kChunkBytes, 0, 128);
                        if constexpr (PAIR) tc_cp_32x128b_warpx4_pair(sfaCol + 4 * q, da);  // each CTA from its own shared memory
                        else tc_cp_32x128b_warpx4(sfaCol + 4 * q, da);
#pragma unroll
                        for (int t = 0; t < BN / 128; ++t) {
                            const uint64_t db = smem_desc_noswizzle(sfbSmem + (t * SFC + q) * kChunkBytes, 0, 128);
                            if constexpr (PAIR) tc_cp_32x128b_warpx4_pair(sfbCol + q * (BN / 32) + 4 * t, db);
                            else tc_cp_32x128b_warpx4(sfbCol + q * (BN / 32) + 4 * t, db);
                        }
                    }
                    const uint64_t descA = smem_desc_sw128(base);
                    const uint64_t descB = smem_desc_sw128(base + C::kABytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if constexpr (SFC == 2) {
                            // 4-bit: K = 64 per MMA = 32 bytes: chunk k/2, scale bytes (k%2)*2 and (k%2)*2+1 of each column
                            const uint32_t sfId = (k & 1) * 2;
                            if constexpr (PAIR)
                                mma_mxf4_pair(tmemD, descA + 2 * k, descB + 2 * k, idesc_mxf4(kTileM, BN, sfId, sfId), (kb | k) != 0,
                                              sfaCol + 4 * (k >> 1), sfbCol + (k >> 1) * (BN / 32));
                            else
                                mma_mxf4(tmemD, descA + 2 * k, descB + 2 * k, idesc_mxf4(kTileM, BN, sfId, sfId), (kb | k) != 0,
                                         sfaCol + 4 * (k >> 1), sfbCol + (k >> 1) * (BN / 32));
                        } else {
                            // 8-bit: K = 32 per MMA = 32 bytes: one chunk per k-block, scale byte k of each column
                            const uint32_t id = idesc_mxf8(kTileM, BN, p.aFmt, p.bFmt, k, k);
                            if constexpr (PAIR) mma_mxf8_pair(tmemD, descA + 2 * k, descB + 2 * k, id, (kb | k) != 0, sfaCol, sfbCol);
                            else mma_mxf8(tmemD, descA + 2 * k, descB + 2 * k, id, (kb | k) != 0, sfaCol, sfbCol);
                        }
                    }
                    if constexpr (PAIR) tc_commit_pair(&emptyBar[s], 3);
                    else tc_commit(&emptyBar[s]);
                }
                if (ok) {
                    if constexpr (PAIR) tc_commit_pair(&tmemFull[acc], 3);
                    else tc_commit(&tmemFull[acc]);
                }
            }
        }
    } else {
        // epilogue: warp w reads TMEM lanes 32*(w%4)..; warps 2..5 take the lower half of the accumulator columns,
        // warps 6..9 the upper half.  Each warp first pulls its whole share into registers and hands the accumulator
        // back to the MMA warp, so the conversion and the stores overlap the next tile's main loop even when there
        // is only one accumulator stage.
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        constexpr int kChunks = BN / 64;  // 32-column chunks per warp
        uint32_t local = 0;
        bool ok = true;
        for (int tile = unit; tile < numTiles && ok; tile += numUnits, ++local) {
            const int acc = local % C::kAccStages;
            const uint32_t accPh = (local / C::kAccStages) & 1;
            int mt, nt;
            tile_coords(tile, p.numTilesM, p.tilesN, mt, nt);
            mt = mt * (PAIR ? 2 : 1) + static_cast<int>(rank);
            const TileInfo ti = p.tiles[mt];
            const int n0 = nt * BN + half * (BN / 2);
            if (!(ok = mbar_wait_bounded(&tmemFull[acc], accPh, abortFlag))) break;
            tc_fence_after();
            const uint32_t taddr = tmemBase + acc * BN + half * (BN / 2) + (static_cast<uint32_t>(q * 32) << 16);
            uint32_t r[kChunks][32];
#pragma unroll
            for (int c = 0; c < kChunks; ++c) tmem_ld_32x32b_x32(taddr + c * 32, r[c]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                // The leader's barrier.  A relaxed arrive: the barrier guards tensor memory only, whose reads are complete
                // (tcgen05.wait::ld above); a release would also wait for this thread's earlier stores of the previous
                // tile to become visible, which the MMA thread never reads -- and with one accumulator stage the tensor
                // pipe stands still for that long (measured: 119 -> 112 us per call on config 5).
                if constexpr (PAIR) mbar_arrive_cluster_relaxed(mapa_u32(smem_u32(&tmemEmpty[acc]), 0));
                else mbar_arrive(&tmemEmpty[acc]);
            }

            const int rIn = q * 32 + lane;
            const bool rowOk = rIn < ti.rowsValid;
            bool vecStore = (p.N % 8 == 0);
            for (int pi = 0; pi < p.nPeers; ++pi) vecStore = vecStore && ((reinterpret_cast<uintptr_t>(p.C[pi]) & 15u) == 0);
            uint8_t* stageW = outStage + (warp - 2) * C::kWarpStageBytes;
            if (p.tmaStore && ti.rowsValid != kBM) {
                // this tile takes a per-thread path through the same staging bytes: the TMA stores of the previous tile
                // must have read them
                if (lane == 0) bulk_wait_group_read<0>();
                __syncwarp();
            }
#pragma unroll
            for (int cp = 0; cp < kChunks / 2; ++cp) {  // two 32-column chunks = 64 columns = 128 bytes of bf16 per row
                const int n = n0 + cp * 64;
                if (n >= p.N) continue;  // uniform over the warp
                if (p.outF32) {  // fp32 output: every thread writes its own row (no conversion, no transpose)
                    if (rowOk) {
                        for (int pi = 0; pi < p.nPeers; ++pi) {
                            float* crow = reinterpret_cast<float*>(p.C[pi]) + static_cast<size_t>(ti.outRow + rIn) * p.N + n;
#pragma unroll
                            for (int j = 0; j < 64; ++j)
                                if (n + j < p.N) crow[j] = __uint_as_float(r[2 * cp + (j >> 5)][j & 31]);
                        }
                    }
                    continue;
                }
                // fp32 -> bfloat16 pairs without a branch per pair (a branch keeps the conversions from overlapping); the
                // saturation of finite overflow is applied afterwards, only if an infinity came out at all
                uint32_t packed[32];
                uint32_t inf = 0;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    uint32_t w;
                    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(__uint_as_float(r[2 * cp + (j >> 4)][2 * (j & 15) + 1])),
                        "f"(__uint_as_float(r[2 * cp + (j >> 4)][2 * (j & 15)])));
                    inf |= (w & 0x7FFF7FFFu) + 0x00800080u;   // bit 15 / 31 set: exponent all ones
                    packed[j] = w;
                }
                if (__builtin_expect((inf & 0x80008000u) != 0, 0)) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        packed[j] = pack_bf16x2_sat(__uint_as_float(r[2 * cp + (j >> 4)][2 * (j & 15)]),
                                                    __uint_as_float(r[2 * cp + (j >> 4)][2 * (j & 15) + 1]));
                }
                if (p.tmaStore && ti.rowsValid == kBM) {
                    // A whole tile of one aligned matrix: sixteen rows at a time go into the warp's swizzled staging rows
                    // (16-byte piece v of row r at v ^ (r & 7)) and leave as one TMA store; columns past N are clipped
                    // by the tensor map.  (A tile that ends inside its group's rows must not touch the next group's.)
                    // 2 KiB at the first 1024-byte boundary inside this warp's own staging region (the region is 2.5 KiB and
                    // starts at a multiple of 512 bytes), so that warps on different paths never share staging bytes
                    uint8_t* stageT = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(stageW) + 1023) & ~uintptr_t(1023));
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
                        if (lane == 0) {
                            // one store per output matrix (this GPU's and the peers'), all reading the same staged rows
                            for (int pi = 0; pi < p.nPeers; ++pi) {
                                int b = p.firstPeer + pi;
                                if (b >= p.nPeers) b -= p.nPeers;
                                tma_store_2d(&tmapC.m[b], stageT, n, ti.outRow + q * 32 + h * 16);
                            }
                            bulk_commit_group();
                        }
                    }
                } else if (n + 64 <= p.N && vecStore && !p.wideStores) {
                    // One output buffer in this GPU's memory: 64-byte row segments, all thirty-two rows in one pass
                    // (fewer instructions and warp barriers than the 128-byte form below, and L2 merges the halves).
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
#pragma unroll
                        for (int v = 0; v < 4; ++v)
                            *reinterpret_cast<uint4*>(stageW + lane * kNarrowPitch + v * 16) =
                                make_uint4(packed[16 * c + 4 * v], packed[16 * c + 4 * v + 1], packed[16 * c + 4 * v + 2],
                                           packed[16 * c + 4 * v + 3]);
                        __syncwarp();
                        const int piece = lane & 3;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int rl = i * 8 + (lane >> 2);
                            const uint4 val = *reinterpret_cast<const uint4*>(stageW + rl * kNarrowPitch + piece * 16);
                            if (q * 32 + rl < ti.rowsValid)
                                *reinterpret_cast<uint4*>(p.C[0] + static_cast<size_t>(ti.outRow + q * 32 + rl) * p.N + n + c * 32 +
                                                          piece * 8) = val;
                        }
                        __syncwarp();
                    }
                } else if (n + 64 <= p.N && vecStore) {
                    // Transpose through this warp's staging rows, sixteen rows at a time: every store instruction then
                    // writes four complete 128-byte row segments (whole lines, which is what both L2 and NVLink move
                    // best) instead of thirty-two 16-byte pieces of thirty-two different rows.
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
                            const int row = q * 32 + h * 16 + rl;
                            const uint4 val = *reinterpret_cast<const uint4*>(stageW + rl * kStagePitch + piece * 16);
                            if (row < ti.rowsValid) {
                                const size_t off = static_cast<size_t>(ti.outRow + row) * p.N + n + piece * 8;
                                for (int pi = 0; pi < p.nPeers; ++pi) {
                                    int b = p.firstPeer + pi;
                                    if (b >= p.nPeers) b -= p.nPeers;
                                    *reinterpret_cast<uint4*>(p.C[b] + off) = val;
                                }
                            }
                        }
                        __syncwarp();
                    }
                } else if (rowOk) {
                    for (int pi = 0; pi < p.nPeers; ++pi) {
                        __nv_bfloat16* crow = p.C[pi] + static_cast<size_t>(ti.outRow + rIn) * p.N + n;
#pragma unroll
                        for (int w = 0; w < 32; ++w) {
                            if (n + 2 * w < p.N) crow[2 * w] = __ushort_as_bfloat16(static_cast<unsigned short>(packed[w] & 0xFFFFu));
                            if (n + 2 * w + 1 < p.N) crow[2 * w + 1] = __ushort_as_bfloat16(static_cast<unsigned short>(packed[w] >> 16));
                        }
                    }
                }
            }
        }
        if (lane == 0) {
            // the staging rows must stay valid until the last TMA store has read them; with an exchange at the end of
            // the step the stores must also have been performed before this CTA reports itself done
            if (p.comm.nranks > 1) bulk_wait_group_all();
            else bulk_wait_group_read<0>();
        }
    }

    __syncthreads();
    if (p.comm.nranks > 1 && threadIdx.x == 0) {
        if (!comm_finish(p.comm, gridDim.x, c_waitCycles)) atomicExch(&g_mxfp4_status, 2);
    }
    if constexpr (PAIR) {  // neither CTA may leave (or free tensor memory) while its partner can still touch it
        cluster_arrive();
        cluster_wait();
    }
    if (*abortFlag) {
        if (threadIdx.x == 0) atomicExch(&g_mxfp4_status, 1);
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

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Layout {
    size_t tileOff, sfaOff, sfbOff, total;
    int tilesM, kBlocks, nTiles128;
};
Layout make_layout(int64_t sumM, int G, int K, int N, int sfc = 2)
{
    Layout L{};
    // upper bound on 128-row entries: with 256-row pair tiles every group may add up to two partly filled entries
    L.tilesM = static_cast<int>((sumM + kBM - 1) / kBM + 2 * static_cast<int64_t>(G) + 2);
    L.kBlocks = (K + 128 * sfc - 1) / (128 * sfc);  // a k-block row is 128 bytes: 256 4-bit or 128 8-bit elements
    L.nTiles128 = 2 * ((N + 255) / 256);  // even, so a 256-wide N tile always finds both of its 128-row halves
    L.tileOff = 0;
    L.sfaOff = align_up(static_cast<size_t>(L.tilesM) * sizeof(TileInfo), 256);
    L.sfbOff = L.sfaOff + align_up(static_cast<size_t>(L.tilesM) * L.kBlocks * sfc * kChunkBytes, 256);
    L.total = L.sfbOff + align_up(static_cast<size_t>(G) * L.nTiles128 * L.kBlocks * sfc * kChunkBytes, 256);
    return L;
}

template <int BN, bool PAIR, int SFC = 2>
ascq_status launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb,
                   const OutMaps& tc, Params p, cudaStream_t st)
{
    using C = Cfg<BN, PAIR, SFC>;
    static PerDeviceOnce attrSet;  // the attribute is per device: a process may drive several GPUs
    const int dev = current_device();
    if (!attrSet.done(dev)) {
        ASCQ_CUDA_CHECK(cudaFuncSetAttribute(mxfp4_kernel<BN, PAIR, SFC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(C::kSmemBytes)));
        attrSet.mark(dev);
    }
    p.tilesN = (p.N + BN - 1) / BN;
    const int tiles = p.numTilesM * p.tilesN;
    // Programmatic dependent launch: the CTAs may become resident and run their set-up (barriers, tensor memory,
    // descriptor prefetch) while the scale-repack launch before this one drains; they wait for its results with
    // griddepcontrol.wait before the first dependent read.
    const int units = PAIR ? sm_count() / 2 : sm_count();
    const int grid = (tiles < units ? tiles : units) * (PAIR ? 2 : 1);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
    if constexpr (PAIR) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 2;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    ASCQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, mxfp4_kernel<BN, PAIR, SFC>, ta, tb, tsa, tsb, tc, p));
    ASCQ_CUDA_CHECK(cudaGetLastError());
    return ASCQ_OK;
}

}  // namespace
}  // namespace ascq

using namespace ascq;

extern "C" size_t ascq_group_matmul_mxfp4_workspace_size(int64_t sumM, int G, int K, int N)
{
    if (sumM < 0 || G <= 0 || K <= 0 || N <= 0) return 0;
    return make_layout(sumM, G, K, N).total;
}

// Shared body of the entry points.  outBufs: nBufs bf16 matrices with row stride N; group g's rows go to rows
// outRowStart_host[g].. of each (NULL: the groups follow each other as in A).
struct Mx8Args {  // 8-bit operands (kind::mxf8f6f4): formats 0 = E4M3, 1 = E5M2; output bf16 or fp32
    uint32_t aFmt, bFmt;
    int outF32;
};
static ascq_status run_mxfp4(void* const* outBufs, int nBufs, int firstBuf, const int64_t* outRowStart_host,
                             const uint8_t* A_fp4, const uint8_t* sA_e8m0, const uint8_t* B_fp4, const uint8_t* sB_e8m0,
                             const int64_t* groupList_host, int G, int K, int N, void* workspace, size_t workspaceBytes,
                             void* stream, const Mx8Args* mx8 = nullptr, const uint8_t* sB_packed = nullptr,
                             const ascq_comm* comm = nullptr)
{
    // sB_packed: the scales of B already in the packed order (weights are static: ascq_group_matmul_mxfp4_pack_scale_b once)
    const int sfc = mx8 ? 1 : 2;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!outBufs || nBufs < 1 || nBufs > kMaxPeers)
        return fail(ASCQ_ERR_INVALID_ARG, "between 1 and %d output buffers are supported", kMaxPeers);
    for (int i = 0; i < nBufs; ++i)
        if (!outBufs[i]) return fail(ASCQ_ERR_INVALID_ARG, "output buffer %d is NULL", i);
    if (!A_fp4 || !sA_e8m0 || !B_fp4 || (!sB_e8m0 && !sB_packed) || !groupList_host)
        return fail(ASCQ_ERR_INVALID_ARG, "C, A, sA, B, sB and groupList must not be NULL");
    if (sB_packed && (reinterpret_cast<uintptr_t>(sB_packed) & 255u))
        return fail(ASCQ_ERR_ALIGNMENT, "packed scales must be 256-byte aligned");
    if (G <= 0 || N <= 0 || K <= 0) return fail(ASCQ_ERR_INVALID_ARG, "G, N, K must be positive");
    if (K % 128 != 0) return fail(ASCQ_ERR_ALIGNMENT, "K %d must be a multiple of 128", K);
    if (!aligned16(A_fp4) || !aligned16(B_fp4)) return fail(ASCQ_ERR_ALIGNMENT, "A and B must be 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(sA_e8m0) & 3u) || (reinterpret_cast<uintptr_t>(sB_e8m0) & 3u))
        return fail(ASCQ_ERR_ALIGNMENT, "scale tensors must be 4-byte aligned");
    int64_t sumM = 0;
    for (int g = 0; g < G; ++g) {
        if (groupList_host[g] < 0) return fail(ASCQ_ERR_INVALID_ARG, "groupList[%d] is negative", g);
        sumM += groupList_host[g];
    }
    if (sumM == 0) return comm ? ascq_comm_barrier(const_cast<ascq_comm*>(comm), stream) : ASCQ_OK;
    if (sumM > 0x7FFFFFFF - 256 || static_cast<int64_t>(G) * N > 0x7FFFFFFF)
        return fail(ASCQ_ERR_INVALID_ARG, "problem too large for 32-bit row indices");
    if (outRowStart_host)
        for (int g = 0; g < G; ++g)
            if (outRowStart_host[g] < 0 || outRowStart_host[g] > 0x7FFFFFFF - 256)
                return fail(ASCQ_ERR_INVALID_ARG, "outRowStart[%d] is out of range", g);
    const Layout L = make_layout(sumM, G, K, N, sfc);
    if (!workspace || workspaceBytes < L.total)
        return fail(ASCQ_ERR_INVALID_ARG, "workspace of %zu bytes needed, %zu given", L.total, workspaceBytes);
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(ASCQ_ERR_ALIGNMENT, "workspace must be 256-byte aligned");

    // CTA pairs on 256-row tiles (B fetched once per pair) when N allows; ASCQ_MXFP4_TILE=single selects single
    // CTAs on 128-row tiles, which waste fewer rows when the groups are much shorter than 256 rows.
    // The pair variant is taken unless rounding every group up to 256 rows adds more than a tenth to the rows that
    // rounding up to 128 already computes.
    int64_t padded128 = 0, padded256 = 0;
    for (int g = 0; g < G; ++g) {
        padded128 += (groupList_host[g] + 127) / 128 * 128;
        padded256 += (groupList_host[g] + 255) / 256 * 256;
    }
    bool pair = N >= 256 && padded256 * 10 <= padded128 * 11;
    if (const char* e = getenv("ASCQ_MXFP4_TILE")) {
        if (!strcmp(e, "single")) pair = false;
        else if (!strcmp(e, "pair")) pair = N >= 256;
    }
    // Row-tile table: zero-row groups are skipped (quant_group_matmul_custom.asc:265-267).  One entry per 128 rows;
    // in pair mode entries come in twos (the two halves of a 256-row tile, the second possibly empty).
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    const int64_t step = pair ? 2 * kBM : kBM;
    int numTilesM = 0;
    GroupRows gr{};
    const bool inlineGroups = G <= kInlineGroups;
    if (inlineGroups) {
        int64_t start = 0;
        for (int g = 0; g < G; ++g) {
            gr.rows[g] = static_cast<int>(groupList_host[g]);
            gr.outStart[g] = static_cast<int>(outRowStart_host ? outRowStart_host[g] : start);
            start += groupList_host[g];
            numTilesM += static_cast<int>((groupList_host[g] + step - 1) / step * (step / kBM));
        }
    } else {
        std::vector<TileInfo> tiles;
        tiles.reserve(L.tilesM);
        int64_t start = 0;
        for (int g = 0; g < G; ++g) {
            const int64_t mg = groupList_host[g];
            for (int64_t r = 0; r < mg; r += step) {
                for (int64_t h = 0; h < step; h += kBM) {
                    const int64_t left = mg - (r + h);
                    const int64_t out0 = outRowStart_host ? outRowStart_host[g] : start;
                    TileInfo t{static_cast<int>(start + r + h), static_cast<int>(left <= 0 ? 0 : (left < kBM ? left : kBM)), g,
                               static_cast<int>(out0 + r + h)};
                    tiles.push_back(t);
                }
            }
            start += mg;
        }
        ASCQ_CUDA_CHECK(cudaMemcpyAsync(ws + L.tileOff, tiles.data(), tiles.size() * sizeof(TileInfo), cudaMemcpyHostToDevice, st));
        // the copy above stages pageable memory before returning, so `tiles` may go out of scope afterwards
        numTilesM = static_cast<int>(tiles.size());
    }

    const int kChunks = L.kBlocks * sfc;
    const int sfRowBytes = K / 32;
    {
        // with prepacked scales of B only the A tiles are repacked
        const dim3 grid(static_cast<unsigned>(numTilesM + (sB_packed ? 0 : G * L.nTiles128)),
                        static_cast<unsigned>((kChunks + kSlab - 1) / kSlab));
        repack_sf_kernel<<<grid, 256, 0, st>>>(ws + L.sfaOff, ws + L.sfbOff, sA_e8m0, sB_e8m0,
                                               reinterpret_cast<TileInfo*>(ws + L.tileOff), gr, inlineGroups ? G : 0,
                                               static_cast<int>(step), numTilesM, kChunks, K / 128, sfRowBytes, N, L.nTiles128, sumM);
        ASCQ_CUDA_CHECK(cudaGetLastError());
    }

    Params p{};
    p.nPeers = nBufs;
    for (int i = 0; i < nBufs; ++i) p.C[i] = static_cast<__nv_bfloat16*>(outBufs[i]);
    p.firstPeer = ((firstBuf % nBufs) + nBufs) % nBufs;
    p.wideStores = nBufs > 1;
    p.comm = comm_args(comm);
    if (mx8) { p.aFmt = mx8->aFmt; p.bFmt = mx8->bFmt; p.outF32 = mx8->outF32; }
    if (const char* e = getenv("ASCQ_MXFP4_STORE")) p.wideStores = !strcmp(e, "wide") ? 1 : (!strcmp(e, "narrow") && nBufs == 1 ? 0 : p.wideStores);
    p.tiles = reinterpret_cast<const TileInfo*>(ws + L.tileOff);
    p.sfaPacked = ws + L.sfaOff;
    p.sfbPacked = sB_packed ? sB_packed : ws + L.sfbOff;
    p.numTilesM = pair ? numTilesM / 2 : numTilesM;
    p.N = N; p.K = K; p.kBlocks = L.kBlocks; p.nTilesPerGroup128 = L.nTiles128;

    const bool wide = N >= 256;
    CUtensorMap ta, tb, tsa, tsb;
    const uint64_t rowBytes = mx8 ? static_cast<uint64_t>(K) : static_cast<uint64_t>(K / 2);
    // (a matrix of fewer than 16 rows loads at two thirds of the speed through a 128-row box: see gemm_w8a8.cu; the rows
    // of the stage the short box leaves stale feed accumulator rows that are never stored)
    const int aBoxRows = (sumM < 16 && !pair) ? 16 : kBM;
    p.aBoxShort = (kBM - aBoxRows) * 128;
    ascq_status rc = make_tmap_u8(&ta, A_fp4, static_cast<uint64_t>(sumM), rowBytes, aBoxRows);
    if (rc != ASCQ_OK) return rc;
    rc = make_tmap_u8(&tb, B_fp4, static_cast<uint64_t>(G) * N, rowBytes, pair ? 128 : (wide ? 256 : 128));
    if (rc != ASCQ_OK) return rc;
    // the packed scales as 1 KiB records (pair mode loads them with tensor copies so that the partner CTA's loads
    // can be counted on the leader's barrier)
    rc = make_tmap_kib_rows(&tsa, ws + L.sfaOff, static_cast<uint64_t>(numTilesM) * L.kBlocks, sfc * kChunkBytes);
    if (rc != ASCQ_OK) return rc;
    rc = make_tmap_kib_rows(&tsb, p.sfbPacked, static_cast<uint64_t>(G) * L.nTiles128 * L.kBlocks, sfc * kChunkBytes);
    if (rc != ASCQ_OK) return rc;
    // bf16 result in one 16-byte aligned matrix whose rows are whole 16-byte pieces: TMA stores for whole tiles
    // (ASCQ_MXFP4_STORE=narrow|wide keeps the per-thread stores).  The row extent of the map only bounds the clipping;
    // tiles that are written this way lie inside the matrix by construction.
    OutMaps tc;
    for (int i = 0; i < kMaxPeers; ++i) tc.m[i] = ta;  // placeholders; the kernel reads maps [0, nPeers) and only for TMA stores
    p.tmaStore = !p.outF32 && N % 8 == 0 && getenv("ASCQ_MXFP4_STORE") == nullptr;
    for (int i = 0; i < nBufs && p.tmaStore; ++i) p.tmaStore = aligned16(outBufs[i]);
    if (p.tmaStore) {
        // one map per output matrix (this GPU's and the peer-mapped ones): the store path only
        for (int i = 0; i < nBufs; ++i) {
            rc = make_tmap_out16(&tc.m[i], outBufs[i], 1ull << 30, static_cast<uint64_t>(N), static_cast<uint64_t>(N), 16);
            if (rc != ASCQ_OK) return rc;
        }
    }
    if (mx8) {
        if (pair) return launch<256, true, 1>(ta, tb, tsa, tsb, tc, p, st);
        return wide ? launch<256, false, 1>(ta, tb, tsa, tsb, tc, p, st) : launch<128, false, 1>(ta, tb, tsa, tsb, tc, p, st);
    }
    if (pair) return launch<256, true>(ta, tb, tsa, tsb, tc, p, st);
    return wide ? launch<256, false>(ta, tb, tsa, tsb, tc, p, st) : launch<128, false>(ta, tb, tsa, tsb, tc, p, st);
}

extern "C" ascq_status ascq_group_matmul_mxfp4(void* C_bf16, const uint8_t* A_fp4, const uint8_t* sA_e8m0,
                                               const uint8_t* B_fp4, const uint8_t* sB_e8m0, const int64_t* groupList_host,
                                               int G, int K, int N, void* workspace, size_t workspaceBytes, void* stream)
{
    if (!C_bf16) return fail(ASCQ_ERR_INVALID_ARG, "C, A, sA, B, sB and groupList must not be NULL");
    void* bufs[1] = {C_bf16};
    return run_mxfp4(bufs, 1, 0, nullptr, A_fp4, sA_e8m0, B_fp4, sB_e8m0, groupList_host, G, K, N, workspace, workspaceBytes,
                     stream);
}

// ---- static weights: pack the scales of B once --------------------------------------------------------------------
extern "C" size_t ascq_group_matmul_mxfp4_packed_scale_b_size(int G, int K, int N)
{
    if (G <= 0 || K <= 0 || N <= 0) return 0;
    const Layout L = make_layout(0, G, K, N);
    return align_up(static_cast<size_t>(G) * L.nTiles128 * L.kBlocks * 2 * kChunkBytes, 256);
}

extern "C" ascq_status ascq_group_matmul_mxfp4_pack_scale_b(uint8_t* sB_packed, const uint8_t* sB_e8m0, int G, int K, int N,
                                                            void* stream)
{
    if (!sB_packed || !sB_e8m0) return fail(ASCQ_ERR_INVALID_ARG, "sB_packed and sB must not be NULL");
    if (G <= 0 || N <= 0 || K <= 0) return fail(ASCQ_ERR_INVALID_ARG, "G, N, K must be positive");
    if (K % 128 != 0) return fail(ASCQ_ERR_ALIGNMENT, "K %d must be a multiple of 128", K);
    if ((reinterpret_cast<uintptr_t>(sB_packed) & 255u) || (reinterpret_cast<uintptr_t>(sB_e8m0) & 3u))
        return fail(ASCQ_ERR_ALIGNMENT, "sB_packed must be 256-byte aligned, sB 4-byte aligned");
    const Layout L = make_layout(0, G, K, N);
    const int kChunks = L.kBlocks * 2;
    const dim3 grid(static_cast<unsigned>(G * L.nTiles128), static_cast<unsigned>((kChunks + kSlab - 1) / kSlab));
    const GroupRows none{};
    repack_sf_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(nullptr, sB_packed, nullptr, sB_e8m0, nullptr, none, 0, 128, 0,
                                                                          kChunks, K / 128, K / 32, N, L.nTiles128, 0);
    ASCQ_CUDA_CHECK(cudaGetLastError());
    return ASCQ_OK;
}

extern "C" ascq_status ascq_group_matmul_mxfp4_prepacked(void* C_bf16, const uint8_t* A_fp4, const uint8_t* sA_e8m0,
                                                         const uint8_t* B_fp4, const uint8_t* sB_packed,
                                                         const int64_t* groupList_host, int G, int K, int N, void* workspace,
                                                         size_t workspaceBytes, void* stream)
{
    if (!C_bf16 || !sB_packed) return fail(ASCQ_ERR_INVALID_ARG, "C, A, sA, B, sB and groupList must not be NULL");
    void* bufs[1] = {C_bf16};
    return run_mxfp4(bufs, 1, 0, nullptr, A_fp4, sA_e8m0, B_fp4, nullptr, groupList_host, G, K, N, workspace, workspaceBytes,
                     stream, nullptr, sB_packed);
}

extern "C" ascq_status ascq_group_matmul_mxfp4_scatter(void* const* C_bufs, int nBufs, int firstBuf,
                                                       const int64_t* outRowStart_host, const uint8_t* A_fp4,
                                                       const uint8_t* sA_e8m0, const uint8_t* B_fp4, const uint8_t* sB_e8m0,
                                                       const int64_t* groupList_host, int G, int K, int N, void* workspace,
                                                       size_t workspaceBytes, void* stream)
{
    return run_mxfp4(C_bufs, nBufs, firstBuf, outRowStart_host, A_fp4, sA_e8m0, B_fp4, sB_e8m0, groupList_host, G, K, N,
                     workspace, workspaceBytes, stream);
}

extern "C" size_t ascq_group_matmul_mxfp8_workspace_size(int64_t sumM, int G, int K, int N)
{
    if (sumM < 0 || G <= 0 || K <= 0 || N <= 0) return 0;
    return make_layout(sumM, G, K, N, 1).total;
}

extern "C" ascq_status ascq_group_matmul_mxfp8(void* C, ascq_dtype cT, const uint8_t* A_fp8, ascq_dtype aT, const uint8_t* sA_e8m0,
                                               const uint8_t* B_fp8, ascq_dtype bT, const uint8_t* sB_e8m0,
                                               const int64_t* groupList_host, int G, int K, int N, void* workspace,
                                               size_t workspaceBytes, void* stream)
{
    if (!C) return fail(ASCQ_ERR_INVALID_ARG, "C, A, sA, B, sB and groupList must not be NULL");
    if ((aT != ASCQ_DT_FP8_E4M3 && aT != ASCQ_DT_FP8_E5M2) || (bT != ASCQ_DT_FP8_E4M3 && bT != ASCQ_DT_FP8_E5M2))
        return fail(ASCQ_ERR_UNSUPPORTED, "operands must be fp8_e4m3fn or fp8_e5m2");
    if (cT != ASCQ_DT_BF16 && cT != ASCQ_DT_F32) return fail(ASCQ_ERR_UNSUPPORTED, "output must be bfloat16_t or float");
    void* bufs[1] = {C};
    const Mx8Args mx8{aT == ASCQ_DT_FP8_E5M2 ? 1u : 0u, bT == ASCQ_DT_FP8_E5M2 ? 1u : 0u, cT == ASCQ_DT_F32 ? 1 : 0};
    return run_mxfp4(bufs, 1, 0, nullptr, A_fp8, sA_e8m0, B_fp8, sB_e8m0, groupList_host, G, K, N, workspace, workspaceBytes,
                     stream, &mx8);
}

// ---- group-parallel form: one rank's share, reassembly and end-of-step exchange inside the launch ----------------
extern "C" ascq_status ascq_group_matmul_mxfp4_sharded(ascq_comm* comm, void* const* C_bufs, const uint8_t* A_local,
                                                       const uint8_t* sA_local, const uint8_t* B_local, const uint8_t* sB_local,
                                                       const int64_t* groupList_host, int G, int K, int N, void* workspace,
                                                       size_t workspaceBytes, void* stream)
{
    if (!comm) return fail(ASCQ_ERR_INVALID_ARG, "the communicator must not be NULL");
    if (!C_bufs || !groupList_host || G <= 0) return fail(ASCQ_ERR_INVALID_ARG, "C_bufs and groupList must not be NULL and G positive");
    // this rank's groups in ascending order, as its A / B hold them; their output rows are the groups' global row offsets
    std::vector<int> owner(static_cast<size_t>(G));
    const ascq_status rc = ascq_shard_groups_lpt(groupList_host, G, comm->nranks, owner.data());
    if (rc != ASCQ_OK) return rc;
    std::vector<int64_t> mine, outStart;
    int64_t start = 0;
    for (int g = 0; g < G; ++g) {
        if (owner[g] == comm->rank) {
            mine.push_back(groupList_host[g]);
            outStart.push_back(start);
        }
        start += groupList_host[g];
    }
    if (mine.empty()) return ascq_comm_barrier(comm, stream);  // no work here, but the other ranks wait for this one
    return run_mxfp4(C_bufs, comm->nranks, comm->rank + 1, outStart.data(), A_local, sA_local, B_local, sB_local, mine.data(),
                     static_cast<int>(mine.size()), K, N, workspace, workspaceBytes, stream, nullptr, nullptr, comm);
}

ascq_status ascq::mxfp4_set_wait_cycles(long long cycles)
{
    ASCQ_CUDA_CHECK(cudaMemcpyToSymbol(ptx::c_waitCycles, &cycles, sizeof(cycles)));
    return ASCQ_OK;
}

// ---- entry point for callers that may not allocate device memory ------------------------------------
// The scratch the grouped matmul needs (tile table + repacked scales) lives in this fixed array instead of a
// caller buffer.  Every GPU that loads the library carries it for the life of the process.
constexpr size_t kStaticScratchBytes = size_t(16) << 20;  // 16 MiB: enough for 16 groups x 16384 rows x K 7168 x N 2048
static __device__ __align__(256) unsigned char g_mxfp4_static_scratch[kStaticScratchBytes];

namespace {
// Device address of the array on the current device.  The symbol name is only a host-side handle, so the
// address is asked for once per device (with that device current) and remembered.
ascq_status static_scratch_address(void** out)
{
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static void* addr[kMaxDevices] = {};
    int dev = -1;
    ASCQ_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(ASCQ_ERR_CUDA, "device ordinal %d is outside the supported range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_mxfp4_static_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail(ASCQ_ERR_CUDA, "cudaGetSymbolAddress for the static scratch failed: %s", cudaGetErrorString(e));
        addr[dev] = p;
    }
    *out = addr[dev];
    return ASCQ_OK;
}
}  // namespace

extern "C" size_t ascq_group_matmul_mxfp4_noalloc_max_scratch(void) { return kStaticScratchBytes; }

extern "C" ascq_status ascq_group_matmul_mxfp4_noalloc(void* C_bf16, const uint8_t* A_fp4, const uint8_t* sA_e8m0,
                                                       const uint8_t* B_fp4, const uint8_t* sB_e8m0,
                                                       const int64_t* groupList_host, int G, int K, int N, void* stream)
{
    if (!groupList_host || G <= 0 || K <= 0 || N <= 0)
        return fail(ASCQ_ERR_INVALID_ARG, "groupList must not be NULL and G, N, K must be positive");
    int64_t sumM = 0;
    for (int g = 0; g < G; ++g) {
        if (groupList_host[g] < 0) return fail(ASCQ_ERR_INVALID_ARG, "groupList[%d] is negative", g);
        sumM += groupList_host[g];
    }
    const size_t need = ascq_group_matmul_mxfp4_workspace_size(sumM, G, K, N);
    if (need > kStaticScratchBytes)
        return fail(ASCQ_ERR_INVALID_ARG,
                    "this problem needs %zu bytes of scratch but the built-in scratch holds %zu; use "
                    "ascq_group_matmul_mxfp4 with a caller workspace instead", need, kStaticScratchBytes);
    void* scratch = nullptr;
    const ascq_status rc = static_scratch_address(&scratch);
    if (rc != ASCQ_OK) return rc;
    // Every byte of scratch the kernels read (tile table, packed scales of the tiles in use) is rewritten by
    // this call before it is read, so nothing has to be cleared between calls.
    return ascq_group_matmul_mxfp4(C_bf16, A_fp4, sA_e8m0, B_fp4, sB_e8m0, groupList_host, G, K, N, scratch,
                                   kStaticScratchBytes, stream);
}

// Reads and clears this translation unit's device status word (used by ascq_matmul_status).
ascq_status ascq::mxfp4_read_status(cudaStream_t st)
{
    int v = 0, zero = 0;
    ASCQ_CUDA_CHECK(cudaMemcpyFromSymbolAsync(&v, g_mxfp4_status, sizeof(int), 0, cudaMemcpyDeviceToHost, st));
    ASCQ_CUDA_CHECK(cudaStreamSynchronize(st));
    if (v != 0) {
        ASCQ_CUDA_CHECK(cudaMemcpyToSymbolAsync(g_mxfp4_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, st));
        return fail(ASCQ_ERR_TIMEOUT, "a bounded wait inside the MX-FP4 matmul kernel expired (status %d)", v);
    }
    return ASCQ_OK;
}

// ---- reference layout adapters -----------------------------------------------------------------------
namespace ascq {
namespace {
// B [K, N/2] bytes (pairs along N) -> B [N, K/2] bytes (pairs along K).  One thread per output byte.
__global__ void __launch_bounds__(256) repack_b_kn_to_nk_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, int K, int N)
{
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const long long total = static_cast<long long>(N) * (K / 2);
    if (i >= total) return;
    const int n = static_cast<int>(i / (K / 2));
    const int k = static_cast<int>(i % (K / 2)) * 2;
    const size_t rowBytes = static_cast<size_t>(N) / 2;
    const uint8_t b0 = src[static_cast<size_t>(k) * rowBytes + n / 2];
    const uint8_t b1 = src[static_cast<size_t>(k + 1) * rowBytes + n / 2];
    const uint32_t lo = (n & 1) ? (b0 >> 4) : (b0 & 0x0Fu);
    const uint32_t hi = (n & 1) ? (b1 >> 4) : (b1 & 0x0Fu);
    dst[i] = static_cast<uint8_t>(lo | (hi << 4));
}
// scaleB stored [sK/2, N, 2] -> [N, sK].
__global__ void __launch_bounds__(256) repack_scale_b_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, int sK, int N)
{
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= static_cast<long long>(N) * sK) return;
    const int n = static_cast<int>(i / sK), sk = static_cast<int>(i % sK);
    dst[i] = src[(static_cast<size_t>(sk / 2) * N + n) * 2 + (sk & 1)];
}
}  // namespace
}  // namespace ascq

extern "C" ascq_status ascq_mx_repack_b_kn_to_nk(uint8_t* B_nk, const uint8_t* B_kn, int K, int N, void* stream)
{
    if (!B_nk || !B_kn) return fail(ASCQ_ERR_INVALID_ARG, "null pointer");
    if (K <= 0 || N <= 0 || K % 2 || N % 2) return fail(ASCQ_ERR_INVALID_ARG, "K and N must be positive and even");
    const long long total = static_cast<long long>(N) * (K / 2);
    repack_b_kn_to_nk_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(B_nk, B_kn, K, N);
    ASCQ_CUDA_CHECK(cudaGetLastError());
    return ASCQ_OK;
}

extern "C" ascq_status ascq_mx_repack_scale_b(uint8_t* sB_nk, const uint8_t* sB_ref, int sK, int N, void* stream)
{
    if (!sB_nk || !sB_ref) return fail(ASCQ_ERR_INVALID_ARG, "null pointer");
    if (sK <= 0 || N <= 0 || sK % 2) return fail(ASCQ_ERR_INVALID_ARG, "sK must be positive and even, N positive");
    const long long total = static_cast<long long>(N) * sK;
    repack_scale_b_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(sB_nk, sB_ref, sK, N);
    ASCQ_CUDA_CHECK(cudaGetLastError());
    return ASCQ_OK;
}
