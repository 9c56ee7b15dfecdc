// Store bandwidth from one GPU into a peer's memory over NVLink for the access patterns an epilogue could use: what the
// fused all-gather of the sharded matmuls can reach at best, measured rather than assumed.  One process, two devices,
// peer access enabled; the block written is config 4's share at two ranks, [4096 rows x 2048 bf16 columns] = 16.8 MB inside
// a [4096 x 4096] matrix.  Only stores cross the link; nothing waits on anything; no load ever reads a peer.
// Built and run by tests/test_gpu_multi.py on a box with two GPUs:  nvcc -arch=sm_100a -O3 -o probe p2p_store_probe.cu
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("ERR %s line %d: %s\n", #x, __LINE__, cudaGetErrorString(e)); exit(1); } } while (0)

constexpr int ROWS = 4096, LDC = 4096 /*elements*/, COLS = 2048;  // block columns [c0, c0+COLS)
constexpr size_t PITCH = LDC * 2;

// V1: flat contiguous 16 B/thread stores over `bytes`
__global__ void k_flat(uint4* dst, size_t n16)
{
    uint4 v = make_uint4(threadIdx.x, blockIdx.x, 3, 4);
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) dst[i] = v;
}
// V2: row segments of SEG bytes (pitch PITCH): a warp writes 512 B per instruction = 512/SEG segments of consecutive rows
template <int SEG> __global__ void k_seg(char* dst, int c0Bytes)
{
    constexpr int lanesPerSeg = SEG / 16;            // lanes covering one segment
    constexpr int segsPerInstr = 32 / lanesPerSeg;   // rows per instruction (if SEG <= 512)
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    constexpr int segsPerRow = COLS * 2 / SEG;
    const long totalSegs = (long)ROWS * segsPerRow;
    uint4 v = make_uint4(lane, warp, 3, 4);
    // unit of work: segsPerInstr consecutive rows x one segment column
    const long units = totalSegs / segsPerInstr;
    for (long u = warp; u < units; u += nwarps) {
        const long rowGroup = u / segsPerRow, sc = u % segsPerRow;   // neighbouring warps take neighbouring column segments
        const int row = (int)rowGroup * segsPerInstr + lane / lanesPerSeg;
        *reinterpret_cast<uint4*>(dst + (size_t)row * PITCH + c0Bytes + sc * SEG + (lane % lanesPerSeg) * 16) = v;
    }
}
// V2b: tile-like order: CTA owns a 128 x 256-col tile region; its 8 warps write 16 rows x 128 B pieces (as the epilogue does)
__global__ void k_tile(char* dst, int c0Bytes, int peerLoops)
{
    const int tilesN = COLS / 256, tilesM = ROWS / 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint4 v = make_uint4(lane, warp, 3, 4);
    for (int t = blockIdx.x; t < tilesM * tilesN; t += gridDim.x) {
        const int m0 = (t % tilesM) * 128, n0 = (t / tilesM) * 256;
        const int q = warp & 3, sub = warp >> 2;
        for (int c2 = sub; c2 < 4; c2 += 2)
            for (int h = 0; h < 2; ++h)
                for (int i = 0; i < 4; ++i) {
                    const int rl = i * 4 + (lane >> 3), piece = lane & 7;
                    const int row = m0 + q * 32 + h * 16 + rl;
                    for (int pl = 0; pl < peerLoops; ++pl)
                        *reinterpret_cast<uint4*>(dst + (size_t)row * PITCH + c0Bytes + (n0 + c2 * 64) * 2 + piece * 16) = v;
                }
    }
}
// V3: bulk store (non-tensor) of CH contiguous bytes from smem, flat destination
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
template <int CH> __global__ void k_bulk(char* dst, size_t bytes)
{
    extern __shared__ __align__(128) char sm[];
    for (int i = threadIdx.x; i < CH / 4; i += blockDim.x) reinterpret_cast<int*>(sm)[i] = i;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) {
        const size_t chunks = bytes / CH;
        for (size_t c = blockIdx.x; c < chunks; c += gridDim.x) {
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + c * CH), "r"(smem_u32(sm)), "r"(CH) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
}
// V4: TMA tensor store of a [boxRows x boxCols] box per issue; thread 0 of each of W warps issues
__global__ void k_tma(const __grid_constant__ CUtensorMap tm, int boxCols, int boxRows, int c0Elems, int warpsIssuing)
{
    extern __shared__ __align__(1024) char sm[];
    char* base = (char*)(((uintptr_t)sm + 1023) & ~(uintptr_t)1023);
    const int boxBytes = boxCols * 2 * boxRows;
    for (int i = threadIdx.x; i < boxBytes * warpsIssuing / 4; i += blockDim.x) reinterpret_cast<int*>(base)[i] = i;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0 && warp < warpsIssuing) {
        const int boxesN = COLS / boxCols, boxesM = ROWS / boxRows;
        const long total = (long)boxesN * boxesM;
        const long issuer = (long)blockIdx.x * warpsIssuing + warp, nIssuers = (long)gridDim.x * warpsIssuing;
        for (long b = issuer; b < total; b += nIssuers) {
            const int bn = (int)(b % boxesN), bm = (int)(b / boxesN);
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"((unsigned long long)&tm),
                         "r"(smem_u32(base + warp * boxBytes)), "r"(c0Elems + bn * boxCols), "r"(bm * boxRows) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // as the epilogue does before reusing its staging rows
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                             const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static CUtensorMap make_map(void* base, int boxCols, int boxRows, bool swz)
{
    void* sym = nullptr; cudaDriverEntryPointQueryResult q;
    CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q));
    CUtensorMap m; cuuint64_t dims[2] = {LDC, ROWS}; cuuint64_t str[1] = {PITCH}; cuuint32_t box[2] = {(cuuint32_t)boxCols, (cuuint32_t)boxRows}; cuuint32_t es[2] = {1, 1};
    CUresult rc = ((EncodeFn)sym)(&m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, base, dims, str, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  swz ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) { printf("encode failed %d\n", (int)rc); exit(1); }
    return m;
}

struct Dev { int id; char* buf; cudaStream_t st; cudaEvent_t e0, e1; };
template <typename F> void run(const char* name, Dev* d, int ndir, double bytes, F launch)
{
    // ndir = 1: dev0 -> dev1 only; 2: both directions at once.  d[i] writes into d[1-i].buf
    for (int rep = 0; rep < 3; ++rep) {
        for (int i = 0; i < ndir; ++i) { CK(cudaSetDevice(d[i].id)); CK(cudaDeviceSynchronize()); }
        for (int i = 0; i < ndir; ++i) { CK(cudaSetDevice(d[i].id)); CK(cudaEventRecord(d[i].e0, d[i].st)); for (int k = 0; k < 5; ++k) launch(d[i], d[1 - i].buf); CK(cudaEventRecord(d[i].e1, d[i].st)); }
        for (int i = 0; i < ndir; ++i) { CK(cudaSetDevice(d[i].id)); CK(cudaDeviceSynchronize()); }
    }
    float ms[2] = {0, 0};
    for (int i = 0; i < ndir; ++i) { CK(cudaEventElapsedTime(&ms[i], d[i].e0, d[i].e1)); }
    printf("%-58s dirs=%d  %7.1f us/launch  %7.1f GB/s per direction", name, ndir, ms[0] / 5 * 1e3, bytes / (ms[0] / 5 * 1e-3) / 1e9);
    if (ndir == 2) printf("   (other dir %7.1f us)", ms[1] / 5 * 1e3);
    printf("\n");
}

int main()
{
    int n = 0; CK(cudaGetDeviceCount(&n));
    if (n < 2) { printf("need 2 GPUs\n"); return 0; }
    Dev d[2];
    for (int i = 0; i < 2; ++i) {
        d[i].id = i; CK(cudaSetDevice(i)); CK(cudaDeviceEnablePeerAccess(1 - i, 0));
        CK(cudaMalloc(&d[i].buf, (size_t)ROWS * PITCH)); CK(cudaStreamCreate(&d[i].st)); CK(cudaEventCreate(&d[i].e0)); CK(cudaEventCreate(&d[i].e1));
    }
    const double blockBytes = (double)ROWS * COLS * 2;
    for (int i = 0; i < 2; ++i) { CK(cudaSetDevice(i)); CK(cudaFuncSetAttribute(k_tma, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024)); }
    for (int nd = 1; nd <= 2; ++nd) {
        // local baseline (write own memory) for reference, only once
        if (nd == 1) {
            Dev loc[2] = {d[0], d[0]};
            run("flat 16B/thread, LOCAL memory, 1184 CTAs x 256", loc, 1, blockBytes, [&](Dev& s, char* dst) { k_flat<<<1184, 256, 0, s.st>>>((uint4*)dst, (size_t)blockBytes / 16); });
        }
        for (int ctas : {148, 296, 592, 1184})
        {
            char nm[128]; snprintf(nm, sizeof nm, "flat 16B/thread contiguous, %d CTAs x 256", ctas);
            run(nm, d, nd, blockBytes, [&](Dev& s, char* dst) { k_flat<<<ctas, 256, 0, s.st>>>((uint4*)dst, (size_t)blockBytes / 16); });
        }
        run("row segments 128 B, pitch 8 KB, 592 CTAs x 256", d, nd, blockBytes, [&](Dev& s, char* dst) { k_seg<128><<<592, 256, 0, s.st>>>(dst, 0); });
        run("row segments 256 B, pitch 8 KB, 592 CTAs x 256", d, nd, blockBytes, [&](Dev& s, char* dst) { k_seg<256><<<592, 256, 0, s.st>>>(dst, 0); });
        run("row segments 512 B, pitch 8 KB, 592 CTAs x 256", d, nd, blockBytes, [&](Dev& s, char* dst) { k_seg<512><<<592, 256, 0, s.st>>>(dst, 0); });
        run("epilogue-like tiles (16 rows x 128 B per instr), 148 x 256", d, nd, blockBytes, [&](Dev& s, char* dst) { k_tile<<<148, 256, 0, s.st>>>(dst, 0, 1); });
        run("epilogue-like tiles, 296 CTAs x 256", d, nd, blockBytes, [&](Dev& s, char* dst) { k_tile<<<296, 256, 0, s.st>>>(dst, 0, 1); });
        run("bulk store 2 KB contiguous chunks, 148 CTAs", d, nd, blockBytes, [&](Dev& s, char* dst) { k_bulk<2048><<<148, 64, 2048, s.st>>>(dst, (size_t)blockBytes); });
        run("bulk store 16 KB contiguous chunks, 148 CTAs", d, nd, blockBytes, [&](Dev& s, char* dst) { k_bulk<16384><<<148, 64, 16384, s.st>>>(dst, (size_t)blockBytes); });
        run("bulk store 16 KB contiguous chunks, 592 CTAs", d, nd, blockBytes, [&](Dev& s, char* dst) { k_bulk<16384><<<592, 64, 16384, s.st>>>(dst, (size_t)blockBytes); });
        for (int i = 0; i < 2; ++i) CK(cudaSetDevice(i));
        {
            CUtensorMap m0[2] = {make_map(d[1].buf, 64, 16, true), make_map(d[0].buf, 64, 16, true)};
            run("TMA box 64 cols x 16 rows (128 B rows, swizzled), 148 CTAs x 8 issuers", d, nd, blockBytes,
                [&](Dev& s, char* dst) { k_tma<<<148, 256, 8 * 2048 + 1024, s.st>>>(m0[s.id], 64, 16, 0, 8); });
            CUtensorMap m1[2] = {make_map(d[1].buf, 256, 16, false), make_map(d[0].buf, 256, 16, false)};
            run("TMA box 256 cols x 16 rows (512 B rows), 148 CTAs x 4 issuers", d, nd, blockBytes,
                [&](Dev& s, char* dst) { k_tma<<<148, 256, 4 * 8192 + 1024, s.st>>>(m1[s.id], 256, 16, 0, 4); });
            CUtensorMap m2[2] = {make_map(d[1].buf, 256, 64, false), make_map(d[0].buf, 256, 64, false)};
            run("TMA box 256 cols x 64 rows (512 B rows, 32 KB), 148 CTAs x 2 issuers", d, nd, blockBytes,
                [&](Dev& s, char* dst) { k_tma<<<148, 256, 2 * 32768 + 1024, s.st>>>(m2[s.id], 256, 64, 0, 2); });
            CUtensorMap m3[2] = {make_map(d[1].buf, 64, 128, true), make_map(d[0].buf, 64, 128, true)};
            run("TMA box 64 cols x 128 rows (128 B rows, 16 KB), 148 CTAs x 4 issuers", d, nd, blockBytes,
                [&](Dev& s, char* dst) { k_tma<<<148, 256, 4 * 16384 + 1024, s.st>>>(m3[s.id], 64, 128, 0, 4); });
        }
        // plain cudaMemcpy2DAsync of the block (copy engine)
        {
            char* src[2]; for (int i = 0; i < 2; ++i) { CK(cudaSetDevice(i)); CK(cudaMalloc(&src[i], (size_t)ROWS * PITCH)); }
            run("cudaMemcpy2DAsync of the block (copy engine)", d, nd, blockBytes,
                [&](Dev& s, char* dst) { CK(cudaMemcpy2DAsync(dst, PITCH, src[s.id], PITCH, COLS * 2, ROWS, cudaMemcpyDeviceToDevice, s.st)); });
            run("cudaMemcpyAsync 16.8 MB contiguous (copy engine)", d, nd, blockBytes,
                [&](Dev& s, char* dst) { CK(cudaMemcpyAsync(dst, src[s.id], (size_t)blockBytes, cudaMemcpyDeviceToDevice, s.st)); });
        }
    }
    printf("done\n");
    return 0;
}
