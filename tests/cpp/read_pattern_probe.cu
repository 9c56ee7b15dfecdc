// Read-rate yardstick of the few-row matmuls (gemm_w8a8_small.cu, gemm_w8a16_small.cu): an [N, K] int8 matrix is read once,
// nothing else, with the work split as in those kernels (a CTA owns 16 rows over the whole of K) and three request shapes:
// the MMA-fragment shape the kernels use (every warp request is eight 128-byte pieces, K bytes apart), the same with
// 16-byte loads, and whole 1 KB runs of one row per request.  What it shows on B200: the request shape does not matter
// (all within 10 %), and reading 8192 x 8192 bytes this way takes 12.4 to 14.4 us (4.6 to 5.4 TB/s), 4096 x 4096 bytes
// 6.2 us -- launch, ramp-up and tail are a third to a half of a launch that moves so little.  Built and run by
// tests/test_gpu_matmul_w8a8.py; prints one line per variant.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include <vector>
#include <algorithm>
struct W8 { uint32_t w[8]; };
__device__ __forceinline__ W8 ld32(const void* p) {
    W8 v;
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7]) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t fold(const W8& v) { return v.w[0] ^ v.w[1] ^ v.w[2] ^ v.w[3] ^ v.w[4] ^ v.w[5] ^ v.w[6] ^ v.w[7]; }
// P: 0 = fragment pattern (8 rows x 128 B per request, two requests per step: rows g and g+8), warps interleave k chunks
//    1 = same 16 rows per CTA, but each request reads 1 KB of one row (lane l -> 32 l); warp w takes rows w, w+WARPS, ...
//    2 = fragment pattern with 16-byte loads: 8 rows x 64 B per request
template <int P, int WARPS, int DEPTH>
__global__ void __launch_bounds__(32 * WARPS) probe(const int8_t* B, int N, int K, uint32_t* out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    uint32_t acc = 0;
    for (int n0 = blockIdx.x * 16; n0 < N; n0 += gridDim.x * 16) {
        if (P == 0) {
            const int8_t* lo = B + size_t(n0 + g) * K + 32 * c; const int8_t* hi = lo + size_t(8) * K;
            const int step = WARPS * 128;
            for (int k = warp * 128; k < K; k += DEPTH * step) {
                W8 a[DEPTH], b[DEPTH];
#pragma unroll
                for (int d = 0; d < DEPTH; ++d) if (k + d * step < K) { a[d] = ld32(lo + k + d * step); b[d] = ld32(hi + k + d * step); }
#pragma unroll
                for (int d = 0; d < DEPTH; ++d) if (k + d * step < K) acc ^= fold(a[d]) ^ fold(b[d]);
            }
        } else if (P == 1) {
            for (int r = warp; r < 16; r += WARPS) {
                const int8_t* row = B + size_t(n0 + r) * K + 32 * lane;
                for (int k = 0; k < K; k += DEPTH * 1024) {
                    W8 a[DEPTH];
#pragma unroll
                    for (int d = 0; d < DEPTH; ++d) if (k + d * 1024 < K) a[d] = ld32(row + k + d * 1024);
#pragma unroll
                    for (int d = 0; d < DEPTH; ++d) if (k + d * 1024 < K) acc ^= fold(a[d]);
                }
            }
        } else {
            const int8_t* lo = B + size_t(n0 + g) * K + 16 * c; const int8_t* hi = lo + size_t(8) * K;
            const int step = WARPS * 64;
            for (int k = warp * 64; k < K; k += DEPTH * step) {
                uint4 a[DEPTH], b[DEPTH];
#pragma unroll
                for (int d = 0; d < DEPTH; ++d) if (k + d * step < K) { a[d] = __ldg((const uint4*)(lo + k + d * step)); b[d] = __ldg((const uint4*)(hi + k + d * step)); }
#pragma unroll
                for (int d = 0; d < DEPTH; ++d) if (k + d * step < K) acc ^= a[d].x ^ a[d].y ^ a[d].z ^ a[d].w ^ b[d].x ^ b[d].y ^ b[d].z ^ b[d].w;
            }
        }
    }
    if (acc == 0x12345678u) out[0] = acc;
}
template <int P, int WARPS, int DEPTH> void run(const char* name, std::vector<int8_t*>& bufs, int N, int K, uint32_t* out, int ctasPerSm) {
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    const int grid = std::min(N / 16, ctasPerSm * 148);
    for (auto b : bufs) probe<P, WARPS, DEPTH><<<grid, 32 * WARPS>>>(b, N, K, out);
    cudaEventRecord(e0);
    const int reps = 5;
    for (int r = 0; r < reps; ++r) for (auto b : bufs) probe<P, WARPS, DEPTH><<<grid, 32 * WARPS>>>(b, N, K, out);
    cudaEventRecord(e1); cudaEventSynchronize(e1);
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    const double us = ms * 1e3 / (reps * bufs.size());
    printf("%-58s N=%5d K=%5d grid=%4d  %7.1f us  %6.0f GB/s  (%s)\n", name, N, K, grid, us, double(N) * K / us / 1e3, cudaGetErrorString(cudaGetLastError()));
}
int main() {
    uint32_t* out; cudaMalloc(&out, 4);
    for (int cfg = 0; cfg < 2; ++cfg) {
        const int N = cfg == 0 ? 8192 : 4096, K = N;
        std::vector<int8_t*> bufs(cfg == 0 ? 6 : 24);
        for (auto& b : bufs) { cudaMalloc(&b, size_t(N) * K); cudaMemset(b, 1, size_t(N) * K); }
        run<0, 4, 3>("fragment pattern 8 rows x 128 B, 4 warps, depth 3, 4 CTA/SM", bufs, N, K, out, 4);
        run<0, 4, 4>("fragment pattern 8 rows x 128 B, 4 warps, depth 4, 8 CTA/SM", bufs, N, K, out, 8);
        run<0, 8, 4>("fragment pattern 8 rows x 128 B, 8 warps, depth 4, 4 CTA/SM", bufs, N, K, out, 4);
        run<0, 8, 2>("fragment pattern 8 rows x 128 B, 8 warps, depth 2, 8 CTA/SM", bufs, N, K, out, 8);
        run<1, 4, 4>("row pattern 1 row x 1 KB, 4 warps, depth 4, 4 CTA/SM", bufs, N, K, out, 4);
        run<1, 4, 4>("row pattern 1 row x 1 KB, 4 warps, depth 4, 8 CTA/SM", bufs, N, K, out, 8);
        run<1, 8, 4>("row pattern 1 row x 1 KB, 8 warps, depth 4, 4 CTA/SM", bufs, N, K, out, 4);
        run<2, 4, 4>("fragment pattern 8 rows x 64 B (16 B loads), 4 warps, depth 4, 8 CTA/SM", bufs, N, K, out, 8);
        run<2, 8, 4>("fragment pattern 8 rows x 64 B (16 B loads), 8 warps, depth 4, 4 CTA/SM", bufs, N, K, out, 4);
        for (auto b : bufs) cudaFree(b);
    }
    printf("done\n");
    return 0;
}
