// One rank of the column-parallel W8A8 matmul driven from plain C++ through include/ascq.h only -- the call sequence a
// C / C++ host of the reference's sample would use in place of its HCCL AllGather (include/adv_api/hccl/hccl.h:82-100,
// 304-326).  Run as one process per GPU by tests/test_gpu_multi.py:
//
//     sharded_main RANK NRANKS DIR
//
// Set-up: cudaMalloc of the flag block and of this rank's [M, N] output matrix, CUDA IPC handles exchanged through files
// in DIR, ascq_comm_create.  Then two steps of ascq_matmul_w8a8_sharded; after each, this rank's matrix must hold the
// whole result, checked bit for bit against an integer computation on the host (inputs small enough for that).
// Every host-side wait is bounded, so a rank that died cannot hang the others.  Exit code 0 on success.
#include <cuda_runtime.h>
#include <sys/stat.h>
#include <unistd.h>

#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "ascq.h"

#define CK(x)                                                                                  \
    do {                                                                                       \
        cudaError_t e_ = (x);                                                                  \
        if (e_ != cudaSuccess) {                                                               \
            fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e_));                    \
            return 2;                                                                          \
        }                                                                                      \
    } while (0)
#define AQ(x)                                                                                  \
    do {                                                                                       \
        ascq_status s_ = (x);                                                                  \
        if (s_ != ASCQ_OK) {                                                                   \
            fprintf(stderr, "%s: %s: %s\n", #x, ascq_status_string(s_), ascq_last_error());   \
            return 3;                                                                          \
        }                                                                                      \
    } while (0)

static bool wait_for(const std::string& path, double limitSeconds = 60.0)
{
    const auto t0 = std::chrono::steady_clock::now();
    struct stat st;
    while (stat(path.c_str(), &st) != 0) {
        if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > limitSeconds) return false;
        std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
    return true;
}
static bool publish(const std::string& dir, const std::string& name, const void* data, size_t bytes)
{
    const std::string tmp = dir + "/" + name + ".tmp", fin = dir + "/" + name;
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) return false;
    const bool ok = fwrite(data, 1, bytes, f) == bytes;
    fclose(f);
    return ok && rename(tmp.c_str(), fin.c_str()) == 0;
}
static bool host_barrier(const std::string& dir, const std::string& tag, int rank, int n)
{
    if (!publish(dir, tag + "." + std::to_string(rank), "1", 1)) return false;
    for (int r = 0; r < n; ++r)
        if (!wait_for(dir + "/" + tag + "." + std::to_string(r))) return false;
    return true;
}
// round-to-nearest-even float -> bfloat16 bits (finite inputs)
static uint16_t bf16_bits(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}

int main(int argc, char** argv)
{
    if (argc != 4) return 64;
    const int rank = atoi(argv[1]), n = atoi(argv[2]);
    const std::string dir = argv[3];
    CK(cudaSetDevice(rank));
    const int M = 384, N = 1024, K = 256;   // |acc| <= 256 * 127 * 127 < 2^24: float(acc) is exact on the host too
    // the same inputs on every rank (a fixed linear congruential sequence)
    std::vector<int8_t> A(size_t(M) * K), B(size_t(N) * K);
    std::vector<float> sA(M), sB(N);
    uint32_t seed = 12345u;
    auto next = [&seed]() { seed = seed * 1664525u + 1013904223u; return seed >> 8; };
    for (auto& v : A) v = static_cast<int8_t>(int(next() % 255u) - 127);
    for (auto& v : B) v = static_cast<int8_t>(int(next() % 255u) - 127);
    for (auto& v : sA) v = 0.005f + 0.015f * float(next() % 1000u) / 1000.0f;
    for (auto& v : sB) v = 0.001f + 0.009f * float(next() % 1000u) / 1000.0f;

    // shared buffers: flag block (zeroed) and output matrix
    void *flags = nullptr, *out = nullptr;
    const size_t flagBytes = ascq_comm_flag_bytes(), outBytes = size_t(M) * N * 2;
    CK(cudaMalloc(&flags, flagBytes));
    CK(cudaMalloc(&out, outBytes));
    CK(cudaMemset(flags, 0, flagBytes));
    CK(cudaMemset(out, 0xFF, outBytes));
    CK(cudaDeviceSynchronize());
    std::vector<unsigned char> h(ascq_comm_ipc_handle_bytes());
    AQ(ascq_comm_ipc_export(h.data(), flags));
    if (!publish(dir, "flags." + std::to_string(rank), h.data(), h.size())) return 4;
    AQ(ascq_comm_ipc_export(h.data(), out));
    if (!publish(dir, "out." + std::to_string(rank), h.data(), h.size())) return 4;
    std::vector<void*> flagPtrs(n), outPtrs(n);
    for (int r = 0; r < n; ++r) {
        if (r == rank) {
            flagPtrs[r] = flags;
            outPtrs[r] = out;
            continue;
        }
        for (int which = 0; which < 2; ++which) {
            const std::string path = dir + (which ? "/out." : "/flags.") + std::to_string(r);
            if (!wait_for(path)) return 5;
            FILE* f = fopen(path.c_str(), "rb");
            if (!f || fread(h.data(), 1, h.size(), f) != h.size()) return 5;
            fclose(f);
            AQ(ascq_comm_ipc_open(which ? &outPtrs[r] : &flagPtrs[r], h.data()));
        }
    }
    if (!host_barrier(dir, "mapped", rank, n)) return 6;   // every block zeroed and mapped before anyone signals
    ascq_comm* comm = nullptr;
    AQ(ascq_comm_create(&comm, rank, n, flagPtrs.data()));

    int c0 = 0, nl = 0;
    AQ(ascq_shard_columns(N, n, rank, &c0, &nl));
    int8_t *dA = nullptr, *dB = nullptr;
    float *dsA = nullptr, *dsB = nullptr;
    CK(cudaMalloc(&dA, A.size()));
    CK(cudaMalloc(&dB, size_t(nl) * K));
    CK(cudaMalloc(&dsA, M * 4));
    CK(cudaMalloc(&dsB, nl * 4));
    CK(cudaMemcpy(dA, A.data(), A.size(), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dB, B.data() + size_t(c0) * K, size_t(nl) * K, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dsA, sA.data(), M * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dsB, sB.data() + c0, nl * 4, cudaMemcpyHostToDevice));

    std::vector<uint16_t> got(size_t(M) * N);
    for (int step = 0; step < 2; ++step) {
        CK(cudaDeviceSynchronize());
        if (!host_barrier(dir, "step" + std::to_string(step), rank, n)) return 6;
        AQ(ascq_matmul_w8a8_sharded(comm, outPtrs.data(), nullptr, dA, dB, dsA, dsB, nullptr, M, N, K, nullptr));
        AQ(ascq_matmul_status(nullptr));   // synchronises; ASCQ_ERR_TIMEOUT if the wait for the other ranks ran out
        CK(cudaMemcpy(got.data(), out, outBytes, cudaMemcpyDeviceToHost));
        size_t bad = 0;
        for (int m = 0; m < M; ++m)
            for (int c = 0; c < N; ++c) {
                int32_t acc = 0;
                for (int k = 0; k < K; ++k) acc += int32_t(A[size_t(m) * K + k]) * int32_t(B[size_t(c) * K + k]);
                const volatile float f1 = float(acc) * sB[c];   // two separately rounded products, as the epilogue does
                const volatile float f2 = f1 * sA[m];
                if (got[size_t(m) * N + c] != bf16_bits(f2)) ++bad;
            }
        if (bad) {
            fprintf(stderr, "rank %d step %d: %zu of %zu elements differ\n", rank, step, bad, got.size());
            return 1;
        }
        if (!host_barrier(dir, "read" + std::to_string(step), rank, n)) return 6;   // nobody overwrites a matrix still being read
    }
    AQ(ascq_comm_destroy(comm));
    printf("rank %d: ok\n", rank);
    return 0;
}
