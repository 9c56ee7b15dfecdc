// Shared host-side helpers of the C ABI: error reporting, CUDA call checking, dtype sizes.
#ifndef ASCQ_INTERNAL_H_
#define ASCQ_INTERNAL_H_

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/ascq.h"
#include "comm.cuh"

struct CUstream_st;

namespace ascq {

// Records a printf-style message in the thread-local slot behind ascq_last_error() and returns `s`.
ascq_status fail(ascq_status s, const char* fmt, ...);
void clear_error();

inline int dtype_size(ascq_dtype t)
{
    switch (t) {
        case ASCQ_DT_F16: case ASCQ_DT_BF16: return 2;
        case ASCQ_DT_F32: case ASCQ_DT_I32: return 4;
        case ASCQ_DT_I8: case ASCQ_DT_E8M0: case ASCQ_DT_FP4X2_E2M1: case ASCQ_DT_FP4X2_E1M2:
        case ASCQ_DT_FP8_E4M3: case ASCQ_DT_FP8_E5M2: case ASCQ_DT_HIF8: case ASCQ_DT_I4X2: return 1;
        case ASCQ_DT_U64: return 8;
    }
    return 0;
}
// Defined in gemm_mxfp4.cu: reads and clears that kernel's device status word (synchronises the stream).
ascq_status mxfp4_read_status(::CUstream_st* stream);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// gemm_w8a16_small.cu: the weight-only-quantised matmul for at most kW8A16SmallMaxM activation rows
constexpr int kW8A16SmallMaxM = 32;
bool w8a16_small_applies(int M, int N, int K, const void* A, const void* B, const void* workspace, size_t workspaceBytes);
ascq_status w8a16_small(void* C, ascq_dtype cT, const void* A, ascq_dtype aT, const int8_t* B_nk, bool int4, const void* offset,
                        const void* scale, float offsetScalar, float scaleScalar, bool hasOffset, int M, int N, int K, int ldc,
                        void* workspace, size_t workspaceBytes, ::CUstream_st* st);

// gemm_w8a8_small.cu: the W8A8 matmul with dequant epilogue for at most kW8A8SmallMaxM activation rows
constexpr int kW8A8SmallMaxM = 32;
bool w8a8_small_applies(int M, int N, int K, const void* A, const void* B);
ascq_status w8a8_small(void* C, const int8_t* A, const int8_t* B_nk, const float* sA_m, const float* sB_n, const void* bias_bf16,
                       int M, int N, int K, int ldc, int colOffset, ::CUstream_st* st);

// Sets the wait limit (SM cycles) of the bounded waits in each matmul translation unit on the current device.
ascq_status w8a8_set_wait_cycles(long long cycles);
ascq_status mxfp4_set_wait_cycles(long long cycles);

}  // namespace ascq

// The communicator behind ascq_comm_create: this rank's place among the ranks of the box and every rank's flag block
// as mapped into this process.
struct ascq_comm {
    int rank, nranks;
    ascq::CommFlags* flags[ascq::kCommMaxRanks];
};

namespace ascq {
CommArgs comm_args(const ascq_comm* comm);              // kernel argument form (nranks == 0 for NULL)
ascq_status comm_read_status(::CUstream_st* stream);    // comm.cu: status word of the stand-alone exchange kernel
}  // namespace ascq

#define ASCQ_CUDA_CHECK(expr)                                                                      \
    do {                                                                                           \
        cudaError_t err__ = (expr);                                                                \
        if (err__ != cudaSuccess)                                                                  \
            return ::ascq::fail(ASCQ_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__)); \
    } while (0)

#endif  // ASCQ_INTERNAL_H_
