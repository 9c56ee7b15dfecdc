// Status strings, the thread-local error slot, and the host-side tmp-size queries of the C ABI.
#include <algorithm>
#include <cstring>

#include "ascq_internal.h"

namespace ascq {
namespace {
thread_local char g_err[512] = "";
}

ascq_status fail(ascq_status s, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return s;
}
void clear_error() { g_err[0] = '\0'; }
}  // namespace ascq

using ascq::fail;

extern "C" {

const char* ascq_status_string(ascq_status s)
{
    switch (s) {
        case ASCQ_OK: return "ASCQ_OK";
        case ASCQ_ERR_INVALID_ARG: return "ASCQ_ERR_INVALID_ARG";
        case ASCQ_ERR_UNSUPPORTED: return "ASCQ_ERR_UNSUPPORTED";
        case ASCQ_ERR_ALIGNMENT: return "ASCQ_ERR_ALIGNMENT";
        case ASCQ_ERR_CUDA: return "ASCQ_ERR_CUDA";
        case ASCQ_ERR_NCCL: return "ASCQ_ERR_NCCL";
        case ASCQ_ERR_TIMEOUT: return "ASCQ_ERR_TIMEOUT";
    }
    return "ASCQ_ERR_UNKNOWN";
}
const char* ascq_last_error(void) { return ascq::g_err; }
int ascq_version(void) { return ASCQ_VERSION_MAJOR * 100 + ASCQ_VERSION_MINOR; }

// ---- tmp-size queries -------------------------------------------------------------------------
// The CUDA kernels need no temporary buffer; the formulas are kept so that host code written
// against the reference's tiling API keeps computing the same numbers.

static int64_t shape_size(const int64_t* d, int rank)
{
    int64_t s = 1;
    for (int i = 0; i < rank; ++i) s *= d[i];
    return s;
}

// impl/adv_api/tiling/quantization/ascend_quant_tiling_impl.cpp:31-69
ascq_status ascq_get_ascend_quant_max_min_tmp_size(const int64_t* srcDims, int rank, uint32_t typeSize,
                                                   uint32_t* maxValue, uint32_t* minValue)
{
    if (!srcDims || rank <= 0 || !maxValue || !minValue) return fail(ASCQ_ERR_INVALID_ARG, "null argument");
    const int64_t size = shape_size(srcDims, rank);
    if (size <= 0) return fail(ASCQ_ERR_INVALID_ARG, "Input Shape size must be greater than 0.");
    if (size * typeSize % 32 != 0) return fail(ASCQ_ERR_INVALID_ARG, "Input Shape size must be 32B aligned!.");
    if (typeSize != 2 && typeSize != 4) return fail(ASCQ_ERR_INVALID_ARG, "Type size %u is unsupported!", typeSize);
    constexpr uint32_t kOneRepeatBytes = 256, kTwo = 2, kBlk = 32;
    const uint32_t raw = std::max(static_cast<uint32_t>(size) * kTwo, kTwo * kOneRepeatBytes);
    *maxValue = (raw + kBlk - 1) / kBlk * kBlk;
    *minValue = kTwo * kOneRepeatBytes;
    return ASCQ_OK;
}
void ascq_get_ascend_quant_tmp_buffer_factor_size(uint32_t* maxLiveNodeCount, uint32_t* extraBuf)
{
    if (extraBuf) *extraBuf = 0u;
    if (maxLiveNodeCount) *maxLiveNodeCount = 2u;
}

// impl/adv_api/tiling/quantization/ascend_dequant_tiling_impl.cpp:31-106
ascq_status ascq_get_ascend_dequant_max_min_tmp_size(const int64_t* srcDims, int rank, uint32_t typeSize,
                                                     uint32_t* maxValue, uint32_t* minValue)
{
    if (!srcDims || !maxValue || !minValue) return fail(ASCQ_ERR_INVALID_ARG, "null argument");
    if (rank <= 0 || rank > 2) return fail(ASCQ_ERR_INVALID_ARG, "SrcShape dim %d is unsupported, must be 1 or 2!", rank);
    if (shape_size(srcDims, rank) <= 0) return fail(ASCQ_ERR_INVALID_ARG, "Input Shape size must be greater than 0.");
    if (typeSize != 4) return fail(ASCQ_ERR_INVALID_ARG, "Type size %u is unsupported!", typeSize);
    constexpr uint32_t kFloatPerBlock = 8, kFloatPerRepeat = 64;
    const uint32_t outer = rank == 2 ? static_cast<uint32_t>(srcDims[0]) : 1u;
    const uint32_t inner = static_cast<uint32_t>(srcDims[rank - 1]);
    const uint32_t deqScaleSize = inner + kFloatPerBlock;
    *maxValue = (kFloatPerRepeat + outer * inner + deqScaleSize) * sizeof(float);
    *minValue = (kFloatPerRepeat + inner + deqScaleSize) * sizeof(float);
    return ASCQ_OK;
}
void ascq_get_ascend_dequant_tmp_buffer_factor_size(const int64_t* srcDims, int rank, uint32_t* maxLiveNodeCount,
                                                    uint32_t* extraBuf)
{
    uint32_t extra = 8u + 64u, live = 0u;
    if (rank == 2) {
        extra += static_cast<uint32_t>(srcDims[1]);
        live = 1u;
    } else if (rank == 1) {
        live = 2u;
    } else {
        extra = 0u;
    }
    if (extraBuf) *extraBuf = extra;
    if (maxLiveNodeCount) *maxLiveNodeCount = live;
}

// impl/adv_api/tiling/quantization/ascend_antiquant_tiling_impl.cpp:71-181
namespace {
struct AntiQuantSizes { uint32_t maxv, minv, live, extra; };
AntiQuantSizes antiquant_sizes(const int64_t* srcDims, int srcRank, const int64_t* scaleDims, int scaleRank,
                               bool isTranspose, ascq_dtype inputT, ascq_dtype outputT)
{
    AntiQuantSizes r{0, 0, 0, 0};
    const uint32_t scaleSize = static_cast<uint32_t>(shape_size(scaleDims, scaleRank));
    const uint32_t srcSize = static_cast<uint32_t>(shape_size(srcDims, srcRank));
    const bool isPerChannel = scaleSize != 1;
    if (inputT == ASCQ_DT_FP4X2_E2M1 || inputT == ASCQ_DT_FP4X2_E1M2) {
        if (isTranspose) r.maxv = r.minv = r.extra = (scaleSize + 31) / 32 * 32 * 2;
        return r;
    }
    if (outputT == ASCQ_DT_F16) return r;
    if (!isPerChannel) {
        r.maxv = srcSize * sizeof(float);
        r.minv = 1024;
        r.live = 1;
    } else if (isTranspose) {
        r.maxv = r.minv = r.extra = 80u * scaleSize * sizeof(float);  // (8 + 8 + 64) * N fp32
    } else {
        const uint32_t k = static_cast<uint32_t>(srcDims[0]);
        r.maxv = r.minv = r.extra = scaleSize * 2u * sizeof(float) + 64u * k * sizeof(float);
    }
    return r;
}
}  // namespace

ascq_status ascq_get_ascend_antiquant_max_min_tmp_size(const int64_t* srcDims, int srcRank, const int64_t* scaleDims,
                                                       int scaleRank, int isTranspose, ascq_dtype inputT,
                                                       ascq_dtype outputT, uint32_t* maxValue, uint32_t* minValue)
{
    if (!srcDims || !scaleDims || !maxValue || !minValue || srcRank < 2 || scaleRank < 1)
        return fail(ASCQ_ERR_INVALID_ARG, "null argument or rank");
    if (shape_size(srcDims, srcRank) <= 0) return fail(ASCQ_ERR_INVALID_ARG, "Input Shape size must be greater than 0.");
    const AntiQuantSizes r = antiquant_sizes(srcDims, srcRank, scaleDims, scaleRank, isTranspose != 0, inputT, outputT);
    *maxValue = r.maxv;
    *minValue = r.minv;
    return ASCQ_OK;
}
void ascq_get_ascend_antiquant_tmp_buffer_factor_size(const int64_t* srcDims, int srcRank, const int64_t* scaleDims,
                                                      int scaleRank, int isTranspose, ascq_dtype inputT,
                                                      ascq_dtype outputT, uint32_t* maxLiveNodeCount,
                                                      uint32_t* extraBuf)
{
    const AntiQuantSizes r = antiquant_sizes(srcDims, srcRank, scaleDims, scaleRank, isTranspose != 0, inputT, outputT);
    if (maxLiveNodeCount) *maxLiveNodeCount = r.live;
    if (extraBuf) *extraBuf = r.extra;
}

}  // extern "C"
