// ascq_dequant: AscendDequant on global-memory tensors (fp32 arithmetic throughout).
#include "elementwise.cuh"

namespace ascq {
namespace {

template <typename Src, typename Dst, typename Sc>
ascq_status run_fast(const EwArgs& a, int smode, bool hasTok, cudaStream_t st)
{
    return launch_ew_rows<kOpDequant, Src, Dst, Sc, float>(a, smode, false, hasTok, st);
}

template <typename Src, typename Sc>
ascq_status by_dst(const EwArgs& a, ascq_dtype dstT, int smode, bool hasTok, cudaStream_t st)
{
    if (dstT == ASCQ_DT_F16) return run_fast<Src, __half, Sc>(a, smode, hasTok, st);
    if (dstT == ASCQ_DT_BF16) return run_fast<Src, __nv_bfloat16, Sc>(a, smode, hasTok, st);
    return run_fast<Src, float, Sc>(a, smode, hasTok, st);
}

ascq_status dispatch_fast(const EwArgs& a, ascq_dtype srcT, ascq_dtype dstT, ascq_dtype scT, int smode, bool hasTok,
                          cudaStream_t st, bool* handled)
{
    *handled = true;
    if (smode == kSScalar) scT = ASCQ_DT_F32;
    if (srcT == ASCQ_DT_I32) {
        if (scT == ASCQ_DT_F32) return by_dst<int32_t, float>(a, dstT, smode, hasTok, st);
        if (scT == ASCQ_DT_BF16) return by_dst<int32_t, __nv_bfloat16>(a, dstT, smode, hasTok, st);
        if (scT == ASCQ_DT_U64) return by_dst<int32_t, uint64_t>(a, dstT, smode, hasTok, st);
        if (scT == ASCQ_DT_F16) return by_dst<int32_t, __half>(a, dstT, smode, hasTok, st);
    } else {
        if (scT == ASCQ_DT_F32) return by_dst<float, float>(a, dstT, smode, hasTok, st);
        if (scT == ASCQ_DT_BF16) return by_dst<float, __nv_bfloat16>(a, dstT, smode, hasTok, st);
        if (scT == ASCQ_DT_F16) return by_dst<float, __half>(a, dstT, smode, hasTok, st);
    }
    *handled = false;
    return ASCQ_OK;
}
}  // namespace
}  // namespace ascq

using namespace ascq;

extern "C" ascq_status ascq_dequant(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT, const void* scale,
                                    const float* tokScale, ascq_dtype scaleT, float scaleScalar, ascq_policy policy,
                                    const ascq_dequant_param* p, void* stream)
{
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!dst || !src || !p) return fail(ASCQ_ERR_INVALID_ARG, "dst, src and param must not be NULL");
    if (policy == ASCQ_PER_CHANNEL_PER_GROUP || policy == ASCQ_PER_TOKEN_PER_GROUP)
        return fail(ASCQ_ERR_UNSUPPORTED, "unsupported policy for AscendDequant in current device!");
    if (policy < ASCQ_PER_TENSOR || policy > ASCQ_PER_GROUP) return fail(ASCQ_ERR_INVALID_ARG, "unknown policy %d", (int)policy);
    if (dstT != ASCQ_DT_F16 && dstT != ASCQ_DT_BF16 && dstT != ASCQ_DT_F32)
        return fail(ASCQ_ERR_UNSUPPORTED, "dst dtype must be half, bfloat16_t or float");
    if (srcT != ASCQ_DT_I32 && srcT != ASCQ_DT_F32) return fail(ASCQ_ERR_UNSUPPORTED, "src dtype must be int32_t or float");
    if (dst == src) return fail(ASCQ_ERR_INVALID_ARG, "src and dst must not overlap");
    if (p->n == 0) return fail(ASCQ_ERR_INVALID_ARG, "n must be greater than 0");

    EwArgs a{};
    a.src = src;
    a.dst = dst;
    a.tok = tokScale;
    a.roundMode = kRoundRint;
    int smode = kSScalar;

    if (policy == ASCQ_PER_TENSOR || policy == ASCQ_PER_CHANNEL) {
        // impl/adv_api/detail/quantization/dequant/ascend_dequant_common_impl.h:68-106 (IsDequantParamsValid)
        if (srcT != ASCQ_DT_I32) return fail(ASCQ_ERR_UNSUPPORTED, "AscendDequant with DequantParams takes int32_t input");
        if ((static_cast<size_t>(p->n) * sizeof(int32_t)) % 32 != 0)
            return fail(ASCQ_ERR_INVALID_ARG, "params.n %u * sizeof(int32_t) must be divisible by 32", p->n);
        if (p->calCount == 0 || p->calCount > p->n)
            return fail(ASCQ_ERR_INVALID_ARG, "params.calCount is %u, which should be in range (0, params.n %u]", p->calCount, p->n);
        const uint32_t perBlk = 32u / dtype_size(dstT);
        a.rows = p->m;
        a.cols = p->calCount;
        a.srcStride = p->n;
        a.dstStride = (p->n + perBlk - 1) / perBlk * perBlk;
        if (policy == ASCQ_PER_TENSOR) {
            if (scale) return fail(ASCQ_ERR_INVALID_ARG, "per-tensor AscendDequant takes a scalar deqScale; the tensor must be NULL");
            a.scale.scalar = scaleScalar;
        } else {
            if (!scale) return fail(ASCQ_ERR_INVALID_ARG, "deqScale tensor must not be NULL");
            // ascend_dequant_common_impl.h:125-155 (IsTemplateValid)
            const bool ok = (scaleT == ASCQ_DT_U64 && dstT == ASCQ_DT_F16) || (scaleT == ASCQ_DT_F32 && dstT == ASCQ_DT_F32) ||
                            (scaleT == ASCQ_DT_BF16 && dstT == ASCQ_DT_F32) || (scaleT == ASCQ_DT_BF16 && dstT == ASCQ_DT_BF16) ||
                            (scaleT == ASCQ_DT_F32 && dstT == ASCQ_DT_BF16);
            if (!ok)
                return fail(ASCQ_ERR_UNSUPPORTED,
                            "current combination of deqScale dtype and dstTensor dtype is not supported, please check the document");
            smode = kSColVec;
            a.scale.p = scale; a.scale.rdiv = 0; a.scale.cdiv = 1; a.scale.stride = 0;
        }
    } else {
        if (tokScale) return fail(ASCQ_ERR_INVALID_ARG, "tokScale is only combined with PER_CHANNEL");
        if (!scale) return fail(ASCQ_ERR_INVALID_ARG, "scale tensor must not be NULL");
        if (scaleT != ASCQ_DT_F16 && scaleT != ASCQ_DT_BF16 && scaleT != ASCQ_DT_F32)
            return fail(ASCQ_ERR_UNSUPPORTED, "scale dtype must be half, bfloat16_t or float");
        // (scale, dst) pairs of tests/api/adv_api/quantization/dequant/test_ascend_dequant_per_token.cpp:149-159
        const bool ok = (scaleT == ASCQ_DT_F32) ? true : (dstT == scaleT);
        if (!ok) return fail(ASCQ_ERR_UNSUPPORTED, "unsupported (scale, dst) dtype pair for AscendDequant PER_TOKEN/PER_GROUP");
        if (p->calCount % p->n != 0)
            return fail(ASCQ_ERR_INVALID_ARG, "calCount is %u, which should be an integer multiple of n %u", p->calCount, p->n);
        a.rows = p->calCount / p->n;
        a.cols = p->n;
        a.srcStride = a.dstStride = p->n;
        a.scale.p = scale;
        if (policy == ASCQ_PER_TOKEN) {
            a.scale.rdiv = 1; a.scale.cdiv = 0; a.scale.stride = 1;
            smode = kSRowBcast;
        } else {
            if (p->groupSize == 0 || p->groupSize % 32 != 0)
                return fail(ASCQ_ERR_INVALID_ARG, "groupSize is %u, which must be a positive multiple of 32", p->groupSize);
            if (p->kDim == 1) {
                a.scale.rdiv = 1; a.scale.cdiv = p->groupSize; a.scale.stride = (p->n + p->groupSize - 1) / p->groupSize;
                smode = kSRowBcast;
            } else if (p->kDim == 0) {
                a.scale.rdiv = p->groupSize; a.scale.cdiv = 1; a.scale.stride = p->n;
                smode = kSRowVec;
            } else {
                return fail(ASCQ_ERR_INVALID_ARG, "kDim is %d, which must be 0 or 1", p->kDim);
            }
        }
    }
    if (a.rows == 0 || a.cols == 0) return ASCQ_OK;

    const int vec = 16 / (dtype_size(dstT) < 4 ? dtype_size(dstT) : 4);
    {
        EwArgs b = a;
        b.scalarPath = ew_fast_ok(a, vec, smode, dtype_size(scaleT)) ? 0 : 1;  // ragged / unaligned: one element per thread
        bool handled = false;
        ascq_status rc = dispatch_fast(b, srcT, dstT, scaleT, smode, tokScale != nullptr, st, &handled);
        if (rc != ASCQ_OK || handled) return rc;
    }
    GenericArgs g{};
    g.op = kOpDequant; g.srcT = srcT; g.dstT = dstT; g.scT = scaleT; g.ct = ASCQ_DT_F32;
    g.src = src; g.dst = dst; g.rows = a.rows; g.cols = a.cols; g.srcStride = a.srcStride; g.dstStride = a.dstStride;
    g.scale = a.scale; g.scaleIsScalar = (smode == kSScalar); g.hasOff = 0; g.tok = tokScale; g.roundMode = kRoundRint;
    return launch_ew_generic(g, st);
}

// Dequantize (impl/adv_api/detail/quantization/dequantize/dequantize_impl.h:100-215) forwards to the AscendDequant
// implementations with whole rows (calCount = n for PER_TENSOR / PER_CHANNEL, m * n otherwise) and has no offset.
extern "C" ascq_status ascq_dequantize(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT, const void* scale,
                                       ascq_dtype scaleT, float scaleScalar, ascq_policy policy,
                                       const ascq_quantize_param* qp, void* stream)
{
    if (!qp) return fail(ASCQ_ERR_INVALID_ARG, "dst, src and param must not be NULL");
    if (policy < ASCQ_PER_TENSOR || policy > ASCQ_PER_GROUP)
        return fail(ASCQ_ERR_UNSUPPORTED, "Unsupported Dequantize policy on current device");
    if (qp->hasOffset) return fail(ASCQ_ERR_UNSUPPORTED, "Dequantize do not support offset currently");
    const bool rowWise = policy == ASCQ_PER_TENSOR || policy == ASCQ_PER_CHANNEL;
    const uint64_t total = static_cast<uint64_t>(qp->m) * qp->n;
    if (total > 0xFFFFFFFFull) return fail(ASCQ_ERR_INVALID_ARG, "m * n does not fit 32 bits");
    ascq_dequant_param p{qp->m, qp->n, rowWise ? qp->n : static_cast<uint32_t>(total), qp->groupSize, qp->kDim};
    return ascq_dequant(dst, dstT, src, srcT, scale, nullptr, scaleT, scaleScalar, policy, &p, stream);
}
