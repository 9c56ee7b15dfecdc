// C++ host mirror of the Ascend C quantization operator interface on top of the C ABI (ascq.h).
//
// The reference operators are device-side templates over on-chip LocalTensor<T> views
// (include/adv_api/quantization/ascend_quant.h, ascend_dequant.h, ascend_antiquant.h).  Here the same names,
// template parameters and argument order work on global-memory views and enqueue one library call on a CUDA
// stream.  Where the reference asserts (ASCENDC_ASSERT), these functions throw ascq::Error.
//
// Header only; link against libascq.so.  No CUDA headers are needed: a stream is passed as void*.
#ifndef ASCQ_ASCENDC_HPP_
#define ASCQ_ASCENDC_HPP_

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "ascq.h"

namespace ascq {

struct Error : std::runtime_error {
    ascq_status status;
    Error(ascq_status s, const char* msg) : std::runtime_error(std::string(ascq_status_string(s)) + ": " + msg), status(s) {}
};
inline void check(ascq_status s)
{
    if (s != ASCQ_OK) throw Error(s, ascq_last_error());
}

// 16-bit storage tags: the host never does arithmetic on them, it only needs the dtype code.
struct half_t { uint16_t bits; };
struct bfloat16_t { uint16_t bits; };
struct fp4x2_e2m1_t { uint8_t bits; };
struct fp8_e8m0_t { uint8_t bits; };

template <typename T> struct DTypeOf;
template <> struct DTypeOf<half_t> { static constexpr ascq_dtype value = ASCQ_DT_F16; };
template <> struct DTypeOf<bfloat16_t> { static constexpr ascq_dtype value = ASCQ_DT_BF16; };
template <> struct DTypeOf<float> { static constexpr ascq_dtype value = ASCQ_DT_F32; };
template <> struct DTypeOf<int8_t> { static constexpr ascq_dtype value = ASCQ_DT_I8; };
template <> struct DTypeOf<int32_t> { static constexpr ascq_dtype value = ASCQ_DT_I32; };
template <> struct DTypeOf<uint64_t> { static constexpr ascq_dtype value = ASCQ_DT_U64; };
template <> struct DTypeOf<fp4x2_e2m1_t> { static constexpr ascq_dtype value = ASCQ_DT_FP4X2_E2M1; };
template <> struct DTypeOf<fp8_e8m0_t> { static constexpr ascq_dtype value = ASCQ_DT_E8M0; };

// Counterpart of LocalTensor<T>/GlobalTensor<T>: a typed view of device memory (not owning).
template <typename T> struct GlobalTensor {
    T* ptr = nullptr;
    size_t size = 0;  // elements
    GlobalTensor() = default;
    GlobalTensor(T* p, size_t n) : ptr(p), size(n) {}
    T* GetPhyAddr() const { return ptr; }
    size_t GetSize() const { return size; }
    GlobalTensor operator[](size_t offset) const { return GlobalTensor(ptr + offset, size - offset); }
};

}  // namespace ascq

namespace AscendC {

using ascq::GlobalTensor;
using half = ascq::half_t;
using bfloat16_t = ascq::bfloat16_t;

enum class RoundMode { CAST_NONE = 0, CAST_RINT, CAST_FLOOR, CAST_CEIL, CAST_ROUND, CAST_TRUNC };
enum class AscendQuantPolicy : int32_t { PER_TENSOR, PER_CHANNEL, PER_TOKEN, PER_GROUP, PER_CHANNEL_PER_GROUP, PER_TOKEN_PER_GROUP };
using AscendDeQuantPolicy = AscendQuantPolicy;
using AscendAntiQuantPolicy = AscendQuantPolicy;

// include/adv_api/quantization/ascend_quant_utils.h:31-87 (run-time relevant fields)
struct AscendQuantConfig {
    bool hasOffset = false;
    int32_t kDim = 1;
    RoundMode roundMode = RoundMode::CAST_RINT;
};
struct AscendQuantParam { uint32_t m, n, calCount, groupSize = 0; };
struct DequantParams { uint32_t m, n, calCount; };
struct AscendDeQuantParam { uint32_t m, n, calCount, groupSize = 0; };
struct AscendAntiQuantConfig { bool hasOffset = false; bool isTranspose = false; int32_t kDim = 1; };
struct AscendAntiQuantParam { uint32_t m, n, calCount = 0, groupSize = 0; };

// AscendQuant<T>(dst, src, scale, offset, calCount) -- per tensor (ascend_quant.h:63-97)
template <typename T>
inline void AscendQuant(const GlobalTensor<int8_t>& dst, const GlobalTensor<T>& src, float scale, float offset, uint32_t calCount,
                        void* stream = nullptr)
{
    ascq_quant_param p{1, calCount, calCount, 0, 1, 1, ASCQ_CAST_RINT};
    ascq::check(ascq_quant(dst.ptr, ASCQ_DT_I8, src.ptr, ascq::DTypeOf<T>::value, nullptr, nullptr, ASCQ_DT_F32, scale, offset,
                           ASCQ_PER_TENSOR, &p, stream));
}
// AscendQuant<T>(dst, src, scaleTensor, offset, scaleCount, calCount) -- per channel, scalar offset (ascend_quant.h:159-250)
template <typename T>
inline void AscendQuant(const GlobalTensor<int8_t>& dst, const GlobalTensor<T>& src, const GlobalTensor<T>& scaleTensor, float offset,
                        uint32_t scaleCount, uint32_t calCount, void* stream = nullptr)
{
    ascq_quant_param p{scaleCount ? calCount / scaleCount : 0, scaleCount, calCount, 0, 1, 1, ASCQ_CAST_RINT};
    ascq::check(ascq_quant(dst.ptr, ASCQ_DT_I8, src.ptr, ascq::DTypeOf<T>::value, scaleTensor.ptr, nullptr, ascq::DTypeOf<T>::value,
                           0.f, offset, ASCQ_PER_CHANNEL, &p, stream));
}
// AscendQuant<T>(dst, src, scaleTensor, offsetTensor, scaleCount, offsetCount, calCount) (ascend_quant.h:252-347)
template <typename T>
inline void AscendQuant(const GlobalTensor<int8_t>& dst, const GlobalTensor<T>& src, const GlobalTensor<T>& scaleTensor,
                        const GlobalTensor<T>& offsetTensor, uint32_t scaleCount, uint32_t offsetCount, uint32_t calCount,
                        void* stream = nullptr)
{
    if (scaleCount != offsetCount) throw ascq::Error(ASCQ_ERR_INVALID_ARG, "scaleCount should be equal to offsetCount");
    ascq_quant_param p{scaleCount ? calCount / scaleCount : 0, scaleCount, calCount, 0, 1, 1, ASCQ_CAST_RINT};
    ascq::check(ascq_quant(dst.ptr, ASCQ_DT_I8, src.ptr, ascq::DTypeOf<T>::value, scaleTensor.ptr, offsetTensor.ptr,
                           ascq::DTypeOf<T>::value, 0.f, 0.f, ASCQ_PER_CHANNEL, &p, stream));
}
// AscendQuant<dstT, srcT, scaleT, config, policy>(dst, src, scale, offset, para) (ascend_quant.h:667-762)
template <typename dstT, typename srcT, typename scaleT>
inline void AscendQuant(const GlobalTensor<dstT>& dst, const GlobalTensor<srcT>& src, const GlobalTensor<scaleT>& scale,
                        const GlobalTensor<scaleT>& offset, const AscendQuantParam& para, AscendQuantPolicy policy,
                        const AscendQuantConfig& config = {}, void* stream = nullptr)
{
    ascq_quant_param p{para.m, para.n, para.calCount, para.groupSize, config.hasOffset ? 1 : 0, config.kDim,
                       static_cast<ascq_round>(config.roundMode)};
    ascq::check(ascq_quant(dst.ptr, ascq::DTypeOf<dstT>::value, src.ptr, ascq::DTypeOf<srcT>::value, scale.ptr,
                           config.hasOffset ? offset.ptr : nullptr, ascq::DTypeOf<scaleT>::value, 0.f, 0.f,
                           static_cast<ascq_policy>(policy), &p, stream));
}

// AscendDequant<dstT, scaleT>(dst, src, deqScale, params) -- per channel (ascend_dequant.h:59-181)
template <typename dstT, typename scaleT>
inline void AscendDequant(const GlobalTensor<dstT>& dst, const GlobalTensor<int32_t>& src, const GlobalTensor<scaleT>& deqScale,
                          DequantParams params, void* stream = nullptr, const float* perTokenScale = nullptr)
{
    ascq_dequant_param p{params.m, params.n, params.calCount, 0, 1};
    ascq::check(ascq_dequant(dst.ptr, ascq::DTypeOf<dstT>::value, src.ptr, ASCQ_DT_I32, deqScale.ptr, perTokenScale,
                             ascq::DTypeOf<scaleT>::value, 0.f, ASCQ_PER_CHANNEL, &p, stream));
}
// AscendDequant<dstT>(dst, src, scalar deqScale, params) (ascend_dequant.h:186-281)
template <typename dstT>
inline void AscendDequant(const GlobalTensor<dstT>& dst, const GlobalTensor<int32_t>& src, float deqScale, DequantParams params,
                          void* stream = nullptr)
{
    ascq_dequant_param p{params.m, params.n, params.calCount, 0, 1};
    ascq::check(ascq_dequant(dst.ptr, ascq::DTypeOf<dstT>::value, src.ptr, ASCQ_DT_I32, nullptr, nullptr, ASCQ_DT_F32, deqScale,
                             ASCQ_PER_TENSOR, &p, stream));
}
// AscendDequant<dstT, srcT, scaleT, config, policy>(dst, src, scale, offset, para) (ascend_dequant.h:286-307)
template <typename dstT, typename srcT, typename scaleT>
inline void AscendDequant(const GlobalTensor<dstT>& dst, const GlobalTensor<srcT>& src, const GlobalTensor<scaleT>& scale,
                          const AscendDeQuantParam& para, AscendDeQuantPolicy policy, int32_t kDim = 1, void* stream = nullptr)
{
    ascq_dequant_param p{para.m, para.n, para.calCount, para.groupSize, kDim};
    ascq::check(ascq_dequant(dst.ptr, ascq::DTypeOf<dstT>::value, src.ptr, ascq::DTypeOf<srcT>::value, scale.ptr, nullptr,
                             ascq::DTypeOf<scaleT>::value, 0.f, static_cast<ascq_policy>(policy), &p, stream));
}

// AscendAntiQuant<InputDataType, OutputDataType, isTranspose>(dst, src, offset, scale, K) (ascend_antiquant.h:50-134).
// src holds src.size elements: [K, N] or, transposed, [N, K]; scale/offset hold N values per group.
template <typename InT, typename OutT, bool isTranspose>
inline void AscendAntiQuant(const GlobalTensor<OutT>& dst, const GlobalTensor<InT>& src, const GlobalTensor<OutT>& offset,
                            const GlobalTensor<OutT>& scale, uint32_t K, uint32_t groupSize = 0, void* stream = nullptr)
{
    const uint32_t other = static_cast<uint32_t>(src.size / K);
    ascq_antiquant_param p{isTranspose ? other : K, isTranspose ? K : other, 0, groupSize, 1, isTranspose ? 1 : 0, 1};
    ascq::check(ascq_antiquant(dst.ptr, ascq::DTypeOf<OutT>::value, src.ptr, ascq::DTypeOf<InT>::value, offset.ptr, scale.ptr,
                               ascq::DTypeOf<OutT>::value, 0.f, 0.f, ASCQ_PER_CHANNEL, &p, stream));
}
// fp4 + e8m0 overload (ascend_antiquant.h:211-231)
template <typename OutT, bool isTranspose>
inline void AscendAntiQuant(const GlobalTensor<OutT>& dst, const GlobalTensor<ascq::fp4x2_e2m1_t>& src,
                            const GlobalTensor<ascq::fp8_e8m0_t>& scale, uint32_t K, uint32_t elements, void* stream = nullptr)
{
    const uint32_t other = elements / K;
    ascq_antiquant_param p{isTranspose ? other : K, isTranspose ? K : other, 0, 32, 0, isTranspose ? 1 : 0, 1};
    ascq::check(ascq_antiquant(dst.ptr, ascq::DTypeOf<OutT>::value, src.ptr, ASCQ_DT_FP4X2_E2M1, nullptr, scale.ptr, ASCQ_DT_E8M0,
                               0.f, 0.f, ASCQ_PER_GROUP, &p, stream));
}
// AscendAntiQuant<dstT, srcT, scaleT, config, policy>(dst, src, scale, offset, para) (ascend_antiquant.h:233-262)
template <typename dstT, typename srcT, typename scaleT>
inline void AscendAntiQuant(const GlobalTensor<dstT>& dst, const GlobalTensor<srcT>& src, const GlobalTensor<scaleT>& scale,
                            const GlobalTensor<scaleT>& offset, const AscendAntiQuantParam& para, AscendAntiQuantPolicy policy,
                            const AscendAntiQuantConfig& config = {}, void* stream = nullptr)
{
    ascq_antiquant_param p{para.m, para.n, para.calCount, para.groupSize, config.hasOffset ? 1 : 0, config.isTranspose ? 1 : 0,
                           config.kDim};
    ascq::check(ascq_antiquant(dst.ptr, ascq::DTypeOf<dstT>::value, src.ptr, ascq::DTypeOf<srcT>::value,
                               config.hasOffset ? offset.ptr : nullptr, scale.ptr, ascq::DTypeOf<scaleT>::value, 0.f, 0.f,
                               static_cast<ascq_policy>(policy), &p, stream));
}

// ---- the unified interface (include/adv_api/quantization/quantize.h:41-62, dequantize.h, antiquantize.h) ----------
enum class QuantizePolicy : int32_t { PER_TENSOR, PER_CHANNEL, PER_TOKEN, PER_GROUP };
using DequantizePolicy = QuantizePolicy;
using AntiQuantizePolicy = QuantizePolicy;
struct QuantizeConfig {
    QuantizePolicy policy;
    bool hasOffset = false;
    RoundMode roundMode = RoundMode::CAST_RINT;
    int32_t kDim = 1;
};
struct DequantizeConfig { DequantizePolicy policy; bool hasOffset = false; int32_t kDim = 1; };
struct AntiQuantizeConfig { AntiQuantizePolicy policy; bool hasOffset = false; int32_t kDim = 1; };
struct QuantizeParams { uint32_t m, n, groupSize = 0; };
using DequantizeParams = QuantizeParams;
using AntiQuantizeParams = QuantizeParams;

namespace detail {
inline ascq_quantize_param pack(const QuantizeParams& p, bool hasOffset, int32_t kDim, RoundMode mode)
{
    return ascq_quantize_param{p.m, p.n, p.groupSize, hasOffset ? 1 : 0, kDim, static_cast<ascq_round>(mode)};
}
}  // namespace detail

// Quantize, scalar scale and offset (PER_TENSOR)
template <typename DstT, typename SrcT>
inline void Quantize(const QuantizeConfig& config, const GlobalTensor<DstT>& dst, const GlobalTensor<SrcT>& src, float scale,
                     float offset, const QuantizeParams& params, void* stream = nullptr)
{
    const ascq_quantize_param p = detail::pack(params, config.hasOffset, config.kDim, config.roundMode);
    ascq::check(ascq_quantize(dst.ptr, ascq::DTypeOf<DstT>::value, src.ptr, ascq::DTypeOf<SrcT>::value, nullptr, nullptr,
                              ASCQ_DT_F32, scale, offset, static_cast<ascq_policy>(config.policy), &p, stream));
}
// Quantize, tensor scale and offset (PER_CHANNEL / PER_TOKEN / PER_GROUP)
template <typename DstT, typename SrcT, typename ScaleT>
inline void Quantize(const QuantizeConfig& config, const GlobalTensor<DstT>& dst, const GlobalTensor<SrcT>& src,
                     const GlobalTensor<ScaleT>& scale, const GlobalTensor<ScaleT>& offset, const QuantizeParams& params,
                     void* stream = nullptr)
{
    const ascq_quantize_param p = detail::pack(params, config.hasOffset, config.kDim, config.roundMode);
    ascq::check(ascq_quantize(dst.ptr, ascq::DTypeOf<DstT>::value, src.ptr, ascq::DTypeOf<SrcT>::value, scale.ptr,
                              config.hasOffset ? offset.ptr : nullptr, ascq::DTypeOf<ScaleT>::value, 0.f, 0.f,
                              static_cast<ascq_policy>(config.policy), &p, stream));
}
template <typename DstT, typename SrcT>
inline void Dequantize(const DequantizeConfig& config, const GlobalTensor<DstT>& dst, const GlobalTensor<SrcT>& src, float scale,
                       const DequantizeParams& params, void* stream = nullptr)
{
    const ascq_quantize_param p = detail::pack(params, config.hasOffset, config.kDim, RoundMode::CAST_RINT);
    ascq::check(ascq_dequantize(dst.ptr, ascq::DTypeOf<DstT>::value, src.ptr, ascq::DTypeOf<SrcT>::value, nullptr, ASCQ_DT_F32,
                                scale, static_cast<ascq_policy>(config.policy), &p, stream));
}
template <typename DstT, typename SrcT, typename ScaleT>
inline void Dequantize(const DequantizeConfig& config, const GlobalTensor<DstT>& dst, const GlobalTensor<SrcT>& src,
                       const GlobalTensor<ScaleT>& scale, const GlobalTensor<ScaleT>& /*offset: not supported by the reference yet*/,
                       const DequantizeParams& params, void* stream = nullptr)
{
    const ascq_quantize_param p = detail::pack(params, config.hasOffset, config.kDim, RoundMode::CAST_RINT);
    ascq::check(ascq_dequantize(dst.ptr, ascq::DTypeOf<DstT>::value, src.ptr, ascq::DTypeOf<SrcT>::value, scale.ptr,
                                ascq::DTypeOf<ScaleT>::value, 0.f, static_cast<ascq_policy>(config.policy), &p, stream));
}
template <typename DstT, typename SrcT>
inline void AntiQuantize(const AntiQuantizeConfig& config, const GlobalTensor<DstT>& dst, const GlobalTensor<SrcT>& src, float scale,
                         float offset, const AntiQuantizeParams& params, void* stream = nullptr)
{
    const ascq_quantize_param p = detail::pack(params, config.hasOffset, config.kDim, RoundMode::CAST_RINT);
    ascq::check(ascq_antiquantize(dst.ptr, ascq::DTypeOf<DstT>::value, src.ptr, ascq::DTypeOf<SrcT>::value, nullptr, nullptr,
                                  ascq::DTypeOf<DstT>::value, offset, scale, static_cast<ascq_policy>(config.policy), &p, stream));
}
template <typename DstT, typename SrcT, typename ScaleT>
inline void AntiQuantize(const AntiQuantizeConfig& config, const GlobalTensor<DstT>& dst, const GlobalTensor<SrcT>& src,
                         const GlobalTensor<ScaleT>& scale, const GlobalTensor<ScaleT>& offset, const AntiQuantizeParams& params,
                         void* stream = nullptr)
{
    const ascq_quantize_param p = detail::pack(params, config.hasOffset, config.kDim, RoundMode::CAST_RINT);
    ascq::check(ascq_antiquantize(dst.ptr, ascq::DTypeOf<DstT>::value, src.ptr, ascq::DTypeOf<SrcT>::value,
                                  config.hasOffset ? offset.ptr : nullptr, scale.ptr, ascq::DTypeOf<ScaleT>::value, 0.f, 0.f,
                                  static_cast<ascq_policy>(config.policy), &p, stream));
}

// Host tiling helpers (include/adv_api/quantization/ascend_quant_tiling.h etc.); shape = dims + rank.
inline void GetAscendQuantMaxMinTmpSize(const int64_t* dims, int rank, uint32_t typeSize, uint32_t& maxValue, uint32_t& minValue)
{
    ascq::check(ascq_get_ascend_quant_max_min_tmp_size(dims, rank, typeSize, &maxValue, &minValue));
}
inline void GetAscendDequantMaxMinTmpSize(const int64_t* dims, int rank, uint32_t typeSize, uint32_t& maxValue, uint32_t& minValue)
{
    ascq::check(ascq_get_ascend_dequant_max_min_tmp_size(dims, rank, typeSize, &maxValue, &minValue));
}

}  // namespace AscendC
#endif  // ASCQ_ASCENDC_HPP_
