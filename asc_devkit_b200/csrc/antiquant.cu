// ascq_antiquant: AscendAntiQuant on global-memory tensors.
#include "elementwise.cuh"

namespace ascq {
namespace {

template <typename Dst, typename Sc, typename CT>
ascq_status run_fast(const EwArgs& a, int smode, bool hasOff, cudaStream_t st)
{
    return launch_ew_rows<kOpAntiQuant, int8_t, Dst, Sc, CT>(a, smode, hasOff, false, st);
}
// int4b_t sources: the type triples of the legacy overloads (what the weight-only-quantised matmul uses) and of the
// unified interface on half; everything else from int4 goes to the scalar kernel
ascq_status dispatch_fast_i4(const EwArgs& a, ascq_dtype dstT, ascq_dtype scT, ascq_dtype ct, int smode, bool hasOff, cudaStream_t st,
                             bool* handled)
{
    *handled = true;
    if (ct == ASCQ_DT_F16 && dstT == ASCQ_DT_F16 && (scT == ASCQ_DT_F16 || smode == kSScalar))
        return launch_ew_rows<kOpAntiQuant, int4x2_t, __half, __half, __half>(a, smode, hasOff, false, st);
    if (ct == ASCQ_DT_F32 && dstT == ASCQ_DT_BF16 && (scT == ASCQ_DT_BF16 || smode == kSScalar))
        return launch_ew_rows<kOpAntiQuant, int4x2_t, __nv_bfloat16, __nv_bfloat16, float>(a, smode, hasOff, false, st);
    if (ct == ASCQ_DT_F32 && dstT == ASCQ_DT_F16 && (scT == ASCQ_DT_F16 || smode == kSScalar))
        return launch_ew_rows<kOpAntiQuant, int4x2_t, __half, __half, float>(a, smode, hasOff, false, st);
    *handled = false;
    return ASCQ_OK;
}

ascq_status dispatch_fast(const EwArgs& a, ascq_dtype dstT, ascq_dtype scT, ascq_dtype ct, int smode, bool hasOff,
                          cudaStream_t st, bool* handled)
{
    *handled = true;
    if (ct == ASCQ_DT_F16 && dstT == ASCQ_DT_F16 && (scT == ASCQ_DT_F16 || smode == kSScalar))
        return run_fast<__half, __half, __half>(a, smode, hasOff, st);
    if (ct == ASCQ_DT_BF16 && dstT == ASCQ_DT_BF16 && scT == ASCQ_DT_BF16)
        return run_fast<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(a, smode, hasOff, st);
    if (ct == ASCQ_DT_F32) {
        if (dstT == ASCQ_DT_BF16 && (scT == ASCQ_DT_BF16 || smode == kSScalar))
            return run_fast<__nv_bfloat16, __nv_bfloat16, float>(a, smode, hasOff, st);
        if (dstT == ASCQ_DT_F16 && (scT == ASCQ_DT_F16 || smode == kSScalar))  // the unified AntiQuantize interface
            return run_fast<__half, __half, float>(a, smode, hasOff, st);
        if (scT == ASCQ_DT_F32) {
            if (dstT == ASCQ_DT_F32) return run_fast<float, float, float>(a, smode, hasOff, st);
            if (dstT == ASCQ_DT_F16) return run_fast<__half, float, float>(a, smode, hasOff, st);
            if (dstT == ASCQ_DT_BF16) return run_fast<__nv_bfloat16, float, float>(a, smode, hasOff, st);
        }
    }
    *handled = false;
    return ASCQ_OK;
}

// ---- MX decode: fp4x2 (E2M1) + E8M0 scale -> bf16 / half ------------------------------------------
// One lane converts 8 elements: one 4-byte load, one 16-byte store, so every access of a warp is contiguous.  The four
// source bytes go through the hardware conversion (cvt.rn.f16x2.e2m1x2; every E2M1 value is exact in half and in
// bfloat16), the product with the scale is one packed multiply per two elements.  With the groups along the columns
// (transposed layout) the 8 elements share one scale byte; with the groups along the rows the lane reads the 8 scale
// bytes of its columns.  Two rows per thread are requested before the first is worked on.
__device__ __forceinline__ void e2m1x8_to_f16x2(uint32_t w, uint32_t (&h)[4])
{
    asm("{ .reg .b8 b0, b1, b2, b3;\n"
        " mov.b32 {b0, b1, b2, b3}, %4;\n"
        " cvt.rn.f16x2.e2m1x2 %0, b0;\n cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        " cvt.rn.f16x2.e2m1x2 %2, b2;\n cvt.rn.f16x2.e2m1x2 %3, b3; }"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "r"(w));
}
// the scale as the multiplier of the destination type: bfloat16 bits, or the half that the saturating cast gives
template <typename Dst> __device__ __forceinline__ uint32_t mx_scale_bits(uint32_t e)
{
    const unsigned short b = e8m0_to_bf16_bits(e);
    if constexpr (std::is_same<Dst, __nv_bfloat16>::value) return b;
    else return __half_as_ushort(f32_to_f16_sat(__uint_as_float(static_cast<uint32_t>(b) << 16)));
}
template <typename Dst, bool TRANSPOSED>
__global__ void __launch_bounds__(256) mx_decode_kernel(Dst* __restrict__ dst, const uint8_t* __restrict__ src,
                                                        const uint8_t* __restrict__ scale, uint32_t rows, uint32_t cols)
{
    const uint32_t c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8u;
    if (c0 >= cols) return;
    constexpr int U = 2;
    const uint32_t gy = gridDim.y;
    for (uint32_t r0 = blockIdx.y; r0 < rows; r0 += gy * U) {
        uint32_t raw[U];
        uint2 sraw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t r = r0 + u * gy;
            if (r >= rows) break;
            raw[u] = __ldcs(reinterpret_cast<const uint32_t*>(src + (static_cast<size_t>(r) * cols + c0) / 2));
            if (TRANSPOSED) sraw[u].x = scale[static_cast<size_t>(r) * (cols / 32) + c0 / 32];
            else sraw[u] = __ldg(reinterpret_cast<const uint2*>(scale + static_cast<size_t>(r / 32) * cols + c0));
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t r = r0 + u * gy;
            if (r >= rows) break;
            uint32_t h[4], out[4];
            e2m1x8_to_f16x2(raw[u], h);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t s2;
                if (TRANSPOSED) {
                    s2 = mx_scale_bits<Dst>(sraw[u].x) * 0x10001u;
                } else {
                    const uint32_t word = (j < 2) ? sraw[u].x : sraw[u].y;
                    s2 = mx_scale_bits<Dst>((word >> ((j & 1) * 16)) & 0xFFu) | (mx_scale_bits<Dst>((word >> ((j & 1) * 16 + 8)) & 0xFFu) << 16);
                }
                if constexpr (std::is_same<Dst, __nv_bfloat16>::value) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[j]));
                    const __nv_bfloat162 v = __floats2bfloat162_rn(f.x, f.y);  // exact
                    const __nv_bfloat162 y = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&s2), v);
                    out[j] = *reinterpret_cast<const uint32_t*>(&y);
                } else {
                    const __half2 y = __hmul2(*reinterpret_cast<const __half2*>(&s2), *reinterpret_cast<const __half2*>(&h[j]));
                    out[j] = *reinterpret_cast<const uint32_t*>(&y);
                }
            }
            __stcs(reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * cols + c0), make_uint4(out[0], out[1], out[2], out[3]));
        }
    }
}
}  // namespace
}  // namespace ascq

using namespace ascq;

// Shared body.  `unified` selects the numerics of the AntiQuantize interface
// (impl/adv_api/detail/quantization/antiquantize/antiquantize_3510_impl.h:252-381, antiquantize_impl.h:68-190):
// every policy widens source, offset and scale to fp32, adds, multiplies and casts once (RINT, saturating).
static ascq_status antiquant_common(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT, const void* offset,
                                    const void* scale, ascq_dtype scaleT, float offsetScalar, float scaleScalar,
                                    ascq_policy policy, const ascq_antiquant_param* p, void* stream, bool unified)
{
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!dst || !src || !p) return fail(ASCQ_ERR_INVALID_ARG, "dst, src and param must not be NULL");
    if (policy == ASCQ_PER_CHANNEL_PER_GROUP || policy == ASCQ_PER_TOKEN_PER_GROUP)
        return fail(ASCQ_ERR_UNSUPPORTED, "unsupported policy for AscendAntiQuant in current device!");
    if (policy < ASCQ_PER_TENSOR || policy > ASCQ_PER_GROUP) return fail(ASCQ_ERR_INVALID_ARG, "unknown policy %d", (int)policy);
    if (dst == src) return fail(ASCQ_ERR_INVALID_ARG, "src and dst must not overlap");
    if (p->n == 0) return fail(ASCQ_ERR_INVALID_ARG, "n must be greater than 0");
    const uint64_t total64 = p->calCount ? p->calCount : static_cast<uint64_t>(p->m) * p->n;
    if (total64 > 0xFFFFFFFFull) return fail(ASCQ_ERR_INVALID_ARG, "element count exceeds 2^32-1");
    const uint32_t total = static_cast<uint32_t>(total64);
    if (total % p->n != 0) return fail(ASCQ_ERR_INVALID_ARG, "calCount is %u, which should be an integer multiple of n %u", total, p->n);
    const uint32_t rows = total / p->n, n = p->n;
    if (rows == 0) return ASCQ_OK;

    if (srcT == ASCQ_DT_FP4X2_E2M1) {
        // include/adv_api/quantization/ascend_antiquant.h:211-231
        if (scaleT != ASCQ_DT_E8M0 || !scale) return fail(ASCQ_ERR_INVALID_ARG, "fp4 input takes an fp8_e8m0 scale tensor");
        if (offset || p->hasOffset) return fail(ASCQ_ERR_UNSUPPORTED, "AscendAntiQuant from fp4 does not take an offset");
        if (dstT != ASCQ_DT_BF16 && dstT != ASCQ_DT_F16) return fail(ASCQ_ERR_UNSUPPORTED, "fp4 input decodes to half or bfloat16_t");
        const uint32_t kext = p->isTranspose ? n : rows;
        if (kext % 32 != 0) return fail(ASCQ_ERR_INVALID_ARG, "the K extent %u must be a multiple of the group size 32", kext);
        if (n % 2) return fail(ASCQ_ERR_INVALID_ARG, "n must be even for packed fp4");
        if (n % 32 == 0 && aligned16(src) && aligned16(dst) && (p->isTranspose || aligned16(scale))) {
            dim3 grid, block;
            ew_grid(rows, n, 8, &grid, &block);
            uint8_t const* s8 = static_cast<const uint8_t*>(src);
            uint8_t const* sc = static_cast<const uint8_t*>(scale);
            if (dstT == ASCQ_DT_BF16) {
                if (p->isTranspose) mx_decode_kernel<__nv_bfloat16, true><<<grid, block, 0, st>>>(static_cast<__nv_bfloat16*>(dst), s8, sc, rows, n);
                else mx_decode_kernel<__nv_bfloat16, false><<<grid, block, 0, st>>>(static_cast<__nv_bfloat16*>(dst), s8, sc, rows, n);
            } else {
                if (p->isTranspose) mx_decode_kernel<__half, true><<<grid, block, 0, st>>>(static_cast<__half*>(dst), s8, sc, rows, n);
                else mx_decode_kernel<__half, false><<<grid, block, 0, st>>>(static_cast<__half*>(dst), s8, sc, rows, n);
            }
            ASCQ_CUDA_CHECK(cudaGetLastError());
            return ASCQ_OK;
        }
        GenericArgs g{};
        g.op = kOpAntiQuant; g.srcT = srcT; g.dstT = dstT; g.scT = scaleT; g.ct = dstT;
        g.src = src; g.dst = dst; g.rows = rows; g.cols = n; g.srcStride = g.dstStride = n;
        g.scale.p = scale; g.fp4Transposed = p->isTranspose;
        return launch_ew_generic(g, st);
    }
    if (srcT != ASCQ_DT_I8 && srcT != ASCQ_DT_I4X2)
        return fail(ASCQ_ERR_UNSUPPORTED, "AscendAntiQuant source dtype %d is not built (int8, int4b_t and fp4x2_e2m1 are)", (int)srcT);
    if (srcT == ASCQ_DT_I4X2 && (n % 2 != 0))
        return fail(ASCQ_ERR_INVALID_ARG, "n must be even for a packed int4b_t source");

    EwArgs a{};
    a.src = src;
    a.dst = dst;
    a.rows = rows;
    a.cols = n;
    a.srcStride = a.dstStride = n;
    a.roundMode = kRoundRint;
    int smode = kSScalar;
    bool hasOff = true;
    ascq_dtype ct;

    if (policy == ASCQ_PER_TENSOR || policy == ASCQ_PER_CHANNEL) {
        // impl/adv_api/detail/quantization/antiquant/ascend_antiquant_c220_impl.h:33-43
        if (dstT != ASCQ_DT_F16 && dstT != ASCQ_DT_BF16)
            return fail(ASCQ_ERR_UNSUPPORTED, "current api support dtype combination is src: int8_t / int4b_t, dst: half / bfloat16_t.");
        ct = (dstT == ASCQ_DT_F16) ? ASCQ_DT_F16 : ASCQ_DT_F32;
        if (policy == ASCQ_PER_TENSOR) {
            if (scale || offset) return fail(ASCQ_ERR_INVALID_ARG, "per-tensor AscendAntiQuant takes scalar scale/offset; tensors must be NULL");
            hasOff = p->hasOffset != 0;
            // the scalars are dstT values in the reference signature: round them to dstT first
            a.scale.scalar = scaleScalar;
            a.offset.scalar = offsetScalar;
        } else {
            if (!scale) return fail(ASCQ_ERR_INVALID_ARG, "scale tensor must not be NULL");
            if (scaleT != dstT) return fail(ASCQ_ERR_UNSUPPORTED, "scale/offset dtype must equal the output dtype");
            hasOff = unified ? (p->hasOffset != 0) : (offset != nullptr);
            if (hasOff && !offset) return fail(ASCQ_ERR_INVALID_ARG, "hasOffset is set but the offset tensor is NULL");
            const uint32_t K = p->isTranspose ? n : rows;
            const uint32_t gs = p->groupSize ? p->groupSize : K;
            if (K % gs != 0) return fail(ASCQ_ERR_INVALID_ARG, "K %u must be a multiple of groupSize %u", K, gs);
            if (p->isTranspose && (static_cast<size_t>(K) * dtype_size(srcT)) % 32 != 0)
                return fail(ASCQ_ERR_INVALID_ARG, "When isTranspose is true, srcShape is [N, K] where the dimension K must be 32B aligned!");
            a.scale.p = scale;
            if (!p->isTranspose) {
                a.scale.rdiv = gs; a.scale.cdiv = 1; a.scale.stride = n;
                smode = (gs == K) ? kSColVec : kSRowVec;
                if (gs == K) a.scale.rdiv = 0;
            } else {
                a.scale.rdiv = 1; a.scale.cdiv = gs; a.scale.stride = K / gs;
                smode = kSRowBcast;
            }
            a.offset = a.scale;
            a.offset.p = offset;
        }
    } else {
        if (!scale) return fail(ASCQ_ERR_INVALID_ARG, "scale tensor must not be NULL");
        if (scaleT != ASCQ_DT_F16 && scaleT != ASCQ_DT_BF16 && scaleT != ASCQ_DT_F32)
            return fail(ASCQ_ERR_UNSUPPORTED, "scale dtype must be half, bfloat16_t or float");
        if (dstT != ASCQ_DT_F16 && dstT != ASCQ_DT_BF16 && dstT != ASCQ_DT_F32)
            return fail(ASCQ_ERR_UNSUPPORTED, "dst dtype must be half, bfloat16_t or float");
        if (scaleT != ASCQ_DT_F32 && dstT != scaleT)
            return fail(ASCQ_ERR_UNSUPPORTED, "unsupported (dst, scale) dtype pair for AscendAntiQuant PER_TOKEN/PER_GROUP");
        ct = scaleT;
        hasOff = p->hasOffset != 0;
        if (hasOff && !offset) return fail(ASCQ_ERR_INVALID_ARG, "hasOffset is set but the offset tensor is NULL");
        a.scale.p = scale;
        if (policy == ASCQ_PER_TOKEN) {
            if (p->isTranspose) { a.scale.rdiv = 0; a.scale.cdiv = 1; a.scale.stride = 0; smode = kSColVec; }
            else { a.scale.rdiv = 1; a.scale.cdiv = 0; a.scale.stride = 1; smode = kSRowBcast; }
        } else {
            if (p->groupSize == 0 || p->groupSize % 32 != 0)
                return fail(ASCQ_ERR_INVALID_ARG, "groupSize is %u, which must be a positive multiple of 32", p->groupSize);
            // impl/adv_api/detail/quantization/antiquant/ascend_antiquant_3510_impl.h:2214-2220
            const bool alongCols = (p->kDim == 1 && !p->isTranspose) || (p->kDim == 0 && p->isTranspose);
            if (alongCols) {
                a.scale.rdiv = 1; a.scale.cdiv = p->groupSize; a.scale.stride = (n + p->groupSize - 1) / p->groupSize;
                smode = kSRowBcast;
            } else {
                a.scale.rdiv = p->groupSize; a.scale.cdiv = 1; a.scale.stride = n;
                smode = kSRowVec;
            }
        }
        a.offset = a.scale;
        a.offset.p = hasOff ? offset : nullptr;
    }
    if (policy == ASCQ_PER_TENSOR) {
        // round the scalars to the type the reference signature carries them in
        // (include/adv_api/quantization/ascend_antiquant.h:136-205)
        if (dstT == ASCQ_DT_F16) {
            a.scale.scalar = __half2float(__float2half_rn(a.scale.scalar));
            a.offset.scalar = __half2float(__float2half_rn(a.offset.scalar));
        } else {
            a.scale.scalar = __bfloat162float(__float2bfloat16_rn(a.scale.scalar));
            a.offset.scalar = __bfloat162float(__float2bfloat16_rn(a.offset.scalar));
        }
    }

    if (unified) ct = ASCQ_DT_F32;
    if (srcT == ASCQ_DT_I8) {
        EwArgs b = a;
        b.scalarPath = ew_fast_ok(a, 16, smode, dtype_size(scaleT)) ? 0 : 1;  // ragged / unaligned: one element per thread
        bool handled = false;
        ascq_status rc = dispatch_fast(b, dstT, scaleT, ct, smode, hasOff, st, &handled);
        if (rc != ASCQ_OK || handled) return rc;
    }
    if (srcT == ASCQ_DT_I4X2 && ew_fast_ok(a, 16, smode, dtype_size(scaleT))) {
        bool handled = false;
        ascq_status rc = dispatch_fast_i4(a, dstT, scaleT, ct, smode, hasOff, st, &handled);
        if (rc != ASCQ_OK || handled) return rc;
    }
    GenericArgs g{};
    g.op = kOpAntiQuant; g.srcT = srcT; g.dstT = dstT; g.scT = scaleT; g.ct = ct;
    g.src = src; g.dst = dst; g.rows = a.rows; g.cols = a.cols; g.srcStride = a.srcStride; g.dstStride = a.dstStride;
    g.scale = a.scale; g.offset = a.offset; g.scaleIsScalar = (smode == kSScalar); g.hasOff = hasOff;
    g.offIsScalar = (smode == kSScalar); g.roundMode = kRoundRint;
    return launch_ew_generic(g, st);
}

extern "C" ascq_status ascq_antiquant(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT, const void* offset,
                                      const void* scale, ascq_dtype scaleT, float offsetScalar, float scaleScalar,
                                      ascq_policy policy, const ascq_antiquant_param* p, void* stream)
{
    return antiquant_common(dst, dstT, src, srcT, offset, scale, scaleT, offsetScalar, scaleScalar, policy, p, stream, false);
}

extern "C" ascq_status ascq_antiquantize(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT, const void* offset,
                                         const void* scale, ascq_dtype scaleT, float offsetScalar, float scaleScalar,
                                         ascq_policy policy, const ascq_quantize_param* qp, void* stream)
{
    if (!qp) return fail(ASCQ_ERR_INVALID_ARG, "dst, src and param must not be NULL");
    if (policy < ASCQ_PER_TENSOR || policy > ASCQ_PER_GROUP)
        return fail(ASCQ_ERR_UNSUPPORTED, "Unsupported AntiQuantize policy on current device");
    ascq_antiquant_param p{qp->m, qp->n, 0, policy == ASCQ_PER_GROUP ? qp->groupSize : 0, qp->hasOffset, 0, qp->kDim};
    return antiquant_common(dst, dstT, src, srcT, offset, scale, scaleT, offsetScalar, scaleScalar, policy, &p, stream, true);
}
