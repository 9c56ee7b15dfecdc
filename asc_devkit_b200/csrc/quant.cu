// ascq_quant / ascq_dynamic_quant_per_token: AscendQuant on global-memory tensors.
#include "elementwise.cuh"

namespace ascq {
namespace {

bool is_float_type(ascq_dtype t) { return t == ASCQ_DT_F16 || t == ASCQ_DT_BF16 || t == ASCQ_DT_F32; }

// Scale / offset addressing of the PER_TOKEN / PER_GROUP overloads
// (impl/adv_api/detail/quantization/quant/ascend_quant_per_group_3510_impl.h:142-178, 498-538, 1000-1044).
ascq_status policy_sref(SRef* s, const void* p, ascq_policy policy, uint32_t n, uint32_t groupSize, int kDim,
                        int* smode)
{
    s->p = p;
    s->scalar = 0.f;
    if (policy == ASCQ_PER_TOKEN) {
        s->rdiv = 1; s->cdiv = 0; s->stride = 1;
        *smode = kSRowBcast;
        return ASCQ_OK;
    }
    if (groupSize == 0 || groupSize % 32 != 0)
        return fail(ASCQ_ERR_INVALID_ARG, "groupSize is %u, which must be a positive multiple of 32", groupSize);
    if (kDim == 1) {
        s->rdiv = 1; s->cdiv = groupSize; s->stride = (n + groupSize - 1) / groupSize;
        *smode = kSRowBcast;
    } else if (kDim == 0) {
        s->rdiv = groupSize; s->cdiv = 1; s->stride = n;
        *smode = kSRowVec;
    } else {
        return fail(ASCQ_ERR_INVALID_ARG, "kDim is %d, which must be 0 or 1", kDim);
    }
    return ASCQ_OK;
}

template <typename Src, typename Sc, typename CT>
ascq_status run_fast(const EwArgs& a, int smode, bool hasOff, cudaStream_t st)
{
    return launch_ew_rows<kOpQuant, Src, int8_t, Sc, CT>(a, smode, hasOff, false, st);
}

ascq_status dispatch_fast(const EwArgs& a, ascq_dtype srcT, ascq_dtype scT, ascq_dtype ct, int smode, bool hasOff,
                          cudaStream_t st, bool* handled)
{
    *handled = true;
    if (ct == ASCQ_DT_F16) {
        // scalar operands carry no storage type: reuse the half instantiation
        const ascq_dtype sc = (smode == kSScalar) ? ASCQ_DT_F16 : scT;
        if (srcT == ASCQ_DT_F16 && sc == ASCQ_DT_F16) return run_fast<__half, __half, __half>(a, smode, hasOff, st);
        if (srcT == ASCQ_DT_F16 && sc == ASCQ_DT_F32) return run_fast<__half, float, __half>(a, smode, hasOff, st);
        if (srcT == ASCQ_DT_F32 && sc == ASCQ_DT_F16) return run_fast<float, __half, __half>(a, smode, hasOff, st);
        if (srcT == ASCQ_DT_F32 && sc == ASCQ_DT_F32) return run_fast<float, float, __half>(a, smode, hasOff, st);
        if (srcT == ASCQ_DT_BF16 && sc == ASCQ_DT_F16) return run_fast<__nv_bfloat16, __half, __half>(a, smode, hasOff, st);
    } else if (ct == ASCQ_DT_BF16) {
        if (srcT == ASCQ_DT_BF16 && scT == ASCQ_DT_BF16)
            return run_fast<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(a, smode, hasOff, st);
    } else {
        // scalar operands carry no storage type: reuse the float-scale instantiation
        const ascq_dtype sc = (smode == kSScalar) ? ASCQ_DT_F32 : scT;
        if (sc == ASCQ_DT_F32) {
            if (srcT == ASCQ_DT_F16) return run_fast<__half, float, float>(a, smode, hasOff, st);
            if (srcT == ASCQ_DT_BF16) return run_fast<__nv_bfloat16, float, float>(a, smode, hasOff, st);
            if (srcT == ASCQ_DT_F32) return run_fast<float, float, float>(a, smode, hasOff, st);
        }
        // the unified Quantize interface: 16-bit scales widened to fp32
        if (srcT == ASCQ_DT_F16 && sc == ASCQ_DT_F16) return run_fast<__half, __half, float>(a, smode, hasOff, st);
        if (srcT == ASCQ_DT_BF16 && sc == ASCQ_DT_BF16) return run_fast<__nv_bfloat16, __nv_bfloat16, float>(a, smode, hasOff, st);
    }
    *handled = false;
    return ASCQ_OK;
}

}  // namespace
}  // namespace ascq

using namespace ascq;

// Shared body.  `unified` selects the numerics of the Quantize interface
// (impl/adv_api/detail/quantization/quantize/quantize_impl.h:832-975): every policy computes in fp32 (source and
// scale/offset widened to fp32, one rounded multiply, one rounded add), honours hasOffset and roundMode, and takes
// the tensor as m rows of n (calCount = m * n).
// ---- AscendQuant PER_GROUP to fp4x2_e2m1, round to nearest even -------------------------------------------------
// (impl/adv_api/detail/quantization/quant/ascend_quant_per_group_3510_impl.h:346-379, ascend_quant_3510_impl.h:994-1032:
// the product in the scale's type, then -> bfloat16 -> E2M1.)  One lane per 8 elements: contiguous loads, one 4-byte
// store; the scale is one value per lane (groups along the columns) or 8 consecutive values (groups along the rows).
// The last conversion is the hardware's (a NaN becomes +6: the multiply before it has already dropped a NaN's sign).
namespace ascq {
namespace {
template <typename T> struct Two;
template <> struct Two<__half> { using type = __half2; };
template <> struct Two<__nv_bfloat16> { using type = __nv_bfloat162; };
__device__ __forceinline__ uint32_t bf16x2_to_e2m1x2(uint32_t b2)
{
    unsigned short r;
    asm("{ .reg .b8 t;\n cvt.rn.satfinite.e2m1x2.f32 t, %2, %1;\n mov.b16 %0, {t, 0}; }"
        : "=h"(r) : "f"(__uint_as_float(b2 << 16)), "f"(__uint_as_float(b2 & 0xFFFF0000u)));
    return r;
}
template <typename CT, typename T> __device__ __forceinline__ CT to_ct(T v)
{
    if constexpr (std::is_same<CT, T>::value) return v;
    else return Ct<CT>::from_f32(to_f32<T>(v));
}
template <typename Src, typename Sc, typename CT>
__global__ void __launch_bounds__(256) quant_fp4_kernel(uint8_t* __restrict__ dst, const Src* __restrict__ src, const SRef scale,
                                                        uint32_t rows, uint32_t cols)
{
    const uint32_t c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8u;
    if (c0 >= cols) return;
    constexpr int U = 2;
    const bool perLane = scale.cdiv != 1;  // groups along the columns: the lane's 8 elements share one scale
    const uint32_t scol = perLane ? c0 / scale.cdiv : c0;
    const uint32_t gy = gridDim.y;
    for (uint32_t r0 = blockIdx.y; r0 < rows; r0 += gy * U) {
        Pack<Src, 8> in[U];
        Pack<Sc, 8> sv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t r = r0 + u * gy;
            if (r >= rows) break;
            in[u] = load_pack<Src, 8, true>(src + static_cast<size_t>(r) * cols + c0);
            const Sc* sp = static_cast<const Sc*>(scale.p) + static_cast<size_t>(r / scale.rdiv) * scale.stride + scol;
            if (perLane) sv[u].v[0] = __ldg(sp);
            else sv[u] = load_pack<Sc, 8, false>(sp);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t r = r0 + u * gy;
            if (r >= rows) break;
            uint32_t word = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t b2;  // the two products as bfloat16
                if constexpr (std::is_same<CT, Src>::value && std::is_same<CT, Sc>::value && sizeof(CT) == 2) {
                    // half or bfloat16 throughout: one packed multiply (each lane rounded on its own)
                    using CT2 = typename Two<CT>::type;
                    CT2 x2, s2;
                    x2.x = in[u].v[2 * j]; x2.y = in[u].v[2 * j + 1];
                    s2.x = sv[u].v[perLane ? 0 : 2 * j]; s2.y = sv[u].v[perLane ? 0 : 2 * j + 1];
                    const CT2 y2 = __hmul2(x2, s2);
                    if constexpr (std::is_same<CT, __nv_bfloat16>::value) {
                        b2 = *reinterpret_cast<const uint32_t*>(&y2);
                    } else {
                        const float2 f = __half22float2(y2);
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(b2) : "f"(f.y), "f"(f.x));
                    }
                } else {
                    const CT s0 = to_ct<CT>(sv[u].v[perLane ? 0 : 2 * j]), s1 = to_ct<CT>(sv[u].v[perLane ? 0 : 2 * j + 1]);
                    const float y0 = Ct<CT>::to_f32(Ct<CT>::mul(to_ct<CT>(in[u].v[2 * j]), s0));
                    const float y1 = Ct<CT>::to_f32(Ct<CT>::mul(to_ct<CT>(in[u].v[2 * j + 1]), s1));
                    // a product beyond bfloat16's range becomes an infinity here and +-6 in the next step, as it would
                    // after saturating to the largest bfloat16 first
                    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(b2) : "f"(y1), "f"(y0));
                }
                word |= bf16x2_to_e2m1x2(b2) << (8 * j);
            }
            *reinterpret_cast<uint32_t*>(dst + (static_cast<size_t>(r) * cols + c0) / 2) = word;
        }
    }
}
template <typename Src, typename Sc, typename CT>
ascq_status launch_quant_fp4(const EwArgs& a, cudaStream_t st)
{
    dim3 grid, block;
    ew_grid(a.rows, a.cols, 8, &grid, &block);
    quant_fp4_kernel<Src, Sc, CT><<<grid, block, 0, st>>>(static_cast<uint8_t*>(a.dst), static_cast<const Src*>(a.src), a.scale, a.rows, a.cols);
    ASCQ_CUDA_CHECK(cudaGetLastError());
    return ASCQ_OK;
}
// (src, scale, compute) type triples of the PER_GROUP overloads: compute = scale type (legacy) or float (unified)
ascq_status dispatch_quant_fp4(const EwArgs& a, ascq_dtype srcT, ascq_dtype scT, ascq_dtype ct, cudaStream_t st, bool* handled)
{
    *handled = true;
    if (srcT == ASCQ_DT_F16 && scT == ASCQ_DT_F16 && ct == ASCQ_DT_F16) return launch_quant_fp4<__half, __half, __half>(a, st);
    if (srcT == ASCQ_DT_BF16 && scT == ASCQ_DT_BF16 && ct == ASCQ_DT_BF16) return launch_quant_fp4<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(a, st);
    if (srcT == ASCQ_DT_F16 && scT == ASCQ_DT_F16 && ct == ASCQ_DT_F32) return launch_quant_fp4<__half, __half, float>(a, st);
    if (srcT == ASCQ_DT_BF16 && scT == ASCQ_DT_BF16 && ct == ASCQ_DT_F32) return launch_quant_fp4<__nv_bfloat16, __nv_bfloat16, float>(a, st);
    if (srcT == ASCQ_DT_F16 && scT == ASCQ_DT_F32 && ct == ASCQ_DT_F32) return launch_quant_fp4<__half, float, float>(a, st);
    if (srcT == ASCQ_DT_BF16 && scT == ASCQ_DT_F32 && ct == ASCQ_DT_F32) return launch_quant_fp4<__nv_bfloat16, float, float>(a, st);
    if (srcT == ASCQ_DT_F32 && scT == ASCQ_DT_F32 && ct == ASCQ_DT_F32) return launch_quant_fp4<float, float, float>(a, st);
    *handled = false;
    return ASCQ_OK;
}
}  // namespace
}  // namespace ascq

static ascq_status quant_common(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT, const void* scale,
                                const void* offset, ascq_dtype scaleT, float scaleScalar, float offsetScalar,
                                ascq_policy policy, const ascq_quant_param* p, void* stream, bool unified)
{
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!dst || !src || !p) return fail(ASCQ_ERR_INVALID_ARG, "dst, src and param must not be NULL");
    if (policy == ASCQ_PER_CHANNEL_PER_GROUP || policy == ASCQ_PER_TOKEN_PER_GROUP)
        return fail(ASCQ_ERR_UNSUPPORTED, "unsupported policy for AscendQuant in current device!");
    if (policy < ASCQ_PER_TENSOR || policy > ASCQ_PER_GROUP) return fail(ASCQ_ERR_INVALID_ARG, "unknown policy %d", (int)policy);
    if (!is_float_type(srcT)) return fail(ASCQ_ERR_UNSUPPORTED, "AscendQuant only supports half/float/bfloat16_t input dtype");
    if (dstT != ASCQ_DT_I8 && dstT != ASCQ_DT_FP4X2_E2M1)
        return fail(ASCQ_ERR_UNSUPPORTED, "AscendQuant destination dtype %d is not built (int8 and fp4x2_e2m1 are)", (int)dstT);
    if (dst == src) return fail(ASCQ_ERR_INVALID_ARG, "src and dst must not overlap");

    EwArgs a{};
    a.src = src;
    a.dst = dst;
    a.roundMode = kRoundRint;
    int smode = kSScalar;
    bool hasOff = true;
    ascq_dtype ct = ASCQ_DT_F16;

    if (unified) {
        if (!is_float_type(scaleT)) return fail(ASCQ_ERR_UNSUPPORTED, "Quantize only support half/float/bfloat16_t scale dtype");
        if (scaleT != ASCQ_DT_F32 && scaleT != srcT)
            return fail(ASCQ_ERR_UNSUPPORTED, "Failed to check data type for Quantize: (src, scale) must be (T, T) or (T, float)");
        if (p->roundMode < ASCQ_CAST_NONE || p->roundMode > ASCQ_CAST_TRUNC)
            return fail(ASCQ_ERR_INVALID_ARG, "unknown roundMode %d", (int)p->roundMode);
        ct = ASCQ_DT_F32;
        hasOff = p->hasOffset != 0;
        a.roundMode = static_cast<int>(p->roundMode);
    }
    if (policy == ASCQ_PER_TENSOR) {
        if (dstT != ASCQ_DT_I8) return fail(ASCQ_ERR_UNSUPPORTED, "per-tensor AscendQuant writes int8 only");
        if (scale || offset) return fail(ASCQ_ERR_INVALID_ARG, "per-tensor AscendQuant takes scalar scale/offset; tensors must be NULL");
        a.scale.scalar = scaleScalar;
        a.offset.scalar = offsetScalar;
        a.rows = 1;
        a.cols = p->calCount;
        a.srcStride = a.dstStride = p->calCount;
    } else {
        if (p->n == 0) return fail(ASCQ_ERR_INVALID_ARG, "n (scaleCount) must be greater than 0");
        if (p->calCount % p->n != 0)
            return fail(ASCQ_ERR_INVALID_ARG, "calCount is %u, which should be an integer multiple of n/scaleCount %u", p->calCount, p->n);
        if (!scale) return fail(ASCQ_ERR_INVALID_ARG, "scale tensor must not be NULL");
        a.rows = p->calCount / p->n;
        a.cols = p->n;
        a.srcStride = a.dstStride = p->n;
        if (policy == ASCQ_PER_CHANNEL) {
            if (dstT != ASCQ_DT_I8) return fail(ASCQ_ERR_UNSUPPORTED, "per-channel AscendQuant writes int8 only");
            if (!unified && scaleT != ASCQ_DT_F16 && scaleT != ASCQ_DT_F32)
                return fail(ASCQ_ERR_UNSUPPORTED, "per-channel scale dtype must be half or float");
            if (!unified && (static_cast<size_t>(p->n) * dtype_size(scaleT)) % 32 != 0)
                return fail(ASCQ_ERR_INVALID_ARG, "scaleCount is %u, which should be 32B aligned", p->n);
            smode = kSColVec;
            a.scale.p = scale; a.scale.rdiv = 0; a.scale.cdiv = 1; a.scale.stride = 0;
            a.offset = a.scale;
            a.offset.p = offset;  // NULL: scalar offset
            a.offset.scalar = offsetScalar;
        } else {
            if (!is_float_type(scaleT)) return fail(ASCQ_ERR_UNSUPPORTED, "scale dtype must be half, bfloat16_t or float");
            if (scaleT != ASCQ_DT_F32 && scaleT != srcT)
                return fail(ASCQ_ERR_UNSUPPORTED, "unsupported (src, scale) dtype pair for AscendQuant PER_TOKEN/PER_GROUP");
            ct = unified ? ASCQ_DT_F32 : scaleT;
            hasOff = p->hasOffset != 0;
            if (hasOff && !offset) return fail(ASCQ_ERR_INVALID_ARG, "hasOffset is set but the offset tensor is NULL");
            if (p->roundMode < ASCQ_CAST_NONE || p->roundMode > ASCQ_CAST_TRUNC)
                return fail(ASCQ_ERR_INVALID_ARG, "unknown roundMode %d", (int)p->roundMode);
            a.roundMode = static_cast<int>(p->roundMode);
            ascq_status rc = policy_sref(&a.scale, scale, policy, p->n, p->groupSize, p->kDim, &smode);
            if (rc != ASCQ_OK) return rc;
            a.offset = a.scale;
            a.offset.p = offset;
            if (dstT == ASCQ_DT_FP4X2_E2M1) {
                if (policy != ASCQ_PER_GROUP) return fail(ASCQ_ERR_UNSUPPORTED, "fp4 destination needs PER_GROUP");
                if (hasOff) return fail(ASCQ_ERR_UNSUPPORTED, "AscendQuant to fp4 does not take an offset");
                if (p->n % 2) return fail(ASCQ_ERR_INVALID_ARG, "n must be even for a packed fp4 destination");
            }
        }
    }
    if (a.rows == 0 || a.cols == 0) return ASCQ_OK;

    constexpr int kVec = 16;
    if (dstT == ASCQ_DT_I8) {
        if (policy == ASCQ_PER_TENSOR) {
            // flat tensor: full rows of kVec*256 elements through the vector kernel, the tail through the scalar one
            const uint32_t width = kVec * 256;
            const uint32_t fullRows = (aligned16(src) && aligned16(dst)) ? p->calCount / width : 0;
            if (fullRows) {
                EwArgs b = a;
                b.rows = fullRows; b.cols = width; b.srcStride = b.dstStride = width;
                bool handled = false;
                ascq_status rc = dispatch_fast(b, srcT, scaleT, ct, smode, hasOff, st, &handled);
                if (rc != ASCQ_OK) return rc;
                if (!handled) return fail(ASCQ_ERR_UNSUPPORTED, "unsupported dtype combination");
            }
            const uint32_t done = fullRows * width;
            if (done == p->calCount) return ASCQ_OK;
            a.cols = p->calCount - done;
            GenericArgs g{};
            g.op = kOpQuant; g.srcT = srcT; g.dstT = dstT; g.scT = scaleT; g.ct = ct;
            g.src = src; g.dst = dst; g.rows = 1; g.cols = a.cols; g.srcStride = g.dstStride = a.cols;
            g.scale = a.scale; g.offset = a.offset; g.scaleIsScalar = 1; g.hasOff = hasOff; g.offIsScalar = 1;
            g.roundMode = a.roundMode; g.srcBase = g.dstBase = done;
            return launch_ew_generic(g, st);
        }
        if (ew_fast_ok(a, kVec, smode, dtype_size(scaleT))) {
            bool handled = false;
            ascq_status rc = dispatch_fast(a, srcT, scaleT, ct, smode, hasOff, st, &handled);
            if (rc != ASCQ_OK || handled) return rc;
        } else {  // ragged width or unaligned tensors: the same types, one element per thread
            EwArgs b = a;
            b.scalarPath = 1;
            bool handled = false;
            ascq_status rc = dispatch_fast(b, srcT, scaleT, ct, smode, hasOff, st, &handled);
            if (rc != ASCQ_OK || handled) return rc;
        }
    }
    if (dstT == ASCQ_DT_FP4X2_E2M1 && (a.roundMode == kRoundRint || a.roundMode == kRoundNone) && a.cols % 8 == 0 && aligned16(src) &&
        (reinterpret_cast<uintptr_t>(dst) & 3u) == 0 && a.scale.rdiv != 0 &&
        (a.scale.cdiv % 8 == 0 ? a.scale.cdiv != 0 : (a.scale.cdiv == 1 && aligned16(scale) && (a.cols * dtype_size(scaleT)) % 16 == 0))) {
        bool handled = false;
        ascq_status rc = dispatch_quant_fp4(a, srcT, scaleT, ct, st, &handled);
        if (rc != ASCQ_OK || handled) return rc;
    }
    GenericArgs g{};
    g.op = kOpQuant; g.srcT = srcT; g.dstT = dstT; g.scT = scaleT; g.ct = ct;
    g.src = src; g.dst = dst; g.rows = a.rows; g.cols = a.cols; g.srcStride = a.srcStride; g.dstStride = a.dstStride;
    g.scale = a.scale; g.offset = a.offset;
    g.scaleIsScalar = (smode == kSScalar);
    g.hasOff = hasOff;
    g.offIsScalar = (smode == kSScalar) || (policy == ASCQ_PER_CHANNEL && !offset);
    g.roundMode = a.roundMode;
    return launch_ew_generic(g, st);
}

extern "C" ascq_status ascq_quant(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT, const void* scale,
                                  const void* offset, ascq_dtype scaleT, float scaleScalar, float offsetScalar,
                                  ascq_policy policy, const ascq_quant_param* p, void* stream)
{
    return quant_common(dst, dstT, src, srcT, scale, offset, scaleT, scaleScalar, offsetScalar, policy, p, stream, false);
}

extern "C" ascq_status ascq_quantize(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT, const void* scale,
                                     const void* offset, ascq_dtype scaleT, float scaleScalar, float offsetScalar,
                                     ascq_policy policy, const ascq_quantize_param* qp, void* stream)
{
    if (!qp) return fail(ASCQ_ERR_INVALID_ARG, "dst, src and param must not be NULL");
    if (policy < ASCQ_PER_TENSOR || policy > ASCQ_PER_GROUP)
        return fail(ASCQ_ERR_UNSUPPORTED, "unsupported policy for Quantize in current device!");
    const uint64_t total = static_cast<uint64_t>(qp->m) * qp->n;
    if (total > 0xFFFFFFFFull) return fail(ASCQ_ERR_INVALID_ARG, "m * n does not fit 32 bits");
    ascq_quant_param p{qp->m, qp->n, static_cast<uint32_t>(total), qp->groupSize, qp->hasOffset, qp->kDim, qp->roundMode};
    return quant_common(dst, dstT, src, srcT, scale, offset, scaleT, scaleScalar, offsetScalar, policy, &p, stream, true);
}

// ---- dynamic per-token quantisation -------------------------------------------------------------
namespace ascq {
namespace {

template <typename Src> __device__ __forceinline__ float absmax8(const Pack<Src, 8>& v)
{
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(to_f32<Src>(v.v[i])));
    return m;
}

// One CTA per row.  Pass 1 streams the row (8 elements per thread per step) and reduces |x| with
// warp shuffles, then across the CTA's warps through shared memory; pass 2 writes int8.  RES > 0: the row has at
// most RES * 2048 elements and stays in the threads' registers between the passes (one read of the source);
// otherwise pass 2 re-reads it (it is L2 resident: a row is at most a few hundred KB).
template <typename Src, int RES> __global__ void __launch_bounds__(256) dyn_quant_kernel(int8_t* __restrict__ dst,
                                                                                float* __restrict__ scaleOut,
                                                                                float* __restrict__ deqOut,
                                                                                const Src* __restrict__ src,
                                                                                uint32_t n, int vecOk)
{
    __shared__ float warpMax[8];
    __shared__ float rowScale;
    const uint32_t r = blockIdx.x;
    const Src* row = src + static_cast<size_t>(r) * n;
    int8_t* out = dst + static_cast<size_t>(r) * n;
    float m = 0.f;
    Pack<Src, 8> held[RES > 0 ? RES : 1];
    if constexpr (RES > 0) {
#pragma unroll
        for (int i = 0; i < RES; ++i) {
            const uint32_t c = (i * 256 + threadIdx.x) * 8;
            if (c < n) {
                held[i] = load_pack<Src, 8, true>(row + c);
                m = fmaxf(m, absmax8<Src>(held[i]));
            }
        }
    } else if (vecOk) {
        for (uint32_t c = threadIdx.x * 8; c < n; c += blockDim.x * 8) m = fmaxf(m, absmax8<Src>(load_pack<Src, 8, false>(row + c)));
    } else {
        for (uint32_t c = threadIdx.x; c < n; c += blockDim.x) m = fmaxf(m, fabsf(to_f32<Src>(row[c])));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
    if ((threadIdx.x & 31) == 0) warpMax[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        float w = (threadIdx.x < (blockDim.x >> 5)) ? warpMax[threadIdx.x] : 0.f;
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) w = fmaxf(w, __shfl_xor_sync(0xFFFFFFFFu, w, off));
        if (threadIdx.x == 0) {
            const float s = (w > 0.f) ? __fdiv_rn(127.0f, w) : 1.0f;
            rowScale = s;
            scaleOut[r] = s;
            if (deqOut) deqOut[r] = (w > 0.f) ? __fdiv_rn(w, 127.0f) : 1.0f;
        }
    }
    __syncthreads();
    const float s = rowScale;
    auto quant8 = [&](const Pack<Src, 8>& v, uint32_t c) {
        uint2 q;
        q.x = pack_i8x4_rni(__fmul_rn(to_f32<Src>(v.v[0]), s), __fmul_rn(to_f32<Src>(v.v[1]), s), __fmul_rn(to_f32<Src>(v.v[2]), s),
                            __fmul_rn(to_f32<Src>(v.v[3]), s));
        q.y = pack_i8x4_rni(__fmul_rn(to_f32<Src>(v.v[4]), s), __fmul_rn(to_f32<Src>(v.v[5]), s), __fmul_rn(to_f32<Src>(v.v[6]), s),
                            __fmul_rn(to_f32<Src>(v.v[7]), s));
        __stcs(reinterpret_cast<uint2*>(out + c), q);
    };
    if constexpr (RES > 0) {
#pragma unroll
        for (int i = 0; i < RES; ++i) {
            const uint32_t c = (i * 256 + threadIdx.x) * 8;
            if (c < n) quant8(held[i], c);
        }
    } else if (vecOk) {
        for (uint32_t c = threadIdx.x * 8; c < n; c += blockDim.x * 8) quant8(load_pack<Src, 8, true>(row + c), c);
    } else {
        for (uint32_t c = threadIdx.x; c < n; c += blockDim.x)
            out[c] = static_cast<int8_t>(f32_to_i8_sat(__fmul_rn(to_f32<Src>(row[c]), s), kRoundRint));
    }
}
}  // namespace
}  // namespace ascq

extern "C" ascq_status ascq_dynamic_quant_per_token(int8_t* dst, float* scaleOut, float* deqScaleOut, const void* src,
                                                    ascq_dtype srcT, uint32_t m, uint32_t n, void* stream)
{
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!dst || !scaleOut || !src) return fail(ASCQ_ERR_INVALID_ARG, "dst, scaleOut and src must not be NULL");
    if (!is_float_type(srcT)) return fail(ASCQ_ERR_UNSUPPORTED, "src dtype must be half, bfloat16_t or float");
    if (m == 0 || n == 0) return ASCQ_OK;
    const int vecOk = (n % 8 == 0) && aligned16(src) && ((reinterpret_cast<uintptr_t>(dst) & 7u) == 0);
    auto run = [&](auto tag) {
        using Src = decltype(tag);
        const Src* sp = static_cast<const Src*>(src);
        if (vecOk && n <= 2048u) dyn_quant_kernel<Src, 1><<<m, 256, 0, st>>>(dst, scaleOut, deqScaleOut, sp, n, vecOk);
        else if (vecOk && n <= 8192u) dyn_quant_kernel<Src, 4><<<m, 256, 0, st>>>(dst, scaleOut, deqScaleOut, sp, n, vecOk);
        else dyn_quant_kernel<Src, 0><<<m, 256, 0, st>>>(dst, scaleOut, deqScaleOut, sp, n, vecOk);
    };
    if (srcT == ASCQ_DT_F16) run(__half{});
    else if (srcT == ASCQ_DT_BF16) run(__nv_bfloat16{});
    else run(float{});
    ASCQ_CUDA_CHECK(cudaGetLastError());
    return ASCQ_OK;
}

// ---- dynamic MX-FP4 block quantisation ---------------------------------------------------------------
// Per block of 32 consecutive elements of a row: amax -> shared exponent -> E8M0 byte, then every value is scaled by the
// exact power of two and converted float -> bfloat16 (RINT) -> E2M1 (RINT, saturating; cvt.rn.satfinite.e2m1x2.f32), the
// conversion chain of AscendQuant's fp4 destination.
namespace ascq {
namespace {
// Two fp32 values -> one byte of two E2M1 codes (first value in the low nibble), round to nearest even, saturating.
__device__ __forceinline__ uint32_t f32x2_to_e2m1x2(float first, float second)
{
    unsigned short r;
    asm("{ .reg .b8 t;\n cvt.rn.satfinite.e2m1x2.f32 t, %2, %1;\n mov.b16 %0, {t, 0}; }" : "=h"(r) : "f"(first), "f"(second));
    return r;
}

// max that returns NaN when either operand is NaN
__device__ __forceinline__ float fmax_nan(float a, float b)
{
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

// One lane owns one 16-byte vector of the source (8 half / bfloat16 or 4 float elements); the 4 or 8 lanes that share
// a 32-element block combine their maxima with shuffles.  Every load, code store and scale store of a warp is
// contiguous.  U vectors per thread are requested before the first is worked on.
template <typename Src>
__global__ void __launch_bounds__(256) dyn_quant_mxfp4_kernel(uint8_t* __restrict__ dst, uint8_t* __restrict__ scaleOut,
                                                              const Src* __restrict__ src, uint64_t vectors)
{
    constexpr int EPL = 16 / static_cast<int>(sizeof(Src));  // elements per lane
    constexpr int LPB = 32 / EPL;                            // lanes per block
    constexpr int U = 4;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const uint32_t lane = threadIdx.x & 31u;
    for (uint64_t g0 = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g0 - lane < vectors; g0 += stride * U) {
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint64_t g = g0 + u * stride;
            raw[u] = g < vectors ? __ldcs(reinterpret_cast<const uint4*>(src) + g) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint64_t g = g0 + u * stride;
            if (g - lane >= vectors) break;  // uniform over the warp
            const uint32_t ws[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
            // largest magnitude of the lane's elements, NaN propagating (so that one test at the end finds NaN and infinity)
            float amax;
            if constexpr (sizeof(Src) == 2) {
                using Src2 = typename Two<Src>::type;
                Src2 mx = __habs2(*reinterpret_cast<const Src2*>(&ws[0]));
#pragma unroll
                for (int j = 1; j < 4; ++j) mx = __hmax2_nan(mx, __habs2(*reinterpret_cast<const Src2*>(&ws[j])));
                amax = fmax_nan(to_f32<Src>(mx.x), to_f32<Src>(mx.y));
            } else {
                amax = fmax_nan(fmax_nan(fabsf(__uint_as_float(ws[0])), fabsf(__uint_as_float(ws[1]))),
                                fmax_nan(fabsf(__uint_as_float(ws[2])), fabsf(__uint_as_float(ws[3]))));
            }
#pragma unroll
            for (int o = 1; o < LPB; o <<= 1) amax = fmax_nan(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
            const bool bad = !(amax <= 3.4028234663852886e38f);  // a NaN or an infinity in the block
            // shared exponent = floor(log2(amax)) - 2 (E2M1's largest exponent), clamped to the E8M0 range; all-zero blocks get 2^0
            int e = 0;
            if (amax > 0.f) {
                const int ex = static_cast<int>((__float_as_uint(amax) >> 23) & 0xFF);
                e = (ex == 0 ? -126 : ex - 127) - 2;  // subnormal amax: floor(log2) is below -126; -126 is close enough to clamp
                e = min(max(e, -127), 127);
            }
            // x * 2^-e is exact; the factor is split in two only when 2^-e itself is not a normal number (|e| > 126)
            const bool twoSteps = e > 126 || e < -127 + 1;
            const int h1 = twoSteps ? (-e) / 2 : -e, h2 = (-e) - h1;
            const uint32_t f1b = static_cast<uint32_t>(h1 + 127) << 23, f2b = static_cast<uint32_t>(h2 + 127) << 23;
            uint32_t word = 0;
            if constexpr (std::is_same<Src, __nv_bfloat16>::value) {
                // bfloat16 times a power of two is a bfloat16: the scaled values stay packed, no rounding step is needed
                const uint32_t s1 = (f1b >> 16) * 0x10001u, s2 = (f2b >> 16) * 0x10001u;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 y = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&ws[j]), *reinterpret_cast<const __nv_bfloat162*>(&s1));
                    if (twoSteps) y = __hmul2(y, *reinterpret_cast<const __nv_bfloat162*>(&s2));
                    const uint32_t b2 = *reinterpret_cast<const uint32_t*>(&y);
                    word |= f32x2_to_e2m1x2(__uint_as_float(b2 << 16), __uint_as_float(b2 & 0xFFFF0000u)) << (8 * j);
                }
            } else {
                const float f1 = __uint_as_float(f1b), f2 = __uint_as_float(f2b);
#pragma unroll
                for (int j = 0; j < EPL / 2; ++j) {
                    float y0, y1;
                    if constexpr (sizeof(Src) == 2) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&ws[j]));
                        y0 = f.x; y1 = f.y;
                    } else {
                        y0 = __uint_as_float(ws[2 * j]); y1 = __uint_as_float(ws[2 * j + 1]);
                    }
                    y0 = __fmul_rn(y0, f1); y1 = __fmul_rn(y1, f1);
                    if (twoSteps) { y0 = __fmul_rn(y0, f2); y1 = __fmul_rn(y1, f2); }
                    // scaled value -> bfloat16 (round to nearest even; |y| < 8, nothing to saturate) -> E2M1
                    uint32_t b2;
                    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(b2) : "f"(y1), "f"(y0));
                    word |= f32x2_to_e2m1x2(__uint_as_float(b2 << 16), __uint_as_float(b2 & 0xFFFF0000u)) << (8 * j);
                }
            }
            if (bad) word = 0;
            if (g < vectors) {
                if constexpr (EPL == 8) reinterpret_cast<uint32_t*>(dst)[g] = word;
                else reinterpret_cast<unsigned short*>(dst)[g] = static_cast<unsigned short>(word);
                if ((lane & (LPB - 1)) == 0) scaleOut[g / LPB] = static_cast<uint8_t>(bad ? 0xFFu : static_cast<uint32_t>(e + 127));
            }
        }
    }
}
}  // namespace
}  // namespace ascq

extern "C" ascq_status ascq_dynamic_quant_mxfp4(uint8_t* dst_fp4, uint8_t* scale_e8m0, const void* src, ascq_dtype srcT,
                                                uint32_t m, uint32_t n, void* stream)
{
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!dst_fp4 || !scale_e8m0 || !src) return fail(ASCQ_ERR_INVALID_ARG, "dst, scale and src must not be NULL");
    if (!is_float_type(srcT)) return fail(ASCQ_ERR_UNSUPPORTED, "src dtype must be half, bfloat16_t or float");
    if (n % 32 != 0) return fail(ASCQ_ERR_INVALID_ARG, "n is %u, which must be a multiple of the MX block size 32", n);
    if (!aligned16(src) || !aligned16(dst_fp4)) return fail(ASCQ_ERR_ALIGNMENT, "src and dst must be 16-byte aligned");
    const uint64_t blocks = static_cast<uint64_t>(m) * (n / 32);
    if (blocks == 0) return ASCQ_OK;
    // one lane per 16-byte source vector, four vectors per thread and pass; at most 16 CTAs of 256 threads per SM
    const uint64_t vectors = blocks * (srcT == ASCQ_DT_F32 ? 8u : 4u);
    const uint64_t want = (vectors + 1023) / 1024;
    const unsigned grid = static_cast<unsigned>(want < static_cast<unsigned>(ascq::sm_count()) * 16u ? want : static_cast<unsigned>(ascq::sm_count()) * 16u);
    if (srcT == ASCQ_DT_F16) dyn_quant_mxfp4_kernel<__half><<<grid, 256, 0, st>>>(dst_fp4, scale_e8m0, static_cast<const __half*>(src), vectors);
    else if (srcT == ASCQ_DT_BF16)
        dyn_quant_mxfp4_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(dst_fp4, scale_e8m0, static_cast<const __nv_bfloat16*>(src), vectors);
    else dyn_quant_mxfp4_kernel<float><<<grid, 256, 0, st>>>(dst_fp4, scale_e8m0, static_cast<const float*>(src), vectors);
    ASCQ_CUDA_CHECK(cudaGetLastError());
    return ASCQ_OK;
}

