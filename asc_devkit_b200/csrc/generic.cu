// Runtime-typed, one-element-per-thread kernel: the catch-all for shapes and pointers the vector
// kernel cannot take (ragged extents, unaligned bases, odd group sizes) and for the 4-bit formats.
// Same arithmetic, one element at a time; correctness first, bandwidth second.
#include "elementwise.cuh"

namespace ascq {
namespace {

__device__ __forceinline__ float load_any_f32(const void* p, int dt, size_t i)
{
    switch (dt) {
        case ASCQ_DT_F16: return __half2float(static_cast<const __half*>(p)[i]);
        case ASCQ_DT_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
        case ASCQ_DT_F32: return static_cast<const float*>(p)[i];
        case ASCQ_DT_I8: return static_cast<float>(static_cast<const int8_t*>(p)[i]);
        case ASCQ_DT_I4X2: {  // int4b_t: two signed 4-bit values per byte, the even element in the low nibble
            const uint32_t byte = static_cast<const uint8_t*>(p)[i >> 1];
            const int32_t nib = static_cast<int32_t>((i & 1) ? (byte >> 4) : (byte & 0xFu));
            return static_cast<float>((nib ^ 8) - 8);
        }
        case ASCQ_DT_I32: return __int2float_rn(static_cast<const int32_t*>(p)[i]);
        case ASCQ_DT_U64: return to_f32<uint64_t>(static_cast<const uint64_t*>(p)[i]);
        default: return 0.f;
    }
}
__device__ __forceinline__ float sref_get(const SRef& s, int isScalar, int dt, uint32_t r, uint32_t c)
{
    if (isScalar) return s.scalar;
    const size_t idx = static_cast<size_t>(s.rdiv ? r / s.rdiv : 0u) * s.stride + (s.cdiv ? c / s.cdiv : 0u);
    return load_any_f32(s.p, dt, idx);
}
__device__ __forceinline__ void store_any(void* p, int dt, size_t i, float v)
{
    if (dt == ASCQ_DT_F32) static_cast<float*>(p)[i] = v;
    else if (dt == ASCQ_DT_BF16) static_cast<__nv_bfloat16*>(p)[i] = f32_to_bf16_sat(v);
    else static_cast<__half*>(p)[i] = f32_to_f16_sat(v);
}

// One element of quant / dequant / antiquant in compute type CT; returns the CT result as float
// (exact) -- the caller converts to the destination.
template <typename CT> __device__ __forceinline__ float compute_one(const GenericArgs& g, uint32_t r, uint32_t c, float xin)
{
    CT x = Ct<CT>::from_f32(xin);
    const CT s = Ct<CT>::from_f32(sref_get(g.scale, g.scaleIsScalar, g.scT, r, c));
    CT o = Ct<CT>::from_f32(0.f);
    if (g.hasOff) o = Ct<CT>::from_f32(sref_get(g.offset, g.offIsScalar, g.scT, r, c));
    if (g.op == kOpQuant) {
        x = Ct<CT>::mul(x, s);
        if (g.hasOff) x = Ct<CT>::add(x, o);
    } else if (g.op == kOpDequant) {
        x = Ct<CT>::mul(x, s);
        if (g.tok) x = Ct<CT>::mul(x, Ct<CT>::from_f32(g.tok[r]));
    } else {
        if (g.hasOff) x = Ct<CT>::add(x, o);
        x = Ct<CT>::mul(x, s);
    }
    return Ct<CT>::to_f32(x);
}
__device__ __forceinline__ float compute_any(const GenericArgs& g, uint32_t r, uint32_t c, float xin)
{
    if (g.ct == ASCQ_DT_F16) return compute_one<__half>(g, r, c, xin);
    if (g.ct == ASCQ_DT_BF16) return compute_one<__nv_bfloat16>(g, r, c, xin);
    return compute_one<float>(g, r, c, xin);
}

__global__ void __launch_bounds__(256) ew_generic_kernel(const GenericArgs g)
{
    const bool fp4dst = g.dstT == ASCQ_DT_FP4X2_E2M1;
    const bool fp4src = g.srcT == ASCQ_DT_FP4X2_E2M1;
    const uint32_t step = fp4dst ? 2u : 1u;  // a thread owns a whole destination byte
    const size_t units = static_cast<size_t>(g.rows) * (g.cols / step);
    for (size_t u = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; u < units;
         u += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t r = static_cast<uint32_t>(u / (g.cols / step));
        const uint32_t c = static_cast<uint32_t>(u % (g.cols / step)) * step;
        const size_t si = g.srcBase + static_cast<size_t>(r) * g.srcStride + c;
        const size_t di = g.dstBase + static_cast<size_t>(r) * g.dstStride + c;
        if (fp4src) {
            // MX decode: bf16(e2m1) * bf16(2^(e-127)), or both cast to half first for a half result.
            const uint8_t byte = static_cast<const uint8_t*>(g.src)[si >> 1];
            const uint32_t code = (si & 1) ? (byte >> 4) : (byte & 0x0Fu);
            const size_t sidx = g.fp4Transposed ? static_cast<size_t>(r) * (g.cols / 32) + c / 32
                                                : static_cast<size_t>(r / 32) * g.cols + c;
            const __nv_bfloat16 sb = __ushort_as_bfloat16(e8m0_to_bf16_bits(static_cast<const uint8_t*>(g.scale.p)[sidx]));
            const __nv_bfloat16 vb = __float2bfloat16_rn(e2m1_to_f32(code));
            if (g.dstT == ASCQ_DT_BF16) static_cast<__nv_bfloat16*>(g.dst)[di] = Ct<__nv_bfloat16>::mul(sb, vb);
            else static_cast<__half*>(g.dst)[di] =
                    __hmul_rn(f32_to_f16_sat(__bfloat162float(sb)), f32_to_f16_sat(__bfloat162float(vb)));
            continue;
        }
        const float y0 = compute_any(g, r, c, load_any_f32(g.src, g.srcT, si));
        if (g.dstT == ASCQ_DT_I8) {
            static_cast<int8_t*>(g.dst)[di] = static_cast<int8_t>(f32_to_i8_sat(y0, g.roundMode));
        } else if (fp4dst) {
            const float y1 = compute_any(g, r, c + 1, load_any_f32(g.src, g.srcT, si + 1));
            const uint32_t lo = f32_to_e2m1(__bfloat162float(f32_to_bf16_sat(y0)), g.roundMode);
            const uint32_t hi = f32_to_e2m1(__bfloat162float(f32_to_bf16_sat(y1)), g.roundMode);
            static_cast<uint8_t*>(g.dst)[di >> 1] = static_cast<uint8_t>(lo | (hi << 4));
        } else {
            store_any(g.dst, g.dstT, di, y0);
        }
    }
}
}  // namespace

ascq_status launch_ew_generic(const GenericArgs& g, cudaStream_t stream)
{
    const size_t step = g.dstT == ASCQ_DT_FP4X2_E2M1 ? 2 : 1;
    const size_t units = static_cast<size_t>(g.rows) * (g.cols / step);
    if (units == 0) return ASCQ_OK;
    size_t blocks = (units + 255) / 256;
    if (blocks > static_cast<unsigned>(ascq::sm_count()) * 16u) blocks = static_cast<unsigned>(ascq::sm_count()) * 16u;
    ew_generic_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(g);
    ASCQ_CUDA_CHECK(cudaGetLastError());
    return ASCQ_OK;
}

}  // namespace ascq
