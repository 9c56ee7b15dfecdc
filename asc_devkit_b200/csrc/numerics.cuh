// Device-side numeric primitives with the rounding / saturation rules of the Ascend C vector unit:
//   - every arithmetic step is one correctly rounded IEEE operation (never contracted into an FMA);
//   - casts round to nearest even unless a round mode says otherwise and saturate on overflow
//     (docs/zh/api/SIMD-API/基础API/数据结构/precision_conversion.md:15-30).
#ifndef ASCQ_NUMERICS_CUH_
#define ASCQ_NUMERICS_CUH_

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace ascq {

enum : int { kRoundNone = 0, kRoundRint = 1, kRoundFloor = 2, kRoundCeil = 3, kRoundRound = 4, kRoundTrunc = 5 };

// float -> half, RINT; finite overflow saturates to +-65504.
__device__ __forceinline__ __half f32_to_f16_sat(float f)
{
    __half h = __float2half_rn(f);
    const unsigned short b = __half_as_ushort(h);
    if ((b & 0x7FFFu) == 0x7C00u && fabsf(f) != INFINITY) h = __ushort_as_half((b & 0x8000u) | 0x7BFFu);
    return h;
}
// float -> bf16, RINT; finite overflow saturates to the largest finite bf16.
__device__ __forceinline__ __nv_bfloat16 f32_to_bf16_sat(float f)
{
    __nv_bfloat16 h = __float2bfloat16_rn(f);
    const unsigned short b = __bfloat16_as_ushort(h);
    if ((b & 0x7FFFu) == 0x7F80u && fabsf(f) != INFINITY) h = __ushort_as_bfloat16((b & 0x8000u) | 0x7F7Fu);
    return h;
}

__device__ __forceinline__ float round_by_mode(float v, int mode)
{
    switch (mode) {
        case kRoundFloor: return floorf(v);
        case kRoundCeil: return ceilf(v);
        case kRoundRound: return roundf(v);  // half away from zero
        case kRoundTrunc: return truncf(v);
        default: return rintf(v);            // half to even
    }
}
// round, then clamp to [-128, 127]; NaN gives 0.
__device__ __forceinline__ int f32_to_i8_sat(float v, int mode)
{
    if (v != v) return 0;
    const float r = round_by_mode(v, mode);
    return static_cast<int>(fminf(fmaxf(r, -128.f), 127.f));
}

// E2M1 code (low 4 bits) -> float.
__device__ __forceinline__ float e2m1_to_f32(uint32_t code)
{
    // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6
    const uint32_t mag = code & 7u;
    float v = (mag < 2u) ? 0.5f * static_cast<float>(mag)
                         : __uint_as_float(((126u + (mag >> 1)) << 23) | ((mag & 1u) << 22));
    return (code & 8u) ? -v : v;
}
// E8M0 scale byte -> bf16 bits: e << 7, with 0x00 -> 2^-127 and 0xFF -> NaN.
__device__ __forceinline__ unsigned short e8m0_to_bf16_bits(uint32_t e)
{
    if (e == 0u) return 0x0040u;
    if (e == 0xFFu) return 0x7FFFu;
    return static_cast<unsigned short>(e << 7);
}
// float (already a bf16 value) -> E2M1 code with round mode and saturation to +-6.
__device__ __forceinline__ uint32_t f32_to_e2m1(float f, int mode)
{
    const uint32_t sign = (__float_as_uint(f) >> 31) ? 8u : 0u;
    const float a = fabsf(f);
    if (!(a < 6.0f)) return sign | 7u;  // also NaN
    // candidates: lo = largest code magnitude <= a
    const float mags[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    int lo = 0;
#pragma unroll
    for (int i = 1; i < 7; ++i)
        if (a >= mags[i]) lo = i;
    const int hi = lo + 1;
    const float dl = a - mags[lo], dh = mags[hi] - a;
    int pick;
    if (dl == 0.0f) pick = lo;
    else if (mode == kRoundFloor) pick = sign ? hi : lo;
    else if (mode == kRoundCeil) pick = sign ? lo : hi;
    else if (mode == kRoundTrunc) pick = lo;
    else if (mode == kRoundRound) pick = (dh <= dl) ? hi : lo;
    else pick = (dl < dh) ? lo : (dh < dl) ? hi : ((lo & 1) ? hi : lo);
    return sign | static_cast<uint32_t>(pick);
}

// ---- packed conversions used by the vector kernels -------------------------------------------------
// Two floats -> packed bf16x2 / f16x2 (RINT) in one instruction; the saturation rule (finite overflow ->
// largest finite value, Inf and NaN kept) is applied only when a lane came out as Inf/NaN, which is rare.
__device__ __forceinline__ uint32_t pack_bf16x2_sat(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    const uint32_t t = r & 0x7F807F80u;
    if (__builtin_expect(t >= 0x7F800000u || (t & 0xFFFFu) == 0x7F80u, 0)) {
        r = static_cast<uint32_t>(__bfloat16_as_ushort(f32_to_bf16_sat(lo))) |
            (static_cast<uint32_t>(__bfloat16_as_ushort(f32_to_bf16_sat(hi))) << 16);
    }
    return r;
}
__device__ __forceinline__ uint32_t pack_f16x2_sat(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    const uint32_t t = r & 0x7C007C00u;
    if (__builtin_expect(t >= 0x7C000000u || (t & 0xFFFFu) == 0x7C00u, 0)) {
        r = static_cast<uint32_t>(__half_as_ushort(f32_to_f16_sat(lo))) |
            (static_cast<uint32_t>(__half_as_ushort(f32_to_f16_sat(hi))) << 16);
    }
    return r;
}
// Four floats -> four saturated int8 in one word, round-half-even: cvt.rni.s32.f32 clamps to int32 and
// turns NaN into 0; cvt.pack.sat.s8.s32 clamps to [-128, 127] while packing.
__device__ __forceinline__ uint32_t pack_i8x4_rni(float x0, float x1, float x2, float x3)
{
    int a, b, c, d;
    asm("cvt.rni.s32.f32 %0, %1;" : "=r"(a) : "f"(x0));
    asm("cvt.rni.s32.f32 %0, %1;" : "=r"(b) : "f"(x1));
    asm("cvt.rni.s32.f32 %0, %1;" : "=r"(c) : "f"(x2));
    asm("cvt.rni.s32.f32 %0, %1;" : "=r"(d) : "f"(x3));
    uint32_t hi, r;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));
    return r;
}
// Two fp32 lanes per instruction (add.f32x2 / mul.f32x2: each lane rounded on its own, no flush to zero), which
// halves the issue slots the fp32 paths need.
__device__ __forceinline__ void add2_rn(float& x0, float& x1, float b0, float b1)
{
    asm("{\n\t.reg .b64 a, b, d;\n\tmov.b64 a, {%0, %1};\n\tmov.b64 b, {%2, %3};\n\tadd.rn.f32x2 d, a, b;\n\tmov.b64 {%0, %1}, d;\n\t}"
        : "+f"(x0), "+f"(x1)
        : "f"(b0), "f"(b1));
}
__device__ __forceinline__ void mul2_rn(float& x0, float& x1, float b0, float b1)
{
    asm("{\n\t.reg .b64 a, b, d;\n\tmov.b64 a, {%0, %1};\n\tmov.b64 b, {%2, %3};\n\tmul.rn.f32x2 d, a, b;\n\tmov.b64 {%0, %1}, d;\n\t}"
        : "+f"(x0), "+f"(x1)
        : "f"(b0), "f"(b1));
}
// Four int8 of one word -> four floats without the conversion pipe: byte ^ 0x80 placed in the mantissa
// of 2^23 gives 2^23 + (v + 128); subtracting 2^23 + 128 is exact.
__device__ __forceinline__ void unpack_i8x4_f32(uint32_t w, float (&f)[4])
{
    const uint32_t b = w ^ 0x80808080u;
    f[0] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7650));
    f[1] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7651));
    f[2] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7652));
    f[3] = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7653));
    add2_rn(f[0], f[1], -8388736.0f, -8388736.0f);
    add2_rn(f[2], f[3], -8388736.0f, -8388736.0f);
}

// ---- compute-type algebra: CT in {__half, __nv_bfloat16, float} ------------------------------
template <typename CT> struct Ct;
template <> struct Ct<float> {
    static __device__ __forceinline__ float from_f32(float v) { return v; }
    static __device__ __forceinline__ float to_f32(float v) { return v; }
    static __device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
    static __device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
};
template <> struct Ct<__half> {
    static __device__ __forceinline__ __half from_f32(float v) { return f32_to_f16_sat(v); }
    static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half mul(__half a, __half b) { return __hmul_rn(a, b); }
    static __device__ __forceinline__ __half add(__half a, __half b) { return __hadd_rn(a, b); }
};
template <> struct Ct<__nv_bfloat16> {
    // products of two bf16 are exact in fp32 and a sum rounded to fp32 then to bf16 equals the
    // directly rounded sum, so fp32 intermediates give the correctly rounded bf16 result.
    static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return f32_to_bf16_sat(v); }
    static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 mul(__nv_bfloat16 a, __nv_bfloat16 b)
    {
        return __float2bfloat16_rn(__fmul_rn(__bfloat162float(a), __bfloat162float(b)));
    }
    static __device__ __forceinline__ __nv_bfloat16 add(__nv_bfloat16 a, __nv_bfloat16 b)
    {
        return __float2bfloat16_rn(__fadd_rn(__bfloat162float(a), __bfloat162float(b)));
    }
};

// ---- storage-type loads as float (all exact) -------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<int8_t>(int8_t v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float to_f32<int32_t>(int32_t v) { return __int2float_rn(v); }
// AscendDequant's uint64 scale keeps the fp32 bit pattern in its low word.
template <> __device__ __forceinline__ float to_f32<uint64_t>(uint64_t v)
{
    return __uint_as_float(static_cast<uint32_t>(v & 0xFFFFFFFFull));
}

}  // namespace ascq
#endif  // ASCQ_NUMERICS_CUH_
