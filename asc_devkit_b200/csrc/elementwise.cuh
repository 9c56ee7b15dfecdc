// Row-streaming elementwise kernel shared by AscendQuant / AscendDequant / AscendAntiQuant.
//
// Data layout in HBM: src is a row-major [rows, cols] matrix (row stride srcStride elements), dst
// likewise with dstStride.  One thread owns VEC consecutive columns (16 bytes of the narrower of the
// two element types) and walks down the rows blockIdx.y, blockIdx.y + gridDim.y, ...; a warp therefore
// reads and writes fully coalesced 128-bit segments.  Per-column scale/offset vectors are loaded once
// per thread and stay in registers; per-row (per-token / per-group) scales are one broadcast load per
// row.  src is read with ld.global.cs and dst written with st.global.cs (both are touched exactly
// once); scales go through the read-only path and stay cached.
//
// The roofline is HBM: algorithmic bytes = rows*cols*(sizeof(Src)+sizeof(Dst)) + the scale vectors.
#ifndef ASCQ_ELEMENTWISE_CUH_
#define ASCQ_ELEMENTWISE_CUH_

#include <cuda_runtime.h>

#include <cstdlib>

#include <type_traits>

#include "ascq_internal.h"
#include "numerics.cuh"
#include "tma_host.h"

namespace ascq {

enum : int { kOpQuant = 0, kOpDequant = 1, kOpAntiQuant = 2 };
// How a scale / offset operand is addressed for element (r, c):
enum : int {
    kSScalar = 0,   // one value for the whole tensor (passed by value)
    kSColVec = 1,   // p[c]                           -- per channel, row invariant
    kSRowBcast = 2, // p[(r/rdiv)*stride + c/cdiv]    -- one value per VEC columns (per token; groups along columns)
    kSRowVec = 3    // p[(r/rdiv)*stride + c]         -- groups along rows
};

struct SRef {
    const void* p;
    uint32_t rdiv, cdiv, stride;  // rdiv / cdiv == 0: the index does not depend on r / c
    float scalar;
};

struct EwArgs {
    const void* src;
    void* dst;
    uint32_t rows, cols, srcStride, dstStride;
    SRef scale, offset;
    const float* tok;  // dequant only: optional fp32 per-row multiplier applied after the scale
    int roundMode;
    int wide32;        // src / dst bases and row pitches are 32-byte aligned: 32-byte vectors move as one 256-bit access
    int scalarPath;    // ragged widths / unaligned tensors: one element per thread, same types and arithmetic
    int offsetIsScalar;  // set by the launcher: a scale tensor with a scalar offset (offset.p then aliases scale.p)
};

template <int BYTES> struct Chunk;
template <> struct Chunk<16> { using type = uint4; };
template <> struct Chunk<8> { using type = uint2; };
template <> struct Chunk<4> { using type = uint32_t; };

template <typename T, int N> struct alignas((sizeof(T) * N >= 16) ? 16 : sizeof(T) * N) Pack { T v[N]; };

template <typename T, int N, bool STREAM> __device__ __forceinline__ Pack<T, N> load_pack(const T* p)
{
    constexpr int BYTES = sizeof(T) * N;
    constexpr int CB = BYTES >= 16 ? 16 : BYTES;
    using C = typename Chunk<CB>::type;
    Pack<T, N> r;
    const C* q = reinterpret_cast<const C*>(p);
    C* o = reinterpret_cast<C*>(&r);
#pragma unroll
    for (int i = 0; i < BYTES / CB; ++i) o[i] = STREAM ? __ldcs(q + i) : __ldg(q + i);
    return r;
}
// 256-bit streaming accesses (sm_100): one instruction per 32-byte vector; the address must be 32-byte aligned.
__device__ __forceinline__ void ld_cs_256(const void* p, uint32_t (&a)[8])
{
    asm volatile("ld.global.cs.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7])
                 : "l"(p));
}
__device__ __forceinline__ void st_cs_256(void* p, const uint32_t (&a)[8])
{
    asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]),
                 "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7])
                 : "memory");
}
template <typename T, int N> __device__ __forceinline__ Pack<T, N> load_pack_wide(const T* p, bool wide)
{
    if constexpr (sizeof(T) * N == 32) {
        if (wide) {
            Pack<T, N> r;
            ld_cs_256(p, *reinterpret_cast<uint32_t(*)[8]>(&r));
            return r;
        }
    }
    return load_pack<T, N, true>(p);
}
template <typename T, int N> __device__ __forceinline__ void store_pack(T* p, const Pack<T, N>& r)
{
    constexpr int BYTES = sizeof(T) * N;
    constexpr int CB = BYTES >= 16 ? 16 : BYTES;
    using C = typename Chunk<CB>::type;
    C* q = reinterpret_cast<C*>(p);
    const C* o = reinterpret_cast<const C*>(&r);
#pragma unroll
    for (int i = 0; i < BYTES / CB; ++i) __stcs(q + i, o[i]);
}

template <typename T, int N> __device__ __forceinline__ void store_pack_wide(T* p, const Pack<T, N>& r, bool wide)
{
    if constexpr (sizeof(T) * N == 32) {
        if (wide) {
            st_cs_256(p, *reinterpret_cast<const uint32_t(*)[8]>(&r));
            return;
        }
    }
    store_pack<T, N>(p, r);
}

// int4b_t source: two signed 4-bit values per byte, the even element in the low nibble.  The tag stands for one byte;
// a thread's 16 elements are 8 source bytes, widened to sixteen int8 in registers right after the load, so that the
// rest of the kernel is the int8 one.
struct int4x2_t { uint8_t bits; };
template <typename Src> struct SrcValue { using type = Src; };
template <> struct SrcValue<int4x2_t> { using type = int8_t; };
// four nibbles (16 bits) -> four sign-extended bytes
__device__ __forceinline__ uint32_t widen_i4x4(uint32_t x)
{
    const uint32_t w = __byte_perm(x & 0x0F0Fu, (x >> 4) & 0x0F0Fu, 0x5140);  // bytes n0, n1, n2, n3
    return w | ((w & 0x08080808u) * 0x1Eu);                                   // bit 3 of each byte copied into bits 4..7
}
template <int VEC> __device__ __forceinline__ Pack<int8_t, VEC> load_i4_as_i8(const void* base, size_t elemIndex)
{
    static_assert(VEC == 16, "sixteen int4 elements = one 8-byte load");
    const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(base) + (elemIndex >> 1)));
    Pack<int8_t, VEC> r;
    uint32_t* w = reinterpret_cast<uint32_t*>(&r);
    w[0] = widen_i4x4(raw.x & 0xFFFFu);
    w[1] = widen_i4x4(raw.x >> 16);
    w[2] = widen_i4x4(raw.y & 0xFFFFu);
    w[3] = widen_i4x4(raw.y >> 16);
    return r;
}

template <typename Src, typename Dst> struct VecOf {
    static constexpr int kMin = sizeof(Src) < sizeof(Dst) ? sizeof(Src) : sizeof(Dst);
    static constexpr int value = 16 / kMin;
};

// Source vector -> compute type.
template <typename Src, typename CT, int VEC>
__device__ __forceinline__ void unpack_src(const Pack<Src, VEC>& in, CT (&x)[VEC])
{
    if constexpr (std::is_same<Src, int8_t>::value && std::is_same<CT, float>::value) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&in);
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
            float f[4];
            unpack_i8x4_f32(w[q], f);
#pragma unroll
            for (int j = 0; j < 4; ++j) x[q * 4 + j] = f[j];
        }
    } else if constexpr (std::is_same<Src, int8_t>::value && std::is_same<CT, __half>::value && (VEC % 4 == 0)) {
        // byte ^ 0x80 in the low byte of the half 1024.0 (0x6400) is 1024 + (v + 128); subtracting 1152 is exact
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&in);
        __half2* x2 = reinterpret_cast<__half2*>(x);
        const uint32_t bias = 0x64806480u;  // 1152.0 twice
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
            const uint32_t b = w[q] ^ 0x80808080u;
            const uint32_t lo = __byte_perm(b, 0x64646464u, 0x4140), hi = __byte_perm(b, 0x64646464u, 0x4342);
            x2[2 * q] = __hsub2(*reinterpret_cast<const __half2*>(&lo), *reinterpret_cast<const __half2*>(&bias));
            x2[2 * q + 1] = __hsub2(*reinterpret_cast<const __half2*>(&hi), *reinterpret_cast<const __half2*>(&bias));
        }
    } else if constexpr (std::is_same<Src, int8_t>::value && std::is_same<CT, __nv_bfloat16>::value && (VEC % 4 == 0)) {
        // through fp32 (no conversion pipe), then two exact narrowing conversions per instruction
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&in);
        __nv_bfloat162* x2 = reinterpret_cast<__nv_bfloat162*>(x);
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
            float f[4];
            unpack_i8x4_f32(w[q], f);
            x2[2 * q] = __floats2bfloat162_rn(f[0], f[1]);
            x2[2 * q + 1] = __floats2bfloat162_rn(f[2], f[3]);
        }
    } else if constexpr (std::is_same<Src, CT>::value) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) x[i] = in.v[i];
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) x[i] = Ct<CT>::from_f32(to_f32<Src>(in.v[i]));
    }
}

// Compute-type results -> destination vector (final cast: RINT + saturation, or the round mode for int8).
template <typename Dst, typename CT, int VEC>
__device__ __forceinline__ void pack_dst(const CT (&x)[VEC], Pack<Dst, VEC>& out, int roundMode)
{
    if constexpr (std::is_same<Dst, int8_t>::value) {
        uint32_t* w = reinterpret_cast<uint32_t*>(&out);
        if (roundMode <= kRoundRint) {
#pragma unroll
            for (int q = 0; q < VEC / 4; ++q)
                w[q] = pack_i8x4_rni(Ct<CT>::to_f32(x[q * 4]), Ct<CT>::to_f32(x[q * 4 + 1]), Ct<CT>::to_f32(x[q * 4 + 2]),
                                     Ct<CT>::to_f32(x[q * 4 + 3]));
        } else {
            // the other modes: round to an integral float first (one instruction for floor / ceil / trunc), then the
            // same saturating pack (NaN -> 0, out-of-range values clamp)
            auto packRounded = [&](auto rnd) {
#pragma unroll
                for (int q = 0; q < VEC / 4; ++q)
                    w[q] = pack_i8x4_rni(rnd(Ct<CT>::to_f32(x[q * 4])), rnd(Ct<CT>::to_f32(x[q * 4 + 1])), rnd(Ct<CT>::to_f32(x[q * 4 + 2])),
                                         rnd(Ct<CT>::to_f32(x[q * 4 + 3])));
            };
            if (roundMode == kRoundFloor) packRounded([](float v) { return floorf(v); });
            else if (roundMode == kRoundCeil) packRounded([](float v) { return ceilf(v); });
            else if (roundMode == kRoundTrunc) packRounded([](float v) { return truncf(v); });
            else packRounded([](float v) { return round_by_mode(v, kRoundRound); });
        }
    } else if constexpr (std::is_same<Dst, CT>::value) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) out.v[i] = x[i];
    } else if constexpr (std::is_same<Dst, __nv_bfloat16>::value) {
        uint32_t* w = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
        for (int q = 0; q < VEC / 2; ++q) w[q] = pack_bf16x2_sat(Ct<CT>::to_f32(x[2 * q]), Ct<CT>::to_f32(x[2 * q + 1]));
    } else if constexpr (std::is_same<Dst, __half>::value) {
        uint32_t* w = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
        for (int q = 0; q < VEC / 2; ++q) w[q] = pack_f16x2_sat(Ct<CT>::to_f32(x[2 * q]), Ct<CT>::to_f32(x[2 * q + 1]));
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) out.v[i] = Ct<CT>::to_f32(x[i]);
    }
}

// The arithmetic of one vector: quant x*s(+o), dequant x*s(*tok), antiquant (x+o)*s.  Half math runs two
// lanes per instruction (HMUL2 / HADD2, each lane individually rounded).
template <int OP, typename CT, int VEC, int SV, bool HAS_OFF, bool HAS_TOK>
__device__ __forceinline__ void apply_op(CT (&x)[VEC], const CT (&s)[SV], const CT (&o)[SV], float tok)
{
    constexpr bool kVecScale = SV != 1;
    if constexpr (std::is_same<CT, __half>::value && (VEC % 2 == 0)) {
        __half2* x2 = reinterpret_cast<__half2*>(x);
#pragma unroll
        for (int q = 0; q < VEC / 2; ++q) {
            const __half2 s2 = kVecScale ? __halves2half2(s[2 * q], s[2 * q + 1]) : __half2half2(s[0]);
            const __half2 o2 = kVecScale ? __halves2half2(o[2 * q], o[2 * q + 1]) : __half2half2(o[0]);
            __half2 v = x2[q];
            if constexpr (OP == kOpQuant) {
                v = __hmul2_rn(v, s2);
                if constexpr (HAS_OFF) v = __hadd2_rn(v, o2);
            } else if constexpr (OP == kOpDequant) {
                v = __hmul2_rn(v, s2);
            } else {
                if constexpr (HAS_OFF) v = __hadd2_rn(v, o2);
                v = __hmul2_rn(v, s2);
            }
            x2[q] = v;
        }
    } else if constexpr (std::is_same<CT, __nv_bfloat16>::value && (VEC % 2 == 0)) {
        // bfloat16 likewise (mul.rn.bf16x2 / add.rn.bf16x2: each lane is the exact result rounded once, which is what the
        // scalar form computes through fp32)
        __nv_bfloat162* x2 = reinterpret_cast<__nv_bfloat162*>(x);
#pragma unroll
        for (int q = 0; q < VEC / 2; ++q) {
            const __nv_bfloat162 s2 = kVecScale ? __halves2bfloat162(s[2 * q], s[2 * q + 1]) : __bfloat162bfloat162(s[0]);
            const __nv_bfloat162 o2 = kVecScale ? __halves2bfloat162(o[2 * q], o[2 * q + 1]) : __bfloat162bfloat162(o[0]);
            __nv_bfloat162 v = x2[q];
            if constexpr (OP == kOpQuant) {
                v = __hmul2_rn(v, s2);
                if constexpr (HAS_OFF) v = __hadd2_rn(v, o2);
            } else if constexpr (OP == kOpDequant) {
                v = __hmul2_rn(v, s2);
                if constexpr (HAS_TOK) v = __hmul2_rn(v, __bfloat162bfloat162(Ct<CT>::from_f32(tok)));
            } else {
                if constexpr (HAS_OFF) v = __hadd2_rn(v, o2);
                v = __hmul2_rn(v, s2);
            }
            x2[q] = v;
        }
    } else if constexpr (std::is_same<CT, float>::value && (VEC % 2 == 0)) {
#pragma unroll
        for (int q = 0; q < VEC / 2; ++q) {
            const int s0 = kVecScale ? 2 * q : 0, s1 = kVecScale ? 2 * q + 1 : 0;
            float& v0 = x[2 * q];
            float& v1 = x[2 * q + 1];
            if constexpr (OP == kOpQuant) {
                mul2_rn(v0, v1, s[s0], s[s1]);
                if constexpr (HAS_OFF) add2_rn(v0, v1, o[s0], o[s1]);
            } else if constexpr (OP == kOpDequant) {
                mul2_rn(v0, v1, s[s0], s[s1]);
                if constexpr (HAS_TOK) mul2_rn(v0, v1, tok, tok);
            } else {
                if constexpr (HAS_OFF) add2_rn(v0, v1, o[s0], o[s1]);
                mul2_rn(v0, v1, s[s0], s[s1]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const int si = kVecScale ? i : 0;
            CT v = x[i];
            if constexpr (OP == kOpQuant) {
                v = Ct<CT>::mul(v, s[si]);
                if constexpr (HAS_OFF) v = Ct<CT>::add(v, o[si]);
            } else if constexpr (OP == kOpDequant) {
                v = Ct<CT>::mul(v, s[si]);
                if constexpr (HAS_TOK) v = Ct<CT>::mul(v, Ct<CT>::from_f32(tok));
            } else {
                if constexpr (HAS_OFF) v = Ct<CT>::add(v, o[si]);
                v = Ct<CT>::mul(v, s[si]);
            }
            x[i] = v;
        }
    }
}

// Tuning constants (measured on config 2/3-sized and larger inputs): four resident CTAs per SM (at most 64
// registers per thread), two row batches in flight per thread, about sixteen CTAs per SM in the grid.
// Per-operator tuning: row batches in flight per thread and CTAs per SM in the grid.  The dequant operator reads
// 4-byte elements (two 16-byte loads per vector already) and does best with one batch and a finer grid.
#define ASCQ_EW_U_DEFAULT 2
template <int OP> struct EwTune {
    static constexpr int kRowsInFlight = ASCQ_EW_U_DEFAULT;
    static constexpr uint32_t kCtasPerSm = 16u;
    static constexpr bool kWide256 = false;  // 256-bit accesses measured no better (antiquant) or worse (quant)
};
template <> struct EwTune<1 /* kOpDequant */> {
    static constexpr int kRowsInFlight = 1;
    static constexpr uint32_t kCtasPerSm = 32u;
    static constexpr bool kWide256 = true;   // its 32-byte source vectors move as one 256-bit load
};
#ifndef ASCQ_EW_MINB
#define ASCQ_EW_MINB 4
#endif
#ifndef ASCQ_EW_TARGET
#define ASCQ_EW_TARGET 16u
#endif
// Resident CTAs per SM the register budget is set for: four (64 registers), or three (80) where a thread holds a vector
// of fp32 scales and one of fp32 offsets next to its data (quant: 32- or 64-byte source vectors) -- those spilled at 64.
template <int OP, typename CT, int SMODE, bool HAS_OFF> struct EwMinBlocks {
    static constexpr int value =
        (OP == kOpQuant && (SMODE == kSColVec || SMODE == kSRowVec) && HAS_OFF && sizeof(CT) == 4) ? 3 : ASCQ_EW_MINB;
};
template <int OP, typename Src, typename Dst, typename Sc, typename CT, int SMODE, bool HAS_OFF, bool HAS_TOK>
__global__ void __launch_bounds__(256, EwMinBlocks<OP, CT, SMODE, HAS_OFF>::value) ew_rows_kernel(const EwArgs a)
{
    constexpr int VEC = VecOf<Src, Dst>::value;
    constexpr bool kVecScale = (SMODE == kSColVec || SMODE == kSRowVec);
    constexpr int SV = kVecScale ? VEC : 1;
    // Programmatic dependent launch: the next launch on the stream may bring its CTAs onto the SMs while this one's last
    // rows drain, and this launch's CTAs were scheduled while its predecessor was still running -- nothing below touches
    // global memory before that predecessor has completed.  For kernels of 9 to 60 us the ramp and the tail of a launch are
    // a visible share; a stream of these operators (one per layer) then runs back to back.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t c0 = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (c0 >= a.cols) return;

    CT s[SV], o[SV];
    if constexpr (SMODE == kSScalar) {
        s[0] = Ct<CT>::from_f32(a.scale.scalar);
        o[0] = Ct<CT>::from_f32(a.offset.scalar);
    } else if constexpr (SMODE == kSColVec) {
        const Pack<Sc, VEC> sp = load_pack<Sc, VEC, false>(static_cast<const Sc*>(a.scale.p) + c0);
#pragma unroll
        for (int i = 0; i < VEC; ++i) s[i] = Ct<CT>::from_f32(to_f32<Sc>(sp.v[i]));
        if constexpr (HAS_OFF) {
            // offsetIsScalar: per-channel scale with a scalar offset; offset.p then holds the scale tensor's address, so
            // that the load below has a valid address even if it is scheduled ahead of the test
            if (!a.offsetIsScalar) {
                const Pack<Sc, VEC> op = load_pack<Sc, VEC, false>(static_cast<const Sc*>(a.offset.p) + c0);
#pragma unroll
                for (int i = 0; i < VEC; ++i) o[i] = Ct<CT>::from_f32(to_f32<Sc>(op.v[i]));
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) o[i] = Ct<CT>::from_f32(a.offset.scalar);
            }
        }
    }
    const uint32_t sc_col = a.scale.cdiv ? c0 / a.scale.cdiv : 0u;

    // Rows are taken U at a time: all U source vectors (and the per-row scalars) are requested before
    // the first result is stored, so every thread keeps U vector loads in flight.
    // Which rows: blockIdx.y + k * gridDim.y in general.  With a scale vector per group of rows (kSRowVec) a block takes a
    // run of consecutive rows instead, so that the vector (and its conversion to the compute type) is fetched once per
    // group and not once per row.
    // one row at a time where two vectors of fp32 parameters are held in registers
    constexpr int U = (SMODE == kSRowVec && HAS_OFF && sizeof(CT) == 4) ? 1 : EwTune<OP>::kRowsInFlight;
    const uint32_t gy = gridDim.y;
    uint32_t rStart = blockIdx.y, rStep = gy, rEnd = a.rows;
    if constexpr (SMODE == kSRowVec) {
        const uint32_t per = (a.rows + gy - 1) / gy;
        rStart = blockIdx.y * per;
        rStep = 1;
        rEnd = min(a.rows, rStart + per);
    }
    uint32_t heldGroup = 0xFFFFFFFFu;
    for (uint32_t r0 = rStart; r0 < rEnd; r0 += rStep * U) {
        using SrcV = typename SrcValue<Src>::type;
        Pack<SrcV, VEC> in[U];
        CT srow[U], orow[U];
        float tok[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t r = r0 + u * rStep;
            if (r < rEnd) {
                if constexpr (std::is_same<Src, int4x2_t>::value)
                    in[u] = load_i4_as_i8<VEC>(a.src, static_cast<size_t>(r) * a.srcStride + c0);
                else
                    in[u] = load_pack_wide<Src, VEC>(static_cast<const Src*>(a.src) + static_cast<size_t>(r) * a.srcStride + c0, a.wide32 != 0);
                if constexpr (SMODE == kSRowBcast) {
                    const size_t idx = static_cast<size_t>(a.scale.rdiv ? r / a.scale.rdiv : 0u) * a.scale.stride + sc_col;
                    srow[u] = Ct<CT>::from_f32(to_f32<Sc>(__ldg(static_cast<const Sc*>(a.scale.p) + idx)));
                    if constexpr (HAS_OFF)
                        orow[u] = Ct<CT>::from_f32(to_f32<Sc>(__ldg(static_cast<const Sc*>(a.offset.p) + idx)));
                }
                if constexpr (HAS_TOK) tok[u] = __ldg(a.tok + r);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t r = r0 + u * rStep;
            if (r >= rEnd) break;
            if constexpr (SMODE == kSRowBcast) {
                s[0] = srow[u];
                if constexpr (HAS_OFF) o[0] = orow[u];
            } else if constexpr (SMODE == kSRowVec) {
                const uint32_t group = a.scale.rdiv ? r / a.scale.rdiv : 0u;
                if (group != heldGroup) {
                heldGroup = group;
                const size_t idx = static_cast<size_t>(group) * a.scale.stride + c0;
                const Pack<Sc, VEC> sp = load_pack<Sc, VEC, false>(static_cast<const Sc*>(a.scale.p) + idx);
#pragma unroll
                for (int i = 0; i < VEC; ++i) s[i] = Ct<CT>::from_f32(to_f32<Sc>(sp.v[i]));
                if constexpr (HAS_OFF) {
                    const Pack<Sc, VEC> op = load_pack<Sc, VEC, false>(static_cast<const Sc*>(a.offset.p) + idx);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) o[i] = Ct<CT>::from_f32(to_f32<Sc>(op.v[i]));
                }
                }
            }
            alignas(4) CT x[VEC];
            unpack_src<SrcV, CT, VEC>(in[u], x);
            apply_op<OP, CT, VEC, SV, HAS_OFF, HAS_TOK>(x, s, o, HAS_TOK ? tok[u] : 1.0f);
            Pack<Dst, VEC> out;
            pack_dst<Dst, CT, VEC>(x, out, a.roundMode);
            store_pack_wide<Dst, VEC>(static_cast<Dst*>(a.dst) + static_cast<size_t>(r) * a.dstStride + c0, out, a.wide32 != 0);
        }
    }
}

// Launch with programmatic stream serialisation allowed (see the kernel's first lines); ASCQ_EW_NOPDL=1 launches plainly.
template <typename K> inline void launch_rows_kernel(K kernel, dim3 grid, dim3 block, cudaStream_t stream, const EwArgs& args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = getenv("ASCQ_EW_NOPDL") == nullptr ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, args);
}

// Grid shape: x covers the column vectors, y strides the rows; about ASCQ_EW_TARGET 256-thread CTAs per SM.
inline void ew_grid(uint32_t rows, uint32_t cols, int vec, dim3* grid, dim3* block, uint32_t ctasPerSm = ASCQ_EW_TARGET)
{
    const uint32_t nvec = (cols + vec - 1) / vec;
    auto waste = [nvec](uint32_t b) { return (nvec + b - 1) / b * b - nvec; };
    uint32_t bx = 256;  // narrower CTAs only when they idle clearly fewer threads on the last column block
    for (uint32_t cand : {128u, 64u})
        if (waste(cand) + nvec / 32 < waste(bx)) bx = cand;
    if (nvec < bx) bx = (nvec + 31) / 32 * 32;
    const uint32_t gx = (nvec + bx - 1) / bx;
    const uint32_t target = static_cast<uint32_t>(sm_count()) * ctasPerSm * 256u / bx;  // CTAs
    uint32_t gy = (target + gx - 1) / gx;
    if (gy > rows) gy = rows;
    if (gy < 1) gy = 1;
    if (gy > 65535u) gy = 65535u;
    *grid = dim3(gx, gy, 1);
    *block = dim3(bx, 1, 1);
}

// The same operators, one element per thread: for widths that are not a multiple of the vector, row pitches or
// pointers that are not 16-byte aligned.  Types are compile-time (the arithmetic is the vector kernel's, element by
// element).  SCALAR_PARAMS (one scale / offset for the whole tensor, passed by value) is a compile-time choice, so that
// the variant without parameter tensors contains no load from them at all; how the tensors are indexed otherwise is
// decided at run time, uniformly over the launch.
template <int OP, typename Src, typename Dst, typename Sc, typename CT, bool SCALAR_PARAMS, bool HAS_TOK>
__global__ void __launch_bounds__(256) ew_scalar_kernel(const EwArgs a, int hasOff)
{
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.cols) return;
    const Sc* sp = static_cast<const Sc*>(a.scale.p);
    const Sc* op = static_cast<const Sc*>(a.offset.p);
    const uint32_t sc_col = a.scale.cdiv ? c / a.scale.cdiv : 0u;
    constexpr int U = 4;
    for (uint32_t r0 = blockIdx.y; r0 < a.rows; r0 += gridDim.y * U) {
        Src in[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t r = r0 + u * gridDim.y;
            if (r < a.rows) in[u] = static_cast<const Src*>(a.src)[static_cast<size_t>(r) * a.srcStride + c];
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t r = r0 + u * gridDim.y;
            if (r >= a.rows) break;
            CT s, o = Ct<CT>::from_f32(0.f);
            if constexpr (SCALAR_PARAMS) {
                s = Ct<CT>::from_f32(a.scale.scalar);
                if (hasOff & 1) o = Ct<CT>::from_f32(a.offset.scalar);
            } else {
                const size_t idx = static_cast<size_t>(a.scale.rdiv ? r / a.scale.rdiv : 0u) * a.scale.stride + sc_col;
                s = Ct<CT>::from_f32(to_f32<Sc>(__ldg(sp + idx)));
                // `op` always points at readable memory here (the launcher passes the scale tensor when the offset is a
                // scalar): the compiler is free to issue this load before it knows which of the two is wanted
                if (hasOff & 1) o = (hasOff & 2) ? Ct<CT>::from_f32(a.offset.scalar) : Ct<CT>::from_f32(to_f32<Sc>(__ldg(op + idx)));
            }
            CT x;
            if constexpr (std::is_same<Src, CT>::value) x = in[u];
            else x = Ct<CT>::from_f32(to_f32<Src>(in[u]));
            if constexpr (OP == kOpQuant) {
                x = Ct<CT>::mul(x, s);
                if (hasOff & 1) x = Ct<CT>::add(x, o);
            } else if constexpr (OP == kOpDequant) {
                x = Ct<CT>::mul(x, s);
                if constexpr (HAS_TOK) x = Ct<CT>::mul(x, Ct<CT>::from_f32(__ldg(a.tok + r)));
            } else {
                if (hasOff & 1) x = Ct<CT>::add(x, o);
                x = Ct<CT>::mul(x, s);
            }
            const float y = Ct<CT>::to_f32(x);
            Dst* d = static_cast<Dst*>(a.dst) + static_cast<size_t>(r) * a.dstStride + c;
            if constexpr (std::is_same<Dst, int8_t>::value) *d = static_cast<int8_t>(f32_to_i8_sat(y, a.roundMode));
            else if constexpr (std::is_same<Dst, __nv_bfloat16>::value) *d = f32_to_bf16_sat(y);
            else if constexpr (std::is_same<Dst, __half>::value) *d = f32_to_f16_sat(y);
            else *d = y;
        }
    }
}

// Launches the instantiation selected by (smode, hasOff, hasTok).  Offsets exist for quant and
// antiquant, the per-row multiplier for dequant.
template <int OP, typename Src, typename Dst, typename Sc, typename CT>
ascq_status launch_ew_rows(const EwArgs& a, int smode, bool hasOff, bool hasTok, cudaStream_t stream)
{
    if (a.rows == 0 || a.cols == 0) return ASCQ_OK;
    dim3 grid, block;
    if (a.scalarPath) {
        if constexpr (std::is_same<Src, int4x2_t>::value) {
            return fail(ASCQ_ERR_UNSUPPORTED, "packed sources have no element-per-thread form");
        } else {
            ew_grid(a.rows, a.cols, 1, &grid, &block, 16u);
            EwArgs b = a;
            if (!hasTok) b.tok = nullptr;
            int off = hasOff ? 1 : 0;  // bit 0: there is an offset; bit 1: it is the scalar
            if (smode != kSScalar && hasOff && b.offset.p == nullptr) {
                off |= 2;
                b.offset.p = b.scale.p;
            }
            if constexpr (OP == kOpDequant) {
                if (hasTok) {
                    if (smode == kSScalar) ew_scalar_kernel<OP, Src, Dst, Sc, CT, true, true><<<grid, block, 0, stream>>>(b, off);
                    else ew_scalar_kernel<OP, Src, Dst, Sc, CT, false, true><<<grid, block, 0, stream>>>(b, off);
                    ASCQ_CUDA_CHECK(cudaGetLastError());
                    return ASCQ_OK;
                }
            }
            if (smode == kSScalar) ew_scalar_kernel<OP, Src, Dst, Sc, CT, true, false><<<grid, block, 0, stream>>>(b, off);
            else ew_scalar_kernel<OP, Src, Dst, Sc, CT, false, false><<<grid, block, 0, stream>>>(b, off);
            ASCQ_CUDA_CHECK(cudaGetLastError());
            return ASCQ_OK;
        }
    }
    ew_grid(a.rows, a.cols, VecOf<Src, Dst>::value, &grid, &block, EwTune<OP>::kCtasPerSm);
    EwArgs b = a;
    if (smode == kSColVec && hasOff && b.offset.p == nullptr) {
        b.offsetIsScalar = 1;
        b.offset.p = b.scale.p;
    }
    b.wide32 = EwTune<OP>::kWide256 && ((reinterpret_cast<uintptr_t>(a.src) | reinterpret_cast<uintptr_t>(a.dst)) & 31u) == 0 &&
               (static_cast<size_t>(a.srcStride) * sizeof(Src)) % 32 == 0 && (static_cast<size_t>(a.dstStride) * sizeof(Dst)) % 32 == 0;
#define ASCQ_EW_LAUNCH(SM, OFF, TOK) \
    launch_rows_kernel(ew_rows_kernel<OP, Src, Dst, Sc, CT, SM, OFF, TOK>, grid, block, stream, b)
#define ASCQ_EW_SMODE(OFF, TOK)                            \
    switch (smode) {                                       \
        case kSScalar: ASCQ_EW_LAUNCH(kSScalar, OFF, TOK); break;     \
        case kSColVec: ASCQ_EW_LAUNCH(kSColVec, OFF, TOK); break;     \
        case kSRowBcast: ASCQ_EW_LAUNCH(kSRowBcast, OFF, TOK); break; \
        default: ASCQ_EW_LAUNCH(kSRowVec, OFF, TOK); break;           \
    }
    if constexpr (OP == kOpDequant) {
        if (hasTok) { ASCQ_EW_SMODE(false, true) } else { ASCQ_EW_SMODE(false, false) }
    } else {
        if (hasOff) { ASCQ_EW_SMODE(true, false) } else { ASCQ_EW_SMODE(false, false) }
    }
#undef ASCQ_EW_SMODE
#undef ASCQ_EW_LAUNCH
    ASCQ_CUDA_CHECK(cudaGetLastError());
    return ASCQ_OK;
}

// ---- runtime-typed scalar kernel for everything the vector kernel cannot take --------------------
// (ragged extents, unaligned pointers, odd group sizes, fp4 sources and destinations).
struct GenericArgs {
    int op;
    int srcT, dstT, scT, ct;  // ascq_dtype codes; ct in {F16, BF16, F32}
    const void* src;
    void* dst;
    uint32_t rows, cols, srcStride, dstStride;
    SRef scale, offset;
    int scaleIsScalar, hasOff, offIsScalar;
    const float* tok;
    int roundMode;
    int fp4Transposed;  // fp4 source: scale index (r, c/32) instead of (r/32, c)
    size_t srcBase, dstBase;  // element offsets added to the flat index (tail launches)
};
ascq_status launch_ew_generic(const GenericArgs& g, cudaStream_t stream);

// True when the vector kernel can be used for this shape and these pointers.
inline bool ew_fast_ok(const EwArgs& a, int vec, int smode, int scSize)
{
    if (a.cols % vec || a.srcStride % vec || a.dstStride % vec) return false;
    if (!aligned16(a.src) || !aligned16(a.dst)) return false;
    if (smode != kSScalar) {
        if (!aligned16(a.scale.p) || (a.offset.p && !aligned16(a.offset.p))) return false;
        if (smode == kSRowBcast && a.scale.cdiv && a.scale.cdiv % vec) return false;
        if (smode == kSRowVec && (a.scale.stride * scSize) % 16) return false;
    }
    return true;
}

// One int8 row segment of 16 weights -> 16 half / bfloat16 values with AscendAntiQuant's arithmetic (the elementwise
// operator's own code: bfloat16 through fp32, half in half), as two 16-byte chunks.
template <typename CT, typename Dst, bool HAS_OFF>
__device__ __forceinline__ void antiquant16(const uint4& raw, CT s, CT o, uint4& lo, uint4& hi)
{
    Pack<int8_t, 16> in;
    *reinterpret_cast<uint4*>(&in) = raw;
    alignas(4) CT x[16];
    unpack_src<int8_t, CT, 16>(in, x);
    const CT sv[1] = {s}, ov[1] = {o};
    apply_op<kOpAntiQuant, CT, 16, 1, HAS_OFF, false>(x, sv, ov, 1.0f);
    Pack<Dst, 16> out;
    pack_dst<Dst, CT, 16>(x, out, kRoundRint);
    lo = reinterpret_cast<const uint4*>(&out)[0];
    hi = reinterpret_cast<const uint4*>(&out)[1];
}

}  // namespace ascq
#endif  // ASCQ_ELEMENTWISE_CUH_
