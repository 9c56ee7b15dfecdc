// Weight-only-quantised matmul for a few activation rows (M <= 32): C[M, N] = A[M, K] x AscendAntiQuant(B)[N, K]^T with the
// int8 weight converted in registers on its way from HBM to the tensor cores, so the 16-bit weight is never written
// anywhere.  At these sizes the product is bound by reading the N x K weight bytes once; the two-launch form (AscendAntiQuant
// into a workspace, then the half / bfloat16 matmul) moves five times as many.  Same arithmetic as that form: each weight
// goes through AscendAntiQuant's own per-element code (include/adv_api/quantization/ascend_antiquant.h:136-205 with
// isTranspose = true: one scale / offset per weight row n; half in half, bfloat16 through fp32), the products are
// accumulated in fp32 and the sum is cast once (impl/adv_api/detail/matmul/stage/copy_cube_in/antiquant/
// antiquant_processor_using_ub.h:86-137 feeds the cube unit the same way).
//
// Shape of the kernel.  The weight rows play the M side of mma.sync.m16n8k16 (16 rows per warp, 4 warps and so 64 rows per
// CTA) and the activation rows the N side (blocks of 8); K may be split over gridDim.y.  Lane (g, c) = (lane / 4, lane % 4)
// loads the 32 consecutive int8 weights k0 + 32c .. k0 + 32c + 31 of rows g and g + 8 and the 32 activations at the same
// k of row g of each block: because a dot product does not care in which order k is visited, those registers are used
// as the fragments of eight MMAs directly (MMA j takes elements 4j .. 4j + 3 of every lane), with no shuffle and no
// staging.  Weight loads run a few steps ahead in a register ring; the activations, which the four warps of a CTA read
// at the same addresses and so mostly find in L1, are fetched one step ahead.  With K split, the fp32 partial sums go to
// the workspace as [split][M][N] and a second small kernel adds the splits in order and casts; with one split the warp
// casts and writes the result itself.  Either way the result does not depend on scheduling.
#include "ascq_internal.h"
#include "elementwise.cuh"
#include "tma_host.h"

namespace ascq {
namespace {

constexpr int kWarps = 4;
constexpr int kRowsPerCta = 16 * kWarps;  // weight rows (output columns) per CTA
constexpr int kChunkK = 128;              // k values one warp consumes per step (4 lanes x 32)

struct SmallParams {
    const int8_t* B;      // [N, K] int8, or [N, K / 2] bytes of int4b_t pairs (even k in the low nibble)
    const void* A;        // [M, K] half / bfloat16
    const void* scale;    // [N] of the activation type, or null: scaleScalar / offsetScalar
    const void* offset;   // [N] or null
    float scaleScalar, offsetScalar;
    float* partial;       // [splits][M][N] fp32 (more than one split)
    void* C;              // [M, ldc] (one split)
    int M, N, K, kPerSplit, ldc, outKind;  // outKind: 0 half, 1 bfloat16, 2 float
};

struct Word8 {
    uint32_t w[8];
};
// 32 bytes per lane in one request: a warp's request covers 128 contiguous bytes of each of its 8 rows
__device__ __forceinline__ Word8 ld_stream32(const void* p)
{
    Word8 v;
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7])
                 : "l"(p));
    return v;
}
__device__ __forceinline__ Word8 ld_cached32(const void* p)
{
    Word8 v;
    asm volatile("ld.global.nc.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7])
                 : "l"(p));
    return v;
}

template <typename Dst>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    if constexpr (std::is_same<Dst, __half>::value)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The 32 weights of one lane and row as they lie in memory: 32 bytes of int8 or 16 bytes of int4b_t pairs.
template <bool I4> struct RawRow {
    uint32_t w[I4 ? 4 : 8];
};
template <bool I4> __device__ __forceinline__ RawRow<I4> ld_weights(const void* p)
{
    RawRow<I4> v;
    if constexpr (I4) {
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(p));
    } else {
        const Word8 t = ld_stream32(p);
#pragma unroll
        for (int i = 0; i < 8; ++i) v.w[i] = t.w[i];
    }
    return v;
}

// 32 int8 weights of one row -> 16 words of two half / bfloat16 values, bit for bit what AscendAntiQuant computes
// ((w + offset) * scale; half: both steps in half; bfloat16: both steps in fp32, then one rounding to bfloat16), without
// the conversion pipe: int8 -> half by placing the biased byte in the mantissa of 1024.0 and subtracting 1152.0 (exact),
// int8 -> float the same way around 2^23.  The bfloat16 form rounds with cvt.rn, which overflows to infinity where
// AscendAntiQuant saturates; `plain` is false for a row whose (|offset| + 128) * |scale| could get there, and such a row
// goes through the elementwise operator's own code.
template <typename CT, typename Dst, bool HAS_OFF>
__device__ __forceinline__ void antiquant32(const RawRow<false>& raw, CT s, CT o, bool plain, uint32_t (&out)[16])
{
    if constexpr (std::is_same<Dst, __half>::value) {
        const __half2 s2 = __half2half2(s), o2 = __half2half2(o), bias = __half2half2(__ushort_as_half(0x6480));  // 1152.0
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const uint32_t b = raw.w[q] ^ 0x80808080u;
            uint32_t p01 = __byte_perm(b, 0x64646464u, 0x4140), p23 = __byte_perm(b, 0x64646464u, 0x4342);
            __half2 h01 = __hsub2_rn(*reinterpret_cast<__half2*>(&p01), bias), h23 = __hsub2_rn(*reinterpret_cast<__half2*>(&p23), bias);
            if constexpr (HAS_OFF) {
                h01 = __hadd2_rn(h01, o2);
                h23 = __hadd2_rn(h23, o2);
            }
            h01 = __hmul2_rn(h01, s2);
            h23 = __hmul2_rn(h23, s2);
            out[2 * q] = *reinterpret_cast<uint32_t*>(&h01);
            out[2 * q + 1] = *reinterpret_cast<uint32_t*>(&h23);
        }
    } else {
        if (plain) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                float f[4];
                unpack_i8x4_f32(raw.w[q], f);
                if constexpr (HAS_OFF) {
                    add2_rn(f[0], f[1], o, o);
                    add2_rn(f[2], f[3], o, o);
                }
                mul2_rn(f[0], f[1], s, s);
                mul2_rn(f[2], f[3], s, s);
                asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(out[2 * q]) : "f"(f[1]), "f"(f[0]));
                asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(out[2 * q + 1]) : "f"(f[3]), "f"(f[2]));
            }
        } else {
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
                const uint4 r4 = make_uint4(raw.w[4 * hlf], raw.w[4 * hlf + 1], raw.w[4 * hlf + 2], raw.w[4 * hlf + 3]);
                uint4 lo, hi;
                antiquant16<CT, Dst, HAS_OFF>(r4, s, o, lo, hi);
                out[8 * hlf + 0] = lo.x; out[8 * hlf + 1] = lo.y; out[8 * hlf + 2] = lo.z; out[8 * hlf + 3] = lo.w;
                out[8 * hlf + 4] = hi.x; out[8 * hlf + 5] = hi.y; out[8 * hlf + 6] = hi.z; out[8 * hlf + 7] = hi.w;
            }
        }
    }
}

// The int4b_t form of antiquant32: byte j of a word holds the weights k = 2j (low nibble) and 2j + 1.  Half: the byte goes
// into both halves of a word whose upper bytes are 0x64 (PRMT), a mask keeps the low nibble in one half and the high
// nibble, in place, in the other (1024 + n and 1024 + 16 n, n biased by 8), and one HFMA2 with the constants
// {1, 1/16} and {-1032, -72} turns both into the signed weight exactly; then the same two roundings as for int8.
// bfloat16: the nibbles go through fp32 as for int8.  Rows whose scale could overflow take the elementwise
// operator's code on nibbles widened to int8, as AscendAntiQuant itself does.
template <typename CT, typename Dst, bool HAS_OFF>
__device__ __forceinline__ void antiquant32_i4(const RawRow<true>& raw, CT s, CT o, bool plain, uint32_t (&out)[16])
{
    if constexpr (std::is_same<Dst, __half>::value) {
        const __half2 s2 = __half2half2(s), o2 = __half2half2(o);
        const __half2 mul = __halves2half2(__ushort_as_half(0x3C00), __ushort_as_half(0x2C00));   // {1, 1/16}
        const __half2 add = __halves2half2(__ushort_as_half(0xE408), __ushort_as_half(0xD480));   // {-1032, -72}
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t b = raw.w[q] ^ 0x88888888u;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t pr = __byte_perm(b, 0x64646464u, 0x4040 + 0x0101 * j) & 0x64F0640Fu;
                __half2 h = __hfma2(*reinterpret_cast<__half2*>(&pr), mul, add);
                if constexpr (HAS_OFF) h = __hadd2_rn(h, o2);
                h = __hmul2_rn(h, s2);
                out[4 * q + j] = *reinterpret_cast<uint32_t*>(&h);
            }
        }
    } else {
        if (plain) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t b = raw.w[q] ^ 0x88888888u;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // 2^23 + (n + 8) in the mantissa, minus 2^23 + 8: exact
                    float f0 = __uint_as_float(0x4B000000u | ((b >> (8 * j)) & 0xFu));
                    float f1 = __uint_as_float(0x4B000000u | ((b >> (8 * j + 4)) & 0xFu));
                    add2_rn(f0, f1, -8388616.0f, -8388616.0f);
                    if constexpr (HAS_OFF) add2_rn(f0, f1, o, o);
                    mul2_rn(f0, f1, s, s);
                    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(out[4 * q + j]) : "f"(f1), "f"(f0));
                }
            }
        } else {
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
                uint32_t w8[4];   // 16 weights widened to int8
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t src = raw.w[2 * hlf + (i >> 1)] >> (16 * (i & 1));   // two bytes = four nibbles
                    uint32_t word = 0;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int n = static_cast<int>((src >> (4 * e)) & 0xFu);
                        word |= static_cast<uint32_t>(((n ^ 8) - 8) & 0xFF) << (8 * e);
                    }
                    w8[i] = word;
                }
                uint4 lo, hi;
                antiquant16<CT, Dst, HAS_OFF>(make_uint4(w8[0], w8[1], w8[2], w8[3]), s, o, lo, hi);
                out[8 * hlf + 0] = lo.x; out[8 * hlf + 1] = lo.y; out[8 * hlf + 2] = lo.z; out[8 * hlf + 3] = lo.w;
                out[8 * hlf + 4] = hi.x; out[8 * hlf + 5] = hi.y; out[8 * hlf + 6] = hi.z; out[8 * hlf + 7] = hi.w;
            }
        }
    }
}

// MB: blocks of 8 activation rows (M <= 8 * MB); DEPTH: weight chunks in flight per lane; XAHEAD: the activations of the
// next step are requested before this step's arithmetic (costs 16 * MB registers), else at the start of their own step
template <typename CT, typename Dst, bool HAS_OFF, int MB, int DEPTH, bool XAHEAD, int MINB, bool I4>
__global__ void __launch_bounds__(32 * kWarps, MINB) w8a16_small_kernel(const SmallParams p)
{
    // launched programmatically, and so is what follows (the reduction, or the next call's kernel): each may be scheduled
    // early and waits for its predecessor's end before it touches memory
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int n0 = blockIdx.x * kRowsPerCta + warp * 16;
    if (n0 >= p.N) return;
    const int kBeg = blockIdx.y * p.kPerSplit, kEnd = min(p.K, kBeg + p.kPerSplit);
    // weight rows of this lane; a row past N is read as row N - 1 and its sums are dropped
    const int nLo = n0 + g, nHi = n0 + g + 8;
    const int rLo = min(nLo, p.N - 1), rHi = min(nHi, p.N - 1);
    float fsLo = p.scaleScalar, fsHi = p.scaleScalar, foLo = HAS_OFF ? p.offsetScalar : 0.f, foHi = foLo;
    if (p.scale != nullptr) {
        fsLo = to_f32<Dst>(static_cast<const Dst*>(p.scale)[rLo]);
        fsHi = to_f32<Dst>(static_cast<const Dst*>(p.scale)[rHi]);
        if (HAS_OFF) {
            foLo = to_f32<Dst>(static_cast<const Dst*>(p.offset)[rLo]);
            foHi = to_f32<Dst>(static_cast<const Dst*>(p.offset)[rHi]);
        }
    }
    const CT sLo = Ct<CT>::from_f32(fsLo), sHi = Ct<CT>::from_f32(fsHi), oLo = Ct<CT>::from_f32(foLo), oHi = Ct<CT>::from_f32(foHi);
    // warp-uniform, so the conversion does not diverge
    const bool plain = __all_sync(0xFFFFFFFFu, !((fabsf(foLo) + 128.f) * fabsf(fsLo) >= 3.0e38f) && !((fabsf(foHi) + 128.f) * fabsf(fsHi) >= 3.0e38f));
    constexpr int kPack = I4 ? 2 : 1;   // weights per byte
    const int8_t* wLo = p.B + (static_cast<size_t>(rLo) * p.K + 32 * c) / kPack;
    const int8_t* wHi = p.B + (static_cast<size_t>(rHi) * p.K + 32 * c) / kPack;
    const Dst* x = static_cast<const Dst*>(p.A) + 32 * c;

    float acc[MB][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mb][i] = 0.f;

    // activations of one step: 64 bytes per lane and block of 8 rows (rows past M read as zero)
    auto load_x = [&](int k0, Word8 (&xv)[MB][2]) {
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            const int m = mb * 8 + g;
            xv[mb][0] = Word8{};
            xv[mb][1] = Word8{};
            if (m < p.M && k0 < kEnd) {
                const Dst* xp = x + static_cast<size_t>(m) * p.K + k0;
                xv[mb][0] = ld_cached32(xp);
                xv[mb][1] = ld_cached32(xp + 16);
            }
        }
    };
    // a ring of DEPTH weight chunks in flight per lane: the loads of step s + DEPTH are issued before step s is consumed
    RawRow<I4> ringLo[DEPTH], ringHi[DEPTH];
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
        const int k = kBeg + d * kChunkK;
        if (k < kEnd) {
            ringLo[d] = ld_weights<I4>(wLo + k / kPack);
            ringHi[d] = ld_weights<I4>(wHi + k / kPack);
        }
    }
    Word8 xCur[MB][2];
    if constexpr (XAHEAD) load_x(kBeg, xCur);
    for (int kBase = kBeg; kBase < kEnd; kBase += DEPTH * kChunkK) {
#pragma unroll
        for (int d = 0; d < DEPTH; ++d) {
            const int k0 = kBase + d * kChunkK;
            if (k0 >= kEnd) break;
            const RawRow<I4> rawLo = ringLo[d], rawHi = ringHi[d];
            const int kNext = k0 + DEPTH * kChunkK;
            if (kNext < kEnd) {
                ringLo[d] = ld_weights<I4>(wLo + kNext / kPack);
                ringHi[d] = ld_weights<I4>(wHi + kNext / kPack);
            }
            Word8 xNext[XAHEAD ? MB : 1][2];
            if constexpr (XAHEAD) load_x(k0 + kChunkK, xNext);
            else load_x(k0, xCur);
            uint32_t al[16], ah[16];  // word i: elements 2i, 2i + 1 of the lane's 32
            if constexpr (I4) {
                antiquant32_i4<CT, Dst, HAS_OFF>(rawLo, sLo, oLo, plain, al);
                antiquant32_i4<CT, Dst, HAS_OFF>(rawHi, sHi, oHi, plain, ah);
            } else {
                antiquant32<CT, Dst, HAS_OFF>(rawLo, sLo, oLo, plain, al);
                antiquant32<CT, Dst, HAS_OFF>(rawHi, sHi, oHi, plain, ah);
            }
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    mma16816<Dst>(acc[mb], al[2 * j], ah[2 * j], al[2 * j + 1], ah[2 * j + 1], xCur[mb][0].w[2 * j], xCur[mb][0].w[2 * j + 1]);
                    mma16816<Dst>(acc[mb], al[8 + 2 * j], ah[8 + 2 * j], al[8 + 2 * j + 1], ah[8 + 2 * j + 1], xCur[mb][1].w[2 * j],
                                  xCur[mb][1].w[2 * j + 1]);
                }
            }
            if constexpr (XAHEAD) {
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                    xCur[mb][0] = xNext[mb][0];
                    xCur[mb][1] = xNext[mb][1];
                }
            }
        }
    }
    // accumulator element i of block mb: weight row (i < 2 ? nLo : nHi), activation row mb * 8 + 2c + (i & 1)
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int m = mb * 8 + 2 * c + (i & 1), n = (i < 2) ? nLo : nHi;
            const float sum = acc[mb][i];
            if (m >= p.M || n >= p.N) continue;
            if (gridDim.y > 1) {
                p.partial[(static_cast<size_t>(blockIdx.y) * p.M + m) * p.N + n] = sum;
            } else if (p.outKind == 2) {
                static_cast<float*>(p.C)[static_cast<size_t>(m) * p.ldc + n] = sum;
            } else {
                // the casts of the half / bfloat16 matmul's epilogue: RINT; bfloat16 saturates, half overflows to infinity
                const uint16_t bits = p.outKind == 1 ? static_cast<uint16_t>(pack_bf16x2_sat(sum, 0.f)) : __half_as_ushort(__float2half_rn(sum));
                static_cast<uint16_t*>(p.C)[static_cast<size_t>(m) * p.ldc + n] = bits;
            }
        }
}

// C[m, n] = cast(sum over splits, in split order); four columns per thread
template <int OUT>  // 0 half, 1 bfloat16, 2 float
__global__ void __launch_bounds__(256) w8a16_small_reduce_kernel(void* __restrict__ C, const float* __restrict__ partial, int M, int N,
                                                                  int ldc, int splits)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");  // launched programmatically behind the kernel that writes `partial`
    const int quadsPerRow = N / 4;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= M * quadsPerRow) return;
    const int m = idx / quadsPerRow, n = (idx - m * quadsPerRow) * 4;
    float4 s = *reinterpret_cast<const float4*>(partial + static_cast<size_t>(m) * N + n);
    for (int sp = 1; sp < splits; ++sp) {
        const float4 v = *reinterpret_cast<const float4*>(partial + (static_cast<size_t>(sp) * M + m) * N + n);
        s.x = __fadd_rn(s.x, v.x);
        s.y = __fadd_rn(s.y, v.y);
        s.z = __fadd_rn(s.z, v.z);
        s.w = __fadd_rn(s.w, v.w);
    }
    const size_t o = static_cast<size_t>(m) * ldc + n;
    if constexpr (OUT == 2) {
        float* c = static_cast<float*>(C) + o;
        c[0] = s.x; c[1] = s.y; c[2] = s.z; c[3] = s.w;
    } else {
        // the casts of the half / bfloat16 matmul's epilogue: RINT; bfloat16 saturates, half overflows to infinity
        uint32_t w0, w1;
        if constexpr (OUT == 1) {
            w0 = pack_bf16x2_sat(s.x, s.y);
            w1 = pack_bf16x2_sat(s.z, s.w);
        } else {
            const __half2 h0 = __floats2half2_rn(s.x, s.y), h1 = __floats2half2_rn(s.z, s.w);
            w0 = *reinterpret_cast<const uint32_t*>(&h0);
            w1 = *reinterpret_cast<const uint32_t*>(&h1);
        }
        uint16_t* c = static_cast<uint16_t*>(C) + o;
        c[0] = static_cast<uint16_t>(w0); c[1] = static_cast<uint16_t>(w0 >> 16);
        c[2] = static_cast<uint16_t>(w1); c[3] = static_cast<uint16_t>(w1 >> 16);
    }
}

// CTAs per SM the variant chosen below is compiled for (its __launch_bounds__)
int small_ctas_per_sm(int M, bool half) { return M <= 8 ? 5 : (M <= 16 ? (half ? 4 : 3) : 3); }

template <typename CT, typename Dst, bool HAS_OFF, bool I4>
cudaError_t launch_small(const SmallParams& p, dim3 grid, cudaStream_t st)
{
    const int mb = (p.M + 7) / 8;
    // Measured on B200 at N = K = 4096 and 8192: resident warps count for more than loads in flight per warp, so the
    // variants trade registers (ring depth 1, activations ahead only where they fit) for CTAs per SM.
    constexpr bool kHalf = std::is_same<Dst, __half>::value;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(32 * kWarps, 1, 1);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (mb <= 1) return cudaLaunchKernelEx(&cfg, w8a16_small_kernel<CT, Dst, HAS_OFF, 1, 1, kHalf, 5, I4>, p);
    if (mb <= 2) return cudaLaunchKernelEx(&cfg, w8a16_small_kernel<CT, Dst, HAS_OFF, 2, 1, true, kHalf ? 4 : 3, I4>, p);
    return cudaLaunchKernelEx(&cfg, w8a16_small_kernel<CT, Dst, HAS_OFF, 4, 1, false, 3, I4>, p);
}

template <int OUT> cudaError_t launch_reduce(void* C, const float* partial, int M, int N, int ldc, int splits, cudaStream_t st)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>((M * (N / 4) + 255) / 256), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, w8a16_small_reduce_kernel<OUT>, C, partial, M, N, ldc, splits);
}

}  // namespace

bool w8a16_small_applies(int M, int N, int K, const void* A, const void* B, const void* workspace, size_t workspaceBytes)
{
    if (M < 1 || M > kW8A16SmallMaxM || K % kChunkK || N % 4) return false;
    if ((reinterpret_cast<uintptr_t>(A) & 31u) || (reinterpret_cast<uintptr_t>(B) & 31u) || !aligned16(workspace)) return false;
    return workspaceBytes >= static_cast<size_t>(M) * N * sizeof(float);
}

// The K split.  Three to five CTAs fit an SM and all CTAs take about the same time per step of 128 values of k, so a launch
// lasts about (number of CTA waves) x (steps per CTA + a fixed start-up cost of about two steps).  The split with the
// smallest such estimate wins, among those whose partial sums stay below a quarter of the weight bytes and fit the
// workspace the caller sized for the two-launch form.
ascq_status w8a16_small(void* C, ascq_dtype cT, const void* A, ascq_dtype aT, const int8_t* B_nk, bool int4, const void* offset,
                        const void* scale, float offsetScalar, float scaleScalar, bool hasOffset, int M, int N, int K, int ldc,
                        void* workspace, size_t workspaceBytes, cudaStream_t st)
{
    const int rowBlocks = (N + kRowsPerCta - 1) / kRowsPerCta, chunks = K / kChunkK;
    const int slots = small_ctas_per_sm(M, aT == ASCQ_DT_F16) * static_cast<int>(sm_count());
    const size_t perSplit = static_cast<size_t>(M) * N * sizeof(float);
    const int maxSplits = static_cast<int>(std::min<size_t>(std::max(1, K / (16 * M)), workspaceBytes / perSplit));
    int chunksPerSplit = chunks;
    double best = 1e30;
    for (int sp = 1; sp <= std::min(chunks / 2, std::max(1, maxSplits)); ++sp) {
        const int cps = (chunks + sp - 1) / sp, ctas = rowBlocks * ((chunks + cps - 1) / cps);
        const double cost = static_cast<double>((ctas + slots - 1) / slots) * (cps + 2.0) + (sp > 1 ? 1.0 : 0.0);
        if (cost < best - 1e-9) {
            best = cost;
            chunksPerSplit = cps;
        }
    }
    const int kPerSplit = chunksPerSplit * kChunkK;
    const int splits = (K + kPerSplit - 1) / kPerSplit;
    if (splits > 1 && static_cast<size_t>(splits) * perSplit > workspaceBytes) return fail(ASCQ_ERR_INVALID_ARG, "workspace too small for the partial sums");
    const int outKind = cT == ASCQ_DT_F16 ? 0 : (cT == ASCQ_DT_BF16 ? 1 : 2);
    SmallParams p{B_nk, A, scale, offset, scaleScalar, offsetScalar, static_cast<float*>(workspace), C, M, N, K, kPerSplit, ldc, outKind};
    const dim3 grid(static_cast<unsigned>(rowBlocks), static_cast<unsigned>(splits), 1);
    cudaError_t e;
    auto go = [&](auto off, auto i4) {
        constexpr bool kOff = decltype(off)::value, kI4 = decltype(i4)::value;
        return aT == ASCQ_DT_F16 ? launch_small<__half, __half, kOff, kI4>(p, grid, st) : launch_small<float, __nv_bfloat16, kOff, kI4>(p, grid, st);
    };
    if (int4) e = hasOffset ? go(std::true_type{}, std::true_type{}) : go(std::false_type{}, std::true_type{});
    else e = hasOffset ? go(std::true_type{}, std::false_type{}) : go(std::false_type{}, std::false_type{});
    ASCQ_CUDA_CHECK(e);
    if (splits == 1) return ASCQ_OK;
    if (cT == ASCQ_DT_F16) e = launch_reduce<0>(C, p.partial, M, N, ldc, splits, st);
    else if (cT == ASCQ_DT_BF16) e = launch_reduce<1>(C, p.partial, M, N, ldc, splits, st);
    else e = launch_reduce<2>(C, p.partial, M, N, ldc, splits, st);
    ASCQ_CUDA_CHECK(e);
    return ASCQ_OK;
}

}  // namespace ascq
