/*
 * ascq_oracle.c -- CPU restatement of the Ascend C quantization operators and the quantized
 * matmuls around them.  TEST INFRASTRUCTURE ONLY: it is the checker the parity tests, the smoke
 * test and the benchmark's CPU-baseline leg compare the CUDA kernels against.  Nothing in the
 * product path may call it.
 *
 * Every function states which reference file:line (paths inside the asc-devkit tree) it follows.
 * The reference's own CPU-debug execution needs the closed `tikicpulib` library of the CANN
 * toolkit, which is not part of the source tree; the operator arithmetic is therefore restated
 * here from the operator sources and the documented conversion rules.
 *
 * Parity pins: the conversion helpers are checked against the worked examples of
 * docs/zh/api/SIMD-API/基础API/数据结构/precision_conversion.md, the operators against the numpy
 * golden generators of the reference's examples (tests/golden), the tmp-size formulas against
 * tests/api/adv_api/tiling/test_tiling.cpp:6540-6712.  Outputs of the operators through the real
 * CPU-debug model are not available: for NaN / Inf / fp16 overflow inside the arithmetic the
 * parity is unpinned (IEEE behaviour is assumed).
 *
 * Plain C, scalar, optionally OpenMP across rows (used only to time the CPU baseline).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- dtype / policy / round codes: numerically identical to include/ascq.h ---------------- */
enum { DT_F16 = 0, DT_BF16 = 1, DT_F32 = 2, DT_I8 = 3, DT_I32 = 4, DT_U64 = 5, DT_FP4X2_E2M1 = 6, DT_E8M0 = 7, DT_I4X2 = 12 };
enum { PER_TENSOR = 0, PER_CHANNEL = 1, PER_TOKEN = 2, PER_GROUP = 3 };
enum { CAST_NONE = 0, CAST_RINT = 1, CAST_FLOOR = 2, CAST_CEIL = 3, CAST_ROUND = 4, CAST_TRUNC = 5 };
enum { OR_OK = 0, OR_INVALID = 1, OR_UNSUPPORTED = 2 };

/* ------------------------------------------------------------------------------------------
 * Conversion helpers.  Rounding of a binary significand: precision_conversion.md:5-27.
 * Overflow saturates by default (precision_conversion.md:30).
 * ---------------------------------------------------------------------------------------- */
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* half -> float, exact (precision_conversion.md:323). */
float orc_f16_to_f32(uint16_t h)
{
    uint32_t s = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu;
    uint32_t m = h & 0x3FFu;
    if (e == 0) {
        if (m == 0) return bits_f32(s);
        /* subnormal: value = m * 2^-24 */
        float v = (float)m * 5.9604644775390625e-8f;
        return (s ? -v : v);
    }
    if (e == 31) return bits_f32(s | 0x7F800000u | (m << 13));
    return bits_f32(s | ((e + 112u) << 23) | (m << 13));
}

/* Round a double to the nearest half (ties to even); overflow saturates to +-65504
 * (float -> half, precision_conversion.md:520-539, saturation rule :30).
 * A double intermediate holds any sum or product of two halves exactly, and any fp32 value. */
uint16_t orc_f64_to_f16_sat(double d)
{
    uint16_t sign = (uint16_t)(signbit(d) ? 0x8000u : 0);
    if (isnan(d)) return (uint16_t)(sign | 0x7E00u);
    double a = fabs(d);
    if (isinf(d)) return (uint16_t)(sign | 0x7C00u);
    if (a == 0.0) return sign;
    int e;
    double fr = frexp(a, &e); /* a = fr * 2^e, fr in [0.5,1) */
    int exp = e - 1;          /* a = (2fr) * 2^exp, 2fr in [1,2) */
    if (exp < -14) {
        /* subnormal: quantum 2^-24 */
        double q = nearbyint(ldexp(a, 24)); /* default rounding mode = ties to even */
        uint32_t m = (uint32_t)q;           /* may reach 1024 = smallest normal, encoding still right */
        return (uint16_t)(sign | m);
    }
    double sig = nearbyint(ldexp(fr, 11)); /* 11-bit significand in [1024, 2048] */
    if (sig == 2048.0) { sig = 1024.0; exp += 1; }
    if (exp > 15) return (uint16_t)(sign | 0x7BFFu); /* saturate */
    uint32_t m = (uint32_t)sig - 1024u;
    return (uint16_t)(sign | ((uint32_t)(exp + 15) << 10) | m);
}
uint16_t orc_f32_to_f16_sat(float f) { return orc_f64_to_f16_sat((double)f); }

/* half arithmetic: one correctly rounded operation each (Muls/Adds/Mul/Add on half,
 * impl/adv_api/detail/quantization/quant/ascend_quant_pre_impl.h:320-333).  IEEE overflow. */
static uint16_t f64_to_f16_ieee(double d)
{
    uint16_t r = orc_f64_to_f16_sat(d);
    if ((r & 0x7FFFu) == 0x7BFFu && fabs(d) >= 65520.0) r = (uint16_t)((r & 0x8000u) | 0x7C00u);
    return r;
}
uint16_t orc_f16_mul(uint16_t a, uint16_t b) { return f64_to_f16_ieee((double)orc_f16_to_f32(a) * (double)orc_f16_to_f32(b)); }
uint16_t orc_f16_add(uint16_t a, uint16_t b) { return f64_to_f16_ieee((double)orc_f16_to_f32(a) + (double)orc_f16_to_f32(b)); }

/* bf16 <-> float (precision_conversion.md:387, :541-555).  RINT, finite overflow saturates. */
float orc_bf16_to_f32(uint16_t b) { return bits_f32((uint32_t)b << 16); }
uint16_t orc_f32_to_bf16_sat(float f)
{
    uint32_t u = f32_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
    if ((u & 0x7FFFFFFFu) == 0x7F800000u) return (uint16_t)(u >> 16);            /* Inf */
    uint32_t lsb = (u >> 16) & 1u;
    uint32_t r = u + 0x7FFFu + lsb;
    uint16_t out = (uint16_t)(r >> 16);
    if ((out & 0x7FFFu) == 0x7F80u) out = (uint16_t)((out & 0x8000u) | 0x7F7Fu); /* saturate */
    return out;
}
static uint16_t f32_to_bf16_ieee(float f)
{
    uint32_t u = f32_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t lsb = (u >> 16) & 1u;
    return (uint16_t)((u + 0x7FFFu + lsb) >> 16);
}
/* bf16 arithmetic: the product of two bf16 is exact in fp32; a sum rounded to fp32 and then to
 * bf16 equals the directly rounded sum (24 >= 2*8+2 bits), so fp32 intermediates are exact enough. */
uint16_t orc_bf16_mul(uint16_t a, uint16_t b) { return f32_to_bf16_ieee(orc_bf16_to_f32(a) * orc_bf16_to_f32(b)); }
uint16_t orc_bf16_add(uint16_t a, uint16_t b)
{
    float s = orc_bf16_to_f32(a) + orc_bf16_to_f32(b);
    return f32_to_bf16_ieee(s);
}

/* Round-to-integer in the six modes (precision_conversion.md:15-27). */
static double round_mode(double v, int mode)
{
    switch (mode) {
        case CAST_FLOOR: return floor(v);
        case CAST_CEIL: return ceil(v);
        case CAST_ROUND: return round(v); /* half away from zero */
        case CAST_TRUNC: return trunc(v);
        default: return nearbyint(v);     /* NONE, RINT: half to even */
    }
}
/* half -> int8: round, then saturate to [-128, 127] (precision_conversion.md:242-248). */
int8_t orc_f16_to_i8(uint16_t h, int mode)
{
    float f = orc_f16_to_f32(h);
    if (isnan(f)) return 0;
    double r = round_mode((double)f, mode);
    if (r > 127.0) r = 127.0;
    if (r < -128.0) r = -128.0;
    return (int8_t)r;
}
/* float -> int16 with saturation (precision_conversion.md:506-518). */
int16_t orc_f32_to_i16(float f, int mode)
{
    if (isnan(f)) return 0;
    double r = round_mode((double)f, mode);
    if (r > 32767.0) r = 32767.0;
    if (r < -32768.0) r = -32768.0;
    return (int16_t)r;
}
/* int32 -> float, RINT (precision_conversion.md:427-440; CAST_NONE in
 * impl/.../dequant/ascend_dequant_common_impl.h:262-267). */
float orc_i32_to_f32(int32_t v) { return (float)v; }

/* E2M1 code -> value (docs .../内置数据类型.md:145-147: 1 sign, 2 exponent, 1 mantissa bit, range +-6). */
float orc_e2m1_to_f32(uint8_t code)
{
    static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float v = mag[code & 7u];
    return (code & 8u) ? -v : v;
}
/* E8M0 scale byte -> bf16 bit pattern: bits << 7, 0x00 -> 0x0040 (2^-127), 0xFF -> 0x7FFF (NaN)
 * (impl/adv_api/detail/quantization/antiquant/ascend_antiquant_3510_impl.h:49-74). */
uint16_t orc_e8m0_to_bf16(uint8_t e)
{
    if (e == 0) return 0x0040u;
    if (e == 0xFFu) return 0x7FFFu;
    return (uint16_t)((uint16_t)e << 7);
}
/* bf16 -> E2M1 code, RINT + saturation (precision_conversion.md:331-343). */
uint8_t orc_f32_to_e2m1(float f, int mode)
{
    static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    uint8_t sign = (uint8_t)(signbit(f) ? 8u : 0u);
    float a = fabsf(f);
    if (isnan(f)) return (uint8_t)(sign | 7u);
    if (a >= 6.0f) return (uint8_t)(sign | 7u);
    int lo = 0;
    for (int i = 0; i < 7; ++i) if (a >= mag[i]) lo = i;
    int hi = lo + 1;
    float dl = a - mag[lo], dh = mag[hi] - a;
    int pick;
    if (dl == 0.0f) pick = lo;
    else switch (mode) {
        case CAST_FLOOR: pick = sign ? hi : lo; break;
        case CAST_CEIL: pick = sign ? lo : hi; break;
        case CAST_TRUNC: pick = lo; break;
        case CAST_ROUND: pick = (dh <= dl) ? hi : lo; break;
        default: /* ties to the code with an even mantissa bit */
            if (dl < dh) pick = lo; else if (dh < dl) pick = hi; else pick = (lo & 1) ? hi : lo;
    }
    return (uint8_t)(sign | (uint8_t)pick);
}

/* ------------------------------------------------------------------------------------------
 * Generic typed load/store.
 * ---------------------------------------------------------------------------------------- */
static int dt_size(int dt)
{
    switch (dt) {
        case DT_F16: case DT_BF16: return 2;
        case DT_F32: case DT_I32: return 4;
        case DT_I8: case DT_E8M0: return 1;
        case DT_U64: return 8;
        default: return 0;
    }
}
/* load a scale/offset/source element as float (exact for every type) */
static float load_as_f32(const void* p, int dt, size_t i)
{
    switch (dt) {
        case DT_F16: return orc_f16_to_f32(((const uint16_t*)p)[i]);
        case DT_BF16: return orc_bf16_to_f32(((const uint16_t*)p)[i]);
        case DT_F32: return ((const float*)p)[i];
        case DT_I8: return (float)((const int8_t*)p)[i];
        case DT_I32: return orc_i32_to_f32(((const int32_t*)p)[i]);
        case DT_U64: return bits_f32((uint32_t)(((const uint64_t*)p)[i] & 0xFFFFFFFFu)); /* low word = fp32 bits,
                        ascend_dequant_common_impl.h:239-249 */
        default: return 0.0f;
    }
}

/* A value held in the compute type CT (half / bf16 / float). */
typedef struct { int ct; uint16_t h; float f; } cval;

static cval cv_from_f32(float v, int ct)
{
    cval c; c.ct = ct; c.h = 0; c.f = 0.f;
    if (ct == DT_F16) c.h = orc_f32_to_f16_sat(v);
    else if (ct == DT_BF16) c.h = orc_f32_to_bf16_sat(v);
    else c.f = v;
    return c;
}
static float cv_to_f32(cval c)
{
    if (c.ct == DT_F16) return orc_f16_to_f32(c.h);
    if (c.ct == DT_BF16) return orc_bf16_to_f32(c.h);
    return c.f;
}
static cval cv_mul(cval a, cval b)
{
    cval r = a;
    if (a.ct == DT_F16) r.h = orc_f16_mul(a.h, b.h);
    else if (a.ct == DT_BF16) r.h = orc_bf16_mul(a.h, b.h);
    else { float t = a.f * b.f; r.f = t; }
    return r;
}
static cval cv_add(cval a, cval b)
{
    cval r = a;
    if (a.ct == DT_F16) r.h = orc_f16_add(a.h, b.h);
    else if (a.ct == DT_BF16) r.h = orc_bf16_add(a.h, b.h);
    else { float t = a.f + b.f; r.f = t; }
    return r;
}

/* Scale / offset addressing shared by the three operators:
 *   index(r, c) = (r / rdiv) * stride + (c / cdiv); rdiv or cdiv == 0 means "does not depend on it". */
typedef struct { const void* p; int dt; uint32_t rdiv, cdiv, stride; int is_scalar; float scalar; } sref;
static float sref_get(const sref* s, uint32_t r, uint32_t c)
{
    if (s->is_scalar) return s->scalar;
    size_t idx = (size_t)(s->rdiv ? r / s->rdiv : 0) * s->stride + (s->cdiv ? c / s->cdiv : 0);
    return load_as_f32(s->p, s->dt, idx);
}
static void sref_scalar(sref* s, float v) { memset(s, 0, sizeof(*s)); s->is_scalar = 1; s->scalar = v; }
static void sref_tensor(sref* s, const void* p, int dt, uint32_t rdiv, uint32_t cdiv, uint32_t stride)
{
    memset(s, 0, sizeof(*s)); s->p = p; s->dt = dt; s->rdiv = rdiv; s->cdiv = cdiv; s->stride = stride;
}
static int policy_sref(sref* s, const void* p, int dt, int policy, uint32_t m, uint32_t n, uint32_t gs, int kDim)
{
    (void)m;
    if (policy == PER_TOKEN) { sref_tensor(s, p, dt, 1, 0, 1); return OR_OK; }
    if (policy == PER_GROUP) {
        if (gs == 0 || gs % 32 != 0) return OR_INVALID;
        if (kDim == 1) sref_tensor(s, p, dt, 1, gs, (n + gs - 1) / gs);
        else sref_tensor(s, p, dt, gs, 1, n);
        return OR_OK;
    }
    return OR_UNSUPPORTED;
}

/* ------------------------------------------------------------------------------------------
 * AscendQuant
 *   per-tensor   impl/adv_api/detail/quantization/quant/ascend_quant_pre_impl.h:320-397
 *                (and ascend_quant_3510_impl.h:35-142): src -> half (RINT, sat), half * half(scale),
 *                half + half(offset), half -> int8 (RINT, sat).
 *   per-channel  ascend_quant_pre_impl.h:101-209, 399-483: same with scale[n] (fp32 scale first cast
 *                to half) and scalar or tensor offset.
 *   PER_TOKEN / PER_GROUP  ascend_quant_per_group_3510_impl.h:54-90 (per token), :498-538 (kDim 1),
 *                :1000-1044 (kDim 0): src -> scaleT, mul, add (if hasOffset) in scaleT, then the
 *                to-int8 chain of ascend_quant_3510_impl.h:934-992:
 *                   scaleT float : float -> int16 (roundMode, sat) -> half -> int8 (RINT, sat)
 *                   scaleT bf16  : bf16 -> float, then as float
 *                   scaleT half  : half -> int8 (roundMode, sat)
 *                fp4 destination (PER_GROUP, no offset; ascend_quant_3510_impl.h:994-1032):
 *                   result -> bf16 (RINT) -> e2m1 (roundMode, sat), two codes per byte.
 * ---------------------------------------------------------------------------------------- */
typedef struct { uint32_t m, n, calCount, groupSize; int32_t hasOffset, kDim; int32_t roundMode; } quant_param;

/* unified != 0: the Quantize interface (impl/adv_api/detail/quantization/quantize/quantize_impl.h:832-975):
 * every policy in fp32 -- src and scale/offset widened to fp32, multiply, add (if hasOffset), then the
 * float -> int16 (roundMode, sat) -> half -> int8 chain (quantize_impl.h:146-157) or, for fp4, float -> bf16 (RINT)
 * -> e2m1 (roundMode) (:170-185). */
static int quant_common(void* dst, int dstT, const void* src, int srcT, const void* scale, const void* offset,
                        int scaleT, float scaleScalar, float offsetScalar, int policy, const quant_param* p, int unified)
{
    if (!dst || !src || !p) return OR_INVALID;
    if (srcT != DT_F16 && srcT != DT_BF16 && srcT != DT_F32) return OR_UNSUPPORTED;
    if (dstT != DT_I8 && dstT != DT_FP4X2_E2M1) return OR_UNSUPPORTED;
    uint32_t n, rows;
    int ct, mode = CAST_RINT, has_off = 1, legacy = (policy == PER_TENSOR || policy == PER_CHANNEL);
    sref ss, so;
    if (policy == PER_TENSOR) {
        if (dstT != DT_I8) return OR_UNSUPPORTED;
        ct = DT_F16;
        sref_scalar(&ss, scaleScalar); sref_scalar(&so, offsetScalar);
        n = p->calCount; rows = 1; /* flat */
        if (unified) { has_off = p->hasOffset; mode = p->roundMode; }
    } else if (policy == PER_CHANNEL) {
        if (dstT != DT_I8) return OR_UNSUPPORTED;
        if (!scale || p->n == 0 || p->calCount % p->n != 0) return OR_INVALID;
        if (!unified && scaleT != DT_F16 && scaleT != DT_F32) return OR_UNSUPPORTED;
        ct = DT_F16;
        n = p->n; rows = p->calCount / n;
        sref_tensor(&ss, scale, scaleT, 0, 1, 0);
        if (offset) sref_tensor(&so, offset, scaleT, 0, 1, 0); else sref_scalar(&so, offsetScalar);
        if (unified) { has_off = p->hasOffset; mode = p->roundMode; }
    } else {
        if (!scale || p->n == 0 || p->calCount % p->n != 0) return OR_INVALID;
        if (scaleT != DT_F16 && scaleT != DT_BF16 && scaleT != DT_F32) return OR_UNSUPPORTED;
        /* (src, scale) pairs: (h,h) (bf,bf) (f,f) (h,f) (bf,f) -- tests/api/adv_api/quantization/quant/
         * test_ascend_quant_per_token.cpp:146-173 */
        if (scaleT != DT_F32 && scaleT != srcT) return OR_UNSUPPORTED;
        ct = scaleT; mode = p->roundMode; has_off = p->hasOffset;
        n = p->n; rows = p->calCount / n;
        int rc = policy_sref(&ss, scale, scaleT, policy, rows, n, p->groupSize, p->kDim);
        if (rc) return rc;
        if (has_off) { if (!offset) return OR_INVALID; policy_sref(&so, offset, scaleT, policy, rows, n, p->groupSize, p->kDim); }
        if (dstT == DT_FP4X2_E2M1 && (policy != PER_GROUP || has_off || (n & 1))) return OR_UNSUPPORTED;
    }
    if (unified) {
        if (scaleT != DT_F16 && scaleT != DT_BF16 && scaleT != DT_F32) return OR_UNSUPPORTED;
        if (scaleT != DT_F32 && scaleT != srcT) return OR_UNSUPPORTED;
        ct = DT_F32; legacy = 0;
    }
#pragma omp parallel for schedule(static)
    for (uint32_t r = 0; r < rows; ++r) {
        for (uint32_t c = 0; c < n; ++c) {
            size_t i = (size_t)r * n + c;
            cval x = cv_from_f32(load_as_f32(src, srcT, i), ct);
            cval s = cv_from_f32(sref_get(&ss, r, c), ct);
            x = cv_mul(x, s);
            if (has_off) x = cv_add(x, cv_from_f32(sref_get(&so, r, c), ct));
            if (dstT == DT_I8) {
                int8_t q;
                if (ct == DT_F16) q = orc_f16_to_i8(x.h, legacy ? CAST_RINT : mode);
                else {
                    int16_t t = orc_f32_to_i16(cv_to_f32(x), mode);
                    q = orc_f16_to_i8(orc_f32_to_f16_sat((float)t), CAST_RINT);
                }
                ((int8_t*)dst)[i] = q;
            } else {
                float v = orc_bf16_to_f32(orc_f32_to_bf16_sat(cv_to_f32(x)));
                uint8_t code = orc_f32_to_e2m1(v, mode);
                uint8_t* d = (uint8_t*)dst + i / 2;
                /* each (r, c/2) byte is written by one thread only when n is even */
                if (i & 1) *d = (uint8_t)((*d & 0x0Fu) | (code << 4)); else *d = (uint8_t)((*d & 0xF0u) | code);
            }
        }
    }
    return OR_OK;
}

int ascq_oracle_quant(void* dst, int dstT, const void* src, int srcT, const void* scale, const void* offset,
                      int scaleT, float scaleScalar, float offsetScalar, int policy, const quant_param* p)
{
    return quant_common(dst, dstT, src, srcT, scale, offset, scaleT, scaleScalar, offsetScalar, policy, p, 0);
}

typedef struct { uint32_t m, n, groupSize; int32_t hasOffset, kDim; int32_t roundMode; } quantize_param;

int ascq_oracle_quantize(void* dst, int dstT, const void* src, int srcT, const void* scale, const void* offset,
                         int scaleT, float scaleScalar, float offsetScalar, int policy, const quantize_param* q)
{
    if (!q) return OR_INVALID;
    quant_param p = {q->m, q->n, q->m * q->n, q->groupSize, q->hasOffset, q->kDim, q->roundMode};
    return quant_common(dst, dstT, src, srcT, scale, offset, scaleT, scaleScalar, offsetScalar, policy, &p, 1);
}

/* Build-defined dynamic per-token quantisation (no reference counterpart): fp32 absmax per row,
 * scale = 127 / absmax (1 when the row is all zero), then the PER_TOKEN float chain above. */
int ascq_oracle_dynamic_quant_per_token(int8_t* dst, float* scaleOut, float* deqScaleOut, const void* src, int srcT,
                                        uint32_t m, uint32_t n)
{
    if (!dst || !src || !scaleOut) return OR_INVALID;
#pragma omp parallel for schedule(static)
    for (uint32_t r = 0; r < m; ++r) {
        float amax = 0.f;
        for (uint32_t c = 0; c < n; ++c) { float v = fabsf(load_as_f32(src, srcT, (size_t)r * n + c)); if (v > amax) amax = v; }
        float s = (amax > 0.f) ? 127.0f / amax : 1.0f;
        scaleOut[r] = s;
        if (deqScaleOut) { float d = (amax > 0.f) ? amax / 127.0f : 1.0f; deqScaleOut[r] = d; }
        for (uint32_t c = 0; c < n; ++c) {
            float t = load_as_f32(src, srcT, (size_t)r * n + c) * s;
            int16_t q = orc_f32_to_i16(t, CAST_RINT);
            dst[(size_t)r * n + c] = orc_f16_to_i8(orc_f32_to_f16_sat((float)q), CAST_RINT);
        }
    }
    return OR_OK;
}

/* Build-defined dynamic MX-FP4 block quantisation (no reference counterpart): per 32 elements amax -> shared exponent
 * floor(log2(amax)) - 2 clamped to [-127, 127] (0 when amax == 0) -> byte e + 127 (0xFF with codes 0 when the block
 * holds NaN / Inf); code = e2m1(bf16(x * 2^-e)) with RINT twice, saturating (the fp4 chain of AscendQuant above). */
int ascq_oracle_dynamic_quant_mxfp4(uint8_t* dst, uint8_t* scaleOut, const void* src, int srcT, uint32_t m, uint32_t n)
{
    if (!dst || !scaleOut || !src || n % 32 != 0) return OR_INVALID;
    const uint64_t blocks = (uint64_t)m * (n / 32);
#pragma omp parallel for schedule(static)
    for (uint64_t b = 0; b < blocks; ++b) {
        float v[32], amax = 0.f;
        int bad = 0;
        for (int i = 0; i < 32; ++i) {
            v[i] = load_as_f32(src, srcT, (size_t)b * 32 + i);
            float a = fabsf(v[i]);
            if (!(a <= 3.4028234663852886e38f)) bad = 1;
            if (a > amax) amax = a;
        }
        int e = 0;
        if (amax > 0.f) {
            uint32_t bits = f32_bits(amax);
            int ex = (int)((bits >> 23) & 0xFF);
            e = (ex == 0 ? -126 : ex - 127) - 2;
            if (e < -127) e = -127;
            if (e > 127) e = 127;
        }
        scaleOut[b] = bad ? 0xFFu : (uint8_t)(e + 127);
        for (int i = 0; i < 32; ++i) {
            /* x * 2^-e: exact unless it underflows; two steps keep both factors normal, as the kernel does */
            int h1 = (-e) / 2, h2 = (-e) - h1;
            float y = (v[i] * ldexpf(1.0f, h1)) * ldexpf(1.0f, h2);
            uint8_t code = bad ? 0 : orc_f32_to_e2m1(orc_bf16_to_f32(orc_f32_to_bf16_sat(y)), CAST_RINT);
            uint8_t* d = dst + ((size_t)b * 32 + i) / 2;
            if (i & 1) *d = (uint8_t)((*d & 0x0Fu) | (code << 4)); else *d = (uint8_t)((*d & 0xF0u) | code);
        }
    }
    return OR_OK;
}

/* ------------------------------------------------------------------------------------------
 * AscendDequant
 *   per-channel / scalar  impl/adv_api/detail/quantization/dequant/ascend_dequant_common_impl.h:
 *      CastDeqscale :225-255 (u64 low word / bf16 / fp32 -> fp32), CastSrc :260-267 (int32 -> fp32),
 *      DequantMul :273-325 (fp32 multiply of the first calCount columns of every row),
 *      CastDst :328-362 with GetFP32CastMode :194-204 (bf16: RINT, half: NONE = RINT),
 *      row stride of dst = n rounded up to 32 bytes (:100-105, :380).
 *   PER_TOKEN / PER_GROUP ascend_dequant_3510_impl.h:226-296, 337-446 (fp32 multiply by the token /
 *      group scale converted to fp32; result cast RINT + sat).
 *   tokScale: optional second fp32 multiply by tokScale[row], applied after the channel scale as in
 *      examples/.../quant_group_matmul_custom.asc:433-441.
 * Only the first calCount columns of a row are written.
 * ---------------------------------------------------------------------------------------- */
typedef struct { uint32_t m, n, calCount, groupSize; int32_t kDim; } dequant_param;

static void store_from_f32(void* dst, int dstT, size_t i, float v)
{
    if (dstT == DT_F32) ((float*)dst)[i] = v;
    else if (dstT == DT_BF16) ((uint16_t*)dst)[i] = orc_f32_to_bf16_sat(v);
    else ((uint16_t*)dst)[i] = orc_f32_to_f16_sat(v);
}

uint32_t ascq_oracle_dequant_dst_stride(uint32_t n, int dstT)
{
    uint32_t per_blk = 32u / (uint32_t)dt_size(dstT);
    return (n + per_blk - 1) / per_blk * per_blk;
}

int ascq_oracle_dequant(void* dst, int dstT, const void* src, int srcT, const void* scale, const float* tokScale,
                        int scaleT, float scaleScalar, int policy, const dequant_param* p)
{
    if (!dst || !src || !p || p->n == 0) return OR_INVALID;
    if (dstT != DT_F16 && dstT != DT_BF16 && dstT != DT_F32) return OR_UNSUPPORTED;
    if (srcT != DT_I32 && srcT != DT_F32) return OR_UNSUPPORTED;
    uint32_t rows, cols, n = p->n, dstStride = n;
    sref ss;
    if (policy == PER_TENSOR || policy == PER_CHANNEL) {
        if (srcT != DT_I32) return OR_UNSUPPORTED;
        if (p->calCount == 0 || p->calCount > n) return OR_INVALID;
        rows = p->m; cols = p->calCount; dstStride = ascq_oracle_dequant_dst_stride(n, dstT);
        if (policy == PER_TENSOR) sref_scalar(&ss, scaleScalar);
        else {
            if (!scale) return OR_INVALID;
            if (scaleT != DT_U64 && scaleT != DT_F32 && scaleT != DT_BF16) return OR_UNSUPPORTED;
            sref_tensor(&ss, scale, scaleT, 0, 1, 0);
        }
    } else {
        if (!scale || p->calCount % n != 0) return OR_INVALID;
        if (scaleT != DT_F16 && scaleT != DT_BF16 && scaleT != DT_F32) return OR_UNSUPPORTED;
        rows = p->calCount / n; cols = n;
        int rc = policy_sref(&ss, scale, scaleT, policy, rows, n, p->groupSize, p->kDim);
        if (rc) return rc;
    }
#pragma omp parallel for schedule(static)
    for (uint32_t r = 0; r < rows; ++r) {
        for (uint32_t c = 0; c < cols; ++c) {
            float f = load_as_f32(src, srcT, (size_t)r * n + c);
            f = f * sref_get(&ss, r, c);
            if (tokScale) f = f * tokScale[r];
            store_from_f32(dst, dstT, (size_t)r * dstStride + c, f);
        }
    }
    return OR_OK;
}

/* ------------------------------------------------------------------------------------------
 * AscendAntiQuant:  dst = scale * (src + offset)   (include/adv_api/quantization/ascend_antiquant.h:37)
 *   legacy, dst bf16: int8 -> half -> fp32 (exact), fp32 add of float(offset), fp32 multiply by
 *      float(scale), RINT to bf16   (antiquant/ascend_antiquant_c220_impl.h:45-102)
 *   legacy, dst half: int8 -> half, half add, half multiply (antiquant/ascend_antiquant_impl.h:62-76)
 *   layouts (ascend_antiquant_impl.h:283-408; docs .../AscendAntiQuant.md:35-49):
 *      !isTranspose: src [K,N], scale/offset [K/groupSize, N] -> index (i/groupSize, j)
 *       isTranspose: src [N,K], scale/offset [N, K/groupSize] -> index (i, j/groupSize)
 *   PER_TOKEN / PER_GROUP (antiquant/ascend_antiquant_3510_impl.h:1385-1495): src -> scaleT
 *      (bf16 via half, RINT), add offset, multiply scale in scaleT, cast to dstT (RINT, sat).
 *      A transposed PER_TOKEN applies scale[col] (ascend_antiquant_3510_impl.h:1311-1327).
 *   fp4 source + e8m0 scale (:49-138): scale byte -> bf16 (0x00 -> 2^-127, 0xFF -> NaN), value =
 *      bf16(fp4) * scale in bf16 (dst bf16) or both cast to half first (dst half); groups of 32
 *      along K: rows when !isTranspose, columns when isTranspose.
 * ---------------------------------------------------------------------------------------- */
typedef struct { uint32_t m, n, calCount, groupSize; int32_t hasOffset, isTranspose, kDim; } antiquant_param;

/* unified != 0: the AntiQuantize interface (antiquantize/antiquantize_3510_impl.h:252-381, antiquantize_impl.h:
 * 68-190): int8 -> half -> fp32 (exact), fp32 add of float(offset) when hasOffset, fp32 multiply by float(scale),
 * one cast to dstT (RINT, sat), for every policy; PER_CHANNEL takes scale[n] / offset[n], never transposed. */
static int antiquant_common(void* dst, int dstT, const void* src, int srcT, const void* offset, const void* scale,
                            int scaleT, float offsetScalar, float scaleScalar, int policy, const antiquant_param* p,
                            int unified)
{
    if (!dst || !src || !p || p->n == 0) return OR_INVALID;
    uint32_t n = p->n;
    uint32_t total = p->calCount ? p->calCount : p->m * n;
    if (total % n != 0) return OR_INVALID;
    uint32_t rows = total / n;
    sref ss, so; int has_off = 1, ct;

    if (srcT == DT_FP4X2_E2M1) {
        if (scaleT != DT_E8M0 || !scale) return OR_INVALID;
        if (dstT != DT_BF16 && dstT != DT_F16) return OR_UNSUPPORTED;
        if (n & 1) return OR_INVALID;
        uint32_t kext = p->isTranspose ? n : rows;
        if (kext % 32 != 0) return OR_INVALID;
#pragma omp parallel for schedule(static)
        for (uint32_t r = 0; r < rows; ++r)
            for (uint32_t c = 0; c < n; ++c) {
                size_t i = (size_t)r * n + c;
                uint8_t byte = ((const uint8_t*)src)[i / 2];
                uint8_t code = (i & 1) ? (byte >> 4) : (byte & 0x0Fu);
                size_t si = p->isTranspose ? (size_t)r * (n / 32) + c / 32 : (size_t)(r / 32) * n + c;
                uint16_t sb = orc_e8m0_to_bf16(((const uint8_t*)scale)[si]);
                uint16_t vb = orc_f32_to_bf16_sat(orc_e2m1_to_f32(code));
                if (dstT == DT_BF16) ((uint16_t*)dst)[i] = orc_bf16_mul(sb, vb);
                else {
                    uint16_t sh = orc_f32_to_f16_sat(orc_bf16_to_f32(sb)), vh = orc_f32_to_f16_sat(orc_bf16_to_f32(vb));
                    ((uint16_t*)dst)[i] = orc_f16_mul(sh, vh);
                }
            }
        return OR_OK;
    }
    /* int4b_t (ascend_antiquant_impl.h:246-247, 512: Cast<half, int4b_t>): two signed nibbles per byte, even element low */
    if (srcT != DT_I8 && srcT != DT_I4X2) return OR_UNSUPPORTED;
    if (srcT == DT_I4X2 && (n & 1)) return OR_INVALID;

    if (policy == PER_TENSOR || policy == PER_CHANNEL) {
        if (dstT != DT_F16 && dstT != DT_BF16) return OR_UNSUPPORTED;
        ct = (dstT == DT_F16) ? DT_F16 : DT_F32;
        has_off = (policy == PER_TENSOR || unified) ? p->hasOffset : (offset != NULL);
        if (unified && policy == PER_CHANNEL && has_off && !offset) return OR_INVALID;
        if (policy == PER_TENSOR) {
            /* the scalars arrive as dstT values (ascend_antiquant.h:136-205) */
            float sc = (dstT == DT_F16) ? orc_f16_to_f32(orc_f32_to_f16_sat(scaleScalar)) : orc_bf16_to_f32(orc_f32_to_bf16_sat(scaleScalar));
            float of = (dstT == DT_F16) ? orc_f16_to_f32(orc_f32_to_f16_sat(offsetScalar)) : orc_bf16_to_f32(orc_f32_to_bf16_sat(offsetScalar));
            sref_scalar(&ss, sc); sref_scalar(&so, of);
        } else {
            if (!scale || scaleT != dstT) return OR_INVALID;
            uint32_t K = p->isTranspose ? n : rows;
            uint32_t gs = p->groupSize ? p->groupSize : K;
            if (gs == 0 || K % gs != 0) return OR_INVALID;
            if (!p->isTranspose) { sref_tensor(&ss, scale, scaleT, gs, 1, n); sref_tensor(&so, offset, scaleT, gs, 1, n); }
            else { sref_tensor(&ss, scale, scaleT, 1, gs, K / gs); sref_tensor(&so, offset, scaleT, 1, gs, K / gs); }
        }
    } else {
        if (!scale) return OR_INVALID;
        if (scaleT != DT_F16 && scaleT != DT_BF16 && scaleT != DT_F32) return OR_UNSUPPORTED;
        /* (dst, scale): (h,h) (bf,bf) (f,f) (h,f) (bf,f) -- tests/api/adv_api/quantization/antiquant/
         * test_ascend_antiquant_per_token.cpp:151-174 */
        if (scaleT != DT_F32 && dstT != scaleT) return OR_UNSUPPORTED;
        if (dstT != DT_F16 && dstT != DT_BF16 && dstT != DT_F32) return OR_UNSUPPORTED;
        ct = scaleT; has_off = p->hasOffset;
        if (has_off && !offset) return OR_INVALID;
        if (policy == PER_TOKEN) {
            if (p->isTranspose) { sref_tensor(&ss, scale, scaleT, 0, 1, 0); sref_tensor(&so, offset, scaleT, 0, 1, 0); }
            else { sref_tensor(&ss, scale, scaleT, 1, 0, 1); sref_tensor(&so, offset, scaleT, 1, 0, 1); }
        } else if (policy == PER_GROUP) {
            /* groups run along columns when (kDim==1 && !isTranspose) || (kDim==0 && isTranspose)
             * (ascend_antiquant_3510_impl.h:2214-2220) */
            int along_cols = (p->kDim == 1 && !p->isTranspose) || (p->kDim == 0 && p->isTranspose);
            int rc = policy_sref(&ss, scale, scaleT, PER_GROUP, rows, n, p->groupSize, along_cols ? 1 : 0);
            if (rc) return rc;
            policy_sref(&so, offset, scaleT, PER_GROUP, rows, n, p->groupSize, along_cols ? 1 : 0);
        } else return OR_UNSUPPORTED;
    }
    if (unified) ct = DT_F32;
#pragma omp parallel for schedule(static)
    for (uint32_t r = 0; r < rows; ++r) {
        for (uint32_t c = 0; c < n; ++c) {
            size_t i = (size_t)r * n + c;
            float xin;
            if (srcT == DT_I8) xin = (float)((const int8_t*)src)[i];
            else { uint8_t byte = ((const uint8_t*)src)[i >> 1]; int nib = (i & 1) ? (byte >> 4) : (byte & 0xF); xin = (float)((nib ^ 8) - 8); }
            cval x = cv_from_f32(xin, ct);
            if (has_off) x = cv_add(x, cv_from_f32(sref_get(&so, r, c), ct));
            x = cv_mul(x, cv_from_f32(sref_get(&ss, r, c), ct));
            if (ct == DT_F32) store_from_f32(dst, dstT, i, x.f);
            else ((uint16_t*)dst)[i] = x.h; /* dstT == ct */
        }
    }
    return OR_OK;
}

int ascq_oracle_antiquant(void* dst, int dstT, const void* src, int srcT, const void* offset, const void* scale,
                          int scaleT, float offsetScalar, float scaleScalar, int policy, const antiquant_param* p)
{
    return antiquant_common(dst, dstT, src, srcT, offset, scale, scaleT, offsetScalar, scaleScalar, policy, p, 0);
}

int ascq_oracle_antiquantize(void* dst, int dstT, const void* src, int srcT, const void* offset, const void* scale,
                             int scaleT, float offsetScalar, float scaleScalar, int policy, const quantize_param* q)
{
    if (!q) return OR_INVALID;
    antiquant_param p = {q->m, q->n, 0, policy == PER_GROUP ? q->groupSize : 0, q->hasOffset, 0, q->kDim};
    return antiquant_common(dst, dstT, src, srcT, offset, scale, scaleT, offsetScalar, scaleScalar, policy, &p, 1);
}

/* ------------------------------------------------------------------------------------------
 * W8A8 matmul with the vector-epilogue order of
 * examples/01_simd_cpp_api/05_best_practices/03_fusion_compute/quant_group_matmul_high_performance/
 * quant_group_matmul_custom.asc:425-454 (AscendDequant by the per-channel scale, Mul by the
 * per-token scale, cast).  The int32 accumulation is exact (Mmad, impl/adv_api/detail/matmul/stage/
 * compute/mmad_compute.h:83).  Adding a bf16 bias after the dequant is this library's definition
 * (the reference only has an int32 bias before the dequant).
 * A [M,K] int8 row-major, B [N,K] int8 row-major.
 * ---------------------------------------------------------------------------------------- */
int ascq_oracle_matmul_w8a8(uint16_t* C, const int8_t* A, const int8_t* B, const float* sA, const float* sB,
                            const uint16_t* bias, int M, int N, int K, int ldc, int32_t* accDump)
{
    if (!A || !B || M < 0 || N < 0 || K < 0) return OR_INVALID;
#pragma omp parallel for schedule(dynamic, 8)
    for (int m = 0; m < M; ++m) {
        const int8_t* a = A + (size_t)m * K;
        for (int n = 0; n < N; ++n) {
            const int8_t* b = B + (size_t)n * K;
            int32_t acc = 0;
            for (int k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
            if (accDump) accDump[(size_t)m * N + n] = acc;
            if (C) {
                float f = orc_i32_to_f32(acc);
                if (sB) f = f * sB[n];
                if (sA) f = f * sA[m];
                if (bias) f = f + orc_bf16_to_f32(bias[n]);
                C[(size_t)m * ldc + n] = orc_f32_to_bf16_sat(f);
            }
        }
    }
    return OR_OK;
}

/* ------------------------------------------------------------------------------------------
 * Grouped W8A8 matmul with per-group channel scales, per-token scales and an optional FasterGelu:
 * examples/01_simd_cpp_api/05_best_practices/03_fusion_compute/quant_group_matmul_high_performance/
 * quant_group_matmul_custom.asc:257-289 (group loop: groupList = rows per group, zero-row groups skipped),
 * :425-454 (vector side: AscendDequant x scale[g][n] -> Mul x perTokenScale[m] -> FasterGelu -> Cast to half).
 *   acc = sum_k A[m,k] * B[g,n,k]  (int32, exact);   f = (float(acc) * sB[g,n]) * sA[m]  (+ float(bias[g,n]));
 *   act: f = f / (1 + exp(-1.702 f))  -- impl/adv_api/detail/activation/gelu/gelu_impl.h:134-166, each step one fp32
 *        operation, the exponential correctly rounded here (the hardware's Exp is not pinned by anything in the tree);
 *   C = half(f) or bf16(f), round to nearest even.
 * A [sumM,K], B [G,N,K] (K-major), sA [sumM], sB [G,N], bias bf16 bits [G,N] or NULL (this library's addition).
 * outKind: 0 = half, 1 = bfloat16.
 * ---------------------------------------------------------------------------------------- */
int ascq_oracle_group_matmul_w8a8(uint16_t* C, const int8_t* A, const int8_t* B, const float* sA, const float* sB,
                                  const uint16_t* bias, const int64_t* groupList, int G, int N, int K, int outKind,
                                  int act, int32_t* accDump)
{
    if (!C || !A || !B || !groupList || G < 0 || N < 0 || K < 0) return OR_INVALID;
    int64_t start = 0;
    for (int g = 0; g < G; ++g) {
        const int64_t mg = groupList[g];
        if (mg < 0) return OR_INVALID;
#pragma omp parallel for schedule(dynamic, 8)
        for (int64_t r = 0; r < mg; ++r) {
            const int64_t m = start + r;
            const int8_t* a = A + (size_t)m * K;
            for (int n = 0; n < N; ++n) {
                const int8_t* b = B + ((size_t)g * N + n) * K;
                int32_t acc = 0;
                for (int k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
                if (accDump) accDump[(size_t)m * N + n] = acc;
                float f = orc_i32_to_f32(acc);
                if (sB) f = f * sB[(size_t)g * N + n];
                if (sA) f = f * sA[m];
                if (bias) f = f + orc_bf16_to_f32(bias[(size_t)g * N + n]);
                if (act) {
                    const float t = f * -1.702f;
                    const float e = (float)exp((double)t);
                    const float d = e + 1.0f;
                    f = f / d;
                }
                C[(size_t)m * N + n] = outKind == 1 ? orc_f32_to_bf16_sat(f) : orc_f32_to_f16_sat(f);
            }
        }
        start += mg;
    }
    return OR_OK;
}

/* ------------------------------------------------------------------------------------------
 * int8 matmul leaving through the fixpipe quantisation (Matmul::SetQuantScalar / SetQuantVector, mode DEQF16:
 * impl/adv_api/detail/matmul/stage/copy_cube_out/quant/quant_processor_fixpipe.h:80-119), with the arithmetic of
 * the sample's golden, examples/01_simd_cpp_api/04_advanced_api/00_matmul/matmul_quant/scripts/gen_data.py:26-44:
 *   y = A.B + bias (int32);  h = half(y) (RINT, overflow -> inf);
 *   scalar mode: C = h * half(quantScalar) in half;
 *   vector mode: C = half(float(h) * s), s = fp32 from the low word of quantVec[n] with the low 13 mantissa bits
 *                cleared ("1 sign bit, 8 exponent bits and 10 mantissa bits").
 * A [M,K], B [N,K] int8 row-major (the sample stores B [K,N]; the caller transposes).
 * ---------------------------------------------------------------------------------------- */
static uint16_t i32_to_f16_rint(int32_t v) { return f64_to_f16_ieee((double)v); } /* one rounding, IEEE overflow */

int ascq_oracle_matmul_i8_quant(uint16_t* C, const int8_t* A, const int8_t* B, const int32_t* bias,
                                const uint64_t* quantVec, float quantScalar, int M, int N, int K, int ldc)
{
    if (!C || !A || !B || M < 0 || N < 0 || K < 0) return OR_INVALID;
    const uint16_t hs = orc_f32_to_f16_sat(quantScalar);
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        for (int n = 0; n < N; ++n) {
            int32_t acc = 0;
            const int8_t* a = A + (size_t)m * K;
            const int8_t* b = B + (size_t)n * K;
            for (int k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
            if (bias) acc = (int32_t)((uint32_t)acc + (uint32_t)bias[n]);
            uint16_t h = i32_to_f16_rint(acc);
            uint16_t out;
            if (quantVec) {
                uint32_t bits = (uint32_t)(quantVec[n] & 0xFFFFFFFFull) & 0xFFFFE000u;
                float s; memcpy(&s, &bits, 4);
                out = f64_to_f16_ieee((double)(orc_f16_to_f32(h) * s)); /* fp32 product, then half (IEEE overflow) */
            } else {
                out = orc_f16_mul(h, hs);
            }
            C[(size_t)m * ldc + n] = out;
        }
    }
    return OR_OK;
}

/* ------------------------------------------------------------------------------------------
 * Fixpipe requantisation int32 -> int8 / uint8 ((V)REQ8), following the reference's description of the unit:
 * examples/01_simd_cpp_api/03_basic_api/03_matrix_compute/fixpipe_l0c2gm/scripts/gen_data_s322s8.py:39-64
 * (fields of the 64-bit parameter) and :75-97 (arithmetic), without the ReLU branch (negative values take the
 * same scale).  The scale is read as the fp32 whose low 13 bits are cleared; for a zero exponent field that
 * differs from the script's (1 + m/1024) * 2^-127, but either product is far below one half and rounds to 0.
 * Returns the result as an integer in [-128, 255].
 * ---------------------------------------------------------------------------------------- */
int ascq_oracle_req8(int32_t data, uint64_t q)
{
    uint32_t bits = (uint32_t)(q & 0xFFFFFFFFull) & 0xFFFFE000u;
    float alpha; memcpy(&alpha, &bits, 4);
    const unsigned shift = (unsigned)(q >> 32) & 15u, mcb = (unsigned)(q >> 36) & 1u;
    const int offset = (int)((q >> 37) & 0x1FFu), sign = (int)((q >> 46) & 1u);
    if (mcb) {
        data >>= shift; /* arithmetic */
        if (data < -32768) data = -32768;
        if (data > 32767) data = 32767;
    }
    volatile float f = (float)data * alpha; /* one fp32 rounding, as numpy does for float32 * python float */
    float c = f;
    if (!(c >= -256.0f)) c = -256.0f;
    if (c > 255.0f) c = 255.0f;
    int t = (int)nearbyintf(c) + offset;
    if (sign) { if (t < -128) t = -128; if (t > 127) t = 127; }
    else { if (t < 0) t = 0; if (t > 255) t = 255; }
    return t;
}

/* int8 matmul + int32 bias + (V)REQ8 (Matmul<int8, int8, int8> with SetQuantScalar / SetQuantVector,
 * quant_processor_fixpipe.h:93-95, 201-203).  C is a byte matrix [M, ldc]. */
int ascq_oracle_matmul_i8_requant(uint8_t* C, const int8_t* A, const int8_t* B, const int32_t* bias,
                                  const uint64_t* quantVec, uint64_t quantScalar, int M, int N, int K, int ldc)
{
    if (!C || !A || !B || M < 0 || N < 0 || K < 0) return OR_INVALID;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        for (int n = 0; n < N; ++n) {
            int32_t acc = 0;
            const int8_t* a = A + (size_t)m * K;
            const int8_t* b = B + (size_t)n * K;
            for (int k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
            if (bias) acc = (int32_t)((uint32_t)acc + (uint32_t)bias[n]);
            C[(size_t)m * ldc + n] = (uint8_t)(ascq_oracle_req8(acc, quantVec ? quantVec[n] : quantScalar) & 0xFF);
        }
    }
    return OR_OK;
}

/* ------------------------------------------------------------------------------------------
 * MX-FP4 grouped matmul.  Golden semantics of
 * examples/.../matmul_mxfp4_high_performance/scripts/gen_data.py:38-72 and
 * examples/.../03_matrix_compute/mmad_mx/scripts/gen_data.py: operands are dequantised
 * (value * 2^(e8m0-127), one scale per 32 K-elements), multiplied with double accumulation and cast
 * to bf16.  Grouping: groupList[g] rows per group, groups contiguous along M
 * (quant_group_matmul_custom.asc:257-289).  B is taken K-major: [G, N, K/2] bytes, sB [G, N, K/32].
 * ---------------------------------------------------------------------------------------- */
static double e8m0_to_f64(uint8_t e) { return (e == 0xFFu) ? NAN : ldexp(1.0, (int)e - 127); }

int ascq_oracle_group_matmul_mxfp4(uint16_t* C, float* C_f32, const uint8_t* A, const uint8_t* sA, const uint8_t* B,
                                   const uint8_t* sB, const int64_t* groupList, int G, int K, int N)
{
    if (!A || !B || !sA || !sB || !groupList || K % 32 != 0) return OR_INVALID;
    int64_t start = 0;
    const int KB = K / 2, KS = K / 32;
    for (int g = 0; g < G; ++g) {
        int64_t mg = groupList[g];
        if (mg < 0) return OR_INVALID;
        const uint8_t* Bg = B + (size_t)g * N * KB;
        const uint8_t* sBg = sB + (size_t)g * N * KS;
#pragma omp parallel
        {
            double* arow = (double*)malloc(sizeof(double) * (size_t)K);
#pragma omp for schedule(dynamic, 4)
            for (int64_t r = start; r < start + mg; ++r) {
                for (int k = 0; k < K; ++k) {
                    uint8_t byte = A[(size_t)r * KB + k / 2];
                    uint8_t code = (k & 1) ? (byte >> 4) : (byte & 0x0Fu);
                    arow[k] = (double)orc_e2m1_to_f32(code) * e8m0_to_f64(sA[(size_t)r * KS + k / 32]);
                }
                for (int n = 0; n < N; ++n) {
                    double acc = 0.0;
                    const uint8_t* brow = Bg + (size_t)n * KB;
                    for (int kb = 0; kb < KS; ++kb) {
                        double part = 0.0;
                        for (int k = kb * 32; k < kb * 32 + 32; ++k) {
                            uint8_t byte = brow[k / 2];
                            uint8_t code = (k & 1) ? (byte >> 4) : (byte & 0x0Fu);
                            part += arow[k] * (double)orc_e2m1_to_f32(code);
                        }
                        acc += part * e8m0_to_f64(sBg[(size_t)n * KS + kb]);
                    }
                    if (C) C[(size_t)r * N + n] = orc_f32_to_bf16_sat((float)acc);
                    if (C_f32) C_f32[(size_t)r * N + n] = (float)acc;
                }
            }
            free(arow);
        }
        start += mg;
    }
    return OR_OK;
}

/* half / bfloat16 matmul: products exact, sum in double (the samples' goldens use fp64 / fp32 numpy matmuls), one
 * cast to the output type.  A [M,K], B [N,K] as 16-bit patterns; returns fp32 and, when C16 is given, the cT cast.
 * The weight-only-quantised matmul of the reference (Matmul::SetAntiQuantVector, antiquant_processor_using_ub.h:86-137)
 * is this matmul applied to AscendAntiQuant's output. */
int ascq_oracle_matmul_f16(uint16_t* C16, float* C_f32, int cT, const uint16_t* A, const uint16_t* B, int abT, int M, int N, int K)
{
    if (!A || !B || M < 0 || N < 0 || K < 0) return OR_INVALID;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            double acc = 0.0;
            for (int k = 0; k < K; ++k) {
                const uint16_t a = A[(size_t)m * K + k], b = B[(size_t)n * K + k];
                const double af = abT == DT_BF16 ? (double)orc_bf16_to_f32(a) : (double)orc_f16_to_f32(a);
                const double bf = abT == DT_BF16 ? (double)orc_bf16_to_f32(b) : (double)orc_f16_to_f32(b);
                acc += af * bf;
            }
            if (C_f32) C_f32[(size_t)m * N + n] = (float)acc;
            if (C16) C16[(size_t)m * N + n] = cT == DT_BF16 ? orc_f32_to_bf16_sat((float)acc) : f64_to_f16_ieee((double)(float)acc);
        }
    return OR_OK;
}

/* Fixpipe quantisation of an fp32 accumulator to int8 / uint8 ((V)QF322B8_PRE), following
 * examples/01_simd_cpp_api/03_basic_api/03_matrix_compute/fixpipe_l0c2gm/scripts/gen_data_f322s8.py:75-97 without its
 * ReLU branch: data * scale in fp32, clamp to [-256, 255], RINT, + offset, clamp to the result type.  The shift
 * fields of the parameter word do not apply to this mode (随路量化.md:54-55) and are ignored. */
int ascq_oracle_qf322b8(float data, uint64_t q)
{
    uint32_t bits = (uint32_t)(q & 0xFFFFFFFFull) & 0xFFFFE000u;
    float alpha; memcpy(&alpha, &bits, 4);
    const int offset = (int)((q >> 37) & 0x1FFu), sign = (int)((q >> 46) & 1u);
    volatile float f = data * alpha;
    float c = f;
    if (!(c >= -256.0f)) c = -256.0f;
    if (c > 255.0f) c = 255.0f;
    int t = (int)nearbyintf(c) + offset;
    if (sign) { if (t < -128) t = -128; if (t > 127) t = 127; }
    else { if (t < 0) t = 0; if (t > 255) t = 255; }
    return t;
}

/* half / bfloat16 matmul (products summed in double, rounded once to fp32) + (V)QF322B8_PRE: Matmul<half, half, int8>
 * with SetQuantScalar / SetQuantVector (quant_processor_fixpipe.h:95-97, 203-205).  C is a byte matrix [M, ldc]. */
int ascq_oracle_matmul_f16_quant(uint8_t* C, const uint16_t* A, const uint16_t* B, int abT, const uint64_t* quantVec,
                                 uint64_t quantScalar, int M, int N, int K, int ldc)
{
    if (!C || !A || !B || M < 0 || N < 0 || K < 0) return OR_INVALID;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            double acc = 0.0;
            for (int k = 0; k < K; ++k) {
                const uint16_t a = A[(size_t)m * K + k], b = B[(size_t)n * K + k];
                const double af = abT == DT_BF16 ? (double)orc_bf16_to_f32(a) : (double)orc_f16_to_f32(a);
                const double bf = abT == DT_BF16 ? (double)orc_bf16_to_f32(b) : (double)orc_f16_to_f32(b);
                acc += af * bf;
            }
            C[(size_t)m * ldc + n] = (uint8_t)(ascq_oracle_qf322b8((float)acc, quantVec ? quantVec[n] : quantScalar) & 0xFF);
        }
    return OR_OK;
}

/* MX matmul with 8-bit operands (fp8_e4m3fn / fp8_e5m2, one E8M0 scale per 32 elements of K), grouped like the fp4
 * one.  Golden formula: examples/01_simd_cpp_api/04_advanced_api/00_matmul/matmul_mx/scripts/gen_data.py:52-66 and
 * examples/01_simd_cpp_api/03_basic_api/03_matrix_compute/mmad_mx/scripts/gen_data.py (mx_decompress, fp64 matmul,
 * result cast to fp32).  aFmt / bFmt: 0 = E4M3 (bias 7, no infinity, S.1111.111 = NaN), 1 = E5M2 (the top byte of a half). */
double orc_fp8_to_f64(uint8_t v, int fmt)
{
    if (fmt == 1) return (double)orc_f16_to_f32((uint16_t)((uint16_t)v << 8));
    int sign = v >> 7, e = (v >> 3) & 0xF, m = v & 7;
    double r;
    if (e == 0xF && m == 7) return NAN;
    if (e == 0) r = ldexp((double)m, -9);            /* subnormal: m/8 * 2^-6 */
    else r = ldexp(1.0 + (double)m / 8.0, e - 7);
    return sign ? -r : r;
}

int ascq_oracle_group_matmul_mxfp8(uint16_t* C, float* C_f32, const uint8_t* A, int aFmt, const uint8_t* sA, const uint8_t* B,
                                   int bFmt, const uint8_t* sB, const int64_t* groupList, int G, int K, int N)
{
    if (!A || !B || !sA || !sB || !groupList || K % 32 != 0) return OR_INVALID;
    int64_t start = 0;
    const int KS = K / 32;
    for (int g = 0; g < G; ++g) {
        int64_t mg = groupList[g];
        if (mg < 0) return OR_INVALID;
        const uint8_t* Bg = B + (size_t)g * N * K;
        const uint8_t* sBg = sB + (size_t)g * N * KS;
#pragma omp parallel
        {
            double* arow = (double*)malloc(sizeof(double) * (size_t)K);
#pragma omp for schedule(dynamic, 4)
            for (int64_t r = start; r < start + mg; ++r) {
                for (int k = 0; k < K; ++k)
                    arow[k] = orc_fp8_to_f64(A[(size_t)r * K + k], aFmt) * e8m0_to_f64(sA[(size_t)r * KS + k / 32]);
                for (int n = 0; n < N; ++n) {
                    double acc = 0.0;
                    const uint8_t* brow = Bg + (size_t)n * K;
                    for (int kb = 0; kb < KS; ++kb) {
                        double part = 0.0;
                        for (int k = kb * 32; k < kb * 32 + 32; ++k) part += arow[k] * orc_fp8_to_f64(brow[k], bFmt);
                        acc += part * e8m0_to_f64(sBg[(size_t)n * KS + kb]);
                    }
                    if (C) C[(size_t)r * N + n] = orc_f32_to_bf16_sat((float)acc);
                    if (C_f32) C_f32[(size_t)r * N + n] = (float)acc;
                }
            }
            free(arow);
        }
        start += mg;
    }
    return OR_OK;
}

/* ------------------------------------------------------------------------------------------
 * Host tmp-size formulas.
 *   impl/adv_api/tiling/quantization/ascend_quant_tiling_impl.cpp:31-69
 *   impl/adv_api/tiling/quantization/ascend_dequant_tiling_impl.cpp:31-106
 *   impl/adv_api/tiling/quantization/ascend_antiquant_tiling_impl.cpp:71-181
 * ---------------------------------------------------------------------------------------- */
static int64_t shape_size(const int64_t* d, int rank) { int64_t s = 1; for (int i = 0; i < rank; ++i) s *= d[i]; return s; }

int ascq_oracle_quant_tmp_size(const int64_t* dims, int rank, uint32_t typeSize, uint32_t* maxV, uint32_t* minV)
{
    int64_t sz = shape_size(dims, rank);
    if (sz <= 0 || (sz * typeSize) % 32 != 0 || (typeSize != 2 && typeSize != 4)) return OR_INVALID;
    uint32_t mx = (uint32_t)sz * 2u; if (mx < 512u) mx = 512u;
    *maxV = (mx + 31u) / 32u * 32u; *minV = 512u;
    return OR_OK;
}
void ascq_oracle_quant_factor(uint32_t* live, uint32_t* extra) { *live = 2; *extra = 0; }

int ascq_oracle_dequant_tmp_size(const int64_t* dims, int rank, uint32_t typeSize, uint32_t* maxV, uint32_t* minV)
{
    if (shape_size(dims, rank) <= 0 || rank < 1 || rank > 2 || typeSize != 4) return OR_INVALID;
    uint32_t outer = (rank == 2) ? (uint32_t)dims[0] : 1u, inner = (rank == 2) ? (uint32_t)dims[1] : (uint32_t)dims[0];
    uint32_t deq = inner + 8u;
    *maxV = (64u + outer * inner + deq) * 4u; *minV = (64u + inner + deq) * 4u;
    return OR_OK;
}
void ascq_oracle_dequant_factor(const int64_t* dims, int rank, uint32_t* live, uint32_t* extra)
{
    *extra = 8u + 64u;
    if (rank == 2) { *extra += (uint32_t)dims[1]; *live = 1; }
    else if (rank == 1) *live = 2;
    else { *extra = 0; *live = 0; }
}
static uint32_t antiquant_tmp(const int64_t* sd, int sr, const int64_t* cd, int cr, int tr, int inT, int outT, int want_max)
{
    uint32_t scaleSize = (uint32_t)shape_size(cd, cr), srcSize = (uint32_t)shape_size(sd, sr);
    if (inT == DT_FP4X2_E2M1) return tr ? (scaleSize + 31u) / 32u * 32u * 2u : 0u;
    if (outT == DT_F16) return 0;
    int perch = scaleSize != 1;
    if (!perch) return want_max ? srcSize * 4u : 1024u;
    if (tr) return 80u * scaleSize * 4u;
    return scaleSize * 2u * 4u + 64u * (uint32_t)sd[0] * 4u;
}
int ascq_oracle_antiquant_tmp_size(const int64_t* sd, int sr, const int64_t* cd, int cr, int tr, int inT, int outT,
                                   uint32_t* maxV, uint32_t* minV)
{
    if (shape_size(sd, sr) <= 0 || sr < 2) return OR_INVALID;
    *maxV = antiquant_tmp(sd, sr, cd, cr, tr, inT, outT, 1);
    *minV = antiquant_tmp(sd, sr, cd, cr, tr, inT, outT, 0);
    return OR_OK;
}
void ascq_oracle_antiquant_factor(const int64_t* sd, int sr, const int64_t* cd, int cr, int tr, int inT, int outT,
                                  uint32_t* live, uint32_t* extra)
{
    (void)sr;
    uint32_t scaleSize = (uint32_t)shape_size(cd, cr);
    int perch = scaleSize != 1;
    *extra = 0; *live = 0;
    if (inT == DT_FP4X2_E2M1) { if (tr) *extra = (scaleSize + 31u) / 32u * 32u * 2u; }
    else if (outT == DT_F16) *live = 0;
    else if (tr && perch) *extra = 80u * scaleSize * 4u;
    else if (!perch) *live = 1;
    else *extra = scaleSize * 2u * 4u + 64u * (uint32_t)sd[0] * 4u;
}

int ascq_oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
