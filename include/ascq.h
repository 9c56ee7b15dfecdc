/*
 * ascq.h -- C ABI of the B200 (sm_100a) quantized-inference operators.
 *
 * Every entry point replaces one operator (or one host helper) of the Ascend C
 * high-level API; the reference file:line each one follows is cited beside it
 * (paths are relative to the asc-devkit source tree).
 *
 * Conventions (all entry points):
 *   - every tensor pointer is a DEVICE pointer owned by the caller;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = the
 *     legacy default stream) and the call returns without synchronising;
 *   - no entry point allocates or frees device memory unless its comment says so;
 *   - argument errors are reported by return code (the reference aborts through
 *     ASCENDC_ASSERT in CPU-debug builds, impl/basic_api/kernel_log.h:41-71);
 *     ascq_last_error() returns a thread-local description of the last failure;
 *   - there is no CPU fallback: without a CUDA device the compute calls fail
 *     with ASCQ_ERR_CUDA.
 */
#ifndef ASCQ_H_
#define ASCQ_H_

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ASCQ_VERSION_MAJOR 0
#define ASCQ_VERSION_MINOR 1

typedef enum {
    ASCQ_OK = 0,
    ASCQ_ERR_INVALID_ARG = 1,  /* a rule the reference checks with ASCENDC_ASSERT is violated          */
    ASCQ_ERR_UNSUPPORTED = 2,  /* dtype / policy combination the reference static_asserts away         */
    ASCQ_ERR_ALIGNMENT = 3,    /* pointer or extent not aligned for the vectorised path                */
    ASCQ_ERR_CUDA = 4,         /* a CUDA runtime / driver call failed                                  */
    ASCQ_ERR_NCCL = 5,         /* multi-GPU set-up failed: invalid communicator, peer memory could not be mapped   */
    ASCQ_ERR_TIMEOUT = 6       /* a bounded device-side wait expired (kernel left cleanly)             */
} ascq_status;

/* Element types.  fp4x2 = two E2M1 values per byte, element 2i in the low nibble
 * (include of impl/utils/common_types.h:33-47; packing as in
 * examples/.../matmul_mxfp4_high_performance/scripts/gen_data.py:25-35). */
typedef enum {
    ASCQ_DT_F16 = 0,
    ASCQ_DT_BF16 = 1,
    ASCQ_DT_F32 = 2,
    ASCQ_DT_I8 = 3,
    ASCQ_DT_I32 = 4,
    ASCQ_DT_U64 = 5,        /* AscendDequant scale: low 32 bits hold fp32 bits */
    ASCQ_DT_FP4X2_E2M1 = 6,
    ASCQ_DT_E8M0 = 7,
    ASCQ_DT_FP8_E4M3 = 8,   /* fp8_e4m3fn_t / fp8_e5m2_t: operands of ascq_group_matmul_mxfp8 only; as quantisation */
    ASCQ_DT_FP8_E5M2 = 9,   /* targets or antiquant sources they are declared by the reference and not built here  */
    ASCQ_DT_HIF8 = 10,      /* declared by the reference, not built here: ASCQ_ERR_UNSUPPORTED */
    ASCQ_DT_FP4X2_E1M2 = 11,
    ASCQ_DT_I4X2 = 12       /* int4b_t, two per byte (even element in the low nibble): AscendAntiQuant source only */
} ascq_dtype;

/* include/adv_api/quantization/ascend_quant_utils.h:73-80 (same order in the
 * antiquant enum, impl/adv_api/detail/quantization/antiquant/ascend_antiquant_common.h:51-58). */
typedef enum {
    ASCQ_PER_TENSOR = 0,
    ASCQ_PER_CHANNEL = 1,
    ASCQ_PER_TOKEN = 2,
    ASCQ_PER_GROUP = 3,
    ASCQ_PER_CHANNEL_PER_GROUP = 4, /* declared, static_assert'ed away by every implementation */
    ASCQ_PER_TOKEN_PER_GROUP = 5
} ascq_policy;

/* impl/basic_api/utils/kernel_utils_mode.h:94-108.  CAST_NONE behaves as CAST_RINT
 * whenever the conversion is lossy (docs .../precision_conversion.md:19-20). */
typedef enum {
    ASCQ_CAST_NONE = 0,
    ASCQ_CAST_RINT = 1,  /* round half to even            */
    ASCQ_CAST_FLOOR = 2,
    ASCQ_CAST_CEIL = 3,
    ASCQ_CAST_ROUND = 4, /* round half away from zero     */
    ASCQ_CAST_TRUNC = 5
} ascq_round;

/* AscendQuantParam + the run-time relevant fields of AscendQuantConfig
 * (include/adv_api/quantization/ascend_quant_utils.h:31-87). */
typedef struct {
    uint32_t m;          /* rows (tokens)                                                     */
    uint32_t n;          /* columns (channels); PER_CHANNEL: scaleCount                       */
    uint32_t calCount;   /* elements to process; multiple of n for every policy but PER_TENSOR */
    uint32_t groupSize;  /* PER_GROUP only; multiple of 32                                    */
    int32_t hasOffset;   /* PER_TOKEN / PER_GROUP: add the offset tensor                      */
    int32_t kDim;        /* PER_GROUP: 1 = groups along n, 0 = groups along m                 */
    ascq_round roundMode;
} ascq_quant_param;

/* DequantParams / AscendDeQuantParam (include/adv_api/quantization/ascend_dequant_utils.h:26-44). */
typedef struct {
    uint32_t m;
    uint32_t n;
    uint32_t calCount;   /* PER_TENSOR / PER_CHANNEL: columns of each row that are scaled (<= n);
                            PER_TOKEN / PER_GROUP: total element count (multiple of n)           */
    uint32_t groupSize;
    int32_t kDim;
} ascq_dequant_param;

/* AscendAntiQuantParam + AscendAntiQuantConfig + the K / AntiQuantShapeInfo arguments of the
 * legacy overloads (ascend_antiquant_common.h:45-66, include/adv_api/quantization/ascend_antiquant_utils.h:27-32). */
typedef struct {
    uint32_t m;          /* src rows    : K when !isTranspose, N when isTranspose (legacy);
                            tokens for the policy overloads                                     */
    uint32_t n;          /* src columns : N when !isTranspose, K when isTranspose               */
    uint32_t calCount;   /* elements to process (multiple of n); 0 = m*n                        */
    uint32_t groupSize;  /* PER_CHANNEL: 0 = one scale row/column for the whole K extent
                            (scale shape [1,N] or [N,1]); else K/groupSize scale rows/columns.
                            PER_GROUP: group length; fp4 source: fixed to 32                    */
    int32_t hasOffset;
    int32_t isTranspose;
    int32_t kDim;
} ascq_antiquant_param;

const char* ascq_status_string(ascq_status s);
/* Thread-local text of the most recent non-OK status returned on this thread ("" if none). */
const char* ascq_last_error(void);
/* major*100 + minor */
int ascq_version(void);

/*
 * AscendQuant.  dst = sat(round(x * scale + offset)) evaluated with the reference's operation
 * sequence (two separately rounded operations, never a fused multiply-add):
 *   PER_TENSOR  include/adv_api/quantization/ascend_quant.h:63-97, arithmetic
 *               impl/adv_api/detail/quantization/quant/ascend_quant_pre_impl.h:320-397: src -> half,
 *               half mul, half add, half -> int8 (RINT, saturate).  scale/offset come from
 *               scaleScalar/offsetScalar; `scale`/`offset` must be NULL.
 *   PER_CHANNEL ascend_quant.h:159-347, ascend_quant_pre_impl.h:101-209,399-483: same half
 *               arithmetic with scale[n] (dtype scaleT = half or float; float is rounded to half
 *               first) and either offset[n] (offset != NULL) or offsetScalar.
 *   PER_TOKEN / PER_GROUP  ascend_quant.h:667-762, impl .../ascend_quant_per_group_3510_impl.h:
 *               arithmetic in scaleT, scale (and offset when hasOffset) shaped [m] /
 *               [m, ceil(n/groupSize)] (kDim 1) / [ceil(m/groupSize), n] (kDim 0);
 *               to-int8 chain .../ascend_quant_3510_impl.h:934-992.
 * dstT: ASCQ_DT_I8 (all policies) or ASCQ_DT_FP4X2_E2M1 (PER_GROUP, no offset).
 */
ascq_status ascq_quant(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT,
                       const void* scale, const void* offset, ascq_dtype scaleT,
                       float scaleScalar, float offsetScalar, ascq_policy policy,
                       const ascq_quant_param* param, void* stream);

/*
 * Dynamic per-token quantisation front end (no counterpart in the reference, which always takes
 * the scale as an input): scaleOut[row] = 127 / max|x[row,:]| in fp32 (1.0 for an all-zero row),
 * then AscendQuant PER_TOKEN with scaleT = float, no offset, CAST_RINT.  One pass over src.
 * deqScaleOut[row] (optional) receives max|x|/127, the per-token scale the W8A8 matmul wants.
 */
ascq_status ascq_dynamic_quant_per_token(int8_t* dst, float* scaleOut, float* deqScaleOut, const void* src,
                                         ascq_dtype srcT, uint32_t m, uint32_t n, void* stream);

/*
 * Dynamic MX-FP4 block quantisation (no counterpart in the reference, which always takes its scales as inputs): turns
 * activations into the operand format of ascq_group_matmul_mxfp4 on the GPU.  For every block of 32 consecutive
 * elements of a row: amax = max |x|; shared exponent e = floor(log2(amax)) - 2 clamped to [-127, 127] (0 for an
 * all-zero block), scale byte = e + 127 (0xFF if the block holds a NaN or an infinity, its codes are then 0);
 * code = e2m1(bf16(x * 2^-e)), both roundings to nearest even, saturating at +-6 -- the conversion chain of
 * AscendQuant's fp4 destination (ascend_quant_3510_impl.h:994-1032).  dst [m, n/2] bytes (even element in the low
 * nibble), scale [m, n/32]; n % 32 == 0.
 */
ascq_status ascq_dynamic_quant_mxfp4(uint8_t* dst_fp4, uint8_t* scale_e8m0, const void* src, ascq_dtype srcT, uint32_t m,
                                     uint32_t n, void* stream);

/*
 * AscendDequant.  dst = cast(float(src) * scale), fp32 arithmetic, final cast RINT + saturate.
 *   PER_TENSOR  scalar deqScale overloads, include/adv_api/quantization/ascend_dequant.h:186-281
 *               (scaleScalar; `scale` NULL).
 *   PER_CHANNEL ascend_dequant.h:59-181, impl .../dequant/ascend_dequant_common_impl.h:365-429:
 *               scale[>=calCount] of scaleT in {U64, F32, BF16}; the first calCount columns of
 *               each of the m rows are scaled; dst rows start every dstStride elements, where
 *               dstStride = n rounded up to 32 bytes of dstT (ascend_dequant_common_impl.h:100-105).
 *               tokScale (optional, fp32 [m]) multiplies each row AFTER the per-channel scale,
 *               still in fp32 -- the order of the grouped-matmul epilogue,
 *               examples/.../quant_group_matmul_high_performance/quant_group_matmul_custom.asc:433-441.
 *   PER_TOKEN / PER_GROUP  ascend_dequant.h:286-307, impl .../ascend_dequant_3510_impl.h:226-296,
 *               337-446: srcT in {I32, F32}; scale [m] or grouped as for AscendQuant.
 * dstT in {F16, BF16, F32}.
 */
ascq_status ascq_dequant(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT,
                         const void* scale, const float* tokScale, ascq_dtype scaleT, float scaleScalar,
                         ascq_policy policy, const ascq_dequant_param* param, void* stream);

/*
 * AscendAntiQuant.  dst = scale * (src + offset)  (include/adv_api/quantization/ascend_antiquant.h:37).
 *   PER_TENSOR  scalar overloads ascend_antiquant.h:136-205 (offsetScalar / scaleScalar).
 *   PER_CHANNEL legacy tensor overloads ascend_antiquant.h:50-134; layouts
 *               impl/.../antiquant/ascend_antiquant_impl.h:283-408: !isTranspose: src [K,N],
 *               scale/offset [K/groupSize, N]; isTranspose: src [N,K], scale/offset [N, K/groupSize].
 *               dst bf16: int8 -> fp32, fp32 add, fp32 mul, RINT to bf16
 *               (ascend_antiquant_c220_impl.h:45-102); dst half: half add, half mul
 *               (ascend_antiquant_impl.h:62-76).  scaleT must equal dstT.
 *   PER_TOKEN / PER_GROUP  ascend_antiquant.h:233-262, impl .../ascend_antiquant_3510_impl.h:
 *               1458-1495, 2167-2222: arithmetic in scaleT, result cast to dstT.
 *   srcT = FP4X2_E2M1 with scaleT = E8M0 (ascend_antiquant.h:211-231, impl :49-138): one scale per
 *               32 K-elements, no offset; scale byte e -> 2^(e-127), 0x00 -> 2^-127, 0xFF -> NaN.
 */
ascq_status ascq_antiquant(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT,
                           const void* offset, const void* scale, ascq_dtype scaleT,
                           float offsetScalar, float scaleScalar, ascq_policy policy,
                           const ascq_antiquant_param* param, void* stream);

/*
 * The unified interface Quantize / Dequantize / AntiQuantize (include/adv_api/quantization/quantize.h:41-62,
 * dequantize.h, antiquantize.h; QuantizeConfig{policy, hasOffset, roundMode, kDim} and QuantizeParams{m, n, groupSize}
 * in quantize_utils.h:34-47 become one run-time struct).  Same tensors and policies as the Ascend* calls above, but
 * every policy computes in fp32: operands widened to fp32, one rounded multiply and one rounded add, one final cast
 * (impl/adv_api/detail/quantization/quantize/quantize_impl.h:832-975,
 *  antiquantize/antiquantize_3510_impl.h:252-381, dequantize/dequantize_impl.h:100-215).
 *   ascq_quantize      dst = cast(float(src) * float(scale) [+ float(offset)]), cast with roundMode + saturation;
 *                      PER_TENSOR: scalars; PER_CHANNEL: scale[n] and offset[n] (or scalar offset when `offset` is
 *                      NULL); PER_TOKEN: [m]; PER_GROUP: as ascq_quant.  (src, scale) dtypes (T, T) or (T, float).
 *   ascq_dequantize    forwards to ascq_dequant on whole rows; hasOffset must be 0.
 *   ascq_antiquantize  dst = cast((float(src) + float(offset)) * float(scale)); int8 source, never transposed;
 *                      PER_TENSOR: scalars rounded to dstT; PER_CHANNEL: [n] of dstT; PER_TOKEN: [m]; PER_GROUP.
 */
typedef struct ascq_quantize_param {
    uint32_t m, n, groupSize;
    int32_t hasOffset;
    int32_t kDim;
    ascq_round roundMode; /* ascq_quantize only */
} ascq_quantize_param;
ascq_status ascq_quantize(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT, const void* scale,
                          const void* offset, ascq_dtype scaleT, float scaleScalar, float offsetScalar,
                          ascq_policy policy, const ascq_quantize_param* param, void* stream);
ascq_status ascq_dequantize(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT, const void* scale,
                            ascq_dtype scaleT, float scaleScalar, ascq_policy policy,
                            const ascq_quantize_param* param, void* stream);
ascq_status ascq_antiquantize(void* dst, ascq_dtype dstT, const void* src, ascq_dtype srcT, const void* offset,
                              const void* scale, ascq_dtype scaleT, float offsetScalar, float scaleScalar,
                              ascq_policy policy, const ascq_quantize_param* param, void* stream);

/*
 * W8A8 matmul with fused dequant epilogue (AscendC::Matmul<int8,int8,int32> +
 * AscendDequant per-channel x per-token; include/adv_api/matmul/matmul.h:79-398,
 * impl/adv_api/detail/matmul/stage/compute/mmad_compute.h:83, epilogue order
 * examples/.../quant_group_matmul_custom.asc:425-454):
 *   acc[m,n] = sum_k A[m,k] * B[n,k]                       (int32, exact)
 *   C[m,n]   = bf16_rint( (float(acc) * sB[n]) * sA[m] + float(bias[n]) )
 * A [M,K] row-major int8; B [N,K] row-major ("K-major", SetTensorB(..., isTransposeB=true)).
 * sA fp32 [M] or NULL (=1), sB fp32 [N] or NULL (=1), bias bf16 [N] or NULL.  The bf16 bias added
 * after the dequantisation is this library's definition (the reference's bias is int32, added
 * before it).  ldc = row stride of C in elements (>= N).  accDump (optional) receives the raw
 * int32 accumulators, [M,N] row-major; C may be NULL when only accDump is wanted.
 * K % 16 == 0; A, B 16-byte aligned (TMA).
 * Two kernels produce the same bits: the tcgen05 kernel, and -- for M <= 32 with K % 128 == 0, A and B 32-byte aligned,
 * no accDump -- a kernel shaped for reading the weight once (the product is then bound by the N x K weight bytes;
 * ASCQ_W8A8_SMALL=0 in the environment keeps such calls on the tcgen05 kernel).
 */
ascq_status ascq_matmul_w8a8(void* C_bf16, const int8_t* A, const int8_t* B_nk, const float* sA_m,
                             const float* sB_n, const void* bias_bf16, int M, int N, int K, int ldc,
                             int32_t* accDump, void* stream);

/*
 * Grouped W8A8 matmul with per-group channel scales and per-token scales: the reference's fused sample
 * examples/01_simd_cpp_api/05_best_practices/03_fusion_compute/quant_group_matmul_high_performance
 * (quant_group_matmul_custom.asc:257-289 group loop, :425-454 vector side; golden scripts/gen_data.py:26-69).
 *   for each group g with rows [s_g, s_g + groupList[g]):
 *     acc[r, n] = sum_k A[r, k] * B[g, n, k]                                    (int32, exact)
 *     f = (float(acc) * sB[g, n]) * sA[r]   (+ float(bias[g, n]))               (separately rounded fp32 operations)
 *     activation 1:  f = f / (1 + exp(-1.702 f))   (FasterGelu, impl/adv_api/detail/activation/gelu/gelu_impl.h:134-166)
 *     C[r, n] = half(f) or bfloat16(f)
 * A int8 [sumM, K]; B int8 [G, N, K] K-major (the sample's [G, K, N] weight is turned once per group with
 * ascq_transpose_i8_kn_to_nk); sA fp32 [sumM] or NULL; sB fp32 [G, N] or NULL; bias bf16 [G, N] or NULL (this library's
 * addition, as in ascq_matmul_w8a8); groupList int64 [G] on the HOST = rows per group, zero-row groups are skipped;
 * C [sumM, N] of cT = ASCQ_DT_F16 (the sample's type) or ASCQ_DT_BF16.  K % 16 == 0, G <= 128.
 * Without the activation the result is bit-exact; the exponential of FasterGelu is the CUDA library's expf (the
 * reference's Exp instruction is not pinned by anything in its tree), so results can differ from a correctly rounded
 * evaluation by one step of the output type.
 */
ascq_status ascq_group_matmul_w8a8(void* C, ascq_dtype cT, const int8_t* A, const int8_t* B_gnk, const float* sA_m,
                                   const float* sB_gn, const void* bias_bf16_gn, const int64_t* groupList_host,
                                   int G, int N, int K, int activation, void* stream);

/*
 * MX-FP4 grouped matmul (MatmulWithScalePolicy, impl/adv_api/detail/matmul/mx_matmul_impl.h:29-181;
 * grouping examples/.../quant_group_matmul_custom.asc:257-289):
 *   for each group g with rows [s_g, s_g + groupList[g]):
 *     C[r, n] = bf16( sum_k (A[r,k] * 2^(sA[r,k/32]-127)) * (B[g,n,k] * 2^(sB[g,n,k/32]-127)) )
 * A  fp4x2 [sumM, K/2] bytes, sA e8m0 [sumM, K/32];
 * B  fp4x2 [G, N, K/2] bytes (K-major), sB e8m0 [G, N, K/32];
 * groupList int64 [G] on the HOST = rows per group (not cumulative); zero-row groups are skipped.
 * C bf16 [sumM, N].  fp32 accumulation.  K % 128 == 0, N % 8 == 0.
 * workspace: device scratch of at least ascq_group_matmul_mxfp4_workspace_size() bytes, 256-byte
 * aligned, private to this call until the stream reaches the end of it.
 */
ascq_status ascq_group_matmul_mxfp4(void* C_bf16, const uint8_t* A_fp4, const uint8_t* sA_e8m0,
                                    const uint8_t* B_fp4, const uint8_t* sB_e8m0,
                                    const int64_t* groupList_host, int G, int K, int N,
                                    void* workspace, size_t workspaceBytes, void* stream);
size_t ascq_group_matmul_mxfp4_workspace_size(int64_t sumM, int G, int K, int N);

/*
 * Static weights: the scales of B can be brought into the kernel's packed order once instead of on every call.
 * ascq_group_matmul_mxfp4_pack_scale_b writes ascq_group_matmul_mxfp4_packed_scale_b_size(G, K, N) bytes (256-byte
 * aligned); ascq_group_matmul_mxfp4_prepacked takes that buffer in place of sB_e8m0 and repacks only the scales of A
 * (the reference likewise expects its weights in a prepared layout: README_en.md:64-67 of matmul_mxfp4_high_performance).
 */
size_t ascq_group_matmul_mxfp4_packed_scale_b_size(int G, int K, int N);
ascq_status ascq_group_matmul_mxfp4_pack_scale_b(uint8_t* sB_packed, const uint8_t* sB_e8m0, int G, int K, int N, void* stream);
ascq_status ascq_group_matmul_mxfp4_prepacked(void* C_bf16, const uint8_t* A_fp4, const uint8_t* sA_e8m0,
                                              const uint8_t* B_fp4, const uint8_t* sB_packed,
                                              const int64_t* groupList_host, int G, int K, int N, void* workspace,
                                              size_t workspaceBytes, void* stream);

/*
 * The same grouped matmul for callers that cannot hand over scratch memory.  It has no counterpart in
 * the reference.  Some hosts of this library must not create device allocations of their own: an
 * inference server that has given all of HBM to its own memory pool at start-up (a cudaMalloc from a
 * plug-in then fails, or eats into what the pool counted on), or a latency-critical serving thread that
 * cannot afford the device-wide synchronisation a cudaMalloc / cudaFree implies.  For them the tile
 * table and the repacked scales go into an array that is compiled into the library (16 MiB, reported by
 * ascq_group_matmul_mxfp4_noalloc_max_scratch(); every GPU that loads the library keeps it until the
 * process exits).  The call makes no cudaMalloc, cudaFree or other allocating call.
 *   - Problems whose scratch need (ascq_group_matmul_mxfp4_workspace_size) exceeds the array are
 *     rejected with ASCQ_ERR_INVALID_ARG; use the workspace variant for those.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current); make that first call outside any stream capture.
 *   - All calls on a device share the one array and it keeps what the previous call left there.  Each
 *     call rewrites everything it later reads, so no clearing is needed, but two calls whose kernels can
 *     overlap on the GPU (different streams, no ordering between them) race on it: serialise them.
 * Arguments and results are those of ascq_group_matmul_mxfp4.
 */
ascq_status ascq_group_matmul_mxfp4_noalloc(void* C_bf16, const uint8_t* A_fp4, const uint8_t* sA_e8m0,
                                            const uint8_t* B_fp4, const uint8_t* sB_e8m0,
                                            const int64_t* groupList_host, int G, int K, int N, void* stream);
size_t ascq_group_matmul_mxfp4_noalloc_max_scratch(void);

/* Reference layout adapters for the MX matmul (one-off weight preparation):
 * B given as [K, N] fp4 pairs along N and scaleB stored [sK/2, N, 2]
 * (examples/.../matmul_mxfp4_high_performance/README_en.md:64-67, scripts/gen_data.py:65)
 * are rewritten into the K-major form ascq_group_matmul_mxfp4 takes. */
ascq_status ascq_mx_repack_b_kn_to_nk(uint8_t* B_nk, const uint8_t* B_kn, int K, int N, void* stream);
ascq_status ascq_mx_repack_scale_b(uint8_t* sB_nk, const uint8_t* sB_ref, int sK, int N, void* stream);

/*
 * The same matmul with the all-gather of a column-parallel layout fused into its epilogue: the [M, N]
 * block this call computes is written to columns [colOffset, colOffset + N) of EVERY buffer in
 * C_bufs (each a bf16 [M, ldc] matrix, ldc >= colOffset + N).  With one process per GPU, C_bufs holds
 * this GPU's output matrix and the peer-mapped addresses of the other GPUs' output matrices (CUDA IPC /
 * symmetric memory); the tiles then cross NVLink as plain stores while the tensor cores work on the
 * next tile, and no separate collective is needed.  Stores start with buffer `firstBuf` and wrap
 * around, so ranks passing their own rank + 1 do not all write to the same GPU at once.  nBufs <= 8.
 * The call returns when the kernel is enqueued; a cross-GPU barrier after it (after all ranks' kernels)
 * is the caller's job before anyone reads the assembled matrix.  The reference reassembles with a
 * separate HCCL AllGather (include/adv_api/hccl/hccl.h:77-253); this entry point has no counterpart.
 */
ascq_status ascq_matmul_w8a8_scatter(void* const* C_bufs, int nBufs, int firstBuf, int colOffset, int ldc,
                                     const int8_t* A, const int8_t* B_nk, const float* sA_m, const float* sB_n,
                                     const void* bias_bf16, int M, int N, int K, void* stream);

/*
 * int8 x int8 matmul with the result quantised on the way out the way the reference's fixpipe does it
 * (Matmul::SetQuantScalar / SetQuantVector, include/adv_api/matmul/matmul.h:150-160,
 * impl/adv_api/detail/matmul/stage/copy_cube_out/quant/quant_processor_fixpipe.h:80-119, mode DEQF16), with the
 * arithmetic of the sample's golden (examples/01_simd_cpp_api/04_advanced_api/00_matmul/matmul_quant/scripts/
 * gen_data.py:26-44):  h = half(acc + bias_i32[n]);  C = h * half(quantScalar)            (quantVector NULL)
 *                                                    C = half(float(h) * s19(quantVector[n]))  (per channel),
 * where s19 keeps sign, exponent and the top 10 mantissa bits of the fp32 held in the low word of the uint64.
 * A [M,K], B_nk [N,K] int8 K-major, bias_i32 [N] or NULL, C fp16 [M, ldc].  A weight stored [K,N] (the sample's
 * CubeFormat::ND B) is turned once with ascq_transpose_i8_kn_to_nk.
 */
ascq_status ascq_matmul_i8_quant(void* C_f16, const int8_t* A, const int8_t* B_nk, const int32_t* bias_i32,
                                 const uint64_t* quantVector, float quantScalar, int M, int N, int K, int ldc,
                                 void* stream);

/*
 * The same matmul with an int8 or uint8 result: the fixpipe's requantisation (quant_processor_fixpipe.h:93-95 and
 * 201-203, modes REQ8 / VREQ8), with the arithmetic of the reference's own description of it
 * (examples/01_simd_cpp_api/03_basic_api/03_matrix_compute/fixpipe_l0c2gm/scripts/gen_data_s322s8.py:39-97; field
 * layout docs/zh/api/SIMD-API/基础API/矩阵计算（ISASI）/矩阵计算的搬出/关键特性说明/随路量化.md:53-58).  Per column n the
 * 64-bit parameter q = quantVector[n] (or quantScalar when quantVector is NULL) holds
 *   bits 31:13  scale: fp32 sign, exponent and the top 10 mantissa bits      bit  36     shift enable
 *   bits 35:32  shift count                                                   bits 45:37  offset (0..511)
 *   bit  46     1: int8 result, 0: uint8 result
 * and   a = acc + bias_i32[n];   if shift enabled: a = sat_int16(a >> count);
 *       t = RINT(clamp(float(a) * scale, -256, 255)) + offset;   C = clamp(t, -128..127 or 0..255).
 * No ReLU stage (the Matmul object does not expose one), so negative values take the same scale.  C is a byte
 * matrix [M, ldc]; everything else as in ascq_matmul_i8_quant.
 */
ascq_status ascq_matmul_i8_requant(void* C_b8, const int8_t* A, const int8_t* B_nk, const int32_t* bias_i32,
                                   const uint64_t* quantVector, uint64_t quantScalar, int M, int N, int K, int ldc,
                                   void* stream);
ascq_status ascq_transpose_i8_kn_to_nk(int8_t* B_nk, const int8_t* B_kn, int K, int N, void* stream);

/*
 * half / bfloat16 matmul, fp32 accumulation (AscendC::Matmul<half, half, half|float>; tcgen05 kind::f16, the same
 * kernel template and tile shapes as the int8 matmul).  A [M,K], B_nk [N,K] of abT, K-major; C [M, ldc] of cT = half,
 * bfloat16_t or float; K % 8 == 0.
 */
ascq_status ascq_matmul_f16(void* C, ascq_dtype cT, const void* A, const void* B_nk, ascq_dtype abT, int M, int N, int K,
                            int ldc, void* stream);

/*
 * The same matmul with an int8 or uint8 result: the fixpipe's quantisation of an fp32 accumulator
 * (Matmul<half, half, int8_t> with SetQuantScalar / SetQuantVector, quant_processor_fixpipe.h:95-97 and 203-205, modes
 * QF322B8_PRE / VQF322B8_PRE; arithmetic of .../fixpipe_l0c2gm/scripts/gen_data_f322s8.py:75-97).  The 64-bit
 * parameter has the layout given for ascq_matmul_i8_requant; its shift fields do not apply to this mode:
 *       t = RINT(clamp(acc * scale, -256, 255)) + offset;   C = clamp(t, -128..127 or 0..255).
 * The accumulator is the tensor cores' fp32 sum, so a product that lands within rounding distance of a tie can come
 * out one step away from a result computed with another summation order.
 */
ascq_status ascq_matmul_f16_quant(void* C_b8, const void* A, const void* B_nk, ascq_dtype abT, const uint64_t* quantVector,
                                  uint64_t quantScalar, int M, int N, int K, int ldc, void* stream);
/*
 * Weight-only-quantised matmul: A half / bfloat16, B int8 dequantised on its way to the tensor cores with
 * Matmul::SetAntiQuantScalar / SetAntiQuantVector (include/adv_api/matmul/matmul.h:155-168; the reference converts each
 * weight tile with AscendAntiQuant<int8_t, TransT, isTranspose> before the cube unit reads it,
 * impl/adv_api/detail/matmul/stage/copy_cube_in/antiquant/antiquant_processor_using_ub.h:86-137).
 *   W[n, k] = AscendAntiQuant(B_nk[n, k]) = scale[n] * (B + offset[n]) in aT arithmetic (half: half add, half multiply;
 *   bfloat16: fp32 intermediates) -- offset / scale [N] tensors of aT, or (scale NULL) the two scalars;
 *   C = A . W^T with fp32 accumulation, cast to cT.
 * M <= 32 (with K % 128 == 0, N % 4 == 0, A and B_nk 32-byte aligned): the weight is converted in registers between its
 * load from HBM and the tensor cores -- it is read once and written nowhere; `workspace` then receives at most fp32
 * partial sums of a K split.  Otherwise two launches: the dequantised weight goes through `workspace` (N * K * 2 bytes,
 * 16-byte aligned) and stays in L2 for the matmul when it fits; K % 32 == 0.  Either way the weight the tensor cores
 * multiply is AscendAntiQuant's output bit for bit; the contents of `workspace` after the call are unspecified.
 * (Environment: ASCQ_W8A16=twostep always takes two launches; ASCQ_W8A16=fused runs the conversion inside the tcgen05
 * matmul instead -- converter warps between the copy stage and the MMA stage, same bits, no workspace traffic; it is
 * slower on B200 and kept as a tested alternative.)
 */
ascq_status ascq_matmul_w8a16(void* C, ascq_dtype cT, const void* A, ascq_dtype aT, const int8_t* B_nk, const void* offset,
                              const void* scale, float offsetScalar, float scaleScalar, int M, int N, int K, int ldc,
                              void* workspace, size_t workspaceBytes, void* stream);
size_t ascq_matmul_w8a16_workspace_size(int N, int K);
/* The same with int4b_t weights (B_nk_int4: [N, K/2] bytes, two signed nibbles per byte, even k in the low nibble;
 * AscendAntiQuant's int4b_t source, ascend_antiquant_impl.h:246-247).  Same workspace size and the same forms: M <= 32
 * converts the weight in registers, larger M takes two launches (there is no converter-warp form for int4). */
ascq_status ascq_matmul_w4a16(void* C, ascq_dtype cT, const void* A, ascq_dtype aT, const uint8_t* B_nk_int4, const void* offset,
                              const void* scale, float offsetScalar, float scaleScalar, int M, int N, int K, int ldc,
                              void* workspace, size_t workspaceBytes, void* stream);

/*
 * The grouped MX matmul with 8-bit operands (fp8_e4m3fn / fp8_e5m2 in any combination, one E8M0 scale per 32 elements
 * of K): MatmulWithScalePolicy on fp8 types (impl/adv_api/detail/matmul/mx_matmul_impl.h:29-181, sample
 * examples/01_simd_cpp_api/04_advanced_api/00_matmul/matmul_mx, basic-API form .../03_matrix_compute/mmad_mx).
 * tcgen05 kind::mxf8f6f4.block_scale; same kernel, tile shapes, scratch scheme and grouping as ascq_group_matmul_mxfp4.
 * A [sumM, K], B [G, N, K] one byte per element, K-major; scales [rows, K/32]; K % 128 == 0; C [sumM, N] of
 * cT = ASCQ_DT_BF16 or ASCQ_DT_F32 (the samples' output type); aT / bT = ASCQ_DT_FP8_E4M3 or ASCQ_DT_FP8_E5M2.
 * A weight stored [K, N] is turned once with ascq_transpose_i8_kn_to_nk (bytes), scales stored [sK/2, N, 2] with
 * ascq_mx_repack_scale_b.
 */
ascq_status ascq_group_matmul_mxfp8(void* C, ascq_dtype cT, const uint8_t* A_fp8, ascq_dtype aT, const uint8_t* sA_e8m0,
                                    const uint8_t* B_fp8, ascq_dtype bT, const uint8_t* sB_e8m0,
                                    const int64_t* groupList_host, int G, int K, int N, void* workspace,
                                    size_t workspaceBytes, void* stream);
size_t ascq_group_matmul_mxfp8_workspace_size(int64_t sumM, int G, int K, int N);

/*
 * The grouped MX-FP4 matmul with the reassembly of a group-parallel layout fused into its epilogue.  With the
 * groups dealt out over the GPUs of one box (one process per GPU), every rank computes the output rows of its own
 * groups and writes them into EVERY buffer of C_bufs: group g's rows go to rows outRowStart_host[g] .. of each bf16
 * [*, N] matrix.  C_bufs holds this GPU's output matrix and the peer-mapped addresses of the other GPUs' matrices
 * (plain stores over NVLink; nothing is loaded from a peer).  firstBuf rotates the store order so that the ranks do
 * not all write to the same peer at the same time.  The caller orders the step: a barrier across the ranks after
 * the launches, before anyone reads its matrix.  outRowStart_host may be NULL (groups follow each other as in A).
 * It replaces the all-gather (of ragged row blocks) that the reference's grouped matmul leaves to its caller
 * (examples/03_libraries/00_matmul/quant_group_matmul_custom: one core group per group, output rows disjoint).
 * 1 <= nBufs <= 8; all other arguments as for ascq_group_matmul_mxfp4.
 */
ascq_status ascq_group_matmul_mxfp4_scatter(void* const* C_bufs, int nBufs, int firstBuf,
                                            const int64_t* outRowStart_host, const uint8_t* A_fp4,
                                            const uint8_t* sA_e8m0, const uint8_t* B_fp4, const uint8_t* sB_e8m0,
                                            const int64_t* groupList_host, int G, int K, int N, void* workspace,
                                            size_t workspaceBytes, void* stream);

/*
 * ---- Multi-GPU: one process per GPU, the GPUs of one box --------------------------------------------------------
 * The two matmuls shard the way the reference's samples would (column blocks of the W8A8 weight; whole groups of the
 * grouped matmul, one core group per group in examples/.../quant_group_matmul_custom.asc:257-289), and reassemble with
 * the exchange the reference's kernels would use: HCCL's kernel-side AllGather followed by Commit / Wait
 * (include/adv_api/hccl/hccl.h:82-100, 304-326).  Here both are part of the matmul launch: the epilogue stores each
 * finished tile into EVERY rank's output matrix over NVLink (TMA stores into peer-mapped memory; nothing is loaded
 * from a peer), and when the last CTA of a launch has finished, the rank writes an arrival flag into every peer's flag
 * block and waits -- bounded -- for theirs.  When a *_sharded kernel has completed on a rank, that rank's output
 * matrix holds every rank's part.  A wait that runs out makes ascq_matmul_status return ASCQ_ERR_TIMEOUT.
 *
 * Set-up (once):  every rank allocates a flag block of ascq_comm_flag_bytes() bytes (128-byte aligned, ZEROED) and
 * its output matrices in memory the other ranks can map -- CUDA IPC (ascq_comm_ipc_export / _open wrap
 * cudaIpcGetMemHandle / cudaIpcOpenMemHandle for cudaMalloc'ed memory; the handle bytes travel over whatever channel
 * the host program has) or a symmetric-memory allocator.  After a host-side barrier (every block zeroed and mapped),
 * ascq_comm_create(rank, nranks, flagBlocks) with flagBlocks[r] = rank r's block as mapped in THIS process
 * (flagBlocks[rank] = the local one).  All ranks must issue the same sequence of *_sharded / ascq_comm_barrier calls
 * on a communicator, stream-ordered; the calls may be captured into a CUDA graph (the step counter lives on the
 * device).  Failures of the set-up calls return ASCQ_ERR_NCCL.
 */
typedef struct ascq_comm ascq_comm;
size_t ascq_comm_flag_bytes(void);
ascq_status ascq_comm_create(ascq_comm** comm, int rank, int nranks, void* const* flagBlocks);
ascq_status ascq_comm_destroy(ascq_comm* comm);
ascq_status ascq_comm_rank(const ascq_comm* comm, int* rank, int* nranks);
size_t ascq_comm_ipc_handle_bytes(void);
ascq_status ascq_comm_ipc_export(void* handleOut, const void* devPtr);   /* handle of a cudaMalloc'ed buffer of this process  */
ascq_status ascq_comm_ipc_open(void** devPtrOut, const void* handle);    /* maps a peer's buffer; enables peer access lazily  */
ascq_status ascq_comm_ipc_close(void* devPtr);
/* The end-of-step exchange as a launch of its own (hccl.h:304-326 Commit + Wait): returns at once; when the kernel has
 * completed, every rank has reached this point of its stream. */
ascq_status ascq_comm_barrier(ascq_comm* comm, void* stream);

/* The partition.  Columns: rank r owns columns [r * N / nranks, (r + 1) * N / nranks); N % nranks == 0.
 * Groups: longest group first onto the rank with the fewest rows so far (ties: lower group index, lower rank);
 * owner[g] = rank of group g.  A rank stores its groups back to back in ascending group order. */
ascq_status ascq_shard_columns(int N, int nranks, int rank, int* firstColumn, int* columns);
ascq_status ascq_shard_groups_lpt(const int64_t* groupList_host, int G, int nranks, int* owner);

/*
 * ascq_matmul_w8a8, column-parallel.  C_bufs[r] = rank r's bf16 [M, N] output matrix (row stride N) as mapped in this
 * process; B_local [N / nranks, K], sB_local, bias_local = this rank's column block; A, sA_m whole (replicated in each
 * GPU's own memory).  N / nranks % 8 == 0.  C_multicast (optional, may be NULL): the multicast address of the output
 * matrix (all ranks' matrices bound to one NVSwitch multicast object); when given, every 16-byte piece leaves as one
 * multimem.st and the switch replicates it, instead of one TMA store per rank (needs N / nranks % 64 == 0).
 */
ascq_status ascq_matmul_w8a8_sharded(ascq_comm* comm, void* const* C_bufs, void* C_multicast, const int8_t* A,
                                     const int8_t* B_local, const float* sA_m, const float* sB_local,
                                     const void* bias_local, int M, int N, int K, void* stream);
/*
 * ascq_group_matmul_mxfp4, group-parallel.  groupList_host holds ALL G groups; A_local / sA_local / B_local /
 * sB_local hold the rows and weights of this rank's groups (ascq_shard_groups_lpt) back to back in ascending group
 * order; C_bufs[r] = rank r's bf16 [sum(groupList), N] matrix.  Workspace sized for this rank's share
 * (ascq_group_matmul_mxfp4_workspace_size(local rows, local groups, K, N)).  A rank without groups only takes part in
 * the exchange.
 */
ascq_status ascq_group_matmul_mxfp4_sharded(ascq_comm* comm, void* const* C_bufs, const uint8_t* A_local,
                                            const uint8_t* sA_local, const uint8_t* B_local, const uint8_t* sB_local,
                                            const int64_t* groupList_host, int G, int K, int N, void* workspace,
                                            size_t workspaceBytes, void* stream);

/*
 * Limit of every bounded device-side wait (mbarrier waits inside the matmul kernels, the wait for the other ranks), in
 * SM cycles, on the current device; the default is about two seconds, cycles <= 0 restores it.  No reference counterpart.
 */
ascq_status ascq_set_wait_limit_cycles(long long cycles);
/*
 * Measured ceiling of the tensor-core matmuls, no reference counterpart: enqueues a kernel that issues nothing but the
 * matmul kernels' own MMA instructions (tcgen05.mma.cta_group::2 on 256 x 256 tiles, kind::i8 for ASCQ_DT_I8, kind::mxf4
 * with unit block scales for ASCQ_DT_FP4X2_E2M1), `kBlocks` k-blocks of four instructions per SM pair, operands resident
 * in shared memory.  *opsPerLaunch receives the operation count (2 x multiply-accumulates); the caller times the launch
 * (CUDA events) and divides.  What the result leaves out is everything a real matmul adds: copies, barriers, epilogue.
 */
ascq_status ascq_measure_tensor_rate(ascq_dtype operandT, int kBlocks, double* opsPerLaunch, void* stream);

/*
 * Test hook, no reference counterpart: the copy-engine producers of the NEXT int8 / half matmul launch of this process
 * stop after `kBlocks` k-blocks (< 0 cancels).  The kernel's other roles then run into their wait limit, leave through
 * the abort path (tensor memory released, status word set) and ascq_matmul_status reports ASCQ_ERR_TIMEOUT; the output
 * of that launch is undefined.  It exists so that the abort path can be exercised without faulting or hanging a GPU;
 * lower the wait limit first.
 */
ascq_status ascq_test_withhold_after(int kBlocks);

/*
 * Synchronises `stream`, then reads and clears the status word the matmul kernels keep on the
 * current device.  ASCQ_ERR_TIMEOUT when a kernel gave up a bounded wait (its output is then
 * undefined); no counterpart in the reference, whose kernels cannot report.
 */
ascq_status ascq_matmul_status(void* stream);

/*
 * Host-side temporary-buffer size queries, kept for API parity (the CUDA kernels need no
 * temporary buffer).  Formulas: impl/adv_api/tiling/quantization/ascend_quant_tiling_impl.cpp:31-69,
 * ascend_dequant_tiling_impl.cpp:31-106, ascend_antiquant_tiling_impl.cpp:71-181.
 * Shapes are passed as (dims pointer, rank).  Return ASCQ_ERR_INVALID_ARG where the reference's
 * ASCENDC_HOST_ASSERT fires.
 */
ascq_status ascq_get_ascend_quant_max_min_tmp_size(const int64_t* srcDims, int rank, uint32_t typeSize,
                                                   uint32_t* maxValue, uint32_t* minValue);
void ascq_get_ascend_quant_tmp_buffer_factor_size(uint32_t* maxLiveNodeCount, uint32_t* extraBuf);
ascq_status ascq_get_ascend_dequant_max_min_tmp_size(const int64_t* srcDims, int rank, uint32_t typeSize,
                                                     uint32_t* maxValue, uint32_t* minValue);
void ascq_get_ascend_dequant_tmp_buffer_factor_size(const int64_t* srcDims, int rank,
                                                    uint32_t* maxLiveNodeCount, uint32_t* extraBuf);
ascq_status ascq_get_ascend_antiquant_max_min_tmp_size(const int64_t* srcDims, int srcRank,
                                                       const int64_t* scaleDims, int scaleRank,
                                                       int isTranspose, ascq_dtype inputT, ascq_dtype outputT,
                                                       uint32_t* maxValue, uint32_t* minValue);
void ascq_get_ascend_antiquant_tmp_buffer_factor_size(const int64_t* srcDims, int srcRank,
                                                      const int64_t* scaleDims, int scaleRank,
                                                      int isTranspose, ascq_dtype inputT, ascq_dtype outputT,
                                                      uint32_t* maxLiveNodeCount, uint32_t* extraBuf);

#ifdef __cplusplus
}
#endif
#endif /* ASCQ_H_ */
