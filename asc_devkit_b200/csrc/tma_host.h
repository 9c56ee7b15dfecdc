// Host-side helpers shared by the GEMM translation units: the cuTensorMapEncodeTiled entry point (looked up
// through the runtime so the library carries no link-time dependency on libcuda) and the SM count.
#ifndef ASCQ_TMA_HOST_H_
#define ASCQ_TMA_HOST_H_

#include <cuda.h>
#include <cuda_runtime.h>

#include "ascq_internal.h"

namespace ascq {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// uint8 [rows, colsBytes] row-major tensor map with a [boxRows, 128-byte] box and the 128B swizzle.
// colsBytes must be a multiple of 16 and base 16-byte aligned.
inline ascq_status make_tmap_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t colsBytes, uint32_t boxRows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(ASCQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    const cuuint64_t dims[2] = {colsBytes, rows};
    const cuuint64_t strides[1] = {colsBytes};
    const cuuint32_t box[2] = {128, boxRows};
    const cuuint32_t elemStrides[2] = {1, 1};
    const CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elemStrides,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(ASCQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(rc));
    return ASCQ_OK;
}

// uint8 [rows, colsBytes] row-major tensor map with a [boxRows, boxBytes] box and no swizzle (rows land back to back).
inline ascq_status make_tmap_u8_plain(CUtensorMap* out, const void* base, uint64_t rows, uint64_t colsBytes, uint32_t boxBytes,
                                      uint32_t boxRows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(ASCQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    const cuuint64_t dims[2] = {colsBytes, rows};
    const cuuint64_t strides[1] = {colsBytes};
    const cuuint32_t box[2] = {boxBytes, boxRows};
    const cuuint32_t elemStrides[2] = {1, 1};
    const CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elemStrides,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(ASCQ_ERR_CUDA, "cuTensorMapEncodeTiled (plain) failed with CUresult %d", static_cast<int>(rc));
    return ASCQ_OK;
}

// uint32 [rows, words] tensor map (rows of recordBytes, no swizzle) with a one-row box: one load moves one record.
inline ascq_status make_tmap_kib_rows(CUtensorMap* out, const void* base, uint64_t rows, uint32_t recordBytes = 1024)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(ASCQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    const cuuint64_t dims[2] = {recordBytes / 4, rows};
    const cuuint64_t strides[1] = {recordBytes};
    const cuuint32_t box[2] = {recordBytes / 4, 1};
    const cuuint32_t elemStrides[2] = {1, 1};
    const CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, elemStrides,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(ASCQ_ERR_CUDA, "cuTensorMapEncodeTiled (records) failed with CUresult %d", static_cast<int>(rc));
    return ASCQ_OK;
}

// 16-bit [rows, cols] row-major output matrix with row pitch ldElems: a [boxRows, 64-element] box (128 bytes) with the
// 128B swizzle, for TMA stores.  base 16-byte aligned, ldElems a multiple of 8.
inline ascq_status make_tmap_out16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ldElems, uint32_t boxRows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(ASCQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ldElems * 2};
    const cuuint32_t box[2] = {64, boxRows};
    const cuuint32_t elemStrides[2] = {1, 1};
    const CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, elemStrides,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(ASCQ_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with CUresult %d", static_cast<int>(rc));
    return ASCQ_OK;
}

inline int sm_count()
{
    static int n = [] {
        int dev = 0, v = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        return v;
    }();
    return n;
}

}  // namespace ascq
#endif  // ASCQ_TMA_HOST_H_
