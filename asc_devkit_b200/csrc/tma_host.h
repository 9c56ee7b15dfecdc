// Host-side helpers shared by the GEMM translation units: the cuTensorMapEncodeTiled entry point (looked up
// through the runtime so the library carries no link-time dependency on libcuda) and the SM count.
#ifndef ASCQ_TMA_HOST_H_
#define ASCQ_TMA_HOST_H_

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>

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

// Encoded 2-D tensor maps are remembered per thread, keyed by everything that goes into them: a matmul that is
// launched again on the same buffers (every step of a serving loop) then pays a table lookup instead of three to
// eleven driver calls before each launch.  A tensor map is a pure function of its arguments, so a hit can never be
// stale; 128 direct-mapped slots.
struct TmapKey {
    const void* base;
    uint64_t d0, d1, stride;
    uint32_t box0, box1;
    int dtype, swizzle, promo;
    bool operator==(const TmapKey& o) const
    {
        return base == o.base && d0 == o.d0 && d1 == o.d1 && stride == o.stride && box0 == o.box0 && box1 == o.box1 &&
               dtype == o.dtype && swizzle == o.swizzle && promo == o.promo;
    }
};
inline ascq_status encode_2d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, uint64_t d0, uint64_t d1, uint64_t strideBytes,
                             uint32_t box0, uint32_t box1, CUtensorMapSwizzle sw, CUtensorMapL2promotion promo, const char* what)
{
    struct Slot {
        TmapKey key;
        CUtensorMap map;
        bool valid;
    };
    static thread_local Slot slots[128] = {};
    const TmapKey key{base, d0, d1, strideBytes, box0, box1, static_cast<int>(dt), static_cast<int>(sw), static_cast<int>(promo)};
    uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
    h ^= d0 * 0x9E3779B97F4A7C15ull;
    h ^= (d1 + (static_cast<uint64_t>(box1) << 32) + box0) * 0xC2B2AE3D27D4EB4Full;
    h ^= h >> 29;
    Slot& sl = slots[h & 127u];
    if (sl.valid && sl.key == key) {
        *out = sl.map;
        return ASCQ_OK;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(ASCQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    const cuuint64_t dims[2] = {d0, d1};
    const cuuint64_t strides[1] = {strideBytes};
    const cuuint32_t box[2] = {box0, box1};
    const cuuint32_t elemStrides[2] = {1, 1};
    const CUresult rc = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, promo,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(ASCQ_ERR_CUDA, "cuTensorMapEncodeTiled (%s) failed with CUresult %d", what, static_cast<int>(rc));
    sl.key = key;
    sl.map = *out;
    sl.valid = true;
    return ASCQ_OK;
}

// uint8 [rows, colsBytes] row-major tensor map with a [boxRows, 128-byte] box and the 128B swizzle.
// colsBytes must be a multiple of 16 and base 16-byte aligned.
inline ascq_status make_tmap_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t colsBytes, uint32_t boxRows)
{
    return encode_2d(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, base, colsBytes, rows, colsBytes, 128, boxRows, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "operand");
}

// uint8 [rows, colsBytes] row-major tensor map with a [boxRows, boxBytes] box and no swizzle (rows land back to back).
inline ascq_status make_tmap_u8_plain(CUtensorMap* out, const void* base, uint64_t rows, uint64_t colsBytes, uint32_t boxBytes,
                                      uint32_t boxRows)
{
    return encode_2d(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, base, colsBytes, rows, colsBytes, boxBytes, boxRows, CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "plain");
}

// uint32 [rows, words] tensor map (rows of recordBytes, no swizzle) with a one-row box: one load moves one record.
inline ascq_status make_tmap_kib_rows(CUtensorMap* out, const void* base, uint64_t rows, uint32_t recordBytes = 1024)
{
    return encode_2d(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, base, recordBytes / 4, rows, recordBytes, recordBytes / 4, 1,
                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "records");
}

// 16-bit [rows, cols] row-major output matrix with row pitch ldElems: a [boxRows, 64-element] box (128 bytes) with the
// 128B swizzle, for TMA stores.  base 16-byte aligned, ldElems a multiple of 8.
inline ascq_status make_tmap_out16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ldElems, uint32_t boxRows,
                                   uint32_t boxCols = 64, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B)
{
    // (boxCols = 32 with CU_TENSOR_MAP_SWIZZLE_64B: 64-byte rows)
    return encode_2d(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, base, cols, rows, ldElems * 2, boxCols, boxRows, swizzle,
                     CU_TENSOR_MAP_L2_PROMOTION_NONE, "output");
}

// The current device's ordinal, clamped to the per-device tables below.
constexpr int kMaxDevices = 64;
inline int current_device()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
    return dev;
}

// "Done once on this device" marker for per-device set-up (kernel attributes are per device, and one process may
// drive several GPUs).  Two threads racing through the same set-up do it twice, which is harmless.
struct PerDeviceOnce {
    std::atomic<uint64_t> mask{0};
    bool done(int dev) const { return (mask.load(std::memory_order_acquire) >> dev) & 1u; }
    void mark(int dev) { mask.fetch_or(1ull << dev, std::memory_order_release); }
};

inline int sm_count()
{
    static std::atomic<int> n[kMaxDevices] = {};
    const int dev = current_device();
    int v = n[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        v = 148;
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        n[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

}  // namespace ascq
#endif  // ASCQ_TMA_HOST_H_
