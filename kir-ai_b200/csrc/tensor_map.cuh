// Host side of TMA: encodes tiled tensor maps through the driver entry point
// (found with cudaGetDriverEntryPoint, so the library does not link libcuda)
// and remembers them by (pointer, shape, box), since weights are encoded again
// and again with the same arguments.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <tuple>
#include <unordered_map>

namespace tmap {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
            status == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    });
    return fn;
}

struct Key {
    const void* ptr;
    uint64_t rows, cols, row_stride;
    uint32_t box_rows, box_cols;
    bool operator==(const Key& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && row_stride == o.row_stride &&
               box_rows == o.box_rows && box_cols == o.box_cols;
    }
};
struct KeyHash {
    size_t operator()(const Key& k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ k.rows;
        h = h * 1000003u ^ k.cols;
        h = h * 1000003u ^ k.row_stride;
        h = h * 1000003u ^ ((size_t)k.box_rows << 16 | k.box_cols);
        return h;
    }
};

// A bf16 matrix [rows, cols] with `row_stride` elements between rows, read in
// boxes of [box_rows, box_cols] with the 128-byte swizzle (box_cols * 2 == 128);
// elements outside the matrix read as zero.  Returns false when the driver
// refuses (alignment: base 16 bytes, row stride a multiple of 16 bytes).
inline bool bf16_2d_sw128(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t row_stride,
                          uint32_t box_rows, uint32_t box_cols) {
    static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
    static std::mutex mutex;
    const Key key{ptr, rows, cols, row_stride, box_rows, box_cols};
    std::lock_guard<std::mutex> lock(mutex);
    auto found = cache.find(key);
    if (found != cache.end()) {
        *out = found->second;
        return true;
    }
    EncodeTiledFn encode = encode_fn();
    if (!encode) return false;
    if (((uintptr_t)ptr & 15) || (row_stride * 2) % 16 != 0) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUtensorMap map;
    const CUresult status =
        encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS) return false;
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return true;
}

// The rows of a paged key/value cache, [rows, head_dim] bf16 with head_dim a multiple of 64, read in boxes of
// `box_rows` whole rows (a multiple of 8) by ONE request each: the map has the dimensions (64 columns, 8 rows,
// head_dim / 64 panels, rows / 8 groups), in that order, so that a box lands in shared memory as
// [group of 8 rows][panel][8 rows][128 bytes] with the 128-byte swizzle: every 8 x 128-byte atom that a matrix
// descriptor addresses is whole, the panels of a group 1,024 bytes apart, the groups head_dim / 64 * 1,024 bytes
// apart.  Coordinates of a load: (0, 0, 0, first row / 8).
inline bool bf16_kv_boxes_sw128(CUtensorMap* out, const void* ptr, uint64_t rows, uint32_t head_dim, uint32_t box_rows) {
    static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
    static std::mutex mutex;
    if (head_dim == 0 || head_dim % 64 != 0 || box_rows == 0 || box_rows % 8 != 0 || rows % 8 != 0) return false;
    const Key key{ptr, rows, head_dim, 0, box_rows, 0xffffu};
    std::lock_guard<std::mutex> lock(mutex);
    auto found = cache.find(key);
    if (found != cache.end()) {
        *out = found->second;
        return true;
    }
    EncodeTiledFn encode = encode_fn();
    if (!encode) return false;
    if ((uintptr_t)ptr & 15) return false;
    const cuuint64_t row_bytes = (cuuint64_t)head_dim * 2;
    cuuint64_t dims[4] = {64, 8, head_dim / 64, rows / 8};
    cuuint64_t strides[3] = {row_bytes, 128, 8 * row_bytes};
    cuuint32_t box[4] = {64, 8, head_dim / 64, box_rows / 8};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUtensorMap map;
    const CUresult status =
        encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS) return false;
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return true;
}

}  // namespace tmap
