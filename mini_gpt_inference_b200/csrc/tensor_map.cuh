// Tensor maps of row-major bfloat16 matrices for the TMA kernels, made on the host and kept by
// (pointer, shape, box): boxes of box_rows x 64 columns (one 128-byte row each), 128-byte swizzle,
// out-of-range rows and columns read as zeros; or, for matrices that are streamed whole rows at a
// time, boxes of box_rows x (several 64-column blocks of the same rows).
#pragma once

#include <cuda.h>

#include <functional>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

struct MapKey {
    const void* ptr;
    int rows, k, box_rows;
    int box_blocks;                  // 0: 2-D boxes of 64 columns; else 64-column blocks per 3-D box
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && k == o.k && box_rows == o.box_rows && box_blocks == o.box_blocks;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& m) const {
        size_t h = std::hash<const void*>()(m.ptr);
        h = h * 1000003u ^ (size_t)m.rows;
        h = h * 1000003u ^ (size_t)m.k;
        h = h * 1000003u ^ (size_t)m.box_rows;
        return h * 1000003u ^ (size_t)m.box_blocks;
    }
};

// Tensor map of a row-major [rows, k] bfloat16 matrix, boxes of box_rows x 64, 128-byte swizzle.
inline int tensor_map(const void* ptr, int rows, int k, int box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    MapKey key{ptr, rows, k, box_rows, 0};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return MG_OK; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return mg_set_error(MG_ERR_CUDA, "linear: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return mg_set_error(MG_ERR_CUDA, "linear: cuTensorMapEncodeTiled failed (%d)", (int)r);
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, *out);
    return MG_OK;
}


// Tensor map of a row-major [rows, k] bfloat16 matrix, k a multiple of 64, seen as
// [rows][k / 64 blocks][64 columns]: a box holds box_blocks consecutive blocks of box_rows rows, so
// a row's bytes are asked of memory as one run.  In shared memory the box is [row][block][128
// bytes], 128-byte swizzle by line (line = row * box_blocks + block): eight rows of one block sit
// in eight different swizzle phases exactly if box_blocks is odd.  Blocks past k / 64 and rows past
// the matrix read as zeros.  Coordinates: (0, first block, first row).
inline int tensor_map_rows(const void* ptr, int rows, int k, int box_rows, int box_blocks, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (k % 64 != 0 || box_blocks < 1 || box_blocks > 256 || box_rows < 1 || box_rows > 256)
        return mg_set_error(MG_ERR_UNSUPPORTED, "linear: no row boxes for k=%d, %d blocks, %d rows", k, box_blocks, box_rows);
    MapKey key{ptr, rows, k, box_rows, box_blocks};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return MG_OK; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return mg_set_error(MG_ERR_CUDA, "linear: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {64u, (cuuint64_t)(k / 64), (cuuint64_t)rows};
    cuuint64_t strides[2] = {128u, (cuuint64_t)k * 2};
    cuuint32_t box[3] = {64u, (cuuint32_t)box_blocks, (cuuint32_t)box_rows};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return mg_set_error(MG_ERR_CUDA, "linear: cuTensorMapEncodeTiled failed (%d)", (int)r);
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, *out);
    return MG_OK;
}
