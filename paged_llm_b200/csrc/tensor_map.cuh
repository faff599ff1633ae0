// Tensor maps for TMA (cp.async.bulk.tensor) over row-major bfloat16 matrices: boxes of
// `box_rows` rows by 64 columns (128 bytes) that land in shared memory in the 128-byte swizzle
// the tcgen05 shared-memory descriptors read.  A map is made once per (address, shape, box) with
// the driver's cuTensorMapEncodeTiled (looked up through the runtime, so no link against the
// driver library) and kept for the life of the process.
#pragma once

#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"

struct TensorMapKey {
    const void* base;
    unsigned long long rows, cols, row_stride;
    unsigned box_rows;
    bool operator==(const TensorMapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && row_stride == o.row_stride && box_rows == o.box_rows;
    }
};

// The map for `rows` x `cols` bfloat16 at `base`, rows `row_stride` elements apart (a multiple
// of 8), boxes of box_rows x 64, copied to `out`.  Out-of-range parts of a box read zeros.  False
// (with the error recorded) if the driver refuses.
inline bool tensor_map_bf16(CUtensorMap* out, const void* base, unsigned long long rows, unsigned long long cols,
                            unsigned long long row_stride, unsigned box_rows) {
    typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static std::mutex mu;
    static std::vector<std::pair<TensorMapKey, CUtensorMap*>> maps;
    static EncodeTiledFn encode = nullptr;
    std::lock_guard<std::mutex> lock(mu);
    const TensorMapKey key{base, rows, cols, row_stride, box_rows};
    for (auto& m : maps)
        if (m.first == key) {
            *out = *m.second;
            return true;
        }
    // Activations come at ever new addresses when steps are not replayed from graphs: the list is
    // kept short by starting over (callers get copies).
    if (maps.size() >= 1024) {
        for (auto& m : maps) free(m.second);
        maps.clear();
    }
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &res) != cudaSuccess ||
            res != cudaDriverEntryPointSuccess || !fn) {
            pl_fail("tensor map: the driver has no cuTensorMapEncodeTiled");
            return false;
        }
        encode = (EncodeTiledFn)fn;
    }
    if (((uintptr_t)base & 15) != 0 || row_stride % 8 != 0 || box_rows == 0 || box_rows > 256 || rows == 0 || cols == 0) {
        pl_fail("tensor map: base must be 16-byte aligned, rows a multiple of 16 bytes apart, boxes of 1..256 rows");
        return false;
    }
    void* mem = nullptr;
    if (posix_memalign(&mem, 64, sizeof(CUtensorMap)) != 0) {
        pl_fail("tensor map: out of host memory");
        return false;
    }
    CUtensorMap* map = (CUtensorMap*)mem;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        free(mem);
        pl_fail("tensor map: cuTensorMapEncodeTiled failed (%d)", (int)rc);
        return false;
    }
    maps.emplace_back(key, map);
    *out = *map;
    return true;
}
