// Host side of TMA: tensor maps over row-major bfloat16 matrices, made through the driver entry
// point (no link against libcuda) and kept by address and shape.
// Include after ABK_REFUSE is defined (common.cuh with ABK_DEFINE_ERROR).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>
#include <unordered_map>

namespace tmap {

typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_tiled() {
    static EncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    });
    return fn;
}

struct Key {
    const void *ptr;
    long long rows, cols, ld;
    int box_rows;
    bool operator==(const Key &o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct KeyHash {
    size_t operator()(const Key &k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ (size_t)k.rows, h = h * 1000003u ^ (size_t)k.cols;
        return h * 1000003u ^ (size_t)k.ld ^ ((size_t)k.box_rows << 48);
    }
};

// A map over a bfloat16 matrix [rows, cols] with row pitch ld (elements): boxes of [box_rows, 64]
// elements (128 bytes a row), 128-byte swizzle, zeros outside. 0 on success.
static int bf16_rows_of_128_bytes(const void *ptr, long long rows, long long cols, long long ld, int box_rows,
                                  CUtensorMap *out) {
    static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
    static std::mutex lock;
    Key key{ptr, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> guard(lock);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return 0;
    }
    EncodeTiled enc = encode_tiled();
    if (!enc) ABK_REFUSE("the driver gives no cuTensorMapEncodeTiled");
    if (((uintptr_t)ptr & 15) || (ld * 2) % 16) ABK_REFUSE("a TMA operand must be 16-byte aligned with a pitch that is a multiple of 16 bytes");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void *)ptr, dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) ABK_REFUSE("cuTensorMapEncodeTiled failed with %d", (int)r);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return 0;
}

}  // namespace tmap
