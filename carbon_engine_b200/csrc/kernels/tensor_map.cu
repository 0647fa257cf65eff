// Encoding and caching of tensor maps: see tensor_map.h.  cuTensorMapEncodeTiled is taken from the
// driver through the runtime (cudaGetDriverEntryPoint), so the library does not link against libcuda.
#include "tensor_map.h"
#include <mutex>
#include <unordered_map>

namespace {

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    });
    return fn;
}

struct MapKey {
    const void* ptr; long long rows, cols, ld; int box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows; }
};
struct MapHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        for (long long v : {k.rows, k.cols, k.ld, (long long)k.box_rows}) h = h * 1000003u ^ (size_t)v;
        return h;
    }
};

}  // namespace

int ce_tensor_map_bf16(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out,
                       const char* who) {
    static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return CE_OK; }
    EncodeTiled enc = encode_fn();
    if (!enc) return ce_fail(CE_ERR_CUDA, "%s: cuTensorMapEncodeTiled is not available in this driver", who);
    if (((uintptr_t)ptr & 15) || (ld * 2) % 16 || box_rows < 1 || box_rows > 256)
        return ce_fail(CE_ERR_SIZE, "%s: a tensor map needs a 16-byte aligned base and row stride, and 1..256 rows a box", who);
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ce_fail(CE_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed (%d)", who, (int)r);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return CE_OK;
}
