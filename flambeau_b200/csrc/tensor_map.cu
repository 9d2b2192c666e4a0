// TMA tensor maps are encoded by the driver; the entry point is looked up through the runtime so that the
// library needs no link against libcuda.  Maps are cached: weights and cache pools keep their addresses.
#include "tensor_map.cuh"

#include "common.cuh"

#include <mutex>
#include <stdint.h>
#include <unordered_map>

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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
    const void* ptr; long rows, cols, ld; int box_cols, box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_cols == o.box_cols &&
               box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ (size_t)k.rows;
        h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.ld;
        h = h * 1000003u ^ (size_t)k.box_cols;
        return h * 1000003u ^ (size_t)k.box_rows;
    }
};

}  // namespace

int fb_tensor_map_bf16(CUtensorMap* out, const void* ptr, long rows, long cols, long ld, int box_cols, int box_rows) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    const MapKey key{ptr, rows, cols, ld, box_cols, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fb_fail(-3, "tensor map: the driver does not provide cuTensorMapEncodeTiled");
    if (box_cols * 2 != 128 || box_rows < 1 || box_rows > 256)
        return fb_fail(-3, "tensor map: box of %d x %d elements is not supported", box_rows, box_cols);
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fb_fail(-3, "tensor map: cuTensorMapEncodeTiled failed with code %d", (int)r);
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

// The same encoding without the cache: nothing is kept and no host memory is taken, for callers that must not
// allocate.  (The encoder writes the 128-byte map into *out and touches nothing else.)
int fb_tensor_map_bf16_uncached(CUtensorMap* out, const void* ptr, long rows, long cols, long ld, int box_cols,
                                int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fb_fail(-3, "tensor map: the driver does not provide cuTensorMapEncodeTiled");
    if (box_cols * 2 != 128 || box_rows < 1 || box_rows > 256)
        return fb_fail(-3, "tensor map: box of %d x %d elements is not supported", box_rows, box_cols);
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fb_fail(-3, "tensor map: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

// An output of a product: [slabs][rows][cols] of float32 or bfloat16 (row stride ld, slab stride slab_stride, in
// elements), written in boxes of box_rows x box_cols elements of one slab as they lie in shared memory (no swizzle).
// Not cached: outputs are workspace views that differ from call to call more often than not, and the encoder takes
// no memory.  Returns 1 if such a map cannot be made for these strides and this address (the caller then stores
// without it), 0 if it was made, a negative code after fb_fail() if the driver refused it.
int fb_tensor_map_out(CUtensorMap* out, void* ptr, int elem_bytes, long rows, long cols, long ld, long slabs,
                      long slab_stride, int box_cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return 1;
    if (slabs < 1) slabs = 1;
    if (slabs == 1) slab_stride = rows * ld;
    const bool ok = ((uintptr_t)ptr & 15) == 0 && (ld * elem_bytes) % 16 == 0 && (slab_stride * elem_bytes) % 16 == 0 &&
                    (box_cols * elem_bytes) % 16 == 0 && box_cols <= 256 && box_rows <= 256 && rows > 0 && cols > 0;
    if (!ok) return 1;
    const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)slabs};
    const cuuint64_t strides[2] = {(cuuint64_t)ld * elem_bytes, (cuuint64_t)slab_stride * elem_bytes};
    const cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = fn(out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, ptr,
                    dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fb_fail(-3, "tensor map: cuTensorMapEncodeTiled failed with code %d for an output", (int)r);
    return 0;
}
