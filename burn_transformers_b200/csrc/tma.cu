#include "tma.cuh"

#include <cstring>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace bt {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encoder() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

struct MapKey {
  const void* base;
  unsigned long long rows, cols, row_stride;
  unsigned box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && row_stride == o.row_stride && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.base;
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.cols;
    h = h * 1000003u ^ (size_t)k.row_stride;
    h = h * 1000003u ^ (size_t)k.box_rows;
    return h;
  }
};

int tensor_map_2d_bf16(CUtensorMap* map, const void* base, unsigned long long rows, unsigned long long cols,
                       unsigned long long row_stride, unsigned box_rows) {
  static std::mutex mutex;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  BT_CHECK(((unsigned long long)base & 15ull) == 0, "tensor map: the tensor must start on a 16-byte boundary");
  BT_CHECK(row_stride % 8 == 0 && cols >= 1 && rows >= 1, "tensor map: rows of %llu bfloat16 are not 16-byte multiples", row_stride);
  BT_CHECK(box_rows >= 1 && box_rows <= 256, "tensor map: a box of %u rows is outside 1..256", box_rows);
  MapKey key{base, rows, cols, row_stride, box_rows};
  std::lock_guard<std::mutex> lock(mutex);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *map = it->second;
    return 0;
  }
  EncodeTiledFn fn = encoder();
  BT_CHECK(fn != nullptr, "tensor map: the driver does not offer cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {cols, rows};                       // innermost first
  cuuint64_t strides[1] = {row_stride * 2ull};             // bytes between rows
  cuuint32_t box[2] = {64u, box_rows};                     // 64 bfloat16 = 128 bytes = the swizzle span
  cuuint32_t elem_strides[2] = {1u, 1u};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  BT_CHECK(r == CUDA_SUCCESS, "tensor map: cuTensorMapEncodeTiled failed with code %d (rows %llu, cols %llu, stride %llu)",
           (int)r, rows, cols, row_stride);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *map);
  return 0;
}

}  // namespace bt

// A tensor map for a caller that keeps it in its own memory (128 bytes, to be placed on a 64-byte boundary).
extern "C" int bt_tensor_map_2d_bf16(void* out, const void* base, unsigned long long rows, unsigned long long cols,
                                     unsigned long long row_stride, unsigned box_rows) {
  static_assert(sizeof(CUtensorMap) == 128, "a tensor map is 128 bytes");
  CUtensorMap map;
  if (bt::tensor_map_2d_bf16(&map, base, rows, cols, row_stride, box_rows) != 0) return 1;
  std::memcpy(out, &map, sizeof(map));
  return 0;
}
