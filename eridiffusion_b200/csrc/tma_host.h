// Host-side helpers shared by the TMA-fed kernels: the driver's tensor-map encoder is fetched
// through the runtime (no link against libcuda), and encoded maps are cached by their geometry.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

namespace eri {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct MapKey {
  uint64_t ptr, d0, d1, d2, d3, s1, s2, s3;
  uint32_t b0, b1, b2, b3, rank, swz, esz;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && d3 == o.d3 && s1 == o.s1 &&
           s2 == o.s2 && s3 == o.s3 && b0 == o.b0 && b1 == o.b1 && b2 == o.b2 && b3 == o.b3 &&
           rank == o.rank && swz == o.swz && esz == o.esz;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    const uint64_t v[] = {k.ptr, k.d0, k.d1, k.d2, k.d3, k.s1, k.s2, k.s3,
                          ((uint64_t)k.b0 << 32) | k.b1, ((uint64_t)k.b2 << 32) | k.b3,
                          ((uint64_t)k.rank << 40) | ((uint64_t)k.swz << 8) | k.esz};
    for (uint64_t x : v) {
      h ^= x;
      h *= 1099511628211ull;
    }
    return (size_t)h;
  }
};

// Encode (or fetch from the cache) a tiled map over a tensor of up to four dimensions.
// dims/box are innermost first; strides are in bytes for dimensions 1..rank-1.
// swizzle_bytes: 0 (none), 32, 64 or 128. elem_bytes: 2 (bf16) or 4 (fp32).
inline int make_tensor_map(CUtensorMap* out, const void* ptr, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes,
                           int elem_bytes = 2) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -2;
  MapKey k{};
  k.ptr = (uint64_t)ptr;
  k.rank = rank;
  k.swz = swizzle_bytes;
  k.esz = elem_bytes;
  uint64_t* kd[] = {&k.d0, &k.d1, &k.d2, &k.d3};
  uint64_t* ks[] = {nullptr, &k.s1, &k.s2, &k.s3};
  uint32_t* kb[] = {&k.b0, &k.b1, &k.b2, &k.b3};
  for (int i = 0; i < rank; ++i) {
    *kd[i] = dims[i];
    *kb[i] = box[i];
    if (i > 0) *ks[i] = strides_bytes[i - 1];
  }
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(k);
    if (it != cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  cuuint64_t gd[4];
  cuuint64_t gs[3];
  cuuint32_t bx[4], es[4];
  for (int i = 0; i < rank; ++i) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) gs[i - 1] = strides_bytes[i - 1];
  }
  CUtensorMapSwizzle sw = swizzle_bytes == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUtensorMapDataType dt =
      elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(out, dt, (cuuint32_t)rank, const_cast<void*>(ptr), gd, gs, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -3;
  {
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 65536) cache.clear();
    cache.emplace(k, *out);
  }
  return 0;
}

}  // namespace eri
