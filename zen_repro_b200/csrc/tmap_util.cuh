// Host-side helpers shared by the TMA kernels: cached 2-D bf16 tensor maps and the SM count.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

namespace zen_tmap {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(f);
  });
  return fn;
}

struct Key {
  const void* ptr; uint64_t d0, d1, ld; uint32_t b0, b1; int dev;
  bool operator==(const Key& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && ld == o.ld && b0 == o.b0 && b1 == o.b1 && dev == o.dev;
  }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    for (uint64_t v : {k.d0, k.d1, k.ld, (uint64_t)k.b0, (uint64_t)k.b1, (uint64_t)k.dev}) h = h * 1000003u ^ v;
    return h;
  }
};

// bf16 tensor map: dims {d0 (contiguous), d1}, row stride ld elements, box {b0, b1}, 128-byte swizzle, zero fill.
inline int get(const void* ptr, uint64_t d0, uint64_t d1, uint64_t ld, uint32_t b0, uint32_t b1, CUtensorMap* out) {
  static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);                                      // the same address can name different memory on another device
  Key key{ptr, d0, d1, ld, b0, b1, dev};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
  }
  EncodeTiledFn enc = get_encode();
  if (!enc) return -10;
  cuuint64_t dims[2] = {d0, d1};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {b0, b1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -11;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() >= 4096) {
    // drop about half of the entries (every other one in iteration order) instead of all: the maps of the running
    // step mostly survive, and the table stays bounded
    bool drop = false;
    for (auto it = cache.begin(); it != cache.end();) {
      if ((drop = !drop)) it = cache.erase(it); else ++it;
    }
  }
  cache[key] = *out;
  return 0;
}

inline int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace zen_tmap
