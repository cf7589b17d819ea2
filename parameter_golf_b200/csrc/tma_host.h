// Host-side TMA tensor-map encoding without linking libcuda: the driver entry point is looked up
// through the runtime so the extension imports on machines that have no driver installed.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstring>
#include <stdexcept>
#include <string>
#include <unordered_map>

namespace pgb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
      throw std::runtime_error("cuTensorMapEncodeTiled is not available (no CUDA driver?)");
    fn = (EncodeTiledFn)p;
  }
  return fn;
}

// Everything `cuTensorMapEncodeTiled` is given. The encoded map is a pure function of these values, so a map built once for
// a (pointer, shape, box) can be reused by every later launch on the same buffers: the training step calls each product with
// the same pre-allocated tensors, step after step.
struct TmapKey {
  const void* base;
  uint64_t dims[4];
  uint64_t strides[3];
  uint32_t box[4];
  int32_t rank;
  int32_t swz;
  bool operator==(const TmapKey& o) const { return std::memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    const unsigned char* b = reinterpret_cast<const unsigned char*>(&k);
    uint64_t h = 1469598103934665603ull;                     // FNV-1a over the (zero-padded) key
    for (size_t i = 0; i < sizeof(TmapKey); ++i) h = (h ^ b[i]) * 1099511628211ull;
    return (size_t)h;
  }
};

// bf16 tensor of up to 4 dims. dims[0] is the contiguous one; strides_bytes[i] is the stride of dim i+1.
// 128-byte swizzle; out-of-range elements read as zero. Encoded maps are cached per host thread.
inline CUtensorMap make_tmap_bf16(const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                                  const uint32_t* box, CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  if (rank < 1 || rank > 4) throw std::runtime_error("TMA tensor maps of rank 1 to 4 only");
  thread_local std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  TmapKey key;
  std::memset(&key, 0, sizeof(key));
  key.base = base;
  key.rank = rank;
  key.swz = (int32_t)swz;
  for (int i = 0; i < rank; ++i) {
    key.dims[i] = dims[i];
    key.box[i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) key.strides[i] = strides_bytes[i];
  auto hit = cache.find(key);
  if (hit != cache.end()) return hit->second;
  CUtensorMap m;
  cuuint64_t gd[5];
  cuuint64_t gs[4];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = strides_bytes[i];
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) throw std::runtime_error("TMA base address must be 16-byte aligned");
  for (int i = 0; i + 1 < rank; ++i)
    if (gs[i] % 16 != 0) throw std::runtime_error("TMA strides must be multiples of 16 bytes");
  CUresult r = encode_tiled_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gd, gs, bx, es,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  if (cache.size() >= 8192) cache.clear();                   // evaluation over many differently shaped views: start over
  cache.emplace(key, m);
  return m;
}

}  // namespace pgb
