// Host-side helpers shared by the launchers: TMA tensor-map encoding through the driver entry
// point (no link-time dependency on libcuda) and a small error-string channel for the C ABI.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <cstring>

namespace ua {

// Last error text of this library; read through ua_last_error().
inline char* err_buf() {
  static thread_local char buf[512];
  return buf;
}
#define UA_FAIL(...)                               \
  do {                                             \
    snprintf(ua::err_buf(), 512, __VA_ARGS__);     \
    return -1;                                     \
  } while (0)
#define UA_CUDA(expr)                                                                   \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess) UA_FAIL("%s failed: %s", #expr, cudaGetErrorString(_e));     \
  } while (0)

// Trace buffers registered by ua_set_kernel_trace: [0 = forward, 1 = backward][device].
struct TraceSlot {
  unsigned long long* buf;
  int cap;
};
inline TraceSlot* trace_registry() {
  static TraceSlot slots[2][64] = {};
  return &slots[0][0];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// ---- tensor-map cache ---------------------------------------------------------------------------
// A training loop encodes the same few dozen tensor maps every step (same buffers, same shapes).
// encode_tiled_cached keeps the encoded 128-byte maps in a fixed table (no heap, so the
// allocation-free entry points may use it): 1024 slots, four probes, the oldest probe is replaced.
// A map depends on nothing but the arguments in the key, so a hit is always valid, also after the
// buffer behind `base` was freed and reallocated.
struct TmapKey {
  uint64_t base;
  uint64_t dims[5];
  uint64_t strides[4];
  uint32_t box[5];
  int32_t rank;
  int32_t kind;      // 0: bf16, 128-byte swizzle; 1: fp32, no swizzle
  uint32_t pad;
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  uint64_t stamp;    // 0: empty
};
struct TmapCache {
  static constexpr int SLOTS = 1024;
  TmapSlot slot[SLOTS];
  uint64_t clock = 0;
  uint64_t hits = 0, misses = 0;
  std::atomic_flag busy = ATOMIC_FLAG_INIT;
};
inline TmapCache& tmap_cache() {
  static TmapCache c;
  return c;
}

inline int encode_tiled_cached(CUtensorMap* out, int kind, const void* base, int rank, const uint64_t* dims,
                               const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) UA_FAIL("cuTensorMapEncodeTiled entry point not found");
  if (rank < 1 || rank > 5) UA_FAIL("tensor map rank %d not in 1..5", rank);
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) UA_FAIL("TMA base not 16-byte aligned");
  TmapKey key;
  std::memset(&key, 0, sizeof(key));
  key.base = reinterpret_cast<uint64_t>(base);
  key.rank = rank;
  key.kind = kind;
  for (int i = 0; i < rank; ++i) {
    key.dims[i] = dims[i];
    key.box[i] = box[i];
    if (i > 0) {
      key.strides[i - 1] = strides_bytes[i - 1];
      if (strides_bytes[i - 1] % 16 != 0)
        UA_FAIL("TMA stride %d (%llu B) not a multiple of 16", i - 1, (unsigned long long)strides_bytes[i - 1]);
    }
  }
  uint64_t h = 1469598103934665603ull;
  const unsigned char* kb = reinterpret_cast<const unsigned char*>(&key);
  for (size_t i = 0; i < sizeof(key); ++i) h = (h ^ kb[i]) * 1099511628211ull;
  TmapCache& c = tmap_cache();
  while (c.busy.test_and_set(std::memory_order_acquire)) {}
  int victim = -1;
  uint64_t oldest = ~0ull;
  for (int pr = 0; pr < 4; ++pr) {
    const int i = static_cast<int>((h + pr) % TmapCache::SLOTS);
    TmapSlot& sl = c.slot[i];
    if (sl.stamp != 0 && std::memcmp(&sl.key, &key, sizeof(key)) == 0) {
      sl.stamp = ++c.clock;
      *out = sl.map;
      ++c.hits;
      c.busy.clear(std::memory_order_release);
      return 0;
    }
    if (sl.stamp < oldest) { oldest = sl.stamp; victim = i; }
  }
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bx[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  const CUresult r =
      kind == 0 ? fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gdim, gstr, bx, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                : fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, rank, const_cast<void*>(base), gdim, gstr, bx, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) {
    TmapSlot& sl = c.slot[victim];
    sl.key = key;
    sl.map = *out;
    sl.stamp = ++c.clock;
    ++c.misses;
  }
  c.busy.clear(std::memory_order_release);
  if (r != CUDA_SUCCESS) UA_FAIL("cuTensorMapEncodeTiled (%s) failed with code %d", kind == 0 ? "bf16" : "f32", (int)r);
  return 0;
}

// bf16 (or any 2-byte) tiled map with 128-byte swizzle. dims/strides innermost first;
// strides_bytes has rank-1 entries (stride of dim 1, 2, ...). The inner box extent must be 64
// elements (128 bytes) to match the swizzle span.
inline int make_tmap_2byte(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box) {
  return encode_tiled_cached(out, 0, base, rank, dims, strides_bytes, box);
}

// fp32 tiled map without swizzle (used as the destination of TMA reduce-add stores).
inline int make_tmap_f32(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box) {
  return encode_tiled_cached(out, 1, base, rank, dims, strides_bytes, box);
}

}  // namespace ua
