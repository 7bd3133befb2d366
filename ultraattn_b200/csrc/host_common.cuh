// Host-side helpers shared by the launchers: TMA tensor-map encoding through the driver entry
// point (no link-time dependency on libcuda) and a small error-string channel for the C ABI.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

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

// bf16 (or any 2-byte) tiled map with 128-byte swizzle. dims/strides innermost first;
// strides_bytes has rank-1 entries (stride of dim 1, 2, ...). The inner box extent must be 64
// elements (128 bytes) to match the swizzle span.
inline int make_tmap_2byte(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) UA_FAIL("cuTensorMapEncodeTiled entry point not found");
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) UA_FAIL("TMA base not 16-byte aligned");
  for (int i = 0; i + 1 < rank; ++i)
    if (gstr[i] % 16 != 0) UA_FAIL("TMA stride %d (%llu B) not a multiple of 16", i,
                                   (unsigned long long)gstr[i]);
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gdim, gstr,
                  bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) UA_FAIL("cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

// fp32 tiled map without swizzle (used as the destination of TMA reduce-add stores).
inline int make_tmap_f32(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) UA_FAIL("cuTensorMapEncodeTiled entry point not found");
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) UA_FAIL("TMA base not 16-byte aligned");
  for (int i = 0; i + 1 < rank; ++i)
    if (gstr[i] % 16 != 0) UA_FAIL("TMA stride %d (%llu B) not a multiple of 16", i,
                                   (unsigned long long)gstr[i]);
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, rank, const_cast<void*>(base), gdim, gstr,
                  bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) UA_FAIL("cuTensorMapEncodeTiled (f32) failed with code %d", (int)r);
  return 0;
}

}  // namespace ua
