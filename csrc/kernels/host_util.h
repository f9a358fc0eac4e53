// Host-side helpers for the kernel launchers: error codes, device attributes and
// TMA tensor-map encoding through the driver entry point (no link against libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#define TB_EXPORT extern "C" __attribute__((visibility("default")))

namespace tb {

// Launcher return codes (negative = refused before launch).
enum : int {
  TB_LAUNCH_OK = 0,
  TB_E_ARG = -1,        // bad shape / alignment / null pointer
  TB_E_CUDA = -2,       // a CUDA runtime call failed (see tb_last_error)
  TB_E_TMAP = -3,       // tensor map could not be encoded
  TB_E_TOO_LARGE = -4,  // size beyond a stated maximum
};

inline char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}
#define TB_FAIL(code, ...)                                   \
  do {                                                       \
    snprintf(tb::last_error_buf(), 512, __VA_ARGS__);        \
    return (code);                                           \
  } while (0)

#define TB_CUDA_CHECK(expr)                                                              \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess)                                                               \
      TB_FAIL(tb::TB_E_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),     \
              __FILE__, __LINE__);                                                       \
  } while (0)

// The library links the CUDA runtime statically, so its notion of "current device" is separate
// from the one of the process that loaded it, and it starts at device 0 in every new thread
// (autograd worker threads included). tb_set_device records the device the caller works on; every
// launcher makes it current on its own thread before touching the runtime or the driver.
inline std::atomic<int>& g_device() {
  static std::atomic<int> d{0};
  return d;
}
inline int ensure_device() {
  static thread_local int bound = -1;
  const int want = g_device().load(std::memory_order_relaxed);
  if (bound != want) {
    // cudaSetDevice initialises the device's primary context and makes it current on this thread (CUDA 12
    // semantics); no allocation routine is involved, which the allocation-free entry points rely on
    TB_CUDA_CHECK(cudaSetDevice(want));
    bound = want;
  }
  return 0;
}
#define TB_ENSURE_DEVICE()                       \
  do {                                           \
    if (int _r = tb::ensure_device()) return _r; \
  } while (0)

inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// rank-N bf16/f32 tiled map with 128-byte swizzle. dims[0] is the innermost extent,
// strides_bytes[i] is the byte stride of dims[i+1]. Returns 0 on success.
inline int make_tmap(CUtensorMap* map, const void* base, int elem_bytes, int rank,
                     const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                     bool swizzle128 = true) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) TB_FAIL(TB_E_TMAP, "cuTensorMapEncodeTiled entry point not available");
  if (((uintptr_t)base & 15) != 0) TB_FAIL(TB_E_ARG, "TMA base address not 16-byte aligned");
  for (int i = 0; i + 1 < rank; ++i)
    if (strides_bytes[i] % 16 != 0)
      TB_FAIL(TB_E_ARG, "TMA stride %d (%llu bytes) is not a multiple of 16", i,
              (unsigned long long)strides_bytes[i]);
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(map, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) TB_FAIL(TB_E_TMAP, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

}  // namespace tb
