// Host-side helpers shared by the launchers: error bookkeeping, TMA tensor-map
// construction through the driver entry point (no link-time dependency on
// libcuda), and shared-memory opt-in.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <mutex>
#include <utility>

#include "../../include/splash_sm100.h"

namespace splash {

inline char* last_error_buf() {
  static thread_local char buf[512] = "";
  return buf;
}

inline int fail(int status, const char* what, const char* detail = "") {
  snprintf(last_error_buf(), 512, "%s%s%s", what, detail[0] ? ": " : "", detail);
  return status;
}

#define SPLASH_CUDA_CHECK(expr)                                                      \
  do {                                                                               \
    cudaError_t _e = (expr);                                                         \
    if (_e != cudaSuccess) return ::splash::fail(SPLASH_CUDA_ERROR, #expr, cudaGetErrorString(_e)); \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes`-wide elements, box
// [box_rows, box_cols].  box_cols * elem_bytes must not exceed the swizzle span.
inline int make_tmap_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows,
                        uint64_t cols, uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(SPLASH_CUDA_ERROR, "cuTensorMapEncodeTiled entry point not found");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail(SPLASH_INVALID_ARGUMENT, "tensor base not 16-byte aligned");
  if ((cols * elem_bytes) % 16 != 0) return fail(SPLASH_INVALID_ARGUMENT, "row pitch not a multiple of 16 bytes");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char d[64];
    snprintf(d, sizeof d, "CUresult %d", static_cast<int>(r));
    return fail(SPLASH_CUDA_ERROR, "cuTensorMapEncodeTiled", d);
  }
  return SPLASH_OK;
}

inline CUtensorMapDataType tmap_dtype(int dtype) {
  return dtype == SPLASH_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

// Raises a kernel's dynamic shared-memory limit.  The attribute is per function and device and only
// ever needs to grow, so the largest size set so far is remembered per (function, device) and later
// calls cost one map lookup instead of a driver call.
inline int opt_in_smem_impl(const void* kernel, size_t bytes) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, int> granted;
  int dev = 0;
  SPLASH_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  int& have = granted[std::make_pair(kernel, dev)];
  if (have >= static_cast<int>(bytes)) return SPLASH_OK;
  SPLASH_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
  have = static_cast<int>(bytes);
  return SPLASH_OK;
}

template <typename Kernel>
inline int opt_in_smem(Kernel kernel, size_t bytes) {
  return opt_in_smem_impl(reinterpret_cast<const void*>(kernel), bytes);
}

constexpr size_t kMaxDynamicSmem = 227 * 1024;

}  // namespace splash
