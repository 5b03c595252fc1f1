// Shared helpers for the spconv_b200 translation units (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/spconv_b200.h"

namespace spc {

// Thread-local text of the last failure, returned by spc_last_error().
char* error_buffer();
// Process-wide count of kernels this library has launched (spc_launch_count()).
void note_launch();

inline int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return status;
}

#define SPC_CUDA_OK(expr)                                                                  \
  do {                                                                                     \
    cudaError_t e__ = (expr);                                                              \
    if (e__ != cudaSuccess)                                                                \
      return ::spc::fail(SPC_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                     \
                         cudaGetErrorString(e__), __FILE__, __LINE__);                     \
  } while (0)

#define SPC_LAUNCH_OK()                                                                    \
  do {                                                                                     \
    cudaError_t e__ = cudaGetLastError();                                                  \
    if (e__ != cudaSuccess)                                                                \
      return ::spc::fail(SPC_ERR_CUDA, "kernel launch failed: %s (%s:%d)",                 \
                         cudaGetErrorString(e__), __FILE__, __LINE__);                     \
    ::spc::note_launch();                                                                  \
  } while (0)

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline int sm_count() {
  static int cached = 0;
  if (cached == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
    if (cached <= 0) cached = 148;
  }
  return cached;
}

inline size_t dtype_size(int dtype) {
  switch (dtype) {
    case SPC_F16:
    case SPC_BF16:
      return 2;
    case SPC_F32:
      return 4;
    case SPC_F64:
      return 8;
    default:
      return 0;
  }
}

// Scalar conversions used by the CUDA-core kernels.
template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

}  // namespace spc
