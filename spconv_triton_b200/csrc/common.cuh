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

constexpr int kMaxDevices = 64;

// Ordinal of the current device, or -1 when it is outside the per-device tables below.
inline int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

// Multiprocessor count of the CURRENT device (remembered per device ordinal).
inline int sm_count() {
  static int cached[kMaxDevices] = {0};
  const int dev = current_device_slot();
  if (dev < 0) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

// The dynamic shared memory opt-in of a kernel is a per-device attribute: `done` (one flag per
// device ordinal, owned by the launcher of that kernel) remembers where it has been set.
template <typename Kernel>
inline cudaError_t ensure_dynamic_smem(Kernel kernel, int bytes, bool (&done)[kMaxDevices]) {
  const int dev = current_device_slot();
  if (dev >= 0 && done[dev]) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && dev >= 0) done[dev] = true;
  return e;
}

// What happens to an accumulator row before it is stored:
//   v = acc (+ bias[n]);  v = v * scale[n] + shift[n] (if scale);  v = act(v);  v += residual[row, n]
// bias has the dtype of the inputs; scale and shift are fp32 (a folded
// inference BatchNorm); act is an spc_activation; residual is a row-major
// [rows, n_dim] matrix of the OUTPUT dtype, added in fp32 before the one rounding
// of the store (a residual connection fused into the convolution).
struct Epilogue {
  const void* bias = nullptr;
  const float* scale = nullptr;
  const float* shift = nullptr;
  int act = 0;
  float alpha = 0.f;
  const void* residual = nullptr;
};

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

// residual[row, n .. n + 16) added to 16 consecutive accumulators (16-byte loads).
template <typename TO>
__device__ __forceinline__ void add_residual16(float* v, const TO* r) {
  if constexpr (sizeof(TO) == 4) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(r) + q);
      v[4 * q] += a.x; v[4 * q + 1] += a.y; v[4 * q + 2] += a.z; v[4 * q + 3] += a.w;
    }
  } else {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(r) + q);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        TO lo, hi;
        const unsigned short l16 = static_cast<unsigned short>(w[t] & 0xffffu), h16 = static_cast<unsigned short>(w[t] >> 16);
        lo = *reinterpret_cast<const TO*>(&l16);
        hi = *reinterpret_cast<const TO*>(&h16);
        v[8 * q + 2 * t] += to_float(lo);
        v[8 * q + 2 * t + 1] += to_float(hi);
      }
    }
  }
}

template <typename T>
__device__ __forceinline__ float apply_epilogue(float v, const Epilogue& e, int n) {
  if (e.bias != nullptr) v += to_float(static_cast<const T*>(e.bias)[n]);
  if (e.scale != nullptr) v = fmaf(v, __ldg(&e.scale[n]), __ldg(&e.shift[n]));
  if (e.act == SPC_ACT_RELU) v = fmaxf(v, 0.f);
  else if (e.act == SPC_ACT_LEAKY_RELU) v = v > 0.f ? v : v * e.alpha;
  else if (e.act == SPC_ACT_SIGMOID) v = 1.f / (1.f + __expf(-v));
  return v;
}

// The same epilogue with bias, scale and shift pre-combined per channel in
// shared memory by stage_epilogue(): v = act(v * sc[n] + sh[n]).
template <typename T>
__device__ __forceinline__ void stage_epilogue(const Epilogue& e, int n_dim, float* sc, float* sh, int tid,
                                               int n_threads) {
  for (int n = tid; n < n_dim; n += n_threads) {
    const float scale = e.scale != nullptr ? e.scale[n] : 1.f;
    float shift = e.shift != nullptr ? e.shift[n] : 0.f;
    if (e.bias != nullptr) shift = fmaf(to_float(static_cast<const T*>(e.bias)[n]), scale, shift);
    sc[n] = scale;
    sh[n] = shift;
  }
}
// 16 consecutive channels at once; sc / sh point to 16-byte aligned shared memory.
__device__ __forceinline__ void finish_epilogue16(float* v, const float* sc, const float* sh, int act, float alpha) {
  float s[16], t[16];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float4 a = reinterpret_cast<const float4*>(sc)[q];
    const float4 b = reinterpret_cast<const float4*>(sh)[q];
    s[4 * q] = a.x; s[4 * q + 1] = a.y; s[4 * q + 2] = a.z; s[4 * q + 3] = a.w;
    t[4 * q] = b.x; t[4 * q + 1] = b.y; t[4 * q + 2] = b.z; t[4 * q + 3] = b.w;
  }
  if (act == SPC_ACT_RELU) {
#pragma unroll
    for (int q = 0; q < 16; ++q) v[q] = fmaxf(fmaf(v[q], s[q], t[q]), 0.f);
  } else if (act == SPC_ACT_NONE) {
#pragma unroll
    for (int q = 0; q < 16; ++q) v[q] = fmaf(v[q], s[q], t[q]);
  } else {
#pragma unroll
    for (int q = 0; q < 16; ++q) {
      const float x = fmaf(v[q], s[q], t[q]);
      v[q] = act == SPC_ACT_LEAKY_RELU ? (x > 0.f ? x : x * alpha) : 1.f / (1.f + __expf(-x));
    }
  }
}
__device__ __forceinline__ float finish_epilogue(float v, float sc, float sh, int act, float alpha) {
  v = fmaf(v, sc, sh);
  if (act == SPC_ACT_RELU) v = fmaxf(v, 0.f);
  else if (act == SPC_ACT_LEAKY_RELU) v = v > 0.f ? v : v * alpha;
  else if (act == SPC_ACT_SIGMOID) v = 1.f / (1.f + __expf(-v));
  return v;
}

}  // namespace spc
