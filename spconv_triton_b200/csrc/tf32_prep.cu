// Operand preparation for the fp32 convolutions on the tensor cores.
//
// tcgen05.mma kind::tf32 reads fp32 operands and uses their upper 19 bits (sign, 8 exponent
// bits, 10 mantissa bits).  Two preparations make that exact arithmetic on chosen operands:
//
//   SPC_TF32_ROUND   x -> rna(x): every value rounded to the nearest TF32 number (ties away from
//                    zero), the same rounding the reference's Triton dot applies to its operands
//                    when SPCONV_ALLOW_TF32 is set (_impl/gemm.py:55-62).  Without it the tensor
//                    core would truncate, which biases every product towards zero.
//   SPC_TF32_SPLIT_* x -> (hi, lo) with hi = rna(x), lo = rna(x - hi): x = hi + lo up to 2^-22 |x|.
//                    A convolution with reduction [hi_f | lo_f | hi_f] . [hi_w | hi_w | lo_w]
//                    = hi_f hi_w + lo_f hi_w + hi_f lo_w carries fp32-level accuracy (the dropped
//                    lo_f lo_w term is 2^-22 relative) through the TF32 tensor-core path at three
//                    times its work: this is how IEEE-mode fp32 layers reach the tensor cores.
//                    SPLIT_A lays a row out as [hi | lo | hi] (features, gradients), SPLIT_B as
//                    [hi | hi | lo] (weights).
#include <algorithm>

#include "common.cuh"

namespace spc {
namespace {

__device__ __forceinline__ float rna_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// ROUND mode on 16-byte vectors (the whole matrix is one contiguous run)
__global__ void __launch_bounds__(256)
tf32_round4_kernel(const float4* __restrict__ src, float4* __restrict__ dst, long long n4) {
  const long long stride = static_cast<long long>(gridDim.x) * 256;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n4; i += stride) {
    float4 v = __ldg(src + i);
    v.x = rna_tf32(v.x); v.y = rna_tf32(v.y); v.z = rna_tf32(v.z); v.w = rna_tf32(v.w);
    dst[i] = v;
  }
}

// one thread per source element
__global__ void __launch_bounds__(256)
tf32_prepare_kernel(const float* __restrict__ src, float* __restrict__ dst, long long rows, int cols, int mode) {
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  if (i >= rows * cols) return;
  const long long r = i / cols;
  const int c = static_cast<int>(i - r * cols);
  const float x = src[i];
  const float hi = rna_tf32(x);
  if (mode == SPC_TF32_ROUND) {
    dst[i] = hi;
    return;
  }
  const float lo = rna_tf32(x - hi);
  float* row = dst + r * 3 * cols;
  row[c] = hi;
  row[cols + c] = mode == SPC_TF32_SPLIT_A ? lo : hi;
  row[2 * cols + c] = mode == SPC_TF32_SPLIT_A ? hi : lo;
}

// weight [c_out, kv, c_in] -> dst [c_out, kv, m * c_in], or with `transpose` [c_in, kv, m * c_out]
// (dst[c][k][n] = w[n][k][c]): the reduction index innermost, as the forward-form kernel reads it.
__global__ void __launch_bounds__(256)
tf32_prepare_weight_kernel(const float* __restrict__ w, float* __restrict__ dst, int c_out, int kv, int c_in,
                           int transpose, int mode) {
  const long long i = blockIdx.x * 256ll + threadIdx.x;
  const long long total = static_cast<long long>(c_out) * kv * c_in;
  if (i >= total) return;
  const int c = static_cast<int>(i % c_in);
  const int k = static_cast<int>((i / c_in) % kv);
  const int n = static_cast<int>(i / (static_cast<long long>(c_in) * kv));
  const float x = w[i];
  const float hi = rna_tf32(x);
  const int m = mode == SPC_TF32_ROUND ? 1 : 3;
  const int red = transpose ? c_out : c_in;   // reduction extent of the prepared weight
  const int r = transpose ? n : c;            // this element's reduction index
  const int o = transpose ? c : n;            // and its output-channel index
  float* row = dst + (static_cast<long long>(o) * kv + k) * m * red;
  row[r] = hi;
  if (m == 3) {
    const float lo = rna_tf32(x - hi);
    row[red + r] = mode == SPC_TF32_SPLIT_A ? lo : hi;
    row[2 * red + r] = mode == SPC_TF32_SPLIT_A ? hi : lo;
  }
}

}  // namespace
}  // namespace spc

extern "C" int spc_tf32_prepare(const float* src, float* dst, int64_t rows, int cols, int mode, void* stream) {
  using namespace spc;
  if (!src || !dst || rows < 0 || cols <= 0 || mode < SPC_TF32_ROUND || mode > SPC_TF32_SPLIT_B)
    return fail(SPC_ERR_INVALID_ARGUMENT, "tf32_prepare: bad arguments");
  if (rows == 0) return SPC_OK;
  const long long total = static_cast<long long>(rows) * cols;
  const bool aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
  if (mode == SPC_TF32_ROUND && total % 4 == 0 && aligned) {
    const long long n4 = total / 4;
    const unsigned blocks = static_cast<unsigned>(std::min<long long>(ceil_div(n4, 256), 8ll * sm_count()));
    tf32_round4_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4*>(src), reinterpret_cast<float4*>(dst), n4);
    SPC_LAUNCH_OK();
    return SPC_OK;
  }
  tf32_prepare_kernel<<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, dst, rows, cols, mode);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

extern "C" int spc_tf32_prepare_weight(const float* weight, float* dst, int c_out, int kv, int c_in, int transpose,
                                       int mode, void* stream) {
  using namespace spc;
  if (!weight || !dst || c_out <= 0 || kv <= 0 || c_in <= 0 || mode < SPC_TF32_ROUND || mode > SPC_TF32_SPLIT_B)
    return fail(SPC_ERR_INVALID_ARGUMENT, "tf32_prepare_weight: bad arguments");
  const long long total = static_cast<long long>(c_out) * kv * c_in;
  tf32_prepare_weight_kernel<<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0,
                               static_cast<cudaStream_t>(stream)>>>(weight, dst, c_out, kv, c_in, transpose, mode);
  SPC_LAUNCH_OK();
  return SPC_OK;
}
