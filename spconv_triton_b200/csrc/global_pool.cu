// Per-sample reduction over all voxels of a sparse tensor.
//
// Replaces SparseGlobalMaxOrAvgPool.forward, spconv_triton/pytorch/pool.py:238-265, which
// rearranges the rows per sample (ops.py:436-450: bincount, stable argsort, index_put), reads
// the counts on the host and then runs one gather + torch.max / torch.mean per sample.
//   max:  out[b, c] = max over rows r of sample b of features[r, c]   (NaN wins, as torch.max)
//         argmax[b, c] = the smallest such row (for the gradient)
//   mean: out[b]    = mean over rows of sample b of features[r, 0]    (upstream returns channel 0
//         of the mean vector only, pool.py:258-261)
// One pass over the features, any row order.  A thread walks a run of rows of one channel and
// flushes to global memory only when the sample changes, so tensors in batch order (what every
// rulebook emits) cost one atomic per thread.  HBM-bound: algorithmic bytes = N * C * e (max) or
// N * 32 B (mean: one sector per row), + N * 4 for the batch column.
#include <algorithm>

#include "common.cuh"

namespace spc {
namespace {

constexpr int kGpThreads = 128;
constexpr int kGpRows = 128;  // rows per CTA in the max kernel, per thread in the count kernel

template <typename T> __device__ __forceinline__ float as_float(T v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float as_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float as_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Monotone map float -> uint32 (NaN above +inf), and back.
__device__ __forceinline__ uint32_t ordered(float f) {
  if (f != f) return 0xffc00000u;
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float unordered(uint32_t o) {
  if (o == 0xffc00000u) return __int_as_float(0x7fc00000);
  return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}

struct GpWs {
  unsigned long long* best;  // [batch, channels] (ordered value << 32) | (0xffffffff - row)
  double* sum;               // [batch] sum of channel 0
  int* count;                // [batch]
};

inline size_t gp_bytes(int batch, int channels) {
  return align_up(static_cast<size_t>(batch) * channels * 8, 256) + align_up(static_cast<size_t>(batch) * 8, 256) +
         align_up(static_cast<size_t>(batch) * 4, 256);
}

inline GpWs gp_view(void* ws, int batch, int channels) {
  char* p = static_cast<char*>(ws);
  GpWs w;
  w.best = reinterpret_cast<unsigned long long*>(p);
  p += align_up(static_cast<size_t>(batch) * channels * 8, 256);
  w.sum = reinterpret_cast<double*>(p);
  p += align_up(static_cast<size_t>(batch) * 8, 256);
  w.count = reinterpret_cast<int*>(p);
  return w;
}

// Rows per sample and the sum of channel 0; each thread owns kGpRows consecutive rows.
template <typename T>
__global__ void __launch_bounds__(kGpThreads)
gp_count_kernel(const T* __restrict__ feats, const int32_t* __restrict__ idx, long long n, int channels, int width,
                int batch, GpWs w, int with_sum) {
  const long long t = static_cast<long long>(blockIdx.x) * kGpThreads + threadIdx.x;
  const long long r0 = t * kGpRows, r1 = min(n, r0 + kGpRows);
  int cur = -1, cnt = 0;
  double acc = 0.0;
  for (long long r = r0; r < r1; ++r) {
    const int b = __ldg(&idx[r * width]);
    if (b != cur) {
      if (cur >= 0 && cur < batch) {
        atomicAdd(&w.count[cur], cnt);
        if (with_sum) atomicAdd(&w.sum[cur], acc);
      }
      cur = b, cnt = 0, acc = 0.0;
    }
    ++cnt;
    if (with_sum) acc += static_cast<double>(as_float(feats[r * channels]));
  }
  if (cur >= 0 && cur < batch) {
    atomicAdd(&w.count[cur], cnt);
    if (with_sum) atomicAdd(&w.sum[cur], acc);
  }
}

// A CTA takes kGpRows rows; thread c walks them for channels c, c + 128, ...
template <typename T>
__global__ void __launch_bounds__(kGpThreads)
gp_max_kernel(const T* __restrict__ feats, const int32_t* __restrict__ idx, long long n, int channels, int width,
              int batch, GpWs w) {
  __shared__ int sample[kGpRows];
  const long long r0 = static_cast<long long>(blockIdx.x) * kGpRows;
  const int rows = static_cast<int>(min(static_cast<long long>(kGpRows), n - r0));
  for (int i = threadIdx.x; i < rows; i += kGpThreads) sample[i] = __ldg(&idx[(r0 + i) * width]);
  __syncthreads();
  for (int c = threadIdx.x; c < channels; c += kGpThreads) {
    int cur = -1;
    unsigned long long best = 0;
    constexpr int kAhead = 8;  // loads of eight rows are issued before any of them is compared
    for (int i0 = 0; i0 < rows; i0 += kAhead) {
      float v[kAhead];
#pragma unroll
      for (int j = 0; j < kAhead; ++j)
        v[j] = i0 + j < rows ? as_float(feats[(r0 + i0 + j) * channels + c]) : 0.f;
#pragma unroll
      for (int j = 0; j < kAhead; ++j) {
        const int i = i0 + j;
        if (i >= rows) break;
        const int b = sample[i];
        if (b != cur) {
          if (cur >= 0 && cur < batch) atomicMax(&w.best[static_cast<long long>(cur) * channels + c], best);
          cur = b, best = 0;
        }
        const unsigned long long cand = (static_cast<unsigned long long>(ordered(v[j])) << 32) |
                                        (0xffffffffu - static_cast<uint32_t>(r0 + i));
        best = cand > best ? cand : best;
      }
    }
    if (cur >= 0 && cur < batch) atomicMax(&w.best[static_cast<long long>(cur) * channels + c], best);
  }
}

template <typename T>
__global__ void __launch_bounds__(kGpThreads)
gp_finish_kernel(GpWs w, int batch, int channels, int is_mean, T* __restrict__ out, int32_t* __restrict__ argmax,
                 int32_t* __restrict__ counts) {
  const int i = blockIdx.x * kGpThreads + threadIdx.x;
  if (i < batch && counts != nullptr) counts[i] = w.count[i];
  if (is_mean) {
    if (i < batch) out[i] = from_float<T>(static_cast<float>(w.sum[i] / static_cast<double>(w.count[i])));
    return;
  }
  if (i >= batch * channels) return;
  const unsigned long long v = w.best[i];
  out[i] = from_float<T>(unordered(static_cast<uint32_t>(v >> 32)));
  if (argmax != nullptr) argmax[i] = v == 0 ? -1 : static_cast<int32_t>(0xffffffffu - static_cast<uint32_t>(v));
}

template <typename T>
int gp_typed(const void* feats, const int32_t* idx, int64_t n, int channels, int width, int batch, int is_mean,
             void* ws, void* out, int32_t* argmax, int32_t* counts, cudaStream_t st) {
  GpWs w = gp_view(ws, batch, channels);
  SPC_CUDA_OK(cudaMemsetAsync(ws, 0, gp_bytes(batch, channels), st));
  if (n > 0) {
    const int64_t threads = ceil_div(n, kGpRows);
    gp_count_kernel<T><<<static_cast<int>(ceil_div(threads, kGpThreads)), kGpThreads, 0, st>>>(
        static_cast<const T*>(feats), idx, n, channels, width, batch, w, is_mean);
    SPC_LAUNCH_OK();
    if (!is_mean) {
      gp_max_kernel<T><<<static_cast<int>(ceil_div(n, kGpRows)), kGpThreads, 0, st>>>(
          static_cast<const T*>(feats), idx, n, channels, width, batch, w);
      SPC_LAUNCH_OK();
    }
  }
  const int outs = is_mean ? batch : batch * channels;
  gp_finish_kernel<T><<<static_cast<int>(ceil_div(std::max(outs, batch), kGpThreads)), kGpThreads, 0, st>>>(
      w, batch, channels, is_mean, static_cast<T*>(out), argmax, counts);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

}  // namespace
}  // namespace spc

using namespace spc;

extern "C" size_t spc_global_pool_workspace_bytes(int batch, int channels) {
  return batch > 0 && channels > 0 ? gp_bytes(batch, channels) : 0;
}

extern "C" int spc_global_pool(const void* features, const int32_t* indices, int64_t n, int channels, int idx_width,
                               int batch, int dtype, int is_mean, void* ws, size_t ws_bytes, void* out,
                               int32_t* argmax, int32_t* counts, void* stream) {
  if (n < 0 || n > 0xfffffffell || channels < 1 || idx_width < 1 || batch < 1 || out == nullptr)
    return fail(SPC_ERR_INVALID_ARGUMENT, "global_pool: bad argument");
  if (ws == nullptr || ws_bytes < gp_bytes(batch, channels))
    return fail(SPC_ERR_WORKSPACE_TOO_SMALL, "global_pool: workspace %zu < %zu", ws_bytes, gp_bytes(batch, channels));
  auto st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SPC_F16: return gp_typed<__half>(features, indices, n, channels, idx_width, batch, is_mean, ws, out, argmax, counts, st);
    case SPC_BF16: return gp_typed<__nv_bfloat16>(features, indices, n, channels, idx_width, batch, is_mean, ws, out, argmax, counts, st);
    case SPC_F32: return gp_typed<float>(features, indices, n, channels, idx_width, batch, is_mean, ws, out, argmax, counts, st);
    default: return fail(SPC_ERR_UNSUPPORTED, "global_pool: dtype %d (fp16, bf16 and fp32 only)", dtype);
  }
}
