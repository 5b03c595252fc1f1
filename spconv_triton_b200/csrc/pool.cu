// Sparse max / average pooling over implicit-gemm pair tables.
//
// HBM-bound gather-reduce: one thread owns one 16-byte channel vector of one
// output row, walks the kv table entries of that row (pair[k*n + row] is
// shared by the threads of the row and served from L1), loads the gathered
// rows with 16-byte accesses and writes the result with one 16-byte store.
// Algorithmic bytes per output row: kv*4 (table) + pairs*C*e (gathered
// rows) + C*e (store).
//
// Semantics follow spconv_triton/pytorch/_impl/pool.py: the max accumulator starts at 0
// (pool.py:75-76), max backward credits every input equal to the output
// (pool.py:148-149), average divides by the number of inputs present
// (pool.py:200-201) and its backward MULTIPLIES by that count (pool.py:250-252).
// fp16/bf16/fp32 accumulate in fp32, fp64 in fp64 (pool.py:72-74).
#include <algorithm>

#include "common.cuh"

namespace spc {
namespace {

template <typename T> struct PoolAcc { using type = float; };
template <> struct PoolAcc<double> { using type = double; };

template <typename T> __device__ __forceinline__ typename PoolAcc<T>::type up(T v) { return to_float(v); }
template <> __device__ __forceinline__ double up<double>(double v) { return v; }
template <typename T> __device__ __forceinline__ T down(typename PoolAcc<T>::type v) { return from_float<T>(v); }
template <> __device__ __forceinline__ double down<double>(double v) { return v; }

template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };

template <typename T, int VEC>
__device__ __forceinline__ Pack<T, VEC> load_pack(const T* p) {
  return *reinterpret_cast<const Pack<T, VEC>*>(p);
}
template <typename T, int VEC>
__device__ __forceinline__ void store_pack(T* p, const Pack<T, VEC>& v) {
  *reinterpret_cast<Pack<T, VEC>*>(p) = v;
}

enum PoolOp { kMaxFwd, kAvgFwd };

template <typename T, int VEC, int OP>
__global__ void __launch_bounds__(256)
pool_fwd_kernel(const T* __restrict__ feats, const int32_t* __restrict__ pairs, T* __restrict__ out,
                int32_t* __restrict__ count, long long n_out, int channels, int kv) {
  using A = typename PoolAcc<T>::type;
  const int tpr = channels / VEC;
  const long long e = blockIdx.x * 256ll + threadIdx.x;
  const long long row = e / tpr;
  if (row >= n_out) return;
  const int c0 = static_cast<int>(e % tpr) * VEC;
  A acc[VEC];
#pragma unroll
  for (int u = 0; u < VEC; ++u) acc[u] = A(0);
  int cnt = 0;
  for (int k = 0; k < kv; ++k) {
    const int j = __ldg(&pairs[static_cast<long long>(k) * n_out + row]);
    if (j < 0) continue;
    const Pack<T, VEC> p = load_pack<T, VEC>(feats + static_cast<long long>(j) * channels + c0);
    ++cnt;
#pragma unroll
    for (int u = 0; u < VEC; ++u) {
      const A v = up<T>(p.v[u]);
      if (OP == kMaxFwd) acc[u] = v > acc[u] ? v : acc[u];
      else acc[u] += v;
    }
  }
  Pack<T, VEC> o;
  if (OP == kAvgFwd) {
    const A d = static_cast<A>(cnt > 1 ? cnt : 1);
#pragma unroll
    for (int u = 0; u < VEC; ++u) o.v[u] = down<T>(acc[u] / d);
    if (count != nullptr && c0 == 0) count[row] = cnt;
  } else {
#pragma unroll
    for (int u = 0; u < VEC; ++u) o.v[u] = down<T>(acc[u]);
  }
  store_pack<T, VEC>(out + row * channels + c0, o);
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256)
maxpool_bwd_kernel(const T* __restrict__ feats, const T* __restrict__ outf, const T* __restrict__ gout,
                   const int32_t* __restrict__ pair_bwd, T* __restrict__ din, long long n_in,
                   int channels, int kv) {
  using A = typename PoolAcc<T>::type;
  const int tpr = channels / VEC;
  const long long e = blockIdx.x * 256ll + threadIdx.x;
  const long long row = e / tpr;
  if (row >= n_in) return;
  const int c0 = static_cast<int>(e % tpr) * VEC;
  const Pack<T, VEC> f = load_pack<T, VEC>(feats + row * channels + c0);
  A acc[VEC];
#pragma unroll
  for (int u = 0; u < VEC; ++u) acc[u] = A(0);
  for (int k = 0; k < kv; ++k) {
    const int o = __ldg(&pair_bwd[static_cast<long long>(k) * n_in + row]);
    if (o < 0) continue;
    const Pack<T, VEC> ov = load_pack<T, VEC>(outf + static_cast<long long>(o) * channels + c0);
    const Pack<T, VEC> gv = load_pack<T, VEC>(gout + static_cast<long long>(o) * channels + c0);
#pragma unroll
    for (int u = 0; u < VEC; ++u)
      if (up<T>(ov.v[u]) == up<T>(f.v[u])) acc[u] += up<T>(gv.v[u]);
  }
  Pack<T, VEC> r;
#pragma unroll
  for (int u = 0; u < VEC; ++u) r.v[u] = down<T>(acc[u]);
  store_pack<T, VEC>(din + row * channels + c0, r);
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256)
avgpool_bwd_kernel(const T* __restrict__ gout, const int32_t* __restrict__ pair_bwd,
                   const int32_t* __restrict__ count, T* __restrict__ din, long long n_in, int channels,
                   int kv) {
  using A = typename PoolAcc<T>::type;
  const int tpr = channels / VEC;
  const long long e = blockIdx.x * 256ll + threadIdx.x;
  const long long row = e / tpr;
  if (row >= n_in) return;
  const int c0 = static_cast<int>(e % tpr) * VEC;
  A acc[VEC];
#pragma unroll
  for (int u = 0; u < VEC; ++u) acc[u] = A(0);
  for (int k = 0; k < kv; ++k) {
    const int o = __ldg(&pair_bwd[static_cast<long long>(k) * n_in + row]);
    if (o < 0) continue;
    const A cnt = static_cast<A>(__ldg(&count[o]));
    const Pack<T, VEC> gv = load_pack<T, VEC>(gout + static_cast<long long>(o) * channels + c0);
#pragma unroll
    for (int u = 0; u < VEC; ++u) acc[u] += up<T>(gv.v[u]) * cnt;
  }
  Pack<T, VEC> r;
#pragma unroll
  for (int u = 0; u < VEC; ++u) r.v[u] = down<T>(acc[u]);
  store_pack<T, VEC>(din + row * channels + c0, r);
}

template <typename T>
int vec_for(int channels, const void* a, const void* b, const void* c = nullptr, const void* d = nullptr) {
  constexpr int full = 16 / sizeof(T);
  auto aligned = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (channels % full == 0 && aligned(a) && aligned(b) && aligned(c) && aligned(d)) return full;
  return 1;
}

inline unsigned grid_for(long long rows, int tpr) {
  return static_cast<unsigned>(ceil_div(std::max<long long>(rows * tpr, 1), 256));
}

template <typename T, int OP>
int pool_fwd(const void* feats, const int32_t* pairs, void* out, int32_t* count, int64_t n_out, int channels,
             int kv, cudaStream_t st) {
  constexpr int full = 16 / sizeof(T);
  if (vec_for<T>(channels, feats, out) == full)
    pool_fwd_kernel<T, full, OP><<<grid_for(n_out, channels / full), 256, 0, st>>>(
        static_cast<const T*>(feats), pairs, static_cast<T*>(out), count, n_out, channels, kv);
  else
    pool_fwd_kernel<T, 1, OP><<<grid_for(n_out, channels), 256, 0, st>>>(
        static_cast<const T*>(feats), pairs, static_cast<T*>(out), count, n_out, channels, kv);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

template <typename T>
int maxpool_bwd(const void* feats, const void* outf, const void* gout, const int32_t* pb, void* din,
                int64_t n_in, int channels, int kv, cudaStream_t st) {
  constexpr int full = 16 / sizeof(T);
  if (vec_for<T>(channels, feats, outf, gout, din) == full)
    maxpool_bwd_kernel<T, full><<<grid_for(n_in, channels / full), 256, 0, st>>>(
        static_cast<const T*>(feats), static_cast<const T*>(outf), static_cast<const T*>(gout), pb,
        static_cast<T*>(din), n_in, channels, kv);
  else
    maxpool_bwd_kernel<T, 1><<<grid_for(n_in, channels), 256, 0, st>>>(
        static_cast<const T*>(feats), static_cast<const T*>(outf), static_cast<const T*>(gout), pb,
        static_cast<T*>(din), n_in, channels, kv);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

template <typename T>
int avgpool_bwd(const void* gout, const int32_t* pb, const int32_t* count, void* din, int64_t n_in,
                int channels, int kv, cudaStream_t st) {
  constexpr int full = 16 / sizeof(T);
  if (vec_for<T>(channels, gout, din) == full)
    avgpool_bwd_kernel<T, full><<<grid_for(n_in, channels / full), 256, 0, st>>>(
        static_cast<const T*>(gout), pb, count, static_cast<T*>(din), n_in, channels, kv);
  else
    avgpool_bwd_kernel<T, 1><<<grid_for(n_in, channels), 256, 0, st>>>(
        static_cast<const T*>(gout), pb, count, static_cast<T*>(din), n_in, channels, kv);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

#define SPC_POOL_DISPATCH(dtype, CALL)                                        \
  switch (dtype) {                                                            \
    case SPC_F16: { using T = __half; return CALL; }                          \
    case SPC_BF16: { using T = __nv_bfloat16; return CALL; }                  \
    case SPC_F32: { using T = float; return CALL; }                           \
    case SPC_F64: { using T = double; return CALL; }                          \
    default: return fail(SPC_ERR_UNSUPPORTED, "pool: dtype %d not supported", dtype); \
  }

bool pool_args_ok(const void* a, const void* b, const void* c, int64_t n, int channels, int kv) {
  return a && b && c && n >= 0 && channels > 0 && kv > 0;
}

}  // namespace
}  // namespace spc

using namespace spc;

extern "C" int spc_maxpool_forward(const void* features, const int32_t* pair_fwd, void* out, int64_t n_out,
                                   int channels, int kv, int dtype, void* stream) {
  if (!pool_args_ok(features, pair_fwd, out, n_out, channels, kv))
    return fail(SPC_ERR_INVALID_ARGUMENT, "maxpool_forward: bad arguments");
  if (n_out == 0) return SPC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SPC_POOL_DISPATCH(dtype, (pool_fwd<T, kMaxFwd>(features, pair_fwd, out, nullptr, n_out, channels, kv, st)));
}

extern "C" int spc_avgpool_forward(const void* features, const int32_t* pair_fwd, void* out, int32_t* count,
                                   int64_t n_out, int channels, int kv, int dtype, void* stream) {
  if (!pool_args_ok(features, pair_fwd, out, n_out, channels, kv))
    return fail(SPC_ERR_INVALID_ARGUMENT, "avgpool_forward: bad arguments");
  if (n_out == 0) return SPC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SPC_POOL_DISPATCH(dtype, (pool_fwd<T, kAvgFwd>(features, pair_fwd, out, count, n_out, channels, kv, st)));
}

extern "C" int spc_maxpool_backward(const void* features, const void* out_features, const void* grad_out,
                                    const int32_t* pair_bwd, void* din, int64_t n_in, int channels, int kv,
                                    int dtype, void* stream) {
  if (!pool_args_ok(features, pair_bwd, din, n_in, channels, kv) || !out_features || !grad_out)
    return fail(SPC_ERR_INVALID_ARGUMENT, "maxpool_backward: bad arguments");
  if (n_in == 0) return SPC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SPC_POOL_DISPATCH(dtype, (maxpool_bwd<T>(features, out_features, grad_out, pair_bwd, din, n_in, channels, kv, st)));
}

extern "C" int spc_avgpool_backward(const void* grad_out, const int32_t* pair_bwd, const int32_t* count,
                                    void* din, int64_t n_in, int channels, int kv, int dtype, void* stream) {
  if (!pool_args_ok(grad_out, pair_bwd, din, n_in, channels, kv) || !count)
    return fail(SPC_ERR_INVALID_ARGUMENT, "avgpool_backward: bad arguments");
  if (n_in == 0) return SPC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SPC_POOL_DISPATCH(dtype, (avgpool_bwd<T>(grad_out, pair_bwd, count, din, n_in, channels, kv, st)));
}
