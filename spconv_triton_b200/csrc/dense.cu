// Sparse -> dense scatter and its gradient (dense -> sparse gather).
//
// Replaces SparseConvTensor.dense() of the reference
// (spconv_triton/pytorch/core.py:320-334: scatter_nd into a zero tensor
// [B, *spatial, C], then permute(...).contiguous() to [B, C, *spatial]), which
// costs a zero fill, an index_put and a full read + write of the dense tensor.
// Here: one cudaMemsetAsync and one kernel that writes each voxel's channels
// straight into the requested layout; the gather is the same walk backwards.
// Pure data movement on 2-, 4- and 8-byte elements.  HBM-bound: algorithmic
// bytes = dense size (zero fill) + 2 * N * C * e (+ N * (ndim + 1) * 4).
//
// Channels-first writes are strided by the spatial volume, so a CTA stages a
// tile of 32 rows x up to 128 channels in shared memory and writes it
// transposed: one warp store covers 32 rows of one channel, which are
// neighbours in memory whenever the rows are neighbours along the last axis
// (the order every rulebook of this library emits).  Rows that share a
// coordinate overwrite each other in an unspecified order, as in the reference.
#include <algorithm>

#include "common.cuh"

namespace spc {
namespace {

constexpr int kDenseThreads = 256;
constexpr int kTileRows = 32;
constexpr int kTileCols = 128;

struct DenseGeo {
  int ndim;
  int batch;
  int shape[4];
  long long volume;
};

// Offset of row `r` in units of spatial cells (b * volume + linear coordinate), or -1 if outside.
__device__ __forceinline__ long long cell_of(const DenseGeo& g, const int32_t* __restrict__ idx, long long r) {
  const int32_t* p = idx + r * (g.ndim + 1);
  const int b = __ldg(&p[0]);
  if (b < 0 || b >= g.batch) return -1;
  long long lin = 0;
  for (int d = 0; d < g.ndim; ++d) {
    const int c = __ldg(&p[d + 1]);
    if (c < 0 || c >= g.shape[d]) return -1;
    lin = lin * g.shape[d] + c;
  }
  return static_cast<long long>(b) * g.volume + lin;
}

// GATHER = false: dense <- features ; true: features <- dense.  Channels first.
template <typename E, bool GATHER>
__global__ void __launch_bounds__(kDenseThreads)
dense_cf_kernel(const __grid_constant__ DenseGeo g, const int32_t* __restrict__ idx, long long n, int channels,
                E* __restrict__ feats, E* __restrict__ dense) {
  __shared__ E tile[kTileRows][kTileCols + 2];
  __shared__ long long base[kTileRows];
  const long long row0 = static_cast<long long>(blockIdx.x) * kTileRows;
  const int c0 = blockIdx.y * kTileCols;
  const int cw = min(kTileCols, channels - c0);
  const int tid = threadIdx.x;
  if (tid < kTileRows) {
    const long long r = row0 + tid;
    long long cell = r < n ? cell_of(g, idx, r) : -1;
    // element offset of channel 0 of this cell: (b * C) * volume + lin
    if (cell >= 0) {
      const long long b = cell / g.volume, lin = cell - b * g.volume;
      cell = b * channels * g.volume + lin;
    }
    base[tid] = cell;
  }
  if (!GATHER) {
    for (int e = tid; e < kTileRows * cw; e += kDenseThreads) {
      const int r = e / cw, c = e - r * cw;
      if (row0 + r < n) tile[r][c] = feats[(row0 + r) * channels + c0 + c];
    }
  }
  __syncthreads();
  for (int e = tid; e < kTileRows * cw; e += kDenseThreads) {
    const int c = e / kTileRows, r = e - c * kTileRows;
    const long long at = base[r];
    if (at < 0) {
      if (GATHER) tile[r][c] = E(0);
      continue;
    }
    E* cell = dense + at + static_cast<long long>(c0 + c) * g.volume;
    if (GATHER) tile[r][c] = *cell;
    else *cell = tile[r][c];
  }
  if (GATHER) {
    __syncthreads();
    for (int e = tid; e < kTileRows * cw; e += kDenseThreads) {
      const int r = e / cw, c = e - r * cw;
      if (row0 + r < n) feats[(row0 + r) * channels + c0 + c] = tile[r][c];
    }
  }
}

// Channels last: a row's channels are contiguous on both sides.
template <typename E, bool GATHER>
__global__ void __launch_bounds__(kDenseThreads)
dense_cl_kernel(const __grid_constant__ DenseGeo g, const int32_t* __restrict__ idx, long long n, int channels,
                E* __restrict__ feats, E* __restrict__ dense) {
  const long long e = blockIdx.x * static_cast<long long>(kDenseThreads) + threadIdx.x;
  const long long r = e / channels;
  if (r >= n) return;
  const int c = static_cast<int>(e - r * channels);
  const long long cell = cell_of(g, idx, r);
  if (cell < 0) {
    if (GATHER) feats[e] = E(0);
    return;
  }
  if (GATHER) feats[e] = dense[cell * channels + c];
  else dense[cell * channels + c] = feats[e];
}

template <typename E, bool GATHER>
int dense_launch(const DenseGeo& g, const int32_t* idx, int64_t n, int channels, int channels_first, void* feats,
                 void* dense, cudaStream_t st) {
  if (channels_first) {
    dim3 grid(static_cast<unsigned>(ceil_div(n, kTileRows)), static_cast<unsigned>(ceil_div(channels, kTileCols)));
    dense_cf_kernel<E, GATHER><<<grid, kDenseThreads, 0, st>>>(g, idx, n, channels, static_cast<E*>(feats),
                                                              static_cast<E*>(dense));
  } else {
    const unsigned blocks = static_cast<unsigned>(ceil_div(n * channels, kDenseThreads));
    dense_cl_kernel<E, GATHER><<<blocks, kDenseThreads, 0, st>>>(g, idx, n, channels, static_cast<E*>(feats),
                                                               static_cast<E*>(dense));
  }
  SPC_LAUNCH_OK();
  return SPC_OK;
}

template <bool GATHER>
int dense_dispatch(const int32_t* indices, int64_t n, int channels, int ndim, int batch, const int32_t* shape,
                   int channels_first, int elem_size, void* feats, void* dense, cudaStream_t st) {
  if (ndim < 1 || ndim > 4 || batch < 1 || channels < 1 || n < 0 || !shape || !dense || (n > 0 && (!indices || !feats)))
    return fail(SPC_ERR_INVALID_ARGUMENT, "dense: bad arguments");
  DenseGeo g{};
  g.ndim = ndim;
  g.batch = batch;
  g.volume = 1;
  for (int d = 0; d < ndim; ++d) {
    if (shape[d] < 1) return fail(SPC_ERR_INVALID_ARGUMENT, "dense: bad spatial shape");
    g.shape[d] = shape[d];
    g.volume *= shape[d];
  }
  if (!GATHER)
    SPC_CUDA_OK(cudaMemsetAsync(dense, 0, static_cast<size_t>(batch) * g.volume * channels * elem_size, st));
  if (n == 0) return SPC_OK;
  switch (elem_size) {
    case 2: return dense_launch<uint16_t, GATHER>(g, indices, n, channels, channels_first, feats, dense, st);
    case 4: return dense_launch<uint32_t, GATHER>(g, indices, n, channels, channels_first, feats, dense, st);
    case 8: return dense_launch<unsigned long long, GATHER>(g, indices, n, channels, channels_first, feats, dense, st);
    default: return fail(SPC_ERR_UNSUPPORTED, "dense: element size %d", elem_size);
  }
}

}  // namespace
}  // namespace spc

using namespace spc;

extern "C" int spc_dense_scatter(const void* features, const int32_t* indices, int64_t n, int channels, int ndim,
                                 int batch_size, const int32_t* spatial_shape, int channels_first, int elem_size,
                                 void* dense, void* stream) {
  return dense_dispatch<false>(indices, n, channels, ndim, batch_size, spatial_shape, channels_first, elem_size,
                               const_cast<void*>(features), dense, static_cast<cudaStream_t>(stream));
}

extern "C" int spc_dense_gather(const void* dense, const int32_t* indices, int64_t n, int channels, int ndim,
                                int batch_size, const int32_t* spatial_shape, int channels_first, int elem_size,
                                void* features, void* stream) {
  return dense_dispatch<true>(indices, n, channels, ndim, batch_size, spatial_shape, channels_first, elem_size,
                              features, const_cast<void*>(dense), static_cast<cudaStream_t>(stream));
}
