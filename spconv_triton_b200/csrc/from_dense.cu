// Dense -> sparse: which cells of a channels-last dense tensor hold a non-zero channel.
//
// Replaces SparseConvTensor.from_dense, spconv_triton/pytorch/core.py:296-318, which calls
// torch's to_sparse(ndim - 1): a cell becomes a row when any of its channels is non-zero, rows in
// ascending row-major cell order, all channels of the cell kept.  Here: one pass over the dense
// tensor marks cells (16-byte loads; value != 0 is a bit test with the sign bit cleared for
// floating types, so -0.0 is zero and NaN is not), a CUB exclusive sum numbers them, the host reads
// the count, and one kernel writes the coordinate rows.  The features are then read with
// spc_dense_gather.  HBM-bound: algorithmic bytes = cells * C * e (read) + 8 * cells (flags and
// numbers) + rows * ((ndim + 1) * 4 + 2 * C * e).
#include <cub/cub.cuh>

#include "common.cuh"

namespace spc {
namespace {

constexpr int kFdThreads = 256;

struct FdLayout {
  size_t off_flags, off_pos, off_cub, cub_bytes, total;
};

FdLayout fd_layout(int64_t cells) {
  FdLayout L;
  const size_t n = static_cast<size_t>(cells > 0 ? cells : 1);
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
  L.off_flags = take(n * 4);
  L.off_pos = take(n * 4);
  L.cub_bytes = 0;
  cub::DeviceScan::ExclusiveSum(nullptr, L.cub_bytes, static_cast<int*>(nullptr), static_cast<int*>(nullptr),
                                static_cast<int>(n));
  L.off_cub = take(L.cub_bytes);
  L.total = off;
  return L;
}

// E: unsigned integer of the element's size; `mask` clears the sign bit of floating types.
template <typename E>
__global__ void __launch_bounds__(kFdThreads)
fd_flag_kernel(const E* __restrict__ dense, long long total, int channels, E mask, int vectors, int* __restrict__ flags) {
  constexpr int kVec = 16 / sizeof(E);
  const long long stride = static_cast<long long>(gridDim.x) * kFdThreads;
  const long long t = static_cast<long long>(blockIdx.x) * kFdThreads + threadIdx.x;
  if (vectors) {
    struct alignas(16) Pack { E v[kVec]; };
    const long long nvec = total / kVec;
    for (long long v = t; v < nvec; v += stride) {
      const Pack p = reinterpret_cast<const Pack*>(dense)[v];
      long long cell = -1;
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        if ((p.v[j] & mask) != 0) {
          const long long c = (v * kVec + j) / channels;
          if (c != cell) flags[c] = 1;  // every writer stores the same value
          cell = c;
        }
      }
    }
    for (long long e = nvec * kVec + t; e < total; e += stride)
      if ((dense[e] & mask) != 0) flags[e / channels] = 1;
  } else {
    for (long long e = t; e < total; e += stride)
      if ((dense[e] & mask) != 0) flags[e / channels] = 1;
  }
}

struct FdGeo {
  int ndim;
  int shape[4];
};

__global__ void __launch_bounds__(kFdThreads)
fd_indices_kernel(const __grid_constant__ FdGeo g, const int* __restrict__ flags, const int* __restrict__ pos,
                  long long cells, int32_t* __restrict__ indices) {
  const long long cell = static_cast<long long>(blockIdx.x) * kFdThreads + threadIdx.x;
  if (cell >= cells || flags[cell] == 0) return;
  int32_t* row = indices + static_cast<long long>(pos[cell]) * (g.ndim + 1);
  long long rest = cell;
  for (int d = g.ndim - 1; d >= 0; --d) {
    row[d + 1] = static_cast<int32_t>(rest % g.shape[d]);
    rest /= g.shape[d];
  }
  row[0] = static_cast<int32_t>(rest);
}

template <typename E>
int fd_flag(const void* dense, int64_t total, int channels, E mask, int* flags, cudaStream_t st) {
  const int vectors = reinterpret_cast<uintptr_t>(dense) % 16 == 0;
  const int64_t work = vectors ? ceil_div(total, 16 / sizeof(E)) : total;
  const int blocks = static_cast<int>(std::min<int64_t>(ceil_div(work, kFdThreads), static_cast<int64_t>(sm_count()) * 32));
  fd_flag_kernel<E><<<blocks, kFdThreads, 0, st>>>(static_cast<const E*>(dense), total, channels, mask, vectors, flags);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

}  // namespace
}  // namespace spc

using namespace spc;

extern "C" size_t spc_from_dense_workspace_bytes(int64_t cells) { return fd_layout(cells).total; }

extern "C" int spc_from_dense_count(const void* dense, int64_t cells, int channels, int elem_size, int is_float,
                                    void* ws, size_t ws_bytes, int64_t* count, void* stream) {
  if (cells < 0 || cells >= (1ll << 31) || channels < 1 || count == nullptr)
    return fail(SPC_ERR_INVALID_ARGUMENT, "from_dense_count: bad argument");
  *count = 0;
  if (cells == 0) return SPC_OK;
  const FdLayout L = fd_layout(cells);
  if (ws == nullptr || ws_bytes < L.total)
    return fail(SPC_ERR_WORKSPACE_TOO_SMALL, "from_dense_count: workspace %zu < %zu", ws_bytes, L.total);
  auto st = static_cast<cudaStream_t>(stream);
  char* w = static_cast<char*>(ws);
  int* flags = reinterpret_cast<int*>(w + L.off_flags);
  int* pos = reinterpret_cast<int*>(w + L.off_pos);
  SPC_CUDA_OK(cudaMemsetAsync(flags, 0, static_cast<size_t>(cells) * 4, st));
  const int64_t total = cells * channels;
  int rc;
  switch (elem_size) {
    case 1: rc = fd_flag<uint8_t>(dense, total, channels, 0xffu, flags, st); break;
    case 2: rc = fd_flag<uint16_t>(dense, total, channels, is_float ? 0x7fffu : 0xffffu, flags, st); break;
    case 4: rc = fd_flag<uint32_t>(dense, total, channels, is_float ? 0x7fffffffu : 0xffffffffu, flags, st); break;
    case 8: rc = fd_flag<unsigned long long>(dense, total, channels, is_float ? 0x7fffffffffffffffull : ~0ull, flags, st); break;
    default: return fail(SPC_ERR_UNSUPPORTED, "from_dense_count: element size %d", elem_size);
  }
  if (rc != SPC_OK) return rc;
  size_t cub_bytes = L.cub_bytes;
  SPC_CUDA_OK(cub::DeviceScan::ExclusiveSum(w + L.off_cub, cub_bytes, flags, pos, static_cast<int>(cells), st));
  note_launch();
  int last[2] = {0, 0};
  SPC_CUDA_OK(cudaMemcpyAsync(&last[0], flags + cells - 1, 4, cudaMemcpyDeviceToHost, st));
  SPC_CUDA_OK(cudaMemcpyAsync(&last[1], pos + cells - 1, 4, cudaMemcpyDeviceToHost, st));
  SPC_CUDA_OK(cudaStreamSynchronize(st));
  *count = static_cast<int64_t>(last[0]) + last[1];
  return SPC_OK;
}

extern "C" int spc_from_dense_indices(const void* ws, int64_t cells, int ndim, const int32_t* spatial_shape,
                                      int32_t* indices, void* stream) {
  if (cells < 0 || cells >= (1ll << 31) || ndim < 1 || ndim > 4 || spatial_shape == nullptr || ws == nullptr)
    return fail(SPC_ERR_INVALID_ARGUMENT, "from_dense_indices: bad argument");
  if (cells == 0) return SPC_OK;
  const FdLayout L = fd_layout(cells);
  const char* w = static_cast<const char*>(ws);
  FdGeo g;
  g.ndim = ndim;
  for (int d = 0; d < 4; ++d) g.shape[d] = d < ndim ? spatial_shape[d] : 1;
  fd_indices_kernel<<<static_cast<int>(ceil_div(cells, kFdThreads)), kFdThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      g, reinterpret_cast<const int*>(w + L.off_flags), reinterpret_cast<const int*>(w + L.off_pos), cells, indices);
  SPC_LAUNCH_OK();
  return SPC_OK;
}
