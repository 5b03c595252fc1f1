// Point cloud voxelisation (points -> voxels) on the GPU, first come first served.
//
// Semantics follow PointToVoxel.generate_voxel_with_id,
// spconv_triton/pytorch/utils.py:72-163, which states them with torch sorts:
//   * a point's voxel is floor((p - cmin) / vsize) per axis, in the dtype of the
//     points (fp32 here: one IEEE subtraction, one IEEE division, floor);
//   * voxels are numbered in the order of their first point (utils.py:107-114);
//     only the first max_voxels voxels are kept, points of the others get id -1;
//   * inside a voxel the points keep their arrival order; the first max_points
//     are stored, the others keep the voxel id but are not stored (utils.py:129-144);
//   * num_per_voxel is the true count clamped at max_points (utils.py:119-120);
//   * voxel coordinates are written reversed (z, y, x) (utils.py:122-128);
//   * empty_mean fills the unused slots of a voxel with the mean of its stored
//     points (utils.py:146-153).
// The result is deterministic and equal to the reference's, bit for bit.
//
// How it is computed here (no global sort of the points by voxel key):
//   1. quantize_insert: key per point; a hash table keeps, per key, the lowest
//      point index (one packed 64-bit atomicMin: key << 32 | index);
//   2. mark_first: a point is "first" when the table returns its own index;
//      an exclusive prefix sum over these flags IS the voxel number of each
//      first point, because voxel order = order of first points;
//   3. the host reads the number of voxels (the reference reads uniq.numel() too);
//   4. assign: every point looks up its voxel's number, counts itself in and
//      becomes a (voxel number, point index) pair; first points write the
//      voxel coordinates;
//   5. a stable radix sort of the pairs by voxel number keeps arrival order
//      inside a voxel; position - (start of the voxel's segment) is the slot;
//   6. scatter copies the stored points; fill_mean pads when asked.
// HBM-bound; algorithmic bytes per point: 4*F read + 4*F written (stored
// points) + 8 (voxel id) + the clear of the voxel buffer when requested.
#include <cub/cub.cuh>

#include <algorithm>

#include "common.cuh"

namespace spc {
namespace {

constexpr int kVoxThreads = 256;
constexpr int kVoxMaxDim = 4;
constexpr unsigned long long kVoxEmpty = ~0ull;
constexpr uint32_t kNoKey = 0xffffffffu;

struct VoxGeo {
  int ndim;
  float cmin[kVoxMaxDim];
  float vsize[kVoxMaxDim];
  int grid[kVoxMaxDim];  // x, y, z order, as given
};

__device__ __forceinline__ uint32_t vox_mix(uint32_t h) {
  h ^= h >> 16;
  h *= 0x85ebca6bu;
  h ^= h >> 13;
  h *= 0xc2b2ae35u;
  h ^= h >> 16;
  return h;
}

inline unsigned vox_blocks(int64_t n) { return static_cast<unsigned>(ceil_div(std::max<int64_t>(n, 1), kVoxThreads)); }

__global__ void __launch_bounds__(kVoxThreads)
quantize_insert_kernel(const __grid_constant__ VoxGeo g, const float* __restrict__ points, long long n,
                       int point_stride, unsigned long long* __restrict__ slots, uint32_t cap_mask,
                       uint32_t* __restrict__ keys, int* __restrict__ status) {
  const long long i = blockIdx.x * static_cast<long long>(kVoxThreads) + threadIdx.x;
  if (i >= n) return;
  const float* p = points + i * point_stride;
  uint32_t key = 0;
  bool in_range = true;
  for (int d = 0; d < g.ndim; ++d) {
    const float q = floorf(__fdiv_rn(__fsub_rn(__ldg(&p[d]), g.cmin[d]), g.vsize[d]));
    // NaN and out-of-range both fail the comparison chain
    if (!(q >= 0.f && q < static_cast<float>(g.grid[d]))) {
      in_range = false;
      break;
    }
    key = key * static_cast<uint32_t>(g.grid[d]) + static_cast<uint32_t>(q);
  }
  if (!in_range) {
    keys[i] = kNoKey;
    return;
  }
  keys[i] = key;
  const unsigned long long packed = (static_cast<unsigned long long>(key) << 32) | static_cast<uint32_t>(i);
  uint32_t s = vox_mix(key) & cap_mask;
  for (uint32_t probe = 0; probe <= cap_mask; ++probe) {
    const unsigned long long old = atomicCAS(&slots[s], kVoxEmpty, packed);
    if (old == kVoxEmpty) return;
    if (static_cast<uint32_t>(old >> 32) == key) {
      atomicMin(&slots[s], packed);
      return;
    }
    s = (s + 1) & cap_mask;
  }
  atomicExch(status, SPC_ERR_HASH_TABLE_FULL);
}

__device__ __forceinline__ int vox_find(const unsigned long long* __restrict__ slots, uint32_t cap_mask, uint32_t key) {
  uint32_t s = vox_mix(key) & cap_mask;
  for (uint32_t probe = 0; probe <= cap_mask; ++probe) {
    const unsigned long long v = slots[s];
    if (v == kVoxEmpty) return -1;
    if (static_cast<uint32_t>(v >> 32) == key) return static_cast<int>(v & 0xffffffffu);
    s = (s + 1) & cap_mask;
  }
  return -1;
}

// first[i] = index of the first point of i's voxel (or -1); flag[i] = 1 when that is i itself.
__global__ void __launch_bounds__(kVoxThreads)
mark_first_kernel(const uint32_t* __restrict__ keys, long long n, const unsigned long long* __restrict__ slots,
                  uint32_t cap_mask, int* __restrict__ first, int* __restrict__ flag) {
  const long long i = blockIdx.x * static_cast<long long>(kVoxThreads) + threadIdx.x;
  if (i >= n) return;
  const uint32_t key = keys[i];
  const int f = key == kNoKey ? -1 : vox_find(slots, cap_mask, key);
  first[i] = f;
  flag[i] = (f == static_cast<int>(i)) ? 1 : 0;
}

// status[1] = number of voxels found (rank of the last point + its flag): one word for the host to read.
__global__ void total_kernel(const int* __restrict__ rank, const int* __restrict__ flag, long long n, int* __restrict__ status) {
  status[1] = rank[n - 1] + flag[n - 1];
}

__global__ void __launch_bounds__(kVoxThreads)
assign_kernel(const __grid_constant__ VoxGeo g, const uint32_t* __restrict__ keys, const int* __restrict__ first,
              const int* __restrict__ rank, long long n, long long num_voxels, int* __restrict__ counts,
              uint32_t* __restrict__ sort_keys, int* __restrict__ sort_vals, long long* __restrict__ pc_voxel_id,
              int32_t* __restrict__ indices) {
  const long long i = blockIdx.x * static_cast<long long>(kVoxThreads) + threadIdx.x;
  if (i >= n) return;
  const int f = first[i];
  long long vid = -1;
  if (f >= 0) {
    vid = rank[f];
    if (vid >= num_voxels) vid = -1;  // beyond the voxel cap
  }
  pc_voxel_id[i] = vid;
  sort_keys[i] = vid >= 0 ? static_cast<uint32_t>(vid) : static_cast<uint32_t>(num_voxels);  // dropped: behind every voxel
  sort_vals[i] = static_cast<int>(i);
  if (vid < 0) return;
  atomicAdd(&counts[vid], 1);
  if (f == static_cast<int>(i)) {
    // the voxel's coordinates, reversed to (z, y, x)
    uint32_t rem = keys[i];
    for (int d = g.ndim - 1; d >= 0; --d) {
      const uint32_t gd = static_cast<uint32_t>(g.grid[d]);
      indices[vid * g.ndim + (g.ndim - 1 - d)] = static_cast<int32_t>(rem % gd);
      rem /= gd;
    }
  }
}

__global__ void __launch_bounds__(kVoxThreads)
clamp_counts_kernel(const int* __restrict__ counts, long long num_voxels, int max_points,
                    int32_t* __restrict__ num_per_voxel) {
  const long long v = blockIdx.x * static_cast<long long>(kVoxThreads) + threadIdx.x;
  if (v < num_voxels) num_per_voxel[v] = min(counts[v], max_points);
}

// One thread per (sorted position, feature).
__global__ void __launch_bounds__(kVoxThreads)
scatter_points_kernel(const float* __restrict__ points, int point_stride, int num_features,
                      const uint32_t* __restrict__ sorted_vid, const int* __restrict__ sorted_idx,
                      const int* __restrict__ seg_start, long long n_kept, long long num_voxels, int max_points,
                      float* __restrict__ voxels) {
  const long long e = blockIdx.x * static_cast<long long>(kVoxThreads) + threadIdx.x;
  const long long pos = e / num_features;
  if (pos >= n_kept) return;
  const int c = static_cast<int>(e - pos * num_features);
  const uint32_t vid = sorted_vid[pos];
  if (vid >= num_voxels) return;  // out of range or beyond the voxel cap: sorted behind every kept point
  const long long slot = pos - seg_start[vid];
  if (slot >= max_points) return;
  voxels[(static_cast<long long>(vid) * max_points + slot) * num_features + c] =
      __ldg(&points[static_cast<long long>(sorted_idx[pos]) * point_stride + c]);
}

// One thread per (voxel, feature): unused slots take the mean of the stored points,
// summed in slot order over ALL max_points slots as the reference's sum(dim=1) does.
__global__ void __launch_bounds__(kVoxThreads)
fill_mean_kernel(float* __restrict__ voxels, const int32_t* __restrict__ num_per_voxel, long long num_voxels,
                 int max_points, int num_features) {
  const long long e = blockIdx.x * static_cast<long long>(kVoxThreads) + threadIdx.x;
  const long long v = e / num_features;
  if (v >= num_voxels) return;
  const int c = static_cast<int>(e - v * num_features);
  const int npv = num_per_voxel[v];
  float* base = voxels + (v * max_points) * num_features + c;
  float sum = 0.f;
  for (int s = 0; s < max_points; ++s) sum += base[static_cast<long long>(s) * num_features];
  const float mean = __fdiv_rn(sum, static_cast<float>(npv > 1 ? npv : 1));
  for (int s = npv; s < max_points; ++s) base[static_cast<long long>(s) * num_features] = mean;
}

uint32_t vox_pow2_at_least(int64_t v) {
  uint32_t c = 1;
  while (static_cast<int64_t>(c) < v && c < (1u << 31)) c <<= 1;
  return c;
}

struct VoxLayout {
  uint32_t cap;
  size_t off_status, off_slots, off_keys, off_first, off_flag, off_rank, off_counts, off_seg, off_sk_a, off_sk_b,
      off_sv_a, off_sv_b, off_cub, cub_bytes, total;
};

VoxLayout vox_layout(int64_t n, int64_t max_voxels) {
  VoxLayout L{};
  L.cap = vox_pow2_at_least(2 * std::max<int64_t>(n, 1));
  size_t scan_bytes = 0, sort_bytes = 0;
  cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, static_cast<int*>(nullptr), static_cast<int*>(nullptr),
                                static_cast<int>(std::max<int64_t>(n, max_voxels)));
  cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, static_cast<uint32_t*>(nullptr), static_cast<uint32_t*>(nullptr),
                                  static_cast<int*>(nullptr), static_cast<int*>(nullptr), static_cast<int>(n));
  L.cub_bytes = std::max(scan_bytes, sort_bytes);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off = align_up(off + bytes, 256);
    return at;
  };
  const size_t np = static_cast<size_t>(std::max<int64_t>(n, 1));
  const size_t nv = static_cast<size_t>(std::max<int64_t>(max_voxels, 1));
  L.off_status = take(256);
  L.off_slots = take(static_cast<size_t>(L.cap) * 8);
  L.off_keys = take(np * 4);
  L.off_first = take(np * 4);
  L.off_flag = take(np * 4);
  L.off_rank = take(np * 4);
  L.off_counts = take(nv * 4);
  L.off_seg = take(nv * 4);
  L.off_sk_a = take(np * 4);
  L.off_sk_b = take(np * 4);
  L.off_sv_a = take(np * 4);
  L.off_sv_b = take(np * 4);
  L.off_cub = take(L.cub_bytes);
  L.total = off;
  return L;
}

}  // namespace
}  // namespace spc

using namespace spc;

extern "C" size_t spc_voxelize_workspace_bytes(int64_t n_points, int64_t max_voxels) {
  if (n_points < 0 || max_voxels <= 0 || n_points >= (1ll << 30)) return 0;
  return vox_layout(n_points, max_voxels).total;
}

extern "C" int spc_voxelize(const float* points, int64_t n_points, int point_stride, int ndim, int num_features,
                            const float* cmin, const float* vsize, const int32_t* grid_xyz, int64_t max_voxels,
                            int max_points, int clear_voxels, int empty_mean, void* workspace,
                            size_t workspace_bytes, float* voxels, int32_t* indices, int32_t* num_per_voxel,
                            int64_t* pc_voxel_id, int64_t* num_voxels_host, void* stream) {
  if (!num_voxels_host || !cmin || !vsize || !grid_xyz || ndim < 1 || ndim > kVoxMaxDim || num_features < 1 ||
      point_stride < std::max(ndim, num_features) || max_voxels <= 0 || max_points <= 0 || n_points < 0 ||
      !voxels || !indices || !num_per_voxel || !workspace)
    return fail(SPC_ERR_INVALID_ARGUMENT, "voxelize: bad arguments");
  if (n_points >= (1ll << 30)) return fail(SPC_ERR_SIZE_LIMIT, "voxelize: %lld points", static_cast<long long>(n_points));
  VoxGeo g{};
  g.ndim = ndim;
  double volume = 1;
  for (int d = 0; d < ndim; ++d) {
    if (grid_xyz[d] <= 0 || !(vsize[d] > 0.f)) return fail(SPC_ERR_INVALID_ARGUMENT, "voxelize: bad grid");
    g.cmin[d] = cmin[d];
    g.vsize[d] = vsize[d];
    g.grid[d] = grid_xyz[d];
    volume *= grid_xyz[d];
  }
  if (volume >= 4294967295.0) return fail(SPC_ERR_SIZE_LIMIT, "voxelize: grid of %.0f cells needs keys beyond 32 bits", volume);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  *num_voxels_host = 0;
  if (clear_voxels)
    SPC_CUDA_OK(cudaMemsetAsync(voxels, 0, static_cast<size_t>(max_voxels) * max_points * num_features * sizeof(float), st));
  if (n_points == 0) return SPC_OK;
  if (!points || !pc_voxel_id) return fail(SPC_ERR_INVALID_ARGUMENT, "voxelize: null points");
  const VoxLayout L = vox_layout(n_points, max_voxels);
  if (workspace_bytes < L.total)
    return fail(SPC_ERR_WORKSPACE_TOO_SMALL, "voxelize: workspace %zu < %zu bytes", workspace_bytes, L.total);
  char* ws = static_cast<char*>(workspace);
  int* status = reinterpret_cast<int*>(ws + L.off_status);
  unsigned long long* slots = reinterpret_cast<unsigned long long*>(ws + L.off_slots);
  uint32_t* keys = reinterpret_cast<uint32_t*>(ws + L.off_keys);
  int* first = reinterpret_cast<int*>(ws + L.off_first);
  int* flag = reinterpret_cast<int*>(ws + L.off_flag);
  int* rank = reinterpret_cast<int*>(ws + L.off_rank);
  int* counts = reinterpret_cast<int*>(ws + L.off_counts);
  int* seg = reinterpret_cast<int*>(ws + L.off_seg);
  uint32_t* sk_a = reinterpret_cast<uint32_t*>(ws + L.off_sk_a);
  uint32_t* sk_b = reinterpret_cast<uint32_t*>(ws + L.off_sk_b);
  int* sv_a = reinterpret_cast<int*>(ws + L.off_sv_a);
  int* sv_b = reinterpret_cast<int*>(ws + L.off_sv_b);
  const uint32_t cap_mask = L.cap - 1;
  const int n = static_cast<int>(n_points);

  SPC_CUDA_OK(cudaMemsetAsync(status, 0, 256, st));
  SPC_CUDA_OK(cudaMemsetAsync(slots, 0xFF, static_cast<size_t>(L.cap) * 8, st));
  quantize_insert_kernel<<<vox_blocks(n), kVoxThreads, 0, st>>>(g, points, n, point_stride, slots, cap_mask, keys, status);
  SPC_LAUNCH_OK();
  mark_first_kernel<<<vox_blocks(n), kVoxThreads, 0, st>>>(keys, n, slots, cap_mask, first, flag);
  SPC_LAUNCH_OK();
  size_t cub_bytes = L.cub_bytes;
  SPC_CUDA_OK(cub::DeviceScan::ExclusiveSum(ws + L.off_cub, cub_bytes, flag, rank, n, st));
  total_kernel<<<1, 1, 0, st>>>(rank, flag, n, status);
  SPC_LAUNCH_OK();
  int host[2] = {0, 0};  // status, voxels found
  SPC_CUDA_OK(cudaMemcpyAsync(host, status, sizeof(host), cudaMemcpyDeviceToHost, st));
  SPC_CUDA_OK(cudaStreamSynchronize(st));
  if (host[0] != 0) return fail(host[0], "voxelize: hash table full (status %d)", host[0]);
  const int64_t total_voxels = host[1];
  const int64_t num_voxels = std::min<int64_t>(total_voxels, max_voxels);
  *num_voxels_host = num_voxels;
  if (num_voxels == 0) {
    SPC_CUDA_OK(cudaMemsetAsync(pc_voxel_id, 0xFF, static_cast<size_t>(n) * sizeof(int64_t), st));
    return SPC_OK;
  }
  SPC_CUDA_OK(cudaMemsetAsync(counts, 0, static_cast<size_t>(num_voxels) * 4, st));
  assign_kernel<<<vox_blocks(n), kVoxThreads, 0, st>>>(g, keys, first, rank, n, num_voxels, counts, sk_a, sv_a,
                                                    reinterpret_cast<long long*>(pc_voxel_id), indices);
  SPC_LAUNCH_OK();
  clamp_counts_kernel<<<vox_blocks(num_voxels), kVoxThreads, 0, st>>>(counts, num_voxels, max_points, num_per_voxel);
  SPC_LAUNCH_OK();
  cub_bytes = L.cub_bytes;
  SPC_CUDA_OK(cub::DeviceScan::ExclusiveSum(ws + L.off_cub, cub_bytes, counts, seg, static_cast<int>(num_voxels), st));
  // stable: arrival order survives inside a voxel; dropped points carry the key num_voxels and
  // sort behind all others; only the bits that key needs are sorted
  int bits = 1;
  while (bits < 32 && (1ll << bits) <= num_voxels) ++bits;
  cub_bytes = L.cub_bytes;
  SPC_CUDA_OK(cub::DeviceRadixSort::SortPairs(ws + L.off_cub, cub_bytes, sk_a, sk_b, sv_a, sv_b, n, 0, bits, st));
  const long long work = static_cast<long long>(n) * num_features;
  scatter_points_kernel<<<vox_blocks(work), kVoxThreads, 0, st>>>(points, point_stride, num_features, sk_b, sv_b, seg,
                                                                 n, num_voxels, max_points, voxels);
  SPC_LAUNCH_OK();
  if (empty_mean) {
    fill_mean_kernel<<<vox_blocks(num_voxels * num_features), kVoxThreads, 0, st>>>(voxels, num_per_voxel, num_voxels,
                                                                                    max_points, num_features);
    SPC_LAUNCH_OK();
  }
  return SPC_OK;
}
