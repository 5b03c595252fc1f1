// Rulebook (indice-pair) generation for sparse convolution on B200.
//
// Design (differs from the reference on purpose): the reference materialises
// the kv*N candidate grid (out_lin, valid, out_row) in HBM, sorts the input
// coordinates, runs kv*N binary searches and scatters into -1 pre-filled
// tables (spconv_triton/pytorch/_impl/pairs.py:126-426).  Here two open-addressing hash
// tables keyed by the batch-major linear coordinate replace the sorts and
// searches, and every table is produced by a GATHER pass with one thread per
// table column: thread r owns column r of pair_fwd, looks each of the kv
// neighbour coordinates up (the tables are a few MB and stay in the 126 MB
// L2), writes pair_fwd[k*n+r] fully coalesced and keeps the row's offset
// bitmask in a register.  No candidate grid, no pre-fill, no atomics on the
// tables, and the only ordered step is a radix sort of the n_out unique
// output coordinates, which reproduces the ascending row numbering that
// torch.unique gives the reference.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include <algorithm>
#include <climits>
#include <type_traits>

#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "gemm_internal.cuh"
#include "rulebook_internal.cuh"

namespace spc {
namespace {

constexpr int kThreads = 256;

struct Geo {
  int ndim, batch, subm, transpose, kv;
  int in_shape[SPC_MAX_NDIM], out_shape[SPC_MAX_NDIM];
  int ksize[SPC_MAX_NDIM], stride[SPC_MAX_NDIM], pad[SPC_MAX_NDIM], dil[SPC_MAX_NDIM];
  // Tile key (kv <= 32 only, off unless a caller of rulebook_igemm_chained asks for it): the mask
  // sort then orders the rows by a transformed mask word instead of the word itself, see below.
  int tile_key;
  unsigned char key_pos[32];  // bit k of the mask word goes to bit key_pos[k] of the key
};

// The order the gather-GEMM wants is not the numeric order of the mask words but one in which the
// 128 rows of a tile share as many kernel offsets as possible.  Two cheap changes to the sort key
// get most of what a data-dependent order would: the offsets far from the kernel's centre (the
// corners of the window, the rarest in surface-like data) become the most significant bits, so that
// rows are grouped by their rare offsets first, and the key is Gray-decoded, so that neighbouring
// keys (hence neighbouring tiles) differ in few offsets.  On the VoxelNet-style backbone: 6 - 9 % fewer
// (tile, offset) stages on the submanifold levels, 2 - 16 % on the strided ones.
__device__ __forceinline__ uint32_t gray_decode(uint32_t key) {
  key ^= key >> 1;
  key ^= key >> 2;
  key ^= key >> 4;
  key ^= key >> 8;
  key ^= key >> 16;
  return key;
}

// ------------------------------------------------------------------------
// Hash tables.  K64 = false: key < 2^31, slot = (key << 32) | value in one
// 64-bit word, so a probe is one 8-byte access and an insert one atomicCAS.
// K64 = true: 64-bit keys with a separate value array.
// Probing is linear and bounded by the capacity; a full table raises a status
// flag instead of spinning.
// ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t mix32(uint32_t h) {
  h ^= h >> 16;
  h *= 0x85ebca6bu;
  h ^= h >> 13;
  h *= 0xc2b2ae35u;
  h ^= h >> 16;
  return h;
}

template <bool K64>
struct Table;

template <>
struct Table<false> {
  using key_t = uint32_t;
  unsigned long long* slots;
  uint32_t cap_mask;
  // Dense numbering (output side of strided layers on a grid small enough for a bitmap): one bit per
  // cell and, per 32-bit word, the number of set bits before it.  The value of a key is then its
  // rank among the set bits = its row in ascending key order, with no hash table and no sort.
  uint32_t* obits = nullptr;
  const uint32_t* oprefix = nullptr;
  // Input side: rows equal ranks only when the rows came in ascending key order (the outputs of an
  // earlier layer do); `unsorted` points at a device flag that says they did not.
  const int* unsorted = nullptr;
  __device__ __forceinline__ bool ranked() const {
    return obits != nullptr && (unsorted == nullptr || *unsorted == 0);
  }
  __device__ __forceinline__ int rank_of(key_t key) const {
    const uint32_t w = __ldg(&obits[key >> 5]);
    if (!((w >> (key & 31u)) & 1u)) return -1;
    return static_cast<int>(__ldg(&oprefix[key >> 5]) + __popc(w & ((1u << (key & 31u)) - 1u)));
  }
  static constexpr unsigned long long kEmpty = ~0ull;

  // Four consecutive keys (neighbours along the fastest coordinate) share one
  // 32-byte sector: the block is chosen by hashing key >> 2, the lane inside it
  // by key & 3, and probing moves a whole block at a time.  The three x
  // neighbours of a voxel then cost one or two sectors instead of three.
  static constexpr uint32_t kStep = 4;
  __device__ __forceinline__ uint32_t home(key_t k) const { return ((mix32(k >> 2) << 2) | (k & 3u)) & cap_mask; }

  // Keeps the smallest value among equal keys (duplicate coordinates resolve
  // to the lowest row, as a stable sort + lower bound does in the reference).
  __device__ bool insert_min(key_t key, uint32_t val) const {
    const unsigned long long packed = (static_cast<unsigned long long>(key) << 32) | val;
    uint32_t s = home(key);
    for (uint32_t probe = 0; probe <= (cap_mask >> 2); ++probe) {
      unsigned long long old = atomicCAS(&slots[s], kEmpty, packed);
      if (old == kEmpty) return true;
      if (static_cast<key_t>(old >> 32) == key) {
        atomicMin(&slots[s], packed);
        return true;
      }
      s = (s + kStep) & cap_mask;
    }
    return false;
  }
  // 1: this call inserted the key, 0: already present, -1: table full.
  __device__ int insert_unique(key_t key) const {
    const unsigned long long packed = (static_cast<unsigned long long>(key) << 32) | 0x7fffffffu;
    uint32_t s = home(key);
    for (uint32_t probe = 0; probe <= (cap_mask >> 2); ++probe) {
      unsigned long long old = atomicCAS(&slots[s], kEmpty, packed);
      if (old == kEmpty) return 1;
      if (static_cast<key_t>(old >> 32) == key) return 0;
      s = (s + kStep) & cap_mask;
    }
    return -1;
  }
  __device__ int find(key_t key) const {
    if (ranked()) return rank_of(key);
    uint32_t s = home(key);
    for (uint32_t probe = 0; probe <= (cap_mask >> 2); ++probe) {
      const unsigned long long v = __ldg(&slots[s]);
      if (v == kEmpty) return -1;
      if (static_cast<key_t>(v >> 32) == key) return static_cast<int>(v & 0xffffffffu);
      s = (s + kStep) & cap_mask;
    }
    return -1;
  }
  // A look-up split in two so that several keys' first probes can be in flight at once:
  // first_probe() returns the home slot's word, finish() resolves it (almost always at once).
  __device__ __forceinline__ unsigned long long first_probe(key_t key) const { return __ldg(&slots[home(key)]); }
  __device__ __forceinline__ int finish(key_t key, unsigned long long v) const {
    if (v == kEmpty) return -1;
    if (static_cast<key_t>(v >> 32) == key) return static_cast<int>(v & 0xffffffffu);
    uint32_t s = (home(key) + kStep) & cap_mask;
    for (uint32_t probe = 1; probe <= (cap_mask >> 2); ++probe) {
      const unsigned long long w = __ldg(&slots[s]);
      if (w == kEmpty) return -1;
      if (static_cast<key_t>(w >> 32) == key) return static_cast<int>(w & 0xffffffffu);
      s = (s + kStep) & cap_mask;
    }
    return -1;
  }
  __device__ void set_value(key_t key, uint32_t val) const {
    uint32_t s = home(key);
    for (uint32_t probe = 0; probe <= (cap_mask >> 2); ++probe) {
      const unsigned long long v = slots[s];
      if (v == kEmpty) return;
      if (static_cast<key_t>(v >> 32) == key) {
        slots[s] = (static_cast<unsigned long long>(key) << 32) | val;
        return;
      }
      s = (s + kStep) & cap_mask;
    }
  }
};

template <>
struct Table<true> {
  using key_t = unsigned long long;
  unsigned long long* slots;  // keys
  int* vals;
  uint32_t cap_mask;
  static constexpr unsigned long long kEmpty = ~0ull;

  static constexpr uint32_t kStep = 4;
  __device__ __forceinline__ uint32_t home(key_t k) const {
    const key_t b = k >> 2;
    return ((mix32(static_cast<uint32_t>(b) ^ mix32(static_cast<uint32_t>(b >> 32))) << 2) |
            (static_cast<uint32_t>(k) & 3u)) & cap_mask;
  }
  __device__ bool insert_min(key_t key, uint32_t val) const {
    uint32_t s = home(key);
    for (uint32_t probe = 0; probe <= (cap_mask >> 2); ++probe) {
      unsigned long long old = atomicCAS(&slots[s], kEmpty, key);
      if (old == kEmpty || old == key) {
        atomicMin(&vals[s], static_cast<int>(val));
        return true;
      }
      s = (s + kStep) & cap_mask;
    }
    return false;
  }
  __device__ int insert_unique(key_t key) const {
    uint32_t s = home(key);
    for (uint32_t probe = 0; probe <= (cap_mask >> 2); ++probe) {
      unsigned long long old = atomicCAS(&slots[s], kEmpty, key);
      if (old == kEmpty) return 1;
      if (old == key) return 0;
      s = (s + kStep) & cap_mask;
    }
    return -1;
  }
  __device__ int find(key_t key) const {
    uint32_t s = home(key);
    for (uint32_t probe = 0; probe <= (cap_mask >> 2); ++probe) {
      const unsigned long long v = __ldg(&slots[s]);
      if (v == kEmpty) return -1;
      if (v == key) return __ldg(&vals[s]);
      s = (s + kStep) & cap_mask;
    }
    return -1;
  }
  __device__ __forceinline__ unsigned long long first_probe(key_t) const { return 0; }
  __device__ __forceinline__ int finish(key_t key, unsigned long long) const { return find(key); }
  __device__ void set_value(key_t key, uint32_t val) const {
    uint32_t s = home(key);
    for (uint32_t probe = 0; probe <= (cap_mask >> 2); ++probe) {
      const unsigned long long v = slots[s];
      if (v == kEmpty) return;
      if (v == key) {
        vals[s] = static_cast<int>(val);
        return;
      }
      s = (s + kStep) & cap_mask;
    }
  }
};

// ------------------------------------------------------------------------
// Coordinate arithmetic (follows spconv_triton/pytorch/_impl/pair_kernels.py:66-91).
// Kernel offsets are enumerated row-major, last dimension fastest, never
// flipped (spconv_triton/pytorch/_impl/pairs.py:43-48).
// ------------------------------------------------------------------------
template <int ND>
struct Odometer {
  int pos[ND];
  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int d = 0; d < ND; ++d) pos[d] = 0;
  }
  __device__ __forceinline__ void set(const Geo& g, int k) {
#pragma unroll
    for (int d = ND - 1; d >= 0; --d) {
      pos[d] = k % g.ksize[d];
      k /= g.ksize[d];
    }
  }
  __device__ __forceinline__ void next(const Geo& g) {
#pragma unroll
    for (int d = ND - 1; d >= 0; --d) {
      if (++pos[d] < g.ksize[d]) return;
      pos[d] = 0;
    }
  }
};

// Output linear coordinate reached from input coordinate `c` through kernel
// offset `kp`, or -1 if that offset does not produce an output.
template <int ND>
__device__ __forceinline__ long long out_key_from_input(const Geo& g, const int* c, const int* kp) {
  long long lin = c[0];
#pragma unroll
  for (int d = 0; d < ND; ++d) {
    int o;
    if (g.transpose) {
      o = c[d + 1] * g.stride[d] + kp[d] * g.dil[d] - g.pad[d];
    } else {
      const int num = c[d + 1] + g.pad[d] - kp[d] * g.dil[d];
      if (num < 0) return -1;
      o = num / g.stride[d];
      if (o * g.stride[d] != num) return -1;
    }
    if (o < 0 || o >= g.out_shape[d]) return -1;
    lin = lin * g.out_shape[d] + o;
  }
  return lin;
}

// Input linear coordinate that feeds output coordinate `o` through kernel
// offset `kp` (the inverse map of out_key_from_input), or -1.
template <int ND>
__device__ __forceinline__ long long in_key_from_output(const Geo& g, const int* o, const int* kp) {
  long long lin = o[0];
#pragma unroll
  for (int d = 0; d < ND; ++d) {
    int x;
    if (g.transpose) {
      const int num = o[d + 1] + g.pad[d] - kp[d] * g.dil[d];
      if (num < 0) return -1;
      x = num / g.stride[d];
      if (x * g.stride[d] != num) return -1;
    } else {
      x = o[d + 1] * g.stride[d] - g.pad[d] + kp[d] * g.dil[d];
    }
    if (x < 0 || x >= g.in_shape[d]) return -1;
    lin = lin * g.in_shape[d] + x;
  }
  return lin;
}

template <int ND>
__device__ __forceinline__ void load_coord(const int32_t* __restrict__ idx, long long row, int* c) {
#pragma unroll
  for (int d = 0; d <= ND; ++d) c[d] = __ldg(&idx[row * (ND + 1) + d]);
}

// A row whose batch index or coordinates lie outside [0, batch) x [0, in_shape) must not be
// turned into a bitmap or table index.  Kernels skip such rows (they get no pairs); the phase-1
// kernels also record SPC_ERR_INVALID_ARGUMENT so that the host raises.
template <int ND>
__device__ __forceinline__ bool coord_in_grid(const Geo& g, const int* c) {
  bool ok = c[0] >= 0 && c[0] < g.batch;
#pragma unroll
  for (int d = 0; d < ND; ++d) ok = ok && c[d + 1] >= 0 && c[d + 1] < g.in_shape[d];
  return ok;
}
__device__ __forceinline__ void flag_bad_row(int* counters, int* dev_status) {
  atomicExch(&counters[1], SPC_ERR_INVALID_ARGUMENT);  // counters[kStatus]
  if (dev_status != nullptr) atomicExch(dev_status, SPC_ERR_INVALID_ARGUMENT);
}

template <int ND>
__device__ __forceinline__ long long in_key_of(const Geo& g, const int* c) {
  long long lin = c[0];
#pragma unroll
  for (int d = 0; d < ND; ++d) lin = lin * g.in_shape[d] + c[d + 1];
  return lin;
}

template <int ND>
__device__ __forceinline__ void delinearize_out(const Geo& g, long long lin, int* c) {
#pragma unroll
  for (int d = ND - 1; d >= 0; --d) {
    c[d + 1] = static_cast<int>(lin % g.out_shape[d]);
    lin /= g.out_shape[d];
  }
  c[0] = static_cast<int>(lin);
}

enum Counter { kUniqueCount = 0, kStatus = 1, kUnsorted = 2 };

// ------------------------------------------------------------------------
// Phase 1 kernels
// ------------------------------------------------------------------------
template <int ND, bool K64>
__global__ void __launch_bounds__(kThreads)
insert_inputs_kernel(const __grid_constant__ Geo g, const int32_t* __restrict__ idx, long long n,
                     Table<K64> tin, int* counters, uint32_t* __restrict__ bitmap, int* dev_status) {
  const long long j = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  if (j >= n) return;
  if (bitmap != nullptr && counters[kUnsorted] == 0) return;  // rows are ranks of the bitmap
  int c[ND + 1];
  load_coord<ND>(idx, j, c);
  if (!coord_in_grid<ND>(g, c)) {
    flag_bad_row(counters, dev_status);
    return;
  }
  using key_t = typename Table<K64>::key_t;
  const long long key = in_key_of<ND>(g, c);
  if (!tin.insert_min(static_cast<key_t>(key), static_cast<uint32_t>(j)))
    atomicExch(&counters[kStatus], SPC_ERR_HASH_TABLE_FULL);
}

// With a bitmap of the input grid: sets the bit of every input cell and notes whether the rows are in
// strictly ascending key order.  If they are, a row number is the rank of its bit and the hash table
// is not needed (insert_inputs_kernel then returns at once).
template <int ND>
__global__ void __launch_bounds__(kThreads)
mark_inputs_kernel(const __grid_constant__ Geo g, const int32_t* __restrict__ idx, long long n,
                   uint32_t* __restrict__ bitmap, int* counters, int* dev_status) {
  const long long j = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  if (j >= n) return;
  int c[ND + 1];
  load_coord<ND>(idx, j, c);
  if (!coord_in_grid<ND>(g, c)) {
    flag_bad_row(counters, dev_status);
    counters[kUnsorted] = 1;  // a skipped row breaks "row number = rank of its bit"
    return;
  }
  const long long key = in_key_of<ND>(g, c);
  atomicOr(&bitmap[key >> 5], 1u << (key & 31));
  if (j > 0) {
    load_coord<ND>(idx, j - 1, c);
    if (in_key_of<ND>(g, c) >= key) counters[kUnsorted] = 1;
  }
}

// One thread per input row walks the kv offsets and inserts each candidate
// output coordinate into the output table.  Offsets are handled in groups of
// 32: a thread remembers in a bitmask which of its candidates were first-time
// inserts, the warp reserves room for all of them in `uniq` with ONE atomicAdd
// per group (a per-insert counter serialises on a single address), and a
// second walk over the group writes the keys.
__device__ __forceinline__ uint32_t* dense_bits(const Table<false>& t) { return t.obits; }
__device__ __forceinline__ uint32_t* dense_bits(const Table<true>&) { return nullptr; }

__device__ __forceinline__ bool table_ranked(const Table<false>& t) { return t.ranked(); }
__device__ __forceinline__ bool table_ranked(const Table<true>&) { return false; }
__device__ __forceinline__ uint32_t rank_prefix(const Table<false>& t, long long key) { return __ldg(&t.oprefix[key >> 5]); }
__device__ __forceinline__ uint32_t rank_prefix(const Table<true>&, long long) { return 0; }

// Dense numbering, step 2: set bits per word (scanned in place afterwards).
__global__ void __launch_bounds__(kThreads)
count_bits_kernel(const uint32_t* __restrict__ bits, long long words, uint32_t* __restrict__ counts) {
  const long long i = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  if (i < words) counts[i] = __popc(bits[i]);
}

// Dense numbering, step 3: the keys of the set bits in ascending order, and their total.
__global__ void __launch_bounds__(kThreads)
expand_bits_kernel(const uint32_t* __restrict__ bits, const uint32_t* __restrict__ prefix, long long words,
                   long long limit, uint32_t* __restrict__ sorted, int* counters) {
  const long long i = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  if (i >= words) return;
  uint32_t w = bits[i];
  long long at = prefix[i];
  if (i == words - 1) counters[kUniqueCount] = static_cast<int>(at + __popc(w));
  while (w != 0 && at < limit) {
    const int b = __ffs(w) - 1;
    sorted[at++] = static_cast<uint32_t>(i * 32 + b);
    w &= w - 1;
  }
}

// Dense numbering, step 1: the bits of every output cell an input row reaches.  Per axis only the
// kernel offsets that land on an output coordinate are kept (a bitmask over the offsets of that axis:
// with stride 2 and a 3-wide kernel one or two of three), and the cells are the product of the axes,
// so a k3 s2 layer visits at most 8 candidates per input instead of testing all 27.
template <int D, int ND>
__device__ __forceinline__ void mark_cells(const Geo& g, const int* c, const uint32_t* mask, long long lin,
                                           uint32_t* __restrict__ bits) {
  if constexpr (D == ND) {
    uint32_t* word = bits + (lin >> 5);
    const uint32_t bit = 1u << (lin & 31);
    if (!(*word & bit)) atomicOr(word, bit);
  } else {
    for (uint32_t m = mask[D]; m != 0; m &= m - 1) {
      const int k = __ffs(m) - 1;
      const int o = g.transpose ? c[D + 1] * g.stride[D] + k * g.dil[D] - g.pad[D]
                                : (c[D + 1] + g.pad[D] - k * g.dil[D]) / g.stride[D];
      mark_cells<D + 1, ND>(g, c, mask, lin * g.out_shape[D] + o, bits);
    }
  }
}

template <int ND>
__global__ void __launch_bounds__(kThreads)
mark_outputs_kernel(const __grid_constant__ Geo g, const int32_t* __restrict__ idx, long long n,
                    uint32_t* __restrict__ bits) {
  const long long j = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  if (j >= n) return;
  int c[ND + 1];
  load_coord<ND>(idx, j, c);
  if (!coord_in_grid<ND>(g, c)) return;  // recorded by the input pass
  uint32_t mask[ND];
#pragma unroll
  for (int d = 0; d < ND; ++d) {
    uint32_t m = 0;
    for (int k = 0; k < g.ksize[d]; ++k) {
      int o;
      if (g.transpose) {
        o = c[d + 1] * g.stride[d] + k * g.dil[d] - g.pad[d];
      } else {
        const int num = c[d + 1] + g.pad[d] - k * g.dil[d];
        if (num < 0) continue;
        o = num / g.stride[d];
        if (o * g.stride[d] != num) continue;
      }
      if (o >= 0 && o < g.out_shape[d]) m |= 1u << k;
    }
    if (m == 0) return;
    mask[d] = m;
  }
  mark_cells<0, ND>(g, c, mask, c[0], bits);
}

template <int ND, bool K64>
__global__ void __launch_bounds__(kThreads)
enumerate_outputs_kernel(const __grid_constant__ Geo g, const int32_t* __restrict__ idx, long long n,
                         Table<K64> tout, typename Table<K64>::key_t* __restrict__ uniq,
                         int* counters) {
  using key_t = typename Table<K64>::key_t;
  const long long j = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  bool live = j < n;
  int c[ND + 1];
  if (live) {
    load_coord<ND>(idx, j, c);
    live = coord_in_grid<ND>(g, c);  // a row outside the grid (recorded by the input pass) reaches no output
  }
  const unsigned lane = threadIdx.x & 31u;
  for (int k0 = 0; k0 < g.kv; k0 += 32) {
    const int gcount = min(32, g.kv - k0);
    Odometer<ND> od;
    od.set(g, k0);
    uint32_t fresh = 0;
    if (live) {
      for (int kk = 0; kk < gcount; ++kk) {
        const long long key = out_key_from_input<ND>(g, c, od.pos);
        if (key >= 0) {
          if (dense_bits(tout) != nullptr) {
            uint32_t* word = dense_bits(tout) + (key >> 5);
            const uint32_t bit = 1u << (key & 31);
            if (!(*word & bit)) atomicOr(word, bit);
          } else {
            const int r = tout.insert_unique(static_cast<key_t>(key));
            if (r < 0) atomicExch(&counters[kStatus], SPC_ERR_HASH_TABLE_FULL);
            fresh |= static_cast<uint32_t>(r > 0) << kk;
          }
        }
        od.next(g);
      }
    }
    // warp-inclusive prefix of the per-thread counts
    const int mine = __popc(fresh);
    int incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= static_cast<unsigned>(off)) incl += t;
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    if (total == 0) continue;
    int base = 0;
    if (lane == 31) base = atomicAdd(&counters[kUniqueCount], total);
    base = __shfl_sync(0xffffffffu, base, 31) + incl - mine;
    if (fresh) {
      od.set(g, k0);
      for (int kk = 0; kk < gcount; ++kk) {
        if ((fresh >> kk) & 1u) uniq[base++] = static_cast<key_t>(out_key_from_input<ND>(g, c, od.pos));
        od.next(g);
      }
    }
  }
}

// counters[kUniqueCount], counters[kStatus] and the device status word -> page-locked host memory.
__global__ void publish_counters_kernel(const int* __restrict__ counters, const int* __restrict__ dev_status,
                                        int* __restrict__ host_box) {
  if (threadIdx.x == 0) {
    host_box[0] = counters[0];
    host_box[1] = counters[1];
    host_box[2] = dev_status != nullptr ? *dev_status : 0;
    __threadfence_system();
  }
}

template <bool K64>
__global__ void __launch_bounds__(kThreads)
assign_ranks_kernel(Table<K64> tout, const typename Table<K64>::key_t* __restrict__ sorted,
                    long long n_out) {
  const long long r = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  if (r < n_out) tout.set_value(sorted[r], static_cast<uint32_t>(r));
}

// ------------------------------------------------------------------------
// Phase 2 kernels (implicit-gemm tables)
// ------------------------------------------------------------------------
// Column r of pair_fwd: for each offset the input row that feeds output row r.
// SUBM_BWD additionally writes pair_bwd, which for a submanifold layer is
// pair_fwd with the offset axis reversed (offset k seen from the input side is
// offset kv-1-k seen from the output side).
template <int ND, bool K64, bool SUBM_BWD>
__global__ void __launch_bounds__(kThreads)
fill_fwd_kernel(const __grid_constant__ Geo g, const int32_t* __restrict__ idx,
                const typename Table<K64>::key_t* __restrict__ sorted_out, long long n_out,
                Table<K64> tin, int32_t* __restrict__ out_indices, int32_t* __restrict__ pair_fwd,
                int32_t* __restrict__ pair_bwd, uint32_t* __restrict__ words, int mic,
                int32_t* __restrict__ fwd_rm, int32_t* __restrict__ bwd_rm, int kvp,
                const uint32_t* __restrict__ bitmap, int32_t* __restrict__ iota, int staged) {
  using key_t = typename Table<K64>::key_t;
  const long long r = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  // Row-major copies: a thread owns one row of kvp entries, so direct stores are 16 (or 4) bytes at
  // a stride of kvp * 4 bytes -- a warp-wide store then touches 32 sectors and writes half (an
  // eighth) of each.  With `staged` the warp collects its 32 rows in shared memory and writes the
  // 32 * kvp * 4 contiguous bytes with full 16-byte-per-lane stores.
  extern __shared__ int32_t stage_s[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t* tile_f = stage_s + static_cast<size_t>(warp) * (SUBM_BWD ? 2 : 1) * 32 * kvp;
  int32_t* tile_b = tile_f + 32 * kvp;
  const bool live = r < n_out;
  if (live) {
  if (iota != nullptr) iota[r] = static_cast<int32_t>(r);  // the values the mask sort permutes
  int o[ND + 1];
  int quad[4] = {-1, -1, -1, -1};  // four consecutive offsets of the row-major copy
  bool row_ok = true;
  if (g.subm) {
    load_coord<ND>(idx, r, o);
    row_ok = coord_in_grid<ND>(g, o);  // a row outside the grid gets no pairs
  } else {
    delinearize_out<ND>(g, static_cast<long long>(sorted_out[r]), o);
#pragma unroll
    for (int d = 0; d <= ND; ++d) out_indices[r * (ND + 1) + d] = o[d];
  }
  Odometer<ND> od;
  od.reset();
  uint32_t word = 0;
  // Non-transposed layers: the input cell of offset (p_0, .., p_last) is base + sum p_d * step_d, and
  // whether it lies inside the grid is one bit per dimension; both are set up once per row so that
  // the loop over the kv offsets does no coordinate arithmetic.
  bool fast = !g.transpose;
  long long base = o[0];
  long long step[ND];
  uint32_t inside[ND];
  if (fast) {
    long long mult = 1;
#pragma unroll
    for (int d = ND - 1; d >= 0; --d) {
      step[d] = mult * g.dil[d];
      mult *= g.in_shape[d];
      if (g.ksize[d] > 32) fast = false;
    }
  }
  if (fast) {
#pragma unroll
    for (int d = 0; d < ND; ++d) {
      const int x0 = o[d + 1] * g.stride[d] - g.pad[d];
      base = base * g.in_shape[d] + x0;
      uint32_t m = 0;
      for (int q = 0; q < g.ksize[d]; ++q) {
        const int x = x0 + q * g.dil[d];
        m |= static_cast<uint32_t>(x >= 0 && x < g.in_shape[d]) << q;
      }
      inside[d] = m;
    }
  }
  // rows in ascending key order: a neighbour's row is the rank of its bit (one load of the word's prefix)
  const bool ranked = bitmap != nullptr && table_ranked(tin);
  // what is written for offset k once its input row j (-1: none) is known
  auto emit = [&](int k, int j) {
    if (pair_fwd != nullptr) pair_fwd[static_cast<long long>(k) * n_out + r] = j;
    if (SUBM_BWD) {
      pair_bwd[static_cast<long long>(g.kv - 1 - k) * n_out + r] = j;
      if (bwd_rm != nullptr) {
        if (staged) tile_b[lane * kvp + (g.kv - 1 - k)] = j;
        else bwd_rm[r * kvp + (g.kv - 1 - k)] = j;
      }
    }
    if (fwd_rm != nullptr) {
      if (staged) {
        tile_f[lane * kvp + k] = j;
      } else {
        quad[k & 3] = j;
        if ((k & 3) == 3 || k == g.kv - 1) {
          *reinterpret_cast<int4*>(&fwd_rm[r * kvp + (k & ~3)]) = make_int4(quad[0], quad[1], quad[2], quad[3]);
          quad[0] = quad[1] = quad[2] = quad[3] = -1;
        }
      }
    }
    // with the tile key the bit goes straight to its place in the key (single word)
    word |= static_cast<uint32_t>(j >= 0) << (g.tile_key ? g.key_pos[k] : (k & 31));
    if ((k & 31) == 31 || k == g.kv - 1) {
      words[r * mic + (k >> 5)] = g.tile_key ? gray_decode(word) : word;
      word = 0;
    }
  };
  const int kl = g.ksize[ND - 1];
  if (fast && row_ok && bitmap != nullptr && g.dil[ND - 1] == 1) {
    // Window path.  The kl offsets along the last axis are kl consecutive cells, i.e. consecutive
    // bits of the occupancy bitmap: one (at a word boundary two) loads test all of them, and in
    // ranked mode one prefix load numbers all of them, since the prefix of the next word is this
    // word's prefix plus its population count.  A scattered load costs an L1 wavefront per lane, so
    // 2-3 loads per axis line instead of one or two per offset is what this kernel's time follows.
    const uint32_t in_mask = inside[ND - 1] & (kl >= 32 ? 0xffffffffu : ((1u << kl) - 1u));
    for (int k0 = 0; k0 < g.kv; k0 += kl) {
      uint32_t ok = in_mask != 0;
      long long kk = base;
#pragma unroll
      for (int d = 0; d < ND - 1; ++d) {
        ok &= inside[d] >> od.pos[d];
        kk += od.pos[d] * step[d];
      }
      uint32_t present = 0, w0 = 0, w1 = 0, pfx0 = 0;
      int qlo = 0, sh = 0;
      long long kb = 0;
      if (ok & 1u) {
        qlo = __ffs(in_mask) - 1;                 // first offset of the line that lies inside the grid
        const int qhi = 31 - __clz(in_mask);      // and the last one
        kb = kk + qlo;                            // its cell: a valid key
        const long long wi = kb >> 5;
        sh = static_cast<int>(kb & 31);
        w0 = __ldg(&bitmap[wi]);
        if (sh + (qhi - qlo) >= 32) w1 = __ldg(&bitmap[wi + 1]);  // the word of a valid cell as well
        const unsigned long long win = ((static_cast<unsigned long long>(w1) << 32) | w0) >> sh;
        present = (static_cast<uint32_t>(win) << qlo) & in_mask;
        if (present != 0 && ranked) pfx0 = rank_prefix(tin, kb);
      }
      for (int q = 0; q < kl; ++q) {
        int j = -1;
        if ((present >> q) & 1u) {
          if (ranked) {
            const int bit = sh + (q - qlo);
            j = bit < 32 ? static_cast<int>(pfx0) + __popc(w0 & ((1u << bit) - 1u))
                         : static_cast<int>(pfx0) + __popc(w0) + __popc(w1 & ((1u << (bit - 32)) - 1u));
          } else {
            j = tin.find(static_cast<key_t>(kb + (q - qlo)));
          }
        }
        emit(k0 + q, j);
        od.next(g);
      }
    }
  } else {
  // Offsets are handled three at a time (the three neighbours along the last axis of a 3^3
  // kernel): their bitmap words, then their first hash probes, are requested together, so a row
  // has up to three L2 accesses in flight instead of one after the other.
  constexpr int kBatch = 3;
  for (int k0 = 0; k0 < g.kv; k0 += kBatch) {
    long long key[kBatch];
    uint32_t bits[kBatch];
    unsigned long long probe[kBatch];
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      key[b] = -1;
      if (k0 + b < g.kv) {
        if (!row_ok) {
        } else if (fast) {
          uint32_t ok = 1u;
          long long kk = base;
#pragma unroll
          for (int d = 0; d < ND; ++d) {
            ok &= inside[d] >> od.pos[d];
            kk += od.pos[d] * step[d];
          }
          if (ok & 1u) key[b] = kk;
        } else {
          key[b] = in_key_from_output<ND>(g, o, od.pos);
        }
        od.next(g);
      }
    }
#pragma unroll
    for (int b = 0; b < kBatch; ++b)
      bits[b] = (key[b] >= 0 && bitmap != nullptr) ? __ldg(&bitmap[key[b] >> 5]) : 0xffffffffu;
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      if (key[b] >= 0 && !((bits[b] >> (key[b] & 31)) & 1u)) key[b] = -1;
      probe[b] = key[b] < 0 ? 0ull
                 : ranked  ? static_cast<unsigned long long>(rank_prefix(tin, key[b]))
                           : tin.first_probe(static_cast<key_t>(key[b]));
    }
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const int k = k0 + b;
      if (k >= g.kv) break;
      const int j = key[b] < 0 ? -1
                    : ranked  ? static_cast<int>(probe[b]) + __popc(bits[b] & ((1u << (key[b] & 31)) - 1u))
                              : tin.finish(static_cast<key_t>(key[b]), probe[b]);
      emit(k, j);
    }
  }
  }
  if (staged) {
    for (int k = g.kv; k < kvp; ++k) {
      if (fwd_rm != nullptr) tile_f[lane * kvp + k] = -1;
      if (SUBM_BWD && bwd_rm != nullptr) tile_b[lane * kvp + k] = -1;
    }
  } else if (SUBM_BWD && bwd_rm != nullptr) {
    for (int k = g.kv; k < kvp; ++k) bwd_rm[r * kvp + k] = -1;
  }
  }  // live
  if (staged) {
    __syncwarp();
    const long long row0 = r - lane;  // first row of this warp
    const long long left = n_out - row0;
    if (left > 0) {
      const int n4 = static_cast<int>(left < 32 ? left : 32) * kvp / 4;  // kvp is a multiple of 4
      if (fwd_rm != nullptr) {
        int4* dst = reinterpret_cast<int4*>(fwd_rm + row0 * kvp);
        const int4* src = reinterpret_cast<const int4*>(tile_f);
        for (int i = lane; i < n4; i += 32) dst[i] = src[i];
      }
      if (SUBM_BWD && bwd_rm != nullptr) {
        int4* dst = reinterpret_cast<int4*>(bwd_rm + row0 * kvp);
        const int4* src = reinterpret_cast<const int4*>(tile_b);
        for (int i = lane; i < n4; i += 32) dst[i] = src[i];
      }
    }
  }
}

// Column j of pair_bwd (strided / transposed layers): for each offset the
// output row that input row j contributes to.
template <int ND, bool K64>
__global__ void __launch_bounds__(kThreads)
fill_bwd_kernel(const __grid_constant__ Geo g, const int32_t* __restrict__ idx, long long n_in,
                long long n_out, Table<K64> tout, int32_t* __restrict__ pair_bwd,
                uint32_t* __restrict__ words, int mic, int32_t* __restrict__ bwd_rm, int kvp,
                int32_t* __restrict__ iota) {
  using key_t = typename Table<K64>::key_t;
  const long long j = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  if (j >= n_in) return;
  if (iota != nullptr) iota[j] = static_cast<int32_t>(j);
  int quad[4] = {-1, -1, -1, -1};
  int c[ND + 1];
  load_coord<ND>(idx, j, c);
  const bool row_ok = coord_in_grid<ND>(g, c);  // a row outside the grid contributes to no output
  Odometer<ND> od;
  od.reset();
  uint32_t word = 0;
  for (int k = 0; k < g.kv; ++k) {
    const long long key = row_ok ? out_key_from_input<ND>(g, c, od.pos) : -1;
    int r = key >= 0 ? tout.find(static_cast<key_t>(key)) : -1;
    if (r >= n_out) r = -1;  // rows cut off by num_out_act_bound
    pair_bwd[static_cast<long long>(k) * n_in + j] = r;
    if (bwd_rm != nullptr) {
      quad[k & 3] = r;
      if ((k & 3) == 3 || k == g.kv - 1) {
        *reinterpret_cast<int4*>(&bwd_rm[j * kvp + (k & ~3)]) = make_int4(quad[0], quad[1], quad[2], quad[3]);
        quad[0] = quad[1] = quad[2] = quad[3] = -1;
      }
    }
    if (words != nullptr) {
      word |= static_cast<uint32_t>(r >= 0) << (k & 31);
      if ((k & 31) == 31 || k == g.kv - 1) {
        words[j * mic + (k >> 5)] = word;
        word = 0;
      }
    }
    od.next(g);
  }
}

// keys[i] = words[rows[i], w] & and_mask ; rows == nullptr means identity.
__global__ void __launch_bounds__(kThreads)
gather_mask_word_kernel(const uint32_t* __restrict__ words, const int32_t* __restrict__ rows,
                        long long n, int mic, int w, uint32_t and_mask, uint32_t* __restrict__ keys,
                        int32_t* __restrict__ iota) {
  const long long i = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  if (i >= n) return;
  const long long row = rows ? rows[i] : i;
  keys[i] = words[row * mic + w] & and_mask;
  if (iota) iota[i] = static_cast<int32_t>(i);
}

// mask_out[i, w] = words[rows[i], w] (word 0 ANDed with and_mask); argsort_out[i] = rows[i].
__global__ void __launch_bounds__(kThreads)
emit_sorted_masks_kernel(const uint32_t* __restrict__ words, const int32_t* __restrict__ rows,
                         long long n, int mic, uint32_t and_mask, int32_t* __restrict__ mask_out,
                         int32_t* __restrict__ argsort_out) {
  const long long i = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  if (i >= n) return;
  const long long row = rows ? rows[i] : i;
  for (int w = 0; w < mic; ++w) {
    uint32_t v = words[row * mic + w];
    if (w == 0) v &= and_mask;
    mask_out[i * mic + w] = static_cast<int32_t>(v);
  }
  argsort_out[i] = static_cast<int32_t>(row);
}

// ------------------------------------------------------------------------
// Phase 2 kernels (Native format): per offset, a stable compaction of the
// contributing input rows.  Grid = (row blocks, kv).
// ------------------------------------------------------------------------
template <int ND, bool K64>
__device__ __forceinline__ int native_out_row(const Geo& g, const int32_t* __restrict__ idx,
                                              long long j, int k, long long n_out,
                                              const Table<K64>& lookup) {
  using key_t = typename Table<K64>::key_t;
  int c[ND + 1];
  load_coord<ND>(idx, j, c);
  if (!coord_in_grid<ND>(g, c)) return -1;
  Odometer<ND> od;
  od.set(g, k);
  const long long key = out_key_from_input<ND>(g, c, od.pos);
  if (key < 0) return -1;
  const int r = lookup.find(static_cast<key_t>(key));
  return (r >= n_out) ? -1 : r;
}

template <int ND, bool K64>
__global__ void __launch_bounds__(kThreads)
native_count_kernel(const __grid_constant__ Geo g, const int32_t* __restrict__ idx, long long n_in,
                    long long n_out, Table<K64> lookup, int* __restrict__ block_counts) {
  const long long j = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  const int k = blockIdx.y;
  const int ok = (j < n_in) && native_out_row<ND, K64>(g, idx, j, k, n_out, lookup) >= 0;
  const int total = __syncthreads_count(ok);
  if (threadIdx.x == 0) block_counts[static_cast<long long>(k) * gridDim.x + blockIdx.x] = total;
}

// One block per offset: exclusive scan of that offset's block counts (in place)
// and the per-offset total.
__global__ void __launch_bounds__(kThreads)
native_scan_kernel(int* __restrict__ block_counts, int n_blocks, int32_t* __restrict__ npl, int kv,
                   int subm) {
  __shared__ int warp_sums[kThreads / 32];
  __shared__ int carry;
  const int k = blockIdx.x;
  int* row = block_counts + static_cast<long long>(k) * n_blocks;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < n_blocks; base += kThreads) {
    const int i = base + threadIdx.x;
    const int v = i < n_blocks ? row[i] : 0;
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, off);
      if ((threadIdx.x & 31) >= off) incl += t;
    }
    if ((threadIdx.x & 31) == 31) warp_sums[threadIdx.x >> 5] = incl;
    __syncthreads();
    int warp_off = 0;
    for (int w = 0; w < (threadIdx.x >> 5); ++w) warp_off += warp_sums[w];
    const int excl = carry + warp_off + incl - v;
    if (i < n_blocks) row[i] = excl;
    __syncthreads();
    if (threadIdx.x == kThreads - 1) carry = excl + v;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    // subm: counts are reported only for offsets before the centre
    // (spconv_triton/pytorch/_impl/pairs.py:269-277); the pair content is still complete.
    npl[k] = (subm && k >= kv / 2) ? 0 : carry;
  }
}

template <int ND, bool K64>
__global__ void __launch_bounds__(kThreads)
native_write_kernel(const __grid_constant__ Geo g, const int32_t* __restrict__ idx, long long n_in,
                    long long n_out, Table<K64> lookup, const int* __restrict__ block_offsets,
                    int32_t* __restrict__ pair) {
  __shared__ int warp_sums[kThreads / 32];
  const long long j = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  const int k = blockIdx.y;
  const int r = (j < n_in) ? native_out_row<ND, K64>(g, idx, j, k, n_out, lookup) : -1;
  const unsigned ballot = __ballot_sync(0xffffffffu, r >= 0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) warp_sums[warp] = __popc(ballot);
  __syncthreads();
  if (r >= 0) {
    int pos = block_offsets[static_cast<long long>(k) * gridDim.x + blockIdx.x];
    for (int w = 0; w < warp; ++w) pos += warp_sums[w];
    pos += __popc(ballot & ((1u << lane) - 1u));
    pair[static_cast<long long>(k) * n_in + pos] = static_cast<int32_t>(j);
    pair[(static_cast<long long>(g.kv) + k) * n_in + pos] = r;
  }
}

// out[row, 4q..4q+3] = pairs[4q..4q+3, row]; one thread per (row, q), q fastest, so
// that the 16-byte stores of a row are contiguous.
__global__ void __launch_bounds__(kThreads)
pairs_to_rowmajor_kernel(const int32_t* __restrict__ pairs, int kv, int kvp, long long n,
                         int32_t* __restrict__ out) {
  const long long e = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  const int quads = kvp / 4;
  const long long row = e / quads;
  if (row >= n) return;
  const int k0 = static_cast<int>(e % quads) * 4;
  int v[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) v[u] = (k0 + u < kv) ? __ldg(&pairs[static_cast<long long>(k0 + u) * n + row]) : -1;
  *reinterpret_cast<int4*>(&out[row * kvp + k0]) = make_int4(v[0], v[1], v[2], v[3]);
}

__global__ void __launch_bounds__(kThreads)
native_to_tables_kernel(const int32_t* __restrict__ pair_in, const int32_t* __restrict__ pair_out,
                        int kv, long long n_pair, int32_t* __restrict__ pair_fwd, long long n_out,
                        int32_t* __restrict__ pair_bwd, long long n_in) {
  const long long p = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  const int k = blockIdx.y;
  if (p >= n_pair) return;
  const int i = pair_in[static_cast<long long>(k) * n_pair + p];
  const int o = pair_out[static_cast<long long>(k) * n_pair + p];
  if (i < 0 || o < 0) return;
  if (o < n_out) pair_fwd[static_cast<long long>(k) * n_out + o] = i;
  if (pair_bwd != nullptr && i < n_in) pair_bwd[static_cast<long long>(k) * n_in + i] = o;
}

// ------------------------------------------------------------------------
// Host side: workspace layout
// ------------------------------------------------------------------------
struct Layout {
  bool k64;
  int key_bits;
  int mic;
  int64_t bound;  // upper bound on n_out
  int64_t obits_words = 0;  // dense numbering of the outputs: words of the bitmap (0 = hash table + sort)
  size_t off_obits = 0, off_oprefix = 0, off_scan = 0, scan_bytes = 0, off_iprefix = 0;
  uint32_t cap_in, cap_out;
  int64_t n_blocks_native;
  size_t off_counters, off_tin, off_tin_vals, off_tout, off_tout_vals, off_uniq, off_sorted;
  size_t off_words, off_keys_a, off_keys_b, off_vals_a, off_vals_b, off_cub, off_native;
  size_t cub_bytes, total;
  size_t off_bitmap, bitmap_bytes;  // occupancy bitmap of the input grid (0 bytes: not used)
  // Chained rulebooks: the input rows are exactly the output rows of an earlier strided layer whose
  // output bitmap and prefix (in ITS workspace) then serve as this layer's input bitmap; rows are
  // ranks by construction, and no input hash table is built.
  const uint32_t* shared_bits = nullptr;
  const uint32_t* shared_prefix = nullptr;
};

uint32_t pow2_at_least(int64_t v) {
  uint64_t c = 64;
  while (c < static_cast<uint64_t>(v)) c <<= 1;
  return static_cast<uint32_t>(std::min<uint64_t>(c, 1ull << 31));
}

int gcd_int(int a, int b) { return b == 0 ? a : gcd_int(b, a % b); }

bool make_geo(const spc_geometry* s, Geo* g) {
  if (s == nullptr || s->ndim < 1 || s->ndim > SPC_MAX_NDIM || s->batch_size <= 0) return false;
  g->ndim = s->ndim;
  g->batch = s->batch_size;
  g->subm = s->subm != 0;
  g->transpose = (!g->subm) && s->transpose != 0;
  g->kv = 1;
  for (int d = 0; d < SPC_MAX_NDIM; ++d) {
    const bool live = d < s->ndim;
    g->in_shape[d] = live ? s->in_shape[d] : 1;
    g->ksize[d] = live ? s->ksize[d] : 1;
    g->dil[d] = live ? s->dilation[d] : 1;
    if (live && (g->ksize[d] <= 0 || g->in_shape[d] <= 0 || g->dil[d] <= 0)) return false;
    if (g->subm) {
      g->out_shape[d] = g->in_shape[d];
      g->stride[d] = 1;
      g->pad[d] = (g->ksize[d] / 2) * g->dil[d];
    } else {
      g->out_shape[d] = live ? s->out_shape[d] : 1;
      g->stride[d] = live ? s->stride[d] : 1;
      g->pad[d] = live ? s->padding[d] : 0;
      if (live && (g->out_shape[d] <= 0 || g->stride[d] <= 0)) return false;
    }
    g->kv *= g->ksize[d];
  }
  g->tile_key = 0;
  for (int k = 0; k < 32; ++k) g->key_pos[k] = static_cast<unsigned char>(k);
  if (g->kv <= 32) {
    // distance of every offset from the kernel's centre (sum over the axes), then positions in
    // ascending distance, ties in offset order
    int dist[32];
    for (int k = 0; k < g->kv; ++k) {
      int rest = k, sum = 0;
      for (int d = g->ndim - 1; d >= 0; --d) {
        const int pos = rest % g->ksize[d];
        rest /= g->ksize[d];
        sum += std::abs(2 * pos - (g->ksize[d] - 1));
      }
      dist[k] = sum;
    }
    for (int k = 0; k < g->kv; ++k) {
      int rank = 0;
      for (int q = 0; q < g->kv; ++q) rank += dist[q] < dist[k] || (dist[q] == dist[k] && q < k);
      g->key_pos[k] = static_cast<unsigned char>(rank);
    }
  }
  return true;
}

Layout make_layout(const Geo& g, int64_t n_in) {
  Layout L{};
  double vol_in = g.batch, vol_out = g.batch;
  for (int d = 0; d < g.ndim; ++d) {
    vol_in *= g.in_shape[d];
    vol_out *= g.out_shape[d];
  }
  const double max_lin = std::max(vol_in, vol_out);
  L.k64 = max_lin >= 2147483648.0;
  L.key_bits = 1;
  while (L.key_bits < 63 && static_cast<double>(1ull << L.key_bits) < max_lin) ++L.key_bits;
  L.mic = (g.kv + 31) / 32;
  double per_input = 1;
  for (int d = 0; d < g.ndim; ++d) {
    int m = g.ksize[d];
    if (!g.transpose && !g.subm && gcd_int(g.dil[d], g.stride[d]) == 1)
      m = (g.ksize[d] + g.stride[d] - 1) / g.stride[d];
    per_input *= m;
  }
  if (g.subm) {
    L.bound = n_in;
  } else {
    const double b = std::min(static_cast<double>(n_in) * per_input, vol_out);
    L.bound = static_cast<int64_t>(std::max(b, 1.0));
  }
  L.cap_in = pow2_at_least(4 * n_in);  // load <= 0.25: most neighbour look-ups miss, keep their probe chains short
  L.cap_out = g.subm ? 0 : pow2_at_least(2 * L.bound);
  const int64_t n_max = std::max<int64_t>(n_in, L.bound);
  L.n_blocks_native = ceil_div(std::max<int64_t>(n_in, 1), kThreads);
  const size_t key_sz = L.k64 ? 8 : 4;

  size_t sort_keys_bytes = 0, sort_pairs_bytes = 0;
  if (L.k64)
    cub::DeviceRadixSort::SortKeys(nullptr, sort_keys_bytes, static_cast<unsigned long long*>(nullptr),
                                   static_cast<unsigned long long*>(nullptr), L.bound);
  else
    cub::DeviceRadixSort::SortKeys(nullptr, sort_keys_bytes, static_cast<uint32_t*>(nullptr),
                                   static_cast<uint32_t*>(nullptr), L.bound);
  cub::DeviceRadixSort::SortPairs(nullptr, sort_pairs_bytes, static_cast<uint32_t*>(nullptr),
                                  static_cast<uint32_t*>(nullptr), static_cast<int32_t*>(nullptr),
                                  static_cast<int32_t*>(nullptr), n_max);
  L.cub_bytes = std::max(sort_keys_bytes, sort_pairs_bytes);

  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off = align_up(off + bytes, 256);
    return at;
  };
  L.off_counters = take(256);
  L.off_tin = take(static_cast<size_t>(L.cap_in) * 8);
  L.off_tin_vals = take(L.k64 ? static_cast<size_t>(L.cap_in) * 4 : 0);
  L.off_tout = take(static_cast<size_t>(L.cap_out) * 8);
  L.off_tout_vals = take(L.k64 ? static_cast<size_t>(L.cap_out) * 4 : 0);
  L.off_uniq = take(g.subm ? 0 : static_cast<size_t>(L.bound) * key_sz);
  L.off_sorted = take(g.subm ? 0 : static_cast<size_t>(L.bound) * key_sz);
  L.off_words = take(static_cast<size_t>(n_max) * L.mic * 4);
  L.off_keys_a = take(static_cast<size_t>(n_max) * 4);
  L.off_keys_b = take(static_cast<size_t>(n_max) * 4);
  L.off_vals_a = take(static_cast<size_t>(n_max) * 4);
  L.off_vals_b = take(static_cast<size_t>(n_max) * 4);
  L.off_cub = take(L.cub_bytes);
  L.off_native = take(static_cast<size_t>(L.n_blocks_native) * g.kv * 4);
  // One bit per input cell, when that is small enough to live in L2 beside the hash table: most of
  // the kv neighbour cells of a voxel are empty, and a bit test (neighbours share bytes) then
  // answers "absent" without a hash probe.
  L.bitmap_bytes = (!L.k64 && vol_in / 8.0 <= 24.0 * 1024 * 1024) ? align_up(static_cast<size_t>(vol_in / 8.0) + 4, 256) : 0;
  L.off_bitmap = take(L.bitmap_bytes);
  L.off_iprefix = take(L.bitmap_bytes);  // set bits before each word of the input bitmap
  // The same for the output grid of a strided layer; there the bitmap also numbers the outputs.
  L.obits_words = (!g.subm && !L.k64 && vol_out / 8.0 <= 24.0 * 1024 * 1024) ? static_cast<int64_t>(vol_out / 32.0) + 1 : 0;
  L.off_obits = take(static_cast<size_t>(L.obits_words) * 4);
  L.off_oprefix = take(static_cast<size_t>(L.obits_words) * 4);
  const int64_t scan_words = std::max<int64_t>(L.obits_words, static_cast<int64_t>(L.bitmap_bytes / 4));
  if (scan_words) {
    size_t scan_bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, static_cast<uint32_t*>(nullptr), static_cast<uint32_t*>(nullptr),
                                  static_cast<int>(scan_words));
    L.off_scan = take(scan_bytes);
    L.scan_bytes = scan_bytes;
  }
  L.total = off;
  return L;
}

template <bool K64>
Table<K64> table_at(char* ws, size_t off_slots, size_t off_vals, uint32_t cap);
template <>
Table<false> table_at<false>(char* ws, size_t off_slots, size_t, uint32_t cap) {
  Table<false> t;
  t.slots = reinterpret_cast<unsigned long long*>(ws + off_slots);
  t.cap_mask = cap ? cap - 1 : 0;
  return t;
}
template <>
Table<true> table_at<true>(char* ws, size_t off_slots, size_t off_vals, uint32_t cap) {
  Table<true> t;
  t.slots = reinterpret_cast<unsigned long long*>(ws + off_slots);
  t.vals = reinterpret_cast<int*>(ws + off_vals);
  t.cap_mask = cap ? cap - 1 : 0;
  return t;
}

template <bool K64>
Table<K64> tin_at(char* ws, const Layout& L);
template <>
Table<false> tin_at<false>(char* ws, const Layout& L) {
  Table<false> t = table_at<false>(ws, L.off_tin, L.off_tin_vals, L.cap_in);
  if (L.shared_bits != nullptr) {
    t.obits = const_cast<uint32_t*>(L.shared_bits);
    t.oprefix = L.shared_prefix;
    return t;  // `unsorted` stays null: the rows are the ranks
  }
  if (L.bitmap_bytes) {
    t.obits = reinterpret_cast<uint32_t*>(ws + L.off_bitmap);
    t.oprefix = reinterpret_cast<const uint32_t*>(ws + L.off_iprefix);
    t.unsorted = reinterpret_cast<const int*>(ws + L.off_counters) + kUnsorted;
  }
  return t;
}
template <>
Table<true> tin_at<true>(char* ws, const Layout& L) {
  return table_at<true>(ws, L.off_tin, L.off_tin_vals, L.cap_in);
}

template <bool K64>
Table<K64> tout_at(char* ws, const Layout& L);
template <>
Table<false> tout_at<false>(char* ws, const Layout& L) {
  Table<false> t = table_at<false>(ws, L.off_tout, L.off_tout_vals, L.cap_out);
  if (L.obits_words) {
    t.obits = reinterpret_cast<uint32_t*>(ws + L.off_obits);
    t.oprefix = reinterpret_cast<const uint32_t*>(ws + L.off_oprefix);
  }
  return t;
}
template <>
Table<true> tout_at<true>(char* ws, const Layout& L) {
  return table_at<true>(ws, L.off_tout, L.off_tout_vals, L.cap_out);
}

// Byte fill of scratch regions by a kernel of this library rather than cudaMemsetAsync: the
// regions are 16-byte multiples at 16-byte aligned offsets, and a kernel can neither be routed
// to a copy engine (where it would queue behind a large transfer of the application) nor
// cost a driver memset's set-up.
__global__ void __launch_bounds__(256) fill_bytes_kernel(uint4* __restrict__ dst, uint32_t word, long long n16) {
  const long long stride = static_cast<long long>(gridDim.x) * 256;
  const uint4 v = make_uint4(word, word, word, word);
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n16; i += stride) dst[i] = v;
}
int fill_bytes(void* dst, int byte, size_t bytes, cudaStream_t st) {
  if (bytes == 0) return SPC_OK;
  if ((reinterpret_cast<uintptr_t>(dst) & 15u) != 0 || bytes % 16 != 0) {
    SPC_CUDA_OK(cudaMemsetAsync(dst, byte, bytes, st));
    return SPC_OK;
  }
  const long long n16 = static_cast<long long>(bytes / 16);
  const uint32_t b = static_cast<uint32_t>(byte) & 0xffu;
  const unsigned blocks = static_cast<unsigned>(std::min<long long>(ceil_div(n16, 256), 16ll * sm_count()));
  fill_bytes_kernel<<<blocks, 256, 0, st>>>(static_cast<uint4*>(dst), b * 0x01010101u, n16);
  SPC_LAUNCH_OK();
  return SPC_OK;
}
#define SPC_FILL(dst, byte, bytes, st)                              \
  do {                                                              \
    const int rc__ = fill_bytes((dst), (byte), (bytes), (st));      \
    if (rc__ != SPC_OK) return rc__;                                \
  } while (0)

// A few page-locked words per host thread and device that kernels write and the host reads after
// synchronising (host memory: the library still allocates no device memory).
int host_mailbox(volatile int** out) {
  static thread_local int* boxes[kMaxDevices] = {nullptr};
  const int dev = current_device_slot();
  if (dev < 0) return fail(SPC_ERR_CUDA, "rulebook: no current device");
  if (boxes[dev] == nullptr) {
    void* p = nullptr;
    SPC_CUDA_OK(cudaHostAlloc(&p, 64, cudaHostAllocPortable | cudaHostAllocMapped));
    boxes[dev] = static_cast<int*>(p);
  }
  *out = boxes[dev];
  return SPC_OK;
}

// How the host waits for a count.  cudaStreamSynchronize spins on a core for the whole wait, which is
// the fastest wake-up (a pass alone: 2.28 ms against 2.59 ms with a blocking event) but needs an idle
// core per pass in flight; with SPC_HOST_WAIT=block in the environment (read once) the thread sleeps
// on a blocking event instead, for processes that keep several passes in flight on few cores (one
// process per GPU, eight GPUs, three host threads each).  One event per host thread and device.
int wait_for_stream(cudaStream_t st) {
  static const bool block = [] {
    const char* v = std::getenv("SPC_HOST_WAIT");
    return v != nullptr && std::strcmp(v, "block") == 0;
  }();
  if (!block) {
    SPC_CUDA_OK(cudaStreamSynchronize(st));
    return SPC_OK;
  }
  static thread_local cudaEvent_t events[kMaxDevices] = {nullptr};
  const int dev = current_device_slot();
  if (dev < 0) return fail(SPC_ERR_CUDA, "rulebook: no current device");
  if (events[dev] == nullptr)
    SPC_CUDA_OK(cudaEventCreateWithFlags(&events[dev], cudaEventBlockingSync | cudaEventDisableTiming));
  SPC_CUDA_OK(cudaEventRecord(events[dev], st));
  SPC_CUDA_OK(cudaEventSynchronize(events[dev]));
  return SPC_OK;
}

inline unsigned blocks_for(int64_t n) { return static_cast<unsigned>(ceil_div(std::max<int64_t>(n, 1), kThreads)); }

// ------------------------------------------------------------------------
// Phase 1
// ------------------------------------------------------------------------
template <int ND, bool K64>
int prepare_impl(const Geo& g, const Layout& L, const int32_t* idx, int64_t n_in, char* ws,
                 int64_t* n_out_host, cudaStream_t st) {
  using key_t = typename Table<K64>::key_t;
  int* counters = reinterpret_cast<int*>(ws + L.off_counters);
  // Submanifold layers return without a host read, so a row outside the grid is also recorded in the
  // device status word, which the host reads at its next synchronisation point.
  int* dev_status = device_status_ptr();
  SPC_FILL(counters, 0, 256, st);
  const bool chained = L.shared_bits != nullptr;  // input bitmap and prefix exist already, no input table
  if (!chained) {
    SPC_FILL(ws + L.off_tin, 0xFF, static_cast<size_t>(L.cap_in) * 8, st);
    if (K64) SPC_FILL(ws + L.off_tin_vals, 0x7F, static_cast<size_t>(L.cap_in) * 4, st);
  }
  Table<K64> tin = tin_at<K64>(ws, L);
  uint32_t* bitmap = (L.bitmap_bytes && !chained) ? reinterpret_cast<uint32_t*>(ws + L.off_bitmap) : nullptr;
  if (bitmap != nullptr) {
    SPC_FILL(bitmap, 0, L.bitmap_bytes, st);
    mark_inputs_kernel<ND><<<blocks_for(n_in), kThreads, 0, st>>>(g, idx, n_in, bitmap, counters, dev_status);
    SPC_LAUNCH_OK();
    const int64_t words = static_cast<int64_t>(L.bitmap_bytes / 4);
    uint32_t* iprefix = reinterpret_cast<uint32_t*>(ws + L.off_iprefix);
    count_bits_kernel<<<blocks_for(words), kThreads, 0, st>>>(bitmap, words, iprefix);
    SPC_LAUNCH_OK();
    size_t scan_bytes = L.scan_bytes;
    SPC_CUDA_OK(cub::DeviceScan::ExclusiveSum(ws + L.off_scan, scan_bytes, iprefix, iprefix, static_cast<int>(words), st));
  }
  if (!chained) {
    insert_inputs_kernel<ND, K64><<<blocks_for(n_in), kThreads, 0, st>>>(g, idx, n_in, tin, counters, bitmap,
                                                                         dev_status);
    SPC_LAUNCH_OK();
  }
  if (g.subm) {
    *n_out_host = n_in;
    return SPC_OK;
  }
  const bool dense_out = L.obits_words != 0;
  if (dense_out) {
    SPC_FILL(ws + L.off_obits, 0, align_up(static_cast<size_t>(L.obits_words) * 4, 16), st);
  } else {
    SPC_FILL(ws + L.off_tout, 0xFF, static_cast<size_t>(L.cap_out) * 8, st);
    if (K64) SPC_FILL(ws + L.off_tout_vals, 0x7F, static_cast<size_t>(L.cap_out) * 4, st);
  }
  Table<K64> tout = tout_at<K64>(ws, L);
  key_t* uniq = reinterpret_cast<key_t*>(ws + L.off_uniq);
  key_t* sorted = reinterpret_cast<key_t*>(ws + L.off_sorted);
  bool axes_fit = true;  // mark_outputs_kernel keeps one bit per kernel offset of an axis
  for (int d = 0; d < ND; ++d) axes_fit = axes_fit && g.ksize[d] <= 32;
  if (dense_out && axes_fit) {
    mark_outputs_kernel<ND><<<blocks_for(n_in), kThreads, 0, st>>>(
        g, idx, n_in, reinterpret_cast<uint32_t*>(ws + L.off_obits));
  } else {
    enumerate_outputs_kernel<ND, K64><<<blocks_for(n_in), kThreads, 0, st>>>(g, idx, n_in, tout, uniq, counters);
  }
  SPC_LAUNCH_OK();
  if (dense_out) {
    uint32_t* bits = reinterpret_cast<uint32_t*>(ws + L.off_obits);
    uint32_t* prefix = reinterpret_cast<uint32_t*>(ws + L.off_oprefix);
    count_bits_kernel<<<blocks_for(L.obits_words), kThreads, 0, st>>>(bits, L.obits_words, prefix);
    SPC_LAUNCH_OK();
    size_t scan_bytes = L.scan_bytes;
    SPC_CUDA_OK(cub::DeviceScan::ExclusiveSum(ws + L.off_scan, scan_bytes, prefix, prefix,
                                              static_cast<int>(L.obits_words), st));
    expand_bits_kernel<<<blocks_for(L.obits_words), kThreads, 0, st>>>(
        bits, prefix, L.obits_words, L.bound, reinterpret_cast<uint32_t*>(sorted), counters);
    SPC_LAUNCH_OK();
  }
  // The output count reaches the host through a page-locked word that a one-thread kernel writes,
  // not through a device-to-host copy: a copy would queue on the copy engine behind whatever
  // transfer the application has in flight (a previous result going back to the host, say) and
  // stall the whole rulebook chain for its duration.
  volatile int* box = nullptr;
  int rc_box = host_mailbox(&box);
  if (rc_box != SPC_OK) return rc_box;
  publish_counters_kernel<<<1, 32, 0, st>>>(counters, dev_status, const_cast<int*>(box));
  SPC_LAUNCH_OK();
  {
    const int rc_wait = wait_for_stream(st);
    if (rc_wait != SPC_OK) return rc_wait;
  }
  int host[2] = {box[kUniqueCount], box[kStatus]};
  const int sticky = box[2];  // the device status word: a bounded wait of an earlier kernel, or a bad row of an earlier layer
  if (host[kStatus] != 0 || sticky != 0) {
    if (dev_status != nullptr && sticky != 0) SPC_CUDA_OK(cudaMemsetAsync(dev_status, 0, sizeof(int), st));
    const int code = host[kStatus] != 0 ? host[kStatus] : sticky;
    if (code == SPC_ERR_INVALID_ARGUMENT)
      return fail(code, "rulebook: an index row lies outside batch_size / spatial_shape");
    if (code == SPC_ERR_DEVICE_WAIT_EXPIRED)
      return fail(code, "a bounded device-side wait of an earlier kernel expired; its output is incomplete");
    return fail(code, "rulebook: hash table full (status %d)", code);
  }
  const int64_t n_out = host[kUniqueCount];
  *n_out_host = n_out;
  if (n_out == 0) return SPC_OK;
  if (n_out > L.bound) return fail(SPC_ERR_WORKSPACE_TOO_SMALL, "rulebook: %lld outputs exceed bound %lld",
                                   static_cast<long long>(n_out), static_cast<long long>(L.bound));
  if (dense_out) return SPC_OK;  // numbered and listed in ascending order already
  size_t cub_bytes = L.cub_bytes;
  SPC_CUDA_OK(cub::DeviceRadixSort::SortKeys(ws + L.off_cub, cub_bytes, uniq, sorted, n_out, 0,
                                              std::min<int>(L.key_bits, sizeof(key_t) * 8), st));
  assign_ranks_kernel<K64><<<blocks_for(n_out), kThreads, 0, st>>>(tout, sorted, n_out);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

// Sorts the per-row bitmasks (stable, ascending as unsigned, highest word most
// significant) and emits pair_mask / mask_argsort for every split.
// One mask word per row, one split that keeps every bit, sorted: the words are the sort keys as
// they stand and the sort can write pair_mask / mask_argsort itself, if the kernel that produced the
// words also left 0..n-1 in the value scratch (mask_iota()).
bool masks_sort_in_place(const Layout& L, const uint32_t* split_masks, int n_split, int do_sort) {
  return L.mic == 1 && n_split == 1 && do_sort != 0 && split_masks[0] == 0xffffffffu;
}
int32_t* mask_iota(const Layout& L, char* ws, const uint32_t* split_masks, int n_split, int do_sort) {
  return masks_sort_in_place(L, split_masks, n_split, do_sort) ? reinterpret_cast<int32_t*>(ws + L.off_vals_a)
                                                                 : nullptr;
}

int emit_masks(const Layout& L, char* ws, int64_t n, int kv, const uint32_t* split_masks, int n_split,
               int do_sort, int32_t* mask_out, int32_t* argsort_out, cudaStream_t st) {
  const uint32_t* words = reinterpret_cast<const uint32_t*>(ws + L.off_words);
  if (masks_sort_in_place(L, split_masks, n_split, do_sort)) {
    size_t cub_bytes = L.cub_bytes;
    SPC_CUDA_OK(cub::DeviceRadixSort::SortPairs(ws + L.off_cub, cub_bytes, words, reinterpret_cast<uint32_t*>(mask_out),
                                                 reinterpret_cast<const int32_t*>(ws + L.off_vals_a), argsort_out, n, 0,
                                                 std::min(32, kv), st));
    return SPC_OK;
  }
  uint32_t* keys_a = reinterpret_cast<uint32_t*>(ws + L.off_keys_a);
  uint32_t* keys_b = reinterpret_cast<uint32_t*>(ws + L.off_keys_b);
  int32_t* vals_a = reinterpret_cast<int32_t*>(ws + L.off_vals_a);
  int32_t* vals_b = reinterpret_cast<int32_t*>(ws + L.off_vals_b);
  const int mic = L.mic;
  for (int s = 0; s < n_split; ++s) {
    const uint32_t and0 = split_masks[s];
    int32_t* m_out = mask_out + static_cast<int64_t>(s) * n * mic;
    int32_t* a_out = argsort_out + static_cast<int64_t>(s) * n;
    const int32_t* rows = nullptr;
    if (do_sort) {
      int32_t* cur = vals_a;
      int32_t* nxt = vals_b;
      for (int w = 0; w < mic; ++w) {
        const uint32_t andw = (w == 0) ? and0 : 0xffffffffu;
        gather_mask_word_kernel<<<blocks_for(n), kThreads, 0, st>>>(
            words, w == 0 ? nullptr : cur, n, mic, w, andw, keys_a, w == 0 ? cur : nullptr);
        SPC_LAUNCH_OK();
        const int bits = std::min(32, kv - 32 * w);
        size_t cub_bytes = L.cub_bytes;
        SPC_CUDA_OK(cub::DeviceRadixSort::SortPairs(ws + L.off_cub, cub_bytes, keys_a, keys_b, cur, nxt,
                                                     n, 0, bits, st));
        std::swap(cur, nxt);
      }
      rows = cur;
    }
    emit_sorted_masks_kernel<<<blocks_for(n), kThreads, 0, st>>>(words, rows, n, mic, and0, m_out, a_out);
    SPC_LAUNCH_OK();
  }
  return SPC_OK;
}

// Input-side tables of a strided / transposed layer: pair_bwd and its masks.
// Reads the output hash the forward phase ranked; shares the mask scratch with
// it, so it must follow the forward phase of the same workspace.
template <int ND, bool K64>
int igemm_backward_impl(const Geo& g, const Layout& L, const int32_t* idx, int64_t n_in, int64_t n_out, char* ws,
                        int32_t* pair_bwd, int32_t* mask_bwd, int32_t* argsort_bwd, const uint32_t* split_masks,
                        int n_split, int do_sort, int32_t* bwd_rm, cudaStream_t st) {
  const int kvp = (g.kv + 3) & ~3;
  Table<K64> tout = tout_at<K64>(ws, L);
  uint32_t* words = reinterpret_cast<uint32_t*>(ws + L.off_words);
  int32_t* iota = mask_bwd != nullptr ? mask_iota(L, ws, split_masks, n_split, do_sort) : nullptr;
  fill_bwd_kernel<ND, K64><<<blocks_for(n_in), kThreads, 0, st>>>(
      g, idx, n_in, n_out, tout, pair_bwd, mask_bwd ? words : nullptr, L.mic, bwd_rm, kvp, iota);
  SPC_LAUNCH_OK();
  if (mask_bwd != nullptr) return emit_masks(L, ws, n_in, g.kv, split_masks, n_split, do_sort, mask_bwd, argsort_bwd, st);
  return SPC_OK;
}

template <int ND, bool K64>
int igemm_impl(const Geo& g, const Layout& L, const int32_t* idx, int64_t n_in, int64_t n_out, char* ws,
               int32_t* out_indices, int32_t* pair_fwd, int32_t* pair_bwd, int32_t* mask_fwd,
               int32_t* argsort_fwd, int32_t* mask_bwd, int32_t* argsort_bwd,
               const uint32_t* split_masks, int n_split, int do_sort, int32_t* fwd_rm, int32_t* bwd_rm,
               cudaStream_t st) {
  using key_t = typename Table<K64>::key_t;
  const int kvp = (g.kv + 3) & ~3;
  Table<K64> tin = tin_at<K64>(ws, L);
  Table<K64> tout = tout_at<K64>(ws, L);
  const key_t* sorted = reinterpret_cast<const key_t*>(ws + L.off_sorted);
  uint32_t* words = reinterpret_cast<uint32_t*>(ws + L.off_words);
  const uint32_t* bitmap = L.shared_bits != nullptr ? L.shared_bits
                           : (L.bitmap_bytes ? reinterpret_cast<const uint32_t*>(ws + L.off_bitmap) : nullptr);
  int32_t* iota = mask_iota(L, ws, split_masks, n_split, do_sort);
  // the row-major copies go through shared memory when a warp's 32 rows fit (kernel volumes up to 32)
  const bool with_bwd = g.subm && pair_bwd != nullptr;
  const int staged = (fwd_rm != nullptr && kvp <= 32 && (reinterpret_cast<uintptr_t>(fwd_rm) & 15u) == 0 &&
                      (!with_bwd || bwd_rm == nullptr || (reinterpret_cast<uintptr_t>(bwd_rm) & 15u) == 0)) ? 1 : 0;
  const size_t stage_bytes = staged ? static_cast<size_t>(kThreads / 32) * (with_bwd ? 2 : 1) * 32 * kvp * 4 : 0;
  if (with_bwd) {
    static bool configured[kMaxDevices] = {false};
    SPC_CUDA_OK(ensure_dynamic_smem(fill_fwd_kernel<ND, K64, true>, 64 * 1024, configured));
    fill_fwd_kernel<ND, K64, true><<<blocks_for(n_out), kThreads, stage_bytes, st>>>(
        g, idx, sorted, n_out, tin, out_indices, pair_fwd, pair_bwd, words, L.mic, fwd_rm, bwd_rm, kvp, bitmap, iota,
        staged);
  } else {
    fill_fwd_kernel<ND, K64, false><<<blocks_for(n_out), kThreads, stage_bytes, st>>>(
        g, idx, sorted, n_out, tin, out_indices, pair_fwd, nullptr, words, L.mic, fwd_rm, nullptr, kvp, bitmap, iota,
        staged);
  }
  SPC_LAUNCH_OK();
  int rc = emit_masks(L, ws, n_out, g.kv, split_masks, n_split, do_sort, mask_fwd, argsort_fwd, st);
  if (rc != SPC_OK) return rc;
  if (!g.subm && pair_bwd != nullptr)
    return igemm_backward_impl<ND, K64>(g, L, idx, n_in, n_out, ws, pair_bwd, mask_bwd, argsort_bwd, split_masks,
                                        n_split, do_sort, bwd_rm, st);
  return SPC_OK;
}

template <int ND, bool K64>
int native_impl(const Geo& g, const Layout& L, const int32_t* idx, int64_t n_in, int64_t n_out, char* ws,
                int32_t* out_indices, int32_t* pair, int32_t* npl, cudaStream_t st) {
  using key_t = typename Table<K64>::key_t;
  Table<K64> tin = tin_at<K64>(ws, L);
  Table<K64> tout = tout_at<K64>(ws, L);
  const Table<K64>& lookup = g.subm ? tin : tout;
  const key_t* sorted = reinterpret_cast<const key_t*>(ws + L.off_sorted);
  int* block_counts = reinterpret_cast<int*>(ws + L.off_native);
  const unsigned nb = static_cast<unsigned>(L.n_blocks_native);
  dim3 grid(nb, static_cast<unsigned>(g.kv));
  SPC_CUDA_OK(cudaMemsetAsync(pair, 0xFF, static_cast<size_t>(2) * g.kv * n_in * sizeof(int32_t), st));
  native_count_kernel<ND, K64><<<grid, kThreads, 0, st>>>(g, idx, n_in, n_out, lookup, block_counts);
  SPC_LAUNCH_OK();
  native_scan_kernel<<<g.kv, kThreads, 0, st>>>(block_counts, static_cast<int>(nb), npl, g.kv, g.subm);
  SPC_LAUNCH_OK();
  native_write_kernel<ND, K64><<<grid, kThreads, 0, st>>>(g, idx, n_in, n_out, lookup, block_counts, pair);
  SPC_LAUNCH_OK();
  (void)sorted;
  (void)out_indices;
  return SPC_OK;
}

template <int ND, bool K64>
__global__ void __launch_bounds__(kThreads)
write_out_indices_kernel(const __grid_constant__ Geo g,
                         const typename Table<K64>::key_t* __restrict__ sorted, long long n_out,
                         int32_t* __restrict__ out_indices) {
  const long long r = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x;
  if (r >= n_out) return;
  int o[ND + 1];
  delinearize_out<ND>(g, static_cast<long long>(sorted[r]), o);
#pragma unroll
  for (int d = 0; d <= ND; ++d) out_indices[r * (ND + 1) + d] = o[d];
}

template <typename F>
int dispatch(int ndim, bool k64, F&& f) {
  switch (ndim * 2 + (k64 ? 1 : 0)) {
    case 2: return f(std::integral_constant<int, 1>{}, std::false_type{});
    case 3: return f(std::integral_constant<int, 1>{}, std::true_type{});
    case 4: return f(std::integral_constant<int, 2>{}, std::false_type{});
    case 5: return f(std::integral_constant<int, 2>{}, std::true_type{});
    case 6: return f(std::integral_constant<int, 3>{}, std::false_type{});
    case 7: return f(std::integral_constant<int, 3>{}, std::true_type{});
    case 8: return f(std::integral_constant<int, 4>{}, std::false_type{});
    case 9: return f(std::integral_constant<int, 4>{}, std::true_type{});
    default: return fail(SPC_ERR_INVALID_ARGUMENT, "ndim %d not in 1..4", ndim);
  }
}

// Points `L` at the output bitmap of `producer` if that strided layer numbered its outputs through
// one and its output grid is this layer's input grid.
void adopt_producer_bits(const Geo& g, Layout* L, const RulebookProducer* producer) {
  if (producer == nullptr || producer->geom == nullptr || producer->workspace == nullptr || L->k64 ||
      L->bitmap_bytes == 0)
    return;
  Geo gp;
  if (!make_geo(producer->geom, &gp) || gp.subm || gp.ndim != g.ndim || gp.batch != g.batch) return;
  for (int d = 0; d < g.ndim; ++d)
    if (gp.out_shape[d] != g.in_shape[d]) return;
  const Layout Lp = make_layout(gp, producer->n_in);
  if (Lp.obits_words == 0) return;
  const char* wp = static_cast<const char*>(producer->workspace);
  L->shared_bits = reinterpret_cast<const uint32_t*>(wp + Lp.off_obits);
  L->shared_prefix = reinterpret_cast<const uint32_t*>(wp + Lp.off_oprefix);
}

}  // namespace

int rulebook_prepare_chained(const spc_geometry* sg, const int32_t* indices, int64_t n_in, void* workspace,
                             size_t workspace_bytes, int64_t* n_out_host, const RulebookProducer* producer,
                             cudaStream_t st) {
  Geo g;
  if (!make_geo(sg, &g)) return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook: bad geometry");
  if (n_in <= 0 || indices == nullptr || n_out_host == nullptr || workspace == nullptr)
    return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook: n_in must be > 0 and pointers non-null");
  if (n_in >= (1ll << 30)) return fail(SPC_ERR_SIZE_LIMIT, "rulebook: n_in %lld too large", (long long)n_in);
  Layout L = make_layout(g, n_in);
  if (workspace_bytes < L.total)
    return fail(SPC_ERR_WORKSPACE_TOO_SMALL, "rulebook: workspace %zu < %zu bytes", workspace_bytes, L.total);
  adopt_producer_bits(g, &L, producer);
  char* ws = static_cast<char*>(workspace);
  return dispatch(g.ndim, L.k64, [&](auto nd, auto k64) {
    return prepare_impl<decltype(nd)::value, decltype(k64)::value>(g, L, indices, n_in, ws, n_out_host, st);
  });
}

int rulebook_igemm_chained(const spc_geometry* sg, const int32_t* indices, int64_t n_in, int64_t n_out,
                           void* workspace, size_t workspace_bytes, int32_t* out_indices, int32_t* pair_fwd,
                           int32_t* pair_bwd, int32_t* mask_fwd, int32_t* argsort_fwd, int32_t* mask_bwd,
                           int32_t* argsort_bwd, const uint32_t* split_masks, int n_split, int do_sort,
                           int32_t* pair_fwd_rowmajor, int32_t* pair_bwd_rowmajor, const RulebookProducer* producer,
                           cudaStream_t st) {
  Geo g;
  if (!make_geo(sg, &g)) return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook: bad geometry");
  // pair_fwd may be absent when the row-major copy is all the caller's GEMMs read (native pass)
  if (n_in <= 0 || n_out <= 0 || !indices || !workspace || (!pair_fwd && (!pair_fwd_rowmajor || pair_bwd)) || !mask_fwd ||
      !argsort_fwd || !split_masks || n_split < 1 || n_split > 2)
    return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook igemm: bad arguments");
  if (!g.subm && out_indices == nullptr)
    return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook igemm: out_indices required for non-subm layers");
  if (g.subm && n_out != n_in) return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook igemm: subm needs n_out == n_in");
  if ((mask_bwd == nullptr) != (argsort_bwd == nullptr))
    return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook igemm: mask_bwd and argsort_bwd go together");
  Layout L = make_layout(g, n_in);
  if (workspace_bytes < L.total)
    return fail(SPC_ERR_WORKSPACE_TOO_SMALL, "rulebook: workspace %zu < %zu bytes", workspace_bytes, L.total);
  if (n_out > L.bound) return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook igemm: n_out exceeds prepared bound");
  adopt_producer_bits(g, &L, producer);
  // do_sort == 2 (callers inside the library only): order the rows by the tile key.  mask_fwd then
  // receives the sorted KEYS, not the sorted mask words, and argsort_fwd the tile order.
  g.tile_key = do_sort == 2 && rulebook_tile_key_applies(sg, pair_bwd != nullptr || mask_bwd != nullptr, split_masks, n_split);
  do_sort = do_sort != 0;
  char* ws = static_cast<char*>(workspace);
  return dispatch(g.ndim, L.k64, [&](auto nd, auto k64) {
    return igemm_impl<decltype(nd)::value, decltype(k64)::value>(
        g, L, indices, n_in, n_out, ws, out_indices, pair_fwd, pair_bwd, mask_fwd, argsort_fwd, mask_bwd,
        argsort_bwd, split_masks, n_split, do_sort, pair_fwd_rowmajor, pair_bwd_rowmajor, st);
  });
}

bool rulebook_tile_key_applies(const spc_geometry* sg, bool with_backward, const uint32_t* split_masks, int n_split) {
  Geo g;
  return make_geo(sg, &g) && g.kv > 1 && g.kv <= 31 && !with_backward && n_split == 1 && split_masks != nullptr &&
         split_masks[0] == 0xffffffffu;
}

}  // namespace spc

using namespace spc;

extern "C" size_t spc_rulebook_workspace_bytes(const spc_geometry* sg, int64_t n_in) {
  Geo g;
  if (!make_geo(sg, &g) || n_in <= 0) return 0;
  return make_layout(g, n_in).total;
}

extern "C" int spc_rulebook_prepare(const spc_geometry* sg, const int32_t* indices, int64_t n_in,
                                    void* workspace, size_t workspace_bytes, int64_t* n_out_host,
                                    void* stream) {
  return rulebook_prepare_chained(sg, indices, n_in, workspace, workspace_bytes, n_out_host, nullptr,
                                  static_cast<cudaStream_t>(stream));
}

extern "C" int spc_rulebook_igemm(const spc_geometry* sg, const int32_t* indices, int64_t n_in,
                                  int64_t n_out, void* workspace, size_t workspace_bytes,
                                  int32_t* out_indices, int32_t* pair_fwd, int32_t* pair_bwd,
                                  int32_t* mask_fwd, int32_t* argsort_fwd, int32_t* mask_bwd,
                                  int32_t* argsort_bwd, const uint32_t* split_masks, int n_split,
                                  int do_sort, int32_t* pair_fwd_rowmajor, int32_t* pair_bwd_rowmajor,
                                  void* stream) {
  if (!pair_fwd) return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook igemm: bad arguments");
  return rulebook_igemm_chained(sg, indices, n_in, n_out, workspace, workspace_bytes, out_indices, pair_fwd, pair_bwd,
                                mask_fwd, argsort_fwd, mask_bwd, argsort_bwd, split_masks, n_split, do_sort != 0,
                                pair_fwd_rowmajor, pair_bwd_rowmajor, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int spc_rulebook_igemm_backward(const spc_geometry* sg, const int32_t* indices, int64_t n_in,
                                           int64_t n_out, void* workspace, size_t workspace_bytes,
                                           int32_t* pair_bwd, int32_t* mask_bwd, int32_t* argsort_bwd,
                                           const uint32_t* split_masks, int n_split, int do_sort,
                                           int32_t* pair_bwd_rowmajor, void* stream) {
  Geo g;
  if (!make_geo(sg, &g)) return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook: bad geometry");
  if (g.subm) return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook igemm backward: submanifold tables come from the forward call");
  if (n_in <= 0 || n_out <= 0 || !indices || !workspace || !pair_bwd || !split_masks || n_split < 1 || n_split > 2)
    return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook igemm backward: bad arguments");
  if ((mask_bwd == nullptr) != (argsort_bwd == nullptr))
    return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook igemm backward: mask_bwd and argsort_bwd go together");
  const Layout L = make_layout(g, n_in);
  if (workspace_bytes < L.total)
    return fail(SPC_ERR_WORKSPACE_TOO_SMALL, "rulebook: workspace %zu < %zu bytes", workspace_bytes, L.total);
  if (n_out > L.bound) return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook igemm backward: n_out exceeds prepared bound");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  char* ws = static_cast<char*>(workspace);
  return dispatch(g.ndim, L.k64, [&](auto nd, auto k64) {
    return igemm_backward_impl<decltype(nd)::value, decltype(k64)::value>(
        g, L, indices, n_in, n_out, ws, pair_bwd, mask_bwd, argsort_bwd, split_masks, n_split, do_sort,
        pair_bwd_rowmajor, st);
  });
}

extern "C" int spc_rulebook_native(const spc_geometry* sg, const int32_t* indices, int64_t n_in,
                                   int64_t n_out, void* workspace, size_t workspace_bytes,
                                   int32_t* out_indices, int32_t* pair, int32_t* indice_num_per_loc,
                                   void* stream) {
  Geo g;
  if (!make_geo(sg, &g)) return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook: bad geometry");
  if (n_in <= 0 || n_out <= 0 || !indices || !workspace || !pair || !indice_num_per_loc)
    return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook native: bad arguments");
  if (!g.subm && out_indices == nullptr)
    return fail(SPC_ERR_INVALID_ARGUMENT, "rulebook native: out_indices required for non-subm layers");
  const Layout L = make_layout(g, n_in);
  if (workspace_bytes < L.total)
    return fail(SPC_ERR_WORKSPACE_TOO_SMALL, "rulebook: workspace %zu < %zu bytes", workspace_bytes, L.total);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  char* ws = static_cast<char*>(workspace);
  return dispatch(g.ndim, L.k64, [&](auto nd, auto k64) {
    constexpr int ND = decltype(nd)::value;
    constexpr bool K64 = decltype(k64)::value;
    if (!g.subm) {
      using key_t = typename Table<K64>::key_t;
      write_out_indices_kernel<ND, K64><<<blocks_for(n_out), kThreads, 0, st>>>(
          g, reinterpret_cast<const key_t*>(ws + L.off_sorted), n_out, out_indices);
      SPC_LAUNCH_OK();
    }
    return native_impl<ND, K64>(g, L, indices, n_in, n_out, ws, out_indices, pair, indice_num_per_loc, st);
  });
}

extern "C" int spc_pairs_to_rowmajor(const int32_t* pairs, int kv, int64_t n, int32_t* out, void* stream) {
  if (!pairs || !out || kv <= 0 || n < 0) return fail(SPC_ERR_INVALID_ARGUMENT, "pairs_to_rowmajor: bad arguments");
  if (n == 0) return SPC_OK;
  const int kvp = (kv + 3) & ~3;
  pairs_to_rowmajor_kernel<<<blocks_for(n * (kvp / 4)), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      pairs, kv, kvp, n, out);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

extern "C" int spc_native_to_tables(const int32_t* pair, int kv, int64_t n_pair, int inverse,
                                    int32_t* pair_fwd, int64_t n_out, int32_t* pair_bwd, int64_t n_in,
                                    void* stream) {
  if (!pair || !pair_fwd || kv <= 0 || n_pair < 0 || n_out < 0 || n_in < 0)
    return fail(SPC_ERR_INVALID_ARGUMENT, "native_to_tables: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_out > 0) SPC_CUDA_OK(cudaMemsetAsync(pair_fwd, 0xFF, static_cast<size_t>(kv) * n_out * 4, st));
  if (pair_bwd && n_in > 0) SPC_CUDA_OK(cudaMemsetAsync(pair_bwd, 0xFF, static_cast<size_t>(kv) * n_in * 4, st));
  if (n_pair == 0) return SPC_OK;
  const int32_t* pair_in = pair + static_cast<int64_t>(inverse ? 1 : 0) * kv * n_pair;
  const int32_t* pair_out = pair + static_cast<int64_t>(inverse ? 0 : 1) * kv * n_pair;
  dim3 grid(blocks_for(n_pair), static_cast<unsigned>(kv));
  native_to_tables_kernel<<<grid, kThreads, 0, st>>>(pair_in, pair_out, kv, n_pair, pair_fwd, n_out, pair_bwd, n_in);
  SPC_LAUNCH_OK();
  return SPC_OK;
}
