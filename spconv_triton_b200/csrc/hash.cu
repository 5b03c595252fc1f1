// Fixed-capacity key -> value hash table on the GPU, and the row scatter-add that
// the misaligned sparse add is made of.
//
// Replaces spconv_triton/pytorch/hash.py:15-110 (HashTable: sorted arrays +
// searchsorted, re-sorted with torch.sort / unique_consecutive on every insert)
// and the table traffic of sparse_add_hash_based
// (spconv_triton/pytorch/functional.py:429-490).  Same observable behaviour:
//   * a key inserted twice keeps the value of the LAST occurrence;
//   * assign_arange_ numbers the stored keys in ascending key order;
//   * items() lists the pairs in ascending key order.
// Here the table is open addressing with linear probing over int64 keys
// (int32 keys are widened on load): insert / query / update are one kernel
// each with no sort; only items / assign_arange sort, and only the stored keys.
//
// Memory of a table with `cap` slots (cap a power of two), one caller-owned buffer:
//   keys  [cap] int64   (kEmptyKey = INT64_MIN marks a free slot)
//   vals  [cap] 8 bytes (the value's bits, zero-extended)
//   stamp [cap] uint64  ((epoch << 40) | index of the writer within its call)
//   counters [2] int64  (stored keys, keys dropped because no slot was free)
// All HBM/L2-bound pointer chasing: algorithmic bytes per key = key + value + one
// 8-byte slot probe and one 8-byte value access.
#include <algorithm>

#include <cub/cub.cuh>

#include "common.cuh"

namespace spc {
namespace {

constexpr int kHashThreads = 256;
constexpr long long kEmptyKey = static_cast<long long>(0x8000000000000000ull);

struct HashView {
  long long* keys;
  unsigned long long* vals;
  unsigned long long* stamp;
  long long* counters;
  unsigned long long mask;
};

inline size_t hash_bytes(int64_t cap) { return static_cast<size_t>(cap) * 24 + 16; }

inline HashView view_of(void* table, int64_t cap) {
  HashView v;
  char* p = static_cast<char*>(table);
  v.keys = reinterpret_cast<long long*>(p);
  v.vals = reinterpret_cast<unsigned long long*>(p + static_cast<size_t>(cap) * 8);
  v.stamp = reinterpret_cast<unsigned long long*>(p + static_cast<size_t>(cap) * 16);
  v.counters = reinterpret_cast<long long*>(p + static_cast<size_t>(cap) * 24);
  v.mask = static_cast<unsigned long long>(cap - 1);
  return v;
}

__device__ __forceinline__ unsigned long long mix(long long key) {
  unsigned long long x = static_cast<unsigned long long>(key);
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdull;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ull;
  x ^= x >> 33;
  return x;
}

__device__ __forceinline__ long long load_key(const void* keys, int key_bytes, long long i) {
  return key_bytes == 4 ? static_cast<long long>(static_cast<const int32_t*>(keys)[i])
                        : static_cast<const long long*>(keys)[i];
}

__device__ __forceinline__ unsigned long long load_val(const void* vals, int val_bytes, long long i) {
  switch (val_bytes) {
    case 1: return static_cast<const uint8_t*>(vals)[i];
    case 2: return static_cast<const uint16_t*>(vals)[i];
    case 4: return static_cast<const uint32_t*>(vals)[i];
    default: return static_cast<const unsigned long long*>(vals)[i];
  }
}

__device__ __forceinline__ void store_val(void* vals, int val_bytes, long long i, unsigned long long v) {
  switch (val_bytes) {
    case 1: static_cast<uint8_t*>(vals)[i] = static_cast<uint8_t>(v); break;
    case 2: static_cast<uint16_t*>(vals)[i] = static_cast<uint16_t>(v); break;
    case 4: static_cast<uint32_t*>(vals)[i] = static_cast<uint32_t>(v); break;
    default: static_cast<unsigned long long*>(vals)[i] = v;
  }
}

// Slot of `key`, or -1.  Bounded: at most one pass over the table.
__device__ __forceinline__ long long find_slot(const HashView& t, long long key) {
  unsigned long long s = mix(key) & t.mask;
  for (unsigned long long probe = 0; probe <= t.mask; ++probe) {
    const long long k = t.keys[s];
    if (k == key) return static_cast<long long>(s);
    if (k == kEmptyKey) return -1;
    s = (s + 1) & t.mask;
  }
  return -1;
}

__global__ void __launch_bounds__(kHashThreads) hash_clear_kernel(HashView t) {
  for (unsigned long long s = static_cast<unsigned long long>(blockIdx.x) * kHashThreads + threadIdx.x; s <= t.mask;
       s += static_cast<unsigned long long>(gridDim.x) * kHashThreads)
    t.keys[s] = kEmptyKey;
}

// Pass 1 of insert: claims a slot per distinct key and leaves, per slot, the
// stamp of the last occurrence of its key in this call.
__global__ void __launch_bounds__(kHashThreads)
hash_claim_kernel(HashView t, const void* __restrict__ keys, int key_bytes, long long n, unsigned long long epoch) {
  const long long i = static_cast<long long>(blockIdx.x) * kHashThreads + threadIdx.x;
  const long long key = i < n ? load_key(keys, key_bytes, i) : kEmptyKey;
  int outcome = 0;  // 1: claimed a free slot, 2: no slot left
  if (key != kEmptyKey) {
    const unsigned long long stamp = (epoch << 40) | static_cast<unsigned long long>(i);
    unsigned long long s = mix(key) & t.mask;
    outcome = 2;
    for (unsigned long long probe = 0; probe <= t.mask; ++probe) {
      long long k = t.keys[s];
      bool fresh = false;
      if (k == kEmptyKey) {
        k = static_cast<long long>(atomicCAS(reinterpret_cast<unsigned long long*>(&t.keys[s]),
                                             static_cast<unsigned long long>(kEmptyKey),
                                             static_cast<unsigned long long>(key)));
        if (k == kEmptyKey) {
          fresh = true;
          k = key;
        }
      }
      if (k == key) {
        atomicMax(&t.stamp[s], stamp);
        outcome = fresh ? 1 : 0;
        break;
      }
      s = (s + 1) & t.mask;
    }
  }
  // one atomic per warp on the two counters instead of one per key
  const unsigned claimed = __ballot_sync(0xffffffffu, outcome == 1);
  const unsigned dropped = __ballot_sync(0xffffffffu, outcome == 2);
  if ((threadIdx.x & 31) == 0) {
    if (claimed) atomicAdd(reinterpret_cast<unsigned long long*>(&t.counters[0]), static_cast<unsigned long long>(__popc(claimed)));
    if (dropped) atomicAdd(reinterpret_cast<unsigned long long*>(&t.counters[1]), static_cast<unsigned long long>(__popc(dropped)));
  }
}

// Pass 2 of insert: the occurrence whose stamp won writes its value.
__global__ void __launch_bounds__(kHashThreads)
hash_write_kernel(HashView t, const void* __restrict__ keys, int key_bytes, const void* __restrict__ values,
                  int val_bytes, long long n, unsigned long long epoch) {
  const long long i = static_cast<long long>(blockIdx.x) * kHashThreads + threadIdx.x;
  if (i >= n) return;
  const long long key = load_key(keys, key_bytes, i);
  if (key == kEmptyKey) return;
  const long long s = find_slot(t, key);
  if (s < 0) return;
  if (t.stamp[s] == ((epoch << 40) | static_cast<unsigned long long>(i)))
    t.vals[s] = values != nullptr ? load_val(values, val_bytes, i) : 0ull;
}

__global__ void __launch_bounds__(kHashThreads)
hash_query_kernel(HashView t, const void* __restrict__ keys, int key_bytes, long long n, void* __restrict__ out,
                  int val_bytes, uint8_t* __restrict__ is_empty) {
  const long long i = static_cast<long long>(blockIdx.x) * kHashThreads + threadIdx.x;
  if (i >= n) return;
  const long long key = load_key(keys, key_bytes, i);
  const long long s = key == kEmptyKey ? -1 : find_slot(t, key);
  store_val(out, val_bytes, i, s >= 0 ? t.vals[s] : 0ull);
  is_empty[i] = s < 0;
}

// insert_exist_keys: overwrites the value of keys that are stored, reports which were.
__global__ void __launch_bounds__(kHashThreads)
hash_update_kernel(HashView t, const void* __restrict__ keys, int key_bytes, const void* __restrict__ values,
                   int val_bytes, long long n, uint8_t* __restrict__ found) {
  const long long i = static_cast<long long>(blockIdx.x) * kHashThreads + threadIdx.x;
  if (i >= n) return;
  const long long key = load_key(keys, key_bytes, i);
  const long long s = key == kEmptyKey ? -1 : find_slot(t, key);
  if (s >= 0) t.vals[s] = load_val(values, val_bytes, i);
  found[i] = s >= 0;
}

// Lists the occupied slots (any order; the sort that follows orders them by key).
__global__ void __launch_bounds__(kHashThreads)
hash_dump_kernel(HashView t, long long limit, unsigned long long* __restrict__ cursor,
                 long long* __restrict__ dump_keys, uint32_t* __restrict__ dump_slots) {
  // one atomic on the cursor per CTA: warp ballots, then a prefix over the CTA's eight warps
  __shared__ unsigned int warp_count[kHashThreads / 32];
  __shared__ unsigned long long cta_base;
  const unsigned long long s = static_cast<unsigned long long>(blockIdx.x) * kHashThreads + threadIdx.x;
  const long long k = s <= t.mask ? t.keys[s] : kEmptyKey;
  const unsigned used = __ballot_sync(0xffffffffu, k != kEmptyKey);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) warp_count[warp] = __popc(used);
  __syncthreads();
  unsigned before = 0, total = 0;
#pragma unroll
  for (int w = 0; w < kHashThreads / 32; ++w) {
    const unsigned c = warp_count[w];
    before += w < warp ? c : 0u;
    total += c;
  }
  if (threadIdx.x == 0 && total > 0) cta_base = atomicAdd(cursor, static_cast<unsigned long long>(total));
  __syncthreads();
  if (k == kEmptyKey) return;
  const unsigned long long pos = cta_base + before + __popc(used & ((1u << lane) - 1u));
  if (static_cast<long long>(pos) < limit) {
    dump_keys[pos] = k;
    dump_slots[pos] = static_cast<uint32_t>(s);
  }
}

// assign_kind: -1 keep the values; 0 / 1 / 2 store the rank as integer / float / double.
__global__ void __launch_bounds__(kHashThreads)
hash_emit_kernel(HashView t, const long long* __restrict__ sorted_keys, const uint32_t* __restrict__ sorted_slots,
                 long long count, int assign_kind, void* __restrict__ out_keys, int key_bytes,
                 void* __restrict__ out_vals, int val_bytes, long long out_limit) {
  const long long r = static_cast<long long>(blockIdx.x) * kHashThreads + threadIdx.x;
  if (r >= count) return;
  const uint32_t s = sorted_slots[r];
  unsigned long long v;
  if (assign_kind < 0) {
    v = t.vals[s];
  } else {
    if (assign_kind == 0) v = static_cast<unsigned long long>(r);
    else if (assign_kind == 1) v = __float_as_uint(static_cast<float>(r));
    else v = static_cast<unsigned long long>(__double_as_longlong(static_cast<double>(r)));
    t.vals[s] = v;
  }
  if (r < out_limit) {
    if (out_keys != nullptr) {
      if (key_bytes == 4) static_cast<int32_t*>(out_keys)[r] = static_cast<int32_t>(sorted_keys[r]);
      else static_cast<long long*>(out_keys)[r] = sorted_keys[r];
    }
    if (out_vals != nullptr) store_val(out_vals, val_bytes, r, v);
  }
}

struct ItemsLayout {
  size_t off_cursor, off_keys, off_slots, off_skeys, off_sslots, off_cub, cub_bytes, total;
};

ItemsLayout items_layout(int64_t count) {
  ItemsLayout L;
  const size_t n = static_cast<size_t>(count > 0 ? count : 1);
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
  L.off_cursor = take(16);
  L.off_keys = take(n * 8);
  L.off_slots = take(n * 4);
  L.off_skeys = take(n * 8);
  L.off_sslots = take(n * 4);
  L.cub_bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, L.cub_bytes, static_cast<long long*>(nullptr), static_cast<long long*>(nullptr),
                                  static_cast<uint32_t*>(nullptr), static_cast<uint32_t*>(nullptr), static_cast<int>(n));
  L.off_cub = take(L.cub_bytes);
  L.total = off;
  return L;
}

template <typename T> struct AddOp {
  static __device__ __forceinline__ T add(T a, T b) { return a + b; }
};
template <> struct AddOp<__half> {
  static __device__ __forceinline__ __half add(__half a, __half b) { return __hadd(a, b); }
};
template <> struct AddOp<__nv_bfloat16> {
  static __device__ __forceinline__ __nv_bfloat16 add(__nv_bfloat16 a, __nv_bfloat16 b) { return __hadd(a, b); }
};

// GATHER = false: dst[rows[i], :] += src[i, :] (rows are distinct within a call, so no atomics);
// GATHER = true:  dst[i, :] = src[rows[i], :].  One thread moves VEC elements (16 bytes when VEC > 1).
template <typename T, int VEC, bool GATHER>
__global__ void __launch_bounds__(kHashThreads)
rows_add_kernel(const T* __restrict__ src, const int32_t* __restrict__ rows, long long n, int channels,
                long long dst_rows, T* __restrict__ dst) {
  const int per_row = channels / VEC;
  const long long total = n * per_row;
  for (long long e = static_cast<long long>(blockIdx.x) * kHashThreads + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * kHashThreads) {
    const long long i = e / per_row;
    const int c = static_cast<int>(e - i * per_row) * VEC;
    const long long r = __ldg(&rows[i]);
    if (r < 0 || r >= dst_rows) continue;
    struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
    if (GATHER) {
      *reinterpret_cast<Pack*>(&dst[i * channels + c]) = *reinterpret_cast<const Pack*>(&src[r * channels + c]);
    } else {
      const Pack a = *reinterpret_cast<const Pack*>(&src[i * channels + c]);
      Pack b = *reinterpret_cast<Pack*>(&dst[r * channels + c]);
#pragma unroll
      for (int j = 0; j < VEC; ++j) b.v[j] = AddOp<T>::add(b.v[j], a.v[j]);
      *reinterpret_cast<Pack*>(&dst[r * channels + c]) = b;
    }
  }
}

template <typename T, bool GATHER>
int rows_add_typed(const void* src, const int32_t* rows, int64_t n, int channels, int64_t dst_rows, void* dst,
                   cudaStream_t st) {
  constexpr int kVec = 16 / sizeof(T);
  const bool vec = channels % kVec == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(dst) % 16 == 0;
  const int64_t work = n * (vec ? channels / kVec : channels);
  const int blocks = static_cast<int>(std::min<int64_t>(ceil_div(work, kHashThreads), static_cast<int64_t>(sm_count()) * 32));
  if (vec)
    rows_add_kernel<T, kVec, GATHER><<<blocks, kHashThreads, 0, st>>>(
        static_cast<const T*>(src), rows, n, channels, dst_rows, static_cast<T*>(dst));
  else
    rows_add_kernel<T, 1, GATHER><<<blocks, kHashThreads, 0, st>>>(
        static_cast<const T*>(src), rows, n, channels, dst_rows, static_cast<T*>(dst));
  SPC_LAUNCH_OK();
  return SPC_OK;
}

struct KeyShape {
  int width;
  long long stride[8];
};

// keys[i] = sum_d indices[i, d] * stride[d]: the row-major linear coordinate over [batch, *spatial].
__global__ void __launch_bounds__(kHashThreads)
coords_to_keys_kernel(const __grid_constant__ KeyShape g, const int32_t* __restrict__ indices, long long n,
                      void* __restrict__ keys, int key_bytes) {
  const long long i = static_cast<long long>(blockIdx.x) * kHashThreads + threadIdx.x;
  if (i >= n) return;
  long long lin = 0;
  for (int d = 0; d < g.width; ++d) lin += g.stride[d] * __ldg(&indices[i * g.width + d]);
  if (key_bytes == 4) static_cast<int32_t*>(keys)[i] = static_cast<int32_t>(lin);
  else static_cast<long long*>(keys)[i] = lin;
}

// idx_dst[rows[i], :] = idx_src[i, :]: the coordinates that go with scattered feature rows.
__global__ void __launch_bounds__(kHashThreads)
rows_index_kernel(const int32_t* __restrict__ rows, long long n, long long dst_rows, const int32_t* __restrict__ idx_src,
                  int idx_width, int32_t* __restrict__ idx_dst) {
  const long long e = static_cast<long long>(blockIdx.x) * kHashThreads + threadIdx.x;
  if (e >= n * idx_width) return;
  const long long i = e / idx_width;
  const int d = static_cast<int>(e - i * idx_width);
  const long long r = __ldg(&rows[i]);
  if (r >= 0 && r < dst_rows) idx_dst[r * idx_width + d] = __ldg(&idx_src[e]);
}

bool bad_bytes(int b) { return b != 1 && b != 2 && b != 4 && b != 8; }
bool bad_cap(int64_t cap) { return cap < 2 || (cap & (cap - 1)) != 0 || cap > (1ll << 32); }

template <bool GATHER>
int rows_dispatch(const void* src, const int32_t* rows, int64_t n, int channels, int dtype, int64_t dst_rows,
                  void* dst, cudaStream_t st) {
  switch (dtype) {
    case SPC_F16: return rows_add_typed<__half, GATHER>(src, rows, n, channels, dst_rows, dst, st);
    case SPC_BF16: return rows_add_typed<__nv_bfloat16, GATHER>(src, rows, n, channels, dst_rows, dst, st);
    case SPC_F32: return rows_add_typed<float, GATHER>(src, rows, n, channels, dst_rows, dst, st);
    case SPC_F64: return rows_add_typed<double, GATHER>(src, rows, n, channels, dst_rows, dst, st);
    default: return fail(SPC_ERR_INVALID_ARGUMENT, "rows: unknown dtype %d", dtype);
  }
}

}  // namespace
}  // namespace spc

using namespace spc;

extern "C" size_t spc_hash_bytes(int64_t capacity) { return bad_cap(capacity) ? 0 : hash_bytes(capacity); }

extern "C" int spc_hash_clear(void* table, int64_t capacity, void* stream) {
  if (table == nullptr || bad_cap(capacity)) return fail(SPC_ERR_INVALID_ARGUMENT, "hash_clear: bad table");
  auto st = static_cast<cudaStream_t>(stream);
  HashView t = view_of(table, capacity);
  SPC_CUDA_OK(cudaMemsetAsync(t.vals, 0, hash_bytes(capacity) - static_cast<size_t>(capacity) * 8, st));
  hash_clear_kernel<<<static_cast<int>(std::min<int64_t>(ceil_div(capacity, kHashThreads), sm_count() * 16)),
                      kHashThreads, 0, st>>>(t);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

extern "C" int spc_hash_insert(void* table, int64_t capacity, const void* keys, int key_bytes, const void* values,
                               int val_bytes, int64_t n, uint64_t epoch, void* stream) {
  if (table == nullptr || bad_cap(capacity) || (key_bytes != 4 && key_bytes != 8) || bad_bytes(val_bytes) || n < 0 ||
      n >= (1ll << 40))
    return fail(SPC_ERR_INVALID_ARGUMENT, "hash_insert: bad argument");
  if (n == 0) return SPC_OK;
  auto st = static_cast<cudaStream_t>(stream);
  HashView t = view_of(table, capacity);
  const int blocks = static_cast<int>(ceil_div(n, kHashThreads));
  hash_claim_kernel<<<blocks, kHashThreads, 0, st>>>(t, keys, key_bytes, n, epoch);
  SPC_LAUNCH_OK();
  hash_write_kernel<<<blocks, kHashThreads, 0, st>>>(t, keys, key_bytes, values, val_bytes, n, epoch);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

extern "C" int spc_hash_counters(const void* table, int64_t capacity, int64_t* stored, int64_t* dropped, void* stream) {
  if (table == nullptr || bad_cap(capacity)) return fail(SPC_ERR_INVALID_ARGUMENT, "hash_counters: bad table");
  auto st = static_cast<cudaStream_t>(stream);
  int64_t host[2] = {0, 0};
  SPC_CUDA_OK(cudaMemcpyAsync(host, view_of(const_cast<void*>(table), capacity).counters, 16, cudaMemcpyDeviceToHost, st));
  SPC_CUDA_OK(cudaStreamSynchronize(st));
  if (stored != nullptr) *stored = host[0];
  if (dropped != nullptr) *dropped = host[1];
  return SPC_OK;
}

extern "C" int spc_hash_query(const void* table, int64_t capacity, const void* keys, int key_bytes, int64_t n,
                              void* out_values, int val_bytes, uint8_t* is_empty, void* stream) {
  if (table == nullptr || bad_cap(capacity) || (key_bytes != 4 && key_bytes != 8) || bad_bytes(val_bytes) || n < 0)
    return fail(SPC_ERR_INVALID_ARGUMENT, "hash_query: bad argument");
  if (n == 0) return SPC_OK;
  hash_query_kernel<<<static_cast<int>(ceil_div(n, kHashThreads)), kHashThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      view_of(const_cast<void*>(table), capacity), keys, key_bytes, n, out_values, val_bytes, is_empty);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

extern "C" int spc_hash_update(void* table, int64_t capacity, const void* keys, int key_bytes, const void* values,
                               int val_bytes, int64_t n, uint8_t* found, void* stream) {
  if (table == nullptr || bad_cap(capacity) || (key_bytes != 4 && key_bytes != 8) || bad_bytes(val_bytes) || n < 0 ||
      values == nullptr)
    return fail(SPC_ERR_INVALID_ARGUMENT, "hash_update: bad argument");
  if (n == 0) return SPC_OK;
  hash_update_kernel<<<static_cast<int>(ceil_div(n, kHashThreads)), kHashThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      view_of(table, capacity), keys, key_bytes, values, val_bytes, n, found);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

extern "C" size_t spc_hash_items_workspace_bytes(int64_t count) { return items_layout(count).total; }

extern "C" int spc_hash_items(void* table, int64_t capacity, int64_t count, int assign_kind, int key_bits, void* ws,
                              size_t ws_bytes, void* out_keys, int key_bytes, void* out_values, int val_bytes,
                              int64_t out_limit, void* stream) {
  if (table == nullptr || bad_cap(capacity) || count < 0 || count > capacity || assign_kind < -1 || assign_kind > 2 ||
      (key_bytes != 4 && key_bytes != 8) || bad_bytes(val_bytes))
    return fail(SPC_ERR_INVALID_ARGUMENT, "hash_items: bad argument");
  if (count == 0) return SPC_OK;
  const ItemsLayout L = items_layout(count);
  if (ws == nullptr || ws_bytes < L.total)
    return fail(SPC_ERR_WORKSPACE_TOO_SMALL, "hash_items: workspace %zu < %zu", ws_bytes, L.total);
  auto st = static_cast<cudaStream_t>(stream);
  char* w = static_cast<char*>(ws);
  HashView t = view_of(table, capacity);
  auto* cursor = reinterpret_cast<unsigned long long*>(w + L.off_cursor);
  auto* dkeys = reinterpret_cast<long long*>(w + L.off_keys);
  auto* dslots = reinterpret_cast<uint32_t*>(w + L.off_slots);
  auto* skeys = reinterpret_cast<long long*>(w + L.off_skeys);
  auto* sslots = reinterpret_cast<uint32_t*>(w + L.off_sslots);
  SPC_CUDA_OK(cudaMemsetAsync(cursor, 0, 16, st));
  hash_dump_kernel<<<static_cast<int>(ceil_div(capacity, kHashThreads)), kHashThreads, 0, st>>>(t, count, cursor, dkeys, dslots);
  SPC_LAUNCH_OK();
  size_t cub_bytes = L.cub_bytes;
  SPC_CUDA_OK(cub::DeviceRadixSort::SortPairs(w + L.off_cub, cub_bytes, dkeys, skeys, dslots, sslots,
                                              static_cast<int>(count), 0, (key_bits > 0 && key_bits < 64) ? key_bits : 64, st));
  note_launch();
  hash_emit_kernel<<<static_cast<int>(ceil_div(count, kHashThreads)), kHashThreads, 0, st>>>(
      t, skeys, sslots, count, assign_kind, out_keys, key_bytes, out_values, val_bytes, out_limit);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

extern "C" int spc_coords_to_keys(const int32_t* indices, int64_t n, int width, const int64_t* shape, int key_bytes,
                                  void* keys, void* stream) {
  if (n < 0 || width < 1 || width > 8 || shape == nullptr || (key_bytes != 4 && key_bytes != 8))
    return fail(SPC_ERR_INVALID_ARGUMENT, "coords_to_keys: bad argument");
  if (n == 0) return SPC_OK;
  KeyShape g;
  g.width = width;
  long long stride = 1;
  for (int d = width - 1; d >= 0; --d) {
    g.stride[d] = stride;
    stride *= shape[d];
  }
  coords_to_keys_kernel<<<static_cast<int>(ceil_div(n, kHashThreads)), kHashThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      g, indices, n, keys, key_bytes);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

extern "C" int spc_rows_scatter_add(const void* src, const int32_t* rows, int64_t n, int channels, int dtype,
                                    int64_t dst_rows, void* dst, const int32_t* idx_src, int idx_width,
                                    int32_t* idx_dst, void* stream) {
  if (n < 0 || channels < 0 || dst_rows < 0) return fail(SPC_ERR_INVALID_ARGUMENT, "rows_scatter_add: bad size");
  if (n == 0) return SPC_OK;
  auto st = static_cast<cudaStream_t>(stream);
  if (channels > 0) {
    const int rc = rows_dispatch<false>(src, rows, n, channels, dtype, dst_rows, dst, st);
    if (rc != SPC_OK) return rc;
  }
  if (idx_src != nullptr && idx_width > 0) {
    rows_index_kernel<<<static_cast<int>(ceil_div(n * idx_width, kHashThreads)), kHashThreads, 0, st>>>(
        rows, n, dst_rows, idx_src, idx_width, idx_dst);
    SPC_LAUNCH_OK();
  }
  return SPC_OK;
}

extern "C" int spc_rows_gather(const void* src, const int32_t* rows, int64_t n, int channels, int dtype,
                               int64_t src_rows, void* dst, void* stream) {
  if (n < 0 || channels < 0 || src_rows < 0) return fail(SPC_ERR_INVALID_ARGUMENT, "rows_gather: bad size");
  if (n == 0 || channels == 0) return SPC_OK;
  return rows_dispatch<true>(src, rows, n, channels, dtype, src_rows, dst, static_cast<cudaStream_t>(stream));
}
