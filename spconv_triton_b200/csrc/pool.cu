// Sparse max / average pooling over implicit-gemm pair tables.
//
// HBM-bound gather-reduce.  pool_group_kernel: an output row is owned by a group
// of 4..32 lanes, each holding up to four 16-byte channel vectors; the group
// reads 32 table entries of the row with one round of loads, a ballot per load
// builds the presence mask and the lanes walk only the set bits (the entry is
// passed around by shuffle), with the gathers of two rows in flight and the
// table entries of the next row group fetched ahead.  pool_compact_kernel
// (entries compacted per CTA in shared memory, one thread per 16-byte vector)
// takes the channel counts the group shape cannot.
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

// Whole-vector conversions.  The 16-bit types convert two lanes per instruction
// on the FMA pipe; one-lane conversions issue on the quarter-rate XU pipe, which
// made the gather-reduce instruction-bound.
template <typename T, int VEC>
__device__ __forceinline__ void unpack(const Pack<T, VEC>& p, typename PoolAcc<T>::type (&out)[VEC]) {
#pragma unroll
  for (int v = 0; v < VEC; ++v) out[v] = up<T>(p.v[v]);
}
template <>
__device__ __forceinline__ void unpack<__half, 8>(const Pack<__half, 8>& p, float (&out)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(p.v);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 f = __half22float2(h[q]);
    out[2 * q] = f.x;
    out[2 * q + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void unpack<__nv_bfloat16, 8>(const Pack<__nv_bfloat16, 8>& p, float (&out)[8]) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(p.v);
#pragma unroll
  for (int q = 0; q < 4; ++q) {  // bf16 is the upper half of an fp32
    out[2 * q] = __uint_as_float(w[q] << 16);
    out[2 * q + 1] = __uint_as_float(w[q] & 0xffff0000u);
  }
}

template <typename T, int VEC>
__device__ __forceinline__ Pack<T, VEC> pack(const typename PoolAcc<T>::type (&in)[VEC]) {
  Pack<T, VEC> o;
#pragma unroll
  for (int v = 0; v < VEC; ++v) o.v[v] = down<T>(in[v]);
  return o;
}
template <>
__device__ __forceinline__ Pack<__half, 8> pack<__half, 8>(const float (&in)[8]) {
  Pack<__half, 8> o;
  __half2* h = reinterpret_cast<__half2*>(o.v);
#pragma unroll
  for (int q = 0; q < 4; ++q) h[q] = __floats2half2_rn(in[2 * q], in[2 * q + 1]);
  return o;
}
template <>
__device__ __forceinline__ Pack<__nv_bfloat16, 8> pack<__nv_bfloat16, 8>(const float (&in)[8]) {
  Pack<__nv_bfloat16, 8> o;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(o.v);
#pragma unroll
  for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(in[2 * q], in[2 * q + 1]);
  return o;
}

enum PoolOp { kMaxFwd = 0, kAvgFwd = 1, kAvgBwd = 2, kMaxBwd = 3 };
// Independent 16-byte gathers one thread keeps in flight (rows in flight = in_flight / U), and
// 16-byte vectors of a row one thread owns, per operator; each pair is the measured best on B200
// for 512-byte rows (C = 256 fp16): max forward has few present entries per row and gains from
// four rows in flight with two vectors each (0.26 ms = 0.81 of the copy peak, against 0.31 with
// 4 x 2); average forward over a 3^3 window prefers four vectors and one row; max backward
// reads two rows per entry and keeps its own row in registers: one vector and one row per thread
// (more resident threads) is best for it.
template <int OP> struct PoolTune;
template <> struct PoolTune<0> { static constexpr int in_flight = 8, max_u = 2; };  // kMaxFwd
template <> struct PoolTune<1> { static constexpr int in_flight = 4, max_u = 4; };  // kAvgFwd
template <> struct PoolTune<2> { static constexpr int in_flight = 8, max_u = 2; };  // kAvgBwd
template <> struct PoolTune<3> { static constexpr int in_flight = 1, max_u = 1; };  // kMaxBwd
constexpr int kChunk = 32;    // table entries of one row compacted per pass (one per lane)
constexpr int kMaxRows = 64;  // rows per CTA

// What the four operators do with the rows their table names:
//   kMaxFwd : dst[row] = max(0, src[j])                        table = pair_fwd
//   kAvgFwd : dst[row] = sum(src[j]) / max(1, #j), aux_out=#j  table = pair_fwd
//   kMaxBwd : dst[row] = sum(src[o] where own[row]==ref[o])    table = pair_bwd, src = grad_out, ref = pooled
//   kAvgBwd : dst[row] = sum(src[o] * aux_in[o])               table = pair_bwd, src = grad_out
//
// One thread owns U 16-byte channel vectors of one row, spaced so that the
// threads of a row read contiguous 16*nt bytes per load; a random 512-byte
// row needs several loads in flight per thread to cover HBM latency, and the
// table walk is paid once per U vectors.
template <typename T, int VEC, int U, int OP>
struct PoolRow {
  using A = typename PoolAcc<T>::type;
  A acc[U][VEC];
  Pack<T, VEC> f[U];
  int total = 0;

  __device__ __forceinline__ void begin(const T* own, long long row, int channels, int c0, int cstep) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[u][v] = A(0);
      if (OP == kMaxBwd) f[u] = load_pack<T, VEC>(own + row * channels + c0 + u * cstep);
    }
  }

  // B rows at once (entries < 0 are skipped); B * U loads are issued before the first use.
  template <int B>
  __device__ __forceinline__ void gather(const int (&j)[B], const T* src, const T* ref, const int32_t* aux_in,
                                         int channels, int c0, int cstep) {
    Pack<T, VEC> pk[B][U], rk[B][U];
    A w[B];
#pragma unroll
    for (int b = 0; b < B; ++b) {
      if (j[b] < 0) continue;
      const long long off = static_cast<long long>(j[b]) * channels + c0;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        pk[b][u] = load_pack<T, VEC>(src + off + u * cstep);
        if (OP == kMaxBwd) rk[b][u] = load_pack<T, VEC>(ref + off + u * cstep);
      }
      if (OP == kAvgBwd) w[b] = static_cast<A>(__ldg(&aux_in[j[b]]));
    }
#pragma unroll
    for (int b = 0; b < B; ++b) {
      if (j[b] < 0) continue;
      ++total;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        A x[VEC], r[VEC], o[VEC];
        unpack<T, VEC>(pk[b][u], x);
        if (OP == kMaxBwd) {
          unpack<T, VEC>(rk[b][u], r);
          unpack<T, VEC>(f[u], o);
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          if (OP == kMaxFwd) acc[u][v] = x[v] > acc[u][v] ? x[v] : acc[u][v];
          else if (OP == kAvgFwd) acc[u][v] += x[v];
          else if (OP == kMaxBwd) { if (r[v] == o[v]) acc[u][v] += x[v]; }
          else acc[u][v] += x[v] * w[b];
        }
      }
    }
  }

  __device__ __forceinline__ void finish(T* dst, int32_t* aux_out, long long row, int channels, int c0,
                                         int cstep) {
    const A d = static_cast<A>(total > 1 ? total : 1);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (OP == kAvgFwd) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[u][v] /= d;
      }
      store_pack<T, VEC>(dst + row * channels + c0 + u * cstep, pack<T, VEC>(acc[u]));
    }
    if (OP == kAvgFwd && aux_out != nullptr && c0 == 0) aux_out[row] = total;
  }
};

// Launch geometry of the shared-memory kernel: `nt` threads per row (U vectors
// each), of which a CTA holds `tpb` (grid.y covers the rest), `rpb` rows per CTA.
struct PoolGeom { int nt, tpb, rpb; };

// Rows whose nt threads are a power of two between 4 and 32 (every channel count
// from 128 bytes to 2 KiB that is a multiple of 64 bytes): the nt lanes of a row
// read up to 32 table entries of the row with ONE round of loads (lane l takes
// entries l, l+nt, ...), a ballot per load builds the row's 32-bit presence
// mask, and the lanes then walk only the set bits, fetching each index from its
// owner lane by shuffle.  No shared memory, no CTA barrier.
// Each warp takes kGroupIters consecutive row groups and loads the table entries
// of the next group before it gathers for the current one, so a table latency is
// exposed once per warp and gathers are in flight the rest of the time.
constexpr int kGroupIters = 8;  // row groups per warp

template <typename T, int VEC, int U, int OP, int LGNT>
__global__ void __launch_bounds__(256)
pool_group_kernel(const T* __restrict__ src, const T* __restrict__ own, const T* __restrict__ ref,
                  const int32_t* __restrict__ table, const int32_t* __restrict__ aux_in, T* __restrict__ dst,
                  int32_t* __restrict__ aux_out, long long n_rows, int channels, int kv) {
  // the threads per row are a compile-time power of two: the entry loops below unroll to
  // exactly 32 / nt loads, ballots and selects
  constexpr int lg_nt = LGNT;
  constexpr int kE = 32 >> LGNT;  // table entries per lane per round == rows per warp
  constexpr int B = PoolTune<OP>::in_flight / U > 0 ? PoolTune<OP>::in_flight / U : 1;
  constexpr unsigned kFull = 0xffffffffu;
  constexpr int nt = 1 << lg_nt;
  const int lane = threadIdx.x & 31;
  const int kl = lane & (nt - 1), gbase = lane - kl;
  const unsigned gmask = nt == 32 ? kFull : ((1u << nt) - 1u);
  const int c0 = kl * VEC, cstep = nt * VEC;
  constexpr int per_lane = kE;
  const long long warp_id = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long row_first = warp_id * kGroupIters * per_lane + (lane >> lg_nt);

  auto load_entries = [&](long long row, int k0, int (&v)[kE]) {
#pragma unroll
    for (int e = 0; e < kE; ++e) {
      const int k = k0 + e * nt + kl;
      v[e] = (row < n_rows && e < per_lane && k < kv) ? __ldg(&table[static_cast<long long>(k) * n_rows + row]) : -1;
    }
  };

  int vn[kE];
  load_entries(row_first, 0, vn);
#pragma unroll 1
  for (int it = 0; it < kGroupIters; ++it) {
    const long long row = row_first + static_cast<long long>(it) * per_lane;
    if (row - (lane >> lg_nt) >= n_rows) break;  // warp-uniform: the whole group is past the end
    const bool live = row < n_rows;
    int v[kE];
#pragma unroll
    for (int e = 0; e < kE; ++e) v[e] = vn[e];
    if (it + 1 < kGroupIters) load_entries(row + per_lane, 0, vn);

    PoolRow<T, VEC, U, OP> pr;
    if (live) pr.begin(own, row, channels, c0, cstep);
    for (int k0 = 0; k0 < kv; k0 += 32) {
      if (k0 != 0) load_entries(row, k0, v);
      unsigned gm = 0;
#pragma unroll
      for (int e = 0; e < kE; ++e) {
        if (e < per_lane) {  // warp-uniform
          const unsigned m = __ballot_sync(kFull, v[e] >= 0);
          gm |= ((m >> gbase) & gmask) << (e * nt);
        }
      }
      while (__any_sync(kFull, gm != 0)) {
        int j[B];
#pragma unroll
        for (int b = 0; b < B; ++b) {
          const int p = gm ? __ffs(gm) - 1 : 0;
          const int e = p >> lg_nt;
          int mine = v[0];
#pragma unroll
          for (int q = 1; q < kE; ++q) mine = e == q ? v[q] : mine;
          const int got = __shfl_sync(kFull, mine, gbase + (p & (nt - 1)));
          j[b] = gm ? got : -1;
          gm &= gm - 1;
        }
        pr.template gather<B>(j, src, ref, aux_in, channels, c0, cstep);
      }
    }
    if (live) pr.finish(dst, aux_out, row, channels, c0, cstep);
  }
}

// Every other channel count.  Tables are mostly -1 (a 3^3 stride-1 pool over a
// LiDAR scene has about 3 of 27 entries present), so walking them per thread costs
// far more instructions than the gathers.  The CTA stages the [kv, rpb] tile of the
// table with coalesced loads, one warp per row compacts the entries that are
// present with a ballot (order of k preserved, so sums are formed in the same
// order as a plain walk), and every thread then reads only the compacted list.
template <typename T, int VEC, int U, int OP>
__global__ void __launch_bounds__(256)
pool_compact_kernel(const T* __restrict__ src, const T* __restrict__ own, const T* __restrict__ ref,
                    const int32_t* __restrict__ table, const int32_t* __restrict__ aux_in, T* __restrict__ dst,
                    int32_t* __restrict__ aux_out, long long n_rows, int channels, int kv, PoolGeom g) {
  constexpr int B = PoolTune<OP>::in_flight / U > 0 ? PoolTune<OP>::in_flight / U : 1;
  __shared__ int32_t tab[kChunk][kMaxRows + 1];
  __shared__ int32_t lst[kMaxRows][kChunk];
  __shared__ int32_t cnt[kMaxRows];
  const int t = threadIdx.x, nthr = blockDim.x;
  const int lane = t & 31, warp = t >> 5, nwarps = nthr >> 5;
  const long long row0 = static_cast<long long>(blockIdx.x) * g.rpb;
  const int rl = t / g.tpb;
  const int ct = t - rl * g.tpb + static_cast<int>(blockIdx.y) * g.tpb;
  const long long row = row0 + rl;
  const bool live = rl < g.rpb && row < n_rows && ct < g.nt;
  const int c0 = ct * VEC, cstep = g.nt * VEC;

  PoolRow<T, VEC, U, OP> pr;
  if (live) pr.begin(own, row, channels, c0, cstep);

  for (int k0 = 0; k0 < kv; k0 += kChunk) {
    const int kc = min(kChunk, kv - k0);
    if (k0 != 0) __syncthreads();
    for (int i = t; i < kc * g.rpb; i += nthr) {
      const int k = i / g.rpb, r = i - k * g.rpb;
      const long long rr = row0 + r;
      tab[k][r] = rr < n_rows ? __ldg(&table[static_cast<long long>(k0 + k) * n_rows + rr]) : -1;
    }
    __syncthreads();
    for (int r = warp; r < g.rpb; r += nwarps) {
      const int v = lane < kc ? tab[lane][r] : -1;
      const unsigned m = __ballot_sync(0xffffffffu, v >= 0);
      if (v >= 0) lst[r][__popc(m & ((1u << lane) - 1u))] = v;
      if (lane == 0) cnt[r] = __popc(m);
    }
    __syncthreads();
    if (!live) continue;
    const int n = cnt[rl];
    for (int i = 0; i < n; i += B) {
      int j[B];
#pragma unroll
      for (int b = 0; b < B; ++b) j[b] = i + b < n ? lst[rl][i + b] : -1;
      pr.template gather<B>(j, src, ref, aux_in, channels, c0, cstep);
    }
  }
  if (live) pr.finish(dst, aux_out, row, channels, c0, cstep);
}

template <typename T>
int vec_for(int channels, const void* a, const void* b, const void* c = nullptr, const void* d = nullptr) {
  constexpr int full = 16 / sizeof(T);
  auto aligned = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (channels % full == 0 && aligned(a) && aligned(b) && aligned(c) && aligned(d)) return full;
  return 1;
}

template <typename T, int VEC, int U, int OP>
void pool_launch_u(const T* src, const T* own, const T* ref, const int32_t* table, const int32_t* aux_in, T* dst,
                   int32_t* aux_out, int64_t n_rows, int channels, int kv, cudaStream_t st) {
  PoolGeom g;
  g.nt = channels / (VEC * U);
  g.tpb = std::min(g.nt, 256);
  g.rpb = std::min(kMaxRows, std::max(1, 256 / g.tpb));
  const int threads = static_cast<int>(ceil_div(static_cast<long long>(g.tpb) * g.rpb, 32) * 32);
  const dim3 grid(static_cast<unsigned>(ceil_div(static_cast<long long>(n_rows), g.rpb)),
                  static_cast<unsigned>(ceil_div(g.nt, g.tpb)));
  if (g.nt >= 4 && g.nt <= 32 && (g.nt & (g.nt - 1)) == 0) {
    int lg = 0;
    while ((1 << lg) < g.nt) ++lg;
    const long long warps = ceil_div(static_cast<long long>(n_rows), (32 >> lg) * kGroupIters);
    const unsigned blocks = static_cast<unsigned>(ceil_div(warps, 8));
    switch (lg) {
      case 2: pool_group_kernel<T, VEC, U, OP, 2><<<blocks, 256, 0, st>>>(src, own, ref, table, aux_in, dst, aux_out, n_rows, channels, kv); break;
      case 3: pool_group_kernel<T, VEC, U, OP, 3><<<blocks, 256, 0, st>>>(src, own, ref, table, aux_in, dst, aux_out, n_rows, channels, kv); break;
      case 4: pool_group_kernel<T, VEC, U, OP, 4><<<blocks, 256, 0, st>>>(src, own, ref, table, aux_in, dst, aux_out, n_rows, channels, kv); break;
      default: pool_group_kernel<T, VEC, U, OP, 5><<<blocks, 256, 0, st>>>(src, own, ref, table, aux_in, dst, aux_out, n_rows, channels, kv); break;
    }
  } else {
    pool_compact_kernel<T, VEC, U, OP><<<grid, threads, 0, st>>>(src, own, ref, table, aux_in, dst, aux_out,
                                                                n_rows, channels, kv, g);
  }
}

template <typename T, int OP>
int pool_launch(const void* src_, const void* own_, const void* ref_, const int32_t* table,
                const int32_t* aux_in, void* dst_, int32_t* aux_out, int64_t n_rows, int channels, int kv,
                cudaStream_t st) {
  constexpr int full = 16 / sizeof(T);
  const T* src = static_cast<const T*>(src_);
  const T* own = static_cast<const T*>(own_);
  const T* ref = static_cast<const T*>(ref_);
  T* dst = static_cast<T*>(dst_);
  if (vec_for<T>(channels, src_, own_, ref_, dst_) != full) {
    pool_launch_u<T, 1, 1, OP>(src, own, ref, table, aux_in, dst, aux_out, n_rows, channels, kv, st);
  } else {
    // most vectors per thread that still leave a row at least 4 threads (the warp-group kernel)
    const int tpr = channels / full;
    int u = PoolTune<OP>::max_u;
    while (u > 1 && (tpr % u != 0 || tpr / u < 4)) u /= 2;
    if (u == 4)
      pool_launch_u<T, full, 4, OP>(src, own, ref, table, aux_in, dst, aux_out, n_rows, channels, kv, st);
    else if (u == 2)
      pool_launch_u<T, full, 2, OP>(src, own, ref, table, aux_in, dst, aux_out, n_rows, channels, kv, st);
    else
      pool_launch_u<T, full, 1, OP>(src, own, ref, table, aux_in, dst, aux_out, n_rows, channels, kv, st);
  }
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
  SPC_POOL_DISPATCH(dtype, (pool_launch<T, kMaxFwd>(features, nullptr, nullptr, pair_fwd, nullptr, out, nullptr, n_out, channels, kv, st)));
}

extern "C" int spc_avgpool_forward(const void* features, const int32_t* pair_fwd, void* out, int32_t* count,
                                   int64_t n_out, int channels, int kv, int dtype, void* stream) {
  if (!pool_args_ok(features, pair_fwd, out, n_out, channels, kv))
    return fail(SPC_ERR_INVALID_ARGUMENT, "avgpool_forward: bad arguments");
  if (n_out == 0) return SPC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SPC_POOL_DISPATCH(dtype, (pool_launch<T, kAvgFwd>(features, nullptr, nullptr, pair_fwd, nullptr, out, count, n_out, channels, kv, st)));
}

extern "C" int spc_maxpool_backward(const void* features, const void* out_features, const void* grad_out,
                                    const int32_t* pair_bwd, void* din, int64_t n_in, int channels, int kv,
                                    int dtype, void* stream) {
  if (!pool_args_ok(features, pair_bwd, din, n_in, channels, kv) || !out_features || !grad_out)
    return fail(SPC_ERR_INVALID_ARGUMENT, "maxpool_backward: bad arguments");
  if (n_in == 0) return SPC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SPC_POOL_DISPATCH(dtype, (pool_launch<T, kMaxBwd>(grad_out, features, out_features, pair_bwd, nullptr, din, nullptr, n_in, channels, kv, st)));
}

extern "C" int spc_avgpool_backward(const void* grad_out, const int32_t* pair_bwd, const int32_t* count,
                                    void* din, int64_t n_in, int channels, int kv, int dtype, void* stream) {
  if (!pool_args_ok(grad_out, pair_bwd, din, n_in, channels, kv) || !count)
    return fail(SPC_ERR_INVALID_ARGUMENT, "avgpool_backward: bad arguments");
  if (n_in == 0) return SPC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SPC_POOL_DISPATCH(dtype, (pool_launch<T, kAvgBwd>(grad_out, nullptr, nullptr, pair_bwd, count, din, nullptr, n_in, channels, kv, st)));
}
