// CUDA-core implicit gather-GEMM: forward, input gradient and weight gradient.
//
// These kernels carry the fp32 IEEE path (Blackwell tensor cores have no IEEE
// fp32 mode; the reference's default fp32 arithmetic is IEEE,
// spconv_triton/pytorch/_impl/gemm.py:11-13) and every 16-bit shape the tcgen05
// kernels do not take (channel counts that are not multiples of 16).  They
// accumulate in fp32 with fused multiply-add.
//
// Forward and input gradient are one kernel with different weight strides,
// as in the reference (spconv_triton/pytorch/_impl/gemm.py:541-567,604-630).  A tile of
// BM output rows loops over the kernel offsets; offsets with no contributing
// row in the tile are skipped after one block-wide vote, which is the
// reference's tile-bitmask trick (gemm.py:282-296) without needing the mask
// words, so it also works for kernel volumes above 32.
#include <algorithm>
#include <atomic>

#include "common.cuh"
#include "gemm_internal.cuh"

namespace spc {
namespace {

template <typename T>
struct AccOf { using type = float; };

template <typename A, typename T>
__device__ __forceinline__ A to_acc(T v) { return static_cast<A>(to_float(v)); }

template <typename T, typename A>
__device__ __forceinline__ T from_acc(A v) { return from_float<T>(static_cast<float>(v)); }

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
constexpr int kGemmThreads = (BM / TM) * (BN / TN);  // 256

// out[rm, n] = sum_k sum_r src[pairs[k, rm], r] * w[n*s_wn + k*s_wk + r*s_wr] (+ bias[n])
template <typename T, typename TO>
__global__ void __launch_bounds__(kGemmThreads)
gather_gemm_simt_kernel(const T* __restrict__ src, const T* __restrict__ w, const Epilogue epi,
                        const int32_t* __restrict__ pairs, const int32_t* __restrict__ order,
                        TO* __restrict__ out, long long m_rows, int n_dim, int r_dim, int kv,
                        long long s_wk, long long s_wr, long long s_wn) {
  using A = typename AccOf<T>::type;
  __shared__ A As[BK][BM + 4];
  __shared__ A Bs[BK][BN + 4];
  __shared__ long long rows_s[BM];
  __shared__ int idx_s[BM];

  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const long long m0 = static_cast<long long>(blockIdx.x) * BM;
  const int n0 = blockIdx.y * BN;

  if (tid < BM) {
    const long long slot = m0 + tid;
    rows_s[tid] = slot < m_rows ? (order ? static_cast<long long>(order[slot]) : slot) : -1;
  }
  __syncthreads();

  A acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = A(0);

  for (int k = 0; k < kv; ++k) {
    int mine = -1;
    if (tid < BM && rows_s[tid] >= 0) mine = __ldg(&pairs[static_cast<long long>(k) * m_rows + rows_s[tid]]);
    if (tid < BM) idx_s[tid] = mine;
    if (!__syncthreads_or(mine >= 0)) continue;
    for (int r0 = 0; r0 < r_dim; r0 += BK) {
      // A tile: BM x BK, thread loads 4 consecutive reduction channels of one row.
      {
        const int row = tid / (BK / 4), c4 = (tid % (BK / 4)) * 4;
        const int j = idx_s[row];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int r = r0 + c4 + u;
          A v = A(0);
          if (j >= 0 && r < r_dim) v = to_acc<A>(src[static_cast<long long>(j) * r_dim + r]);
          As[c4 + u][row] = v;
        }
      }
      // B tile: BK x BN.
      {
        const int n = tid / (BK / 4), c4 = (tid % (BK / 4)) * 4;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int r = r0 + c4 + u;
          A v = A(0);
          if (n0 + n < n_dim && r < r_dim) v = to_acc<A>(w[(n0 + n) * s_wn + k * s_wk + r * s_wr]);
          Bs[c4 + u][n] = v;
        }
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) {
        A a[TM], b[TN];
#pragma unroll
        for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
        for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) acc[i][j] += a[i] * b[j];
      }
      __syncthreads();
    }
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const long long rm = rows_s[ty * TM + i];
    if (rm < 0) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= n_dim) continue;
      float v = apply_epilogue<T>(acc[i][j], epi, n);
      if (epi.residual != nullptr) v += to_float(static_cast<const TO*>(epi.residual)[rm * n_dim + n]);
      out[rm * n_dim + n] = from_acc<TO>(v);
    }
  }
}

// Weight gradient partial sums.  grid.x = kv * splits, grid.y tiles c_in,
// grid.z tiles c_out.  Each block walks its chunk of pair_fwd[k, :], compacts
// the rows that exist into shared lists with warp ballots, and accumulates
// g[o,:]^T f[i,:] over them.
constexpr int WP = 16;  // pairs per accumulation step

template <typename T>
__global__ void __launch_bounds__(kGemmThreads)
wgrad_simt_kernel(const T* __restrict__ feats, const T* __restrict__ gout,
                  const int32_t* __restrict__ pair_fwd, float* __restrict__ partial, long long n_out,
                  int c_in, int c_out, int kv, int splits, long long rows_per_split) {
  using A = typename AccOf<T>::type;
  __shared__ A Gs[WP][BM + 4];  // [pair][out channel]
  __shared__ A Fs[WP][BN + 4];  // [pair][in channel]
  __shared__ int list_i[kGemmThreads];
  __shared__ int list_o[kGemmThreads];
  __shared__ int warp_cnt[kGemmThreads / 32];

  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int k = blockIdx.x / splits, split = blockIdx.x % splits;
  const int c0 = blockIdx.y * BN, n0 = blockIdx.z * BM;
  const long long lo = split * rows_per_split;
  const long long hi = min(n_out, lo + rows_per_split);

  A acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = A(0);

  for (long long base = lo; base < hi; base += kGemmThreads) {
    const long long m = base + tid;
    const int in_row = m < hi ? __ldg(&pair_fwd[static_cast<long long>(k) * n_out + m]) : -1;
    const unsigned ballot = __ballot_sync(0xffffffffu, in_row >= 0);
    const int lane = tid & 31, warp = tid >> 5;
    if (lane == 0) warp_cnt[warp] = __popc(ballot);
    __syncthreads();
    int total = 0, before = 0;
#pragma unroll
    for (int wi = 0; wi < kGemmThreads / 32; ++wi) {
      const int c = warp_cnt[wi];
      if (wi < warp) before += c;
      total += c;
    }
    if (in_row >= 0) {
      const int pos = before + __popc(ballot & ((1u << lane) - 1u));
      list_i[pos] = in_row;
      list_o[pos] = static_cast<int>(m - base);
    }
    __syncthreads();
    for (int p0 = 0; p0 < total; p0 += WP) {
      {
        const int p = tid / 16, ch4 = (tid % 16) * 4;  // 16 pairs x 64 channels
        const bool live = p0 + p < total;
        const long long o = live ? base + list_o[p0 + p] : 0;
        const long long i = live ? list_i[p0 + p] : 0;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int n = n0 + ch4 + u, c = c0 + ch4 + u;
          Gs[p][ch4 + u] = (live && n < c_out) ? to_acc<A>(gout[o * c_out + n]) : A(0);
          Fs[p][ch4 + u] = (live && c < c_in) ? to_acc<A>(feats[i * c_in + c]) : A(0);
        }
      }
      __syncthreads();
#pragma unroll
      for (int pp = 0; pp < WP; ++pp) {
        A a[TM], b[TN];
#pragma unroll
        for (int i = 0; i < TM; ++i) a[i] = Gs[pp][ty * TM + i];
#pragma unroll
        for (int j = 0; j < TN; ++j) b[j] = Fs[pp][tx * TN + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) acc[i][j] += a[i] * b[j];
      }
      __syncthreads();
    }
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int n = n0 + ty * TM + i;
    if (n >= c_out) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int c = c0 + tx * TN + j;
      if (c >= c_in) continue;
      partial[((static_cast<long long>(split) * c_out + n) * kv + k) * c_in + c] = static_cast<float>(acc[i][j]);
    }
  }
}


// Weight gradient of thin layers (c_out * c_in <= 256, e.g. the 4 -> 32 stem of a UNet): the
// 64 x 64 tile of wgrad_simt_kernel would be almost all padding there (measured 8.1 ms for 1.2 M
// rows, 15 % of a training step).  Here a thread owns ONE element dW[n, k, c] of the block's
// offset k; the 256 threads form G = 256 / E groups (E = c_out * c_in rounded up to a power of
// two) that take the existing pairs of a 256-row chunk in turn (pair p goes to group p mod G), so
// every pair costs each thread two small loads and one multiply-add.  Groups are summed in a fixed
// order; partial[split] is then reduced by wgrad_reduce_kernel as for the tiled kernel.
template <typename T>
__global__ void __launch_bounds__(kGemmThreads)
wgrad_thin_kernel(const T* __restrict__ feats, const T* __restrict__ gout, const int32_t* __restrict__ pair_fwd,
                  float* __restrict__ partial, long long n_out, int c_in, int c_out, int kv, int splits,
                  long long rows_per_split, int e_pad) {
  __shared__ int list_i[kGemmThreads];
  __shared__ int list_o[kGemmThreads];
  __shared__ int warp_cnt[kGemmThreads / 32];
  __shared__ float red[kGemmThreads];

  const int tid = threadIdx.x;
  const int k = blockIdx.x / splits, split = blockIdx.x % splits;
  const long long lo = split * rows_per_split;
  const long long hi = min(n_out, lo + rows_per_split);
  const int groups = kGemmThreads / e_pad;
  const int e = tid % e_pad, grp = tid / e_pad;
  const bool owner = e < c_out * c_in;
  const int n = owner ? e / c_in : 0, c = owner ? e % c_in : 0;
  float acc = 0.f;

  for (long long base = lo; base < hi; base += kGemmThreads) {
    const long long m = base + tid;
    const int in_row = m < hi ? __ldg(&pair_fwd[static_cast<long long>(k) * n_out + m]) : -1;
    const unsigned ballot = __ballot_sync(0xffffffffu, in_row >= 0);
    const int lane = tid & 31, warp = tid >> 5;
    if (lane == 0) warp_cnt[warp] = __popc(ballot);
    __syncthreads();
    int total = 0, before = 0;
#pragma unroll
    for (int wi = 0; wi < kGemmThreads / 32; ++wi) {
      const int cnt = warp_cnt[wi];
      if (wi < warp) before += cnt;
      total += cnt;
    }
    if (in_row >= 0) {
      const int pos = before + __popc(ballot & ((1u << lane) - 1u));
      list_i[pos] = in_row;
      list_o[pos] = static_cast<int>(m - base);
    }
    __syncthreads();
    if (owner) {
      int p = grp;
      // The blocks of the offsets most rows have (the in-plane ones of a wall or floor) carry most
      // pairs and run on after the others have left the SM, so what a block's time follows is the
      // number of dependent load round trips: sixteen pairs in flight per thread, then four.
      for (; p + 15 * groups < total; p += 16 * groups) {
        T g[16], f[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int q = p + u * groups;
          g[u] = gout[(base + list_o[q]) * c_out + n];
          f[u] = feats[static_cast<long long>(list_i[q]) * c_in + c];
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) acc = fmaf(to_float(g[u]), to_float(f[u]), acc);
      }
      for (; p + 3 * groups < total; p += 4 * groups) {
        float g[4], f[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int q = p + u * groups;
          g[u] = to_float(gout[(base + list_o[q]) * c_out + n]);
          f[u] = to_float(feats[static_cast<long long>(list_i[q]) * c_in + c]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) acc = fmaf(g[u], f[u], acc);
      }
      for (; p < total; p += groups)
        acc = fmaf(to_float(gout[(base + list_o[p]) * c_out + n]),
                   to_float(feats[static_cast<long long>(list_i[p]) * c_in + c]), acc);
    }
    __syncthreads();  // the lists are rewritten by the next chunk
  }
  red[tid] = acc;
  __syncthreads();
  if (grp == 0 && owner) {
    float sum = 0.f;
    for (int gi = 0; gi < groups; ++gi) sum += red[gi * e_pad + e];
    partial[((static_cast<long long>(split) * c_out + n) * kv + k) * c_in + c] = sum;
  }
}

inline bool wgrad_is_thin(int c_in, int c_out) { return c_in <= 8 && c_in * c_out <= kGemmThreads; }

// Stem layers with four input channels and 16 or 32 output channels: a THREAD takes a pair (and
// 16 of the output channels: PARTS = c_out / 16 thread groups per block walk the same rows).  It
// loads the pair's 8 bytes of features and 32 bytes of output gradient with vector loads and keeps
// its 64 products in registers, so a pair costs three loads in one or two threads instead of two
// loads in each of 64 - 128 threads; two rows are in flight per thread, and the block's sums are
// combined once at the end (warp shuffles, then shared memory, in a fixed order).  16-bit inputs.
template <typename T, int PARTS>
__global__ void __launch_bounds__(kGemmThreads, 2)
wgrad_stem4_kernel(const T* __restrict__ feats, const T* __restrict__ gout, const int32_t* __restrict__ pair_fwd,
                   float* __restrict__ partial, long long n_out, int kv, int splits, long long rows_per_split) {
  constexpr int CIN = 4, NT = 16, COUT = NT * PARTS, GT = kGemmThreads / PARTS;
  static_assert(sizeof(T) == 2, "16-bit inputs");
  __shared__ float red[kGemmThreads / 32][CIN * NT];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int part = tid / GT, gt = tid % GT;
  const int k = blockIdx.x / splits, split = blockIdx.x % splits;
  const long long lo = split * rows_per_split;
  const long long hi = min(n_out, lo + rows_per_split);
  float acc[NT][CIN];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int c = 0; c < CIN; ++c) acc[n][c] = 0.f;
  const int32_t* col = pair_fwd + static_cast<long long>(k) * n_out;
  const T* gcol = gout + part * NT;
  for (long long m0 = lo + gt; m0 < hi; m0 += 2 * GT) {
    const long long m1 = m0 + GT;
    const int r0 = __ldg(col + m0);
    const int r1 = m1 < hi ? __ldg(col + m1) : -1;
    uint2 f0 = make_uint2(0u, 0u), f1 = make_uint2(0u, 0u);
    uint4 g0[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
    uint4 g1[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
    if (r0 >= 0) {
      f0 = __ldg(reinterpret_cast<const uint2*>(feats + static_cast<long long>(r0) * CIN));
      g0[0] = __ldg(reinterpret_cast<const uint4*>(gcol + m0 * COUT));
      g0[1] = __ldg(reinterpret_cast<const uint4*>(gcol + m0 * COUT) + 1);
    }
    if (r1 >= 0) {
      f1 = __ldg(reinterpret_cast<const uint2*>(feats + static_cast<long long>(r1) * CIN));
      g1[0] = __ldg(reinterpret_cast<const uint4*>(gcol + m1 * COUT));
      g1[1] = __ldg(reinterpret_cast<const uint4*>(gcol + m1 * COUT) + 1);
    }
    // an absent pair contributes zeros (its registers were cleared), in the same row order as a
    // thread that walks one row at a time
    {
      const T* fh = reinterpret_cast<const T*>(&f0);
      const T* gh = reinterpret_cast<const T*>(g0);
      if (r0 >= 0) {
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const float g = to_float(gh[n]);
#pragma unroll
          for (int c = 0; c < CIN; ++c) acc[n][c] = fmaf(g, to_float(fh[c]), acc[n][c]);
        }
      }
    }
    {
      const T* fh = reinterpret_cast<const T*>(&f1);
      const T* gh = reinterpret_cast<const T*>(g1);
      if (r1 >= 0) {
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const float g = to_float(gh[n]);
#pragma unroll
          for (int c = 0; c < CIN; ++c) acc[n][c] = fmaf(g, to_float(fh[c]), acc[n][c]);
        }
      }
    }
  }
  // warps never straddle two parts (GT is a multiple of 32)
  for (int pp = 0; pp < PARTS; ++pp) {
    if (part == pp) {
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int c = 0; c < CIN; ++c) {
          float v = acc[n][c];
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
          if (lane == 0) red[warp][n * CIN + c] = v;
        }
    }
    __syncthreads();
    if (tid < CIN * NT) {
      float sum = 0.f;
      for (int w = pp * (GT / 32); w < (pp + 1) * (GT / 32); ++w) sum += red[w][tid];
      const int n = pp * NT + tid / CIN, c = tid % CIN;
      partial[((static_cast<long long>(split) * COUT + n) * kv + k) * CIN + c] = sum;
    }
    __syncthreads();
  }
}

inline bool wgrad_is_stem4(int c_in, int c_out, int dtype) {
  return c_in == 4 && (c_out == 16 || c_out == 32) && (dtype == SPC_F16 || dtype == SPC_BF16);
}

template <typename T>
__global__ void __launch_bounds__(256)
wgrad_reduce_kernel(const float* __restrict__ partial, T* __restrict__ dw, long long elems, int splits) {
  const long long e = blockIdx.x * 256ll + threadIdx.x;
  if (e >= elems) return;
  float s = 0.f;
  for (int sp = 0; sp < splits; ++sp) s += partial[sp * elems + e];
  dw[e] = from_acc<T, float>(s);
}

// Thin layers (the 4 -> 16 stem of a LiDAR backbone): a 64x64x16 tile would be three quarters
// padding in two dimensions.  Here one thread owns one output row and all of its n_dim <= NP
// outputs in registers; the whole weight tensor sits in shared memory as fp32 [kv][r_dim][NP] and
// is read as broadcasts; the table column pairs[k, row] is read coalesced.  Same sums in the same
// offset order as the tiled kernel (fp32 accumulation).
constexpr int kThinThreads = 128;

template <typename T, typename TO, int NP>
__global__ void __launch_bounds__(kThinThreads)
gather_gemm_thin_kernel(const T* __restrict__ src, const T* __restrict__ w, const Epilogue epi,
                        const int32_t* __restrict__ pairs, TO* __restrict__ out, long long m_rows, int n_dim,
                        int r_dim, int kv, long long s_wk, long long s_wr, long long s_wn) {
  extern __shared__ float w_s[];  // [kv][r_dim][NP]
  for (int i = threadIdx.x; i < kv * r_dim * NP; i += kThinThreads) {
    const int n = i % NP, r = (i / NP) % r_dim, k = i / (NP * r_dim);
    w_s[i] = n < n_dim ? to_float(w[n * s_wn + k * s_wk + r * s_wr]) : 0.f;
  }
  __syncthreads();
  const long long row = static_cast<long long>(blockIdx.x) * kThinThreads + threadIdx.x;
  if (row >= m_rows) return;
  float acc[NP];
#pragma unroll
  for (int n = 0; n < NP; ++n) acc[n] = 0.f;
  int j_next = __ldg(&pairs[row]);
  for (int k = 0; k < kv; ++k) {
    const int j = j_next;
    if (k + 1 < kv) j_next = __ldg(&pairs[static_cast<long long>(k + 1) * m_rows + row]);
    if (j < 0) continue;
    const T* f = src + static_cast<long long>(j) * r_dim;
    const float* wk = w_s + k * r_dim * NP;
    for (int r = 0; r < r_dim; ++r) {
      const float a = to_float(f[r]);
      const float4* wr = reinterpret_cast<const float4*>(wk + r * NP);
#pragma unroll
      for (int q = 0; q < NP / 4; ++q) {
        const float4 v = wr[q];
        acc[4 * q + 0] += a * v.x;
        acc[4 * q + 1] += a * v.y;
        acc[4 * q + 2] += a * v.z;
        acc[4 * q + 3] += a * v.w;
      }
    }
  }
  TO* o = out + row * n_dim;
#pragma unroll
  for (int n = 0; n < NP; ++n)
    if (n < n_dim) {
      float v = apply_epilogue<T>(acc[n], epi, n);
      if (epi.residual != nullptr) v += to_float(static_cast<const TO*>(epi.residual)[row * n_dim + n]);
      o[n] = from_acc<TO>(v);
    }
}

template <typename T, typename TO>
int launch_thin(const void* src, const void* w, const Epilogue& epi, const int32_t* pairs, void* out,
                long long m_rows, int n_dim, int r_dim, int kv, long long s_wk, long long s_wr, long long s_wn,
                cudaStream_t st) {
  const int np = n_dim <= 8 ? 8 : n_dim <= 16 ? 16 : 32;
  const size_t smem = static_cast<size_t>(kv) * r_dim * np * sizeof(float);
  const unsigned blocks = static_cast<unsigned>(ceil_div(m_rows, kThinThreads));
#define SPC_THIN(NP)                                                                                         \
  gather_gemm_thin_kernel<T, TO, NP><<<blocks, kThinThreads, smem, st>>>(                                    \
      static_cast<const T*>(src), static_cast<const T*>(w), epi, pairs, static_cast<TO*>(out), m_rows, n_dim, \
      r_dim, kv, s_wk, s_wr, s_wn)
  if (np == 8) SPC_THIN(8);
  else if (np == 16) SPC_THIN(16);
  else SPC_THIN(32);
#undef SPC_THIN
  SPC_LAUNCH_OK();
  return SPC_OK;
}

template <typename T, typename TO>
int launch_gather(const void* src, const void* w, const Epilogue& epi, const int32_t* pairs,
                  const int32_t* order, void* out, long long m_rows, int n_dim, int r_dim, int kv,
                  long long s_wk, long long s_wr, long long s_wn, cudaStream_t st) {
  if (r_dim <= 8 && n_dim <= 32 && static_cast<size_t>(kv) * r_dim * 32 * sizeof(float) <= 40 * 1024 && m_rows > 0)
    return launch_thin<T, TO>(src, w, epi, pairs, out, m_rows, n_dim, r_dim, kv, s_wk, s_wr, s_wn, st);
  dim3 grid(static_cast<unsigned>(ceil_div(m_rows, BM)), static_cast<unsigned>(ceil_div(n_dim, BN)));
  gather_gemm_simt_kernel<T, TO><<<grid, kGemmThreads, 0, st>>>(
      static_cast<const T*>(src), static_cast<const T*>(w), epi, pairs, order,
      static_cast<TO*>(out), m_rows, n_dim, r_dim, kv, s_wk, s_wr, s_wn);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

}  // namespace

int gather_gemm_simt(const void* src, const void* w, const Epilogue& epi, const int32_t* pairs,
                     const int32_t* order, void* out, long long m_rows, int n_dim, int r_dim, int kv,
                     long long s_wk, long long s_wr, long long s_wn, int dtype, int out_dtype,
                     cudaStream_t st) {
#define SPC_GG(T, TO) \
  return launch_gather<T, TO>(src, w, epi, pairs, order, out, m_rows, n_dim, r_dim, kv, s_wk, s_wr, s_wn, st)
  if (dtype == SPC_F16 && out_dtype == SPC_F16) SPC_GG(__half, __half);
  if (dtype == SPC_F16 && out_dtype == SPC_F32) SPC_GG(__half, float);
  if (dtype == SPC_BF16 && out_dtype == SPC_BF16) SPC_GG(__nv_bfloat16, __nv_bfloat16);
  if (dtype == SPC_BF16 && out_dtype == SPC_F32) SPC_GG(__nv_bfloat16, float);
  if (dtype == SPC_F32 && out_dtype == SPC_F32) SPC_GG(float, float);
  if (dtype == SPC_F32 && out_dtype == SPC_F16) SPC_GG(float, __half);
#undef SPC_GG
  return fail(SPC_ERR_UNSUPPORTED, "gather-GEMM: dtype %d -> %d not supported", dtype, out_dtype);
}

WgradSplit wgrad_split(int64_t n_out, int c_in, int c_out, int kv) {
  WgradSplit s;
  const int64_t tiles = static_cast<int64_t>(kv) * ceil_div(c_in, BN) * ceil_div(c_out, BM);
  // the thin kernel's blocks are light (one element per thread): eight of them per multiprocessor
  int64_t want = ceil_div((wgrad_is_thin(c_in, c_out) ? 8 : 2) * static_cast<int64_t>(sm_count()),
                          std::max<int64_t>(tiles, 1));
  const int64_t by_len = std::max<int64_t>(1, n_out / 2048);
  want = std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(want, by_len), 64));
  s.splits = static_cast<int>(want);
  s.rows_per_split = ceil_div(std::max<int64_t>(n_out, 1), s.splits);
  s.bytes = static_cast<size_t>(s.splits) * c_out * kv * c_in * sizeof(float);
  return s;
}

int wgrad_reduce(const float* partial, void* dw, long long elems, int splits, int dtype, cudaStream_t st) {
  const unsigned rblocks = static_cast<unsigned>(ceil_div(elems, 256));
  if (dtype == SPC_F16) wgrad_reduce_kernel<__half><<<rblocks, 256, 0, st>>>(partial, static_cast<__half*>(dw), elems, splits);
  else if (dtype == SPC_BF16)
    wgrad_reduce_kernel<__nv_bfloat16><<<rblocks, 256, 0, st>>>(partial, static_cast<__nv_bfloat16*>(dw), elems, splits);
  else if (dtype == SPC_F32) wgrad_reduce_kernel<float><<<rblocks, 256, 0, st>>>(partial, static_cast<float*>(dw), elems, splits);
  else return fail(SPC_ERR_UNSUPPORTED, "wgrad reduce: dtype %d not supported", dtype);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

int wgrad_simt(const void* feats, const void* gout, const int32_t* pair_fwd, void* dw, float* partial,
               int64_t n_out, int c_in, int c_out, int kv, int dtype, cudaStream_t st) {
  const WgradSplit s = wgrad_split(n_out, c_in, c_out, kv);
  dim3 grid(static_cast<unsigned>(kv * s.splits), static_cast<unsigned>(ceil_div(c_in, BN)),
            static_cast<unsigned>(ceil_div(c_out, BM)));
  const long long elems = static_cast<long long>(c_out) * kv * c_in;
  const unsigned rblocks = static_cast<unsigned>(ceil_div(elems, 256));
  const bool thin = wgrad_is_thin(c_in, c_out);
  int e_pad = 1;
  while (e_pad < c_in * c_out) e_pad <<= 1;
  if (wgrad_is_stem4(c_in, c_out, dtype) && (reinterpret_cast<uintptr_t>(feats) & 7u) == 0 &&
      (reinterpret_cast<uintptr_t>(gout) & 15u) == 0) {
    const unsigned blocks = static_cast<unsigned>(kv * s.splits);
#define SPC_STEM(T, N)                                                                                  \
    wgrad_stem4_kernel<T, N><<<blocks, kGemmThreads, 0, st>>>(static_cast<const T*>(feats),            \
                                                               static_cast<const T*>(gout), pair_fwd, partial, \
                                                               n_out, kv, s.splits, s.rows_per_split)
    if (dtype == SPC_F16 && c_out == 16) SPC_STEM(__half, 1);
    else if (dtype == SPC_F16) SPC_STEM(__half, 2);
    else if (c_out == 16) SPC_STEM(__nv_bfloat16, 1);
    else SPC_STEM(__nv_bfloat16, 2);
#undef SPC_STEM
    SPC_LAUNCH_OK();
    return wgrad_reduce(partial, dw, elems, s.splits, dtype, st);
  }
#define SPC_WG(T)                                                                                   \
  do {                                                                                              \
    if (thin)                                                                                       \
      wgrad_thin_kernel<T><<<static_cast<unsigned>(kv * s.splits), kGemmThreads, 0, st>>>(         \
          static_cast<const T*>(feats), static_cast<const T*>(gout), pair_fwd, partial, n_out, c_in, \
          c_out, kv, s.splits, s.rows_per_split, e_pad);                                            \
    else                                                                                            \
      wgrad_simt_kernel<T><<<grid, kGemmThreads, 0, st>>>(static_cast<const T*>(feats),             \
                                                          static_cast<const T*>(gout), pair_fwd,    \
                                                          partial, n_out, c_in, c_out, kv, s.splits, \
                                                          s.rows_per_split);                        \
    SPC_LAUNCH_OK();                                                                                \
    wgrad_reduce_kernel<T><<<rblocks, 256, 0, st>>>(partial, static_cast<T*>(dw), elems, s.splits); \
    SPC_LAUNCH_OK();                                                                                \
    return SPC_OK;                                                                                  \
  } while (0)
  if (dtype == SPC_F16) SPC_WG(__half);
  if (dtype == SPC_BF16) SPC_WG(__nv_bfloat16);
  if (dtype == SPC_F32) SPC_WG(float);
#undef SPC_WG
  return fail(SPC_ERR_UNSUPPORTED, "wgrad: dtype %d not supported", dtype);
}

}  // namespace spc

// ---------------------------------------------------------------------------
// Weight gradient without any workspace from the caller.
//
// Some hosts can give this library nothing but the tensors of the operation
// itself: a C/C++ inference or training runtime that embeds the library as a
// plugin, plans every byte of device memory up front, forbids cudaMalloc from
// plugin code and has no workspace argument in its operator interface.  For
// them the fp32 partial sums of the split reduction live in the fixed array
// below instead of a caller-provided buffer.
//
// The array is part of the library image: every GPU that loads the library
// holds these 16 MiB until the process exits.  All calls on a device share it,
// so two calls that overlap on the GPU (different streams, or graphs launched
// concurrently) race on it; callers must serialise them.  Nothing in it has to
// start at zero: the partial-sum kernel writes every element the reduction
// kernel reads, so contents left by an earlier call are never observed.
// ---------------------------------------------------------------------------
namespace spc {
namespace {

constexpr size_t kNoAllocScratchFloats = size_t(4) << 20;  // 4 Mi floats = 16 MiB
static __device__ __align__(256) float g_wgrad_scratch[kNoAllocScratchFloats];

// In host code `g_wgrad_scratch` is only a handle for the symbol, not an
// address a kernel could use; the device address is looked up once per device
// (with that device current) and remembered.  Two host threads that make the
// first call on a device at the same time both look the address up and store
// the same value (atomic pointer-sized stores), so no lock is taken.
int wgrad_scratch_address(float** out) {
  static std::atomic<float*> per_device[64];
  int dev = 0;
  SPC_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(SPC_ERR_SIZE_LIMIT, "device ordinal %d out of range", dev);
  float* addr = per_device[dev].load(std::memory_order_acquire);
  if (addr == nullptr) {
    void* raw = nullptr;
    SPC_CUDA_OK(cudaGetSymbolAddress(&raw, g_wgrad_scratch));
    addr = static_cast<float*>(raw);
    per_device[dev].store(addr, std::memory_order_release);
  }
  *out = addr;
  return SPC_OK;
}

}  // namespace
}  // namespace spc

extern "C" size_t spc_conv_backward_weight_noalloc_max_bytes(void) {
  return spc::kNoAllocScratchFloats * sizeof(float);
}

extern "C" int spc_conv_backward_weight_noalloc(const void* features, const void* grad_out,
                                                const int32_t* pair_fwd, void* dweight, int64_t n_in,
                                                int64_t n_out, int c_in, int c_out, int kv, int dtype,
                                                void* stream) {
  using namespace spc;
  (void)n_in;
  if (!features || !grad_out || !pair_fwd || !dweight || n_out < 0 || c_in <= 0 || c_out <= 0 || kv <= 0)
    return fail(SPC_ERR_INVALID_ARGUMENT, "conv_backward_weight_noalloc: bad arguments");
  if (dtype != SPC_F16 && dtype != SPC_BF16 && dtype != SPC_F32)
    return fail(SPC_ERR_UNSUPPORTED, "conv_backward_weight_noalloc: dtype %d not supported", dtype);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_out == 0) {
    SPC_CUDA_OK(cudaMemsetAsync(dweight, 0, static_cast<size_t>(c_out) * kv * c_in * dtype_size(dtype), st));
    return SPC_OK;
  }
  const WgradSplit s = wgrad_split(n_out, c_in, c_out, kv);
  if (s.bytes > kNoAllocScratchFloats * sizeof(float))
    return fail(SPC_ERR_SIZE_LIMIT,
                "conv_backward_weight_noalloc: this shape needs %zu bytes of partial sums (%d splits x %d x %d x %d "
                "fp32) but the built-in scratch holds %zu; use spc_conv_backward_weight with a workspace",
                s.bytes, s.splits, c_out, kv, c_in, kNoAllocScratchFloats * sizeof(float));
  float* scratch = nullptr;
  const int rc = wgrad_scratch_address(&scratch);
  if (rc != SPC_OK) return rc;
  return wgrad_simt(features, grad_out, pair_fwd, dweight, scratch, n_out, c_in, c_out, kv, dtype, st);
}
