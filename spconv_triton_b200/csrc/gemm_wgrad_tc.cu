// Weight gradient of the sparse convolution on tcgen05 / TMEM.
//
//   dW[n, k, c] = sum over rows m with pair_fwd[k, m] >= 0 of
//                 grad_out[m, n] * features[pair_fwd[k, m], c]
//
// For one kernel offset k this is a dense contraction D[n, c] = G^T F over the
// list of existing (output row, input row) pairs, with the pairs as the
// reduction dimension.  One CTA owns (offset k, a contiguous range of output
// rows, a block of <= 128 output channels) and keeps D (128 lanes x c_in fp32
// columns) in tensor memory:
//   warps 0-7  scan pair_fwd[k, lo:hi] 256 entries at a time, compact the
//              existing pairs into a shared-memory ring with warp ballots (no
//              host-side nonzero(), unlike spconv_triton/pytorch/_impl/gemm.py:663),
//              and for every 64 pairs copy the 64 grad_out rows and the 64
//              feature rows into a swizzled stage with 16-byte cp.async
//              (completion delivered by cp.async.mbarrier.arrive.noinc)
//   warp 8     issues tcgen05.mma with BOTH operands MN-major: a stage row is
//              one pair and holds its channels contiguously, which is exactly
//              how gathered rows arrive, so nothing is transposed
//   warps 0-3  finally read TMEM and write the fp32 partial tile
//              partial[split, n, k, c]; the partials of the splits are added
//              in a fixed order by the reduction kernel of gemm_simt.cu.
// Rows of the accumulator beyond c_out are computed from whatever the stage
// buffer holds and are never stored.  Every wait is bounded.
#include <algorithm>

#include "common.cuh"
#include "gemm_internal.cuh"
#include "tc_common.cuh"

namespace spc {
namespace {

using namespace tc;

// The number of copy warps is a template parameter: four (160-thread CTAs, three per SM) where a pair
// is at most 384 bytes of rows, eight (two CTAs per SM) for wider rows, which need the copy throughput.
constexpr int kWgMaxIssueWarps = 8;
constexpr int kPairsPerStage = 64;
constexpr int kScanBatch = 4;                        // table entries per thread per scan round
constexpr int kRing = 2048;                          // capacity of the pair list (power of two, > 64 + 1024)

struct WgParams {
  const void* feats;
  const void* gout;
  const int32_t* pair_fwd;
  float* partial;
  long long n_out, rows_per_split;
  int c_in, c_out, kv, splits;
  int g_row_bytes, f_row_bytes;  // swizzle span of the grad_out / feature rows (32, 64 or 128)
  int g_stage_bytes, f_stage_bytes, stages, tmem_cols;
  int* status;
};

__host__ __device__ inline uint32_t wg_layout_type(int row_bytes) {
  return row_bytes == 128 ? 2u : (row_bytes == 64 ? 4u : 6u);
}

// Copies `pieces_per_row` 16-byte pieces of `n_rows` gathered rows into an
// MN-major stage region: column block b of row p lands at
// base + b * (kPairsPerStage * row_bytes) + p * row_bytes (+ swizzle).
template <int ELEM>
__device__ __forceinline__ void copy_rows(uint32_t dst_base, const uint8_t* src, uint32_t src_pitch,
                                          const int* rows, int n_rows, int n_rows_padded, int pieces_per_row,
                                          int row_bytes, int tid, int nthreads) {
  const int per_block = row_bytes / 16;  // 2, 4 or 8
  const uint32_t swz_mask = static_cast<uint32_t>(per_block - 1);
  const int lg_pb = per_block == 8 ? 3 : (per_block == 4 ? 2 : 1);
  const int total = n_rows_padded * pieces_per_row;
  const bool pow2 = (pieces_per_row & (pieces_per_row - 1)) == 0;
  const int lg_ppr = 31 - __clz(pieces_per_row);
  for (int q = tid; q < total; q += nthreads) {
    int p, piece;
    if (pow2) {  // the usual case: no integer division per copy
      p = q >> lg_ppr;
      piece = q & (pieces_per_row - 1);
    } else {
      p = q / pieces_per_row;
      piece = q - p * pieces_per_row;
    }
    const int block = piece >> lg_pb, chunk = piece & (per_block - 1);
    const uint32_t lin = static_cast<uint32_t>(p * row_bytes + chunk * 16);
    const uint32_t off = static_cast<uint32_t>(block * kPairsPerStage * row_bytes) + (lin ^ (((lin >> 7) & swz_mask) << 4));
    const bool live = p < n_rows;
    const uint32_t row = live ? static_cast<uint32_t>(rows[p]) : 0u;
    cp_async16(dst_base + off, src + static_cast<unsigned long long>(row) * src_pitch + piece * 16, live ? 16u : 0u);
  }
}

template <typename T, int W>
__global__ void __maxnreg__(W == 4 ? 96 : 80)
wgrad_tc_kernel(const __grid_constant__ WgParams p) {
  constexpr int kWgIssueWarps = W;
  constexpr int kWgIssueThreads = W * 32;
  constexpr int kWgMmaWarp = W;
  constexpr int kScanEntries = kScanBatch * kWgIssueThreads;
  constexpr int ELEM = sizeof(T);
  constexpr int UMMA_K = 32 / ELEM;  // 16 pairs per MMA

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = p.g_stage_bytes + p.f_stage_bytes;
  uint8_t* stage_base = smem;
  int* ring_m = reinterpret_cast<int*>(smem + static_cast<size_t>(p.stages) * stage_bytes);  // output rows
  int* ring_i = ring_m + kRing;                                                                // input rows
  int* rows_m = ring_i + kRing;            // [stages][64] row lists of the stages in flight
  int* rows_i = rows_m + kMaxStages * kPairsPerStage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(rows_i + kMaxStages * kPairsPerStage);
  StageInfo* info = reinterpret_cast<StageInfo*>(bars + 2 * kMaxStages + 1);
  int* warp_cnt = reinterpret_cast<int*>(info + kMaxStages);  // [kScanBatch][8]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(warp_cnt + kScanBatch * kWgIssueWarps);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  if (*reinterpret_cast<volatile int*>(p.status) != 0) return;
  const int k = blockIdx.x / p.splits, split = blockIdx.x % p.splits;
  const int n0 = blockIdx.y * kTileM;  // first output channel of this CTA
  const long long lo = split * p.rows_per_split;
  const long long hi = min(p.n_out, lo + p.rows_per_split);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = smem_u32(bars + kMaxStages);
  const uint32_t bar_accum = smem_u32(bars + 2 * kMaxStages);

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(bar_full + 8 * s, kWgIssueThreads + 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_accum, 1);
    fence_mbar_init();
  }
  if (warp == kWgMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  int real_stages = 0;
  if (warp < kWgIssueWarps) {
    int stage = 0;
    uint32_t empty_parity = 1;
    bool ok = true;
    int head = 0, tail = 0;  // ring positions (uniform over the 256 threads)
    long long pos = lo;
    const int g_cols = min(kTileM, p.c_out - n0);          // output channels this CTA owns
    const int g_pieces = g_cols * ELEM / 16;
    const int f_pieces = p.c_in * ELEM / 16;
    const uint8_t* g_src = static_cast<const uint8_t*>(p.gout) + static_cast<size_t>(n0) * ELEM;
    const uint8_t* f_src = static_cast<const uint8_t*>(p.feats);
    const uint32_t g_pitch = static_cast<uint32_t>(p.c_out) * ELEM, f_pitch = static_cast<uint32_t>(p.c_in) * ELEM;

    // Table entries are fetched one scan round (1024 entries, four per thread) ahead:
    // the loads of the next round are in flight while the stages of this one are built,
    // so the walk over a sparse table does not pay a memory latency per round.
    const int32_t* table = p.pair_fwd + static_cast<long long>(k) * p.n_out;
    int ahead[kScanBatch];
    auto fetch = [&](long long at) {
#pragma unroll
      for (int j = 0; j < kScanBatch; ++j) {
        const long long m = at + j * kWgIssueThreads + tid;
        ahead[j] = m < hi ? __ldg(&table[m]) : -1;
      }
    };
    fetch(pos);
    while (pos < hi || tail > head) {
      if (tail - head < kPairsPerStage && pos < hi) {
        // ---- append the existing pairs of one scan round to the ring, in table order ----
        int cur[kScanBatch];
        unsigned ballot[kScanBatch];
#pragma unroll
        for (int j = 0; j < kScanBatch; ++j) {
          cur[j] = ahead[j];
          ballot[j] = __ballot_sync(0xffffffffu, cur[j] >= 0);
          if (lane == 0) warp_cnt[j * kWgIssueWarps + warp] = __popc(ballot[j]);
        }
        const long long at = pos;
        pos += kScanEntries;
        if (pos < hi) fetch(pos);
        named_bar_sync(1, kWgIssueThreads);
        int before[kScanBatch];
        int run = 0;
#pragma unroll
        for (int j = 0; j < kScanBatch; ++j) {
#pragma unroll
          for (int w = 0; w < kWgIssueWarps; ++w) {
            if (w == warp) before[j] = run;
            run += warp_cnt[j * kWgIssueWarps + w];
          }
        }
#pragma unroll
        for (int j = 0; j < kScanBatch; ++j) {
          if (cur[j] >= 0) {
            const int slot = (tail + before[j] + __popc(ballot[j] & ((1u << lane) - 1u))) & (kRing - 1);
            ring_m[slot] = static_cast<int>(at + j * kWgIssueThreads + tid);
            ring_i[slot] = cur[j];
          }
        }
        named_bar_sync(1, kWgIssueThreads);
        tail += run;
        continue;
      }
      // ---- one stage: up to 64 pairs from the head of the ring ----
      const int n = min(kPairsPerStage, tail - head);
      const int n_pad = (n + UMMA_K - 1) / UMMA_K * UMMA_K;  // rows the MMAs will read; the tail is zero filled
      ++real_stages;
      if (ok && !mbar_wait(bar_empty + 8 * stage, empty_parity)) ok = false;
      if (ok) {
        // private copy of the stage's row lists (the ring may be overwritten by the next scan)
        int* sm = rows_m + stage * kPairsPerStage;
        int* si = rows_i + stage * kPairsPerStage;
        if (tid < n) {
          sm[tid] = ring_m[(head + tid) & (kRing - 1)];
          si[tid] = ring_i[(head + tid) & (kRing - 1)];
        }
        named_bar_sync(2, kWgIssueThreads);
        const uint32_t g_dst = smem_u32(stage_base + static_cast<size_t>(stage) * stage_bytes);
        const uint32_t f_dst = g_dst + p.g_stage_bytes;
        const uint32_t full = bar_full + 8 * stage;
        copy_rows<ELEM>(g_dst, g_src, g_pitch, sm, n, n_pad, g_pieces, p.g_row_bytes, tid, kWgIssueThreads);
        copy_rows<ELEM>(f_dst, f_src, f_pitch, si, n, n_pad, f_pieces, p.f_row_bytes, tid, kWgIssueThreads);
        cp_async_arrive_noinc(full);
        if (tid == 0) {
          info[stage].ksteps = n_pad / UMMA_K;
          info[stage].last = 0;
          mbar_arrive(full);
        }
        if (++stage == p.stages) {
          stage = 0;
          empty_parity ^= 1;
        }
      } else {
        named_bar_sync(2, kWgIssueThreads);
      }
      head += n;
    }
    // terminator
    if (ok && !mbar_wait(bar_empty + 8 * stage, empty_parity)) ok = false;
    if (ok) {
      mbar_arrive(bar_full + 8 * stage);
      if (tid == 0) {
        info[stage].ksteps = 0;
        info[stage].last = 1;
        mbar_arrive(bar_full + 8 * stage);
      }
    } else {
      atomicExch(p.status, SPC_ERR_DEVICE_WAIT_EXPIRED);
    }
    cp_async_wait_all();

    // ---------------- epilogue (warps 0-3): fp32 partial tile ----------------
    if (warp < 4) {
      bool have_acc = mbar_wait(bar_accum, 0);
      if (!have_acc) atomicExch(p.status, SPC_ERR_DEVICE_WAIT_EXPIRED);
      have_acc = __all_sync(0xffffffffu, have_acc);
      tc_fence_after();
      if (have_acc) {
        const int n = n0 + tid;  // output channel held by this TMEM lane
        float* dst = p.partial + ((static_cast<long long>(split) * p.c_out + (n < p.c_out ? n : 0)) * p.kv + k) * p.c_in;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
        for (int c0 = 0; c0 < p.c_in; c0 += 16) {
          float v[16];
          if (real_stages > 0) {
            uint32_t raw[16];
            tmem_ld16(lane_addr + c0, raw);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 16; ++q) v[q] = __uint_as_float(raw[q]);
          } else {
#pragma unroll
            for (int q = 0; q < 16; ++q) v[q] = 0.f;
          }
          if (n < p.c_out) store_row16<float>(dst + c0, v);
        }
      }
      tc_fence_before();
    }
  } else {
    // ---------------- MMA issuer ----------------
    // This one thread paces the CTA: the loop keeps running descriptor words (a stage advance
    // is one add to the address field) and unrolls the four 16-pair steps of a stage.
    if (lane == 0) {
      // fp32 accumulate, both operands MN-major, M = 128, N = c_in
      const uint32_t idesc = (1u << 4) | (TcType<T>::fmt << 7) | (TcType<T>::fmt << 10) | (1u << 15) | (1u << 16) |
                             (static_cast<uint32_t>(p.c_in >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
      const uint32_t g_type = wg_layout_type(p.g_row_bytes), f_type = wg_layout_type(p.f_row_bytes);
      const uint32_t g_addr0 = smem_u32(stage_base);
      const uint64_t a_desc0 = make_desc(g_addr0, kPairsPerStage * p.g_row_bytes, 8 * p.g_row_bytes, g_type);
      const uint64_t b_desc0 = make_desc(g_addr0 + p.g_stage_bytes, kPairsPerStage * p.f_row_bytes, 8 * p.f_row_bytes, f_type);
      const uint32_t a_hi = static_cast<uint32_t>(a_desc0 >> 32), b_hi = static_cast<uint32_t>(b_desc0 >> 32);
      const uint32_t a_lo0 = static_cast<uint32_t>(a_desc0), b_lo0 = static_cast<uint32_t>(b_desc0);
      const uint32_t stage_step = static_cast<uint32_t>(stage_bytes >> 4);
      const uint32_t a_step = static_cast<uint32_t>(UMMA_K * p.g_row_bytes / 16);
      const uint32_t b_step = static_cast<uint32_t>(UMMA_K * p.f_row_bytes / 16);
      const uint32_t info0 = smem_u32(info);
      uint32_t a_lo = a_lo0, b_lo = b_lo0, full = bar_full, empty = bar_empty, inf = info0;
      int stage = 0;
      uint32_t full_parity = 0, accumulate = 0;
      bool ok = true;
      while (true) {
        if (!mbar_wait(full, full_parity)) {
          ok = false;
          break;
        }
        fence_proxy_async();  // stage was written by cp.async (generic proxy)
        tc_fence_after();
        uint32_t ksteps;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(ksteps) : "r"(inf) : "memory");
        if (ksteps == 0) {  // terminator
          tc_commit(bar_accum);
          break;
        }
#pragma unroll
        for (int ks = 0; ks < kPairsPerStage / UMMA_K; ++ks) {
          if (static_cast<uint32_t>(ks) < ksteps) {
            const uint64_t a_desc = (static_cast<uint64_t>(a_hi) << 32) | (a_lo + a_step * ks);
            const uint64_t b_desc = (static_cast<uint64_t>(b_hi) << 32) | (b_lo + b_step * ks);
            tc_mma<false>(tmem_base, a_desc, b_desc, idesc, accumulate);
            accumulate = 1;
          }
        }
        tc_commit(empty);
        a_lo += stage_step;
        b_lo += stage_step;
        full += 8;
        empty += 8;
        inf += static_cast<uint32_t>(sizeof(StageInfo));
        if (++stage == p.stages) {
          stage = 0;
          full_parity ^= 1;
          a_lo = a_lo0;
          b_lo = b_lo0;
          full = bar_full;
          empty = bar_empty;
          inf = info0;
        }
      }
      if (!ok) {
        atomicExch(p.status, SPC_ERR_DEVICE_WAIT_EXPIRED);
        mbar_arrive(bar_accum);
      }
    }
    __syncwarp();
  }

  __syncthreads();
  if (warp == kWgMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

int span_of(int elems, int elem_size) {
  const int bytes = elems * elem_size;
  if (bytes == 32 || bytes == 64) return bytes;
  if (bytes >= 128 && bytes % 128 == 0) return 128;
  return 0;
}

template <typename T, int W>
int launch_wgrad_tc(const WgParams& p, size_t smem_bytes, cudaStream_t st) {
  static bool configured[kMaxDevices] = {false};  // per instantiation and device
  SPC_CUDA_OK(ensure_dynamic_smem(wgrad_tc_kernel<T, W>, 200 * 1024, configured));
  dim3 grid(static_cast<unsigned>(p.kv * p.splits), static_cast<unsigned>(ceil_div(p.c_out, kTileM)));
  wgrad_tc_kernel<T, W><<<grid, W * 32 + 32, smem_bytes, st>>>(p);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

}  // namespace

bool wgrad_tc_supported(int c_in, int c_out, int kv, int dtype) {
  (void)kv;
  if (dtype != SPC_F16 && dtype != SPC_BF16) return false;
  if (c_in < 16 || c_in > 256 || c_in % 16 != 0 || c_out < 16 || c_out % 16 != 0) return false;
  // a CTA's slice of grad_out columns must also fit a swizzle span
  const int g_cols = std::min(c_out, tc::kTileM);
  if (c_out > tc::kTileM && c_out % tc::kTileM != 0) return false;
  return span_of(c_in, 2) != 0 && span_of(g_cols, 2) != 0;
}

// Split of the row range; same formula family as the CUDA-core kernel, with the
// tensor-core tile (128 output channels x all input channels per CTA).
WgradSplit wgrad_tc_split(int64_t n_out, int c_in, int c_out, int kv) {
  WgradSplit s;
  const int64_t tiles = static_cast<int64_t>(kv) * ceil_div(c_out, tc::kTileM);
  // several CTAs per resident slot: offsets differ a lot in how many pairs they have (the centre
  // offset of a submanifold layer has all of them), and surplus CTAs even that out
  int64_t want = ceil_div(16 * static_cast<int64_t>(sm_count()), std::max<int64_t>(tiles, 1));
  const int64_t by_len = std::max<int64_t>(1, n_out / 4096);
  want = std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(want, by_len), 64));
  s.splits = static_cast<int>(want);
  s.rows_per_split = ceil_div(std::max<int64_t>(n_out, 1), s.splits);
  s.bytes = static_cast<size_t>(s.splits) * c_out * kv * c_in * sizeof(float);
  return s;
}

int wgrad_tc(const void* feats, const void* gout, const int32_t* pair_fwd, float* partial, int64_t n_out, int c_in,
             int c_out, int kv, int dtype, const WgradSplit& split, cudaStream_t st) {
  if (!wgrad_tc_supported(c_in, c_out, kv, dtype)) return fail(SPC_ERR_UNSUPPORTED, "tcgen05 wgrad: unsupported shape");
  if ((reinterpret_cast<uintptr_t>(feats) | reinterpret_cast<uintptr_t>(gout) | reinterpret_cast<uintptr_t>(partial)) & 15u)
    return fail(SPC_ERR_UNSUPPORTED, "tcgen05 wgrad: operands must be 16-byte aligned");
  WgParams p{};
  p.feats = feats; p.gout = gout; p.pair_fwd = pair_fwd; p.partial = partial;
  p.n_out = n_out; p.rows_per_split = split.rows_per_split; p.splits = split.splits;
  p.c_in = c_in; p.c_out = c_out; p.kv = kv;
  const int g_cols = std::min(c_out, tc::kTileM);
  p.g_row_bytes = span_of(g_cols, 2);
  p.f_row_bytes = span_of(c_in, 2);
  // the A region always spans 128 channels (M = 128); columns beyond c_out hold stale data
  p.g_stage_bytes = static_cast<int>(align_up(static_cast<size_t>(tc::kTileM) * 2 * kPairsPerStage, 1024));
  p.f_stage_bytes = static_cast<int>(align_up(static_cast<size_t>(c_in) * 2 * kPairsPerStage, 1024));
  const int stage_bytes = p.g_stage_bytes + p.f_stage_bytes;
  const size_t fixed = 1024 + 2 * kRing * 4 + 2 * tc::kMaxStages * kPairsPerStage * 4 + (2 * tc::kMaxStages + 1) * 8 +
                       tc::kMaxStages * sizeof(tc::StageInfo) + kScanBatch * kWgMaxIssueWarps * 4 + 64;
  const bool narrow = (c_in + g_cols) * 2 <= 384;  // bytes of rows per pair
  const size_t budget = narrow ? 74 * 1024 : 110 * 1024;  // three / two CTAs per SM
  p.stages = std::max(2, std::min<int>(tc::kMaxStages, static_cast<int>((budget - fixed) / stage_bytes)));
  const size_t smem_bytes = fixed + static_cast<size_t>(p.stages) * stage_bytes;
  int cols = 32;
  while (cols < c_in) cols <<= 1;
  p.tmem_cols = cols;
  p.status = device_status_ptr();
  if (p.status == nullptr) return fail(SPC_ERR_CUDA, "tcgen05 wgrad: no device status word");
  if (narrow) {
    if (dtype == SPC_F16) return launch_wgrad_tc<__half, 4>(p, smem_bytes, st);
    return launch_wgrad_tc<__nv_bfloat16, 4>(p, smem_bytes, st);
  }
  if (dtype == SPC_F16) return launch_wgrad_tc<__half, 8>(p, smem_bytes, st);
  return launch_wgrad_tc<__nv_bfloat16, 8>(p, smem_bytes, st);
}

}  // namespace spc
