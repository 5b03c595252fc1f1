// Implicit gather-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   out[rm, n] = sum_k sum_r src[pairs[k, rm], r] * B_k[r, n]  (+ bias[n])
//
// used for the forward pass (B_k[r, n] = W[n, k, r]) and, with the weight read
// "transposed", for the input gradient (B_k[r, n] = W[r, k, n]).
//
// One CTA owns a tile of 128 output rows (taken in mask-sorted order when the
// caller passes the rulebook's argsort, so the rows of a tile share their
// active offsets).  The accumulator, 128 lanes x N fp32 columns, lives in
// tensor memory.  Warp roles:
//   warps 0-3  producers: vote on which kernel offsets have any row in the
//              tile, then for every active (offset, reduction chunk) gather
//              the 128 feature rows and the weight slab into a 128-byte-
//              swizzled shared-memory stage with 16-byte cp.async (zero fill
//              for absent rows, completion delivered to the stage's mbarrier by
//              cp.async.mbarrier.arrive.noinc, so nobody waits for a copy);
//              afterwards they are the epilogue warps that
//              read TMEM with tcgen05.ld, add the bias and store the rows
//   warp 4     one elected lane issues tcgen05.mma (kind::f16 / kind::tf32,
//              fp32 accumulate) for each filled stage and releases the stage
//              with tcgen05.commit
// Stages are handed over through mbarriers.  Every wait is bounded: if one
// expires the kernel records SPC_ERR_DEVICE_WAIT_EXPIRED in a device status
// word, drains its copies, frees its tensor memory and returns.
//
// Shared-memory operand layouts (canonical UMMA layouts, 128-byte swizzle):
//   A (gathered rows) and forward B: K-major; row = 128 bytes of the reduction
//     dimension; 8-row groups 1024 bytes apart (SBO); one MMA reads 32 bytes
//     of every row, so the descriptor advances by 32 bytes per K step.
//   input-gradient B: MN-major; row = one reduction index holding 128 bytes
//     of output channels; column blocks LBO apart, 8-row groups 1024 bytes
//     apart (SBO); the descriptor advances by UMMA_K rows per K step.
#include <algorithm>

#include "common.cuh"
#include "gemm_internal.cuh"
#include "tc_common.cuh"

namespace spc {

__device__ int g_device_status = 0;

namespace {

using namespace tc;

struct TcParams {
  const void* src;
  const void* w;
  Epilogue epi;
  const int32_t* pairs;
  const int32_t* order;
  void* out;
  long long m_rows;
  int n_dim, r_dim, kv;
  int stages, b_stage_bytes, tmem_cols;
  int* status;
};

template <typename T, typename TO, bool B_MN>
__global__ void __launch_bounds__(kThreadsTc, 1)
gather_gemm_tc_kernel(const __grid_constant__ TcParams p) {
  constexpr int ELEM = sizeof(T);
  constexpr int EPR = kRowBytes / ELEM;   // elements per 128-byte row
  constexpr int UMMA_K = 32 / ELEM;       // reduction elements per MMA
  constexpr int EP16 = 16 / ELEM;         // elements per 16-byte piece
  constexpr bool TF32 = TcType<T>::tf32;

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled stages
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = kAStageBytes + p.b_stage_bytes;
  uint8_t* stage_base = smem;
  int* idx_s = reinterpret_cast<int*>(smem + static_cast<size_t>(p.stages) * stage_bytes);  // [kGroup][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(idx_s + kGroup * kTileM);  // full[S], empty[S], accum
  StageInfo* info = reinterpret_cast<StageInfo*>(bars + 2 * kMaxStages + 1);
  uint32_t* vote = reinterpret_cast<uint32_t*>(info + kMaxStages);  // [4]
  uint32_t* tmem_slot = vote + 4;
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  float* epi_scale = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(abort_flag + 1) + 15) & ~uintptr_t(15));  // [256]
  float* epi_shift = epi_scale + 256;                             // [256] per-channel shift (bias folded in)

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  // once any CTA has given up on a wait, the remaining CTAs return at once
  if (*reinterpret_cast<volatile int*>(p.status) != 0) return;
  // tiles are taken from the END of the mask-sorted order first: those rows have the most
  // kernel offsets, and starting the long tiles first leaves the short ones to fill the tail
  const long long m0 = static_cast<long long>(gridDim.x - 1 - blockIdx.x) * kTileM;
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = smem_u32(bars + kMaxStages);
  const uint32_t bar_accum = smem_u32(bars + 2 * kMaxStages);

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(bar_full + 8 * s, kProducers + 1);  // 128 copy completions + the header writer
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_accum, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(tmem_slot), static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  const bool has_epilogue = p.epi.bias != nullptr || p.epi.scale != nullptr || p.epi.act != SPC_ACT_NONE;
  if (has_epilogue) stage_epilogue<T>(p.epi, p.n_dim, epi_scale, epi_shift, tid, kThreadsTc);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_rchunks = (p.r_dim + EPR - 1) / EPR;
  int real_stages = 0;

  if (warp < 4) {
    // ---------------- producers ----------------
    const long long slot = m0 + tid;
    const long long my_row = slot < p.m_rows ? (p.order ? static_cast<long long>(__ldg(&p.order[slot])) : slot) : -1;
    const int chunk = tid & 7, row_lo = tid >> 3;
    const uint8_t* src_b = static_cast<const uint8_t*>(p.src);
    const uint8_t* w_b = static_cast<const uint8_t*>(p.w);
    int stage = 0;
    uint32_t empty_parity = 1;  // a fresh barrier passes a wait on parity 1
    bool ok = true;

    // A thread whose wait expired keeps walking the loops (so that every named
    // barrier is still reached by all 128 producers) but issues nothing more.
    for (int k0 = 0; k0 < p.kv; k0 += kGroup) {
      const int gcount = min(kGroup, p.kv - k0);
      uint32_t mine = 0;
#pragma unroll 8
      for (int kk = 0; kk < gcount; ++kk) {
        int j = -1;
        if (my_row >= 0) j = __ldg(&p.pairs[static_cast<long long>(k0 + kk) * p.m_rows + my_row]);
        idx_s[kk * kTileM + tid] = j;
        mine |= static_cast<uint32_t>(j >= 0) << kk;
      }
      mine = __reduce_or_sync(0xffffffffu, mine);
      if (lane == 0) vote[warp] = mine;
      named_bar_sync(1, kProducers);
      const uint32_t active = vote[0] | vote[1] | vote[2] | vote[3];

      for (uint32_t rest = active; rest != 0; rest &= rest - 1) {
        const int kk = __ffs(rest) - 1;
        const int k = k0 + kk;
        for (int rc = 0; rc < n_rchunks; ++rc) {
          ++real_stages;
          if (ok && !mbar_wait(bar_empty + 8 * stage, empty_parity)) ok = false;
          if (!ok) continue;
          const int r0 = rc * EPR;
          const int r_len = min(EPR, p.r_dim - r0);
          const int pieces = r_len / EP16;  // 16-byte pieces per gathered row
          uint8_t* a_st = stage_base + static_cast<size_t>(stage) * stage_bytes;
          uint8_t* b_st = a_st + kAStageBytes;
          // A: 8 lanes cover the 128 bytes of one gathered row
          if (chunk < pieces) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int row = row_lo + 16 * i;
              const int j = idx_s[kk * kTileM + row];
              const uint8_t* g = j >= 0 ? src_b + (static_cast<long long>(j) * p.r_dim + r0) * ELEM + chunk * 16 : src_b;
              cp_async16(smem_u32(a_st + row * kRowBytes + ((chunk ^ (row & 7)) << 4)), g, j >= 0 ? 16u : 0u);
            }
          }
          if (!B_MN) {
            // B rows = output channels n, 128 bytes of reduction each: W[n, k, r0 + ...]
            if (chunk < pieces) {
              for (int row = row_lo; row < p.n_dim; row += 16) {
                const uint8_t* g = w_b + ((static_cast<long long>(row) * p.kv + k) * p.r_dim + r0) * ELEM + chunk * 16;
                cp_async16(smem_u32(b_st + row * kRowBytes + ((chunk ^ (row & 7)) << 4)), g, 16u);
              }
            }
          } else {
            // B rows = reduction index r, column blocks of EPR output channels: W[r0 + r, k, cb*EPR + ...]
            const int ncb = (p.n_dim + EPR - 1) / EPR;
            const int total = r_len * ncb;
            for (int q = row_lo; q < total; q += 16) {
              const int r = q % r_len, cb = q / r_len;
              const int col = cb * EPR + chunk * EP16;
              if (col < p.n_dim) {
                const uint8_t* g = w_b + ((static_cast<long long>(r0 + r) * p.kv + k) * p.n_dim + col) * ELEM;
                cp_async16(smem_u32(b_st + cb * (EPR * kRowBytes) + r * kRowBytes + ((chunk ^ (r & 7)) << 4)), g, 16u);
              }
            }
          }
          // hand-over without waiting: each thread's arrival is delivered by the
          // copy unit when its copies have landed; thread 0 adds the stage header
          cp_async_arrive_noinc(bar_full + 8 * stage);
          if (tid == 0) {
            info[stage].ksteps = r_len / UMMA_K;
            info[stage].last = 0;
            mbar_arrive(bar_full + 8 * stage);
          }
          if (++stage == p.stages) {
            stage = 0;
            empty_parity ^= 1;
          }
        }
      }
      named_bar_sync(1, kProducers);  // idx_s may be overwritten by the next group
    }
    // terminator stage: no data, tells the MMA warp the tile is complete
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
      atomicExch(abort_flag, 1);
    }

    cp_async_wait_all();
    // ---------------- epilogue ----------------
    bool have_acc = ok && mbar_wait(bar_accum, 0);
    if (ok && !have_acc) atomicExch(p.status, SPC_ERR_DEVICE_WAIT_EXPIRED);
    // the TMEM loads are warp-wide (.sync.aligned): take them only if the whole warp can
    have_acc = __all_sync(0xffffffffu, have_acc);
    tc_fence_after();
    if (have_acc) {
      TO* out_row = static_cast<TO*>(p.out) + (my_row >= 0 ? my_row : 0) * p.n_dim;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
      for (int c0 = 0; c0 < p.n_dim; c0 += 16) {
        float v[16];
        if (real_stages > 0) {  // uniform over the CTA
          uint32_t raw[16];
          tmem_ld16(lane_addr + c0, raw);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 16; ++q) v[q] = __uint_as_float(raw[q]);
        } else {
#pragma unroll
          for (int q = 0; q < 16; ++q) v[q] = 0.f;
        }
        if (my_row >= 0) {
            if (has_epilogue) finish_epilogue16(v, epi_scale + c0, epi_shift + c0, p.epi.act, p.epi.alpha);
            if (p.epi.residual != nullptr)
              add_residual16<TO>(v, static_cast<const TO*>(p.epi.residual) + my_row * p.n_dim + c0);
          store_row16<TO>(out_row + c0, v);
        }
      }
    }
    tc_fence_before();
  } else {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (TcType<T>::fmt << 7) | (TcType<T>::fmt << 10) |
                             ((B_MN ? 1u : 0u) << 16) | (static_cast<uint32_t>(p.n_dim >> 3) << 17) |
                             (static_cast<uint32_t>(kTileM >> 4) << 24);
      int stage = 0;
      uint32_t full_parity = 0;
      uint32_t accumulate = 0;
      bool ok = true;
      while (true) {
        if (!mbar_wait(bar_full + 8 * stage, full_parity)) {
          ok = false;
          break;
        }
        // the stage was written through the generic proxy (cp.async); order those
        // writes before the tensor core's async-proxy reads
        fence_proxy_async();
        tc_fence_after();
        const StageInfo si = info[stage];
        const uint32_t a_addr = smem_u32(stage_base + static_cast<size_t>(stage) * stage_bytes);
        const uint32_t b_addr = a_addr + kAStageBytes;
        const uint64_t a_desc = make_desc(a_addr, 16, 1024);
        const uint64_t b_desc = B_MN ? make_desc(b_addr, EPR * kRowBytes, 1024) : make_desc(b_addr, 16, 1024);
        for (int ks = 0; ks < si.ksteps; ++ks) {
          // descriptors address in 16-byte units: +32 bytes per step along a K-major row,
          // +UMMA_K rows (of 128 bytes) per step for the MN-major weight slab
          const uint64_t a_step = static_cast<uint64_t>(ks * 2);
          const uint64_t b_step = static_cast<uint64_t>(B_MN ? ks * (UMMA_K * kRowBytes / 16) : ks * 2);
          tc_mma<TF32>(tmem_base, a_desc + a_step, b_desc + b_step, idesc, accumulate);
          accumulate = 1;
        }
        if (si.last) {
          tc_commit(bar_accum);
          break;
        }
        tc_commit(bar_empty + 8 * stage);
        if (++stage == p.stages) {
          stage = 0;
          full_parity ^= 1;
        }
      }
      if (!ok && atomicAdd(abort_flag, 0) == 0) atomicExch(p.status, SPC_ERR_DEVICE_WAIT_EXPIRED);
    }
    __syncwarp();
  }

  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

struct TcPlan {
  int stages, b_stage_bytes, tmem_cols;
  size_t smem_bytes;
};

TcPlan make_plan(int n_dim, int r_dim, int elem, bool b_mn) {
  TcPlan pl;
  const int epr = kRowBytes / elem;
  if (b_mn) {
    const int ncb = (n_dim + epr - 1) / epr;
    pl.b_stage_bytes = ncb * epr * kRowBytes;
  } else {
    pl.b_stage_bytes = ((n_dim + 7) / 8 * 8) * kRowBytes;
  }
  pl.b_stage_bytes = static_cast<int>(align_up(pl.b_stage_bytes, 1024));
  const int stage_bytes = kAStageBytes + pl.b_stage_bytes;
  const size_t fixed = 1024 /*alignment slack*/ + kGroup * kTileM * 4 + (2 * kMaxStages + 1) * 8 +
                       kMaxStages * sizeof(StageInfo) + 64 + 2 * 256 * sizeof(float) + 16;
  const size_t budget = 110 * 1024;  // two CTAs per SM
  int stages = static_cast<int>((budget - fixed) / stage_bytes);
  stages = std::max(2, std::min(stages, 6));
  pl.stages = stages;
  pl.smem_bytes = fixed + static_cast<size_t>(stages) * stage_bytes;
  int cols = 32;
  while (cols < n_dim) cols <<= 1;
  pl.tmem_cols = cols;
  (void)r_dim;
  return pl;
}

template <typename T, typename TO, bool B_MN>
int launch_tc(const TcParams& base, cudaStream_t st) {
  TcParams p = base;
  const TcPlan pl = make_plan(p.n_dim, p.r_dim, sizeof(T), B_MN);
  p.stages = pl.stages;
  p.b_stage_bytes = pl.b_stage_bytes;
  p.tmem_cols = pl.tmem_cols;
  static bool configured[kMaxDevices] = {false};  // per instantiation and device
  SPC_CUDA_OK(ensure_dynamic_smem(gather_gemm_tc_kernel<T, TO, B_MN>, 200 * 1024, configured));
  const unsigned grid = static_cast<unsigned>(ceil_div(p.m_rows, kTileM));
  gather_gemm_tc_kernel<T, TO, B_MN><<<grid, kThreadsTc, pl.smem_bytes, st>>>(p);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

}  // namespace

// Address of the current device's status word (every device that loads the
// library has its own copy of the symbol).
int* device_status_ptr() {
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (ptrs[dev] == nullptr) {
    void* raw = nullptr;
    if (cudaGetSymbolAddress(&raw, g_device_status) == cudaSuccess) ptrs[dev] = static_cast<int*>(raw);
  }
  return ptrs[dev];
}

bool gather_gemm_tc_supported(int n_dim, int r_dim, int kv, int dtype, int out_dtype, int precision,
                              bool transposed_weight) {
  (void)kv;
  const bool sixteen = dtype == SPC_F16 || dtype == SPC_BF16;
  const bool tf32 = dtype == SPC_F32 && precision == SPC_PREC_TF32;
  if (!sixteen && !tf32) return false;
  // The MN-major weight slab of the input gradient is laid out for 16-bit
  // elements only; TF32 input gradients run on the CUDA cores in IEEE fp32.
  if (tf32 && transposed_weight) return false;
  if (tf32 && out_dtype != SPC_F32) return false;
  if (sixteen && out_dtype != dtype && out_dtype != SPC_F32) return false;
  if (n_dim < 16 || n_dim > 256 || n_dim % 16 != 0) return false;
  const int umma_k = sixteen ? 16 : 8;
  if (r_dim < umma_k || r_dim % umma_k != 0) return false;
  return true;
}

int gather_gemm_tc(const void* src, const void* w, const Epilogue& epi, const int32_t* pairs,
                   const int32_t* order, void* out, long long m_rows, int n_dim, int r_dim, int kv,
                   bool transposed_weight, int dtype, int out_dtype, int precision, cudaStream_t st) {
  if (!gather_gemm_tc_supported(n_dim, r_dim, kv, dtype, out_dtype, precision, transposed_weight))
    return fail(SPC_ERR_UNSUPPORTED, "tcgen05 gather-GEMM: unsupported shape");
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15u)
    return fail(SPC_ERR_UNSUPPORTED, "tcgen05 gather-GEMM: operands must be 16-byte aligned");
  TcParams p{};
  p.src = src; p.w = w; p.epi = epi; p.pairs = pairs; p.order = order; p.out = out;
  p.m_rows = m_rows; p.n_dim = n_dim; p.r_dim = r_dim; p.kv = kv;
  p.status = device_status_ptr();
  if (p.status == nullptr) return fail(SPC_ERR_CUDA, "tcgen05 gather-GEMM: no device status word");
#define SPC_TC(T, TO)                                                        \
  return transposed_weight ? launch_tc<T, TO, true>(p, st) : launch_tc<T, TO, false>(p, st)
  if (dtype == SPC_F16 && out_dtype == SPC_F16) SPC_TC(__half, __half);
  if (dtype == SPC_F16 && out_dtype == SPC_F32) SPC_TC(__half, float);
  if (dtype == SPC_BF16 && out_dtype == SPC_BF16) SPC_TC(__nv_bfloat16, __nv_bfloat16);
  if (dtype == SPC_BF16 && out_dtype == SPC_F32) SPC_TC(__nv_bfloat16, float);
  if (dtype == SPC_F32 && out_dtype == SPC_F32) SPC_TC(float, float);
#undef SPC_TC
  return fail(SPC_ERR_UNSUPPORTED, "tcgen05 gather-GEMM: dtype combination");
}

__global__ void post_status_kernel(const int* __restrict__ status, int* __restrict__ host_word) {
  *host_word = *status;
  __threadfence_system();
}

int read_device_status(cudaStream_t st, int* host_value) {
  int* ptr = device_status_ptr();
  *host_value = 0;
  if (ptr == nullptr) return SPC_OK;
  SPC_CUDA_OK(cudaMemcpyAsync(host_value, ptr, sizeof(int), cudaMemcpyDeviceToHost, st));
  SPC_CUDA_OK(cudaStreamSynchronize(st));
  if (*host_value != 0) SPC_CUDA_OK(cudaMemsetAsync(ptr, 0, sizeof(int), st));
  return SPC_OK;
}

}  // namespace spc

extern "C" int spc_post_device_status(int* pinned_host_word, void* stream) {
  if (pinned_host_word == nullptr) return spc::fail(SPC_ERR_INVALID_ARGUMENT, "post_device_status: null mailbox");
  int* ptr = spc::device_status_ptr();
  if (ptr == nullptr) return SPC_OK;
  // written by a kernel, not copied: a device-to-host copy would wait on the copy engine behind
  // whatever transfer the application has in flight and hold up the stream
  spc::post_status_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(ptr, pinned_host_word);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

extern "C" int spc_check_device_status(void* stream) {
  int value = 0;
  const int rc = spc::read_device_status(static_cast<cudaStream_t>(stream), &value);
  if (rc != SPC_OK) return rc;
  if (value == SPC_ERR_INVALID_ARGUMENT)
    return spc::fail(value, "a rulebook kernel met an index row outside batch_size / spatial_shape (device status %d)", value);
  if (value != 0) return spc::fail(value, "a kernel of this library recorded device status %d (a bounded wait expired)", value);
  return SPC_OK;
}
