// Implicit gather-GEMM on tcgen05: cp.async-gathered feature rows, TMA-loaded
// weight slabs.
//
// Same computation and tiling as gemm_tc.cu (128 output rows per CTA, fp32
// accumulator in tensor memory).  What differs is how a shared-memory stage is
// filled:
//   * the 128 gathered feature rows are copied with 16-byte cp.async by two
//     groups of two warps that take the stages in turn (a row's pieces go to
//     neighbouring lanes, a thread copies one piece of 16, 8 or 4 rows, absent
//     rows are zero-filled by predicate); each thread's completion is
//     delivered to the stage's mbarrier by cp.async.mbarrier.arrive.noinc, so
//     nobody waits for data;
//   * the weight slab W[:, k, chunk] arrives through one tiled 3-D TMA load
//     (one per column block for the input gradient) completing on the same
//     mbarrier with complete_tx::bytes.
// The row pitch in shared memory equals the swizzle span (32 / 64 / 128 bytes),
// so channel counts of 16, 32 and multiples of 64 (16-bit) or 8, 16 and
// multiples of 32 (TF32) are taken; other widths stay with gemm_tc.cu.
//
// Measured alternatives on B200 (64 -> 64 channels, 723k rows, 7.1M pairs):
// feeding the rows with TMA tile::gather4 (4 rows per instruction) reached
// 590 us issued by one warp and 400 us issued by four: the gather4 path
// sustains roughly one 512-byte operation per ~30 cycles per SM, below what
// the LSU path reaches, so the rows go through cp.async.
//
// Other things measured on the same kernel (SubMConv3d k3, 383k rows, 67.6k
// stages): one barrier arrival per warp instead of per thread (needs a
// blocking cp.async.wait_group: slower), one polling warp per CTA with the
// others parked in a hardware barrier (slower), mbarrier.test_wait spinning
// instead of try_wait (same), the table tile in registers with shuffles
// instead of shared memory (a fourth CTA per SM at 64 channels, but slower:
// the select tree costs more than the table read), skipping the zero fill of
// pieces that are still zero (slower: the bookkeeping costs more than the
// copies), two CTAs with four stages instead of three with two (slower).
// Timing the two loops with clock64 shows where a stage's ~1 000 cycles go at
// 64 -> 64: the MMA thread waits ~500 cycles for the stage and spends ~560
// issuing its four tcgen05.mma (about 100 cycles each with three CTAs feeding
// one tensor core from shared memory), the copy warps ~220 cycles in the slot
// wait and ~450 issuing copies and the arrival.
//
// Warp roles (160 threads): warps 0-3 load the tile's table entries, vote on the
// active kernel offsets (32 at a time), issue the row copies and later run the
// epilogue; the first thread of a copy group also issues its stages' TMA
// weight loads; warp 4 issues tcgen05.mma and counts the stages from the same
// vote.  All waits are bounded.
#include <cuda.h>

#include <algorithm>
#include <type_traits>

#include "common.cuh"
#include "gemm_internal.cuh"
#include "tc_common.cuh"

namespace spc {
namespace {

using namespace tc;

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

struct TmaParams {
  const void* src;
  Epilogue epi;
  const int32_t* pairs;
  const int32_t* pairs_rm;  // optional row-major copy [m_rows, kvp]
  const int32_t* order;
  void* out;
  long long m_rows;
  int kvp;
  int src_rows;  // rows of the gathered matrix; also the "absent row" index
  int n_dim, r_dim, kv;
  int stages, a_stage_bytes, b_stage_bytes, tmem_cols;
  int group_rows;  // kernel offsets voted on together: min(kv, 32); sizes the table tile in shared memory
  int epi_pad;     // output channels rounded up to 16; sizes the epilogue scale / shift arrays
  int a_row_bytes, b_row_bytes;  // swizzle span of the A rows / of the MN-major B rows
  int* status;
};

__host__ __device__ inline uint32_t layout_type_for(int row_bytes) {
  return row_bytes == 128 ? 2u : (row_bytes == 64 ? 4u : 6u);
}

// Four copy warps + the MMA warp: 160 threads.  A small CTA lets three or four of them share an SM
// (shared memory permitting), i.e. three or four MMA issuers and that many tiles whose table
// load, pipeline drain and epilogue overlap the others' stages: 64 -> 64 went from 166 us with
// 2 x 288 threads to 141 us with 3 x 160, 32 -> 32 from 149 us to 103 us with 4 x 160.
//
// The copy warps are bound by the instructions they issue per stage, not by bytes: with the
// copies, the multiplications and the stores all removed the kernel still took 60 % of its time.
// So a stage costs a copy thread as few instructions as the job allows: one vector read of its
// rows' table entries (the table tile is stored in the order the copy threads read it), per row
// one clamp, one address and one copy whose zero fill is a predicate, destinations that are
// compile-time offsets from the stage base; the MMA warp counts the stages itself from the same
// vote, so no per-stage record goes through shared memory and no terminator stage exists.
constexpr int kIssueWarps = 4;                        // warps that issue the feature-row copies
constexpr int kIssueThreads = kIssueWarps * 32;       // 128
constexpr int kMmaWarp = kIssueWarps;                 // warp 4
constexpr int kThreadsHybrid = kIssueThreads + 32;    // 160
constexpr int kCopyGroups = 2;                        // halves of the copy warps; stages alternate between them
constexpr int kGroupThreads = kIssueThreads / kCopyGroups;  // 64
constexpr int kPassBytes = kGroupThreads * 16;        // one copy per thread of a group covers 1024 bytes of the tile
constexpr int kMaxCtasPerSm = 4;                      // 4 x 160 threads x 96 registers fit the register file

// 16-byte copy into shared memory; zeros instead when row < 0 (the source is then not read).
__device__ __forceinline__ void cp_async16_row(uint32_t dst, const void* src, int row) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.lt.s32 p, %2, 0;\n\t"
      "cp.async.cg.shared.global [%0], [%1], 16, p;\n\t}" ::"r"(dst), "l"(src), "r"(row)
      : "memory");
}

// LPR: lanes per row = 16-byte pieces of one A row in a stage (8, 4 or 2 for rows of 128, 64 or 32
// bytes).  128 / LPR rows are covered by one copy per thread, so a thread copies piece
// tid % LPR of rows tid / LPR + i * (128 / LPR), i < LPR.
template <typename T, typename TO, bool B_MN, int LPR>
__global__ void __maxnreg__(96)
gather_gemm_tma_kernel(const __grid_constant__ TmaParams p, const __grid_constant__ CUtensorMap map_b) {
  constexpr int ELEM = sizeof(T);
  constexpr int UMMA_K = 32 / ELEM;
  constexpr bool TF32 = TcType<T>::tf32;
  constexpr int A_ROW_BYTES = 16 * LPR;
  constexpr int kRowsPass = kGroupThreads / LPR;  // rows one copy per thread of a group covers: 8, 16, 32
  constexpr int CP = kTileM / kRowsPass;          // copies per thread and stage: 16, 8, 4

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = p.a_stage_bytes + p.b_stage_bytes;
  uint8_t* stage_base = smem;
  // table entries of the group, [offset][row / kRowsPass-th copy of thread row % kRowsPass]
  int* idx_s = reinterpret_cast<int*>(smem + static_cast<size_t>(p.stages) * stage_bytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(idx_s + p.group_rows * kTileM);
  uint32_t* vote = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 1);  // [2][4]: groups alternate
  uint32_t* tmem_slot = vote + 8;
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  float* epi_scale = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(abort_flag + 1) + 15) & ~uintptr_t(15));  // [epi_pad]
  float* epi_shift = epi_scale + p.epi_pad;                       // [epi_pad] per-channel shift (bias folded in)

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  if (*reinterpret_cast<volatile int*>(p.status) != 0) return;
  // tiles are taken from the END of the mask-sorted order first: those rows have the most
  // kernel offsets, and starting the long tiles first leaves the short ones to fill the tail
  const long long m0 = static_cast<long long>(gridDim.x - 1 - blockIdx.x) * kTileM;
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = smem_u32(bars + kMaxStages);
  const uint32_t bar_accum = smem_u32(bars + 2 * kMaxStages);

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(bar_full + 8 * s, kGroupThreads + 1);  // every thread of the stage's copy group + the weight-slab transaction
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_accum, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_b);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  const bool has_epilogue = p.epi.bias != nullptr || p.epi.scale != nullptr || p.epi.act != SPC_ACT_NONE;
  if (has_epilogue) stage_epilogue<T>(p.epi, p.n_dim, epi_scale, epi_shift, tid, kThreadsHybrid);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int epr = A_ROW_BYTES / ELEM;  // reduction elements per stage
  const int n_rchunks = (p.r_dim + epr - 1) / epr;
  constexpr int KSTEPS = A_ROW_BYTES / 32;  // tcgen05.mma instructions per stage
  const uint32_t stage0 = smem_u32(stage_base);
  const uint32_t ring_end = stage0 + static_cast<uint32_t>(p.stages * stage_bytes);

  if (warp < kIssueWarps) {
    long long my_row = -1;
    {
      const long long slot = m0 + tid;
      if (slot < p.m_rows) my_row = p.order ? static_cast<long long>(__ldg(&p.order[slot])) : slot;
    }
    int real_stages = 0;
    bool ok = true;
    const int b_cols = p.b_row_bytes / ELEM;  // MN-major: output channels per column block
    const int ncb = B_MN ? (p.n_dim + b_cols - 1) / b_cols : 1;
    const uint32_t b_bytes = B_MN ? static_cast<uint32_t>(ncb * epr * p.b_row_bytes)
                                  : static_cast<uint32_t>(p.n_dim * A_ROW_BYTES);
    // Two copy groups of 64 threads take the stages in turn.  What a stage costs a copy warp
    // besides its copies (the slot wait, the arrival, the loop) is a chain of some hundred
    // cycles of latency that the MMA warp ends up waiting for; with two groups the chains of
    // neighbouring stages overlap.
    const int grp = tid / kGroupThreads, gt = tid % kGroupThreads;
    const int chunk = gt & (LPR - 1), row_lo = gt / LPR;
    // 64 / LPR rows further down the tile is 1024 bytes further and leaves the swizzle term
    // (row modulo 8, 4 or 2) alone: the i-th copy goes to a_dst + i * kPassBytes
    const uint32_t lin0 = static_cast<uint32_t>(row_lo * A_ROW_BYTES + chunk * 16);
    uint32_t a_dst = stage0 + (lin0 ^ (((lin0 >> 7) & static_cast<uint32_t>(LPR - 1)) << 4));  // this thread's piece of row_lo
    uint32_t full = bar_full, empty = bar_empty, empty_parity = 1;
    uint32_t turn = 0;  // whose stage comes next
    const uint32_t a_dst0 = a_dst;
    const uint8_t* src_chunk = static_cast<const uint8_t*>(p.src) + chunk * 16;
    const uint32_t src_pitch = static_cast<uint32_t>(p.r_dim) * ELEM;
    // the tile row `tid` is the (tid / kRowsPass)-th copy of the copy threads with row_lo = tid % kRowsPass
    int* const wr_ptr = idx_s + (tid % kRowsPass) * CP + tid / kRowsPass;
    const int* const rd_ptr = idx_s + row_lo * CP;

    int group = 0;
    for (int k0 = 0; k0 < p.kv; k0 += kGroup, ++group) {
      const int gcount = min(kGroup, p.kv - k0);
      {
        // all table entries of the group are requested before any is used
        int jj[kGroup];
        if (p.pairs_rm != nullptr) {
          // the row's entries are contiguous: 16-byte loads
          const int4* rowp = reinterpret_cast<const int4*>(p.pairs_rm + (my_row >= 0 ? my_row : 0) * p.kvp + k0);
#pragma unroll
          for (int q = 0; q < kGroup / 4; ++q) {
            int4 v = make_int4(-1, -1, -1, -1);
            if (4 * q < gcount && my_row >= 0) v = __ldg(rowp + q);
            jj[4 * q] = v.x; jj[4 * q + 1] = v.y; jj[4 * q + 2] = v.z; jj[4 * q + 3] = v.w;
          }
        } else {
#pragma unroll
          for (int kk = 0; kk < kGroup; ++kk) {
            jj[kk] = -1;
            if (kk < gcount && my_row >= 0)
              jj[kk] = __ldg(&p.pairs[static_cast<long long>(k0 + kk) * p.m_rows + my_row]);
          }
        }
        uint32_t mine = 0;
#pragma unroll
        for (int kk = 0; kk < kGroup; ++kk) {
          mine |= static_cast<uint32_t>(jj[kk] >= 0) << kk;
          if (kk < gcount) wr_ptr[kk * kTileM] = jj[kk];
        }
        mine = __reduce_or_sync(0xffffffffu, mine);
        if (lane == 0) vote[(group & 1) * 4 + warp] = mine;
      }
      named_bar_sync(1, kThreadsHybrid);  // the MMA warp reads the vote too
      const uint32_t* v4 = vote + (group & 1) * 4;
      const uint32_t active = v4[0] | v4[1] | v4[2] | v4[3];
      real_stages += __popc(active) * n_rchunks;

      for (uint32_t rest = ok ? active : 0u; rest != 0; rest &= rest - 1) {
        const int kk = __ffs(rest) - 1;
        const int k = k0 + kk;
        // this group's stages of the offset: every other one
        if (n_rchunks == 1 && turn != static_cast<uint32_t>(grp)) {
          turn ^= 1u;
          a_dst += stage_bytes;
          full += 8;
          empty += 8;
          if (a_dst >= ring_end) {
            a_dst = a_dst0;
            full = bar_full;
            empty = bar_empty;
            empty_parity ^= 1;
          }
          continue;
        }
        int j[CP];
#pragma unroll
        for (int q = 0; q < CP / 4; ++q) {
          const int4 v = *reinterpret_cast<const int4*>(rd_ptr + kk * kTileM + 4 * q);
          j[4 * q] = v.x; j[4 * q + 1] = v.y; j[4 * q + 2] = v.z; j[4 * q + 3] = v.w;
        }
        for (int rc = 0; rc < n_rchunks; ++rc) {
          if (turn == static_cast<uint32_t>(grp)) {
            if (!mbar_wait(empty, empty_parity)) {
              ok = false;
              rest = 0;  // leaves the offset loop after this one
              break;
            }
            const int r0 = rc * epr;
            const uint8_t* base = src_chunk + static_cast<long long>(r0) * ELEM;
#pragma unroll
            for (int i = 0; i < CP; ++i)
              cp_async16_row(a_dst + i * kPassBytes,
                             base + static_cast<unsigned long long>(static_cast<uint32_t>(max(j[i], 0))) * src_pitch, j[i]);
            // delivered to the barrier by the copy unit once this thread's copies have landed
            cp_async_arrive_noinc(full);
            if (gt == 0) {
              mbar_expect_tx(full, b_bytes);
              const uint32_t b_dst = a_dst - (a_dst0 - stage0) + p.a_stage_bytes;
              if (!B_MN) {
                // weight viewed as [c_out][kv][c_in]: rows n = 0..n_dim-1 of offset k, reduction chunk r0
                tma_load_3d(b_dst, &map_b, r0, k, 0, full);
              } else {
                // weight viewed as [c_out = reduction][kv][c_in]: rows r0.., one load per column block
                for (int cb = 0; cb < ncb; ++cb)
                  tma_load_3d(b_dst + cb * epr * p.b_row_bytes, &map_b, cb * b_cols, k, r0, full);
              }
            }
          }
          turn ^= 1u;
          a_dst += stage_bytes;
          full += 8;
          empty += 8;
          if (a_dst >= ring_end) {
            a_dst = a_dst0;
            full = bar_full;
            empty = bar_empty;
            empty_parity ^= 1;
          }
        }
      }
      // the table tile may be overwritten by the next group once every copy thread is done with it
      if (k0 + kGroup < p.kv) named_bar_sync(2, kIssueThreads);
    }
    if (!ok) {
      atomicExch(p.status, SPC_ERR_DEVICE_WAIT_EXPIRED);
      atomicExch(abort_flag, 1);
    }
    cp_async_wait_all();

    // ---------------- epilogue ----------------
    bool have_acc = mbar_wait(bar_accum, 0);
    if (!have_acc) atomicExch(p.status, SPC_ERR_DEVICE_WAIT_EXPIRED);
    have_acc = __all_sync(0xffffffffu, have_acc);
    tc_fence_after();
    if (have_acc) {
      TO* out_row = static_cast<TO*>(p.out) + (my_row >= 0 ? my_row : 0) * p.n_dim;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
      for (int c0 = 0; c0 < p.n_dim; c0 += 16) {
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
    // One thread paces the whole CTA: every instruction between "stage full" and the commit is
    // on the critical path, so the loop carries running descriptor words (a stage advance is one
    // add to the address field) and the reduction steps are unrolled.  The number of stages of a
    // group follows from the copy warps' vote.
    const uint32_t idesc = (1u << 4) | (TcType<T>::fmt << 7) | (TcType<T>::fmt << 10) |
                           ((B_MN ? 1u : 0u) << 16) | (static_cast<uint32_t>(p.n_dim >> 3) << 17) |
                           (static_cast<uint32_t>(kTileM >> 4) << 24);
    const uint32_t a_type = layout_type_for(A_ROW_BYTES);
    const uint32_t b_type = B_MN ? layout_type_for(p.b_row_bytes) : a_type;
    const uint64_t a_desc0 = make_desc(stage0, 16, 8 * A_ROW_BYTES, a_type);
    const uint64_t b_desc0 = B_MN ? make_desc(stage0 + p.a_stage_bytes, epr * p.b_row_bytes, 8 * p.b_row_bytes, b_type)
                                  : make_desc(stage0 + p.a_stage_bytes, 16, 8 * A_ROW_BYTES, a_type);
    const uint32_t a_hi = static_cast<uint32_t>(a_desc0 >> 32), b_hi = static_cast<uint32_t>(b_desc0 >> 32);
    const uint32_t a_lo0 = static_cast<uint32_t>(a_desc0), b_lo0 = static_cast<uint32_t>(b_desc0);
    const uint32_t stage_step = static_cast<uint32_t>(stage_bytes >> 4);  // address field counts 16-byte units
    const uint32_t b_step = static_cast<uint32_t>(B_MN ? UMMA_K * p.b_row_bytes / 16 : 2);
    uint32_t a_lo = a_lo0, b_lo = b_lo0, full = bar_full, empty = bar_empty;
    uint32_t full_parity = 0, accumulate = 0;
    int stage = 0;
    bool ok = true;
    int group = 0;
    for (int k0 = 0; k0 < p.kv; k0 += kGroup, ++group) {
      named_bar_sync(1, kThreadsHybrid);
      const uint32_t* v4 = vote + (group & 1) * 4;
      const int n_stages = __popc(v4[0] | v4[1] | v4[2] | v4[3]) * n_rchunks;
      if (lane == 0 && ok) {
        for (int s = 0; s < n_stages; ++s) {
          // a wait that expires here is either a real failure or the copy warps having aborted
          if (!mbar_wait(full, full_parity)) {
            ok = false;
            break;
          }
          // the feature rows were written through the generic proxy (cp.async): order
          // those writes before the tensor core's async-proxy reads
          fence_proxy_async();
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ++ks) {
            const uint64_t a_desc = (static_cast<uint64_t>(a_hi) << 32) | (a_lo + 2u * ks);
            const uint64_t b_desc = (static_cast<uint64_t>(b_hi) << 32) | (b_lo + b_step * ks);
            tc_mma<TF32>(tmem_base, a_desc, b_desc, idesc, accumulate);
            accumulate = 1;
          }
          tc_commit(empty);
          a_lo += stage_step;
          b_lo += stage_step;
          full += 8;
          empty += 8;
          if (++stage == p.stages) {
            stage = 0;
            full_parity ^= 1;
            a_lo = a_lo0;
            b_lo = b_lo0;
            full = bar_full;
            empty = bar_empty;
          }
        }
      }
      __syncwarp();
    }
    if (lane == 0) {
      if (ok) {
        tc_commit(bar_accum);  // arrives once every multiplication above has completed
      } else {
        atomicExch(p.status, SPC_ERR_DEVICE_WAIT_EXPIRED);
        // release the epilogue warps: nothing more will be accumulated
        mbar_arrive(bar_accum);
      }
    }
    __syncwarp();
  }

  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

// ---- host side ------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* raw = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &raw, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(raw);
  }
  return fn;
}

CUtensorMapSwizzle swizzle_for(int row_bytes) {
  return row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : (row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

CUtensorMapDataType tma_dtype(int dtype) {
  return dtype == SPC_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                          : (dtype == SPC_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
}

// Swizzle span of rows holding `elems` contiguous elements: 32, 64 or 128 bytes
// (the latter for any multiple of 128 bytes); 0 if the width does not fit.
int row_span(int elems, int elem_size) {
  const int bytes = elems * elem_size;
  if (bytes == 32 || bytes == 64) return bytes;
  if (bytes >= 128 && bytes % 128 == 0) return 128;
  return 0;
}

template <typename T, typename TO, bool B_MN, int LPR>
int launch_tma_rows(const TmaParams& p, const CUtensorMap& map_b, size_t smem_bytes, cudaStream_t st) {
  static bool configured[kMaxDevices] = {false};  // per instantiation and device
  SPC_CUDA_OK(ensure_dynamic_smem(gather_gemm_tma_kernel<T, TO, B_MN, LPR>, 226 * 1024, configured));
  const unsigned grid = static_cast<unsigned>(ceil_div(p.m_rows, kTileM));
  gather_gemm_tma_kernel<T, TO, B_MN, LPR><<<grid, kThreadsHybrid, smem_bytes, st>>>(p, map_b);
  SPC_LAUNCH_OK();
  return SPC_OK;
}

template <typename T, typename TO, bool B_MN>
int launch_tma(const TmaParams& p, const CUtensorMap& map_b, size_t smem_bytes, cudaStream_t st) {
  if (p.a_row_bytes == 128) return launch_tma_rows<T, TO, B_MN, 8>(p, map_b, smem_bytes, st);
  if (p.a_row_bytes == 64) return launch_tma_rows<T, TO, B_MN, 4>(p, map_b, smem_bytes, st);
  return launch_tma_rows<T, TO, B_MN, 2>(p, map_b, smem_bytes, st);
}

}  // namespace

bool gather_gemm_tma_supported(int n_dim, int r_dim, int kv, int dtype, int out_dtype, int precision,
                               bool transposed_weight) {
  if (!gather_gemm_tc_supported(n_dim, r_dim, kv, dtype, out_dtype, precision, transposed_weight)) return false;
  const int elem = (dtype == SPC_F32) ? 4 : 2;
  if (row_span(r_dim, elem) == 0) return false;
  if (transposed_weight && row_span(n_dim, elem) == 0) return false;
  return encode_fn() != nullptr;
}

int gather_gemm_tma(const void* src, const void* w, const Epilogue& epi, const int32_t* pairs,
                    const int32_t* pairs_rowmajor, const int32_t* order, void* out, long long src_rows, long long m_rows, int n_dim, int r_dim,
                    int kv, bool transposed_weight, int dtype, int out_dtype, int precision, cudaStream_t st) {
  if (!gather_gemm_tma_supported(n_dim, r_dim, kv, dtype, out_dtype, precision, transposed_weight))
    return fail(SPC_ERR_UNSUPPORTED, "TMA gather-GEMM: unsupported shape");
  if (src_rows <= 0 || src_rows >= (1ll << 31) - 1)
    return fail(SPC_ERR_SIZE_LIMIT, "TMA gather-GEMM: %lld source rows", static_cast<long long>(src_rows));
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15u)
    return fail(SPC_ERR_UNSUPPORTED, "TMA gather-GEMM: operands must be 16-byte aligned");
  const int elem = (dtype == SPC_F32) ? 4 : 2;
  EncodeTiledFn encode = encode_fn();

  TmaParams p{};
  p.src = src; p.epi = epi; p.pairs = pairs; p.pairs_rm = pairs_rowmajor; p.kvp = (kv + 3) & ~3; p.order = order; p.out = out;
  p.m_rows = m_rows; p.src_rows = static_cast<int>(src_rows);
  p.n_dim = n_dim; p.r_dim = r_dim; p.kv = kv;
  p.a_row_bytes = row_span(r_dim, elem);
  p.b_row_bytes = transposed_weight ? row_span(n_dim, elem) : p.a_row_bytes;
  const int epr = p.a_row_bytes / elem;
  p.a_stage_bytes = static_cast<int>(align_up(static_cast<size_t>(kTileM) * p.a_row_bytes, 1024));
  if (transposed_weight) {
    const int b_cols = p.b_row_bytes / elem;
    const int ncb = (n_dim + b_cols - 1) / b_cols;
    p.b_stage_bytes = ncb * epr * p.b_row_bytes;
  } else {
    p.b_stage_bytes = n_dim * p.a_row_bytes;
  }
  p.b_stage_bytes = static_cast<int>(align_up(p.b_stage_bytes, 1024));
  const int stage_bytes = p.a_stage_bytes + p.b_stage_bytes;
  // Everything besides the stages is sized to the layer.  As many CTAs per SM as shared memory
  // (228 KB per SM, 1 KB reserved per CTA), tensor memory (512 columns) and registers allow, as
  // long as each keeps at least two stages.
  p.epi_pad = (n_dim + 15) / 16 * 16;
  int cols = 32;
  while (cols < n_dim) cols <<= 1;
  p.tmem_cols = cols;
  p.group_rows = std::min(kv, kGroup);
  const size_t fixed = 1024 + static_cast<size_t>(p.group_rows) * kTileM * 4 + (2 * kMaxStages + 1) * 8 + 64 + 2 * p.epi_pad * sizeof(float) + 16;
  p.stages = 0;
  int ctas = std::min(kMaxCtasPerSm, 512 / cols) + 1;
  // 256 output channels: two CTAs per SM keep two 48 KB stages each.  That wins on large grids
  // (SparseConvTranspose3d C256, 10k tiles: 1.12 against 1.25 ms, the stores of one tile overlap
  // the multiplications of the other) and loses on small ones, where one CTA with four stages
  // finishes a tile sooner (SubMConv3d C256 on 50k rows, 391 tiles: 0.048 against 0.059 ms).
  const long long tiles = ceil_div(m_rows, kTileM);
  if (cols >= 256 && tiles < 4ll * sm_count()) ctas = 2;
  while (p.stages < 2 && ctas > 1) {
    --ctas;
    const size_t per_cta = (228 * 1024 - static_cast<size_t>(ctas) * 1024) / ctas - 256;
    p.stages = per_cta > fixed ? std::min<int>(kMaxStages, static_cast<int>((per_cta - fixed) / stage_bytes)) : 0;
  }
  // the kernel's dynamic shared memory limit is set to 200 KB
  while (p.stages > 2 && fixed + static_cast<size_t>(p.stages) * stage_bytes > 226 * 1024) --p.stages;
  // shared memory is carved out of the L1: beyond two stages, keep about 36 KB of the SM as cache
  // for the table and epilogue traffic (a third stage that took it cost 8 % on 64 -> 128)
  // (layers whose reduction spans several stages per offset keep the deeper pipeline: 128 -> 128
  // lost 10 % without its third stage)
  const bool long_reduction = r_dim * elem > p.a_row_bytes;
  while (!long_reduction && p.stages > 2 && ctas * (fixed + static_cast<size_t>(p.stages) * stage_bytes) > 192 * 1024)
    --p.stages;
  if (p.stages < 2) return fail(SPC_ERR_UNSUPPORTED, "TMA gather-GEMM: a stage of %d bytes does not fit twice", stage_bytes);
  const size_t smem_bytes = fixed + static_cast<size_t>(p.stages) * stage_bytes;
  p.status = device_status_ptr();
  if (p.status == nullptr) return fail(SPC_ERR_CUDA, "TMA gather-GEMM: no device status word");

  CUtensorMap map_b;
  // B: the KRSC weight [c_out][kv][c_in] as a 3-D tensor (c_in innermost)
  {
    const int c_in = transposed_weight ? n_dim : r_dim;
    const int c_out = transposed_weight ? r_dim : n_dim;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(c_in), static_cast<cuuint64_t>(kv),
                                static_cast<cuuint64_t>(c_out)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(c_in) * elem, static_cast<cuuint64_t>(kv) * c_in * elem};
    cuuint32_t box[3];
    if (transposed_weight) {
      box[0] = static_cast<cuuint32_t>(p.b_row_bytes / elem);  // output channels of one column block
      box[1] = 1;
      box[2] = static_cast<cuuint32_t>(epr);                   // reduction rows of one stage
    } else {
      box[0] = static_cast<cuuint32_t>(epr);
      box[1] = 1;
      box[2] = static_cast<cuuint32_t>(n_dim);
    }
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = encode(&map_b, tma_dtype(dtype), 3, const_cast<void*>(w), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(p.b_row_bytes),
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SPC_ERR_CUDA, "cuTensorMapEncodeTiled(B) failed: %d", static_cast<int>(r));
  }

#define SPC_TMA(T, TO)                                                                                   \
  return transposed_weight ? launch_tma<T, TO, true>(p, map_b, smem_bytes, st)                    \
                           : launch_tma<T, TO, false>(p, map_b, smem_bytes, st)
  if (dtype == SPC_F16 && out_dtype == SPC_F16) SPC_TMA(__half, __half);
  if (dtype == SPC_F16 && out_dtype == SPC_F32) SPC_TMA(__half, float);
  if (dtype == SPC_BF16 && out_dtype == SPC_BF16) SPC_TMA(__nv_bfloat16, __nv_bfloat16);
  if (dtype == SPC_BF16 && out_dtype == SPC_F32) SPC_TMA(__nv_bfloat16, float);
  if (dtype == SPC_F32 && out_dtype == SPC_F32) SPC_TMA(float, float);
#undef SPC_TMA
  return fail(SPC_ERR_UNSUPPORTED, "TMA gather-GEMM: dtype combination");
}

}  // namespace spc
