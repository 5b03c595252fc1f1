// Device-side building blocks shared by the tcgen05 kernels: PTX wrappers for
// mbarriers, cp.async, TMA, tensor memory and tcgen05.mma, the shared-memory
// matrix descriptor and the epilogue row store.
#pragma once

#include "common.cuh"

namespace spc {
namespace tc {

constexpr int kTileM = 128;
constexpr int kRowBytes = 128;
constexpr int kAStageBytes = kTileM * kRowBytes;  // 16 KB
constexpr int kProducers = 128;
constexpr int kThreadsTc = 160;
constexpr int kGroup = 32;  // kernel offsets voted on together
constexpr int kMaxStages = 8;
// A wait polls kSpinLimit times, then keeps polling against a wall-clock limit, so that a slow
// tile (a long reduction, a preempted SM) is not mistaken for a failure while every wait still ends.
constexpr uint32_t kSpinLimit = 1u << 10;
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // one second

// ---- PTX wrappers --------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One try: the hardware may park the thread until the phase completes or, at the latest, for
// about kWaitHintNs; a parked warp issues nothing, a spinning one takes issue slots and
// shared-memory cycles from the warps that copy and multiply.
constexpr uint32_t kWaitHintNs = 20000;
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kWaitHintNs)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity) {
  const unsigned long long t0 = global_timer_ns();
  do {
    for (uint32_t it = 0; it < 16; ++it)
      if (mbar_try_wait(bar, parity)) return true;
  } while (global_timer_ns() - t0 < kWaitLimitNs);
  return false;
}
// Bounded wait; false means the limit was reached.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < kSpinLimit; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// The barrier receives this thread's arrival once all cp.async it has issued so
// far have landed; the thread itself does not wait.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <bool TF32>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       uint32_t accumulate) {
  if (TF32) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: start address, leading / stride byte
// offsets (all >> 4), descriptor version 1, 128-byte swizzle.
// layout_type: 2 = 128-byte swizzle, 4 = 64-byte, 6 = 32-byte.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type = 2) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fffu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= 1ull << 46;
  d |= static_cast<uint64_t>(layout_type) << 61;
  return d;
}

template <typename T> struct TcType;
template <> struct TcType<__half> { static constexpr uint32_t fmt = 0; static constexpr bool tf32 = false; };
template <> struct TcType<__nv_bfloat16> { static constexpr uint32_t fmt = 1; static constexpr bool tf32 = false; };
template <> struct TcType<float> { static constexpr uint32_t fmt = 2; static constexpr bool tf32 = true; };


struct StageInfo {
  int ksteps;
  int last;
};

// 16 consecutive fp32 accumulators -> 16 output elements of one row.
template <typename TO>
__device__ __forceinline__ void store_row16(TO* dst, const float* v);
template <>
__device__ __forceinline__ void store_row16<float>(float* dst, const float* v) {
#pragma unroll
  for (int q = 0; q < 4; ++q)
    reinterpret_cast<float4*>(dst)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
}
template <>
__device__ __forceinline__ void store_row16<__half>(__half* dst, const float* v) {
  uint32_t packed[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    __half2 h = __floats2half2_rn(v[2 * q], v[2 * q + 1]);
    packed[q] = *reinterpret_cast<uint32_t*>(&h);
  }
  reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
}
template <>
__device__ __forceinline__ void store_row16<__nv_bfloat16>(__nv_bfloat16* dst, const float* v) {
  uint32_t packed[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
    packed[q] = *reinterpret_cast<uint32_t*>(&h);
  }
  reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
}


}  // namespace tc
}  // namespace spc
