// Shared device helpers of the B200 (sm_100a) MoE FFN kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define DEVI __device__ __forceinline__

namespace dmoe {

constexpr int kWarp = 32;
// Status word bits written by kernels instead of trapping or hanging.
constexpr unsigned kStatusWaitTimeout = 1u;   // a bounded wait ran out
constexpr unsigned kStatusBadRoute = 2u;      // expert id out of range / duplicate in a token

// ---- programmatic dependent launch -------------------------------------------------------
// `pdl_wait` blocks until every grid this launch depends on has finished and flushed its
// memory (returns at once when the launch carries no PDL attribute). `pdl_launch` lets the
// next PDL launch in the stream start scheduling its blocks.
DEVI void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
DEVI void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- warp helpers ------------------------------------------------------------------------
DEVI float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
DEVI float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
DEVI float sigmoid_precise(float x) { return 1.f / (1.f + expf(-x)); }
DEVI float silu_mul(float g, float u) { return g * (1.f / (1.f + expf(-g))) * u; }
// hardware exp2 / reciprocal approximations (about 2 ulp each): for products that are rounded to bf16 right after
DEVI float silu_mul_fast(float g, float u) { return __fdividef(g * u, 1.f + __expf(-g)); }

DEVI uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- shared-memory barriers and bulk copies (TMA engine, untiled form) ----------------------
DEVI uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

DEVI void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
DEVI void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
DEVI void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
DEVI void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
DEVI bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity to complete. Never spins without bound: after
// `kWaitLimitNs` the status bit is set and false is returned so that the caller can unwind.
constexpr uint64_t kWaitLimitNs = 2000000000ull;
DEVI bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned* status) {
  if (mbar_test(bar, parity)) return true;
  const uint64_t start = global_timer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_test(bar, parity)) return true;
    if ((spin & 63u) == 0) {
      __nanosleep(64);
      if (global_timer_ns() - start > kWaitLimitNs) {
        atomicOr(status, kStatusWaitTimeout);
        return false;
      }
    }
  }
}
// Same contract, but each probe lets the hardware suspend the thread until the phase completes or a short
// time limit passes, so that many waiting warps do not fill the issue slots with polling.
DEVI bool mbar_wait_suspend(uint64_t* bar, uint32_t parity, unsigned* status) {
  const uint32_t addr = smem_u32(bar);
  uint64_t start = 0;
  for (uint32_t spin = 0;; ++spin) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity), "r"(20000u)
        : "memory");
    if (ok) return true;
    if ((spin & 15u) == 0) {
      const uint64_t now = global_timer_ns();
      if (spin == 0) start = now;
      else if (now - start > kWaitLimitNs) {
        atomicOr(status, kStatusWaitTimeout);
        return false;
      }
    }
  }
}
// Global -> shared bulk copy completing on an mbarrier. Both addresses 16-byte aligned and the
// size a multiple of 16 bytes.
DEVI void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
DEVI void named_barrier(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

// ---- small-integer bytes -> float without I2F ---------------------------------------------------
// Byte `i` of `w` placed in the low mantissa byte of 2^23: the float 8388608 + byte, exactly.
constexpr float kMagic = 8388608.f;
template <int I>
DEVI float byte_magic(uint32_t w) {
  return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650 + I));
}

DEVI float half_lo(uint32_t w) { return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xffffu))); }
DEVI float half_hi(uint32_t w) { return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16))); }

}  // namespace dmoe
