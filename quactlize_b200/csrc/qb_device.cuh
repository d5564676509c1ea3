// Device-side building blocks shared by the GEMV kernels (sm_100a).
//
//  * bulk asynchronous copies (cp.async.bulk, the untiled TMA path) global -> shared, completing on an mbarrier,
//    with BOUNDED waits: a wait that does not complete within kWaitNs records a code in the status word and the
//    kernel finishes normally instead of hanging the GPU;
//  * the "subnormal pattern" integer -> fp16 conversion: a 16-bit lane whose upper 6 bits are zero IS the fp16
//    subnormal  value * 2^-24, so  (w & 0x000F000F)  is already a half2 holding two codes, with no magic-number
//    subtraction.  Activations are pre-scaled by a power of two per warp so the products stay in fp16's normal range.
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cstdint>

namespace qb {

constexpr unsigned long long kWaitNs = 2000000000ull;   // 2 s: far beyond any legitimate copy latency

enum DeviceWaitCode : unsigned int { kWaitOk = 0, kWaitStageTimeout = 0x51A6E001u, kWaitTmemTimeout = 0x51A6E002u,
                                     kWaitMmaTimeout = 0x51A6E003u };

__device__ __forceinline__ uint32_t smem_u32(void const* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false after kWaitNs, having written `code` to *status (first writer wins).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity, unsigned int* status, unsigned code,
                                                  unsigned long long limit_ns = kWaitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0;                                    // the clock is first read after 64 failed polls
  unsigned spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0) {
      unsigned long long const now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) {
        if (status) atomicCAS(status, 0u, code);
        return false;
      }
    }
  }
  return true;
}

// 1-D bulk copy global -> this CTA's shared memory; dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, void const* src, unsigned bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst_smem)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ uint4 lds128(void const* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
  return v;
}

__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Power-of-two activation scale for one warp: max|x| * 2^e lands in [2^(top-1), 2^top).  Zero / non-finite input -> e = 0.
__device__ __forceinline__ int pow2_scale_exponent(float maxabs, int top) {
  if (!(maxabs > 0.f) || !isfinite(maxabs)) return 0;
  int const ex = ilogbf(maxabs);          // floor(log2(maxabs)), exact for subnormals too
  return (top - 1) - ex;
}

// sum of both lanes of a half2, in fp32
__device__ __forceinline__ float h2_sum(__half2 a) {
  float2 const f = __half22float2(a);
  return f.x + f.y;
}

// byte pair (b_lo, b_hi of `w` selected by sel) -> half2 of fp16 subnormals (b * 2^-24 each)
__device__ __forceinline__ float2 bytes_to_f2(uint32_t w, uint32_t sel) {
  return __half22float2(u32_as_h2(__byte_perm(w, 0u, sel)));
}

}  // namespace qb
