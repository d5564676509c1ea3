// Shared-memory access, mbarrier polling and small bit helpers common to the warp-per-row-pair GEMV kernels
// (qb_gemv_kquant1.cu: raw blocks; qb_gemv_bc1.cu: planes + packed units).
#pragma once

#include <cstdint>

#include "qb_device.cuh"

namespace qb {

__device__ __forceinline__ uint32_t k_lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t k_lds16(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 k_lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void k_sts128(uint32_t a, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ bool k_try_wait(uint32_t bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
static __device__ __noinline__ bool k_slow_wait(uint32_t bar, unsigned parity, unsigned int* status, unsigned long long limit) {
  unsigned long long t0 = 0;                                    // the clock is first read after 64 failed polls
  unsigned spins = 0;
  while (!k_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0) {
      unsigned long long const now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit) {
        if (status) atomicCAS(status, 0u, unsigned(kWaitStageTimeout));
        return false;
      }
    }
  }
  return true;
}

// NW consecutive 32-bit words starting at shared address a.  ALIGN 16: a is 16-byte aligned (NW == 4); 4: word aligned;
// 2: only 2-byte aligned, read as NW+1 aligned words and funnel-shifted by the misalignment.
template <int ALIGN, int NW>
__device__ __forceinline__ void k_run(uint32_t a, uint32_t (&w)[NW]) {
  if constexpr (ALIGN == 16 && NW == 4) {
    uint4 const v = k_lds128(a);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
  } else if constexpr (ALIGN >= 4) {
#pragma unroll
    for (int i = 0; i < NW; ++i) w[i] = k_lds32(a + 4u * i);
  } else {
    uint32_t const a0 = a & ~3u, sh = (a & 2u) * 8u;
    uint32_t t[NW + 1];
#pragma unroll
    for (int i = 0; i <= NW; ++i) t[i] = k_lds32(a0 + 4u * i);
#pragma unroll
    for (int i = 0; i < NW; ++i) w[i] = __funnelshift_r(t[i], t[i + 1], sh);
  }
}

// byte `i` of v as a float (exact), through the 2^23 magic: (0x4B000000 | byte) - 2^23 - bias
template <int I>
__device__ __forceinline__ float k_byte_f(uint32_t v, float bias) {
  return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7440u + I)) - (8388608.f + bias);
}

}  // namespace qb
