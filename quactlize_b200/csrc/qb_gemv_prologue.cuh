// Activation prologue shared by the plane GEMV kernels: statistics of a 16-byte piece of a 16-bit activation row, and the
// conversion of one row into "pattern order" -- the half2 operands that a masked plane word multiplies directly.
//
// A plane word of B-bit codes holds CW = 32/B codes.  Masking it with M << (o*B) (M = two B-bit fields 16 bits apart) leaves
// the codes (h*PER + o) and (h*PER + o + 16/B) of byte lane h as an fp16 pair of value code * 2^(o*B) * 2^-24, so the
// operand for that mask is the pair of activations at those two codes times 2^(ex - o*B).  Operands are stored in the
// order the kernels consume them: word, byte lane h, field o -- NP = 16/B operands of 4 bytes per word -- in runs of
// `part_codes` codes that start `part_stride` bytes apart (the padding spreads the runs over the banks).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

#include "qb_device.cuh"

namespace qb {

// max |x| and the sum of the eight 16-bit values of one piece (fp16 or bf16); NaNs do not raise the maximum
template <bool BF16>
__device__ __forceinline__ void piece_stats(uint4 v, float& mx, float& sum) {
  uint32_t const w[4] = {v.x, v.y, v.z, v.w};
  float s = 0.f;
  if constexpr (BF16) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float const lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xFFFF0000u);
      mx = fmaxf(mx, fmaxf(fabsf(lo), fabsf(hi)));
      s += lo + hi;
    }
  } else {
    __half2 m2 = __float2half2_rn(0.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      m2 = __hmax2(m2, u32_as_h2(w[j] & 0x7FFF7FFFu));
      float2 const f = __half22float2(u32_as_h2(w[j]));
      s += f.x + f.y;
    }
    float2 const mf = __half22float2(m2);
    mx = fmaxf(mx, fmaxf(mf.x, mf.y));
  }
  sum = s;
}

template <bool BF16>
__device__ __forceinline__ float act16_to_f32(uint32_t h) {
  if constexpr (BF16) return __uint_as_float(h << 16);
  else return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}

// One activation row, raw in shared memory (`xraw`, k values), into pattern order for a B-bit plane at `dst_row`.
// `ex` is the power-of-two exponent of the row's pre-scale (operand = x * 2^(ex - o*B)).  Called by the whole CTA; one work
// item is (word, byte lane): PER = 8/B operands read from two runs of PER consecutive activations and written as one run.
// Stores are 8 bytes wide, so `dst_row` and `part_stride` need 8-byte alignment only.
template <int B, bool BF16>
__device__ __forceinline__ void pattern_row(uint16_t const* xraw, uint8_t* dst_row, int k, int ex, int part_codes, int part_stride) {
  constexpr int CW = 32 / B, PER = 8 / B, NP = 16 / B;
  uint32_t const base = uint32_t(127 + ex) << 23;
  for (int it = threadIdx.x; it < (k / CW) * 2; it += blockDim.x) {
    int const word = it >> 1, h = it & 1;
    uint16_t const* s0 = xraw + word * CW + h * PER;          // (PER * 2)-byte aligned
    uint32_t a[PER / 2], b[PER / 2];                           // two activations per 32-bit word
    if constexpr (PER == 2) {
      a[0] = *reinterpret_cast<uint32_t const*>(s0); b[0] = *reinterpret_cast<uint32_t const*>(s0 + 2 * PER);
    } else if constexpr (PER == 4) {
      uint2 const va = *reinterpret_cast<uint2 const*>(s0), vb = *reinterpret_cast<uint2 const*>(s0 + 2 * PER);
      a[0] = va.x; a[1] = va.y; b[0] = vb.x; b[1] = vb.y;
    } else {
      uint4 const va = *reinterpret_cast<uint4 const*>(s0), vb = *reinterpret_cast<uint4 const*>(s0 + 2 * PER);
      a[0] = va.x; a[1] = va.y; a[2] = va.z; a[3] = va.w; b[0] = vb.x; b[1] = vb.y; b[2] = vb.z; b[3] = vb.w;
    }
    uint32_t out[PER];
#pragma unroll
    for (int o = 0; o < PER; ++o) {
      float const mul = __uint_as_float(base - (uint32_t(o * B) << 23));
      uint32_t const e0 = (a[o >> 1] >> (16 * (o & 1))) & 0xFFFFu, e1 = (b[o >> 1] >> (16 * (o & 1))) & 0xFFFFu;
      out[o] = h2_as_u32(__floats2half2_rn(act16_to_f32<BF16>(e0) * mul, act16_to_f32<BF16>(e1) * mul));
    }
    int const pt = (word * CW) / part_codes;
    uint8_t* dst = dst_row + size_t(pt) * part_stride + size_t(word * NP + h * PER - pt * (part_codes / 2)) * 4;
#pragma unroll
    for (int o = 0; o < PER; o += 2) *reinterpret_cast<uint2*>(dst + o * 4) = make_uint2(out[o], out[o + 1]);
  }
}

}  // namespace qb
