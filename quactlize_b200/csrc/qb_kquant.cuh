// GGUF k-quant super-block formats: field offsets and the meaning of every bit, usable from host and device code.
//
// Restates the behaviour of the reference's format definitions (quactlize/include/gguf_scale_layout.hpp:56-236,
// quactlize/include/gguf_vecdot.hpp:66-281) as plain byte arithmetic.  A block holds 256 weights in G groups;
// group g has a sub-scale sc (and a sub-min mn when the format is affine); the weight of element (g,j) is
//     W = float(d)*sc*code(g,j) - float(dmin)*mn .
// ggml type numbers: Q2_K=10 Q3_K=11 Q4_K=12 Q5_K=13 Q6_K=14.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define QB_HD __host__ __device__ __forceinline__
#else
#define QB_HD inline
#endif

namespace qb {
namespace kq {

template <int QT> struct Fmt;
template <> struct Fmt<10> {  // Q2_K: scales[16] qs[64] d dmin
  static constexpr int kBytes = 84, kGroups = 16, kLo = 2, kHi = 0, kCodeBias = 0, kScaleBias = 0;
  static constexpr bool kHasMin = true, kSignedScale = false;
  static constexpr int kD = 80, kDmin = 82, kScaleOff = 0, kScaleBytes = 16, kScaleBits = 4, kMinBits = 4;
};
template <> struct Fmt<11> {  // Q3_K: hmask[32] qs[64] scales[12] d
  static constexpr int kBytes = 110, kGroups = 16, kLo = 2, kHi = 1, kCodeBias = 4, kScaleBias = 32;
  static constexpr bool kHasMin = false, kSignedScale = false;
  static constexpr int kD = 108, kDmin = -1, kScaleOff = 96, kScaleBytes = 12, kScaleBits = 6, kMinBits = 0;
};
template <> struct Fmt<12> {  // Q4_K: d dmin scales[12] qs[128]
  static constexpr int kBytes = 144, kGroups = 8, kLo = 4, kHi = 0, kCodeBias = 0, kScaleBias = 0;
  static constexpr bool kHasMin = true, kSignedScale = false;
  static constexpr int kD = 0, kDmin = 2, kScaleOff = 4, kScaleBytes = 12, kScaleBits = 6, kMinBits = 6;
};
template <> struct Fmt<13> {  // Q5_K: d dmin scales[12] qh[32] qs[128]
  static constexpr int kBytes = 176, kGroups = 8, kLo = 4, kHi = 1, kCodeBias = 0, kScaleBias = 0;
  static constexpr bool kHasMin = true, kSignedScale = false;
  static constexpr int kD = 0, kDmin = 2, kScaleOff = 4, kScaleBytes = 12, kScaleBits = 6, kMinBits = 6;
};
template <> struct Fmt<14> {  // Q6_K: ql[128] qh[64] int8 scales[16] d
  static constexpr int kBytes = 210, kGroups = 16, kLo = 4, kHi = 2, kCodeBias = 32, kScaleBias = 0;
  static constexpr bool kHasMin = false, kSignedScale = true;
  static constexpr int kD = 208, kDmin = -1, kScaleOff = 192, kScaleBytes = 16, kScaleBits = 8, kMinBits = 0;
};

template <int QT> struct Unit {          // byte-neutral packed scale unit, quactlize/include/gguf_packed_unit.hpp:39-107
  using F = Fmt<QT>;
  static constexpr int kHdr = F::kHasMin ? 4 : 2;
  static constexpr int kSbBytes = kHdr + F::kGroups * (F::kScaleBits + F::kMinBits) / 8;
  static constexpr int kSbPerUnit = (kSbBytes % 4 == 0) ? 1 : 2;
  static constexpr int kUnitTotal = kSbBytes * kSbPerUnit;
  static constexpr int kRun = F::kHasMin ? F::kGroups / 2 : F::kGroups;
  static constexpr int kRunBits = kRun * (F::kScaleBits + F::kMinBits);
  static QB_HD int bit_of(int g, int which) {
    int const base = 8 * kHdr + (g / kRun) * kRunBits;
    return which ? base + kRun * F::kScaleBits + (g % kRun) * F::kMinBits : base + (g % kRun) * F::kScaleBits;
  }
};

QB_HD int raw_bytes(int qt) { return qt == 10 ? 84 : qt == 11 ? 110 : qt == 12 ? 144 : qt == 13 ? 176 : qt == 14 ? 210 : 0; }
QB_HD int group_size(int qt) { return (qt == 12 || qt == 13) ? 32 : 16; }
QB_HD int lo_bits(int qt) { return (qt == 10 || qt == 11) ? 2 : 4; }
QB_HD int hi_bits(int qt) { return (qt == 11 || qt == 13) ? 1 : qt == 14 ? 2 : 0; }

// Integer sub-scale (the value that multiplies d) and sub-min of group g, from the format's scale bytes `s`.
template <int QT> QB_HD void scale_min(uint8_t const* s, int g, int& sc, int& mn) {
  if constexpr (QT == 12 || QT == 13) {
    int const t = g & 3;
    if (g < 4) { sc = s[t] & 63; mn = s[4 + t] & 63; }
    else { sc = (s[8 + t] & 0xF) | ((s[t] >> 6) << 4); mn = (s[8 + t] >> 4) | ((s[4 + t] >> 6) << 4); }
  } else if constexpr (QT == 10) {
    sc = s[g] & 0xF; mn = s[g] >> 4;
  } else if constexpr (QT == 14) {
    sc = int(int8_t(s[g])); mn = 0;
  } else {
    sc = (((s[g & 7] >> (4 * (g >> 3))) & 0xF) | (((s[8 + (g & 3)] >> (2 * (g >> 2))) & 3) << 4)) - 32; mn = 0;
  }
}

// Logical (signed where the format is) code of element j of group g.
template <int QT> QB_HD int code(uint8_t const* b, int g, int j) {
  if constexpr (QT == 12) {
    return (b[16 + j + 32 * (g >> 1)] >> (4 * (g & 1))) & 0xF;
  } else if constexpr (QT == 13) {
    return ((b[48 + j + 32 * (g >> 1)] >> (4 * (g & 1))) & 0xF) | (((b[16 + j] >> g) & 1) << 4);
  } else if constexpr (QT == 14) {
    int const p = g & 1, q1 = (g >> 1) & 1, n = (g >> 2) & 1, h = g >> 3;
    int const lo = (b[j + 16 * p + 32 * q1 + 64 * h] >> (4 * n)) & 0xF;
    int const hi = (b[128 + j + 16 * p + 32 * h] >> (2 * q1 + 4 * n)) & 3;
    return (lo | (hi << 4)) - 32;
  } else if constexpr (QT == 11) {
    int const lo = (b[32 + j + 16 * (g & 1) + 32 * (g >> 3)] >> (2 * ((g >> 1) & 3))) & 3;
    int const hb = (b[j + 16 * (g & 1)] >> (((g >> 1) & 3) + 4 * (g >> 3))) & 1;
    return lo - ((hb ^ 1) << 2);
  } else {
    return (b[16 + j + 16 * (g & 1) + 32 * (g >> 3)] >> (2 * ((g >> 1) & 3))) & 3;
  }
}

QB_HD uint16_t load_u16(uint8_t const* p) { return uint16_t(p[0] | (uint16_t(p[1]) << 8)); }

// Field of `bits` (<= 8) bits at bit offset `bit` of a byte string; may straddle one byte boundary.
QB_HD int get_bits(uint8_t const* u, int bit, int bits) {
  uint32_t w = u[bit >> 3];
  if ((bit & 7) + bits > 8) w |= uint32_t(u[(bit >> 3) + 1]) << 8;
  return int((w >> (bit & 7)) & ((1u << bits) - 1u));
}
QB_HD void put_bits(uint8_t* u, int bit, int bits, int v) {
  uint32_t const sh = uint32_t(v & ((1 << bits) - 1)) << (bit & 7);
  u[bit >> 3] |= uint8_t(sh & 0xFF);
  if ((bit & 7) + bits > 8) u[(bit >> 3) + 1] |= uint8_t(sh >> 8);
}

// One superblock's share of a packed unit -> integer sub-scale (bias removed / sign restored) and sub-min of group g.
template <int QT> QB_HD void unit_scale_min(uint8_t const* sb, int g, int& sc, int& mn) {
  using F = Fmt<QT>;
  using U = Unit<QT>;
  sc = get_bits(sb, U::bit_of(g, 0), F::kScaleBits);
  if constexpr (F::kSignedScale) { if (sc & (1 << (F::kScaleBits - 1))) sc -= (1 << F::kScaleBits); }
  sc -= F::kScaleBias;
  mn = 0;
  if constexpr (F::kHasMin) mn = get_bits(sb, U::bit_of(g, 1), F::kMinBits);
}

}  // namespace kq
}  // namespace qb
