// Merged-artifact decode GEMV (bit planes + packed scale units), one activation row per (expert, row): the copy
// structure of the raw-block single-row kernels applied to the plane layout.
//
//   out[t, r] = sum_k x[t, k] * W[r, k]
//   low   [E][n][k*lo/8]   element k of a row at bit k*lo, LSB first (lo = 2 or 4)
//   high  [E][n][k*hi/8]   the bits above the low field (hi = 0, 1 or 2); Q3_K / Q6_K codes are offset binary
//   units [E][k/256/P][n][P*sb]   per superblock: d (, dmin), then the sub-scales (and sub-mins) as bit runs
//
// Same contract as the reference's merged GEMV for these artifacts (quactlize/include/gguf_bc_vecdot.hpp:91-318; unit
// layout quactlize/include/gguf_packed_unit.hpp:39-107).
//
// Structure (sm_100a): one 16-warp CTA per SM owns a run of output rows; a warp owns (row pair, K segment of <= 16
// superblocks); a ring stage receives the pair's low-plane and high-plane row segments by cp.async.bulk and the pair's
// share of the packed units -- runs of 2 x unit bytes that lie `n` units apart in memory and are only 8-byte aligned -- as
// 8-byte cp.async pieces issued by all lanes, everything completing on ONE mbarrier (bounded waits).
//
// Lane l owns the 16-byte low-plane chunks l, l+32, ... of the segment (32 codes of a 4-bit plane, 64 of a 2-bit one):
// a warp's loads of a plane are consecutive in shared memory, where a lane that owned a contiguous run of a power-of-two
// layout would meet its neighbours in the same banks.  The lanes of one superblock read its unit share by broadcast.
// A lane keeps the 128 activations of its chunks in 64 half2 REGISTERS for the whole kernel, ordered as the planes pair
// them: an octet's registers are (x0,x4), (x1,x5), (x2,x6), (x3,x7).
//
// Arithmetic.  A 16-bit lane whose bits above bit 9 are zero read as fp16 is (field value) * 2^(shift-24), exact.  A
// 4-bit plane word holds the eight codes of an octet: its two 16-bit lanes are codes (0..3) and (4..7), so masks at bits
// 0 and 4 of the word and of the word shifted by 8 are the pairs (i, i+4).  2-bit planes hold an octet in two bytes and
// 1-bit planes in one: one byte permute puts (codes 0..3, codes 4..7) into the two lanes and field masks do the rest.
// Fields at different bit positions of one scale group carry different powers of two: they accumulate apart (8-16
// products per fp16 lane) and are joined per group by HFMA2s with constants.  Sub-scales are unpacked from the unit
// with word shifts; sub-mins and code biases use per-group sums of x from the prologue.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <map>
#include <mutex>

#include "qb_device.cuh"
#include "qb_internal.hpp"
#include "qb_kquant.cuh"
#include "qb_rowpair.cuh"
#include "qb_runtime.hpp"

namespace qb {
namespace {

struct BcArgs {
  uint8_t const* low;
  uint8_t const* high;
  uint8_t const* units;
  __half const* x;
  float* out;
  int const* offsets;        // cumulative [experts+1] (grouped) or nullptr (dense)
  int n, bpr, max_rows;      // grid.y = activation rows (dense) or experts*max_rows (grouped)
  int S, nbs, RS;            // K segments per row, superblocks per segment, row slots per CTA
  int hi_base, un_base;      // byte offsets of the high-plane and unit regions inside a ring stage
  int stage_bytes;
  int rows_q, rows_r;        // rows are dealt in pairs: CTA c owns rows_q (+2 if c < rows_r) consecutive rows, rows_q even
  unsigned int* status;
};

constexpr int kBcWarps = 16;
constexpr int kBcStages = 2;
constexpr int kBcMaxPieces = 4;      // 16-byte activation pieces per thread in the prologue (K <= 16384)

#define BC_H2(v) u32_as_h2(v)

// One 4-bit plane word = octet Q: the pairs (i, i+4) at bits 0 and 4 of the word and of the word >> 8.
// A collects the fields read at bit 0 (weight 1), B those read at bit 4 (weight 1/16).
#define BC_LO4(word, Q, A, B)                                                   \
  {                                                                             \
    uint32_t const w_ = (word), u_ = w_ >> 8;                                   \
    A = __hfma2(BC_H2(w_ & 0x000F000Fu), xr[4 * (Q) + 0], A);                   \
    B = __hfma2(BC_H2(w_ & 0x00F000F0u), xr[4 * (Q) + 1], B);                   \
    A = __hfma2(BC_H2(u_ & 0x000F000Fu), xr[4 * (Q) + 2], A);                   \
    B = __hfma2(BC_H2(u_ & 0x00F000F0u), xr[4 * (Q) + 3], B);                   \
  }
// The two 16-bit lanes hold (codes 0..3, codes 4..7) of octet Q as BITS-bit fields: field f is the pair (f, f+4),
// accumulated into ACC(f) with weight 2^(-BITS*f) still to be applied.
#define BC_FIELDS(lanes, BITS, Q, ACC)                                          \
  {                                                                             \
    uint32_t const l_ = (lanes);                                                \
    _Pragma("unroll") for (int f = 0; f < 4; ++f)                               \
      ACC(f) = __hfma2(BC_H2(l_ & (uint32_t((1u << BITS) - 1u) * 0x00010001u) << (BITS * f)), xr[4 * (Q) + f], ACC(f)); \
  }

__device__ __forceinline__ float bc_u6(uint32_t v, float bias) {      // low six bits of v as a float, minus bias (exact)
  return __uint_as_float((v & 63u) | 0x4B000000u) - (8388608.f + bias);
}
__device__ __forceinline__ float bc_u4(uint32_t v) {
  return __uint_as_float((v & 15u) | 0x4B000000u) - 8388608.f;
}

__device__ __forceinline__ uint2 bc_lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}

// Codes per 16-byte low-plane chunk, chunks per superblock, scale groups per chunk.
template <int QT> struct BcGeom {
  using F = kq::Fmt<QT>;
  static constexpr int kCodes = 128 / F::kLo;                      // 32 or 64
  static constexpr int kCps = 256 / kCodes;                        // 8 or 4
  static constexpr int kOct = kCodes / 8;                          // octets (= 16-byte activation pieces) per chunk: 4 or 8
  static constexpr int kGpc = kCodes / (256 / F::kGroups);         // 1, 2 or 4
  static constexpr int kSlots = 128 / kCodes;                      // chunks per lane for a 16-superblock segment: 4 or 2
};

// One chunk of one output row.  L, H: shared addresses of the chunk's low / high plane bytes; U: of its superblock's
// share of the packed unit; ci: the chunk's position inside its superblock.  XB, SB: where the chunk's activations and
// group sums start in xr (scaled by 2^ex, plane pair order) and sxg (sums of the unscaled x); fm = 2^(24-ex).
// Returns the chunk's share of the dot product.
template <int QT, int XB, int SB>
__device__ __forceinline__ float bc_chunk(uint32_t L, uint32_t H, uint32_t U, int ci, __half2 const (&xr)[64], float const (&sxg)[8], float fm) {
  __half2 const z = __float2half2_rn(0.f);
  uint4 const lw = k_lds128(L);
  if constexpr (QT == 14) {
    // ---- Q6_K: 4 + 2 bits, groups of 16 (two per chunk), int8 sub-scales, code - 32
    uint2 const hw = bc_lds64(H);
    uint32_t const s2 = k_lds16(U + 2u + 2u * ci) ^ 0x8080u;        // the chunk's two int8 sub-scales -> offset binary
    float const d = __half2float(__ushort_as_half((unsigned short)k_lds16(U)));
    float dsum = 0.f, bsum = 0.f;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      // weights: low at bit 0: 1, at bit 4: 1/16; high field f (read at bit 2f, worth 16): 16, 4, 1, 1/4
      __half2 a = z, b = z, h0 = z, h1 = z, h3 = z;
      BC_LO4(t ? lw.z : lw.x, XB / 4 + 2 * t, a, b)
      BC_LO4(t ? lw.w : lw.y, XB / 4 + 2 * t + 1, a, b)
      uint32_t const hw_t = t ? hw.y : hw.x;
      uint32_t const l0 = __byte_perm(hw_t, 0u, 0x4140), l1 = __byte_perm(hw_t, 0u, 0x4342);
      h0 = __hfma2(BC_H2(l0 & 0x00030003u), xr[XB + 8 * t + 0], h0);
      h1 = __hfma2(BC_H2(l0 & 0x000C000Cu), xr[XB + 8 * t + 1], h1);
      a = __hfma2(BC_H2(l0 & 0x00300030u), xr[XB + 8 * t + 2], a);
      h3 = __hfma2(BC_H2(l0 & 0x00C000C0u), xr[XB + 8 * t + 3], h3);
      h0 = __hfma2(BC_H2(l1 & 0x00030003u), xr[XB + 8 * t + 4], h0);
      h1 = __hfma2(BC_H2(l1 & 0x000C000Cu), xr[XB + 8 * t + 5], h1);
      a = __hfma2(BC_H2(l1 & 0x00300030u), xr[XB + 8 * t + 6], a);
      h3 = __hfma2(BC_H2(l1 & 0x00C000C0u), xr[XB + 8 * t + 7], h3);
      __half2 tot = __hfma2(b, __float2half2_rn(0.0625f), a);
      tot = __hfma2(h3, __float2half2_rn(0.25f), tot);
      tot = __hfma2(h1, __float2half2_rn(4.f), tot);
      tot = __hfma2(h0, __float2half2_rn(16.f), tot);
      float const sc = t ? k_byte_f<1>(s2, 128.f) : k_byte_f<0>(s2, 128.f);
      dsum = fmaf(sc, h2_sum(tot), dsum);
      bsum = fmaf(sc, sxg[SB + t], bsum);
    }
    return d * fmaf(fm, dsum, -32.f * bsum);
  } else if constexpr (QT == 13 || QT == 12) {
    // ---- Q5_K: 4 + 1 bits, Q4_K: 4 bits; groups of 32 (one per chunk), 6-bit sub-scales and sub-mins
    uint4 const un = k_lds128(U);                                   // the whole 16-byte unit: d dmin | run 0 | run 1
    // run h = 3 bytes of four 6-bit sub-scales, then 3 bytes of four 6-bit sub-mins, at byte 4 + 6h
    int const h = ci >> 2, g6 = 6 * (ci & 3);
    uint32_t const r0 = h ? __funnelshift_r(un.z, un.w, 16) : un.y; // bytes 0-3 of the run
    uint32_t const r1 = h ? (un.w >> 16) : un.z;                    // bytes 4-5
    uint32_t const mn24 = __funnelshift_r(r0, r1, 24);
    float2 const dd = __half22float2(u32_as_h2(un.x));
    __half2 a = z, b = z;
    BC_LO4(lw.x, XB / 4 + 0, a, b)
    BC_LO4(lw.y, XB / 4 + 1, a, b)
    BC_LO4(lw.z, XB / 4 + 2, a, b)
    BC_LO4(lw.w, XB / 4 + 3, a, b)
    __half2 tot = __hfma2(b, __float2half2_rn(0.0625f), a);
    if constexpr (QT == 13) {
      // a byte of the 1-bit plane is an octet: lanes (byte, byte >> 4) hold (codes 0..3, codes 4..7) at bits 0..3;
      // the bit read at position f is worth 16: weights 16, 8, 4, 2
      uint32_t const w = k_lds32(H), sft = w >> 4;
      __half2 hh[4] = {z, z, z, z};
#define ACC_(f) hh[f]
      BC_FIELDS(__byte_perm(w, sft, 0x4400), 1, XB / 4 + 0, ACC_)
      BC_FIELDS(__byte_perm(w, sft, 0x5511), 1, XB / 4 + 1, ACC_)
      BC_FIELDS(__byte_perm(w, sft, 0x6622), 1, XB / 4 + 2, ACC_)
      BC_FIELDS(__byte_perm(w, sft, 0x7733), 1, XB / 4 + 3, ACC_)
#undef ACC_
      __half2 hs = __hfma2(hh[3], __float2half2_rn(0.5f), hh[2]);
      hs = __hfma2(hs, __float2half2_rn(0.5f), hh[1]);
      hs = __hfma2(hs, __float2half2_rn(0.5f), hh[0]);
      tot = __hfma2(hs, __float2half2_rn(16.f), tot);
    }
    float const sc = bc_u6(r0 >> g6, 0.f), mn = bc_u6(mn24 >> g6, 0.f);
    return fmaf(dd.x * fm, sc * h2_sum(tot), -dd.y * (mn * sxg[SB]));
  } else {
    // ---- Q3_K: 2 + 1 bits, 6-bit sub-scales minus 32, code - 4; Q2_K: 2 bits, 4-bit sub-scales and sub-mins;
    // groups of 16 (four per chunk: word t of the chunk is group t)
    uint32_t sv, mv = 0u;
    float d, dmin = 0.f;
    uint2 hw = make_uint2(0u, 0u);
    if constexpr (QT == 11) {
      hw = bc_lds64(H);
      uint32_t const at = U + 2u + 3u * ci, a0 = at & ~3u;          // four 6-bit sub-scales: 3 bytes at any byte address
      sv = __funnelshift_r(k_lds32(a0), k_lds32(a0 + 4u), (at & 3u) * 8u);
      d = __half2float(__ushort_as_half((unsigned short)k_lds16(U)));
    } else {
      uint32_t const at = U + 4u + 8u * (ci >> 1) + 2u * (ci & 1);  // four scale nibbles; the four min nibbles 4 bytes on
      sv = k_lds16(at); mv = k_lds16(at + 4u);
      float2 const dd = __half22float2(u32_as_h2(k_lds32(U)));
      d = dd.x; dmin = dd.y;
    }
    float dsum = 0.f, bsum = 0.f;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      uint32_t const w = t == 0 ? lw.x : t == 1 ? lw.y : t == 2 ? lw.z : lw.w;   // 16 codes = the group's two octets
      // low field f read at bit 2f: weights 1, 1/4, 1/16, 1/64; the high bit read at position f is worth 4: 4, 2, 1, 1/2
      __half2 l0 = z, l1 = z, l2 = z, l3 = z;
      uint32_t const p0 = __byte_perm(w, 0u, 0x4140), p1 = __byte_perm(w, 0u, 0x4342);
      l0 = __hfma2(BC_H2(p0 & 0x00030003u), xr[XB + 8 * t + 0], l0);
      l1 = __hfma2(BC_H2(p0 & 0x000C000Cu), xr[XB + 8 * t + 1], l1);
      l2 = __hfma2(BC_H2(p0 & 0x00300030u), xr[XB + 8 * t + 2], l2);
      l3 = __hfma2(BC_H2(p0 & 0x00C000C0u), xr[XB + 8 * t + 3], l3);
      l0 = __hfma2(BC_H2(p1 & 0x00030003u), xr[XB + 8 * t + 4], l0);
      l1 = __hfma2(BC_H2(p1 & 0x000C000Cu), xr[XB + 8 * t + 5], l1);
      l2 = __hfma2(BC_H2(p1 & 0x00300030u), xr[XB + 8 * t + 6], l2);
      l3 = __hfma2(BC_H2(p1 & 0x00C000C0u), xr[XB + 8 * t + 7], l3);
      __half2 tot;
      if constexpr (QT == 11) {
        // the group's two octets are bytes 2*(t&1), 2*(t&1)+1 of high word t>>1
        uint32_t const m = (t >> 1) ? hw.y : hw.x, sft = m >> 4;
        uint32_t const q0 = (t & 1) ? __byte_perm(m, sft, 0x6622) : __byte_perm(m, sft, 0x4400);
        uint32_t const q1 = (t & 1) ? __byte_perm(m, sft, 0x7733) : __byte_perm(m, sft, 0x5511);
        __half2 g0 = z, g1 = z, g3 = z;                             // the bit at position 2 (worth 1) joins l0
        g0 = __hfma2(BC_H2(q0 & 0x00010001u), xr[XB + 8 * t + 0], g0);
        g1 = __hfma2(BC_H2(q0 & 0x00020002u), xr[XB + 8 * t + 1], g1);
        l0 = __hfma2(BC_H2(q0 & 0x00040004u), xr[XB + 8 * t + 2], l0);
        g3 = __hfma2(BC_H2(q0 & 0x00080008u), xr[XB + 8 * t + 3], g3);
        g0 = __hfma2(BC_H2(q1 & 0x00010001u), xr[XB + 8 * t + 4], g0);
        g1 = __hfma2(BC_H2(q1 & 0x00020002u), xr[XB + 8 * t + 5], g1);
        l0 = __hfma2(BC_H2(q1 & 0x00040004u), xr[XB + 8 * t + 6], l0);
        g3 = __hfma2(BC_H2(q1 & 0x00080008u), xr[XB + 8 * t + 7], g3);
        __half2 lo = __hfma2(l3, __float2half2_rn(0.25f), l2);      // (l2 + l3/4) / 16 + l1/4 + l0
        lo = __hfma2(lo, __float2half2_rn(0.0625f), l0);
        lo = __hfma2(l1, __float2half2_rn(0.25f), lo);
        lo = __hfma2(g3, __float2half2_rn(0.5f), lo);
        lo = __hfma2(g1, __float2half2_rn(2.f), lo);
        tot = __hfma2(g0, __float2half2_rn(4.f), lo);
      } else {
        __half2 lo = __hfma2(l3, __float2half2_rn(0.25f), l2);
        lo = __hfma2(lo, __float2half2_rn(0.0625f), l0);
        tot = __hfma2(l1, __float2half2_rn(0.25f), lo);
      }
      float const gsum = h2_sum(tot);
      if constexpr (QT == 11) {
        float const sc = bc_u6(sv >> (6 * t), 32.f);
        dsum = fmaf(sc, gsum, dsum);
        bsum = fmaf(sc, sxg[SB + t], bsum);
      } else {
        dsum = fmaf(bc_u4(sv >> (4 * t)), gsum, dsum);
        bsum = fmaf(bc_u4(mv >> (4 * t)), sxg[SB + t], bsum);
      }
    }
    if constexpr (QT == 11) return d * fmaf(fm, dsum, -4.f * bsum);
    else return fmaf(d * fm, dsum, -dmin * bsum);
  }
}

// A lane's chunks of one row: slot j is chunk (lane + 32j) of the segment.  lo / hi / un: the slots' byte offsets inside
// the stage for the first row of the pair.
template <int QT>
__device__ __forceinline__ float bc_row_dot(uint32_t st, uint32_t dl, uint32_t dh, uint32_t du, uint32_t const (&lo)[4],
                                            uint32_t const (&hi)[4], uint32_t const (&un)[4], int ci,
                                            __half2 const (&xr)[64], float const (&sxg)[8], float fm) {
  using GM = BcGeom<QT>;
  uint32_t const sl = st + dl, sh = st + dh, su = st + du;        // dl, dh, du: the row's offsets inside the stage's regions
  float r = bc_chunk<QT, 0, 0>(sl + lo[0], sh + hi[0], su + un[0], ci, xr, sxg, fm);
  r += bc_chunk<QT, 64 / GM::kSlots, GM::kGpc>(sl + lo[1], sh + hi[1], su + un[1], ci, xr, sxg, fm);
  if constexpr (GM::kSlots == 4) {
    r += bc_chunk<QT, 32, 2 * GM::kGpc>(sl + lo[2], sh + hi[2], su + un[2], ci, xr, sxg, fm);
    r += bc_chunk<QT, 48, 3 * GM::kGpc>(sl + lo[3], sh + hi[3], su + un[3], ci, xr, sxg, fm);
  }
  return r;
}

template <int QT>
__global__ void __launch_bounds__(kBcWarps * 32, 1) bc_gemv1_kernel(BcArgs a) {
  using F = kq::Fmt<QT>;
  using UN = kq::Unit<QT>;
  using GM = BcGeom<QT>;
  constexpr int G = F::kGroups;
  constexpr int LBS = 32 * F::kLo, HBS = 32 * F::kHi;              // plane bytes per superblock
  constexpr int UB = UN::kUnitTotal, P = UN::kSbPerUnit, SBB = UN::kSbBytes;
  constexpr int UD2 = UB / 4;                                      // 8-byte pieces of one unit for a row pair (2 * UB / 8)
  constexpr int PPG = (256 / G) / 8;                               // 16-byte activation pieces per group: 2 or 4
  constexpr int OPC = GM::kOct, CPS = GM::kCps, GPC = GM::kGpc, SLOTS = GM::kSlots;
  constexpr int HCB = 16 * F::kHi / F::kLo;                        // high-plane bytes per chunk
  static_assert((P == 1 ? 16 : 9) * UD2 <= 96, "a segment's unit pieces fit three per lane");
  extern __shared__ __align__(128) uint8_t smem[];
  int const T = blockDim.x, W = T >> 5, warp = __shfl_sync(0xffffffffu, int(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  int const seg = warp % a.S, rslot = warp / a.S;
  int e = 0, arow;
  // Under programmatic dependent launch the offsets and the activation may be the preceding kernel's output: nothing of
  // them is read before this wait (it also precedes the early return of surplus CTAs).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (a.offsets) {
    e = blockIdx.y / a.max_rows;
    int const r = blockIdx.y % a.max_rows, r0 = a.offsets[e], r1 = a.offsets[e + 1];
    if (r >= r1 - r0) return;                                     // uniform for the CTA
    arow = r0 + r;
  } else {
    arow = blockIdx.y;
  }
  int const bpr = a.bpr, k = bpr * 256;
  // shared memory map: activations (octet o of the row's chunk c at (o*(NC+1) + c)*16, NC chunks per row: the lanes of a
  // warp read consecutive pieces, the prologue's writes are spread by the odd pitch), group sums, scratch, rings, barriers
  int const NC = bpr * CPS;
  uint32_t const s0 = smem_u32(smem);
  uint32_t const xa32 = s0;
  uint32_t const sx32 = xa32 + uint32_t(OPC * (NC + 1)) * 16u;    // bpr*G floats
  uint32_t const red32 = sx32 + uint32_t(bpr) * G * 4u;           // 32 words of reduction scratch and claim counters
  uint32_t const stage_bytes = uint32_t(a.stage_bytes);
  uint32_t const ring32 = red32 + 128u + uint32_t(warp) * kBcStages * stage_bytes;
  uint32_t const bar32 = red32 + 128u + uint32_t(W) * kBcStages * stage_bytes + uint32_t(warp) * kBcStages * 8u;
  uint32_t const part32 = red32 + 128u + uint32_t(W) * kBcStages * (stage_bytes + 8u);
  float* red = reinterpret_cast<float*>(smem + (red32 - s0));
  float* part = reinterpret_cast<float*>(smem + (part32 - s0));

  // ---- 1. activation pieces -> registers, requested BEFORE the weight copies so they do not queue behind them
  int const npieces = k >> 3;
  uint4 const* xg = reinterpret_cast<uint4 const*>(a.x + size_t(arow) * k);
  uint4 pc[kBcMaxPieces];
#pragma unroll
  for (int j = 0; j < kBcMaxPieces; ++j) {
    int const p = threadIdx.x + j * T;
    pc[j] = p < npieces ? __ldg(xg + p) : make_uint4(0, 0, 0, 0);
  }

  // ---- 2. weight ring: barriers and the first row pairs
  int const b0 = seg * a.nbs;                                      // first superblock of the warp's segment
  int const nb_seg = min(a.nbs, bpr - b0);
  int const u_first = b0 / P, nu_seg = (b0 + nb_seg - 1) / P - u_first + 1;
  int const cx = blockIdx.x;
  int const row0 = cx * a.rows_q + 2 * min(cx, a.rows_r);
  int const nrows = a.rows_q + (cx < a.rows_r ? 2 : 0);
  int const npairs = nrows >> 1;
  unsigned const lo_row = unsigned(bpr) * LBS, hi_row = unsigned(bpr) * HBS;       // plane bytes of a whole row
  unsigned const lo_copy = unsigned(nb_seg) * LBS, hi_copy = unsigned(nb_seg) * HBS;
  unsigned const lo_stride = unsigned(a.nbs) * LBS, hi_stride = unsigned(a.nbs) * HBS;   // row 1 of a pair inside a stage
  bool const contiguous = a.S == 1;                               // a whole row per segment: the two rows are adjacent
  size_t const wrow = size_t(e) * a.n + size_t(row0);
  uint8_t const* lo_base = a.low + wrow * lo_row + size_t(b0) * LBS;
  uint8_t const* hi_base = HBS ? a.high + wrow * hi_row + size_t(b0) * HBS : nullptr;
  // unit u of row r of expert e lies at ((e*(bpr/P) + u)*n + r)*UB: the units of a row pair are 2*UB contiguous bytes
  uint8_t const* un_base = a.units + ((size_t(e) * (bpr / P) + size_t(u_first)) * a.n + size_t(row0)) * UB;
  unsigned const un_pitch = unsigned(a.n) * UB;                    // bytes between consecutive units of a row
  // this lane's 8-byte pieces of a pair's units: piece i = lane + 32t is piece (i % UD2) of unit (i / UD2)
  unsigned uo[3];
#pragma unroll
  for (int t = 0; t < 3; ++t) {
    unsigned const i = unsigned(lane) + 32u * t, ul = i / unsigned(UD2), rem = i - ul * unsigned(UD2);
    uo[t] = i < unsigned(nu_seg) * UD2 ? ul * un_pitch + 8u * rem : 0xFFFFFFFFu;
  }
  auto bulk = [](uint32_t dst, uint8_t const* src, unsigned bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
  };
  // Executed by the whole warp: lane 0 arms the barrier and issues the plane copies, every lane issues its pieces of the
  // units and lets the barrier track them.  A barrier phase = 1 arrival with the byte count + 32 tracked arrivals.
  // (Every CTA owns whole row pairs: the rows are dealt in pairs.)
  auto issue_pair = [&](int pair, uint32_t dst, uint32_t bar) {
    if (lane == 0) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2u * (lo_copy + hi_copy)) : "memory");
      uint8_t const* ls = lo_base + size_t(2 * pair) * lo_row;
      if (contiguous) {
        bulk(dst, ls, 2u * lo_copy, bar);
      } else {
        bulk(dst, ls, lo_copy, bar);
        bulk(dst + lo_stride, ls + lo_row, lo_copy, bar);
      }
      if constexpr (HBS != 0) {
        uint8_t const* hs = hi_base + size_t(2 * pair) * hi_row;
        uint32_t const hd = dst + uint32_t(a.hi_base);
        if (contiguous) {
          bulk(hd, hs, 2u * hi_copy, bar);
        } else {
          bulk(hd, hs, hi_copy, bar);
          bulk(hd + hi_stride, hs + hi_row, hi_copy, bar);
        }
      }
    }
    uint8_t const* us = un_base + size_t(2 * pair) * UB;
    uint32_t const ud = dst + uint32_t(a.un_base) + 8u * lane;
#pragma unroll
    for (int t = 0; t < 3; ++t)
      if (uo[t] != 0xFFFFFFFFu)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(ud + 256u * t), "l"(us + uo[t]) : "memory");
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
  };
  // Beyond the first two pairs of every warp, row pairs are claimed from a per-segment counter by whichever warp has a
  // free stage: the CTA's pairs rarely divide evenly over its warps.  Which warp computes a row does not change the
  // row's arithmetic.
  static_assert(kBcStages == 2, "the claim bookkeeping below keeps two pairs per warp");
  int* claim = reinterpret_cast<int*>(red) + 16;                  // [S] next unclaimed pair per K segment (S <= 16)
  if (int(threadIdx.x) < a.S) claim[threadIdx.x] = kBcStages * a.RS;   // visible after the prologue's barriers
  int cur = rslot < npairs ? rslot : -1;                          // pair held by the stage consumed next
  int nxt = rslot + a.RS < npairs ? rslot + a.RS : -1;            // ... and by the other stage
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kBcStages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 33;" ::"r"(bar32 + 8u * s) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  if (cur >= 0) issue_pair(cur, ring32, bar32);
  if (nxt >= 0) issue_pair(nxt, ring32 + stage_bytes, bar32 + 8u);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // ---- 3. CTA-wide max|x| -> power-of-two scale
  __half2 m2 = __float2half2_rn(0.f);
#pragma unroll
  for (int j = 0; j < kBcMaxPieces; ++j) {
    if (j * T >= npieces) break;
    uint32_t const* v = reinterpret_cast<uint32_t const*>(&pc[j]);
#pragma unroll
    for (int q = 0; q < 4; ++q) m2 = __hmax2_nan(m2, u32_as_h2(v[q] & 0x7FFF7FFFu));
  }
  float mx = fmaxf(__low2float(m2), __high2float(m2));
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < W; ++w) mx = fmaxf(mx, red[w]);
  int const ex = pow2_scale_exponent(mx, 15);
  float const scl = __int_as_float((ex + 127) << 23);             // exact power of two (ex is within [-2, 39])
  float const fm = __int_as_float((24 - ex + 127) << 23);

  // ---- 4. scaled activations in plane pair order ((x0,x4),(x1,x5),(x2,x6),(x3,x7) per octet) and group sums -> shared memory
#pragma unroll
  for (int j = 0; j < kBcMaxPieces; ++j) {
    if (j * T >= npieces) break;                                  // uniform for the CTA
    int const p = threadIdx.x + j * T;
    bool const valid = p < npieces;                               // whole warps are valid or not (npieces % 32 == 0)
    uint32_t const* v = reinterpret_cast<uint32_t const*>(&pc[j]);
    float2 const f0 = __half22float2(u32_as_h2(v[0])), f1 = __half22float2(u32_as_h2(v[1]));
    float2 const f2 = __half22float2(u32_as_h2(v[2])), f3 = __half22float2(u32_as_h2(v[3]));
    float gsum = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
    gsum += __shfl_xor_sync(0xffffffffu, gsum, 1);
    if (PPG == 4) gsum += __shfl_xor_sync(0xffffffffu, gsum, 2);
    if (valid) {
      uint4 o;
      o.x = h2_as_u32(__floats2half2_rn(f0.x * scl, f2.x * scl)); o.y = h2_as_u32(__floats2half2_rn(f0.y * scl, f2.y * scl));
      o.z = h2_as_u32(__floats2half2_rn(f1.x * scl, f3.x * scl)); o.w = h2_as_u32(__floats2half2_rn(f1.y * scl, f3.y * scl));
      k_sts128(xa32 + uint32_t(((p % OPC) * (NC + 1) + p / OPC) * 16), o);
      if ((p & (PPG - 1)) == 0) reinterpret_cast<float*>(smem + (sx32 - s0))[p / PPG] = gsum;
    }
  }
  __syncthreads();

  // ---- 5. this lane's activation registers and stage offsets: slot j is chunk (lane + 32j) of the warp's segment.  Slots
  // beyond the segment keep zero activations (their weights, read from chunk 0, then add nothing).
  int const nch = nb_seg * CPS;
  int const ci = lane % CPS;
  __half2 xr[64];
  float sxg[8];
  uint32_t lo_o[4], hi_o[4], un_o[4];
#pragma unroll
  for (int i = 0; i < 8; ++i) sxg[i] = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (j >= SLOTS) { lo_o[j] = 0u; hi_o[j] = 0u; un_o[j] = 0u; continue; }
    int const c = lane + 32 * j;
    bool const valid = c < nch;
    int const cs = valid ? c : 0, b = b0 + cs / CPS;
    lo_o[j] = uint32_t(cs) * 16u;
    hi_o[j] = uint32_t(a.hi_base) + uint32_t(cs) * HCB;
    un_o[j] = uint32_t(a.un_base) + uint32_t(b / P - u_first) * (2u * UB) + uint32_t(b % P) * SBB;
    int const cg = b0 * CPS + cs;                                  // the chunk's index in the row
#pragma unroll
    for (int o = 0; o < OPC; ++o) {
      uint4 v = k_lds128(xa32 + uint32_t((o * (NC + 1) + cg) * 16));
      if (!valid) v = make_uint4(0u, 0u, 0u, 0u);
      int const q = j * OPC + o;
      xr[4 * q + 0] = u32_as_h2(v.x); xr[4 * q + 1] = u32_as_h2(v.y); xr[4 * q + 2] = u32_as_h2(v.z); xr[4 * q + 3] = u32_as_h2(v.w);
    }
#pragma unroll
    for (int t = 0; t < GPC; ++t) {
      float const sv = __uint_as_float(k_lds32(sx32 + uint32_t((cg * GPC + t) * 4)));
      sxg[j * GPC + t] = valid ? sv : 0.f;
    }
  }

  // ---- 6. main loop: one stage = the segments of two consecutive rows
  uint32_t st_addr = ring32, st_bar = bar32;
  unsigned phase = 0;
  int st = 0;
  float p0 = 0.f, p1 = 0.f;                                       // previous pair's per-lane partial sums
  int plr = nrows;                                                // ... and its CTA-local row (nrows = scratch slot)
  auto reduce_store = [&](float t0, float t1, int row_l) {
    float v = (lane & 16) ? t1 : t0;
    float const u = (lane & 16) ? t0 : t1;
    v += __shfl_xor_sync(0xffffffffu, u, 16);
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    if ((lane & 15) == 0) part[(row_l + (lane >> 4)) * a.S + seg] = v;   // rows nrows, nrows+1 are scratch
  };
  bool gave_up = false;
  while (cur >= 0) {
    if (!k_try_wait(st_bar, phase) && !k_slow_wait(st_bar, phase, a.status, kWaitNs)) { gave_up = true; break; }
    float const t0 = bc_row_dot<QT>(st_addr, 0u, 0u, 0u, lo_o, hi_o, un_o, ci, xr, sxg, fm);
    float const t1 = bc_row_dot<QT>(st_addr, lo_stride, hi_stride, uint32_t(UB), lo_o, hi_o, un_o, ci, xr, sxg, fm);
    reduce_store(p0, p1, plr);
    p0 = t0; p1 = t1;
    plr = 2 * cur;
    __syncwarp();
    int c = -1;
    if (lane == 0) {
      c = atomicAdd(&claim[seg], 1);
      if (c >= npairs) c = -1;
    }
    c = __shfl_sync(0xffffffffu, c, 0);
    if (c >= 0) issue_pair(c, st_addr, st_bar);
    cur = nxt; nxt = c;
    st_addr += stage_bytes; st_bar += 8u;
    if (++st == kBcStages) { st = 0; st_addr = ring32; st_bar = bar32; phase ^= 1u; }
  }
  reduce_store(p0, p1, plr);
  if (gave_up && nxt >= 0) {
    // a wait gave up: drain this warp's other copy still in flight (bounded, short) before the shared memory can be handed
    // to another CTA
    uint32_t const ob = st == 0 ? bar32 + 8u : bar32;
    unsigned const op = st == 0 ? phase : (phase ^ 1u);
    if (!k_try_wait(ob, op)) (void)k_slow_wait(ob, op, nullptr, 250000000ull);
  }
  __syncthreads();
  for (int r = threadIdx.x; r < nrows; r += T) {
    float s = 0.f;
    for (int sg = 0; sg < a.S; ++sg) s += part[r * a.S + sg];
    a.out[size_t(arow) * a.n + row0 + r] = s;
  }
}

struct BcPlan { int S, nbs, RS, gx, W, hi_base, un_base, stage_bytes; size_t smem; bool ok; };

template <int QT>
BcPlan const& bc_plan(int n, int bpr, int gy) {
  using F = kq::Fmt<QT>;
  using UN = kq::Unit<QT>;
  struct Key { int n, bpr, gy, dev; bool operator<(Key const& o) const {
    return n != o.n ? n < o.n : bpr != o.bpr ? bpr < o.bpr : gy != o.gy ? gy < o.gy : dev < o.dev; } };
  static std::map<Key, BcPlan> cache;
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(mu);
  Key const key{n, bpr, gy, dev};
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  BcPlan p{};
  auto kern = bc_gemv1_kernel<QT>;
  constexpr int LBS = 32 * F::kLo, HBS = 32 * F::kHi, P = UN::kSbPerUnit, UB = UN::kUnitTotal;
  p.S = (bpr + 15) / 16;
  // rows come in pairs whose units are copied together: n even; a unit never straddles two rows' superblock counts
  p.ok = p.S <= kBcWarps && n % 2 == 0 && bpr % P == 0 && size_t(bpr / P) * n * UB < (size_t(1) << 31);
  if (p.ok) {
    p.nbs = (bpr + p.S - 1) / p.S;
    p.RS = std::max(1, kBcWarps / p.S);
    p.W = p.S * p.RS;
    if (p.W * 32 * kBcMaxPieces * 8 < bpr * 256) p.ok = false;
    int const nu_max = P == 1 ? p.nbs : p.nbs / 2 + 1;             // units a segment can touch
    p.hi_base = 2 * p.nbs * LBS;
    p.un_base = p.hi_base + 2 * p.nbs * HBS;
    // the sub-scale runs are read as aligned words and may reach two words past the last unit
    p.stage_bytes = (p.un_base + nu_max * 2 * UB + 16 + 15) / 16 * 16;
    size_t const fixed = size_t(bpr) * 512 + 128 + size_t(bpr) * F::kGroups * 4 + 128 + size_t(p.W) * kBcStages * (p.stage_bytes + 8);
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) { (void)cudaGetLastError(); p.ok = false; }
    int const sms = rt_sm_count();
    int const resident = std::max(1, sms / std::max(1, std::min(gy, 8)));
    // every CTA starts on an even row: rows_q even, and the first rows_r CTAs (one extra row each) would break that,
    // so the rows are dealt in pairs
    int const pairs = n / 2;
    p.gx = std::max(1, std::min(resident, (pairs + p.RS - 1) / p.RS));
    p.smem = fixed + size_t(2 * ((pairs + p.gx - 1) / p.gx) + 4) * p.S * 4;
    if (p.smem > 227 * 1024) p.ok = false;
  }
  return cache.emplace(key, p).first->second;
}

template <int QT>
int enqueue_bc1(PlaneGemvDesc const& d, unsigned int* status, cudaStream_t stream) {
  int const bpr = d.k / 256;
  int const gy = d.offsets ? d.experts * d.max_rows : d.m_rows;
  if (gy <= 0 || gy > 65535) return 40;
  BcPlan const& p = bc_plan<QT>(d.n, bpr, gy);
  if (!p.ok) return 40;
  BcArgs a{};
  a.low = d.low; a.high = d.high; a.units = d.units; a.x = static_cast<__half const*>(d.act); a.out = static_cast<float*>(d.out);
  a.offsets = d.offsets; a.n = d.n; a.bpr = bpr; a.max_rows = d.max_rows;
  a.S = p.S; a.nbs = p.nbs; a.RS = p.RS; a.hi_base = p.hi_base; a.un_base = p.un_base; a.stage_bytes = p.stage_bytes; a.status = status;
  // rows are dealt to the CTAs in pairs, so that every CTA starts on an even row
  int const pairs = d.n / 2;
  a.rows_q = 2 * (pairs / p.gx); a.rows_r = pairs % p.gx;
  static bool const no_pdl = std::getenv("QUACTLIZE_B200_NO_PDL") != nullptr;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.gx, gy); cfg.blockDim = dim3(p.W * 32); cfg.dynamicSmemBytes = p.smem; cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = no_pdl ? 0 : 1;
  if (cudaLaunchKernelEx(&cfg, bc_gemv1_kernel<QT>, a) != cudaSuccess) { (void)cudaGetLastError(); return 40; }
  return 0;
}

}  // namespace

// Merged artifact (scale_mode 1), fp16 activations, fp32 output, one activation row per weight pass.  0 = enqueued;
// 40 = outside this kernel's envelope (the caller then uses another kernel).
int enqueue_bc_gemv1(PlaneGemvDesc const& d, cudaStream_t stream) {
  if (d.scale_mode != 1 || d.act_bf16 || d.out_kind != 1 || d.k <= 0 || d.k % 256) return 40;
  auto aligned = [](void const* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (!aligned(d.low) || (d.hi_bits && !aligned(d.high)) || !aligned(d.units) || !aligned(d.act)) return 40;
  unsigned int* status = rt_device_status_ptr();
  if (!status) return 40;
  switch (d.qtype) {
    case 10: return enqueue_bc1<10>(d, status, stream);
    case 11: return enqueue_bc1<11>(d, status, stream);
    case 12: return enqueue_bc1<12>(d, status, stream);
    case 13: return enqueue_bc1<13>(d, status, stream);
    case 14: return enqueue_bc1<14>(d, status, stream);
    default: return 40;
  }
}

}  // namespace qb
