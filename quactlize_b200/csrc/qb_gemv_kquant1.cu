// Raw-block decode GEMV for the four k-quant formats beside Q4_K (Q2_K, Q3_K, Q5_K, Q6_K), one activation row per
// (expert, row): the copy structure of the Q4_K single-row kernel with a decode per format.
//
//   out[t, r] = sum_k x[t, k] * W[r, k],   W = raw blocks [E][n][k/256][84|110|176|210] row-major by output row.
//
// Same contract as vecdot_rows_kernel of the reference for these formats (quactlize/include/gguf_vecdot.hpp:604-760, one
// template over the five formats there too; bit meaning quactlize/include/gguf_vecdot.hpp:66-281).
//
// Structure (sm_100a), as in qb_gemv_q4k.cu: one 16-warp CTA per SM owns a run of output rows; a warp owns (row pair,
// K segment of <= 16 blocks); row segments arrive by cp.async.bulk into the warp's private ring (mbarrier completion,
// bounded waits); two lanes share a block, each taking the half with groups [G/2*prt, G/2*prt + G/2) = 128 codes, whose
// 128 activations it keeps in 64 half2 REGISTERS for the whole kernel.  The activation is scaled by one power of two per
// CTA; programmatic dependent launch.
//
// Arithmetic.  The code bytes of these formats hold several fields per byte, each field belonging to ANOTHER group but
// the same element position, and neighbouring bytes hold neighbouring elements.  So one PRMT spreads bytes (j, j+1) of a
// word over the two 16-bit lanes of a register, and (lanes & field mask) read as half2 is (c_j, c_j+1) * 2^(shift-24): an
// fp16 subnormal pair, exact, multiplied straight into the natural-order activation pair by one HFMA2.  The high planes
// (Q3_K's hmask bit, Q5_K's fifth bit, Q6_K's two high bits) are further fields of the same kind, accumulated apart and
// joined to their low plane by one HFMA2 with a power of two per group.  Group sums (8 or 16 products per fp16 lane) go
// to fp32 with the group's sub-scale; sub-mins and code biases use per-group sums of x from the prologue.
//
// Blocks of 84, 110 and 210 bytes are only 4- or 2-byte aligned in a row: code runs are read as aligned words and, for the
// 2-byte case, funnel-shifted by the lane's misalignment.  A K segment that does not start on a 16-byte boundary is
// copied from the boundary below it (the row itself must be a multiple of 16 bytes, else the caller uses the plain kernel).
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

struct KqArgs {
  uint8_t const* blocks;
  __half const* x;
  float* out;
  int const* offsets;        // cumulative [experts+1] (grouped) or nullptr (dense)
  int n, bpr, max_rows;      // grid.y = activation rows (dense) or experts*max_rows (grouped)
  int S, nbs, RS;            // K segments per row, blocks per segment, row slots per CTA
  int seg_stride;            // bytes between the two row segments of a ring stage
  int rows_q, rows_r;        // n = gridDim.x*rows_q + rows_r: CTA c owns rows_q (+1 if c < rows_r) consecutive rows
  unsigned int* status;
};

constexpr int kKqWarps = 16;
constexpr int kKqStages = 2;
constexpr int kKqMaxPieces = 4;      // 16-byte activation pieces per thread in the prologue (K <= 16384)

// A word of code bytes (elements j..j+3) with NF fields of BITS bits per byte: field f of the word multiplies the
// activation pairs xa[f][0], xa[f][1] into acc[f].  MASK0 is the mask of field 0 in both 16-bit lanes.
#define KQ_WORD(word, NF, BITS, MASK0, ACC, XI)                                                   \
  {                                                                                                \
    uint32_t const l01 = __byte_perm(word, 0u, 0x4140), l23 = __byte_perm(word, 0u, 0x4342);       \
    _Pragma("unroll") for (int f = 0; f < NF; ++f) {                                               \
      uint32_t const m = uint32_t(MASK0) << (BITS * f);                                            \
      ACC(f) = __hfma2(u32_as_h2(l01 & m), xr[XI(f)], ACC(f));                                     \
      ACC(f) = __hfma2(u32_as_h2(l23 & m), xr[XI(f) + 1], ACC(f));                                 \
    }                                                                                              \
  }

// One lane's half block (128 weights) of one output row: B = shared address of the block, h = which half.
// Returns the lane's share of the dot product.  xr: the 128 activations of the half in natural order, scaled by 2^ex;
// sxg: sums of the unscaled x over the half's groups; fm = 2^(24-ex).
template <int QT>
__device__ __forceinline__ float kq_half_block_dot(uint32_t B, int h, __half2 const (&xr)[64], float const (&sxg)[8], float fm);

// ---- Q6_K: ql[128] qh[64] int8 sc[16] d; group g = p + 2*q1 + 4*n + 8*h, code = lo | hi<<4, minus 32 ------------------------
template <>
__device__ __forceinline__ float kq_half_block_dot<14>(uint32_t B, int h, __half2 const (&xr)[64], float const (&sxg)[8], float fm) {
  __half2 const z = __float2half2_rn(0.f);
  __half2 acc[8] = {z, z, z, z, z, z, z, z}, ahi[8] = {z, z, z, z, z, z, z, z};
#pragma unroll
  for (int r = 0; r < 4; ++r) {                                   // ql run r = p + 2*q1: low nibble group r, high nibble group r+4
    uint32_t w[4];
    k_run<2, 4>(B + 64u * h + 16u * r, w);
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
#define ACC_(f) acc[r + 4 * (f)]
#define XI_(f) ((r + 4 * (f)) * 8 + 2 * wi)
      KQ_WORD(w[wi], 2, 4, 0x000F000Fu, ACC_, XI_)
#undef ACC_
#undef XI_
    }
  }
#pragma unroll
  for (int p = 0; p < 2; ++p) {                                   // qh run p: field f = q1 + 2n -> group p + 2*q1 + 4*n
    uint32_t w[4];
    k_run<2, 4>(B + 128u + 32u * h + 16u * p, w);
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
#define ACC_(f) ahi[p + 2 * ((f) & 1) + 4 * ((f) >> 1)]
#define XI_(f) ((p + 2 * ((f) & 1) + 4 * ((f) >> 1)) * 8 + 2 * wi)
      KQ_WORD(w[wi], 4, 2, 0x00030003u, ACC_, XI_)
#undef ACC_
#undef XI_
    }
  }
  uint32_t s[2];
  k_run<2, 2>(B + 192u + 8u * h, s);
  s[0] ^= 0x80808080u; s[1] ^= 0x80808080u;                       // int8 -> offset binary (sc + 128)
  float const d = __half2float(__ushort_as_half((unsigned short)k_lds16(B + 208u)));
  float dsum = 0.f, bsum = 0.f;
#pragma unroll
  for (int gl = 0; gl < 8; ++gl) {
    float const sc = gl == 0 ? k_byte_f<0>(s[0], 128.f) : gl == 1 ? k_byte_f<1>(s[0], 128.f) : gl == 2 ? k_byte_f<2>(s[0], 128.f)
                   : gl == 3 ? k_byte_f<3>(s[0], 128.f) : gl == 4 ? k_byte_f<0>(s[1], 128.f) : gl == 5 ? k_byte_f<1>(s[1], 128.f)
                   : gl == 6 ? k_byte_f<2>(s[1], 128.f) : k_byte_f<3>(s[1], 128.f);
    // lo + 16*hi: the hi field of group (q1, n) sits at bit 2*(q1 + 2n), its low nibble at bit 4n
    __half2 const kk = __float2half2_rn(((gl >> 1) & 1) ? 4.f : 16.f);
    float const gsum = h2_sum(__hfma2(ahi[gl], kk, acc[gl]));
    dsum = fmaf(gl >= 4 ? sc * 0.0625f : sc, gsum, dsum);
    bsum = fmaf(sc, sxg[gl], bsum);
  }
  return d * fmaf(fm, dsum, -32.f * bsum);
}

// ---- Q2_K: sc|mn nibbles[16] qs[64] d dmin; group g = p + 2*f + 8*h, 2-bit field f of byte j + 16p + 32h -----------------------
template <>
__device__ __forceinline__ float kq_half_block_dot<10>(uint32_t B, int h, __half2 const (&xr)[64], float const (&sxg)[8], float fm) {
  __half2 const z = __float2half2_rn(0.f);
  __half2 acc[8] = {z, z, z, z, z, z, z, z};
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    uint32_t w[4];
    k_run<4, 4>(B + 16u + 32u * h + 16u * p, w);
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
#define ACC_(f) acc[p + 2 * (f)]
#define XI_(f) ((p + 2 * (f)) * 8 + 2 * wi)
      KQ_WORD(w[wi], 4, 2, 0x00030003u, ACC_, XI_)
#undef ACC_
#undef XI_
    }
  }
  uint32_t s[2];
  k_run<4, 2>(B + 8u * h, s);
  uint32_t const scn[2] = {s[0] & 0x0F0F0F0Fu, s[1] & 0x0F0F0F0Fu}, mnn[2] = {(s[0] >> 4) & 0x0F0F0F0Fu, (s[1] >> 4) & 0x0F0F0F0Fu};
  float2 const dd = __half22float2(u32_as_h2(k_lds32(B + 80u)));   // (d, dmin)
  float dsum = 0.f, msum = 0.f;
#pragma unroll
  for (int gl = 0; gl < 8; ++gl) {
    uint32_t const sw = scn[gl >> 2], mw = mnn[gl >> 2];
    float const sc = (gl & 3) == 0 ? k_byte_f<0>(sw, 0.f) : (gl & 3) == 1 ? k_byte_f<1>(sw, 0.f) : (gl & 3) == 2 ? k_byte_f<2>(sw, 0.f) : k_byte_f<3>(sw, 0.f);
    float const mn = (gl & 3) == 0 ? k_byte_f<0>(mw, 0.f) : (gl & 3) == 1 ? k_byte_f<1>(mw, 0.f) : (gl & 3) == 2 ? k_byte_f<2>(mw, 0.f) : k_byte_f<3>(mw, 0.f);
    float const fs = 1.f / float(1 << (2 * (gl >> 1)));            // the field of group gl = p + 2f sits at bit 2f
    dsum = fmaf(sc * fs, h2_sum(acc[gl]), dsum);
    msum = fmaf(mn, sxg[gl], msum);
  }
  return fmaf(dd.x * fm, dsum, -dd.y * msum);
}

// ---- Q3_K: hmask[32] qs[64] sc6[12] d; group g = p + 2*f + 8*h, code = lo + 4*hb - 4, sub-scale = sc6 - 32 --------------------
template <>
__device__ __forceinline__ float kq_half_block_dot<11>(uint32_t B, int h, __half2 const (&xr)[64], float const (&sxg)[8], float fm) {
  __half2 const z = __float2half2_rn(0.f);
  __half2 acc[8] = {z, z, z, z, z, z, z, z}, ahi[8] = {z, z, z, z, z, z, z, z};
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    uint32_t w[4], m[4];
    k_run<2, 4>(B + 32u + 32u * h + 16u * p, w);
    k_run<2, 4>(B + 16u * p, m);                                  // hmask: bit f + 4h of byte j + 16p
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
#define ACC_(f) acc[p + 2 * (f)]
#define AHI_(f) ahi[p + 2 * (f)]
#define XI_(f) ((p + 2 * (f)) * 8 + 2 * wi)
      KQ_WORD(w[wi], 4, 2, 0x00030003u, ACC_, XI_)
      uint32_t const mw = m[wi] >> (4 * h);
      KQ_WORD(mw, 4, 1, 0x00010001u, AHI_, XI_)
#undef ACC_
#undef AHI_
#undef XI_
    }
  }
  uint32_t s[3];
  k_run<2, 3>(B + 96u, s);
  int const sh4 = 4 * h;
  uint32_t const sc6[2] = {((s[0] >> sh4) & 0x0F0F0F0Fu) | (((s[2] >> sh4) & 0x03030303u) << 4),
                           ((s[1] >> sh4) & 0x0F0F0F0Fu) | (((s[2] >> (sh4 + 2)) & 0x03030303u) << 4)};
  float const d = __half2float(__ushort_as_half((unsigned short)k_lds16(B + 108u)));
  float dsum = 0.f, bsum = 0.f;
#pragma unroll
  for (int gl = 0; gl < 8; ++gl) {
    uint32_t const sw = sc6[gl >> 2];
    float const sc = (gl & 3) == 0 ? k_byte_f<0>(sw, 32.f) : (gl & 3) == 1 ? k_byte_f<1>(sw, 32.f) : (gl & 3) == 2 ? k_byte_f<2>(sw, 32.f) : k_byte_f<3>(sw, 32.f);
    int const f = gl >> 1;                                        // lo field at bit 2f, hmask bit (after the shift) at bit f
    __half2 const kk = __float2half2_rn(float(4 << f));
    float const gsum = h2_sum(__hfma2(ahi[gl], kk, acc[gl]));
    dsum = fmaf(sc * (1.f / float(1 << (2 * f))), gsum, dsum);
    bsum = fmaf(sc, sxg[gl], bsum);
  }
  return d * fmaf(fm, dsum, -4.f * bsum);
}

// ---- Q5_K: d dmin sc6/mn6[12] qh[32] qs[128]; groups of 32: group g = nibble (g & 1) of qs byte j + 32*(g >> 1), bit g of qh[j]
template <>
__device__ __forceinline__ float kq_half_block_dot<13>(uint32_t B, int h, __half2 const (&xr)[64], float const (&sxg)[8], float fm) {
  __half2 const z = __float2half2_rn(0.f);
  __half2 acc[4] = {z, z, z, z}, ahi[4] = {z, z, z, z};
#pragma unroll
  for (int c = 0; c < 2; ++c)
#pragma unroll
    for (int u = 0; u < 2; ++u) {                                 // qs bytes 64h + 32c + 16u + (0..15): groups 2c (low), 2c+1 (high)
      uint32_t w[4];
      k_run<16, 4>(B + 48u + 64u * h + 32u * c + 16u * u, w);
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {
#define ACC_(f) acc[2 * c + (f)]
#define XI_(f) ((2 * c + (f)) * 16 + 8 * u + 2 * wi)
        KQ_WORD(w[wi], 2, 4, 0x000F000Fu, ACC_, XI_)
#undef ACC_
#undef XI_
      }
    }
#pragma unroll
  for (int u = 0; u < 2; ++u) {                                   // qh bytes 16u + (0..15): bit 4h + gl belongs to group gl
    uint32_t w[4];
    k_run<16, 4>(B + 16u + 16u * u, w);
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      uint32_t const mw = w[wi] >> (4 * h);
#define AHI_(f) ahi[f]
#define XI_(f) ((f) * 16 + 8 * u + 2 * wi)
      KQ_WORD(mw, 4, 1, 0x00010001u, AHI_, XI_)
#undef AHI_
#undef XI_
    }
  }
  uint4 const hdr = k_lds128(B);
  // groups 0-3 (h 0): the low six bits of scale bytes 0-3 / 4-7; groups 4-7 (h 1): nibbles of bytes 8-11 plus the top two
  // bits of bytes 0-3 / 4-7
  uint32_t const ma = h ? 0x0F0F0F0Fu : 0x3F3F3F3Fu, mb = h ? 0x30303030u : 0u;
  uint32_t const sc4 = ((h ? hdr.w : hdr.y) & ma) | ((hdr.y >> 2) & mb);
  uint32_t const mn4 = ((h ? (hdr.w >> 4) : hdr.z) & ma) | ((hdr.z >> 2) & mb);
  float2 const dd = __half22float2(u32_as_h2(hdr.x));
  float dsum = 0.f, msum = 0.f;
#pragma unroll
  for (int gl = 0; gl < 4; ++gl) {
    float const sc = gl == 0 ? k_byte_f<0>(sc4, 0.f) : gl == 1 ? k_byte_f<1>(sc4, 0.f) : gl == 2 ? k_byte_f<2>(sc4, 0.f) : k_byte_f<3>(sc4, 0.f);
    float const mn = gl == 0 ? k_byte_f<0>(mn4, 0.f) : gl == 1 ? k_byte_f<1>(mn4, 0.f) : gl == 2 ? k_byte_f<2>(mn4, 0.f) : k_byte_f<3>(mn4, 0.f);
    // the fifth bit (after the shift by 4h) sits at bit gl; the low code at bit 0 (even gl) or 4 (odd gl)
    __half2 const kk = __float2half2_rn((gl & 1) ? float(256 >> gl) : float(16 >> gl));
    float const gsum = h2_sum(__hfma2(ahi[gl], kk, acc[gl]));
    dsum = fmaf((gl & 1) ? sc * 0.0625f : sc, gsum, dsum);
    msum = fmaf(mn, sxg[gl], msum);
  }
  return fmaf(dd.x * fm, dsum, -dd.y * msum);
}

template <int QT>
__global__ void __launch_bounds__(kKqWarps * 32, 1) kquant_gemv1_kernel(KqArgs a) {
  using F = kq::Fmt<QT>;
  constexpr int KB = F::kBytes, G = F::kGroups, GH = G / 2;       // block bytes; groups per block and per half
  constexpr int PPG = (256 / G) / 8;                               // 16-byte activation pieces per group: 2 or 4
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
  // shared memory map: activations (piece q of half-block slot s at (q*2*bpr + s)*16), group sums, scratch, rings, barriers
  uint32_t const s0 = smem_u32(smem);
  uint32_t const xa32 = s0;
  uint32_t const sx32 = xa32 + uint32_t(k) * 2u;                  // bpr*G floats
  uint32_t const red32 = sx32 + uint32_t(bpr) * G * 4u;           // 32 floats of reduction scratch
  int const stage_bytes = 2 * a.seg_stride;                       // a stage holds the segments of two rows
  uint32_t const ring32 = red32 + 128u + uint32_t(warp) * kKqStages * stage_bytes;
  uint32_t const bar32 = red32 + 128u + uint32_t(W) * kKqStages * stage_bytes + uint32_t(warp) * kKqStages * 8u;
  uint32_t const part32 = red32 + 128u + uint32_t(W) * kKqStages * (stage_bytes + 8);
  float* red = reinterpret_cast<float*>(smem + (red32 - s0));
  float* part = reinterpret_cast<float*>(smem + (part32 - s0));

  // ---- 1. activation pieces -> registers, requested BEFORE the weight copies so they do not queue behind them
  int const npieces = k >> 3;
  uint4 const* xg = reinterpret_cast<uint4 const*>(a.x + size_t(arow) * k);
  uint4 pc[kKqMaxPieces];
#pragma unroll
  for (int j = 0; j < kKqMaxPieces; ++j) {
    int const p = threadIdx.x + j * T;
    pc[j] = p < npieces ? __ldg(xg + p) : make_uint4(0, 0, 0, 0);
  }

  // ---- 2. weight ring: barriers and the first row pairs.  A segment that starts off a 16-byte boundary is copied from
  // the boundary below (`lead` bytes early); rows are multiples of 16 bytes, so this is the same for every row.
  int const nb_seg = min(a.nbs, bpr - seg * a.nbs);
  int const cx = blockIdx.x;
  int const row0 = cx * a.rows_q + min(cx, a.rows_r);
  int const nrows = a.rows_q + (cx < a.rows_r ? 1 : 0);
  int const npairs = (nrows + 1) >> 1;
  size_t const row_stride = size_t(bpr) * KB;
  unsigned const seg_off = unsigned(seg) * unsigned(a.nbs) * KB, lead = seg_off & 15u;
  unsigned const copy_bytes = (lead + unsigned(nb_seg) * KB + 15u) & ~15u;
  bool const contiguous = a.S == 1;                               // a whole row per segment: the two rows are adjacent
  // Beyond the first two pairs of every warp, row pairs are claimed from a per-segment counter by whichever warp has a
  // free stage (see qb_gemv_q4k.cu): the CTA's pairs rarely divide evenly over its warps.  Which warp computes a row does
  // not change the row's arithmetic.
  static_assert(kKqStages == 2, "the claim bookkeeping below keeps two pairs per warp");
  uint8_t const* seg_base = a.blocks + (size_t(e) * a.n + size_t(row0)) * row_stride + (seg_off - lead);
  auto issue_pair = [&](int pair, uint32_t dst, uint32_t bar) {
    uint8_t const* src = seg_base + size_t(2 * pair) * row_stride;
    bool const two = 2 * pair + 1 < nrows;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(two ? 2u * copy_bytes : copy_bytes) : "memory");
    if (two && contiguous) {
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(dst), "l"(src), "r"(2u * copy_bytes), "r"(bar) : "memory");
    } else {
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(dst), "l"(src), "r"(copy_bytes), "r"(bar) : "memory");
      if (two)
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(dst + uint32_t(a.seg_stride)), "l"(src + row_stride), "r"(copy_bytes), "r"(bar) : "memory");
    }
  };
  int* claim = reinterpret_cast<int*>(red) + 16;                  // [S] next unclaimed pair per K segment (S <= 16)
  if (int(threadIdx.x) < a.S) claim[threadIdx.x] = kKqStages * a.RS;   // visible after the prologue's barriers
  int cur = rslot < npairs ? rslot : -1;                          // pair held by the stage consumed next
  int nxt = rslot + a.RS < npairs ? rslot + a.RS : -1;            // ... and by the other stage
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kKqStages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar32 + 8u * s) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (cur >= 0) issue_pair(cur, ring32, bar32);
    if (nxt >= 0) issue_pair(nxt, ring32 + stage_bytes, bar32 + 8u);
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // ---- 3. CTA-wide max|x| -> power-of-two scale
  __half2 m2 = __float2half2_rn(0.f);
#pragma unroll
  for (int j = 0; j < kKqMaxPieces; ++j) {
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

  // ---- 4. scaled activations (natural order) and group sums -> shared memory
#pragma unroll
  for (int j = 0; j < kKqMaxPieces; ++j) {
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
      o.x = h2_as_u32(__floats2half2_rn(f0.x * scl, f0.y * scl)); o.y = h2_as_u32(__floats2half2_rn(f1.x * scl, f1.y * scl));
      o.z = h2_as_u32(__floats2half2_rn(f2.x * scl, f2.y * scl)); o.w = h2_as_u32(__floats2half2_rn(f3.x * scl, f3.y * scl));
      k_sts128(xa32 + uint32_t(((p & 15) * 2 * bpr + (p >> 4)) * 16), o);
      if ((p & (PPG - 1)) == 0) reinterpret_cast<float*>(smem + (sx32 - s0))[p / PPG] = gsum;
    }
  }
  __syncthreads();

  // ---- 5. this lane's activation registers: half h of block blk of the warp's segment
  int const blk = lane >> 1, h = lane & 1;
  bool const active = blk < nb_seg;
  int const b_in_row = seg * a.nbs + blk;
  __half2 xr[64];
  float sxg[8];
  if (active) {
    int const slot = b_in_row * 2 + h;
#pragma unroll
    for (int q = 0; q < 16; ++q) {
      uint4 const v = k_lds128(xa32 + uint32_t((q * 2 * bpr + slot) * 16));
      xr[4 * q + 0] = u32_as_h2(v.x); xr[4 * q + 1] = u32_as_h2(v.y); xr[4 * q + 2] = u32_as_h2(v.z); xr[4 * q + 3] = u32_as_h2(v.w);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sxg[i] = 0.f;
#pragma unroll
    for (int i = 0; i < GH; i += 4) {
      uint4 const sv = k_lds128(sx32 + uint32_t((b_in_row * G + GH * h + i) * 4));
      sxg[i] = __uint_as_float(sv.x); sxg[i + 1] = __uint_as_float(sv.y); sxg[i + 2] = __uint_as_float(sv.z); sxg[i + 3] = __uint_as_float(sv.w);
    }
  } else {
#pragma unroll
    for (int q = 0; q < 64; ++q) xr[q] = __float2half2_rn(0.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) sxg[i] = 0.f;
  }

  // ---- 6. main loop: one stage = the segments of two consecutive rows
  uint32_t const lane_off = lead + uint32_t(active ? blk : 0) * KB;   // lanes without a block read block 0 and are masked
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
    float const t0 = kq_half_block_dot<QT>(st_addr + lane_off, h, xr, sxg, fm);
    float const t1 = kq_half_block_dot<QT>(st_addr + uint32_t(contiguous ? copy_bytes : unsigned(a.seg_stride)) + lane_off, h, xr, sxg, fm);
    reduce_store(p0, p1, plr);
    int const lr = 2 * cur;
    p0 = active ? t0 : 0.f;
    p1 = (active && lr + 1 < nrows) ? t1 : 0.f;
    plr = lr;
    __syncwarp();
    int c = -1;
    if (lane == 0) {
      c = atomicAdd(&claim[seg], 1);
      if (c < npairs) issue_pair(c, st_addr, st_bar); else c = -1;
    }
    c = __shfl_sync(0xffffffffu, c, 0);
    cur = nxt; nxt = c;
    st_addr += stage_bytes; st_bar += 8u;
    if (++st == kKqStages) { st = 0; st_addr = ring32; st_bar = bar32; phase ^= 1u; }
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

struct KqPlan { int S, nbs, RS, gx, W, seg_stride; size_t smem; bool ok; };

template <int QT>
KqPlan const& kq_plan(int n, int bpr, int gy) {
  using F = kq::Fmt<QT>;
  struct Key { int n, bpr, gy, dev; bool operator<(Key const& o) const {
    return n != o.n ? n < o.n : bpr != o.bpr ? bpr < o.bpr : gy != o.gy ? gy < o.gy : dev < o.dev; } };
  static std::map<Key, KqPlan> cache;
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(mu);
  Key const key{n, bpr, gy, dev};
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  KqPlan p{};
  auto kern = kquant_gemv1_kernel<QT>;
  p.S = (bpr + 15) / 16;
  p.ok = p.S <= kKqWarps && (size_t(bpr) * F::kBytes) % 16 == 0;
  if (p.ok) {
    p.nbs = (bpr + p.S - 1) / p.S;
    p.RS = std::max(1, kKqWarps / p.S);
    p.W = p.S * p.RS;
    if (p.W * 32 * kKqMaxPieces * 8 < bpr * 256) p.ok = false;
    // a lone segment is the whole row (two rows adjacent, one copy); otherwise a segment may start up to 15 bytes early
    // and end up to 15 bytes late, and the word reads of a misaligned run reach 4 bytes further
    p.seg_stride = p.S == 1 ? bpr * F::kBytes : ((p.nbs * F::kBytes + 15 + 15) / 16 + 1) * 16;
    size_t const tail = p.S == 1 ? 16 : 0;                         // room for the last run's extra word
    size_t const fixed = size_t(bpr) * 512 + size_t(bpr) * F::kGroups * 4 + 128 + size_t(p.W) * kKqStages * (2 * p.seg_stride + 8) + tail;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) { (void)cudaGetLastError(); p.ok = false; }
    int const sms = rt_sm_count();
    int const resident = std::max(1, sms / std::max(1, std::min(gy, 8)));
    p.gx = std::max(1, std::min(resident, (n + p.RS - 1) / p.RS));
    p.smem = fixed + size_t((n + p.gx - 1) / p.gx + 4) * p.S * 4;
    if (p.smem > 227 * 1024) p.ok = false;
  }
  return cache.emplace(key, p).first->second;
}

template <int QT>
bool enqueue_kq1(uint8_t const* blocks, __half const* x, float* out, int const* offsets, int n, int bpr, int experts, int rows,
                 int max_rows, unsigned int* status, cudaStream_t stream) {
  int const gy = offsets ? experts * max_rows : rows;
  if (gy <= 0 || gy > 65535) return false;
  KqPlan const& p = kq_plan<QT>(n, bpr, gy);
  if (!p.ok) return false;
  KqArgs a{};
  a.blocks = blocks; a.x = x; a.out = out; a.offsets = offsets;
  a.n = n; a.bpr = bpr; a.max_rows = max_rows;
  a.S = p.S; a.nbs = p.nbs; a.RS = p.RS; a.seg_stride = p.seg_stride; a.status = status;
  a.rows_q = n / p.gx; a.rows_r = n % p.gx;
  static bool const no_pdl = std::getenv("QUACTLIZE_B200_NO_PDL") != nullptr;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.gx, gy); cfg.blockDim = dim3(p.W * 32); cfg.dynamicSmemBytes = p.smem; cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = no_pdl ? 0 : 1;
  if (cudaLaunchKernelEx(&cfg, kquant_gemv1_kernel<QT>, a) != cudaSuccess) { (void)cudaGetLastError(); return false; }
  return true;
}

}  // namespace

// Enqueue; false when the format or the shape is outside this kernel's envelope (the caller then uses another kernel).
bool enqueue_kquant_gemv1(uint8_t const* blocks, __half const* x, float* out, int const* offsets, int n, int bpr, int experts,
                          int rows, int max_rows, int qtype, unsigned int* status, cudaStream_t stream) {
  switch (qtype) {
    case 10: return enqueue_kq1<10>(blocks, x, out, offsets, n, bpr, experts, rows, max_rows, status, stream);
    case 11: return enqueue_kq1<11>(blocks, x, out, offsets, n, bpr, experts, rows, max_rows, status, stream);
    case 13: return enqueue_kq1<13>(blocks, x, out, offsets, n, bpr, experts, rows, max_rows, status, stream);
    case 14: return enqueue_kq1<14>(blocks, x, out, offsets, n, bpr, experts, rows, max_rows, status, stream);
    default: return false;
  }
}

}  // namespace qb
