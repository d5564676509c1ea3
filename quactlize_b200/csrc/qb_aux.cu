// Bit-exact helper kernels around the GEMVs: raw block -> fp16 weights, scale pre-pass (raw scale blocks or packed
// units -> fp16 scale/zero planes).  Every product and sum is an explicit round-to-nearest intrinsic so the device
// result equals the reference's host definition bit for bit:
//   weight  = half( (float(d)*sc) * q - float(dmin)*mn )                quactlize/include/gguf_vecdot.hpp:313-321
//   scale   = half( float(d) * float(sc) ),  zero = -half( float(dmin) * float(mn) ),
//   zero   := half( float(zero) + zmul * float(scale) )                 quactlize/include/gguf_scale_prepass.hpp:64-98
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "qb_kquant.cuh"
#include "qb_runtime.hpp"

namespace qb {

// Eight consecutive codes (elements j0 .. j0+7 of group g, j0 a multiple of 8) of a block as the bytes of two words,
// unsigned and before the format's bias: the same bits kq::code<QT> reads one element at a time, taken a word at a time.
// The block may be only 2-byte aligned (84-, 110-, 210-byte blocks), so bytes are fetched in pairs.
__device__ __forceinline__ void load8(uint8_t const* p, uint32_t& w0, uint32_t& w1) {
  unsigned short const* h = reinterpret_cast<unsigned short const*>(p);
  w0 = uint32_t(h[0]) | (uint32_t(h[1]) << 16);
  w1 = uint32_t(h[2]) | (uint32_t(h[3]) << 16);
}
template <int QT>
__device__ __forceinline__ void codes8(uint8_t const* b, int g, int j0, uint32_t& c0, uint32_t& c1) {
  uint32_t l0, l1, h0, h1;
  if constexpr (QT == 12) {
    load8(b + 16 + j0 + 32 * (g >> 1), l0, l1);
    int const s = 4 * (g & 1);
    c0 = (l0 >> s) & 0x0F0F0F0Fu; c1 = (l1 >> s) & 0x0F0F0F0Fu;
  } else if constexpr (QT == 13) {
    load8(b + 48 + j0 + 32 * (g >> 1), l0, l1);
    load8(b + 16 + j0, h0, h1);
    int const s = 4 * (g & 1);
    c0 = ((l0 >> s) & 0x0F0F0F0Fu) | (((h0 >> g) & 0x01010101u) << 4);
    c1 = ((l1 >> s) & 0x0F0F0F0Fu) | (((h1 >> g) & 0x01010101u) << 4);
  } else if constexpr (QT == 14) {
    int const p = g & 1, q1 = (g >> 1) & 1, n = (g >> 2) & 1, h = g >> 3;
    load8(b + j0 + 16 * p + 32 * q1 + 64 * h, l0, l1);
    load8(b + 128 + j0 + 16 * p + 32 * h, h0, h1);
    int const s = 4 * n, sh = 2 * q1 + 4 * n;
    c0 = ((l0 >> s) & 0x0F0F0F0Fu) | (((h0 >> sh) & 0x03030303u) << 4);
    c1 = ((l1 >> s) & 0x0F0F0F0Fu) | (((h1 >> sh) & 0x03030303u) << 4);
  } else if constexpr (QT == 11) {
    load8(b + 32 + j0 + 16 * (g & 1) + 32 * (g >> 3), l0, l1);
    load8(b + j0 + 16 * (g & 1), h0, h1);
    int const s = 2 * ((g >> 1) & 3), sh = ((g >> 1) & 3) + 4 * (g >> 3);
    c0 = ((l0 >> s) & 0x03030303u) | (((h0 >> sh) & 0x01010101u) << 2);     // lo + 4*hb; the bias of 4 is the format's
    c1 = ((l1 >> s) & 0x03030303u) | (((h1 >> sh) & 0x01010101u) << 2);
  } else {
    load8(b + 16 + j0 + 16 * (g & 1) + 32 * (g >> 3), l0, l1);
    int const s = 2 * ((g >> 1) & 3);
    c0 = (l0 >> s) & 0x03030303u; c1 = (l1 >> s) & 0x03030303u;
  }
}

// Raw blocks -> fp16 weights.  A CTA takes kDqBlocks consecutive blocks: their bytes are one contiguous run, staged in
// shared memory by 16-byte loads (coalesced whatever the block size; the ragged ends by byte loads), then a warp owns a
// block, lane -> 8 consecutive elements, one 16-byte store per lane (a warp writes 512 contiguous bytes).  DRAM traffic
// is the algorithmic 144..210 B in + 512 B out per block; the reference's warp-per-256 kernel has the same shape
// (quactlize/include/gguf_vecdot.hpp:782-854, 78 % of peak published at :762-770).
constexpr int kDqBlocks = 32;
template <int QT, bool WORDS>          // WORDS: the blocks start on an even address, codes are taken a word at a time
__global__ void __launch_bounds__(256) dequant_kernel(uint8_t const* __restrict__ blocks, __half* __restrict__ out, int count) {
  using F = kq::Fmt<QT>;
  constexpr int GS = 256 / F::kGroups;
  __shared__ __align__(16) uint8_t stage[kDqBlocks * F::kBytes + 16];
  int const b0 = blockIdx.x * kDqBlocks;
  int const nb = min(kDqBlocks, count - b0);
  if (nb <= 0) return;
  uint8_t const* src = blocks + size_t(b0) * F::kBytes;
  int const bytes = nb * F::kBytes;
  // align the staged copy to the source's 16-byte grid: stage[lead + i] = src[i]
  int const lead = int(reinterpret_cast<uintptr_t>(src) & 15u);
  int const head = lead ? min(16 - lead, bytes) : 0;
  for (int i = threadIdx.x; i < head; i += blockDim.x) stage[lead + i] = src[i];
  int const body = (bytes - head) >> 4;
  for (int i = threadIdx.x; i < body; i += blockDim.x)
    *reinterpret_cast<uint4*>(stage + lead + head + 16 * i) = __ldg(reinterpret_cast<uint4 const*>(src + head) + i);
  for (int i = head + 16 * body + threadIdx.x; i < bytes; i += blockDim.x) stage[lead + i] = src[i];
  __syncthreads();
  int const lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int lb = warp; lb < nb; lb += (blockDim.x >> 5)) {
    uint8_t const* blk = stage + lead + lb * F::kBytes;
    float const d = __half2float(__ushort_as_half(kq::load_u16(blk + F::kD)));
    float dmin = 0.f;
    if constexpr (F::kHasMin) dmin = __half2float(__ushort_as_half(kq::load_u16(blk + F::kDmin)));
    int const i0 = lane * 8, g = i0 / GS, j0 = i0 % GS;
    int sc, mn;
    kq::scale_min<QT>(blk + F::kScaleOff, g, sc, mn);
    float const dl = __fmul_rn(d, float(sc)), ml = __fmul_rn(dmin, float(mn));
    // the lane's eight codes as bytes of two words (unsigned, before the format's bias), then byte -> float through the
    // 2^23 magic (exact) and the reference's three roundings
    __align__(16) __half2 w[4];
    if constexpr (!WORDS) {
#pragma unroll
      for (int t = 0; t < 4; ++t)
        w[t] = __halves2half2(__float2half_rn(__fsub_rn(__fmul_rn(dl, float(kq::code<QT>(blk, g, j0 + 2 * t))), ml)),
                              __float2half_rn(__fsub_rn(__fmul_rn(dl, float(kq::code<QT>(blk, g, j0 + 2 * t + 1))), ml)));
    } else {
    uint32_t c0, c1;
    codes8<QT>(blk, g, j0, c0, c1);
    float const bias = 8388608.f + float(F::kCodeBias);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      uint32_t const cw = t < 2 ? c0 : c1;
      float const qa = __uint_as_float(__byte_perm(cw, 0x4B000000u, (t & 1) ? 0x7442u : 0x7440u)) - bias;
      float const qb2 = __uint_as_float(__byte_perm(cw, 0x4B000000u, (t & 1) ? 0x7443u : 0x7441u)) - bias;
      w[t] = __floats2half2_rn(__fsub_rn(__fmul_rn(dl, qa), ml), __fsub_rn(__fmul_rn(dl, qb2), ml));
    }
    }
    *reinterpret_cast<uint4*>(out + size_t(b0 + lb) * 256 + i0) = *reinterpret_cast<uint4 const*>(w);
  }
}

// Raw blocks -> (codes int8 [rows][256], scale fp16 [rows][G], zero fp16 [rows][G]) with W = code*scale + zero:
// scale = half(float(d)*sc), zero = half(-(float(dmin)*mn)) (quactlize/include/gguf_vecdot.hpp:336-343, the
// gguf_unpack op).  One warp per block, a lane writes eight codes.
template <int QT>
__global__ void __launch_bounds__(256) unpack_kernel(uint8_t const* __restrict__ blocks, int8_t* __restrict__ codes,
                                                     __half* __restrict__ scale, __half* __restrict__ zero, int count) {
  using F = kq::Fmt<QT>;
  constexpr int GS = 256 / F::kGroups;
  int const lane = threadIdx.x & 31;
  int const b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (b >= count) return;
  uint8_t const* blk = blocks + size_t(b) * F::kBytes;
  int const i0 = lane * 8, g = i0 / GS, j0 = i0 % GS;
  __align__(8) int8_t c[8];
#pragma unroll
  for (int t = 0; t < 8; ++t) c[t] = int8_t(kq::code<QT>(blk, g, j0 + t));
  *reinterpret_cast<uint2*>(codes + size_t(b) * 256 + i0) = *reinterpret_cast<uint2 const*>(c);
  if (lane < F::kGroups) {
    float const d = __half2float(__ushort_as_half(kq::load_u16(blk + F::kD)));
    float dmin = 0.f;
    if constexpr (F::kHasMin) dmin = __half2float(__ushort_as_half(kq::load_u16(blk + F::kDmin)));
    int sc, mn;
    kq::scale_min<QT>(blk + F::kScaleOff, lane, sc, mn);
    scale[size_t(b) * F::kGroups + lane] = __float2half_rn(__fmul_rn(d, float(sc)));
    zero[size_t(b) * F::kGroups + lane] = __float2half_rn(-__fmul_rn(dmin, float(mn)));
  }
}

// Plane artifact -> fp16 [E][n][k]:  half( float(lo + 2^LO*hi + shift) * float(scale) + float(zero) ), product and sum
// rounded separately as the host definition does (quactlize/csrc/preprocess/thop/gguf_prepass_ops.cpp:1194-1202).
// A thread converts eight consecutive k of one row (one 16-byte store); planes are K-contiguous per row, the fp16
// planes are [E][k/gs][n].
__global__ void __launch_bounds__(256) planes_dequant_kernel(uint8_t const* __restrict__ low, uint8_t const* __restrict__ high,
                                                             __half const* __restrict__ scale, __half const* __restrict__ zero,
                                                             __half* __restrict__ out, int64_t rows, int n, int k, int lo, int hi,
                                                             int gs, int shift) {
  int64_t const idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  int const per_row = k >> 3;
  if (idx >= rows * per_row) return;
  int64_t const row = idx / per_row;                    // e*n + col
  int const k0 = int(idx % per_row) * 8;
  int64_t const e = row / n;
  int const col = int(row % n);
  uint8_t const* lp = low + (row * k * lo >> 3) + (int64_t(k0) * lo >> 3);
  uint32_t lw = 0;
  for (int i = 0; i < lo; ++i) lw |= uint32_t(lp[i]) << (8 * i);      // eight codes of `lo` bits = lo bytes
  uint32_t hw = 0;
  if (hi) {
    uint8_t const* hp = high + (row * k * hi >> 3) + (int64_t(k0) * hi >> 3);
    for (int i = 0; i < hi; ++i) hw |= uint32_t(hp[i]) << (8 * i);
  }
  __align__(16) __half w[8];
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    int q = int((lw >> (t * lo)) & ((1u << lo) - 1u));
    if (hi) q |= int((hw >> (t * hi)) & ((1u << hi) - 1u)) << lo;
    int64_t const a = (e * (k / gs) + (k0 + t) / gs) * n + col;
    float const z = zero ? __half2float(zero[a]) : 0.f;
    w[t] = __float2half_rn(__fadd_rn(__fmul_rn(float(q + shift), __half2float(scale[a])), z));
  }
  *reinterpret_cast<uint4*>(out + row * k + k0) = *reinterpret_cast<uint4 const*>(w);
}

__device__ __forceinline__ void scale_zero_from_codes(float d, float dmin, int sc, int mn, bool has_min, int zmul,
                                                      __half& scale, __half& zero) {
  scale = __float2half_rn(__fmul_rn(d, float(sc)));
  zero = has_min ? __hneg(__float2half_rn(__fmul_rn(dmin, float(mn)))) : __float2half_rn(0.f);
  if (zmul != 0) zero = __float2half_rn(__fadd_rn(__half2float(zero), __fmul_rn(float(zmul), __half2float(scale))));
}

// scale blocks [count][scale_bytes] + headers d,dmin [count] -> planes [count][groups]; one thread per (row, group)
template <int QT>
__global__ void __launch_bounds__(256) prepass_kernel(uint8_t const* __restrict__ sblocks, uint16_t const* __restrict__ d,
                                                      uint16_t const* __restrict__ dmin, int count, int zmul,
                                                      __half* __restrict__ scale, __half* __restrict__ zero) {
  using F = kq::Fmt<QT>;
  int const idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= count * F::kGroups) return;
  int const r = idx / F::kGroups, g = idx % F::kGroups;
  int sc, mn;
  kq::scale_min<QT>(sblocks + size_t(r) * F::kScaleBytes, g, sc, mn);
  float const df = __half2float(__ushort_as_half(d[r]));
  float const mf = F::kHasMin ? __half2float(__ushort_as_half(dmin[r])) : 0.f;
  __half s, z;
  scale_zero_from_codes(df, mf, sc, mn, F::kHasMin, zmul, s, z);
  scale[idx] = s; zero[idx] = z;
}

// units [E][K/256/P][N][unit_total] -> planes [E][K/gs][N]; one thread per (expert, superblock, column), column fastest:
// it reads its superblock's share of the unit once (2-byte loads: shares are 14-20 bytes and 2-byte aligned), decodes all
// the groups from registers and writes one element of G consecutive plane rows; a warp's stores are 64 contiguous bytes.
template <int QT>
__global__ void __launch_bounds__(256) prepass_unit_kernel(uint8_t const* __restrict__ units, __half* __restrict__ scale,
                                                           __half* __restrict__ zero, int experts, int n, int nsb, int zmul) {
  using F = kq::Fmt<QT>;
  using U = kq::Unit<QT>;
  int64_t const total = int64_t(experts) * nsb * n;
  int64_t const idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  int const col = int(idx % n);
  int64_t const r = idx / n;
  int const sb = int(r % nsb);
  int const e = int(r / nsb);
  int const nu = nsb / U::kSbPerUnit;
  uint8_t const* u = units + ((int64_t(e) * nu + sb / U::kSbPerUnit) * n + col) * U::kUnitTotal + (sb % U::kSbPerUnit) * U::kSbBytes;
  static_assert(U::kSbBytes % 2 == 0 && U::kUnitTotal % 2 == 0, "shares are read two bytes at a time");
  uint8_t loc[U::kSbBytes];
#pragma unroll
  for (int i = 0; i < U::kSbBytes / 2; ++i) {
    unsigned short const v = __ldg(reinterpret_cast<unsigned short const*>(u) + i);
    loc[2 * i] = uint8_t(v & 0xFF); loc[2 * i + 1] = uint8_t(v >> 8);
  }
  float const df = __half2float(__ushort_as_half(kq::load_u16(loc)));
  float const mf = F::kHasMin ? __half2float(__ushort_as_half(kq::load_u16(loc + 2))) : 0.f;
  int64_t const o0 = ((int64_t(e) * nsb + sb) * F::kGroups) * n + col;
#pragma unroll
  for (int g = 0; g < F::kGroups; ++g) {
    int sc, mn;
    kq::unit_scale_min<QT>(loc, g, sc, mn);
    __half s, z;
    scale_zero_from_codes(df, mf, sc, mn, F::kHasMin, zmul, s, z);
    scale[o0 + int64_t(g) * n] = s; zero[o0 + int64_t(g) * n] = z;
  }
}

#define QB_QT_SWITCH(qtype, CALL)                                                        \
  switch (qtype) { case 10: CALL(10); break; case 11: CALL(11); break; case 12: CALL(12); break; \
                   case 13: CALL(13); break; case 14: CALL(14); break; default: return false; }

bool enqueue_dequantize(uint8_t const* blocks, __half* out, int count, int qtype, cudaStream_t s) {
#define CALL(Q) { if (reinterpret_cast<uintptr_t>(blocks) & 1) dequant_kernel<Q, false><<<(count + kDqBlocks - 1) / kDqBlocks, 256, 0, s>>>(blocks, out, count); \
                  else dequant_kernel<Q, true><<<(count + kDqBlocks - 1) / kDqBlocks, 256, 0, s>>>(blocks, out, count); }
  QB_QT_SWITCH(qtype, CALL)
#undef CALL
  return true;
}

bool enqueue_unpack(uint8_t const* blocks, int8_t* codes, __half* scale, __half* zero, int count, int qtype, cudaStream_t s) {
#define CALL(Q) unpack_kernel<Q><<<(count + 7) / 8, 256, 0, s>>>(blocks, codes, scale, zero, count)
  QB_QT_SWITCH(qtype, CALL)
#undef CALL
  return true;
}

bool enqueue_planes_dequantize(uint8_t const* low, uint8_t const* high, __half const* scale, __half const* zero, __half* out,
                               int experts, int n, int k, int lo, int hi, int gs, int shift, cudaStream_t s) {
  int64_t const rows = int64_t(experts) * n, total = rows * (k >> 3);
  if (total <= 0 || total > int64_t(0x7fffffff) * 256) return false;
  planes_dequant_kernel<<<unsigned((total + 255) / 256), 256, 0, s>>>(low, high, scale, zero, out, rows, n, k, lo, hi, gs, shift);
  return true;
}

bool enqueue_prepass(uint8_t const* sblocks, uint16_t const* d, uint16_t const* dmin, int count, int qtype, int zmul,
                     __half* scale, __half* zero, cudaStream_t s) {
#define CALL(Q) prepass_kernel<Q><<<(count * kq::Fmt<Q>::kGroups + 255) / 256, 256, 0, s>>>(sblocks, d, dmin, count, zmul, scale, zero)
  QB_QT_SWITCH(qtype, CALL)
#undef CALL
  return true;
}

bool enqueue_prepass_unit(uint8_t const* units, __half* scale, __half* zero, int experts, int n, int nsb, int qtype,
                          int zmul, cudaStream_t s) {
#define CALL(Q) { int64_t const total = int64_t(experts) * nsb * n; \
                  prepass_unit_kernel<Q><<<unsigned((total + 255) / 256), 256, 0, s>>>(units, scale, zero, experts, n, nsb, zmul); }
  QB_QT_SWITCH(qtype, CALL)
#undef CALL
  return true;
}

}  // namespace qb
