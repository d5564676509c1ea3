// Mixed-input (fp16/bf16 activation x low-bit weight) GEMM on the 5th-generation tensor cores: dense fpA_intB and
// MoE grouped (ragged rows per expert) in one kernel.
//
//   D[m, n] = sum_k A[m, k] * ( (u[n, k] + off) * S[k/gs, n] + Z[k/gs, n] ),     u = lo + 2^LO * hi
//
//   A     fp16/bf16 [rows][K] row-major; grouped: rows concatenated in expert order, cumulative int offsets [E+1]
//   low   [E][N][K*LO/8], high [E][N][K*HI/8]   Native planes (element k of a row at bit k*bits, LSB first)
//   S, Z  fp16 [E][K/gs][N]  (Z optional)
//   D     fp16/bf16 [rows][N]
//
// Replaces the reference's PPU collectives: dense (quactlize/include/fpA_intB_ppu.cuh:67-194, mainloop
// quactlize/include/quactlize_extensions/cutlass/gemm/collective/quactlize_mma_mixed_input.hpp:985-1250) and grouped
// (quactlize/include/ppu_aiu_gemm_mixed_input_group.hpp:35-311, launcher quactlize/include/moe_grouped_ppu.cuh:69-361).
//
// One CTA computes MT x NT UMMA tiles of 128 rows x 128 weight columns (2 x 2 for prefill-sized problems, 1 x 1 for small
// ones); K advances in stages of 64.  Warp-specialised:
//   warp 0        TMA producer: activation tiles (SWIZZLE_128B, K-major) into their own ring; raw weight planes and
//                 scale/zero rows, in 128-k pieces, into a second ring
//   warp 1        one elected thread issues tcgen05.mma (M=128, N=128*NT, K=16, fp32 accumulators in TMEM) and commits
//   warp 2        allocates / frees the 128*MT*NT TMEM columns
//   warps 4..     4*MT dequant warps: thread = weight column; 64 codes -> 64 fp16/bf16 values written in the UMMA
//                 canonical 128-byte-swizzled K-major layout (third ring); afterwards the same warps read the
//                 accumulators (tcgen05.ld) and store D
// The three rings are sized so that about a microsecond of copies is in flight: a tile's worth of tensor-core work per
// byte of shared memory is what the 2 x 2 shape buys (half the activation bytes per flop of 2 x 1).
// Every mbarrier wait is bounded; a wait that gives up raises a CTA-wide abort flag, records a status code, and the
// CTA drains its copies, frees its TMEM and exits.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "qb_device.cuh"
#include "qb_internal.hpp"
#include "qb_runtime.hpp"
#include "qb_tma.hpp"

namespace qb {

constexpr int kTM = 128, kTN = 128, kTK = 64;       // UMMA tile and K stage
constexpr int kRawK = 128;                          // weight planes and scale rows arrive in 128-k pieces
constexpr int kATileBytes = kTM * kTK * 2;          // 16 KB
constexpr int kBTileBytes = kTN * kTK * 2;          // 16 KB
constexpr int kScaleRows = kRawK / 16;              // 8 group rows per piece at gs = 16
constexpr int kScaleBytes = kScaleRows * kTN * 2;   // 2 KB each for scale and zero

struct GemmArgs {
  int const* offsets;      // cumulative [E+1] (grouped) or nullptr (dense: rows = m_rows)
  void* out;
  int m_rows, n, k, experts, group_size;
  int code_offset, has_zero;
  int splits;              // K slices (gridDim.z); > 1: slice z accumulates its own 128-k pieces and writes fp32 to `partial`
  float* partial;          // [splits][m_rows][n] fp32 (split-K only), summed by splitk_reduce_kernel
  unsigned long long const* out_rows;   // optional: the address output row r is stored at (n elements), instead of out + r*n
  unsigned int* status;
};

// DEPTH 0: rings sized for one CTA per SM (prefill tiles).  DEPTH 1 (128 x 128 only): two-deep rings, about 75 KB, so that
// two or three CTAs share an SM -- decode-sized grouped problems are bound by the latency of one CTA's
// copy -> dequantise -> MMA chain, and co-resident CTAs overlap those chains.
template <int LO, int HI, int MT, int NT, int DEPTH = 0> struct GemmSmem {
  static constexpr bool kBig = MT * NT == 4;
#ifndef QB_GEMM_AST                                          // ring depths of the 256 x 256 tile (compile-time experiment switches)
#define QB_GEMM_AST 3
#endif
#ifndef QB_GEMM_BST
#define QB_GEMM_BST 2
#endif
  // DEPTH 2: the CTA is one of a PAIR (cluster of two along the rows, tcgen05 cta_group::2): it holds only its half of the
  // weight columns (NTB tiles), which pays for deeper rings.
  static constexpr int NTB = DEPTH == 2 ? NT / 2 : NT;
  static constexpr int AST = DEPTH == 2 ? 4 : DEPTH ? 2 : (kBig ? QB_GEMM_AST : 4);   // activation ring: 64-k tiles of 128*MT rows
  static constexpr int BST = DEPTH == 2 ? 3 : DEPTH ? 2 : (kBig ? QB_GEMM_BST : 4);   // dequantised operand ring: 64-k tiles of 128*NTB columns
  static constexpr int RST = DEPTH == 2 ? 3 : DEPTH ? 2 : (kBig ? 2 : 3);             // raw ring: 128-k pieces of planes + scale rows
  static constexpr int kLoBytes = kTN * kRawK * LO / 8, kHiBytes = HI ? kTN * kRawK * HI / 8 : 1024;
  alignas(1024) uint8_t a[AST][MT * kATileBytes];
  alignas(1024) uint8_t b[BST][NTB * kBTileBytes];
  alignas(1024) uint8_t raw_lo[RST][NTB][kLoBytes];  // rows of 16*LO bytes, TMA-swizzled when 64 or 32 bytes long
  alignas(1024) uint8_t raw_hi[RST][NTB][kHiBytes];
  alignas(128) uint8_t scale[RST][NTB][kScaleBytes];
  alignas(128) uint8_t zero[RST][NTB][kScaleBytes];
  alignas(8) uint64_t a_full[AST];             // TMA -> MMA (activation tile landed)
  alignas(8) uint64_t a_empty[AST];            // MMA (tcgen05.commit) -> TMA
  alignas(8) uint64_t b_full[BST];             // dequant warps -> MMA (operand tile written)
  alignas(8) uint64_t b_empty[BST];            // MMA (tcgen05.commit) -> dequant warps
  alignas(8) uint64_t raw_full[RST];           // TMA -> dequant
  alignas(8) uint64_t raw_empty[RST];          // dequant -> TMA
  alignas(8) uint64_t acc_full;                // MMA -> epilogue
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ void tma_load_2d(void* dst, CUtensorMap const* map, int c0, int c1, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, CUtensorMap const* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart (SBO), version 1, layout type 2
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFFu) >> 4);
  d |= uint64_t(1) << 16;                        // leading byte offset (unused for swizzled K-major), 16-byte units
  d |= uint64_t(1024 >> 4) << 32;                // stride byte offset
  d |= uint64_t(1) << 46;                        // descriptor version
  d |= uint64_t(2) << 61;                        // SWIZZLE_128B
  return d;
}
// kind::f16, fp32 accumulate, A and B K-major, M = 128, N = 128; fmt 0 = fp16, 1 = bf16 for both operands
__host__ __device__ constexpr uint32_t umma_idesc(int fmt, int m, int n) {
  return (1u << 4) | (uint32_t(fmt) << 7) | (uint32_t(fmt) << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- the pair form (cluster of two CTAs, tcgen05 cta_group::2) ------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the shared::cluster address of this CTA's shared address `a` in the CTA of rank `rank`
__device__ __forceinline__ uint32_t cluster_addr(uint32_t a, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on a barrier of the partner CTA.  Relaxed: what the arrival publishes (this CTA's operand tile, written for its
// own tensor core) has been made visible by the proxy fence before it; a release at cluster scope here stalls every
// dequantising warp on a cluster-wide memory barrier once per stage.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// activation tile of this CTA, completion counted on the barrier at cluster address `cluster_bar` (the leader's)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, CUtensorMap const* map, int c0, int c1, uint32_t cluster_bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrival on one barrier (cluster address: this CTA's or the partner's) once the pair's MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}

template <class SM>
__device__ __forceinline__ bool gemm_wait(SM& sm, uint64_t* bar, unsigned parity, unsigned int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0;                                  // the clock is first read after 32 failed polls: ordinary waits
  unsigned spins = 0;                                         // of the pipeline never pay for it
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 31u) == 0) {
      if (sm.abort_flag) return false;
      unsigned long long const now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitNs) {
        sm.abort_flag = 1;
        if (status) atomicCAS(status, 0u, unsigned(kWaitMmaTimeout));
        return false;
      }
    }
  }
  return true;
}

// ---- dequantisation of one weight column (64 consecutive k) into the swizzled operand row ---------------------------

template <bool BF16> struct Pack2;
template <> struct Pack2<false> {
  using T2 = __half2;
  static constexpr uint32_t kMagic = 0x64006400u;     // 1024 + u, exact for u < 1024
  __device__ static __forceinline__ T2 bias() { return __float2half2_rn(1024.f); }
  __device__ static __forceinline__ T2 from_f(float a, float b) { return __floats2half2_rn(a, b); }
  __device__ static __forceinline__ uint32_t affine(uint32_t v, T2 s, T2 zo) {
    T2 const u = __hsub2(*reinterpret_cast<T2*>(&v), bias());
    T2 const w = __hfma2(u, s, zo);
    return *reinterpret_cast<uint32_t const*>(&w);
  }
};
template <> struct Pack2<true> {
  using T2 = __nv_bfloat162;
  static constexpr uint32_t kMagic = 0x43004300u;     // 128 + u, exact for u < 128
  __device__ static __forceinline__ T2 bias() { return __float2bfloat162_rn(128.f); }
  __device__ static __forceinline__ T2 from_f(float a, float b) { return __floats2bfloat162_rn(a, b); }
  __device__ static __forceinline__ uint32_t affine(uint32_t v, T2 s, T2 zo) {
    T2 const u = __hsub2(*reinterpret_cast<T2*>(&v), bias());
    T2 const w = __hfma2(u, s, zo);
    return *reinterpret_cast<uint32_t const*>(&w);
  }
};

// Raw plane rows of a 128-k piece are 16*BITS bytes; consecutive columns therefore sit 64 / 32 / 16 bytes apart, which
// would put a warp's loads on a few banks.  The TMA writes 64- and 32-byte rows with the matching swizzle (16-byte chunk
// index XOR row bits), and this reads through the same XOR with the widest load that covers the thread's bytes.
__device__ __forceinline__ uint4 g_lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 g_lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t g_lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ float g_ldsh(uint32_t a) {          // one fp16 -> float
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
  return __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ void g_sts128(uint32_t a, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <int NB, int RB>
__device__ __forceinline__ void load_raw(uint32_t tile, uint32_t off, uint32_t* out) {
  constexpr uint32_t mask = RB == 64 ? 3u : (RB == 32 ? 1u : 0u);
  if constexpr (NB >= 16) {
#pragma unroll
    for (int i = 0; i < NB / 16; ++i) {
      uint32_t const o = off + 16 * i;
      uint4 const v = g_lds128(tile + (o ^ (((o >> 7) & mask) << 4)));
      out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w;
    }
  } else if constexpr (NB == 8) {
    uint2 const v = g_lds64(tile + (off ^ (((off >> 7) & mask) << 4)));
    out[0] = v.x; out[1] = v.y;
  } else {
    static_assert(NB == 4, "a thread converts at least four 8-element chunks of a 1-bit plane");
    out[0] = g_lds32(tile + (off ^ (((off >> 7) & mask) << 4)));
  }
}

// the BITS*8 plane bits of local chunk i out of the words load_raw() returned
template <int BITS>
__device__ __forceinline__ uint32_t chunk_bits(uint32_t const* w, int i) {
  if constexpr (BITS == 4) return w[i];
  else if constexpr (BITS == 2) return (w[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
  else return (w[i >> 2] >> (8 * (i & 3))) & 0xFFu;
}

// One thread converts NC consecutive 8-element chunks (from chunk c0 of the 64-k half h) of weight column `col`.
// lo_tile/hi_tile: the stage's raw 128-k pieces; sc/zr: [group 0][this column] of the scale rows for this half
// (row stride kTN halves).  Output chunk c lands at 16-byte position c ^ (col & 7) of the operand row (SWIZZLE_128B).
// ONE: the whole 64-k stage lies in one scale group (gs >= 64): scale and zero are fetched once and the chunks form one
// straight-line block, which lets the compiler overlap the byte permutes, the half2 arithmetic and the stores of all of them.
template <int LO, int HI, bool BF16, int NC, bool ONE>
__device__ __forceinline__ void dequant_col(uint32_t lo_tile, uint32_t hi_tile, uint32_t sc, uint32_t zr, bool has_zero,
                                            int gs, float coff, uint32_t brow, int col, int h, int c0) {
  using P = Pack2<BF16>;
  uint32_t lw[(NC * LO + 3) / 4], hw[HI ? (NC * HI + 3) / 4 : 1];
  load_raw<NC * LO, 16 * LO>(lo_tile, uint32_t(col * (16 * LO) + h * (8 * LO) + c0 * LO), lw);
  if constexpr (HI > 0) load_raw<NC * HI, 16 * HI>(hi_tile, uint32_t(col * (16 * HI) + h * (8 * HI) + c0 * HI), hw);
  int const gshift = gs >= 64 ? 31 : (gs == 32 ? 2 : 1);          // chunks per group: >= 8 -> one group, 4, or 2
  int gprev = -1;
  typename P::T2 s2, z2;
  if constexpr (ONE) {
    float const s = g_ldsh(sc);
    float const z = (has_zero ? g_ldsh(zr) : 0.f) + coff * s;
    s2 = P::from_f(s, s); z2 = P::from_f(z, z);
  }
#pragma unroll
  for (int i = 0; i < NC; ++i) {
    int const c = c0 + i;
    if constexpr (!ONE) {
      int const g = c >> gshift;
      if (g != gprev) {
        float const s = g_ldsh(sc + uint32_t(g * kTN * 2));
        float const z = (has_zero ? g_ldsh(zr + uint32_t(g * kTN * 2)) : 0.f) + coff * s;
        s2 = P::from_f(s, s); z2 = P::from_f(z, z);
        gprev = g;
      }
    }
    uint32_t v[4];
    if constexpr (LO == 4 && HI == 0) {
      uint32_t const w = lw[i], w4 = w >> 4;
#pragma unroll
      for (int j = 0; j < 4; ++j)                               // byte j: (low nibble, high nibble) = elements 2j, 2j+1
        v[j] = (__byte_perm(w, w4, 0x4400u + 0x1111u * j) & 0x000F000Fu) | P::kMagic;
    } else {
      uint32_t const L = chunk_bits<LO>(lw, i);
      uint32_t const H = HI ? chunk_bits<HI ? HI : 1>(hw, i) : 0u;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t const u0 = ((L >> (2 * j * LO)) & ((1u << LO) - 1u)) | (HI ? (((H >> (2 * j * HI)) & ((1u << HI) - 1u)) << LO) : 0u);
        uint32_t const u1 = ((L >> ((2 * j + 1) * LO)) & ((1u << LO) - 1u)) | (HI ? (((H >> ((2 * j + 1) * HI)) & ((1u << HI) - 1u)) << LO) : 0u);
        v[j] = u0 | (u1 << 16) | P::kMagic;
      }
    }
    uint4 o;
    o.x = P::affine(v[0], s2, z2); o.y = P::affine(v[1], s2, z2);
    o.z = P::affine(v[2], s2, z2); o.w = P::affine(v[3], s2, z2);
    g_sts128(brow + uint32_t((c ^ (col & 7)) << 4), o);
  }
}

// ---- the kernel -----------------------------------------------------------------------------------------------------

// Dequantising warps per epilogue warp.  The 256 x 256 tile converts 16 K codes per 64-k stage; with one warp per 32 rows
// (eight warps, two per scheduler) that conversion, a dependent chain of loads, byte permutes and half2 arithmetic behind
// two barrier waits, took longer than the stage's MMAs and set the pace of the whole kernel (timed with either side
// removed: conversion alone 776 us, MMAs alone 633 us, together 977 us on the 4096 -> 14336 grouped problem).  Twice the
// warps, each converting half of a column's 64 codes, put the tensor pipe back in charge.
#ifndef QB_GEMM_DQ
#define QB_GEMM_DQ 1
#endif
template <int MT, int NT, int DEPTH> constexpr int gemm_dq() { return (MT == 2 && NT == 2 && DEPTH == 0) ? QB_GEMM_DQ : 1; }

template <int LO, int HI, bool BF16, int MT, int NT, int DEPTH>
__global__ void __launch_bounds__(128 + 128 * MT * gemm_dq<MT, NT, DEPTH>(), DEPTH == 1 ? 2 : 1)
mixed_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_lo,
                  const __grid_constant__ CUtensorMap map_hi, const __grid_constant__ CUtensorMap map_s,
                  const __grid_constant__ CUtensorMap map_z, GemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  using SM = GemmSmem<LO, HI, MT, NT, DEPTH>;
  constexpr int AST = SM::AST, BST = SM::BST, RST = SM::RST, kRows = kTM * MT, kCols = kTN * NT;
  constexpr bool PAIR = DEPTH == 2;                           // one of two CTAs of a cluster: rows 256*rank.. of a 512-row tile,
  constexpr int NTB = SM::NTB, kColsB = kTN * NTB;            // all 256 accumulator columns, but only half of the weight columns
  constexpr int kRowsTile = PAIR ? 2 * kRows : kRows;         // rows of the tile a row-tile index names
  static_assert(!PAIR || (MT == 2 && NT == 2), "the pair form is the 512 x 256 tile");
  constexpr int DQ = gemm_dq<MT, NT, DEPTH>();
  constexpr int kDqWarps = 4 * MT * DQ;                       // the first 4*MT of them also run the epilogue: one per 32 accumulator lanes
  constexpr int NC = 8 * NTB / MT / DQ;                       // 8-element chunks a dequant thread converts per stage
  static_assert(NC >= 1 && NC * MT * DQ == 8 * NTB, "the dequant threads tile a stage's chunks exactly");
  uint32_t const crank = PAIR ? cluster_ctarank() : 0u;
  SM& sm = *reinterpret_cast<SM*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  int const warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- which tile: blockIdx.x = weight-column tile, blockIdx.y = row tile (grouped: searched in the per-expert counts)
  int e = 0, m0, mrows;
  if (g.offsets) {
    // warp 0 scans the per-expert tile counts 32 experts at a time (a decode launch has over a hundred experts and
    // most CTAs of the grid's upper bound find no tile: the lookup is their whole cost)
    __shared__ int tile_of[4];                                // expert, first row, rows, found
    if (warp == 0) {
      int const t = blockIdx.y;
      int carry = 0, hit_e = -1, hit_m0 = 0, hit_rows = 0;
      for (int base = 0; base < g.experts && hit_e < 0; base += 32) {
        int const x = base + lane;
        int r0 = 0, rows = 0;
        if (x < g.experts) { r0 = g.offsets[x]; rows = g.offsets[x + 1] - r0; }
        int const cnt = (rows + kRowsTile - 1) / kRowsTile;
        int incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { int const u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
        int const lo = carry + incl - cnt;                    // tiles before this expert
        bool const mine = cnt > 0 && t >= lo && t < lo + cnt;
        unsigned const who = __ballot_sync(0xffffffffu, mine);
        if (who) {
          int const src = __ffs(who) - 1;
          hit_e = __shfl_sync(0xffffffffu, x, src);
          int const lo_s = __shfl_sync(0xffffffffu, lo, src), r0_s = __shfl_sync(0xffffffffu, r0, src),
                    rows_s = __shfl_sync(0xffffffffu, rows, src);
          hit_m0 = r0_s + (t - lo_s) * kRowsTile;
          hit_rows = min(kRowsTile, rows_s - (t - lo_s) * kRowsTile);
        }
        carry += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) { tile_of[0] = hit_e; tile_of[1] = hit_m0; tile_of[2] = hit_rows; }
    }
    __syncthreads();
    e = tile_of[0]; m0 = tile_of[1]; mrows = tile_of[2];
    if (e < 0) return;                                        // uniform for the CTA (and the pair), before any mbarrier or TMEM allocation
  } else {
    int const t = blockIdx.y;
    m0 = t * kRowsTile; mrows = min(kRowsTile, g.m_rows - m0);
    if (mrows <= 0) return;
  }
  // Row blocks the MMAs cover: in the pair form block mt is rows 128*mt.. of BOTH CTAs' halves, and the leader's half is
  // the fuller one, so the count comes from the whole tile's rows.  Then this CTA's own rows (none, for the partner of a
  // tile of up to 256 rows: it still runs the pipeline, its half of the operand is needed, and stores nothing).
  int const mt_here = min(MT, (mrows + kTM - 1) / kTM);       // a ragged row tile may end in the first 128 rows
  if constexpr (PAIR) { m0 += int(crank) * kRows; mrows = max(0, min(kRows, mrows - int(crank) * kRows)); }
  int const n0 = (PAIR ? int(blockIdx.x >> 1) : int(blockIdx.x)) * kCols;   // the pair's two CTAs are neighbours along x
  int const nb0 = n0 + int(crank) * kColsB;                   // first weight column this CTA converts (pair form: its half)
  int const nt_here = PAIR ? NT : min(NT, (g.n - n0) / kTN);  // a 256-wide tile may hang over the last 128 columns
  // split-K: slice z owns a contiguous run of 128-k pieces (pieces are dealt as evenly as they divide); its stages are
  // numbered from 0 for the rings, and offset by ks0 stages / p0 pieces where global k coordinates are formed
  int const pieces = g.k / kRawK, z = blockIdx.z, S = g.splits;
  int const p0 = int((long long)pieces * z / S), p1 = int((long long)pieces * (z + 1) / S);
  int const ks0 = 2 * p0;
  int const nks = 2 * (p1 - p0);                              // 64-k stages of this slice (k is a multiple of 256)
  int const gs = g.group_size;
  int const srows = gs >= kRawK ? 1 : kRawK / gs;             // scale rows per 128-k piece

  if (threadIdx.x == 0) {
    for (int s = 0; s < AST; ++s) { mbar_init(&sm.a_full[s], 1); mbar_init(&sm.a_empty[s], 1); }
    for (int s = 0; s < BST; ++s) { mbar_init(&sm.b_full[s], PAIR ? 2 * kDqWarps : kDqWarps); mbar_init(&sm.b_empty[s], 1); }
    for (int s = 0; s < RST; ++s) { mbar_init(&sm.raw_full[s], 1); mbar_init(&sm.raw_empty[s], kDqWarps); }
    mbar_init(&sm.acc_full, 1);
    sm.abort_flag = 0;
    mbar_init_fence();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 2) {
    if constexpr (PAIR) {                                     // the same warp of both CTAs, the same destination offset
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(uint32_t(kTN * MT * NT)) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(uint32_t(kTN * MT * NT)) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if constexpr (PAIR) cluster_sync_all();                     // the partner's barriers exist before anything arrives on them
  uint32_t const tmem = sm.tmem_base;

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      unsigned const raw_bytes = unsigned(NTB) * (unsigned(kTN * kRawK * LO / 8) + unsigned(kTN * kRawK * HI / 8) +
                                                 unsigned(srows * kTN * 2) * (g.has_zero ? 2u : 1u));
      for (int i = 0; i < nks; ++i) {
        int const sa = i % AST;
        if ((i & 1) == 0) {
          int const j = i >> 1, r = j % RST;
          if (j >= RST && !gemm_wait(sm, &sm.raw_empty[r], unsigned(j / RST - 1) & 1u, g.status)) break;
          mbar_expect_tx(&sm.raw_full[r], raw_bytes);
          int const kk = (p0 + j) * kRawK;
#pragma unroll
          for (int nt = 0; nt < NTB; ++nt) {                   // columns past n are out of bounds: zero-filled, still counted
            tma_load_3d(sm.raw_lo[r][nt], &map_lo, kk * LO / 8, nb0 + nt * kTN, e, &sm.raw_full[r]);
            if constexpr (HI != 0) tma_load_3d(sm.raw_hi[r][nt], &map_hi, kk * HI / 8, nb0 + nt * kTN, e, &sm.raw_full[r]);
            tma_load_3d(sm.scale[r][nt], &map_s, nb0 + nt * kTN, kk / gs, e, &sm.raw_full[r]);
            if (g.has_zero) tma_load_3d(sm.zero[r][nt], &map_z, nb0 + nt * kTN, kk / gs, e, &sm.raw_full[r]);
          }
        }
        if (i >= AST && !gemm_wait(sm, &sm.a_empty[sa], unsigned(i / AST - 1) & 1u, g.status)) break;
#ifdef QB_GABL_NOA
        if (i >= AST) { mbar_arrive(&sm.a_full[sa]); continue; }
#endif
        if constexpr (PAIR) {
          // both CTAs' activation tiles are counted on the LEADER's barrier, which the leader arms for both
          if (crank == 0) mbar_expect_tx(&sm.a_full[sa], 2 * MT * kATileBytes);
          tma_load_2d_pair(sm.a[sa], &map_a, (ks0 + i) * kTK, m0, cluster_addr(smem_u32(&sm.a_full[sa]), 0));
        } else {
          mbar_expect_tx(&sm.a_full[sa], MT * kATileBytes);
          tma_load_2d(sm.a[sa], &map_a, (ks0 + i) * kTK, m0, &sm.a_full[sa]);
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0 && crank == 0) {                             // pair form: the leader issues for both CTAs
      uint32_t const idesc = umma_idesc(BF16 ? 1 : 0, PAIR ? 2 * kTM : kTM, kTN * nt_here);
      bool ok = true;
      for (int i = 0; i < nks && ok; ++i) {
        int const sa = i % AST, sb = i % BST;
        ok = gemm_wait(sm, &sm.a_full[sa], unsigned(i / AST) & 1u, g.status) &&
             gemm_wait(sm, &sm.b_full[sb], unsigned(i / BST) & 1u, g.status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t const a_addr = smem_u32(sm.a[sa]), b_addr = smem_u32(sm.b[sb]);
#ifndef QB_GABL_NOMMA
#pragma unroll
        for (int kk = 0; kk < kTK / 16; ++kk)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)                      // every row block multiplies the same dequantised operand tile
            if (mt < mt_here) {
              if constexpr (PAIR)
                umma_f16_pair(tmem + mt * kCols, umma_desc_sw128(a_addr + mt * kATileBytes + kk * 32), umma_desc_sw128(b_addr + kk * 32),
                              idesc, (i | kk) ? 1u : 0u);
              else
                umma_f16(tmem + mt * kCols, umma_desc_sw128(a_addr + mt * kATileBytes + kk * 32), umma_desc_sw128(b_addr + kk * 32),
                         idesc, (i | kk) ? 1u : 0u);
            }
#endif
        if constexpr (PAIR) {                                  // frees the slots in BOTH CTAs once these MMAs have read them
          uint32_t const ae = smem_u32(&sm.a_empty[sa]), be = smem_u32(&sm.b_empty[sb]);
          umma_commit_pair(cluster_addr(ae, 0)); umma_commit_pair(cluster_addr(ae, 1));
          umma_commit_pair(cluster_addr(be, 0)); umma_commit_pair(cluster_addr(be, 1));
        } else {
          umma_commit(&sm.a_empty[sa]);                        // frees the rings' slots once these MMAs have read them
          umma_commit(&sm.b_empty[sb]);
        }
      }
      if (ok) {
        if constexpr (PAIR) {
          uint32_t const af = smem_u32(&sm.acc_full);
          umma_commit_pair(cluster_addr(af, 0)); umma_commit_pair(cluster_addr(af, 1));
        } else {
          umma_commit(&sm.acc_full);
        }
      }
    }
  } else if (warp >= 4) {
    // ================= dequantise (thread = weight column), then epilogue =================
    int const t = threadIdx.x - 128;
    int const col = t % kColsB, part = t / kColsB;             // the CTA's weight columns x (128*MT*DQ / columns) chunk ranges
    int const nt = col >> 7, cin = col & 127;
    bool const live = nt < nt_here;
    float const coff = float(g.code_offset);
    bool ok = true;
    for (int i = 0; i < nks && ok; ++i) {
      int const sb = i % BST, j = i >> 1, r = j % RST, h = i & 1;
      if (h == 0) ok = gemm_wait(sm, &sm.raw_full[r], unsigned(j / RST) & 1u, g.status);
      if (ok && i >= BST) ok = gemm_wait(sm, &sm.b_empty[sb], unsigned(i / BST - 1) & 1u, g.status);
      if (!ok) break;
      int const srow = gs >= kRawK ? 0 : h * (srows / 2);
#ifndef QB_GABL_NODEQ
      if (live) {
        uint32_t const sc_a = smem_u32(sm.scale[r][nt]) + uint32_t((srow * kTN + cin) * 2);
        uint32_t const zr_a = smem_u32(sm.zero[r][nt]) + uint32_t((srow * kTN + cin) * 2);
        if (gs >= 64)
          dequant_col<LO, HI, BF16, NC, true>(smem_u32(sm.raw_lo[r][nt]), smem_u32(sm.raw_hi[r][nt]), sc_a, zr_a, g.has_zero != 0,
                                              gs, coff, smem_u32(sm.b[sb]) + uint32_t(col * 128), cin, h, part * NC);
        else
          dequant_col<LO, HI, BF16, NC, false>(smem_u32(sm.raw_lo[r][nt]), smem_u32(sm.raw_hi[r][nt]), sc_a, zr_a, g.has_zero != 0,
                                               gs, coff, smem_u32(sm.b[sb]) + uint32_t(col * 128), cin, h, part * NC);
      }
#endif
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy writes -> visible to the MMA
      __syncwarp();
      if (lane == 0) {
        if (PAIR && crank != 0) mbar_arrive_cluster(cluster_addr(smem_u32(&sm.b_full[sb]), 0));   // the leader's barrier counts both CTAs' warps
        else mbar_arrive(&sm.b_full[sb]);
        if (h == 1) mbar_arrive(&sm.raw_empty[r]);
      }
    }
    // epilogue: this warp owns TMEM lanes 32*(warp%4) .. +31 of row block mt = 32 output rows of the tile
    if (ok) ok = gemm_wait(sm, &sm.acc_full, 0, g.status);
    int const q = warp & 3, mt = (warp - 4) >> 2, row = mt * kTM + q * 32 + lane;
    if (ok && mt < mt_here) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      size_t const orow = size_t(m0 + row) * g.n + n0;
#pragma unroll 1
      for (int c = 0; c < kTN * nt_here; c += 32) {
        uint32_t v[32];
        uint32_t const taddr = tmem + (uint32_t(q * 32) << 16) + uint32_t(mt * kCols + c);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
              "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
              "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
              "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(taddr) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (S > 1) {                                           // fp32 partial sums of this K slice
          if (row < mrows) {
            float4* dst = reinterpret_cast<float4*>(g.partial + (size_t(z) * g.m_rows + size_t(m0 + row)) * g.n + n0 + c);
#pragma unroll
            for (int u = 0; u < 8; ++u)
              dst[u] = make_float4(__uint_as_float(v[4 * u]), __uint_as_float(v[4 * u + 1]), __uint_as_float(v[4 * u + 2]),
                                   __uint_as_float(v[4 * u + 3]));
          }
        } else if (row < mrows) {
          uint32_t pk[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            float const f0 = __uint_as_float(v[2 * u]), f1 = __uint_as_float(v[2 * u + 1]);
            if constexpr (BF16) { __nv_bfloat162 const hh = __floats2bfloat162_rn(f0, f1); pk[u] = *reinterpret_cast<uint32_t const*>(&hh); }
            else { __half2 const hh = __floats2half2_rn(f0, f1); pk[u] = *reinterpret_cast<uint32_t const*>(&hh); }
          }
          // a row map sends every output row to its own destination (another rank's buffer in expert parallelism: plain
          // 16-byte stores, peer memory is written but never read here)
          uint4* dst = g.out_rows ? reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(g.out_rows[m0 + row]) + n0 + c)
                                  : reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(g.out) + orow + c);
#pragma unroll
          for (int u = 0; u < 4; ++u) dst[u] = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
        }
      }
    }
  }
  // ---- teardown: everyone meets here (all waits are bounded), then the allocating warp frees the TMEM columns
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (sm.abort_flag && threadIdx.x == 0) {
    // drain copies that may still be in flight so they do not land in shared memory handed to another CTA
    for (int s = 0; s < AST; ++s) { (void)mbar_wait_bounded(&sm.a_full[s], 0, nullptr, 0, 100000000ull); (void)mbar_wait_bounded(&sm.a_full[s], 1, nullptr, 0, 100000000ull); }
    for (int s = 0; s < RST; ++s) { (void)mbar_wait_bounded(&sm.raw_full[s], 0, nullptr, 0, 100000000ull); (void)mbar_wait_bounded(&sm.raw_full[s], 1, nullptr, 0, 100000000ull); }
  }
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();                     // neither CTA's shared or tensor memory goes while the other may use it
  if (warp == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if constexpr (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(uint32_t(kTN * MT * NT)) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(uint32_t(kTN * MT * NT)) : "memory");
  }
}

// ---- the swapped form: weights as the A operand, converted straight into TENSOR MEMORY -------------------------------------
//
// In the kernel above every dequantised weight crosses shared memory twice more than it has to (the converting thread
// stores it, the tensor core reads it back once per row block).  tcgen05.mma can take its A operand from tensor memory,
// so here the roles are swapped: D[n][token] = W[n][k] * X[token][k]^T with A = 128 weight rows (one per TMEM lane, two
// 16-bit elements per 32-bit column) and B = up to 192 activation rows from shared memory.  A converting thread owns ONE
// weight row: it reads the 64 codes of the row's stage from the raw ring, converts them in registers and writes them
// with one tcgen05.st (left in flight while the next stage is converted) into a ring of TMEM columns; the dequantised
// operand never touches shared memory.  The CTA tile is 256 weight rows (two blocks of 128 = two accumulators) x 192
// tokens: the 512 TMEM columns hold 2 x 192 accumulator columns and a two-deep operand ring of 32 columns per block.
// The accumulator holds [weight row][token], so the epilogue stores transposed: for one token the 32 lanes of a warp
// write 32 consecutive outputs.  int4 planes (LO = 4, HI = 0), one K slice; the other formats and split-K use the kernel
// above.  Results are bit-identical to the kernel above (same conversion arithmetic, same K order).
//
// Measured on the 4096 -> 14336 grouped problem (8192 rows): 1.10 ms against 0.97 ms above, so this form is opt-in.  What
// it showed: with the MMAs compiled out (QB_SWAP_NOMMA) 0.94 ms, with the TMEM stores compiled out (QB_SWAP_NOST)
// 0.89 ms, deeper activation rings (QB_SWAP_XS = 6) no change, smaller token tiles slower (160: 1.24 ms, 128: 1.44 ms);
// a first version with one block of 128 rows x 256 tokens, which re-reads the activations once per 128 weight rows, took
// 1.21 ms while moving 8.4 GB from L2, i.e. 7 TB/s.  Every variant, and the kernel above with its conversion compiled out
// (0.63 ms, 4.7 GB), tops out at about 26 bytes per clock and SM of tensor copies into shared memory -- about 4 cycles
// per box row of at most 128 bytes (388 rows per stage above: 1 570 cycles; 324 here: 1 300-1 490): the rows a tile needs
// per flop set the floor, the rings' depth does not, and the conversion path comes on top of it.
#ifndef QB_SWAP_TOKENS
#define QB_SWAP_TOKENS 192
#endif
constexpr int kSwapTokens = QB_SWAP_TOKENS;                    // activation rows per CTA tile (the MMAs' N)
constexpr int kSwapACol = 2 * kSwapTokens;                     // first TMEM column of the operand ring (the accumulators are below)
struct SwapSmem {
#ifndef QB_SWAP_XS
#define QB_SWAP_XS 4
#endif
  static constexpr int XS = QB_SWAP_XS, RS = 3;                // activation ring, raw ring
  static constexpr int TS = (512 - 2 * kSwapTokens) / 64;      // TMEM operand ring per block: what the accumulators leave
  static_assert(kSwapTokens % 16 == 0 && kSwapTokens <= 192 && TS >= 2, "two accumulators and at least a two-deep operand ring");
  alignas(1024) uint8_t x[XS][kSwapTokens * kTK * 2];          // 192 tokens x 64 k, K-major, 128-byte swizzle
  alignas(1024) uint8_t raw_lo[RS][2][kTN * kRawK / 2];        // per block: 128 weight rows x 64 bytes (128 k), TMA-swizzled
  alignas(128) uint8_t scale[RS][2][kScaleBytes];
  alignas(128) uint8_t zero[RS][2][kScaleBytes];
  alignas(8) uint64_t x_full[XS];                              // TMA -> MMA
  alignas(8) uint64_t x_empty[XS];                             // MMA (tcgen05.commit) -> TMA
  alignas(8) uint64_t raw_full[RS];                            // TMA -> converting warps
  alignas(8) uint64_t raw_empty[RS];                           // converting warps -> TMA
  alignas(8) uint64_t a_full[2][TS];                           // a block's converting warps (tcgen05.st done) -> MMA
  alignas(8) uint64_t a_empty[2][TS];                          // MMA (tcgen05.commit) -> the block's converting warps
  alignas(8) uint64_t acc_full;
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

template <bool BF16>
__global__ void __launch_bounds__(384, 1)
mixed_gemm_swap_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_lo,
                       const __grid_constant__ CUtensorMap map_s, const __grid_constant__ CUtensorMap map_z, GemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  using SM = SwapSmem;
  using P = Pack2<BF16>;
  constexpr int XS = SM::XS, RS = SM::RS, TS = SM::TS;
  SM& sm = *reinterpret_cast<SM*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  int const warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- which tile: blockIdx.x = tile of 256 weight rows, blockIdx.y = tile of 192 tokens (grouped: searched in the counts)
  int e = 0, m0, mrows;
  if (g.offsets) {
    __shared__ int tile_of[4];
    if (warp == 0) {
      int const t = blockIdx.y;
      int carry = 0, hit_e = -1, hit_m0 = 0, hit_rows = 0;
      for (int base = 0; base < g.experts && hit_e < 0; base += 32) {
        int const x = base + lane;
        int r0 = 0, rows = 0;
        if (x < g.experts) { r0 = g.offsets[x]; rows = g.offsets[x + 1] - r0; }
        int const cnt = (rows + kSwapTokens - 1) / kSwapTokens;
        int incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { int const u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
        int const lo = carry + incl - cnt;
        bool const mine = cnt > 0 && t >= lo && t < lo + cnt;
        unsigned const who = __ballot_sync(0xffffffffu, mine);
        if (who) {
          int const src = __ffs(who) - 1;
          hit_e = __shfl_sync(0xffffffffu, x, src);
          int const lo_s = __shfl_sync(0xffffffffu, lo, src), r0_s = __shfl_sync(0xffffffffu, r0, src),
                    rows_s = __shfl_sync(0xffffffffu, rows, src);
          hit_m0 = r0_s + (t - lo_s) * kSwapTokens;
          hit_rows = min(kSwapTokens, rows_s - (t - lo_s) * kSwapTokens);
        }
        carry += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) { tile_of[0] = hit_e; tile_of[1] = hit_m0; tile_of[2] = hit_rows; }
    }
    __syncthreads();
    e = tile_of[0]; m0 = tile_of[1]; mrows = tile_of[2];
    if (e < 0) return;                                        // uniform for the CTA, before any mbarrier or TMEM allocation
  } else {
    m0 = int(blockIdx.y) * kSwapTokens; mrows = min(kSwapTokens, g.m_rows - m0);
    if (mrows <= 0) return;
  }
  // a wait of an earlier CTA of this process gave up: do not queue thousands of CTAs behind the same failure
  if (g.status && *reinterpret_cast<volatile unsigned int*>(g.status) != 0u) return;
  int const n0 = int(blockIdx.x) * (2 * kTN);
  int const ncols = max(16, (mrows + 15) & ~15);              // the MMAs' N: tokens of this tile, in sixteens
  int const nks = g.k / kTK;                                  // 64-k stages (k is a multiple of 128)
  int const gs = g.group_size;
  int const srows = gs >= kRawK ? 1 : kRawK / gs;             // scale rows per 128-k piece

  if (threadIdx.x == 0) {
    for (int s = 0; s < XS; ++s) { mbar_init(&sm.x_full[s], 1); mbar_init(&sm.x_empty[s], 1); }
    for (int s = 0; s < RS; ++s) { mbar_init(&sm.raw_full[s], 1); mbar_init(&sm.raw_empty[s], 8); }
    for (int b = 0; b < 2; ++b)
      for (int s = 0; s < TS; ++s) { mbar_init(&sm.a_full[b][s], 4); mbar_init(&sm.a_empty[b][s], 1); }
    mbar_init(&sm.acc_full, 1);
    sm.abort_flag = 0;
    mbar_init_fence();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  uint32_t const tmem = sm.tmem_base;

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      unsigned const raw_bytes = 2u * (unsigned(kTN * kRawK / 2) + unsigned(srows * kTN * 2) * (g.has_zero ? 2u : 1u));
      for (int i = 0; i < nks; ++i) {
        if ((i & 1) == 0) {
          int const j = i >> 1, r = j % RS;
          if (j >= RS && !gemm_wait(sm, &sm.raw_empty[r], unsigned(j / RS - 1) & 1u, g.status)) break;
          mbar_expect_tx(&sm.raw_full[r], raw_bytes);
          int const kk = j * kRawK;
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            tma_load_3d(sm.raw_lo[r][b], &map_lo, kk / 2, n0 + b * kTN, e, &sm.raw_full[r]);
            tma_load_3d(sm.scale[r][b], &map_s, n0 + b * kTN, kk / gs, e, &sm.raw_full[r]);
            if (g.has_zero) tma_load_3d(sm.zero[r][b], &map_z, n0 + b * kTN, kk / gs, e, &sm.raw_full[r]);
          }
        }
        int const sx = i % XS;
        if (i >= XS && !gemm_wait(sm, &sm.x_empty[sx], unsigned(i / XS - 1) & 1u, g.status)) break;
        mbar_expect_tx(&sm.x_full[sx], kSwapTokens * kTK * 2);
        tma_load_2d(sm.x[sx], &map_x, i * kTK, m0, &sm.x_full[sx]);
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0) {
      uint32_t const idesc = umma_idesc(BF16 ? 1 : 0, kTM, ncols);
      bool ok = true;
      for (int i = 0; i < nks && ok; ++i) {
        int const sx = i % XS, sa = i % TS;
        ok = gemm_wait(sm, &sm.x_full[sx], unsigned(i / XS) & 1u, g.status);
        uint32_t const x_addr = smem_u32(sm.x[sx]);
#pragma unroll
        for (int b = 0; b < 2 && ok; ++b) {
          ok = gemm_wait(sm, &sm.a_full[b][sa], unsigned(i / TS) & 1u, g.status);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
#ifndef QB_SWAP_NOMMA
          for (int kk = 0; kk < kTK / 16; ++kk)                // 16 k per instruction = 8 TMEM columns of the operand
            umma_f16_ts(tmem + uint32_t(b * kSwapTokens), tmem + uint32_t(kSwapACol + (b * TS + sa) * 32 + kk * 8),
                        umma_desc_sw128(x_addr + kk * 32), idesc, (i | kk) ? 1u : 0u);
#endif
          umma_commit(&sm.a_empty[b][sa]);                     // frees the block's operand slot once these MMAs have read it
        }
        if (ok) umma_commit(&sm.x_empty[sx]);
      }
      if (ok) umma_commit(&sm.acc_full);
    }
  } else if (warp >= 4) {
    // ================= convert (warpgroup = block of 128 weight rows, thread = weight row = TMEM lane), then epilogue =====
    int const t = threadIdx.x - 128, blk = t >> 7, q = warp & 3, rr = q * 32 + lane;
    float const coff = float(g.code_offset);
    int const gsh = 31 - __clz(gs);
    uint32_t const lane_base = uint32_t(q * 32) << 16;
    // The store of stage i into tensor memory is left in flight while stage i+1 is loaded and converted: its completion
    // is awaited (and the stage handed to the MMA warp) just before the next store is issued.
    bool ok = true;
    int pending = -1;                                          // operand slot whose tcgen05.st has been issued but not yet published
    for (int i = 0; i < nks && ok; ++i) {
      int const sa = i % TS, j = i >> 1, r = j % RS, h = i & 1;
      if (h == 0) ok = gemm_wait(sm, &sm.raw_full[r], unsigned(j / RS) & 1u, g.status);
      if (!ok) break;
      int const kofs = h * 64;                                 // this stage's 64 codes inside the 128-k piece
      uint32_t lw[8];
      load_raw<32, 64>(smem_u32(sm.raw_lo[r][blk]), uint32_t(rr * 64 + kofs / 2), lw);
      uint32_t o[32];
      int gprev = -1;
      typename P::T2 s2, z2;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        int const grow = gs >= kRawK ? 0 : ((kofs + 8 * c) >> gsh);
        if (grow != gprev) {
          float const s = g_ldsh(smem_u32(sm.scale[r][blk]) + uint32_t((grow * kTN + rr) * 2));
          float const z = (g.has_zero ? g_ldsh(smem_u32(sm.zero[r][blk]) + uint32_t((grow * kTN + rr) * 2)) : 0.f) + coff * s;
          s2 = P::from_f(s, s); z2 = P::from_f(z, z);
          gprev = grow;
        }
        uint32_t const w = lw[c], w4 = w >> 4;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)                          // byte jj: (low nibble, high nibble) = elements 2jj, 2jj+1
          o[4 * c + jj] = P::affine((__byte_perm(w, w4, 0x4400u + 0x1111u * jj) & 0x000F000Fu) | P::kMagic, s2, z2);
      }
      __syncwarp();                                            // every lane has read its codes and scales of this piece
      if (lane == 0 && h == 1) mbar_arrive(&sm.raw_empty[r]);
      if (pending >= 0) {                                      // publish the previous stage
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.a_full[blk][pending]);
      }
      if (i >= TS) ok = gemm_wait(sm, &sm.a_empty[blk][sa], unsigned(i / TS - 1) & 1u, g.status);
      if (!ok) { pending = -1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t const taddr = tmem + lane_base + uint32_t(kSwapACol + (blk * TS + sa) * 32);
#ifndef QB_SWAP_NOST
      asm volatile(
          "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
          "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
          ::"r"(taddr), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]), "r"(o[8]),
            "r"(o[9]), "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]), "r"(o[14]), "r"(o[15]), "r"(o[16]), "r"(o[17]),
            "r"(o[18]), "r"(o[19]), "r"(o[20]), "r"(o[21]), "r"(o[22]), "r"(o[23]), "r"(o[24]), "r"(o[25]), "r"(o[26]),
            "r"(o[27]), "r"(o[28]), "r"(o[29]), "r"(o[30]), "r"(o[31]) : "memory");
#else
      asm volatile("" ::"r"(taddr), "r"(o[0] ^ o[7] ^ o[13] ^ o[31]) : "memory");
#endif
      pending = sa;
    }
    if (pending >= 0) {
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.a_full[blk][pending]);
    }
    // epilogue: TMEM lane rr of accumulator blk = weight row n0 + 128*blk + rr; 32 tokens at a time
    if (ok) ok = gemm_wait(sm, &sm.acc_full, 0, g.status);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c = 0; c < mrows; c += 32) {
        uint32_t v[32];
        uint32_t const taddr = tmem + lane_base + uint32_t(blk * kSwapTokens + c);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
              "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
              "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
              "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(taddr) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int u = 0; u < 32; ++u) {
          if (c + u < mrows) {                                  // uniform for the warp
            float const f = __uint_as_float(v[u]);
            uint16_t bits;
            if constexpr (BF16) { __nv_bfloat16 const hh = __float2bfloat16_rn(f); bits = *reinterpret_cast<uint16_t const*>(&hh); }
            else { __half const hh = __float2half_rn(f); bits = *reinterpret_cast<uint16_t const*>(&hh); }
            // a row map sends every output row to its own destination (peer memory is written, never read)
            uint16_t* dst = g.out_rows ? reinterpret_cast<uint16_t*>(g.out_rows[m0 + c + u]) + n0 + blk * kTN + rr
                                       : reinterpret_cast<uint16_t*>(g.out) + size_t(m0 + c + u) * g.n + n0 + blk * kTN + rr;
            *dst = bits;
          }
        }
      }
    }
  }
  // ---- teardown: everyone meets here (all waits are bounded), then the allocating warp frees the TMEM columns
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (sm.abort_flag && threadIdx.x == 0) {
    // drain copies that may still be in flight so they do not land in shared memory handed to another CTA
    for (int s = 0; s < XS; ++s) { (void)mbar_wait_bounded(&sm.x_full[s], 0, nullptr, 0, 100000000ull); (void)mbar_wait_bounded(&sm.x_full[s], 1, nullptr, 0, 100000000ull); }
    for (int s = 0; s < RS; ++s) { (void)mbar_wait_bounded(&sm.raw_full[s], 0, nullptr, 0, 100000000ull); (void)mbar_wait_bounded(&sm.raw_full[s], 1, nullptr, 0, 100000000ull); }
  }
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// Light reduce of the split-K partial planes: out[r][c] = sum_z partial[z][r][c], converted to the output type.  A thread
// owns four consecutive columns; slices are summed in slice order, so the result does not depend on scheduling.
template <bool BF16>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(float const* __restrict__ partial, void* __restrict__ out,
                                                            int64_t elems, int splits) {
  int64_t const i = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i >= elems) return;
  float4 acc = *reinterpret_cast<float4 const*>(partial + i);
  for (int z = 1; z < splits; ++z) {
    float4 const v = *reinterpret_cast<float4 const*>(partial + int64_t(z) * elems + i);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  uint2 o;
  if constexpr (BF16) {
    __nv_bfloat162 const a = __floats2bfloat162_rn(acc.x, acc.y), b = __floats2bfloat162_rn(acc.z, acc.w);
    o.x = *reinterpret_cast<uint32_t const*>(&a); o.y = *reinterpret_cast<uint32_t const*>(&b);
  } else {
    __half2 const a = __floats2half2_rn(acc.x, acc.y), b = __floats2half2_rn(acc.z, acc.w);
    o.x = *reinterpret_cast<uint32_t const*>(&a); o.y = *reinterpret_cast<uint32_t const*>(&b);
  }
  *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(out) + i) = o;
}

// ---- host side: tensor maps and launch ---------------------------------------------------------------------------------

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, cuuint64_t const*, cuuint64_t const*,
                                   cuuint32_t const*, cuuint32_t const*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

bool make_map(CUtensorMap* m, CUtensorMapDataType dt, int rank, void const* base, cuuint64_t const* dims,
              cuuint64_t const* strides_bytes, cuuint32_t const* box, CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint32_t const ones[3] = {1, 1, 1};
  return fn(m, dt, cuuint32_t(rank), const_cast<void*>(base), dims, strides_bytes, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// swizzle of a raw plane tile by its row length (what load_raw() undoes)
inline CUtensorMapSwizzle plane_swizzle(int row_bytes) {
  return row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : (row_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE);
}

// The four maps over a weight artifact depend only on its pointers and shape: a model's weights are launched again and
// again, so they are encoded once and kept (per plane-width instantiation; the map of the activations is encoded per launch).
template <int LO, int HI>
int weight_maps(GemmDesc const& d, int E, CUtensorMap& ml, CUtensorMap& mh, CUtensorMap& ms, CUtensorMap& mz) {
  int const gs = d.group_size;
  int const srows = gs >= kRawK ? 1 : kRawK / gs;
  struct WKey {
    void const *lo, *hi, *sc, *ze; int n, k, e, gs;
    bool operator<(WKey const& o) const {
      return std::tie(lo, hi, sc, ze, n, k, e, gs) < std::tie(o.lo, o.hi, o.sc, o.ze, o.n, o.k, o.e, o.gs);
    }
  };
  struct WMaps { CUtensorMap ml, mh, ms, mz; };
  static std::map<WKey, WMaps> cache;
  static std::mutex cmu;
  WKey const key{d.low, HI ? d.high : nullptr, d.scale, d.zero, d.n, d.k, E, gs};
  std::lock_guard<std::mutex> lock(cmu);
  auto it = cache.find(key);
  if (it == cache.end()) {
    WMaps w{};
    {
      cuuint64_t const rb = cuuint64_t(d.k) * LO / 8;
      cuuint64_t dims[3] = {rb, cuuint64_t(d.n), cuuint64_t(E)};
      cuuint64_t str[2] = {rb, rb * d.n};
      cuuint32_t box[3] = {cuuint32_t(kRawK * LO / 8), cuuint32_t(kTN), 1};
      if (!make_map(&w.ml, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d.low, dims, str, box, plane_swizzle(16 * LO))) return kRuntimeError;
    }
    if constexpr (HI != 0) {
      cuuint64_t const rb = cuuint64_t(d.k) * HI / 8;
      cuuint64_t dims[3] = {rb, cuuint64_t(d.n), cuuint64_t(E)};
      cuuint64_t str[2] = {rb, rb * d.n};
      cuuint32_t box[3] = {cuuint32_t(kRawK * HI / 8), cuuint32_t(kTN), 1};
      if (!make_map(&w.mh, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d.high, dims, str, box, plane_swizzle(16 * HI))) return kRuntimeError;
    } else {
      w.mh = w.ml;
    }
    {
      cuuint64_t const kg = cuuint64_t(d.k / gs);
      cuuint64_t dims[3] = {cuuint64_t(d.n), kg, cuuint64_t(E)};
      cuuint64_t str[2] = {cuuint64_t(d.n) * 2, cuuint64_t(d.n) * 2 * kg};
      cuuint32_t box[3] = {cuuint32_t(kTN), cuuint32_t(srows), 1};
      if (!make_map(&w.ms, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, d.scale, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return kRuntimeError;
      if (d.zero) {
        if (!make_map(&w.mz, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, d.zero, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return kRuntimeError;
      } else {
        w.mz = w.ms;
      }
    }
    if (cache.size() >= 8192) cache.clear();                  // bounded: far more artifacts than a model has
    it = cache.emplace(key, w).first;
  }
  ml = it->second.ml; mh = it->second.mh; ms = it->second.ms; mz = it->second.mz;
  return 0;
}

template <int LO, int HI, bool BF16, int MT, int NT, int DEPTH = 0>
int launch_mixed_gemm(GemmDesc const& d, cudaStream_t stream) {
  int const E = d.experts > 0 ? d.experts : 1;
  int const gs = d.group_size;
  CUtensorMap ma, ml, mh, ms, mz;
  {
    cuuint64_t dims[2] = {cuuint64_t(d.k), cuuint64_t(d.total_rows)};
    cuuint64_t str[1] = {cuuint64_t(d.k) * 2};
    cuuint32_t box[2] = {cuuint32_t(kTK), cuuint32_t(kTM * MT)};
    if (!make_map(&ma, BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, d.act, dims, str, box,
                  CU_TENSOR_MAP_SWIZZLE_128B)) return kRuntimeError;
  }
  if (int const rc = weight_maps<LO, HI>(d, E, ml, mh, ms, mz)) return rc;
  GemmArgs g{};
  g.offsets = d.experts > 0 ? d.offsets : nullptr;
  g.out = d.out; g.m_rows = d.total_rows; g.n = d.n; g.k = d.k; g.experts = E; g.group_size = gs;
  g.code_offset = d.code_offset; g.has_zero = d.zero ? 1 : 0;
  int const splits = d.splits > 1 ? d.splits : 1;
  if (splits > d.k / kRawK || splits > 64 || (splits > 1 && !d.partial)) return 30;    // every slice owns at least one piece
  g.splits = splits; g.partial = d.partial;
  g.out_rows = d.out_rows;
  if (d.out_rows && splits > 1) return 30;                     // the reduce kernel writes the dense layout only
  g.status = rt_device_status_ptr();
  if (!g.status) return kRuntimeError;
  auto kern = mixed_gemm_kernel<LO, HI, BF16, MT, NT, DEPTH>;
  size_t const smem = sizeof(GemmSmem<LO, HI, MT, NT, DEPTH>) + 1024;
  static_assert(sizeof(GemmSmem<LO, HI, MT, NT, DEPTH>) + 1024 <= 232448, "shared memory of one CTA");
  static_assert(DEPTH != 1 || sizeof(GemmSmem<LO, HI, MT, NT, DEPTH>) + 1024 <= 113 * 1024, "two CTAs of the shallow form share an SM");
  constexpr bool PAIR = DEPTH == 2;
  if (PAIR && (d.n % (kTN * NT) != 0 || splits > 1)) return 30;  // the pair form covers whole 256-column tiles, one K slice
  {  // the opt-in to large dynamic shared memory is a per-device attribute of the function
    static std::mutex mu;
    static bool attr_set[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { (void)cudaGetLastError(); return kRuntimeError; }
    std::lock_guard<std::mutex> lock(mu);
    if (!attr_set[dev]) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
        (void)cudaGetLastError();
        return kRuntimeError;
      }
      attr_set[dev] = true;
    }
  }
  // row tiles: sum over experts of ceil(rows_e / tile) <= floor(total / tile) + the experts that hold rows
  int const tile_rows = kTM * MT * (PAIR ? 2 : 1);
  int const mtiles = d.experts > 0 ? d.total_rows / tile_rows + std::min(d.experts, d.total_rows)
                                   : (d.total_rows + tile_rows - 1) / tile_rows;
  if (mtiles > 65535) return 30;
  if constexpr (PAIR) {                                        // clusters of two CTAs (neighbours along grid x; they split a tile's rows)
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * ((d.n + kTN * NT - 1) / (kTN * NT)), mtiles, 1);
    cfg.blockDim = dim3(128 + 128 * MT * gemm_dq<MT, NT, DEPTH>());
    cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    cudaError_t const le = cudaLaunchKernelEx(&cfg, kern, ma, ml, mh, ms, mz, g);
    if (le != cudaSuccess) {
      int ncl = -1;
      cudaError_t const oe = cudaOccupancyMaxActiveClusters(&ncl, kern, &cfg);
      std::fprintf(stderr, "[quactlize_b200] pair-form GEMM launch failed: %s (grid %u x %u, block %u, smem %zu, active clusters %d / %s)\n",
                   cudaGetErrorString(le), cfg.gridDim.x, cfg.gridDim.y, cfg.blockDim.x, smem, ncl, cudaGetErrorString(oe));
      (void)cudaGetLastError();
      return kRuntimeError;
    }
    return 0;
  }
  kern<<<dim3((d.n + kTN * NT - 1) / (kTN * NT), mtiles, splits), 128 + 128 * MT * gemm_dq<MT, NT, DEPTH>(), smem, stream>>>(ma, ml, mh, ms, mz, g);
  if (splits > 1) {
    int64_t const elems = int64_t(d.total_rows) * d.n;         // n % 128 == 0: whole float4 groups
    splitk_reduce_kernel<BF16><<<unsigned((elems / 4 + 255) / 256), 256, 0, stream>>>(d.partial, d.out, elems, splits);
  }
  return 0;
}

std::atomic<long long> g_swap_launches{0};

// The swapped form (int4 planes, one K slice): see mixed_gemm_swap_kernel.
template <bool BF16>
int launch_mixed_gemm_swap(GemmDesc const& d, cudaStream_t stream) {
  int const E = d.experts > 0 ? d.experts : 1;
  CUtensorMap mx, ml, mh, ms, mz;
  {
    cuuint64_t dims[2] = {cuuint64_t(d.k), cuuint64_t(d.total_rows)};
    cuuint64_t str[1] = {cuuint64_t(d.k) * 2};
    cuuint32_t box[2] = {cuuint32_t(kTK), cuuint32_t(kSwapTokens)};
    if (!make_map(&mx, BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, d.act, dims, str, box,
                  CU_TENSOR_MAP_SWIZZLE_128B)) return kRuntimeError;
  }
  if (int const rc = weight_maps<4, 0>(d, E, ml, mh, ms, mz)) return rc;
  GemmArgs g{};
  g.offsets = d.experts > 0 ? d.offsets : nullptr;
  g.out = d.out; g.m_rows = d.total_rows; g.n = d.n; g.k = d.k; g.experts = E; g.group_size = d.group_size;
  g.code_offset = d.code_offset; g.has_zero = d.zero ? 1 : 0;
  g.splits = 1; g.partial = nullptr; g.out_rows = d.out_rows;
  g.status = rt_device_status_ptr();
  if (!g.status) return kRuntimeError;
  auto kern = mixed_gemm_swap_kernel<BF16>;
  size_t const smem = sizeof(SwapSmem) + 1024;
  static_assert(sizeof(SwapSmem) + 1024 <= 232448, "shared memory of one CTA");
  {
    static std::mutex mu;
    static bool attr_set[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { (void)cudaGetLastError(); return kRuntimeError; }
    std::lock_guard<std::mutex> lock(mu);
    if (!attr_set[dev]) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
        (void)cudaGetLastError();
        return kRuntimeError;
      }
      attr_set[dev] = true;
    }
  }
  int const mtiles = d.experts > 0 ? d.total_rows / kSwapTokens + std::min(d.experts, d.total_rows)
                                   : (d.total_rows + kSwapTokens - 1) / kSwapTokens;
  if (mtiles > 65535) return 30;
  kern<<<dim3(d.n / (2 * kTN), mtiles, 1), 384, smem, stream>>>(mx, ml, ms, mz, g);
  g_swap_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

}  // namespace

bool tma_make_map(CUtensorMap* m, CUtensorMapDataType dt, int rank, void const* base, cuuint64_t const* dims,
                  cuuint64_t const* strides_bytes, cuuint32_t const* box, CUtensorMapSwizzle sw) {
  return make_map(m, dt, rank, base, dims, strides_bytes, box, sw);
}

long long gemm_swap_launches() { return g_swap_launches.load(std::memory_order_relaxed); }

int enqueue_mixed_gemm(GemmDesc const& d, cudaStream_t stream) {
  if (!d.act || !d.low || !d.scale || (!d.out && !d.out_rows) || d.total_rows <= 0 || d.n <= 0 || d.n % kTN || d.k <= 0 || d.k % 256 ||
      d.group_size < 16 || (d.group_size & (d.group_size - 1)) || d.k % d.group_size || (d.hi_bits && !d.high) ||
      (d.experts > 0 && !d.offsets)) return 30;
  auto al = [](void const* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (!al(d.act) || !al(d.low) || !al(d.scale) || (d.out && !al(d.out)) || (d.zero && !al(d.zero)) || (d.hi_bits && !al(d.high))) return 30;
  int const key = d.lo_bits * 10 + d.hi_bits;
  // 256 x 256 CTA tiles (four accumulators = all 512 TMEM columns) for prefill-sized problems; small ones keep 128 x 128
  int const avg_rows = d.experts > 0 ? d.total_rows / d.experts : d.total_rows;
  bool const big = d.tile == 256 || d.tile == 512 || d.tile == 1024 || (d.tile == 0 && avg_rows >= 192);
  if (d.shallow && !big) {                        // decode tactic: 128 x 128 tiles, two-deep rings, several CTAs per SM
#define QB_GEMM_SHALLOW(K, L, H) case K: return d.act_bf16 ? launch_mixed_gemm<L, H, true, 1, 1, 1>(d, stream) : launch_mixed_gemm<L, H, false, 1, 1, 1>(d, stream);
    switch (key) {
      QB_GEMM_SHALLOW(40, 4, 0) QB_GEMM_SHALLOW(41, 4, 1) QB_GEMM_SHALLOW(42, 4, 2) QB_GEMM_SHALLOW(20, 2, 0) QB_GEMM_SHALLOW(21, 2, 1)
      QB_GEMM_SHALLOW(10, 1, 0)
      default: return 33;
    }
#undef QB_GEMM_SHALLOW
  }
  // The pair form (512 x 256 tile over a cluster of two CTAs, tcgen05 cta_group::2; each CTA converts half of the weight
  // columns): int4 planes, whole 256-column tiles, one K slice.  Opt-in (QUACTLIZE_B200_GEMM_PAIR in the environment, read
  // per call): measured on par with the single-CTA tile on dense problems (64 us both at M = 2048, N = K = 4096) and 9-12 %
  // behind it on the ragged MoE problems, whose experts pad to 512 rows instead of 256.  Halving the conversion did not
  // raise the tensor pipe's duty (47 % against 45 %): each SM still serves the operand reads of both tensor cores.
  // The swapped form (weights as the A operand, converted into tensor memory): int4 planes, whole 256-row weight tiles,
  // one K slice.  Opt-in (QUACTLIZE_B200_GEMM_SWAP in the environment, read per call, or tile = 1024): it is slower than
  // the tiles below on the problems measured (see mixed_gemm_swap_kernel).
  char const* const swap_env = std::getenv("QUACTLIZE_B200_GEMM_SWAP");   // set: prefill-sized problems; "all": every size
  bool const swap_on = swap_env != nullptr && (big || swap_env[0] == 'a');
  if (key == 40 && d.splits <= 1 && !d.shallow && d.n % (2 * kTN) == 0 && (d.tile == 1024 || (d.tile == 0 && swap_on)))
    return d.act_bf16 ? launch_mixed_gemm_swap<true>(d, stream) : launch_mixed_gemm_swap<false>(d, stream);
  bool const pair_on = std::getenv("QUACTLIZE_B200_GEMM_PAIR") != nullptr;
  if (big && key == 40 && d.n % 256 == 0 && d.splits <= 1 && (d.tile == 512 || (d.tile == 0 && pair_on)))
    return d.act_bf16 ? launch_mixed_gemm<4, 0, true, 2, 2, 2>(d, stream) : launch_mixed_gemm<4, 0, false, 2, 2, 2>(d, stream);
#define QB_GEMM_CASE(K, L, H) case K: return d.act_bf16 ? (big ? launch_mixed_gemm<L, H, true, 2, 2>(d, stream) : launch_mixed_gemm<L, H, true, 1, 1>(d, stream)) \
                                                        : (big ? launch_mixed_gemm<L, H, false, 2, 2>(d, stream) : launch_mixed_gemm<L, H, false, 1, 1>(d, stream));
  switch (key) {
    QB_GEMM_CASE(40, 4, 0) QB_GEMM_CASE(41, 4, 1) QB_GEMM_CASE(42, 4, 2) QB_GEMM_CASE(20, 2, 0) QB_GEMM_CASE(21, 2, 1)
    QB_GEMM_CASE(10, 1, 0)
    default: return 33;
  }
#undef QB_GEMM_CASE
}

}  // namespace qb

namespace qb {
int splitk_auto(int row_tiles, int n, int k) {
  int const tiles = std::max(1, row_tiles) * ((n + kTN - 1) / kTN);
  int const want = 2 * rt_sm_count();                      // two shallow CTAs per SM
  int s = (want + tiles - 1) / tiles;
  s = std::min(s, std::min(8, k / kRawK / 2));             // a slice keeps at least two 128-k pieces
  return std::max(1, s);
}
}  // namespace qb
