// Decode GEMV over the bit-plane artifacts, "row-thread" form: every lane owns (one weight row, one quarter of a
// 256-code K slice), so the scale channel -- fp16 planes [E][k/gs][n] or packed units [E][k/256/P][n][bytes], both with
// n innermost -- is read with consecutive lanes on consecutive columns, and nothing is reduced across lanes until the
// very end.  Same math as the segment-per-warp kernel in qb_gemv_planes.cu:
//
//   out[t, r] = sum_k a[t, k] * ( (u[r,k] + off) * s[r, k/gs] + z[r, k/gs] ),   u = lo + 2^LO * hi
//
// Replaces the reference kernels gemv_kernel (quactlize/include/gemv_lowbit/gemv_kernel.hpp:44-246) and
// bc_vecdot::rows_kernel (quactlize/include/gguf_bc_vecdot.hpp:152-227); the reference names the scale loads, not
// the weight stream, as what limits its kernel (gemv_kernel.hpp:147-161) -- this layout is the answer to that.
//
// Work decomposition.  A tile is 8 rows x 256 codes of a plane: a tiled TMA copy with the swizzle matching its row
// length (128 / 64 / 32 bytes), so the 8 x 4 lanes of a warp read it without bank conflicts.  A CTA of 16 warps owns a
// set of 8-row blocks; the tiles of those blocks, listed block by block, are cut into 16 equal contiguous runs, one
// per warp, each streamed through the warp's own ring of mbarrier-tracked stages.  A run may begin and end inside a
// block, so a warp leaves one partial sum per block it touched in shared memory; after the only CTA barrier the
// contributions of each block are added in warp order, so results do not depend on timing.
//
// Activations: the CTA turns its activation row once into "pattern order" in shared memory -- for each plane word the
// half2 operands that the mask-only code extraction needs ((w & mask) read as fp16 IS code * 2^shift * 2^-24; the
// power-of-two activation pre-scale and the shift are folded into the operand) -- plus the sums of x over every
// 16/32/64-code run for the zero / code-offset terms.  Lanes fetch these with 128-bit broadcast loads.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <type_traits>

#include "qb_device.cuh"
#include "qb_gemv_prologue.cuh"
#include "qb_internal.hpp"
#include "qb_kquant.cuh"
#include "qb_runtime.hpp"
#include "qb_tma.hpp"

namespace qb {

namespace {

constexpr int kRows = 8;             // rows of a tile
constexpr int kSlice = 256;          // codes of a tile along K
constexpr int kPart = 64;            // codes one lane converts per tile (4 lanes per row)
constexpr int kPartStride = 144;     // bytes between the pattern runs of consecutive parts: 128 + 16 keeps the four
                                     // parts a warp reads at once on different banks

struct RtArgs {
  PlaneGemvDesc d;
  int ns, nblocks;                   // K slices per block, row blocks
  unsigned int* status;
};

__device__ __forceinline__ void tma_tile_3d(void* dst, CUtensorMap const* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

__device__ __forceinline__ float act_at(void const* base, size_t i, int bf16) {
  uint16_t const h = __ldg(reinterpret_cast<uint16_t const*>(base) + i);
  return bf16 ? __uint_as_float(uint32_t(h) << 16) : __half2float(__ushort_as_half(h));
}

// shared-memory accesses by 32-bit shared-space address (keeps the address arithmetic in 32 bits)
__device__ __forceinline__ uint4 lds128_a(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
// bytes one ring stage keeps for a tile's scale channel: fp16 scale and zero of 8 rows x up to 4 * NQ groups (two halves),
// or the packed units of 8 rows
template <int MODE, int QT, int NQ, int WR>
constexpr int sc_tile_bytes() {
  if constexpr (MODE == 0) return NQ * WR <= 2 ? 256 : NQ * WR * 128;   // each half starts 128-byte aligned, as a tiled copy's destination must
  else return kRows * WR * kq::Unit<QT>::kUnitTotal;             // an untiled bulk copy needs 16-byte alignment only
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

// one 32-bit plane word of B-bit codes against its NP = 16/B pattern operands
template <int B>
__device__ __forceinline__ __half2 rt_acc_word(uint32_t w, __half2 const* xs, __half2 acc) {
  constexpr int PER = 8 / B;
  constexpr uint32_t M1 = ((1u << B) - 1u) * 0x00010001u;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t const ws = h ? (w >> 8) : w;
#pragma unroll
    for (int o = 0; o < PER; ++o) acc = __hfma2(u32_as_h2(ws & (M1 << (o * B))), xs[h * PER + o], acc);
  }
  return acc;
}

// this lane's 64 codes of plane row `r`, part `kp`, out of a swizzled tile whose rows are 32*B bytes
// byte offset(s) of this lane's codes inside a tile: fixed per lane, computed once
// (RB = bytes of a tile row: 128, 64 or 32; a lane's quarter of it is 32, 16 or 8 bytes)
template <int RB>
__device__ __forceinline__ void part_offsets(int r, int kp, uint32_t* off) {
  if constexpr (RB == 128) { off[0] = r * 128 + (((2 * kp) ^ r) << 4); off[1] = r * 128 + (((2 * kp + 1) ^ r) << 4); }
  else if constexpr (RB == 64) { off[0] = r * 64 + ((kp ^ ((r >> 1) & 3)) << 4); off[1] = 0; }
  else { off[0] = r * 32 + ((((kp >> 1) ^ ((r >> 2) & 1))) << 4) + (kp & 1) * 8; off[1] = 0; }
}
template <int RB>
__device__ __forceinline__ void load_part(uint32_t tile, uint32_t const* off, uint32_t* w) {
  if constexpr (RB == 128) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      uint4 const v = lds128_a(tile + off[j]);
      w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
    }
  } else if constexpr (RB == 64) {
    uint4 const v = lds128_a(tile + off[0]);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
  } else {
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(tile + off[0]));
  }
}

// 32 bits starting at bit `bit` of a little-endian bit string held in words u[0..N-1]
template <int N>
__device__ __forceinline__ uint32_t bits_at(uint32_t const* u, int bit) {
  int const wi = bit >> 5;
  uint32_t lo = u[0], hi = N > 1 ? u[1] : 0u;
#pragma unroll
  for (int i = 1; i < N; ++i) {
    if (wi == i) { lo = u[i]; hi = i + 1 < N ? u[i + 1] : 0u; }
  }
  return __funnelshift_r(lo, hi, bit & 31);
}

// LO/HI plane bits; MODE 0 fp16 scale(+zero) planes with NQ = 64/min(gs,64) runs per part, MODE 1 packed units of QT
// MR activation rows share every weight tile (1, or up to 4 rows of one expert)
// SL: 256-code slices per tile (1; 2 or 4 for a lone 2- or 1-bit plane, whose tile then is 1 KB like the 4-bit one and the
// per-tile bookkeeping is paid per 512 / 1024 codes); NQ counts the runs of one lane's 64*SL codes
// WR: weight rows per lane (1, or 2: tile rows r and r + 8 of a 16-row tile share the lane's activation operands and every
// per-tile step -- wait, copy issue, scale addressing -- is paid once per two rows)
template <int LO, int HI, int MODE, int QT, int NQ, int STAGES, int MR, int SL, int WR>
__global__ void __launch_bounds__(512, 1)
rowthread_gemv_kernel(const __grid_constant__ CUtensorMap map_lo, const __grid_constant__ CUtensorMap map_hi,
                      const __grid_constant__ CUtensorMap map_sc, const __grid_constant__ CUtensorMap map_zr, RtArgs a) {
  static_assert(SL == 1 || (MODE == 0 && HI == 0 && LO * SL <= 4), "wide tiles are for a lone low plane");
  constexpr int KS = kSlice * SL, KP = kPart * SL, KPS = KP * 2 + 16;   // codes per tile, per lane, bytes between pattern runs
  constexpr int Q = KP / NQ;                          // codes per run: one scale group (or 64 codes of a wider one)
  constexpr int NWL = KP * LO / 32;                   // low-plane words per part: 8 / 4 / 2
  constexpr int NWH = HI ? KP * HI / 32 : 1;          // high-plane words per part: 4 / 2
  constexpr int CWL = 32 / LO, CWH = HI ? 32 / HI : 32;
  constexpr int NPL = 16 / LO, NPH = HI ? 16 / HI : 1;
  constexpr int U = Q < 32 ? Q : 32;                  // codes per fp16 accumulation run (then fp32)
  constexpr int NU = KP / U;
  constexpr int RBL = 32 * LO * SL, RBH = HI ? 32 * HI : 32;           // bytes of a tile row
  constexpr int TR = kRows * WR;                                       // rows of a tile
  constexpr int LO_TILE = TR * RBL, HI_TILE = HI ? TR * RBH : 0;
  constexpr int SC_TILE = sc_tile_bytes<MODE, QT, NQ, WR>(), SC_HALF = SC_TILE / 2;   // scale channel of one tile, copied with it
  static_assert(CWL <= U, "a low-plane word must not straddle accumulation runs");
  constexpr bool kCrossHi = HI && CWH > U;            // a high word spans two runs (1-bit plane, 16-code groups)
  static_assert(!kCrossHi || CWH == 2 * U, "a high-plane word may span at most two runs");

  PlaneGemvDesc const& d = a.d;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  // the warp index is broadcast from lane 0: the compiler then keeps what derives from it (tile counts, ring and barrier
  // addresses, copy coordinates) in uniform registers and the per-tile bookkeeping off the vector pipes
  int const warp = __shfl_sync(0xffffffffu, int(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  int const kp = lane >> 3, r = lane & 7;

  // ---- which activation rows / expert ---------------------------------------------------------------------------------
  // grid.y is a group of up to MR activation rows of one expert.  MR == 1: the row itself, whose expert a ragged launch
  // looks up in the cumulative offsets (one probe per thread).  MR > 1, ragged: group y of the list "ceil(rows_e / MR)
  // groups per expert, in expert order", located by a block-wide scan of the per-expert group counts.
  int e = 0, arow = 0, nrows = 1;
  // Under programmatic dependent launch the activations (and a router's offsets) may be the preceding kernel's output:
  // nothing of them is read before this wait.  Without the launch attribute it returns at once.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // The first activation row is requested at once where its index does not depend on the expert look-up (always, except
  // for ragged groups of several rows): the look-up's own global loads then overlap it.
  constexpr int kPre = 4;                                   // 16-byte pieces per thread held in registers: K <= 16384 is covered
  uint4 pre[kPre];
  bool const early_x = MR == 1 || d.offsets == nullptr;
  if (early_x) {
    uint16_t const* x0 = reinterpret_cast<uint16_t const*>(d.act) + size_t(blockIdx.y) * MR * d.k;
    bool const have = d.offsets != nullptr || int(blockIdx.y) * MR < d.m_rows;
#pragma unroll
    for (int j = 0; j < kPre; ++j) {
      int const i = (int(threadIdx.x) + j * 512) * 8;
      pre[j] = (have && i < d.k) ? __ldg(reinterpret_cast<uint4 const*>(x0 + i)) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
  if (d.offsets) {
    volatile int* sh = reinterpret_cast<volatile int*>(smem);            // ring space, not yet in use
    if (threadIdx.x < 4) sh[threadIdx.x] = -1;
    __syncthreads();
    if constexpr (MR == 1) {
      arow = blockIdx.y;
      for (int t = threadIdx.x; t < d.experts; t += blockDim.x)
        if (arow >= d.offsets[t] && arow < d.offsets[t + 1]) sh[0] = t;
      __syncthreads();
      e = sh[0];
    } else {
      volatile int* cnt = sh + 8;                                          // [experts] inclusive scan of group counts
      for (int t = threadIdx.x; t < d.experts; t += blockDim.x) cnt[t] = (d.offsets[t + 1] - d.offsets[t] + MR - 1) / MR;
      __syncthreads();
      if (warp == 0) {                                                     // inclusive scan, 32 experts per step
        int carry = 0;
        for (int base = 0; base < d.experts; base += 32) {
          int v = base + lane < d.experts ? cnt[base + lane] : 0;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) { int const u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
          v += carry;
          if (base + lane < d.experts) cnt[base + lane] = v;
          carry = __shfl_sync(0xffffffffu, v, 31);
        }
      }
      __syncthreads();
      for (int t = threadIdx.x; t < d.experts; t += blockDim.x) {
        int const hi = cnt[t], lo = t ? cnt[t - 1] : 0;
        if (int(blockIdx.y) >= lo && int(blockIdx.y) < hi) { sh[0] = t; sh[1] = int(blockIdx.y) - lo; }
      }
      __syncthreads();
      e = sh[0];
      if (e >= 0) {
        int const r0 = d.offsets[e], r1 = d.offsets[e + 1];
        arow = r0 + sh[1] * MR;
        nrows = min(MR, r1 - arow);
      }
    }
    __syncthreads();                                  // everyone has read the scratch before the first copy may land there
    if (e < 0) return;                                // uniform for the CTA: a group beyond the last expert
  } else {
    arow = blockIdx.y * MR;
    nrows = min(MR, d.m_rows - arow);
    if (nrows <= 0) return;
  }
  e = __shfl_sync(0xffffffffu, e, 0);                 // uniform for the compiler too (it was read from shared memory)
  int const k = d.k, n = d.n;

  // ---- shared memory carve-up -----------------------------------------------------------------------------------------
  constexpr int W = 16;
  int const nparts = k / KP;
  uint8_t* lo_ring = smem;                                              // [W][STAGES][LO_TILE]
  uint8_t* hi_ring = lo_ring + size_t(W) * STAGES * LO_TILE;             // [W][STAGES][HI_TILE]
  uint32_t const xrow = uint32_t(nparts) * KPS;                  // bytes of one activation row in pattern order
  uint8_t* sc_ring = hi_ring + size_t(W) * STAGES * HI_TILE;             // [W][STAGES][SC_TILE]
  uint8_t* xlo = sc_ring + size_t(W) * STAGES * SC_TILE;                 // [MR][nparts][kPartStride]
  uint8_t* xhi = xlo + size_t(MR) * xrow;                                // same, if HI
  float* sxq = reinterpret_cast<float*>(xhi + (HI ? size_t(MR) * xrow : 0));   // [MR][k/Q]
  uint16_t* xraw = reinterpret_cast<uint16_t*>(sxq + MR * (k / Q));      // [k] raw activations (prologue only, one row at a time)
  float* red = reinterpret_cast<float*>(xraw + k);                       // [16]
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 16);                // [W][STAGES]
  float* part = reinterpret_cast<float*>(bars + W * STAGES);             // [blocks of this CTA + 16][MR][TR]
  (void)xhi;

  // ---- this warp's share of the work ------------------------------------------------------------------------------------
  // The CTA owns blocks blockIdx.x, blockIdx.x + gridDim.x, ...; their tiles, listed block by block, are cut into 16
  // equal runs, one per warp, so a warp's run may start and end inside a block.
  int const ns = a.ns;
  int const nb_c = blockIdx.x < a.nblocks ? (a.nblocks - 1 - blockIdx.x) / gridDim.x + 1 : 0;   // blocks of this CTA
  int const T = nb_c * ns;
  int const t0 = ((warp * T) >> 4), t1 = (((warp + 1) * T) >> 4);
  int const ntiles = t1 - t0;
  uint64_t* mybars = bars + warp * STAGES;
  uint8_t* mylo = lo_ring + size_t(warp) * STAGES * LO_TILE;
  uint8_t* myhi = hi_ring + size_t(warp) * STAGES * HI_TILE;
  uint8_t* mysc = sc_ring + size_t(warp) * STAGES * SC_TILE;

  static_assert((STAGES & (STAGES - 1)) == 0, "ring depth is a power of two");
  int const b_first = ntiles > 0 ? t0 / ns : 0, s_first = ntiles > 0 ? t0 % ns : 0;
  // next tile to request (lane 0 only): everything the copy needs is kept in registers and advanced by additions
  int is_s = s_first;
  int is_row0 = (blockIdx.x + b_first * gridDim.x) * TR;
  int const row_step = gridDim.x * TR;
  uint32_t const bar_a = smem_u32(mybars), ring_lo_a = smem_u32(mylo), ring_hi_a = smem_u32(myhi), ring_sc_a = smem_u32(mysc);
  uint64_t const map_lo_p = reinterpret_cast<uint64_t>(&map_lo), map_hi_p = reinterpret_cast<uint64_t>(&map_hi);
  uint64_t const map_sc_p = reinterpret_cast<uint64_t>(&map_sc), map_zr_p = reinterpret_cast<uint64_t>(&map_zr);
  // The scale channel of a tile travels with it, on the same mbarrier: the scale (and zero) values of the tile's 8 rows
  // and its 256/gs groups as one box of each fp16 plane, or the 8 rows' packed units as one contiguous bulk copy.  (A
  // per-lane global load of the scales, even one tile ahead, cost 40% of the kernel's time: it queues behind the ring.)
  int const gs = d.group_size;
  int const gshift = 31 - __clz(gs > 0 ? gs : 1);           // group size is a power of two
  bool const has_zero = MODE == 0 && d.zero != nullptr;
  using UnitT = kq::Unit<(MODE == 1 ? QT : 12)>;
  int const sc_groups = MODE == 0 ? max(1, KS >> gshift) : 0;
  uint32_t const tx_bytes = LO_TILE + HI_TILE + (MODE == 0 ? uint32_t(sc_groups) * uint32_t(TR * 2) * (has_zero ? 2u : 1u) : uint32_t(TR * UnitT::kUnitTotal));
  uint8_t const* const un_e = MODE == 1 ? d.units + size_t(e) * ((k / 256) / UnitT::kSbPerUnit) * n * UnitT::kUnitTotal : nullptr;
  // called with q = 0, 1, 2, ... in order; every lane keeps the (uniform) bookkeeping, lane 0 issues the copies
  auto issue = [&](int q) {
    uint32_t const st = uint32_t(q) & (STAGES - 1), bar = bar_a + st * 8;
    int const gy = MODE == 0 ? (is_s * KS) >> gshift : 0;
    if (lane == 0) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(tx_bytes) : "memory");
      if constexpr (MODE == 0) {
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                     ::"r"(ring_sc_a + st * SC_TILE), "l"(map_sc_p), "r"(bar), "r"(is_row0), "r"(gy), "r"(e) : "memory");
        if (has_zero)
          asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                       ::"r"(ring_sc_a + st * SC_TILE + SC_HALF), "l"(map_zr_p), "r"(bar), "r"(is_row0), "r"(gy), "r"(e) : "memory");
      } else {
        uint8_t const* src = un_e + (size_t(is_s / UnitT::kSbPerUnit) * n + is_row0) * UnitT::kUnitTotal;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(ring_sc_a + st * SC_TILE), "l"(src), "n"(TR * UnitT::kUnitTotal), "r"(bar) : "memory");
      }
      asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                   ::"r"(ring_lo_a + st * LO_TILE), "l"(map_lo_p), "r"(bar), "r"(is_s * (KS * LO / 8)), "r"(is_row0), "r"(e) : "memory");
      if constexpr (HI != 0)
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                     ::"r"(ring_hi_a + st * HI_TILE), "l"(map_hi_p), "r"(bar), "r"(is_s * (KS * HI / 8)), "r"(is_row0), "r"(e) : "memory");
    }
    if (++is_s == ns) { is_s = 0; is_row0 += row_step; }
  };
  // Activation rows are requested BEFORE the weight stream: a load issued after it queues behind the ring's copies
  // (128 KB per SM) and costs a microsecond per row.  Row m + 1 is loaded into registers while row m is converted, and
  // the stream starts as soon as the last row's loads are in flight.
  auto load_row = [&](int m) {
    uint16_t const* x0 = reinterpret_cast<uint16_t const*>(d.act) + size_t(arow + m) * k;
#pragma unroll
    for (int j = 0; j < kPre; ++j) {
      if (j * 4096 >= k) break;                            // uniform: no thread has a piece j
      int const i = (int(threadIdx.x) + j * 512) * 8;
      pre[j] = i < k ? __ldg(reinterpret_cast<uint4 const*>(x0 + i)) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  if (!early_x) load_row(0);
  if (MODE == 0 && !has_zero) {                             // no copy ever lands in the zero halves: they read as zero
    for (int i = lane; i < STAGES * (SC_HALF / 4); i += 32)
      *reinterpret_cast<uint32_t*>(mysc + (i / (SC_HALF / 4)) * SC_TILE + SC_HALF + (i % (SC_HALF / 4)) * 4) = 0u;
    __syncwarp();
  }
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(&mybars[s], 1);
    mbar_init_fence();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  auto start_stream = [&]() {
    for (int q = 0; q < STAGES && q < ntiles; ++q) issue(q);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  };
  if (nrows == 1) start_stream();
  for (int i = threadIdx.x; i < (nb_c + 16) * MR * TR; i += blockDim.x) part[i] = 0.f;

  // ---- CTA prologue: activations into pattern order, one activation row at a time ---------------------------------------
  float fm[MR];
#pragma unroll
  for (int m = 0; m < MR; ++m) fm[m] = 0.f;
  auto prologue = [&](auto bf16_tag) {
    constexpr bool BF = decltype(bf16_tag)::value;
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      if (m >= nrows) continue;                            // uniform for the CTA
      // pass 1: raw 16-bit activations to shared memory, max |x|, and the sum of x over every Q-code run (lanes hold
      // consecutive 8-element pieces, so a run is Q/8 neighbouring lanes)
      float mx = 0.f;
      uint4 cur[kPre];
#pragma unroll
      for (int j = 0; j < kPre; ++j) cur[j] = pre[j];
      if (m + 1 < nrows) {                                 // uniform for the CTA
        load_row(m + 1);
        if (m + 2 == nrows) start_stream();
      }
      auto piece = [&](int i, uint4 v) {                   // k % 256 == 0: whole warps in or out
        *reinterpret_cast<uint4*>(xraw + i) = v;
        float p;
        piece_stats<BF>(v, mx, p);
#pragma unroll
        for (int o = 1; o < Q / 8; o <<= 1) p += __shfl_xor_sync(0xffffffffu, p, o);
        if ((lane & (Q / 8 - 1)) == 0) sxq[m * (k / Q) + i / Q] = p;
      };
      uint4 const* xg = reinterpret_cast<uint4 const*>(reinterpret_cast<uint16_t const*>(d.act) + size_t(arow + m) * k);
#pragma unroll
      for (int j = 0; j < kPre; ++j) {
        if (j * 4096 >= k) break;                          // uniform
        int const i = (int(threadIdx.x) + j * 512) * 8;
        if (i < k) piece(i, cur[j]);
      }
      for (int i = (int(threadIdx.x) + kPre * 512) * 8; i < k; i += 512 * 8) piece(i, __ldg(xg + i / 8));
      mx = warp_max(mx);
      if (lane == 0) red[warp] = mx;
      __syncthreads();
      mx = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {                            // red is 16-byte aligned
        float4 const v = reinterpret_cast<float4 const*>(red)[i];
        mx = fmaxf(fmaxf(mx, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
      }
      int const ex = pow2_scale_exponent(mx, HI ? 15 - LO : 15);
      fm[m] = ldexpf(1.f, 24 - ex);
      // pass 2: one half2 operand per code pair and mask position, multiplier 2^(ex - shift)
      pattern_row<LO, BF>(xraw, xlo + size_t(m) * xrow, k, ex, KP, KPS);
      if constexpr (HI != 0) pattern_row<(HI ? HI : 1), BF>(xraw, xhi + size_t(m) * xrow, k, ex + LO, KP, KPS);
      __syncthreads();                                     // xraw and red are reused by the next row
    }
  };
  if (d.act_bf16) prologue(std::true_type{});
  else prologue(std::false_type{});

  // ---- where this lane finds its runs' scales inside the staged scale channel (fixed per lane) -----------------------------
  // (weight row w of the lane is tile row r + 8*w: 16 bytes further in a scale row, 8 units further in the packed units)
  uint32_t sc_off[MODE == 0 ? NQ : 1];
  if constexpr (MODE == 0) {
#pragma unroll
    for (int j = 0; j < NQ; ++j) sc_off[j] = uint32_t(gs <= KS ? (kp * KP + j * Q) >> gshift : 0) * uint32_t(TR * 2) + uint32_t(r) * 2u;
  } else {
    sc_off[0] = uint32_t(r) * UnitT::kUnitTotal;
  }
  constexpr int NSC = MODE == 0 ? NQ : 5;
  constexpr uint32_t SC_ROW8 = MODE == 0 ? 16u : 8u * UnitT::kUnitTotal;   // from tile row r to tile row r + 8
  uint32_t const sc_a = smem_u32(mysc);

  float const coff = float(d.code_offset);
  bool dead = false;
  int q = 0;
  float tot[MR][WR];
#pragma unroll
  for (int m = 0; m < MR; ++m)
#pragma unroll
    for (int w = 0; w < WR; ++w) tot[m][w] = 0.f;
  uint32_t offl[2], offh[2];
  part_offsets<RBL>(r, kp, offl);
  part_offsets<RBH>(r, kp, offh);
  uint32_t const lo_a = smem_u32(mylo), hi_a = smem_u32(myhi), xlo_a = smem_u32(xlo), xhi_a = smem_u32(xhi), sxq_a = smem_u32(sxq);
  uint32_t const sx_row = uint32_t(k / Q) * 4;
  // a warp's sums for one block go to slot (block + warp): runs are contiguous and ordered, so slots never collide
  auto flush = [&](int bi) {
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
      for (int w = 0; w < WR; ++w) {
        float v = tot[m][w];
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        if (lane < kRows) part[((bi + warp) * MR + m) * TR + 8 * w + lane] = v;
        tot[m][w] = 0.f;
      }
  };
  for (int bi = b_first, s_begin = s_first; q < ntiles; ++bi, s_begin = 0) {
   int const s_end = min(ns, s_begin + (ntiles - q));
   for (int s = s_begin; s < s_end; ++s, ++q) {
    uint32_t const st = uint32_t(q) & (STAGES - 1);
    if (!mbar_wait_bounded(&mybars[st], unsigned(q / STAGES) & 1u, a.status, kWaitStageTimeout)) { dead = true; break; }
    int const pt = s * (KS / KP) + kp;
    uint32_t wl[WR][NWL], wh[WR][NWH];
    uint32_t cur[WR][NSC];                                   // MODE 0: scale | zero << 16 per run; MODE 1: the superblock's scale bytes
#pragma unroll
    for (int w = 0; w < WR; ++w) {
      load_part<RBL>(lo_a + st * LO_TILE + w * (8 * RBL), offl, wl[w]);      // the swizzle pattern repeats every 8 rows
      if constexpr (HI != 0) load_part<RBH>(hi_a + st * HI_TILE + w * (8 * RBH), offh, wh[w]);
      if constexpr (MODE == 0) {
#pragma unroll
        for (int j = 0; j < NQ; ++j) {
          uint32_t const at = sc_a + st * SC_TILE + sc_off[j] + w * SC_ROW8;
          cur[w][j] = lds_u16(at) | (lds_u16(at + SC_HALF) << 16);   // the zero half holds zeros when there is no zero plane
        }
      } else {
        uint32_t const at = sc_a + st * SC_TILE + sc_off[0] + w * SC_ROW8 + uint32_t(s % UnitT::kSbPerUnit) * UnitT::kSbBytes;
#pragma unroll
        for (int i = 0; i < NSC; ++i) cur[w][i] = 0u;
#pragma unroll
        for (int i = 0; i < (UnitT::kSbBytes + 3) / 4; ++i) {
          uint32_t const lo16 = lds_u16(at + 4 * i);
          uint32_t const hi16 = (4 * i + 2 < UnitT::kSbBytes) ? lds_u16(at + 4 * i + 2) : 0u;
          cur[w][i] = lo16 | (hi16 << 16);
        }
      }
    }
    // Once the loads above have returned, the slot can be refilled while the rows are multiplied.  The mov reads one word of
    // every load instruction, so it cannot issue before they have completed for the whole warp; the copy is issued after it.
    {
      uint32_t dep = 0u, sink;
#pragma unroll
      for (int w = 0; w < WR; ++w) {
        dep ^= wl[w][0] ^ wl[w][NWL - 1] ^ (HI ? wh[w][0] : 0u);
#pragma unroll
        for (int i = 0; i < (MODE == 0 ? NQ : (UnitT::kSbBytes + 3) / 4); ++i) dep ^= cur[w][i];
      }
      asm volatile("mov.u32 %0, %1;" : "=r"(sink) : "r"(dep) : "memory");
      __syncwarp();
      if (q + STAGES < ntiles) issue(q + STAGES);
    }
    // scale channel of this lane's NQ runs, decoded once for all activation rows: weight = sv * (code + off) + zv
    float sv[WR][NQ], oz[WR][NQ];                            // scale, and (code offset * scale + zero)
#pragma unroll
    for (int w = 0; w < WR; ++w)
#pragma unroll
      for (int j = 0; j < NQ; ++j) {
        if constexpr (MODE == 0) {
          float2 const sz = __half22float2(u32_as_h2(cur[w][j]));
          sv[w][j] = sz.x; oz[w][j] = fmaf(coff, sz.x, sz.y);
        } else {
          using F = kq::Fmt<QT>;
          using UU = kq::Unit<QT>;
          int const grp = kp * NQ + j;                     // group inside the superblock
          float2 const dd = __half22float2(u32_as_h2(cur[w][0]));    // (d, dmin); dmin lane meaningless without a min
          uint32_t const sraw = bits_at<5>(cur[w], UU::bit_of(grp, 0)) & ((1u << F::kScaleBits) - 1u);
          int sc = int(sraw);
          if constexpr (F::kSignedScale) sc = int(int8_t(sraw));
          sc -= F::kScaleBias;
          sv[w][j] = dd.x * float(sc);
          float zz = 0.f;
          if constexpr (F::kHasMin) {
            uint32_t const mraw = bits_at<5>(cur[w], UU::bit_of(grp, 1)) & ((1u << F::kMinBits) - 1u);
            zz = -dd.y * float(mraw);
          }
          oz[w][j] = -float(F::kCodeBias) * sv[w][j] + zz;
        }
      }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      if (MR > 1 && m >= nrows) continue;                // uniform for the CTA
      float usum[WR][NU];
      uint32_t const xp = xlo_a + uint32_t(m) * xrow + uint32_t(pt) * KPS;
      uint32_t const xq = xhi_a + uint32_t(m) * xrow + uint32_t(pt) * KPS;
      (void)xq;
#pragma unroll
      for (int u = 0; u < NU; ++u) {
        // two independent fp16 chains per run and weight row (even and odd words) when the run has several words: half the
        // dependent latency, half the products per fp16 accumulator.  The operands of a word are loaded once for both rows.
        constexpr int WPR = U / CWL;                      // low-plane words per run
        __half2 acc[WR], acc_b[WR];
#pragma unroll
        for (int w = 0; w < WR; ++w) { acc[w] = __float2half2_rn(0.f); acc_b[w] = __float2half2_rn(0.f); }
#pragma unroll
        for (int wi = u * WPR; wi < (u + 1) * WPR; ++wi) {
          __half2 xs[NPL];
#pragma unroll
          for (int v = 0; v < NPL / 4; ++v) {
            uint4 const xv = lds128_a(xp + wi * (NPL * 4) + v * 16);
            xs[4 * v] = u32_as_h2(xv.x); xs[4 * v + 1] = u32_as_h2(xv.y); xs[4 * v + 2] = u32_as_h2(xv.z); xs[4 * v + 3] = u32_as_h2(xv.w);
          }
#pragma unroll
          for (int w = 0; w < WR; ++w) {
            if (WPR > 1 && (wi & 1)) acc_b[w] = rt_acc_word<LO>(wl[w][wi], xs, acc_b[w]);
            else acc[w] = rt_acc_word<LO>(wl[w][wi], xs, acc[w]);
          }
        }
        if constexpr (WPR > 1) {
#pragma unroll
          for (int w = 0; w < WR; ++w) acc[w] = __hadd2(acc[w], acc_b[w]);
        }
        if constexpr (HI != 0 && !kCrossHi) {
#pragma unroll
          for (int wi = u * (U / CWH); wi < (u + 1) * (U / CWH); ++wi) {
            __half2 xs[NPH];
#pragma unroll
            for (int v = 0; v < NPH / 4; ++v) {
              uint4 const xv = lds128_a(xq + wi * (NPH * 4) + v * 16);
              xs[4 * v] = u32_as_h2(xv.x); xs[4 * v + 1] = u32_as_h2(xv.y); xs[4 * v + 2] = u32_as_h2(xv.z); xs[4 * v + 3] = u32_as_h2(xv.w);
            }
#pragma unroll
            for (int w = 0; w < WR; ++w) acc[w] = rt_acc_word<(HI ? HI : 1)>(wh[w][wi], xs, acc[w]);
          }
        }
#pragma unroll
        for (int w = 0; w < WR; ++w) usum[w][u] = h2_sum(acc[w]);
      }
      if constexpr (kCrossHi) {                         // the low half-lane of a high word is run 2w, the high one run 2w+1
#pragma unroll
        for (int wi = 0; wi < NWH; ++wi) {
          __half2 xs[NPH];
#pragma unroll
          for (int v = 0; v < NPH / 4; ++v) {
            uint4 const xv = lds128_a(xq + wi * (NPH * 4) + v * 16);
            xs[4 * v] = u32_as_h2(xv.x); xs[4 * v + 1] = u32_as_h2(xv.y); xs[4 * v + 2] = u32_as_h2(xv.z); xs[4 * v + 3] = u32_as_h2(xv.w);
          }
#pragma unroll
          for (int w = 0; w < WR; ++w) {
            float2 const f = __half22float2(rt_acc_word<(HI ? HI : 1)>(wh[w][wi], xs, __float2half2_rn(0.f)));
            usum[w][2 * wi] += f.x; usum[w][2 * wi + 1] += f.y;
          }
        }
      }
      // runs -> scale groups
#pragma unroll
      for (int j = 0; j < NQ; ++j) {
        float const sx = lds_f32(sxq_a + uint32_t(m) * sx_row + uint32_t(pt * NQ + j) * 4);
#pragma unroll
        for (int w = 0; w < WR; ++w) {
          float gsum = 0.f;
#pragma unroll
          for (int u = j * (NU / NQ); u < (j + 1) * (NU / NQ); ++u) gsum += usum[w][u];
          tot[m][w] = fmaf(sv[w][j] * fm[m], gsum, tot[m][w]);
          tot[m][w] = fmaf(oz[w][j], sx, tot[m][w]);
        }
      }
    }
   }
   if (dead) break;
   flush(bi);
  }
  if (dead)                                               // let copies already in flight land before the CTA's memory is reused
    for (int i = q + 1; i < ntiles && i < q + STAGES; ++i)
      (void)mbar_wait_bounded(&mybars[i % STAGES], unsigned(i / STAGES) & 1u, nullptr, 0, 250000000ull);
  __syncthreads();
  // ---- every block's contributions, added in warp order (fixed: results do not depend on timing) ------------------------------
  for (int o = threadIdx.x; o < nb_c * MR * TR; o += blockDim.x) {
    int const bi = o / (MR * TR), m = (o / TR) % MR, rr = o % TR;
    int const row = (blockIdx.x + bi * gridDim.x) * TR + rr;
    if (row >= n || m >= nrows) continue;
    float sum = 0.f;
    // with many blocks per CTA only the warps whose run can touch block bi are visited (a conservative range; the test
    // below is exact); with one or two blocks the two divisions would cost more than the full loop
    int w_lo = 0, w_hi = 15;
    if (nb_c > 2) { w_lo = max(0, (bi * ns * 16) / T - 1); w_hi = min(15, ((bi + 1) * ns * 16) / T + 1); }
    for (int w2 = w_lo; w2 <= w_hi; ++w2) {
      int const u0 = ((w2 * T) >> 4), u1 = (((w2 + 1) * T) >> 4);
      if (u1 > u0 && u0 < (bi + 1) * ns && u1 > bi * ns) sum += part[((bi + w2) * MR + m) * TR + rr];
    }
    size_t const oi = size_t(arow + m) * n + row;
    if (d.out_kind == 1) reinterpret_cast<float*>(d.out)[oi] = sum;
    else if (d.out_kind == 0) reinterpret_cast<__half*>(d.out)[oi] = __float2half_rn(sum);
    else reinterpret_cast<__nv_bfloat16*>(d.out)[oi] = __float2bfloat16_rn(sum);
  }
}

struct RtPlan { int gx, rc; size_t smem; };
struct RtMaps { CUtensorMap lo, hi, sc, zr; };

template <int LO, int HI, int MODE, int QT, int NQ, int MR, int SL, int WR>
int launch_rowthread_mr(PlaneGemvDesc const& d, cudaStream_t stream) {
  constexpr int STAGES = ((LO + HI >= 5) ? 4 : 8) / WR;   // a power of two; 64-96 KB in flight per SM for the wide tiles
  constexpr int KS = kSlice * SL, KP = kPart * SL, KPS = KP * 2 + 16;
  constexpr int Q = KP / NQ;
  constexpr int TR = kRows * WR;
  constexpr int LO_TILE = TR * 32 * LO * SL, HI_TILE = HI ? TR * 32 * HI : 0;
  constexpr int SC_TILE = sc_tile_bytes<MODE, QT, NQ, WR>();
  auto kern = rowthread_gemv_kernel<LO, HI, MODE, QT, NQ, STAGES, MR, SL, WR>;
  // grid rows: one per group of up to MR activation rows of one expert (ragged: an upper bound, surplus CTAs exit at once)
  int const gy = MR == 1 ? d.m_rows : (d.offsets ? std::min(d.m_rows, d.m_rows / MR + d.experts) : (d.m_rows + MR - 1) / MR);
  if (gy <= 0 || gy > 65535) return 40;
  int const E = d.experts > 0 ? d.experts : 1;
  int dev = 0;
  cudaGetDevice(&dev);
  // ---- launch geometry: cached per (n, k, grid.y, device) ----------------------------------------------------------------
  struct Key { int n, k, gy, dev; bool operator<(Key const& o) const {
    return n != o.n ? n < o.n : k != o.k ? k < o.k : gy != o.gy ? gy < o.gy : dev < o.dev; } };
  static std::map<Key, RtPlan> plans;
  static std::mutex mu;
  RtPlan p{};
  {
    std::lock_guard<std::mutex> lk(mu);
    Key const key{d.n, d.k, gy, dev};
    auto it = plans.find(key);
    if (it == plans.end()) {
      int const nblocks = (d.n + TR - 1) / TR, sms = rt_sm_count();
      int const act_rows = MR == 1 ? gy : std::max(1, (d.m_rows + MR - 1) / MR);    // groups that do work
      int const share = std::max(1, sms / std::max(1, std::min(act_rows, sms)));   // CTAs per activation row: one wave in all
      p.gx = std::max(1, std::min(nblocks, share));
      int per = std::min(512, (nblocks + p.gx - 1) / p.gx);            // blocks per CTA, evened; bounded by the partial-sum table
      p.gx = (nblocks + per - 1) / per;
      int const nparts = d.k / KP;
      p.smem = 1024 + size_t(16) * STAGES * (LO_TILE + HI_TILE + SC_TILE) + size_t(MR) * nparts * KPS * (HI ? 2 : 1) +
               size_t(MR) * (d.k / Q) * 4 + size_t(d.k) * 2 + 16 * 4 + size_t(16) * STAGES * 8 + size_t(per + 16) * MR * TR * 4;
      p.rc = p.smem > 227 * 1024 ? 40 : 0;
      // one ceiling for every shape of this instantiation: plans of other shapes are cached and never set it again
      if (!p.rc && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) { (void)cudaGetLastError(); p.rc = 40; }
      it = plans.emplace(key, p).first;
    }
    p = it->second;
  }
  if (p.rc) {
    if (std::getenv("QUACTLIZE_B200_DEBUG")) std::fprintf(stderr, "[quactlize_b200] row-thread GEMV declines n=%d k=%d gy=%d: smem %zu\n", d.n, d.k, gy, p.smem);
    return p.rc;
  }
  // ---- tensor maps: cached per plane pointer -------------------------------------------------------------------------------
  struct MKey { void const* lo; void const* hi; void const* sc; void const* zr; int n, k, e, gs; bool operator<(MKey const& o) const {
    return lo != o.lo ? lo < o.lo : hi != o.hi ? hi < o.hi : sc != o.sc ? sc < o.sc : zr != o.zr ? zr < o.zr :
           n != o.n ? n < o.n : k != o.k ? k < o.k : e != o.e ? e < o.e : gs < o.gs; } };
  static std::map<MKey, RtMaps> maps;
  static std::mutex mmu;
  RtMaps m;
  {
    std::lock_guard<std::mutex> lk(mmu);
    MKey const key{d.low, HI ? d.high : nullptr, MODE == 0 ? d.scale : nullptr, MODE == 0 ? d.zero : nullptr, d.n, d.k, E, MODE == 0 ? d.group_size : 0};
    auto it = maps.find(key);
    if (it == maps.end()) {
      if (maps.size() > 4096) maps.clear();
      RtMaps nm{};
      {
        cuuint64_t const rb = cuuint64_t(d.k) * LO / 8;
        cuuint64_t dims[3] = {rb, cuuint64_t(d.n), cuuint64_t(E)};
        cuuint64_t str[2] = {rb, rb * d.n};
        cuuint32_t box[3] = {cuuint32_t(KS * LO / 8), cuuint32_t(TR), 1};
        if (!tma_make_map(&nm.lo, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d.low, dims, str, box, tma_row_swizzle(KS * LO / 8))) return kRuntimeError;
      }
      if constexpr (HI != 0) {
        cuuint64_t const rb = cuuint64_t(d.k) * HI / 8;
        cuuint64_t dims[3] = {rb, cuuint64_t(d.n), cuuint64_t(E)};
        cuuint64_t str[2] = {rb, rb * d.n};
        cuuint32_t box[3] = {cuuint32_t(kSlice * HI / 8), cuuint32_t(TR), 1};
        if (!tma_make_map(&nm.hi, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d.high, dims, str, box, tma_row_swizzle(kSlice * HI / 8))) return kRuntimeError;
      } else {
        nm.hi = nm.lo;
      }
      nm.sc = nm.lo; nm.zr = nm.lo;
      if constexpr (MODE == 0) {                            // fp16 [E][k/gs][n]: a box is 8 rows x the groups of one slice
        cuuint64_t const kg = cuuint64_t(d.k / d.group_size);
        cuuint64_t dims[3] = {cuuint64_t(d.n), kg, cuuint64_t(E)};
        cuuint64_t str[2] = {cuuint64_t(d.n) * 2, cuuint64_t(d.n) * 2 * kg};
        cuuint32_t box[3] = {cuuint32_t(TR), cuuint32_t(std::max(1, KS / d.group_size)), 1};
        if (!tma_make_map(&nm.sc, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, d.scale, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return kRuntimeError;
        if (d.zero && !tma_make_map(&nm.zr, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, d.zero, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return kRuntimeError;
      }
      it = maps.emplace(key, nm).first;
    }
    m = it->second;
  }
  RtArgs a{};
  a.d = d;
  a.ns = d.k / KS; a.nblocks = (d.n + TR - 1) / TR;
  a.status = rt_device_status_ptr();
  if (!a.status) return kRuntimeError;
  // Programmatic dependent launch: this kernel may be scheduled while the previous kernel of the stream drains; it reads
  // activations and offsets only after griddepcontrol.wait.  QUACTLIZE_B200_NO_PDL=1 launches it the plain way.
  static bool const no_pdl = std::getenv("QUACTLIZE_B200_NO_PDL") != nullptr;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.gx, gy); cfg.blockDim = dim3(512); cfg.dynamicSmemBytes = p.smem; cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = no_pdl ? 0 : 1;
  if (cudaLaunchKernelEx(&cfg, kern, m.lo, m.hi, m.sc, m.zr, a) != cudaSuccess) { (void)cudaGetLastError(); return kRuntimeError; }
  return 0;
}

// Rows per weight pass: several rows of one expert (or of a dense batch) share every tile when there are enough of them;
// a long K may leave no room for four rows of activations, then every row streams the weights itself.
template <int LO, int HI, int MODE, int QT, int NQ, int SL = 1>
int launch_rowthread(PlaneGemvDesc const& d, cudaStream_t stream) {
  bool const many = d.offsets ? d.m_rows >= 2 * std::max(1, d.experts) : d.m_rows >= 2;
  if (many) {
    int const rc = launch_rowthread_mr<LO, HI, MODE, QT, NQ, 4, SL, 1>(d, stream);
    if (rc != 40) return rc;
  }
  if constexpr (HI == 0 && MODE == 0) {
    // 32-row tiles, four weight rows per lane, where every warp of a CTA still gets two tiles or more
    int const nb32 = d.n / 32, sms = rt_sm_count();
    int const ctas = std::max(1, std::min(nb32, std::max(1, sms / std::max(1, std::min(d.m_rows, sms)))));
    if (d.n % 32 == 0 && (long long)nb32 * (d.k / (kSlice * SL)) / ctas >= 32) {
      int const rc = launch_rowthread_mr<LO, HI, MODE, QT, NQ, 1, SL, 4>(d, stream);
      if (rc != 40) return rc;
    }
  }
  if (d.n % 16 == 0) {                                 // 16-row tiles, two weight rows per lane
    int const rc = launch_rowthread_mr<LO, HI, MODE, QT, NQ, 1, SL, 2>(d, stream);
    if (rc != 40) return rc;
  }
  return launch_rowthread_mr<LO, HI, MODE, QT, NQ, 1, SL, 1>(d, stream);
}

}  // namespace

// 0 launched; 40 = this form does not cover the shape (the caller falls back to the segment-per-warp kernel)
int enqueue_rowthread_gemv(PlaneGemvDesc const& d, cudaStream_t s) {
  if (std::getenv("QUACTLIZE_B200_DEBUG"))
    std::fprintf(stderr, "[quactlize_b200] row-thread GEMV n=%d k=%d rows=%d experts=%d max_rows=%d bits=%d+%d gs=%d mode=%d act=%p low=%p\n",
                 d.n, d.k, d.m_rows, d.experts, d.max_rows, d.lo_bits, d.hi_bits, d.group_size, d.scale_mode, d.act, (void const*)d.low);
  if (d.k <= 0 || d.k % 256 || d.n < 8 || d.n % 8) return 40;    // the scale channel is copied in 16-byte runs of 8 rows
  auto aligned = [](void const* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (!aligned(d.low) || (d.hi_bits && !aligned(d.high)) || !aligned(d.act)) return 40;
  if (d.scale_mode == 1 ? !aligned(d.units) : (!aligned(d.scale) || (d.zero && !aligned(d.zero)))) return 40;
  if (d.scale_mode == 1) {
    switch (d.qtype) {
      case 10: return launch_rowthread<2, 0, 1, 10, 4>(d, s);
      case 11: return launch_rowthread<2, 1, 1, 11, 4>(d, s);
      case 12: return launch_rowthread<4, 0, 1, 12, 2>(d, s);
      case 13: return launch_rowthread<4, 1, 1, 13, 2>(d, s);
      case 14: return launch_rowthread<4, 2, 1, 14, 4>(d, s);
      default: return 40;
    }
  }
  int const gs = d.group_size;
  if (gs < 16 || (gs & (gs - 1)) || d.k % gs) return 40;
  int const nq = gs >= 64 ? 1 : 64 / gs;
  // a lone 2- or 1-bit plane takes 512- or 1024-code tiles (1 KB, as the 4-bit plane's) when K is a multiple of them
  if (d.hi_bits == 0 && d.lo_bits == 2 && d.k % 512 == 0 && gs >= 32) {
    int const rc = gs >= 64 ? launch_rowthread<2, 0, 0, 0, 2, 2>(d, s) : launch_rowthread<2, 0, 0, 0, 4, 2>(d, s);
    if (rc != 40) return rc;
  }
  if (d.hi_bits == 0 && d.lo_bits == 1 && d.k % 1024 == 0 && gs >= 64) {
    int const rc = launch_rowthread<1, 0, 0, 0, 4, 4>(d, s);
    if (rc != 40) return rc;
  }
  int const key = d.lo_bits * 100 + d.hi_bits * 10 + nq;
  switch (key) {
    case 401: return launch_rowthread<4, 0, 0, 0, 1>(d, s);
    case 402: return launch_rowthread<4, 0, 0, 0, 2>(d, s);
    case 404: return launch_rowthread<4, 0, 0, 0, 4>(d, s);
    case 412: return launch_rowthread<4, 1, 0, 0, 2>(d, s);
    case 411: return launch_rowthread<4, 1, 0, 0, 1>(d, s);
    case 424: return launch_rowthread<4, 2, 0, 0, 4>(d, s);
    case 421: return launch_rowthread<4, 2, 0, 0, 1>(d, s);
    case 201: return launch_rowthread<2, 0, 0, 0, 1>(d, s);
    case 202: return launch_rowthread<2, 0, 0, 0, 2>(d, s);
    case 204: return launch_rowthread<2, 0, 0, 0, 4>(d, s);
    case 214: return launch_rowthread<2, 1, 0, 0, 4>(d, s);
    case 211: return launch_rowthread<2, 1, 0, 0, 1>(d, s);
    case 101: return launch_rowthread<1, 0, 0, 0, 1>(d, s);
    case 102: return launch_rowthread<1, 0, 0, 0, 2>(d, s);
    default: return 40;
  }
}

}  // namespace qb
