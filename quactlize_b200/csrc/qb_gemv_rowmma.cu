// Small-batch GEMV over scale-first bit planes on the tensor cores (mma.sync m16n8k16): up to 8 activation rows of one
// expert (or of a dense batch) share every weight tile, and the per-row multiply-accumulate work of the CUDA-core
// kernel (qb_gemv_rowthread.cu) collapses into one MMA per 16 weight rows x 16 codes x 8 activation rows.
//
//   out[t, r] = sum_k a[t, k] * ( (u[r,k] + off) * s[r, k/gs] + z[r, k/gs] ),   u = low-plane code, gs >= 32
//
// Serves the MoE decode shapes of the reference's grouped / split-K family at a handful of rows per expert
// (quactlize/include/moe_grouped_ppu.cuh:69-361) and small dense batches of the scale-first GEMV
// (quactlize/include/gemv_lowbit/gemv_kernel.hpp:44-246).
//
// The weights never leave their packed form: (word & mask) read as fp16 IS code * 2^shift * 2^-24, and that register is
// an A-fragment register as it stands; the power of two goes into the B fragment, which is the activation row in
// "pattern order" prepared once per CTA in shared memory.  Lane (g, t) of a warp owns weight rows g and g+8 of a
// 16-row tile and the t-th word (or part of a word) of every step along K, so the 16 codes of one MMA come from the
// four lanes of a quad and always lie inside one scale group; products are accumulated in fp32 by the MMA, scaled per
// (weight row, group) and added to running sums.  Tiles arrive by tiled TMA into per-warp mbarrier rings; every wait is
// bounded.  Work split, partial sums and their fixed-order reduction are those of the row-thread kernel.
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
#include "qb_runtime.hpp"
#include "qb_tma.hpp"

namespace qb {

namespace {

constexpr int kTRows = 16;           // weight rows of a tile
constexpr int kTSlice = 256;         // codes of a tile along K
constexpr int kCols = 8;             // activation rows per group (the n of m16n8k16)
constexpr int kXPart = 64;           // codes per run of the pattern-order activation array
constexpr int kXPartStride = 144;    // bytes between runs (128 + 16: neighbouring runs on different banks)

struct MmaArgs {
  PlaneGemvDesc d;
  int ns, nblocks;                   // K slices per block, 16-row blocks
  int xrows;                         // activation rows kept in shared memory (1..8): the most any group has
  unsigned int* status;
};

__device__ __forceinline__ void tma_tile3(void* dst, CUtensorMap const* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ float2 lds_f32x2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
// D(16x8, fp32) += A(16x16, fp16, row) * B(16x8, fp16, col)
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// byte offset of 32-bit word `w` of plane row `rr` inside a TMA-swizzled tile whose rows are 32*LO bytes
template <int LO>
__device__ __forceinline__ uint32_t word_offset(int rr, int w) {
  if constexpr (LO == 4) return uint32_t(rr * 128 + ((((w >> 2) ^ rr) & 7) << 4) + (w & 3) * 4);
  else if constexpr (LO == 2) return uint32_t(rr * 64 + ((((w >> 2) ^ (rr >> 1)) & 3) << 4) + (w & 3) * 4);
  else return uint32_t(rr * 32 + ((((w >> 2) ^ (rr >> 2)) & 1) << 4) + (w & 3) * 4);
}

// LO plane bits; WL distinct words per step across a quad (4, 2 or 1); GQ = min(group size, 256) codes
// RB: 16-row blocks per tile (1 or 2).  With two, the activation fragments of an MMA and every per-tile step are shared by
// 32 weight rows.
template <int LO, int WL, int GQ, int STAGES, int RB>
__global__ void __launch_bounds__(512, 1)
rowmma_gemv_kernel(const __grid_constant__ CUtensorMap map_lo, const __grid_constant__ CUtensorMap map_sc,
                   const __grid_constant__ CUtensorMap map_zr, MmaArgs a) {
  constexpr int CW = 32 / LO;                         // codes per word
  constexpr int NP = 16 / LO;                         // half2 operands ("patterns") per word
  constexpr int PER = 8 / LO;                         // codes per byte
  constexpr int L = 4 / WL;                           // lanes of a quad that share a word
  constexpr int S = WL * CW;                          // codes per step
  constexpr int NSTEP = kTSlice / S;
  constexpr int MSTEP = WL * NP / 8;                  // MMAs per step
  constexpr int NGT = kTSlice / GQ;                   // scale groups per tile (1, 2, 4 or 8)
  constexpr int NGR = NGT > 4 ? NGT / 4 : 1;          // scale registers per row and lane
  constexpr int TR = kTRows * RB;                     // weight rows of a tile
  constexpr int TILE = TR * 32 * LO;
  // fp16 scale, then zero: [group][16 rows], copied with the tile; each half 128-byte aligned (destination of a tiled copy)
  constexpr int SC_HALF = NGT * TR * 2 < 128 ? 128 : NGT * TR * 2, SC_TILE = 2 * SC_HALF;
  constexpr int XPAD = LO == 4 ? 24 : 8;              // skew between activation rows: B-fragment loads spread over the banks
  static_assert(S <= GQ && GQ % S == 0, "the codes of one MMA must lie inside one scale group");
  static_assert((STAGES & (STAGES - 1)) == 0, "ring depth is a power of two");

  PlaneGemvDesc const& d = a.d;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  // the warp index is broadcast from lane 0: the compiler then keeps what derives from it (tile counts, ring and barrier
  // addresses, copy coordinates) in uniform registers and the per-tile bookkeeping off the vector pipes
  int const warp = __shfl_sync(0xffffffffu, int(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  int const g = lane >> 2, t = lane & 3;

  // ---- which group of activation rows / which expert (as in the row-thread kernel, 8 rows per group) ----------------------
  int e = 0, arow = 0, nrows = 1;
  // Under programmatic dependent launch the activations (and a router's offsets) may be the preceding kernel's output:
  // nothing of them is read before this wait.  Without the launch attribute it returns at once.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (d.offsets) {
    volatile int* sh = reinterpret_cast<volatile int*>(smem);            // ring space, not yet in use
    if (threadIdx.x < 4) sh[threadIdx.x] = -1;
    __syncthreads();
    volatile int* cnt = sh + 8;                                          // [experts] inclusive scan of group counts
    for (int x = threadIdx.x; x < d.experts; x += blockDim.x) cnt[x] = (d.offsets[x + 1] - d.offsets[x] + kCols - 1) / kCols;
    __syncthreads();
    if (warp == 0) {
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
    for (int x = threadIdx.x; x < d.experts; x += blockDim.x) {
      int const hi = cnt[x], lo = x ? cnt[x - 1] : 0;
      if (int(blockIdx.y) >= lo && int(blockIdx.y) < hi) { sh[0] = x; sh[1] = int(blockIdx.y) - lo; }
    }
    __syncthreads();
    e = sh[0];
    if (e >= 0) {
      int const r0 = d.offsets[e], r1 = d.offsets[e + 1];
      arow = r0 + sh[1] * kCols;
      nrows = min(min(kCols, a.xrows), r1 - arow);     // (a bound smaller than an expert's rows drops the surplus, as the grid bound does elsewhere)
    }
    __syncthreads();                                  // the scratch has been read before the first copy may land there
    if (e < 0) return;                                // uniform for the CTA
  } else {
    arow = blockIdx.y * kCols;
    nrows = min(min(kCols, a.xrows), d.m_rows - arow);
    if (nrows <= 0) return;
  }
  e = __shfl_sync(0xffffffffu, e, 0);                 // uniform for the compiler too (it was read from shared memory)
  int const k = d.k, n = d.n;

  // ---- shared memory carve-up -----------------------------------------------------------------------------------------
  constexpr int W = 16;
  int const nparts = k / kXPart;
  uint32_t const xrow = uint32_t(nparts) * kXPartStride + XPAD;          // bytes of one activation row in pattern order
  uint8_t* ring = smem;                                                  // [W][STAGES][TILE]
  uint8_t* sc_ring = ring + size_t(W) * STAGES * TILE;                   // [W][STAGES][SC_TILE]
  uint8_t* xpat = sc_ring + size_t(W) * STAGES * SC_TILE;                // [8][xrow]
  // [k/GQ][8]; the rows are skewed by 8 or 24 bytes, so their total is rounded up: the raw row behind is stored 16 bytes at a time
  float* sxq = reinterpret_cast<float*>(xpat + ((size_t(a.xrows) * xrow + 15) & ~size_t(15)));
  float* fmv = sxq + (k / GQ) * kCols;                                   // [8] 2^(24-ex) per activation row
  uint16_t* xraw = reinterpret_cast<uint16_t*>(fmv + kCols);             // [k] (prologue only)
  float* red = reinterpret_cast<float*>(xraw + k);                       // [16]
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 16);                // [W][STAGES]
  float* part = reinterpret_cast<float*>(bars + W * STAGES);             // [blocks of this CTA + 16][16 rows][8 cols]

  // ---- this warp's contiguous run of tiles ----------------------------------------------------------------------------------
  int const ns = a.ns;
  int const nb_c = blockIdx.x < a.nblocks ? (a.nblocks - 1 - blockIdx.x) / gridDim.x + 1 : 0;
  int const T = nb_c * ns;
  int const t0 = ((warp * T) >> 4), t1 = (((warp + 1) * T) >> 4);
  int const ntiles = t1 - t0;
  uint64_t* mybars = bars + warp * STAGES;
  uint8_t* myring = ring + size_t(warp) * STAGES * TILE;
  uint8_t* mysc = sc_ring + size_t(warp) * STAGES * SC_TILE;
  int const b_first = ntiles > 0 ? t0 / ns : 0, s_first = ntiles > 0 ? t0 % ns : 0;
  // next tile to request (lane 0 only): addresses and coordinates live in registers and advance by additions
  int is_s = s_first;
  int is_row0 = (blockIdx.x + b_first * gridDim.x) * TR;
  int const row_step = gridDim.x * TR;
  uint32_t const bar_a = smem_u32(mybars), ring_issue_a = smem_u32(myring);
  uint64_t const map_p = reinterpret_cast<uint64_t>(&map_lo);
  uint64_t const map_sc_p = reinterpret_cast<uint64_t>(&map_sc), map_zr_p = reinterpret_cast<uint64_t>(&map_zr);
  // the scale channel of a tile (fp16 scale and zero of its 16 rows and 256/gs groups) travels with it on the same mbarrier;
  // per-lane global loads of the scales queue behind the ring and were the largest stall of this kernel
  uint32_t const sc_issue_a = smem_u32(mysc);
  int const gs = d.group_size;
  int const gshift = 31 - __clz(gs);
  bool const has_zero = d.zero != nullptr;
  uint32_t const tx_bytes = TILE + uint32_t(NGT * TR * 2) * (has_zero ? 2u : 1u);   // the boxes' bytes, not the padded halves
  // called with q = 0, 1, 2, ... in order; every lane keeps the (uniform) bookkeeping, lane 0 issues the copies
  auto issue = [&](int q) {
    uint32_t const st = uint32_t(q) & (STAGES - 1), bar = bar_a + st * 8;
    int const gy = (is_s * kTSlice) >> gshift;
    if (lane == 0) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(tx_bytes) : "memory");
      asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                   ::"r"(sc_issue_a + st * SC_TILE), "l"(map_sc_p), "r"(bar), "r"(is_row0), "r"(gy), "r"(e) : "memory");
      if (has_zero)
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                     ::"r"(sc_issue_a + st * SC_TILE + SC_HALF), "l"(map_zr_p), "r"(bar), "r"(is_row0), "r"(gy), "r"(e) : "memory");
      asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                   ::"r"(ring_issue_a + st * TILE), "l"(map_p), "r"(bar), "r"(is_s * (kTSlice * LO / 8)), "r"(is_row0), "r"(e) : "memory");
    }
    if (++is_s == ns) { is_s = 0; is_row0 += row_step; }
  };
  // Activation rows are requested BEFORE the weight stream: a load issued after it queues behind the ring's copies and
  // costs a microsecond per row.  Row m + 1 is loaded into registers while row m is converted, and the stream starts as
  // soon as the last row's loads are in flight.
  constexpr int kPre = 4;                                   // 16-byte pieces per thread held in registers (K <= 16384)
  uint4 pre[kPre];
  auto load_row = [&](int m) {
    uint16_t const* x0 = reinterpret_cast<uint16_t const*>(d.act) + size_t(arow + m) * k;
#pragma unroll
    for (int j = 0; j < kPre; ++j) {
      if (j * 4096 >= k) break;                            // uniform: no thread has a piece j
      int const i = (int(threadIdx.x) + j * 512) * 8;
      pre[j] = i < k ? __ldg(reinterpret_cast<uint4 const*>(x0 + i)) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  load_row(0);
  if (!has_zero) {                                          // no copy ever lands in the zero halves: they read as zero
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
  for (int i = threadIdx.x; i < (nb_c + 16) * TR * kCols; i += blockDim.x) part[i] = 0.f;

  // ---- CTA prologue: every activation row of the group into pattern order --------------------------------------------------
  auto prologue = [&](auto bf16_tag) {
    constexpr bool BF = decltype(bf16_tag)::value;
    for (int m = 0; m < nrows; ++m) {
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
        for (int o = 1; o < GQ / 8; o <<= 1) p += __shfl_xor_sync(0xffffffffu, p, o);
        if ((lane & (GQ / 8 - 1)) == 0) sxq[(i / GQ) * kCols + m] = p;
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
      int const ex = pow2_scale_exponent(mx, 15);
      if (threadIdx.x == 0) fmv[m] = ldexpf(1.f, 24 - ex);
      pattern_row<LO, BF>(xraw, xpat + size_t(m) * xrow, k, ex, kXPart, kXPartStride);   // one half2 operand per code pair
      __syncthreads();                                     // xraw and red are reused by the next row
    }
  };
  if (d.act_bf16) prologue(std::true_type{});
  else prologue(std::false_type{});

  // ---- per-lane constants of the fragment addressing ------------------------------------------------------------------------
  constexpr uint32_t M1 = ((1u << LO) - 1u) * 0x00010001u;
  int const wsel = t / L, lsel = t % L;                      // which word of the step, which share of its patterns
  uint32_t const sc_a = smem_u32(mysc) + uint32_t(g) * 2;    // this lane's rows g (and g + 8) of the staged scales
  uint32_t const ring_a = smem_u32(myring), xpat_a = smem_u32(xpat) + uint32_t(min(g, a.xrows - 1)) * xrow,   // columns beyond the group's rows re-read a held row; their results are dropped
       sxq_a = smem_u32(sxq) + uint32_t(t) * 8;
  float const coff = float(d.code_offset);
  float totA[RB][4], totB[RB][4];
#pragma unroll
  for (int rb = 0; rb < RB; ++rb)
#pragma unroll
    for (int i = 0; i < 4; ++i) { totA[rb][i] = 0.f; totB[rb][i] = 0.f; }
  bool dead = false;
  int q = 0, cur_b = b_first, c_b = b_first, c_s = s_first;
  float const fm0 = fmv[2 * t], fm1 = fmv[2 * t + 1];
  // a warp's sums for one block go to slot (block + warp): runs are contiguous and ordered, so slots never collide
  auto flush = [&](int bi) {
#pragma unroll
    for (int rb = 0; rb < RB; ++rb) {
      float* p0 = part + (size_t(bi + warp) * TR + 16 * rb + g) * kCols + 2 * t;
      *reinterpret_cast<float2*>(p0) = make_float2(fmaf(totA[rb][0], fm0, totB[rb][0]), fmaf(totA[rb][1], fm1, totB[rb][1]));
      *reinterpret_cast<float2*>(p0 + 8 * kCols) = make_float2(fmaf(totA[rb][2], fm0, totB[rb][2]), fmaf(totA[rb][3], fm1, totB[rb][3]));
#pragma unroll
      for (int i = 0; i < 4; ++i) { totA[rb][i] = 0.f; totB[rb][i] = 0.f; }
    }
  };
  for (; q < ntiles; ++q) {
    int const st = q & (STAGES - 1);
    int const bi = c_b, s = c_s;
    if (++c_s == ns) { c_s = 0; ++c_b; }
    if (bi != cur_b) { flush(cur_b); cur_b = bi; }
    if (!mbar_wait_bounded(&mybars[st], unsigned(q / STAGES) & 1u, a.status, kWaitStageTimeout)) { dead = true; break; }
    uint32_t const tile_a = ring_a + st * TILE;
    float c[RB][4];
#pragma unroll
    for (int rb = 0; rb < RB; ++rb) c[rb][0] = c[rb][1] = c[rb][2] = c[rb][3] = 0.f;
    uint32_t dep = 0u;
#pragma unroll
    for (int j = 0; j < NSTEP; ++j) {
      int const w = j * WL + wsel;                           // word of the row's 256 codes this lane reads in this step
      uint32_t w_lo[RB], w_hi[RB];
#pragma unroll
      for (int rb = 0; rb < RB; ++rb) {                      // the swizzle pattern repeats every 8 rows
        w_lo[rb] = lds32(tile_a + rb * (16 * 32 * LO) + word_offset<LO>(g, w));
        w_hi[rb] = lds32(tile_a + rb * (16 * 32 * LO) + word_offset<LO>(g + 8, w));
      }
      // pattern-order activations of that word: run (s*4 + code/64), word inside the run, then this lane's patterns
      int const code0 = j * S + wsel * CW;
      uint32_t const xw = xpat_a + uint32_t(s * (kTSlice / kXPart) + code0 / kXPart) * kXPartStride + uint32_t((code0 % kXPart) / CW) * (NP * 4);
#pragma unroll
      for (int i = 0; i < MSTEP; ++i) {
        int const p = i * 2 * L + 2 * lsel;                  // this lane's two patterns of MMA i (compile-time when L == 1)
        int const h = p / PER, o = p % PER;
        uint32_t const mA = M1 << (o * LO), mB = M1 << ((o + 1) * LO);
        uint2 const b = lds64(xw + uint32_t(p) * 4);         // one activation fragment for every row block
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) {
          uint32_t const src_lo = w_lo[rb] >> (8 * h), src_hi = w_hi[rb] >> (8 * h);
          mma16816(c[rb], src_lo & mA, src_hi & mA, src_lo & mB, src_hi & mB, b.x, b.y);
        }
      }
      if (((j + 1) * S) % GQ == 0) {                         // a scale group is complete (compile-time condition)
        int const jg = (j * S) / GQ;
        float2 const sx = lds_f32x2(sxq_a + uint32_t(s * NGT + jg) * (kCols * 4));                     // sums of x, columns 2t, 2t+1
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) {
          uint32_t const sat = sc_a + st * SC_TILE + jg * (TR * 2) + rb * 32;
          uint32_t const raw_lo = lds_u16(sat) | (lds_u16(sat + SC_HALF) << 16);        // the zero half holds zeros when there is no zero plane
          uint32_t const raw_hi = lds_u16(sat + 16) | (lds_u16(sat + SC_HALF + 16) << 16);
          dep ^= raw_lo ^ raw_hi;
          float2 const lo = __half22float2(u32_as_h2(raw_lo)), hi = __half22float2(u32_as_h2(raw_hi));   // (scale, zero)
          totA[rb][0] = fmaf(lo.x, c[rb][0], totA[rb][0]); totA[rb][1] = fmaf(lo.x, c[rb][1], totA[rb][1]);
          totA[rb][2] = fmaf(hi.x, c[rb][2], totA[rb][2]); totA[rb][3] = fmaf(hi.x, c[rb][3], totA[rb][3]);
          float const oz_lo = fmaf(coff, lo.x, lo.y), oz_hi = fmaf(coff, hi.x, hi.y);
          totB[rb][0] = fmaf(oz_lo, sx.x, totB[rb][0]); totB[rb][1] = fmaf(oz_lo, sx.y, totB[rb][1]);
          totB[rb][2] = fmaf(oz_hi, sx.x, totB[rb][2]); totB[rb][3] = fmaf(oz_hi, sx.y, totB[rb][3]);
          c[rb][0] = c[rb][1] = c[rb][2] = c[rb][3] = 0.f;
        }
      }
    }
    {                                                        // the scale loads have returned before the slot is refilled
      uint32_t sink;
      asm volatile("mov.u32 %0, %1;" : "=r"(sink) : "r"(dep) : "memory");
    }
    __syncwarp();                                            // every lane's loads of this tile were consumed by its MMAs
    if (q + STAGES < ntiles) issue(q + STAGES);
  }
  if (ntiles > 0 && !dead) flush(cur_b);
  if (dead)                                                  // let copies already in flight land before the CTA's memory is reused
    for (int i = q + 1; i < ntiles && i < q + STAGES; ++i)
      (void)mbar_wait_bounded(&mybars[i % STAGES], unsigned(i / STAGES) & 1u, nullptr, 0, 250000000ull);
  __syncthreads();
  // ---- every block's contributions, added in warp order (fixed: results do not depend on timing) ------------------------------
  for (int o = threadIdx.x; o < nb_c * TR * kCols; o += blockDim.x) {
    int const bi = o / (TR * kCols), col = (o / TR) % kCols, rr = o % TR;                 // consecutive threads: consecutive rows
    int const row = (blockIdx.x + bi * gridDim.x) * TR + rr;
    if (row >= n || col >= nrows) continue;
    float sum = 0.f;
    // with many blocks per CTA only the warps whose run can touch block bi are visited (a conservative range; the test
    // below is exact); with one or two blocks the two divisions would cost more than the full loop
    int w_lo = 0, w_hi = 15;
    if (nb_c > 2) { w_lo = max(0, (bi * ns * 16) / T - 1); w_hi = min(15, ((bi + 1) * ns * 16) / T + 1); }
    for (int w2 = w_lo; w2 <= w_hi; ++w2) {
      int const u0 = ((w2 * T) >> 4), u1 = (((w2 + 1) * T) >> 4);
      if (u1 > u0 && u0 < (bi + 1) * ns && u1 > bi * ns) sum += part[(size_t(bi + w2) * TR + rr) * kCols + col];
    }
    size_t const oi = size_t(arow + col) * n + row;
    if (d.out_kind == 1) reinterpret_cast<float*>(d.out)[oi] = sum;
    else if (d.out_kind == 0) reinterpret_cast<__half*>(d.out)[oi] = __float2half_rn(sum);
    else reinterpret_cast<__nv_bfloat16*>(d.out)[oi] = __float2bfloat16_rn(sum);
  }
}

struct MmaPlan { int gx, rc; size_t smem; };

template <int LO, int WL, int GQ, int STAGES, int RB>
int launch_rowmma_st(PlaneGemvDesc const& d, cudaStream_t stream) {
  constexpr int TR = kTRows * RB;
  constexpr int TILE = TR * 32 * LO;
  constexpr int XPAD = LO == 4 ? 24 : 8;
  constexpr int SC_TILE = 2 * std::max(128, (kTSlice / GQ) * TR * 2);
  auto kern = rowmma_gemv_kernel<LO, WL, GQ, STAGES, RB>;
  // grid rows: one per group of up to 8 activation rows of one expert (ragged: an upper bound, surplus CTAs exit at once)
  int const gy = d.offsets ? std::min(d.m_rows, d.m_rows / kCols + d.experts) : (d.m_rows + kCols - 1) / kCols;
  if (gy <= 0 || gy > 65535) return 40;
  int const E = d.experts > 0 ? d.experts : 1;
  int dev = 0;
  cudaGetDevice(&dev);
  // activation rows to hold: a dense batch's own count, or the caller's bound on any expert's rows
  int const xrows = std::max(1, std::min(kCols, d.offsets ? (d.max_rows > 0 ? d.max_rows : kCols) : d.m_rows));
  struct Key { int n, k, gy, rows, xrows, dev; bool operator<(Key const& o) const {
    return n != o.n ? n < o.n : k != o.k ? k < o.k : gy != o.gy ? gy < o.gy : rows != o.rows ? rows < o.rows : xrows != o.xrows ? xrows < o.xrows : dev < o.dev; } };
  static std::map<Key, MmaPlan> plans;
  static std::mutex mu;
  MmaPlan p{};
  {
    std::lock_guard<std::mutex> lk(mu);
    Key const key{d.n, d.k, gy, d.m_rows, xrows, dev};
    auto it = plans.find(key);
    if (it == plans.end()) {
      int const nblocks = (d.n + TR - 1) / TR, sms = rt_sm_count();
      // groups that do work: between rows/8 and one per expert with rows; a ragged launch cannot know, assume the mean
      int const groups = d.offsets ? std::max(1, std::min(d.m_rows, (d.m_rows / kCols + std::min(d.experts, d.m_rows) + 1) / 2))
                                   : (d.m_rows + kCols - 1) / kCols;
      int const share = std::max(1, sms / std::max(1, std::min(groups, sms)));
      p.gx = std::max(1, std::min(nblocks, share));
      int const per = std::min(256, (nblocks + p.gx - 1) / p.gx);
      p.gx = (nblocks + per - 1) / per;
      int const nparts = d.k / kXPart;
      p.smem = 1024 + size_t(16) * STAGES * (TILE + SC_TILE) + ((size_t(xrows) * (size_t(nparts) * kXPartStride + XPAD) + 15) & ~size_t(15)) +
               size_t(d.k / GQ) * kCols * 4 + kCols * 4 + size_t(d.k) * 2 + 16 * 4 + size_t(16) * STAGES * 8 +
               size_t(per + 16) * TR * kCols * 4;
      p.rc = p.smem > 227 * 1024 ? 40 : 0;
      if (!p.rc && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) { (void)cudaGetLastError(); p.rc = 40; }
      it = plans.emplace(key, p).first;
    }
    p = it->second;
  }
  if (p.rc) return p.rc;
  struct MKey { void const* lo; void const* sc; void const* zr; int n, k, e, gs; bool operator<(MKey const& o) const {
    return lo != o.lo ? lo < o.lo : sc != o.sc ? sc < o.sc : zr != o.zr ? zr < o.zr : n != o.n ? n < o.n : k != o.k ? k < o.k :
           e != o.e ? e < o.e : gs < o.gs; } };
  struct Maps { CUtensorMap lo, sc, zr; };
  static std::map<MKey, Maps> maps;
  static std::mutex mmu;
  Maps m;
  {
    std::lock_guard<std::mutex> lk(mmu);
    MKey const key{d.low, d.scale, d.zero, d.n, d.k, E, d.group_size};
    auto it = maps.find(key);
    if (it == maps.end()) {
      if (maps.size() > 4096) maps.clear();
      Maps nm;
      cuuint64_t const rb = cuuint64_t(d.k) * LO / 8;
      cuuint64_t dims[3] = {rb, cuuint64_t(d.n), cuuint64_t(E)};
      cuuint64_t str[2] = {rb, rb * d.n};
      cuuint32_t box[3] = {cuuint32_t(kTSlice * LO / 8), cuuint32_t(TR), 1};
      if (!tma_make_map(&nm.lo, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d.low, dims, str, box, tma_row_swizzle(kTSlice * LO / 8))) return kRuntimeError;
      {                                                     // fp16 [E][k/gs][n]: a box is 16 rows x the groups of one slice
        cuuint64_t const kg = cuuint64_t(d.k / d.group_size);
        cuuint64_t sdims[3] = {cuuint64_t(d.n), kg, cuuint64_t(E)};
        cuuint64_t sstr[2] = {cuuint64_t(d.n) * 2, cuuint64_t(d.n) * 2 * kg};
        cuuint32_t sbox[3] = {cuuint32_t(TR), cuuint32_t(kTSlice / GQ), 1};
        if (!tma_make_map(&nm.sc, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, d.scale, sdims, sstr, sbox, CU_TENSOR_MAP_SWIZZLE_NONE)) return kRuntimeError;
        nm.zr = nm.sc;
        if (d.zero && !tma_make_map(&nm.zr, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, d.zero, sdims, sstr, sbox, CU_TENSOR_MAP_SWIZZLE_NONE)) return kRuntimeError;
      }
      it = maps.emplace(key, nm).first;
    }
    m = it->second;
  }
  MmaArgs a{};
  a.d = d;
  a.ns = d.k / kTSlice; a.nblocks = (d.n + TR - 1) / TR; a.xrows = xrows;
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
  if (cudaLaunchKernelEx(&cfg, kern, m.lo, m.sc, m.zr, a) != cudaSuccess) { (void)cudaGetLastError(); return kRuntimeError; }
  return 0;
}

// Ring depth: 64-128 KB in flight per SM (32 KB for the 1-bit plane).  A 4-bit plane with a long K leaves no room for
// eight rows of activations beside a 128 KB ring; it runs with half the depth rather than falling back to a kernel
// that streams the weights once per four rows.
template <int LO, int WL, int GQ>
int launch_rowmma(PlaneGemvDesc const& d, cudaStream_t stream) {
  constexpr int ST = LO == 1 ? 8 : 4;
  if (d.n % 32 == 0) {                                 // 32-row tiles: the same bytes per ring with half the stages
    int const rc = launch_rowmma_st<LO, WL, GQ, ST / 2, 2>(d, stream);
    if (rc != 40) return rc;
  }
  int const rc = launch_rowmma_st<LO, WL, GQ, ST, 1>(d, stream);
  if constexpr (LO == 4) {
    if (rc == 40) return launch_rowmma_st<LO, WL, GQ, 2, 1>(d, stream);
  }
  return rc;
}

}  // namespace

// 0 launched; 40 = this form does not cover the shape (scale-first planes without a high plane, group size >= 32, n >= 16)
int enqueue_rowmma_gemv(PlaneGemvDesc const& d, cudaStream_t s) {
  if (d.scale_mode != 0 || d.hi_bits != 0 || d.k <= 0 || d.k % 256 || d.n < 16 || d.n % 8) return 40;   // scale rows are copied in 16-byte units
  auto aligned = [](void const* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (!aligned(d.low) || !aligned(d.act) || !aligned(d.scale) || (d.zero && !aligned(d.zero))) return 40;
  int const gs = d.group_size;
  if (gs < 32 || (gs & (gs - 1)) || d.k % gs) return 40;
  int const gq = gs >= 256 ? 256 : gs;
  switch (d.lo_bits * 1000 + gq) {
    case 4032: return launch_rowmma<4, 4, 32>(d, s);
    case 4064: return launch_rowmma<4, 4, 64>(d, s);
    case 4128: return launch_rowmma<4, 4, 128>(d, s);
    case 4256: return launch_rowmma<4, 4, 256>(d, s);
    case 2032: return launch_rowmma<2, 2, 32>(d, s);
    case 2064: return launch_rowmma<2, 4, 64>(d, s);
    case 2128: return launch_rowmma<2, 4, 128>(d, s);
    case 2256: return launch_rowmma<2, 4, 256>(d, s);
    case 1032: return launch_rowmma<1, 1, 32>(d, s);
    case 1064: return launch_rowmma<1, 2, 64>(d, s);
    case 1128: return launch_rowmma<1, 4, 128>(d, s);
    case 1256: return launch_rowmma<1, 4, 256>(d, s);
    default: return 40;
  }
}

}  // namespace qb
