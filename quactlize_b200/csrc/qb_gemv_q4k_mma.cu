// Raw GGUF Q4_K blocks, small batches (2..16 activation rows), on the tensor cores (mma.sync m16n8k16).
//
//   out[t, r] = sum_b sum_g ( d_rb*sc_rbg * sum_j q_rbgj x[t, 256b+32g+j]  -  dmin_rb*mn_rbg * sum_j x[t, 256b+32g+j] )
//
// The M = 1 kernel (qb_gemv_q4k.cu) pays four HFMA2 per eight weights and per activation row; here the packed nibbles go
// to the MMA as they are -- (w >> s) & 0x000F000F read as fp16 IS two codes * 2^-24, which is an A-fragment register --
// and one instruction multiplies 16 weight rows x 16 codes by up to 8 activation rows.  Replaces the M > 1 arm of the
// reference's vecdot_rows_kernel (quactlize/include/gguf_vecdot.hpp:604-760, launch policy :564-602).
//
// Tile = 16 rows x one 144-byte superblock, fetched by a tiled TMA copy (row pitch 144*bpr bytes) into per-warp
// mbarrier rings.  Lane (g, t) owns rows g, g+8 and, in each 32-byte chunk of qs, words t and t+4: the low nibbles of a
// word are four codes of group 2c, the high nibbles four codes of group 2c+1, so the 16 codes of one MMA come from the
// four lanes of a quad and stay inside one 32-code group.  fp32 products from the MMA are scaled per (row, group) with
// d*sc; the min term uses the sums of x over each group.  The 6-bit sub-scales are unpacked with word-wide masks, two
// groups per lane, and handed round the quad by shuffles.  Activations are converted once per CTA into the order the
// fragments want ([x0 x2 x1 x3] per four elements, pre-scaled by a power of two).  Work split, partial sums and their
// fixed-order reduction follow the row-thread plane kernel.  Every mbarrier wait is bounded.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <map>
#include <mutex>

#include "qb_device.cuh"
#include "qb_internal.hpp"
#include "qb_runtime.hpp"
#include "qb_tma.hpp"

namespace qb {

namespace {

constexpr int kQRows = 16;               // weight rows of a tile
constexpr int kQBlock = 144;             // bytes of a Q4_K superblock
constexpr int kQTile = kQRows * kQBlock; // 2304
constexpr int kQCols = 8;                // the n of m16n8k16

struct Q4MmaArgs {
  uint8_t const* blocks;
  __half const* x;
  float* out;
  int const* offsets;                    // cumulative [experts+1] (grouped) or nullptr
  int n, bpr, experts, m_rows;
  int cpg;                               // activation rows per group: 8, or 4 when eight rows of activations do not fit
  int nblocks;                           // 16-row blocks
  unsigned int* status;
};

__device__ __forceinline__ void q_tma3(void* dst, CUtensorMap const* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ uint32_t q_lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 q_lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ float2 q_ldsf2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ void q_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// d*sc and dmin*mn of groups t and t+4 of one row, from the block's first four words (d|dmin, 12 scale bytes)
__device__ __forceinline__ void q4k_lane_scales(uint32_t hdr, uint32_t s0, uint32_t s1, uint32_t s2, int t, float* dl, float* ml) {
  // bytes of s0: 6-bit sc of groups 0..3 (top 2 bits: high bits of sc 4..7); s1: mn 0..3 (top bits: mn 4..7);
  // s2: low nibbles sc 4..7, high nibbles mn 4..7
  uint32_t const sc_lo = s0 & 0x3F3F3F3Fu, mn_lo = s1 & 0x3F3F3F3Fu;
  uint32_t const sc_hi = (s2 & 0x0F0F0F0Fu) | (((s0 >> 6) & 0x03030303u) << 4);
  uint32_t const mn_hi = ((s2 >> 4) & 0x0F0F0F0Fu) | (((s1 >> 6) & 0x03030303u) << 4);
  float2 const dd = __half22float2(u32_as_h2(hdr));
  int const sh = 8 * t;
  dl[0] = dd.x * float((sc_lo >> sh) & 0xFFu); ml[0] = dd.y * float((mn_lo >> sh) & 0xFFu);
  dl[1] = dd.x * float((sc_hi >> sh) & 0xFFu); ml[1] = dd.y * float((mn_hi >> sh) & 0xFFu);
}

template <int STAGES>
__global__ void __launch_bounds__(512, 1) q4k_mma_kernel(const __grid_constant__ CUtensorMap map_b, Q4MmaArgs a) {
  static_assert((STAGES & (STAGES - 1)) == 0, "ring depth is a power of two");
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  // the warp index is broadcast from lane 0: the compiler then keeps what derives from it (tile counts, ring and barrier
  // addresses, copy coordinates) in uniform registers and the per-tile bookkeeping off the vector pipes
  int const warp = __shfl_sync(0xffffffffu, int(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  int const g = lane >> 2, t = lane & 3;
  int const cpg = a.cpg;

  // ---- which group of activation rows / which expert ----------------------------------------------------------------------
  int e = 0, arow = 0, nrows = 1;
  // Under programmatic dependent launch the activations (and a router's offsets) may be the preceding kernel's output:
  // nothing of them is read before this wait.  Without the launch attribute it returns at once.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (a.offsets) {
    volatile int* sh = reinterpret_cast<volatile int*>(smem);            // ring space, not yet in use
    if (threadIdx.x < 4) sh[threadIdx.x] = -1;
    __syncthreads();
    volatile int* cnt = sh + 8;
    for (int x = threadIdx.x; x < a.experts; x += blockDim.x) cnt[x] = (a.offsets[x + 1] - a.offsets[x] + cpg - 1) / cpg;
    __syncthreads();
    if (warp == 0) {                                                     // inclusive scan of the per-expert group counts
      int carry = 0;
      for (int base = 0; base < a.experts; base += 32) {
        int v = base + lane < a.experts ? cnt[base + lane] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { int const u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
        v += carry;
        if (base + lane < a.experts) cnt[base + lane] = v;
        carry = __shfl_sync(0xffffffffu, v, 31);
      }
    }
    __syncthreads();
    for (int x = threadIdx.x; x < a.experts; x += blockDim.x) {
      int const hi = cnt[x], lo = x ? cnt[x - 1] : 0;
      if (int(blockIdx.y) >= lo && int(blockIdx.y) < hi) { sh[0] = x; sh[1] = int(blockIdx.y) - lo; }
    }
    __syncthreads();
    e = sh[0];
    if (e >= 0) {
      int const r0 = a.offsets[e], r1 = a.offsets[e + 1];
      arow = r0 + sh[1] * cpg;
      nrows = min(cpg, r1 - arow);
    }
    __syncthreads();
    if (e < 0) return;                                                   // uniform for the CTA
  } else {
    arow = blockIdx.y * cpg;
    nrows = min(cpg, a.m_rows - arow);
    if (nrows <= 0) return;
  }
  e = __shfl_sync(0xffffffffu, e, 0);                                    // uniform for the compiler too (it was read from shared memory)
  int const n = a.n, bpr = a.bpr, k = bpr * 256;

  // ---- shared memory carve-up -----------------------------------------------------------------------------------------
  constexpr int W = 16;
  uint32_t const xrow = uint32_t(k) * 2 + 32;                            // bytes per activation row (+32: the eight rows a B fragment reads sit on different banks)
  uint8_t* ring = smem;                                                  // [W][STAGES][kQTile]
  uint8_t* xpat = ring + size_t(W) * STAGES * kQTile;                    // [cpg][xrow] fp16, [x0 x2 x1 x3] order, pre-scaled
  float* sxq = reinterpret_cast<float*>(xpat + size_t(cpg) * xrow);      // [k/32][8] sums of x per group
  float* fmv = sxq + (k / 32) * kQCols;                                  // [8]
  float* red = fmv + kQCols;                                             // [16]
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 16);                // [W][STAGES]
  float* part = reinterpret_cast<float*>(bars + W * STAGES);             // [blocks of this CTA + 16][16][8]

  // ---- this warp's contiguous run of tiles ----------------------------------------------------------------------------------
  int const nb_c = blockIdx.x < a.nblocks ? (a.nblocks - 1 - blockIdx.x) / gridDim.x + 1 : 0;
  int const T = nb_c * bpr;
  int const t0 = ((warp * T) >> 4), t1 = (((warp + 1) * T) >> 4);
  int const ntiles = t1 - t0;
  uint64_t* mybars = bars + warp * STAGES;
  uint8_t* myring = ring + size_t(warp) * STAGES * kQTile;
  int const b_first = ntiles > 0 ? t0 / bpr : 0, s_first = ntiles > 0 ? t0 % bpr : 0;
  // next tile to request (lane 0 only): addresses and coordinates live in registers and advance by additions
  int is_s = s_first;
  int is_row0 = (blockIdx.x + b_first * gridDim.x) * kQRows;
  int const row_step = gridDim.x * kQRows;
  uint32_t const bar_a = smem_u32(mybars), ring_issue_a = smem_u32(myring);
  uint64_t const map_p = reinterpret_cast<uint64_t>(&map_b);
  // called with q = 0, 1, 2, ... in order; every lane keeps the (uniform) bookkeeping, lane 0 issues the copies
  auto issue = [&](int q) {
    uint32_t const st = uint32_t(q) & (STAGES - 1), bar = bar_a + st * 8;
    if (lane == 0) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "n"(kQTile) : "memory");
      asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                   ::"r"(ring_issue_a + st * kQTile), "l"(map_p), "r"(bar), "r"(is_s * kQBlock), "r"(is_row0), "r"(e) : "memory");
    }
    if (++is_s == bpr) { is_s = 0; is_row0 += row_step; }
  };
  // Activation rows are requested BEFORE the weight stream: a load issued after it queues behind the ring's copies and
  // costs a microsecond per row.  Row m + 1 is loaded into registers while row m is converted, and the stream starts as
  // soon as the last row's loads are in flight.
  constexpr int kPre = 4;                                   // 16-byte pieces per thread held in registers (K <= 16384)
  uint4 pre[kPre];
  auto load_row = [&](int m) {
    uint16_t const* x0 = reinterpret_cast<uint16_t const*>(a.x) + size_t(arow + m) * k;
#pragma unroll
    for (int j = 0; j < kPre; ++j) {
      if (j * 4096 >= k) break;                            // uniform: no thread has a piece j
      int const i = (int(threadIdx.x) + j * 512) * 8;
      pre[j] = i < k ? __ldg(reinterpret_cast<uint4 const*>(x0 + i)) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  load_row(0);
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
  for (int i = threadIdx.x; i < (nb_c + 16) * kQRows * kQCols; i += blockDim.x) part[i] = 0.f;

  // ---- CTA prologue: activations into fragment order -------------------------------------------------------------------------
  for (int m = 0; m < nrows; ++m) {
    uint16_t const* xr = reinterpret_cast<uint16_t const*>(a.x) + size_t(arow + m) * k;
    float mx = 0.f;
    uint4 cur[kPre];
#pragma unroll
    for (int j = 0; j < kPre; ++j) cur[j] = pre[j];
    if (m + 1 < nrows) {                                                 // uniform for the CTA
      load_row(m + 1);
      if (m + 2 == nrows) start_stream();
    }
    auto piece = [&](int i, uint4 v) {                                   // k % 256 == 0: whole warps in or out
      uint32_t const w4[4] = {v.x, v.y, v.z, v.w};
      float p = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 const f = __half22float2(u32_as_h2(w4[j]));
        mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
        p += f.x + f.y;
      }
      p += __shfl_xor_sync(0xffffffffu, p, 1);
      p += __shfl_xor_sync(0xffffffffu, p, 2);
      if ((lane & 3) == 0) sxq[(i / 32) * kQCols + m] = p;
    };
#pragma unroll
    for (int j = 0; j < kPre; ++j) {
      if (j * 4096 >= k) break;                            // uniform
      int const i = (int(threadIdx.x) + j * 512) * 8;
      if (i < k) piece(i, cur[j]);
    }
    for (int i = (int(threadIdx.x) + kPre * 512) * 8; i < k; i += 512 * 8) piece(i, __ldg(reinterpret_cast<uint4 const*>(xr + i)));
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
    float const mul = __int_as_float((127 + ex) << 23);
    auto convert = [&](int i, uint4 v) {
      float2 const f0 = __half22float2(u32_as_h2(v.x)), f1 = __half22float2(u32_as_h2(v.y));
      float2 const f2 = __half22float2(u32_as_h2(v.z)), f3 = __half22float2(u32_as_h2(v.w));
      uint4 o;                                                           // [x0 x2 | x1 x3] [x4 x6 | x5 x7]
      o.x = h2_as_u32(__floats2half2_rn(f0.x * mul, f1.x * mul)); o.y = h2_as_u32(__floats2half2_rn(f0.y * mul, f1.y * mul));
      o.z = h2_as_u32(__floats2half2_rn(f2.x * mul, f3.x * mul)); o.w = h2_as_u32(__floats2half2_rn(f2.y * mul, f3.y * mul));
      uint8_t* dst = xpat + size_t(m) * xrow + size_t(i) * 2;            // 16-byte aligned
      *reinterpret_cast<uint2*>(dst) = make_uint2(o.x, o.y);
      *reinterpret_cast<uint2*>(dst + 8) = make_uint2(o.z, o.w);
    };
#pragma unroll
    for (int j = 0; j < kPre; ++j) {                                     // the pieces are still in registers
      if (j * 4096 >= k) break;                                          // uniform
      int const i = (int(threadIdx.x) + j * 512) * 8;
      if (i < k) convert(i, cur[j]);
    }
    for (int i = (int(threadIdx.x) + kPre * 512) * 8; i < k; i += 512 * 8) convert(i, __ldg(reinterpret_cast<uint4 const*>(xr + i)));
    __syncthreads();                                                     // red is reused by the next row
  }

  // ---- main loop ----------------------------------------------------------------------------------------------------------
  uint32_t const ring_a = smem_u32(myring);
  uint32_t const xcol_a = smem_u32(xpat) + uint32_t(g % cpg) * xrow + uint32_t(t) * 8;   // column g of the MMA = activation row g
  uint32_t const sxq_a = smem_u32(sxq) + uint32_t(t) * 8;
  uint32_t const row_lo = uint32_t(g) * kQBlock, row_hi = uint32_t(g + 8) * kQBlock;
  float totA[4] = {0.f, 0.f, 0.f, 0.f}, totB[4] = {0.f, 0.f, 0.f, 0.f};
  float const fm0 = fmv[2 * t], fm1 = fmv[2 * t + 1];
  bool dead = false;
  int q = 0, cur_b = b_first, c_b = b_first, c_s = s_first;
  auto flush = [&](int bi) {
    float* p0 = part + (size_t(bi + warp) * kQRows + g) * kQCols + 2 * t;
    *reinterpret_cast<float2*>(p0) = make_float2(fmaf(totA[0], fm0, -totB[0]), fmaf(totA[1], fm1, -totB[1]));
    *reinterpret_cast<float2*>(p0 + 8 * kQCols) = make_float2(fmaf(totA[2], fm0, -totB[2]), fmaf(totA[3], fm1, -totB[3]));
#pragma unroll
    for (int i = 0; i < 4; ++i) { totA[i] = 0.f; totB[i] = 0.f; }
  };
  for (; q < ntiles; ++q) {
    int const st = q & (STAGES - 1);
    int const bi = c_b, s = c_s;
    if (++c_s == bpr) { c_s = 0; ++c_b; }
    if (bi != cur_b) { flush(cur_b); cur_b = bi; }
    if (!mbar_wait_bounded(&mybars[st], unsigned(q / STAGES) & 1u, a.status, kWaitStageTimeout)) { dead = true; break; }
    uint32_t const lo_a = ring_a + st * kQTile + row_lo, hi_a = ring_a + st * kQTile + row_hi;
    // sub-scales: this lane unpacks groups t and t+4 of its two rows
    float dl_lo[2], ml_lo[2], dl_hi[2], ml_hi[2];
    q4k_lane_scales(q_lds32(lo_a), q_lds32(lo_a + 4), q_lds32(lo_a + 8), q_lds32(lo_a + 12), t, dl_lo, ml_lo);
    q4k_lane_scales(q_lds32(hi_a), q_lds32(hi_a + 4), q_lds32(hi_a + 8), q_lds32(hi_a + 12), t, dl_hi, ml_hi);
    uint32_t const xb = xcol_a + uint32_t(s) * 512;                       // this block's 256 activations of column g
    uint32_t const sb = sxq_a + uint32_t(s) * (8 * kQCols * 4);
#pragma unroll
    for (int c = 0; c < 4; ++c) {                                         // 32-byte chunk of qs: groups 2c (low nibbles), 2c+1 (high)
      float ce[4] = {0.f, 0.f, 0.f, 0.f}, co[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int hw = 0; hw < 2; ++hw) {
        uint32_t const wl = q_lds32(lo_a + 16 + 32 * c + 16 * hw + 4 * t), wh = q_lds32(hi_a + 16 + 32 * c + 16 * hw + 4 * t);
        // elements 16*hw + 4t .. +3 of each group: B registers [x_j x_{j+2}], [x_{j+1} x_{j+3}]
        uint2 const be = q_lds64(xb + uint32_t(64 * c + 16 * hw) * 2);
        uint2 const bo = q_lds64(xb + uint32_t(64 * c + 32 + 16 * hw) * 2);
        q_mma(ce, wl & 0x000F000Fu, wh & 0x000F000Fu, (wl >> 8) & 0x000F000Fu, (wh >> 8) & 0x000F000Fu, be.x, be.y);
        q_mma(co, (wl >> 4) & 0x000F000Fu, (wh >> 4) & 0x000F000Fu, (wl >> 12) & 0x000F000Fu, (wh >> 12) & 0x000F000Fu, bo.x, bo.y);
      }
#pragma unroll
      for (int par = 0; par < 2; ++par) {                                 // group jg = 2c + par, held by lane (jg & 3), slot (jg >> 2)
        int const jg = 2 * c + par, src = (lane & ~3) | (jg & 3), slot = jg >> 2;
        float const dlo = __shfl_sync(0xffffffffu, dl_lo[slot], src), mlo = __shfl_sync(0xffffffffu, ml_lo[slot], src);
        float const dhi = __shfl_sync(0xffffffffu, dl_hi[slot], src), mhi = __shfl_sync(0xffffffffu, ml_hi[slot], src);
        float2 const sx = q_ldsf2(sb + uint32_t(jg) * (kQCols * 4));
        float const* cc = par ? co : ce;
        totA[0] = fmaf(dlo, cc[0], totA[0]); totA[1] = fmaf(dlo, cc[1], totA[1]);
        totA[2] = fmaf(dhi, cc[2], totA[2]); totA[3] = fmaf(dhi, cc[3], totA[3]);
        totB[0] = fmaf(mlo, sx.x, totB[0]); totB[1] = fmaf(mlo, sx.y, totB[1]);
        totB[2] = fmaf(mhi, sx.x, totB[2]); totB[3] = fmaf(mhi, sx.y, totB[3]);
      }
    }
    __syncwarp();                                                         // every lane's loads of this tile fed its MMAs
    if (q + STAGES < ntiles) issue(q + STAGES);
  }
  if (ntiles > 0 && !dead) flush(cur_b);
  if (dead)
    for (int i = q + 1; i < ntiles && i < q + STAGES; ++i)
      (void)mbar_wait_bounded(&mybars[i % STAGES], unsigned(i / STAGES) & 1u, nullptr, 0, 250000000ull);
  __syncthreads();
  // ---- every block's contributions, added in warp order (fixed: results do not depend on timing) ------------------------------
  for (int o = threadIdx.x; o < nb_c * kQRows * kQCols; o += blockDim.x) {
    int const bi = o / (kQRows * kQCols), col = (o / kQRows) % kQCols, rr = o % kQRows;
    int const row = (blockIdx.x + bi * gridDim.x) * kQRows + rr;
    if (row >= n || col >= nrows) continue;
    float sum = 0.f;
    // with many blocks per CTA only the warps whose run can touch block bi are visited (a conservative range; the test
    // below is exact); with one or two blocks the two divisions would cost more than the full loop
    int w_lo = 0, w_hi = 15;
    if (nb_c > 2) { w_lo = max(0, (bi * bpr * 16) / T - 1); w_hi = min(15, ((bi + 1) * bpr * 16) / T + 1); }
    for (int w2 = w_lo; w2 <= w_hi; ++w2) {
      int const u0 = ((w2 * T) >> 4), u1 = (((w2 + 1) * T) >> 4);
      if (u1 > u0 && u0 < (bi + 1) * bpr && u1 > bi * bpr) sum += part[(size_t(bi + w2) * kQRows + rr) * kQCols + col];
    }
    a.out[size_t(arow + col) * n + row] = sum;
  }
}

struct Q4MmaPlan { int gx, cpg, stages, ok; size_t smem; };

}  // namespace

// Enqueue; false when the shape is outside this kernel's envelope (the caller then uses another kernel).
bool enqueue_q4k_mma(uint8_t const* blocks, __half const* x, float* out, int const* offsets, int n, int bpr, int experts,
                     int rows, unsigned int* status, cudaStream_t stream) {
  if (n < kQRows || bpr <= 0 || rows <= 0 || !status) return false;
  int const E = offsets ? experts : 1;
  int dev = 0;
  cudaGetDevice(&dev);
  struct Key { int n, bpr, rows, e, dev; bool operator<(Key const& o) const {
    return n != o.n ? n < o.n : bpr != o.bpr ? bpr < o.bpr : rows != o.rows ? rows < o.rows : e != o.e ? e < o.e : dev < o.dev; } };
  static std::map<Key, Q4MmaPlan> plans;
  static std::mutex mu;
  Q4MmaPlan p{};
  {
    std::lock_guard<std::mutex> lk(mu);
    Key const key{n, bpr, rows, offsets ? experts : 0, dev};
    auto it = plans.find(key);
    if (it == plans.end()) {
      int const k = bpr * 256, nblocks = (n + kQRows - 1) / kQRows, sms = rt_sm_count();
      p.ok = 0;
      for (int cpg : {8, 4}) {
        for (int stages : {4, 2}) {
          int const groups = offsets ? std::max(1, std::min(rows, (rows / cpg + std::min(experts, rows) + 1) / 2)) : (rows + cpg - 1) / cpg;
          int const share = std::max(1, sms / std::max(1, std::min(groups, sms)));
          int gx = std::max(1, std::min(nblocks, share));
          int const per = std::min(256, (nblocks + gx - 1) / gx);
          gx = (nblocks + per - 1) / per;
          size_t const smem = 1024 + size_t(16) * stages * kQTile + size_t(cpg) * (size_t(k) * 2 + 32) + size_t(k / 32) * kQCols * 4 +
                              (kQCols + 16) * 4 + size_t(16) * stages * 8 + size_t(per + 16) * kQRows * kQCols * 4;
          if (smem <= 227 * 1024) { p.gx = gx; p.cpg = cpg; p.stages = stages; p.smem = smem; p.ok = 1; break; }
        }
        if (p.ok) break;
      }
      if (p.ok) {
        bool const a1 = cudaFuncSetAttribute(q4k_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess;
        bool const a2 = cudaFuncSetAttribute(q4k_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess;
        if (!a1 || !a2) { (void)cudaGetLastError(); p.ok = 0; }
      }
      it = plans.emplace(key, p).first;
    }
    p = it->second;
  }
  if (!p.ok) return false;
  int const gy = offsets ? std::min(rows, rows / p.cpg + experts) : (rows + p.cpg - 1) / p.cpg;
  if (gy <= 0 || gy > 65535) return false;
  struct MKey { void const* b; int n, bpr, e; bool operator<(MKey const& o) const {
    return b != o.b ? b < o.b : n != o.n ? n < o.n : bpr != o.bpr ? bpr < o.bpr : e < o.e; } };
  static std::map<MKey, CUtensorMap> maps;
  static std::mutex mmu;
  CUtensorMap m;
  {
    std::lock_guard<std::mutex> lk(mmu);
    MKey const key{blocks, n, bpr, E};
    auto it = maps.find(key);
    if (it == maps.end()) {
      if (maps.size() > 4096) maps.clear();
      CUtensorMap nm;
      cuuint64_t const rb = cuuint64_t(bpr) * kQBlock;
      cuuint64_t dims[3] = {rb, cuuint64_t(n), cuuint64_t(E)};
      cuuint64_t str[2] = {rb, rb * n};
      cuuint32_t box[3] = {cuuint32_t(kQBlock), cuuint32_t(kQRows), 1};
      if (!tma_make_map(&nm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, blocks, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return false;
      it = maps.emplace(key, nm).first;
    }
    m = it->second;
  }
  Q4MmaArgs a{};
  a.blocks = blocks; a.x = x; a.out = out; a.offsets = offsets;
  a.n = n; a.bpr = bpr; a.experts = E; a.m_rows = rows; a.cpg = p.cpg; a.nblocks = (n + kQRows - 1) / kQRows;
  a.status = status;
  // Programmatic dependent launch: this kernel may be scheduled while the previous kernel of the stream drains; it reads
  // activations and offsets only after griddepcontrol.wait.  QUACTLIZE_B200_NO_PDL=1 launches it the plain way.
  static bool const no_pdl = std::getenv("QUACTLIZE_B200_NO_PDL") != nullptr;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.gx, gy); cfg.blockDim = dim3(512); cfg.dynamicSmemBytes = p.smem; cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = no_pdl ? 0 : 1;
  cudaError_t const le = p.stages == 4 ? cudaLaunchKernelEx(&cfg, q4k_mma_kernel<4>, m, a) : cudaLaunchKernelEx(&cfg, q4k_mma_kernel<2>, m, a);
  if (le != cudaSuccess) { (void)cudaGetLastError(); return false; }
  return true;
}

}  // namespace qb
