// Dense raw GGUF Q4_K GEMV for 2..8 activation rows: the tensor-core arithmetic of the small-batch kernel on the copy
// structure of the single-row kernel, so that eight rows cost what one row costs -- the weights are streamed once,
// in large contiguous pieces, and the kernel stays bound by that stream.
//
//   out[t, r] = sum_b sum_g ( d_rb*sc_rbg * sum_j q_rbgj x[t, 256b+32g+j]  -  dmin_rb*mn_rbg * sum_j x[t, 256b+32g+j] )
//
// Same contract as the M > 1 arm of the reference's vecdot_rows_kernel (quactlize/include/gguf_vecdot.hpp:604-760).
//
// Work split.  A CTA (16 warps, one per SM) owns a run of consecutive output rows (dealt over the grid in units of eight)
// and walks it in TILES of 16 rows.  K is covered in PASSES of at most 16 superblocks; in a pass warp w owns superblock w
// of every row of the tile.  A stage of the shared-memory ring is one (pass, tile): 16 bulk copies, one per row, each
// the row's contiguous run of this pass's superblocks (2.3 KB at K = 4096), completing on one mbarrier; rows are padded
// apart so the fragment loads of a warp fall on 32 different banks.  Every wait is bounded.
//
// Arithmetic.  mma.sync.m16n8k16: the packed nibbles ARE the A fragments -- (word & 0x000F000F) read as fp16 is two codes
// * 2^-24, (word & 0x00F000F0) two codes * 2^-20 of the neighbouring group -- and the activations of up to eight rows,
// pre-scaled by a power of two per (row, superblock), are the B fragments, held in REGISTERS for the whole pass (32 per
// lane).  The fp32 products of a 32-code group are scaled by d*sc and accumulated; lane t of a quad unpacks the 6-bit
// sub-scales and sub-mins of groups 2t, 2t+1 of its two rows, the quad exchanges d*sc through 512 bytes of shared memory,
// and the sub-mins go through one more MMA (m16n8k8) against the per-group sums of x, split in two fp16 halves so the
// fp32 sums are kept.  A warp keeps its K-slice of every tile of the CTA in its own area of shared memory across the
// passes (registers go to the B fragments); the slices of a row are added in warp order at the end, so results do not
// depend on timing.  The activations of the first pass are requested before the first weight copy: a load requested
// behind the ring's copies is served after them.
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

namespace qb {
namespace {

constexpr int kTileRows = 16;
constexpr int kRWarps = 16;
constexpr int kMaxTiles = 7;             // tiles per CTA (at most 112 rows): bounds the shared memory of the K-slices
constexpr int kCols = 8;                 // the n of the MMA = activation rows per launch

struct RowsArgs {
  uint8_t const* blocks;
  __half const* x;
  float* out;
  int n, bpr, m;                         // output rows, superblocks per row, activation rows (1..8)
  int passes, nbp;                       // K passes; superblocks per pass (<= 16)
  int pitch, stages;                     // bytes between the rows of a staged tile; ring depth
  int units_q, units_r;                  // CTA c owns units_q (+1 if c < units_r) units of eight rows
  unsigned int* status;
};

__device__ __forceinline__ uint2 r_lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 r_lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ float2 r_ldsf2(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ void r_stsf2(uint32_t a, float x, float y) {
  asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(a), "f"(x), "f"(y) : "memory");
}
__device__ __forceinline__ void r_mma16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D = A*B with a zero accumulator: the first MMA of a chain needs no cleared registers
__device__ __forceinline__ void r_mma16z(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void r_mma8z(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
               : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3]) : "r"(a0), "r"(a1), "r"(b0), "f"(0.f));
}
__device__ __forceinline__ void r_mma8(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint4 r_ldg128(uint4 const* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ bool r_try_wait(uint32_t bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __noinline__ bool r_slow_wait(uint32_t bar, unsigned parity, unsigned int* status, unsigned long long limit) {
  unsigned long long t0 = 0;                                    // the clock is first read after 64 failed polls
  unsigned spins = 0;
  while (!r_try_wait(bar, parity)) {
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
__device__ __forceinline__ bool r_wait(uint32_t bar, unsigned parity, unsigned int* status) {
  return r_try_wait(bar, parity) || r_slow_wait(bar, parity, status, kWaitNs);
}

__global__ void __launch_bounds__(kRWarps * 32, 1) q4k_rows_kernel(RowsArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  int const warp = __shfl_sync(0xffffffffu, int(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  int const g = lane >> 2, t = lane & 3;
  int const S = a.stages;
  // ---- this CTA's rows ---------------------------------------------------------------------------------------------------
  int const cx = blockIdx.x;
  int const u0 = cx * a.units_q + min(cx, a.units_r), nu = a.units_q + (cx < a.units_r ? 1 : 0);
  int const row0 = u0 * 8, nrows = min(a.n, row0 + nu * 8) - row0;
  if (nrows <= 0) return;                                                 // uniform, before any barrier
  int const ntiles = (nrows + kTileRows - 1) / kTileRows;
  int const total = ntiles * a.passes;                                    // stages this CTA consumes
  // ---- shared memory: ring | barriers | d*sc exchange ---------------------------------------------------------------------
  uint32_t const s0 = smem_u32(smem);
  uint32_t const stage_bytes = uint32_t(kTileRows) * uint32_t(a.pitch);
  uint32_t const ring32 = s0;
  uint32_t const full32 = ring32 + uint32_t(S) * stage_bytes, empty32 = full32 + 8u * uint32_t(S);
  uint32_t const dl32 = empty32 + 8u * uint32_t(S) + uint32_t(warp) * (kTileRows * 8 * 4);   // [16 rows][8 groups] floats
  uint32_t const red32 = empty32 + 8u * uint32_t(S) + uint32_t(kRWarps) * (kTileRows * 8 * 4);
  size_t const row_stride = size_t(a.bpr) * 144;

  // Under programmatic dependent launch the activations may be the preceding kernel's output: nothing of them is read
  // (and, to keep the order of the stream's memory operations, no weight copy is requested) before this wait.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full32 + 8u * s) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty32 + 8u * s), "r"(kRWarps) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  // stage q = (pass q / ntiles, tile q % ntiles); warp 0 issues it: lane 0 arms the barrier, lane r copies row r
  auto issue = [&](int p, int tl, int s) {
    int const rows_t = min(kTileRows, nrows - tl * kTileRows), nb = min(a.nbp, a.bpr - p * a.nbp);
    unsigned const bytes = unsigned(nb) * 144u;
    uint32_t const bar = full32 + 8u * s;
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(unsigned(rows_t) * bytes) : "memory");
    __syncwarp();
    if (lane < rows_t) {
      uint8_t const* src = a.blocks + size_t(row0 + tl * kTileRows + lane) * row_stride + size_t(p) * a.nbp * 144;
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(ring32 + uint32_t(s) * stage_bytes + uint32_t(lane) * uint32_t(a.pitch)), "l"(src), "r"(bytes), "r"(bar) : "memory");
    }
  };
  int ip = 0, itl = 0;                                                    // (pass, tile) of the next stage to request
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  uint16_t const* xg = reinterpret_cast<uint16_t const*>(a.x) + size_t(g) * (size_t(a.bpr) * 256);   // activation row g = MMA column g
  bool const col_live = g < a.m;
  bool dead = false;
  int q = 0, s = 0, ps = 0;                                                // stage counter; its ring slot; the previous slot
  unsigned par = 0u, ppar = 0u;                                            // ... and their phase parities
  for (int p = 0; p < a.passes && !dead; ++p) {
    int const nb = min(a.nbp, a.bpr - p * a.nbp);
    bool const active = warp < nb;                                         // this warp has a superblock in this pass
    int const blk = p * a.nbp + warp;
    // ---- B fragments of this warp's superblock: eight columns (activation rows), pre-scaled by a power of two per
    // (column, superblock); group sums for the sub-min term ------------------------------------------------------------
    uint32_t xb[4][8];
    uint32_t sx_hi = 0u, sx_lo = 0u;
    float f0 = 0.f, f1 = 0.f;
    {
      // The loads of the activations are requested BEFORE the first weight copies: a load requested behind the ring's
      // copies is served after them (microseconds later).  Volatile so the compiler keeps that order.
      uint4 raw[8];
      float mx = 0.f;
      bool const ld = active && col_live;
      uint4 const* xp = reinterpret_cast<uint4 const*>(xg + size_t(blk) * 256);
      if (ld) {
#pragma unroll
        for (int gr = 0; gr < 8; ++gr) raw[gr] = r_ldg128(xp + gr * 4 + t);   // elements 8t..8t+7 of group gr
      }
      if (p == 0) {
        __syncthreads();                                                   // every warp's loads are requested
        if (warp == 0)
          for (int qq = 0; qq < S && qq < total; ++qq) {
            issue(ip, itl, qq);
            if (++itl == ntiles) { itl = 0; ++ip; }
          }
      }
      // group sums for the sub-min term, from the registers: this lane has eight elements of each of the eight groups;
      // a two-step exchange inside the quad leaves lane t with the whole sums of groups 2t and 2t+1
      float ps[8];
#pragma unroll
      for (int gr = 0; gr < 8; ++gr) {
        ps[gr] = 0.f;
        if (ld) {
          uint32_t const w4[4] = {raw[gr].x, raw[gr].y, raw[gr].z, raw[gr].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 const f = __half22float2(u32_as_h2(w4[j]));
            ps[gr] += f.x + f.y;
            mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
          }
        } else {
          raw[gr] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      {
        bool const up = (t & 2) != 0, odd = (t & 1) != 0;
        float q4[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float const got = __shfl_xor_sync(0xffffffffu, up ? ps[j] : ps[4 + j], 2);
          q4[j] = (up ? ps[4 + j] : ps[j]) + got;
        }
        float const g0 = __shfl_xor_sync(0xffffffffu, odd ? q4[0] : q4[2], 1);
        float const g1 = __shfl_xor_sync(0xffffffffu, odd ? q4[1] : q4[3], 1);
        float const sa = (odd ? q4[2] : q4[0]) + g0, sb = (odd ? q4[3] : q4[1]) + g1;
        __half const ha = __float2half_rn(sa), hb = __float2half_rn(sb);
        sx_hi = h2_as_u32(__halves2half2(ha, hb));
        sx_lo = h2_as_u32(__floats2half2_rn(sa - __half2float(ha), sb - __half2float(hb)));
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      int const ex = pow2_scale_exponent(mx, 15);
      // exact powers of two built from the exponent field (ex is within [-2, 39]); the product is formed in fp32, where
      // the factor itself always fits, and rounded to fp16 once
      float const se = __int_as_float((ex + 127) << 23), so = __int_as_float((ex - 4 + 127) << 23);
      auto scaled = [](uint32_t pr, float sc) {
        float2 const f = __half22float2(u32_as_h2(pr));
        return h2_as_u32(__floats2half2_rn(f.x * sc, f.y * sc));
      };
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int par = 0; par < 2; ++par) {
          uint4 const v = raw[2 * c + par];
          float const sc = par ? so : se;
          // (h0 h1)(h2 h3)(h4 h5)(h6 h7) -> (h0 h2)(h1 h3)(h4 h6)(h5 h7): the order the nibble masks deliver codes
          xb[c][4 * par + 0] = scaled(__byte_perm(v.x, v.y, 0x5410), sc);
          xb[c][4 * par + 1] = scaled(__byte_perm(v.x, v.y, 0x7632), sc);
          xb[c][4 * par + 2] = scaled(__byte_perm(v.z, v.w, 0x5410), sc);
          xb[c][4 * par + 3] = scaled(__byte_perm(v.z, v.w, 0x7632), sc);
        }
      }
      // accumulator columns of this lane are 2t, 2t+1: their factors 2^(24 - ex) live in the lanes whose g is that column
      float const fm = __int_as_float((24 - ex + 127) << 23);
      f0 = __shfl_sync(0xffffffffu, fm, 8 * t);
      f1 = __shfl_sync(0xffffffffu, fm, 8 * t + 4);
    }
    // ---- the tiles of this pass ---------------------------------------------------------------------------------------
    // The body appears once (unrolled over the tiles it would not fit the instruction cache); the accumulator set of the
    // tile is picked by a switch at the end, so the sets stay in registers.
#pragma unroll 1
    for (int tl = 0; tl < ntiles; ++tl) {
      if (dead) break;                                                     // uniform for the warp
      if (warp == 0 && q >= 1 && ip < a.passes) {                          // refill the slot the CTA finished one stage ago
        if (!r_wait(empty32 + 8u * ps, ppar, a.status)) dead = true;
        else {
          issue(ip, itl, ps);
          if (++itl == ntiles) { itl = 0; ++ip; }
        }
      }
      dead = __shfl_sync(0xffffffffu, int(dead), 0) != 0;
      if (!dead && !r_wait(full32 + 8u * s, par, a.status)) dead = true;
      dead = __any_sync(0xffffffffu, dead);
      if (dead) break;
      if (active) {
        uint32_t const lo_a = ring32 + uint32_t(s) * stage_bytes + uint32_t(g) * uint32_t(a.pitch) + uint32_t(warp) * 144u;
        uint32_t const hi_a = lo_a + 8u * uint32_t(a.pitch);
        uint4 const hl = r_lds128(lo_a), hh = r_lds128(hi_a);             // d|dmin, 12 scale bytes, of rows g and g+8
        // lane t unpacks groups 2t, 2t+1 (half t >> 1 of the block: two different bit layouts, selected by masks)
        uint32_t const ma = (t & 2) ? 0x0F0F0F0Fu : 0x3F3F3F3Fu, mb = (t & 2) ? 0x30303030u : 0u;
        int const sh = 16 * (t & 1);
        uint32_t const scl = ((((t & 2) ? hl.w : hl.y) & ma) | ((hl.y >> 2) & mb)) >> sh;
        uint32_t const mnl = ((((t & 2) ? (hl.w >> 4) : hl.z) & ma) | ((hl.z >> 2) & mb)) >> sh;
        uint32_t const sch = ((((t & 2) ? hh.w : hh.y) & ma) | ((hh.y >> 2) & mb)) >> sh;
        uint32_t const mnh = ((((t & 2) ? (hh.w >> 4) : hh.z) & ma) | ((hh.z >> 2) & mb)) >> sh;
        float2 const ddl = __half22float2(u32_as_h2(hl.x)), ddh = __half22float2(u32_as_h2(hh.x));
        // byte -> float without a conversion instruction: 2^23 + b, minus 2^23
        auto b2f = [](uint32_t b) { return __uint_as_float(0x4B000000u | b) - 8388608.f; };
        r_stsf2(dl32 + uint32_t((g * 8 + 2 * t) * 4), ddl.x * b2f(scl & 0xFFu), ddl.x * b2f((scl >> 8) & 0xFFu));
        r_stsf2(dl32 + uint32_t(((g + 8) * 8 + 2 * t) * 4), ddh.x * b2f(sch & 0xFFu), ddh.x * b2f((sch >> 8) & 0xFFu));
        __half2 const k1024 = __float2half2_rn(1024.f);
        uint32_t const am0 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(mnl, 0x64646464u, 0x4140)), k1024));   // (mn[2t], mn[2t+1]) of row g
        uint32_t const am1 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(mnh, 0x64646464u, 0x4140)), k1024));   // ... of row g+8
        __syncwarp();
        float bacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4; c += 2) {
          // d*sc of groups 2c .. 2c+3 of both rows: one 16-byte load each
          uint4 const dlo4 = r_lds128(dl32 + uint32_t((g * 8 + 2 * c) * 4)), dhi4 = r_lds128(dl32 + uint32_t(((g + 8) * 8 + 2 * c) * 4));
          float const dlo[4] = {__uint_as_float(dlo4.x), __uint_as_float(dlo4.y), __uint_as_float(dlo4.z), __uint_as_float(dlo4.w)};
          float const dhi[4] = {__uint_as_float(dhi4.x), __uint_as_float(dhi4.y), __uint_as_float(dhi4.z), __uint_as_float(dhi4.w)};
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            int const ch = c + cc;
            uint2 const wl = r_lds64(lo_a + 16u + 32u * ch + 8u * t), wh = r_lds64(hi_a + 16u + 32u * ch + 8u * t);
            float ce[4], co[4];
            uint32_t const l0 = wl.x, l1 = wl.y, h0 = wh.x, h1 = wh.y;
            uint32_t const l0s = l0 >> 8, l1s = l1 >> 8, h0s = h0 >> 8, h1s = h1 >> 8;
            r_mma16z(ce, l0 & 0x000F000Fu, h0 & 0x000F000Fu, l0s & 0x000F000Fu, h0s & 0x000F000Fu, xb[ch][0], xb[ch][1]);
            r_mma16z(co, l0 & 0x00F000F0u, h0 & 0x00F000F0u, l0s & 0x00F000F0u, h0s & 0x00F000F0u, xb[ch][4], xb[ch][5]);
            r_mma16(ce, l1 & 0x000F000Fu, h1 & 0x000F000Fu, l1s & 0x000F000Fu, h1s & 0x000F000Fu, xb[ch][2], xb[ch][3]);
            r_mma16(co, l1 & 0x00F000F0u, h1 & 0x00F000F0u, l1s & 0x00F000F0u, h1s & 0x00F000F0u, xb[ch][6], xb[ch][7]);
            bacc[0] = fmaf(dlo[2 * cc], ce[0], bacc[0]); bacc[1] = fmaf(dlo[2 * cc], ce[1], bacc[1]);
            bacc[2] = fmaf(dhi[2 * cc], ce[2], bacc[2]); bacc[3] = fmaf(dhi[2 * cc], ce[3], bacc[3]);
            bacc[0] = fmaf(dlo[2 * cc + 1], co[0], bacc[0]); bacc[1] = fmaf(dlo[2 * cc + 1], co[1], bacc[1]);
            bacc[2] = fmaf(dhi[2 * cc + 1], co[2], bacc[2]); bacc[3] = fmaf(dhi[2 * cc + 1], co[3], bacc[3]);
          }
        }
        float cm[4];                                                      // sum over groups of mn * sum(x)
        r_mma8z(cm, am0, am1, sx_hi);
        r_mma8(cm, am0, am1, sx_lo);
        float const r0 = fmaf(f0, bacc[0], -ddl.y * cm[0]), r1 = fmaf(f1, bacc[1], -ddl.y * cm[1]);
        float const r2 = fmaf(f0, bacc[2], -ddh.y * cm[2]), r3 = fmaf(f1, bacc[3], -ddh.y * cm[3]);
        // this warp's K-slice of the tile: kept in shared memory across the passes (its own area: no other warp touches it)
        uint32_t const ra = red32 + uint32_t(((warp * ntiles + tl) * kTileRows + g) * kCols + 2 * t) * 4u;
        if (p == 0) {
          r_stsf2(ra, r0, r1);
          r_stsf2(ra + 8u * kCols * 4u, r2, r3);
        } else {
          float2 const o0 = r_ldsf2(ra), o1 = r_ldsf2(ra + 8u * kCols * 4u);
          r_stsf2(ra, o0.x + r0, o0.y + r1);
          r_stsf2(ra + 8u * kCols * 4u, o1.x + r2, o1.y + r3);
        }
      }
      __syncwarp();                                                        // every lane's reads of the stage are done
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty32 + 8u * s) : "memory");
      ++q;
      ps = s; ppar = par;
      if (++s == S) { s = 0; par ^= 1u; }
    }
  }
  if (dead) {
    // a wait gave up: let the copies still in flight land (bounded, short) before the shared memory is handed on
    if (threadIdx.x == 0)
      for (int s = 0; s < S; ++s) { (void)r_try_wait(full32 + 8u * s, 0) ; (void)r_slow_wait(full32 + 8u * s, 0, nullptr, 100000000ull); }
  }
  __syncthreads();
  if (dead) return;
  // ---- the K-slices of every (row, column), added in warp order ----------------------------------------------------------
  float const* red = reinterpret_cast<float const*>(smem + (red32 - s0));   // [warp][tile][16 rows][8 cols]
  for (int o = threadIdx.x; o < ntiles * kTileRows * kCols; o += blockDim.x) {
    int const col = o / (ntiles * kTileRows), rr = o % (ntiles * kTileRows);  // consecutive threads -> consecutive output rows
    if (rr >= nrows || col >= a.m) continue;
    float sum = 0.f;
    for (int w = 0; w < a.nbp; ++w) sum += red[(size_t(w) * ntiles * kTileRows + rr) * kCols + col];   // warps >= nbp never had a superblock
    a.out[size_t(col) * a.n + row0 + rr] = sum;
  }
}

struct RowsPlan { int gx, passes, nbp, pitch, stages, units_q, units_r, ok; size_t smem; };

}  // namespace

// Enqueue; false when the shape is outside this kernel's envelope (the caller then uses another kernel).
bool enqueue_q4k_rows(uint8_t const* blocks, __half const* x, float* out, int n, int bpr, int rows, unsigned int* status,
                      cudaStream_t stream) {
  if (n <= 0 || bpr <= 0 || rows <= 0 || rows > kCols || !status) return false;
  if ((reinterpret_cast<uintptr_t>(blocks) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return false;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); return false; }
  struct Key { int n, bpr, dev; bool operator<(Key const& o) const { return n != o.n ? n < o.n : bpr != o.bpr ? bpr < o.bpr : dev < o.dev; } };
  static std::map<Key, RowsPlan> plans;
  static std::mutex mu;
  RowsPlan p{};
  {
    std::lock_guard<std::mutex> lk(mu);
    Key const key{n, bpr, dev};
    auto it = plans.find(key);
    if (it == plans.end()) {
      int const sms = rt_sm_count();
      p.passes = (bpr + kRWarps - 1) / kRWarps;
      p.nbp = (bpr + p.passes - 1) / p.passes;
      // rows of a staged tile sit pitch bytes apart with (pitch / 4) % 32 == 8: an 8-byte fragment load is served half a
      // warp at a time (rows g = 0..3 or 4..7, four lanes of 8 bytes each), and those four rows then tile the 32 banks
      int const words = p.nbp * 36;
      p.pitch = (words + ((8 - words % 32) + 32) % 32) * 4;
      int const units = (n + 7) / 8;
      p.gx = std::max(std::min(sms, units), (units + (kMaxTiles * 2) - 1) / (kMaxTiles * 2));
      p.units_q = units / p.gx; p.units_r = units % p.gx;
      int const max_rows = (p.units_q + (p.units_r ? 1 : 0)) * 8;
      int const tiles = (max_rows + kTileRows - 1) / kTileRows;
      size_t const stage = size_t(kTileRows) * p.pitch;
      size_t const fixed = size_t(kRWarps) * kTileRows * 8 * 4 + size_t(kRWarps) * tiles * kTileRows * kCols * 4 + 128;
      p.stages = fixed + 2 * (stage + 16) <= 227 * 1024 ? int(std::min<size_t>(6, (227 * 1024 - fixed) / (stage + 16))) : 0;
      p.smem = size_t(p.stages) * (stage + 16) + fixed;
      p.ok = tiles <= kMaxTiles && p.stages >= 2 && p.smem <= 227 * 1024 && p.pitch % 16 == 0;
      if (p.ok && cudaFuncSetAttribute(q4k_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
        (void)cudaGetLastError();
        p.ok = 0;
      }
      it = plans.emplace(key, p).first;
    }
    p = it->second;
  }
  if (!p.ok) return false;
  RowsArgs a{};
  a.blocks = blocks; a.x = x; a.out = out; a.n = n; a.bpr = bpr; a.m = rows;
  a.passes = p.passes; a.nbp = p.nbp; a.pitch = p.pitch; a.stages = p.stages; a.units_q = p.units_q; a.units_r = p.units_r;
  a.status = status;
  static bool const no_pdl = std::getenv("QUACTLIZE_B200_NO_PDL") != nullptr;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.gx); cfg.blockDim = dim3(kRWarps * 32); cfg.dynamicSmemBytes = p.smem; cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = no_pdl ? 0 : 1;
  if (cudaLaunchKernelEx(&cfg, q4k_rows_kernel, a) != cudaSuccess) { (void)cudaGetLastError(); return false; }
  return true;
}

}  // namespace qb
