// Q4_K decode GEMV, one activation row per (expert, row) -- the headline kernel.
//
//   out[t, r] = sum_k x[t, k] * W[r, k],   W = raw Q4_K blocks [E][n][k/256][144] row-major by output row.
//
// Same contract as vecdot_rows_kernel of the reference (quactlize/include/gguf_vecdot.hpp:604-760, launch policy
// quactlize/csrc/device/ppu_backend.cu:52-131) for Q4_K with a shared activation.
//
// Structure (sm_100a):
//   prologue, once per CTA  the activation vector is scaled by one power of two, laid out in the order the nibble bit
//                           tricks emit codes, and parked in shared memory together with the per-group sums of x;
//                           every lane then pulls its 64 half2 registers with 16 conflict-free LDS.128.  The
//                           activation loads are issued BEFORE the weight copies so they are not queued behind them.
//   main loop, per warp     a warp owns (output row, K segment of <= 16 blocks); row segments arrive by cp.async.bulk
//                           into a private ring of STAGES buffers (mbarrier completion, bounded waits); two lanes
//                           share a block: 1 header LDS.128 + 4 code LDS.128 per lane per row.
//   arithmetic              (w & 0x000F000F) reinterpreted as half2 IS (q0, q2) * 2^-24 (fp16 subnormals); 5 integer +
//                           4 HFMA2 per 8 weights; the 6-bit sub-scales are applied in the fp16 domain as exact
//                           integers (1024+sc magic), one fp32 flush per lane per block; mins use the per-group sums.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <map>
#include <mutex>

#include "qb_device.cuh"
#include "qb_runtime.hpp"

namespace qb {

struct Q4Args {
  uint8_t const* blocks;
  __half const* x;
  float* out;
  int const* offsets;        // cumulative [experts+1] (grouped) or nullptr (dense)
  int n, bpr, max_rows;      // grid.y = activation rows (dense) or experts*max_rows (grouped)
  int S, nbs, RS, iters;     // K segments per row, blocks per segment, row slots per CTA, rows per slot
  int rows_q, rows_r;        // n = gridDim.x*rows_q + rows_r: CTA c owns rows_q (+1 if c < rows_r) consecutive rows
  unsigned int* status;
  // A second matrix of the same K that shares the activation row (dense only): output rows n_first .. n-1 are its rows
  // 0 .. n - n_first - 1 and go to out2.  nullptr: one matrix (n_first == n).
  uint8_t const* blocks2;
  float* out2;
  int n_first;
};

__device__ __forceinline__ uint4 lds128_a(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts64_a(uint32_t addr, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ bool try_wait_a(uint32_t bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __noinline__ bool slow_wait_a(uint32_t bar, unsigned parity, unsigned int* status, unsigned long long limit) {
  unsigned long long t0 = 0;                                    // the clock is first read after 64 failed polls
  unsigned spins = 0;
  while (!try_wait_a(bar, parity)) {
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
__device__ __forceinline__ void issue_copy_a(uint32_t dst, void const* src, unsigned bytes, uint32_t bar) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

constexpr int kQ4MaxPieces = 4;      // 16-byte activation pieces per thread in the prologue (K <= 16384 at 512+ threads)
#ifndef QB_Q4_WARPS
#define QB_Q4_WARPS 16
#endif
constexpr int kQ4Warps = QB_Q4_WARPS;         // warps per CTA (one CTA per SM); bounded by registers: 65536 / (32 * regs)

// One lane's share (half a block: four groups, 128 weights) of one output row.  `base` is the shared address of the
// lane's block, `code` of its 64 code bytes.
__device__ __forceinline__ float q4k_half_block_dot(uint32_t base, uint32_t code, __half2 const (&xr)[4][16],
                                                    float const (&sxg)[4], int prt, uint32_t mask_a, uint32_t mask_b,
                                                    float fm) {
  uint4 const hdr = lds128_a(base);
  // groups 0-3 (prt 0): the low six bits of scale bytes 0-3 / 4-7; groups 4-7 (prt 1): nibbles of bytes 8-11 plus the
  // top two bits of bytes 0-3 / 4-7.  Both forms are  (A & ma) | ((B >> 2) & mb)  with per-lane constants.
#if defined(QB_ABL_NOHDR)
  uint32_t const sc4 = hdr.y, mn4 = hdr.z;
#else
  uint32_t const sA = prt ? hdr.w : hdr.y, mA = prt ? (hdr.w >> 4) : hdr.z;
  uint32_t const sc4 = (sA & mask_a) | ((hdr.y >> 2) & mask_b);
  uint32_t const mn4 = (mA & mask_a) | ((hdr.z >> 2) & mask_b);
#endif
  __half2 const k1024 = __float2half2_rn(1024.f);
  __half2 sch[4];                                               // the four sub-scales as exact fp16 integers, broadcast
  sch[0] = __hsub2(u32_as_h2(__byte_perm(sc4, 0x64646464u, 0x4040)), k1024);
  sch[1] = __hsub2(u32_as_h2(__byte_perm(sc4, 0x64646464u, 0x4141)), k1024);
  sch[2] = __hsub2(u32_as_h2(__byte_perm(sc4, 0x64646464u, 0x4242)), k1024);
  sch[3] = __hsub2(u32_as_h2(__byte_perm(sc4, 0x64646464u, 0x4343)), k1024);
  float dsum = 0.f;
  __half2 pair;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 const qv = lds128_a(code + 16u * c);
    uint32_t const qw[4] = {qv.x, qv.y, qv.z, qv.w};
    __half2 alo, ahi;
#if defined(QB_ABL_NOCORE)
    alo = u32_as_h2((qw[0] ^ qw[1]) & 0x03FF03FFu); ahi = u32_as_h2((qw[2] ^ qw[3]) & 0x03FF03FFu);
#else
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      uint32_t const w = qw[wi], w8 = w >> 8;
      if (wi == 0) {
        alo = __hmul2(u32_as_h2(w & 0x000F000Fu), xr[c][0]);
        ahi = __hmul2(u32_as_h2(w & 0x00F000F0u), xr[c][2]);
      } else {
        alo = __hfma2(u32_as_h2(w & 0x000F000Fu), xr[c][4 * wi + 0], alo);
        ahi = __hfma2(u32_as_h2(w & 0x00F000F0u), xr[c][4 * wi + 2], ahi);
      }
      alo = __hfma2(u32_as_h2(w8 & 0x000F000Fu), xr[c][4 * wi + 1], alo);
      ahi = __hfma2(u32_as_h2(w8 & 0x00F000F0u), xr[c][4 * wi + 3], ahi);
    }
#endif
    // chunks 2j and 2j+1 cover the same two groups: scale in fp16, one fp32 flush per chunk pair
    if ((c & 1) == 0) pair = __hfma2(ahi, sch[c + 1], __hmul2(alo, sch[c]));
    else dsum += h2_sum(__hfma2(ahi, sch[c], __hfma2(alo, sch[c - 1], pair)));
  }
#if defined(QB_ABL_NOMIN)
  return __low2float(u32_as_h2(hdr.x)) * fm * dsum;
#endif
  float2 const dd = __half22float2(u32_as_h2(hdr.x));           // (d, dmin)
  float2 const m01 = bytes_to_f2(mn4, 0x4140), m23 = bytes_to_f2(mn4, 0x4342);   // mins * 2^-24
  float const msum = fmaf(m01.x, sxg[0], fmaf(m01.y, sxg[1], fmaf(m23.x, sxg[2], m23.y * sxg[3])));
  return fmaf(dd.x * fm, dsum, -(dd.y * 16777216.f) * msum);
}

template <int STAGES>
__global__ void __launch_bounds__(kQ4Warps * 32, 1) q4k_gemv1_kernel(Q4Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  // the warp index is broadcast from lane 0 so the compiler keeps everything derived from it in uniform registers
  int const T = blockDim.x, W = T >> 5, warp = __shfl_sync(0xffffffffu, int(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  int const seg = warp % a.S, rslot = warp / a.S;
  int e = 0, arow;
  // Under programmatic dependent launch the offsets and the activation may be the preceding kernel's output: nothing
  // of them is read before this wait (it also precedes the early return of surplus CTAs).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (a.offsets) {
    e = blockIdx.y / a.max_rows;
    int const r = blockIdx.y % a.max_rows, r0 = a.offsets[e], r1 = a.offsets[e + 1];
    if (r >= r1 - r0) return;                                   // uniform for the CTA
    arow = r0 + r;
  } else {
    arow = blockIdx.y;
  }
#if defined(QB_ABL_EMPTY)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0 && blockIdx.x == 0) a.out[0] = 1.f;
  return;
#endif
  int const bpr = a.bpr, k = bpr * 256;
  // shared memory map
  uint32_t const s0 = smem_u32(smem);
  uint32_t const xa32 = s0;                                     // arranged activations, k*2 bytes
  uint32_t const sx32 = xa32 + uint32_t(k) * 2u;                // per-group sums, bpr*8 floats
  uint32_t const red32 = sx32 + uint32_t(bpr) * 32u;            // 32 floats of reduction scratch
  int const seg_bytes = a.nbs * 144, stage_bytes = 2 * seg_bytes;   // a stage holds the segments of two rows
  uint32_t const ring32 = red32 + 128u + uint32_t(warp) * STAGES * stage_bytes;
  uint32_t const bar32 = red32 + 128u + uint32_t(W) * STAGES * stage_bytes + uint32_t(warp) * STAGES * 8u;
  uint32_t const part32 = red32 + 128u + uint32_t(W) * STAGES * (stage_bytes + 8);
  float* red = reinterpret_cast<float*>(smem + (red32 - s0));
  float* part = reinterpret_cast<float*>(smem + (part32 - s0));

  // ---- 1. activation pieces -> registers, issued BEFORE the weight copies so they do not queue behind them.
  int const npieces = k >> 3;
  uint4 const* xg = reinterpret_cast<uint4 const*>(a.x + size_t(arow) * k);
  uint4 pc[kQ4MaxPieces];
#pragma unroll
  for (int j = 0; j < kQ4MaxPieces; ++j) {
    int const p = threadIdx.x + j * T;
    pc[j] = p < npieces ? __ldg(xg + p) : make_uint4(0, 0, 0, 0);
  }

  // ---- 2. weight ring: barriers and the first STAGES row pairs --------------------------------------------------------
  // output rows are split evenly over the grid (CTA row counts differ by at most one); a warp takes PAIRS of rows
  // round-robin, so the per-row bookkeeping (wait, issue, reduce) is paid once per two rows
  int const nb_seg = min(a.nbs, bpr - seg * a.nbs);
  int const cx = blockIdx.x;
  int const row0 = cx * a.rows_q + min(cx, a.rows_r);
  int const nrows = a.rows_q + (cx < a.rows_r ? 1 : 0);
  int const npairs = (nrows + 1) >> 1;
  size_t const row_stride = size_t(bpr) * 144;
  unsigned const copy_bytes = unsigned(nb_seg) * 144u;
  bool const contiguous = a.S == 1;                              // a whole row per segment: the two rows are adjacent
  // Row pairs are not dealt to the warps in advance beyond the first STAGES: a warp that has finished a stage claims the
  // next unclaimed pair of its K segment from a shared counter, so the 48.4 pairs of a CTA (14336 rows over 148 CTAs) do not
  // cost the four rounds of the warps that would own four of them while the others own three.  Which warp computes a row
  // does not change the row's arithmetic, so results do not depend on the claiming order.
  static_assert(STAGES == 2, "the claim bookkeeping below keeps two pairs per warp");
  size_t const seg_off = size_t(seg) * a.nbs * 144;
  // the row's segment in memory: rows of the first matrix (of expert e), then, for a two-matrix launch, of the second
  auto row_src = [&](int grow) -> uint8_t const* {
    return grow < a.n_first ? a.blocks + (size_t(e) * a.n_first + size_t(grow)) * row_stride + seg_off
                            : a.blocks2 + size_t(grow - a.n_first) * row_stride + seg_off;
  };
  auto issue_pair = [&](int pair, uint32_t dst, uint32_t bar) {
    int const grow = row0 + 2 * pair;
    uint8_t const* src = row_src(grow);
    bool const two = 2 * pair + 1 < nrows;
    bool const adjacent = grow + 1 != a.n_first;                 // a pair that straddles the two matrices is two copies
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(two ? 2u * copy_bytes : copy_bytes) : "memory");
    if (two && contiguous && adjacent) {
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(dst), "l"(src), "r"(2u * copy_bytes), "r"(bar) : "memory");
    } else {
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(dst), "l"(src), "r"(copy_bytes), "r"(bar) : "memory");
      if (two)
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(dst + uint32_t(seg_bytes)), "l"(adjacent ? src + row_stride : row_src(grow + 1)), "r"(copy_bytes), "r"(bar) : "memory");
    }
  };
  int* claim = reinterpret_cast<int*>(red) + 16;                 // [S] next unclaimed pair per K segment (S <= 16)
  if (int(threadIdx.x) < a.S) claim[threadIdx.x] = STAGES * a.RS;   // visible after the prologue's barriers, long before the first claim
  int cur = rslot < npairs ? rslot : -1;                         // pair held by the stage consumed next
  int nxt = rslot + a.RS < npairs ? rslot + a.RS : -1;           // ... and by the other stage
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar32 + 8u * s) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (cur >= 0) issue_pair(cur, ring32, bar32);
    if (nxt >= 0) issue_pair(nxt, ring32 + stage_bytes, bar32 + 8u);
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // ---- 3. CTA-wide max|x| -> power-of-two scale ---------------------------------------------------------------------
  __half2 m2 = __float2half2_rn(0.f);
#pragma unroll
  for (int j = 0; j < kQ4MaxPieces; ++j) {
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
  // exact powers of two built from the exponent field (ex is within [-2, 39])
  float const sc_lo = __int_as_float((ex + 127) << 23), sc_hi = __int_as_float((ex - 4 + 127) << 23);
  float const fm = __int_as_float((24 - ex + 127) << 23);

  // ---- 4. arranged, scaled activations and group sums -> shared memory ----------------------------------------------
  // piece p covers elements 8p..8p+7: block b, group g, offset j0 in the group.  Its first four elements belong to
  // code word wi0 of chunk ci = 2*(g/2) + j0/16, its last four to word wi0+1; even groups ride the low nibbles (bytes
  // 0-7 of the 16-byte item), odd groups the high nibbles (bytes 8-15, scaled by a further 2^-4).
#pragma unroll
  for (int j = 0; j < kQ4MaxPieces; ++j) {
    if (j * T >= npieces) break;                                 // uniform for the CTA
    int const p = threadIdx.x + j * T;
    bool const valid = p < npieces;                              // whole warps are valid or not (npieces % 32 == 0)
    uint32_t const* v = reinterpret_cast<uint32_t const*>(&pc[j]);
    float2 const f0 = __half22float2(u32_as_h2(v[0])), f1 = __half22float2(u32_as_h2(v[1]));
    float2 const f2 = __half22float2(u32_as_h2(v[2])), f3 = __half22float2(u32_as_h2(v[3]));
    float gsum = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
    gsum += __shfl_xor_sync(0xffffffffu, gsum, 1);
    gsum += __shfl_xor_sync(0xffffffffu, gsum, 2);
    if (valid) {
      int const b = p >> 5, g = (p >> 2) & 7, j0 = (p & 3) * 8;
      int const ci = 2 * (g >> 1) + (j0 >> 4), prt = ci >> 2, c = ci & 3, wi0 = (j0 & 15) >> 2;
      float const s = (g & 1) ? sc_hi : sc_lo;
      uint32_t const w0a = h2_as_u32(__floats2half2_rn(f0.x * s, f1.x * s)), w0b = h2_as_u32(__floats2half2_rn(f0.y * s, f1.y * s));
      uint32_t const w1a = h2_as_u32(__floats2half2_rn(f2.x * s, f3.x * s)), w1b = h2_as_u32(__floats2half2_rn(f2.y * s, f3.y * s));
      uint32_t const item0 = xa32 + uint32_t((((c * 4 + wi0) * bpr + b) * 2 + prt) * 16 + (g & 1) * 8);
      sts64_a(item0, w0a, w0b);
      sts64_a(item0 + uint32_t(bpr) * 32u, w1a, w1b);             // word wi0+1: items are bpr*2*16 bytes apart
      if ((p & 3) == 0) reinterpret_cast<float*>(smem + (sx32 - s0))[p >> 2] = gsum;
    }
  }
  __syncthreads();

  // ---- 5. this lane's activation registers ---------------------------------------------------------------------------
  int const blk = lane >> 1, prt = lane & 1;
  bool const active = blk < nb_seg;
  int const b_in_row = seg * a.nbs + blk;
  __half2 xr[4][16];       // [chunk][4*word + {lo(e0,e2), lo(e1,e3), hi(e0,e2), hi(e1,e3)}]
  float sxg[4];            // sums of x over the lane's four groups (4*prt .. 4*prt+3)
  if (active) {
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {
        uint4 const v = lds128_a(xa32 + uint32_t((((c * 4 + wi) * bpr + b_in_row) * 2 + prt) * 16));
        xr[c][4 * wi + 0] = u32_as_h2(v.x); xr[c][4 * wi + 1] = u32_as_h2(v.y);
        xr[c][4 * wi + 2] = u32_as_h2(v.z); xr[c][4 * wi + 3] = u32_as_h2(v.w);
      }
    uint4 const sv = lds128_a(sx32 + uint32_t((b_in_row * 8 + 4 * prt) * 4));
    sxg[0] = __uint_as_float(sv.x); sxg[1] = __uint_as_float(sv.y); sxg[2] = __uint_as_float(sv.z); sxg[3] = __uint_as_float(sv.w);
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
      for (int q = 0; q < 16; ++q) xr[c][q] = __float2half2_rn(0.f);
    sxg[0] = sxg[1] = sxg[2] = sxg[3] = 0.f;
  }

  // ---- 6. main loop: one stage = the segments of two consecutive rows -------------------------------------------------
  uint32_t const lane_off = uint32_t(blk) * 144u;
  uint32_t const code_off = lane_off + 16u + uint32_t(prt) * 64u;
  uint32_t const mask_a = prt ? 0x0F0F0F0Fu : 0x3F3F3F3Fu, mask_b = prt ? 0x30303030u : 0u;
  uint32_t st_addr = ring32, st_bar = bar32;
  unsigned phase = 0;
  int st = 0;
  // The loop body is branch-free apart from the wait and the single-lane claim and refill: lanes without a block and the
  // missing second row of an odd tail compute on whatever the buffer holds and are masked at the end, and the warp
  // reduction of pair i-1 is carried into iteration i so its shuffle latency hides under the next pair's arithmetic.
  float p0 = 0.f, p1 = 0.f;                                      // previous pair's per-lane partial sums
  int plr = nrows;                                               // ... and its CTA-local row (nrows = scratch slot)
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
    if (!try_wait_a(st_bar, phase) && !slow_wait_a(st_bar, phase, a.status, kWaitNs)) { gave_up = true; break; }
#if defined(QB_ABL_NOCOMPUTE)
    float t0 = __uint_as_float(lds128_a(st_addr + lane_off).x & 0x3FFFFFFFu), t1 = 0.f;
#else
    float t0 = q4k_half_block_dot(st_addr + lane_off, st_addr + code_off, xr, sxg, prt, mask_a, mask_b, fm);
    float t1 = q4k_half_block_dot(st_addr + seg_bytes + lane_off, st_addr + seg_bytes + code_off, xr, sxg, prt, mask_a, mask_b, fm);
#endif
    reduce_store(p0, p1, plr);
    int const lr = 2 * cur;                                      // CTA-local row of the pair's first row
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
    if (++st == STAGES) { st = 0; st_addr = ring32; st_bar = bar32; phase ^= 1u; }
  }
  reduce_store(p0, p1, plr);
  if (gave_up && nxt >= 0) {
    // a wait gave up: drain this warp's other copy still in flight (bounded, short) before the shared memory can be handed
    // to another CTA
    uint32_t const ob = st == 0 ? bar32 + 8u : bar32;
    unsigned const op = st == 0 ? phase : (phase ^ 1u);
    if (!try_wait_a(ob, op)) (void)slow_wait_a(ob, op, nullptr, 250000000ull);
  }
  __syncthreads();
  for (int r = threadIdx.x; r < nrows; r += T) {
    float s = 0.f;
    for (int sg = 0; sg < a.S; ++sg) s += part[r * a.S + sg];
    int const grow = row0 + r;
    if (grow < a.n_first) a.out[size_t(arow) * a.n_first + grow] = s;
    else a.out2[size_t(arow) * (a.n - a.n_first) + (grow - a.n_first)] = s;
  }
}

namespace {
struct Q4Plan1 { int S, nbs, RS, iters, gx, W; size_t smem; bool ok; };
constexpr int kStages1 = 2;          // x two rows per stage, 16 warps per SM

Q4Plan1 const& q4k_plan1(int n, int bpr, int gy) {
  struct Key { int n, bpr, gy, dev; bool operator<(Key const& o) const {
    return n != o.n ? n < o.n : bpr != o.bpr ? bpr < o.bpr : gy != o.gy ? gy < o.gy : dev < o.dev; } };
  static std::map<Key, Q4Plan1> cache;
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(mu);
  Key const key{n, bpr, gy, dev};
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  Q4Plan1 p{};
  auto kern = q4k_gemv1_kernel<kStages1>;
  p.S = (bpr + 15) / 16;
  p.ok = p.S <= kQ4Warps;
  if (p.ok) {
    p.nbs = (bpr + p.S - 1) / p.S;
    p.RS = std::max(1, kQ4Warps / p.S);   // one CTA per SM shares a single activation prologue
    p.W = p.S * p.RS;
    if (p.W * 32 * kQ4MaxPieces * 8 < bpr * 256) p.ok = false;
    size_t const fixed = size_t(bpr) * 512 + size_t(bpr) * 32 + 128 + size_t(p.W) * kStages1 * (2 * p.nbs * 144 + 8);
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    int const sms = rt_sm_count();
    // grid.x = the CTAs that are resident at once (never more than one row slot per warp needs), rows split evenly
    size_t smem = fixed + 8 * size_t(p.RS) * p.S;
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, p.W * 32, smem + 4096) != cudaSuccess || occ < 1) occ = 1;
    int const resident = std::max(1, occ * sms / std::max(1, std::min(gy, 8)));
    p.gx = std::max(1, std::min(resident, (n + p.RS - 1) / p.RS));
    p.iters = ((n + p.gx - 1) / p.gx + p.RS - 1) / p.RS;          // rows per slot in the largest CTA
    p.smem = fixed + size_t((n + p.gx - 1) / p.gx + 4) * p.S * 4;
    if (p.smem > 227 * 1024) p.ok = false;
  }
  return cache.emplace(key, p).first->second;
}
}  // namespace

// Enqueue; false when the shape is outside this kernel's envelope (the caller then uses another kernel).
bool enqueue_q4k_gemv1(uint8_t const* blocks, __half const* x, float* out, int const* offsets, int n, int bpr,
                       int experts, int rows, int max_rows, unsigned int* status, cudaStream_t stream) {
  int const gy = offsets ? experts * max_rows : rows;
  if (gy <= 0 || gy > 65535) return false;
  Q4Plan1 const& p = q4k_plan1(n, bpr, gy);
  if (!p.ok) return false;
  Q4Args a{};
  a.blocks = blocks; a.x = x; a.out = out; a.offsets = offsets;
  a.n = n; a.bpr = bpr; a.max_rows = max_rows;
  a.blocks2 = nullptr; a.out2 = nullptr; a.n_first = n;
  a.S = p.S; a.nbs = p.nbs; a.RS = p.RS; a.iters = p.iters; a.status = status;
  a.rows_q = n / p.gx; a.rows_r = n % p.gx;
  // Programmatic dependent launch: the next kernel of the stream may start its prologue (barrier set-up and weight
  // prefetch) while this one drains; it reads activations only after griddepcontrol.wait.
  static bool const no_pdl = std::getenv("QUACTLIZE_B200_NO_PDL") != nullptr;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.gx, gy); cfg.blockDim = dim3(p.W * 32); cfg.dynamicSmemBytes = p.smem; cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = no_pdl ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, q4k_gemv1_kernel<kStages1>, a) == cudaSuccess;
}

// Two Q4_K matrices of the same K against ONE activation row in one launch (a layer's gate and up projections): the CTAs
// split the n1 + n2 rows evenly as if they were one matrix.  false outside the single-row kernel's envelope.
bool enqueue_q4k_gemv1_dual(uint8_t const* blocks1, int n1, uint8_t const* blocks2, int n2, __half const* x, float* out1, float* out2,
                            int bpr, unsigned int* status, cudaStream_t stream) {
  if (n1 <= 0 || n2 <= 0) return false;
  Q4Plan1 const& p = q4k_plan1(n1 + n2, bpr, 1);
  if (!p.ok) return false;
  Q4Args a{};
  a.blocks = blocks1; a.x = x; a.out = out1; a.offsets = nullptr;
  a.n = n1 + n2; a.bpr = bpr; a.max_rows = 1;
  a.blocks2 = blocks2; a.out2 = out2; a.n_first = n1;
  a.S = p.S; a.nbs = p.nbs; a.RS = p.RS; a.iters = p.iters; a.status = status;
  a.rows_q = a.n / p.gx; a.rows_r = a.n % p.gx;
  static bool const no_pdl = std::getenv("QUACTLIZE_B200_NO_PDL") != nullptr;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.gx, 1); cfg.blockDim = dim3(p.W * 32); cfg.dynamicSmemBytes = p.smem; cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = no_pdl ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, q4k_gemv1_kernel<kStages1>, a) == cudaSuccess;
}

}  // namespace qb
