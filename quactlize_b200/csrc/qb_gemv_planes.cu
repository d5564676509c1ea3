// Decode GEMV over the offline BIT-PLANE artifact (scale-first planes or the merged planes + packed units form).
//
//   out[t, r] = sum_k a[t, k] * ( (u[r,k] + off) * s[r, k/gs] + z[r, k/gs] ),   u = lo + 2^LO * hi
//
//   low  [E][n][k*LO/8], high [E][n][k*HI/8]   Native planes: element k of a row at bit k*bits, LSB first
//   scale-first mode : fp16 scale, zero [E][k/gs][n] (zero optional)
//   merged mode      : packed k-quant units [E][k/256/P][n][unit bytes]; s = d*sc, z = -dmin*mn - bias*s in fp32
//
// Replaces the reference kernels gemv_kernel (quactlize/include/gemv_lowbit/gemv_kernel.hpp:44-246, launched by
// gemv_launcher.hpp:213-246) and bc_vecdot::rows_kernel (quactlize/include/gguf_bc_vecdot.hpp:152-227).
//
// Design (same skeleton as the raw Q4_K kernel): one warp owns (output row, K segment); its activation slice lives in
// registers, pre-scaled by a per-warp power of two and laid out in the order the plane bit tricks emit codes; plane
// row segments arrive by cp.async.bulk into a per-warp shared-memory ring; codes are consumed as fp16 subnormal
// patterns ((w & mask) IS code*2^p*2^-24) by HFMA2, two planes accumulate into the same group sum because the high
// plane's activations carry the extra 2^LO; scales for the NEXT row are prefetched while the current row computes.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstdint>
#include <map>
#include <mutex>

#include "qb_device.cuh"
#include "qb_internal.hpp"
#include "qb_kquant.cuh"
#include "qb_runtime.hpp"

namespace qb {

struct PlaneArgs {
  PlaneGemvDesc d;
  int S, cps, RS, iters, nch;      // K segments, lane-chunks per segment, row slots per CTA, rows per slot, chunks per row
  unsigned int* status;
};

// element e of a register-resident activation chunk (two 16-bit values per word), as float
__device__ __forceinline__ float act_elem(uint32_t const* xraw, int e, int bf16) {
  uint32_t const h = (xraw[e >> 1] >> (16 * (e & 1))) & 0xFFFFu;
  return bf16 ? __uint_as_float(h << 16) : __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}
// CPC 16-bit activations starting at element idx0 (a multiple of 8) -> registers; zeros when !valid
template <int CPC>
__device__ __forceinline__ void load_act_chunk(void const* base, size_t idx0, bool valid, uint32_t* xraw) {
  uint4 const* p = reinterpret_cast<uint4 const*>(reinterpret_cast<uint16_t const*>(base) + idx0);
#pragma unroll
  for (int v = 0; v < CPC / 8; ++v) {
    uint4 const q = valid ? __ldg(p + v) : make_uint4(0, 0, 0, 0);
    xraw[4 * v] = q.x; xraw[4 * v + 1] = q.y; xraw[4 * v + 2] = q.z; xraw[4 * v + 3] = q.w;
  }
}

// accumulate one 32-bit plane word of B-bit codes; xs[pi] holds the matching activation pairs
template <int B>
__device__ __forceinline__ __half2 acc_word(uint32_t w, __half2 const* xs, __half2 acc) {
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

// activation pairs for one plane word whose first code is element e0 of the chunk: codes a = (h*8)/B + o and
// a + 16/B, multiplier 2^(ex - o*B)
template <int B>
__device__ __forceinline__ void build_x_word(uint32_t const* xraw, int e0, int bf16, int ex, __half2* xs) {
  constexpr int PER = 8 / B;
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int o = 0; o < PER; ++o) {
      int const a = (h * 8) / B + o, b = a + 16 / B;
      float const m = ldexpf(1.f, ex - o * B);
      xs[h * PER + o] = __floats2half2_rn(act_elem(xraw, e0 + a, bf16) * m, act_elem(xraw, e0 + b, bf16) * m);
    }
}

template <int LO, int HI, int NG, int CPL, int MODE, int QT, int STAGES>
__global__ void __launch_bounds__(512, 1) plane_gemv_kernel(PlaneArgs a) {
  constexpr int CPC = 128 / LO;                 // codes per 16-byte lane-chunk of the low plane
  constexpr int CW = 32 / LO;                   // codes per low word
  constexpr int NPL = 2 * (8 / LO);             // patterns per low word
  constexpr int HB = CPC * HI / 8;              // high-plane bytes per lane-chunk (0, 4 or 8)
  constexpr int HW = HB / 4;                    // high words per lane-chunk
  constexpr int CWH = HI ? 32 / HI : 1;         // codes per high word
  constexpr int NPH = HI ? 2 * (8 / HI) : 1;
  constexpr int GC = CPC / NG;                  // codes of one group inside a chunk (group size, or the whole chunk)
  constexpr bool kCross = HI && (CWH > GC);     // a high word spans two groups (Q3_K's 1-bit plane at gs 16)
  PlaneGemvDesc const& d = a.d;
  extern __shared__ __align__(128) uint8_t smem[];
  int const W = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int const seg = warp % a.S, rslot = warp / a.S;

  int e = 0, arow;
  if (d.offsets) {
    e = blockIdx.y / d.max_rows;
    int const r = blockIdx.y % d.max_rows, r0 = d.offsets[e], r1 = d.offsets[e + 1];
    if (r >= r1 - r0) return;
    arow = r0 + r;
  } else {
    arow = blockIdx.y;
  }
  int const k = d.k, n = d.n, gs = d.group_size;
  int const lo_stage = a.cps * 16, hi_stage = a.cps * HB, stage_bytes = lo_stage + hi_stage;
  int const ch0 = seg * a.cps;
  int const nch_seg = min(a.cps, a.nch - ch0);
  uint8_t* ring = smem + size_t(warp) * STAGES * stage_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + size_t(W) * STAGES * stage_bytes) + warp * STAGES;
  float* part = reinterpret_cast<float*>(smem + size_t(W) * STAGES * stage_bytes + size_t(W) * STAGES * 8);

  int const row0 = blockIdx.x * (a.RS * a.iters);
  int n_my = 0;
  if (row0 + rslot < n) n_my = min(a.iters, (n - 1 - (row0 + rslot)) / a.RS + 1);

  size_t const lo_row = size_t(k) * LO / 8, hi_row = size_t(k) * HI / 8;
  uint8_t const* lo_base = d.low + size_t(e) * n * lo_row + size_t(ch0) * 16;
  uint8_t const* hi_base = HI ? d.high + size_t(e) * n * hi_row + size_t(ch0) * HB : nullptr;
  unsigned const lo_bytes = unsigned(nch_seg) * 16u, hi_bytes = unsigned(nch_seg) * unsigned(HB);

  auto issue = [&](int it, int st) {
    size_t const row = size_t(row0 + rslot + it * a.RS);
    mbar_expect_tx(&bars[st], lo_bytes + hi_bytes);
    bulk_g2s(ring + st * stage_bytes, lo_base + row * lo_row, lo_bytes, &bars[st]);
    if constexpr (HI != 0) bulk_g2s(ring + st * stage_bytes + lo_stage, hi_base + row * hi_row, hi_bytes, &bars[st]);
  };
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(&bars[s], 1);
    mbar_init_fence();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    for (int s = 0; s < STAGES && s < n_my; ++s) issue(s, s);
  }
  __syncwarp();

  // ---- activations -> registers --------------------------------------------------------------------------------
  __half2 xl[CPL][4][NPL];
  __half2 xh[CPL][HW ? HW : 1][NPH];
  float sx[CPL][NG];
  bool cvalid[CPL];
  size_t const xoff = size_t(arow) * k;
  float mx = 0.f;
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    int const cis = c * 32 + lane;
    cvalid[c] = cis < nch_seg;
    uint32_t xraw[CPC / 2];
    load_act_chunk<CPC>(d.act, xoff + size_t(ch0 + cis) * CPC, cvalid[c], xraw);
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < GC; ++j) { float const f = act_elem(xraw, g * GC + j, d.act_bf16); s += f; mx = fmaxf(mx, fabsf(f)); }
      sx[c][g] = s;
    }
  }
  mx = warp_max(mx);
  int const ex = pow2_scale_exponent(mx, HI ? 15 - LO : 15);
  float const fm = ldexpf(1.f, 24 - ex);
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    uint32_t xraw[CPC / 2];
    load_act_chunk<CPC>(d.act, xoff + size_t(ch0 + c * 32 + lane) * CPC, cvalid[c], xraw);
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) build_x_word<LO>(xraw, wi * CW, d.act_bf16, ex, xl[c][wi]);
    if constexpr (HI != 0) {
#pragma unroll
      for (int hw = 0; hw < HW; ++hw) build_x_word<(HI ? HI : 1)>(xraw, hw * CWH, d.act_bf16, ex + LO, xh[c][hw]);
    }
  }

  // ---- per-row scale channel, fetched one row ahead ---------------------------------------------------------------
  // MODE 0: raw fp16 bits of (scale, zero) per (chunk, group).  MODE 1: up to 3 raw words of the chunk's unit share.
  constexpr int NSR = MODE == 0 ? CPL * NG : CPL * 3;
  uint32_t cur[NSR], nxt[NSR];
  int const kg = k / gs;
  auto fetch_scales = [&](int it, uint32_t* dst) {
    size_t const row = size_t(row0 + rslot + it * a.RS);
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
      if (!cvalid[c]) continue;
      int const ci = ch0 + c * 32 + lane;                   // lane-chunk index inside the row
      if constexpr (MODE == 0) {
        uint16_t const* sp = reinterpret_cast<uint16_t const*>(d.scale);
        uint16_t const* zp = reinterpret_cast<uint16_t const*>(d.zero);
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          size_t const gi = (size_t(e) * kg + size_t(ci) * CPC / gs + (NG > 1 ? g : 0)) * n + row;
          uint32_t const s = __ldg(sp + gi), z = zp ? uint32_t(__ldg(zp + gi)) : 0u;
          dst[c * NG + g] = s | (z << 16);
        }
      } else {
        using U = kq::Unit<QT>;
        constexpr int CPS = 256 / CPC;                       // lane-chunks per superblock
        int const sb = ci / CPS, q = ci % CPS;
        int const nu = (k / 256) / U::kSbPerUnit;
        uint8_t const* u = d.units + ((size_t(e) * nu + sb / U::kSbPerUnit) * n + row) * U::kUnitTotal + (sb % U::kSbPerUnit) * U::kSbBytes;
        uint16_t const* u16 = reinterpret_cast<uint16_t const*>(u);
        if constexpr (QT == 12 || QT == 13) {               // 16-byte unit, one group (= q) per chunk
          uint32_t const* u32 = reinterpret_cast<uint32_t const*>(u);
          int const bit = 32 + (q & 3) * 6 + (q >> 2) * 48;   // sub-scale; the sub-min sits 24 bits further
          uint32_t const w0 = __ldg(u32 + (bit >> 5)), w1 = __ldg(u32 + ((bit + 29) >> 5));
          uint32_t const sc = __funnelshift_r(w0, w1, bit & 31) & 63u;
          uint32_t const mn = (__funnelshift_r(w0, w1, bit & 31) >> 24) & 63u;
          dst[c * 3 + 0] = __ldg(u32);                       // d | dmin << 16
          dst[c * 3 + 1] = sc | (mn << 8);
          dst[c * 3 + 2] = 0;
        } else if constexpr (QT == 14) {                    // 18-byte share: d, then 16 int8; chunk = groups 2q, 2q+1
          dst[c * 3 + 0] = __ldg(u16);
          dst[c * 3 + 1] = __ldg(u16 + 1 + q);
          dst[c * 3 + 2] = 0;
        } else if constexpr (QT == 11) {                    // 14-byte share: d, then 16 x 6 bits; chunk = groups 4q..4q+3
          int const off = 2 + 3 * q;                         // 3 bytes of fields
          uint32_t const lo16 = __ldg(u16 + (off >> 1)), hi16 = __ldg(u16 + (off >> 1) + 1);
          dst[c * 3 + 0] = __ldg(u16);
          dst[c * 3 + 1] = ((lo16 | (hi16 << 16)) >> (8 * (off & 1))) & 0xFFFFFFu;
          dst[c * 3 + 2] = 0;
        } else {                                            // Q2_K 20-byte unit: d,dmin, 2 runs of (8x4 scale bits, 8x4 min bits)
          int const g0 = 4 * q, run = g0 >> 3, in = (g0 & 7) >> 2;       // 16 bits of scales, 16 bits of mins
          dst[c * 3 + 0] = __ldg(reinterpret_cast<uint32_t const*>(u));
          dst[c * 3 + 1] = __ldg(u16 + 2 + run * 4 + in);
          dst[c * 3 + 2] = __ldg(u16 + 2 + run * 4 + 2 + in);
        }
      }
    }
  };
#pragma unroll
  for (int t = 0; t < NSR; ++t) nxt[t] = 0;
  if (n_my > 0) fetch_scales(0, nxt);

  float const coff = float(d.code_offset);
  int dead_at = -1;
  for (int i = 0; i < n_my; ++i) {
    int const st = i % STAGES;
#pragma unroll
    for (int t = 0; t < NSR; ++t) cur[t] = nxt[t];
    if (i + 1 < n_my) fetch_scales(i + 1, nxt);
    if (!mbar_wait_bounded(&bars[st], unsigned(i / STAGES) & 1u, a.status, kWaitStageTimeout)) { dead_at = i; break; }
    float tot = 0.f;
    uint8_t const* sl = ring + st * stage_bytes;
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
      if (!cvalid[c]) continue;
      int const cis = c * 32 + lane;
      uint4 const qv = lds128(sl + 16 * cis);
      uint32_t const qw[4] = {qv.x, qv.y, qv.z, qv.w};
      __half2 acc[NG];
#pragma unroll
      for (int g = 0; g < NG; ++g) acc[g] = __float2half2_rn(0.f);
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) acc[(wi * CW) / GC] = acc_word<LO>(qw[wi], xl[c][wi], acc[(wi * CW) / GC]);
      float gsum[NG];
      if constexpr (HI != 0) {
        uint32_t hwv[HW];
        if constexpr (HW == 1) {
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(hwv[0]) : "r"(smem_u32(sl + lo_stage + 4 * cis)));
        } else {
          asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(hwv[0]), "=r"(hwv[HW - 1]) : "r"(smem_u32(sl + lo_stage + 8 * cis)));
        }
        if constexpr (kCross) {
          __half2 cx[HW];
#pragma unroll
          for (int hw = 0; hw < HW; ++hw) cx[hw] = acc_word<(HI ? HI : 1)>(hwv[hw], xh[c][hw], __float2half2_rn(0.f));
#pragma unroll
          for (int g = 0; g < NG; ++g) {
            float2 const f = __half22float2(cx[g >> 1]);
            gsum[g] = h2_sum(acc[g]) + ((g & 1) ? f.y : f.x);
          }
        } else {
#pragma unroll
          for (int hw = 0; hw < HW; ++hw) acc[(hw * CWH) / GC] = acc_word<(HI ? HI : 1)>(hwv[hw], xh[c][hw], acc[(hw * CWH) / GC]);
#pragma unroll
          for (int g = 0; g < NG; ++g) gsum[g] = h2_sum(acc[g]);
        }
      } else {
#pragma unroll
        for (int g = 0; g < NG; ++g) gsum[g] = h2_sum(acc[g]);
      }
      // scale channel
      if constexpr (MODE == 0) {
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          float2 const sz = __half22float2(u32_as_h2(cur[c * NG + g]));
          tot = fmaf(sz.x, fmaf(fm, gsum[g], coff * sx[c][g]), tot);
          tot = fmaf(sz.y, sx[c][g], tot);
        }
      } else {
        using F = kq::Fmt<QT>;
        uint32_t const r0 = cur[c * 3], r1 = cur[c * 3 + 1], r2 = cur[c * 3 + 2];
        float2 const dd = __half22float2(u32_as_h2(r0));        // (d, dmin) -- dmin lane is garbage for Q3_K/Q6_K, unused
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          float sc, mn = 0.f;
          if constexpr (QT == 12 || QT == 13) { sc = float(r1 & 0xFFu); mn = float((r1 >> 8) & 0xFFu); }
          else if constexpr (QT == 14) { sc = float(int(int8_t((r1 >> (8 * g)) & 0xFFu))); }
          else if constexpr (QT == 11) { sc = float(int((r1 >> (6 * g)) & 63u) - 32); }
          else { sc = float((r1 >> (4 * g)) & 15u); mn = float((r2 >> (4 * g)) & 15u); }
          float const s = dd.x * sc;
          tot = fmaf(s, fmaf(fm, gsum[g], -float(F::kCodeBias) * sx[c][g]), tot);
          if constexpr (F::kHasMin) tot = fmaf(-dd.y * mn, sx[c][g], tot);
        }
      }
    }
    __syncwarp();
    if (lane == 0 && i + STAGES < n_my) issue(i + STAGES, st);
    tot = warp_sum(tot);
    if (lane == 0) part[size_t(i * a.RS + rslot) * a.S + seg] = tot;
  }
  if (dead_at >= 0)
    for (int i = dead_at + 1; i < n_my && i < dead_at + STAGES; ++i)
      (void)mbar_wait_bounded(&bars[i % STAGES], unsigned(i / STAGES) & 1u, nullptr, 0, 250000000ull);
  __syncthreads();
  int const rows_cta = a.RS * a.iters;
  for (int lr = threadIdx.x; lr < rows_cta; lr += blockDim.x) {
    int const row = row0 + lr;
    if (row >= n) continue;
    float s = 0.f;
    for (int sg = 0; sg < a.S; ++sg) s += part[size_t(lr) * a.S + sg];
    size_t const oi = size_t(arow) * n + row;
    if (d.out_kind == 1) reinterpret_cast<float*>(d.out)[oi] = s;
    else if (d.out_kind == 0) reinterpret_cast<__half*>(d.out)[oi] = __float2half_rn(s);
    else reinterpret_cast<__nv_bfloat16*>(d.out)[oi] = __float2bfloat16_rn(s);
  }
}

namespace {

struct PlanePlan { int S, cps, RS, iters, gx, W, nch; size_t smem; int rc; };

template <int LO, int HI, int NG, int CPL, int MODE, int QT>
int launch_plane(PlaneGemvDesc const& d, cudaStream_t stream) {
  constexpr int STAGES = 6;
  constexpr int CPC = 128 / LO, HB = CPC * HI / 8;
  auto kern = plane_gemv_kernel<LO, HI, NG, CPL, MODE, QT, STAGES>;
  int const gy = d.offsets ? d.experts * d.max_rows : d.m_rows;
  if (gy <= 0 || gy > 65535) return 40;
  // launch geometry depends only on (n, k, grid.y, device): computed once, then cached
  struct Key { int n, k, gy, dev; bool operator<(Key const& o) const {
    return n != o.n ? n < o.n : k != o.k ? k < o.k : gy != o.gy ? gy < o.gy : dev < o.dev; } };
  static std::map<Key, PlanePlan> cache;
  static std::mutex mu;
  PlanePlan p{};
  {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(mu);
    Key const key{d.n, d.k, gy, dev};
    auto it = cache.find(key);
    if (it == cache.end()) {
      p.nch = d.k / CPC;
      p.S = (p.nch + 32 * CPL - 1) / (32 * CPL);
      p.rc = p.S > 16 ? 40 : 0;
      if (!p.rc) {
        p.cps = ((p.nch + p.S - 1) / p.S + 3) & ~3;        // keeps every high-plane segment 16-byte aligned
        p.RS = std::max(1, 8 / p.S);
        p.W = p.S * p.RS;
        size_t const ring = size_t(p.W) * STAGES * p.cps * (16 + HB) + size_t(p.W) * STAGES * 8;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        int const sms = rt_sm_count();
        int iters = 1;
        for (int pass = 0; pass < 2 && !p.rc; ++pass) {
          size_t const smem = ring + size_t(iters) * p.RS * p.S * 4;
          if (smem > 227 * 1024) { p.rc = 40; break; }
          int occ = 0;
          if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, p.W * 32, smem) != cudaSuccess || occ < 1) occ = 1;
          int const resident = std::max(1, occ * sms / std::max(1, std::min(gy, 8)));
          int const slots = (d.n + p.RS - 1) / p.RS;
          iters = std::min(64, std::max(1, (slots + resident - 1) / resident));
        }
        p.iters = iters;
        p.smem = ring + size_t(iters) * p.RS * p.S * 4;
        if (p.smem > 227 * 1024) p.rc = 40;
        p.gx = (d.n + p.RS * iters - 1) / (p.RS * iters);
      }
      it = cache.emplace(key, p).first;
    }
    p = it->second;
  }
  if (p.rc) return p.rc;
  PlaneArgs a{};
  a.d = d;
  a.status = rt_device_status_ptr();
  if (!a.status) return kRuntimeError;
  a.nch = p.nch; a.S = p.S; a.cps = p.cps; a.RS = p.RS; a.iters = p.iters;
  kern<<<dim3(p.gx, gy), p.W * 32, p.smem, stream>>>(a);
  return 0;
}

// chunks-per-lane: the smallest of {1,2,4} (capped by the register budget of the format) that covers the row
template <int LO, int HI, int NG, int MODE, int QT, int CPLMAX>
int launch_plane_cpl(PlaneGemvDesc const& d, cudaStream_t s) {
  int const nch = d.k / (128 / LO);
  if constexpr (CPLMAX >= 4) { if (nch > 64) return launch_plane<LO, HI, NG, 4, MODE, QT>(d, s); }
  if constexpr (CPLMAX >= 2) { if (nch > 32) return launch_plane<LO, HI, NG, 2, MODE, QT>(d, s); }
  return launch_plane<LO, HI, NG, 1, MODE, QT>(d, s);
}

}  // namespace

int enqueue_plane_gemv(PlaneGemvDesc const& d, cudaStream_t s) {
  if (d.k <= 0 || d.k % 256 || d.n <= 0) return 40;
  // Kernel choice: the tensor-core small-batch kernel when several activation rows can share a weight pass, else the
  // row-thread kernel, else the segment-per-warp kernel below.  QUACTLIZE_B200_PLANE_GEMV = mma | rowthread | segment
  // forces one of them (for comparisons); "pair" forces the row-pair kernel of the merged artifact where it applies.
  static int const forced = [] {
    char const* v = std::getenv("QUACTLIZE_B200_PLANE_GEMV");
    return !v ? 0 : v[0] == 'm' ? 1 : v[0] == 'r' ? 2 : v[0] == 's' ? 3 : v[0] == 'p' ? 4 : 0;
  }();
  bool const batch = d.offsets ? d.m_rows >= 2 * std::max(1, d.experts) : d.m_rows >= 2;
  if (forced == 1 || (forced == 0 && batch)) {
    int const rc = enqueue_rowmma_gemv(d, s);
    if (rc != 40) return rc;
  }
  // merged artifact, one activation row per expert at most: the row-pair kernel (with more rows per expert the row-thread
  // kernel shares a weight tile between up to four of them)
  int const passes = d.offsets ? d.max_rows : d.m_rows;
  if (d.scale_mode == 1 && (forced == 4 || (forced == 0 && passes == 1))) {
    int const rc = enqueue_bc_gemv1(d, s);
    if (rc != 40) return rc;
  }
  if (forced != 3) {
    int const rc = enqueue_rowthread_gemv(d, s);
    if (rc != 40) return rc;
  }
  auto aligned = [](void const* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (!aligned(d.low) || (d.hi_bits && !aligned(d.high)) || !aligned(d.act)) return 40;
  if (d.scale_mode == 1) {
    switch (d.qtype) {
      case 10: return launch_plane_cpl<2, 0, 4, 1, 10, 2>(d, s);
      case 11: return launch_plane_cpl<2, 1, 4, 1, 11, 1>(d, s);
      case 12: return launch_plane_cpl<4, 0, 1, 1, 12, 4>(d, s);
      case 13: return launch_plane_cpl<4, 1, 1, 1, 13, 2>(d, s);
      case 14: return launch_plane_cpl<4, 2, 2, 1, 14, 2>(d, s);
      default: return 40;
    }
  }
  int const gs = d.group_size;
  if (gs <= 0 || d.k % gs) return 40;
  int const key = d.lo_bits * 100 + d.hi_bits * 10;
  int const cpc = 128 / d.lo_bits;
  int const ng = gs >= cpc ? 1 : cpc / gs;
  if (gs < 16 || (gs & (gs - 1))) return 40;
  switch (key) {
    case 400: if (ng == 1) return launch_plane_cpl<4, 0, 1, 0, 0, 4>(d, s);
              if (ng == 2) return launch_plane_cpl<4, 0, 2, 0, 0, 4>(d, s); break;
    case 410: if (ng == 1) return launch_plane_cpl<4, 1, 1, 0, 0, 2>(d, s); break;
    case 420: if (ng == 2) return launch_plane_cpl<4, 2, 2, 0, 0, 2>(d, s); break;
    case 200: if (ng == 1) return launch_plane_cpl<2, 0, 1, 0, 0, 2>(d, s);
              if (ng == 2) return launch_plane_cpl<2, 0, 2, 0, 0, 2>(d, s);
              if (ng == 4) return launch_plane_cpl<2, 0, 4, 0, 0, 2>(d, s); break;
    case 210: if (ng == 4) return launch_plane_cpl<2, 1, 4, 0, 0, 1>(d, s); break;
    case 100: if (ng == 1) return launch_plane_cpl<1, 0, 1, 0, 0, 1>(d, s);
              if (ng == 2) return launch_plane_cpl<1, 0, 2, 0, 0, 1>(d, s);
              if (ng == 4) return launch_plane_cpl<1, 0, 4, 0, 0, 1>(d, s); break;
    default: break;
  }
  return 40;
}

}  // namespace qb
