// Decode GEMV over RAW GGUF k-quant blocks (the checkpoint's own bytes; nothing is materialised).
//
//   out[t, r] = sum_k x[t, k] * W[r, k],   W from blocks [E][n][k/256][block_bytes] row-major by output row,
//   x fp16 [rows, k] (dense: shared by all rows; grouped: gathered in expert order with cumulative offsets),
//   out fp32.
//
// Replaces the reference kernel vecdot_rows_kernel (quactlize/include/gguf_vecdot.hpp:604-760) and its launch policy
// (quactlize/csrc/device/ppu_backend.cu:52-131).  The arithmetic identity is the reference's
// (gguf_vecdot.hpp:12-19): sum_i W_i x_i = sum_g [ dl_g * sum(q x) - ml_g * sum(x) ], but group sums are carried to
// fp32 after at most 16 fp16 products instead of accumulating the whole row in fp16.
//
// Q4_K fast kernel (sm_100a design):
//   * one warp owns (output row, K segment); the activation slice of that segment lives in REGISTERS for the whole
//     kernel, pre-scaled by a per-warp power of two and pre-arranged in the order the bit tricks emit codes;
//   * the row segment (<= 16 blocks = 2304 B, contiguous) is fetched by one cp.async.bulk into a private
//     shared-memory ring (mbarrier completion, 6-8 stages deep per warp), so up to ~220 KB per SM is in flight;
//   * codes never pass through an integer->float conversion: (w & 0x000F000F) reinterpreted as half2 is two fp16
//     subnormals q*2^-24, fed straight to HFMA2; 5 integer + 4 HFMA2 instructions per 8 weights;
//   * 6-bit sub-scales/mins are unpacked once per (lane, block) with three 32-bit words and byte permutes.
// Other formats / unaligned inputs use a simpler warp-per-row kernel that reads blocks through L1.
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
#include "qb_runtime.hpp"

namespace qb {

struct NativeArgs {
  uint8_t const* blocks;
  __half const* x;
  float* out;
  int const* offsets;     // cumulative [experts+1] (grouped) or nullptr (dense)
  int n, bpr, experts, m_rows, mtiles;
  int S, nbs, RS, iters;
  int per_row_x;          // generic kernel only: row r has its own activation slice (the per-block vecdot contract)
  unsigned int* status;
};

// ------------------------------------------------------------------------------------------------------------------
// Q4_K, bulk-copy staged.

template <int M, int LPB, int STAGES>
__global__ void __launch_bounds__(M >= 4 ? 256 : 384, 1) q4k_gemv_kernel(NativeArgs a) {
  constexpr int CH = 8 / LPB;          // 16-byte qs chunks per lane per block
  extern __shared__ __align__(128) uint8_t smem[];
  int const W = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int const seg = warp % a.S, rslot = warp / a.S;

  int e = 0, mt = blockIdx.y, row_base, mvalid;
  if (a.offsets) {
    e = blockIdx.y / a.mtiles; mt = blockIdx.y % a.mtiles;
    int const r0 = a.offsets[e], r1 = a.offsets[e + 1];
    row_base = r0 + mt * M; mvalid = min(M, r1 - row_base);
  } else {
    row_base = mt * M; mvalid = min(M, a.m_rows - row_base);
  }
  if (mvalid <= 0) return;                                    // uniform for the whole CTA

  int const k = a.bpr * 256;
  int const stage_bytes = a.nbs * 144;
  int const nb_seg = min(a.nbs, a.bpr - seg * a.nbs);          // blocks in this warp's segment (>= 1)
  uint8_t* ring = smem + size_t(warp) * STAGES * stage_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + size_t(W) * STAGES * stage_bytes) + warp * STAGES;
  float* part = reinterpret_cast<float*>(smem + size_t(W) * STAGES * stage_bytes + size_t(W) * STAGES * 8);

  int const row0 = blockIdx.x * (a.RS * a.iters);
  int n_my = 0;
  if (row0 + rslot < a.n) n_my = min(a.iters, (a.n - 1 - (row0 + rslot)) / a.RS + 1);

  uint8_t const* wbase = a.blocks + (size_t(e) * a.n * a.bpr + size_t(seg) * a.nbs) * 144;
  size_t const row_stride = size_t(a.bpr) * 144;
  unsigned const copy_bytes = unsigned(nb_seg) * 144u;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(&bars[s], 1);
    mbar_init_fence();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    for (int s = 0; s < STAGES && s < n_my; ++s) {
      mbar_expect_tx(&bars[s], copy_bytes);
      bulk_g2s(ring + s * stage_bytes, wbase + size_t(row0 + rslot + s * a.RS) * row_stride, copy_bytes, &bars[s]);
    }
  }
  __syncwarp();

  // ---- activation slice -> registers, scaled and arranged for the code patterns -------------------------------
  int const blk = lane / LPB, prt = lane % LPB;
  bool const active = blk < nb_seg;
  int const b_in_row = seg * a.nbs + blk;
  __half2 xr[M][CH][16];        // per word wi: [4wi+0]=(lo e0,e2) [4wi+1]=(lo e1,e3) [4wi+2]=(hi e0,e2) [4wi+3]=(hi e1,e3)
  float sx[M][CH][2];           // sum of the unscaled activations of the lane's 16 elements of the lo / hi group
  float fm[M];                  // 2^48 / scale_m
#pragma unroll
  for (int m = 0; m < M; ++m) {
    float mx = 0.f;
    bool const mv = active && m < mvalid;
    __half const* xrow = a.x + size_t(row_base + (m < mvalid ? m : 0)) * k + size_t(b_in_row) * 256;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      int const ci = prt * CH + c;
      int const klo = (ci >> 1) * 64 + (ci & 1) * 16;
      uint4 v[4];
      if (mv) {
        uint4 const* p0 = reinterpret_cast<uint4 const*>(xrow + klo);
        uint4 const* p1 = reinterpret_cast<uint4 const*>(xrow + klo + 32);
        v[0] = __ldg(p0); v[1] = __ldg(p0 + 1); v[2] = __ldg(p1); v[3] = __ldg(p1 + 1);
      } else {
        v[0] = v[1] = v[2] = v[3] = make_uint4(0, 0, 0, 0);
      }
      // v[0..1] = 16 lo-group halves e0..e15, v[2..3] = 16 hi-group halves.  Stash raw; scale after the max is known.
      uint32_t const* lo = reinterpret_cast<uint32_t const*>(&v[0]);
      uint32_t const* hi = reinterpret_cast<uint32_t const*>(&v[2]);
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {
        // natural order pairs: lo[2wi] = (e0,e1), lo[2wi+1] = (e2,e3)  ->  (e0,e2), (e1,e3)
        uint32_t const a01 = lo[2 * wi], a23 = lo[2 * wi + 1], b01 = hi[2 * wi], b23 = hi[2 * wi + 1];
        xr[m][c][4 * wi + 0] = u32_as_h2(__byte_perm(a01, a23, 0x5410));
        xr[m][c][4 * wi + 1] = u32_as_h2(__byte_perm(a01, a23, 0x7632));
        xr[m][c][4 * wi + 2] = u32_as_h2(__byte_perm(b01, b23, 0x5410));
        xr[m][c][4 * wi + 3] = u32_as_h2(__byte_perm(b01, b23, 0x7632));
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float2 const f = __half22float2(xr[m][c][4 * wi + q]);
          mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
          if (q < 2) s0 += f.x + f.y; else s1 += f.x + f.y;
        }
      }
      sx[m][c][0] = s0; sx[m][c][1] = s1;
    }
    mx = warp_max(mx);
    int const ex = pow2_scale_exponent(mx, 15);
    float const sc_lo = ldexpf(1.f, ex), sc_hi = ldexpf(1.f, ex - 4);
    fm[m] = ldexpf(1.f, 48 - ex);
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        float2 f = __half22float2(xr[m][c][q]);
        float const s = ((q & 3) < 2) ? sc_lo : sc_hi;
        xr[m][c][q] = __floats2half2_rn(f.x * s, f.y * s);
      }
  }
  // byte selectors of this lane's (sub-scale, sub-min) pair inside the 4-byte words built below
  uint32_t sel[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) sel[c] = (((prt * CH + c) >> 1) & 1) ? 0x4342u : 0x4140u;
  bool const upper = ((prt * CH) >> 2) != 0;                   // groups 4..7

  int dead_at = -1;
  for (int i = 0; i < n_my; ++i) {
    int const st = i % STAGES;
    unsigned const ph = unsigned(i / STAGES) & 1u;
    if (!mbar_wait_bounded(&bars[st], ph, a.status, kWaitStageTimeout)) { dead_at = i; break; }
    float tot[M];
#pragma unroll
    for (int m = 0; m < M; ++m) tot[m] = 0.f;
    if (active) {
      uint8_t const* sb = ring + st * stage_bytes + blk * 144;
      uint4 const hdr = lds128(sb);
      uint32_t sc4, mn4;
      if (!upper) { sc4 = hdr.y & 0x3F3F3F3Fu; mn4 = hdr.z & 0x3F3F3F3Fu; }
      else {
        sc4 = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
        mn4 = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
      }
      float2 const dd = __half22float2(u32_as_h2(hdr.x));       // (d, dmin)
      float dsum[M], msum[M];
#pragma unroll
      for (int m = 0; m < M; ++m) { dsum[m] = 0.f; msum[m] = 0.f; }
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        uint4 const qv = lds128(sb + 16 + 16 * (prt * CH + c));
        uint32_t const qw[4] = {qv.x, qv.y, qv.z, qv.w};
        __half2 alo[M], ahi[M];
#pragma unroll
        for (int m = 0; m < M; ++m) { alo[m] = __float2half2_rn(0.f); ahi[m] = alo[m]; }
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          uint32_t const w = qw[wi], w8 = w >> 8;
          __half2 const p0 = u32_as_h2(w & 0x000F000Fu), p1 = u32_as_h2(w & 0x00F000F0u);
          __half2 const p2 = u32_as_h2(w8 & 0x000F000Fu), p3 = u32_as_h2(w8 & 0x00F000F0u);
#pragma unroll
          for (int m = 0; m < M; ++m) {
            alo[m] = __hfma2(p0, xr[m][c][4 * wi + 0], alo[m]);
            ahi[m] = __hfma2(p1, xr[m][c][4 * wi + 2], ahi[m]);
            alo[m] = __hfma2(p2, xr[m][c][4 * wi + 1], alo[m]);
            ahi[m] = __hfma2(p3, xr[m][c][4 * wi + 3], ahi[m]);
          }
        }
        float2 const scf = bytes_to_f2(sc4, sel[c]);             // (sc_lo, sc_hi) * 2^-24
        float2 const mnf = bytes_to_f2(mn4, sel[c]);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          dsum[m] = fmaf(scf.x, h2_sum(alo[m]), dsum[m]);
          dsum[m] = fmaf(scf.y, h2_sum(ahi[m]), dsum[m]);
          msum[m] = fmaf(mnf.x, sx[m][c][0], msum[m]);
          msum[m] = fmaf(mnf.y, sx[m][c][1], msum[m]);
        }
      }
#pragma unroll
      for (int m = 0; m < M; ++m) tot[m] = dd.x * fm[m] * dsum[m] - dd.y * 16777216.f * msum[m];
    }
    __syncwarp();
    if (lane == 0 && i + STAGES < n_my) {
      mbar_expect_tx(&bars[st], copy_bytes);
      bulk_g2s(ring + st * stage_bytes, wbase + size_t(row0 + rslot + (i + STAGES) * a.RS) * row_stride,
               copy_bytes, &bars[st]);
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float const t = warp_sum(tot[m]);
      if (lane == 0) part[(size_t(i * a.RS + rslot) * a.S + seg) * M + m] = t;
    }
  }
  if (dead_at >= 0) {
    // a wait gave up: drain this warp's other copies still in flight (bounded, short) before the shared memory can
    // be handed to another CTA
    for (int i = dead_at + 1; i < n_my && i < dead_at + STAGES; ++i)
      (void)mbar_wait_bounded(&bars[i % STAGES], unsigned(i / STAGES) & 1u, nullptr, 0, 250000000ull);
  }
  __syncthreads();
  int const rows_cta = a.RS * a.iters;
  for (int idx = threadIdx.x; idx < rows_cta * M; idx += blockDim.x) {
    int const m = idx / rows_cta, lr = idx % rows_cta, row = row0 + lr;
    if (row < a.n && m < mvalid) {
      float s = 0.f;
      for (int sg = 0; sg < a.S; ++sg) s += part[(size_t(lr) * a.S + sg) * M + m];
      a.out[size_t(row_base + m) * a.n + row] = s;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Any k-quant, any alignment: one warp per output row, lanes stride over (block, group) items.

template <int QT, int M>
__global__ void __launch_bounds__(256) kquant_gemv_generic_kernel(NativeArgs a) {
  using F = kq::Fmt<QT>;
  constexpr int G = F::kGroups, GS = 256 / G;
  int const warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int const row = blockIdx.x * (blockDim.x >> 5) + warp;
  int e = 0, mt = blockIdx.y, row_base, mvalid;
  if (a.offsets) {
    e = blockIdx.y / a.mtiles; mt = blockIdx.y % a.mtiles;
    int const r0 = a.offsets[e], r1 = a.offsets[e + 1];
    row_base = r0 + mt * M; mvalid = min(M, r1 - row_base);
  } else {
    row_base = mt * M; mvalid = min(M, a.m_rows - row_base);
  }
  if (mvalid <= 0 || row >= a.n) return;
  int const k = a.bpr * 256;
  uint8_t const* rb = a.blocks + (size_t(e) * a.n + row) * a.bpr * F::kBytes;
  __half const* xb = a.per_row_x ? a.x + size_t(row) * k : a.x + size_t(row_base) * k;
  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  for (int it = lane; it < a.bpr * G; it += 32) {
    int const b = it / G, g = it % G;
    uint8_t const* blk = rb + size_t(b) * F::kBytes;
    float const d = __half2float(__ushort_as_half(kq::load_u16(blk + F::kD)));
    float dmin = 0.f;
    if constexpr (F::kHasMin) dmin = __half2float(__ushort_as_half(kq::load_u16(blk + F::kDmin)));
    int sc, mn;
    kq::scale_min<QT>(blk + F::kScaleOff, g, sc, mn);
    float const dl = d * float(sc), ml = dmin * float(mn);
    float sqx[M], sxx[M];
#pragma unroll
    for (int m = 0; m < M; ++m) { sqx[m] = 0.f; sxx[m] = 0.f; }
    for (int j = 0; j < GS; ++j) {
      float const q = float(kq::code<QT>(blk, g, j));
#pragma unroll
      for (int m = 0; m < M; ++m) {
        if (m < mvalid) {
          float const xv = __half2float(xb[size_t(m) * k + b * 256 + g * GS + j]);
          sqx[m] = fmaf(q, xv, sqx[m]);
          sxx[m] += xv;
        }
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] += dl * sqx[m] - ml * sxx[m];
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    float const t = warp_sum(acc[m]);
    if (lane == 0 && m < mvalid) {
      if (a.per_row_x) a.out[row] = t; else a.out[size_t(row_base + m) * a.n + row] = t;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// host launch policy

namespace {

// Launch geometry is a pure function of (kernel, n, bpr, grid.y, device); it is computed once and cached so the
// enqueue path does no occupancy queries or attribute calls (decode launches are only a few microseconds long).
struct Q4Plan { int S, nbs, RS, iters, gx, W; size_t smem; bool ok; };

template <int M, int LPB, int STAGES>
Q4Plan const& q4k_plan(int n, int bpr, int gy) {
  struct Key { int n, bpr, gy, dev; bool operator<(Key const& o) const {
    return n != o.n ? n < o.n : bpr != o.bpr ? bpr < o.bpr : gy != o.gy ? gy < o.gy : dev < o.dev; } };
  static std::map<Key, Q4Plan> cache;
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(mu);
  Key const key{n, bpr, gy, dev};
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  Q4Plan p{};
  constexpr int BW = 32 / LPB;
  constexpr int MAXW = M >= 4 ? 8 : 12;          // warps per CTA the register budget of this tile allows
  auto kern = q4k_gemv_kernel<M, LPB, STAGES>;
  p.S = (bpr + BW - 1) / BW;
  p.ok = p.S <= MAXW;
  if (p.ok) {
    p.nbs = (bpr + p.S - 1) / p.S;
    p.RS = std::max(1, MAXW / p.S);
    p.W = p.S * p.RS;
    size_t const ring = size_t(p.W) * STAGES * p.nbs * 144 + size_t(p.W) * STAGES * 8;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    int const sms = rt_sm_count();
    int iters = 1;
    for (int pass = 0; pass < 2 && p.ok; ++pass) {
      size_t const smem = ring + size_t(iters) * p.RS * p.S * M * 4;
      if (smem > 227 * 1024) { p.ok = false; break; }
      int occ = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, p.W * 32, smem) != cudaSuccess || occ < 1) occ = 1;
      int const resident = std::max(1, occ * sms / std::max(1, gy));
      int const slots = (n + p.RS - 1) / p.RS;
      iters = std::min(64, std::max(1, (slots + resident - 1) / resident));
    }
    p.iters = iters;
    p.smem = ring + size_t(iters) * p.RS * p.S * M * 4;
    if (p.smem > 227 * 1024) p.ok = false;
    p.gx = (n + p.RS * iters - 1) / (p.RS * iters);
  }
  return cache.emplace(key, p).first->second;
}

template <int M, int LPB, int STAGES>
bool launch_q4k_fast(NativeArgs a, int gy, cudaStream_t stream) {
  Q4Plan const& p = q4k_plan<M, LPB, STAGES>(a.n, a.bpr, gy);
  if (!p.ok) return false;
  a.S = p.S; a.nbs = p.nbs; a.RS = p.RS; a.iters = p.iters;
  q4k_gemv_kernel<M, LPB, STAGES><<<dim3(p.gx, gy), p.W * 32, p.smem, stream>>>(a);
  return true;
}

template <int QT, int M>
void launch_generic(NativeArgs const& a, int gy, cudaStream_t stream) {
  kquant_gemv_generic_kernel<QT, M><<<dim3((a.n + 7) / 8, gy), 256, 0, stream>>>(a);
}

template <int M>
void launch_generic_qt(int qtype, NativeArgs const& a, int gy, cudaStream_t stream) {
  switch (qtype) {
    case 10: launch_generic<10, M>(a, gy, stream); break;
    case 11: launch_generic<11, M>(a, gy, stream); break;
    case 12: launch_generic<12, M>(a, gy, stream); break;
    case 13: launch_generic<13, M>(a, gy, stream); break;
    default: launch_generic<14, M>(a, gy, stream); break;
  }
}

}  // namespace

// Enqueue a raw-block GEMV.  max_rows bounds the activation rows of any expert (dense: the row count).
// force_generic selects the simple kernel (used by tests to cross-check the two implementations).
int enqueue_native_gemv(uint8_t const* blocks, __half const* x, float* out, int const* offsets,
                        int n, int bpr, int experts, int m_rows, int max_rows, int qtype, bool per_row_x,
                        bool force_generic, cudaStream_t stream) {
  NativeArgs a{};
  a.blocks = blocks; a.x = x; a.out = out; a.offsets = offsets;
  a.n = n; a.bpr = bpr; a.experts = experts > 0 ? experts : 1; a.m_rows = m_rows;
  a.per_row_x = per_row_x ? 1 : 0;
  a.status = rt_device_status_ptr();
  int const rows_hint = offsets ? max_rows : m_rows;
  bool const aligned = (reinterpret_cast<uintptr_t>(blocks) % 16 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0);
  // several activation rows per weight pass: the tensor-core kernel (QUACTLIZE_B200_Q4K_SMALLM=off keeps the CUDA-core ones)
  static bool const no_mma = [] { char const* v = std::getenv("QUACTLIZE_B200_Q4K_SMALLM"); return v && v[0] == 'o'; }();
  bool const batch = offsets ? m_rows >= 2 * a.experts : m_rows >= 2;
  // dense, 2..8 rows: a CTA per row range, a warp per superblock of the K pass, all eight rows as one MMA operand.  Where
  // K needs more than one pass (more than 16 superblocks per row) it pays an activation prologue per pass and is used from
  // five rows up only (measured on 14336-deep rows: 19.3-19.7 us for any row count against 14.7-17.4 us of the tile kernel
  // at 2-4 rows and 26 us at 5-8).  QUACTLIZE_B200_Q4K_ROWS=off skips it, =all sends every count from one row through it.
  static int const rows_mode = [] { char const* v = std::getenv("QUACTLIZE_B200_Q4K_ROWS"); return !v ? 1 : (v[0] == 'o' ? 0 : (v[0] == 'a' ? 2 : 1)); }();
  bool const rows_fit = rows_mode == 2 || (m_rows >= 2 && (bpr <= 16 || m_rows >= 5));
  if (qtype == 12 && !per_row_x && !force_generic && !offsets && a.status && rows_mode && m_rows <= 8 && rows_fit) {
    if (enqueue_q4k_rows(blocks, x, out, n, bpr, m_rows, a.status, stream)) return 0;
  }
  if (qtype == 12 && !per_row_x && !force_generic && aligned && a.status && batch && !no_mma) {
    if (enqueue_q4k_mma(blocks, x, out, offsets, n, bpr, a.experts, m_rows, a.status, stream)) return 0;
  }
  if (qtype == 12 && !per_row_x && !force_generic && aligned && a.status && rows_hint <= 2) {
    // one or two activation rows: the single-row kernel, once per row (the second pass hits L2)
    if (enqueue_q4k_gemv1(blocks, x, out, offsets, n, bpr, a.experts, m_rows, max_rows, a.status, stream)) return 0;
  }
  if (qtype == 12 && !per_row_x && !force_generic && aligned && a.status) {
    int const mt = rows_hint >= 3 ? 4 : rows_hint == 2 ? 2 : 1;
    a.mtiles = (rows_hint + mt - 1) / mt;
    int const gy = (offsets ? a.experts : 1) * a.mtiles;
    bool ok = false;
    if (mt == 1) ok = launch_q4k_fast<1, 2, 6>(a, gy, stream);
    else if (mt == 2) ok = launch_q4k_fast<2, 4, 8>(a, gy, stream);
    else ok = launch_q4k_fast<4, 8, 8>(a, gy, stream);   // more rows: several 4-row tiles share the weight reads in L2
    if (ok) return 0;
    // long rows leave no room for a multi-row tile's activations: stream the weights once per row instead (the first
    // pass pulls them into L2 for the others) rather than fall back to plain loads
    if (rows_hint <= 16 && enqueue_q4k_gemv1(blocks, x, out, offsets, n, bpr, a.experts, m_rows, max_rows, a.status, stream)) return 0;
  }
  if (qtype != 12 && !per_row_x && !force_generic && aligned && a.status && rows_hint <= 64) {
    // the other four formats: the single-row kernel once per activation row (rows after the first hit L2)
    if (enqueue_kquant_gemv1(blocks, x, out, offsets, n, bpr, a.experts, m_rows, max_rows, qtype, a.status, stream)) return 0;
  }
  if (per_row_x) {
    a.mtiles = 1;
    launch_generic_qt<1>(qtype, a, 1, stream);
    return 0;
  }
  int const mt = rows_hint >= 2 ? 4 : 1;
  a.mtiles = (rows_hint + mt - 1) / mt;
  int const gy = (offsets ? a.experts : 1) * a.mtiles;
  if (mt == 1) launch_generic_qt<1>(qtype, a, gy, stream); else launch_generic_qt<4>(qtype, a, gy, stream);
  return 0;
}

}  // namespace qb
