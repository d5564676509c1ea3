// Host-only producers of the offline weight artifacts (no device work, no torch types).
//
//   raw GGUF blocks [E][N][K/256][bytes]
//      -> Native code planes  low [E][N][K*lo/8], high [E][N][K*hi/8]   element (e,n,k) at bit ((e*N+n)*K+k)*bits,
//         LSB first; signed formats stored offset-binary (Q3_K +4, Q6_K +32)
//      -> fp16 planes scale/zero [E][K/gs][N]           (scale-first artifact)
//      -> packed units [E][K/256/P][N][P*sb_bytes]      (byte-neutral scale channel; Q3_K/Q6_K pair two superblocks)
// and the byte-exact inverse.  Behaviour follows quactlize/csrc/preprocess/thop/gguf_prepass_ops.cpp:809-878
// (gguf_prepare_gemv), quactlize/include/gguf_unit_pack.hpp:58-72 and quactlize/csrc/device/ppu_unit_pack.cpp:72-184.
//
// PLANE PLACEMENT.  The reference's device library permutes the planes into a PPU-specific "xplane" byte order
// (quactlize/csrc/device/ppu_dense_layout.cu:53-74) for its tensor-core converter.  That order encodes PPU hardware
// delivery and is not reproduced: this library's placement IS the Native order, so prepare_dense / recover_dense are
// byte-identical copies and every consumer here (GEMV and GEMM) reads Native planes.
#include <cuda_fp16.h>

#include <cstdint>
#include <cstring>
#include <vector>

#include "qb_kquant.cuh"

namespace qb {
namespace {

inline float h2f(uint16_t b) { return __half2float(__ushort_as_half(b)); }
inline uint16_t f2h(float f) { return __half_as_ushort(__float2half_rn(f)); }

template <int Bits> inline void plane_put(uint8_t* plane, int64_t logical, int v) {
  int64_t const bit = logical * Bits;
  plane[bit >> 3] |= uint8_t((v & ((1 << Bits) - 1)) << (bit & 7));
}
template <int Bits> inline int plane_get(uint8_t const* plane, int64_t logical) {
  int64_t const bit = logical * Bits;
  return (plane[bit >> 3] >> (bit & 7)) & ((1 << Bits) - 1);
}

template <int QT>
void pack_unit_sb(uint8_t const* block, uint8_t* sb) {
  using F = kq::Fmt<QT>;
  using U = kq::Unit<QT>;
  std::memset(sb, 0, U::kSbBytes);
  sb[0] = block[F::kD]; sb[1] = block[F::kD + 1];
  if constexpr (F::kHasMin) { sb[2] = block[F::kDmin]; sb[3] = block[F::kDmin + 1]; }
  for (int g = 0; g < F::kGroups; ++g) {
    int sc, mn;
    kq::scale_min<QT>(block + F::kScaleOff, g, sc, mn);
    kq::put_bits(sb, U::bit_of(g, 0), F::kScaleBits, sc + F::kScaleBias);
    if constexpr (F::kHasMin) kq::put_bits(sb, U::bit_of(g, 1), F::kMinBits, mn);
  }
}

template <int QT>
int pack_units(uint8_t const* blocks, uint8_t* units, int n, int k, int experts) {
  using F = kq::Fmt<QT>;
  using U = kq::Unit<QT>;
  int64_t const nsb = k / 256;
  if (nsb % U::kSbPerUnit) return 24;
  int64_t const nu = nsb / U::kSbPerUnit;
  for (int e = 0; e < experts; ++e)
    for (int col = 0; col < n; ++col)
      for (int64_t sb = 0; sb < nsb; ++sb)
        pack_unit_sb<QT>(blocks + ((int64_t(e) * n + col) * nsb + sb) * F::kBytes,
                         units + ((int64_t(e) * nu + sb / U::kSbPerUnit) * n + col) * U::kUnitTotal +
                             (sb % U::kSbPerUnit) * U::kSbBytes);
  return 0;
}

// planes (+ optional fp16 planes) from raw blocks
template <int QT>
void raw_to_planes(uint8_t const* blocks, uint8_t* low, uint8_t* high, uint16_t* scale, uint16_t* zero,
                   int n, int k, int experts) {
  using F = kq::Fmt<QT>;
  constexpr int G = F::kGroups, GS = 256 / G;
  int64_t const nsb = k / 256;
  std::memset(low, 0, size_t(experts) * n * k * F::kLo / 8);
  if (F::kHi && high) std::memset(high, 0, size_t(experts) * n * k * F::kHi / 8);
  int64_t const scale_k = nsb * G;
  for (int e = 0; e < experts; ++e)
    for (int col = 0; col < n; ++col)
      for (int64_t sb = 0; sb < nsb; ++sb) {
        uint8_t const* blk = blocks + ((int64_t(e) * n + col) * nsb + sb) * F::kBytes;
        float const d = h2f(kq::load_u16(blk + F::kD));
        float const dmin = F::kHasMin ? h2f(kq::load_u16(blk + F::kDmin)) : 0.f;
        for (int g = 0; g < G; ++g) {
          int sc, mn;
          kq::scale_min<QT>(blk + F::kScaleOff, g, sc, mn);
          for (int j = 0; j < GS; ++j) {
            int const u = kq::code<QT>(blk, g, j) + F::kCodeBias;
            int64_t const logical = (int64_t(e) * n + col) * k + sb * 256 + g * GS + j;
            plane_put<F::kLo>(low, logical, u);
            if constexpr (F::kHi != 0) plane_put<(F::kHi ? F::kHi : 1)>(high, logical, u >> F::kLo);
          }
          if (scale) {
            // scale = half(dl), zero = half(-ml), then the offset-binary bias folded in float and rounded once
            uint16_t const s = f2h(d * float(sc));
            uint16_t const z0 = f2h(-(dmin * float(mn)));
            uint16_t const z = f2h(h2f(z0) - float(F::kCodeBias) * h2f(s));
            int64_t const dst = (int64_t(e) * scale_k + sb * G + g) * n + col;
            scale[dst] = s; zero[dst] = z;
          }
        }
      }
}

template <int QT>
int recover(uint8_t const* low, uint8_t const* high, uint8_t const* units, uint8_t* out, int n, int k, int experts) {
  using F = kq::Fmt<QT>;
  using U = kq::Unit<QT>;
  constexpr int G = F::kGroups, GS = 256 / G;
  int64_t const nsb = k / 256;
  if (nsb % U::kSbPerUnit) return 24;
  int64_t const nu = nsb / U::kSbPerUnit;
  std::memset(out, 0, size_t(experts) * n * nsb * F::kBytes);
  for (int e = 0; e < experts; ++e)
    for (int col = 0; col < n; ++col)
      for (int64_t sb = 0; sb < nsb; ++sb) {
        uint8_t* blk = out + ((int64_t(e) * n + col) * nsb + sb) * F::kBytes;
        uint8_t const* u = units + ((int64_t(e) * nu + sb / U::kSbPerUnit) * n + col) * U::kUnitTotal +
                           (sb % U::kSbPerUnit) * U::kSbBytes;
        blk[F::kD] = u[0]; blk[F::kD + 1] = u[1];
        if constexpr (F::kHasMin) { blk[F::kDmin] = u[2]; blk[F::kDmin + 1] = u[3]; }
        uint8_t* s = blk + F::kScaleOff;
        for (int g = 0; g < G; ++g) {
          int const sc = kq::get_bits(u, U::bit_of(g, 0), F::kScaleBits);          // raw stored pattern
          int const mn = F::kHasMin ? kq::get_bits(u, U::bit_of(g, 1), F::kMinBits) : 0;
          if constexpr (QT == 12 || QT == 13) {
            int const t = g & 3;
            if (g < 4) { s[t] |= uint8_t(sc & 63); s[4 + t] |= uint8_t(mn & 63); }
            else { s[8 + t] |= uint8_t((sc & 0xF) | ((mn & 0xF) << 4)); s[t] |= uint8_t((sc >> 4) << 6); s[4 + t] |= uint8_t((mn >> 4) << 6); }
          } else if constexpr (QT == 10) {
            s[g] = uint8_t((sc & 0xF) | (mn << 4));
          } else if constexpr (QT == 14) {
            s[g] = uint8_t(sc);
          } else {
            s[g & 7] |= uint8_t((sc & 0xF) << (4 * (g >> 3)));
            s[8 + (g & 3)] |= uint8_t(((sc >> 4) & 3) << (2 * (g >> 2)));
          }
          for (int j = 0; j < GS; ++j) {
            int64_t const logical = (int64_t(e) * n + col) * k + sb * 256 + g * GS + j;
            int q = plane_get<F::kLo>(low, logical);
            if constexpr (F::kHi != 0) q |= plane_get<(F::kHi ? F::kHi : 1)>(high, logical) << F::kLo;
            if constexpr (QT == 12 || QT == 13) {
              blk[(QT == 12 ? 16 : 48) + j + 32 * (g >> 1)] |= uint8_t((q & 0xF) << (4 * (g & 1)));
              if constexpr (QT == 13) blk[16 + j] |= uint8_t(((q >> 4) & 1) << g);
            } else if constexpr (QT == 14) {
              int const p = g & 1, q1 = (g >> 1) & 1, nn = (g >> 2) & 1, h = g >> 3;
              blk[j + 16 * p + 32 * q1 + 64 * h] |= uint8_t((q & 0xF) << (4 * nn));
              blk[128 + j + 16 * p + 32 * h] |= uint8_t(((q >> 4) & 3) << (2 * q1 + 4 * nn));
            } else {
              int const base = (QT == 11 ? 32 : 16) + j + 16 * (g & 1) + 32 * (g >> 3);
              blk[base] |= uint8_t((q & 3) << (2 * ((g >> 1) & 3)));
              if constexpr (QT == 11) blk[j + 16 * (g & 1)] |= uint8_t(((q >> 2) & 1) << (((g >> 1) & 3) + 4 * (g >> 3)));
            }
          }
        }
      }
  return 0;
}

bool shape_ok(int n, int k) { return n > 0 && n % 256 == 0 && k > 0 && k % 256 == 0; }

}  // namespace
}  // namespace qb

using namespace qb;

#define QT_DISPATCH(qtype, EXPR, DEFAULT)                                                             \
  switch (qtype) { case 10: { constexpr int Q = 10; return EXPR; } case 11: { constexpr int Q = 11; return EXPR; } \
                   case 12: { constexpr int Q = 12; return EXPR; } case 13: { constexpr int Q = 13; return EXPR; } \
                   case 14: { constexpr int Q = 14; return EXPR; } default: return DEFAULT; }

extern "C" int64_t quactlize_ppu_units_bytes(int n, int k, int qtype) {
  if (!shape_ok(n, k)) return -1;
  int64_t const nsb = k / 256;
#define EXPR ((nsb % kq::Unit<Q>::kSbPerUnit) ? int64_t(-1) : int64_t(n) * (nsb / kq::Unit<Q>::kSbPerUnit) * kq::Unit<Q>::kUnitTotal)
  QT_DISPATCH(qtype, EXPR, int64_t(-1))
#undef EXPR
}

extern "C" int quactlize_ppu_prepare_units_grouped(uint8_t const* blocks, uint8_t* units, int n, int k, int experts, int qtype) {
  if (!blocks || !units || experts <= 0 || !shape_ok(n, k)) return 20;
  QT_DISPATCH(qtype, pack_units<Q>(blocks, units, n, k, experts), 22)
}
extern "C" int quactlize_ppu_prepare_units(uint8_t const* blocks, uint8_t* units, int n, int k, int qtype) {
  return quactlize_ppu_prepare_units_grouped(blocks, units, n, k, 1, qtype);
}

// Same producer without the n%256 restriction of the GEMM-facing entries (GEMV artifacts accept any n).
extern "C" int quactlize_b200_pack_units(uint8_t const* blocks, uint8_t* units, int n, int k, int experts, int qtype) {
  if (!blocks || !units || experts <= 0 || n <= 0 || k <= 0 || k % 256) return 20;
  QT_DISPATCH(qtype, pack_units<Q>(blocks, units, n, k, experts), 22)
}

extern "C" int quactlize_ppu_prepare_fully_quantized_v1(uint8_t const* blocks, uint8_t* low, uint8_t* high, uint8_t* units,
                                                         int n, int k, int experts, int qtype) {
  if (!blocks || !low || !units || experts <= 0 || !shape_ok(n, k)) return 20;
  if ((qtype == 11 || qtype == 13 || qtype == 14) && !high) return 21;
#define EXPR ((k / 256) % kq::Unit<Q>::kSbPerUnit ? 24 : (raw_to_planes<Q>(blocks, low, high, nullptr, nullptr, n, k, experts), \
                                                       pack_units<Q>(blocks, units, n, k, experts)))
  QT_DISPATCH(qtype, EXPR, 22)
#undef EXPR
}

extern "C" int quactlize_ppu_recover_fully_quantized_v1(uint8_t const* low, uint8_t const* high, uint8_t const* units,
                                                         uint8_t* recovered, int n, int k, int experts, int qtype) {
  if (!low || !units || !recovered || experts <= 0 || !shape_ok(n, k)) return 20;
  if ((qtype == 11 || qtype == 13 || qtype == 14) && !high) return 21;
  QT_DISPATCH(qtype, recover<Q>(low, high, units, recovered, n, k, experts), 22)
}

// Scale-first artifact producer (the reference keeps this one in its torch extension, gguf_prepass_ops.cpp:809-878).
extern "C" int quactlize_b200_prepare_gemv(uint8_t const* blocks, uint8_t* low, uint8_t* high, uint16_t* scale,
                                            uint16_t* zero, int n, int k, int experts, int qtype) {
  if (!blocks || !low || !scale || !zero || experts <= 0 || n <= 0 || k <= 0 || k % 256) return 20;
  if ((qtype == 11 || qtype == 13 || qtype == 14) && !high) return 21;
  QT_DISPATCH(qtype, (raw_to_planes<Q>(blocks, low, high, scale, zero, n, k, experts), 0), 22)
}

// Placement entries: the placement of this library is the Native order, so both directions are copies.
static int copy_planes(uint8_t const* lo_in, uint8_t const* hi_in, uint8_t* lo_out, uint8_t* hi_out, int n, int k, int qtype) {
  if (!lo_in || !lo_out || !shape_ok(n, k) || kq::raw_bytes(qtype) == 0) return 20;
  int const hb = kq::hi_bits(qtype);
  if (hb && (!hi_in || !hi_out)) return 21;
  std::memcpy(lo_out, lo_in, size_t(n) * k * kq::lo_bits(qtype) / 8);
  if (hb) std::memcpy(hi_out, hi_in, size_t(n) * k * hb / 8);
  return 0;
}
extern "C" int quactlize_ppu_prepare_dense(uint8_t const* a, uint8_t const* b, uint8_t* c, uint8_t* d, int n, int k, int qtype) {
  return copy_planes(a, b, c, d, n, k, qtype);
}
extern "C" int quactlize_ppu_recover_dense(uint8_t const* a, uint8_t const* b, uint8_t* c, uint8_t* d, int n, int k, int qtype) {
  return copy_planes(a, b, c, d, n, k, qtype);
}
extern "C" int quactlize_ppu_prepare_dense_for_tile(uint8_t const* a, uint8_t const* b, uint8_t* c, uint8_t* d, int n, int k,
                                                     int qtype, int tile_k) {
  if (tile_k <= 0 || tile_k > 256 || (tile_k & (tile_k - 1))) return 23;
  return copy_planes(a, b, c, d, n, k, qtype);
}
extern "C" int quactlize_ppu_recover_dense_for_tile(uint8_t const* a, uint8_t const* b, uint8_t* c, uint8_t* d, int n, int k,
                                                     int qtype, int tile_k) {
  if (tile_k <= 0 || tile_k > 256 || (tile_k & (tile_k - 1))) return 23;
  return copy_planes(a, b, c, d, n, k, qtype);
}

// ---- planes placed by the reference's device library ("xplane" order) <-> Native planes -----------------------------
//
// The reference places code planes for its tensor-core converter in tiles of 64 columns x TileK codes (TileK 256; 128 for
// Q6_K).  Inside a tile the logical index  n_in_tile*TileK + k_in_tile  is mapped to a physical code slot by a pure
// BIT PERMUTATION, stated per (format, plane) as one stride per input bit, least significant first
// (quactlize/include/gguf_bc_vecdot.hpp:34-72); tiles are laid out k-tile-major, then 64-column tile, 256 code rows of
// 64 columns each, and TileK = 128 interleaves two k-tiles into one 256-row band (:81-95).  The same maps run both ways
// here, so an artifact placed for that library can be read (to Native, which every kernel of this library consumes)
// and written back byte for byte.
namespace qb {
namespace {

struct XplaneMap { int bits; int tile_k; uint16_t stride[14]; };

// input bit i of (n_in_tile*TileK + k_in_tile) -> stride[i]
constexpr XplaneMap kXLow2  = {14, 256, {0x8, 0x10, 0x20, 0x1, 0x2, 0x4, 0x40, 0x80, 0x100, 0x200, 0x400, 0x800, 0x1000, 0x2000}};
constexpr XplaneMap kXQ3Hi  = {14, 256, {0x10, 0x20, 0x40, 0x1, 0x2, 0x4, 0x8, 0x80, 0x100, 0x200, 0x400, 0x800, 0x1000, 0x2000}};
constexpr XplaneMap kXLow4  = {14, 256, {0x4, 0x8, 0x10, 0x1, 0x2, 0x20, 0x40, 0x80, 0x100, 0x200, 0x400, 0x800, 0x1000, 0x2000}};
constexpr XplaneMap kXQ5Hi  = {14, 256, {0x10, 0x20, 0x40, 0x1, 0x2, 0x4, 0x80, 0x800, 0x100, 0x200, 0x400, 0x8, 0x1000, 0x2000}};
constexpr XplaneMap kXQ6Lo  = {13, 128, {0x4, 0x8, 0x10, 0x1, 0x2, 0x20, 0x40, 0x80, 0x100, 0x200, 0x400, 0x800, 0x1000, 0}};
constexpr XplaneMap kXQ6Hi  = {13, 128, {0x8, 0x10, 0x20, 0x1, 0x2, 0x4, 0x40, 0x80, 0x100, 0x200, 0x400, 0x800, 0x1000, 0}};

XplaneMap const* xplane_map(int qtype, bool high) {
  switch (qtype) {
    case 10: return high ? nullptr : &kXLow2;
    case 11: return high ? &kXQ3Hi : &kXLow2;
    case 12: return high ? nullptr : &kXLow4;
    case 13: return high ? &kXQ5Hi : &kXLow4;
    case 14: return high ? &kXQ6Hi : &kXQ6Lo;
    default: return nullptr;
  }
}

inline int64_t xplane_slot(XplaneMap const& m, int n, int k, int num_cols) {
  int const kt = k / m.tile_k, kr = k % m.tile_k, nt = n / 64, nr = n % 64;
  int const logical = nr * m.tile_k + kr;
  int rel = 0;
  for (int i = 0; i < m.bits; ++i) if ((logical >> i) & 1) rel += m.stride[i];
  if (m.tile_k == 128) {
    int const rows = (rel & 127) | ((rel & ~127) << 1) | ((kt & 1) << 7);
    return int64_t(kt / 2) * num_cols * 256 + int64_t(nt) * 64 * 256 + rows;
  }
  return int64_t(kt) * num_cols * 256 + int64_t(nt) * 64 * 256 + rel;
}

template <int Bits>
void xplane_move(XplaneMap const& m, uint8_t const* src, uint8_t* dst, int n, int k, bool to_native) {
  std::memset(dst, 0, size_t(n) * k * Bits / 8);
  for (int col = 0; col < n; ++col)
    for (int kk = 0; kk < k; ++kk) {
      int64_t const native = int64_t(col) * k + kk, placed = xplane_slot(m, col, kk, n);
      if (to_native) plane_put<Bits>(dst, native, plane_get<Bits>(src, placed));
      else plane_put<Bits>(dst, placed, plane_get<Bits>(src, native));
    }
}

int xplane_convert(uint8_t const* lo_in, uint8_t const* hi_in, uint8_t* lo_out, uint8_t* hi_out, int n, int k, int qtype,
                   bool to_native) {
  if (!lo_in || !lo_out || n <= 0 || k <= 0 || n % 64 || k % 256 || kq::raw_bytes(qtype) == 0) return 20;
  int const hb = kq::hi_bits(qtype);
  if (hb && (!hi_in || !hi_out)) return 21;
  XplaneMap const* ml = xplane_map(qtype, false);
  if (kq::lo_bits(qtype) == 2) xplane_move<2>(*ml, lo_in, lo_out, n, k, to_native);
  else xplane_move<4>(*ml, lo_in, lo_out, n, k, to_native);
  if (hb) {
    XplaneMap const* mh = xplane_map(qtype, true);
    if (hb == 1) xplane_move<1>(*mh, hi_in, hi_out, n, k, to_native);
    else xplane_move<2>(*mh, hi_in, hi_out, n, k, to_native);
  }
  return 0;
}

}  // namespace
}  // namespace qb

extern "C" int quactlize_b200_xplane_to_native(uint8_t const* low_placed, uint8_t const* high_placed, uint8_t* low_native,
                                                uint8_t* high_native, int n, int k, int qtype) {
  return qb::xplane_convert(low_placed, high_placed, low_native, high_native, n, k, qtype, true);
}
extern "C" int quactlize_b200_native_to_xplane(uint8_t const* low_native, uint8_t const* high_native, uint8_t* low_placed,
                                                uint8_t* high_placed, int n, int k, int qtype) {
  return qb::xplane_convert(low_native, high_native, low_placed, high_placed, n, k, qtype, false);
}
// The physical code slot of logical (n, k) in a placed plane of `num_cols` columns; -1 for a plane the format lacks.
extern "C" long long quactlize_b200_xplane_slot(int qtype, int high, int n, int k, int num_cols) {
  qb::XplaneMap const* m = qb::xplane_map(qtype, high != 0);
  if (!m || n < 0 || k < 0 || num_cols <= 0 || n >= num_cols) return -1;
  return qb::xplane_slot(*m, n, k, num_cols);
}
