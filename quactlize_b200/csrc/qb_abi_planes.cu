// C ABI of the bit-plane GEMV family: scale-first artifact (planes + fp16 scale/zero), merged artifact (planes +
// packed units), and the additive generic per-group entries (W4/W2/W1, fp16 or bf16 activations).
// Signatures and return codes follow quactlize/csrc/device/ppu_backend.cu:241-293,398-509 of the reference.
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "qb_internal.hpp"
#include "qb_kquant.cuh"
#include "qb_runtime.hpp"
#include "../../include/quactlize_b200.h"

using namespace qb;

namespace {
constexpr char const* kDenseCudaConfig = "gemv_lowbit";

PlaneGemvDesc kquant_planes(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                            uint16_t const* zero, void* out, int total_rows, int n, int k, int qtype, int experts,
                            int const* offsets, int max_rows) {
  PlaneGemvDesc d{};
  d.act = act; d.low = low; d.high = high; d.scale = scale; d.zero = zero; d.out = out;
  d.offsets = experts > 0 ? offsets : nullptr;
  d.n = n; d.k = k; d.experts = experts > 0 ? experts : 1; d.m_rows = total_rows; d.max_rows = max_rows;
  d.lo_bits = kq::lo_bits(qtype); d.hi_bits = kq::hi_bits(qtype); d.group_size = kq::group_size(qtype);
  d.scale_mode = 0; d.qtype = qtype; d.code_offset = 0; d.act_bf16 = 0; d.out_kind = 0;
  return d;
}
}  // namespace

extern "C" int32_t quactlize_ppu_gemv_lowbit_config_valid_v1(int m, int n, int k, int group_size, int qtype,
                                                             char const* config_name) {
  bool const name_ok = !config_name || !config_name[0] || std::strcmp(config_name, kDenseCudaConfig) == 0;
  return name_ok && kq::raw_bytes(qtype) != 0 && m > 0 && n > 0 && n % 256 == 0 && k > 0 && k % 256 == 0 &&
         group_size == kq::group_size(qtype);
}

extern "C" int quactlize_ppu_gemv_lowbit(uint16_t const* a, uint8_t const* low, uint8_t const* high,
                                         uint16_t const* scale, uint16_t const* zero, uint16_t* out, int total_rows,
                                         int n, int k, int group_size, int qtype, int experts, int const* offsets,
                                         int max_rows) {
  if (kq::raw_bytes(qtype) == 0) return 6;
  if (!a || !low || !scale || !zero || !out || total_rows <= 0 || n <= 0 || k <= 0 || k % 256 ||
      group_size != kq::group_size(qtype) || (kq::hi_bits(qtype) && !high) || (experts > 0 && (!offsets || max_rows <= 0)))
    return 40;
  rt_clear_error();
  int const we = experts > 0 ? experts : 1;
  size_t const lo_per = size_t(n) * k * kq::lo_bits(qtype) / 8, hi_per = size_t(n) * k * kq::hi_bits(qtype) / 8;
  size_t const sc_per = size_t(k / group_size) * n;
  DevBuf da(size_t(total_rows) * k * 2), dl(we * lo_per), dh(we * hi_per), ds(we * sc_per * 2), dz(we * sc_per * 2),
      dout(size_t(total_rows) * n * 2), doff(experts > 0 ? size_t(experts + 1) * 4 : 0);
  da.from_host(a); dl.from_host(low); if (hi_per) dh.from_host(high); ds.from_host(scale); dz.from_host(zero);
  if (experts > 0) doff.from_host(offsets);
  if (!rt_ok()) return kRuntimeError;
  PlaneGemvDesc d = kquant_planes(da.as<uint16_t>(), dl.as<uint8_t>(), hi_per ? dh.as<uint8_t>() : nullptr, ds.as<uint16_t>(),
                                  dz.as<uint16_t>(), dout.p, total_rows, n, k, qtype, experts, doff.as<int>(),
                                  experts > 0 ? max_rows : total_rows);
  int const rc = enqueue_plane_gemv(d, nullptr);
  if (rc) return rc;
  if (!rt_check_launch("scale-first GEMV") || !rt_sync(nullptr, "scale-first GEMV") ||
      !rt_device_status_ok(nullptr, "scale-first GEMV")) return kRuntimeError;
  return rt_copy_out(dout.p, out, size_t(total_rows) * n * 2, nullptr) ? 0 : kRuntimeError;
}

extern "C" int quactlize_ppu_gemv_lowbit_config_v1(uint16_t const* a, uint8_t const* low, uint8_t const* high,
                                                   uint16_t const* scale, uint16_t const* zero, uint16_t* out, int m,
                                                   int n, int k, int group_size, int qtype, char const* config_name) {
  if (config_name && config_name[0] && std::strcmp(config_name, kDenseCudaConfig) != 0)
    std::fprintf(stderr, "[quactlize_b200] dense CUDA config '%s' is not compiled in; running default '%s'\n",
                 config_name, kDenseCudaConfig);
  return quactlize_ppu_gemv_lowbit(a, low, high, scale, zero, out, m, n, k, group_size, qtype, 0, nullptr, m);
}

extern "C" int quactlize_ppu_gemv_lowbit_dev_v1(uint16_t const* a, uint8_t const* low, uint8_t const* high,
                                                uint16_t const* scale, uint16_t const* zero, uint16_t* out, int m, int n,
                                                int k, int group_size, int qtype, void* stream, char const* config_name) {
  if (!a || !low || !scale || !zero || !out || (kq::hi_bits(qtype) && !high) ||
      !quactlize_ppu_gemv_lowbit_config_valid_v1(m, n, k, group_size, qtype, config_name)) return 40;
  rt_clear_error();
  PlaneGemvDesc d = kquant_planes(a, low, high, scale, zero, out, m, n, k, qtype, 0, nullptr, m);
  int const rc = enqueue_plane_gemv(d, static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return rt_check_launch("scale-first GEMV enqueue") ? 0 : kRuntimeError;
}

// Ragged MoE on device pointers (the reference exposes the grouped form only through its host-pointer entry).
extern "C" int quactlize_b200_gemv_lowbit_moe_dev_v1(uint16_t const* a, uint8_t const* low, uint8_t const* high,
                                                     uint16_t const* scale, uint16_t const* zero, uint16_t* out,
                                                     int total_rows, int n, int k, int group_size, int qtype, int experts,
                                                     int const* offsets, int max_rows, void* stream) {
  if (kq::raw_bytes(qtype) == 0) return 6;
  if (!a || !low || !scale || !zero || !out || !offsets || total_rows <= 0 || n <= 0 || k <= 0 || k % 256 || experts <= 0 ||
      max_rows <= 0 || group_size != kq::group_size(qtype) || (kq::hi_bits(qtype) && !high)) return 40;
  rt_clear_error();
  PlaneGemvDesc d = kquant_planes(a, low, high, scale, zero, out, total_rows, n, k, qtype, experts, offsets, max_rows);
  int const rc = enqueue_plane_gemv(d, static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return rt_check_launch("scale-first MoE GEMV enqueue") ? 0 : kRuntimeError;
}

// ---- merged artifact: planes + packed units ----------------------------------------------------------------------
static int bc_check(uint16_t const* x, uint8_t const* low, uint8_t const* high, uint8_t const* units, int const* offsets,
                    float* out, int total_rows, int n, int k, int experts, int max_rows, int qtype) {
  if (!x || !low || !units || !out || total_rows <= 0 || n <= 0 || n % 256 || k <= 0 || k % 256 || experts < 0 ||
      (experts > 0 && (!offsets || max_rows <= 0)) || (experts == 0 && total_rows != 1)) return 13;
  if (kq::raw_bytes(qtype) == 0) return 16;
  if (kq::hi_bits(qtype) && !high) return 14;
  if ((k / 256) % ((qtype == 11 || qtype == 14) ? 2 : 1)) return 15;
  return 0;
}
static PlaneGemvDesc bc_desc(uint16_t const* x, uint8_t const* low, uint8_t const* high, uint8_t const* units,
                             int const* offsets, float* out, int total_rows, int n, int k, int experts, int max_rows, int qtype) {
  PlaneGemvDesc d{};
  d.act = x; d.low = low; d.high = high; d.units = units; d.out = out;
  d.offsets = experts > 0 ? offsets : nullptr;
  d.n = n; d.k = k; d.experts = experts > 0 ? experts : 1; d.m_rows = total_rows; d.max_rows = experts > 0 ? max_rows : total_rows;
  d.lo_bits = kq::lo_bits(qtype); d.hi_bits = kq::hi_bits(qtype); d.group_size = kq::group_size(qtype);
  d.scale_mode = 1; d.qtype = qtype; d.out_kind = 1;
  return d;
}

extern "C" int quactlize_ppu_bc_gemv_dev_v1(uint16_t const* x, uint8_t const* low, uint8_t const* high,
                                            uint8_t const* units, int const* offsets, float* out, int total_rows, int n,
                                            int k, int experts, int max_rows, int qtype, void* stream) {
  int const bad = bc_check(x, low, high, units, offsets, out, total_rows, n, k, experts, max_rows, qtype);
  if (bad) return bad;
  rt_clear_error();
  int const rc = enqueue_plane_gemv(bc_desc(x, low, high, units, offsets, out, total_rows, n, k, experts, max_rows, qtype),
                                    static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return rt_check_launch("merged-artifact GEMV enqueue") ? 0 : kRuntimeError;
}

extern "C" int quactlize_ppu_bc_gemv(uint16_t const* x, uint8_t const* low, uint8_t const* high, uint8_t const* units,
                                     int const* offsets, float* out, int total_rows, int n, int k, int experts,
                                     int max_rows, int qtype) {
  int const bad = bc_check(x, low, high, units, offsets, out, total_rows, n, k, experts, max_rows, qtype);
  if (bad) return bad;
  rt_clear_error();
  int const we = experts > 0 ? experts : 1;
  int const p = (qtype == 11 || qtype == 14) ? 2 : 1;
  int const sbb = qtype == 10 ? 20 : qtype == 11 ? 14 : qtype == 14 ? 18 : 16;
  size_t const lo_b = size_t(we) * n * k * kq::lo_bits(qtype) / 8, hi_b = size_t(we) * n * k * kq::hi_bits(qtype) / 8;
  size_t const un_b = size_t(we) * (k / 256 / p) * n * (size_t(sbb) * p);
  DevBuf dx(size_t(total_rows) * k * 2), dl(lo_b), dh(hi_b), du(un_b), doff(experts > 0 ? size_t(experts + 1) * 4 : 0),
      dout(size_t(total_rows) * n * 4);
  dx.from_host(x); dl.from_host(low); if (hi_b) dh.from_host(high); du.from_host(units);
  if (experts > 0) doff.from_host(offsets);
  if (!rt_ok()) return kRuntimeError;
  int const rc = enqueue_plane_gemv(bc_desc(dx.as<uint16_t>(), dl.as<uint8_t>(), hi_b ? dh.as<uint8_t>() : nullptr,
                                            du.as<uint8_t>(), doff.as<int>(), dout.as<float>(), total_rows, n, k, experts,
                                            max_rows, qtype), nullptr);
  if (rc) return rc;
  if (!rt_check_launch("merged-artifact GEMV") || !rt_sync(nullptr, "merged-artifact GEMV") ||
      !rt_device_status_ok(nullptr, "merged-artifact GEMV")) return kRuntimeError;
  return rt_copy_out(dout.p, out, size_t(total_rows) * n * 4, nullptr) ? 0 : kRuntimeError;
}

// ---- generic per-group planes (W4A16 / W2A16 / W1A16 and two-plane combinations) ---------------------------------
extern "C" int quactlize_b200_gemv_plane_dev_v1(void const* act, uint8_t const* low, uint8_t const* high,
                                                uint16_t const* scale, uint16_t const* zero, void* out, int total_rows,
                                                int n, int k, int bits_lo, int bits_hi, int group_size, int code_offset,
                                                int act_dtype, int out_dtype, int experts, int const* offsets,
                                                int max_rows, void* stream) {
  if (!act || !low || !scale || !out || total_rows <= 0 || n <= 0 || k <= 0 || k % 256 || group_size <= 0 ||
      (bits_hi && !high) || experts < 0 || (experts > 0 && (!offsets || max_rows <= 0)) ||
      act_dtype < 0 || act_dtype > 1 || out_dtype < 0 || out_dtype > 2) return 40;
  rt_clear_error();
  PlaneGemvDesc d{};
  d.act = act; d.low = low; d.high = bits_hi ? high : nullptr; d.scale = scale; d.zero = zero; d.out = out;
  d.offsets = experts > 0 ? offsets : nullptr;
  d.n = n; d.k = k; d.experts = experts > 0 ? experts : 1; d.m_rows = total_rows;
  d.max_rows = experts > 0 ? max_rows : total_rows;
  d.lo_bits = bits_lo; d.hi_bits = bits_hi; d.group_size = group_size; d.scale_mode = 0; d.qtype = 0;
  d.code_offset = code_offset; d.act_bf16 = act_dtype; d.out_kind = out_dtype;
  int const rc = enqueue_plane_gemv(d, static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return rt_check_launch("plane GEMV enqueue") ? 0 : kRuntimeError;
}
