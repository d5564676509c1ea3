// C ABI of the tensor-core family: dense and grouped mixed-input GEMM over the scale-first artifact (planes + fp16
// scale/zero) and over the fully-quantized artifact (planes + packed units), plus the config inventory.
// Signatures and return codes follow quactlize/csrc/device/ppu_dense_backend.cu:603-1251 of the reference
// (30 bad arguments, 32 wrong group size, 33 unsupported format, 37 workspace too small, 41 runtime failure).
//
// Code conventions of the reference's converters, kept at this boundary: the int4-low formats (Q4_K, Q5_K, Q6_K)
// arrive with zero planes that assume the converter emits (low - 8) (gguf_prepass_ops.cpp:912-920), the int2-low
// formats (Q2_K, Q3_K) with an unbiased converter; the scale-only grouped entry centres two-plane codes at 2^(W-1).
// The fully-quantized entries derive fp16 scale/zero planes from the packed units into the caller's workspace
// (one bit-exact pre-pass launch) and then run the same GEMM.
#include <cstdint>
#include <cstdio>
#include <algorithm>
#include <cstring>

#include "qb_internal.hpp"
#include "qb_kquant.cuh"
#include "qb_runtime.hpp"
#include "../../include/quactlize_b200.h"

using namespace qb;

namespace {
// Two tensor-core tactics are compiled (CTA tile 256 x 256 and 128 x 128, K stage 64); a null or empty name lets the launcher
// choose by rows per expert, a known name forces that tile, an unknown name is declined with a message and the default runs.
constexpr char const* kTensorConfig = "256x256x64:tcgen05";
constexpr char const* kTensorConfigSmall = "128x128x64:tcgen05";
// grouped only: the decode tactic -- 128 x 128 tiles with two-deep rings (several CTAs per SM) and K split over gridDim.z
// into fp32 partial planes that a light reduce kernel sums (quactlize/include/ppu_aiu_gemm_mixed_input_group.hpp:120-131,
// 289-309 in the reference: slice z writes its own D plane).  Needs workspace for the partials; without it, it runs unsplit.
constexpr char const* kTensorConfigSplitK = "128x128x64:tcgen05:splitk";
quactlize_ppu_config_v1 const kDenseConfigs[] = {{false, kTensorConfig, 256, 256, 128, 256, 3}, {false, kTensorConfigSmall, 128, 128, 128, 128, 4},
                                                 {true, "gemv_lowbit", 0, 0, 0, 0, 0}};
quactlize_ppu_config_v1 const kGroupedConfigs[] = {{false, kTensorConfig, 256, 256, 128, 256, 3}, {false, kTensorConfigSmall, 128, 128, 128, 128, 4},
                                                   {false, kTensorConfigSplitK, 128, 128, 128, 128, 2}, {true, "vecdot_moe", 0, 0, 0, 0, 0}};
constexpr int kSplitKTile = 129;                   // tile_of() value of the split-K tactic (a 128 tile, shallow, split)

int tile_of(char const* name) {                    // 0 = default choice, 128 / 256 = forced tile, -1 = unknown name
  if (!name || !name[0]) return 0;
  if (std::strcmp(name, kTensorConfig) == 0) return 256;
  if (std::strcmp(name, kTensorConfigSmall) == 0) return 128;
  if (std::strcmp(name, kTensorConfigSplitK) == 0) return kSplitKTile;
  return -1;
}
bool tensor_name_ok(char const* name) { return tile_of(name) >= 0; }
int decline(char const* name) {                    // the tile to run
  int const t = tile_of(name);
  if (t >= 0) return t;
  std::fprintf(stderr, "[quactlize_b200] tensor config '%s' is not compiled in; running the default choice\n", name);
  return 0;
}
bool shape_ok(int n, int k) { return n > 0 && n % 256 == 0 && k > 0 && k % 256 == 0; }
int converter_offset(int qtype) { return (qtype == 12 || qtype == 13 || qtype == 14) ? -8 : 0; }
int placed_zmul(int qtype) { return qtype == 11 ? -4 : (qtype == 12 || qtype == 13) ? 8 : qtype == 14 ? -24 : 0; }
int centred_offset(int qtype) {                     // scale-only grouped: centre of the concatenated code
  int const w = kq::lo_bits(qtype) + kq::hi_bits(qtype);
  return kq::hi_bits(qtype) ? -(1 << (w - 1)) : (kq::lo_bits(qtype) == 4 ? -8 : 0);
}
int sb_per_unit(int qtype) { return (qtype == 11 || qtype == 14) ? 2 : 1; }
int unit_sb_bytes(int qtype) { return qtype == 10 ? 20 : qtype == 11 ? 14 : qtype == 14 ? 18 : 16; }
int64_t plane_elems(int n, int k, int experts, int qtype) { return int64_t(experts) * (k / kq::group_size(qtype)) * n; }

GemmDesc kq_desc(void const* act, uint8_t const* low, uint8_t const* high, void const* scale, void const* zero, void* out,
                 int rows, int n, int k, int qtype, int experts, int const* offsets, int code_offset, int tile) {
  GemmDesc d{};
  d.act = act; d.low = low; d.high = kq::hi_bits(qtype) ? high : nullptr; d.scale = scale; d.zero = zero; d.out = out;
  d.offsets = offsets; d.total_rows = rows; d.n = n; d.k = k; d.experts = experts;
  d.group_size = kq::group_size(qtype); d.lo_bits = kq::lo_bits(qtype); d.hi_bits = kq::hi_bits(qtype);
  d.code_offset = code_offset; d.act_bf16 = 0; d.tile = tile == kSplitKTile ? 128 : tile;
  d.shallow = tile == kSplitKTile ? 1 : 0;
  return d;
}

// split-K partial planes carved from what is left of a workspace; no room (or nothing to gain) leaves the launch unsplit
void attach_splitk(GemmDesc& d, int tile, void* ws, int64_t ws_bytes) {
  if (tile != kSplitKTile || d.experts <= 0) return;
  int const s = splitk_auto(std::min(d.experts, d.total_rows), d.n, d.k);
  int64_t const need = int64_t(s) * d.total_rows * d.n * 4;
  uintptr_t const base = (reinterpret_cast<uintptr_t>(ws) + 15) & ~uintptr_t(15);
  if (s > 1 && ws && int64_t(base - reinterpret_cast<uintptr_t>(ws)) + need <= ws_bytes) { d.splits = s; d.partial = reinterpret_cast<float*>(base); }
}
int64_t splitk_extra_bytes(int experts, int max_rows, int n) {      // room for 8 slices of a decode-sized problem, else none
  int64_t const rows = int64_t(experts) * max_rows;
  return rows <= 4096 ? 8 * rows * n * 4 + 16 : 0;
}

// cumulative offsets from per-expert row counts; false if a count is negative or the sum disagrees
bool make_offsets(int const* rows_per_expert, int experts, int total_rows, int* off) {
  off[0] = 0;
  for (int e = 0; e < experts; ++e) { if (rows_per_expert[e] < 0) return false; off[e + 1] = off[e] + rows_per_expert[e]; }
  return off[experts] == total_rows;
}

// host-pointer scale-first GEMM (dense: experts == 0)
int host_planes_gemm(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale, uint16_t const* zero,
                     uint16_t* out, int rows, int n, int k, int qtype, int experts, int const* rows_per_expert,
                     int code_offset, int tile, char const* what) {
  rt_clear_error();
  int const we = experts > 0 ? experts : 1;
  size_t const lo_b = size_t(we) * n * k * kq::lo_bits(qtype) / 8, hi_b = size_t(we) * n * k * kq::hi_bits(qtype) / 8;
  size_t const pe = size_t(plane_elems(n, k, we, qtype));
  int offs[1025];
  if (experts > 1024) return 30;
  if (experts > 0 && !make_offsets(rows_per_expert, experts, rows, offs)) return 30;
  DevBuf da(size_t(rows) * k * 2), dl(lo_b), dh(hi_b), ds(pe * 2), dz(zero ? pe * 2 : 0), dout(size_t(rows) * n * 2),
      doff(experts > 0 ? size_t(experts + 1) * 4 : 0);
  da.from_host(act); dl.from_host(low); if (hi_b) dh.from_host(high); ds.from_host(scale); if (zero) dz.from_host(zero);
  if (experts > 0) doff.from_host(offs);
  if (!rt_ok()) return kRuntimeError;
  GemmDesc d = kq_desc(da.p, dl.as<uint8_t>(), dh.as<uint8_t>(), ds.p, zero ? dz.p : nullptr, dout.p, rows, n, k, qtype,
                       experts, doff.as<int>(), code_offset, tile);
  int const rc = enqueue_mixed_gemm(d, nullptr);
  if (rc) return rc;
  if (!rt_check_launch(what) || !rt_sync(nullptr, what) || !rt_device_status_ok(nullptr, what)) return kRuntimeError;
  return rt_copy_out(dout.p, out, size_t(rows) * n * 2, nullptr) ? 0 : kRuntimeError;
}

// device-pointer fully-quantized GEMM: units -> fp16 planes in the workspace -> GEMM
int dev_units_gemm(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint8_t const* units, int const* offsets,
                   uint16_t* out, int rows, int n, int k, int experts, int qtype, void* workspace, int64_t workspace_bytes,
                   cudaStream_t s, int tile, char const* what) {
  int const we = experts > 0 ? experts : 1;
  int64_t const pe = plane_elems(n, k, we, qtype);
  if (!workspace || workspace_bytes < pe * 4) return 37;
  __half* sc = reinterpret_cast<__half*>(workspace);
  __half* zr = sc + pe;
  rt_clear_error();
  // the reference's placed-code convention (quactlize/formats.py:315-321): int4-low codes are converted as (low - 8) and
  // the zero plane carries the matching correction, which keeps |zero| small and its fp16 rounding with it
  if (!enqueue_prepass_unit(units, sc, zr, we, n, k / 256, qtype, placed_zmul(qtype), s)) return 33;
  GemmDesc d = kq_desc(act, low, high, sc, zr, out, rows, n, k, qtype, experts, offsets, converter_offset(qtype), tile);
  attach_splitk(d, tile, reinterpret_cast<uint8_t*>(workspace) + pe * 4, workspace_bytes - pe * 4);
  int const rc = enqueue_mixed_gemm(d, s);
  if (rc) return rc;
  return rt_check_launch(what) ? 0 : kRuntimeError;
}

int host_units_gemm(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint8_t const* units,
                    int const* rows_per_expert, uint16_t* out, int rows, int n, int k, int experts, int qtype, int tile,
                    char const* what) {
  rt_clear_error();
  int const we = experts > 0 ? experts : 1;
  size_t const lo_b = size_t(we) * n * k * kq::lo_bits(qtype) / 8, hi_b = size_t(we) * n * k * kq::hi_bits(qtype) / 8;
  size_t const un_b = size_t(we) * (k / 256) * n * unit_sb_bytes(qtype);
  int64_t const pe = plane_elems(n, k, we, qtype);
  int offs[1025];
  if (experts > 1024) return 30;
  if (experts > 0 && !make_offsets(rows_per_expert, experts, rows, offs)) return 30;
  DevBuf da(size_t(rows) * k * 2), dl(lo_b), dh(hi_b), du(un_b), ws(size_t(pe) * 4), dout(size_t(rows) * n * 2),
      doff(experts > 0 ? size_t(experts + 1) * 4 : 0);
  da.from_host(act); dl.from_host(low); if (hi_b) dh.from_host(high); du.from_host(units);
  if (experts > 0) doff.from_host(offs);
  if (!rt_ok()) return kRuntimeError;
  int const rc = dev_units_gemm(da.as<uint16_t>(), dl.as<uint8_t>(), dh.as<uint8_t>(), du.as<uint8_t>(), doff.as<int>(),
                                dout.as<uint16_t>(), rows, n, k, experts, qtype, ws.p, pe * 4, nullptr, tile, what);
  if (rc) return rc;
  if (!rt_sync(nullptr, what) || !rt_device_status_ok(nullptr, what)) return kRuntimeError;
  return rt_copy_out(dout.p, out, size_t(rows) * n * 2, nullptr) ? 0 : kRuntimeError;
}

bool fq_ok(int k, int qtype) { return kq::raw_bytes(qtype) != 0 && (k / 256) % sb_per_unit(qtype) == 0; }
}  // namespace

// ---- config inventory (quactlize/include/quactlize_ppu_config.h:42-119) ------------------------------------------------
extern "C" int32_t quactlize_ppu_list_configs(quactlize_ppu_config_v1 const** configs) {
  if (configs) *configs = kDenseConfigs;
  return 3;
}
extern "C" int32_t quactlize_ppu_list_grouped_configs(quactlize_ppu_config_v1 const** configs) {
  if (configs) *configs = kGroupedConfigs;
  return 4;
}
extern "C" int32_t quactlize_ppu_dense_lowbit_config_valid_v1(int m, int n, int k, int group_size, int qtype, char const* name) {
  return tensor_name_ok(name) && tile_of(name) != kSplitKTile && kq::raw_bytes(qtype) != 0 && m > 0 && shape_ok(n, k) && group_size == kq::group_size(qtype);
}
extern "C" int32_t quactlize_ppu_dense_fully_quantized_config_valid_v1(int m, int n, int k, int group_size, int qtype, char const* name) {
  return quactlize_ppu_dense_lowbit_config_valid_v1(m, n, k, group_size, qtype, name) && fq_ok(k, qtype);
}
extern "C" int32_t quactlize_ppu_grouped_lowbit_config_valid_v1(int total_rows, int n, int k, int group_size, int experts,
                                                                int max_rows, int qtype, char const* name) {
  return tensor_name_ok(name) && kq::raw_bytes(qtype) != 0 && total_rows > 0 && experts > 0 && max_rows > 0 && shape_ok(n, k) &&
         group_size == kq::group_size(qtype);
}
extern "C" int32_t quactlize_ppu_grouped_fully_quantized_config_valid_v1(int total_rows, int n, int k, int group_size, int experts,
                                                                         int max_rows, int qtype, char const* name) {
  return quactlize_ppu_grouped_lowbit_config_valid_v1(total_rows, n, k, group_size, experts, max_rows, qtype, name) && fq_ok(k, qtype);
}
static int32_t list_one(quactlize_ppu_config_v2* configs, int32_t capacity, bool valid) {   // both tactics run every valid shape
  if (valid && configs && capacity > 0) configs[0] = {false, kTensorConfig, 256, 256, 64, 128, 256, 3};
  if (valid && configs && capacity > 1) configs[1] = {false, kTensorConfigSmall, 128, 128, 64, 128, 128, 4};
  return valid ? 2 : 0;
}
extern "C" int32_t quactlize_ppu_list_valid_dense_lowbit_configs_v2(quactlize_ppu_config_v2* c, int32_t cap, int m, int n, int k, int gs, int qtype) {
  return list_one(c, cap, quactlize_ppu_dense_lowbit_config_valid_v1(m, n, k, gs, qtype, nullptr));
}
extern "C" int32_t quactlize_ppu_list_valid_dense_fully_quantized_configs_v2(quactlize_ppu_config_v2* c, int32_t cap, int m, int n, int k, int gs, int qtype) {
  return list_one(c, cap, quactlize_ppu_dense_fully_quantized_config_valid_v1(m, n, k, gs, qtype, nullptr));
}
extern "C" int32_t quactlize_ppu_list_valid_grouped_fully_quantized_configs_v2(quactlize_ppu_config_v2* c, int32_t cap, int total_rows,
                                                                               int n, int k, int gs, int experts, int max_rows, int qtype) {
  bool const valid = quactlize_ppu_grouped_fully_quantized_config_valid_v1(total_rows, n, k, gs, experts, max_rows, qtype, nullptr);
  int32_t const base = list_one(c, cap, valid);
  if (valid && c && cap > 2) c[2] = {false, kTensorConfigSplitK, 128, 128, 64, 128, 128, 2};
  return valid ? base + 1 : 0;
}

// ---- dense, scale-first ------------------------------------------------------------------------------------------------
extern "C" int quactlize_ppu_dense_lowbit_config_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                    uint16_t const* scale, uint16_t const* zero, uint16_t* out, int m, int n,
                                                    int k, int group_size, int qtype, char const* config_name) {
  if (!act || !low || !scale || !zero || !out || m <= 0 || !shape_ok(n, k)) return 30;
  if (kq::raw_bytes(qtype) == 0) return 33;
  if (group_size != kq::group_size(qtype) || (kq::hi_bits(qtype) && !high)) return 32;
  int const tile = decline(config_name);
  return host_planes_gemm(act, low, high, scale, zero, out, m, n, k, qtype, 0, nullptr, converter_offset(qtype), tile, "scale-first dense GEMM");
}
extern "C" int quactlize_ppu_dense_lowbit(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                          uint16_t const* zero, uint16_t* out, int m, int n, int k, int group_size, int qtype) {
  return quactlize_ppu_dense_lowbit_config_v1(act, low, high, scale, zero, out, m, n, k, group_size, qtype, nullptr);
}

// ---- dense, fully quantized ----------------------------------------------------------------------------------------------
extern "C" int quactlize_ppu_dense_fully_quantized_config_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                             uint8_t const* units, uint16_t* out, int m, int n, int k, int qtype,
                                                             char const* config_name) {
  if (!act || !low || !units || !out || m <= 0 || !shape_ok(n, k)) return 30;
  if (!fq_ok(k, qtype) || (kq::hi_bits(qtype) && !high)) return 33;
  int const tile = decline(config_name);
  return host_units_gemm(act, low, high, units, nullptr, out, m, n, k, 0, qtype, tile, "fully-quantized dense GEMM");
}
extern "C" int quactlize_ppu_dense_fully_quantized(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                   uint8_t const* units, uint16_t* out, int m, int n, int k, int qtype) {
  return quactlize_ppu_dense_fully_quantized_config_v1(act, low, high, units, out, m, n, k, qtype, nullptr);
}
extern "C" int64_t quactlize_ppu_dense_fully_quantized_workspace_bytes_v1(int m, int n, int k, int qtype) {
  if (m <= 0 || !shape_ok(n, k) || !fq_ok(k, qtype)) return -1;
  return plane_elems(n, k, 1, qtype) * 4;
}
extern "C" int quactlize_ppu_dense_fully_quantized_dev_v2(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                          uint8_t const* units, uint16_t* out, int m, int n, int k, int qtype,
                                                          void* workspace, int64_t workspace_bytes, void* stream,
                                                          char const* config_name) {
  int64_t const need = quactlize_ppu_dense_fully_quantized_workspace_bytes_v1(m, n, k, qtype);
  if (!act || !low || !units || !out || !workspace || need < 0 || workspace_bytes < need || (kq::hi_bits(qtype) && !high)) return 30;
  int const tile = decline(config_name);
  return dev_units_gemm(act, low, high, units, nullptr, out, m, n, k, 0, qtype, workspace, workspace_bytes,
                        static_cast<cudaStream_t>(stream), tile, "fully-quantized dense GEMM enqueue");
}
extern "C" int quactlize_ppu_dense_fully_quantized_dev_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                          uint8_t const* units, uint16_t* out, int m, int n, int k, int qtype,
                                                          void* workspace, int64_t workspace_bytes, void* stream) {
  return quactlize_ppu_dense_fully_quantized_dev_v2(act, low, high, units, out, m, n, k, qtype, workspace, workspace_bytes, stream, nullptr);
}

// ---- grouped, scale-first (scale only) -------------------------------------------------------------------------------------
extern "C" int quactlize_ppu_grouped_lowbit_config_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                      uint16_t const* scale, int const* rows_per_expert, uint16_t* out,
                                                      int total_rows, int n, int k, int group_size, int experts, int qtype,
                                                      char const* config_name) {
  if (!act || !low || !scale || !rows_per_expert || !out || total_rows <= 0 || experts <= 0 || !shape_ok(n, k)) return 30;
  if (kq::raw_bytes(qtype) == 0) return 33;
  if (group_size != kq::group_size(qtype) || (kq::hi_bits(qtype) && !high)) return 32;
  int const tile = decline(config_name);
  return host_planes_gemm(act, low, high, scale, nullptr, out, total_rows, n, k, qtype, experts, rows_per_expert,
                          centred_offset(qtype), tile, "scale-first grouped GEMM");
}
extern "C" int quactlize_ppu_grouped_lowbit(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                            int const* rows_per_expert, uint16_t* out, int total_rows, int n, int k,
                                            int group_size, int experts, int qtype) {
  return quactlize_ppu_grouped_lowbit_config_v1(act, low, high, scale, rows_per_expert, out, total_rows, n, k, group_size, experts, qtype, nullptr);
}
extern "C" int64_t quactlize_ppu_grouped_lowbit_workspace_bytes_v1(int max_rows, int n, int k, int group_size, int experts, int qtype) {
  if (!quactlize_ppu_grouped_lowbit_config_valid_v1(max_rows, n, k, group_size, experts, max_rows, qtype, nullptr)) return -1;
  return 256 + splitk_extra_bytes(experts, max_rows, n);   // only the split-K tactic uses a workspace (its fp32 partial planes)
}
extern "C" int quactlize_ppu_grouped_lowbit_dev_v2(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                   uint16_t const* scale, int const* offsets, uint16_t* out, int total_rows, int n,
                                                   int k, int group_size, int experts, int max_rows, int qtype, void* workspace,
                                                   int64_t workspace_bytes, void* stream, char const* config_name) {
  int64_t const need = quactlize_ppu_grouped_lowbit_workspace_bytes_v1(max_rows, n, k, group_size, experts, qtype);
  if (!act || !low || !scale || !offsets || !out || total_rows <= 0 || need < 0 || workspace_bytes < need ||
      (kq::hi_bits(qtype) && !high)) return 30;
  int const tile = decline(config_name);
  rt_clear_error();
  GemmDesc d = kq_desc(act, low, high, scale, nullptr, out, total_rows, n, k, qtype, experts, offsets, centred_offset(qtype), tile);
  attach_splitk(d, tile, workspace, workspace_bytes);
  int const rc = enqueue_mixed_gemm(d, static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return rt_check_launch("scale-first grouped GEMM enqueue") ? 0 : kRuntimeError;
}
extern "C" int quactlize_ppu_grouped_lowbit_dev_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                   uint16_t const* scale, int const* offsets, uint16_t* out, int total_rows, int n,
                                                   int k, int group_size, int experts, int max_rows, int qtype, void* workspace,
                                                   int64_t workspace_bytes, void* stream) {
  return quactlize_ppu_grouped_lowbit_dev_v2(act, low, high, scale, offsets, out, total_rows, n, k, group_size, experts, max_rows,
                                             qtype, workspace, workspace_bytes, stream, nullptr);
}

// ---- grouped, fully quantized ------------------------------------------------------------------------------------------------
extern "C" int quactlize_ppu_grouped_fully_quantized_config_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                               uint8_t const* units, int const* rows_per_expert, uint16_t* out,
                                                               int total_rows, int n, int k, int experts, int qtype,
                                                               char const* config_name) {
  if (!act || !low || !units || !rows_per_expert || !out || total_rows <= 0 || experts <= 0 || !shape_ok(n, k)) return 30;
  if (!fq_ok(k, qtype) || (kq::hi_bits(qtype) && !high)) return 33;
  int const tile = decline(config_name);
  return host_units_gemm(act, low, high, units, rows_per_expert, out, total_rows, n, k, experts, qtype, tile, "fully-quantized grouped GEMM");
}
extern "C" int quactlize_ppu_grouped_fully_quantized(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                     uint8_t const* units, int const* rows_per_expert, uint16_t* out,
                                                     int total_rows, int n, int k, int experts, int qtype) {
  return quactlize_ppu_grouped_fully_quantized_config_v1(act, low, high, units, rows_per_expert, out, total_rows, n, k, experts, qtype, nullptr);
}
extern "C" int64_t quactlize_ppu_grouped_fully_quantized_workspace_bytes_v1(int max_rows, int n, int k, int experts, int qtype) {
  if (max_rows <= 0 || !shape_ok(n, k) || experts <= 0 || !fq_ok(k, qtype)) return -1;
  return plane_elems(n, k, experts, qtype) * 4 + splitk_extra_bytes(experts, max_rows, n);
}
extern "C" int quactlize_ppu_grouped_fully_quantized_dev_v2(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                            uint8_t const* units, int const* offsets, uint16_t* out,
                                                            int total_rows, int n, int k, int experts, int max_rows, int qtype,
                                                            void* workspace, int64_t workspace_bytes, void* stream,
                                                            char const* config_name) {
  int64_t const need = quactlize_ppu_grouped_fully_quantized_workspace_bytes_v1(max_rows, n, k, experts, qtype);
  if (!act || !low || !units || !offsets || !out || !workspace || total_rows <= 0 || need < 0 || workspace_bytes < need ||
      (kq::hi_bits(qtype) && !high)) return 30;
  int const tile = decline(config_name);
  return dev_units_gemm(act, low, high, units, offsets, out, total_rows, n, k, experts, qtype, workspace, workspace_bytes,
                        static_cast<cudaStream_t>(stream), tile, "fully-quantized grouped GEMM enqueue");
}
extern "C" int quactlize_ppu_grouped_fully_quantized_dev_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                            uint8_t const* units, int const* offsets, uint16_t* out,
                                                            int total_rows, int n, int k, int experts, int max_rows, int qtype,
                                                            void* workspace, int64_t workspace_bytes, void* stream) {
  return quactlize_ppu_grouped_fully_quantized_dev_v2(act, low, high, units, offsets, out, total_rows, n, k, experts, max_rows,
                                                      qtype, workspace, workspace_bytes, stream, nullptr);
}

// ---- additive: generic per-group planes, fp16 or bf16 activations, dense (experts == 0) or grouped ------------------------
extern "C" int64_t quactlize_b200_gemm_plane_splitk_workspace_bytes_v1(int total_rows, int n, int splits) {
  if (total_rows <= 0 || n <= 0 || splits < 0 || splits > 64) return -1;
  return int64_t(splits > 1 ? splits : 8) * total_rows * n * 4;       // splits 0 = chosen by the library, at most 8
}
extern "C" int quactlize_b200_gemm_plane_splitk_dev_v1(void const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                                       uint16_t const* zero, void* out, int total_rows, int n, int k, int bits_lo,
                                                       int bits_hi, int group_size, int code_offset, int act_dtype, int experts,
                                                       int const* offsets, int splits, void* workspace, int64_t workspace_bytes,
                                                       void* stream) {
  if (act_dtype < 0 || act_dtype > 1 || experts < 0 || splits < 0 || total_rows <= 0 || n <= 0) return 30;
  rt_clear_error();
  GemmDesc d{};
  d.act = act; d.low = low; d.high = bits_hi ? high : nullptr; d.scale = scale; d.zero = zero; d.out = out;
  d.offsets = offsets; d.total_rows = total_rows; d.n = n; d.k = k; d.experts = experts; d.group_size = group_size;
  d.lo_bits = bits_lo; d.hi_bits = bits_hi; d.code_offset = code_offset; d.act_bf16 = act_dtype;
  d.tile = 128; d.shallow = 1;
  int const row_tiles = experts > 0 ? std::min(experts, total_rows) : (total_rows + 127) / 128;
  d.splits = splits ? splits : splitk_auto(row_tiles, n, k);
  if (d.splits > 1) {
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15) || workspace_bytes < int64_t(d.splits) * total_rows * n * 4) return 37;
    d.partial = static_cast<float*>(workspace);
  }
  int const rc = enqueue_mixed_gemm(d, static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return rt_check_launch("split-K plane GEMM enqueue") ? 0 : kRuntimeError;
}

extern "C" int quactlize_b200_gemm_plane_dev_v2(void const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                                uint16_t const* zero, void* out, int total_rows, int n, int k, int bits_lo,
                                                int bits_hi, int group_size, int code_offset, int act_dtype, int experts,
                                                int const* offsets, unsigned long long const* out_rows, void* stream) {
  if (act_dtype < 0 || act_dtype > 1 || experts < 0) return 30;
  rt_clear_error();
  GemmDesc d{};
  d.act = act; d.low = low; d.high = bits_hi ? high : nullptr; d.scale = scale; d.zero = zero; d.out = out;
  d.offsets = offsets; d.total_rows = total_rows; d.n = n; d.k = k; d.experts = experts; d.group_size = group_size;
  d.lo_bits = bits_lo; d.hi_bits = bits_hi; d.code_offset = code_offset; d.act_bf16 = act_dtype;
  d.out_rows = out_rows;
  int const rc = enqueue_mixed_gemm(d, static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return rt_check_launch("plane GEMM enqueue") ? 0 : kRuntimeError;
}

extern "C" int quactlize_b200_gemm_plane_dev_v1(void const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                                uint16_t const* zero, void* out, int total_rows, int n, int k, int bits_lo,
                                                int bits_hi, int group_size, int code_offset, int act_dtype, int experts,
                                                int const* offsets, void* stream) {
  if (act_dtype < 0 || act_dtype > 1 || experts < 0) return 30;
  rt_clear_error();
  GemmDesc d{};
  d.act = act; d.low = low; d.high = bits_hi ? high : nullptr; d.scale = scale; d.zero = zero; d.out = out;
  d.offsets = offsets; d.total_rows = total_rows; d.n = n; d.k = k; d.experts = experts; d.group_size = group_size;
  d.lo_bits = bits_lo; d.hi_bits = bits_hi; d.code_offset = code_offset; d.act_bf16 = act_dtype;
  int const rc = enqueue_mixed_gemm(d, static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return rt_check_launch("plane GEMM enqueue") ? 0 : kRuntimeError;
}

extern "C" long long quactlize_b200_debug_gemm_swap_launches(void) { return qb::gemm_swap_launches(); }
