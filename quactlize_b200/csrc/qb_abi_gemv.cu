// C ABI of the CUDA-core family: raw-block GEMV (rows / dense / ragged MoE), raw-block dequantise, scale pre-pass.
// Host-pointer entries allocate device temporaries, copy in, launch, synchronise and copy out; `_dev_v1` entries take
// device pointers and a stream, only enqueue, and neither allocate nor synchronise.
// Signatures and return codes follow quactlize/csrc/device/ppu_backend.cu:297-509 of the reference.
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "qb_internal.hpp"
#include "qb_kquant.cuh"
#include "qb_runtime.hpp"
#include "../../include/quactlize_b200.h"

using namespace qb;

namespace {
constexpr char const* kGroupedCudaConfig = "vecdot_moe";

int native_host(uint8_t const* blocks, uint16_t const* x, int const* offsets, float* out, int n, int bpr, int experts,
                int x_rows, int max_rows, int qtype, bool per_row_x, char const* what) {
  rt_clear_error();
  int const bb = kq::raw_bytes(qtype);
  int const we = experts > 0 ? experts : 1;
  size_t const out_elems = per_row_x ? size_t(n) : size_t(x_rows) * n;
  DevBuf db(size_t(we) * n * bpr * bb), dx(size_t(x_rows) * bpr * 256 * 2), dout(out_elems * 4),
      doff(experts > 0 ? size_t(experts + 1) * 4 : 0);
  db.from_host(blocks); dx.from_host(x); if (experts > 0) doff.from_host(offsets);
  if (!rt_ok()) return kRuntimeError;
  enqueue_native_gemv(db.as<uint8_t>(), dx.as<__half>(), dout.as<float>(), experts > 0 ? doff.as<int>() : nullptr,
                      n, bpr, we, per_row_x ? 1 : x_rows, max_rows, qtype, per_row_x, false, nullptr);
  if (!rt_check_launch(what)) return kRuntimeError;
  if (!rt_sync(nullptr, what) || !rt_device_status_ok(nullptr, what)) return kRuntimeError;
  return rt_copy_out(dout.p, out, out_elems * 4, nullptr) ? 0 : kRuntimeError;
}
}  // namespace

extern "C" int quactlize_ppu_vecdot(uint8_t const* b, int64_t block_bytes, uint16_t const* x, float* out,
                                    int rows, int bpr, int qtype) {
  if (kq::raw_bytes(qtype) == 0) return 1;
  if (block_bytes != kq::raw_bytes(qtype) || rows <= 0 || bpr <= 0 || !b || !x || !out) return 10;
  return native_host(b, x, nullptr, out, rows, bpr, 0, rows, 1, qtype, true, "raw-block row vecdot");
}

extern "C" int quactlize_b200_vecdot_dev_v1(uint8_t const* b, int64_t block_bytes, uint16_t const* x, float* out,
                                           int rows, int bpr, int qtype, void* stream) {
  if (kq::raw_bytes(qtype) == 0) return 1;
  if (block_bytes != kq::raw_bytes(qtype) || rows <= 0 || bpr <= 0 || !b || !x || !out) return 10;
  rt_clear_error();
  enqueue_native_gemv(b, reinterpret_cast<__half const*>(x), out, nullptr, rows, bpr, 1, 1, 1, qtype, true, false,
                      static_cast<cudaStream_t>(stream));
  return rt_check_launch("raw-block row vecdot enqueue") ? 0 : kRuntimeError;
}

// Two raw-block matrices of the same K against one activation row in ONE launch (a layer's gate and up projections share
// their input): out_a[n_a] and out_b[n_b].  Q4_K through the single-row kernel with the rows of both matrices split over
// the CTAs as one; any other format, alignment or shape runs as two launches.  Device pointers, enqueue only.
extern "C" int quactlize_b200_vecdot_dense2_dev_v1(uint8_t const* blocks_a, int n_a, uint8_t const* blocks_b, int n_b, int64_t block_bytes,
                                                  uint16_t const* x, float* out_a, float* out_b, int bpr, int qtype, void* stream) {
  if (!blocks_a || !blocks_b || !x || !out_a || !out_b || n_a <= 0 || n_b <= 0 || bpr <= 0) return 12;
  if (kq::raw_bytes(qtype) == 0) return 3;
  if (block_bytes != kq::raw_bytes(qtype)) return 12;
  rt_clear_error();
  auto al = [](void const* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  unsigned int* status = rt_device_status_ptr();
  bool done = false;
  if (qtype == 12 && status && al(blocks_a) && al(blocks_b) && al(x))
    done = enqueue_q4k_gemv1_dual(blocks_a, n_a, blocks_b, n_b, reinterpret_cast<__half const*>(x), out_a, out_b, bpr, status,
                                  static_cast<cudaStream_t>(stream));
  if (!done) {
    (void)cudaGetLastError();
    enqueue_native_gemv(blocks_a, reinterpret_cast<__half const*>(x), out_a, nullptr, n_a, bpr, 1, 1, 1, qtype, false, false,
                        static_cast<cudaStream_t>(stream));
    enqueue_native_gemv(blocks_b, reinterpret_cast<__half const*>(x), out_b, nullptr, n_b, bpr, 1, 1, 1, qtype, false, false,
                        static_cast<cudaStream_t>(stream));
  }
  return rt_check_launch("two-matrix raw-block GEMV enqueue") ? 0 : kRuntimeError;
}

extern "C" int quactlize_ppu_vecdot_dense(uint8_t const* b, int64_t block_bytes, uint16_t const* x, float* out,
                                          int rows, int bpr, int qtype) {
  if (kq::raw_bytes(qtype) == 0) return 3;
  if (block_bytes != kq::raw_bytes(qtype) || rows <= 0 || bpr <= 0 || !b || !x || !out) return 12;
  return native_host(b, x, nullptr, out, rows, bpr, 0, 1, 1, qtype, false, "raw-block dense GEMV");
}

extern "C" int quactlize_ppu_vecdot_dense_dev_v1(uint8_t const* b, int64_t block_bytes, uint16_t const* x, float* out,
                                                 int rows, int bpr, int qtype, void* stream) {
  if (!b || !x || !out || rows <= 0 || bpr <= 0) return 12;
  if (kq::raw_bytes(qtype) == 0) return 3;
  if (block_bytes != kq::raw_bytes(qtype)) return 12;
  rt_clear_error();
  enqueue_native_gemv(b, reinterpret_cast<__half const*>(x), out, nullptr, rows, bpr, 1, 1, 1, qtype, false, false,
                      static_cast<cudaStream_t>(stream));
  return rt_check_launch("raw-block dense GEMV enqueue") ? 0 : kRuntimeError;
}

extern "C" int quactlize_b200_vecdot_rows_dev_v1(uint8_t const* b, int64_t block_bytes, uint16_t const* x, float* out,
                                                 int m, int rows, int bpr, int qtype, int force_generic, void* stream) {
  if (!b || !x || !out || rows <= 0 || bpr <= 0 || m <= 0) return 12;
  if (kq::raw_bytes(qtype) == 0) return 3;
  if (block_bytes != kq::raw_bytes(qtype)) return 12;
  rt_clear_error();
  enqueue_native_gemv(b, reinterpret_cast<__half const*>(x), out, nullptr, rows, bpr, 1, m, m, qtype, false,
                      force_generic != 0, static_cast<cudaStream_t>(stream));
  return rt_check_launch("raw-block multi-row GEMV enqueue") ? 0 : kRuntimeError;
}

extern "C" int32_t quactlize_ppu_vecdot_moe_config_valid_v1(int total_rows, int n, int k, int group_size, int experts,
                                                            int max_rows, int qtype, char const* config_name) {
  bool const name_ok = !config_name || !config_name[0] || std::strcmp(config_name, kGroupedCudaConfig) == 0;
  return name_ok && kq::raw_bytes(qtype) != 0 && total_rows > 0 && n > 0 && k > 0 && k % 256 == 0 && experts > 0 &&
         max_rows > 0 && group_size == kq::group_size(qtype);
}

extern "C" int32_t quactlize_ppu_list_valid_vecdot_moe_configs_v2(quactlize_ppu_config_v2* configs, int32_t capacity,
                                                                  int total_rows, int n, int k, int group_size,
                                                                  int experts, int max_rows, int qtype) {
  bool const valid = quactlize_ppu_vecdot_moe_config_valid_v1(total_rows, n, k, group_size, experts, max_rows, qtype,
                                                              kGroupedCudaConfig);
  if (valid && configs && capacity > 0) configs[0] = {true, kGroupedCudaConfig, 0, 0, 0, 0, 0, 0};
  return valid ? 1 : 0;
}

extern "C" int quactlize_ppu_vecdot_moe_config_v1(uint8_t const* b, int64_t block_bytes, uint16_t const* x,
                                                  int const* offsets, float* out, int n, int bpr, int experts,
                                                  int total_rows, int max_rows, int qtype, char const* config_name) {
  if (config_name && config_name[0] && std::strcmp(config_name, kGroupedCudaConfig) != 0)
    std::fprintf(stderr, "[quactlize_b200] grouped CUDA config '%s' is not compiled in; running default '%s'\n",
                 config_name, kGroupedCudaConfig);
  if (kq::raw_bytes(qtype) == 0) return 2;
  if (block_bytes != kq::raw_bytes(qtype) || n <= 0 || bpr <= 0 || experts <= 0 || total_rows <= 0 || max_rows <= 0 ||
      !b || !x || !offsets || !out) return 11;
  return native_host(b, x, offsets, out, n, bpr, experts, total_rows, max_rows, qtype, false, "raw-block MoE GEMV");
}

extern "C" int quactlize_ppu_vecdot_moe(uint8_t const* b, int64_t block_bytes, uint16_t const* x, int const* offsets,
                                        float* out, int n, int bpr, int experts, int total_rows, int max_rows, int qtype) {
  return quactlize_ppu_vecdot_moe_config_v1(b, block_bytes, x, offsets, out, n, bpr, experts, total_rows, max_rows, qtype, nullptr);
}

extern "C" int quactlize_b200_vecdot_moe_dev_v1(uint8_t const* b, int64_t block_bytes, uint16_t const* x,
                                                int const* offsets, float* out, int n, int bpr, int experts,
                                                int total_rows, int max_rows, int qtype, void* stream) {
  if (kq::raw_bytes(qtype) == 0) return 2;
  if (block_bytes != kq::raw_bytes(qtype) || n <= 0 || bpr <= 0 || experts <= 0 || total_rows <= 0 || max_rows <= 0 ||
      !b || !x || !offsets || !out) return 11;
  rt_clear_error();
  enqueue_native_gemv(b, reinterpret_cast<__half const*>(x), out, offsets, n, bpr, experts, total_rows, max_rows, qtype,
                      false, false, static_cast<cudaStream_t>(stream));
  return rt_check_launch("raw-block MoE GEMV enqueue") ? 0 : kRuntimeError;
}

extern "C" int quactlize_ppu_dequantize(uint8_t const* b, int64_t block_bytes, uint16_t* out, int count, int qtype) {
  if (kq::raw_bytes(qtype) == 0) return 3;
  if (block_bytes != kq::raw_bytes(qtype) || count <= 0 || !b || !out) return 12;
  rt_clear_error();
  DevBuf db(size_t(count) * block_bytes), dout(size_t(count) * 512);
  db.from_host(b);
  if (!rt_ok()) return kRuntimeError;
  enqueue_dequantize(db.as<uint8_t>(), dout.as<__half>(), count, qtype, nullptr);
  if (!rt_check_launch("GGUF dequantize") || !rt_sync(nullptr, "GGUF dequantize")) return kRuntimeError;
  return rt_copy_out(dout.p, out, size_t(count) * 512, nullptr) ? 0 : kRuntimeError;
}

extern "C" int quactlize_b200_dequantize_dev_v1(uint8_t const* b, int64_t block_bytes, uint16_t* out, int count,
                                                int qtype, void* stream) {
  if (kq::raw_bytes(qtype) == 0) return 3;
  if (block_bytes != kq::raw_bytes(qtype) || count <= 0 || !b || !out) return 12;
  rt_clear_error();
  enqueue_dequantize(b, reinterpret_cast<__half*>(out), count, qtype, static_cast<cudaStream_t>(stream));
  return rt_check_launch("GGUF dequantize enqueue") ? 0 : kRuntimeError;
}

// Additive: the gguf_unpack op on the device.  codes int8 [count][256], scale/zero fp16 [count][groups].
extern "C" int quactlize_b200_unpack_dev_v1(uint8_t const* b, int64_t block_bytes, int8_t* codes, uint16_t* scale,
                                            uint16_t* zero, int count, int qtype, void* stream) {
  if (kq::raw_bytes(qtype) == 0) return 3;
  if (block_bytes != kq::raw_bytes(qtype) || count <= 0 || !b || !codes || !scale || !zero) return 12;
  rt_clear_error();
  enqueue_unpack(b, codes, reinterpret_cast<__half*>(scale), reinterpret_cast<__half*>(zero), count, qtype,
                 static_cast<cudaStream_t>(stream));
  return rt_check_launch("GGUF unpack enqueue") ? 0 : kRuntimeError;
}

// Additive: dequantise a plane artifact (Native planes + fp16 scale/zero planes [E][k/gs][n]) to fp16 [E][n][k] -- the
// materialisation the dequant-then-dense route pays for.  code_shift is added to the unsigned code (the reference's
// dense contract stores int4-low codes against a zero plane that carries +8*scale: shift -8).
extern "C" int quactlize_b200_planes_dequantize_dev_v1(uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                                       uint16_t const* zero, uint16_t* out, int experts, int n, int k,
                                                       int bits_lo, int bits_hi, int group_size, int code_shift, void* stream) {
  if (!low || !scale || !out || experts <= 0 || n <= 0 || k <= 0) return 20;
  if (!(bits_lo == 1 || bits_lo == 2 || bits_lo == 4) || bits_hi < 0 || bits_hi > 2 || (bits_hi && !high)) return 21;
  if (group_size <= 0 || k % group_size || k % 8) return 24;
  rt_clear_error();
  if (!enqueue_planes_dequantize(low, high, reinterpret_cast<__half const*>(scale), reinterpret_cast<__half const*>(zero),
                                 reinterpret_cast<__half*>(out), experts, n, k, bits_lo, bits_hi, group_size, code_shift,
                                 static_cast<cudaStream_t>(stream)))
    return 30;
  return rt_check_launch("plane dequantize enqueue") ? 0 : kRuntimeError;
}

extern "C" int quactlize_ppu_prepass(uint8_t const* b, int64_t block_bytes, uint16_t const* d, uint16_t const* dm,
                                     int count, uint16_t* scale, uint16_t* zero, int groups, int qtype, int zmul) {
  (void)block_bytes; (void)groups;
  if (zmul != 0 && zmul != 8) return 4;
  if (kq::raw_bytes(qtype) == 0) return 5;
  if (!b || !d || !scale || !zero || count <= 0) return 5;
  bool const has_min = (qtype == 10 || qtype == 12 || qtype == 13);
  if (has_min && !dm) return 5;
  int const sbytes = (qtype == 10 || qtype == 14) ? 16 : 12;
  int const g = kq::group_size(qtype) == 32 ? 8 : 16;
  rt_clear_error();
  DevBuf db(size_t(count) * sbytes), dd(size_t(count) * 2), dmn(has_min ? size_t(count) * 2 : 0),
      ds(size_t(count) * g * 2), dz(size_t(count) * g * 2);
  db.from_host(b); dd.from_host(d); if (has_min) dmn.from_host(dm);
  if (!rt_ok()) return kRuntimeError;
  enqueue_prepass(db.as<uint8_t>(), dd.as<uint16_t>(), dmn.as<uint16_t>(), count, qtype, zmul, ds.as<__half>(), dz.as<__half>(), nullptr);
  if (!rt_check_launch("GGUF scale prepass") || !rt_sync(nullptr, "GGUF scale prepass")) return kRuntimeError;
  if (!rt_copy_out(ds.p, scale, size_t(count) * g * 2, nullptr)) return kRuntimeError;
  return rt_copy_out(dz.p, zero, size_t(count) * g * 2, nullptr) ? 0 : kRuntimeError;
}

static bool zmul_ok(int z) { return z == -32 || z == -24 || z == -4 || z == 0 || z == 8; }

extern "C" int quactlize_ppu_prepass_unit(uint8_t const* units, uint16_t* scale, uint16_t* zero, int n, int k,
                                          int experts, int qtype, int zmul) {
  if (!units || !scale || !zero || n <= 0 || k <= 0 || k % 256 || experts <= 0) return 7;
  if (!zmul_ok(zmul)) return 8;
  if (kq::raw_bytes(qtype) == 0) return 9;
  int const nsb = k / 256;
  int const p = (qtype == 11 || qtype == 14) ? 2 : 1;
  if (nsb % p) return 6;
  int const sbb = qtype == 10 ? 20 : qtype == 11 ? 14 : qtype == 14 ? 18 : 16;
  int const g = kq::group_size(qtype) == 32 ? 8 : 16;
  size_t const ub = size_t(experts) * nsb * n * sbb, pe = size_t(experts) * nsb * g * n;
  rt_clear_error();
  DevBuf du(ub), ds(pe * 2), dz(pe * 2);
  du.from_host(units);
  if (!rt_ok()) return kRuntimeError;
  enqueue_prepass_unit(du.as<uint8_t>(), ds.as<__half>(), dz.as<__half>(), experts, n, nsb, qtype, zmul, nullptr);
  if (!rt_check_launch("packed-unit scale prepass") || !rt_sync(nullptr, "packed-unit scale prepass")) return kRuntimeError;
  if (!rt_copy_out(ds.p, scale, pe * 2, nullptr)) return kRuntimeError;
  return rt_copy_out(dz.p, zero, pe * 2, nullptr) ? 0 : kRuntimeError;
}

extern "C" int quactlize_b200_prepass_unit_dev_v1(uint8_t const* units, uint16_t* scale, uint16_t* zero, int n, int k,
                                                  int experts, int qtype, int zmul, void* stream) {
  if (!units || !scale || !zero || n <= 0 || k <= 0 || k % 256 || experts <= 0) return 7;
  if (!zmul_ok(zmul)) return 8;
  if (kq::raw_bytes(qtype) == 0) return 9;
  int const p = (qtype == 11 || qtype == 14) ? 2 : 1;
  if ((k / 256) % p) return 6;
  rt_clear_error();
  enqueue_prepass_unit(units, reinterpret_cast<__half*>(scale), reinterpret_cast<__half*>(zero), experts, n, k / 256,
                       qtype, zmul, static_cast<cudaStream_t>(stream));
  return rt_check_launch("packed-unit scale prepass enqueue") ? 0 : kRuntimeError;
}
