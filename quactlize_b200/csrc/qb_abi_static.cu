// A fully-quantized dense GEMM entry that allocates nothing and asks the caller for no workspace.
//
// Who needs it: callers that sit where device allocation is off limits -- a decode loop that must not hit the
// allocator's implicit device synchronisation, a plugin host whose memory budget is fixed up front and which treats
// any later allocation as a leak, a C caller with no allocator of its own to produce the workspace the regular entry
// (quactlize_ppu_dense_fully_quantized_dev_v1) takes.  For them the fp16 scale/zero planes that the GEMM derives from
// the packed units live in a fixed array inside this library's device image instead.
//
// What follows from that:
//   * the array has one size, QUACTLIZE_B200_STATIC_SCRATCH_BYTES (16 MiB) per device; a weight whose planes
//     (2 planes x k/group_size x n fp16) do not fit is refused with code 37 and a message, nothing is launched.
//     The array is part of the library's device image: every process that loads the library pays these 16 MiB on
//     every device it creates a context on, whether or not it ever calls this entry, until the process exits;
//   * the first call on each device looks the array's device address up (a runtime query, made with that device
//     current, result kept per device).  Make that first call outside any stream capture;
//   * every call on a device uses the same array.  The planes of a call are rewritten completely by that call's own
//     pre-pass before its GEMM reads them, so nothing has to start at zero and stale contents of an earlier call
//     are never read.  Two calls that may overlap in time on one device (different streams, different host threads)
//     race on the array: keep calls of this entry on one stream per device, or order them with events.
// No counterpart in the reference.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <mutex>

#include "qb_internal.hpp"
#include "qb_kquant.cuh"
#include "qb_runtime.hpp"
#include "../../include/quactlize_b200.h"

using namespace qb;

namespace {

constexpr int64_t kStaticScratchBytes = QUACTLIZE_B200_STATIC_SCRATCH_BYTES;

// The scratch itself.  Host code never uses this name as an address: it asks the runtime for the device address.
static __device__ __align__(256) unsigned char g_static_planes[kStaticScratchBytes];

// Device address of the scratch on the CURRENT device; nullptr (with the error latched) if the query fails.
void* static_scratch_of_current_device() {
  static std::mutex mu;
  static void* ptrs[kMaxDevices] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    rt_record(RtStatus::Launch, "static scratch set-up", e != cudaSuccess ? cudaGetErrorString(e) : "device ordinal out of range");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_planes);
    if (e != cudaSuccess || !p) {
      (void)cudaGetLastError();
      rt_record(RtStatus::Launch, "static scratch set-up (cudaGetSymbolAddress)", cudaGetErrorString(e));
      return nullptr;
    }
    ptrs[dev] = p;
  }
  return ptrs[dev];
}

}  // namespace

extern "C" int quactlize_b200_dense_fully_quantized_static_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                              uint8_t const* units, uint16_t* out, int m, int n, int k,
                                                              int qtype, void* stream) {
  if (!act || !low || !units || !out || m <= 0 || n <= 0 || n % 256 || k <= 0 || k % 256) return 30;
  if (kq::raw_bytes(qtype) == 0) return 33;
  int const per_unit = (qtype == 11 || qtype == 14) ? 2 : 1;          // superblocks per packed unit
  if ((k / 256) % per_unit) return 33;
  if (kq::hi_bits(qtype) && !high) return 30;
  int64_t const plane_elems = int64_t(k / kq::group_size(qtype)) * n;
  int64_t const need = plane_elems * 4;                                 // scale plane + zero plane, fp16
  if (need > kStaticScratchBytes) {
    std::fprintf(stderr,
                 "[quactlize_b200] dense_fully_quantized_static: the scale/zero planes of an (n=%d, k=%d) weight of type %d "
                 "take %lld bytes; the built-in scratch holds %lld. Use quactlize_ppu_dense_fully_quantized_dev_v1 with a "
                 "caller workspace.\n", n, k, qtype, static_cast<long long>(need), static_cast<long long>(kStaticScratchBytes));
    return 37;
  }
  rt_clear_error();
  void* const scratch = static_scratch_of_current_device();
  if (!scratch) return kRuntimeError;
  cudaStream_t const s = static_cast<cudaStream_t>(stream);
  __half* const sc = reinterpret_cast<__half*>(scratch);
  __half* const zr = sc + plane_elems;
  // pre-pass: packed units -> fp16 planes, every element of both planes written.  Same code convention as the regular
  // entry: int4-low codes convert as (low - 8), the zero plane carries the matching correction.
  int const zmul = qtype == 11 ? -4 : (qtype == 12 || qtype == 13) ? 8 : qtype == 14 ? -24 : 0;
  int const code_offset = (qtype == 12 || qtype == 13 || qtype == 14) ? -8 : 0;
  if (!enqueue_prepass_unit(units, sc, zr, 1, n, k / 256, qtype, zmul, s)) return 33;
  GemmDesc d{};
  d.act = act; d.low = low; d.high = kq::hi_bits(qtype) ? high : nullptr; d.scale = sc; d.zero = zr; d.out = out;
  d.offsets = nullptr; d.total_rows = m; d.n = n; d.k = k; d.experts = 0;
  d.group_size = kq::group_size(qtype); d.lo_bits = kq::lo_bits(qtype); d.hi_bits = kq::hi_bits(qtype);
  d.code_offset = code_offset; d.act_bf16 = 0;
  int const rc = enqueue_mixed_gemm(d, s);
  if (rc) return rc;
  return rt_check_launch("fully-quantized dense GEMM (static scratch) enqueue") ? 0 : kRuntimeError;
}
