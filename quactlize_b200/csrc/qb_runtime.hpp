// Runtime shim shared by every C-ABI entry of libquactlize_b200.
//
// Error contract (the reference's, quactlize/include/gemv_lowbit/gemv_rt.hpp:1-48,182-199): an entry returns an int,
// 0 = done (host-pointer entries) or enqueued (device-pointer entries).  Allocation, copy, synchronise and launch
// failures never abort the process: the first one is latched in a thread-local status, reported once on stderr, and
// the entry returns kRuntimeError (41).  Host outputs are staged and written only after the device work succeeded,
// so `out` is untouched on failure.  The status is per host thread, so entries may be called concurrently.
//
// Failures can be injected ON THE HOST for tests (quactlize_b200_rt_fail_next): the next call of the named kind
// fails without touching the GPU.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstring>

namespace qb {

constexpr int kRuntimeError = 41;
constexpr int kMaxDevices = 64;          // device ordinals that per-device caches are sized for

enum class RtStatus : int { Ok = 0, Allocation = 1, HostToDevice = 2, DeviceToHost = 3, Synchronize = 4,
                            HostAllocation = 5, Launch = 6, DeviceWait = 7 };

struct RtTls {
  RtStatus status = RtStatus::Ok;
  RtStatus inject = RtStatus::Ok;
};
inline RtTls& rt_tls() { static thread_local RtTls t; return t; }

inline void rt_clear_error() { rt_tls().status = RtStatus::Ok; }
inline bool rt_ok() { return rt_tls().status == RtStatus::Ok; }
inline bool rt_record(RtStatus s, char const* op, char const* detail) {
  if (rt_tls().status == RtStatus::Ok) {
    rt_tls().status = s;
    std::fprintf(stderr, "[quactlize_b200] %s: %s\n", op, detail ? detail : "device runtime failure");
  }
  return false;
}
inline bool rt_injected(RtStatus s) {
  if (rt_tls().inject != s) return false;
  rt_tls().inject = RtStatus::Ok;
  return true;
}

// Device temporaries of the host-pointer entries come from a small per-thread pool of recently released buffers, so
// a decode loop through those entries does not pay cudaMalloc/cudaFree (both synchronise the device) on every call.
void* rt_pool_take(size_t bytes);                 // nullptr when nothing fits
void rt_pool_give(void* p, size_t bytes);         // keeps or frees
void rt_pool_trim();                              // frees everything the calling thread holds

inline void* rt_malloc(size_t bytes) {
  if (rt_injected(RtStatus::Allocation)) { rt_record(RtStatus::Allocation, "cudaMalloc", "injected failure"); return nullptr; }
  if (void* q = rt_pool_take(bytes)) return q;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes ? bytes : 1);
  if (e != cudaSuccess) { (void)cudaGetLastError(); rt_pool_trim(); e = cudaMalloc(&p, bytes ? bytes : 1); }
  if (e != cudaSuccess) { (void)cudaGetLastError(); rt_record(RtStatus::Allocation, "cudaMalloc", cudaGetErrorString(e)); return nullptr; }
  return p;
}
inline void rt_free(void* p, size_t bytes) { if (p) rt_pool_give(p, bytes); }
inline bool rt_h2d(void* dst, void const* src, size_t bytes, cudaStream_t s) {
  if (rt_injected(RtStatus::HostToDevice)) return rt_record(RtStatus::HostToDevice, "H2D", "injected failure");
  if (!bytes) return true;
  cudaError_t const e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, s);
  return e == cudaSuccess || rt_record(RtStatus::HostToDevice, "H2D", cudaGetErrorString(e));
}
inline bool rt_d2h(void* dst, void const* src, size_t bytes, cudaStream_t s) {
  if (rt_injected(RtStatus::DeviceToHost)) return rt_record(RtStatus::DeviceToHost, "D2H", "injected failure");
  if (!bytes) return true;
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  return e == cudaSuccess || rt_record(RtStatus::DeviceToHost, "D2H", cudaGetErrorString(e));
}
inline bool rt_sync(cudaStream_t s, char const* where) {
  if (rt_injected(RtStatus::Synchronize)) return rt_record(RtStatus::Synchronize, where, "injected failure");
  cudaError_t e = cudaStreamSynchronize(s);
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess || rt_record(RtStatus::Synchronize, where, cudaGetErrorString(e));
}
inline bool rt_check_launch(char const* where) {
  if (rt_injected(RtStatus::Launch)) return rt_record(RtStatus::Launch, where, "injected failure");
  cudaError_t const e = cudaPeekAtLastError();
  if (e != cudaSuccess) (void)cudaGetLastError();
  return e == cudaSuccess || rt_record(RtStatus::Launch, where, cudaGetErrorString(e));
}

// Device temporary owned by a host-pointer entry; released on scope exit whatever happened.
struct DevBuf {
  void* p = nullptr;
  size_t bytes = 0;
  explicit DevBuf(size_t b) : bytes(b) { if (b && rt_ok()) p = rt_malloc(b); }
  ~DevBuf() { rt_free(p, bytes); }
  DevBuf(DevBuf const&) = delete;
  DevBuf& operator=(DevBuf const&) = delete;
  void from_host(void const* src, cudaStream_t s = nullptr) { if (rt_ok() && p && src) rt_h2d(p, src, bytes, s); }
  template <class T> T* as() const { return reinterpret_cast<T*>(p); }
};

// Copy a device result to the caller's host buffer through a staging vector so `out` is untouched on failure.
bool rt_copy_out(void const* dev, void* host, size_t bytes, cudaStream_t s);

// Device-side wait status.  Kernels that wait on an mbarrier give up after a bounded time, record where in this
// device word and finish normally; host-pointer entries read it after synchronising.
unsigned int* rt_device_status_ptr();          // device address of the word for the current device (nullptr on failure)
bool rt_device_status_ok(cudaStream_t s, char const* where);   // reads + clears; latches DeviceWait if non-zero

int rt_sm_count();

}  // namespace qb
