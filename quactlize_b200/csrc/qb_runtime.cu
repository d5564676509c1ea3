// Runtime shim: staged host copies, the device wait-status word, device properties.
#include "qb_runtime.hpp"

#include <mutex>
#include <vector>

namespace qb {

// One word per device that loads the library.  Kernels with bounded waits record a code here when a wait gives up.
static __device__ unsigned int g_wait_status[4];

namespace {
constexpr int kMaxDevices = 64;
unsigned int* g_status_ptr[kMaxDevices];
int g_sm_count[kMaxDevices];
std::mutex g_mu;
}  // namespace

unsigned int* rt_device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_wait_status) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
    g_status_ptr[dev] = static_cast<unsigned int*>(p);
  }
  return g_status_ptr[dev];
}

bool rt_device_status_ok(cudaStream_t s, char const* where) {
  unsigned int* p = rt_device_status_ptr();
  if (!p) return rt_record(RtStatus::DeviceWait, where, "no device status word");
  unsigned int v = 0;
  cudaError_t e = cudaMemcpyAsync(&v, p, sizeof(v), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return rt_record(RtStatus::Synchronize, where, cudaGetErrorString(e));
  if (v != 0) {
    (void)cudaMemsetAsync(p, 0, sizeof(v), s);
    (void)cudaStreamSynchronize(s);
    char msg[96];
    std::snprintf(msg, sizeof(msg), "a bounded device wait gave up (code 0x%08X)", v);
    return rt_record(RtStatus::DeviceWait, where, msg);
  }
  return true;
}

bool rt_copy_out(void const* dev, void* host, size_t bytes, cudaStream_t s) {
  if (!rt_ok()) return false;
  std::vector<unsigned char> stage;
  try { stage.resize(bytes); } catch (...) { return rt_record(RtStatus::HostAllocation, "host staging", "allocation failed"); }
  if (!rt_d2h(stage.data(), dev, bytes, s)) return false;
  std::memcpy(host, stage.data(), bytes);
  return true;
}

int rt_sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (!g_sm_count[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

}  // namespace qb

// ---- additive C entries: fault injection for tests, status query ---------------------------------------------------
extern "C" void quactlize_b200_rt_fail_next(int kind) { qb::rt_tls().inject = static_cast<qb::RtStatus>(kind); }
extern "C" int quactlize_b200_rt_last_status(void) { return static_cast<int>(qb::rt_tls().status); }
extern "C" int quactlize_b200_device_wait_status(void) {
  qb::rt_clear_error();
  return qb::rt_device_status_ok(nullptr, "device wait status") ? 0 : qb::kRuntimeError;
}
