// Runtime shim: staged host copies, the device wait-status word, device properties.
#include "qb_runtime.hpp"

#include "qb_device.cuh"

#include <mutex>
#include <vector>

namespace qb {

// One word per device that loads the library.  Kernels with bounded waits record a code here when a wait gives up.
static __device__ unsigned int g_wait_status[4];

namespace {
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

namespace {
struct PoolEntry { void* p; size_t bytes; int dev; };
struct Pool {
  std::vector<PoolEntry> free_list;
  size_t held = 0;
  ~Pool() { for (auto& e : free_list) (void)cudaFree(e.p); }
};
Pool& pool() { static thread_local Pool p; return p; }
constexpr size_t kPoolCap = size_t(1) << 30;      // bytes a thread may keep parked
}  // namespace

void* rt_pool_take(size_t bytes) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  auto& fl = pool().free_list;
  int best = -1;
  for (int i = 0; i < int(fl.size()); ++i)
    if (fl[i].dev == dev && fl[i].bytes >= bytes && fl[i].bytes <= 2 * bytes + 4096 && (best < 0 || fl[i].bytes < fl[best].bytes)) best = i;
  if (best < 0) return nullptr;
  void* p = fl[best].p;
  pool().held -= fl[best].bytes;
  fl.erase(fl.begin() + best);
  return p;
}

void rt_pool_give(void* p, size_t bytes) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || bytes > kPoolCap / 2) { (void)cudaFree(p); return; }
  auto& pl = pool();
  while (!pl.free_list.empty() && (pl.held + bytes > kPoolCap || pl.free_list.size() >= 32)) {
    (void)cudaFree(pl.free_list.front().p);
    pl.held -= pl.free_list.front().bytes;
    pl.free_list.erase(pl.free_list.begin());
  }
  pl.free_list.push_back({p, bytes, dev});
  pl.held += bytes;
}

void rt_pool_trim() {
  auto& pl = pool();
  for (auto& e : pl.free_list) (void)cudaFree(e.p);
  pl.free_list.clear();
  pl.held = 0;
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

// A one-CTA kernel that waits on an mbarrier nothing ever arms, with a caller-chosen limit.  The wait gives up, records
// its code in the device status word and the kernel returns normally: the path every bounded wait of the library takes
// when a copy never lands, exercised without a fault, a trap or a hang.
namespace {
__global__ void wait_probe_kernel(unsigned int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
    (void)mbar_wait_bounded(&bar, 0u, status, kWaitStageTimeout, limit_ns);
  }
}
}  // namespace

}  // namespace qb

extern "C" int quactlize_b200_debug_wait_probe(long long limit_ns, void* stream) {
  if (limit_ns <= 0 || limit_ns > 100000000ll) return 20;          // at most 100 ms: this is a test hook, not a sleep
  qb::rt_clear_error();
  unsigned int* st = qb::rt_device_status_ptr();
  if (!st) return qb::kRuntimeError;
  qb::wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(st, static_cast<unsigned long long>(limit_ns));
  return qb::rt_check_launch("wait probe enqueue") ? 0 : qb::kRuntimeError;
}

// ---- additive C entries: fault injection for tests, status query ---------------------------------------------------
extern "C" void quactlize_b200_rt_fail_next(int kind) { qb::rt_tls().inject = static_cast<qb::RtStatus>(kind); }
extern "C" void quactlize_b200_rt_trim(void) { qb::rt_pool_trim(); }
extern "C" int quactlize_b200_rt_last_status(void) { return static_cast<int>(qb::rt_tls().status); }
extern "C" int quactlize_b200_device_wait_status(void) {
  qb::rt_clear_error();
  return qb::rt_device_status_ok(nullptr, "device wait status") ? 0 : qb::kRuntimeError;
}
