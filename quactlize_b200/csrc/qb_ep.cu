// Expert-parallel MoE over the GPUs of one node: the pieces that move rows between ranks without a host round trip.
//
// The reference has no multi-device code for this path.  One process drives one GPU; ranks exchange rows through
// buffers every rank can write: each rank allocates its receive buffers with the runtime allocator, exports an IPC
// handle, and opens its peers' handles (NVLink peer access).  Then
//
//   plan       ep_count_kernel (routes per expert) -> the caller's all_gather of the counts -> ep_plan_kernel: every
//              route's owner and final row in the owner's EXPERT-MAJOR receive buffer, one CTA, no host round trip;
//   dispatch   every rank stores each of its routed token rows straight into the owning rank's receive buffer at that
//              row, together with a return tag (source rank, item) (ep_dispatch_kernel: plain 16-byte peer stores);
//   compute    the owner turns the tags into addresses inside ITS mapping of the senders' combine buffers
//              (ep_return_addr_kernel) and runs the single-GPU grouped GEMMs on its receive buffer; the last GEMM's
//              epilogue stores each output row at that address (GemmArgs::out_rows), i.e. directly into the sender's memory;
//   combine    each rank sums its tokens' top-k result rows with the router weights (ep_combine_kernel);
//   ordering   a stream-ordered collective between the phases (the caller's) makes one rank's stores visible before
//              another rank reads them.
//
// Peer memory is only ever WRITTEN with ordinary st.global from these kernels and read by its owner; no TMA load, bulk
// copy or library kernel is handed a peer pointer.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstring>

#include "qb_device.cuh"
#include "qb_runtime.hpp"

namespace qb {
namespace {

// routes per expert: one CTA, shared-memory histogram.  expert ids are int64 (what a router's top-k gives).
__global__ void __launch_bounds__(1024) ep_count_kernel(long long const* __restrict__ expert_of_route, int routes, int experts,
                                                        int* __restrict__ counts) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < routes; r += blockDim.x) {
    long long const e = expert_of_route[r];
    if (e >= 0 && e < experts) atomicAdd(&hist[int(e)], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = hist[e];
}

// One CTA.  counts_all [world][experts] (every rank's ep_count result).  Item i of this rank = the i-th route in
// expert order (inside an expert, in whatever order the atomics grant: any order is a valid plan, each row's result
// does not depend on its neighbours).  Outputs per item: the local token, the owner rank, the row in the owner's
// buffer (experts in order; inside an expert the sources in rank order); per route: its item; and the cumulative rows
// per LOCAL expert of this rank, which its grouped GEMMs read as offsets.
__global__ void __launch_bounds__(1024) ep_plan_kernel(long long const* __restrict__ expert_of_route, int const* __restrict__ counts_all,
                                                       int rank, int world, int experts, int routes, int top_k,
                                                       int* __restrict__ item_token, int* __restrict__ item_rank,
                                                       int* __restrict__ item_pos, int* __restrict__ item_of_route,
                                                       int* __restrict__ local_off) {
  extern __shared__ int sh[];
  int* first_row = sh;                 // [experts] row of (expert, this source) in the owner's buffer
  int* first_item = sh + experts;      // [experts] first item of the expert among this rank's items
  int* cursor = sh + 2 * experts;      // [experts]
  __shared__ int warp_tot[2][32];
  int const per = experts / world;
  // Per expert, in parallel: rows of lower ranks (below), rows of all ranks (total), rows of this rank (mine); then two
  // block-wide exclusive scans over the experts (of mine: first item; of total: rows before the expert, taken relative to
  // the first expert of its owner).  A thread owns a run of consecutive experts so the scans are one pass of shuffles.
  int const chunk = (experts + int(blockDim.x) - 1) / int(blockDim.x), e0 = threadIdx.x * chunk;
  int below_l[4], mine_l[4], total_l[4];                           // experts <= 4096 and 1024 threads: chunk <= 4
  int sum_m = 0, sum_t = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int const e = e0 + i;
    below_l[i] = mine_l[i] = total_l[i] = 0;
    if (i < chunk && e < experts) {
      for (int s2 = 0; s2 < world; ++s2) {
        int const c = counts_all[s2 * experts + e];
        if (s2 < rank) below_l[i] += c;
        if (s2 == rank) mine_l[i] = c;
        total_l[i] += c;
      }
    }
    sum_m += mine_l[i]; sum_t += total_l[i];
  }
  int const lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int inc_m = sum_m, inc_t = sum_t;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int const um = __shfl_up_sync(0xffffffffu, inc_m, o), ut = __shfl_up_sync(0xffffffffu, inc_t, o);
    if (lane >= o) { inc_m += um; inc_t += ut; }
  }
  if (lane == 31) { warp_tot[0][wid] = inc_m; warp_tot[1][wid] = inc_t; }
  __syncthreads();
  if (wid == 0) {
    int vm = lane < int(blockDim.x >> 5) ? warp_tot[0][lane] : 0, vt = lane < int(blockDim.x >> 5) ? warp_tot[1][lane] : 0;
    int im = vm, it = vt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int const um = __shfl_up_sync(0xffffffffu, im, o), ut = __shfl_up_sync(0xffffffffu, it, o);
      if (lane >= o) { im += um; it += ut; }
    }
    warp_tot[0][lane] = im - vm; warp_tot[1][lane] = it - vt;       // exclusive over the warps
  }
  __syncthreads();
  int run_m = warp_tot[0][wid] + inc_m - sum_m, run_t = warp_tot[1][wid] + inc_t - sum_t;   // exclusive prefix of this thread's run
  // rows before each expert, over all experts, parked in `cursor` for the owner-relative subtraction below
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int const e = e0 + i;
    if (i < chunk && e < experts) {
      first_item[e] = run_m;
      cursor[e] = run_t;
      first_row[e] = below_l[i];
      run_m += mine_l[i]; run_t += total_l[i];
    }
  }
  if (e0 <= experts - 1 && e0 + chunk > experts - 1) sh[3 * experts] = run_t;   // grand total, by the thread that owns the last expert
  __syncthreads();
  int const grand = sh[3 * experts];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int const o = e / per, before = cursor[e] - cursor[o * per];
    first_row[e] += before;
    if (o == rank) local_off[e - o * per] = before;
  }
  if (threadIdx.x == 0) {
    int const end = (rank + 1) * per < experts ? cursor[(rank + 1) * per] : grand;
    local_off[per] = end - cursor[rank * per];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cursor[e] = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < routes; r += blockDim.x) {
    long long const e64 = expert_of_route[r];
    if (e64 < 0 || e64 >= experts) { item_of_route[r] = -1; continue; }
    int const e = int(e64), slot = atomicAdd(&cursor[e], 1), i = first_item[e] + slot;
    item_token[i] = r / top_k;
    item_rank[i] = e / per;
    item_pos[i] = first_row[e] + slot;
    item_of_route[r] = i;
  }
}

// One CTA per item.  The token row (row_bytes, a multiple of 16) goes to row item_pos[i] of rank item_rank[i]'s receive
// buffer, and the return tag (this rank << 32 | item) to the same index of its tag array.
__global__ void __launch_bounds__(128) ep_dispatch_kernel(uint8_t const* __restrict__ act, int const* __restrict__ item_token,
                                                          int const* __restrict__ item_rank, int const* __restrict__ item_pos,
                                                          unsigned long long const* __restrict__ peer_rows,
                                                          unsigned long long const* __restrict__ peer_tag,
                                                          int my_rank, int items, int row_bytes) {
  int const i = blockIdx.x;
  if (i >= items) return;
  int const o = item_rank[i], pos = item_pos[i];
  uint4 const* src = reinterpret_cast<uint4 const*>(act + size_t(item_token[i]) * row_bytes);
  uint4* dst = reinterpret_cast<uint4*>(peer_rows[o] + size_t(pos) * row_bytes);
  for (int c = threadIdx.x; c < row_bytes / 16; c += blockDim.x) dst[c] = __ldg(src + c);
  if (threadIdx.x == 0)
    reinterpret_cast<unsigned long long*>(peer_tag[o])[pos] = ((unsigned long long)(unsigned)my_rank << 32) | (unsigned)i;
  __threadfence_system();
}

// tags of the rows this rank received -> addresses in THIS process's mappings of the senders' combine buffers
__global__ void __launch_bounds__(256) ep_return_addr_kernel(unsigned long long const* __restrict__ tags,
                                                             unsigned long long const* __restrict__ peer_comb, int world,
                                                             int const* __restrict__ rows_dev, int max_rows, int row_bytes,
                                                             unsigned long long* __restrict__ addr) {
  int const rows = min(*rows_dev, max_rows);
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
    unsigned long long const t = tags[r];
    unsigned const src = unsigned(t >> 32), item = unsigned(t);
    addr[r] = src < unsigned(world) ? peer_comb[src] + (unsigned long long)item * (unsigned long long)row_bytes : 0ull;
  }
}

// out[t] = sum_j weights[t][j] * comb[item_of_route[t*top_k + j]], fp32 in route order, bf16 out.  One CTA per token.
__global__ void __launch_bounds__(128) ep_combine_kernel(__nv_bfloat16 const* __restrict__ comb, int const* __restrict__ item_of_route,
                                                         float const* __restrict__ weights, __nv_bfloat16* __restrict__ out,
                                                         int top_k, int h) {
  int const t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < h; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      int const i = item_of_route[t * top_k + j];
      if (i < 0) continue;
      float const w = weights[t * top_k + j];
      uint4 const v = *reinterpret_cast<uint4 const*>(comb + size_t(i) * h + c);
      __nv_bfloat162 const* v2 = reinterpret_cast<__nv_bfloat162 const*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) { float2 const f = __bfloat1622float2(v2[q]); acc[2 * q] = fmaf(w, f.x, acc[2 * q]); acc[2 * q + 1] = fmaf(w, f.y, acc[2 * q + 1]); }
    }
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) o2[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    *reinterpret_cast<uint4*>(out + size_t(t) * h + c) = o;
  }
}

// out[r][c] = silu(gu[r][c]) * gu[r][F + c] for the rows a device-side count says exist (bf16 in and out, fp32 math).
__global__ void __launch_bounds__(256) silu_mul_kernel(__nv_bfloat16 const* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                                       int const* __restrict__ rows_dev, int max_rows, int f) {
  int const rows = rows_dev ? min(*rows_dev, max_rows) : max_rows;
  int const per_row = f / 8;
  for (int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; idx < int64_t(rows) * per_row;
       idx += int64_t(gridDim.x) * blockDim.x) {
    int64_t const r = idx / per_row;
    int const c = int(idx % per_row) * 8;
    uint4 const g4 = *reinterpret_cast<uint4 const*>(gu + r * 2 * f + c);
    uint4 const u4 = *reinterpret_cast<uint4 const*>(gu + r * 2 * f + f + c);
    __nv_bfloat162 const* g2 = reinterpret_cast<__nv_bfloat162 const*>(&g4);
    __nv_bfloat162 const* u2 = reinterpret_cast<__nv_bfloat162 const*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 const g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
      o2[j] = __floats2bfloat162_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + r * f + c) = o4;
  }
}

}  // namespace
}  // namespace qb

using namespace qb;

extern "C" int quactlize_b200_peer_alloc(long long bytes, void** ptr, unsigned char* handle64) {
  if (bytes <= 0 || !ptr || !handle64) return 20;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  rt_clear_error();
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, size_t(bytes));
  if (e == cudaSuccess) e = cudaMemset(p, 0, size_t(bytes));
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    if (p) (void)cudaFree(p);
    rt_record(RtStatus::Allocation, "peer buffer", cudaGetErrorString(e));
    return kRuntimeError;
  }
  std::memcpy(handle64, &h, 64);
  *ptr = p;
  return 0;
}
extern "C" int quactlize_b200_peer_open(unsigned char const* handle64, void** ptr) {
  if (!handle64 || !ptr) return 20;
  rt_clear_error();
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t const e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { (void)cudaGetLastError(); rt_record(RtStatus::Allocation, "peer buffer open", cudaGetErrorString(e)); return kRuntimeError; }
  *ptr = p;
  return 0;
}
extern "C" int quactlize_b200_peer_close(void* ptr) {
  if (!ptr) return 20;
  cudaError_t const e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return kRuntimeError; }
  return 0;
}
extern "C" int quactlize_b200_peer_free(void* ptr) {
  if (!ptr) return 20;
  cudaError_t const e = cudaFree(ptr);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return kRuntimeError; }
  return 0;
}

// ---- rendezvous of the ranks through peer memory ---------------------------------------------------------------------------
// Every rank owns a small sync area that all peers have mapped: per barrier id a row of epoch words, one per source rank,
// this rank's own epoch counters (kept on the device so a replayed CUDA graph advances them), and from byte 1024 the
// table counts_all[world][experts].  One CTA: (optionally) store this rank's route counts into every rank's table, fence
// at system scope, store the new epoch into row `id`, word `rank`, of every rank's area, then wait until every word of the
// own row has reached the epoch.  The wait is bounded (2 s): a peer that never arrives leaves a status code, not a hang.
// It runs as one launch per GPU; ranks are different GPUs, so the launches run at the same time by construction.
constexpr int kEpSyncIds = 3, kEpSyncRow = 64, kEpSyncCountsByte = 1024;      // words per row; epochs follow the rows
__global__ void __launch_bounds__(256) ep_sync_kernel(unsigned long long const* __restrict__ peer_sync, int rank, int world, int id,
                                                      int const* __restrict__ counts_local, int experts, unsigned int* status) {
  __shared__ unsigned epoch_s;
  unsigned* mine = reinterpret_cast<unsigned*>(peer_sync[rank]);
  if (counts_local) {
    for (int i = threadIdx.x; i < world * experts; i += blockDim.x) {
      int const w = i / experts, e = i - w * experts;
      int* table = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(peer_sync[w]) + kEpSyncCountsByte);
      table[rank * experts + e] = counts_local[e];
    }
  }
  __threadfence_system();                                      // this thread's stores (and, through the launch order of the
  if (threadIdx.x == 0) epoch_s = ++mine[kEpSyncIds * kEpSyncRow + id];   // stream, the preceding kernels') before the epoch
  __syncthreads();
  unsigned const epoch = epoch_s;
  if (int(threadIdx.x) < world) {
    unsigned* theirs = reinterpret_cast<unsigned*>(peer_sync[threadIdx.x]) + id * kEpSyncRow + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
    unsigned const* flag = mine + id * kEpSyncRow + threadIdx.x;
    unsigned long long const t0 = global_ns();
    unsigned seen = 0, spins = 0;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
      if (int(seen - epoch) >= 0) break;                       // epochs only grow; a fast peer may already be one ahead
      if ((++spins & 255u) == 0 && global_ns() - t0 > kWaitNs) {
        if (status) atomicCAS(status, 0u, unsigned(kWaitStageTimeout));
        break;
      }
    }
  }
  __syncthreads();
}

extern "C" int quactlize_b200_ep_sync_bytes(int world, int experts) {
  if (world <= 0 || world > kEpSyncRow || experts < 0 || experts > 4096) return -1;
  return kEpSyncCountsByte + world * experts * 4;
}

extern "C" int quactlize_b200_ep_sync_dev_v1(unsigned long long const* peer_sync, int rank, int world, int id, int const* counts_local,
                                             int experts, void* stream) {
  if (!peer_sync || world <= 0 || world > kEpSyncRow || rank < 0 || rank >= world || id < 0 || id >= kEpSyncIds ||
      (counts_local && (experts <= 0 || experts > 4096))) return 20;
  rt_clear_error();
  unsigned int* status = rt_device_status_ptr();
  if (!status) return kRuntimeError;
  ep_sync_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(peer_sync, rank, world, id, counts_local, experts, status);
  return rt_check_launch("expert-parallel rendezvous enqueue") ? 0 : kRuntimeError;
}

extern "C" int quactlize_b200_ep_count_dev_v1(long long const* expert_of_route, int routes, int experts, int* counts, void* stream) {
  if (!expert_of_route || !counts || routes < 0 || experts <= 0 || experts > 4096) return 20;
  rt_clear_error();
  ep_count_kernel<<<1, 1024, size_t(experts) * 4, static_cast<cudaStream_t>(stream)>>>(expert_of_route, routes, experts, counts);
  return rt_check_launch("expert-parallel count enqueue") ? 0 : kRuntimeError;
}

extern "C" int quactlize_b200_ep_plan_dev_v1(long long const* expert_of_route, int const* counts_all, int rank, int world, int experts,
                                             int routes, int top_k, int* item_token, int* item_rank, int* item_pos,
                                             int* item_of_route, int* local_off, void* stream) {
  if (!expert_of_route || !counts_all || !item_token || !item_rank || !item_pos || !item_of_route || !local_off || world <= 0 ||
      rank < 0 || rank >= world || experts <= 0 || experts > 4096 || experts % world || routes < 0 || top_k <= 0) return 20;
  rt_clear_error();
  ep_plan_kernel<<<1, 1024, size_t(experts) * 12 + 16, static_cast<cudaStream_t>(stream)>>>(expert_of_route, counts_all, rank, world, experts,
                                                                                      routes, top_k, item_token, item_rank, item_pos,
                                                                                      item_of_route, local_off);
  return rt_check_launch("expert-parallel plan enqueue") ? 0 : kRuntimeError;
}

extern "C" int quactlize_b200_ep_dispatch_dev_v1(void const* act, int const* item_token, int const* item_rank, int const* item_pos,
                                                 unsigned long long const* peer_rows, unsigned long long const* peer_tag,
                                                 int my_rank, int items, int row_bytes, void* stream) {
  if (!act || !item_token || !item_rank || !item_pos || !peer_rows || !peer_tag || items < 0 || row_bytes <= 0 || row_bytes % 16 ||
      my_rank < 0 || (reinterpret_cast<uintptr_t>(act) & 15)) return 20;
  if (items == 0) return 0;
  rt_clear_error();
  ep_dispatch_kernel<<<items, 128, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint8_t const*>(act), item_token, item_rank,
                                                                           item_pos, peer_rows, peer_tag, my_rank, items, row_bytes);
  return rt_check_launch("expert-parallel dispatch enqueue") ? 0 : kRuntimeError;
}

extern "C" int quactlize_b200_ep_return_addr_dev_v1(unsigned long long const* tags, unsigned long long const* peer_comb, int world,
                                                    int const* rows_dev, int max_rows, int row_bytes, unsigned long long* addr,
                                                    void* stream) {
  if (!tags || !peer_comb || !rows_dev || !addr || world <= 0 || max_rows <= 0 || row_bytes <= 0) return 20;
  rt_clear_error();
  ep_return_addr_kernel<<<std::min((max_rows + 255) / 256, 64), 256, 0, static_cast<cudaStream_t>(stream)>>>(tags, peer_comb, world, rows_dev,
                                                                                                           max_rows, row_bytes, addr);
  return rt_check_launch("expert-parallel return addresses enqueue") ? 0 : kRuntimeError;
}

extern "C" int quactlize_b200_ep_combine_dev_v1(void const* comb, int const* item_of_route, float const* weights, void* out, int tokens,
                                                int top_k, int h, void* stream) {
  if (!comb || !item_of_route || !weights || !out || tokens < 0 || top_k <= 0 || h <= 0 || h % 8) return 20;
  if (tokens == 0) return 0;
  rt_clear_error();
  ep_combine_kernel<<<tokens, 128, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<__nv_bfloat16 const*>(comb), item_of_route, weights,
                                                                           static_cast<__nv_bfloat16*>(out), top_k, h);
  return rt_check_launch("expert-parallel combine enqueue") ? 0 : kRuntimeError;
}

extern "C" int quactlize_b200_silu_mul_dev_v1(void const* gate_up, void* out, int const* rows_dev, int max_rows, int f, void* stream) {
  if (!gate_up || !out || max_rows <= 0 || f <= 0 || f % 8) return 20;
  rt_clear_error();
  int64_t const work = int64_t(max_rows) * (f / 8);
  unsigned const grid = unsigned(std::min<int64_t>((work + 255) / 256, int64_t(rt_sm_count()) * 16));
  silu_mul_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<__nv_bfloat16 const*>(gate_up),
                                                                       static_cast<__nv_bfloat16*>(out), rows_dev, max_rows, f);
  return rt_check_launch("silu-mul enqueue") ? 0 : kRuntimeError;
}
