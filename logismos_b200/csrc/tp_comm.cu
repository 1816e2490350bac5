// All-reduce of the tensor-parallel partial sums, fused with the residual add, over NVLink peer memory.
//
// The hybrid decoder's tensor-parallel form (logismos_model.h) leaves, after every output projection,
// a partial sum [tokens, hidden] fp32 on each rank; the residual stream needs x += sum over ranks.
// The messages are small (tokens * hidden * 4 B: 256 KB at 32 decode tokens) and there are two per
// layer, so what matters is latency, not bandwidth: ONE kernel per rank does the whole exchange.
//   phase 1  every CTA copies its slices of the local partial sum into each peer's receive buffer
//            (plain 16-byte peer stores over NVLink), fences, and raises its flag in the peer's memory
//   phase 2  it waits (bounded) for the same CTA's flag from every peer, then adds the local partial
//            and the received ones, in rank order on every rank, into the residual stream
// All CTAs of the grid are co-resident (grid <= SM count) and every CTA publishes before it waits, so
// no CTA can wait for one that has not been scheduled. Receive buffers and flags alternate between two
// sets by call parity: a rank can start call e + 1 (writing set (e + 1) & 1 at its peer) while the peer
// still reads set e & 1, and cannot reach call e + 2 before the peer has finished call e, because
// finishing call e + 1 needs the flag the peer raises in ITS call e + 1. Flags carry the call number and
// are never reset. The ranks are processes on different GPUs of one node; the buffers are shared with
// cudaIpc handles. No reference counterpart: the reference has no multi-GPU code at all.
//
// The wait is bounded: after kSpinLimit polls a CTA raises status 3, skips its add and returns, so a
// peer that died between steps costs a wrong step that is reported, not a hung GPU.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "logismos_model.h"

namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 256;     // flags per (set, rank)
constexpr int kThreads = 256;
constexpr uint32_t kSpinLimit = 1u << 21;

struct TpComm {
  int rank = 0, tp = 1, device = 0, grid_cap = 0;
  uint64_t max_elems = 0;
  void* region = nullptr;           // this rank's region (flags, then receive buffers)
  void* peer_region[kMaxRanks] = {nullptr};
  bool opened[kMaxRanks] = {false};
  uint32_t epoch = 0;
  std::mutex mu;
};

// region layout: flags u32 [2][tp][kMaxCtas] | pad to 256 B | recv f32 [2][tp][max_elems]
inline size_t flags_bytes(int tp) { return (((size_t)2 * tp * kMaxCtas * 4) + 255) & ~(size_t)255; }
inline size_t region_bytes(int tp, uint64_t max_elems) { return flags_bytes(tp) + (size_t)2 * tp * max_elems * 4; }

struct Peers {
  float* recv[kMaxRanks];       // recv[r]: rank r's region's receive area (r == me: local)
  uint32_t* flags[kMaxRanks];
};

LG_DEVINL void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory"); }
LG_DEVINL uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kThreads)
tp_reduce_add_kernel(float* __restrict__ x, const float* __restrict__ delta, uint64_t count4, Peers peers, int me, int tp,
                     uint64_t max_elems, uint32_t epoch, int* __restrict__ status) {
  const int set = (int)(epoch & 1u);
  const uint64_t stride = (uint64_t)gridDim.x * kThreads;
  const uint64_t first = (uint64_t)blockIdx.x * kThreads + threadIdx.x;
  const float4* d4 = reinterpret_cast<const float4*>(delta);
  // phase 1: my slices into slot `me` of every peer's receive set
  for (int r = 0; r < tp; ++r) {
    if (r == me) continue;
    float4* dst = reinterpret_cast<float4*>(peers.recv[r] + ((size_t)set * tp + me) * max_elems);
    for (uint64_t i = first; i < count4; i += stride) dst[i] = d4[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0)
    for (int r = 0; r < tp; ++r)
      if (r != me) st_release_sys(peers.flags[r] + ((size_t)set * tp + me) * kMaxCtas + blockIdx.x, epoch);
  // phase 2: wait for every peer's slices of this CTA
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int r = 0; r < tp && ok; ++r) {
      if (r == me) continue;
      const uint32_t* f = peers.flags[me] + ((size_t)set * tp + r) * kMaxCtas + blockIdx.x;
      uint32_t spins = 0;
      while (ld_acquire_sys(f) != epoch) {
        if (++spins > kSpinLimit) { ok = 0; break; }
        __nanosleep(64);
      }
    }
    if (!ok && status) atomicExch(status, 3);
    ok_s = ok;
  }
  __syncthreads();
  if (!ok_s) return;
  float4* x4 = reinterpret_cast<float4*>(x);
  for (uint64_t i = first; i < count4; i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < tp; ++r) {  // rank order on every rank: the replicas stay bit-identical
      const float4 v = r == me ? d4[i] : __ldcg(reinterpret_cast<const float4*>(peers.recv[me] + ((size_t)set * tp + r) * max_elems) + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float4 xv = x4[i];
    xv.x += acc.x; xv.y += acc.y; xv.z += acc.z; xv.w += acc.w;
    x4[i] = xv;
  }
}

}  // namespace

extern "C" {

size_t lg_tp_comm_region_bytes(int32_t tp, uint64_t max_elems) {
  if (tp < 1 || tp > kMaxRanks || max_elems == 0 || (max_elems & 3)) return 0;
  return region_bytes(tp, max_elems);
}

uint32_t lg_tp_comm_alloc(int32_t device, int32_t tp, uint64_t max_elems, void** region, uint8_t* handle_out64) {
  if (!region || !handle_out64 || lg_tp_comm_region_bytes(tp, max_elems) == 0) return 1;
  if (cudaSetDevice(device) != cudaSuccess) return (uint32_t)cudaGetLastError();
  void* p = nullptr;
  const size_t bytes = region_bytes(tp, max_elems);
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return (uint32_t)e;
  e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaFree(p); return (uint32_t)e; }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  std::memcpy(handle_out64, &h, 64);
  *region = p;
  return 0;
}

uint32_t lg_tp_comm_open(int32_t device, void* region, int32_t rank, int32_t tp, uint64_t max_elems, const uint8_t* all_handles,
                         void** comm) {
  if (!region || !comm || !all_handles || rank < 0 || rank >= tp || lg_tp_comm_region_bytes(tp, max_elems) == 0) return 1;
  if (cudaSetDevice(device) != cudaSuccess) return (uint32_t)cudaGetLastError();
  TpComm* c = new TpComm();
  c->rank = rank; c->tp = tp; c->device = device; c->max_elems = max_elems; c->region = region;
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  c->grid_cap = sms > 0 && sms < kMaxCtas ? sms : (sms >= kMaxCtas ? kMaxCtas : 128);
  for (int r = 0; r < tp; ++r) {
    if (r == rank) { c->peer_region[r] = region; continue; }
    cudaIpcMemHandle_t h;
    std::memcpy(&h, all_handles + (size_t)r * 64, 64);
    cudaError_t e = cudaIpcOpenMemHandle(&c->peer_region[r], h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      for (int k = 0; k < r; ++k) if (c->opened[k]) cudaIpcCloseMemHandle(c->peer_region[k]);
      delete c;
      return (uint32_t)e;
    }
    c->opened[r] = true;
  }
  *comm = c;
  return 0;
}

void lg_tp_comm_destroy(void* comm, int32_t free_region) {
  if (!comm) return;
  TpComm* c = static_cast<TpComm*>(comm);
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  for (int r = 0; r < c->tp; ++r) if (c->opened[r]) cudaIpcCloseMemHandle(c->peer_region[r]);
  if (free_region && c->region) cudaFree(c->region);
  delete c;
}

// x += sum over ranks of delta, for count floats (count % 4 == 0, count <= max_elems, 16-byte aligned
// pointers). Every rank must make the same sequence of calls with the same counts. The signature is
// lg_reduce_add_f32_fn (logismos_model.h) with `user` = the communicator.
uint32_t lg_tp_reduce_add_f32(void* comm, void* x_f32, void* delta_f32, uint64_t count, void* status_i32, void* stream) {
  TpComm* c = static_cast<TpComm*>(comm);
  if (!c || !x_f32 || !delta_f32 || (count & 3) || count > c->max_elems || ((uintptr_t)x_f32 & 15) || ((uintptr_t)delta_f32 & 15)) return 1;
  if (count == 0) return 0;
  std::lock_guard<std::mutex> lock(c->mu);
  (void)cudaGetLastError();
  Peers p;
  for (int r = 0; r < kMaxRanks; ++r) { p.recv[r] = nullptr; p.flags[r] = nullptr; }
  for (int r = 0; r < c->tp; ++r) {
    p.flags[r] = (uint32_t*)c->peer_region[r];
    p.recv[r] = (float*)((uint8_t*)c->peer_region[r] + flags_bytes(c->tp));
  }
  const uint64_t count4 = count / 4;
  uint64_t grid = (count4 + kThreads - 1) / kThreads;
  if (grid > (uint64_t)c->grid_cap) grid = (uint64_t)c->grid_cap;
  c->epoch += 1;
  tp_reduce_add_kernel<<<(unsigned)grid, kThreads, 0, (cudaStream_t)stream>>>((float*)x_f32, (const float*)delta_f32, count4, p, c->rank,
                                                                             c->tp, c->max_elems, c->epoch, (int*)status_i32);
  return (uint32_t)cudaGetLastError();
}

}  // extern "C"
