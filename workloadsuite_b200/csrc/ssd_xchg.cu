// All-gather of the sequence shards' (final state, summed log-decay) blocks over NVLink peer memory: the one
// exchange of the sequence-sharded forward, as a kernel of this library instead of a collective-library call.
//
// Every rank owns one device buffer [world slots | entry flags | data flags]; the ranks open each other's buffers
// (CUDA IPC), and one launch per rank and step
//   1. tells every peer "I have entered exchange e" (so what a peer wrote for exchange e-1 has been consumed here:
//      the consumers run before this kernel in stream order),
//   2. waits for a peer's entry flag, then writes this rank's block into its own slot of that peer's buffer with
//      plain 16-byte stores (ordinary st.global to the mapped peer buffer, nothing else),
//   3. publishes "data of rank r for exchange e" on every peer (release at system scope) once all blocks of the
//      grid have finished their stores, and
//   4. waits until every rank's data flag for exchange e is set here (acquire at system scope).
// The exchange number lives in device memory and is advanced by the kernel itself, so a captured launch can be
// replayed.  Every wait is bounded by the clock; a wait that runs out records a status code and the kernel
// ends (the context stays usable).  One process per GPU: the ranks' kernels run on different devices.
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstring>
#include <new>

#include "ssd_b200.h"

namespace {

constexpr int kMaxWorld = 16;
constexpr int kThreads = 256;
constexpr int kChunksPerPeer = 16;
constexpr int32_t kStatusPeerTimeout = 7;

struct XchgDev {
  unsigned char* peer[kMaxWorld];   // base of every rank's buffer as mapped into this process (own buffer included)
  int rank, world;
  size_t slot_bytes;       // multiple of 16
  size_t flags_offset;     // byte offset of entry[world] (uint32), data[world] follows
  uint32_t* epoch;         // this rank's exchange counter (device memory)
  uint32_t* ticket;        // blocks of the current launch that have finished their stores
  long long wait_clocks;
  int32_t* status;
};

struct Xchg {
  XchgDev d;
  void* local;
  void* opened[kMaxWorld];
  size_t total_bytes;
  uint32_t* counters;   // epoch, ticket
  bool connected;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// true once *p has reached e (counters wrap: compare the signed difference)
__device__ bool wait_reached(const uint32_t* p, uint32_t e, long long limit, int32_t* status) {
  const long long t0 = clock64();
  while ((int32_t)(ld_acquire_sys(p) - e) < 0) {
    if (clock64() - t0 > limit) {
      if (status) atomicCAS(status, 0, kStatusPeerTimeout);
      return false;
    }
  }
  return true;
}

__global__ void __launch_bounds__(kThreads) xchg_all_gather_kernel(XchgDev x, const uint4* __restrict__ send, size_t bytes) {
  __shared__ int s_ok, s_last;
  const int tid = threadIdx.x;
  const uint32_t e = *x.epoch + 1;   // (advanced by the last block, which cannot exist before every block has read it)
  const int peer = (x.rank + 1 + blockIdx.x / kChunksPerPeer) % x.world;   // start with the neighbour: spreads the links
  const int chunk = blockIdx.x % kChunksPerPeer;
  uint32_t* my_entry = reinterpret_cast<uint32_t*>(x.peer[x.rank] + x.flags_offset);
  uint32_t* my_data = my_entry + x.world;

  // 1. entry flags: one block tells all peers
  if (blockIdx.x == 0 && tid < x.world)
    st_release_sys(reinterpret_cast<uint32_t*>(x.peer[tid] + x.flags_offset) + x.rank, e);

  // 2. the peer must have entered this exchange before its slot is overwritten
  if (tid == 0) s_ok = wait_reached(my_entry + peer, e, x.wait_clocks, x.status) ? 1 : 0;
  __syncthreads();
  if (s_ok) {
    const size_t n16 = bytes / 16, per = (n16 + kChunksPerPeer - 1) / kChunksPerPeer;
    const size_t lo = per * chunk, hi = lo + per < n16 ? lo + per : n16;
    uint4* dst = reinterpret_cast<uint4*>(x.peer[peer] + (size_t)x.rank * x.slot_bytes);
    for (size_t i = lo + tid; i < hi; i += kThreads) dst[i] = send[i];
  }
  // 3. the last block to finish publishes the data flags ...
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    s_last = (atomicAdd(x.ticket, 1u) == gridDim.x - 1) ? 1 : 0;
    __threadfence();
  }
  __syncthreads();
  if (!s_last) return;
  if (tid < x.world)
    st_release_sys(reinterpret_cast<uint32_t*>(x.peer[tid] + x.flags_offset) + x.world + x.rank, e);
  // 4. ... and waits for everybody's
  if (tid < x.world) wait_reached(my_data + tid, e, x.wait_clocks, x.status);
  __syncthreads();
  if (tid == 0) {
    *x.ticket = 0;
    *x.epoch = e;
  }
}

}  // namespace

extern "C" {

int ssd_b200_xchg_create(size_t slot_bytes, int32_t world, void** ctx_out, void* handle_out) {
  if (!ctx_out || !handle_out) return SSD_ERR_NULL_POINTER;
  if (world < 1 || world > kMaxWorld || slot_bytes == 0) return SSD_ERR_BAD_SHAPE;
  Xchg* x = new (std::nothrow) Xchg();
  if (!x) return SSD_ERR_BAD_SHAPE;
  x->d.world = world;
  x->d.rank = -1;
  x->d.slot_bytes = (slot_bytes + 15) / 16 * 16;
  x->d.flags_offset = x->d.slot_bytes * world;
  x->total_bytes = x->d.flags_offset + 2 * sizeof(uint32_t) * world;
  x->total_bytes = (x->total_bytes + 255) / 256 * 256;
  if (cudaMalloc(&x->local, x->total_bytes) != cudaSuccess ||
      cudaMalloc(reinterpret_cast<void**>(&x->counters), 2 * sizeof(uint32_t)) != cudaSuccess) {
    if (x->local) cudaFree(x->local);
    delete x;
    return SSD_ERR_CUDA;
  }
  cudaMemset(x->local, 0, x->total_bytes);
  cudaMemset(x->counters, 0, 2 * sizeof(uint32_t));
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, x->local) != cudaSuccess) {
    cudaFree(x->local);
    cudaFree(x->counters);
    delete x;
    return SSD_ERR_CUDA;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == SSD_XCHG_HANDLE_BYTES, "handle size");
  memcpy(handle_out, &h, sizeof(h));
  cudaDeviceSynchronize();
  x->d.epoch = x->counters;
  x->d.ticket = x->counters + 1;
  *ctx_out = x;
  return SSD_OK;
}

int ssd_b200_xchg_connect(void* ctx, const void* handles, int32_t rank) {
  Xchg* x = static_cast<Xchg*>(ctx);
  if (!x || !handles || rank < 0 || rank >= x->d.world || x->connected) return SSD_ERR_BAD_SHAPE;
  x->d.rank = rank;
  for (int r = 0; r < x->d.world; ++r) {
    if (r == rank) {
      x->d.peer[r] = static_cast<unsigned char*>(x->local);
      continue;
    }
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const unsigned char*>(handles) + (size_t)r * SSD_XCHG_HANDLE_BYTES, sizeof(h));
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      cudaGetLastError();
      for (int q = 0; q < r; ++q)
        if (x->opened[q]) { cudaIpcCloseMemHandle(x->opened[q]); x->opened[q] = nullptr; }
      return SSD_ERR_CUDA;
    }
    x->opened[r] = p;
    x->d.peer[r] = static_cast<unsigned char*>(p);
  }
  x->connected = true;
  return SSD_OK;
}

void* ssd_b200_xchg_buffer(void* ctx) {
  Xchg* x = static_cast<Xchg*>(ctx);
  return x ? x->local : nullptr;
}

int ssd_b200_xchg_all_gather(void* ctx, const void* send, size_t bytes, int32_t* status, int32_t wait_limit_ms,
                             void* stream) {
  Xchg* x = static_cast<Xchg*>(ctx);
  if (!x || !x->connected || !send || bytes == 0 || bytes % 16 != 0 || bytes > x->d.slot_bytes ||
      (reinterpret_cast<uintptr_t>(send) & 15))
    return SSD_ERR_BAD_SHAPE;
  int dev = 0, khz = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
  XchgDev d = x->d;
  d.wait_clocks = (long long)(wait_limit_ms > 0 ? wait_limit_ms : 2000) * (khz > 0 ? khz : 1965000);
  d.status = status;
  xchg_all_gather_kernel<<<x->d.world * kChunksPerPeer, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      d, static_cast<const uint4*>(send), bytes);
  return cudaGetLastError() == cudaSuccess ? SSD_OK : SSD_ERR_CUDA;
}

int ssd_b200_xchg_destroy(void* ctx) {
  Xchg* x = static_cast<Xchg*>(ctx);
  if (!x) return SSD_ERR_BAD_SHAPE;
  cudaDeviceSynchronize();
  for (int r = 0; r < kMaxWorld; ++r)
    if (x->opened[r]) cudaIpcCloseMemHandle(x->opened[r]);
  cudaFree(x->local);
  cudaFree(x->counters);
  delete x;
  return SSD_OK;
}

}  // extern "C"
