// SSD forward for callers that cannot allocate device memory.
//
// The segmented forward (each sequence cut into independently scanned segments
// joined by a state fold) needs scratch for the per-segment states.  The normal
// entry point takes that scratch from the caller.  Some callers have nothing to
// give: a plugin running inside a host runtime that owns the whole device heap
// and forbids cudaMalloc on its request path (the call synchronises the device
// and fails once the host has reserved the memory), or a thin C/FFI client that
// has no allocator of its own.  For them this file keeps one fixed scratch
// array in the library image and lends it to the existing forward.
#include <mutex>

#include "ssd_common.cuh"

namespace {

constexpr size_t kStaticScratchBytes = SSD_STATIC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// Lives in every GPU that loads the library, from module load until exit.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal

// In host code `g_static_scratch` is only a handle for the runtime, not a device
// address; the address a kernel may use comes from cudaGetSymbolAddress, asked
// once per device while that device is current.
int scratch_for_current_device(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return SSD_ERR_CUDA;
  if (dev < 0 || dev >= kMaxDevices) return SSD_ERR_TOO_LARGE;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return SSD_ERR_CUDA;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return SSD_OK;
}

}  // namespace

extern "C" {

size_t ssd_b200_static_scratch_capacity(void) { return kStaticScratchBytes; }

int ssd_b200_forward_static_scratch(const SsdArgs* args, void* stream) {
  if (!args) return SSD_ERR_NULL_POINTER;
  SsdArgs a = *args;
  a.workspace = nullptr;
  a.workspace_bytes = 0;
  const size_t need = ssd_b200_workspace_bytes(&a);  // 0 for invalid arguments: the forward reports those
  if (need > kStaticScratchBytes) return SSD_ERR_TOO_LARGE;
  if (need > 0) {
    void* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc != SSD_OK) return rc;
    a.workspace = scratch;
    a.workspace_bytes = kStaticScratchBytes;
  }
  // The two-pass forward writes every segment state and log-decay sum before it reads
  // it; the single-launch (chained) forward needs its ready flags at zero and clears
  // them itself with a memset on `stream`.  So the caller never has to clear the array.
  return ssd_b200_forward(&a, stream);
}

}  // extern "C"
