// moe_rd_route_dispatch_noalloc: the routing/dispatch pipeline for callers that
// cannot give it a workspace because they are not allowed to allocate device
// memory at all.  The scratch lives in a fixed array that is part of this
// library's device image.
#include <mutex>

#include "common.cuh"

namespace {

// Scratch shared by every call on a device.  It is reserved on each GPU that
// loads the library, for as long as the library stays loaded.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MOE_RD_NOALLOC_MAX_BYTES];

std::mutex g_mu;
void* g_scratch_ptr[64] = {};  // device address of g_noalloc_scratch, per device

// In host code the name g_noalloc_scratch is only a handle for the runtime, not
// an address a kernel may use: the real device address has to be asked for,
// once per device, with that device current.
int scratch_for_current_device(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MOE_RD_E_CUDA;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr)
      return MOE_RD_E_CUDA;
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return MOE_RD_OK;
}

}  // namespace

extern "C" int moe_rd_route_dispatch_noalloc(const moe_rd_params* p, const moe_rd_buffers* b,
                                             void* stream) {
  size_t need = 0;
  const int rc = moe_rd_workspace_bytes(p, &need);
  if (rc != MOE_RD_OK) return rc;
  if (need > (size_t)MOE_RD_NOALLOC_MAX_BYTES) return MOE_RD_E_TOO_LARGE;
  void* scratch = nullptr;
  const int rs = scratch_for_current_device(&scratch);
  if (rs != MOE_RD_OK) return rs;
  // The pipeline clears the part of the scratch that must start at zero (status
  // block, tile counts, expert counts) at the head of every call, so what an
  // earlier call left behind does not matter.
  return moe_rd_route_dispatch(p, b, scratch, (size_t)MOE_RD_NOALLOC_MAX_BYTES, stream);
}
