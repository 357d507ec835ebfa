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
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    moe_rd::set_last_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidDevice);
    return MOE_RD_E_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      moe_rd::set_last_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
      return MOE_RD_E_CUDA;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return MOE_RD_OK;
}

// The kernels run on the device of the stream; the scratch address belongs to the
// current device.  Refuse a stream of another device instead of handing its
// kernels an address of this one.
int stream_is_on_current_device(void* stream) {
  if (stream == nullptr) return MOE_RD_OK;  // the default stream of the current device
  int cur = 0, sdev = 0;
  cudaError_t e = cudaGetDevice(&cur);
  if (e == cudaSuccess) e = cudaStreamGetDevice(static_cast<cudaStream_t>(stream), &sdev);
  if (e != cudaSuccess) {
    moe_rd::set_last_cuda_error(e);
    return MOE_RD_E_CUDA;
  }
  return sdev == cur ? MOE_RD_OK : MOE_RD_E_UNSUPPORTED;
}

}  // namespace

extern "C" int moe_rd_route_dispatch_noalloc(const moe_rd_params* p, const moe_rd_buffers* b,
                                             void* stream) {
  size_t need = 0;
  const int rc = moe_rd_workspace_bytes(p, &need);
  if (rc != MOE_RD_OK) return rc;
  if (need > (size_t)MOE_RD_NOALLOC_MAX_BYTES) return MOE_RD_E_TOO_LARGE;
  const int rd = stream_is_on_current_device(stream);
  if (rd != MOE_RD_OK) return rd;
  void* scratch = nullptr;
  const int rs = scratch_for_current_device(&scratch);
  if (rs != MOE_RD_OK) return rs;
  // The pipeline clears the part of the scratch that must start at zero (status
  // block, tile counts, expert counts) at the head of every call, so what an
  // earlier call left behind does not matter.
  return moe_rd_route_dispatch(p, b, scratch, (size_t)MOE_RD_NOALLOC_MAX_BYTES, stream);
}

// Device status block of the last moe_rd_route_dispatch_noalloc call on the
// current device (its scratch address is private to this file, so
// moe_rd_read_status cannot be pointed at it).
extern "C" int moe_rd_read_status_noalloc(void* stream, int32_t status[8]) {
  const int rd = stream_is_on_current_device(stream);
  if (rd != MOE_RD_OK) return rd;
  void* scratch = nullptr;
  const int rs = scratch_for_current_device(&scratch);
  if (rs != MOE_RD_OK) return rs;
  return moe_rd_read_status(scratch, stream, status);
}
