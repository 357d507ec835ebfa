// Placeholder translation unit: the tcgen05 gate product is added separately.
#include "common.cuh"

namespace moe_rd {

bool umma_available() { return false; }

cudaError_t init_umma_attributes() { return cudaSuccess; }

cudaError_t launch_gate_umma(const moe_rd_params&, const moe_rd_buffers&, const Plan&, void*,
                             float*, float*, int32_t*, cudaStream_t) {
  return cudaErrorNotSupported;
}

}  // namespace moe_rd
