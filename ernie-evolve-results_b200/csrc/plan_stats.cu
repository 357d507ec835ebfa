// Small consumers of the routed offsets: the device-side plan of a grouped
// (ragged) expert GEMM and per-expert statistics.
//
// gemm_plan_kernel follows plan_kernel of the reference (moe_gemm.cu:613-638):
// one thread per expert turns offsets into a problem shape and the A / B / D
// pointers of its group, with no host synchronisation; a group that holds every
// token exactly once (rows == ident_m) reads the un-permuted x instead of its
// slice of the permuted buffer (moe_gemm.h:66-75).  The reference fills CUTLASS
// stride objects; here the pitches are plain byte counts.
//
// expert_stats_kernel makes first-class outputs of what the reference keeps for
// its own precision selector (wsum / counts, kernel.cu:1903-1919).  The reference
// accumulates wsum with floating-point atomics, whose order is not defined; here
// the weights of an expert's rows are added in a fixed order.
#include "common.cuh"

namespace moe_rd {
namespace {

__global__ void gemm_plan_kernel(const int32_t* __restrict__ offsets, int E, const unsigned char* a_rows,
                                 int64_t a_row_bytes, const unsigned char* ident_a, int64_t ident_m,
                                 const unsigned char* w, int64_t w_expert_bytes, unsigned char* d_rows,
                                 int64_t d_row_bytes, int n, int k, moe_rd_gemm_group* groups) {
  pdl_sync();
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const int64_t start = offsets[e];
  const int m = offsets[e + 1] - offsets[e];
  const bool ident = ident_m > 0 && (int64_t)m == ident_m && ident_a != nullptr;
  moe_rd_gemm_group g;
  g.m = m;
  g.n = n;
  g.k = k;
  g.identity = ident ? 1 : 0;
  g.a = ident ? ident_a : a_rows + start * a_row_bytes;
  g.b = w + (int64_t)e * w_expert_bytes;
  g.d = d_rows + start * d_row_bytes;
  g.lda = a_row_bytes;
  g.ldb = w_expert_bytes;
  g.ldd = d_row_bytes;
  groups[e] = g;
}

constexpr int kStatThreads = 256;

__global__ void __launch_bounds__(kStatThreads)
expert_stats_kernel(const int32_t* __restrict__ offsets, const float* __restrict__ row_weight, int E,
                    float* __restrict__ weight_sum, float* __restrict__ mean_weight,
                    float* __restrict__ load) {
  __shared__ float s_v[kStatThreads];
  pdl_sync();
  const int e = blockIdx.x, tid = threadIdx.x;
  const int lo = offsets[e], hi = offsets[e + 1];
  float v = 0.0f;
  if (row_weight != nullptr)
    for (int i = lo + tid; i < hi; i += kStatThreads) v = __fadd_rn(v, row_weight[i]);
  s_v[tid] = v;
  __syncthreads();
  for (int off = kStatThreads / 2; off; off >>= 1) {
    if (tid < off) s_v[tid] = __fadd_rn(s_v[tid], s_v[tid + off]);
    __syncthreads();
  }
  if (tid == 0) {
    const int rows = hi - lo;
    const int total = offsets[E];
    if (weight_sum != nullptr) weight_sum[e] = s_v[0];
    if (mean_weight != nullptr) mean_weight[e] = __fdiv_rn(s_v[0], (float)(rows > 0 ? rows : 1));
    if (load != nullptr) load[e] = __fdiv_rn((float)rows, (float)(total > 0 ? total : 1));
  }
}

}  // namespace
}  // namespace moe_rd

using namespace moe_rd;

extern "C" int moe_rd_gemm_plan(const int32_t* offsets, int32_t E, const void* a_rows,
                                int64_t a_row_bytes, const void* ident_a, int64_t ident_m,
                                const void* w, int64_t w_expert_bytes, void* d_rows,
                                int64_t d_row_bytes, int32_t n, int32_t k,
                                moe_rd_gemm_group* groups, void* stream) {
  if (offsets == nullptr || groups == nullptr) return MOE_RD_E_NULL;
  if (E <= 0 || E > kMaxE || n < 0 || k < 0 || a_row_bytes < 0 || d_row_bytes < 0 || w_expert_bytes < 0 ||
      ident_m < 0)
    return MOE_RD_E_SHAPE;
  const cudaError_t e = launch_pdl(gemm_plan_kernel, dim3((unsigned)((E + 127) / 128)), dim3(128), 0,
                                   static_cast<cudaStream_t>(stream), offsets, (int)E,
                                   static_cast<const unsigned char*>(a_rows), a_row_bytes,
                                   static_cast<const unsigned char*>(ident_a), ident_m,
                                   static_cast<const unsigned char*>(w), w_expert_bytes,
                                   static_cast<unsigned char*>(d_rows), d_row_bytes, (int)n, (int)k, groups);
  count_launch();
  return e == cudaSuccess ? MOE_RD_OK : MOE_RD_E_CUDA;
}

extern "C" int moe_rd_expert_stats(const int32_t* offsets, const float* row_weight, int32_t E,
                                   float* weight_sum, float* mean_weight, float* load, void* stream) {
  if (offsets == nullptr) return MOE_RD_E_NULL;
  if ((weight_sum != nullptr || mean_weight != nullptr) && row_weight == nullptr) return MOE_RD_E_NULL;
  if (E <= 0 || E > kMaxE) return MOE_RD_E_SHAPE;
  const cudaError_t e = launch_pdl(expert_stats_kernel, dim3((unsigned)E), dim3(kStatThreads), 0,
                                   static_cast<cudaStream_t>(stream), offsets, row_weight, (int)E, weight_sum,
                                   mean_weight, load);
  count_launch();
  return e == cudaSuccess ? MOE_RD_OK : MOE_RD_E_CUDA;
}
