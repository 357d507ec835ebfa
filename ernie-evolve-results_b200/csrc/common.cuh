// Internal declarations shared by the kernels of libmoe_rd.so.
//
// Numerics contract: every fp32 operation on the routing path is a single
// IEEE-754 operation in a fixed order (explicit __fadd_rn/__fmul_rn/__fdiv_rn
// and fmaf), so a CPU restatement that follows the same order reproduces the
// results bit for bit.  The library is compiled with -fmad=false so that the
// compiler never fuses a multiply and an add that the source keeps apart.
#pragma once

#include <cuda_bf16.h>
#include <utility>
#include <cuda_runtime.h>
#include <stdint.h>

#include "moe_rd.h"

namespace moe_rd {

constexpr int kTile = 64;    // tokens per counting tile (granularity of the expert histogram)
constexpr int kTileGroup = 32;  // counting tiles per group (second level of the histogram)
constexpr int kMaxE = 256;
constexpr int kMaxK = 32;
constexpr unsigned kFull = 0xffffffffu;

// Workspace carving, computed identically by moe_rd_workspace_bytes and by
// the call itself.  All offsets are multiples of 256 bytes.
struct Workspace {
  size_t status;       // int32[8]  device status block            } cleared at the
  size_t tile_base;    // int32[E*ntiles] per-tile counts, scanned } start of a call
                       //           in place to bases
  size_t counts;       // int32[E]  pairs per expert before dropping }
  size_t group_counts; // int32[groups*E] pairs per expert and group of kTileGroup tiles }
  size_t dense;        // int32[1+kMaxK] number and first rows of identity experts }
  size_t zero_bytes;   // length of that cleared prefix
  size_t logits;       // float[T*E] when the caller passes no router_logits
  size_t ids;          // int32[T*K] when the caller passes no expert_ids
  size_t wt;           // bf16[N*H]  gate weight in [N,H] order for the tensor-core gate (N = E, or
                       //            2E: hi rows then lo rows of an fp32 weight)
  size_t partial;      // float[S*T*N] split-K partial logits of the tensor-core gate
  size_t total;
};

struct Plan {
  int ntiles;      // ceil(T / kTile)
  int gate;        // resolved MOE_RD_GATE_*
  int scatter;     // resolved MOE_RD_SCATTER_*
  int ksplit;      // split-K factor of the tensor-core gate
  int umma_mh;     // 128-token halves per CTA of the tensor-core gate (1 or 2)
  int umma_pair;   // 1: two-CTA tiles (cta_group::2), each CTA fetching half of every W tile
  int tile_major;  // 1: the routing kernel leaves pair counts per [tile][expert] and per [group of
                   //    tiles][expert] and the positions kernel derives tile bases and offsets from
                   //    them (no scan kernel); 0: counts per [expert][tile], scanned in place
  int umma_fold;   // 1: fp32 gate weight split into bf16 hi and lo rows; the product has 2E columns
                   //    and logit e = column e + column E+e
  int umma_n;      // columns of the tensor-core product: E, or 2E with umma_fold
};

int make_plan(const moe_rd_params& p, Plan* plan);
void carve(const moe_rd_params& p, const Plan& plan, bool need_logits, bool need_ids, Workspace* w);

// Launchers (each returns cudaError_t of the launch).  Defined one per .cu.
cudaError_t launch_gate_simt(const moe_rd_params& p, const moe_rd_buffers& b, float* logits,
                             cudaStream_t s);
cudaError_t launch_gate_umma(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                             void* wt, float* partial, float* logits, int32_t* status, void* zero, size_t zero_bytes,
                             cudaStream_t s);
cudaError_t launch_route(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                         const float* logits, int32_t* ids, int32_t* tile_base, int32_t* counts,
                         int32_t* group_counts, cudaStream_t s);
cudaError_t launch_route_splits(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                                const float* partial, int nsplit, const float* logit_bias,
                                float* logits_out, int32_t* ids, int32_t* tile_base,
                                int32_t* counts, int32_t* group_counts, cudaStream_t s);
cudaError_t launch_gemv_route(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                              float* logits_out, int32_t* ids, int32_t* tile_base, int32_t* counts, int32_t* ticket,
                              cudaStream_t s);
cudaError_t launch_scatter(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                           const int32_t* ids, const int32_t* tile_base, const int32_t* counts,
                           int32_t* status, int32_t* dense, const int32_t* group_counts, cudaStream_t s,
                           cudaEvent_t after_positions = nullptr);
bool fused_front_eligible(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan);
cudaError_t launch_gate_route(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan, void* wt,
                              int32_t* ids, int32_t* tile_counts, int32_t* group_counts, int32_t* status,
                              cudaStream_t s);
bool umma_available();
bool gemv_eligible(const moe_rd_params& p);
void count_launch(int n = 1);
void set_last_cuda_error(cudaError_t e);  // what moe_rd_last_cuda_error reports on this thread

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------
#ifdef __CUDACC__

// Programmatic dependent launch.  Every kernel of the pipeline lets the next
// launch start early (its blocks then park in pdl_sync until this grid has
// completed and its writes are visible) and itself waits for the previous grid
// before it touches global memory.  This hides the launch latency between the
// short kernels of a call.  Without the launch attribute both
// instructions do nothing.
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_sync() {
  pdl_trigger();
  pdl_wait();
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// <<<grid, block, smem, stream>>> with the programmatic-serialization attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// First failing check wins; later ones are dropped.  The caller skips the access.
__device__ __forceinline__ void report(int32_t* status, int id, int a, int b) {
  if (atomicCAS(&status[0], 0, 1) == 0) {
    status[1] = id;
    status[2] = a;
    status[3] = b;
  }
}

__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) {
  return __uint_as_float(packed & 0xffff0000u);
}

__device__ __forceinline__ void unpack8(const uint4& v, float f[8]) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x);
  f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z);
  f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}

// exp(x) from IEEE operations only (no MUFU): n = rint(x*log2 e), two-step
// Cody-Waite reduction, degree-6 polynomial, scale through the exponent field.
__device__ __forceinline__ float exp_ieee(float x) {
  if (x < -87.0f) return 0.0f;
  if (x > 88.0f) return __int_as_float(0x7f800000);
  const float n = rintf(__fmul_rn(x, 1.44269504f));
  const int ni = (int)n;
  float r = fmaf(n, -0.693145752f, x);
  r = fmaf(n, -1.42860677e-6f, r);
  float p = 1.9875691500e-4f;
  p = fmaf(p, r, 1.3981999507e-3f);
  p = fmaf(p, r, 8.3334519073e-3f);
  p = fmaf(p, r, 4.1665795894e-2f);
  p = fmaf(p, r, 1.6666665459e-1f);
  p = fmaf(p, r, 5.0000001201e-1f);
  const float r2 = __fmul_rn(r, r);
  float y = fmaf(p, r2, r);
  y = __fadd_rn(y, 1.0f);
  const float s = __int_as_float((ni + 127) << 23);
  return __fmul_rn(y, s);
}

// Sum over the warp by the tree v[l] += v[l^off], off = 16..1; every lane ends
// with the same value because fp32 addition is commutative.
__device__ __forceinline__ float warp_tree_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(kFull, v, o));
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, o));
  return v;
}

// Arg-max over the warp; on equal values the lower index wins
// (reference: topk_kernel, kernel.cu:1882-1890).
__device__ __forceinline__ void warp_argmax(float& bv, int& bi) {
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(kFull, bv, o);
    const int oi = __shfl_xor_sync(kFull, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
}

#endif  // __CUDACC__

}  // namespace moe_rd
