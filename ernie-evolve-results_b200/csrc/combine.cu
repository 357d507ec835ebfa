// Weighted combine (un-permute): out[t,:] = shared[t,:] + sum_k w[t,k] * y[inverse_perm[t,k],:]
//
// The consumer of inverse_perm and combine_weights; follows combine_kernel of
// the reference (kernel.cu:2365-2428): the K gathered 16-byte vectors are all
// loaded before any arithmetic (so K loads are outstanding per lane), the fp32
// accumulator starts from the shared-expert row (or 0), slots are added in
// order k = 0..K-1 by one fused multiply-add each, the result is rounded once
// to bf16; loads and stores carry streaming hints because every byte is touched
// once (kernel.cu:2391-2404).  Pairs dropped by the capacity limit
// (inverse_perm < 0) contribute nothing.  Work units (a token x 32 vectors of
// 16 bytes) are dealt to warps grid-stride with many more blocks than fit, as
// in the row scatter.
//
// Expert-parallel form (EP == true): the expert outputs stay where the experts
// ran.  The row of pair (t,k) then lives on rank ids[t,k] / experts_per_rank, at
// the row the dispatch stored it to, and is fetched from there with plain
// 16-byte peer loads over NVLink inside the same kernel that weights and adds
// it: the return all-to-all and the un-permute are one pass, and no receive
// buffer exists.  Arithmetic and order are those of the local form.
#include "common.cuh"

namespace moe_rd {
namespace {

constexpr int kCombineThreads = 256;
constexpr int kCombineWarps = kCombineThreads / 32;
constexpr int kCombineBlocksPerSm = 64;

struct CombineArgs {
  const uint4* y;
  const int32_t* inverse_perm;
  const float* weights;
  const uint4* shared;
  uint4* out;
  int64_t T;
  int nvec, K;
  // EP: y of rank d is peer_y[d]; pair (t,k) of expert e is row
  // dest_base[e] + (inverse_perm[t,k] - offsets[e]) there
  const uint4* peer_y[8];
  const int32_t* ids;
  const int32_t* offsets;
  const int32_t* dest_base;
  int epr;
};

// Row of pair (t,k) kept at local row pos; null when the pair has no row on its
// owner (moe_rd_ep_plan found that the expert's rows do not fit there).
template <bool EP>
__device__ __forceinline__ const uint4* row_of(const CombineArgs& a, int64_t t, int k, int pos) {
  if (!EP) return a.y + (size_t)pos * a.nvec;
  const int e = __ldg(a.ids + (size_t)t * a.K + k);
  const int db = __ldg(a.dest_base + e);
  if (db < 0) return nullptr;
  const int64_t row = (int64_t)db + (pos - __ldg(a.offsets + e));
  return a.peer_y[e / a.epr] + (size_t)row * a.nvec;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <int KT, bool EP>
__device__ __forceinline__ void combine_unit(const CombineArgs& a, int64_t t, int v) {
  int pos[KT];
  float w[KT];
  uint4 yv[KT];
#pragma unroll
  for (int k = 0; k < KT; ++k) {
    pos[k] = k < a.K ? __ldg(a.inverse_perm + (size_t)t * a.K + k) : -1;
    w[k] = k < a.K ? __ldg(a.weights + (size_t)t * a.K + k) : 0.0f;
  }
#pragma unroll
  for (int k = 0; k < KT; ++k) {
    if (pos[k] >= 0) {
      const uint4* src = row_of<EP>(a, t, k, pos[k]);
      if (EP && src == nullptr)
        pos[k] = -1;  // no row on the owner: the pair contributes nothing
      else
        yv[k] = __ldcs(src + v);
    }
  }
  float acc[8];
  if (a.shared != nullptr) {
    const uint4 s = __ldcs(a.shared + (size_t)t * a.nvec + v);
    unpack8(s, acc);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  }
#pragma unroll
  for (int k = 0; k < KT; ++k) {
    if (pos[k] >= 0) {
      float f[8];
      unpack8(yv[k], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(w[k], f[j], acc[j]);
    }
  }
  uint4 o;
  o.x = pack_bf16x2(acc[0], acc[1]);
  o.y = pack_bf16x2(acc[2], acc[3]);
  o.z = pack_bf16x2(acc[4], acc[5]);
  o.w = pack_bf16x2(acc[6], acc[7]);
  __stcs(a.out + (size_t)t * a.nvec + v, o);
}

// K > 8: same arithmetic with the loads issued eight at a time.
template <bool EP>
__device__ __forceinline__ void combine_unit_any(const CombineArgs& a, int64_t t, int v) {
  float acc[8];
  if (a.shared != nullptr) {
    const uint4 s = __ldcs(a.shared + (size_t)t * a.nvec + v);
    unpack8(s, acc);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  }
  for (int k0 = 0; k0 < a.K; k0 += 8) {
    int pos[8];
    float w[8];
    uint4 yv[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      pos[k] = k0 + k < a.K ? __ldg(a.inverse_perm + (size_t)t * a.K + k0 + k) : -1;
      w[k] = k0 + k < a.K ? __ldg(a.weights + (size_t)t * a.K + k0 + k) : 0.0f;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (pos[k] >= 0) {
        const uint4* src = row_of<EP>(a, t, k0 + k, pos[k]);
        if (EP && src == nullptr)
          pos[k] = -1;
        else
          yv[k] = __ldcs(src + v);
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (pos[k] >= 0) {
        float f[8];
        unpack8(yv[k], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = fmaf(w[k], f[j], acc[j]);
      }
    }
  }
  uint4 o;
  o.x = pack_bf16x2(acc[0], acc[1]);
  o.y = pack_bf16x2(acc[2], acc[3]);
  o.z = pack_bf16x2(acc[4], acc[5]);
  o.w = pack_bf16x2(acc[6], acc[7]);
  __stcs(a.out + (size_t)t * a.nvec + v, o);
}

template <int KT, bool EP>
__global__ void __launch_bounds__(kCombineThreads) combine_kernel(const CombineArgs a) {
  pdl_sync();
  const int lane = threadIdx.x & 31;
  const int upr = (a.nvec + 31) >> 5;  // units per row
  const int64_t total = a.T * upr;
  const int64_t W = (int64_t)gridDim.x * kCombineWarps;
  for (int64_t u = (int64_t)blockIdx.x * kCombineWarps + (threadIdx.x >> 5); u < total; u += W) {
    const int64_t t = u / upr;
    const int v = (int)(u - t * upr) * 32 + lane;
    if (v >= a.nvec) continue;
    if (KT > 0)
      combine_unit<(KT > 0 ? KT : 1), EP>(a, t, v);
    else
      combine_unit_any<EP>(a, t, v);
  }
}

}  // namespace

int device_sms();

}  // namespace moe_rd

using namespace moe_rd;

namespace moe_rd {
namespace {

template <bool EP>
int launch_combine(CombineArgs& a, int64_t T, int32_t H, int32_t K, void* stream) {
  a.T = T;
  a.nvec = H / 8;
  a.K = K;
  const int64_t units = T * ((a.nvec + 31) / 32);
  const int64_t want = (units + kCombineWarps - 1) / kCombineWarps;
  const int64_t cap = (int64_t)device_sms() * kCombineBlocksPerSm;
  const dim3 grid((unsigned)(want < cap ? want : cap));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (K <= 2)
    e = launch_pdl(combine_kernel<2, EP>, grid, dim3(kCombineThreads), 0, s, a);
  else if (K <= 4)
    e = launch_pdl(combine_kernel<4, EP>, grid, dim3(kCombineThreads), 0, s, a);
  else if (K <= 8)
    e = launch_pdl(combine_kernel<8, EP>, grid, dim3(kCombineThreads), 0, s, a);
  else
    e = launch_pdl(combine_kernel<0, EP>, grid, dim3(kCombineThreads), 0, s, a);
  count_launch();
  return e == cudaSuccess ? MOE_RD_OK : MOE_RD_E_CUDA;
}

// ---------------------------------------------------------------------------
// Residual (accumulating) combine over expert-major rows:
//   out[row_token[p], :] += bf16(row_weight[p] * y[p, :])   for p < *n_rows
// The form the reference uses when most expert outputs were already reduced
// into `out` by a GEMM epilogue and only the rows of the remaining experts are
// left to fold in (raddleft_kernel, kernel.cu:2451-2486): it must add, not
// store, and the number of live rows is a device-side value, so nothing is
// read back.  The product is rounded to bf16 and added by an element-wise bf16
// reduction without return value (kernel.cu:2446-2449); here one 16-byte
// vector reduction (red.global.add.noftz.v4.bf16x2) per lane where the
// reference issues four 4-byte ones.  Adds to one element from different rows
// arrive in no fixed order, each rounding to bf16: results are exact when every
// token receives at most one row and order-dependent in the last bits otherwise
// (as in the reference).  Work units (a row x 32 vectors) are dealt to warps
// grid-stride.
// ---------------------------------------------------------------------------
struct AddRowsArgs {
  const uint4* y;
  const int32_t* row_token;
  const float* row_weight;
  const int32_t* n_rows;  // device value
  uint4* out;
  int64_t max_rows;
  int nvec;
};

__device__ __forceinline__ void red_add_bf16x8(void* p, const uint32_t (&v)[4]) {
  asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v[0]), "r"(v[1]),
               "r"(v[2]), "r"(v[3])
               : "memory");
}

__global__ void __launch_bounds__(kCombineThreads) combine_add_rows_kernel(const AddRowsArgs a) {
  pdl_sync();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kCombineWarps + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kCombineWarps;
  int64_t n = __ldg(a.n_rows);
  n = n < 0 ? 0 : (n > a.max_rows ? a.max_rows : n);
  const int chunks = (a.nvec + 31) / 32;
  for (int64_t u = warp; u < n * chunks; u += nwarps) {
    const int64_t p = u / chunks;
    const int v = (int)(u - p * chunks) * 32 + lane;
    const int t = __ldg(a.row_token + p);
    if (v >= a.nvec || t < 0) continue;
    const float w = __ldg(a.row_weight + p);
    const uint4 yv = __ldcs(a.y + (size_t)p * a.nvec + v);
    const uint32_t in[4] = {yv.x, yv.y, yv.z, yv.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = pack_bf16x2(__fmul_rn(w, __uint_as_float(in[j] << 16)),
                         __fmul_rn(w, __uint_as_float(in[j] & 0xffff0000u)));
    red_add_bf16x8(a.out + (size_t)t * a.nvec + v, o);
  }
}

}  // namespace
}  // namespace moe_rd

extern "C" int moe_rd_combine_add_rows(int32_t H, int64_t max_rows, const void* y, const int32_t* row_token,
                                       const float* row_weight, const int32_t* n_rows, void* out,
                                       void* stream) {
  if (H < 8 || H % 8 != 0 || max_rows < 0 || max_rows > ((int64_t)1 << 31) - 1) return MOE_RD_E_SHAPE;
  if (max_rows == 0) return MOE_RD_OK;
  if (y == nullptr || row_token == nullptr || row_weight == nullptr || n_rows == nullptr || out == nullptr)
    return MOE_RD_E_NULL;
  if ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) & 15) return MOE_RD_E_ALIGN;
  AddRowsArgs a = {};
  a.y = static_cast<const uint4*>(y);
  a.row_token = row_token;
  a.row_weight = row_weight;
  a.n_rows = n_rows;
  a.out = static_cast<uint4*>(out);
  a.max_rows = max_rows;
  a.nvec = H / 8;
  const int64_t units = max_rows * ((a.nvec + 31) / 32);
  const int64_t want = (units + kCombineWarps - 1) / kCombineWarps;
  const int64_t cap = (int64_t)device_sms() * kCombineBlocksPerSm;
  const dim3 grid((unsigned)(want < cap ? want : cap));
  const cudaError_t e =
      launch_pdl(combine_add_rows_kernel, grid, dim3(kCombineThreads), 0, static_cast<cudaStream_t>(stream), a);
  count_launch();
  if (e != cudaSuccess) set_last_cuda_error(e);
  return e == cudaSuccess ? MOE_RD_OK : MOE_RD_E_CUDA;
}

extern "C" int moe_rd_combine(int64_t T, int32_t H, int32_t K, const void* y,
                              const int32_t* inverse_perm, const float* combine_weights,
                              const void* shared, void* out, void* stream) {
  if (T < 0 || H < 8 || H % 8 != 0 || K < 1 || K > kMaxK) return MOE_RD_E_SHAPE;
  if (T == 0) return MOE_RD_OK;
  if (y == nullptr || inverse_perm == nullptr || combine_weights == nullptr || out == nullptr)
    return MOE_RD_E_NULL;
  if ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(shared)) & 15)
    return MOE_RD_E_ALIGN;
  CombineArgs a = {};
  a.y = static_cast<const uint4*>(y);
  a.inverse_perm = inverse_perm;
  a.weights = combine_weights;
  a.shared = static_cast<const uint4*>(shared);
  a.out = static_cast<uint4*>(out);
  return launch_combine<false>(a, T, H, K, stream);
}

extern "C" int moe_rd_ep_combine(int64_t T, int32_t H, int32_t K, int32_t E, int32_t world,
                                 const void* const* peer_y, const int32_t* expert_ids,
                                 const int32_t* inverse_perm, const float* combine_weights,
                                 const int32_t* offsets, const int32_t* dest_base, const void* shared,
                                 void* out, void* stream) {
  if (T < 0 || H < 8 || H % 8 != 0 || K < 1 || K > kMaxK || world < 1 || world > 8 || E < 1 || E > kMaxE ||
      E % world != 0)
    return MOE_RD_E_SHAPE;
  if (T == 0) return MOE_RD_OK;
  if (peer_y == nullptr || expert_ids == nullptr || inverse_perm == nullptr || combine_weights == nullptr ||
      offsets == nullptr || dest_base == nullptr || out == nullptr)
    return MOE_RD_E_NULL;
  CombineArgs a = {};
  for (int d = 0; d < world; ++d) {
    if (peer_y[d] == nullptr) return MOE_RD_E_NULL;
    if (reinterpret_cast<uintptr_t>(peer_y[d]) & 15) return MOE_RD_E_ALIGN;
    a.peer_y[d] = static_cast<const uint4*>(peer_y[d]);
  }
  if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(shared)) & 15) return MOE_RD_E_ALIGN;
  a.inverse_perm = inverse_perm;
  a.weights = combine_weights;
  a.shared = static_cast<const uint4*>(shared);
  a.out = static_cast<uint4*>(out);
  a.ids = expert_ids;
  a.offsets = offsets;
  a.dest_base = dest_base;
  a.epr = E / world;
  return launch_combine<true>(a, T, H, K, stream);
}
