// Destination rows, inverse permutation, drop mask, and the row scatter with
// optional fused fp8-e4m3 quantisation.
//
// Replaces dispatch_body + gather_body of the reference (kernel.cu:2109-2238).
// The reference gathers expert-major: it walks destination rows and reads
// x[tok[row]] once per (token, expert) pair, i.e. K reads of every token row.
// This kernel scatters token-major: a token row is read ONCE, quantised once
// if asked, and written to its K destination rows with 16-byte stores.
//
// A pair's destination is  offsets[e] + tile_base[e][tile] + rank_in_tile ,
// all integers produced by the route and scan kernels, so the slot order is
// the stable (token, slot) order.  Pairs whose rank inside the expert reaches
// the capacity get inverse_perm = -1 and are not written.
//
// fp8 rows follow the reference's per-row int8 quantiser convention
// (xquant_body, kernel.cu:2573-2591) applied per 128 elements with QMAX = 448:
// scale = max(amax, 1e-30) * (1/448), inv = 1/scale, q = rne_satfinite(x*inv).
#include <cuda_fp8.h>

#include "common.cuh"

namespace moe_rd {
namespace {

constexpr int kScatterThreads = 256;
constexpr int kGroup = 8;  // tokens per block iteration = warps per block

struct ScatterArgs {
  const uint16_t* x;
  const int32_t* ids;
  const int32_t* pair_rank;
  const int32_t* tile_base;  // [E][ntiles], scanned
  const int32_t* offsets;    // [E+1]
  int32_t* inverse_perm;
  uint8_t* drop_mask;
  void* rows;
  float* scales;
  int32_t* status;
  int64_t T, capacity, out_rows;
  int H, E, K, ntiles;
};

__device__ __forceinline__ uint32_t abs_bf16x2(uint32_t v) { return v & 0x7fff7fffu; }

__device__ __forceinline__ float amax8(const uint4& v) {
  // |bf16| -> fp32 is exact, so the maximum is order-independent.
  float m = fmaxf(bf16_lo(abs_bf16x2(v.x)), bf16_hi(abs_bf16x2(v.x)));
  m = fmaxf(m, fmaxf(bf16_lo(abs_bf16x2(v.y)), bf16_hi(abs_bf16x2(v.y))));
  m = fmaxf(m, fmaxf(bf16_lo(abs_bf16x2(v.z)), bf16_hi(abs_bf16x2(v.z))));
  m = fmaxf(m, fmaxf(bf16_lo(abs_bf16x2(v.w)), bf16_hi(abs_bf16x2(v.w))));
  return m;
}

__device__ __forceinline__ uint32_t quant4(uint32_t a, uint32_t b, float inv) {
  // two packed bf16 pairs -> four e4m3 bytes, element order preserved
  const float2 f0 = make_float2(__fmul_rn(bf16_lo(a), inv), __fmul_rn(bf16_hi(a), inv));
  const float2 f1 = make_float2(__fmul_rn(bf16_lo(b), inv), __fmul_rn(bf16_hi(b), inv));
  const uint32_t q0 = __nv_cvt_float2_to_fp8x2(f0, __NV_SATFINITE, __NV_E4M3);
  const uint32_t q1 = __nv_cvt_float2_to_fp8x2(f1, __NV_SATFINITE, __NV_E4M3);
  return q0 | (q1 << 16);
}

template <int FMT>
__global__ void __launch_bounds__(kScatterThreads) scatter_kernel(const ScatterArgs a) {
  extern __shared__ int s_pos[];  // [kGroup*K]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t ngroups = (a.T + kGroup - 1) / kGroup;

  for (int64_t g = blockIdx.x; g < ngroups; g += gridDim.x) {
    const int64_t t0 = g * kGroup;
    const int ng = (int)min((int64_t)kGroup, a.T - t0);
    __syncthreads();  // every warp is done reading s_pos of the previous group
    for (int p = tid; p < ng * a.K; p += kScatterThreads) {
      const size_t s = (size_t)t0 * a.K + p;
      const int64_t t = t0 + p / a.K;
      const int e = a.ids[s];
      int pos = -1;
      bool dropped = false;
      if (e < 0 || e >= a.E) {
        report(a.status, 1, e, (int)s);
      } else {
        const int64_t r =
            (int64_t)a.tile_base[(size_t)e * a.ntiles + (int)(t / kTile)] + a.pair_rank[s];
        dropped = a.capacity > 0 && r >= a.capacity;
        if (!dropped) {
          const int64_t q = (int64_t)a.offsets[e] + r;
          if (q < 0 || q >= a.out_rows)
            report(a.status, 2, (int)q, (int)s);
          else
            pos = (int)q;
        }
      }
      a.inverse_perm[s] = pos;
      if (a.drop_mask != nullptr) a.drop_mask[s] = dropped ? 1 : 0;
      s_pos[p] = pos;
    }
    __syncthreads();

    // One warp per token row of the group.
    if (warp < ng) {
      const int64_t t = t0 + warp;
      const int* pos = s_pos + warp * a.K;
      if (FMT == MOE_RD_ROWS_BF16) {
        const int nvec = a.H >> 3;
        const uint4* src = reinterpret_cast<const uint4*>(a.x) + (size_t)t * nvec;
        uint4* dst = reinterpret_cast<uint4*>(a.rows);
        for (int v0 = 0; v0 < nvec; v0 += 128) {
          uint4 val[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int v = v0 + u * 32 + lane;
            if (v < nvec) val[u] = __ldg(src + v);
          }
          for (int k = 0; k < a.K; ++k) {
            const int q = pos[k];
            if (q < 0) continue;
            uint4* d = dst + (size_t)q * nvec;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int v = v0 + u * 32 + lane;
              if (v < nvec) __stcs(d + v, val[u]);
            }
          }
        }
      } else {
        // 16 elements per lane: 8 lanes share one 128-element scale block.
        const int n16 = a.H >> 4;
        const int nb = a.H >> 7;
        const uint4* src = reinterpret_cast<const uint4*>(a.x) + (size_t)t * (n16 * 2);
        uint4* dst = reinterpret_cast<uint4*>(a.rows);
        for (int v0 = 0; v0 < n16; v0 += 32) {
          const int v = v0 + lane;
          const bool act = v < n16;
          uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
          if (act) {
            lo = __ldg(src + 2 * v);
            hi = __ldg(src + 2 * v + 1);
          }
          float am = fmaxf(amax8(lo), amax8(hi));
          am = fmaxf(am, __shfl_xor_sync(kFull, am, 4));
          am = fmaxf(am, __shfl_xor_sync(kFull, am, 2));
          am = fmaxf(am, __shfl_xor_sync(kFull, am, 1));
          const float scale = __fmul_rn(fmaxf(am, 1e-30f), 1.0f / 448.0f);
          const float inv = __fdiv_rn(1.0f, scale);
          uint4 q;
          q.x = quant4(lo.x, lo.y, inv);
          q.y = quant4(lo.z, lo.w, inv);
          q.z = quant4(hi.x, hi.y, inv);
          q.w = quant4(hi.z, hi.w, inv);
          if (act) {
            for (int k = 0; k < a.K; ++k) {
              const int r = pos[k];
              if (r < 0) continue;
              __stcs(dst + (size_t)r * n16 + v, q);
              if ((lane & 7) == 0) a.scales[(size_t)r * nb + (v >> 3)] = scale;
            }
          }
        }
      }
    }
  }
}

}  // namespace

cudaError_t launch_scatter(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                           const int32_t* ids, const int32_t* pair_rank, const int32_t* tile_base,
                           int32_t* status, cudaStream_t s) {
  if (p.T == 0) return cudaSuccess;
  ScatterArgs a;
  a.x = static_cast<const uint16_t*>(b.x);
  a.ids = ids;
  a.pair_rank = pair_rank;
  a.tile_base = tile_base;
  a.offsets = b.offsets;
  a.inverse_perm = b.inverse_perm;
  a.drop_mask = b.drop_mask;
  a.rows = b.permuted;
  a.scales = b.scales;
  a.status = status;
  a.T = p.T;
  a.capacity = p.capacity;
  a.out_rows = p.out_rows;
  a.H = p.H;
  a.E = p.E;
  a.K = p.K;
  a.ntiles = plan.ntiles;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t ngroups = (p.T + kGroup - 1) / kGroup;
  const int64_t cap = (int64_t)sms * 16;
  const unsigned grid = (unsigned)(ngroups < cap ? ngroups : cap);
  const size_t smem = (size_t)kGroup * p.K * sizeof(int);
  if (p.rows_format == MOE_RD_ROWS_BF16)
    scatter_kernel<MOE_RD_ROWS_BF16><<<grid, kScatterThreads, smem, s>>>(a);
  else
    scatter_kernel<MOE_RD_ROWS_FP8_E4M3_B128><<<grid, kScatterThreads, smem, s>>>(a);
  count_launch();
  return cudaGetLastError();
}

}  // namespace moe_rd
