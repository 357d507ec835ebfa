// Gate logits z[t,e] = sum_h x[t,h] * W[h,e] (+ logit_bias[e]) in a FIXED fp32
// order, one warp per token ("warp-level GEMV").
//
// Replaces wsplit_kernel + the library router GEMM of the reference
// (kernel.cu:1786-1824, 4327-4339) where the number of experts is small, and
// serves every E as the order-defining product: lane l keeps two chains, one
// for even and one for odd hidden indices; chain (l, p) accumulates by fused
// multiply-add, from 0, the elements h = 256*c + 8*l + 2*m + p (c = 0,1,..;
// m = 0..3, increasing); the lane's value is chain(l,0) + chain(l,1), and the 32
// lane values are combined by the tree v[l] += v[l^off], off = 16,8,4,2,1.
// (Two chains per lane are what the packed fma.rn.f32x2 of the fused GEMV
// kernel computes from a bf16 pair.)  fp32 gate weights are read directly, so
// no hi/lo bf16 split (kernel.cu:1816-1822) is needed on this path.
#include "common.cuh"

namespace moe_rd {
namespace {

// One row of W (EB consecutive experts of hidden index h), [H,E] layout.
template <int EB, int WD, bool VEC>
__device__ __forceinline__ void load_w_row(const void* __restrict__ w, int h, int e0, int E,
                                           float wv[EB]) {
  if (VEC) {
    // E % 8 == 0 and e0 % 8 == 0: the EB values are 16-byte aligned groups.
    if (WD == MOE_RD_W_BF16) {
      const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(w) +
                                                      (size_t)h * E + e0);
#pragma unroll
      for (int q = 0; q < EB / 8; ++q) {
        const uint4 v = __ldg(p + q);
        unpack8(v, wv + 8 * q);
      }
    } else {
      const float4* p =
          reinterpret_cast<const float4*>(static_cast<const float*>(w) + (size_t)h * E + e0);
#pragma unroll
      for (int q = 0; q < EB / 4; ++q) {
        const float4 v = __ldg(p + q);
        wv[4 * q + 0] = v.x; wv[4 * q + 1] = v.y; wv[4 * q + 2] = v.z; wv[4 * q + 3] = v.w;
      }
    }
  } else {
#pragma unroll
    for (int e = 0; e < EB; ++e) {
      float v = 0.0f;
      if (e0 + e < E) {
        const size_t i = (size_t)h * E + e0 + e;
        v = WD == MOE_RD_W_BF16
                ? __uint_as_float((uint32_t)__ldg(static_cast<const uint16_t*>(w) + i) << 16)
                : __ldg(static_cast<const float*>(w) + i);
      }
      wv[e] = v;
    }
  }
}

// Eight consecutive hidden indices of expert e, [E,H] layout (H % 8 == 0).
template <int WD>
__device__ __forceinline__ void load_w_col8(const void* __restrict__ w, int e, int h0, int H,
                                            float wv[8]) {
  if (WD == MOE_RD_W_BF16) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(w) +
                                                         (size_t)e * H + h0));
    unpack8(v, wv);
  } else {
    const float4* p =
        reinterpret_cast<const float4*>(static_cast<const float*>(w) + (size_t)e * H + h0);
    const float4 a = __ldg(p), b = __ldg(p + 1);
    wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w;
    wv[4] = b.x; wv[5] = b.y; wv[6] = b.z; wv[7] = b.w;
  }
}

constexpr int kWarps = 8;

template <int EB, int WD, int WL, bool VEC>
__global__ void __launch_bounds__(kWarps * 32)
gate_simt_kernel(const uint16_t* __restrict__ x, const void* __restrict__ w,
                 const float* __restrict__ logit_bias, float* __restrict__ logits, int64_t T,
                 int H, int E) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int e0 = blockIdx.y * EB;
  if (t >= T) return;  // warp-uniform; the kernel has no block-level barrier

  float acc[EB], acc1[EB];  // even-h chain, odd-h chain
#pragma unroll
  for (int e = 0; e < EB; ++e) acc[e] = acc1[e] = 0.0f;

  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)t * H);
  const int nchunk = (H + 255) >> 8;
  uint4 xn = make_uint4(0, 0, 0, 0);
  if (lane * 8 < H) xn = __ldg(xr + lane);
  for (int c = 0; c < nchunk; ++c) {
    const int h0 = c * 256 + lane * 8;
    const uint4 xv = xn;
    const int hn = h0 + 256;
    if (c + 1 < nchunk && hn < H) xn = __ldg(xr + (hn >> 3));
    if (h0 < H) {
      float xf[8];
      unpack8(xv, xf);
      if (WL == MOE_RD_W_LAYOUT_HE) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float wv[EB];
          load_w_row<EB, WD, VEC>(w, h0 + j, e0, E, wv);
#pragma unroll
          for (int e = 0; e < EB; ++e) {
            if (j & 1)
              acc1[e] = fmaf(xf[j], wv[e], acc1[e]);
            else
              acc[e] = fmaf(xf[j], wv[e], acc[e]);
          }
        }
      } else {
#pragma unroll
        for (int e = 0; e < EB; ++e) {
          if (e0 + e < E) {
            float wv[8];
            load_w_col8<WD>(w, e0 + e, h0, H, wv);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (j & 1)
                acc1[e] = fmaf(xf[j], wv[j], acc1[e]);
              else
                acc[e] = fmaf(xf[j], wv[j], acc[e]);
            }
          }
        }
      }
    }
  }

#pragma unroll
  for (int e = 0; e < EB; ++e) acc[e] = __fadd_rn(acc[e], acc1[e]);
#pragma unroll
  for (int o = 16; o; o >>= 1) {
#pragma unroll
    for (int e = 0; e < EB; ++e) acc[e] = __fadd_rn(acc[e], __shfl_xor_sync(kFull, acc[e], o));
  }

  float v = 0.0f;
#pragma unroll
  for (int e = 0; e < EB; ++e)
    if (lane == e) v = acc[e];
  if (lane < EB && e0 + lane < E) {
    if (logit_bias != nullptr) v = __fadd_rn(v, __ldg(logit_bias + e0 + lane));
    logits[(size_t)t * E + e0 + lane] = v;
  }
}

template <int EB, int WD, int WL, bool VEC>
cudaError_t launch_one(const moe_rd_params& p, const moe_rd_buffers& b, float* logits,
                       cudaStream_t s) {
  const dim3 grid((unsigned)((p.T + kWarps - 1) / kWarps), (unsigned)((p.E + EB - 1) / EB));
  gate_simt_kernel<EB, WD, WL, VEC><<<grid, kWarps * 32, 0, s>>>(
      static_cast<const uint16_t*>(b.x), b.gate_w, b.logit_bias, logits, p.T, p.H, p.E);
  count_launch();
  return cudaGetLastError();
}

template <int WD, int WL>
cudaError_t launch_wd_wl(const moe_rd_params& p, const moe_rd_buffers& b, float* logits,
                         cudaStream_t s) {
  // [H,E] rows vectorise when groups of 8 experts are 16-byte aligned; [E,H]
  // always vectorises along h.  EB = 8 experts per block keeps 8 accumulators
  // per lane; x is re-read (from L2) once per group of 8 experts.
  const bool vec = WL == MOE_RD_W_LAYOUT_HE && p.E % 8 == 0 &&
                   (reinterpret_cast<uintptr_t>(b.gate_w) & 15) == 0;
  if (WL == MOE_RD_W_LAYOUT_HE && vec) return launch_one<8, WD, WL, true>(p, b, logits, s);
  return launch_one<8, WD, WL, false>(p, b, logits, s);
}

}  // namespace

cudaError_t launch_gate_simt(const moe_rd_params& p, const moe_rd_buffers& b, float* logits,
                             cudaStream_t s) {
  if (p.T == 0) return cudaSuccess;
  if (p.w_dtype == MOE_RD_W_BF16) {
    return p.w_layout == MOE_RD_W_LAYOUT_HE
               ? launch_wd_wl<MOE_RD_W_BF16, MOE_RD_W_LAYOUT_HE>(p, b, logits, s)
               : launch_wd_wl<MOE_RD_W_BF16, MOE_RD_W_LAYOUT_EH>(p, b, logits, s);
  }
  return p.w_layout == MOE_RD_W_LAYOUT_HE
             ? launch_wd_wl<MOE_RD_W_F32, MOE_RD_W_LAYOUT_HE>(p, b, logits, s)
             : launch_wd_wl<MOE_RD_W_F32, MOE_RD_W_LAYOUT_EH>(p, b, logits, s);
}

}  // namespace moe_rd
