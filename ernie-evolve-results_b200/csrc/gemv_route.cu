// Warp-level GEMV gate for few experts (E <= 32) fused with scoring, top-K and
// the expert histogram: one kernel from hidden states to expert ids, weights
// and per-tile expert counts.
//
// Replaces wsplit_kernel + the router GEMM + topk_kernel of the reference
// (kernel.cu:1786-1824, 4327-4339, 1829-1920) where the expert count is far
// too small for a tensor-core tile.  The gate weight is staged once per block
// in shared memory, in a lane-interleaved order that makes every 16-byte read
// conflict-free; a warp carries 32/EB tokens at a time so each weight read
// feeds several tokens, and the products accumulate with packed fma.rn.f32x2
// (two IEEE fp32 FMAs per instruction).  The summation order per (token,
// expert) is the fixed one of gate_simt.cu, so the logits are bit-identical
// to that kernel's.
#include "route_core.cuh"

namespace moe_rd {
namespace {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kMaxDynSmem = 227 * 1024;

typedef unsigned long long u64;

__device__ __forceinline__ void ffma2(u64& d, u64 a, u64 b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}
__device__ __forceinline__ u64 pack2(float lo, float hi) {
  return (u64)__float_as_uint(lo) | ((u64)__float_as_uint(hi) << 32);
}
__device__ __forceinline__ float lo_of(u64 v) { return __uint_as_float((uint32_t)v); }
__device__ __forceinline__ float hi_of(u64 v) { return __uint_as_float((uint32_t)(v >> 32)); }
// two packed bf16 -> packed pair of fp32
__device__ __forceinline__ u64 bf16x2_to_f32x2(uint32_t v) {
  return (u64)(v << 16) | ((u64)(v & 0xffff0000u) << 32);
}

struct GemvArgs {
  const uint16_t* x;
  const void* w;
  const float* logit_bias;
  float* logits_out;  // optional [T,E]
  int H;
  int w_layout;
};

// Bytes of the staged weight: rows padded to whole 256-row chunks.
__host__ __device__ inline size_t staged_w_bytes(int H, int EB, int wb) {
  return (size_t)((H + 255) / 256) * 256 * EB * wb;
}

template <int EB, int WD>
__global__ void __launch_bounds__(kGemvThreads) gemv_route_kernel(const GemvArgs g,
                                                                 const RouteArgs a) {
  constexpr int WB = WD == MOE_RD_W_BF16 ? 2 : 4;  // bytes per weight
  constexpr int U = EB * WB / 16;                  // 16-byte units per weight row
  constexpr int TPW = 32 / EB;                     // tokens a warp carries at once
  constexpr int NP = EB / 2;                       // accumulator pairs per token

  extern __shared__ __align__(16) unsigned char smem[];
  uint4* s_w = reinterpret_cast<uint4*>(smem);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nchunk = (g.H + 255) >> 8;

  // ---- stage the gate weight: element (h, e) of 16-byte unit u = e*WB/16 goes to
  //      unit index ((c*8 + j)*U + u)*32 + l  with h = 256c + 8l + j.
  if (g.w_layout == MOE_RD_W_LAYOUT_HE && a.E == EB) {
    // A weight row is U whole 16-byte units, contiguous in memory: move units.
    const uint4* w4 = static_cast<const uint4*>(g.w);
    const int total = nchunk * 256 * U;
    const int live = g.H * U;
    for (int idx = tid; idx < total; idx += kGemvThreads) {
      const int h = idx / U, u = idx - h * U;
      const int c = h >> 8, l = (h >> 3) & 31, j = h & 7;
      s_w[((c * 8 + j) * U + u) * 32 + l] = idx < live ? __ldg(w4 + idx) : make_uint4(0, 0, 0, 0);
    }
  } else {
    const int Hp = nchunk * 256;
    const int total = Hp * EB;
    for (int idx = tid; idx < total; idx += kGemvThreads) {
      int h, e;
      if (g.w_layout == MOE_RD_W_LAYOUT_HE) {
        h = idx / EB;
        e = idx - h * EB;
      } else {
        e = idx / Hp;
        h = idx - e * Hp;
      }
      const bool live = h < g.H && e < a.E;
      const size_t src = g.w_layout == MOE_RD_W_LAYOUT_HE ? (size_t)h * a.E + e : (size_t)e * g.H + h;
      const int c = h >> 8, l = (h >> 3) & 31, j = h & 7;
      const int byte = (((c * 8 + j) * U + (e * WB) / 16) * 32 + l) * 16 + (e * WB) % 16;
      if (WD == MOE_RD_W_BF16)
        *reinterpret_cast<uint16_t*>(smem + byte) =
            live ? __ldg(static_cast<const uint16_t*>(g.w) + src) : (uint16_t)0;
      else
        *reinterpret_cast<float*>(smem + byte) =
            live ? __ldg(static_cast<const float*>(g.w) + src) : 0.0f;
    }
  }
  __syncthreads();

  // A unit = TPW consecutive tokens carried by one warp.  Block b owns the
  // contiguous unit range [U*b/B, U*(b+1)/B), so with B a multiple of the SM
  // count every SM gets the same work to within one unit.
  const int64_t units = (a.T + TPW - 1) / TPW;
  const int64_t ulo = units * blockIdx.x / gridDim.x;
  const int64_t uhi = units * (blockIdx.x + 1) / gridDim.x;
  for (int64_t unit = ulo + warp; unit < uhi; unit += kGemvWarps) {
    const int64_t tb = unit * TPW;
    const uint4* xr[TPW];
#pragma unroll
    for (int i = 0; i < TPW; ++i) {
      const int64_t t = min(tb + i, a.T - 1);  // clamp: rows past T are computed, not stored
      xr[i] = reinterpret_cast<const uint4*>(g.x + (size_t)t * g.H);
    }
    u64 acc[TPW][NP];
#pragma unroll
    for (int i = 0; i < TPW; ++i)
#pragma unroll
      for (int q = 0; q < NP; ++q) acc[i][q] = 0ull;

    uint4 xn[TPW];
#pragma unroll
    for (int i = 0; i < TPW; ++i) xn[i] = make_uint4(0, 0, 0, 0);
    if (lane * 8 < g.H) {
#pragma unroll
      for (int i = 0; i < TPW; ++i) xn[i] = __ldg(xr[i] + lane);
    }
    for (int c = 0; c < nchunk; ++c) {
      const int h0 = c * 256 + lane * 8;
      uint4 xv[TPW];
#pragma unroll
      for (int i = 0; i < TPW; ++i) xv[i] = xn[i];
      if (c + 1 < nchunk && h0 + 256 < g.H) {
#pragma unroll
        for (int i = 0; i < TPW; ++i) xn[i] = __ldg(xr[i] + ((h0 + 256) >> 3));
      }
      if (h0 < g.H) {
        const uint4* wrow = s_w + (size_t)c * 8 * U * 32 + lane;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          u64 wp[NP];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint4 v = wrow[(j * U + u) * 32];
            if (WD == MOE_RD_W_BF16) {
              wp[4 * u + 0] = bf16x2_to_f32x2(v.x);
              wp[4 * u + 1] = bf16x2_to_f32x2(v.y);
              wp[4 * u + 2] = bf16x2_to_f32x2(v.z);
              wp[4 * u + 3] = bf16x2_to_f32x2(v.w);
            } else {
              wp[2 * u + 0] = (u64)v.x | ((u64)v.y << 32);
              wp[2 * u + 1] = (u64)v.z | ((u64)v.w << 32);
            }
          }
#pragma unroll
          for (int i = 0; i < TPW; ++i) {
            const uint32_t pk = j < 2 ? xv[i].x : j < 4 ? xv[i].y : j < 6 ? xv[i].z : xv[i].w;
            const float xf = (j & 1) ? bf16_hi(pk) : bf16_lo(pk);
            const u64 xx = pack2(xf, xf);
#pragma unroll
            for (int q = 0; q < NP; ++q) ffma2(acc[i][q], xx, wp[q]);
          }
        }
      }
    }

    // lane sums -> token logits by the fixed tree; lane e keeps expert e, then
    // the warp routes the token at once (E <= 32: one expert per lane)
#pragma unroll
    for (int i = 0; i < TPW; ++i) {
      float mine = 0.0f;
#pragma unroll
      for (int q = 0; q < NP; ++q) {
        float v0 = lo_of(acc[i][q]), v1 = hi_of(acc[i][q]);
#pragma unroll
        for (int o = 16; o; o >>= 1) {
          v0 = __fadd_rn(v0, __shfl_xor_sync(kFull, v0, o));
          v1 = __fadd_rn(v1, __shfl_xor_sync(kFull, v1, o));
        }
        if (lane == 2 * q) mine = v0;
        if (lane == 2 * q + 1) mine = v1;
      }
      const int64_t t = tb + i;
      if (t < a.T) {  // warp-uniform
        if (lane < a.E) {
          if (g.logit_bias != nullptr) mine = __fadd_rn(mine, __ldg(g.logit_bias + lane));
          if (g.logits_out != nullptr) g.logits_out[(size_t)t * a.E + lane] = mine;
        } else {
          mine = 0.0f;
        }
        float z[1] = {mine};
        int mysel;
        float myw;
        route_token<1>(a, z, lane, mysel, myw);
        publish_token(a, t, lane, mysel, myw);
      }
    }
  }
}

size_t gemv_smem_bytes(const moe_rd_params& p, int EB) {
  const int wb = p.w_dtype == MOE_RD_W_BF16 ? 2 : 4;
  return staged_w_bytes(p.H, EB, wb);
}

int pick_eb(int E) { return E <= 8 ? 8 : E <= 16 ? 16 : 32; }

template <int EB, int WD>
cudaError_t launch_t(const moe_rd_params& p, const GemvArgs& g, const RouteArgs& a,
                     cudaStream_t s) {
  const size_t smem = gemv_smem_bytes(p, EB);
  // Two blocks per SM when shared memory allows (registers allow no more).
  const int per_sm = smem * 2 + 2048 <= (size_t)kMaxDynSmem ? 2 : 1;
  const int64_t units = (p.T + 32 / EB - 1) / (32 / EB);
  const int64_t need = (units + kGemvWarps - 1) / kGemvWarps;
  const int64_t cap = (int64_t)device_sms() * per_sm;
  const int grid = (int)(need < cap ? need : cap);
  gemv_route_kernel<EB, WD><<<grid, kGemvThreads, smem, s>>>(g, a);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

bool gemv_eligible(const moe_rd_params& p) {
  if (p.E > 32 || p.T <= 0) return false;
  return gemv_smem_bytes(p, pick_eb(p.E)) <= (size_t)kMaxDynSmem;
}

cudaError_t launch_gemv_route(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                              float* logits_out, int32_t* ids, int32_t* tile_base, cudaStream_t s) {
  GemvArgs g;
  g.x = static_cast<const uint16_t*>(b.x);
  g.w = b.gate_w;
  g.logit_bias = b.logit_bias;
  g.logits_out = logits_out;
  g.H = p.H;
  g.w_layout = p.w_layout;
  RouteArgs a;
  fill_route_args(p, b, plan, nullptr, ids, tile_base, &a);
  const int eb = pick_eb(p.E);
  const bool bf = p.w_dtype == MOE_RD_W_BF16;
  if (eb == 8)
    return bf ? launch_t<8, MOE_RD_W_BF16>(p, g, a, s)
              : launch_t<8, MOE_RD_W_F32>(p, g, a, s);
  if (eb == 16)
    return bf ? launch_t<16, MOE_RD_W_BF16>(p, g, a, s)
              : launch_t<16, MOE_RD_W_F32>(p, g, a, s);
  return bf ? launch_t<32, MOE_RD_W_BF16>(p, g, a, s)
            : launch_t<32, MOE_RD_W_F32>(p, g, a, s);
}

cudaError_t init_gemv_attributes() {
  cudaError_t e;
#define SET(EB, WD)                                                                          \
  e = cudaFuncSetAttribute(gemv_route_kernel<EB, WD>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           kMaxDynSmem);                                                     \
  if (e != cudaSuccess) return e;
  SET(8, MOE_RD_W_BF16) SET(8, MOE_RD_W_F32) SET(16, MOE_RD_W_BF16) SET(16, MOE_RD_W_F32)
  SET(32, MOE_RD_W_BF16) SET(32, MOE_RD_W_F32)
#undef SET
  return cudaSuccess;
}

}  // namespace moe_rd
