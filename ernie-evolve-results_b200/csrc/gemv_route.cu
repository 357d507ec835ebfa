// Warp-level GEMV gate for few experts (E <= 32) fused with scoring, top-K and
// the expert histogram: one kernel from hidden states to expert ids, weights
// and per-tile expert counts.
//
// Replaces wsplit_kernel + the router GEMM + topk_kernel of the reference
// (kernel.cu:1786-1824, 4327-4339, 1829-1920) where the expert count is far
// too small for a tensor-core tile.
//
// A lane owns hidden indices h = 256c + 8l + j.  Two consecutive bf16 of x
// (h even, h odd) sit in one 32-bit word, and turning that word into a packed
// pair of fp32 costs two integer operations.  The gate weight is staged once
// per block in shared memory as fp32 in matching pairs {W[h_even][e],
// W[h_odd][e]}, so one fma.rn.f32x2 advances the even-h chain and the odd-h
// chain of one (token, expert) at once, with no conversion or duplication
// inside the loop.  That is exactly the summation order gate_simt.cu defines
// (32 lanes x 2 chains, then the tree), so the logits are bit-identical to that
// kernel's.  A warp carries 32/EB tokens at a time so that every 16-byte weight
// read feeds several tokens.
#include "route_core.cuh"

namespace moe_rd {
namespace {

constexpr int kMaxDynSmem = 227 * 1024;

// Tokens a warp carries at once and threads per block, per padded expert count:
// 2 * TPW * EB accumulator registers per lane.  (Two tokens per warp with 1024
// threads spills at 64 registers and measured 35 % slower on E = 8.)
template <int EB> struct GemvShape;
#ifndef MOE_RD_GEMV8_TPW      // tokens per warp and threads per block of the E <= 8 kernel
#define MOE_RD_GEMV8_TPW 4
#endif
#ifndef MOE_RD_GEMV8_THREADS
#define MOE_RD_GEMV8_THREADS 512
#endif
template <> struct GemvShape<8> { static constexpr int TPW = MOE_RD_GEMV8_TPW, THREADS = MOE_RD_GEMV8_THREADS; };
template <> struct GemvShape<16> { static constexpr int TPW = 2, THREADS = 512; };
template <> struct GemvShape<32> { static constexpr int TPW = 1, THREADS = 512; };

typedef unsigned long long u64;

__device__ __forceinline__ void ffma2(u64& d, u64 a, u64 b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}
__device__ __forceinline__ float lo_of(u64 v) { return __uint_as_float((uint32_t)v); }
__device__ __forceinline__ float hi_of(u64 v) { return __uint_as_float((uint32_t)(v >> 32)); }
// two packed bf16 (even h in the low half) -> packed pair of fp32.  The halves
// are produced straight into the two registers of the 64-bit pair; building the
// pair with 64-bit integer shifts and ors costs extra moves.
__device__ __forceinline__ u64 bf16x2_to_f32x2(uint32_t v) {
  u64 r;
  asm("{\n\t.reg .b32 lo, hi;\n\t"
      "shl.b32 lo, %1, 16;\n\t"
      "and.b32 hi, %1, 0xffff0000;\n\t"
      "mov.b64 %0, {lo, hi};\n\t}"
      : "=l"(r)
      : "r"(v));
  return r;
}

// 16-byte load of x with an L2 evict-last policy: the row scatter reads x again right after this
// kernel, and what is still in L2 then does not come from HBM a second time.
__device__ __forceinline__ uint4 ld_x_keep(const uint4* p, u64 policy) {
  uint4 v;
  asm volatile("ld.global.nc.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(policy));
  return v;
}
__device__ __forceinline__ u64 policy_evict_last() {
  u64 p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

struct GemvArgs {
  const uint16_t* x;
  const void* w;
  const float* logit_bias;
  float* logits_out;  // optional [T,E]
  int H;
  int w_layout;
  // the scans of the counts, done by the last block to finish
  int32_t* ticket;       // zeroed before the kernel
  int32_t* offsets;      // [E+1]
  int32_t* user_counts;  // [E] or null
  int64_t capacity;
};

// Bytes of the staged fp32 weight: rows padded to whole 256-row chunks.
__host__ __device__ inline size_t staged_w_bytes(int H, int EB) {
  return (size_t)((H + 255) / 256) * 256 * EB * 4;
}

// Shared-memory float index of W[h][e]: 16-byte unit (c, m, e/2) holds, for lane
// l, {W[he][e0], W[ho][e0], W[he][e0+1], W[ho][e0+1]} with he = 256c + 8l + 2m.
template <int EB>
__device__ __forceinline__ int staged_index(int h, int e) {
  const int c = h >> 8, l = (h >> 3) & 31, m = (h & 7) >> 1, p = h & 1;
  return ((((c * 4 + m) * (EB / 2) + (e >> 1)) * 32 + l) << 2) + ((e & 1) << 1) + p;
}

template <int EB, int WD>
__global__ void __launch_bounds__(GemvShape<EB>::THREADS, 1)
gemv_route_kernel(const GemvArgs g, const RouteArgs a) {
  constexpr int TPW = GemvShape<EB>::TPW;
  constexpr int kGemvThreads = GemvShape<EB>::THREADS;
  constexpr int kGemvWarps = kGemvThreads / 32;
  pdl_sync();
  extern __shared__ __align__(16) unsigned char smem[];
  float* s_wf = reinterpret_cast<float*>(smem);
  int* s_cnt = reinterpret_cast<int*>(smem + staged_w_bytes(g.H, EB));  // [32] block histogram, [32] = last-block flag
  if (threadIdx.x < 32) s_cnt[threadIdx.x] = 0;
  // read back as two 64-bit halves: each half is already a {W[he], W[ho]} pair
  const ulonglong2* s_w = reinterpret_cast<const ulonglong2*>(smem);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nchunk = (g.H + 255) >> 8;
  const int Hp = nchunk * 256;

  // ---- stage the gate weight (converted to fp32, zero padded) ----
  if (g.w_layout == MOE_RD_W_LAYOUT_HE && a.E == EB && WD == MOE_RD_W_BF16) {
    // a weight row is EB bf16 = EB/8 whole 16-byte vectors
    const uint4* w4 = static_cast<const uint4*>(g.w);
    constexpr int VPR = EB / 8;
    for (int idx = tid; idx < Hp * VPR; idx += kGemvThreads) {
      const int h = idx / VPR, q = idx - h * VPR;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (h < g.H) v = __ldg(w4 + idx);
      float f[8];
      unpack8(v, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) s_wf[staged_index<EB>(h, q * 8 + i)] = f[i];
    }
  } else if (g.w_layout == MOE_RD_W_LAYOUT_HE && a.E == EB && WD == MOE_RD_W_F32) {
    const float4* w4 = static_cast<const float4*>(g.w);
    constexpr int VPR = EB / 4;
    for (int idx = tid; idx < Hp * VPR; idx += kGemvThreads) {
      const int h = idx / VPR, q = idx - h * VPR;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (h < g.H) v = __ldg(w4 + idx);
      s_wf[staged_index<EB>(h, q * 4 + 0)] = v.x;
      s_wf[staged_index<EB>(h, q * 4 + 1)] = v.y;
      s_wf[staged_index<EB>(h, q * 4 + 2)] = v.z;
      s_wf[staged_index<EB>(h, q * 4 + 3)] = v.w;
    }
  } else {
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
      float v = 0.0f;
      if (h < g.H && e < a.E) {
        const size_t src =
            g.w_layout == MOE_RD_W_LAYOUT_HE ? (size_t)h * a.E + e : (size_t)e * g.H + h;
        v = WD == MOE_RD_W_BF16
                ? __uint_as_float((uint32_t)__ldg(static_cast<const uint16_t*>(g.w) + src) << 16)
                : __ldg(static_cast<const float*>(g.w) + src);
      }
      s_wf[staged_index<EB>(h, e)] = v;
    }
  }
  __syncthreads();

  // A unit = TPW consecutive tokens carried by one warp.  Block b owns the
  // contiguous unit range [U*b/B, U*(b+1)/B), so with B = the SM count every SM
  // gets the same work to within one unit.
  const u64 keep_x = policy_evict_last();
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
    u64 acc[TPW][EB];  // low half: even-h chain, high half: odd-h chain
#pragma unroll
    for (int i = 0; i < TPW; ++i)
#pragma unroll
      for (int e = 0; e < EB; ++e) acc[i][e] = 0ull;

    uint4 xn[TPW];
#pragma unroll
    for (int i = 0; i < TPW; ++i) xn[i] = make_uint4(0, 0, 0, 0);
    if (lane * 8 < g.H) {
#pragma unroll
      for (int i = 0; i < TPW; ++i) xn[i] = ld_x_keep(xr[i] + lane, keep_x);
    }
    for (int c = 0; c < nchunk; ++c) {
      const int h0 = c * 256 + lane * 8;
      uint4 xv[TPW];
#pragma unroll
      for (int i = 0; i < TPW; ++i) xv[i] = xn[i];
      if (c + 1 < nchunk && h0 + 256 < g.H) {
#pragma unroll
        for (int i = 0; i < TPW; ++i) xn[i] = ld_x_keep(xr[i] + ((h0 + 256) >> 3), keep_x);
      }
      if (h0 < g.H) {
        const ulonglong2* wc = s_w + (size_t)c * 4 * (EB / 2) * 32 + lane;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          u64 xx[TPW];
#pragma unroll
          for (int i = 0; i < TPW; ++i) {
            const uint32_t pk = m == 0 ? xv[i].x : m == 1 ? xv[i].y : m == 2 ? xv[i].z : xv[i].w;
            xx[i] = bf16x2_to_f32x2(pk);
          }
#pragma unroll
          for (int e2 = 0; e2 < EB / 2; ++e2) {
            const ulonglong2 v = wc[(m * (EB / 2) + e2) * 32];
#pragma unroll
            for (int i = 0; i < TPW; ++i) {
              ffma2(acc[i][2 * e2], xx[i], v.x);
              ffma2(acc[i][2 * e2 + 1], xx[i], v.y);
            }
          }
        }
      }
    }

    // lane value = even chain + odd chain; lanes are summed by the fixed tree
    if (TPW > 1 && a.n_groups <= 1) {
      // all TPW tokens of the warp are routed at once: token i in lanes i*W..i*W+W-1
      constexpr int W = 32 / TPW;
      float zp = 0.0f;
#pragma unroll
      for (int i = 0; i < TPW; ++i) {
#pragma unroll
        for (int e = 0; e < EB; ++e) {
          float v = __fadd_rn(lo_of(acc[i][e]), hi_of(acc[i][e]));
#pragma unroll
          for (int o = 16; o; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(kFull, v, o));
          if (lane == i * W + e) zp = v;
        }
      }
      const int e = lane & (W - 1);
      const int64_t t = tb + lane / W;
      const bool live = t < a.T;
      if (live && e < a.E) {
        if (g.logit_bias != nullptr) zp = __fadd_rn(zp, __ldg(g.logit_bias + e));
        if (g.logits_out != nullptr) g.logits_out[(size_t)t * a.E + e] = zp;
      }
      int mysel;
      float myw;
      route_token_packed<W>(a, zp, lane, mysel, myw);
      if (live) publish_token(a, t, e, mysel, myw, s_cnt);
    } else {
      // lane e keeps expert e, and the warp routes one token at a time
#pragma unroll
      for (int i = 0; i < TPW; ++i) {
        float mine = 0.0f;
#pragma unroll
        for (int e = 0; e < EB; ++e) {
          float v = __fadd_rn(lo_of(acc[i][e]), hi_of(acc[i][e]));
#pragma unroll
          for (int o = 16; o; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(kFull, v, o));
          if (lane == e) mine = v;
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
          route_token<1, false>(a, z, lane, nullptr, mysel, myw);
          publish_token(a, t, lane, mysel, myw, s_cnt);
        }
      }
    }
  }
  __syncthreads();
  flush_counts(a, s_cnt, kGemvThreads);

  // ---- The last block to finish turns the counts into bases and offsets (with
  // at most 32 experts this is a microsecond of work; a kernel of its own costs
  // several).  Follows the scan part of offsets_kernel of the reference
  // (kernel.cu:2074-2086).
  int* s_last = s_cnt + 32;  // (the kernel's whole shared-memory budget is dynamic)
  __threadfence();
  __syncthreads();
  if (tid == 0) *s_last = atomicAdd(g.ticket, 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!*s_last) return;
  __threadfence();
  for (int e = warp; e < a.E; e += kGemvWarps) {
    // exclusive scan, in place, of the expert's per-tile counts: a warp per expert,
    // eight chunks of 32 tiles loaded at a time
    volatile int32_t* col = a.tile_counts + (size_t)e * a.ntiles;
    int carry = 0;
    for (int base = 0; base < a.ntiles; base += 256) {
      int v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = base + 32 * j + lane;
        v[j] = i < a.ntiles ? col[i] : 0;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        int incl = v[j];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int n = __shfl_up_sync(kFull, incl, o);
          if (lane >= o) incl += n;
        }
        const int i = base + 32 * j + lane;
        if (i < a.ntiles) col[i] = carry + incl - v[j];
        carry += __shfl_sync(kFull, incl, 31);
      }
    }
  }
  if (warp == 0) {
    // offsets[e] = rows kept by the experts before e (E <= 32: one lane each)
    int c = lane < a.E ? reinterpret_cast<volatile int32_t*>(a.counts)[lane] : 0;
    if (lane < a.E && g.user_counts != nullptr) g.user_counts[lane] = c;
    if (g.capacity > 0 && (int64_t)c > g.capacity) c = (int)g.capacity;
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(kFull, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane < a.E) g.offsets[lane] = incl - c;
    if (lane == a.E - 1) g.offsets[a.E] = incl;
  }
}

int pick_eb(int E) { return E <= 8 ? 8 : E <= 16 ? 16 : 32; }

template <int EB, int WD>
cudaError_t launch_t(const moe_rd_params& p, const GemvArgs& g, const RouteArgs& a,
                     cudaStream_t s) {
  constexpr int TPW = GemvShape<EB>::TPW;
  constexpr int kGemvThreads = GemvShape<EB>::THREADS;
  constexpr int kGemvWarps = kGemvThreads / 32;
  const size_t smem = staged_w_bytes(p.H, EB) + 256;
  const int64_t units = (p.T + TPW - 1) / TPW;
  const int64_t need = (units + kGemvWarps - 1) / kGemvWarps;
  const int64_t cap = device_sms();  // one block per SM (it fills the register file)
  const int grid = (int)(need < cap ? need : cap);
  const cudaError_t e =
      launch_pdl(gemv_route_kernel<EB, WD>, dim3((unsigned)grid), dim3(kGemvThreads), smem, s, g, a);
  count_launch();
  return e;
}

}  // namespace

bool gemv_eligible(const moe_rd_params& p) {
  if (p.E > 32 || p.T <= 0) return false;
  return staged_w_bytes(p.H, pick_eb(p.E)) + 256 <= (size_t)kMaxDynSmem;
}

cudaError_t launch_gemv_route(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                              float* logits_out, int32_t* ids, int32_t* tile_base, int32_t* counts,
                              int32_t* ticket, cudaStream_t s) {
  GemvArgs g;
  g.ticket = ticket;
  g.offsets = b.offsets;
  g.user_counts = b.counts;
  g.capacity = p.capacity;
  g.x = static_cast<const uint16_t*>(b.x);
  g.w = b.gate_w;
  g.logit_bias = b.logit_bias;
  g.logits_out = logits_out;
  g.H = p.H;
  g.w_layout = p.w_layout;
  RouteArgs a;
  fill_route_args(p, b, plan, nullptr, ids, tile_base, counts, &a);
  const int eb = pick_eb(p.E);
  const bool bf = p.w_dtype == MOE_RD_W_BF16;
  if (eb == 8)
    return bf ? launch_t<8, MOE_RD_W_BF16>(p, g, a, s) : launch_t<8, MOE_RD_W_F32>(p, g, a, s);
  if (eb == 16)
    return bf ? launch_t<16, MOE_RD_W_BF16>(p, g, a, s) : launch_t<16, MOE_RD_W_F32>(p, g, a, s);
  return bf ? launch_t<32, MOE_RD_W_BF16>(p, g, a, s) : launch_t<32, MOE_RD_W_F32>(p, g, a, s);
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
