// Scoring, group-limited top-K, combine weights, and the deterministic
// per-tile expert histogram with in-tile stable ranks.
//
// Replaces topk_kernel of the reference (kernel.cu:1829-1920): one warp per
// token, experts strided over lanes (expert e lives in lane e%32, register
// e/32), softmax as max / exp / sum / reciprocal-multiply (1857-1866), bias
// added to the score to form the selection key (1865-1866), K rounds of warp
// arg-max with lowest-index tie-break (1872-1901), weights u / max(sum u,
// norm_min) (1909).  Added here: sigmoid scoring, selection-only bias,
// group-limited selection, a final scale.
//
// The reference ranks a pair inside its expert with shared and global atomics
// (dispatch_body, kernel.cu:2155-2158), which makes slot order depend on
// scheduling.  Here a block owns a tile of kTile consecutive tokens, counts
// every 32 consecutive pairs with __match_any_sync, and prefix-sums those
// counts in pair order, so the rank of a pair is a pure function of the ids.
#include "common.cuh"

namespace moe_rd {
namespace {

constexpr int kRouteThreads = 512;

struct RouteArgs {
  const float* logits;
  const float* select_bias;
  int32_t* ids;
  float* weights;
  int32_t* pair_rank;
  int32_t* tile_counts;  // [E][ntiles]
  int32_t* ticket;
  int64_t T;
  int E, K, ntiles;
  int n_groups, topk_groups, group_topk;
  int score_fn, weight_from_key, renorm;
  float routed_scale, norm_min;
};

template <int EPL>
__device__ __forceinline__ void route_token(const RouteArgs& a, const float* __restrict__ zr,
                                            int lane, int& mysel, float& myw) {
  const float ninf = __int_as_float(0xff800000);
  float sc[EPL], key[EPL];
  {
    float z[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int e = lane + 32 * i;
      z[i] = e < a.E ? __ldg(zr + e) : ninf;
    }
    if (a.score_fn == MOE_RD_SCORE_SOFTMAX) {
      float m = z[0];
#pragma unroll
      for (int i = 1; i < EPL; ++i) m = fmaxf(m, z[i]);
      m = warp_max(m);
      float part = 0.0f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const int e = lane + 32 * i;
        const float p = e < a.E ? exp_ieee(__fsub_rn(z[i], m)) : 0.0f;
        sc[i] = p;
        part = __fadd_rn(part, p);
      }
      const float s = warp_tree_sum(part);
      const float rs = __fdiv_rn(1.0f, s);
#pragma unroll
      for (int i = 0; i < EPL; ++i) sc[i] = __fmul_rn(sc[i], rs);
    } else {
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const int e = lane + 32 * i;
        sc[i] = e < a.E ? __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_ieee(-z[i]))) : 0.0f;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int e = lane + 32 * i;
    if (e < a.E)
      key[i] = a.select_bias != nullptr ? __fadd_rn(sc[i], __ldg(a.select_bias + e)) : sc[i];
    else
      key[i] = ninf;
  }

  if (a.n_groups > 1) {
    const int gs = a.E / a.n_groups;
    float mygs = ninf;  // lane g keeps the score of group g
    for (int g = 0; g < a.n_groups; ++g) {
      const int lo = g * gs, hi = lo + gs;
      unsigned gtaken = 0;
      float sum = 0.0f;
      for (int r = 0; r < a.group_topk; ++r) {
        float bv = ninf;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          const int e = lane + 32 * i;
          if (e >= lo && e < hi && !((gtaken >> i) & 1u) && key[i] > bv) {
            bv = key[i];
            bi = e;
          }
        }
        warp_argmax(bv, bi);
        if (bi < a.E && (bi & 31) == lane) gtaken |= 1u << (bi >> 5);
        sum = r == 0 ? bv : __fadd_rn(sum, bv);
      }
      if (lane == g) mygs = sum;
    }
    int rank = 0;
    for (int o = 0; o < a.n_groups; ++o) {
      const float og = __shfl_sync(kFull, mygs, o);
      if (og > mygs || (og == mygs && o < lane)) ++rank;
    }
    const unsigned keep = __ballot_sync(kFull, lane < a.n_groups && rank < a.topk_groups);
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int e = lane + 32 * i;
      if (e < a.E && !((keep >> (e / gs)) & 1u)) key[i] = ninf;
    }
  }

  unsigned taken = 0;
  float tot = 0.0f, myu = 0.0f;
  mysel = 0;
  for (int k = 0; k < a.K; ++k) {
    float bv = ninf;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      if (!((taken >> i) & 1u) && key[i] > bv) {
        bv = key[i];
        bi = lane + 32 * i;
      }
    }
    warp_argmax(bv, bi);
    bi = min(max(bi, 0), a.E - 1);  // only non-finite inputs can get here out of range
    const int oi = bi >> 5, ol = bi & 31;
    float cand = 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      if (i == oi) cand = a.weight_from_key ? key[i] : sc[i];
    const float u = __shfl_sync(kFull, cand, ol);
    if (ol == lane) taken |= 1u << oi;
    tot = __fadd_rn(tot, u);
    if (lane == k) {
      mysel = bi;
      myu = u;
    }
  }
  float wv = a.renorm ? __fdiv_rn(myu, fmaxf(tot, a.norm_min)) : myu;
  myw = __fmul_rn(wv, a.routed_scale);
}

template <int EPL>
__global__ void __launch_bounds__(kRouteThreads) route_kernel(const RouteArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  int32_t* s_ids = reinterpret_cast<int32_t*>(smem);                      // [kTile*K]
  uint16_t* s_cc = reinterpret_cast<uint16_t*>(smem + (size_t)kTile * a.K * 4);  // [nch][E]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int nwarps = kRouteThreads / 32;
  const int tile = blockIdx.x;
  const int64_t t0 = (int64_t)tile * kTile;
  const int ntok = (int)min((int64_t)kTile, a.T - t0);
  const int P = ntok * a.K;
  const int nch = (P + 31) >> 5;

  if (tile == 0 && tid < 8) a.ticket[tid] = 0;  // the scan that follows counts arrivals here
  {
    uint32_t* z32 = reinterpret_cast<uint32_t*>(s_cc);
    const int nw = (nch * a.E + 1) >> 1;
    for (int i = tid; i < nw; i += kRouteThreads) z32[i] = 0u;
  }

  for (int tl = warp; tl < ntok; tl += nwarps) {
    int mysel;
    float myw;
    route_token<EPL>(a, a.logits + (size_t)(t0 + tl) * a.E, lane, mysel, myw);
    if (lane < a.K) {
      const size_t s = (size_t)(t0 + tl) * a.K + lane;
      a.ids[s] = mysel;
      a.weights[s] = myw;
      s_ids[tl * a.K + lane] = mysel;
    }
  }
  __syncthreads();

  // Count every 32 consecutive pairs per expert.
  for (int c = warp; c < nch; c += nwarps) {
    const int p = c * 32 + lane;
    const int e = p < P ? s_ids[p] : -1;
    const unsigned m = __match_any_sync(kFull, e);
    if (e >= 0 && (m & ((1u << lane) - 1u)) == 0u) s_cc[c * a.E + e] = (uint16_t)__popc(m);
  }
  __syncthreads();
  // Exclusive prefix over the chunks of each expert, in pair order.
  for (int e = tid; e < a.E; e += kRouteThreads) {
    int run = 0;
    for (int c = 0; c < nch; ++c) {
      const int v = s_cc[c * a.E + e];
      s_cc[c * a.E + e] = (uint16_t)run;
      run += v;
    }
    a.tile_counts[(size_t)e * a.ntiles + tile] = run;
  }
  __syncthreads();
  for (int c = warp; c < nch; c += nwarps) {
    const int p = c * 32 + lane;
    const int e = p < P ? s_ids[p] : -1;
    const unsigned m = __match_any_sync(kFull, e);
    if (e >= 0)
      a.pair_rank[(size_t)t0 * a.K + p] = (int)s_cc[c * a.E + e] + __popc(m & ((1u << lane) - 1u));
  }
}

// ---------------------------------------------------------------------------
// Exclusive scan of the per-tile counts of one expert per block, then (in the
// block that finishes last) the scan across experts with the capacity clamp.
// Replaces the scan part of offsets_kernel (kernel.cu:2074-2086); offsets is
// stored as E+1 exclusive starts instead of the reference's inclusive ends
// `offs` plus exclusive starts `cursor`.
// ---------------------------------------------------------------------------
constexpr int kScanThreads = 256;

// Exclusive scan of v across the block; returns the exclusive prefix and the
// block total.  s_w holds one int per warp.
__device__ __forceinline__ int block_exclusive_scan(int v, int* s_w, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(kFull, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) s_w[warp] = incl;
  __syncthreads();
  int wp = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kScanThreads / 32; ++w) {
    const int sv = s_w[w];
    if (w < warp) wp += sv;
    tot += sv;
  }
  __syncthreads();  // s_w may be reused by the next call
  total = tot;
  return wp + incl - v;
}

__global__ void __launch_bounds__(kScanThreads)
scan_kernel(int32_t* __restrict__ tile_base, int32_t* __restrict__ counts,
            int32_t* __restrict__ user_counts, int32_t* __restrict__ offsets,
            int32_t* __restrict__ ticket, int E, int ntiles, int64_t capacity) {
  __shared__ int s_w[kScanThreads / 32];
  __shared__ int s_last;
  const int e = blockIdx.x, tid = threadIdx.x;
  int32_t* col = tile_base + (size_t)e * ntiles;
  int carry = 0;
  for (int base = 0; base < ntiles; base += kScanThreads) {
    const int i = base + tid;
    const int v = i < ntiles ? col[i] : 0;
    int total;
    const int ex = block_exclusive_scan(v, s_w, total);
    if (i < ntiles) col[i] = carry + ex;
    carry += total;
  }
  if (tid == 0) {
    counts[e] = carry;
    if (user_counts != nullptr) user_counts[e] = carry;
    __threadfence();
    s_last = atomicAdd(ticket, 1) == E - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  int run = 0;
  for (int base = 0; base < E; base += kScanThreads) {
    const int i = base + tid;
    int v = 0;
    if (i < E) {
      v = __ldcg(counts + i);
      if (capacity > 0 && (int64_t)v > capacity) v = (int)capacity;
    }
    int total;
    const int ex = block_exclusive_scan(v, s_w, total);
    if (i < E) offsets[i] = run + ex;
    run += total;
  }
  if (tid == 0) {
    offsets[E] = run;
    *ticket = 0;
  }
}

}  // namespace

cudaError_t launch_route(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                         const float* logits, int32_t* ids, int32_t* pair_rank, int32_t* tile_base,
                         int32_t* ticket, int32_t* status, cudaStream_t s) {
  (void)status;
  RouteArgs a;
  a.logits = logits;
  a.select_bias = b.select_bias;
  a.ids = ids;
  a.weights = b.combine_weights;
  a.pair_rank = pair_rank;
  a.tile_counts = tile_base;
  a.ticket = ticket;
  a.T = p.T;
  a.E = p.E;
  a.K = p.K;
  a.ntiles = plan.ntiles;
  a.n_groups = p.n_groups;
  a.topk_groups = p.topk_groups;
  a.group_topk = p.group_topk;
  a.score_fn = p.score_fn;
  a.weight_from_key = p.weight_from_key;
  a.renorm = p.renorm;
  a.routed_scale = p.routed_scale;
  a.norm_min = p.norm_min;
  const size_t smem = (size_t)kTile * p.K * 4 + (size_t)(kTile * p.K / 32) * p.E * 2 + 16;
  const dim3 grid((unsigned)plan.ntiles);
  if (p.E <= 32)
    route_kernel<1><<<grid, kRouteThreads, smem, s>>>(a);
  else if (p.E <= 64)
    route_kernel<2><<<grid, kRouteThreads, smem, s>>>(a);
  else if (p.E <= 128)
    route_kernel<4><<<grid, kRouteThreads, smem, s>>>(a);
  else
    route_kernel<8><<<grid, kRouteThreads, smem, s>>>(a);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_scan(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                        int32_t* tile_base, int32_t* counts, int32_t* ticket, cudaStream_t s) {
  scan_kernel<<<(unsigned)p.E, kScanThreads, 0, s>>>(tile_base, counts, b.counts, b.offsets, ticket,
                                                     p.E, plan.ntiles, p.capacity);
  count_launch();
  return cudaGetLastError();
}

cudaError_t init_route_attributes() {
  const int max_smem = kTile * kMaxK * 4 + (kTile * kMaxK / 32) * kMaxE * 2 + 16;
  cudaError_t e;
  e = cudaFuncSetAttribute(route_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(route_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(route_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(route_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              max_smem);
}

}  // namespace moe_rd
