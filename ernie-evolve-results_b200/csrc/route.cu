// Scoring / top-K / tile histogram for logits that already sit in memory (the
// tensor-core gate, the order-defining SIMT gate, or caller-supplied logits).
// The per-token device code lives in route_core.cuh.  The kernel leaves pair
// counts per (tile, expert) and per (group of tiles, expert); the positions
// kernel (scatter.cu) turns them into tile bases and offsets.
#include "route_core.cuh"
#include "route_lane.cuh"

namespace moe_rd {
namespace {

#ifndef MOE_RD_ROUTE_PREFETCH
#define MOE_RD_ROUTE_PREFETCH 1
#endif
#ifndef MOE_RD_ROUTE_LANE   // 0: always the lane-strided routing kernel (tuning/validation)
#define MOE_RD_ROUTE_LANE 1
#endif
#ifndef MOE_RD_ROUTE_LANE_THREE   // 1: three resident blocks per SM for E <= 128 in the lane-consecutive kernel
#define MOE_RD_ROUTE_LANE_THREE 1
#endif
constexpr int kRouteThreads = 512;
constexpr int kRouteWarps = kRouteThreads / 32;

// One warp per token.  Block b owns the contiguous token range
// [T*b/B, T*(b+1)/B): with B a multiple of the SM count every SM gets the same
// number of tokens to within one, whatever T is.  With group counts the blocks
// are dealt to the groups of kTileGroup counting tiles, blocks_per_group each,
// and share the tokens of their group the same way, so that a block's histogram
// belongs to one group.  The logits of a warp's next
// token are requested before the current one is scored.  MB = resident blocks
// per SM the register budget is cut for: 3 pays when every warp has several
// tokens to work through, 2 when it has one or two.
template <int EPL, bool FULL>
__device__ __forceinline__ void load_logits(const RouteArgs& a, int64_t t, int lane, float (&z)[EPL]) {
  const int ncol = a.fold ? 2 * a.E : a.E;
  const float* row = a.logits + (size_t)t * ncol + lane;  // split 0; the others are split_stride apart
  const size_t split_stride = (size_t)a.T * ncol;
  // every load of the token is issued before the first add
  float v[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) v[i] = (FULL || lane + 32 * i < a.E) ? __ldg(row + 32 * i) : 0.0f;
  if (a.fold) {
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      if (FULL || lane + 32 * i < a.E) v[i] = __fadd_rn(v[i], __ldg(row + a.E + 32 * i));
  }
  // splits in ascending order; with the hi/lo weight split each split contributes hi + lo
  for (int sp = 1; sp < a.nsplit; ++sp) {
    const float* rs = row + sp * split_stride;
    float p[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) p[i] = (FULL || lane + 32 * i < a.E) ? __ldg(rs + 32 * i) : 0.0f;
    if (a.fold) {
#pragma unroll
      for (int i = 0; i < EPL; ++i)
        if (FULL || lane + 32 * i < a.E) p[i] = __fadd_rn(p[i], __ldg(rs + a.E + 32 * i));
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) v[i] = __fadd_rn(v[i], p[i]);
  }
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int e = lane + 32 * i;
    if (FULL || e < a.E) {
      if (a.logit_bias != nullptr) v[i] = __fadd_rn(v[i], __ldg(a.logit_bias + e));
      if (a.logits_out != nullptr) a.logits_out[(size_t)t * a.E + e] = v[i];
    } else {
      v[i] = 0.0f;
    }
    z[i] = v[i];
  }
}

template <int EPL, bool FULL, int MB>
__global__ void __launch_bounds__(kRouteThreads, MB) route_kernel(const RouteArgs a) {
  __shared__ int s_cnt[kMaxE];
  __shared__ float s_sc[EPL > 1 ? kRouteWarps * 32 * EPL : 1];
  for (int e = threadIdx.x; e < a.E; e += kRouteThreads) s_cnt[e] = 0;
  __syncthreads();
  pdl_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t lo, hi;
  int group = 0;
  if (a.group_counts != nullptr) {
    constexpr int64_t kGroupTokens = (int64_t)kTileGroup * kTile;
    group = blockIdx.x / a.blocks_per_group;
    const int j = blockIdx.x - group * a.blocks_per_group;
    const int64_t glo = group * kGroupTokens;
    const int64_t n = min(kGroupTokens, a.T - glo);
    lo = glo + n * j / a.blocks_per_group;
    hi = glo + n * (j + 1) / a.blocks_per_group;
  } else {
    lo = a.T * blockIdx.x / gridDim.x;
    hi = a.T * (blockIdx.x + 1) / gridDim.x;
  }
  float zn[EPL];
  if (lo + warp < hi) load_logits<EPL, FULL>(a, lo + warp, lane, zn);
  for (int64_t t = lo + warp; t < hi; t += kRouteWarps) {
    float z[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) z[i] = zn[i];
    if (!MOE_RD_ROUTE_PREFETCH && t > lo + warp) load_logits<EPL, FULL>(a, t, lane, z);
    if (MOE_RD_ROUTE_PREFETCH && t + kRouteWarps < hi) load_logits<EPL, FULL>(a, t + kRouteWarps, lane, zn);
    int mysel;
    float myw;
    route_token<EPL, FULL>(a, z, lane, EPL > 1 ? s_sc + warp * 32 * EPL : nullptr, mysel, myw);
    publish_token(a, t, lane, mysel, myw, s_cnt);
  }
  __syncthreads();
  flush_counts(a, s_cnt, kRouteThreads, group);
}


// ---------------------------------------------------------------------------
// The same kernel with consecutive experts per lane (route_lane.cuh) for
// E = 64, 128, 256: the EPL logits of a lane are one or two 16-byte vectors.
// ---------------------------------------------------------------------------
template <int EPL>
__device__ __forceinline__ void load_vec(const float* p, float (&v)[EPL]) {
  if (EPL == 2) {
    const float2 a = __ldg(reinterpret_cast<const float2*>(p));
    v[0] = a.x; v[1] = a.y;
  } else {
#pragma unroll
    for (int q = 0; q < EPL / 4; ++q) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(p) + q);
      v[4 * q] = a.x; v[4 * q + 1] = a.y; v[4 * q + 2] = a.z; v[4 * q + 3] = a.w;
    }
  }
}
template <int EPL>
__device__ __forceinline__ void store_vec(float* p, const float (&v)[EPL]) {
  if (EPL == 2) {
    *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
  } else {
#pragma unroll
    for (int q = 0; q < EPL / 4; ++q)
      reinterpret_cast<float4*>(p)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  }
}

// Final logits of token t for this lane's experts: the splits in ascending order (with the
// hi/lo weight split each contributes hi + lo), then the logit bias lb.
template <int EPL>
__device__ __forceinline__ void load_logits_c(const RouteArgs& a, int64_t t, int lane, float (&z)[EPL]) {
  const int ncol = a.fold ? 2 * a.E : a.E;
  const float* row = a.logits + (size_t)t * ncol + EPL * lane;
  const size_t split_stride = (size_t)a.T * ncol;
  float v[EPL];
  load_vec<EPL>(row, v);
  if (a.fold) {
    float lo[EPL];
    load_vec<EPL>(row + a.E, lo);
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = __fadd_rn(v[j], lo[j]);
  }
  for (int sp = 1; sp < a.nsplit; ++sp) {
    float p[EPL];
    load_vec<EPL>(row + sp * split_stride, p);
    if (a.fold) {
      float lo[EPL];
      load_vec<EPL>(row + sp * split_stride + a.E, lo);
#pragma unroll
      for (int j = 0; j < EPL; ++j) p[j] = __fadd_rn(p[j], lo[j]);
    }
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = __fadd_rn(v[j], p[j]);
  }
  if (a.logit_bias != nullptr) {
    float lb[EPL];
    load_vec<EPL>(a.logit_bias + EPL * lane, lb);
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = __fadd_rn(v[j], lb[j]);
  }
  if (a.logits_out != nullptr) store_vec<EPL>(a.logits_out + (size_t)t * a.E + EPL * lane, v);
#pragma unroll
  for (int j = 0; j < EPL; ++j) z[j] = v[j];
}

template <int EPL, int MB>
__global__ void __launch_bounds__(kRouteThreads, MB) route_lane_kernel(const RouteArgs a) {
  __shared__ int s_cnt[kMaxE];
  __shared__ __align__(16) uint32_t s_cand[kRouteWarps * kLaneCandWords];
  for (int e = threadIdx.x; e < a.E; e += kRouteThreads) s_cnt[e] = 0;
  __syncthreads();
  pdl_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // blocks are dealt to the groups of kTileGroup counting tiles (see route_kernel)
  constexpr int64_t kGroupTokens = (int64_t)kTileGroup * kTile;
  const int group = blockIdx.x / a.blocks_per_group;
  const int jb = blockIdx.x - group * a.blocks_per_group;
  const int64_t glo = group * kGroupTokens;
  const int64_t n = min(kGroupTokens, a.T - glo);
  const int64_t lo = glo + n * jb / a.blocks_per_group;
  const int64_t hi = glo + n * (jb + 1) / a.blocks_per_group;
  float zn[EPL];
  if (lo + warp < hi) load_logits_c<EPL>(a, lo + warp, lane, zn);
  for (int64_t t = lo + warp; t < hi; t += kRouteWarps) {
    float z[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) z[j] = zn[j];
    if (t + kRouteWarps < hi) load_logits_c<EPL>(a, t + kRouteWarps, lane, zn);
    int mysel;
    float myw;
    route_token_c<EPL>(a, z, lane, s_cand + warp * kLaneCandWords, mysel, myw);
    publish_token(a, t, lane, mysel, myw, s_cnt);
  }
  __syncthreads();
  flush_counts(a, s_cnt, kRouteThreads, group);
}

}  // namespace

int device_sms() {
  static int cached[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = sms;
  }
  return cached[dev];
}

void fill_route_args(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                     const float* logits, int32_t* ids, int32_t* tile_base, int32_t* counts,
                     RouteArgs* a) {
  a->logits = logits;
  a->logit_bias = nullptr;
  a->logits_out = nullptr;
  a->nsplit = 1;
  a->fold = 0;
  a->select_bias = b.select_bias;
  a->ids = ids;
  a->weights = b.combine_weights;
  a->tile_counts = tile_base;
  a->counts = counts;
  a->group_counts = nullptr;
  a->blocks_per_group = 1;
  a->T = p.T;
  a->E = p.E;
  a->K = p.K;
  a->ntiles = plan.ntiles;
  a->n_groups = p.n_groups;
  a->topk_groups = p.topk_groups;
  a->group_topk = p.group_topk;
  a->score_fn = p.score_fn;
  a->weight_from_key = p.weight_from_key;
  a->renorm = p.renorm;
  a->routed_scale = p.routed_scale;
  a->norm_min = p.norm_min;
}

cudaError_t launch_route(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                         const float* logits, int32_t* ids, int32_t* tile_base, int32_t* counts,
                         int32_t* group_counts, cudaStream_t s) {
  return launch_route_splits(p, b, plan, logits, 1, nullptr, nullptr, ids, tile_base, counts, group_counts, s);
}

cudaError_t launch_route_splits(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                                const float* partial, int nsplit, const float* logit_bias,
                                float* logits_out, int32_t* ids, int32_t* tile_base,
                                int32_t* counts, int32_t* group_counts, cudaStream_t s) {
  RouteArgs a;
  fill_route_args(p, b, plan, partial, ids, tile_base, counts, &a);
  a.group_counts = plan.tile_major ? group_counts : nullptr;
  a.nsplit = nsplit;
  a.fold = plan.gate == MOE_RD_GATE_UMMA ? plan.umma_fold : 0;
  a.logit_bias = logit_bias;
  a.logits_out = logits_out;
  // Three resident blocks of 512 threads per SM when every warp then still has
  // at least two tokens and 40 registers hold a token (<= 4 experts per lane),
  // else two.
  const int sms = device_sms();
  const int epl = p.E <= 32 ? 1 : p.E <= 64 ? 2 : p.E <= 128 ? 4 : 8;
  const bool three = epl <= 4 && p.T >= (int64_t)sms * 3 * kRouteWarps * 2;
  int64_t nblk = (int64_t)sms * (three ? 3 : 2);
  const int64_t need = (p.T + kRouteWarps - 1) / kRouteWarps;
  if (nblk > need) nblk = need;
  if (a.group_counts != nullptr) {
    const int64_t ngroups = (plan.ntiles + kTileGroup - 1) / kTileGroup;
    int64_t bpg = nblk / ngroups;
    if (bpg < 1) bpg = 1;
    a.blocks_per_group = (int)bpg;
    nblk = ngroups * bpg;
  }
  const dim3 grid((unsigned)nblk);
  const dim3 blk(kRouteThreads);
  const bool full = p.E == 32 * epl;
  cudaError_t e;
  // consecutive experts per lane: E of 64, 128 or 256, tile-major counts, and logits and biases that
  // can be read as 16-byte vectors
  const auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (MOE_RD_ROUTE_LANE && a.group_counts != nullptr &&
      lane_route_supported(p.E, p.K, p.n_groups, p.topk_groups, p.group_topk) && aligned16(a.logits) &&
      aligned16(a.logit_bias) && aligned16(a.select_bias) && aligned16(a.logits_out)) {
    const bool three_c = three && MOE_RD_ROUTE_LANE_THREE;
    if (!three_c && three) {
      // fewer resident blocks: size the grid for two per SM
      int64_t nb2 = (int64_t)sms * 2;
      if (nb2 > need) nb2 = need;
      const int64_t ngroups = (plan.ntiles + kTileGroup - 1) / kTileGroup;
      int64_t bpg = nb2 / ngroups;
      if (bpg < 1) bpg = 1;
      a.blocks_per_group = (int)bpg;
      nblk = ngroups * bpg;
    }
    const dim3 grid_c((unsigned)nblk);
    if (p.E == 64)
      e = three_c ? launch_pdl(route_lane_kernel<2, 3>, grid_c, blk, 0, s, a) : launch_pdl(route_lane_kernel<2, 2>, grid_c, blk, 0, s, a);
    else if (p.E == 128)
      e = three ? launch_pdl(route_lane_kernel<4, 3>, grid, blk, 0, s, a) : launch_pdl(route_lane_kernel<4, 2>, grid, blk, 0, s, a);
    else
      e = launch_pdl(route_lane_kernel<8, 2>, grid, blk, 0, s, a);
    count_launch();
    return e;
  }
#define MOE_RD_ROUTE_CASE(EPL_)                                                              \
  case EPL_:                                                                                 \
    e = full ? (three ? launch_pdl(route_kernel<EPL_, true, 3>, grid, blk, 0, s, a)          \
                      : launch_pdl(route_kernel<EPL_, true, 2>, grid, blk, 0, s, a))         \
             : (three ? launch_pdl(route_kernel<EPL_, false, 3>, grid, blk, 0, s, a)         \
                      : launch_pdl(route_kernel<EPL_, false, 2>, grid, blk, 0, s, a));       \
    break;
  switch (epl) {
    MOE_RD_ROUTE_CASE(1)
    MOE_RD_ROUTE_CASE(2)
    MOE_RD_ROUTE_CASE(4)
    default:
    MOE_RD_ROUTE_CASE(8)
  }
#undef MOE_RD_ROUTE_CASE
  count_launch();
  return e;
}

cudaError_t init_route_attributes() { return cudaSuccess; }

}  // namespace moe_rd
