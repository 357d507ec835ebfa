// Scoring / top-K / tile histogram for logits that already sit in memory (the
// tensor-core gate, the order-defining SIMT gate, or caller-supplied logits).
// The per-token device code lives in route_core.cuh.  The kernel leaves pair
// counts per (tile, expert) and per (group of tiles, expert); the positions
// kernel (scatter.cu) turns them into tile bases and offsets.
#include "route_core.cuh"

namespace moe_rd {
namespace {

#ifndef MOE_RD_ROUTE_PREFETCH
#define MOE_RD_ROUTE_PREFETCH 1
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
  __shared__ uint32_t s_cand[EPL > 1 ? kRouteWarps * kRouteCandWords : 1];
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
    route_token<EPL, FULL>(a, z, lane, EPL > 1 ? s_sc + warp * 32 * EPL : nullptr, mysel, myw,
                           EPL > 1 ? s_cand + warp * kRouteCandWords : nullptr);
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
