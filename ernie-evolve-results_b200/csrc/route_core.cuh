// Device code shared by the routing kernels: per-token scoring / top-K, and
// the deterministic per-tile histogram with in-tile stable ranks.
//
// Follows topk_kernel of the reference (kernel.cu:1829-1920): one warp per
// token, experts strided over lanes (expert e lives in lane e%32, register
// e/32), softmax as max / exp / sum / reciprocal-multiply (1857-1866), bias
// added to the score to form the selection key (1865-1866), K rounds of warp
// arg-max with lowest-index tie-break (1872-1901), weights u / max(sum u,
// norm_min) (1909).  Added: sigmoid scoring, selection-only bias,
// group-limited selection, a final scale.  The reference's 5-step shuffle
// arg-max is replaced by two redux.sync operations on order-preserving integer
// images of the keys (max of the keys, then min of the indices that hold it),
// which selects the same expert.
//
// The reference ranks a pair inside its expert with shared and global atomics
// whose return values become slot positions (dispatch_body,
// kernel.cu:2155-2158), so its slot order depends on scheduling.  Here the
// routing kernels only COUNT with atomics: pairs per (expert, tile of kTile
// consecutive tokens), an integer sum that is the same in any order.  Slot
// order is decided later, from the ids alone (positions_kernel, scatter.cu).
#pragma once

#include "common.cuh"

#ifndef MOE_RD_ROUTE_SORTED
#define MOE_RD_ROUTE_SORTED 1
#endif

namespace moe_rd {

struct RouteArgs {
  const float* logits;       // [nsplit][T,E] (unused by the fused gate kernel)
  const float* logit_bias;   // [E] added after the splits are summed, or null
  float* logits_out;         // [T,E] final logits for the caller, or null
  int nsplit;                // number of K-split partial products to add, in order
  int fold;                  // 1: a row of `logits` has 2E columns (bf16 hi and lo parts of an fp32
                             // gate weight) and logit e = column e + column E+e (kernel.cu:1849-1851)
  const float* select_bias;  // [E] or null
  int32_t* ids;              // [T,K]
  float* weights;            // [T,K]
  int32_t* tile_counts;      // [E][ntiles], zeroed before the kernel
  int32_t* counts;           // [E], zeroed before the kernel
  int32_t* group_counts;     // null, or [ceil(ntiles/kTileGroup)][E] pairs per expert and group of
                             // kTileGroup tiles, zeroed before the kernel; tile_counts is then laid out
                             // [ntiles][E] and `counts` is left alone
  int blocks_per_group;      // with group_counts: consecutive blocks that share a group of tiles
  int64_t T;
  int E, K, ntiles;
  int n_groups, topk_groups, group_topk;
  int score_fn, weight_from_key, renorm;
  float routed_scale, norm_min;
};

// Order-preserving map fp32 -> uint32 (-0.0 is folded onto +0.0 so that keys
// that compare equal as floats have equal images).
__device__ __forceinline__ uint32_t ord_key(float f) {
  uint32_t u = __float_as_uint(f);
  if (u == 0x80000000u) u = 0u;
  return u ^ ((uint32_t)((int32_t)u >> 31) | 0x80000000u);
}
__device__ __forceinline__ float ord_value(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}

// Scores one token held as z[i] = logit of expert lane + 32*i and selects its
// K experts.  On return lane k < K holds slot k: `mysel` the expert, `myw` the
// combine weight.  All 32 lanes of the warp must call.
//
// FULL: E == 32*EPL, so no register needs a bounds test.  s_sc: null, or 32*EPL
// floats of shared memory owned by this warp; the scores are then parked there
// and lane k fetches the score of its expert after the selection, instead of
// every round broadcasting it out of a register picked by a chain of selects.
// A selected key is removed by zeroing its image (0 = not eligible), so a round
// costs one max pass, one index pass and one removal pass over the registers.
template <int EPL, bool FULL>
__device__ __forceinline__ void route_token(const RouteArgs& a, const float (&z)[EPL], int lane,
                                            float* s_sc, int& mysel, float& myw) {
  float sc[EPL];
  uint32_t ok[EPL];  // ordered images of the selection keys; 0 = not eligible
  if (a.score_fn == MOE_RD_SCORE_SOFTMAX) {
    uint32_t mk = 0u;
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      if (FULL || lane + 32 * i < a.E) mk = max(mk, ord_key(z[i]));
    const float m = ord_value(__reduce_max_sync(kFull, mk));
    float part = 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const float p = (FULL || lane + 32 * i < a.E) ? exp_ieee(__fsub_rn(z[i], m)) : 0.0f;
      sc[i] = p;
      part = __fadd_rn(part, p);
    }
    const float rs = __frcp_rn(warp_tree_sum(part));  // correctly rounded: same bits as 1.0f / s
#pragma unroll
    for (int i = 0; i < EPL; ++i) sc[i] = __fmul_rn(sc[i], rs);
  } else {
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      sc[i] = (FULL || lane + 32 * i < a.E) ? __frcp_rn(__fadd_rn(1.0f, exp_ieee(-z[i]))) : 0.0f;
  }
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int e = lane + 32 * i;
    float key = sc[i];
    if ((FULL || e < a.E) && a.select_bias != nullptr) key = __fadd_rn(key, __ldg(a.select_bias + e));
    ok[i] = (FULL || e < a.E) ? ord_key(key) : 0u;
  }
  const bool staged = s_sc != nullptr && EPL > 1 && !a.weight_from_key;

  if (a.n_groups > 1) {
    const int gs = a.E / a.n_groups;
    float mygs = 0.0f;  // lane g keeps the score of group g
    if (gs == 32 && a.group_topk <= 2) {
      // Group g is exactly register g of every lane.
#pragma unroll
      for (int g = 0; g < EPL; ++g) {
        if (g < a.n_groups) {
          const uint32_t l1 = ok[g];
          const uint32_t m1 = __reduce_max_sync(kFull, l1);
          float sum = ord_value(m1);
          if (a.group_topk == 2) {
            // Second largest = largest once ONE instance of m1 is removed.
            const unsigned holders = __ballot_sync(kFull, l1 == m1);
            uint32_t m2 = m1;
            if (__popc(holders) < 2) m2 = __reduce_max_sync(kFull, l1 == m1 ? 0u : l1);
            sum = __fadd_rn(sum, ord_value(m2));
          }
          if (lane == g) mygs = sum;
        }
      }
    } else if ((gs & 31) == 0 && a.group_topk <= 2) {
      // A group is a whole number of registers: m = gs/32 of them per lane.
      const int m = gs >> 5;
      for (int g = 0; g < a.n_groups; ++g) {
        uint32_t l1 = 0u, l2 = 0u;  // the lane's two largest images inside the group
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          if (i >= g * m && i < (g + 1) * m) {
            const uint32_t v = ok[i];
            if (v > l1) {
              l2 = l1;
              l1 = v;
            } else if (v > l2) {
              l2 = v;
            }
          }
        }
        const uint32_t m1 = __reduce_max_sync(kFull, l1);
        float sum = ord_value(m1);
        if (a.group_topk == 2) {
          const unsigned holders = __ballot_sync(kFull, l1 == m1);
          uint32_t m2 = m1;
          if (__popc(holders) < 2) m2 = __reduce_max_sync(kFull, l1 == m1 ? l2 : l1);
          sum = __fadd_rn(sum, ord_value(m2));
        }
        if (lane == g) mygs = sum;
      }
    } else {
      for (int g = 0; g < a.n_groups; ++g) {
        const int lo = g * gs, hi = lo + gs;
        unsigned gtaken = 0;
        float sum = 0.0f;
        for (int r = 0; r < a.group_topk; ++r) {
          uint32_t bk = 0u;
          int bi = 0x7fffffff;
#pragma unroll
          for (int i = 0; i < EPL; ++i) {
            const int e = lane + 32 * i;
            if (e >= lo && e < hi && !((gtaken >> i) & 1u) && ok[i] > bk) {
              bk = ok[i];
              bi = e;
            }
          }
          const uint32_t mx = __reduce_max_sync(kFull, bk);
          const int win = (int)__reduce_min_sync(kFull, (unsigned)(bk == mx ? bi : 0x7fffffff));
          if (win < a.E && (win & 31) == lane) gtaken |= 1u << (win >> 5);
          const float bv = ord_value(mx);
          sum = r == 0 ? bv : __fadd_rn(sum, bv);
        }
        if (lane == g) mygs = sum;
      }
    }
    int rank = 0;
    for (int o = 0; o < a.n_groups; ++o) {
      const float og = __shfl_sync(kFull, mygs, o);
      if (og > mygs || (og == mygs && o < lane)) ++rank;
    }
    const unsigned keep = __ballot_sync(kFull, lane < a.n_groups && rank < a.topk_groups);
    if ((gs & 31) == 0) {
      // register i belongs to group i / (gs/32), the same for every lane
      const int m = gs >> 5;
      int g = 0, c = 0;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        if (!((keep >> g) & 1u)) ok[i] = 0u;
        if (++c == m) {
          c = 0;
          ++g;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const int e = lane + 32 * i;
        if (e < a.E && !((keep >> (e / gs)) & 1u)) ok[i] = 0u;
      }
    }
  }

  float tot = 0.0f, myu = 0.0f;
  mysel = 0;
  if (staged) {
    __syncwarp();  // the previous token's readers are done with s_sc
#pragma unroll
    for (int i = 0; i < EPL; ++i) s_sc[lane + 32 * i] = sc[i];
  }
  // With many registers per lane and many rounds it pays to sort each lane's
  // keys once (descending; odd-even transposition with a strict compare keeps
  // equal keys in index order) and then only look at the head of every lane.
  const bool sorted = MOE_RD_ROUTE_SORTED && EPL >= 4 && (staged || a.weight_from_key) && a.K >= (EPL >= 8 ? 6 : 3);
  if (sorted) {
    int ix[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) ix[i] = lane + 32 * i;
#pragma unroll
    for (int pass = 0; pass < EPL; ++pass) {
#pragma unroll
      for (int i = pass & 1; i + 1 < EPL; i += 2) {
        const bool sw = ok[i + 1] > ok[i];
        const uint32_t ka = ok[i], kb = ok[i + 1];
        const int ia = ix[i], ib = ix[i + 1];
        ok[i] = sw ? kb : ka;
        ok[i + 1] = sw ? ka : kb;
        ix[i] = sw ? ib : ia;
        ix[i + 1] = sw ? ia : ib;
      }
    }
    for (int k = 0; k < a.K; ++k) {
      const uint32_t mx = __reduce_max_sync(kFull, ok[0]);
      int win = (int)__reduce_min_sync(kFull, (unsigned)(ok[0] == mx ? ix[0] : 0x7fffffff));
      if (mx == 0u) win = 0x7fffffff;   // nothing eligible is left
      win = min(max(win, 0), a.E - 1);  // only then is the index out of range
      const bool pop = ix[0] == win;
#pragma unroll
      for (int i = 0; i + 1 < EPL; ++i) {
        ok[i] = pop ? ok[i + 1] : ok[i];
        ix[i] = pop ? ix[i + 1] : ix[i];
      }
      if (pop) ok[EPL - 1] = 0u;
      if (a.weight_from_key) {
        const float cand = ord_value(mx);
        tot = __fadd_rn(tot, cand);
        if (lane == k) myu = cand;
      }
      if (lane == k) mysel = win;
    }
  } else {
  for (int k = 0; k < a.K; ++k) {
    uint32_t bk = ok[0];
#pragma unroll
    for (int i = 1; i < EPL; ++i) bk = max(bk, ok[i]);
    const uint32_t mx = __reduce_max_sync(kFull, bk);
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = EPL - 1; i >= 0; --i)
      if (ok[i] == mx) bi = lane + 32 * i;  // descending: the lowest register wins ties
    int win = (int)__reduce_min_sync(kFull, (unsigned)bi);
    if (mx == 0u) win = 0x7fffffff;          // nothing eligible is left
    win = min(max(win, 0), a.E - 1);         // only then is the index out of range
    const int d = win - lane;                // == 32*i on the lane and register that hold it
    if (staged) {
#pragma unroll
      for (int i = 0; i < EPL; ++i)
        if (d == 32 * i) ok[i] = 0u;
      if (lane == k) mysel = win;
    } else {
      float cand = 0.0f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        if (d == 32 * i) {
          cand = sc[i];
          ok[i] = 0u;
        }
      }
      cand = a.weight_from_key ? ord_value(mx) : __shfl_sync(kFull, cand, win & 31);
      tot = __fadd_rn(tot, cand);
      if (lane == k) {
        mysel = win;
        myu = cand;
      }
    }
  }
  }
  if (staged) {
    __syncwarp();
    if (lane < a.K) myu = s_sc[mysel];
    for (int k = 0; k < a.K; ++k) tot = __fadd_rn(tot, __shfl_sync(kFull, myu, k));
  }
  const float wv = a.renorm ? __fdiv_rn(myu, fmaxf(tot, a.norm_min)) : myu;
  myw = __fmul_rn(wv, a.routed_scale);
}

// Several tokens per warp for few experts: token i of the warp lives in lanes
// i*W .. i*W+W-1 (W = 8 or 16 lanes, E <= W), lane i*W+e holding the logit of
// expert e.  Same arithmetic and order as route_token: the softmax sum of
// route_token is the 32-lane tree over lanes that hold zeros beyond E, and adding
// those zeros changes nothing, so the W-lane tree below gives the same bits.
// No expert groups (callers use route_token when n_groups > 1).  On return lane
// i*W+k (k < K) holds slot k of token i.
template <int W>
__device__ __forceinline__ void route_token_packed(const RouteArgs& a, float z, int lane, int& mysel,
                                                   float& myw) {
  const int e = lane & (W - 1);
  const int base = lane & ~(W - 1);
  const unsigned gmask = (W == 32) ? kFull : (((1u << W) - 1u) << base);
  const bool valid = e < a.E;
  float sc;
  if (a.score_fn == MOE_RD_SCORE_SOFTMAX) {
    const float m = ord_value(__reduce_max_sync(gmask, valid ? ord_key(z) : 0u));
    const float p = valid ? exp_ieee(__fsub_rn(z, m)) : 0.0f;
    float sum = p;
#pragma unroll
    for (int o = W / 2; o; o >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(gmask, sum, o));
    sc = __fmul_rn(p, __frcp_rn(sum));
  } else {
    sc = valid ? __frcp_rn(__fadd_rn(1.0f, exp_ieee(-z))) : 0.0f;
  }
  float key = sc;
  if (valid && a.select_bias != nullptr) key = __fadd_rn(key, __ldg(a.select_bias + e));
  uint32_t ok = valid ? ord_key(key) : 0u;
  float tot = 0.0f, myu = 0.0f;
  mysel = 0;
  for (int k = 0; k < a.K; ++k) {
    const uint32_t mx = __reduce_max_sync(gmask, ok);
    int win = (int)__reduce_min_sync(gmask, (unsigned)(ok == mx ? e : 0x7fffffff));
    if (mx == 0u) win = 0x7fffffff;
    win = min(max(win, 0), a.E - 1);
    const float cand = a.weight_from_key ? ord_value(mx) : __shfl_sync(gmask, sc, base + win);
    if (e == win) ok = 0u;
    tot = __fadd_rn(tot, cand);
    if (e == k) {
      mysel = win;
      myu = cand;
    }
  }
  const float wv = a.renorm ? __fdiv_rn(myu, fmaxf(tot, a.norm_min)) : myu;
  myw = __fmul_rn(wv, a.routed_scale);
}

// Lanes k < K publish slot k of token t: id, weight, one count for the
// (expert, tile) cell, and one count in the block's shared histogram s_cnt[E]
// (a popular expert would otherwise serialise tens of thousands of global
// atomics on one address).
__device__ __forceinline__ void publish_token(const RouteArgs& a, int64_t t, int lane, int mysel,
                                              float myw, int* s_cnt) {
  if (lane < a.K) {
    const size_t s = (size_t)t * a.K + lane;
    a.ids[s] = mysel;
    a.weights[s] = myw;
    if (a.group_counts != nullptr)
      atomicAdd(a.tile_counts + (size_t)(t / kTile) * a.E + mysel, 1);  // [tile][expert]
    else
      atomicAdd(a.tile_counts + (size_t)mysel * a.ntiles + (int)(t / kTile), 1);
    atomicAdd(s_cnt + mysel, 1);
  }
}

// Block-wide: add the shared histogram to counts[E], or to row `group` of
// group_counts.  Call after a barrier.
__device__ __forceinline__ void flush_counts(const RouteArgs& a, const int* s_cnt, int nthreads, int group = 0) {
  int32_t* dst = a.group_counts != nullptr ? a.group_counts + (size_t)group * a.E : a.counts;
  for (int e = threadIdx.x; e < a.E; e += nthreads) {
    const int v = s_cnt[e];
    if (v) atomicAdd(dst + e, v);
  }
}

void fill_route_args(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                     const float* logits, int32_t* ids, int32_t* tile_base, int32_t* counts,
                     RouteArgs* a);
int device_sms();

}  // namespace moe_rd
