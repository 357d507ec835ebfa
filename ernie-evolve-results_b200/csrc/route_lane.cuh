// Scoring / top-K of one token by one warp with CONSECUTIVE experts per lane:
// lane l holds experts EPL*l .. EPL*l+EPL-1 (E = 32*EPL, EPL = 2, 4 or 8).
//
// Same results, bit for bit, as route_token (route_core.cuh), which follows
// topk_kernel of the reference (kernel.cu:1829-1920) and strides the experts
// over the lanes (expert e in lane e % 32).  With consecutive experts a group of
// experts (group-limited routing) is a run of lanes, so all groups are ranked at
// once with a few shuffles inside the runs instead of one warp-wide reduction
// per group, the logits arrive as 16-byte vectors, and the K experts are found
// without K rounds of warp-wide arg-max:
//   1. the lanes are cut into slices (the expert groups, or runs of lanes chosen
//      so that slices * q >= K with q = 1 or 2); every slice that may contribute
//      notes its q-th largest key, and the smallest of those, tau, is a lower
//      bound of the K-th largest key of the token (at least K keys are >= tau);
//   2. the keys >= tau (a dozen or so) are listed in expert order;
//   3. lane c counts the listed keys that beat key c (larger, or equal and listed
//      earlier, i.e. lower expert index): that count is its slot if below K.
// "Larger key first, lower index on ties" is a total order, and every key that
// can be among the K largest is on the list, so these are the experts, in the
// order, that K rounds of arg-max with lowest-index tie-break produce.  (K rounds
// of arg-max over one listed key per lane were measured too: no fewer
// instructions than the count.)
// When more than 32 keys reach tau (long runs of equal keys) or fewer than K are
// eligible, the rounds decide (select_by_rounds_c).
//
// Order-dependent arithmetic is kept as route_token defines it:
//  * softmax sum: partial l = p[l] + p[l+32] + p[l+64] + ... (ascending), then
//    the tree v[l] += v[l^off], off = 16..1 over the 32 partials;
//  * weights: tot = u_0 + u_1 + ... in slot order.
#pragma once

#include "route_core.cuh"

namespace moe_rd {

constexpr int kLaneCandWords = 3 * 32 + 2 * kMaxK;  // per-warp shared memory of route_token_c

// Whether route_token_c covers these routing parameters.
__host__ __device__ inline bool lane_route_supported(int E, int K, int n_groups, int topk_groups, int group_topk) {
  if (E != 64 && E != 128 && E != 256) return false;
  const int epl = E >> 5;
  if (K > kMaxK) return false;
  if (n_groups > 1) {
    const int gs = E / n_groups;
    if (gs % epl != 0) return false;
    const int lpg = gs / epl;  // lanes per group: a power of two
    if ((lpg & (lpg - 1)) != 0 || group_topk > 2) return false;
  }
  return true;
}

// Round-by-round selection in the consecutive layout (the slow path, and the
// path for K beyond what the threshold covers).  ok[]: ordered key images, 0 =
// not eligible.  On return lane k < K holds slot k.
template <int EPL>
__device__ __forceinline__ void select_by_rounds_c(const RouteArgs& a, uint32_t (&ok)[EPL], const float (&sc)[EPL],
                                                    int lane, int& mysel, float& myu, float& tot) {
  tot = 0.0f;
  myu = 0.0f;
  mysel = 0;
  for (int k = 0; k < a.K; ++k) {
    uint32_t bk = ok[0];
#pragma unroll
    for (int j = 1; j < EPL; ++j) bk = max(bk, ok[j]);
    const uint32_t mx = __reduce_max_sync(kFull, bk);
    // the lowest lane that holds the maximum holds its lowest expert index
    const unsigned holders = __ballot_sync(kFull, bk == mx);
    const int wl = __ffs(holders) - 1;
    int wj = EPL - 1;
#pragma unroll
    for (int j = EPL - 2; j >= 0; --j) wj = ok[j] == mx ? j : wj;
    float cand = 0.0f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) cand = j == wj ? sc[j] : cand;
    int win = __shfl_sync(kFull, EPL * lane + wj, wl);
    cand = __shfl_sync(kFull, cand, wl);
    if (mx == 0u) {
      win = a.E - 1;  // nothing eligible is left (route_token clamps the same way)
      cand = __shfl_sync(kFull, sc[EPL - 1], 31);
    } else if (lane == wl) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) ok[j] = j == wj ? 0u : ok[j];
    }
    if (a.weight_from_key) cand = ord_value(mx);
    tot = __fadd_rn(tot, cand);
    if (lane == k) {
      mysel = win;
      myu = cand;
    }
  }
}

// z[j]: final logit of expert EPL*lane + j (a.select_bias, when given, must be
// readable as 16-byte vectors).  On return lane k < K holds slot k: `mysel` the expert, `myw`
// the combine weight.  s_cand: kLaneCandWords words of shared memory owned by
// this warp, 16-byte aligned.  All 32 lanes must call.
template <int EPL>
__device__ __forceinline__ void route_token_c(const RouteArgs& a, const float (&z)[EPL], int lane,
                                              uint32_t* s_cand, int& mysel, float& myw) {
  constexpr int LPB = 32 / EPL;  // lanes per block of 32 consecutive experts
  float sc[EPL];
  if (a.score_fn == MOE_RD_SCORE_SOFTMAX) {
    uint32_t mk = 0u;
#pragma unroll
    for (int j = 0; j < EPL; ++j) mk = max(mk, ord_key(z[j]));
    const float m = ord_value(__reduce_max_sync(kFull, mk));
#pragma unroll
    for (int j = 0; j < EPL; ++j) sc[j] = exp_ieee(__fsub_rn(z[j], m));
    // partial l = p[l] + p[l+32] + ...: expert 32*i + l sits in lane LPB*i + l/EPL, register l%EPL,
    // so the partials are chains over the lanes LPB apart, accumulated in ascending i
    float v[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = sc[j];
    const int blk = lane / LPB;
#pragma unroll
    for (int step = 1; step < EPL; ++step) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const float below = __shfl_up_sync(kFull, v[j], LPB);
        if (blk == step) v[j] = __fadd_rn(below, sc[j]);
      }
    }
    // the lanes of the last block now hold the 32 partials, l = EPL*(lane % LPB) + j; the tree
    // v[l] += v[l^off] runs over lanes for off >= EPL and over registers below that
#pragma unroll
    for (int off = 16; off >= EPL; off >>= 1) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) v[j] = __fadd_rn(v[j], __shfl_xor_sync(kFull, v[j], off / EPL));
    }
#pragma unroll
    for (int off = EPL / 2; off >= 1; off >>= 1) {
#pragma unroll
      for (int j = 0; j < EPL / 2; ++j)
        if (j < off) v[j] = __fadd_rn(v[j], v[j + off]);
    }
    const float rs = __frcp_rn(__shfl_sync(kFull, v[0], 31));  // correctly rounded: the bits of 1.0f / sum
#pragma unroll
    for (int j = 0; j < EPL; ++j) sc[j] = __fmul_rn(sc[j], rs);
  } else {
#pragma unroll
    for (int j = 0; j < EPL; ++j) sc[j] = __frcp_rn(__fadd_rn(1.0f, exp_ieee(-z[j])));
  }
  uint32_t ok[EPL];  // ordered images of the selection keys; 0 = not eligible
  if (a.select_bias != nullptr) {
    if (EPL == 2) {
      const float2 b = __ldg(reinterpret_cast<const float2*>(a.select_bias) + lane);
      ok[0] = ord_key(__fadd_rn(sc[0], b.x));
      ok[1] = ord_key(__fadd_rn(sc[1], b.y));
    } else {
#pragma unroll
      for (int v4 = 0; v4 < EPL / 4; ++v4) {
        const float4 b = __ldg(reinterpret_cast<const float4*>(a.select_bias) + (EPL / 4) * lane + v4);
        ok[4 * v4] = ord_key(__fadd_rn(sc[4 * v4], b.x));
        ok[4 * v4 + 1] = ord_key(__fadd_rn(sc[4 * v4 + 1], b.y));
        ok[4 * v4 + 2] = ord_key(__fadd_rn(sc[4 * v4 + 2], b.z));
        ok[4 * v4 + 3] = ord_key(__fadd_rn(sc[4 * v4 + 3], b.w));
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < EPL; ++j) ok[j] = ord_key(sc[j]);
  }

  // ---- slices: runs of `lps` lanes; each notes its two largest keys (equal keys count separately)
  int lps, q;
  if (a.n_groups > 1) {
    lps = (a.E / a.n_groups) / EPL;
    q = (a.K + a.topk_groups - 1) / a.topk_groups;
  } else {
    int s = 1;
    while (2 * s < a.K) s <<= 1;  // slices: the power of two >= K/2 (K <= 32), two keys from each
    lps = 32 / s;
    q = 2;
  }
  uint32_t m1 = 0u, m2 = 0u;
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    m2 = max(m2, min(m1, ok[j]));
    m1 = max(m1, ok[j]);
  }
  for (int d = 1; d < lps; d <<= 1) {
    const uint32_t o1 = __shfl_xor_sync(kFull, m1, d);
    const uint32_t o2 = __shfl_xor_sync(kFull, m2, d);
    m2 = max(min(m1, o1), max(m2, o2));
    m1 = max(m1, o1);
  }
  bool kept = true;
  if (a.n_groups > 1) {
    // group score = sum of its group_topk <= 2 largest keys; a group is kept when fewer than
    // topk_groups groups beat it (larger score, or equal score and lower index)
    float gsc = ord_value(m1);
    if (a.group_topk == 2) gsc = __fadd_rn(gsc, ord_value(m2));
    const int g = lane / lps;
    int rank = 0;
    for (int o = 0; o < a.n_groups; ++o) {
      const float og = __shfl_sync(kFull, gsc, o * lps);
      if (og > gsc || (og == gsc && o < g)) ++rank;
    }
    kept = rank < a.topk_groups;
    if (!kept) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) ok[j] = 0u;
    }
  }

  float tot = 0.0f, myu = 0.0f;
  mysel = 0;
  bool done = false;
  if (q <= 2) {
    // ---- threshold, short list, rank
    const uint32_t tq = q == 1 ? m1 : m2;
    // (tau >= 1, so that a key that reaches it is eligible; a slice with fewer than q eligible keys
    // gives tau = 1: every eligible key is listed, or the rounds decide)
    const uint32_t tau = max(__reduce_min_sync(kFull, kept ? tq : 0xffffffffu), 1u);
    int n = 0;
#pragma unroll
    for (int j = 0; j < EPL; ++j) n += ok[j] >= tau ? 1 : 0;
    int incl = n;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(kFull, incl, d);
      if (lane >= d) incl += up;
    }
    const int total = __shfl_sync(kFull, incl, 31);
    if (total <= 32 && total >= a.K) {
      uint32_t* s_k = s_cand;                                      // [32] listed keys, in expert order
      int* s_e = reinterpret_cast<int*>(s_cand + 32);              // [32] their experts
      float* s_v = reinterpret_cast<float*>(s_cand + 64);          // [32] their unbiased scores
      int* s_sel = reinterpret_cast<int*>(s_cand + 96);            // [K] slots
      float* s_u = reinterpret_cast<float*>(s_cand + 96 + kMaxK);  // [K]
      __syncwarp();  // the previous token's readers are done
      int pos = incl - n;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        if (ok[j] >= tau) {
          s_k[pos] = ok[j];
          s_e[pos] = EPL * lane + j;
          s_v[pos] = sc[j];
          ++pos;
        }
      }
      if (lane >= total) s_k[lane] = 0u;  // padding: beats nothing
      __syncwarp();
      // lane c takes listed key c and counts the listed keys that beat it: the larger ones (four
      // keys per shared-memory load), plus the equal ones listed earlier - the list is in expert
      // order, so those are the lower expert indices
      const uint32_t k = s_k[lane];
      int rank = 0;
      const uint4* k4 = reinterpret_cast<const uint4*>(s_k);
      for (int c4 = 0; c4 < (total + 3) >> 2; ++c4) {
        const uint4 o = k4[c4];
        rank += (o.x > k ? 1 : 0) + (o.y > k ? 1 : 0) + (o.z > k ? 1 : 0) + (o.w > k ? 1 : 0);
      }
      rank += __popc(__match_any_sync(kFull, k) & ((1u << lane) - 1u));
      if (lane < total && rank < a.K) {
        s_sel[rank] = s_e[lane];
        s_u[rank] = a.weight_from_key ? ord_value(k) : s_v[lane];
      }
      __syncwarp();
      if (lane < a.K) {
        mysel = s_sel[lane];
        myu = s_u[lane];
      }
      for (int kk = 0; kk < a.K; ++kk) tot = __fadd_rn(tot, __shfl_sync(kFull, myu, kk));
      done = true;
    }
  }
  if (!done) select_by_rounds_c<EPL>(a, ok, sc, lane, mysel, myu, tot);
  const float wv = a.renorm ? __fdiv_rn(myu, fmaxf(tot, a.norm_min)) : myu;
  myw = __fmul_rn(wv, a.routed_scale);
}

}  // namespace moe_rd
