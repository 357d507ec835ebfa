/*
 * CPU oracle for MoE sparse routing and dispatch.  TEST INFRASTRUCTURE ONLY:
 * the parity tests, the smoke check and the CPU-baseline leg of the benchmark
 * link this file; no product code path may call it.
 *
 * PARITY UNPINNED: the reference project ships no tests, golden vectors or
 * runnable CPU implementation of this path (its PyTorch reference is not
 * redistributed), so this file is a restatement of the algorithm read from the
 * reference's CUDA source, extended with the routing modes the target configs
 * add.  Every function cites the reference lines it follows.  Citations are
 * relative to sol-execbench/029_moe_sparse_routing_and_dispatch/ of
 * ernie-research/ERNIE-Evolve-Results.
 *
 * The arithmetic is specified down to the order of every fp32 operation so a
 * GPU implementation that follows the same order produces identical bits:
 * only IEEE-754 single operations (add, mul, div, fma, max, round-to-int) are
 * used, never libm transcendentals.  Build with -ffp-contract=off.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* ------------------------------------------------------------------------
 * Gate logits z[t,e] = sum_h x[t,h] * W[h,e]  (+ logit_bias[e]).
 *
 * The reference computes this product with a library GEMM whose summation
 * order is unspecified (kernel.cu:4327-4339) and recovers fp32-weight accuracy
 * by a hi/lo bf16 split (kernel.cu:1816-1822, 1849-1851).  Here the order is
 * fixed ("32 lanes x 2 chains"): chain (l, p), l = 0..31, p = 0..1,
 * accumulates by fused multiply-add, from 0, the elements
 * h = 256*c + 8*l + 2*m + p for c = 0,1,.. and m = 0..3 in increasing (c, m);
 * lane l's value is chain(l,0) + chain(l,1); the 32 lane values are then summed
 * by the binary tree v[l] += v[l+off] for off = 16, 8, 4, 2, 1.  (Two chains
 * per lane are what a packed two-wide fp32 FMA over a bf16 pair computes.)
 *
 * w_dtype: 0 = fp32, 1 = bf16.  w_layout: 0 = [H,E] row-major, 1 = [E,H].
 * ---------------------------------------------------------------------- */
void moe_oracle_logits(const uint16_t* x, const void* w, int w_dtype,
                       int w_layout, const float* logit_bias, int64_t T, int H,
                       int E, float* z) {
  float* wf = (float*)malloc((size_t)H * E * sizeof(float));
  for (int h = 0; h < H; ++h)
    for (int e = 0; e < E; ++e) {
      size_t src = w_layout == 0 ? (size_t)h * E + e : (size_t)e * H + h;
      wf[(size_t)h * E + e] = w_dtype == 0 ? ((const float*)w)[src]
                                           : bf16_to_f32(((const uint16_t*)w)[src]);
    }
  const int nchunk = (H + 255) / 256;
#pragma omp parallel
  {
    float* acc = (float*)malloc((size_t)64 * E * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t t = 0; t < T; ++t) {
      memset(acc, 0, (size_t)64 * E * sizeof(float));
      const uint16_t* xr = x + (size_t)t * H;
      for (int c = 0; c < nchunk; ++c)
        for (int l = 0; l < 32; ++l) {
          const int h0 = c * 256 + l * 8;
          if (h0 >= H) break;
          for (int j = 0; j < 8; ++j) {
            float* a = acc + ((size_t)l * 2 + (j & 1)) * E; /* chain (l, j&1) */
            const float xv = bf16_to_f32(xr[h0 + j]);
            const float* wr = wf + (size_t)(h0 + j) * E;
            for (int e = 0; e < E; ++e) a[e] = fmaf(xv, wr[e], a[e]);
          }
        }
      for (int l = 0; l < 32; ++l) { /* lane value = even chain + odd chain, kept in slot l */
        const float* a0 = acc + ((size_t)l * 2) * E;
        const float* a1 = a0 + E;
        float* d = acc + (size_t)l * E;
        for (int e = 0; e < E; ++e) d[e] = a0[e] + a1[e];
      }
      for (int off = 16; off; off >>= 1)
        for (int l = 0; l < off; ++l) {
          float* a = acc + (size_t)l * E;
          const float* b = acc + (size_t)(l + off) * E;
          for (int e = 0; e < E; ++e) a[e] = a[e] + b[e];
        }
      float* zr = z + (size_t)t * E;
      if (logit_bias)
        for (int e = 0; e < E; ++e) zr[e] = acc[e] + logit_bias[e];
      else
        for (int e = 0; e < E; ++e) zr[e] = acc[e];
    }
    free(acc);
  }
  free(wf);
}

/* The same product in double precision, rounded once: the yardstick for the
 * tolerance check of a tensor-core gate product whose order cannot be fixed. */
void moe_oracle_logits_f64(const uint16_t* x, const void* w, int w_dtype,
                           int w_layout, const float* logit_bias, int64_t T,
                           int H, int E, double* z) {
  double* wd = (double*)malloc((size_t)H * E * sizeof(double));
  for (int h = 0; h < H; ++h)
    for (int e = 0; e < E; ++e) {
      size_t src = w_layout == 0 ? (size_t)h * E + e : (size_t)e * H + h;
      wd[(size_t)h * E + e] = w_dtype == 0
                                  ? (double)((const float*)w)[src]
                                  : (double)bf16_to_f32(((const uint16_t*)w)[src]);
    }
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < T; ++t) {
    double* zr = z + (size_t)t * E;
    for (int e = 0; e < E; ++e) zr[e] = 0.0;
    for (int h = 0; h < H; ++h) {
      const double xv = (double)bf16_to_f32(x[(size_t)t * H + h]);
      const double* wr = wd + (size_t)h * E;
      for (int e = 0; e < E; ++e) zr[e] += xv * wr[e];
    }
    if (logit_bias)
      for (int e = 0; e < E; ++e) zr[e] += (double)logit_bias[e];
  }
  free(wd);
}

/* exp(x) from IEEE operations only: n = rint(x*log2(e)); r = x - n*ln2 in two
 * fused steps; degree-6 polynomial; scale by 2^n through the exponent field.
 * Flushes to 0 below -87 and returns +inf above 88.  About 1 ulp. */
float moe_oracle_expf(float x) {
  if (x < -87.0f) return 0.0f;
  if (x > 88.0f) return INFINITY;
  const float n = rintf(x * 1.44269504f);
  float r = fmaf(n, -0.693145752f, x);
  r = fmaf(n, -1.42860677e-6f, r);
  float p = 1.9875691500e-4f;
  p = fmaf(p, r, 1.3981999507e-3f);
  p = fmaf(p, r, 8.3334519073e-3f);
  p = fmaf(p, r, 4.1665795894e-2f);
  p = fmaf(p, r, 1.6666665459e-1f);
  p = fmaf(p, r, 5.0000001201e-1f);
  const float r2 = r * r;
  float y = fmaf(p, r2, r);
  y = y + 1.0f;
  const uint32_t sb = (uint32_t)((int)n + 127) << 23;
  float s;
  memcpy(&s, &sb, 4);
  return y * s;
}

/* ------------------------------------------------------------------------
 * Scoring, group-limited top-K and combine weights for one batch of logits.
 *
 * Follows topk_kernel (kernel.cu:1829-1920): softmax as max, exp, sum,
 * reciprocal-then-multiply (1857-1866); bias added to the score to form the
 * selection key (1865-1866); K rounds of arg-max where the lowest expert
 * index wins ties (1886) and slot k holds the k-th pick (1892-1895); weights
 * w = u / max(sum u, norm_min) (1891, 1909).
 *
 * The softmax sum order is fixed: partial l (0..31) adds p[l], p[l+32], ... in
 * increasing index from 0, then the same binary tree as the logits.
 *
 * score_fn: 0 softmax, 1 sigmoid = 1/(1+exp(-z)).
 * weight_from_key: 1 reproduces the reference (weights use the biased key);
 *   0 uses the unbiased score (bias steers selection only).
 * n_groups > 1: experts [g*E/G, (g+1)*E/G) form group g; its score is the sum
 *   of its group_topk largest keys (added in descending order); only the
 *   topk_groups best groups (lowest index on ties) stay eligible.
 * Returns 0, or -1 on invalid parameters.
 * ---------------------------------------------------------------------- */
int moe_oracle_route(const float* z, const float* select_bias, int64_t T,
                     int E, int K, int score_fn, int n_groups, int topk_groups,
                     int group_topk, int weight_from_key, int renorm,
                     float routed_scale, float norm_min, int32_t* ids,
                     float* wts) {
  if (E < 1 || K < 1 || K > E) return -1;
  if (n_groups < 1) n_groups = 1;
  if (E % n_groups) return -1;
  const int gs = E / n_groups;
  if (n_groups > 1 &&
      (topk_groups < 1 || topk_groups > n_groups || group_topk < 1 ||
       group_topk > gs || K > topk_groups * gs))
    return -1;
#pragma omp parallel
  {
    float* score = (float*)malloc((size_t)E * sizeof(float));
    float* key = (float*)malloc((size_t)E * sizeof(float));
    float* gsc = (float*)malloc((size_t)n_groups * sizeof(float));
    char* taken = (char*)malloc((size_t)E);
#pragma omp for schedule(static)
    for (int64_t t = 0; t < T; ++t) {
      const float* zr = z + (size_t)t * E;
      if (score_fn == 0) {
        float m = zr[0];
        for (int e = 1; e < E; ++e) m = fmaxf(m, zr[e]);
        float part[32];
        for (int l = 0; l < 32; ++l) part[l] = 0.0f;
        for (int e = 0; e < E; ++e) {
          score[e] = moe_oracle_expf(zr[e] - m);
          part[e & 31] = part[e & 31] + score[e];
        }
        for (int off = 16; off; off >>= 1)
          for (int l = 0; l < off; ++l) part[l] = part[l] + part[l + off];
        const float rs = 1.0f / part[0];
        for (int e = 0; e < E; ++e) score[e] = score[e] * rs;
      } else {
        for (int e = 0; e < E; ++e)
          score[e] = 1.0f / (1.0f + moe_oracle_expf(-zr[e]));
      }
      for (int e = 0; e < E; ++e)
        key[e] = select_bias ? score[e] + select_bias[e] : score[e];
      memset(taken, 0, (size_t)E);
      if (n_groups > 1) {
        for (int g = 0; g < n_groups; ++g) {
          float sum = 0.0f;
          for (int r = 0; r < group_topk; ++r) {
            int bi = -1;
            float bv = 0.0f;
            for (int e = g * gs; e < (g + 1) * gs; ++e)
              if (!taken[e] && (bi < 0 || key[e] > bv)) {
                bi = e;
                bv = key[e];
              }
            if (bi < 0) break;
            taken[bi] = 1;
            sum = r == 0 ? bv : sum + bv;
          }
          gsc[g] = sum;
        }
        memset(taken, 0, (size_t)E);
        for (int g = 0; g < n_groups; ++g) {
          int rank = 0;
          for (int o = 0; o < n_groups; ++o)
            if (gsc[o] > gsc[g] || (gsc[o] == gsc[g] && o < g)) ++rank;
          if (rank >= topk_groups)
            for (int e = g * gs; e < (g + 1) * gs; ++e) taken[e] = 1;
        }
      }
      float u[64];
      float* uk = K <= 64 ? u : (float*)malloc((size_t)K * sizeof(float));
      float tot = 0.0f;
      for (int k = 0; k < K; ++k) {
        int bi = -1;
        float bv = 0.0f;
        for (int e = 0; e < E; ++e)
          if (!taken[e] && (bi < 0 || key[e] > bv)) {
            bi = e;
            bv = key[e];
          }
        if (bi < 0) bi = 0; /* unreachable: K <= eligible experts is validated */
        taken[bi] = 1;
        ids[(size_t)t * K + k] = bi;
        uk[k] = weight_from_key ? key[bi] : score[bi];
        tot = tot + uk[k];
      }
      for (int k = 0; k < K; ++k) {
        float wv = renorm ? uk[k] / fmaxf(tot, norm_min) : uk[k];
        wts[(size_t)t * K + k] = wv * routed_scale;
      }
      if (uk != u) free(uk);
    }
    free(score);
    free(key);
    free(gsc);
    free(taken);
  }
  return 0;
}

/* ------------------------------------------------------------------------
 * Counts, offsets, slot order and drops.
 *
 * offsets[] follows the scan in offsets_kernel (kernel.cu:2074-2086), stored
 * as E+1 exclusive starts with a leading 0 (the reference keeps inclusive ends
 * `offs` and exclusive starts `cursor`).  inverse_perm[s] is the destination
 * row of pair s = t*K+k, the meaning of `inv` in dispatch_body
 * (kernel.cu:2172-2177) as consumed by combine_kernel (2377-2383).  Unlike the
 * reference, whose order inside an expert depends on atomics (2155-2158), the
 * order is stable: a pair's rank is the number of earlier pairs (smaller s)
 * routed to the same expert.  capacity > 0 keeps only ranks < capacity;
 * dropped pairs get inverse_perm = -1 and drop_mask = 1.
 * ---------------------------------------------------------------------- */
void moe_oracle_dispatch(const int32_t* ids, int64_t T, int K, int E,
                         int64_t capacity, int32_t* counts, int32_t* offsets,
                         int32_t* inverse_perm, uint8_t* drop_mask) {
  const int64_t P = T * K;
  int64_t* cnt = (int64_t*)calloc((size_t)E, sizeof(int64_t));
  int32_t* rank = (int32_t*)malloc((size_t)(P > 0 ? P : 1) * sizeof(int32_t));
  for (int64_t s = 0; s < P; ++s) rank[s] = (int32_t)cnt[ids[s]]++;
  offsets[0] = 0;
  for (int e = 0; e < E; ++e) {
    const int64_t kept = capacity > 0 && cnt[e] > capacity ? capacity : cnt[e];
    if (counts) counts[e] = (int32_t)cnt[e];
    offsets[e + 1] = offsets[e] + (int32_t)kept;
  }
  for (int64_t s = 0; s < P; ++s) {
    const int dropped = capacity > 0 && rank[s] >= capacity;
    inverse_perm[s] = dropped ? -1 : offsets[ids[s]] + rank[s];
    if (drop_mask) drop_mask[s] = (uint8_t)dropped;
  }
  free(cnt);
  free(rank);
}

/* Row copy xg[pos,:] = x[t,:] (gather_body, kernel.cu:2223-2228), bit for bit. */
void moe_oracle_permute_bf16(const uint16_t* x, const int32_t* inverse_perm,
                             int64_t T, int K, int H, uint16_t* rows) {
#pragma omp parallel for schedule(static)
  for (int64_t s = 0; s < T * K; ++s) {
    const int32_t pos = inverse_perm[s];
    if (pos < 0) continue;
    memcpy(rows + (size_t)pos * H, x + (size_t)(s / K) * H, (size_t)H * 2);
  }
}

/* float -> fp8 e4m3 (finite-only format), round to nearest even, saturating
 * to +-448; NaN -> 0x7f. */
uint8_t moe_oracle_f32_to_e4m3(float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  const uint8_t sign = (uint8_t)((u >> 24) & 0x80);
  u &= 0x7fffffffu;
  if (u > 0x7f800000u) return (uint8_t)(sign | 0x7f);
  float a;
  memcpy(&a, &u, 4);
  if (a > 448.0f) return (uint8_t)(sign | 0x7e);
  if (a < 0.015625f) /* below 2^-6: subnormal grid of 2^-9 */
    return (uint8_t)(sign | (uint8_t)rintf(a * 512.0f));
  u += 0x7ffffu + ((u >> 20) & 1u);
  u >>= 20;
  u -= (127u - 7u) << 3;
  if (u > 0x7eu) u = 0x7eu;
  return (uint8_t)(sign | (uint8_t)u);
}

float moe_oracle_e4m3_to_f32(uint8_t b) {
  const int e = (b >> 3) & 15, m = b & 7;
  float v;
  if (e == 15 && m == 7)
    v = NAN;
  else if (e == 0)
    v = ldexpf((float)m, -9);
  else
    v = ldexpf((float)(8 + m), e - 10);
  return (b & 0x80) ? -v : v;
}

/* ------------------------------------------------------------------------
 * Row copy with fused fp8 quantisation, one fp32 scale per 128 elements.
 * Convention of the reference's per-row int8 quantiser xquant_body
 * (kernel.cu:2573-2591; moe_wq.h:146-169) with QMAX = 448:
 *   scale = max(amax, 1e-30) * (1/448);  inv = 1/scale;  q = rne(x*inv).
 * ---------------------------------------------------------------------- */
void moe_oracle_permute_fp8(const uint16_t* x, const int32_t* inverse_perm,
                            int64_t T, int K, int H, uint8_t* rows,
                            float* scales) {
  const int nb = H / 128;
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < T; ++t) {
    int any = 0;
    for (int k = 0; k < K; ++k) any |= inverse_perm[(size_t)t * K + k] >= 0;
    if (!any) continue;
    uint8_t* q = (uint8_t*)malloc((size_t)H);
    float* sc = (float*)malloc((size_t)nb * sizeof(float));
    const uint16_t* xr = x + (size_t)t * H;
    for (int b = 0; b < nb; ++b) {
      float am = 0.0f;
      for (int i = 0; i < 128; ++i)
        am = fmaxf(am, fabsf(bf16_to_f32(xr[b * 128 + i])));
      const float s = fmaxf(am, 1e-30f) * (1.0f / 448.0f);
      const float inv = 1.0f / s;
      sc[b] = s;
      for (int i = 0; i < 128; ++i)
        q[b * 128 + i] = moe_oracle_f32_to_e4m3(bf16_to_f32(xr[b * 128 + i]) * inv);
    }
    for (int k = 0; k < K; ++k) {
      const int32_t pos = inverse_perm[(size_t)t * K + k];
      if (pos < 0) continue;
      memcpy(rows + (size_t)pos * H, q, (size_t)H);
      memcpy(scales + (size_t)pos * nb, sc, (size_t)nb * sizeof(float));
    }
    free(q);
    free(sc);
  }
}

/* float -> bf16, round to nearest even (finite inputs). */
static inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* ------------------------------------------------------------------------
 * Weighted combine (un-permute): out[t,:] = shared[t,:] + sum_k w[t,k] * y[inverse_perm[t,k],:]
 * Follows combine_kernel (kernel.cu:2365-2428): fp32 accumulator starting from
 * the shared-expert row (or 0), slots added in order k = 0..K-1 by one fused
 * multiply-add each (the reference's `acc += w * y` contracts to an FMA under
 * nvcc's default -fmad=true), rounded once to bf16 at the end.  Dropped pairs
 * (inverse_perm < 0) contribute nothing.
 * ---------------------------------------------------------------------- */
void moe_oracle_combine(const uint16_t* y, const int32_t* inverse_perm, const float* weights,
                        const uint16_t* shared, int64_t T, int K, int H, uint16_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < T; ++t) {
    for (int h = 0; h < H; ++h) {
      float acc = shared ? bf16_to_f32(shared[(size_t)t * H + h]) : 0.0f;
      for (int k = 0; k < K; ++k) {
        const int32_t pos = inverse_perm[(size_t)t * K + k];
        if (pos < 0) continue;
        acc = fmaf(weights[(size_t)t * K + k], bf16_to_f32(y[(size_t)pos * H + h]), acc);
      }
      out[(size_t)t * H + h] = f32_to_bf16_rne(acc);
    }
  }
}

/* ------------------------------------------------------------------------
 * Residual (accumulating) combine over expert-major rows, raddleft_kernel
 * (kernel.cu:2451-2486): out[tok[p],:] += bf16(w[p] * y[p,:]) for p < n_rows,
 * rows taken in ascending p.  The product is an fp32 multiply rounded to bf16
 * (kernel.cu:2466-2467); the add is one bf16 addition with a single rounding
 * (red.global.add.noftz.bf16x2, kernel.cu:2446-2449), computed here in double,
 * where the sum of two bf16 values cannot be rounded twice to a different bf16.
 * The GPU adds rows of one token in no fixed order: this is the result for ONE
 * order, exact for the GPU only when a token has at most one row.
 * ---------------------------------------------------------------------- */
static inline uint16_t f64_to_bf16_rne(double d) {
  /* double -> fp32 with round-to-odd (truncate toward zero, inexact sets the last bit), then the
   * usual round-to-nearest-even to bf16: with 16 spare bits the two steps equal one rounding */
  float f = (float)d;
  if ((double)f != d && f == f) {
    uint32_t u;
    const double fa = f < 0 ? -(double)f : (double)f, da = d < 0 ? -d : d;
    memcpy(&u, &f, 4);
    if (fa > da) u -= 1u; /* one step toward zero (sign-magnitude encoding) */
    u |= 1u;
    memcpy(&f, &u, 4);
  }
  return f32_to_bf16_rne(f);
}

void moe_oracle_combine_add_rows(const uint16_t* y, const int32_t* row_token, const float* row_weight,
                                 int64_t n_rows, int H, uint16_t* out) {
  for (int64_t p = 0; p < n_rows; ++p) {
    const int32_t t = row_token[p];
    if (t < 0) continue;
    const float w = row_weight[p];
    for (int h = 0; h < H; ++h) {
      const float prod = w * bf16_to_f32(y[(size_t)p * H + h]);
      const double term = (double)bf16_to_f32(f32_to_bf16_rne(prod));
      uint16_t* o = out + (size_t)t * H + h;
      *o = f64_to_bf16_rne((double)bf16_to_f32(*o) + term);
    }
  }
}

int moe_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void moe_oracle_set_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}
