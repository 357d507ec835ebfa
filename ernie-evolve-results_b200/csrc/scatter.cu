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
// the capacity get inverse_perm = -1 and are not written.  positions_kernel
// derives rank_in_tile from the ids (replacing the atomic ranks of the
// reference's dispatch_body, kernel.cu:2155-2158, by a stable count) and
// writes inverse_perm / drop_mask; scatter_kernel is then a
// pure streaming kernel whose work units (a 2 KB slice of a bf16 row, or 512
// elements = four scale blocks of an fp8 row) are dealt to warps grid-stride,
// so the load is even whatever T, H and K are.
//
// fp8 rows follow the reference's per-row int8 quantiser convention
// (xquant_body, kernel.cu:2573-2591) applied per 128 elements with QMAX = 448:
// scale = max(amax, 1e-30) * (1/448), inv = 1/scale, q = rne_satfinite(x*inv).
#include <cuda_fp8.h>

#include "common.cuh"

namespace moe_rd {
namespace {

// Tuning constants of the streaming scatter (defaults are the measured best).
#ifndef MOE_RD_SC_THREADS
#define MOE_RD_SC_THREADS 256
#endif
#ifndef MOE_RD_SC_UNIT_VECS   // 16-byte loads per lane and bf16 work unit
#define MOE_RD_SC_UNIT_VECS 4
#endif
#ifndef MOE_RD_SC_BLOCKS_PER_SM
#define MOE_RD_SC_BLOCKS_PER_SM 64  // far more blocks than fit: late blocks fill the gaps
#endif
#ifndef MOE_RD_SC_PREFETCH_UNITS   // work units per warp whose x is requested before the grid dependency wait
#define MOE_RD_SC_PREFETCH_UNITS 2
#endif
#ifndef MOE_RD_SC_FP8_LANE_ELEMS   // elements a lane quantises per work unit of an fp8 row: 16 or 32
#define MOE_RD_SC_FP8_LANE_ELEMS 16
#endif
#ifndef MOE_RD_SC_VECTOR_SCALES   // 1: the four scales of an fp8 work unit leave in one 16-byte store
#define MOE_RD_SC_VECTOR_SCALES 0
#endif
#ifndef MOE_RD_SC_STREAMING   // 1: st.global.cs (evict-first) for the row stores
#define MOE_RD_SC_STREAMING 1
#endif
constexpr int kScatterThreads = MOE_RD_SC_THREADS;
constexpr int kScatterWarps = kScatterThreads / 32;
constexpr int kUV = MOE_RD_SC_UNIT_VECS;

__device__ __forceinline__ void store_row16(uint4* p, const uint4& v) {
#if MOE_RD_SC_STREAMING
  __stcs(p, v);
#else
  *p = v;
#endif
}

struct PositionArgs {
  const int32_t* ids;
  const int32_t* tile_base;  // scanned mode: [E][ntiles] tile bases; tile mode: [ntiles][E] raw counts
  const int32_t* group_counts;  // tile mode: [groups][E] pairs per expert and group of kTileGroup tiles
  int32_t* offsets;          // [E+1]: read (scanned mode) or written by block 0 (tile mode)
  int32_t* inverse_perm;
  uint8_t* drop_mask;
  int32_t* status;
  const float* weights;      // [T,K] combine weights (read for row_weight)
  int32_t* row_token;        // [out_rows] or null
  float* row_weight;         // [out_rows] or null
  const int32_t* counts;     // scanned mode: [E] pairs per expert before dropping
  int32_t* user_counts;      // tile mode: [E] output of the same, or null
  int32_t* dense;            // [1+kMaxK] identity experts: number, first rows (or null)
  int64_t T, capacity, out_rows;
  int E, K, ntiles;
};

constexpr int kPosThreads = 256;
static_assert(kMaxE <= kPosThreads, "tile mode keeps one expert per thread");

// One block per tile of kTile tokens.  The rank of a pair inside its tile and
// expert is the number of earlier pairs (flat index t*K+k) of the tile with the
// same expert: every 32 consecutive pairs are counted with __match_any_sync and
// the per-chunk counts are prefix-summed per expert in pair order.
//
// Scanned mode (after the fused GEMV kernel, whose last block scanned the counts):
// tile_base [E][ntiles] and offsets are read as they are.
// TILE (after the routing kernel of route.cu): there is no scan; the block
// derives what it needs from the raw counts itself, thread e for expert e, with
// coalesced loads that are all in flight at once: the expert's total (sum of its
// group counts), the pairs in the tiles before this one (group counts of the
// groups before, plus the tile counts of this group's earlier tiles), and, by a
// block-wide scan over the experts, offsets[e] = rows kept by the experts
// before e (the scan part of offsets_kernel of the reference, kernel.cu:2074-2086).
// Block 0 writes offsets[E+1] and the per-expert counts out.
template <bool TILE>
__global__ void __launch_bounds__(kPosThreads) positions_kernel(const PositionArgs a) {
  extern __shared__ __align__(16) uint16_t s_cc[];  // [chunks][E]
  __shared__ int s_off[TILE ? kMaxE : 1], s_tb[TILE ? kMaxE : 1], s_tot[TILE ? kMaxE : 1], s_w[kPosThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int nwarps = kPosThreads / 32;
  constexpr int kRegChunks = 2;  // chunks per warp whose loads stay in registers (all of them for K <= 8)
  const int tile = blockIdx.x;
  const int64_t t0 = (int64_t)tile * kTile;
  const int ntok = (int)min((int64_t)kTile, a.T - t0);
  const int P = ntok * a.K;
  const int nch = (P + 31) >> 5;
  const int32_t* ids = a.ids + (size_t)t0 * a.K;
  {
    // independent of the kernels before: done while they finish
    uint32_t* z32 = reinterpret_cast<uint32_t*>(s_cc);
    const int nw = (nch * a.E + 1) >> 1;
    for (int i = tid; i < nw; i += kPosThreads) z32[i] = 0u;
  }
  pdl_trigger();
  pdl_wait();
  int e_reg[kRegChunks], tb_reg[kRegChunks], off_reg[kRegChunks];
#pragma unroll
  for (int k = 0; k < kRegChunks; ++k) {
    const int p = (warp + k * nwarps) * 32 + lane;
    const int e = p < P ? ids[p] : -1;
    e_reg[k] = e;
    tb_reg[k] = 0;
    off_reg[k] = 0;
    if (!TILE && e >= 0 && e < a.E) {
      // scanned mode: every load is issued up front
      tb_reg[k] = a.tile_base[(size_t)e * a.ntiles + tile];
      off_reg[k] = a.offsets[e];
    }
  }
  if (TILE) {
    // kMaxE <= kPosThreads: one expert per thread
    const int e = tid;
    int total = 0, base = 0;
    if (e < a.E) {
      const int ngroups = (a.ntiles + kTileGroup - 1) / kTileGroup;
      const int g0 = tile / kTileGroup;
      // the earlier tiles of this group: all loads are issued before the first add
      int tv[kTileGroup - 1];
      const int32_t* tc = a.tile_base + (size_t)g0 * kTileGroup * a.E + e;
      const int nt = tile - g0 * kTileGroup;
#pragma unroll
      for (int j = 0; j < kTileGroup - 1; ++j) tv[j] = j < nt ? tc[(size_t)j * a.E] : 0;
      for (int gb = 0; gb < ngroups; gb += 8) {
        int gv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) gv[j] = gb + j < ngroups ? a.group_counts[(size_t)(gb + j) * a.E + e] : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          total += gv[j];
          if (gb + j < g0) base += gv[j];
        }
      }
#pragma unroll
      for (int j = 0; j < kTileGroup - 1; ++j) base += tv[j];
    }
    int kept = total;
    if (a.capacity > 0 && (int64_t)kept > a.capacity) kept = (int)a.capacity;
    int incl = kept;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(kFull, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) s_w[warp] = incl;
    __syncthreads();
    int before = 0, all = 0;
#pragma unroll
    for (int w = 0; w < nwarps; ++w) {
      const int v = s_w[w];
      if (w < warp) before += v;
      all += v;
    }
    const int off = before + incl - kept;
    if (e < a.E) {
      s_off[e] = off;
      s_tb[e] = base;
      s_tot[e] = total;
      if (tile == 0) {
        a.offsets[e] = off;
        if (a.user_counts != nullptr) a.user_counts[e] = total;
      }
    }
    if (tile == 0 && tid == 0) a.offsets[a.E] = all;
  }
  __syncthreads();
  for (int c = warp, k = 0; c < nch; c += nwarps, ++k) {
    const int p = c * 32 + lane;
    int e = -1;
    if (k < kRegChunks) {
#pragma unroll
      for (int kk = 0; kk < kRegChunks; ++kk)
        if (kk == k) e = e_reg[kk];
    } else {
      e = p < P ? ids[p] : -1;
    }
    if (e >= a.E) e = -1;
    const unsigned m = __match_any_sync(kFull, e);
    if (e >= 0 && (m & ((1u << lane) - 1u)) == 0u) s_cc[c * a.E + e] = (uint16_t)__popc(m);
  }
  __syncthreads();
  for (int e = tid; e < a.E; e += kPosThreads) {
    int run = 0;
    for (int c = 0; c < nch; ++c) {
      const int v = s_cc[c * a.E + e];
      s_cc[c * a.E + e] = (uint16_t)run;
      run += v;
    }
  }
  __syncthreads();
  for (int c = warp, k = 0; c < nch; c += nwarps, ++k) {
    const int p = c * 32 + lane;
    int e_raw = -1, tb = 0, off = 0;
    if (k < kRegChunks) {
#pragma unroll
      for (int kk = 0; kk < kRegChunks; ++kk) {
        if (kk == k) {
          e_raw = e_reg[kk];
          tb = tb_reg[kk];
          off = off_reg[kk];
        }
      }
    } else {
      e_raw = p < P ? ids[p] : -1;
      if (!TILE && e_raw >= 0 && e_raw < a.E) {
        tb = a.tile_base[(size_t)e_raw * a.ntiles + tile];
        off = a.offsets[e_raw];
      }
    }
    const int e = e_raw >= a.E ? -1 : e_raw;
    if (TILE && e >= 0) {
      tb = s_tb[e];
      off = s_off[e];
    }
    const unsigned m = __match_any_sync(kFull, e);
    if (p >= P) continue;
    const size_t s = (size_t)t0 * a.K + p;
    int pos = -1;
    bool dropped = false;
    if (e < 0) {
      report(a.status, 1, e_raw, (int)s);
    } else {
      const int64_t r = (int64_t)tb + s_cc[c * a.E + e] + __popc(m & ((1u << lane) - 1u));
      dropped = a.capacity > 0 && r >= a.capacity;
      if (!dropped) {
        const int64_t q = (int64_t)off + r;
        if (q < 0 || q >= a.out_rows)
          report(a.status, 2, (int)q, (int)s);
        else
          pos = (int)q;
      }
    }
    a.inverse_perm[s] = pos;
    if (a.drop_mask != nullptr) a.drop_mask[s] = dropped ? 1 : 0;
    if (pos >= 0) {
      if (a.row_token != nullptr) a.row_token[pos] = (int32_t)(t0 + p / a.K);
      if (a.row_weight != nullptr) a.row_weight[pos] = a.weights[s];
    }
  }
  // Identity experts (every token once, none dropped): their first rows, in
  // expert order, for the row scatter to skip.  At most K experts can qualify.
  if (a.dense != nullptr && tile == 0 && warp == 0) {
    int n = 0;
    for (int e0 = 0; e0 < a.E; e0 += 32) {
      const int e = e0 + lane;
      const int cnt = e < a.E ? (TILE ? s_tot[e] : a.counts[e]) : 0;
      const bool is = e < a.E && (int64_t)cnt == a.T && (a.capacity == 0 || a.T <= a.capacity);
      const unsigned m = __ballot_sync(kFull, is);
      const int j = n + __popc(m & ((1u << lane) - 1u));
      if (is && j < kMaxK) a.dense[1 + j] = TILE ? s_off[e] : a.offsets[e];
      n += __popc(m);
    }
    if (lane == 0) a.dense[0] = n < kMaxK ? n : kMaxK;
  }
}

constexpr int kMaxWorld = 8;

struct ScatterArgs {
  const uint16_t* x;
  const int32_t* inverse_perm;
  void* rows;
  float* scales;
  int64_t T;
  int H, K;
  // expert-parallel destinations (EP == true): the row of pair (t,k) goes to
  // peer_rows[e / epr] at row dest_base[e] + (inverse_perm - offsets[e])
  const int32_t* ids;
  const int32_t* offsets;
  const int32_t* dest_base;
  void* peer_rows[kMaxWorld];
  float* peer_scales[kMaxWorld];
  int epr;
  const int32_t* dense;  // identity experts whose rows are not written (or null)
};

// Destination of pair (t,k): local row index, or (peer buffer, row) when EP.
template <bool EP>
__device__ __forceinline__ bool resolve_dest(const ScatterArgs& a, int64_t t, int k, int q,
                                             void*& rows, float*& scales, int64_t& row) {
  if (q < 0) return false;
  if (!EP) {
    if (a.dense != nullptr) {
      const int nd = __ldg(a.dense);
      for (int j = 0; j < nd; ++j)
        if ((uint32_t)(q - __ldg(a.dense + 1 + j)) < (uint32_t)a.T) return false;
    }
    rows = a.rows;
    scales = a.scales;
    row = q;
    return true;
  }
  const int e = __ldg(a.ids + (size_t)t * a.K + k);
  const int db = __ldg(a.dest_base + e);
  if (db < 0) return false;  // the expert's rows do not fit its owner's buffer (moe_rd_ep_plan reported it)
  const int d = e / a.epr;
  rows = a.peer_rows[d];
  scales = a.peer_scales[d];
  row = (int64_t)db + (q - __ldg(a.offsets + e));
  return true;
}

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

// Work units are numbered u = t * upr + c (row t, slice c).  A warp walks
// u = w, w + W, w + 2W, ...; (t, c) advance without a division.
struct UnitWalk {
  int64_t t;
  int c, dq, dr, upr;
  __device__ UnitWalk(int64_t first, int64_t stride, int units_per_row) {
    upr = units_per_row;
    t = first / upr;
    c = (int)(first - t * upr);
    dq = (int)(stride / upr);
    dr = (int)(stride - (int64_t)dq * upr);
  }
  __device__ void next() {
    t += dq;
    c += dr;
    if (c >= upr) {
      c -= upr;
      ++t;
    }
  }
};

template <int FMT, bool EP>
__global__ void __launch_bounds__(kScatterThreads) scatter_kernel(const ScatterArgs a) {
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int64_t w0 = (int64_t)blockIdx.x * kScatterWarps + (threadIdx.x >> 5);
  const int64_t W = (int64_t)gridDim.x * kScatterWarps;
  // The blocks of this grid become resident while the positions kernel is still
  // running.  x does not depend on it, so every warp asks L2 for the slices of x
  // it will read first and only then waits for the destinations.
  {
    const int upr = FMT == MOE_RD_ROWS_BF16 ? ((a.H >> 3) + 32 * kUV - 1) / (32 * kUV)
                                            : (a.H / MOE_RD_SC_FP8_LANE_ELEMS + 31) >> 5;
    const int unit_bytes = FMT == MOE_RD_ROWS_BF16 ? 512 * kUV : 64 * MOE_RD_SC_FP8_LANE_ELEMS;
    const int row_bytes = a.H * 2;
    UnitWalk pw(w0, W, upr);
    for (int n = 0; n < MOE_RD_SC_PREFETCH_UNITS && pw.t < a.T; ++n, pw.next()) {
      const int off = pw.c * unit_bytes + lane * 128;
      if (lane * 128 < unit_bytes && off < row_bytes)
        prefetch_l2(reinterpret_cast<const unsigned char*>(a.x) + (size_t)(a.T - 1 - pw.t) * row_bytes + off);
    }
  }
  pdl_wait();

  if (FMT == MOE_RD_ROWS_BF16) {
    // unit = 32*kUV uint4 (2 KB for kUV = 4) of a row: kUV 16-byte loads per lane
    const int nvec = a.H >> 3;
    const int upr = (nvec + 32 * kUV - 1) / (32 * kUV);
    const uint4* x4 = reinterpret_cast<const uint4*>(a.x);
    UnitWalk wk(w0, W, upr);
    for (; wk.t < a.T; wk.next()) {
      // Rows are taken last-first: the gate pass read x in ascending order just
      // before, so the tail of x is what is most likely still in L2.
      const int64_t t = a.T - 1 - wk.t;
      const uint4* src = x4 + (size_t)t * nvec;
      const int vb = wk.c * (32 * kUV) + lane;
      uint4 val[kUV];
#pragma unroll
      for (int u = 0; u < kUV; ++u)
        if (vb + 32 * u < nvec) val[u] = __ldg(src + vb + 32 * u);
      // the row's destinations are fetched while its loads are in flight
      int qv[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        qv[k] = k < a.K ? __ldg(a.inverse_perm + (size_t)t * a.K + k) : -1;
#pragma unroll 1
      for (int kb = 0; kb < a.K; kb += 8) {
        if (kb) {
#pragma unroll
          for (int k = 0; k < 8; ++k)
            qv[k] = kb + k < a.K ? __ldg(a.inverse_perm + (size_t)t * a.K + kb + k) : -1;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          void* rows;
          float* scl;
          int64_t q;
          if (!resolve_dest<EP>(a, t, kb + k, qv[k], rows, scl, q)) continue;
          uint4* d = reinterpret_cast<uint4*>(rows) + (size_t)q * nvec;
#pragma unroll
          for (int u = 0; u < kUV; ++u)
            if (vb + 32 * u < nvec) store_row16(d + vb + 32 * u, val[u]);
        }
      }
    }
  } else {
#if MOE_RD_SC_FP8_LANE_ELEMS == 32
    // unit = 1024 elements (eight 128-element scale blocks): 32 elements = four
    // 16-byte loads per lane, 4 lanes per scale block, two 16-byte stores per lane
    // and destination
    const int n32 = a.H >> 5;
    const int nb = a.H >> 7;
    const int upr = (n32 + 31) >> 5;
    const uint4* x4 = reinterpret_cast<const uint4*>(a.x);
    UnitWalk wk(w0, W, upr);
    for (; wk.t < a.T; wk.next()) {
      const int64_t t = a.T - 1 - wk.t;  // last rows first (see above)
      const int v = wk.c * 32 + lane;
      const bool act = v < n32;
      uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0, x2 = x0, x3 = x0;
      if (act) {
        const uint4* src = x4 + (size_t)t * (n32 * 4) + 4 * v;
        x0 = __ldg(src);
        x1 = __ldg(src + 1);
        x2 = __ldg(src + 2);
        x3 = __ldg(src + 3);
      }
      int qv[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        qv[k] = k < a.K ? __ldg(a.inverse_perm + (size_t)t * a.K + k) : -1;
      float am = fmaxf(fmaxf(amax8(x0), amax8(x1)), fmaxf(amax8(x2), amax8(x3)));
      am = fmaxf(am, __shfl_xor_sync(kFull, am, 2));
      am = fmaxf(am, __shfl_xor_sync(kFull, am, 1));
      const float scale = __fmul_rn(fmaxf(am, 1e-30f), 1.0f / 448.0f);
      const float inv = __frcp_rn(scale);  // correctly rounded: the bits of 1.0f / scale
      uint4 q0, q1;
      q0.x = quant4(x0.x, x0.y, inv);
      q0.y = quant4(x0.z, x0.w, inv);
      q0.z = quant4(x1.x, x1.y, inv);
      q0.w = quant4(x1.z, x1.w, inv);
      q1.x = quant4(x2.x, x2.y, inv);
      q1.y = quant4(x2.z, x2.w, inv);
      q1.z = quant4(x3.x, x3.y, inv);
      q1.w = quant4(x3.z, x3.w, inv);
      if (act) {
#pragma unroll 1
        for (int kb = 0; kb < a.K; kb += 8) {
          if (kb) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
              qv[k] = kb + k < a.K ? __ldg(a.inverse_perm + (size_t)t * a.K + kb + k) : -1;
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            void* rows;
            float* scl;
            int64_t r;
            if (!resolve_dest<EP>(a, t, kb + k, qv[k], rows, scl, r)) continue;
            uint4* d = reinterpret_cast<uint4*>(rows) + (size_t)r * (n32 * 2) + 2 * v;
            store_row16(d, q0);
            store_row16(d + 1, q1);
            if ((lane & 3) == 0) scl[(size_t)r * nb + (v >> 2)] = scale;
          }
        }
      }
    }
#else
    // unit = 512 elements (four 128-element scale blocks): 16 elements per lane,
    // 8 lanes per scale block
    const int n16 = a.H >> 4;
    const int nb = a.H >> 7;
    const int upr = (n16 + 31) >> 5;
    const uint4* x4 = reinterpret_cast<const uint4*>(a.x);
    UnitWalk wk(w0, W, upr);
    for (; wk.t < a.T; wk.next()) {
      const int64_t t = a.T - 1 - wk.t;  // last rows first (see above)
      const int v = wk.c * 32 + lane;
      const bool act = v < n16;
      uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
      if (act) {
        const uint4* src = x4 + (size_t)t * (n16 * 2) + 2 * v;
        lo = __ldg(src);
        hi = __ldg(src + 1);
      }
      int qv[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        qv[k] = k < a.K ? __ldg(a.inverse_perm + (size_t)t * a.K + k) : -1;
      float am = fmaxf(amax8(lo), amax8(hi));
      am = fmaxf(am, __shfl_xor_sync(kFull, am, 4));
      am = fmaxf(am, __shfl_xor_sync(kFull, am, 2));
      am = fmaxf(am, __shfl_xor_sync(kFull, am, 1));
      const float scale = __fmul_rn(fmaxf(am, 1e-30f), 1.0f / 448.0f);
      const float inv = __frcp_rn(scale);  // correctly rounded: the bits of 1.0f / scale
      uint4 q;
      q.x = quant4(lo.x, lo.y, inv);
      q.y = quant4(lo.z, lo.w, inv);
      q.z = quant4(hi.x, hi.y, inv);
      q.w = quant4(hi.z, hi.w, inv);
      // the unit's four scales in one 16-byte store by lane 0 (instead of four
      // 4-byte stores by four lanes) when the unit is whole and rows of scales
      // are 16-byte aligned
      const bool vec_scales = MOE_RD_SC_VECTOR_SCALES && (nb & 3) == 0 && wk.c * 4 + 4 <= nb;
      float4 s4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (vec_scales) {
        s4.x = __shfl_sync(kFull, scale, 0);
        s4.y = __shfl_sync(kFull, scale, 8);
        s4.z = __shfl_sync(kFull, scale, 16);
        s4.w = __shfl_sync(kFull, scale, 24);
      }
      if (act) {
#pragma unroll 1
        for (int kb = 0; kb < a.K; kb += 8) {
          if (kb) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
              qv[k] = kb + k < a.K ? __ldg(a.inverse_perm + (size_t)t * a.K + kb + k) : -1;
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            void* rows;
            float* scl;
            int64_t r;
            if (!resolve_dest<EP>(a, t, kb + k, qv[k], rows, scl, r)) continue;
            store_row16(reinterpret_cast<uint4*>(rows) + (size_t)r * n16 + v, q);
            if (vec_scales) {
              if (lane == 0) *reinterpret_cast<float4*>(scl + (size_t)r * nb + wk.c * 4) = s4;
            } else if ((lane & 7) == 0) {
              scl[(size_t)r * nb + (v >> 3)] = scale;
            }
          }
        }
      }
    }
#endif
  }
}

}  // namespace

int device_sms();
cudaError_t launch_scatter_bulk(const moe_rd_params& p, const moe_rd_buffers& b, int32_t* status,
                                cudaStream_t s);
cudaError_t launch_scatter_bulk_ep(const moe_rd_params& p, const void* x, const int32_t* ids,
                                   const int32_t* inverse_perm, const int32_t* offsets,
                                   const int32_t* dest_base, int world, void* const* peer_rows,
                                   float* const* peer_scales, int rank, int32_t* const* peer_copy_of,
                                   int32_t* status, cudaStream_t s);
cudaError_t launch_ep_replicate(void* rows, float* scales, int32_t* copy_of, const int32_t* n_rows,
                                int64_t max_rows, int H, bool fp8, int32_t* status, cudaStream_t s);
bool bulk_scatter_eligible(const moe_rd_params& p);

size_t positions_smem(int K, int E) { return (size_t)((kTile * K + 31) / 32) * E * 2 + 16; }

cudaError_t init_scatter_attributes() {
  cudaError_t e = cudaFuncSetAttribute(positions_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)positions_smem(kMaxK, kMaxE));
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(positions_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)positions_smem(kMaxK, kMaxE));
}

cudaError_t launch_scatter(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                           const int32_t* ids, const int32_t* tile_base, const int32_t* counts,
                           int32_t* status, int32_t* dense, const int32_t* group_counts, cudaStream_t s,
                           cudaEvent_t after_positions) {
  if (p.T == 0) {
    return after_positions ? cudaEventRecord(after_positions, s) : cudaSuccess;
  }
  PositionArgs pa;
  pa.ids = ids;
  pa.tile_base = tile_base;
  pa.offsets = b.offsets;
  pa.inverse_perm = b.inverse_perm;
  pa.drop_mask = b.drop_mask;
  pa.status = status;
  pa.weights = b.combine_weights;
  pa.row_token = b.row_token;
  pa.row_weight = b.row_weight;
  pa.counts = counts;
  pa.group_counts = group_counts;
  pa.user_counts = b.counts;
  pa.dense = (p.flags & MOE_RD_FLAG_SKIP_IDENTITY_ROWS) ? dense : nullptr;
  pa.T = p.T;
  pa.capacity = p.capacity;
  pa.out_rows = p.out_rows;
  pa.E = p.E;
  pa.K = p.K;
  pa.ntiles = plan.ntiles;
  cudaError_t e = plan.tile_major ? launch_pdl(positions_kernel<true>, dim3((unsigned)plan.ntiles),
                                               dim3(kPosThreads), positions_smem(p.K, p.E), s, pa)
                                  : launch_pdl(positions_kernel<false>, dim3((unsigned)plan.ntiles),
                                               dim3(kPosThreads), positions_smem(p.K, p.E), s, pa);
  count_launch();
  if (e != cudaSuccess) return e;
  if (after_positions) {
    e = cudaEventRecord(after_positions, s);
    if (e != cudaSuccess) return e;
  }
  if (plan.scatter == MOE_RD_SCATTER_NONE) return cudaSuccess;
  if (plan.scatter == MOE_RD_SCATTER_BULK) return launch_scatter_bulk(p, b, status, s);

  ScatterArgs a = {};
  a.x = static_cast<const uint16_t*>(b.x);
  a.inverse_perm = b.inverse_perm;
  a.rows = b.permuted;
  a.scales = b.scales;
  a.T = p.T;
  a.H = p.H;
  a.K = p.K;
  a.dense = (p.flags & MOE_RD_FLAG_SKIP_IDENTITY_ROWS) ? dense : nullptr;
  const bool fp8 = p.rows_format == MOE_RD_ROWS_FP8_E4M3_B128;
  const int64_t upr = fp8 ? (p.H / MOE_RD_SC_FP8_LANE_ELEMS + 31) >> 5 : ((p.H >> 3) + 32 * kUV - 1) / (32 * kUV);
  const int64_t units = p.T * upr;
  const int64_t want = (units + kScatterWarps - 1) / kScatterWarps;
  const int64_t cap = (int64_t)device_sms() * MOE_RD_SC_BLOCKS_PER_SM;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  if (fp8)
    e = launch_pdl(scatter_kernel<MOE_RD_ROWS_FP8_E4M3_B128, false>, dim3(grid), dim3(kScatterThreads), 0, s, a);
  else
    e = launch_pdl(scatter_kernel<MOE_RD_ROWS_BF16, false>, dim3(grid), dim3(kScatterThreads), 0, s, a);
  count_launch();
  return e;
}

namespace {

// One block.  kept_all[s][e] = rows rank s dispatches to expert e.
__global__ void __launch_bounds__(256)
ep_plan_kernel(const int32_t* __restrict__ kept_all, int world, int rank, int E, int64_t max_rows,
               int32_t* __restrict__ dest_base, int32_t* __restrict__ cnt,
               int32_t* __restrict__ local_offsets, int32_t* __restrict__ status) {
  __shared__ int s_tot[kMaxE];     // rows expert e receives from all ranks
  __shared__ int s_before[kMaxE];  // rows expert e receives from ranks before `rank`
  __shared__ int s_start[kMaxE];   // first row of expert e in its owner's buffer
  const int epr = E / world;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, before = 0;
    for (int s = 0; s < world; ++s) {
      const int v = max(kept_all[(size_t)s * E + e], 0);
      if (s < rank) before += v;
      tot += v;
    }
    s_tot[e] = tot;
    s_before[e] = before;
  }
  __syncthreads();
  // exclusive prefix of s_tot inside every owner's expert range (<= 256 entries).
  // Every rank computes the same table from the same counts, so every rank sees
  // the same overflow: an expert whose rows would end past max_rows in its
  // owner's buffer gets no destination (-1) on any rank, and its pairs are
  // skipped by the scatter and combine kernels instead of being stored or loaded
  // out of bounds.
  if (threadIdx.x < world) {
    const int d = threadIdx.x;
    int64_t run = 0;
    bool over = false;
    for (int le = 0; le < epr; ++le) {
      over = over || run + s_tot[d * epr + le] > max_rows;
      s_start[d * epr + le] = over ? -1 : (int)run;
      if (d == rank) local_offsets[le] = (int)(run < max_rows ? run : max_rows);
      run += s_tot[d * epr + le];
    }
    if (d == rank) local_offsets[epr] = (int)(run < max_rows ? run : max_rows);
    if (over) report(status, 202, (int)(run > 0x7fffffff ? 0x7fffffff : run), d);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    dest_base[e] = s_start[e] < 0 ? -1 : s_start[e] + s_before[e];
  for (int i = threadIdx.x; i < world * epr; i += blockDim.x) {
    const int s = i / epr, le = i - s * epr;
    cnt[i] = max(kept_all[(size_t)s * E + rank * epr + le], 0);
  }
}

}  // namespace
}  // namespace moe_rd

using namespace moe_rd;

extern "C" int moe_rd_ep_plan(const int32_t* kept_all, int world, int rank, int E, int64_t max_rows,
                              int32_t* dest_base, int32_t* cnt, int32_t* local_offsets,
                              int32_t* status, void* stream) {
  if (kept_all == nullptr || dest_base == nullptr || cnt == nullptr || local_offsets == nullptr ||
      status == nullptr)
    return MOE_RD_E_NULL;
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || E < 1 || E > kMaxE ||
      E % world != 0 || max_rows < 0)
    return MOE_RD_E_SHAPE;
  ep_plan_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      kept_all, world, rank, E, max_rows, dest_base, cnt, local_offsets, status);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? MOE_RD_OK : MOE_RD_E_CUDA;
}

static int ep_scatter_impl(const moe_rd_params* p, const void* x, const int32_t* expert_ids,
                           const int32_t* inverse_perm, const int32_t* offsets, const int32_t* dest_base,
                           int world, void* const* peer_rows, float* const* peer_scales, int rank,
                           int32_t* const* peer_copy_of, int32_t* status, void* stream);

extern "C" int moe_rd_ep_scatter(const moe_rd_params* p, const void* x, const int32_t* expert_ids,
                                 const int32_t* inverse_perm, const int32_t* offsets,
                                 const int32_t* dest_base, int world, void* const* peer_rows,
                                 float* const* peer_scales, int32_t* status, void* stream) {
  return ep_scatter_impl(p, x, expert_ids, inverse_perm, offsets, dest_base, world, peer_rows, peer_scales, -1,
                         nullptr, status, stream);
}

extern "C" int moe_rd_ep_scatter_once(const moe_rd_params* p, const void* x, const int32_t* expert_ids,
                                      const int32_t* inverse_perm, const int32_t* offsets,
                                      const int32_t* dest_base, int world, int rank, void* const* peer_rows,
                                      float* const* peer_scales, int32_t* const* peer_copy_of,
                                      int32_t* status, void* stream) {
  if (peer_copy_of == nullptr) return MOE_RD_E_NULL;
  if (rank < 0 || rank >= world) return MOE_RD_E_SHAPE;
  if (p != nullptr && p->scatter_impl != MOE_RD_SCATTER_BULK) return MOE_RD_E_UNSUPPORTED;
  for (int d = 0; d < world && d < kMaxWorld; ++d)
    if (peer_copy_of[d] == nullptr) return MOE_RD_E_NULL;
  return ep_scatter_impl(p, x, expert_ids, inverse_perm, offsets, dest_base, world, peer_rows, peer_scales, rank,
                         peer_copy_of, status, stream);
}

extern "C" int moe_rd_ep_replicate(const moe_rd_params* p, void* rows, float* scales, int32_t* copy_of,
                                   const int32_t* n_rows, int64_t max_rows, int32_t* status, void* stream) {
  if (p == nullptr || rows == nullptr || copy_of == nullptr || n_rows == nullptr || status == nullptr)
    return MOE_RD_E_NULL;
  const bool fp8 = p->rows_format == MOE_RD_ROWS_FP8_E4M3_B128;
  if (max_rows < 0 || p->H % 8 != 0 || (fp8 && p->H % 512 != 0)) return MOE_RD_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(scales)) & 15) return MOE_RD_E_ALIGN;
  if (max_rows == 0) return MOE_RD_OK;
  const cudaError_t e = launch_ep_replicate(rows, scales, copy_of, n_rows, max_rows, p->H, fp8, status,
                                            static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) set_last_cuda_error(e);
  return e == cudaSuccess ? MOE_RD_OK : MOE_RD_E_CUDA;
}

static int ep_scatter_impl(const moe_rd_params* p, const void* x, const int32_t* expert_ids,
                           const int32_t* inverse_perm, const int32_t* offsets, const int32_t* dest_base,
                           int world, void* const* peer_rows, float* const* peer_scales, int rank,
                           int32_t* const* peer_copy_of, int32_t* status, void* stream) {
  if (p == nullptr || x == nullptr || expert_ids == nullptr || inverse_perm == nullptr ||
      offsets == nullptr || dest_base == nullptr || peer_rows == nullptr)
    return MOE_RD_E_NULL;
  if (world < 1 || world > kMaxWorld || p->E % world != 0 || p->T < 0 || p->H % 8 != 0)
    return MOE_RD_E_SHAPE;
  const bool fp8 = p->rows_format == MOE_RD_ROWS_FP8_E4M3_B128;
  if (fp8 && p->H % 128 != 0) return MOE_RD_E_SHAPE;
  // fp8 rows without a scales buffer: the scales follow each row (bulk copies only)
  const bool packed = fp8 && peer_scales == nullptr;
  if (packed && p->scatter_impl != MOE_RD_SCATTER_BULK) return MOE_RD_E_NULL;
  if (p->T == 0) return MOE_RD_OK;
  if (p->scatter_impl == MOE_RD_SCATTER_BULK) {
    // whole-row bulk copies (TMA engine) into the owners' buffers
    if (!bulk_scatter_eligible(*p)) return MOE_RD_E_UNSUPPORTED;
    for (int d = 0; d < world; ++d)
      if (peer_rows[d] == nullptr || (reinterpret_cast<uintptr_t>(peer_rows[d]) & 15) ||
          (fp8 && !packed && (peer_scales[d] == nullptr || (reinterpret_cast<uintptr_t>(peer_scales[d]) & 15))))
        return MOE_RD_E_ALIGN;
    if (status == nullptr) return MOE_RD_E_NULL;
    const cudaError_t be =
        launch_scatter_bulk_ep(*p, x, expert_ids, inverse_perm, offsets, dest_base, world, peer_rows,
                               peer_scales, rank, peer_copy_of, status, static_cast<cudaStream_t>(stream));
    return be == cudaSuccess ? MOE_RD_OK : MOE_RD_E_CUDA;
  }
  ScatterArgs a = {};
  a.x = static_cast<const uint16_t*>(x);
  a.inverse_perm = inverse_perm;
  a.T = p->T;
  a.H = p->H;
  a.K = p->K;
  a.ids = expert_ids;
  a.offsets = offsets;
  a.dest_base = dest_base;
  a.epr = p->E / world;
  for (int d = 0; d < world; ++d) {
    if (peer_rows[d] == nullptr || (reinterpret_cast<uintptr_t>(peer_rows[d]) & 15))
      return MOE_RD_E_ALIGN;
    a.peer_rows[d] = peer_rows[d];
    a.peer_scales[d] = fp8 ? peer_scales[d] : nullptr;
    if (fp8 && a.peer_scales[d] == nullptr) return MOE_RD_E_NULL;
  }
  const int64_t upr = fp8 ? (p->H / MOE_RD_SC_FP8_LANE_ELEMS + 31) >> 5 : ((p->H >> 3) + 32 * kUV - 1) / (32 * kUV);
  const int64_t units = p->T * upr;
  const int64_t want = (units + kScatterWarps - 1) / kScatterWarps;
  const int64_t cap = (int64_t)device_sms() * MOE_RD_SC_BLOCKS_PER_SM;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (fp8)
    e = launch_pdl(scatter_kernel<MOE_RD_ROWS_FP8_E4M3_B128, true>, dim3(grid),
                   dim3(kScatterThreads), 0, s, a);
  else
    e = launch_pdl(scatter_kernel<MOE_RD_ROWS_BF16, true>, dim3(grid), dim3(kScatterThreads), 0, s, a);
  count_launch();
  return e == cudaSuccess ? MOE_RD_OK : MOE_RD_E_CUDA;
}
