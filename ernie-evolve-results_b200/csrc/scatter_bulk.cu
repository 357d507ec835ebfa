// Row scatter through shared memory with bulk asynchronous copies (the TMA
// engine, non-tensor form): a token row is staged once in shared memory and
// then written to each of its K destination rows by ONE cp.async.bulk
// instruction per copy, so HBM sees whole-row bursts instead of 512-byte pieces
// and the SM issues a handful of instructions per row.
//
// Same contract as scatter_kernel (scatter.cu), which replaces gather_body of
// the reference (kernel.cu:2216-2238): permuted[inverse_perm[t,k], :] = x[t, :]
// (bf16), or its fp8-e4m3 image with one fp32 scale per 128 elements.
//
// bf16:  one warp per CTA owns a ring of stages; lane 0 streams rows in with
//        cp.async.bulk (global -> shared, completion on an mbarrier); lane k
//        reads inverse_perm[t,k] while the row is in flight and, once it has
//        landed, issues the bulk store of copy k.
// fp8:   a CTA quantises the row cooperatively into a shared-memory image
//        (bytes + scales, double buffered) and thread k issues the bulk stores.
// Every mbarrier wait is bounded; on expiry the status block is set and the CTA
// stops taking rows.
#include <cuda_fp8.h>

#include "common.cuh"

namespace moe_rd {
namespace {

constexpr uint32_t kSpinLimit = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

constexpr int kMaxWorld = 8;

struct BulkArgs {
  const uint16_t* x;
  const int32_t* inverse_perm;
  void* rows;
  float* scales;
  int32_t* status;
  int64_t T;
  int H, K, stages;
  // expert-parallel destinations (see ScatterArgs in scatter.cu)
  const int32_t* ids;
  const int32_t* offsets;
  const int32_t* dest_base;
  void* peer_rows[kMaxWorld];
  float* peer_scales[kMaxWorld];
  int epr;
  int packed;  // 1 (expert-parallel fp8): a destination row is H bytes followed by its H/128 scales
  // Send-once exchange: a token that has several experts on one remote rank crosses NVLink once.  Its
  // first pair there carries the row; for every later pair the sender stores only
  // copy_of[row of that pair] = row of the first pair (4 bytes) in the owner's memory, and the owner
  // copies the row locally afterwards (ep_replicate_kernel).  Null pointers: every pair carries its row.
  int rank;
  int32_t* peer_copy_of[kMaxWorld];
};

// Destination of pair (t,k) with local row q >= 0: buffers and row to write;
// false when the pair has none (its expert's rows do not fit the owner's buffer).
template <bool EP>
__device__ __forceinline__ bool bulk_dest(const BulkArgs& a, int64_t t, int k, int q,
                                          unsigned char*& rows, unsigned char*& scales,
                                          int64_t& row) {
  if (!EP) {
    rows = static_cast<unsigned char*>(a.rows);
    scales = reinterpret_cast<unsigned char*>(a.scales);
    row = q;
    return true;
  }
  const int e = __ldg(a.ids + (size_t)t * a.K + k);
  const int db = __ldg(a.dest_base + e);
  if (db < 0) return false;
  const int d = e / a.epr;
  rows = static_cast<unsigned char*>(a.peer_rows[d]);
  scales = reinterpret_cast<unsigned char*>(a.peer_scales[d]);
  row = (int64_t)db + (q - __ldg(a.offsets + e));
  if (d != a.rank && a.peer_copy_of[d] != nullptr) {
    // an earlier pair of this token that has a row on the same rank already carries the bytes
    for (int j = 0; j < k; ++j) {
      const int ej = __ldg(a.ids + (size_t)t * a.K + j);
      if (ej / a.epr != d) continue;
      const int qj = __ldg(a.inverse_perm + (size_t)t * a.K + j);
      const int dbj = __ldg(a.dest_base + ej);
      if (qj < 0 || dbj < 0) continue;
      a.peer_copy_of[d][row] = dbj + (qj - __ldg(a.offsets + ej));
      return false;
    }
  }
  return true;
}

// ------------------------------ bf16 --------------------------------------
template <bool EP>
__global__ void __launch_bounds__(32) scatter_bulk_bf16_kernel(const BulkArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  pdl_sync();
  const int lane = threadIdx.x;
  const uint32_t row_bytes = (uint32_t)a.H * 2;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)a.stages * row_bytes);
  if (lane == 0) {
    for (int s = 0; s < a.stages; ++s) mbar_init(smem_u32(bars + s), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  const int64_t G = gridDim.x;
  const int64_t first = blockIdx.x;
  const unsigned char* xb = reinterpret_cast<const unsigned char*>(a.x);

  if (lane == 0) {
    for (int s = 0; s < a.stages; ++s) {
      const int64_t t = first + (int64_t)s * G;
      if (t >= a.T) break;
      const uint32_t bar = smem_u32(bars + s);
      mbar_expect_tx(bar, row_bytes);
      bulk_load(smem_u32(smem + (size_t)s * row_bytes), xb + (size_t)t * row_bytes, row_bytes, bar);
    }
  }
  int64_t i = 0;
  for (int64_t t = first; t < a.T; t += G, ++i) {
    const int s = (int)(i % a.stages);
    const uint32_t parity = (uint32_t)((i / a.stages) & 1);
    int pos = -1;
    if (lane < a.K) pos = __ldg(a.inverse_perm + (size_t)t * a.K + lane);
    bool ok = mbar_wait(smem_u32(bars + s), parity);
    ok = __all_sync(kFull, ok);
    if (!ok) {
      if (lane == 0) report(a.status, 301, (int)t, s);
      break;
    }
    const uint32_t src = smem_u32(smem + (size_t)s * row_bytes);
    if (pos >= 0) {
      unsigned char *out, *unused;
      int64_t r;
      if (bulk_dest<EP>(a, t, lane, pos, out, unused, r)) bulk_store(out + (size_t)r * row_bytes, src, row_bytes);
    }
    bulk_commit();
    // the stage may be refilled once every lane's stores have read it
    bulk_wait_read<0>();
    __syncwarp();
    const int64_t tn = t + (int64_t)a.stages * G;
    if (lane == 0 && tn < a.T) {
      const uint32_t bar = smem_u32(bars + s);
      mbar_expect_tx(bar, row_bytes);
      bulk_load(src, xb + (size_t)tn * row_bytes, row_bytes, bar);
    }
  }
  // leave only after the loads this warp started have landed (they target its shared memory)
  if (lane == 0) {
    for (int64_t t = first + i * G, j = i; j < i + a.stages; ++j, t += G) {
      // rows [i, i+stages) were requested only if they exist and were not consumed above
      if (t < a.T) mbar_wait(smem_u32(bars + (int)(j % a.stages)), (uint32_t)((j / a.stages) & 1));
    }
  }
}

// ------------------------------ fp8 ---------------------------------------
constexpr int kQThreads = 128;

__device__ __forceinline__ uint32_t abs_bf16x2(uint32_t v) { return v & 0x7fff7fffu; }
__device__ __forceinline__ float amax8(const uint4& v) {
  float m = fmaxf(bf16_lo(abs_bf16x2(v.x)), bf16_hi(abs_bf16x2(v.x)));
  m = fmaxf(m, fmaxf(bf16_lo(abs_bf16x2(v.y)), bf16_hi(abs_bf16x2(v.y))));
  m = fmaxf(m, fmaxf(bf16_lo(abs_bf16x2(v.z)), bf16_hi(abs_bf16x2(v.z))));
  m = fmaxf(m, fmaxf(bf16_lo(abs_bf16x2(v.w)), bf16_hi(abs_bf16x2(v.w))));
  return m;
}
__device__ __forceinline__ uint32_t quant4(uint32_t a, uint32_t b, float inv) {
  const float2 f0 = make_float2(__fmul_rn(bf16_lo(a), inv), __fmul_rn(bf16_hi(a), inv));
  const float2 f1 = make_float2(__fmul_rn(bf16_lo(b), inv), __fmul_rn(bf16_hi(b), inv));
  const uint32_t q0 = __nv_cvt_float2_to_fp8x2(f0, __NV_SATFINITE, __NV_E4M3);
  const uint32_t q1 = __nv_cvt_float2_to_fp8x2(f1, __NV_SATFINITE, __NV_E4M3);
  return q0 | (q1 << 16);
}

// Shared image of one quantised row: H bytes, then H/128 scales (16-byte aligned).
template <bool EP>
__global__ void __launch_bounds__(kQThreads) scatter_bulk_fp8_kernel(const BulkArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  pdl_sync();
  const int tid = threadIdx.x, lane = tid & 31;
  const int n16 = a.H >> 4, nb = a.H >> 7;
  const uint32_t q_bytes = (uint32_t)a.H;
  const uint32_t s_bytes = (uint32_t)nb * 4;
  const uint32_t img = (q_bytes + s_bytes + 127u) & ~127u;
  const uint4* x4 = reinterpret_cast<const uint4*>(a.x);

  int64_t i = 0;
  for (int64_t t = blockIdx.x; t < a.T; t += gridDim.x, ++i) {
    unsigned char* buf = smem + (size_t)(i & 1) * img;
    int pos = -1;
    if (tid < a.K) pos = __ldg(a.inverse_perm + (size_t)t * a.K + tid);
    // the buffer used two rows ago must have been read by its stores
    if (tid < a.K) bulk_wait_read<1>();
    __syncthreads();
    const uint4* src = x4 + (size_t)t * (n16 * 2);
    for (int v0 = 0; v0 < n16; v0 += kQThreads) {
      const int v = v0 + tid;
      const bool act = v < n16;
      uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
      if (act) {
        lo = __ldg(src + 2 * v);
        hi = __ldg(src + 2 * v + 1);
      }
      float am = fmaxf(amax8(lo), amax8(hi));
      am = fmaxf(am, __shfl_xor_sync(kFull, am, 4));
      am = fmaxf(am, __shfl_xor_sync(kFull, am, 2));
      am = fmaxf(am, __shfl_xor_sync(kFull, am, 1));
      const float scale = __fmul_rn(fmaxf(am, 1e-30f), 1.0f / 448.0f);
      const float inv = __fdiv_rn(1.0f, scale);
      uint4 q;
      q.x = quant4(lo.x, lo.y, inv);
      q.y = quant4(lo.z, lo.w, inv);
      q.z = quant4(hi.x, hi.y, inv);
      q.w = quant4(hi.z, hi.w, inv);
      if (act) {
        reinterpret_cast<uint4*>(buf)[v] = q;
        if ((lane & 7) == 0) reinterpret_cast<float*>(buf + q_bytes)[v >> 3] = scale;
      }
    }
    fence_async_smem();  // make this thread's shared-memory writes visible to the bulk engine
    __syncthreads();
    if (tid < a.K) {
      if (pos >= 0) {
        unsigned char *out_q, *out_s;
        int64_t r;
        if (bulk_dest<EP>(a, t, tid, pos, out_q, out_s, r)) {
          if (a.packed) {
            // scales follow their row in the destination: the shared image goes out in one copy
            bulk_store(out_q + (size_t)r * (q_bytes + s_bytes), smem_u32(buf), q_bytes + s_bytes);
          } else {
            bulk_store(out_q + (size_t)r * q_bytes, smem_u32(buf), q_bytes);
            bulk_store(out_s + (size_t)r * s_bytes, smem_u32(buf + q_bytes), s_bytes);
          }
        }
      }
      bulk_commit();
    }
  }
  if (tid < a.K) bulk_wait_read<0>();
}

}  // namespace

int device_sms();

bool bulk_scatter_eligible(const moe_rd_params& p) {
  if (p.T <= 0 || p.K > 32) return false;
  if (p.rows_format == MOE_RD_ROWS_FP8_E4M3_B128)
    return p.H % 512 == 0 && (size_t)2 * ((p.H + (p.H / 128) * 4 + 127) & ~127) <= 200 * 1024;
  return (size_t)p.H * 2 * 2 + 64 <= 200 * 1024;
}

cudaError_t init_bulk_attributes() {
  const auto attr = cudaFuncAttributeMaxDynamicSharedMemorySize;
  cudaError_t e = cudaFuncSetAttribute(scatter_bulk_bf16_kernel<false>, attr, 200 * 1024);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(scatter_bulk_bf16_kernel<true>, attr, 200 * 1024);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(scatter_bulk_fp8_kernel<false>, attr, 200 * 1024);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(scatter_bulk_fp8_kernel<true>, attr, 200 * 1024);
}

static cudaError_t launch_bulk_args(const moe_rd_params& p, BulkArgs& a, bool ep, cudaStream_t s) {
  const int sms = device_sms();
  cudaError_t e;
  if (p.rows_format == MOE_RD_ROWS_FP8_E4M3_B128) {
    const size_t img = ((size_t)p.H + (p.H / 128) * 4 + 127) & ~(size_t)127;
    const size_t smem = 2 * img;
    int per_sm = (int)((200 * 1024) / (smem + 1024));
    if (per_sm > 12) per_sm = 12;
    if (per_sm < 1) per_sm = 1;
    int64_t grid = (int64_t)sms * per_sm;
    if (grid > p.T) grid = p.T;
    a.stages = 2;
    e = ep ? launch_pdl(scatter_bulk_fp8_kernel<true>, dim3((unsigned)grid), dim3(kQThreads), smem, s, a)
           : launch_pdl(scatter_bulk_fp8_kernel<false>, dim3((unsigned)grid), dim3(kQThreads), smem, s, a);
  } else {
    const size_t row = (size_t)p.H * 2;
    // about 160 KB of rows in flight per SM, at least 2 stages per warp
    int stages = 4;
    while (stages > 2 && stages * row + 64 > 48 * 1024) --stages;
    const size_t smem = stages * row + 8 * stages;
    int per_sm = (int)((160 * 1024) / (smem + 1024));
    if (per_sm > 16) per_sm = 16;
    if (per_sm < 1) per_sm = 1;
    int64_t grid = (int64_t)sms * per_sm;
    if (grid > p.T) grid = p.T;
    a.stages = stages;
    e = ep ? launch_pdl(scatter_bulk_bf16_kernel<true>, dim3((unsigned)grid), dim3(32), smem, s, a)
           : launch_pdl(scatter_bulk_bf16_kernel<false>, dim3((unsigned)grid), dim3(32), smem, s, a);
  }
  count_launch();
  return e;
}

cudaError_t launch_scatter_bulk(const moe_rd_params& p, const moe_rd_buffers& b, int32_t* status,
                                cudaStream_t s) {
  BulkArgs a = {};
  a.x = static_cast<const uint16_t*>(b.x);
  a.inverse_perm = b.inverse_perm;
  a.rows = b.permuted;
  a.scales = b.scales;
  a.status = status;
  a.T = p.T;
  a.H = p.H;
  a.K = p.K;
  return launch_bulk_args(p, a, false, s);
}

// Expert-parallel form: destinations are rows of the owners' buffers.
cudaError_t launch_scatter_bulk_ep(const moe_rd_params& p, const void* x, const int32_t* ids,
                                   const int32_t* inverse_perm, const int32_t* offsets,
                                   const int32_t* dest_base, int world, void* const* peer_rows,
                                   float* const* peer_scales, int rank, int32_t* const* peer_copy_of,
                                   int32_t* status, cudaStream_t s) {
  BulkArgs a = {};
  a.x = static_cast<const uint16_t*>(x);
  a.inverse_perm = inverse_perm;
  a.status = status;
  a.T = p.T;
  a.H = p.H;
  a.K = p.K;
  a.ids = ids;
  a.offsets = offsets;
  a.dest_base = dest_base;
  a.epr = p.E / world;
  for (int d = 0; d < world; ++d) {
    a.peer_rows[d] = peer_rows[d];
    a.peer_scales[d] = peer_scales != nullptr ? peer_scales[d] : nullptr;
    a.peer_copy_of[d] = peer_copy_of != nullptr ? peer_copy_of[d] : nullptr;
  }
  a.rank = rank;
  a.packed = (peer_scales == nullptr && p.rows_format == MOE_RD_ROWS_FP8_E4M3_B128) ? 1 : 0;
  return launch_bulk_args(p, a, true, s);
}

// ---------------------------------------------------------------------------
// Owner side of the send-once exchange: row r with copy_of[r] = s >= 0 did not
// cross NVLink; it is a copy of row s of the same buffer (the same token, sent
// for an earlier expert of this rank).  One warp per marked row, 16-byte vectors; the
// mark is cleared for the next step.  Runs after the barrier that orders every
// rank's stores.  A source row is never itself a copy (the sender marks only
// later pairs, and names the first one that carries a row).
// ---------------------------------------------------------------------------
struct ReplicateArgs {
  unsigned char* rows;
  unsigned char* scales;   // null: bf16 rows, or scales inside the row pitch (packed)
  int32_t* copy_of;
  const int32_t* n_rows;   // device value: rows received in this step
  int32_t* status;
  int64_t max_rows;
  uint32_t row_pitch, row_copy, scale_pitch;
};

__device__ __forceinline__ void replicate_row(const ReplicateArgs& a, int64_t r, int src, int lane) {
  const uint4* s4 = reinterpret_cast<const uint4*>(a.rows + (size_t)src * a.row_pitch);
  uint4* d4 = reinterpret_cast<uint4*>(a.rows + (size_t)r * a.row_pitch);
  const uint32_t nvec = a.row_copy / 16;
  uint32_t v = lane;
  for (; v + 224 < nvec; v += 256) {  // eight 16-byte loads in flight per lane
    uint4 x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = __ldcs(s4 + v + 32 * i);
#pragma unroll
    for (int i = 0; i < 8; ++i) __stcs(d4 + v + 32 * i, x[i]);
  }
  for (; v + 96 < nvec; v += 128) {
    const uint4 x0 = __ldcs(s4 + v), x1 = __ldcs(s4 + v + 32), x2 = __ldcs(s4 + v + 64), x3 = __ldcs(s4 + v + 96);
    __stcs(d4 + v, x0);
    __stcs(d4 + v + 32, x1);
    __stcs(d4 + v + 64, x2);
    __stcs(d4 + v + 96, x3);
  }
  for (; v < nvec; v += 32) __stcs(d4 + v, __ldcs(s4 + v));
  if (a.scales != nullptr) {
    const float* sf = reinterpret_cast<const float*>(a.scales + (size_t)src * a.scale_pitch);
    float* df = reinterpret_cast<float*>(a.scales + (size_t)r * a.scale_pitch);
    for (uint32_t i = lane; i < a.scale_pitch / 4; i += 32) df[i] = sf[i];
  }
}

// A block takes 32 consecutive rows at a time: its first warp reads their marks in one coalesced load,
// clears them and lists the marked rows in shared memory; the eight warps then share the listed rows, a
// row per warp at a time (about a third to a half of the rows are marked, unevenly).
__global__ void __launch_bounds__(256) ep_replicate_kernel(const ReplicateArgs a) {
  __shared__ int s_row[32], s_src[32], s_n;
  pdl_sync();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int64_t n = __ldg(a.n_rows);
  n = n < 0 ? 0 : (n > a.max_rows ? a.max_rows : n);
  for (int64_t base = (int64_t)blockIdx.x * 32; base < n; base += (int64_t)gridDim.x * 32) {
    if (w == 0) {
      const int64_t r = base + lane;
      int src = r < n ? a.copy_of[r] : -1;
      if (src >= 0) a.copy_of[r] = -1;
      if (src >= n) {  // cannot happen with marks written by the scatter kernel of a consistent plan
        report(a.status, 203, (int)r, src);
        src = -1;
      }
      const unsigned marked = __ballot_sync(kFull, src >= 0);
      if (src >= 0) {
        const int i = __popc(marked & ((1u << lane) - 1u));
        s_row[i] = lane;
        s_src[i] = src;
      }
      if (lane == 0) s_n = __popc(marked);
    }
    __syncthreads();
    for (int i = w; i < s_n; i += 8) replicate_row(a, base + s_row[i], s_src[i], lane);
    __syncthreads();
  }
}

cudaError_t launch_ep_replicate(void* rows, float* scales, int32_t* copy_of, const int32_t* n_rows,
                                int64_t max_rows, int H, bool fp8, int32_t* status, cudaStream_t s) {
  ReplicateArgs a = {};
  a.rows = static_cast<unsigned char*>(rows);
  a.copy_of = copy_of;
  a.n_rows = n_rows;
  a.status = status;
  a.max_rows = max_rows;
  if (fp8 && scales == nullptr) {  // packed: H bytes + H/128 scales per row
    a.row_pitch = a.row_copy = (uint32_t)(H + (H / 128) * 4);
  } else {
    a.row_pitch = a.row_copy = (uint32_t)(fp8 ? H : 2 * H);
    a.scales = fp8 ? reinterpret_cast<unsigned char*>(scales) : nullptr;
    a.scale_pitch = fp8 ? (uint32_t)(H / 128) * 4 : 0;
  }
  int64_t grid = (max_rows + 31) / 32;
  const int64_t cap = (int64_t)device_sms() * 16;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  const cudaError_t e = launch_pdl(ep_replicate_kernel, dim3((unsigned)grid), dim3(256), 0, s, a);
  count_launch();
  return e;
}

}  // namespace moe_rd
