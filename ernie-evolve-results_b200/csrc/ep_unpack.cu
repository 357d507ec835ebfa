// Expert-parallel receive side: turn the rank-major buffer an all-to-all
// delivers ([source rank][local expert][rows]) into the expert-major layout an
// expert GEMM consumes ([local expert][source rank][rows]).
//
// The reference has no expert parallelism (its only count-then-rows exchange is
// the embedding-row all-to-all of nanogpt-speedrun/track-1,
// track_1_short/sharded_rows.py:72-103, which ships int8 rows and fp32 scales as
// two exchanges, ngram_table.py:343-360).  The order inside an expert is
// (source rank, source slot order), i.e. deterministic.
#include "common.cuh"

namespace moe_rd {
namespace {

constexpr int kUnpackThreads = 256;
constexpr int kMaxChunks = 2048;  // world * experts_per_rank

struct UnpackArgs {
  const int32_t* cnt;  // [W][epr] rows received from source s for local expert le
  const uint4* src_rows;
  uint4* dst_rows;
  const float* src_scales;
  float* dst_scales;
  int32_t* local_offsets;  // [epr+1]
  int32_t* status;
  int64_t max_rows;
  int W, epr, row_vecs, scale_floats;
};

__global__ void __launch_bounds__(kUnpackThreads) ep_unpack_kernel(const UnpackArgs a) {
  __shared__ int s_src[kMaxChunks + 1];  // start of chunk (s, le) in the received buffer
  __shared__ int s_dst[kMaxChunks];      // start of chunk (s, le) in the expert-major buffer
  __shared__ int s_cnt[kMaxChunks];
  __shared__ int s_tot;
  const int n = a.W * a.epr;
  for (int c = threadIdx.x; c < n; c += kUnpackThreads) s_cnt[c] = max(a.cnt[c], 0);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int c = 0; c < n; ++c) {  // (s, le) order = arrival order
      s_src[c] = run;
      run += s_cnt[c];
    }
    s_src[n] = run;
    s_tot = run;
  } else if (threadIdx.x == 32) {
    int d = 0;
    for (int le = 0; le < a.epr; ++le) {
      if (blockIdx.x == 0) a.local_offsets[le] = d;
      for (int s = 0; s < a.W; ++s) {
        s_dst[s * a.epr + le] = d;
        d += s_cnt[s * a.epr + le];
      }
    }
    if (blockIdx.x == 0) a.local_offsets[a.epr] = d;
  }
  __syncthreads();
  const int total = s_tot;
  if (total > a.max_rows) {
    if (threadIdx.x == 0 && blockIdx.x == 0) report(a.status, 201, total, (int)a.max_rows);
    return;
  }
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (kUnpackThreads / 32);
  for (int r = blockIdx.x * (kUnpackThreads / 32) + (threadIdx.x >> 5); r < total; r += warps) {
    // chunk holding row r: last c with s_src[c] <= r
    int lo = 0, hi = n;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_src[mid] <= r) lo = mid; else hi = mid;
    }
    const int q = s_dst[lo] + (r - s_src[lo]);
    const uint4* sp = a.src_rows + (size_t)r * a.row_vecs;
    uint4* dp = a.dst_rows + (size_t)q * a.row_vecs;
    for (int v = lane; v < a.row_vecs; v += 32) __stcs(dp + v, __ldcs(sp + v));
    if (a.src_scales != nullptr) {
      const float* ss = a.src_scales + (size_t)r * a.scale_floats;
      float* ds = a.dst_scales + (size_t)q * a.scale_floats;
      for (int v = lane; v < a.scale_floats; v += 32) ds[v] = ss[v];
    }
  }
}

}  // namespace

int device_sms();

}  // namespace moe_rd

using namespace moe_rd;

extern "C" int moe_rd_ep_unpack(const int32_t* cnt, int world, int experts_per_rank,
                                const void* recv_rows, const float* recv_scales, void* out_rows,
                                float* out_scales, int32_t* local_offsets, int64_t row_bytes,
                                int32_t scale_floats, int64_t max_rows, int32_t* status,
                                void* stream) {
  if (cnt == nullptr || recv_rows == nullptr || out_rows == nullptr || local_offsets == nullptr ||
      status == nullptr)
    return MOE_RD_E_NULL;
  if (world < 1 || experts_per_rank < 1 || (int64_t)world * experts_per_rank > kMaxChunks)
    return MOE_RD_E_SHAPE;
  if (row_bytes <= 0 || row_bytes % 16 != 0 || max_rows < 0 || max_rows > 0x7fffffff)
    return MOE_RD_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(recv_rows) | reinterpret_cast<uintptr_t>(out_rows)) & 15)
    return MOE_RD_E_ALIGN;
  if ((recv_scales == nullptr) != (out_scales == nullptr)) return MOE_RD_E_NULL;
  UnpackArgs a;
  a.cnt = cnt;
  a.src_rows = static_cast<const uint4*>(recv_rows);
  a.dst_rows = static_cast<uint4*>(out_rows);
  a.src_scales = recv_scales;
  a.dst_scales = out_scales;
  a.local_offsets = local_offsets;
  a.status = status;
  a.max_rows = max_rows;
  a.W = world;
  a.epr = experts_per_rank;
  a.row_vecs = (int)(row_bytes / 16);
  a.scale_floats = scale_floats;
  ep_unpack_kernel<<<device_sms() * 8, kUnpackThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? MOE_RD_OK : MOE_RD_E_CUDA;
}
