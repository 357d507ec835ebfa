// C ABI of libmoe_rd.so: parameter validation, workspace carving and launch
// sequencing.  Mirrors the host part of the reference's run()
// (kernel.cu:4067-4079 stream handling, 4202-4268 one arena with 256-byte
// aligned sub-buffers, 4323-4430 launch order) with destination passing: the
// caller owns every buffer, nothing is allocated here.
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace moe_rd {

static std::atomic<int64_t> g_launches{0};
static thread_local cudaError_t t_last_cuda = cudaSuccess;

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
void set_last_cuda_error(cudaError_t e) { t_last_cuda = e; }

cudaError_t init_route_attributes();
cudaError_t init_umma_attributes();
cudaError_t init_gemv_attributes();
cudaError_t init_scatter_attributes();
cudaError_t init_bulk_attributes();
bool bulk_scatter_eligible(const moe_rd_params& p);

static size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

// Columns of the tensor-core product: an fp32 weight is split into bf16 hi and lo
// rows (wsplit_kernel of the reference, kernel.cu:1786-1824), which doubles them.
static int umma_columns(const moe_rd_params& p) { return p.w_dtype == MOE_RD_W_F32 ? 2 * p.E : p.E; }

static bool umma_eligible(const moe_rd_params& p) {
  const int n = umma_columns(p);
  return umma_available() && p.E >= 16 && n <= 256 && n % 16 == 0 && p.H % 64 == 0 && p.T > 0;
}

int make_plan(const moe_rd_params& p, Plan* plan) {
  plan->ntiles = (int)((p.T + kTile - 1) / kTile);
  int gate = p.gate_impl;
  if (gate == MOE_RD_GATE_AUTO) {
    if (gemv_eligible(p))
      gate = MOE_RD_GATE_GEMV;
    else
      gate = (p.E >= 64 && umma_eligible(p)) ? MOE_RD_GATE_UMMA : MOE_RD_GATE_SIMT;
  }
  const bool one_cta = gate == MOE_RD_GATE_UMMA_ONE_CTA;
  if (one_cta) gate = MOE_RD_GATE_UMMA;
  if (gate == MOE_RD_GATE_UMMA && !umma_eligible(p)) return MOE_RD_E_UNSUPPORTED;
  if (gate == MOE_RD_GATE_GEMV && !gemv_eligible(p)) return MOE_RD_E_UNSUPPORTED;
  plan->gate = gate;
  plan->scatter = p.scatter_impl == MOE_RD_SCATTER_AUTO ? MOE_RD_SCATTER_SIMT : p.scatter_impl;
  // Split K only when the token tiles alone cannot fill the SMs (148): every
  // split writes and re-reads a [T,E] fp32 partial, which costs more than a
  // ragged last wave once there is at least one full wave of tiles.
  int ksplit = 1, mh = 1;
  if (gate == MOE_RD_GATE_UMMA) {
    // two 128-token halves per CTA share every weight tile (half the L2 reads of
    // W) once there are enough tokens to still fill the SMs
    mh = (p.T >= 4096 && umma_columns(p) <= 128) ? 2 : 1;  // at 256 columns it measured no faster and doubles the splits
    const int64_t mtiles = (p.T + 128 * mh - 1) / (128 * mh);
    const int kblocks = p.H / 64;
    while (ksplit < 8 && mtiles * ksplit * 2 <= 148 && kblocks / (ksplit * 2) >= 4) ksplit *= 2;
  }
  plan->umma_mh = mh;
  // many experts: the W tiles dominate the bytes a CTA pulls in, and a pair of
  // CTAs can share them
  plan->umma_fold = (gate == MOE_RD_GATE_UMMA && p.w_dtype == MOE_RD_W_F32) ? 1 : 0;
  plan->umma_n = umma_columns(p);
  plan->umma_pair = (gate == MOE_RD_GATE_UMMA && !one_cta && plan->umma_n > 128 && plan->umma_n % 32 == 0) ? 1 : 0;
  plan->ksplit = ksplit;
  plan->tile_major = (gate != MOE_RD_GATE_GEMV && p.T > 0) ? 1 : 0;
  return MOE_RD_OK;
}

void carve(const moe_rd_params& p, const Plan& plan, bool need_logits, bool need_ids,
           Workspace* w) {
  size_t o = 0;
  w->status = o; o += 256;
  w->tile_base = o; o += up256((size_t)p.E * plan.ntiles * 4);
  w->counts = o; o += up256((size_t)p.E * 4);
  w->group_counts = o; o += up256((size_t)p.E * ((plan.ntiles + kTileGroup - 1) / kTileGroup) * 4);
  w->dense = o; o += 256;
  w->zero_bytes = o;
  w->logits = o; if (need_logits) o += up256((size_t)p.T * p.E * 4);
  w->ids = o; if (need_ids) o += up256((size_t)p.T * p.K * 4);
  w->wt = o;
  if (plan.gate == MOE_RD_GATE_UMMA && (p.w_layout == MOE_RD_W_LAYOUT_HE || plan.umma_fold))
    o += up256((size_t)plan.umma_n * p.H * 2);
  w->partial = o;
  if (plan.gate == MOE_RD_GATE_UMMA) o += up256((size_t)plan.ksplit * p.T * plan.umma_n * 4);
  w->total = o;
}

static int validate(const moe_rd_params* p) {
  if (p == nullptr) return MOE_RD_E_NULL;
  if (p->T < 0 || p->T > ((int64_t)1 << 31) / (p->K > 0 ? p->K : 1) - 1) return MOE_RD_E_SHAPE;
  if (p->H < 8 || p->H % 8 != 0 || p->H > (1 << 20)) return MOE_RD_E_SHAPE;
  if (p->E < 1 || p->E > kMaxE) return MOE_RD_E_SHAPE;
  if (p->K < 1 || p->K > kMaxK || p->K > p->E) return MOE_RD_E_SHAPE;
  if (p->n_groups < 1 || p->n_groups > 32 || p->E % p->n_groups != 0) return MOE_RD_E_GROUPS;
  if (p->n_groups > 1) {
    const int gs = p->E / p->n_groups;
    if (p->topk_groups < 1 || p->topk_groups > p->n_groups || p->group_topk < 1 ||
        p->group_topk > gs || p->K > p->topk_groups * gs)
      return MOE_RD_E_GROUPS;
  }
  if (p->score_fn != MOE_RD_SCORE_SOFTMAX && p->score_fn != MOE_RD_SCORE_SIGMOID)
    return MOE_RD_E_ENUM;
  if (p->w_dtype != MOE_RD_W_F32 && p->w_dtype != MOE_RD_W_BF16) return MOE_RD_E_ENUM;
  if (p->w_layout != MOE_RD_W_LAYOUT_HE && p->w_layout != MOE_RD_W_LAYOUT_EH) return MOE_RD_E_ENUM;
  if (p->rows_format != MOE_RD_ROWS_BF16 && p->rows_format != MOE_RD_ROWS_FP8_E4M3_B128)
    return MOE_RD_E_ENUM;
  if (p->gate_impl < MOE_RD_GATE_AUTO || p->gate_impl > MOE_RD_GATE_UMMA_ONE_CTA) return MOE_RD_E_ENUM;
  if (p->scatter_impl < MOE_RD_SCATTER_AUTO || p->scatter_impl > MOE_RD_SCATTER_NONE)
    return MOE_RD_E_ENUM;
  if (p->rows_format == MOE_RD_ROWS_FP8_E4M3_B128 && p->H % 128 != 0) return MOE_RD_E_SHAPE;
  if (p->flags & ~(MOE_RD_FLAG_SKIP_IDENTITY_ROWS | MOE_RD_FLAG_TEST_GATE_STALL |
                   MOE_RD_FLAG_SEPARATE_GATE_AND_ROUTING))
    return MOE_RD_E_ENUM;
  if ((p->flags & MOE_RD_FLAG_SKIP_IDENTITY_ROWS) && p->rows_format != MOE_RD_ROWS_BF16)
    return MOE_RD_E_UNSUPPORTED;
  if (p->capacity < 0 || p->out_rows < 0 || p->out_rows > 0x7fffffff) return MOE_RD_E_SHAPE;
  if ((int64_t)p->E * ((p->T + kTile - 1) / kTile) > 0x7fffffff) return MOE_RD_E_TOO_LARGE;
  return MOE_RD_OK;
}

static bool misaligned(const void* p, size_t a) {
  return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0;
}

static cudaError_t init_device_once() {
  static std::mutex mu;
  static bool done[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (done[dev]) return cudaSuccess;
  e = init_route_attributes();
  if (e != cudaSuccess) return e;
  e = init_umma_attributes();
  if (e != cudaSuccess) return e;
  e = init_gemv_attributes();
  if (e != cudaSuccess) return e;
  e = init_scatter_attributes();
  if (e != cudaSuccess) return e;
  e = init_bulk_attributes();
  if (e != cudaSuccess) return e;
  done[dev] = true;
  return cudaSuccess;
}

}  // namespace moe_rd

using namespace moe_rd;

#define MOE_RD_CUDA(call)              \
  do {                                 \
    cudaError_t e__ = (call);          \
    if (e__ != cudaSuccess) {          \
      t_last_cuda = e__;               \
      return MOE_RD_E_CUDA;            \
    }                                  \
  } while (0)

extern "C" {

int moe_rd_version(void) { return MOE_RD_VERSION; }

int64_t moe_rd_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* moe_rd_last_cuda_error(void) { return cudaGetErrorString(t_last_cuda); }

const char* moe_rd_strerror(int code) {
  switch (code) {
    case MOE_RD_OK: return "ok";
    case MOE_RD_E_NULL: return "a required pointer is NULL";
    case MOE_RD_E_SHAPE: return "T/H/E/K/capacity/out_rows outside the supported range";
    case MOE_RD_E_GROUPS: return "inconsistent group-limited routing parameters";
    case MOE_RD_E_ALIGN: return "pointer not sufficiently aligned";
    case MOE_RD_E_WORKSPACE: return "workspace too small or not 256-byte aligned";
    case MOE_RD_E_ENUM: return "unknown enum value";
    case MOE_RD_E_CUDA: return "a CUDA call failed (see moe_rd_last_cuda_error)";
    case MOE_RD_E_UNSUPPORTED: return "combination not implemented";
    case MOE_RD_E_DEVICE: return "a device-side bound check failed (see moe_rd_read_status)";
    case MOE_RD_E_TOO_LARGE: return "problem exceeds a fixed-size resource";
    default: return "unknown error code";
  }
}

int moe_rd_workspace_bytes(const moe_rd_params* p, size_t* bytes) {
  if (bytes == nullptr) return MOE_RD_E_NULL;
  int rc = validate(p);
  if (rc != MOE_RD_OK) return rc;
  Plan plan;
  rc = make_plan(*p, &plan);
  if (rc != MOE_RD_OK) return rc;
  Workspace w;
  // Sized for the worst case (no caller-provided router_logits / expert_ids).
  carve(*p, plan, true, true, &w);
  *bytes = w.total;
  return MOE_RD_OK;
}

static int run_pipeline(const moe_rd_params* p, const moe_rd_buffers* b, void* workspace,
                        size_t workspace_bytes, cudaStream_t s, cudaEvent_t* ev) {
  int rc = validate(p);
  if (rc != MOE_RD_OK) return rc;
  if (b == nullptr || workspace == nullptr) return MOE_RD_E_NULL;
  Plan plan;
  rc = make_plan(*p, &plan);
  if (rc != MOE_RD_OK) return rc;
  if (plan.scatter == MOE_RD_SCATTER_BULK &&
      (!bulk_scatter_eligible(*p) || misaligned(b->scales, 16) || misaligned(b->permuted, 16)))
    return MOE_RD_E_UNSUPPORTED;
  if (b->offsets == nullptr) return MOE_RD_E_NULL;
  if (p->T > 0 && (b->x == nullptr || (b->permuted == nullptr && plan.scatter != MOE_RD_SCATTER_NONE) ||
                   b->inverse_perm == nullptr ||
                   b->combine_weights == nullptr))
    return MOE_RD_E_NULL;
  if (plan.gate == MOE_RD_GATE_EXTERNAL ? (p->T > 0 && b->router_logits == nullptr)
                                        : (p->T > 0 && b->gate_w == nullptr))
    return MOE_RD_E_NULL;
  if (p->rows_format == MOE_RD_ROWS_FP8_E4M3_B128 && p->T > 0 && b->scales == nullptr &&
      plan.scatter != MOE_RD_SCATTER_NONE)
    return MOE_RD_E_NULL;
  if (misaligned(b->x, 16) || misaligned(b->permuted, 16) || misaligned(b->gate_w, 16) ||
      misaligned(b->scales, 4))
    return MOE_RD_E_ALIGN;
  if (misaligned(workspace, 256)) return MOE_RD_E_WORKSPACE;
  // Without a capacity limit every pair is kept; with one, at most E*capacity.
  if (p->out_rows < p->T * p->K && (p->capacity == 0 || p->out_rows < (int64_t)p->E * p->capacity))
    return MOE_RD_E_SHAPE;

  // The fused GEMV keeps logits in shared memory; it writes them out only on request.
  const bool need_logits = plan.gate == MOE_RD_GATE_SIMT && b->router_logits == nullptr;
  const bool need_ids = b->expert_ids == nullptr;
  Workspace w;
  carve(*p, plan, need_logits, need_ids, &w);
  if (workspace_bytes < w.total) return MOE_RD_E_WORKSPACE;

  MOE_RD_CUDA(init_device_once());
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  int32_t* status = reinterpret_cast<int32_t*>(ws + w.status);
  int32_t* counts = reinterpret_cast<int32_t*>(ws + w.counts);
  float* logits = need_logits ? reinterpret_cast<float*>(ws + w.logits) : b->router_logits;
  int32_t* tile_base = reinterpret_cast<int32_t*>(ws + w.tile_base);
  int32_t* group_counts = reinterpret_cast<int32_t*>(ws + w.group_counts);
  int32_t* ids = need_ids ? reinterpret_cast<int32_t*>(ws + w.ids) : b->expert_ids;

  // status block, the tile counts and the expert counts are adjacent: one clear.  The
  // tensor-core gate clears them itself (its epilogue warps are idle while the
  // first tiles load), which saves the separate memset node.
  // (not in the time-out test: there a CTA may record its status within microseconds of the start,
  // before the first CTA has cleared the block)
  // Gate product and routing in one kernel where that pays (several token tiles per SM): its routing
  // warps add to the group counts while other CTAs are still starting, so the clear comes first.
  const bool fused = p->T > 0 && !(p->flags & MOE_RD_FLAG_SEPARATE_GATE_AND_ROUTING) &&
                     fused_front_eligible(*p, *b, plan);
  const bool gate_clears = plan.gate == MOE_RD_GATE_UMMA && p->T > 0 && !fused &&
                           !(p->flags & MOE_RD_FLAG_TEST_GATE_STALL);
  if (!gate_clears) MOE_RD_CUDA(cudaMemsetAsync(ws + w.status, 0, w.zero_bytes, s));
  if (ev) MOE_RD_CUDA(cudaEventRecord(ev[0], s));
  if (p->T > 0) {
    if (plan.gate == MOE_RD_GATE_SIMT) {
      MOE_RD_CUDA(launch_gate_simt(*p, *b, logits, s));
    } else if (fused) {
      MOE_RD_CUDA(launch_gate_route(*p, *b, plan, ws + w.wt, ids, tile_base, group_counts, status, s));
    } else if (plan.gate == MOE_RD_GATE_UMMA) {
      MOE_RD_CUDA(launch_gate_umma(*p, *b, plan, ws + w.wt,
                                   reinterpret_cast<float*>(ws + w.partial), logits, status,
                                   gate_clears ? ws + w.status : nullptr, w.zero_bytes, s));
    }
  }
  if (ev) MOE_RD_CUDA(cudaEventRecord(ev[1], s));
  if (p->T > 0) {
    if (fused) {
      // routed inside the gate kernel
    } else if (plan.gate == MOE_RD_GATE_GEMV)
      MOE_RD_CUDA(launch_gemv_route(*p, *b, plan, b->router_logits, ids, tile_base, counts, status + 16, s));
    else if (plan.gate == MOE_RD_GATE_UMMA)
      MOE_RD_CUDA(launch_route_splits(*p, *b, plan, reinterpret_cast<float*>(ws + w.partial),
                                      plan.ksplit, b->logit_bias, b->router_logits, ids, tile_base,
                                      counts, group_counts, s));
    else
      MOE_RD_CUDA(launch_route(*p, *b, plan, logits, ids, tile_base, counts, group_counts, s));
  }
  if (ev) MOE_RD_CUDA(cudaEventRecord(ev[2], s));
  // the fused GEMV kernel scans in its last block; after the routing kernel the positions kernel
  // derives bases and offsets itself; with T = 0 nothing ran: every offset and count is zero
  if (p->T == 0) {
    MOE_RD_CUDA(cudaMemsetAsync(b->offsets, 0, (size_t)(p->E + 1) * 4, s));
    if (b->counts != nullptr) MOE_RD_CUDA(cudaMemsetAsync(b->counts, 0, (size_t)p->E * 4, s));
  }
  if (ev) MOE_RD_CUDA(cudaEventRecord(ev[3], s));
  MOE_RD_CUDA(launch_scatter(*p, *b, plan, ids, tile_base, counts, status,
                             reinterpret_cast<int32_t*>(ws + w.dense), group_counts, s, ev ? ev[4] : nullptr));
  if (ev) MOE_RD_CUDA(cudaEventRecord(ev[5], s));
  return MOE_RD_OK;
}

int moe_rd_route_dispatch(const moe_rd_params* p, const moe_rd_buffers* b, void* workspace,
                          size_t workspace_bytes, void* stream) {
  return run_pipeline(p, b, workspace, workspace_bytes, static_cast<cudaStream_t>(stream), nullptr);
}

int moe_rd_route_dispatch_timed(const moe_rd_params* p, const moe_rd_buffers* b, void* workspace,
                                size_t workspace_bytes, void* stream, float stage_ms[5]) {
  if (stage_ms == nullptr) return MOE_RD_E_NULL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaEvent_t ev[6] = {};
  for (int i = 0; i < 6; ++i) {
    cudaError_t e = cudaEventCreate(&ev[i]);
    if (e != cudaSuccess) {
      for (int j = 0; j < i; ++j) cudaEventDestroy(ev[j]);
      t_last_cuda = e;
      return MOE_RD_E_CUDA;
    }
  }
  int rc = run_pipeline(p, b, workspace, workspace_bytes, s, ev);
  if (rc == MOE_RD_OK) {
    cudaError_t e = cudaStreamSynchronize(s);
    for (int i = 0; i < 5 && e == cudaSuccess; ++i)
      e = cudaEventElapsedTime(&stage_ms[i], ev[i], ev[i + 1]);
    if (e != cudaSuccess) {
      t_last_cuda = e;
      rc = MOE_RD_E_CUDA;
    }
  }
  for (int i = 0; i < 6; ++i) cudaEventDestroy(ev[i]);
  return rc;
}

int moe_rd_read_status(const void* workspace, void* stream, int32_t status[8]) {
  if (workspace == nullptr || status == nullptr) return MOE_RD_E_NULL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  MOE_RD_CUDA(cudaMemcpyAsync(status, workspace, 32, cudaMemcpyDeviceToHost, s));
  MOE_RD_CUDA(cudaStreamSynchronize(s));
  return status[0] != 0 ? MOE_RD_E_DEVICE : MOE_RD_OK;
}

}  // extern "C"
