/*
 * moe_rd — MoE sparse routing and dispatch for NVIDIA B200 (sm_100a).
 *
 * C ABI of libmoe_rd.so.  Plain pointers and sizes only; every pointer in
 * moe_rd_buffers is DEVICE memory owned by the caller, and the library never
 * allocates or frees on a call path (destination passing).  All work is
 * enqueued on the caller's stream; no entry point synchronises the host
 * unless its comment says so.  Functions return 0 or a negative MOE_RD_E_*.
 *
 * "Reference" below is ernie-research/ERNIE-Evolve-Results; citations are
 * relative to sol-execbench/029_moe_sparse_routing_and_dispatch/.
 */
#ifndef MOE_RD_H_
#define MOE_RD_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOE_RD_VERSION 1

/* error codes */
#define MOE_RD_OK 0
#define MOE_RD_E_NULL (-1)        /* a required pointer is NULL */
#define MOE_RD_E_SHAPE (-2)       /* T/H/E/K outside the supported range */
#define MOE_RD_E_GROUPS (-3)      /* group-limited routing parameters inconsistent */
#define MOE_RD_E_ALIGN (-4)       /* pointer or row pitch not 16-byte aligned */
#define MOE_RD_E_WORKSPACE (-5)   /* workspace too small or misaligned */
#define MOE_RD_E_ENUM (-6)        /* unknown enum value */
#define MOE_RD_E_CUDA (-7)        /* a CUDA call failed; see moe_rd_last_cuda_error */
#define MOE_RD_E_UNSUPPORTED (-8) /* combination not implemented */
#define MOE_RD_E_DEVICE (-9)      /* device-side check failed; see moe_rd_read_status */
#define MOE_RD_E_TOO_LARGE (-10)  /* problem exceeds a fixed-size resource */

/* enums (int32 fields of moe_rd_params) */
enum { MOE_RD_SCORE_SOFTMAX = 0, MOE_RD_SCORE_SIGMOID = 1 };
enum { MOE_RD_W_F32 = 0, MOE_RD_W_BF16 = 1 };
enum { MOE_RD_W_LAYOUT_HE = 0 /* [H,E] row-major */, MOE_RD_W_LAYOUT_EH = 1 /* [E,H] */ };
enum { MOE_RD_ROWS_BF16 = 0, MOE_RD_ROWS_FP8_E4M3_B128 = 1 };
enum {
  MOE_RD_GATE_AUTO = 0,     /* E <= 32: fused warp GEMV; E >= 64: tcgen05 where MOE_RD_GATE_UMMA is
                               available; otherwise the SIMT product */
  MOE_RD_GATE_SIMT = 1,     /* fixed-order fp32 FMA product, any E (defines the logit bits) */
  MOE_RD_GATE_UMMA = 2,     /* tcgen05/TMEM tiles fed by TMA.  bf16 weights: E % 16 == 0, E <= 256.
                               fp32 weights: split per call into bf16 hi = bf16(W) and
                               lo = bf16(W - hi) rows and folded as z = D[e] + D[E+e], which the
                               reference does to get an fp32-weight product from a bf16 MMA
                               (wsplit_kernel, kernel.cu:1786-1824, 1849-1851); E % 8 == 0, E <= 128 */
  MOE_RD_GATE_EXTERNAL = 3, /* logits supplied by the caller in router_logits */
  MOE_RD_GATE_GEMV = 4,     /* warp GEMV fused with scoring/top-k (E <= 32, weight fits in
                               shared memory); same logit bits as MOE_RD_GATE_SIMT */
  MOE_RD_GATE_UMMA_ONE_CTA = 5 /* MOE_RD_GATE_UMMA without the two-CTA tiles it uses for E > 128 */
};
enum {
  MOE_RD_SCATTER_AUTO = 0,
  MOE_RD_SCATTER_SIMT = 1,
  MOE_RD_SCATTER_BULK = 2,
  MOE_RD_SCATTER_NONE = 3 /* routing, offsets and inverse permutation only; rows are moved by
                             moe_rd_ep_scatter (expert-parallel dispatch) */
};

/*
 * Problem description.  Replaces the compile-time constants NE/TOPK and the
 * scalar arguments of the reference's run() (kernel.cu:1582-1583, 4067-4077).
 */
typedef struct moe_rd_params {
  int64_t T;            /* tokens (rows of x) */
  int32_t H;            /* hidden size; H % 8 == 0, and H % 128 == 0 for fp8 rows */
  int32_t E;            /* experts, 1..256 */
  int32_t K;            /* experts per token, 1..32, K <= E */
  int32_t n_groups;     /* 1 = no group limit; else E % n_groups == 0, n_groups <= 32 */
  int32_t topk_groups;  /* groups kept per token */
  int32_t group_topk;   /* a group's score = sum of its group_topk largest keys */
  int32_t score_fn;     /* MOE_RD_SCORE_* */
  int32_t weight_from_key; /* 1: weights from score+select_bias as the reference does
                              (kernel.cu:1891,1909); 0: from the unbiased score */
  int32_t renorm;       /* 1: w = u / max(sum u, norm_min) */
  float routed_scale;   /* weights are multiplied by this last */
  float norm_min;       /* the reference's norm_min (kernel.cu:1909) */
  int64_t capacity;     /* rows kept per expert, 0 = unlimited; pairs beyond it are
                           dropped in token order */
  int64_t out_rows;     /* rows the caller allocated in permuted/scales (>= kept pairs;
                           T*K always suffices) */
  int32_t rows_format;  /* MOE_RD_ROWS_* */
  int32_t w_dtype;      /* MOE_RD_W_* */
  int32_t w_layout;     /* MOE_RD_W_LAYOUT_* */
  int32_t gate_impl;    /* MOE_RD_GATE_* */
  int32_t scatter_impl; /* MOE_RD_SCATTER_* */
  int32_t flags;        /* MOE_RD_FLAG_* bits, 0 by default */
} moe_rd_params;

/*
 * MOE_RD_FLAG_SKIP_IDENTITY_ROWS (bf16 rows): an expert that received every one
 * of the T tokens (none dropped) holds them exactly once each and in token
 * order, so its slice of `permuted` would be a verbatim copy of x.  With this
 * flag the rows of such experts are not written (their positions in offsets /
 * inverse_perm stay as they are); moe_rd_gemm_plan aims the A pointer of those
 * groups at x instead.  Same shortcut as ident_a / ident_m of the reference
 * (moe_gemm.h:66-75, kernel.cu:2089-2108, 2154).
 */
enum {
  MOE_RD_FLAG_SKIP_IDENTITY_ROWS = 1,
  /* For tests of the time-out path only.  Every wait inside the tensor-core gate
   * kernel is bounded; when one runs out, the kernel records a status (ids
   * 101-103, 111, 112), waits for its own copies in flight, frees its tensor
   * memory and returns, and the call completes with meaningless outputs.  With
   * this flag the kernel's producer issues no loads at all (so nothing is in
   * flight) and the limit is a few hundred polls, which makes that path run:
   * moe_rd_read_status then returns MOE_RD_E_DEVICE and the next call on the same
   * workspace works normally.  Ignored by the other gate implementations. */
  MOE_RD_FLAG_TEST_GATE_STALL = 2,
  /* Keep the gate product and the routing in two kernels where the library would otherwise run them
   * as one (several token tiles per SM, no split over K, at most 128 product columns).  Same results;
   * for measuring the gate product alone. */
  MOE_RD_FLAG_SEPARATE_GATE_AND_ROUTING = 4
};

/*
 * Device buffers.  The data contract between routing and expert compute that
 * the reference keeps in its arena (kernel.cu:4208-4222, 4304-4306): sel,
 * wsel, offs/cursor, inv, xg, router_logits.
 */
typedef struct moe_rd_buffers {
  const void* x;             /* [T,H] bf16 row-major, 16-byte aligned */
  const void* gate_w;        /* [H,E] or [E,H], fp32 or bf16 */
  const float* logit_bias;   /* [E] added to the logits before scoring, or NULL */
  const float* select_bias;  /* [E] added to the scores to form selection keys, or NULL
                                (the reference's e_score_correction_bias) */
  void* permuted;            /* [out_rows,H] bf16, or [out_rows,H] fp8-e4m3 bytes */
  float* scales;             /* [out_rows,H/128] fp32 (fp8 rows only) */
  int32_t* offsets;          /* [E+1] first row of each expert, offsets[E] = kept pairs */
  int32_t* inverse_perm;     /* [T,K] row of pair (t,k) in permuted, -1 if dropped */
  float* combine_weights;    /* [T,K] */
  int32_t* expert_ids;       /* [T,K] slot k = k-th pick, or NULL */
  uint8_t* drop_mask;        /* [T,K] 1 = dropped by the capacity limit, or NULL */
  float* router_logits;      /* [T,E] fp32: optional output; INPUT for MOE_RD_GATE_EXTERNAL */
  int32_t* counts;           /* [E] pairs routed to each expert before dropping, or NULL */
  int32_t* row_token;        /* [out_rows] token of each permuted row (the reference's forward
                                permutation `tok` / `ptok`, kernel.cu:2172-2177), or NULL */
  float* row_weight;         /* [out_rows] combine weight of each permuted row (`pw`), or NULL */
} moe_rd_buffers;

/* Bytes of scratch moe_rd_route_dispatch needs for these parameters. */
int moe_rd_workspace_bytes(const moe_rd_params* p, size_t* bytes);

/*
 * Router -> top-k -> offsets -> dispatch -> row scatter, steps 1-6 of the
 * reference's run() (kernel.cu:4323-4430: wsplit_kernel, the router GEMM,
 * topk_kernel, offsets_kernel, dispatch_kernel, gather_kernel), enqueued on
 * `stream` (a cudaStream_t) with no host synchronisation.  `workspace` is
 * device memory, 256-byte aligned, of at least moe_rd_workspace_bytes bytes.
 * Nothing is allocated and nothing read back, so the call may be recorded into a
 * CUDA graph (stream capture) after one plain call has set the per-device
 * function attributes; the graph holds the buffer addresses of the recorded call.
 */
int moe_rd_route_dispatch(const moe_rd_params* p, const moe_rd_buffers* b,
                          void* workspace, size_t workspace_bytes, void* stream);

/*
 * moe_rd_route_dispatch without a workspace argument, for callers that must
 * not (or cannot) allocate device memory: a plug-in inside a host program that
 * hands out every byte of device memory itself and treats a later cudaMalloc
 * as an error, a service that froze its memory pool after start-up, or a bare
 * C client with no allocator to carve a workspace from.  The scratch is a fixed
 * array of MOE_RD_NOALLOC_MAX_BYTES inside the library's device image; every
 * GPU that loads the library keeps that much reserved until the process exits.
 * The caller still passes all inputs and outputs in `b`.
 *
 * - Problems whose moe_rd_workspace_bytes() exceeds MOE_RD_NOALLOC_MAX_BYTES are
 *   refused with MOE_RD_E_TOO_LARGE before anything is launched.  That size is the
 *   worst case (it includes room for the logits and expert ids even when the
 *   caller passes router_logits / expert_ids buffers of its own), so a problem
 *   can be refused although this particular call would have needed less.
 * - `stream` must belong to the current device (MOE_RD_E_UNSUPPORTED otherwise):
 *   the scratch address is looked up for the current device.
 * - moe_rd_read_status_noalloc reads the device status block of the last such
 *   call on the current device (synchronises `stream`), as moe_rd_read_status
 *   does for a caller-owned workspace.
 * - The call itself makes no cudaMalloc/cudaFree and uses no allocating library.
 * - The first call on each device looks up the array's device address (and, as
 *   with moe_rd_route_dispatch, sets kernel attributes); make that first call
 *   before starting any stream capture on that device.
 * - All calls on a device share the one array.  Each call clears what it needs
 *   zeroed, so calls that follow each other on a stream are fine, but two calls
 *   whose kernels can overlap on the GPU (different streams, no ordering) race
 *   on the scratch and corrupt each other.
 * This entry point has no counterpart in the reference, whose run() allocates
 * its arena with at::empty on every call (kernel.cu:4202-4268).
 */
#define MOE_RD_NOALLOC_MAX_BYTES (32u << 20)
int moe_rd_route_dispatch_noalloc(const moe_rd_params* p, const moe_rd_buffers* b, void* stream);
int moe_rd_read_status_noalloc(void* stream, int32_t status[8]);

/*
 * Expert-parallel receive side.  After an all-to-all delivered, from every
 * source rank s, that rank's rows for this rank's experts (rank-major:
 * [s][local expert][rows], with cnt[s][le] rows each), reorder them into the
 * expert-major buffer an expert GEMM consumes: [local expert][s][rows], and
 * write local_offsets[experts_per_rank+1].  recv_scales/out_scales may both be
 * NULL (bf16 rows).  `status` is an 8-word device block cleared by the caller;
 * word 0 is set if the counts add up to more than max_rows.  The reference has
 * no expert parallelism; its only counts-then-rows exchange is
 * nanogpt-speedrun/track-1/track_1_short/sharded_rows.py:72-103.
 */
int moe_rd_ep_unpack(const int32_t* cnt, int world, int experts_per_rank, const void* recv_rows,
                     const float* recv_scales, void* out_rows, float* out_scales,
                     int32_t* local_offsets, int64_t row_bytes, int32_t scale_floats,
                     int64_t max_rows, int32_t* status, void* stream);

/*
 * Expert-parallel dispatch by direct peer stores (one kernel moves the rows and
 * crosses NVLink; no send buffer, no receive-side reorder).  Rank `rank` of
 * `world` owns experts [rank*E/world, (rank+1)*E/world).
 *
 * moe_rd_ep_plan: from kept_all[world][E] (rows every rank dispatches to every
 * expert, gathered beforehand) computes, on this rank, dest_base[E] = the row in
 * the owner's buffer where THIS rank's rows for expert e start (experts of an
 * owner are contiguous, and inside an expert rows are ordered by source rank),
 * cnt[world][E/world] = rows this rank receives per (source, local expert), and
 * local_offsets[E/world + 1].  max_rows is the number of rows of EVERY rank's
 * buffer.  If the rows of an expert would end past max_rows in its owner's
 * buffer, status word 0 is set (id 202) on every rank, that expert gets
 * dest_base = -1 everywhere, and moe_rd_ep_scatter / moe_rd_ep_combine skip its
 * pairs: nothing is stored or loaded outside a buffer.
 *
 * moe_rd_ep_scatter: for every kept pair (t,k) of this rank, row
 * dest_base[e] + (inverse_perm[t,k] - offsets[e]) of the owner's buffer
 * peer_rows[e / (E/world)] receives the token row (bf16 copy or fp8 bytes plus
 * scales into peer_scales[..]).  peer_rows/peer_scales are host arrays of
 * `world` device pointers that this GPU can store to (peer-mapped memory; the
 * entry for `rank` is local).  Plain 16-byte stores; no multicast.  The caller
 * orders a cross-rank barrier after it before anyone reads the buffers.
 * p->scatter_impl = MOE_RD_SCATTER_BULK moves whole rows with cp.async.bulk
 * through shared memory instead (needs `status`, an 8-word device block).  With
 * bulk copies and fp8 rows peer_scales may be NULL: a row of peer_rows[d] is then
 * H bytes followed by its H/128 fp32 scales (pitch H + H/32 bytes), and a pair
 * crosses NVLink as ONE copy instead of two.
 * Run the local pipeline with MOE_RD_SCATTER_NONE first.  No counterpart in the
 * reference (it has no expert parallelism).
 */
int moe_rd_ep_plan(const int32_t* kept_all, int world, int rank, int E, int64_t max_rows,
                   int32_t* dest_base, int32_t* cnt, int32_t* local_offsets, int32_t* status,
                   void* stream);
int moe_rd_ep_scatter(const moe_rd_params* p, const void* x, const int32_t* expert_ids,
                      const int32_t* inverse_perm, const int32_t* offsets,
                      const int32_t* dest_base, int world, void* const* peer_rows,
                      float* const* peer_scales, int32_t* status, void* stream);

/*
 * Send-once form of moe_rd_ep_scatter (bulk copies only): a token with several
 * experts on one REMOTE rank crosses NVLink once.  The first of its pairs that
 * has a row there carries the bytes; for every later pair the kernel stores only
 *   peer_copy_of[d][row of that pair] = row of the first pair       (4 bytes)
 * in the owner's memory.  After the cross-rank barrier every owner runs
 * moe_rd_ep_replicate on its own buffer: each row r < *n_rows with
 * copy_of[r] >= 0 is copied from that row (local HBM traffic) and the mark is
 * reset to -1.  The buffers end up exactly as moe_rd_ep_scatter leaves them.
 * With group-limited routing (at most 4 of 8 expert groups per token) this
 * halves the NVLink bytes on 8 ranks and quarters them on 2.  Pairs bound for
 * `rank` itself are written directly, as before.
 * peer_copy_of: host array of `world` device pointers to int32 [max_rows], every
 * element -1 before the first use (the owner's own replicate keeps it so).
 * moe_rd_ep_replicate: rows / scales / copy_of are this rank's buffers (scales
 * NULL for bf16 rows and for the packed fp8 layout), n_rows a device int32
 * (local_offsets[E/world] of moe_rd_ep_plan), status an 8-word device block.
 */
int moe_rd_ep_scatter_once(const moe_rd_params* p, const void* x, const int32_t* expert_ids,
                           const int32_t* inverse_perm, const int32_t* offsets,
                           const int32_t* dest_base, int world, int rank, void* const* peer_rows,
                           float* const* peer_scales, int32_t* const* peer_copy_of, int32_t* status,
                           void* stream);
int moe_rd_ep_replicate(const moe_rd_params* p, void* rows, float* scales, int32_t* copy_of,
                        const int32_t* n_rows, int64_t max_rows, int32_t* status, void* stream);

/*
 * Weighted combine, the consumer of inverse_perm and combine_weights:
 *   out[t,:] = shared[t,:] + sum_k combine_weights[t,k] * y[inverse_perm[t,k],:]
 * y [rows,H] bf16 are the expert outputs in the permuted (expert-major) order,
 * shared [T,H] bf16 may be NULL, out [T,H] bf16.  fp32 accumulation from the
 * shared row, one fused multiply-add per slot in slot order, one rounding to
 * bf16: the arithmetic of the reference's combine_kernel (kernel.cu:2365-2428).
 * Dropped pairs (inverse_perm < 0) are skipped.
 */
int moe_rd_combine(int64_t T, int32_t H, int32_t K, const void* y, const int32_t* inverse_perm,
                   const float* combine_weights, const void* shared, void* out, void* stream);

/*
 * Residual (accumulating) combine over expert-major rows, the reference's
 * raddleft_kernel (kernel.cu:2451-2486), for a pipeline in which most expert
 * outputs were already reduced into `out` and only the first *n_rows rows of y
 * are left to fold in:
 *   out[row_token[p],:] += bf16(row_weight[p] * y[p,:])     for p < min(*n_rows, max_rows)
 * y [max_rows,H] bf16; row_token / row_weight as moe_rd_buffers returns them
 * (rows with row_token < 0 are skipped); n_rows is a DEVICE int32 (for example
 * &offsets[E]), so the count is never read back; out [T,H] bf16 is updated in
 * place.  The product is rounded to bf16 and added with an element-wise bf16
 * reduction (red.global.add.noftz, kernel.cu:2446-2449): exact when every token
 * receives at most one row; with several rows per token the adds reach an
 * element in no fixed order and the last bits depend on it, as in the reference.
 */
int moe_rd_combine_add_rows(int32_t H, int64_t max_rows, const void* y, const int32_t* row_token,
                            const float* row_weight, const int32_t* n_rows, void* out, void* stream);

/*
 * Same work as moe_rd_route_dispatch, but with a CUDA event recorded on
 * `stream` between the stages; synchronises the stream and returns the device
 * time of each stage in milliseconds: stage_ms[0] gate product, [1] scoring /
 * top-k / expert histogram (with the fused GEMV gate the product and the scans
 * are in here), [2] unused (no separate scan kernel is launched), [3] positions
 * (tile bases, offsets, inverse permutation), [4] row scatter.  For measurement only
 * (the reference's per-kernel figures come from an external profiler,
 * kernel.cu:865-890); it creates and destroys events, so keep it off hot paths.
 */
int moe_rd_route_dispatch_timed(const moe_rd_params* p, const moe_rd_buffers* b,
                                void* workspace, size_t workspace_bytes, void* stream,
                                float stage_ms[5]);

/*
 * Copies the 8-word device status block of the last call that used
 * `workspace` to the host (synchronises `stream`).  status[0] != 0 means a
 * device-side bound check failed (the offending access was skipped);
 * status[1..3] hold the check id and the bad values.  Returns
 * MOE_RD_E_DEVICE in that case.  The reference has no counterpart: it relies
 * on external compute-sanitizer runs (kernel.cu:4193-4195).
 */
int moe_rd_read_status(const void* workspace, void* stream, int32_t status[8]);

/*
 * Expert-parallel weighted combine: the return path of moe_rd_ep_scatter and the
 * un-permute in one kernel.  The expert outputs stay on the ranks that own the
 * experts, in buffers laid out like the dispatch's receive buffers
 * (peer_y[d] = rank d's [rows, H] bf16 output, mapped into this process); the
 * row of pair (t,k), expert e = expert_ids[t,k], is row
 * dest_base[e] + (inverse_perm[t,k] - offsets[e]) of peer_y[e / (E / world)]
 * (dest_base from moe_rd_ep_plan) and is read from there with 16-byte loads over
 * NVLink.  Arithmetic as moe_rd_combine.  The caller orders the kernel after
 * every rank's outputs are written (a barrier on the stream) and keeps the
 * buffers alive until every rank's kernel has finished.  The reference has no
 * counterpart (single GPU); it is the second half of the exchange of its
 * sharded_rows.py precedent.
 */
int moe_rd_ep_combine(int64_t T, int32_t H, int32_t K, int32_t E, int32_t world,
                      const void* const* peer_y, const int32_t* expert_ids,
                      const int32_t* inverse_perm, const float* combine_weights,
                      const int32_t* offsets, const int32_t* dest_base, const void* shared,
                      void* out, void* stream);

/*
 * One group of a grouped (ragged) expert GEMM  D[m,n] = A[m,k] * B_e : what
 * plan_kernel of the reference builds per expert on the device from the routed
 * offsets (moe_gemm.cu:613-638: problem shape, A / B / D pointers, leading
 * dimensions), as plain integers and pointers.
 */
typedef struct moe_rd_gemm_group {
  int32_t m, n, k;      /* rows of this expert, output columns, reduction length */
  int32_t identity;     /* 1: A is aimed at ident_a (every token once, in token order) */
  const void* a;        /* first row of the group's A operand */
  const void* b;        /* this expert's weight */
  void* d;              /* first row of the group's output */
  int64_t lda, ldb, ldd; /* row pitches in bytes of A and D, bytes per expert of B */
} moe_rd_gemm_group;

/*
 * Builds groups[E] on the device from offsets[E+1] with no host
 * synchronisation.  a_rows is the permuted buffer (row pitch a_row_bytes), w
 * the stacked expert weights (w_expert_bytes apart), d_rows the output (row
 * pitch d_row_bytes).  ident_a / ident_m: when ident_m > 0, a group with
 * exactly ident_m rows reads ident_a (the un-permuted x) instead of its slice
 * of a_rows (see MOE_RD_FLAG_SKIP_IDENTITY_ROWS).
 */
int moe_rd_gemm_plan(const int32_t* offsets, int32_t E, const void* a_rows, int64_t a_row_bytes,
                     const void* ident_a, int64_t ident_m, const void* w, int64_t w_expert_bytes,
                     void* d_rows, int64_t d_row_bytes, int32_t n, int32_t k,
                     moe_rd_gemm_group* groups, void* stream);

/*
 * Per-expert statistics of one routing pass, as first-class outputs (the
 * reference keeps wsum / counts for its own use, kernel.cu:1903-1919):
 * weight_sum[e] = sum of row_weight over the expert's kept rows, added in a
 * fixed order (element i goes to partial i % 256 in ascending order, the 256
 * partials are combined by the tree v[i] += v[i + off], off = 128..1), so the
 * result does not depend on scheduling; mean_weight[e] = weight_sum[e] /
 * max(rows, 1); load[e] = rows / max(total kept rows, 1).  Any output may be NULL.
 */
int moe_rd_expert_stats(const int32_t* offsets, const float* row_weight, int32_t E,
                        float* weight_sum, float* mean_weight, float* load, void* stream);

/* Kernels this library launched since it was loaded (all threads). */
int64_t moe_rd_launch_count(void);

const char* moe_rd_strerror(int code);
/* cudaError_t of the last failed CUDA call on this thread, as text. */
const char* moe_rd_last_cuda_error(void);
int moe_rd_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MOE_RD_H_ */
