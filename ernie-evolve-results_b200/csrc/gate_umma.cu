// Gate logits on the 5th-generation tensor cores: D[128 tokens, E] (fp32, in
// TMEM) += x[128, 64] * W^T[64, E] per 64-wide K block, operands staged in
// shared memory by TMA (no multicast), MMAs issued by one thread with
// tcgen05.mma, accumulator read back with tcgen05.ld.
//
// Replaces the library router GEMM of the reference (cublasGemmEx,
// kernel.cu:4327-4339; the reference ships no hand-written tcgen05 code for
// it).  One CTA owns one 128-token tile and one K split; it writes raw fp32
// partial products [split][T][E]; the routing kernel adds the splits in a fixed
// order (plus the logit bias), so the result does not depend on scheduling.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..5 =
// epilogue (a warp may only touch TMEM lanes 32*(warp%4)..+31, and 2,3,4,5 mod 4
// cover all four quarters).  Every mbarrier wait is bounded: on expiry the
// kernel records a status code, raises a CTA-wide abort flag, skips the
// remaining work, frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"
#include "route_lane.cuh"

namespace moe_rd {
namespace {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;   // 64 bf16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr uint32_t kSpinLimit = 1u << 20;

// Tuning constants (defaults are the measured best).
#ifndef MOE_RD_UMMA_L2_PROMOTION
#define MOE_RD_UMMA_L2_PROMOTION CU_TENSOR_MAP_L2_PROMOTION_L2_128B
#endif
#ifndef MOE_RD_UMMA_SMEM_KB_ONE_CTA   // shared-memory budget when one CTA owns the SM
#define MOE_RD_UMMA_SMEM_KB_ONE_CTA 200
#endif
#ifndef MOE_RD_UMMA_SMEM_KB_TWO_CTA   // ... when two CTAs share it
#define MOE_RD_UMMA_SMEM_KB_TWO_CTA 100
#endif
#ifndef MOE_RD_FUSED_FRONT   // 0: never fuse the routing into the gate kernel (tuning/validation)
#define MOE_RD_FUSED_FRONT 1
#endif
#ifndef MOE_RD_UMMA_TWO_CTA_MAX_E     // largest E for which two CTAs per SM are targeted
#define MOE_RD_UMMA_TWO_CTA_MAX_E 128
#endif

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
// Bounded wait; false when the limit ran out or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t limit = kSpinLimit) {
  for (uint32_t it = 0; it < limit; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}

// Non-blocking look at a barrier phase.  The answer is consumed later, so the
// shared-memory round trip overlaps with the instructions issued in between.
__device__ __forceinline__ uint32_t mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Position in a ring of `stages` slots: the slot and the phase parity to wait
// for.  The producer and the MMA issuer are single threads whose instruction
// count per K block bounds the K loop (measured: with the slot, phase and
// descriptors recomputed from the block index by division, the MMA thread alone
// took 0.43 us per block where the tensor pipe needs 0.28), so everything that
// can be stepped is stepped.
struct Ring {
  uint32_t s, ph;
  __device__ __forceinline__ void next(uint32_t stages) {
    if (++s == stages) {
      s = 0;
      ph ^= 1u;
    }
  }
};

// L2 policy for the loads of x: keep the lines if possible.  The row scatter reads x again right
// after the routing front, and whatever part of x is still in L2 then does not come from HBM a
// second time (measured on T=8192, H=7168: scatter 100.2 -> 97.2 us).
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d_keep(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, groups of 8
// rows 1024 bytes apart (stride byte offset), leading byte offset unused (1).
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version of this architecture
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

// MN-major operand tile (rows = K, 64 elements of N per 128-byte row) with
// 128-byte swizzle: the 8 K-rows of a group are 128 bytes apart, groups of 8
// K-rows 1024 bytes apart (stride byte offset), blocks of 64 N-elements
// `n_block_bytes` apart (leading byte offset).
__device__ __forceinline__ uint64_t make_desc_mn(uint32_t smem_addr, uint32_t n_block_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)((n_block_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

__device__ __forceinline__ void bulk_store_row(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(src_smem), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// ---- helpers of the two-CTA (cta_group::2) kernel -------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load of one CTA of a pair; the bytes are counted on `bar`, a barrier of
// the pair's leader CTA (cluster address).  No multicast: each CTA fetches
// only what lands in its own shared memory.
__device__ __forceinline__ void tma_load_2d_pair_keep(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                      uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// One MMA over both CTAs of the pair: D[256, N] += A[256, 16] * B[16, N]; each
// CTA supplies its 128 rows of A and its N/2 columns of B from the same
// shared-memory offsets and keeps its 128 rows of D in its own TMEM.
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t da, uint64_t db,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this offset in both CTAs of the pair once all MMAs
// issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3)
      : "memory");
}

struct UmmaArgs {
  float* partial;  // [ksplit][T][E]
  int32_t* status;
  int64_t T;
  int E, kblocks, ksplit, stages, tmem_cols;
  int w_mn_major;  // 1: map_w is over W[H,E] and B tiles are MN-major; 0: over W^T[E,H], K-major
  int mh;          // 128-token halves per CTA (1 or 2): two halves share every W tile
  uint4* zero;     // region the epilogue warps clear while the first tiles load (or null)
  uint32_t zero_vecs;
  uint32_t spin_limit;  // polls a wait may take before the kernel gives up
  int no_loads;    // MOE_RD_FLAG_TEST_GATE_STALL: the producer issues nothing, so the waits run out
};

// Epilogue of one CTA (warps 2..5; TMEM lane = token row of the tile): waits for
// the accumulator, parks every row in the free operand ring and writes it out
// with one bulk copy.  `mt` numbers 128*mh-row tiles.
__device__ __forceinline__ void epilogue_rows(const UmmaArgs& a, unsigned char* smem, uint32_t tmem_base,
                                              uint64_t* accum_bar, volatile int* abort_flag, int warp,
                                              int lane, int mt, int ks) {
    const int q = warp & 3;
    if (a.zero != nullptr) {
      // Clear the counters of the later kernels while the first tiles are on
      // their way (the routing kernel starts after this grid has finished).
      // The region starts with the status block (16 vectors).  Only the first CTA clears
      // that, at its very start: a CTA of a later wave must not wipe a time-out another
      // CTA has recorded there (a report is at least 2^20 polls after the kernel began).
      const uint32_t nthr = gridDim.x * gridDim.y * 128u;
      const uint32_t cta = blockIdx.y * gridDim.x + blockIdx.x;
      const uint32_t me = cta * 128u + (uint32_t)(q * 32 + lane);
      for (uint32_t i = me; i < a.zero_vecs; i += nthr)
        if (i >= 16u || cta == 0u) a.zero[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    bool ok = mbar_wait(smem_u32(accum_bar), 0u, abort_flag, a.spin_limit);
    ok = __all_sync(kFull, ok);
    if (!ok) {
      if (lane == 0 && !*abort_flag) report(a.status, 103, mt, ks);
      *abort_flag = 1;
    } else {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // All MMAs have completed, so the operand ring is free: every thread parks
      // its token row there (row pitch E*4 + 16 bytes keeps the 16-byte stores of
      // a warp on different banks) and sends it to memory with one bulk copy.
      const uint32_t pitch = (uint32_t)a.E * 4u + 16u;
      unsigned char* my_row = smem + (size_t)(q * 32 + lane) * pitch;
      for (int h = 0; h < a.mh; ++h) {
        const int64_t row = ((int64_t)mt * a.mh + h) * kBlockM + q * 32 + lane;
        if (h > 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        for (int c = 0; c < a.E; c += 32) {
          uint32_t r[32];
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * a.E + c);
          if (a.E - c >= 32) {
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                  "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
                  "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                  "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                  "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
                  "=r"(r[31])
                : "r"(taddr)
                : "memory");
          } else {
            // E % 32 == 16: the last 16 columns
#pragma unroll
            for (int i = 16; i < 32; ++i) r[i] = 0u;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                  "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
                  "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(taddr)
                : "memory");
          }
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          const int n = a.E - c >= 32 ? 32 : 16;
          uint4* o4 = reinterpret_cast<uint4*>(my_row + (size_t)c * 4);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (4 * i < n) o4[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (row < a.T)
          bulk_store_row(a.partial + ((size_t)ks * a.T + row) * a.E, smem_u32(my_row), (uint32_t)a.E * 4u);
      }
      // the rows must have left shared memory before the CTA may go; their arrival in global
      // memory is ordered before the next kernel by the end of this grid
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
}

__global__ void __launch_bounds__(kThreads, 1)
gate_umma_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const UmmaArgs a) {
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t half_bytes = kBlockM * kBlockK * 2;
  const uint32_t a_bytes = (uint32_t)a.mh * half_bytes;
  const uint32_t b_bytes = (uint32_t)a.E * kBlockK * 2;
  const uint32_t stage_bytes = a_bytes + b_bytes;
  unsigned char* tail = smem + (size_t)a.stages * stage_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
  uint64_t* empty_bar = full_bar + a.stages;
  uint64_t* accum_bar = empty_bar + a.stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = blockIdx.x, ks = blockIdx.y;
  const int kb0 = (int)((int64_t)ks * a.kblocks / a.ksplit);
  const int kb1 = (int)((int64_t)(ks + 1) * a.kblocks / a.ksplit);
  const int nkb = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(smem_u32(full_bar + s), 1);
      mbar_init(smem_u32(empty_bar + s), 1);
    }
    mbar_init(smem_u32(accum_bar), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"((uint32_t)a.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      const uint64_t keep_x = policy_evict_last();
      int issued = 0;
      Ring r{0u, 1u};
      const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar), st0 = smem_u32(smem);
      const int row = mt * a.mh * kBlockM, nbox = a.E / 64;
      int kx = kb0 * kBlockK;
      for (int i = 0; i < nkb && !a.no_loads; ++i) {
        if (!mbar_wait(empty0 + 8u * r.s, r.ph, abort_flag, a.spin_limit)) {
          if (!*abort_flag) report(a.status, 101, mt, i);
          *abort_flag = 1;
          break;
        }
        const uint32_t fb = full0 + 8u * r.s;
        mbar_expect_tx(fb, stage_bytes);
        const uint32_t st = st0 + r.s * stage_bytes;
        tma_load_2d_keep(st, &map_x, kx, row, fb, keep_x);
        if (a.mh == 2) tma_load_2d_keep(st + half_bytes, &map_x, kx, row + kBlockM, fb, keep_x);
        if (a.w_mn_major) {
          // one [64 h][64 e] box per block of 64 experts, 8 KB apart
          for (int nb = 0; nb < nbox; ++nb) tma_load_2d(st + a_bytes + nb * 8192, &map_w, nb * 64, kx, fb);
        } else {
          tma_load_2d(st + a_bytes, &map_w, kx, 0, fb);
        }
        issued = i + 1;
        kx += kBlockK;
        r.next((uint32_t)a.stages);
      }
      if (*abort_flag) {
        // Do not leave the CTA while bulk copies into its shared memory are in
        // flight: wait (bounded) for the barriers of the last `stages` loads.
        volatile int never = 0;
        for (int j = issued > a.stages ? issued - a.stages : 0; j < issued; ++j)
          mbar_wait(smem_u32(full_bar + j % a.stages), (uint32_t)(j / a.stages) & 1u, &never);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.E >> 3) << 17) |
                             ((uint32_t)(kBlockM >> 4) << 24) |
                             (a.w_mn_major ? (1u << 16) : 0u);  // B major: 0 = K, 1 = MN
      bool ok = true;
      Ring r{0u, 0u};
      const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
      const uint64_t da_first = make_desc(smem_u32(smem));
      const uint64_t db_first = a.w_mn_major ? make_desc_mn(smem_u32(smem + a_bytes), 8192u)
                                             : make_desc(smem_u32(smem + a_bytes));
      const uint64_t stage_units = (uint64_t)(stage_bytes >> 4);  // the address field counts 16 bytes
      const uint64_t half_units = (uint64_t)(half_bytes >> 4);
      // one UMMA_K step: 32 bytes inside the 128-byte swizzle row (K-major), two 1024-byte groups (MN-major)
      const uint64_t kstep_a = (uint64_t)((kUmmaK * 2) >> 4);
      const uint64_t kstep_b = a.w_mn_major ? (uint64_t)(2048 >> 4) : kstep_a;
      uint32_t ready = 0;
      for (int i = 0; i < nkb && ok; ++i) {
        if (!ready && !mbar_wait(full0 + 8u * r.s, r.ph, abort_flag, a.spin_limit)) {
          if (!*abort_flag) report(a.status, 102, mt, i);
          *abort_flag = 1;
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da0 = da_first + r.s * stage_units, da1 = da0 + half_units;
        const uint64_t db = db_first + r.s * stage_units;
        const uint32_t empty = empty0 + 8u * r.s;
        r.next((uint32_t)a.stages);
        // look at the next stage's barrier now; the answer is needed after these MMAs are issued
        const uint32_t peek = mbar_test(full0 + 8u * r.s, r.ph);
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k) {
          const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
          umma_f16(tmem_base, da0 + (uint64_t)k * kstep_a, db + (uint64_t)k * kstep_b, idesc, acc);
          // the second 128-token half accumulates E columns further on
          if (a.mh == 2)
            umma_f16(tmem_base + (uint32_t)a.E, da1 + (uint64_t)k * kstep_a, db + (uint64_t)k * kstep_b, idesc, acc);
        }
        umma_commit(empty);  // frees the stage once these MMAs have read it
        ready = peek;
      }
      if (ok) umma_commit(smem_u32(accum_bar));
    }
  } else {
    epilogue_rows(a, smem, tmem_base, accum_bar, abort_flag, warp, lane, mt, ks);
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)a.tmem_cols)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// Two-CTA variant for many experts (E = 256): the CTAs of a cluster of two own
// neighbouring 128-token tiles and share every W tile - each fetches only half
// of its columns (E/2 experts) - and the leader CTA issues one 256-row MMA over
// both (tcgen05 cta_group::2).  A stage is then 16 KB of x + E*64 bytes of W per
// CTA instead of 16 KB + E*128, so the same shared memory holds half as many
// more stages and every SM pulls a third fewer bytes through L2 per tile.
//
// Barriers: full[s] of the LEADER counts the bytes of both CTAs (the peer's
// TMA loads name the leader's barrier); empty[s] and accum exist in both CTAs
// and are signalled together by a multicast commit of the leader's MMA thread.
// ---------------------------------------------------------------------------
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gate_umma_pair_kernel(const __grid_constant__ CUtensorMap map_x,
                      const __grid_constant__ CUtensorMap map_w, const UmmaArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t a_bytes = kBlockM * kBlockK * 2;
  const uint32_t bh_bytes = (uint32_t)(a.E / 2) * kBlockK * 2;  // this CTA's half of a W tile
  const uint32_t stage_bytes = a_bytes + bh_bytes;
  unsigned char* tail = smem + (size_t)a.stages * stage_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
  uint64_t* empty_bar = full_bar + a.stages;
  uint64_t* accum_bar = empty_bar + a.stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int mt = blockIdx.x, ks = blockIdx.y;
  const int kb0 = (int)((int64_t)ks * a.kblocks / a.ksplit);
  const int kb1 = (int)((int64_t)(ks + 1) * a.kblocks / a.ksplit);
  const int nkb = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(smem_u32(full_bar + s), 1);
      mbar_init(smem_u32(empty_bar + s), 1);
    }
    mbar_init(smem_u32(accum_bar), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    __syncwarp();
    // the same warp of both CTAs allocates, with the same slot address
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"((uint32_t)a.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster_sync_all();  // both CTAs' barriers are initialised before either is signalled
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      const uint64_t keep_x = policy_evict_last();
      int issued = 0;
      Ring r{0u, 1u};
      const uint32_t full_lead0 = map_to_cta(smem_u32(full_bar), 0u);  // the leader's full barriers
      const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar), st0 = smem_u32(smem);
      const int row = mt * kBlockM, nbox = a.E / 128;
      int kx = kb0 * kBlockK;
      for (int i = 0; i < nkb && !a.no_loads; ++i) {
        if (!mbar_wait(empty0 + 8u * r.s, r.ph, abort_flag, a.spin_limit)) {
          if (!*abort_flag) report(a.status, 111, mt, i);
          *abort_flag = 1;
          break;
        }
        // the leader expects the bytes of both CTAs
        if (rank == 0) mbar_expect_tx(full0 + 8u * r.s, 2u * stage_bytes);
        const uint32_t fb = full_lead0 + 8u * r.s;
        const uint32_t st = st0 + r.s * stage_bytes;
        tma_load_2d_pair_keep(st, &map_x, kx, row, fb, keep_x);
        if (a.w_mn_major) {
          // this CTA's E/128 boxes of [64 h][64 e], 8 KB apart
          for (int nb = 0; nb < nbox; ++nb)
            tma_load_2d_pair(st + a_bytes + nb * 8192, &map_w, ((int)rank * nbox + nb) * 64, kx, fb);
        } else {
          tma_load_2d_pair(st + a_bytes, &map_w, kx, (int)rank * (a.E / 2), fb);
        }
        issued = i + 1;
        kx += kBlockK;
        r.next((uint32_t)a.stages);
      }
      if (*abort_flag && rank == 0) {
        // the leader's barriers see the loads of both CTAs: wait (bounded) for the
        // last `stages` of them before leaving
        volatile int never = 0;
        for (int j = issued > a.stages ? issued - a.stages : 0; j < issued; ++j)
          mbar_wait(smem_u32(full_bar + j % a.stages), (uint32_t)(j / a.stages) & 1u, &never);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // fp32 accumulate, bf16 x bf16, M = 256 over the pair, N = E
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.E >> 3) << 17) |
                             ((uint32_t)((2 * kBlockM) >> 4) << 24) | (a.w_mn_major ? (1u << 16) : 0u);
      bool ok = true;
      Ring r{0u, 0u};
      const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
      const uint64_t da0 = make_desc(smem_u32(smem));
      const uint64_t db0 = a.w_mn_major ? make_desc_mn(smem_u32(smem + a_bytes), 8192u)
                                        : make_desc(smem_u32(smem + a_bytes));
      const uint64_t stage_units = (uint64_t)(stage_bytes >> 4);  // the address field counts 16 bytes
      // one UMMA_K step: 32 bytes inside the 128-byte swizzle row (K-major), two 1024-byte groups (MN-major)
      const uint64_t kstep_a = (uint64_t)((kUmmaK * 2) >> 4);
      const uint64_t kstep_b = a.w_mn_major ? (uint64_t)(2048 >> 4) : kstep_a;
      uint32_t ready = 0;
      for (int i = 0; i < nkb && ok; ++i) {
        if (!ready && !mbar_wait(full0 + 8u * r.s, r.ph, abort_flag, a.spin_limit)) {
          if (!*abort_flag) report(a.status, 112, mt, i);
          *abort_flag = 1;
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da = da0 + r.s * stage_units, db = db0 + r.s * stage_units;
        const uint32_t empty = empty0 + 8u * r.s;
        r.next((uint32_t)a.stages);
        // look at the next stage's barrier now; the answer is needed after these MMAs are issued
        const uint32_t peek = mbar_test(full0 + 8u * r.s, r.ph);
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k)
          umma_f16_pair(tmem_base, da + (uint64_t)k * kstep_a, db + (uint64_t)k * kstep_b, idesc,
                        (i > 0 || k > 0) ? 1u : 0u);
        umma_commit_pair(empty);  // frees the stage in both CTAs
        ready = peek;
      }
      if (ok) umma_commit_pair(smem_u32(accum_bar));
    }
  } else {
    epilogue_rows(a, smem, tmem_base, accum_bar, abort_flag, warp, lane, mt, ks);
  }

  // Neither CTA may leave (or free TMEM) while its peer can still read its shared
  // memory, write its barriers or run an MMA into its TMEM.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster_sync_all();
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)a.tmem_cols)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// Gate product AND routing in one kernel, for shapes with several 128-token
// tiles per SM, at most 128 product columns and no split over K: the logits
// never leave the SM.  A CTA walks its tiles (b, b + grid, ...); the accumulator
// alternates between two TMEM buffers, so that while the tensor core works on
// tile i+1 the other warps route tile i:
//   warp 0      TMA producer (x tile + W tile per 64-wide K block, one ring over all tiles)
//   warp 1      MMA issuer; tmem_full[buf] when a tile's product is complete
//   warps 2-5   drain: TMEM row -> shared-memory row (raw product columns), tmem_empty[buf];
//               then they route with the others
//   warps 2-31  routing: one token per warp at a time from the shared rows
//               (route_token_c: consecutive experts per lane; the hi/lo columns of an
//               fp32 weight are folded here), ids / weights / pair counts
// Replaces cublasGemmEx + topk_kernel of the reference (kernel.cu:4327-4339,
// 1829-1920) without the router_logits round trip through memory in between
// (they are written only on request).  Every wait is bounded; a role that gives
// up raises the abort flag and keeps passing the named barriers of its group so
// that nobody is left waiting for it.
// ---------------------------------------------------------------------------
constexpr int kFusedThreads = 1024;
constexpr int kRouteWarps0 = 2;                                    // first routing warp (2-5 drain first)
constexpr int kDrainWarps = 4;
constexpr int kFusedRouteWarps = kFusedThreads / 32 - kRouteWarps0;  // 30
constexpr int kFusedRouteThreads = kFusedRouteWarps * 32;

struct FusedArgs {
  RouteArgs r;          // routing parameters and outputs; r.fold: the rows hold 2E columns
  int32_t* status;
  int64_t T;
  int N;                // product columns: E, or 2E
  int kblocks, stages, w_mn_major;
  int ntiles;           // 128-token tiles
  int ncount_tiles;     // kTile-token counting tiles
  uint32_t spin_limit;
  int no_loads;
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

template <int EPL>
__global__ void __launch_bounds__(kFusedThreads, 1)
gate_route_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                  const FusedArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t a_bytes = kBlockM * kBlockK * 2;
  const uint32_t b_bytes = (uint32_t)a.N * kBlockK * 2;
  const uint32_t stage_bytes = a_bytes + b_bytes;
  const uint32_t row_pitch = (uint32_t)a.N * 4u + 16u;  // a 16-byte skew keeps a warp's 16-byte row stores apart
  unsigned char* rows = smem + (size_t)a.stages * stage_bytes;               // [128][row_pitch] logits of one tile
  int* s_cnt = reinterpret_cast<int*>(rows + (size_t)kBlockM * row_pitch);   // [2][E] pairs per counting tile half
  uint32_t* s_cand = reinterpret_cast<uint32_t*>(s_cnt + 2 * a.r.E);         // [route warps][kLaneCandWords]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(s_cand + kFusedRouteWarps * kLaneCandWords);
  uint64_t* empty_bar = full_bar + a.stages;
  uint64_t* tmem_full = empty_bar + a.stages;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;         // [2]
  uint64_t* rows_full = tmem_empty + 2;         // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(rows_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(smem_u32(full_bar + s), 1);
      mbar_init(smem_u32(empty_bar + s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(tmem_full + i), 1);
      mbar_init(smem_u32(tmem_empty + i), 128);
    }
    mbar_init(smem_u32(rows_full), 128);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const uint32_t tmem_cols = 2u * (uint32_t)a.N <= 32u ? 32u : 2u * (uint32_t)a.N <= 64u ? 64u
                             : 2u * (uint32_t)a.N <= 128u ? 128u : 256u;
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  for (int i = threadIdx.x; i < 2 * a.r.E; i += kFusedThreads) s_cnt[i] = 0;
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const int my_tiles = (a.ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;  // b, b+G, ...

  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      const uint64_t keep_x = policy_evict_last();
      int issued = 0;
      bool ok = true;
      Ring r{0u, 1u};
      const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar), st0 = smem_u32(smem);
      const int nbox = a.N / 64;
      for (int it = 0; it < my_tiles && ok && !a.no_loads; ++it) {
        const int tile = (int)blockIdx.x + it * (int)gridDim.x;
        int kx = 0;
        for (int kb = 0; kb < a.kblocks; ++kb) {
          if (!mbar_wait(empty0 + 8u * r.s, r.ph, abort_flag, a.spin_limit)) {
            if (!*abort_flag) report(a.status, 121, tile, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t fb = full0 + 8u * r.s;
          mbar_expect_tx(fb, stage_bytes);
          const uint32_t st = st0 + r.s * stage_bytes;
          tma_load_2d_keep(st, &map_x, kx, tile * kBlockM, fb, keep_x);
          if (a.w_mn_major) {
            for (int nb = 0; nb < nbox; ++nb) tma_load_2d(st + a_bytes + nb * 8192, &map_w, nb * 64, kx, fb);
          } else {
            tma_load_2d(st + a_bytes, &map_w, kx, 0, fb);
          }
          ++issued;
          kx += kBlockK;
          r.next((uint32_t)a.stages);
        }
      }
      if (*abort_flag) {
        // do not leave while copies into this CTA's shared memory are in flight
        volatile int never = 0;
        for (int j = issued > a.stages ? issued - a.stages : 0; j < issued; ++j)
          mbar_wait(smem_u32(full_bar + j % a.stages), (uint32_t)(j / a.stages) & 1u, &never);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.N >> 3) << 17) |
                             ((uint32_t)(kBlockM >> 4) << 24) | (a.w_mn_major ? (1u << 16) : 0u);
      bool ok = true;
      Ring r{0u, 0u};
      const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
      const uint64_t da_first = make_desc(smem_u32(smem));
      const uint64_t db_first = a.w_mn_major ? make_desc_mn(smem_u32(smem + a_bytes), 8192u)
                                             : make_desc(smem_u32(smem + a_bytes));
      const uint64_t stage_units = (uint64_t)(stage_bytes >> 4);  // the address field counts 16 bytes
      const uint64_t kstep_a = (uint64_t)((kUmmaK * 2) >> 4);
      const uint64_t kstep_b = a.w_mn_major ? (uint64_t)(2048 >> 4) : kstep_a;
      uint32_t ready = 0;
      for (int it = 0; it < my_tiles && ok; ++it) {
        const int buf = it & 1;
        const int tile = (int)blockIdx.x + it * (int)gridDim.x;
        // the drain warps have emptied this accumulator (its previous tile, two tiles ago)
        if (!mbar_wait(smem_u32(tmem_empty + buf), ((uint32_t)(it >> 1) & 1u) ^ 1u, abort_flag, a.spin_limit)) {
          if (!*abort_flag) report(a.status, 122, tile, it);
          *abort_flag = 1;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc_cols = tmem_base + (uint32_t)(buf * a.N);
        for (int kb = 0; kb < a.kblocks; ++kb) {
          if (!ready && !mbar_wait(full0 + 8u * r.s, r.ph, abort_flag, a.spin_limit)) {
            if (!*abort_flag) report(a.status, 123, tile, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t da = da_first + r.s * stage_units, db = db_first + r.s * stage_units;
          const uint32_t empty = empty0 + 8u * r.s;
          r.next((uint32_t)a.stages);
          // look at the next stage's barrier now; the answer is needed after these MMAs are issued
          const uint32_t peek = mbar_test(full0 + 8u * r.s, r.ph);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k)
            umma_f16(acc_cols, da + (uint64_t)k * kstep_a, db + (uint64_t)k * kstep_b, idesc,
                     (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty);
          ready = peek;
        }
        if (ok) umma_commit(smem_u32(tmem_full + buf));
      }
    }
  } else {
    // ---- warps 2..31: (warps 2-5: drain the accumulator of the tile, then) route the tile
    const bool drains = warp < kRouteWarps0 + kDrainWarps;
    const int q = warp & 3;  // TMEM lane quarter a drain warp may touch
    const int rw = warp - kRouteWarps0;
    const RouteArgs& ra = a.r;
    uint32_t* my_cand = s_cand + rw * kLaneCandWords;
    bool gave_up = false;
    for (int it = 0; it < my_tiles; ++it) {
      const int buf = it & 1;
      const int tile = (int)blockIdx.x + it * (int)gridDim.x;
      const int64_t t0 = (int64_t)tile * kBlockM;
      if (drains && !gave_up) {
        // (the rows of the previous tile are free: this warp passed the barriers of its routing)
        bool ok = mbar_wait(smem_u32(tmem_full + buf), (uint32_t)(it >> 1) & 1u, abort_flag, a.spin_limit);
        ok = __all_sync(kFull, ok);
        if (!ok) {
          if (lane == 0 && !*abort_flag) report(a.status, 124, tile, it);
          *abort_flag = 1;
          gave_up = true;
        } else {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          unsigned char* my_row = rows + (size_t)(q * 32 + lane) * row_pitch;
          for (int c = 0; c < a.N; c += 32) {
            uint32_t r[32];
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * a.N + c);
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                  "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
                  "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                  "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                  "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
                  "=r"(r[31])
                : "r"(taddr)
                : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            uint4* o4 = reinterpret_cast<uint4*>(my_row + (size_t)c * 4);
#pragma unroll
            for (int i = 0; i < 8; ++i) o4[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
          }
          // the accumulator may be overwritten, and the rows may be read
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          mbar_arrive(smem_u32(tmem_empty + buf));
          mbar_arrive(smem_u32(rows_full));
        }
      }
      if (!gave_up) {
        bool ok = mbar_wait(smem_u32(rows_full), (uint32_t)it & 1u, abort_flag, a.spin_limit);
        ok = __all_sync(kFull, ok);
        if (!ok) {
          if (lane == 0 && !*abort_flag) report(a.status, 125, tile, it);
          *abort_flag = 1;
          gave_up = true;
        }
      }
      if (!gave_up) {
        for (int tk = rw; tk < kBlockM; tk += kFusedRouteWarps) {
          const int64_t t = t0 + tk;
          if (t >= a.T) break;
          // this lane's experts: EPL consecutive columns (plus the lo columns of an fp32 weight)
          const float* row = reinterpret_cast<const float*>(rows + (size_t)tk * row_pitch) + EPL * lane;
          float z[EPL];
          if (EPL == 2) {
            const float2 v = *reinterpret_cast<const float2*>(row);
            z[0] = v.x; z[1] = v.y;
          } else {
#pragma unroll
            for (int v4 = 0; v4 < EPL / 4; ++v4) {
              const float4 v = reinterpret_cast<const float4*>(row)[v4];
              z[4 * v4] = v.x; z[4 * v4 + 1] = v.y; z[4 * v4 + 2] = v.z; z[4 * v4 + 3] = v.w;
            }
          }
          if (ra.fold) {
#pragma unroll
            for (int j = 0; j < EPL; ++j) z[j] = __fadd_rn(z[j], row[ra.E + j]);
          }
          if (ra.logit_bias != nullptr) {
#pragma unroll
            for (int j = 0; j < EPL; ++j) z[j] = __fadd_rn(z[j], __ldg(ra.logit_bias + EPL * lane + j));
          }
          if (ra.logits_out != nullptr) {
#pragma unroll
            for (int j = 0; j < EPL; ++j) ra.logits_out[(size_t)t * ra.E + EPL * lane + j] = z[j];
          }
          int mysel;
          float myw;
          route_token_c<EPL>(ra, z, lane, my_cand, mysel, myw);
          if (lane < ra.K) {
            const size_t o = (size_t)t * ra.K + lane;
            ra.ids[o] = mysel;
            ra.weights[o] = myw;
            atomicAdd(s_cnt + (tk >> 6) * ra.E + mysel, 1);  // kTile = 64: two counting tiles per 128-token tile
          }
        }
      }
      // every one of these warps passes both barriers of every tile, also after it gave up
      named_bar_sync(1, kFusedRouteThreads);
      if (!gave_up) {
        // the tile's pair counts: stored per (counting tile, expert) - this CTA owns both counting
        // tiles whole - and added per (group of counting tiles, expert)
        const int rt = (int)threadIdx.x - kRouteWarps0 * 32;
        for (int i = rt; i < 2 * ra.E; i += kFusedRouteThreads) {
          const int half = i / ra.E, e = i - half * ra.E;
          const int ct = tile * 2 + half;
          const int v = s_cnt[i];
          s_cnt[i] = 0;
          if (ct < a.ncount_tiles) {
            ra.tile_counts[(size_t)ct * ra.E + e] = v;
            if (v) atomicAdd(ra.group_counts + (size_t)(ct / kTileGroup) * ra.E + e, v);
          }
        }
      }
      // after this barrier the rows may be overwritten by the drain warps and the histogram is clear
      named_bar_sync(1, kFusedRouteThreads);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols)
                 : "memory");
  }
}


// W[H,E] -> Wt[E,H] (bf16), 32x32 tiles through shared memory.
__global__ void __launch_bounds__(256) transpose_w_kernel(const uint16_t* __restrict__ w,
                                                          uint16_t* __restrict__ wt, int H, int E) {
  __shared__ uint16_t tile[32][33];
  const int h0 = blockIdx.x * 32, e0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8) {
    const int h = h0 + r, e = e0 + tx;
    tile[r][tx] = (h < H && e < E) ? w[(size_t)h * E + e] : (uint16_t)0;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int e = e0 + r, h = h0 + tx;
    if (e < E && h < H) wt[(size_t)e * H + h] = tile[tx][r];
  }
}

// fp32 gate weight -> two bf16 rows per expert, K-major: wpk[e][h] = hi = bf16(W[e,h])
// and wpk[E + e][h] = lo = bf16(W[e,h] - hi), so that a bf16 product with 2E columns
// followed by  z[e] = D[e] + D[E + e]  reproduces the fp32-weight product to about
// 2^-17 relative per term (wsplit_kernel of the reference, kernel.cu:1786-1824, and
// its fold at 1849-1851; the reference packs [H,2E], here the rows are K-major so
// that the same tiles serve both weight layouts).  W - hi is exact in fp32.
__device__ __forceinline__ void split_bf16(float v, uint16_t& hi, uint16_t& lo) {
  const __nv_bfloat16 h = __float2bfloat16_rn(v);
  const __nv_bfloat16 l = __float2bfloat16_rn(__fsub_rn(v, __bfloat162float(h)));
  hi = __bfloat16_as_ushort(h);
  lo = __bfloat16_as_ushort(l);
}

// W[E,H]: four hidden indices per thread.
__global__ void __launch_bounds__(256) wsplit_eh_kernel(const float* __restrict__ w,
                                                        uint16_t* __restrict__ wpk, int H, int E) {
  const size_t n4 = (size_t)E * H / 4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(w) + i);
    uint16_t h0, h1, h2, h3, l0, l1, l2, l3;
    split_bf16(v.x, h0, l0);
    split_bf16(v.y, h1, l1);
    split_bf16(v.z, h2, l2);
    split_bf16(v.w, h3, l3);
    reinterpret_cast<uint2*>(wpk)[i] = make_uint2(h0 | ((uint32_t)h1 << 16), h2 | ((uint32_t)h3 << 16));
    reinterpret_cast<uint2*>(wpk + (size_t)E * H)[i] =
        make_uint2(l0 | ((uint32_t)l1 << 16), l2 | ((uint32_t)l3 << 16));
  }
}

// W[H,E]: 32x32 tiles through shared memory.
__global__ void __launch_bounds__(256) wsplit_he_kernel(const float* __restrict__ w,
                                                        uint16_t* __restrict__ wpk, int H, int E) {
  __shared__ float tile[32][33];
  const int h0 = blockIdx.x * 32, e0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8) {
    const int h = h0 + r, e = e0 + tx;
    tile[r][tx] = (h < H && e < E) ? __ldg(w + (size_t)h * E + e) : 0.0f;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int e = e0 + r, h = h0 + tx;
    if (e < E && h < H) {
      uint16_t hi, lo;
      split_bf16(tile[tx][r], hi, lo);
      wpk[(size_t)e * H + h] = hi;
      wpk[(size_t)(E + e) * H + h] = lo;
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// rows x cols bf16, row-major; box = box_rows x 64 columns, 128-byte swizzle.
bool make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  if (rows == 0 || cols == 0 || (cols * 2) % 16 != 0) return false;
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBlockK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            MOE_RD_UMMA_L2_PROMOTION, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// One CTA per SM with two token halves (or with E = 256); two CTAs per SM for a
// single half and few experts, so that more than 148 tiles stay resident.
int pick_stages(int E, int mh) {
  const int stage = mh * kBlockM * kBlockK * 2 + E * kBlockK * 2;
  const int budget = (mh == 2 || E > MOE_RD_UMMA_TWO_CTA_MAX_E) ? MOE_RD_UMMA_SMEM_KB_ONE_CTA * 1024
                                                                 : MOE_RD_UMMA_SMEM_KB_TWO_CTA * 1024;
  int s = budget / stage;
  return s > 8 ? 8 : (s < 2 ? 2 : s);
}

size_t umma_smem_bytes(int E, int stages, int mh) {
  return (size_t)stages * (mh * kBlockM * kBlockK * 2 + E * kBlockK * 2) + (2 * stages + 1) * 8 + 16 +
         1024;
}

}  // namespace

bool umma_available() { return true; }

int device_sms();
static int device_sms_cached() { return device_sms(); }
void fill_route_args(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan, const float* logits,
                     int32_t* ids, int32_t* tile_base, int32_t* counts, RouteArgs* a);

cudaError_t init_umma_attributes() {
  cudaError_t e = cudaFuncSetAttribute(gate_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       227 * 1024);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(gate_umma_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(gate_route_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(gate_route_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
}

static_assert(kTile == 64, "gate_route_kernel keeps two counting tiles per 128-token tile");

// Shared memory of gate_route_kernel with `stages` ring stages.
static size_t fused_smem_bytes(int N, int E, int stages) {
  return (size_t)stages * (kBlockM * kBlockK * 2 + N * kBlockK * 2) + (size_t)kBlockM * (N * 4 + 16) +
         (size_t)2 * E * 4 + (size_t)kFusedRouteWarps * kLaneCandWords * 4 + (size_t)(2 * stages + 6) * 8 + 16 + 1024;
}

// Whether the fused gate + routing kernel takes this problem: no split over K, at most 128 product
// columns, E of 64 or 128 (consecutive experts per lane), enough 128-token tiles that most CTAs get two
// or more (the routing of one tile then overlaps the K loop of the next), and biases / logits that can
// be read as 16-byte vectors.
bool fused_front_eligible(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan) {
  if (!MOE_RD_FUSED_FRONT || plan.gate != MOE_RD_GATE_UMMA || plan.ksplit != 1 || plan.umma_pair) return false;
  if (plan.umma_n > 128 || (p.E != 64 && p.E != 128)) return false;
  if (!lane_route_supported(p.E, p.K, p.n_groups, p.topk_groups, p.group_topk)) return false;
  const int64_t ntiles = (p.T + kBlockM - 1) / kBlockM;
  if (ntiles < (int64_t)device_sms_cached() * 5 / 4) return false;
  const auto mis = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) != 0; };
  if (mis(b.logit_bias) || mis(b.select_bias) || mis(b.router_logits)) return false;
  return fused_smem_bytes(plan.umma_n, p.E, 3) <= 227 * 1024;
}

cudaError_t launch_gate_route(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan, void* wt,
                              int32_t* ids, int32_t* tile_counts, int32_t* group_counts, int32_t* status,
                              cudaStream_t s) {
  const int N = plan.umma_n;
  const uint16_t* w_eh = static_cast<const uint16_t*>(b.gate_w);
  const bool mn_major = !plan.umma_fold && p.w_layout == MOE_RD_W_LAYOUT_HE && p.E % 64 == 0;
  if (plan.umma_fold) {
    const float* wf = static_cast<const float*>(b.gate_w);
    if (p.w_layout == MOE_RD_W_LAYOUT_EH) {
      const size_t n4 = (size_t)p.E * p.H / 4;
      const unsigned blocks = (unsigned)((n4 + 255) / 256 < 1184 ? (n4 + 255) / 256 : 1184);
      wsplit_eh_kernel<<<blocks, 256, 0, s>>>(wf, static_cast<uint16_t*>(wt), p.H, p.E);
    } else {
      const dim3 grid((unsigned)((p.H + 31) / 32), (unsigned)((p.E + 31) / 32));
      wsplit_he_kernel<<<grid, 256, 0, s>>>(wf, static_cast<uint16_t*>(wt), p.H, p.E);
    }
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    w_eh = static_cast<const uint16_t*>(wt);
  } else if (p.w_layout == MOE_RD_W_LAYOUT_HE && !mn_major) {
    const dim3 grid((unsigned)((p.H + 31) / 32), (unsigned)((p.E + 31) / 32));
    transpose_w_kernel<<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(b.gate_w), static_cast<uint16_t*>(wt),
                                            p.H, p.E);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    w_eh = static_cast<const uint16_t*>(wt);
  }
  CUtensorMap map_x, map_w;
  if (!make_map(&map_x, b.x, (uint64_t)p.T, (uint64_t)p.H, kBlockM)) return cudaErrorInvalidValue;
  if (mn_major ? !make_map(&map_w, b.gate_w, (uint64_t)p.H, (uint64_t)p.E, 64u)
               : !make_map(&map_w, w_eh, (uint64_t)N, (uint64_t)p.H, (uint32_t)N))
    return cudaErrorInvalidValue;
  FusedArgs a;
  fill_route_args(p, b, plan, nullptr, ids, tile_counts, nullptr, &a.r);
  a.r.group_counts = group_counts;
  a.r.fold = plan.umma_fold;
  a.r.logit_bias = b.logit_bias;
  a.r.logits_out = b.router_logits;
  a.status = status;
  a.T = p.T;
  a.N = N;
  a.kblocks = p.H / kBlockK;
  a.w_mn_major = mn_major ? 1 : 0;
  a.ntiles = (int)((p.T + kBlockM - 1) / kBlockM);
  a.ncount_tiles = plan.ntiles;
  a.no_loads = (p.flags & MOE_RD_FLAG_TEST_GATE_STALL) ? 1 : 0;
  a.spin_limit = a.no_loads ? 256u : kSpinLimit;
  int stages = 8;
  while (stages > 2 && fused_smem_bytes(N, p.E, stages) > 227 * 1024) --stages;
  a.stages = stages;
  // every CTA the same number of tiles: grid = tiles / (tiles per CTA), rounded up
  const int sms = device_sms_cached();
  const int per = (a.ntiles + sms - 1) / sms;
  const unsigned grid = (unsigned)((a.ntiles + per - 1) / per);
  const size_t smem = fused_smem_bytes(N, p.E, stages);
  if (p.E == 64)
    gate_route_kernel<2><<<grid, kFusedThreads, smem, s>>>(map_x, map_w, a);
  else
    gate_route_kernel<4><<<grid, kFusedThreads, smem, s>>>(map_x, map_w, a);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_gate_umma(const moe_rd_params& p, const moe_rd_buffers& b, const Plan& plan,
                             void* wt, float* partial, float* logits, int32_t* status,
                             void* zero, size_t zero_bytes, cudaStream_t s) {
  (void)logits;
  const int N = plan.umma_n;  // columns of the product: E, or 2E (hi and lo rows of an fp32 weight)
  const uint16_t* w_eh = static_cast<const uint16_t*>(b.gate_w);
  // W[H,E] with whole blocks of 64 experts is consumed in place as an MN-major
  // operand; otherwise it is transposed to the K-major W^T[E,H] first.
  const bool mn_major = !plan.umma_fold && p.w_layout == MOE_RD_W_LAYOUT_HE && p.E % (plan.umma_pair ? 128 : 64) == 0;
  if (plan.umma_fold) {
    const float* wf = static_cast<const float*>(b.gate_w);
    if (p.w_layout == MOE_RD_W_LAYOUT_EH) {
      const size_t n4 = (size_t)p.E * p.H / 4;
      const unsigned blocks = (unsigned)((n4 + 255) / 256 < 1184 ? (n4 + 255) / 256 : 1184);
      wsplit_eh_kernel<<<blocks, 256, 0, s>>>(wf, static_cast<uint16_t*>(wt), p.H, p.E);
    } else {
      const dim3 grid((unsigned)((p.H + 31) / 32), (unsigned)((p.E + 31) / 32));
      wsplit_he_kernel<<<grid, 256, 0, s>>>(wf, static_cast<uint16_t*>(wt), p.H, p.E);
    }
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    w_eh = static_cast<const uint16_t*>(wt);
  } else if (p.w_layout == MOE_RD_W_LAYOUT_HE && !mn_major) {
    const dim3 grid((unsigned)((p.H + 31) / 32), (unsigned)((p.E + 31) / 32));
    transpose_w_kernel<<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(b.gate_w),
                                            static_cast<uint16_t*>(wt), p.H, p.E);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    w_eh = static_cast<const uint16_t*>(wt);
  }
  CUtensorMap map_x, map_w;
  if (!make_map(&map_x, b.x, (uint64_t)p.T, (uint64_t)p.H, kBlockM)) return cudaErrorInvalidValue;
  const bool pair = plan.umma_pair != 0;
  // K-major W^T: one box holds the rows (experts) one CTA needs per block of H
  const uint32_t wt_box_rows = (uint32_t)(pair ? N / 2 : N);
  if (mn_major ? !make_map(&map_w, b.gate_w, (uint64_t)p.H, (uint64_t)p.E, 64u)
               : !make_map(&map_w, w_eh, (uint64_t)N, (uint64_t)p.H, wt_box_rows))
    return cudaErrorInvalidValue;
  UmmaArgs a;
  a.partial = partial;
  a.status = status;
  a.T = p.T;
  a.E = N;
  a.kblocks = p.H / kBlockK;
  a.ksplit = plan.ksplit;
  a.mh = pair ? 1 : plan.umma_mh;
  a.w_mn_major = mn_major ? 1 : 0;
  a.zero = static_cast<uint4*>(zero);
  a.zero_vecs = (uint32_t)(zero_bytes / 16);
  a.no_loads = (p.flags & MOE_RD_FLAG_TEST_GATE_STALL) ? 1 : 0;
  a.spin_limit = a.no_loads ? 256u : kSpinLimit;
  int cols = 32;
  while (cols < N * a.mh) cols <<= 1;
  a.tmem_cols = cols;
  const size_t staging = (size_t)kBlockM * (N * 4 + 16);  // the epilogue parks 128 rows in the ring
  if (pair) {
    const int stage = kBlockM * kBlockK * 2 + (N / 2) * kBlockK * 2;
    int st = MOE_RD_UMMA_SMEM_KB_ONE_CTA * 1024 / stage;
    a.stages = st > 8 ? 8 : (st < 2 ? 2 : st);
    if (staging > (size_t)a.stages * stage) return cudaErrorInvalidValue;
    const unsigned mtiles = (unsigned)((p.T + kBlockM - 1) / kBlockM);
    const dim3 grid((mtiles + 1u) & ~1u, (unsigned)plan.ksplit);  // whole pairs; rows past T load as zeros
    const size_t smem = (size_t)a.stages * stage + (2 * a.stages + 1) * 8 + 16 + 1024;
    gate_umma_pair_kernel<<<grid, kThreads, smem, s>>>(map_x, map_w, a);
  } else {
    a.stages = pick_stages(N, a.mh);
    if (staging > (size_t)a.stages * (a.mh * kBlockM * kBlockK * 2 + N * kBlockK * 2))
      return cudaErrorInvalidValue;
    const int tile = kBlockM * a.mh;
    const dim3 grid((unsigned)((p.T + tile - 1) / tile), (unsigned)plan.ksplit);
    gate_umma_kernel<<<grid, kThreads, umma_smem_bytes(N, a.stages, a.mh), s>>>(map_x, map_w, a);
  }
  count_launch();
  return cudaGetLastError();
}

}  // namespace moe_rd
