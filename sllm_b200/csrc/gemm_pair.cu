// bfloat16 matrix product on the 5th-generation tensor cores with two CTAs on one tile:
//   C[M, N] = A[M, K] W[N, K]^T (+ bias), float32 accumulation in tensor memory.
//
// gemm_tcgen05.cu gives a 128 x 256 tile of C to one CTA; every tcgen05.mma there reads 4 KB of A and
// 8 KB of W from shared memory while the TMA unit writes as much, which is more than an SM's shared
// memory moves per cycle, and the tile stops at about 0.7 of the tensor pipe.  Here a pair of CTAs on
// neighbouring SMs (a thread-block cluster of two) shares a 256 x 256 tile: CTA r of the pair loads rows
// m0 + 128 r .. of A and rows n0 + 128 r .. of W (its half of each operand, 16 KB + 16 KB per 64-wide
// k block), and one thread of the pair's first CTA issues tcgen05.mma with cta_group::2 (M = 256, N = 256,
// K = 16): each SM's tensor core multiplies its own 128 rows of A by all 256 rows of W, taking the other
// half of W from its partner's shared memory, and accumulates 128 x 256 in its own tensor memory.  Per
// product a CTA reads 8 KB of shared memory instead of 12, and a stage is 32 KB instead of 48 (six stages
// in flight instead of four).
//
// Who waits for whom (all barriers are mbarriers in shared memory; every wait is bounded in time):
//   full[s]       in the FIRST CTA only: one arrival with the byte count of both CTAs' boxes; the second
//                 CTA's TMA loads signal it across the pair (cp.async.bulk.tensor with cta_group::2, the
//                 barrier's address mapped to the first CTA).  The MMA thread waits on it.
//   empty[s]      in each CTA: the MMA thread's tcgen05.commit arrives at both (multicast to the pair);
//                 each CTA's producer waits on its own before it loads into the stage again.
//   acc_full[b]   in each CTA: committed to both after a tile's last product; the epilogue warps of each
//                 CTA wait on their own and read their CTA's 128 lanes of the accumulator.
//   acc_empty[b]  in the first CTA: eight arrivals, one per epilogue warp of the pair (the second CTA's
//                 arrive across the pair); the MMA thread waits on it before it reuses the buffer.
// Tensor memory is allocated and freed by one warp of EACH CTA with cta_group::2, and both CTAs meet at a
// cluster barrier after set-up (no CTA signals a barrier its partner has not initialised) and before the
// memory is freed (no CTA frees it while its partner's epilogue still reads).  No TMA load is multicast.
//
// Three tile shapes: 256 x 256 (two accumulators: a tile's epilogue under the next tile's products), 256 x 512 (one
// accumulator, a quarter less traffic from L2; further down) and 256 x 128 (for results with few tiles).  The 256 x 256
// and 256 x 128 forms also run in slices of K: a unit of work is then (tile, slice) and the slices leave a stack of
// float32 partial sums for the next kernel to add, so that a result of few tiles still occupies every pair of SMs.
// The epilogues that touch float32 rows of global memory (the plain float32 result and the residual epilogue, which
// reads and writes the stream and writes the next norm's input) go through a box of shared memory per warp and
// walk it four rows an instruction (gemm_epilogue.cuh): in tensor memory a lane holds a row, and lane-by-lane
// accesses would put every 16-byte piece on a line of its own.
//
// The reference has no such kernel: its products are cublasGemmEx calls on one token
// (kernels/cuda/kernels.cu:752-767) and its prefill runs in numpy (serving/executor.py:255-265).
#include <stdio.h>

#include "gemm_epilogue.cuh"

namespace sllm {

constexpr int TP_BM = 128;                                // rows of A (and of C) per CTA; the pair's tile has 256
constexpr int TP_BK = 64;
constexpr int TP_A_BYTES = TP_BM * TP_BK * 2;             // 16 KB
// BN: columns of C per tile, 256 or 128; each CTA loads BN / 2 rows of W.  The slim tile is for results with so few
// tiles of 256 x 256 that most pairs of SMs would have none (a prompt portion of 512 tokens times a matrix of 3,584
// rows: 28 tiles for 74 pairs): twice the tiles at half the width.
template <int BN> struct TpCfg {
  static constexpr int B_BYTES = (BN / 2) * TP_BK * 2;    // 16 or 8 KB
  static constexpr int STAGE_BYTES = TP_A_BYTES + B_BYTES;
  static constexpr int STAGES = BN == 256 ? 6 : 8;        // 192 KB either way
  static constexpr int BOX_BYTES = 4 * 4096;              // a box of 32 rows x 128 bytes per epilogue warp (residual epilogue)
  static constexpr int SMEM = STAGES * STAGE_BYTES + BOX_BYTES + 1024 /* alignment */ + 256 /* barriers */;
  static constexpr int TMEM_COLS = 2 * BN;                // two accumulators
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address, in the cluster's shared window, of the same variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// a TMA box into this CTA's shared memory whose bytes are counted on a barrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(void* smem, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives at the barrier at this offset in BOTH CTAs of the pair once the products issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}

template <int EPI, int BN>
__global__ void __launch_bounds__(192, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                 const float* __restrict__ bias, void* __restrict__ out, int M, int N, int K, int* __restrict__ status,
                 const TgExtra extra, const int ksplits, const int kb_per_split) {
  extern __shared__ unsigned char tp_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tp_smem_raw) + 1023) & ~(uintptr_t)1023);
  using C = TpCfg<BN>;
  constexpr int TP_BN = BN, TP_STAGES = C::STAGES, TP_STAGE_BYTES = C::STAGE_BYTES, TP_TMEM_COLS = C::TMEM_COLS;
  unsigned char* boxes = smem + TP_STAGES * TP_STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(boxes + C::BOX_BYTES);
  uint64_t* empty = full + TP_STAGES;
  uint64_t* acc_full = empty + TP_STAGES;           // [2]
  uint64_t* acc_empty = acc_full + 2;               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: the CTA whose thread issues the products
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int m_tiles = (M + 2 * TP_BM - 1) / (2 * TP_BM), n_tiles = (N + TP_BN - 1) / TP_BN;
  // A unit of work is a tile and a slice of K (ksplits slices of kb_per_split 64-wide blocks; one slice unless the
  // result has so few tiles that most pairs would have none): unit u is slice u % ksplits of tile u / ksplits, and
  // slice s leaves its partial sums in out[s] of a stack [ksplits, M, N] (float32 epilogue only; bias in slice 0).
  const int tiles = m_tiles * n_tiles * ksplits;
  const int k_blocks_all = (K + TP_BK - 1) / TP_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TP_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);                  // the four epilogue warps of each CTA
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TP_TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                               // both CTAs' barriers exist before either signals the other
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                                       // A is the work of the step's earlier kernels

  if (warp == 0) {
    // ---------------- TMA producer (each CTA loads its halves) ----------------
    if (lane == 0) {
      int it = 0;
      bool gave_up = false;
      for (int unit = pair; unit < tiles && !*failed; unit += pairs) {
        const int tile = unit / ksplits, kb0 = (unit % ksplits) * kb_per_split, kb1 = min(k_blocks_all, kb0 + kb_per_split);
        const int m0 = (tile % m_tiles) * 2 * TP_BM + (int)rank * TP_BM;
        const int n0 = (tile / m_tiles) * TP_BN + (int)rank * (TP_BN / 2);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % TP_STAGES, round = it / TP_STAGES;
          if (!mbar_wait(&empty[s], (round & 1) ^ 1) || *failed) {
            if (!*failed) { *failed = 1; atomicExch(status, 41); }
            gave_up = true;
            break;
          }
          unsigned char* sa = smem + s * TP_STAGE_BYTES;
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
          if (rank == 0) mbar_expect_tx(&full[s], 2 * TP_STAGE_BYTES);      // both CTAs' boxes
          tma_load_2d_pair(sa, &map_a, kb * TP_BK, m0, bar);
          tma_load_2d_pair(sa + TP_A_BYTES, &map_w, kb * TP_BK, n0, bar);
        }
        if (gave_up) break;
      }
      if (*failed) {
        // let the copies already issued land before the CTA gives its shared memory back
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < TMA_DRAIN_NS) {}
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: one thread of the pair's first CTA ----------------
    if (lane == 0 && rank == 0) {
      // instruction descriptor: D float32, A and B bfloat16, both K-major, N = 256, M = 256 (the pair's)
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TP_BN >> 3) << 17) | ((uint32_t)((2 * TP_BM) >> 4) << 24);
      const uint64_t desc0 = umma_desc(smem_u32(smem));
      int local = 0;
      uint32_t st = 0, ph = 0;                      // the stage to consume next and its barrier's parity
      for (int unit = pair; unit < tiles && !*failed; unit += pairs, ++local) {
        const int kb0 = (unit % ksplits) * kb_per_split, k_blocks = min(k_blocks_all, kb0 + kb_per_split) - kb0;
        const int b = local & 1;
        if (!mbar_wait(&acc_empty[b], ((local >> 1) & 1) ^ 1) || *failed) {     // both epilogues have drained this buffer
          if (!*failed) { *failed = 2; atomicExch(status, 42); }
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + b * TP_BN;
        bool gave_up = false;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_hot(&full[st], ph)) {
            if (!*failed) { *failed = 2; atomicExch(status, 42); }
            gave_up = true;
            break;
          }
          // the stage's descriptors: 16 k further along the swizzled row is 32 bytes, 2 in the descriptor's address field
          const uint64_t da = desc0 + (uint64_t)(st * (TP_STAGE_BYTES >> 4)), db = da + (TP_A_BYTES >> 4);
          umma_bf16_pair(tmem_d, da, db, idesc, kb ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < TP_BK / 16; ++k) umma_bf16_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, 1u);
          umma_commit_pair(&empty[st]);             // arrives in both CTAs when these products have read the stage
          if (++st == TP_STAGES) { st = 0; ph ^= 1u; }
        }
        if (gave_up) break;
        umma_commit_pair(&acc_full[b]);             // arrives in both CTAs when every product issued so far is done
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5 own TMEM lane quarters 2, 3, 0, 1 of their CTA ----------------
    const int quarter = warp & 3;
    const uint32_t acc_empty_addr[2] = {map_to_cta(smem_u32(&acc_empty[0]), 0), map_to_cta(smem_u32(&acc_empty[1]), 0)};
    int local = 0;
    for (int unit = pair; unit < tiles; unit += pairs, ++local) {
      const int b = local & 1;
      const int tile = unit / ksplits, split = unit % ksplits;
      const int m0 = (tile % m_tiles) * 2 * TP_BM + (int)rank * TP_BM, n0 = (tile / m_tiles) * TP_BN;
      const int m = m0 + quarter * 32 + lane;
      const float row_scale = tg_row_scale(extra, m, M);        // a norm still owed on the input (1 if none): fetched while the products run
      const bool ok = mbar_wait(&acc_full[b], (local >> 1) & 1);
      if (!ok && !*failed) { *failed = 3; atomicExch(status, 43); }
      if (!ok || *failed) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float sq[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (m0 + quarter * 32 >= M) {                 // (warp-uniform) none of this warp's rows is in the matrix
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_addr[b]);
        continue;
      }
#pragma unroll 1
      for (int c0 = 0; c0 < TP_BN; c0 += 32) {
        if (n0 + c0 >= N) break;                    // warp-uniform
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + b * TP_BN + c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if constexpr (EPI == TG_EPI_RESID) {
          if (extra.ssq_in != nullptr) tg_scale(r, row_scale);
          tg_resid_box(r, boxes + (warp - 2) * 4096, lane, m0 + quarter * 32, n0 + c0, M, N, bias, extra, sq);
          if ((c0 & 127) == 96 || n0 + c0 + 32 >= N)      // a block of 128 columns is complete
            tg_resid_box_sums(sq, lane, m0 + quarter * 32, M, (n0 + c0) / 128, extra);
          continue;
        }
        if constexpr (EPI == TG_EPI_F32) {
          if ((N & 3) == 0) {                       // (uniform) whole 16-byte pieces: through the box, four rows an instruction
            if (extra.ssq_in != nullptr) tg_scale(r, row_scale);
            tg_store_box_f32(r, boxes + (warp - 2) * 4096, lane, m0 + quarter * 32, n0 + c0, M, N, split == 0 ? bias : nullptr,
                             reinterpret_cast<float*>(out) + (size_t)split * M * N);
            continue;
          }
        }
        if (m >= M) continue;
        if (extra.ssq_in != nullptr) tg_scale(r, row_scale);
        if constexpr (EPI == TG_EPI_F32)
          tg_store_chunk<EPI>(r, m, n0 + c0, N, split == 0 ? bias : nullptr, reinterpret_cast<float*>(out) + (size_t)split * M * N);
        else if constexpr (EPI != TG_EPI_RESID)
          tg_store_chunk<EPI>(r, m, n0 + c0, N, bias, out);
      }
      // this warp has read its quarter of the buffer: tell the MMA thread (in the pair's first CTA)
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_addr[b]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                               // the partner's epilogue is done with tensor memory too
  pdl_launch_dependents();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TP_TMEM_COLS));
  }
}

// ---- the wide form: 256 x 512 tiles ---------------------------------------------------------------
// With 256 x 256 tiles a CTA's shared memory moves, per 16-wide k step, 8 KB into the tensor core and 8 KB
// in from the TMA unit in the 128 cycles the step's product takes: all of its 128 bytes a cycle, and the
// tensor pipe stays near 0.8 busy.  A tile twice as wide keeps A for two products: per CTA 128 x 512 of C
// (all 512 columns of its tensor memory, one accumulator), per 64-wide k block A 128 x 64 and W 256 x 64
// (48 KB a stage, four stages), two products (N = 256 each) per k step: 16 KB out and 12 KB in per 256
// cycles, and a quarter less traffic from L2.  CTA r loads rows n0 + 256 r .. of W in one box; product h of a
// k step takes rows 128 h .. of each CTA's box, so that columns [0, 128) of accumulator half h are C's columns
// n0 + 128 h .. and its columns [128, 256) are C's columns n0 + 256 + 128 h ...
// With one accumulator the epilogue of a tile cannot run under the next tile's products as a whole; it runs
// under part of them: the epilogue hands half 0 back as soon as it has read it, and the MMA thread starts the
// next tile with the products of half 0 alone for the stages that are loaded (TP_STAGES_WIDE k blocks), then
// waits for half 1, catches up on those stages and goes on with both.
// The tile may also be narrower, 256 + 2 R2 columns with R2 = 96, 64 or 32 (448, 384, 320): the second product of a
// k step then takes R2 rows of each CTA's box of W (N = 2 R2), so that a result whose 512-wide tiles leave pairs of
// SMs idle (3,584 columns by 2,048 rows: 56 tiles for 74 pairs) is cut into more, narrower ones (64 of 448).

constexpr int TP_TMEM_COLS_WIDE = 512;                            // one accumulator of 512 columns
constexpr int TP_BN_WIDE = 512, TP_STAGES_WIDE = 4;
constexpr int TP_B_BYTES_WIDE = (TP_BN_WIDE / 2) * TP_BK * 2;      // 32 KB: this CTA's 256 rows of W
constexpr int TP_STAGE_BYTES_WIDE = TP_A_BYTES + TP_B_BYTES_WIDE;  // 48 KB
constexpr int TP_EPI_WARPS_WIDE = 8;                               // two per quarter of the tensor memory's lanes
constexpr int TP_THREADS_WIDE = (2 + TP_EPI_WARPS_WIDE) * 32;
constexpr int TP_STAGING_BYTES = TP_EPI_WARPS_WIDE * 4096;         // the epilogue warps' boxes on their way to the TMA unit
constexpr int TP_SMEM_WIDE = TP_STAGES_WIDE * TP_STAGE_BYTES_WIDE + TP_STAGING_BYTES + 1024 + 256;
static_assert(TP_SMEM_WIDE <= 227 * 1024, "shared memory of the wide form");

template <int EPI, int R2>
__global__ void __launch_bounds__(TP_THREADS_WIDE, 1)
gemm_pair_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                      const __grid_constant__ CUtensorMap map_out, int tma_out,
                      const float* __restrict__ bias, void* __restrict__ out, int M, int N, int K, int* __restrict__ status,
                      const TgExtra extra) {
  extern __shared__ unsigned char tp_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tp_smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* staging = smem + TP_STAGES_WIDE * TP_STAGE_BYTES_WIDE;     // [epilogue warps][32 rows x 128 bytes]
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + TP_STAGING_BYTES);
  uint64_t* empty = full + TP_STAGES_WIDE;
  uint64_t* acc_full = empty + TP_STAGES_WIDE;      // [1] (a second slot is left unused)
  uint64_t* acc_empty = acc_full + 2;               // [2]: the accumulator's halves
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  static_assert(R2 >= 32 && R2 <= 128 && R2 % TgBox<EPI>::ACC_COLS == 0, "rows of W in the second product");
  constexpr int BNW = 256 + 2 * R2;                  // the tile's columns; a CTA's box of W has half as many rows
  constexpr int STAGE_TX = TP_A_BYTES + (BNW / 2) * TP_BK * 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int m_tiles = (M + 2 * TP_BM - 1) / (2 * TP_BM), n_tiles = (N + BNW - 1) / BNW;
  const int tiles = m_tiles * n_tiles;
  const int k_blocks = (K + TP_BK - 1) / TP_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TP_STAGES_WIDE; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&acc_full[0], 1);
    for (int h = 0; h < 2; ++h) mbar_init(&acc_empty[h], 2 * TP_EPI_WARPS_WIDE);     // the epilogue warps of both CTAs
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TP_TMEM_COLS_WIDE));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int it = 0;
      bool gave_up = false;
      for (int tile = pair; tile < tiles && !*failed; tile += pairs) {
        const int m0 = (tile % m_tiles) * 2 * TP_BM + (int)rank * TP_BM;
        const int n0 = (tile / m_tiles) * BNW + (int)rank * (BNW / 2);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % TP_STAGES_WIDE, round = it / TP_STAGES_WIDE;
          if (!mbar_wait(&empty[s], (round & 1) ^ 1) || *failed) {
            if (!*failed) { *failed = 1; atomicExch(status, 41); }
            gave_up = true;
            break;
          }
          unsigned char* sa = smem + s * TP_STAGE_BYTES_WIDE;
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
          if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE_TX);
          tma_load_2d_pair(sa, &map_a, kb * TP_BK, m0, bar);
          tma_load_2d_pair(sa + TP_A_BYTES, &map_w, kb * TP_BK, n0, bar);
        }
        if (gave_up) break;
      }
      if (*failed) {
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < TMA_DRAIN_NS) {}
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc_common = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((2 * TP_BM) >> 4) << 24);
      constexpr uint32_t idesc0 = idesc_common | ((uint32_t)(256 >> 3) << 17), idesc1 = idesc_common | ((uint32_t)((2 * R2) >> 3) << 17);
      // The loop of the issuing thread is kept lean (its own instructions showed in the kernel's time): stages and
      // parities are counted, not divided; descriptors are made by addition; the flag in shared memory is only read
      // when a wait has run out.
      const uint64_t desc0 = umma_desc(smem_u32(smem));
      // the products of accumulator half h on stage st (kb: the tile's k block, 0 starts the accumulator)
      auto half_products = [&](uint32_t st, int kb, int h) {
        const uint64_t da = desc0 + (uint64_t)(st * (TP_STAGE_BYTES_WIDE >> 4));
        const uint64_t db = da + ((TP_A_BYTES + h * (128 * 128)) >> 4);
        const uint32_t idesc = h ? idesc1 : idesc0;
        umma_bf16_pair(tmem_base + h * 256, da, db, idesc, kb ? 1u : 0u);
#pragma unroll
        for (int k = 1; k < TP_BK / 16; ++k) umma_bf16_pair(tmem_base + h * 256, da + 2 * k, db + 2 * k, idesc, 1u);
      };
      auto wait_or_fail = [&](uint64_t* bar, uint32_t parity) {
        if (mbar_wait_hot(bar, parity)) return true;
        if (!*failed) { *failed = 2; atomicExch(status, 42); }
        return false;
      };
      int local = 0;
      uint32_t st = 0, ph = 0;                      // the stage to consume next and its barrier's parity
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs, ++local) {
        const uint32_t drained = (local & 1) ^ 1;     // the parity of "the epilogue before this tile has read the half"
        const int lead = k_blocks < TP_STAGES_WIDE ? k_blocks : TP_STAGES_WIDE;
        // half 0 alone for the stages that are loaded already, while the epilogue still reads half 1
        ok = wait_or_fail(&acc_empty[0], drained);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t st1 = st, ph1 = ph;
        for (int kb = 0; kb < lead && ok; ++kb) {
          ok = wait_or_fail(&full[st1], ph1);
          if (ok) half_products(st1, kb, 0);
          if (++st1 == TP_STAGES_WIDE) { st1 = 0; ph1 ^= 1u; }
        }
        if (ok) ok = wait_or_fail(&acc_empty[1], drained);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int kb = 0; kb < lead && ok; ++kb) {
          half_products(st, kb, 1);
          umma_commit_pair(&empty[st]);
          if (++st == TP_STAGES_WIDE) { st = 0; ph ^= 1u; }
        }
        // the rest of the tile: both halves per k block
        for (int kb = lead; kb < k_blocks && ok; ++kb) {
          ok = wait_or_fail(&full[st], ph);
          if (!ok) break;
          half_products(st, kb, 0);
          half_products(st, kb, 1);
          umma_commit_pair(&empty[st]);
          if (++st == TP_STAGES_WIDE) { st = 0; ph ^= 1u; }
        }
        if (ok) umma_commit_pair(&acc_full[0]);
      }
    }
  } else {
    // ---------------- epilogue: warps 2..9; warp w reads lanes 32 (w % 4) .., and of every accumulator half the
    // columns of the first CTA's rows of W (warps 2..5) or of the second CTA's (warps 6..9) ----------------
    const int quarter = warp & 3, col_half = (warp - 2) >> 2;
    const uint32_t acc_empty_addr[2] = {map_to_cta(smem_u32(&acc_empty[0]), 0), map_to_cta(smem_u32(&acc_empty[1]), 0)};
    unsigned char* box = staging + (warp - 2) * 4096;
    int local = 0;
    bool staged = false;                            // a box of this warp is on its way out of shared memory
    for (int tile = pair; tile < tiles; tile += pairs, ++local) {
      const int m0 = (tile % m_tiles) * 2 * TP_BM + (int)rank * TP_BM, n0 = (tile / m_tiles) * BNW;
      const int m = m0 + quarter * 32 + lane;
      const float row_scale = tg_row_scale(extra, m, M);        // a norm still owed on the input (1 if none): fetched while the products run
      const bool ok = mbar_wait(&acc_full[0], local & 1);
      if (!ok && !*failed) { *failed = 3; atomicExch(status, 43); }
      if (!ok || *failed) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      constexpr int AC = TgBox<EPI>::ACC_COLS;
      const int row0 = m0 + quarter * 32;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        float sq[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        // accumulator half h holds a product of `width` rows of each CTA's box of W (128 for half 0, R2 for half 1):
        // its columns [0, width) are C's columns n0 + 128 h .. (the first CTA's rows), its columns [width, 2 width)
        // are C's columns n0 + BNW / 2 + 128 h .. (the second CTA's); nb: where this warp's columns start in C
        const int width = h == 0 ? 128 : R2;
        const int nb = n0 + (BNW / 2) * col_half + 128 * h;
#pragma unroll 1
        for (int c0 = width * col_half; c0 < width * col_half + width; c0 += AC) {
          const int n = nb + (c0 - width * col_half);
          if (n >= N || row0 >= M) continue;        // warp-uniform
          if (tma_out && staged) {                  // the box staged before has left shared memory
            if (lane == 0) bulk_wait_read<0>();
            __syncwarp();
          }
#pragma unroll 1
          for (int sub = 0; sub < AC / 32; ++sub) {
            uint32_t r[32];
            tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + h * 256 + c0 + 32 * sub, r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (extra.ssq_in != nullptr) tg_scale(r, row_scale);
            if constexpr (EPI == TG_EPI_RESID) {
              if (n + 32 * sub < N) tg_resid_box(r, box, lane, row0, n + 32 * sub, M, N, bias, extra, sq);      // (warp-uniform)
            } else {
              if (tma_out) tg_stage_chunk<EPI>(r, box, lane, sub, n + 32 * sub, N, bias);
              else if (m < M && n + 32 * sub < N) tg_store_chunk<EPI>(r, m, n + 32 * sub, N, bias, out);
            }
          }
          if (tma_out) {
            fence_async_smem();                     // the lanes' writes, before the TMA unit reads them
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&map_out, box, EPI == TG_EPI_SILU ? n >> 1 : n, row0);
              bulk_commit();
            }
            staged = true;
          }
        }
        if constexpr (EPI == TG_EPI_RESID) {
          // the warp's columns of this half are one block of C's columns: its sum of squares per row (four blocks a tile)
          if (nb < N) tg_resid_box_sums(sq, lane, row0, M, 4 * (tile / m_tiles) + 2 * col_half + h, extra);
        }
        // this warp has read its share of the half: the MMA thread may write it again
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_addr[h]);
      }
    }
    if (lane == 0) bulk_wait<0>();                  // this warp's stores are complete before the kernel ends
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();
  pdl_launch_dependents();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TP_TMEM_COLS_WIDE));
  }
}

// ---- host side --------------------------------------------------------------------------------

static void pair_launch_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute (&attr)[2], int pairs, int threads, int smem,
                               cudaStream_t stream) {
  cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
}

template <int EPI, int R2>
static int launch_tp_wide(const CUtensorMap& ma, const CUtensorMap& mw, const float* bias, void* out, int M, int N, int K,
                          int* status, cudaStream_t stream, const TgExtra& extra) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_pair_wide_kernel<EPI, R2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM_WIDE) != cudaSuccess) {
      set_error("gemm_pair: cannot raise the shared memory limit");
      return SLLM_ERR_LAUNCH;
    }
    configured = true;
  }
  // the result leaves through TMA stores where its rows are whole 16-byte pieces; else lane by lane
  const int out_cols = EPI == TG_EPI_SILU ? N / 2 : N, elem = TgBox<EPI>::ELEM;
  CUtensorMap mo = {};
  int tma_out = 0;
  if (EPI != TG_EPI_RESID && ((size_t)out_cols * elem) % 16 == 0 && ((uintptr_t)out & 15) == 0)
    tma_out = make_map_store(&mo, out, M, out_cols, elem) ? 1 : 0;
  const int pairs_max = sllm::num_sms() / 2;
  constexpr int BNW = 256 + 2 * R2;
  const long long tiles = (long long)((M + 2 * TP_BM - 1) / (2 * TP_BM)) * ((N + BNW - 1) / BNW);
  const int pairs = (int)(tiles < pairs_max ? tiles : pairs_max);
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  pair_launch_config(cfg, attr, pairs, TP_THREADS_WIDE, TP_SMEM_WIDE, stream);
  cudaLaunchKernelEx(&cfg, gemm_pair_wide_kernel<EPI, R2>, ma, mw, mo, tma_out, bias, out, M, N, K, status, extra);
  return launch_status("gemm_pair");
}

template <int EPI, int BN>
static int launch_tp(const CUtensorMap& ma, const CUtensorMap& mw, const float* bias, void* out, int M, int N, int K,
                     int* status, cudaStream_t stream, const TgExtra& extra, int ksplits, int kb_per_split) {
  auto kernel = gemm_pair_kernel<EPI, BN>;
  constexpr int TP_SMEM = TpCfg<BN>::SMEM, TP_BN = BN;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM) != cudaSuccess) {
      set_error("gemm_pair: cannot raise the shared memory limit");
      return SLLM_ERR_LAUNCH;
    }
    configured = true;
  }
  const int pairs_max = sllm::num_sms() / 2;
  const long long tiles = (long long)((M + 2 * TP_BM - 1) / (2 * TP_BM)) * ((N + TP_BN - 1) / TP_BN) * ksplits;
  const int pairs = (int)(tiles < pairs_max ? tiles : pairs_max);       // persistent: a pair per two SMs walks the units
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  pair_launch_config(cfg, attr, pairs, 192, TP_SMEM, stream);
  cudaLaunchKernelEx(&cfg, kernel, ma, mw, bias, out, M, N, K, status, extra, ksplits, kb_per_split);
  return launch_status("gemm_pair");
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_gemm_pair_supports(int M, int N, int K) {
  return M >= 1 && N >= 8 && K >= 8 && K % 8 == 0 && M <= (1 << 24) && sllm::num_sms() >= 2 && encode_fn() != nullptr;
}

// The same product and epilogues as sllm_gemm_tcgen05 (0: float32 out[M, N] (+bias); 1: bfloat16; 2: bfloat16
// out[M, N/2] = silu(gate) * up for W rows interleaved in blocks of 8), by pairs of CTAs on 256 x 256 tiles, and
// 3: residual[M, N] (float32) += the product (+bias) in place (`out` is ignored).
// `wide`: 0 tiles of 256 x 256; 1 tiles of 256 x 512 (for matrices with few rows of W); 2 tiles of 256 x 128 (for results
// with few tiles); 448, 384, 320: tiles of 256 x that many columns (epilogues 0 and 3; where they fill the pairs of SMs
// better than 512-wide ones).
// ssq_in != null: A is bfloat16(stream * gain) of an RMSNorm still owed; ssq_in [M][stride_in] holds parts_in partial
//   sums of squares of the stream's rows (width_in wide) and every row of the product is multiplied by
//   rsqrt(sum / width_in + eps_in) before bias and activation.
// gain != null (epilogue 3): also write xg_out [M, N] = bfloat16(residual * gain) and ssq_out [M][stride_out], the
//   sums of squares of the new residual per row and block of columns (sllm_gemm_pair_parts_of(N, wide) entries a row).
// `status` is one int of device memory, zero before the launch; non-zero afterwards means a wait inside the
// kernel ran out (41 producer, 42 MMA issuer, 43 epilogue) and the result is not valid.
SLLM_EXPORT int sllm_gemm_pair_parts(int N) { return (N + 127) / 128; }

// the same for the tile form `wide` (see sllm_gemm_pair): tiles of 448, 384 or 320 columns leave four sums a tile
// (two of 128 columns, two of 96, 64 or 32); the sums of the last tile's blocks that start beyond N are not made
SLLM_EXPORT int sllm_gemm_pair_parts_of(int N, int wide) {
  if (wide != 448 && wide != 384 && wide != 320) return sllm_gemm_pair_parts(N);
  const int full = N / wide, rest = N - full * wide;
  const int starts[4] = {0, 128, wide / 2, wide / 2 + 128};
  int parts = 4 * full;
  for (int i = 0; i < 4; ++i) parts += rest > starts[i] ? 1 : 0;
  return parts;
}

// slices of K a request for `want` comes to (empty slices are not made): the rows of the stack of partial sums
SLLM_EXPORT int sllm_gemm_pair_splits(int K, int want) {
  const int k_blocks = (K + TP_BK - 1) / TP_BK;
  if (want < 1) want = 1;
  if (want > k_blocks) want = k_blocks;
  const int per = (k_blocks + want - 1) / want;
  return (k_blocks + per - 1) / per;
}

SLLM_EXPORT int sllm_gemm_pair(const void* A, const void* W, const float* bias, void* out, int M, int N, int K,
                               int epilogue, int wide, int want_splits, const float* ssq_in, int parts_in, int stride_in, float eps_in,
                               int width_in, float* residual, const float* gain, void* xg_out, float* ssq_out, int stride_out,
                               int* status, cudaStream_t stream) {
  SLLM_REQUIRE(sllm_gemm_pair_supports(M, N, K), "gemm_pair: sizes M=%d N=%d K=%d (K must be a multiple of 8)", M, N, K);
  SLLM_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_pair: operands must be 16-byte aligned");
  SLLM_REQUIRE(status != nullptr, "gemm_pair: a status word is required");
  SLLM_REQUIRE(epilogue != TG_EPI_SILU || N % 16 == 0, "gemm_pair: the SiLU epilogue needs N %% 16 == 0");
  TgExtra extra;
  if (ssq_in != nullptr) {
    SLLM_REQUIRE(parts_in >= 1 && stride_in >= parts_in && width_in >= 1, "gemm_pair: a table of %d partial sums (row stride %d) over width %d",
                 parts_in, stride_in, width_in);
    extra.ssq_in = ssq_in; extra.parts_in = parts_in; extra.stride_in = stride_in; extra.eps_in = eps_in;
    extra.inv_width_in = 1.0f / (float)width_in;
  }
  if (epilogue == TG_EPI_RESID) {
    SLLM_REQUIRE(residual != nullptr && N % 4 == 0 && ((uintptr_t)residual & 15) == 0, "gemm_pair: the residual epilogue needs a 16-byte aligned float32 residual and N %% 4 == 0");
    extra.residual = residual;
    if (gain != nullptr) {
      SLLM_REQUIRE(xg_out != nullptr && ssq_out != nullptr && stride_out >= sllm_gemm_pair_parts_of(N, wide) && ((uintptr_t)xg_out & 15) == 0,
                   "gemm_pair: the next norm's input needs both destinations (row stride %d, %d parts)", stride_out, sllm_gemm_pair_parts_of(N, wide));
      extra.gain = gain; extra.xg = (__nv_bfloat16*)xg_out; extra.ssq_out = ssq_out; extra.stride_out = stride_out;
    }
  } else {
    SLLM_REQUIRE(out != nullptr, "gemm_pair: no destination");
  }
  CUtensorMap ma, mw;
  const CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_128B;
  const bool wide_form = wide == 1 || wide == 448 || wide == 384 || wide == 320;
  SLLM_REQUIRE((wide >= 0 && wide <= 2) || wide_form, "gemm_pair: tile form %d (0: 256 x 256, 1: 256 x 512, 2: 256 x 128; 448, 384, 320: 256 x that)", wide);
  SLLM_REQUIRE(wide <= 2 || epilogue == TG_EPI_F32 || epilogue == TG_EPI_RESID,
               "gemm_pair: tiles of %d columns only with the float32 and the residual epilogue", wide);
  const int wide_cols = wide == 1 ? TP_BN_WIDE : wide;
  const int ksplits = sllm_gemm_pair_splits(K, want_splits);
  const int kb_per_split = (((K + TP_BK - 1) / TP_BK) + ksplits - 1) / ksplits;
  SLLM_REQUIRE(ksplits == 1 || (epilogue == TG_EPI_F32 && !wide_form && ssq_in == nullptr),
               "gemm_pair: slices of K leave a stack of float32 partial sums (plain epilogue, not the 512-wide tiles, no owed norm)");
  if (!make_map(&ma, A, M, K, TP_BM, promo) || !make_map(&mw, W, N, K, wide_form ? wide_cols / 2 : wide == 2 ? 64 : 128, promo)) {
    set_error("gemm_pair: cuTensorMapEncodeTiled failed");
    return SLLM_ERR_LAUNCH;
  }
#define GO(EPI_)                                                                                   \
  return wide == 1 ? launch_tp_wide<EPI_, 128>(ma, mw, bias, out, M, N, K, status, stream, extra)  \
       : wide == 2 ? launch_tp<EPI_, 128>(ma, mw, bias, out, M, N, K, status, stream, extra, ksplits, kb_per_split) \
                   : launch_tp<EPI_, 256>(ma, mw, bias, out, M, N, K, status, stream, extra, ksplits, kb_per_split);
#define GO_COLS(EPI_)                                                                                          \
  if (wide == 448) return launch_tp_wide<EPI_, 96>(ma, mw, bias, out, M, N, K, status, stream, extra);         \
  if (wide == 384) return launch_tp_wide<EPI_, 64>(ma, mw, bias, out, M, N, K, status, stream, extra);         \
  if (wide == 320) return launch_tp_wide<EPI_, 32>(ma, mw, bias, out, M, N, K, status, stream, extra);
  if (epilogue == TG_EPI_F32) { GO_COLS(TG_EPI_F32) }
  if (epilogue == TG_EPI_RESID) { GO_COLS(TG_EPI_RESID) }
#undef GO_COLS
  switch (epilogue) {
    case TG_EPI_F32: GO(TG_EPI_F32)
    case TG_EPI_BF16: GO(TG_EPI_BF16)
    case TG_EPI_SILU: GO(TG_EPI_SILU)
    case TG_EPI_RESID: GO(TG_EPI_RESID)
  }
#undef GO
  SLLM_REQUIRE(false, "gemm_pair: unknown epilogue %d", epilogue);
}
