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
// The reference has no such kernel: its products are cublasGemmEx calls on one token
// (kernels/cuda/kernels.cu:752-767) and its prefill runs in numpy (serving/executor.py:255-265).
#include <stdio.h>

#include "gemm_epilogue.cuh"

namespace sllm {

constexpr int TP_BM = 128;                                // rows of A (and of C) per CTA; the pair's tile has 256
constexpr int TP_BN = 256;                                // columns of C per tile; each CTA loads 128 rows of W
constexpr int TP_BK = 64, TP_STAGES = 6;
constexpr int TP_A_BYTES = TP_BM * TP_BK * 2;             // 16 KB
constexpr int TP_B_BYTES = (TP_BN / 2) * TP_BK * 2;       // 16 KB
constexpr int TP_STAGE_BYTES = TP_A_BYTES + TP_B_BYTES;
constexpr int TP_SMEM = TP_STAGES * TP_STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */;
constexpr int TP_TMEM_COLS = 512;                         // two accumulators of 256 columns

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

template <int EPI>
__global__ void __launch_bounds__(192, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                 const float* __restrict__ bias, void* __restrict__ out, int M, int N, int K, int* __restrict__ status) {
  extern __shared__ unsigned char tp_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tp_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + TP_STAGES * TP_STAGE_BYTES);
  uint64_t* empty = full + TP_STAGES;
  uint64_t* acc_full = empty + TP_STAGES;           // [2]
  uint64_t* acc_empty = acc_full + 2;               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: the CTA whose thread issues the products
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int m_tiles = (M + 2 * TP_BM - 1) / (2 * TP_BM), n_tiles = (N + TP_BN - 1) / TP_BN;
  const int tiles = m_tiles * n_tiles;
  const int k_blocks = (K + TP_BK - 1) / TP_BK;

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
      for (int tile = pair; tile < tiles && !*failed; tile += pairs) {
        const int m0 = (tile % m_tiles) * 2 * TP_BM + (int)rank * TP_BM;
        const int n0 = (tile / m_tiles) * TP_BN + (int)rank * (TP_BN / 2);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % TP_STAGES, round = it / TP_STAGES;
          if (!mbar_wait(&empty[s], (round & 1) ^ 1) || *failed) {
            if (!*failed) { *failed = 1; atomicExch(status, 1); }
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
      int it = 0, local = 0;
      for (int tile = pair; tile < tiles && !*failed; tile += pairs, ++local) {
        const int b = local & 1;
        if (!mbar_wait(&acc_empty[b], ((local >> 1) & 1) ^ 1) || *failed) {     // both epilogues have drained this buffer
          if (!*failed) { *failed = 2; atomicExch(status, 2); }
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + b * TP_BN;
        bool gave_up = false;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % TP_STAGES, round = it / TP_STAGES;
          if (!mbar_wait(&full[s], round & 1) || *failed) {
            if (!*failed) { *failed = 2; atomicExch(status, 2); }
            gave_up = true;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(smem + s * TP_STAGE_BYTES), b_addr = a_addr + TP_A_BYTES;
#pragma unroll
          for (int k = 0; k < TP_BK / 16; ++k)      // 16 k = 32 bytes further along the swizzled row
            umma_bf16_pair(tmem_d, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc, (kb | k) ? 1u : 0u);
          umma_commit_pair(&empty[s]);              // arrives in both CTAs when these products have read the stage
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
    for (int tile = pair; tile < tiles; tile += pairs, ++local) {
      const int b = local & 1;
      const int m0 = (tile % m_tiles) * 2 * TP_BM + (int)rank * TP_BM, n0 = (tile / m_tiles) * TP_BN;
      const bool ok = mbar_wait(&acc_full[b], (local >> 1) & 1);
      if (!ok && !*failed) { *failed = 3; atomicExch(status, 3); }
      if (!ok || *failed) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int m = m0 + quarter * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < TP_BN; c0 += 32) {
        if (n0 + c0 >= N) break;                    // warp-uniform
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + b * TP_BN + c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (m >= M) continue;
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

// ---- host side --------------------------------------------------------------------------------

template <int EPI>
static int launch_tp(const CUtensorMap& ma, const CUtensorMap& mw, const float* bias, void* out, int M, int N, int K,
                     int* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM) != cudaSuccess) {
      set_error("gemm_pair: cannot raise the shared memory limit");
      return SLLM_ERR_LAUNCH;
    }
    configured = true;
  }
  const int pairs_max = sllm::num_sms() / 2;
  const long long tiles = (long long)((M + 2 * TP_BM - 1) / (2 * TP_BM)) * ((N + TP_BN - 1) / TP_BN);
  const int pairs = (int)(tiles < pairs_max ? tiles : pairs_max);       // persistent: a pair per two SMs walks the tiles
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = TP_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, gemm_pair_kernel<EPI>, ma, mw, bias, out, M, N, K, status);
  return launch_status("gemm_pair");
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_gemm_pair_supports(int M, int N, int K) {
  return M >= 1 && N >= 8 && K >= 8 && K % 8 == 0 && M <= (1 << 24) && sllm::num_sms() >= 2 && encode_fn() != nullptr;
}

// The same product and epilogues as sllm_gemm_tcgen05 (0: float32 out[M, N] (+bias); 1: bfloat16; 2: bfloat16
// out[M, N/2] = silu(gate) * up for W rows interleaved in blocks of 8), by pairs of CTAs on 256 x 256 tiles.
// `status` is one int of device memory, zero before the launch; non-zero afterwards means a wait inside the
// kernel ran out (1 producer, 2 MMA issuer, 3 epilogue) and `out` is not valid.
SLLM_EXPORT int sllm_gemm_pair(const void* A, const void* W, const float* bias, void* out, int M, int N, int K,
                               int epilogue, int* status, cudaStream_t stream) {
  SLLM_REQUIRE(sllm_gemm_pair_supports(M, N, K), "gemm_pair: sizes M=%d N=%d K=%d (K must be a multiple of 8)", M, N, K);
  SLLM_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_pair: operands must be 16-byte aligned");
  SLLM_REQUIRE(status != nullptr, "gemm_pair: a status word is required");
  SLLM_REQUIRE(epilogue != TG_EPI_SILU || N % 16 == 0, "gemm_pair: the SiLU epilogue needs N %% 16 == 0");
  CUtensorMap ma, mw;
  if (!make_map(&ma, A, M, K, TP_BM) || !make_map(&mw, W, N, K, TP_BN / 2)) {
    set_error("gemm_pair: cuTensorMapEncodeTiled failed");
    return SLLM_ERR_LAUNCH;
  }
  switch (epilogue) {
    case TG_EPI_F32: return launch_tp<TG_EPI_F32>(ma, mw, bias, out, M, N, K, status, stream);
    case TG_EPI_BF16: return launch_tp<TG_EPI_BF16>(ma, mw, bias, out, M, N, K, status, stream);
    case TG_EPI_SILU: return launch_tp<TG_EPI_SILU>(ma, mw, bias, out, M, N, K, status, stream);
  }
  SLLM_REQUIRE(false, "gemm_pair: unknown epilogue %d", epilogue);
}
