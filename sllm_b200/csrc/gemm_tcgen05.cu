// bfloat16 matrix product on the 5th-generation tensor cores, for prompt portions:
//   C[M, N] = A[M, K] W[N, K]^T (+ bias), float32 accumulation in tensor memory.
//
// The kernel is persistent: one CTA per SM walks over 128 x 256 tiles of C (M tiles fastest, so
// that the CTAs working at the same time share few W tiles and all of A through L2).  The
// accumulator is double-buffered in tensor memory (2 x 256 of its 512 columns), so the epilogue of
// one tile runs while the next tile's products are issued.  The six warps have three jobs:
//   warp 0  one lane issues the TMA loads: per 64-wide k block a 128 x 64 box of A and a
//           256 x 64 box of W land in shared memory in the 128-byte-swizzled layout the tensor
//           core reads, four stages deep (48 KB a stage), each signalling an mbarrier;
//   warp 1  allocates the tensor memory; one lane waits for an accumulator buffer to be free,
//           issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=256, K=16) four times per stage,
//           commits the stage's "empty" barrier and, after a tile's last stage, the buffer's
//           "accumulator full" barrier;
//   warps 2-5  wait for a full accumulator, read their quarter of its 128 lanes with tcgen05.ld
//           (32 lanes x 32 columns at a time), store C (with bias / as bfloat16 / through
//           SiLU(gate)*up for a gate|up matrix interleaved in blocks of 8) and hand the buffer back.
// Both operands are K-major (rows contiguous in k) as checkpoints store W and as activations lie.
// Out-of-range rows and the k tail are zero-filled by the TMA unit, so any M, N and any K that is
// a multiple of 8 is taken.
//
// Every wait on an mbarrier is bounded: after its limit the waiter records a code in the status
// word the host passes, waits (bounded) for the copies it has in flight, the tensor memory is
// freed, and the kernel returns; the host reads the status after the launch's stream is synchronised.
// No multicast, no clusters: each CTA loads both of its operands.
//
// The reference has no such kernel: its products are cublasGemmEx calls on one token
// (kernels/cuda/kernels.cu:752-767) and its prefill runs in numpy (serving/executor.py:255-265).
#include <stdio.h>

#include "gemm_epilogue.cuh"

namespace sllm {

constexpr int TG_BM = 128, TG_BN = 256, TG_BK = 64, TG_STAGES = 4;
constexpr int TG_A_BYTES = TG_BM * TG_BK * 2;            // 16 KB
constexpr int TG_B_BYTES = TG_BN * TG_BK * 2;            // 32 KB
constexpr int TG_STAGE_BYTES = TG_A_BYTES + TG_B_BYTES;
constexpr int TG_SMEM = TG_STAGES * TG_STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */;
constexpr int TG_TMEM_COLS = 512;                        // two accumulators of 256 columns

template <int EPI>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const float* __restrict__ bias, void* __restrict__ out, int M, int N, int K, int* __restrict__ status) {
  extern __shared__ unsigned char tg_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tg_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + TG_STAGES * TG_STAGE_BYTES);
  uint64_t* empty = full + TG_STAGES;
  uint64_t* acc_full = empty + TG_STAGES;           // [2]
  uint64_t* acc_empty = acc_full + 2;               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + TG_BM - 1) / TG_BM, n_tiles = (N + TG_BN - 1) / TG_BN;
  const int tiles = m_tiles * n_tiles;
  const int k_blocks = (K + TG_BK - 1) / TG_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TG_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);                  // the four epilogue warps
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TG_TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                                     // A is the work of the step's earlier kernels

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int it = 0, issued = 0;                       // k blocks issued so far, over all tiles
      for (int tile = blockIdx.x; tile < tiles && !*failed; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * TG_BM, n0 = (tile / m_tiles) * TG_BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % TG_STAGES, round = it / TG_STAGES;
          if (!mbar_wait(&empty[s], (round & 1) ^ 1) || *failed) {
            if (!*failed) { *failed = 1; atomicExch(status, 1); }
            break;
          }
          unsigned char* sa = smem + s * TG_STAGE_BYTES;
          mbar_expect_tx(&full[s], TG_STAGE_BYTES);
          tma_load_2d(sa, &map_a, kb * TG_BK, m0, &full[s]);
          tma_load_2d(sa + TG_A_BYTES, &map_w, kb * TG_BK, n0, &full[s]);
          issued = it + 1;
        }
      }
      if (*failed) {
        // let the copies already issued land before the CTA gives its shared memory back
        for (int i = issued > TG_STAGES ? issued - TG_STAGES : 0; i < issued; ++i)
          mbar_wait(&full[i % TG_STAGES], (i / TG_STAGES) & 1, TMA_DRAIN_NS);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // instruction descriptor: D float32, A and B bfloat16, both K-major, N = 256, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TG_BN >> 3) << 17) | ((uint32_t)(TG_BM >> 4) << 24);
      int it = 0, local = 0;
      for (int tile = blockIdx.x; tile < tiles && !*failed; tile += gridDim.x, ++local) {
        const int b = local & 1;
        if (!mbar_wait(&acc_empty[b], ((local >> 1) & 1) ^ 1) || *failed) {     // the epilogue has drained this buffer
          if (!*failed) { *failed = 2; atomicExch(status, 2); }
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + b * TG_BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % TG_STAGES, round = it / TG_STAGES;
          if (!mbar_wait(&full[s], round & 1) || *failed) {
            if (!*failed) { *failed = 2; atomicExch(status, 2); }
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(smem + s * TG_STAGE_BYTES), b_addr = a_addr + TG_A_BYTES;
#pragma unroll
          for (int k = 0; k < TG_BK / 16; ++k)      // 16 k = 32 bytes further along the swizzled row
            umma_bf16(tmem_d, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc, (kb | k) ? 1u : 0u);
          umma_commit(&empty[s]);                   // arrives when these MMAs have read the stage
        }
        umma_commit(&acc_full[b]);                  // arrives when every MMA issued so far is done
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5 own TMEM lane quarters 2, 3, 0, 1 ----------------
    const int quarter = warp & 3;
    int local = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      const int b = local & 1;
      const int m0 = (tile % m_tiles) * TG_BM, n0 = (tile / m_tiles) * TG_BN;
      const bool ok = mbar_wait(&acc_full[b], (local >> 1) & 1);
      if (!ok && !*failed) { *failed = 3; atomicExch(status, 3); }
      if (!ok || *failed) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int m = m0 + quarter * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < TG_BN; c0 += 32) {
        if (n0 + c0 >= N) break;                    // warp-uniform
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + b * TG_BN + c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (m >= M) continue;
        tg_store_chunk<EPI>(r, m, n0 + c0, N, bias, out);
      }
      // this warp has read its quarter of the buffer: hand it back to the MMA issuer
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  pdl_launch_dependents();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TG_TMEM_COLS));
  }
}

// ---- host side --------------------------------------------------------------------------------

template <int EPI>
static int launch_tg(const CUtensorMap& ma, const CUtensorMap& mw, const float* bias, void* out, int M, int N, int K,
                     int* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, TG_SMEM) != cudaSuccess) {
      set_error("gemm_tcgen05: cannot raise the shared memory limit");
      return SLLM_ERR_LAUNCH;
    }
    configured = true;
  }
  const int num_sms = sllm::num_sms();
  const long long tiles = (long long)((M + TG_BM - 1) / TG_BM) * ((N + TG_BN - 1) / TG_BN);
  dim3 grid((unsigned)(tiles < num_sms ? tiles : num_sms));      // persistent: one CTA per SM walks the tiles
  launch_kernel(gemm_tcgen05_kernel<EPI>, grid, 192, TG_SMEM, stream, ma, mw, bias, out, M, N, K, status);
  return launch_status("gemm_tcgen05");
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_gemm_tcgen05_supports(int M, int N, int K) {
  return M >= 1 && N >= 8 && K >= 8 && K % 8 == 0 && M <= (1 << 24) && encode_fn() != nullptr;
}

// epilogue 0: float32 out[M, N] (+bias); 1: bfloat16 out[M, N] (+bias); 2: bfloat16 out[M, N/2] =
// silu(gate) * up for W rows interleaved in blocks of 8 (N a multiple of 16).
// `status` is one int of device memory, zero before the launch; non-zero afterwards means a wait
// inside the kernel ran out (1 producer, 2 MMA issuer, 3 epilogue) and `out` is not valid.
SLLM_EXPORT int sllm_gemm_tcgen05(const void* A, const void* W, const float* bias, void* out, int M, int N, int K,
                                  int epilogue, int* status, cudaStream_t stream) {
  SLLM_REQUIRE(M >= 1 && N >= 8 && K >= 8 && K % 8 == 0, "gemm_tcgen05: sizes M=%d N=%d K=%d (K must be a multiple of 8)", M, N, K);
  SLLM_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_tcgen05: operands must be 16-byte aligned");
  SLLM_REQUIRE(status != nullptr, "gemm_tcgen05: a status word is required");
  SLLM_REQUIRE(epilogue != TG_EPI_SILU || N % 16 == 0, "gemm_tcgen05: the SiLU epilogue needs N %% 16 == 0");
  CUtensorMap ma, mw;
  if (!make_map(&ma, A, M, K, TG_BM) || !make_map(&mw, W, N, K, TG_BN)) {
    set_error("gemm_tcgen05: cuTensorMapEncodeTiled failed");
    return SLLM_ERR_LAUNCH;
  }
  switch (epilogue) {
    case TG_EPI_F32: return launch_tg<TG_EPI_F32>(ma, mw, bias, out, M, N, K, status, stream);
    case TG_EPI_BF16: return launch_tg<TG_EPI_BF16>(ma, mw, bias, out, M, N, K, status, stream);
    case TG_EPI_SILU: return launch_tg<TG_EPI_SILU>(ma, mw, bias, out, M, N, K, status, stream);
  }
  SLLM_REQUIRE(false, "gemm_tcgen05: unknown epilogue %d", epilogue);
}
