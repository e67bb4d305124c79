// Weight-streaming linear layer on the 5th-generation tensor cores, for 33..128 tokens:
//   y[M, N] = x[M, K] W[N, K]^T (+ bias), bfloat16 operands, float32 accumulation in tensor memory.
//
// With this many tokens the product is still bound by reading W once, but the tokens no longer fit
// the register tiles of the mma.sync streaming kernel.  Here W is the tensor core's M operand: a CTA
// takes 128 weight rows and all the tokens (padded to BN = 64 or 128 columns of the accumulator), so
// every byte of W is loaded once, by TMA, into a deep ring of shared-memory stages (8 x 24 KB or
// 6 x 32 KB: enough bytes in flight to cover the latency of HBM at its full rate).  The few
// activations are re-read by every CTA, from L2.
//   warp 0      one lane issues the TMA loads: per 64-wide k block a 128 x 64 box of W and a BN x 64
//               box of x (rows beyond M are filled with zeros), 128-byte swizzle;
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (M = 128, N = BN, K = 16) four
//               times per stage and commits the stage's "empty" barrier; after a unit's last k block
//               it commits the accumulator's "full" barrier;
//   warps 2-5   read the accumulator (lane = weight row, column = token) and store it transposed:
//               for each token the 32 lanes of a warp write 32 consecutive outputs.
// Small N would leave most SMs idle, so a unit of work is (tile of 128 rows, slice of K); the
// partial sums of the slices go to a stack [splits, M, N] that the consumer adds in a fixed order
// (bias in the first).  The accumulator is double-buffered, so a CTA with several units stores one
// while the next one's products are issued.
// Epilogues: float32 (+bias), bfloat16 (+bias), SiLU(gate)*up for a gate|up matrix whose rows
// alternate in blocks of 8 (a gate row's up row is 8 lanes further).
//
// Every wait on an mbarrier is bounded; after its limit the waiter records a code in the status word.
// No multicast, no clusters.
//
// The reference's device path calls cublasGemmEx for these products (kernels/cuda/kernels.cu:752-767).
#include <stdio.h>

#include "tcgen05.cuh"

namespace sllm {

constexpr int LT_ROWS = 128, LT_BK = 64;
constexpr int LT_W_BYTES = LT_ROWS * LT_BK * 2;          // 16 KB

template <int BN>
struct LtCfg {
  static constexpr int STAGES = BN == 64 ? 8 : 6;
  static constexpr int X_BYTES = BN * LT_BK * 2;
  static constexpr int STAGE_BYTES = LT_W_BYTES + X_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */;
  static constexpr int TMEM_COLS = 2 * BN;                // two accumulators
};

#define LT_EPI_F32 0
#define LT_EPI_BF16 1
#define LT_EPI_SILU 2

template <int BN, int EPI>
__global__ void __launch_bounds__(192, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 const float* __restrict__ bias, void* __restrict__ out, int M, int N, int K, int splits, int kb_per_split,
                 int* __restrict__ status) {
  using C = LtCfg<BN>;
  extern __shared__ unsigned char lt_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(lt_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* acc_full = empty + C::STAGES;           // [2]
  uint64_t* acc_empty = acc_full + 2;               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = (N + LT_ROWS - 1) / LT_ROWS;
  const int units = tiles * splits;
  const int k_blocks = (K + LT_BK - 1) / LT_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
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
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      // this CTA's k blocks, unit after unit, as one sequence
      struct Cursor { int unit, kb, kb1, n0, it; };
      auto enter = [&](Cursor& c) {
        if (c.unit < units) {
          c.n0 = (c.unit / splits) * LT_ROWS;
          c.kb = (c.unit % splits) * kb_per_split;
          c.kb1 = min(k_blocks, c.kb + kb_per_split);
        }
      };
      auto advance = [&](Cursor& c) {
        ++c.it;
        if (++c.kb >= c.kb1) { c.unit += gridDim.x; enter(c); }
      };
      Cursor cw{(int)blockIdx.x, 0, 0, 0, 0};
      enter(cw);
      Cursor cx = cw;
      // The ring's first round: the weights do not depend on the step's earlier kernels and are
      // requested before the wait for them, the activations after it.
      int first = 0;
      for (; first < C::STAGES && cw.unit < units; ++first) {
        mbar_expect_tx(&full[first], C::STAGE_BYTES);
        tma_load_2d(smem + first * C::STAGE_BYTES, &map_w, cw.kb * LT_BK, cw.n0, &full[first]);
        advance(cw);
      }
      pdl_wait();
      for (int i = 0; i < first; ++i) {
        tma_load_2d(smem + i * C::STAGE_BYTES + LT_W_BYTES, &map_x, cx.kb * LT_BK, 0, &full[i]);
        advance(cx);
      }
      int issued = first;
      while (cw.unit < units && !*failed) {
        const int s = cw.it % C::STAGES, round = cw.it / C::STAGES;
        if (!mbar_wait(&empty[s], (round & 1) ^ 1) || *failed) {
          if (!*failed) { *failed = 1; atomicExch(status, 31); }
          break;
        }
        unsigned char* sw = smem + s * C::STAGE_BYTES;
        mbar_expect_tx(&full[s], C::STAGE_BYTES);
        tma_load_2d(sw, &map_w, cw.kb * LT_BK, cw.n0, &full[s]);
        tma_load_2d(sw + LT_W_BYTES, &map_x, cw.kb * LT_BK, 0, &full[s]);
        advance(cw);
        issued = cw.it;
      }
      if (*failed) {
        // let the copies already issued land before the CTA gives its shared memory back
        for (int i = issued > C::STAGES ? issued - C::STAGES : 0; i < issued; ++i)
          mbar_wait(&full[i % C::STAGES], (i / C::STAGES) & 1, TMA_DRAIN_NS);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // instruction descriptor: D float32, A and B bfloat16, both K-major, N = BN, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(LT_ROWS >> 4) << 24);
      int it = 0, local = 0;
      for (int unit = blockIdx.x; unit < units && !*failed; unit += gridDim.x, ++local) {
        const int split = unit % splits;
        const int kb0 = split * kb_per_split, kb1 = min(k_blocks, kb0 + kb_per_split);
        const int b = local & 1;
        if (!mbar_wait(&acc_empty[b], ((local >> 1) & 1) ^ 1) || *failed) {     // the epilogue has drained this buffer
          if (!*failed) { *failed = 2; atomicExch(status, 32); }
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + b * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % C::STAGES, round = it / C::STAGES;
          if (!mbar_wait(&full[s], round & 1) || *failed) {
            if (!*failed) { *failed = 2; atomicExch(status, 32); }
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t w_addr = smem_u32(smem + s * C::STAGE_BYTES), x_addr = w_addr + LT_W_BYTES;
#pragma unroll
          for (int k = 0; k < LT_BK / 16; ++k)      // 16 k = 32 bytes further along the swizzled row
            umma_bf16(tmem_d, umma_desc(w_addr + k * 32), umma_desc(x_addr + k * 32), idesc, (kb > kb0 || k) ? 1u : 0u);
          umma_commit(&empty[s]);                   // arrives when these MMAs have read the stage
        }
        umma_commit(&acc_full[b]);                  // arrives when every MMA issued so far is done
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5 own TMEM lane quarters 2, 3, 0, 1 ----------------
    const int quarter = warp & 3;
    int local = 0;
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x, ++local) {
      const int b = local & 1;
      const int n0 = (unit / splits) * LT_ROWS, split = unit % splits;
      const bool ok = mbar_wait(&acc_full[b], (local >> 1) & 1);
      if (!ok && !*failed) { *failed = 3; atomicExch(status, 33); }
      if (!ok || *failed) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int n = n0 + quarter * 32 + lane;       // this lane's weight row = output column
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (c0 >= M) break;                         // warp-uniform
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + b * BN + c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if constexpr (EPI == LT_EPI_SILU) {
          // lanes 0-7 and 16-23 hold gate rows, their up rows are 8 lanes further
          const int col = ((n0 + quarter * 32) >> 1) + (lane >> 4) * 8 + (lane & 7);
          const bool writer = (lane & 8) == 0 && n + 8 < N;
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + col;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float g = __uint_as_float(r[j]);
            const float u = __shfl_down_sync(0xffffffffu, g, 8);
            if (writer && c0 + j < M) o[(size_t)(c0 + j) * (N >> 1)] = __float2bfloat16_rn(g * (1.0f / (1.0f + expf(-g))) * u);
          }
        } else {
          if (n < N) {
            const float bv = (bias && split == 0) ? bias[n] : 0.f;
            if constexpr (EPI == LT_EPI_F32) {
              float* o = reinterpret_cast<float*>(out) + (size_t)split * M * N + n;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (c0 + j < M) o[(size_t)(c0 + j) * N] = __uint_as_float(r[j]) + bv;
            } else {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + n;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (c0 + j < M) o[(size_t)(c0 + j) * N] = __float2bfloat16_rn(__uint_as_float(r[j]) + bv);
            }
          }
        }
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS));
  }
}

// ---- host side --------------------------------------------------------------------------------

static int lt_num_sms() { return sllm::num_sms(); }

template <int BN, int EPI>
static int launch_lt(const CUtensorMap& mw, const CUtensorMap& mx, const float* bias, void* out, int M, int N, int K,
                     int splits, int kb_per_split, int* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(linear_tc_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, LtCfg<BN>::SMEM) != cudaSuccess) {
      set_error("linear_tc: cannot raise the shared memory limit");
      return SLLM_ERR_LAUNCH;
    }
    configured = true;
  }
  const int units = ((N + LT_ROWS - 1) / LT_ROWS) * splits, sms = lt_num_sms();
  dim3 grid((unsigned)(units < sms ? units : sms));              // persistent: one CTA per SM walks the units
  launch_kernel(linear_tc_kernel<BN, EPI>, grid, 192, LtCfg<BN>::SMEM, stream, mw, mx, bias, out, M, N, K, splits, kb_per_split, status);
  return launch_status("linear_tc");
}

// k blocks a slice takes when K is cut `want` ways, and how many slices that makes
static void lt_slices(int K, int want, int* kb_per_split, int* splits) {
  const int k_blocks = (K + LT_BK - 1) / LT_BK;
  if (want < 1) want = 1;
  if (want > k_blocks) want = k_blocks;
  *kb_per_split = (k_blocks + want - 1) / want;
  *splits = (k_blocks + *kb_per_split - 1) / *kb_per_split;
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_linear_tc_supports(int M, int N, int K) {
  return M >= 1 && M <= 128 && N >= 8 && K >= 8 && K % 8 == 0 && encode_fn() != nullptr;
}

// the number of partial sums that `want` slices of K come to (empty slices are not made)
SLLM_EXPORT int sllm_linear_tc_splits(int K, int want) {
  int kbps, splits;
  lt_slices(K, want, &kbps, &splits);
  return splits;
}

// epilogue 0: float32 out[splits, M, N] (bias in the first slice); 1: bfloat16 out[M, N] (+bias; one
// slice); 2: bfloat16 out[M, N/2] = silu(gate) * up for W rows interleaved in blocks of 8 (N a multiple
// of 16; one slice).  `status` as for sllm_gemm_tcgen05 (codes 31 producer, 32 MMA issuer, 33 epilogue).
SLLM_EXPORT int sllm_linear_tc(const void* x, const void* W, const float* bias, void* out, int M, int N, int K, int want_splits,
                               int epilogue, int* status, cudaStream_t stream) {
  SLLM_REQUIRE(M >= 1 && M <= 128 && N >= 8 && K >= 8 && K % 8 == 0, "linear_tc: sizes M=%d N=%d K=%d (M <= 128, K a multiple of 8)", M, N, K);
  SLLM_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)W & 15) == 0, "linear_tc: operands must be 16-byte aligned");
  SLLM_REQUIRE(status != nullptr, "linear_tc: a status word is required");
  SLLM_REQUIRE(epilogue != LT_EPI_SILU || N % 16 == 0, "linear_tc: the SiLU epilogue needs N %% 16 == 0");
  SLLM_REQUIRE(epilogue == LT_EPI_F32 || want_splits <= 1, "linear_tc: only the float32 result can be a stack of partial sums");
  int kbps, splits;
  lt_slices(K, want_splits, &kbps, &splits);
  const int bn = M <= 64 ? 64 : 128;
  CUtensorMap mw, mx;
  if (!make_map(&mw, W, N, K, LT_ROWS) || !make_map(&mx, x, M, K, bn)) {
    set_error("linear_tc: cuTensorMapEncodeTiled failed");
    return SLLM_ERR_LAUNCH;
  }
#define LT_LAUNCH(BN_, EPI_) return launch_lt<BN_, EPI_>(mw, mx, bias, out, M, N, K, splits, kbps, status, stream)
  if (bn == 64) {
    switch (epilogue) {
      case LT_EPI_F32: LT_LAUNCH(64, LT_EPI_F32);
      case LT_EPI_BF16: LT_LAUNCH(64, LT_EPI_BF16);
      case LT_EPI_SILU: LT_LAUNCH(64, LT_EPI_SILU);
    }
  } else {
    switch (epilogue) {
      case LT_EPI_F32: LT_LAUNCH(128, LT_EPI_F32);
      case LT_EPI_BF16: LT_LAUNCH(128, LT_EPI_BF16);
      case LT_EPI_SILU: LT_LAUNCH(128, LT_EPI_SILU);
    }
  }
#undef LT_LAUNCH
  SLLM_REQUIRE(false, "linear_tc: unknown epilogue %d", epilogue);
}
