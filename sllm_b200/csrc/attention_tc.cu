// Attention of prompt portions over the paged cache on the 5th-generation tensor cores
// (tcgen05, accumulators in tensor memory): causal GQA with an online softmax, bfloat16 in,
// float32 scores, softmax and output accumulation.
//
// A CTA takes RT (one or two) 128-row tiles of (token, head-in-group) rows of one request and one kv
// head and walks the keys in tiles of 64.  The form in use has one row tile: two CTAs share an SM
// (96 KB of shared memory and 256 columns of tensor memory each), so that one CTA's softmax runs
// while the other's products do.  With two row tiles a key/value tile fetched once serves both and
// the shared memory of a whole SM holds four key/value tiles in flight; it is kept and tested, but
// measured slower at every prompt length tried (the engine does not choose it).
// Per row tile four softmax warps, then one warp for TMA and one for the MMAs:
//   softmax    thread r owns row r.  It reads its row of S = Q K^T from tensor memory
//              (tcgen05.ld), scales and masks it, keeps the row's running maximum and sum, writes
//              P = exp2(S - max) as bfloat16 back into the first half of the same columns
//              (tcgen05.st, two keys per 32-bit column), from where the tensor core takes it as the
//              A operand, and at the end reads O, divides by the sum and stores the row.
//              The maximum in use only moves when a tile's maximum exceeds it by more than 2^8
//              (then O in tensor memory is rescaled: tcgen05.ld, multiply, tcgen05.st); the result
//              is the same sum with a different common factor, which cancels in O / sum.
//   producer   one lane issues the TMA loads: per page and 64-column half of the head one box of
//              K and one of V (page_size x 64 elements, 128-byte swizzle), or one box each for a
//              tile whose pages have consecutive ids; K and V in rings of their own, so that the
//              next keys load as soon as the scores that read a K buffer are done;
//   issuer     allocates the tensor memory; one lane issues S(j) = Q K(j)^T (M=128, N=64, K=16,
//              head_dim/16 times) two tiles ahead of the softmax, and O += P(j) V(j) (M=128,
//              N=head_dim, K=16, four times; V is read as stored, keys down the rows: an MN-major
//              operand) when P(j) is written.  S(j+2) overwrites the columns of P(j): it is issued
//              only when a barrier committed behind P(j) V(j) says that product is complete.  With two row
//              tiles it serves whichever has an event pending, so one's products run under the
//              other's softmax.
// Per row tile S/P is double-buffered in tensor memory (2 x 64 columns) and O takes head_dim columns.
// Nothing in the loop waits for a round trip: the softmax of tile j+1 needs S(j+1), issued long
// before, and only a rescale of O waits for the product before it.
//
// What lies in the cache beyond a request's last key inside its last page, and in the part of a
// stage that no page fills, meets a probability of exactly zero; it must be finite, so the stages
// are zeroed before the first copy, and the cache pool is expected to hold finite numbers only
// (it starts as zeros and only keys and values are written into it).
//
// Every wait on an mbarrier is bounded; a wait that runs out records a code in the status word
// (21 producer, 22 MMA issuer, 23 softmax), the roles fall through, tensor memory is freed and the
// kernel returns.  No multicast, no clusters.
//
// Formulas: ref/qwen3_5.py:373-390 (scores * scale, causal mask, softmax, P.V);
// ref/standard.py:65-68 (query head h reads kv head h / group).  The reference has no such kernel:
// its prefill attention runs in numpy (serving/executor.py:255-265).
#include <math.h>
#include <stdio.h>

#include <mutex>
#include <unordered_map>

#include "tcgen05.cuh"

namespace sllm {

struct AttnTcParams {
  const __nv_bfloat16* q;        // [T, nq, HD]
  __nv_bfloat16* out;            // [T, nq, HD]
  const int* block_tables;       // [S, max_pages]
  const int* q_start;            // [S+1]
  const int* ctx_len;            // [S]
  const int* tile_seq;           // [tiles]
  const int* tile_row0;          // [tiles]
  int* status;
  int max_pages, page_size, nq, nkv;
  int page_runs;                 // the run maps are valid: a key tile whose pages have consecutive ids is one box of K and one of V
  float scale_log2;              // scale * log2(e)
  // the context cut in num_splits ranges of tiles_per_split key tiles each (grid z); with more than one,
  // a CTA writes what its range gives to part_o [splits, T, nq, HD] (normalised) and part_lse
  // [splits, T, nq] (log2 of its sum of exponentials, -inf where its range holds no key of the row)
  int num_splits, tiles_per_split, total_tokens;
  float* part_o;
  float* part_lse;
};

constexpr int TC_BM = 128, TC_BN = 64;
constexpr float TC_RESCALE_STEP = 8.0f;     // log2 units the maximum may lag behind before O is rescaled

template <int HD, int RT> struct TcLayout {
  static constexpr int HALVES = HD / 64;
  static constexpr int STAGES = RT == 1 ? 2 : 4;
  static constexpr int THREADS = 128 * RT + 64;
  static constexpr int Q_BYTES = HALVES * TC_BM * 128;       // one row tile
  static constexpr int KV_BYTES = HALVES * TC_BN * 128;      // one of K or V, one stage
  static constexpr int K_OFF = RT * Q_BYTES;
  static constexpr int V_OFF = K_OFF + STAGES * KV_BYTES;
  static constexpr int BAR_OFF = V_OFF + STAGES * KV_BYTES;
  static constexpr int SMEM = BAR_OFF + 256;
  static constexpr int TMEM_TILE = 256;                      // per row tile: 2 x 64 (S) + HD (O), a power of two
  static constexpr int TMEM_COLS = RT * TMEM_TILE;
  static constexpr int O_COL = 2 * TC_BN;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The softmax thread walks its row's 64 keys alone, and every instruction of that walk lengthens the
// key tile's period, so the walk uses the two-wide float32 forms (one instruction for two
// multiply-adds or two sums, each rounded as the scalar form rounds) and the maximum of three.
__device__ __forceinline__ float2 fma_x2(float a0, float a1, float b, float c) {
  unsigned long long ra, rb, rc, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a0), "f"(a1));
  asm("mov.b64 %0, {%1, %1};" : "=l"(rb) : "f"(b));
  asm("mov.b64 %0, {%1, %1};" : "=l"(rc) : "f"(c));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ float2 add_x2(float2 a, float2 b) {
  unsigned long long ra, rb, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <int HD, int RT>
__global__ void __launch_bounds__(TcLayout<HD, RT>::THREADS, RT == 1 ? 2 : 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const __grid_constant__ CUtensorMap run_k, const __grid_constant__ CUtensorMap run_v,
                    const AttnTcParams p) {
  using L = TcLayout<HD, RT>;
  constexpr int HALVES = L::HALVES;
  constexpr int CHUNKS = HD / 8;
  constexpr int TC_STAGES = L::STAGES, TC_THREADS = L::THREADS;
  constexpr int PRODUCER = 4 * RT, ISSUER = 4 * RT + 1;      // warp numbers
  extern __shared__ __align__(1024) unsigned char tc_smem[];
  unsigned char* smem = tc_smem;
  // K and V have rings of their own: a K buffer is free again when the scores of its tile are done,
  // long before the tile's P.V, so the next keys load under the softmax
  uint64_t* k_full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);    // [STAGES] the buffer's K has landed
  uint64_t* k_empty = k_full + TC_STAGES;                               // [STAGES] the scores that read it are done
  uint64_t* v_full = k_empty + TC_STAGES;                               // [STAGES] the buffer's V has landed
  uint64_t* v_empty = v_full + TC_STAGES;                               // [STAGES] the P.V that read it is done
  uint64_t* s_full = v_empty + TC_STAGES;                               // [RT][2] S buffer holds Q K^T
  uint64_t* p_full = s_full + 2 * RT;                                   // [RT][2] the buffer holds P, O is rescaled
  uint64_t* q_full = p_full + 2 * RT;                                   // [RT] the row tile's queries are in place
  uint64_t* s_free = q_full + RT;                                       // [RT][2] the P.V that read the buffer's P is complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + 2 * RT);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2 * RT; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_free[s], 1);
      mbar_init(&p_full[s], 4);                   // the four softmax warps of the row tile
    }
    for (int t = 0; t < RT; ++t) {
      mbar_init(&q_full[t], 4);
    }
    // a wait that ran out in another CTA voids the result anyway: the CTAs that start after it do nothing
    *failed = *reinterpret_cast<volatile int*>(p.status);
    if ((smem_u32(smem) & 1023u) != 0) {            // the swizzled layouts need a 1024-byte base
      *failed = 20;
      atomicExch(p.status, 20);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == ISSUER) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(L::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  // the stages start as zeros (see the header)
  for (int o = tid * 16; o < 2 * TC_STAGES * L::KV_BYTES; o += TC_THREADS * 16)
    *reinterpret_cast<uint4*>(smem + L::K_OFF + o) = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_wait();       // everything below reads what the step's earlier kernels or its batch upload wrote
  // The KV head is the fastest index of the grid: the row tiles come sorted by their number of keys,
  // longest first, and CTAs start in the grid's order, so every head's long tiles start in the first
  // wave (with the head as the slow index the last heads' long tiles started behind a whole wave: a
  // prompt of 2,048 tokens took 87 us in place of about 50).
  const int tile_i = blockIdx.x / p.nkv, kvh = blockIdx.x % p.nkv;
  const int seq = p.tile_seq[tile_i], row0 = p.tile_row0[tile_i];
  const int G = p.nq / p.nkv;
  const int q0 = p.q_start[seq], q_len = p.q_start[seq + 1] - q0, ctx = p.ctx_len[seq];
  const int rows_total = q_len * G;
  const int pos0 = ctx - q_len;                  // position of the request's first token of this step
  // per row tile t: its keys end at key_end[t] (exclusive), in n_of[t] key tiles; later rows see more keys
  // This CTA's range of the context: key tiles [tile0, tile0 + tiles_per_split).  Key tile j below is
  // the range's j-th, key tile tile0 + j of the request.
  const int tile0 = (int)blockIdx.z * p.tiles_per_split;
  int key_end[RT], n_of[RT];
#pragma unroll
  for (int t = 0; t < RT; ++t) {
    const int lo = row0 + t * TC_BM, hi = min(lo + TC_BM, rows_total);
    key_end[t] = hi > lo ? pos0 + (hi - 1) / G + 1 : 0;
    n_of[t] = min(max((key_end[t] + TC_BN - 1) / TC_BN - tile0, 0), p.tiles_per_split);
  }
  const int key_hi = RT == 1 ? key_end[0] : max(key_end[0], key_end[RT - 1]);
  const int n_tiles = RT == 1 ? n_of[0] : max(n_of[0], n_of[RT - 1]);
  const int* bt = p.block_tables + (size_t)seq * p.max_pages;

  if (warp == PRODUCER) {
    // ---------------- TMA producer ----------------
    if (lane == 0 && !*failed) {
      const int ps = p.page_size, per_tile = TC_BN / ps;
      // the copies of one of K (which = 0) or V (1) for key tile j into its ring buffer
      auto load_tile = [&](int which, int j) {
        const int s = j % TC_STAGES;
        uint64_t* full = which ? &v_full[s] : &k_full[s];
        unsigned char* dst = smem + (which ? L::V_OFF : L::K_OFF) + s * L::KV_BYTES;
        const int kbase = (tile0 + j) * TC_BN;
        const int pages = min(per_tile, (key_hi - kbase + ps - 1) / ps);
        // a tile whose pages have consecutive ids is one box (the run maps walk the pages with a stride
        // of their own): the TMA unit's time goes by the box, not by the byte
        const int first_pi = kbase / ps;
        bool run = p.page_runs && pages == per_tile && first_pi + per_tile <= p.max_pages && bt[first_pi] >= 0;
        for (int i = 1; run && i < per_tile; ++i) run = bt[first_pi + i] == bt[first_pi] + i;
        if (run) {
          mbar_expect_tx(full, (uint32_t)L::KV_BYTES);
          tma_load_5d(dst, which ? &run_v : &run_k, 0, 0, bt[first_pi], 0, kvh, full);
          return;
        }
        mbar_expect_tx(full, (uint32_t)(pages * HALVES * ps * 128));
        for (int i = 0; i < pages; ++i) {
          const int pi = first_pi + i;
          int page = pi < p.max_pages ? bt[pi] : 0;
          if (page < 0) page = 0;                   // no page lies inside a causal range without a window
          const int y = (page * p.nkv + kvh) * ps;
#pragma unroll
          for (int h = 0; h < HALVES; ++h)
            tma_load_2d(dst + h * (TC_BN * 128) + i * ps * 128, which ? &map_v : &map_k, h * 64, y, full);
        }
      };
      // two streams, served as their buffers come free (the keys first: the scores come first)
      int jk = 0, jv = 0;
      uint64_t idle_since = 0;
      uint32_t spins = 0;
      while ((jk < n_tiles || jv < n_tiles) && !*failed) {
        bool progress = false;
        if (jk < n_tiles && mbar_test(&k_empty[jk % TC_STAGES], ((jk / TC_STAGES) & 1) ^ 1)) {
          load_tile(0, jk);
          ++jk;
          progress = true;
        }
        if (jv < n_tiles && jv < jk && mbar_test(&v_empty[jv % TC_STAGES], ((jv / TC_STAGES) & 1) ^ 1)) {
          load_tile(1, jv);
          ++jv;
          progress = true;
        }
        if (progress) {
          idle_since = 0;
          spins = 0;
        } else if ((++spins & 255u) == 0) {
          const uint64_t now = global_ns();
          if (idle_since == 0) idle_since = now;
          else if (now - idle_since > TMA_WAIT_NS) {
            *failed = 21;
            atomicExch(p.status, 21);
          }
        }
      }
      if (*failed) {
        // let the copies already issued land before the CTA gives its shared memory back
        for (int i = jk > TC_STAGES ? jk - TC_STAGES : 0; i < jk; ++i)
          mbar_wait(&k_full[i % TC_STAGES], (i / TC_STAGES) & 1, TMA_DRAIN_NS);
        for (int i = jv > TC_STAGES ? jv - TC_STAGES : 0; i < jv; ++i)
          mbar_wait(&v_full[i % TC_STAGES], (i / TC_STAGES) & 1, TMA_DRAIN_NS);
      }
    }
  } else if (warp == ISSUER) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && !*failed) {
      // D float32, A and B bfloat16; scores: both K-major, N = 64; output: B (V) MN-major, N = HD
      const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
      const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
      bool ok = true;
      // scores of key tile j for row tile t (the stage is known to have landed)
      auto issue_scores = [&](int j, int t) {
        const int s = j % TC_STAGES, b = j & 1;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + L::K_OFF + s * L::KV_BYTES);
        const uint32_t q_addr = smem_u32(smem + t * L::Q_BYTES);
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + t * L::TMEM_TILE + b * TC_BN, umma_desc(q_addr + h * (TC_BM * 128) + k * 32),
                      umma_desc(k_addr + h * (TC_BN * 128) + k * 32), idesc_qk, (h | k) ? 1u : 0u);
        umma_commit(&s_full[t * 2 + b]);
      };
      // The row tiles are served as their events come, not in turn, so that one's products run under
      // the other's softmax.  Per row tile: jq = next key tile whose scores are to be issued (at most
      // two ahead of the softmax: S(j+2) goes into the columns P(j) V(j) has read), jp = next key tile
      // whose P.V is to be issued (when its P is written).
      int jq[RT], jp[RT], q_ready[RT];
#pragma unroll
      for (int t = 0; t < RT; ++t) jq[t] = jp[t] = q_ready[t] = 0;
      int k_released = 0, v_released = 0;
      uint64_t idle_since = 0;
      uint32_t spins = 0;
      while (ok) {
        bool pending = false, progress = false;
#pragma unroll
        for (int t = 0; t < RT; ++t) {
          if (jp[t] < n_of[t]) {
            pending = true;
            const int j = jp[t], s = j % TC_STAGES, b = j & 1;
            if (mbar_test(&p_full[t * 2 + b], (j >> 1) & 1) && mbar_test(&v_full[s], (j / TC_STAGES) & 1)) {
              tc_fence_after();
              const uint32_t v_addr = smem_u32(smem + L::V_OFF + s * L::KV_BYTES);
              const uint32_t p_tmem = tmem_base + t * L::TMEM_TILE + b * TC_BN;
#pragma unroll
              for (int k = 0; k < TC_BN / 16; ++k)     // 16 keys: 8 columns of P, 16 rows of V
                umma_bf16_ta(tmem_base + t * L::TMEM_TILE + L::O_COL, p_tmem + k * 8,
                             umma_desc_mn(v_addr + k * 16 * 128, TC_BN * 128), idesc_pv, (j | k) ? 1u : 0u);
              umma_commit(&s_free[t * 2 + b]);          // the product is complete: P's columns are free, O is still
              jp[t] = j + 1;
              progress = true;
            }
          }
          if (jq[t] < n_of[t] && jq[t] < jp[t] + 2) {
            const int j = jq[t];
            if (!q_ready[t]) q_ready[t] = mbar_test(&q_full[t], 0);
            // S(j) goes into the columns of P(j-2): the product that read them must be complete, not
            // only issued (products with different accumulators are not promised to run in order)
            const bool s_is_free = j < 2 || mbar_test(&s_free[t * 2 + (j & 1)], ((j >> 1) - 1) & 1);
            if (q_ready[t] && s_is_free && mbar_test(&k_full[j % TC_STAGES], (j / TC_STAGES) & 1)) {
              issue_scores(j, t);
              jq[t] = j + 1;
              progress = true;
            }
          }
        }
        // a K buffer goes back when every row tile that reaches its key tile has issued its scores, a V
        // buffer when every such row tile has issued its P.V (a commit covers all that was issued before it)
        while (k_released < n_tiles) {
          bool all = true;
#pragma unroll
          for (int t = 0; t < RT; ++t) all = all && (k_released >= n_of[t] || jq[t] > k_released);
          if (!all) break;
          umma_commit(&k_empty[k_released % TC_STAGES]);
          ++k_released;
        }
        while (v_released < n_tiles) {
          bool all = true;
#pragma unroll
          for (int t = 0; t < RT; ++t) all = all && (v_released >= n_of[t] || jp[t] > v_released);
          if (!all) break;
          umma_commit(&v_empty[v_released % TC_STAGES]);
          ++v_released;
        }
        if (!pending) break;
        if (*failed) ok = false;
        if (progress) {
          idle_since = 0;
          spins = 0;
        } else if ((++spins & 255u) == 0) {
          const uint64_t now = global_ns();
          if (idle_since == 0) idle_since = now;
          else if (now - idle_since > TMA_WAIT_NS) ok = false;
        }
      }
      if (!ok && !*failed) { *failed = 22; atomicExch(p.status, 22); }
    }
  } else {
    // ---------------- softmax: thread r owns row r (TMEM lane r) ----------------
    const int t = warp >> 2;                                           // row tile of this warp
    const int r = (warp & 3) * 32 + lane;
    const int row = row0 + t * TC_BM + r;
    const bool valid = row < rows_total;
    const int my_tiles = RT == 1 ? n_of[0] : (t == 0 ? n_of[0] : n_of[RT - 1]);
    const int hi = valid ? pos0 + row / G + 1 : 0;                     // keys [0, hi) are this row's
    const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + t * L::TMEM_TILE;
    uint64_t* my_s_full = s_full + t * 2;
    uint64_t* my_p_full = p_full + t * 2;
    {
      // the row tile's queries into the swizzled K-major layout [half][row][128 bytes]: all loads first
      constexpr int ROWS_PER_IT = TC_BM / CHUNKS;
      uint4 qv[CHUNKS];
#pragma unroll
      for (int it = 0; it < CHUNKS; ++it) {
        const int qr = it * ROWS_PER_IT + r / CHUNKS, qrow = row0 + t * TC_BM + qr;
        qv[it] = make_uint4(0, 0, 0, 0);
        if (qrow < rows_total)
          qv[it] = *reinterpret_cast<const uint4*>(p.q + ((size_t)(q0 + qrow / G) * p.nq + kvh * G + qrow % G) * HD + (r % CHUNKS) * 8);
      }
#pragma unroll
      for (int it = 0; it < CHUNKS; ++it) {
        const int qr = it * ROWS_PER_IT + r / CHUNKS, ch = r % CHUNKS;
        *reinterpret_cast<uint4*>(smem + t * L::Q_BYTES + (ch >> 3) * (TC_BM * 128) + qr * 128 + (((ch & 7) ^ (qr & 7)) << 4)) = qv[it];
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_full[t]);
    }
    float m_used = -INFINITY, l = 0.f;                                 // the maximum in scaled (log2) units
    bool ok = !*failed;
    for (int j = 0; j < my_tiles && ok; ++j) {
      const int b = j & 1;
      if (!mbar_wait(&my_s_full[b], (j >> 1) & 1) || *failed) { ok = false; break; }
      tc_fence_after();
      uint32_t s0[32], s1[32];
      tmem_ld32(t_lane + b * TC_BN, s0);
      tmem_ld32(t_lane + b * TC_BN + 32, s1);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const int kbase = (tile0 + j) * TC_BN;
      // the scale is positive, so the maximum of the scaled scores is the scaled maximum: the
      // scaling itself is folded into the exponent's multiply-add below
      float mx = -INFINITY;
      if (__all_sync(0xffffffffu, kbase + TC_BN <= hi)) {
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = max3(mx, __uint_as_float(s0[i]), __uint_as_float(s1[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (kbase + i >= hi) s0[i] = 0xff800000u;          // -inf
          if (kbase + 32 + i >= hi) s1[i] = 0xff800000u;
          mx = max3(mx, __uint_as_float(s0[i]), __uint_as_float(s1[i]));
        }
      }
      mx *= p.scale_log2;
      const bool grow = mx > m_used + TC_RESCALE_STEP;      // also the first tile with a key (m_used = -inf)
      // Only a rescale of O waits for the product of the tile before it (O must not change under it).
      // The barrier is the one behind that product, s_free of its buffer: its phases go by every
      // second tile, and S(j) being there means the product of tile j-2, hence of j-3, is complete,
      // so the phase asked for is the pending one or the one before: a parity tells them apart.
      const bool rescale = __any_sync(0xffffffffu, grow);
      if (rescale) {
        const float corr = grow ? ex2(m_used - mx) : 1.f;   // 0 when m_used = -inf (nothing summed yet)
        if (grow) {
          m_used = mx;
          l *= corr;
        }
        if (j > 0) {
          if (!mbar_wait(&s_free[t * 2 + ((j - 1) & 1)], ((j - 1) >> 1) & 1) || *failed) { ok = false; break; }
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < HD; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(t_lane + L::O_COL + c0, o);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
            tmem_st32(t_lane + L::O_COL + c0, o);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
      const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
      uint32_t pk[32];                                      // column i: keys 2i (low half) and 2i+1
      float2 sums = make_float2(0.f, 0.f);                  // of the even and of the odd keys
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float2 x01 = fma_x2(__uint_as_float(s0[2 * i]), __uint_as_float(s0[2 * i + 1]), p.scale_log2, neg_m);
        const float2 x23 = fma_x2(__uint_as_float(s1[2 * i]), __uint_as_float(s1[2 * i + 1]), p.scale_log2, neg_m);
        const float2 e01 = make_float2(ex2(x01.x), ex2(x01.y)), e23 = make_float2(ex2(x23.x), ex2(x23.y));
        sums = add_x2(sums, add_x2(e01, e23));
        pk[i] = pack2(e01.x, e01.y);
        pk[16 + i] = pack2(e23.x, e23.y);
      }
      l += sums.x + sums.y;
      tmem_st32(t_lane + b * TC_BN, pk);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&my_p_full[b]);
    }
    if (ok && my_tiles > 0) {
      // the last product: the barrier behind it (see the rescale above for why a parity suffices)
      if (!mbar_wait(&s_free[t * 2 + ((my_tiles - 1) & 1)], ((my_tiles - 1) >> 1) & 1) || *failed) ok = false;
    }
    if (!ok && !*failed) { *failed = 23; atomicExch(p.status, 23); }
    const size_t orow = valid ? (size_t)(q0 + row / G) * p.nq + kvh * G + row % G : 0;
    if (ok && valid && p.num_splits > 1)
      p.part_lse[(size_t)blockIdx.z * p.total_tokens * p.nq + orow] = (my_tiles > 0 && l > 0.f) ? m_used + log2f(l) : -INFINITY;
    if (ok && my_tiles > 0) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* po = nullptr;
      if (valid) po = p.out + orow * HD;
      float* pp = p.num_splits > 1 ? p.part_o + ((size_t)blockIdx.z * p.total_tokens * p.nq + orow) * HD : nullptr;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t o[32];
        tmem_ld32(t_lane + L::O_COL + c0, o);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (valid && pp) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(pp + c0 + i) = make_float4(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv,
                                                                  __uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
        } else if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            *reinterpret_cast<uint4*>(po + c0 + i) =
                make_uint4(pack2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv),
                           pack2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv),
                           pack2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv),
                           pack2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  pdl_launch_dependents();
  if (warp == ISSUER) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS));
  }
}

// The ranges' results of one (token, head) row merged: weights 2^(lse - max lse), ranges without a key skipped.
template <int HD>
__global__ void attention_tc_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                            __nv_bfloat16* __restrict__ out, int rows, int num_splits) {
  pdl_launch_dependents();       // a short kernel: the successor may be set up behind it
  pdl_wait();
  const int row = blockIdx.x;
  float mt = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mt = fmaxf(mt, part_lse[(size_t)s * rows + row]);
  if (mt == -INFINITY) return;   // no range wrote this row: it belongs to another kernel of the step (a decoded token's)
  float tot = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float l = part_lse[(size_t)s * rows + row];
    tot += l == -INFINITY ? 0.f : exp2f(l - mt);
  }
  const float inv = tot > 0.f ? 1.f / tot : 0.f;
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float l = part_lse[(size_t)s * rows + row];
      if (l != -INFINITY) acc += part_o[((size_t)s * rows + row) * HD + d] * exp2f(l - mt);
    }
    out[(size_t)row * HD + d] = __float2bfloat16_rn(acc * inv);
  }
}

// ---- host side --------------------------------------------------------------------------------

// tensor maps of the caches seen so far: (base, rows, page size, head size) -> map
struct TcMapKey {
  const void* base; long long rows; int ps, hd, nkv_run;      // nkv_run: 0 for the per-page map, else the kv heads of the run map
  bool operator==(const TcMapKey& o) const {
    return base == o.base && rows == o.rows && ps == o.ps && hd == o.hd && nkv_run == o.nkv_run;
  }
};
struct TcMapKeyHash {
  size_t operator()(const TcMapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (std::hash<long long>()(k.rows) * 31) ^ (size_t)(k.ps * 131 + k.hd + k.nkv_run * 7919);
  }
};
static std::unordered_map<TcMapKey, CUtensorMap, TcMapKeyHash> g_tc_maps;
static std::mutex g_tc_maps_mutex;

static bool tc_cache_map(const void* base, long long rows, int ps, int hd, CUtensorMap* out, int nkv_run = 0) {
  std::lock_guard<std::mutex> lock(g_tc_maps_mutex);
  TcMapKey key{base, rows, ps, hd, nkv_run};
  auto it = g_tc_maps.find(key);
  if (it != g_tc_maps.end()) {
    *out = it->second;
    return true;
  }
  if (rows > 0x7fffffffLL) return false;
  if (nkv_run == 0) {
    if (!make_map(out, base, (int)rows, hd, ps)) return false;
  } else {
    if (!make_map_page_run(out, base, rows / ((long long)nkv_run * ps), nkv_run, ps, hd, TC_BN / ps, false)) return false;
  }
  if (g_tc_maps.size() > 4096) g_tc_maps.clear();
  g_tc_maps.emplace(key, *out);
  return true;
}

template <int HD, int RT>
static int launch_tc(const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& rk, const CUtensorMap& rv,
                     const AttnTcParams& p, int tiles, cudaStream_t stream) {
  constexpr int smem = TcLayout<HD, RT>::SMEM;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_tc_kernel<HD, RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
      set_error("attention_tc: cannot raise the shared memory limit");
      return SLLM_ERR_LAUNCH;
    }
    configured = true;
  }
  dim3 grid((unsigned)tiles * p.nkv, 1, p.num_splits);
  launch_kernel(attention_tc_kernel<HD, RT>, grid, TcLayout<HD, RT>::THREADS, (size_t)smem, stream, mk, mv, rk, rv, p);
  int rc = launch_status("attention_tc");
  if (rc != SLLM_OK || p.num_splits == 1) return rc;
  launch_kernel(attention_tc_combine_kernel<HD>, p.total_tokens * p.nq, HD >= 128 ? 128 : 64, 0, stream,
                (const float*)p.part_o, (const float*)p.part_lse, p.out, p.total_tokens * p.nq, p.num_splits);
  return launch_status("attention_tc_combine");
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_attention_tc_supports(int hd, int page_size) {
  // a page's box must start on a 1024-byte boundary of the swizzled tile: page sizes 8, 16, 32, 64
  return (hd == 64 || hd == 128) && page_size >= 8 && page_size <= 64 && 64 % page_size == 0 && encode_fn() != nullptr;
}

// The prefill form: tiles of up to 128 * row_tiles (token, head-in-group) rows (row_tiles 1 or 2; tile_row0
// in steps of that many rows), no window.  num_splits > 1 cuts the context into that many ranges of
// tiles_per_split 64-key tiles (num_splits * tiles_per_split must cover the longest context), each range a
// CTA of its own; part_o [num_splits, total_tokens, nq, hd] and part_lse [num_splits, total_tokens, nq]
// float32 are the scratch the ranges' results pass through; part_lse must be -inf everywhere before the
// launch: the merge writes the rows some range has written and leaves the others as they are.
// num_pages: pages in the cache tensors [num_pages, nkv, page_size, hd].  status: one int of device
// memory, zero before the launch; non-zero afterwards means a wait ran out and `out` is not valid.
SLLM_EXPORT int sllm_attention_tc(const void* q, const void* k_cache, const void* v_cache, long long num_pages, void* out,
                                  const int* block_tables, int max_pages, const int* q_start, const int* ctx_len,
                                  const int* tile_seq, const int* tile_row0, int tiles, int row_tiles, int nq, int nkv,
                                  int hd, int page_size, float scale, int num_splits, int tiles_per_split, int total_tokens,
                                  float* part_o, float* part_lse, int* status, cudaStream_t stream) {
  SLLM_REQUIRE(row_tiles == 1 || row_tiles == 2, "attention_tc: row_tiles=%d must be 1 or 2", row_tiles);
  SLLM_REQUIRE(num_splits >= 1 && num_splits <= 65535 && tiles_per_split >= 1, "attention_tc: bad context split %d x %d",
               num_splits, tiles_per_split);
  SLLM_REQUIRE(num_splits == 1 || (part_o && part_lse && total_tokens > 0), "attention_tc: a context split needs scratch");
  SLLM_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_tc: bad head counts nq=%d nkv=%d", nq, nkv);
  SLLM_REQUIRE(sllm_attention_tc_supports(hd, page_size), "attention_tc: head_dim=%d page_size=%d not taken", hd, page_size);
  SLLM_REQUIRE(max_pages > 0 && tiles >= 0 && num_pages > 0 && nkv <= 65535, "attention_tc: bad sizes");
  SLLM_REQUIRE(status != nullptr, "attention_tc: a status word is required");
  SLLM_REQUIRE(scale > 0.f, "attention_tc: the score scale must be positive (the row maximum is taken before scaling)");
  SLLM_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 && ((uintptr_t)q & 15) == 0 &&
                   ((uintptr_t)out & 15) == 0, "attention_tc: operands must be 16-byte aligned");
  if (tiles == 0) return SLLM_OK;
  CUtensorMap mk, mv;
  const long long rows = num_pages * nkv * page_size;
  if (!tc_cache_map(k_cache, rows, page_size, hd, &mk) || !tc_cache_map(v_cache, rows, page_size, hd, &mv)) {
    set_error("attention_tc: cuTensorMapEncodeTiled failed");
    return SLLM_ERR_LAUNCH;
  }
  CUtensorMap rk = mk, rv = mv;
  const bool runs = page_size < TC_BN && tc_cache_map(k_cache, rows, page_size, hd, &rk, nkv) &&
                    tc_cache_map(v_cache, rows, page_size, hd, &rv, nkv);
  AttnTcParams p;
  p.page_runs = runs ? 1 : 0;
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.block_tables = block_tables; p.q_start = q_start;
  p.ctx_len = ctx_len; p.tile_seq = tile_seq; p.tile_row0 = tile_row0; p.status = status; p.max_pages = max_pages;
  p.page_size = page_size; p.nq = nq; p.nkv = nkv; p.scale_log2 = scale * 1.4426950408889634f;
  p.num_splits = num_splits; p.tiles_per_split = num_splits == 1 ? (1 << 30) / TC_BN : tiles_per_split;
  p.total_tokens = total_tokens; p.part_o = part_o; p.part_lse = part_lse;
  if (row_tiles == 2)
    return hd == 128 ? launch_tc<128, 2>(mk, mv, rk, rv, p, tiles, stream) : launch_tc<64, 2>(mk, mv, rk, rv, p, tiles, stream);
  return hd == 128 ? launch_tc<128, 1>(mk, mv, rk, rv, p, tiles, stream) : launch_tc<64, 1>(mk, mv, rk, rv, p, tiles, stream);
}
