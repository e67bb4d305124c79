// Attention of prompt portions over the paged cache on the 5th-generation tensor cores
// (tcgen05, accumulators in tensor memory): causal GQA with an online softmax, bfloat16 in,
// float32 scores, softmax and output accumulation.
//
// A CTA takes one 128-row tile of (token, head-in-group) rows of one request and one kv head,
// as the mma.sync prefill form does, and walks the keys in tiles of 64.  Two CTAs share an SM
// (112 KB of shared memory and 256 columns of tensor memory each), so that one CTA's softmax
// runs while the other's products do.  Six warps, three jobs:
//   warps 0-3  softmax: thread r owns row r.  It reads its row of S = Q K^T from tensor memory
//              (tcgen05.ld), scales and masks it, keeps the row's running maximum and sum, writes
//              P = exp2(S - max) as bfloat16 into shared memory in the swizzled layout the tensor
//              core reads, and at the end reads O, divides by the sum and stores the row.
//              The maximum in use only moves when a tile's maximum exceeds it by more than 2^8
//              (then O in tensor memory is rescaled: tcgen05.ld, multiply, tcgen05.st); the result
//              is the same sum with a different common factor, which cancels in O / sum.
//   warp 4     one lane issues the TMA loads: per page and 64-column half of the head one box of
//              K and one of V (page_size x 64 elements, 128-byte swizzle), two tiles deep;
//   warp 5     allocates the tensor memory; one lane issues S(j+1) = Q K(j+1)^T (M=128, N=64, K=16,
//              head_dim/16 times) before it waits for P(j), so the score product of the next tile
//              runs under the softmax of this one; then O += P(j) V(j) (M=128, N=head_dim, K=16, four
//              times; V is read as stored, keys down the rows: an MN-major operand).
// S is double-buffered in tensor memory (2 x 64 columns), O takes head_dim columns.
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
  float scale_log2;              // scale * log2(e)
};

constexpr int TC_BM = 128, TC_BN = 64, TC_STAGES = 2, TC_THREADS = 192;
constexpr float TC_RESCALE_STEP = 8.0f;     // log2 units the maximum may lag behind before O is rescaled

template <int HD> struct TcLayout {
  static constexpr int HALVES = HD / 64;
  static constexpr int Q_BYTES = HALVES * TC_BM * 128;
  static constexpr int KV_BYTES = HALVES * TC_BN * 128;      // one of K or V, one stage
  static constexpr int P_BYTES = TC_BM * 128;
  static constexpr int K_OFF = Q_BYTES;
  static constexpr int V_OFF = K_OFF + TC_STAGES * KV_BYTES;
  static constexpr int P_OFF = V_OFF + TC_STAGES * KV_BYTES;
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  static constexpr int SMEM = BAR_OFF + 128;
  static constexpr int TMEM_COLS = 256;                      // 2 x 64 (S) + HD (O), a power of two
  static constexpr int O_COL = 2 * TC_BN;
};

template <int HD>
__global__ void __launch_bounds__(TC_THREADS, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const AttnTcParams p) {
  using L = TcLayout<HD>;
  constexpr int HALVES = L::HALVES;
  constexpr int CHUNKS = HD / 8;
  extern __shared__ __align__(1024) unsigned char tc_smem[];
  unsigned char* smem = tc_smem;
  uint64_t* full_kv = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);   // [2] a stage's K and V have landed
  uint64_t* empty_kv = full_kv + 2;                                     // [2] P.V of the stage's tile is done
  uint64_t* s_full = empty_kv + 2;                                      // [2] S buffer holds Q K^T
  uint64_t* s_empty = s_full + 2;                                       // [2] the softmax warps have read it
  uint64_t* p_full = s_empty + 2;                                       // P is written, O is rescaled
  uint64_t* o_done = p_full + 1;                                        // P.V done: P may be rewritten, O read
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&full_kv[s], 1);
      mbar_init(&empty_kv[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 4);                  // the four softmax warps
    }
    mbar_init(p_full, 4);
    mbar_init(o_done, 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(L::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  // the stages start as zeros (see the header)
  for (int o = tid * 16; o < 2 * TC_STAGES * L::KV_BYTES; o += TC_THREADS * 16)
    *reinterpret_cast<uint4*>(smem + L::K_OFF + o) = make_uint4(0, 0, 0, 0);

  pdl_wait();       // everything below reads what the step's earlier kernels or its batch upload wrote
  const int seq = p.tile_seq[blockIdx.x], row0 = p.tile_row0[blockIdx.x];
  const int kvh = blockIdx.y;
  const int G = p.nq / p.nkv;
  const int q0 = p.q_start[seq], q_len = p.q_start[seq + 1] - q0, ctx = p.ctx_len[seq];
  const int rows_total = q_len * G;
  const int pos0 = ctx - q_len;                  // position of the request's first token of this step
  const int row_hi = min(row0 + TC_BM, rows_total);
  const int key_hi = row_hi > row0 ? pos0 + (row_hi - 1) / G + 1 : 0;   // exclusive
  const int n_tiles = (key_hi + TC_BN - 1) / TC_BN;
  const int* bt = p.block_tables + (size_t)seq * p.max_pages;

  // Q: rows of the tile into the swizzled K-major layout [half][row][128 bytes]
  for (int c = tid; c < TC_BM * CHUNKS; c += TC_THREADS) {
    const int r = c / CHUNKS, ch = c % CHUNKS;
    const int row = row0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < rows_total) {
      const int tok = row / G, hg = row % G;
      v = *reinterpret_cast<const uint4*>(p.q + ((size_t)(q0 + tok) * p.nq + kvh * G + hg) * HD + ch * 8);
    }
    *reinterpret_cast<uint4*>(smem + (ch >> 3) * (TC_BM * 128) + r * 128 + (((ch & 7) ^ (r & 7)) << 4)) = v;
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if ((smem_u32(smem) & 1023u) != 0 && tid == 0) {      // the swizzled layouts need a 1024-byte base
    *failed = 20;
    atomicExch(p.status, 20);
  }
  __syncthreads();

  if (warp == 4) {
    // ---------------- TMA producer ----------------
    if (lane == 0 && !*failed) {
      const int ps = p.page_size, per_tile = TC_BN / ps;
      int issued = 0;
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % TC_STAGES, round = j / TC_STAGES;
        if (!mbar_wait(&empty_kv[s], (round & 1) ^ 1) || *failed) {
          if (!*failed) { *failed = 21; atomicExch(p.status, 21); }
          break;
        }
        const int kbase = j * TC_BN;
        const int pages = min(per_tile, (key_hi - kbase + ps - 1) / ps);
        mbar_expect_tx(&full_kv[s], (uint32_t)(pages * 2 * HALVES * ps * 128));
        unsigned char* ks = smem + L::K_OFF + s * L::KV_BYTES;
        unsigned char* vs = smem + L::V_OFF + s * L::KV_BYTES;
        for (int i = 0; i < pages; ++i) {
          const int pi = kbase / ps + i;
          int page = pi < p.max_pages ? bt[pi] : 0;
          if (page < 0) page = 0;                   // no page lies inside a causal range without a window
          const int y = (page * p.nkv + kvh) * ps;
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            tma_load_2d(ks + h * (TC_BN * 128) + i * ps * 128, &map_k, h * 64, y, &full_kv[s]);
            tma_load_2d(vs + h * (TC_BN * 128) + i * ps * 128, &map_v, h * 64, y, &full_kv[s]);
          }
        }
        issued = j + 1;
      }
      if (*failed) {
        // let the copies already issued land before the CTA gives its shared memory back
        for (int i = issued > TC_STAGES ? issued - TC_STAGES : 0; i < issued; ++i)
          mbar_wait(&full_kv[i % TC_STAGES], (i / TC_STAGES) & 1, 1u << 16);
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && !*failed) {
      // D float32, A and B bfloat16; scores: both K-major, N = 64; output: B (V) MN-major, N = HD
      const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
      const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
      const uint32_t q_addr = smem_u32(smem), p_addr = smem_u32(smem + L::P_OFF);
      bool ok = true;
      auto issue_scores = [&](int j) {
        const int s = j % TC_STAGES, b = j & 1;
        if (!mbar_wait(&full_kv[s], (j / TC_STAGES) & 1) || !mbar_wait(&s_empty[b], ((j >> 1) & 1) ^ 1) || *failed) {
          ok = false;
          return;
        }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + L::K_OFF + s * L::KV_BYTES);
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + b * TC_BN, umma_desc(q_addr + h * (TC_BM * 128) + k * 32),
                      umma_desc(k_addr + h * (TC_BN * 128) + k * 32), idesc_qk, (h | k) ? 1u : 0u);
        umma_commit(&s_full[b]);
      };
      if (n_tiles > 0) issue_scores(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) issue_scores(j + 1);
        if (!ok) break;
        if (!mbar_wait(p_full, j & 1) || *failed) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int s = j % TC_STAGES;
        const uint32_t v_addr = smem_u32(smem + L::V_OFF + s * L::KV_BYTES);
#pragma unroll
        for (int k = 0; k < TC_BN / 16; ++k)         // 16 keys: 32 bytes along P's rows, 16 rows of V
          umma_bf16(tmem_base + L::O_COL, umma_desc(p_addr + k * 32), umma_desc_mn(v_addr + k * 16 * 128, TC_BN * 128),
                    idesc_pv, (j | k) ? 1u : 0u);
        umma_commit(&empty_kv[s]);
        umma_commit(o_done);
      }
      if (!ok && !*failed) { *failed = 22; atomicExch(p.status, 22); }
    }
  } else {
    // ---------------- softmax: thread r owns row r (TMEM lane r) ----------------
    const int r = warp * 32 + lane;
    const int row = row0 + r;
    const bool valid = row < rows_total;
    const int hi = valid ? min(pos0 + row / G + 1, key_hi) : 0;       // keys [0, hi) are this row's
    const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);
    unsigned char* p_row = smem + L::P_OFF + r * 128;
    float m_used = -INFINITY, l = 0.f;
    bool ok = !*failed;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int b = j & 1;
      if (!mbar_wait(&s_full[b], (j >> 1) & 1) || *failed) { ok = false; break; }
      tc_fence_after();
      uint32_t s0[32], s1[32];
      tmem_ld32(t_lane + b * TC_BN, s0);
      tmem_ld32(t_lane + b * TC_BN + 32, s1);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[b]);
      const int kbase = j * TC_BN;
      float mx = -INFINITY;
      if (__all_sync(0xffffffffu, kbase + TC_BN <= hi)) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float a = __uint_as_float(s0[i]) * p.scale_log2, c = __uint_as_float(s1[i]) * p.scale_log2;
          s0[i] = __float_as_uint(a);
          s1[i] = __float_as_uint(c);
          mx = fmaxf(mx, fmaxf(a, c));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float a = kbase + i < hi ? __uint_as_float(s0[i]) * p.scale_log2 : -INFINITY;
          const float c = kbase + 32 + i < hi ? __uint_as_float(s1[i]) * p.scale_log2 : -INFINITY;
          s0[i] = __float_as_uint(a);
          s1[i] = __float_as_uint(c);
          mx = fmaxf(mx, fmaxf(a, c));
        }
      }
      const bool grow = mx > m_used + TC_RESCALE_STEP;      // also the first tile with a key (m_used = -inf)
      // P.V of the tile before must be done: it reads P, and O must not change under a rescale
      if (j > 0) {
        if (!mbar_wait(o_done, (j - 1) & 1) || *failed) { ok = false; break; }
        tc_fence_after();
      }
      if (__any_sync(0xffffffffu, grow)) {
        const float corr = grow ? exp2f(m_used - mx) : 1.f; // 0 when m_used = -inf (nothing summed yet)
        if (grow) {
          m_used = mx;
          l *= corr;
        }
        if (j > 0) {
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
      const float m_eff = m_used == -INFINITY ? 0.f : m_used;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int idx = c8 * 8 + i;
          e[i] = exp2f(__uint_as_float(idx < 32 ? s0[idx] : s1[idx - 32]) - m_eff);
          l += e[i];
        }
        *reinterpret_cast<uint4*>(p_row + ((c8 ^ (r & 7)) << 4)) =
            make_uint4(pack2(e[0], e[1]), pack2(e[2], e[3]), pack2(e[4], e[5]), pack2(e[6], e[7]));
      }
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && n_tiles > 0) {
      if (!mbar_wait(o_done, (n_tiles - 1) & 1) || *failed) ok = false;
    }
    if (!ok && !*failed) { *failed = 23; atomicExch(p.status, 23); }
    if (ok && n_tiles > 0) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* po = nullptr;
      if (valid) po = p.out + ((size_t)(q0 + row / G) * p.nq + kvh * G + row % G) * HD;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t o[32];
        tmem_ld32(t_lane + L::O_COL + c0, o);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (valid) {
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
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS));
  }
}

// ---- host side --------------------------------------------------------------------------------

// tensor maps of the caches seen so far: (base, rows, page size, head size) -> map
struct TcMapKey {
  const void* base; long long rows; int ps, hd;
  bool operator==(const TcMapKey& o) const { return base == o.base && rows == o.rows && ps == o.ps && hd == o.hd; }
};
struct TcMapKeyHash {
  size_t operator()(const TcMapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (std::hash<long long>()(k.rows) * 31) ^ (size_t)(k.ps * 131 + k.hd);
  }
};
static std::unordered_map<TcMapKey, CUtensorMap, TcMapKeyHash> g_tc_maps;
static std::mutex g_tc_maps_mutex;

static bool tc_cache_map(const void* base, long long rows, int ps, int hd, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_tc_maps_mutex);
  TcMapKey key{base, rows, ps, hd};
  auto it = g_tc_maps.find(key);
  if (it != g_tc_maps.end()) {
    *out = it->second;
    return true;
  }
  if (rows > 0x7fffffffLL) return false;
  if (!make_map(out, base, (int)rows, hd, ps)) return false;
  if (g_tc_maps.size() > 4096) g_tc_maps.clear();
  g_tc_maps.emplace(key, *out);
  return true;
}

template <int HD>
static int launch_tc(const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcParams& p, int tiles, cudaStream_t stream) {
  constexpr int smem = TcLayout<HD>::SMEM;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
      set_error("attention_tc: cannot raise the shared memory limit");
      return SLLM_ERR_LAUNCH;
    }
    configured = true;
  }
  dim3 grid(tiles, p.nkv);
  launch_kernel(attention_tc_kernel<HD>, grid, TC_THREADS, (size_t)smem, stream, mk, mv, p);
  return launch_status("attention_tc");
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_attention_tc_supports(int hd, int page_size) {
  // a page's box must start on a 1024-byte boundary of the swizzled tile: page sizes 8, 16, 32, 64
  return (hd == 64 || hd == 128) && page_size >= 8 && page_size <= 64 && 64 % page_size == 0 && encode_fn() != nullptr;
}

// The prefill form: tiles of up to 128 (token, head-in-group) rows, no window, no context split.
// num_pages: pages in the cache tensors [num_pages, nkv, page_size, hd].  status: one int of device
// memory, zero before the launch; non-zero afterwards means a wait ran out and `out` is not valid.
SLLM_EXPORT int sllm_attention_tc(const void* q, const void* k_cache, const void* v_cache, long long num_pages, void* out,
                                  const int* block_tables, int max_pages, const int* q_start, const int* ctx_len,
                                  const int* tile_seq, const int* tile_row0, int tiles, int nq, int nkv, int hd,
                                  int page_size, float scale, int* status, cudaStream_t stream) {
  SLLM_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_tc: bad head counts nq=%d nkv=%d", nq, nkv);
  SLLM_REQUIRE(sllm_attention_tc_supports(hd, page_size), "attention_tc: head_dim=%d page_size=%d not taken", hd, page_size);
  SLLM_REQUIRE(max_pages > 0 && tiles >= 0 && num_pages > 0 && nkv <= 65535, "attention_tc: bad sizes");
  SLLM_REQUIRE(status != nullptr, "attention_tc: a status word is required");
  SLLM_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 && ((uintptr_t)q & 15) == 0 &&
                   ((uintptr_t)out & 15) == 0, "attention_tc: operands must be 16-byte aligned");
  if (tiles == 0) return SLLM_OK;
  CUtensorMap mk, mv;
  const long long rows = num_pages * nkv * page_size;
  if (!tc_cache_map(k_cache, rows, page_size, hd, &mk) || !tc_cache_map(v_cache, rows, page_size, hd, &mv)) {
    set_error("attention_tc: cuTensorMapEncodeTiled failed");
    return SLLM_ERR_LAUNCH;
  }
  AttnTcParams p;
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.block_tables = block_tables; p.q_start = q_start;
  p.ctx_len = ctx_len; p.tile_seq = tile_seq; p.tile_row0 = tile_row0; p.status = status; p.max_pages = max_pages;
  p.page_size = page_size; p.nq = nq; p.nkv = nkv; p.scale_log2 = scale * 1.4426950408889634f;
  return hd == 128 ? launch_tc<128>(mk, mv, p, tiles, stream) : launch_tc<64>(mk, mv, p, tiles, stream);
}
