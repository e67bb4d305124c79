// Decode-form attention fed by the tensor memory accelerator.
//
// Same arithmetic and the same split-KV scheme as the decode form of attention_mma.cu (16 rows per
// CTA: a request's one or two tokens times its group of query heads; four warps take 16-key slices
// of each 64-key tile; partial results per context split, a combine kernel afterwards).  What
// differs is how keys and values reach shared memory.  There, every thread computes addresses and
// issues sixteen 16-byte cp.async per tile, and the kernel is bound by those instructions.  Here a
// fifth warp's one lane issues one TMA box copy per page (cp.async.bulk.tensor.3d over the cache
// seen as [pages * kv heads * page size rows][head size / 64][64], all rows and halves of a page in
// one box, 128-byte swizzle; the TMA unit spends a fixed time per copy, so few large boxes); the copies signal an mbarrier per stage, the compute warps read the
// swizzled tile with ldmatrix and hand the stage back through a second mbarrier.  No thread of the
// compute warps touches an address of the cache.
//
// A whole page is always copied, also where it reaches past the context (its rows are masked by
// position); slots of a tile that have no page (past the last page, or a page a window gave back)
// are zero-filled on the stage's first use so that a masked probability of zero never meets an
// uninitialised value.  Every mbarrier wait is bounded; a wait that runs out records a code in the
// status word and the CTA leaves through the common exit.
//
// Takes head sizes 64 and 128 and page sizes that divide 64; the host falls back to
// attention_mma.cu otherwise.
#include <math.h>
#include <stdio.h>

#include <mutex>
#include <unordered_map>

#include "mma.cuh"
#include "tma.cuh"

namespace sllm {

constexpr int TA_BN = 64;          // keys per tile
constexpr int TA_STAGES = 3;
constexpr int TA_THREADS = 160;    // four compute warps and the producer warp
constexpr int TA_BT_CACHE = 2048;  // block-table entries the producer keeps in shared memory

struct AttnTmaParams {
  const __nv_bfloat16* q;        // [T, nq, HD]
  __nv_bfloat16* out;            // [T, nq, HD]   (num_splits == 1)
  float* part_o;                 // [splits, T, nq, HD]
  float* part_lse;               // [splits, T, nq]
  const int* block_tables;       // [S, max_pages]
  const int* q_start;            // [S+1]
  const int* ctx_len;            // [S]
  const int* tile_seq;           // [tiles]
  const int* tile_row0;          // [tiles]
  int* status;
  int max_pages, page_size, nq, nkv, window, num_splits, total_tokens;
  int page_runs;                 // the run maps are valid: a tile of pages with consecutive ids is fetched as one box
  float scale_log2;
};

// Byte offset of the 16-byte chunk `chunk` (of the head's HD/8) of key row `row` within a stage's K or V.
// A page arrives as one box of whole rows; a row is HD/64 consecutive 128-byte units, and the TMA unit
// swizzles the eight chunks of a unit by the unit's index.
template <int HD>
__device__ __forceinline__ int swz(int row, int chunk) {
  const int unit = row * (HD / 64) + (chunk >> 3);
  return unit * 128 + (((chunk & 7) ^ (unit & 7)) << 4);
}

template <int HD>
__global__ void __launch_bounds__(TA_THREADS)
attention_tma_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const __grid_constant__ CUtensorMap run_k, const __grid_constant__ CUtensorMap run_v,
                            const AttnTmaParams p) {
  constexpr int STRIDE = HD + 8;
  constexpr int KSTEPS = HD / 16;
  constexpr int DT = HD / 8;
  constexpr int HALVES = HD / 64;
  constexpr int KV_BYTES = TA_BN * HD * 2;               // one of K or V of a stage
  extern __shared__ unsigned char ta_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(ta_smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* kv_s = smem;                                                    // [STAGES][K | V]
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem + TA_STAGES * 2 * KV_BYTES);   // [16][STRIDE]
  uint64_t* full = reinterpret_cast<uint64_t*>(q_s + 16 * STRIDE);
  uint64_t* empty = full + TA_STAGES;
  volatile int* failed = reinterpret_cast<volatile int*>(empty + TA_STAGES);
  int* bt_s = const_cast<int*>(reinterpret_cast<volatile int*>(failed + 2));      // [TA_BT_CACHE]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  if (tid == 0) {
    for (int s = 0; s < TA_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 4);                          // the four compute warps
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // The batch description (tiles, lengths, block tables) was copied to the device before the step's
  // first kernel started, so it is read before the wait for the step's earlier kernels: the chain of
  // dependent loads (tile -> request -> lengths -> pages) runs under their tails.  The queries and the
  // new keys and values come from those kernels: each role waits before it touches them.

  // the KV head is the grid's fastest index: tiles come longest first and CTAs start in grid order,
  // so every head's long tiles start in the first wave
  const int tile_i = blockIdx.x / p.nkv, kvh = blockIdx.x % p.nkv, split = blockIdx.z;
  const int seq = p.tile_seq[tile_i], row0 = p.tile_row0[tile_i];
  const int G = p.nq / p.nkv;
  const int q0 = p.q_start[seq], q_len = p.q_start[seq + 1] - q0, ctx = p.ctx_len[seq];
  const int rows_total = q_len * G;
  const int pos0 = ctx - q_len;
  const int row_hi = min(row0 + 16, rows_total);
  const int* bt = p.block_tables + (size_t)seq * p.max_pages;
  const int ps = p.page_size;
  const int pages_per_tile = TA_BN / ps;
  const int pages_in_ctx = (ctx + ps - 1) / ps;

  int key_hi = pos0 + (row_hi - 1) / G + 1;
  int key_lo = 0;
  if (p.window > 0) key_lo = max(0, pos0 + row0 / G - p.window + 1);
  if (p.num_splits > 1) {
    const int chunk = ((ctx + p.num_splits - 1) / p.num_splits + TA_BN - 1) / TA_BN * TA_BN;
    key_lo = max(key_lo, split * chunk);
    key_hi = min(key_hi, (split + 1) * chunk);
  }
  const int tile0 = key_lo / TA_BN * TA_BN;
  const int n_tiles = key_hi > tile0 ? (key_hi - tile0 + TA_BN - 1) / TA_BN : 0;

  if (warp == 4) {
    // ---------------- producer ----------------
    // The pages of this CTA's key range, fetched once by the whole warp: a tile's copies then wait
    // for nothing but a free stage (one lane reading the table from global memory page by page
    // took longer per tile than the copies themselves).
    const int page_first = tile0 / ps;
    const int page_count = n_tiles > 0 ? min(pages_in_ctx, (tile0 + n_tiles * TA_BN + ps - 1) / ps) - page_first : 0;
    const bool bt_cached = page_count <= TA_BT_CACHE;
    if (bt_cached) {
      for (int i = lane; i < page_count; i += 32) bt_s[i] = bt[page_first + i];
      __syncwarp();
    }
    auto page_of = [&](int pi) { return bt_cached ? bt_s[pi - page_first] : bt[pi]; };
    pdl_wait();
    for (int tile = 0; tile < n_tiles; ++tile) {
      const int s = tile % TA_STAGES, round = tile / TA_STAGES;
      bool ok = true;
      if (lane == 0) ok = mbar_wait(&empty[s], (round & 1) ^ 1) && !*failed;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) {
        if (lane == 0 && !*failed) { *failed = 1; atomicExch(p.status, 11); }
        break;
      }
      unsigned char* ks = kv_s + s * 2 * KV_BYTES;
      unsigned char* vs = ks + KV_BYTES;
      const int page0 = (tile0 + tile * TA_BN) / ps;
      // which slots of the tile have a page to copy (the same answer in every lane)
      unsigned valid = 0;
      for (int i = 0; i < pages_per_tile; ++i) {
        const int pi = page0 + i;
        if (pi < pages_in_ctx && page_of(pi) >= 0) valid |= 1u << i;     // at most 8 pages a tile (page size >= 8)
      }
      if (round == 0 && valid != (1u << pages_per_tile) - 1) {
        // first use of this stage: slots without a page must not hold garbage
        for (int i = 0; i < pages_per_tile; ++i) {
          if (valid & (1u << i)) continue;
          for (int o = lane * 16; o < ps * HALVES * 128; o += 32 * 16) {
            *reinterpret_cast<uint4*>(ks + i * ps * HALVES * 128 + o) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(vs + i * ps * HALVES * 128 + o) = make_uint4(0, 0, 0, 0);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
      }
      // a tile whose pages have consecutive ids is one box of K and one of V (the page dimension of
      // the run maps has its own stride); the TMA unit's time goes by the box, not by the byte
      bool run = p.page_runs && valid == (1u << pages_per_tile) - 1;
      for (int i = 1; run && i < pages_per_tile; ++i) run = page_of(page0 + i) == page_of(page0) + i;
      if (lane == 0 && run) {
        mbar_expect_tx(&full[s], (uint32_t)(2 * KV_BYTES));
        tma_load_5d(ks, &run_k, 0, 0, 0, kvh, page_of(page0), &full[s]);
        tma_load_5d(vs, &run_v, 0, 0, 0, kvh, page_of(page0), &full[s]);
      } else if (lane == 0) {
        const uint32_t bytes = (uint32_t)__popc(valid) * ps * HD * 2 * 2;
        if (bytes == 0) {
          mbar_arrive(&full[s]);
        } else {
          mbar_expect_tx(&full[s], bytes);
          for (int i = 0; i < pages_per_tile; ++i) {
            if (!(valid & (1u << i))) continue;
            const int y = (page_of(page0 + i) * p.nkv + kvh) * ps;
            tma_load_3d(ks + i * ps * HALVES * 128, &map_k, 0, 0, y, &full[s]);
            tma_load_3d(vs + i * ps * HALVES * 128, &map_v, 0, 0, y, &full[s]);
          }
        }
      }
    }
  } else {
    // ---------------- compute warps ----------------
    // queries: 16 rows of (token, head-in-group)
    constexpr int CHUNKS = HD / 8;
    pdl_wait();
    for (int c = tid; c < 16 * CHUNKS; c += 128) {
      const int r = c / CHUNKS, ch = c % CHUNKS;
      const int row = row0 + r;
      const bool okr = row < rows_total;
      const int tok = okr ? row / G : 0, hg = okr ? row % G : 0;
      cp_async_16(q_s + r * STRIDE + ch * 8, p.q + ((size_t)(q0 + tok) * p.nq + kvh * G + hg) * HD + ch * 8, okr);
    }
    cp_async_commit();
    cp_async_wait<0>();
    asm volatile("bar.sync 1, 128;" ::: "memory");          // the four compute warps only
    unsigned qf[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
      ldmatrix_x4(qf[ks], q_s + (lane & 15) * STRIDE + ks * 16 + (lane >> 4) * 8);

    int hi_r[2], lo_r[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = row0 + g + 8 * i;
      if (row < rows_total) {
        const int pos = pos0 + row / G;
        hi_r[i] = min(pos + 1, key_hi);
        lo_r[i] = p.window > 0 ? max(key_lo, pos - p.window + 1) : key_lo;
      } else {
        hi_r[i] = 0;
        lo_r[i] = 1;
      }
    }
    float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[d][c] = 0.f;

    const int koff = warp * 16;
    bool alive = true;
    for (int tile = 0; tile < n_tiles && alive; ++tile) {
      const int s = tile % TA_STAGES, round = tile / TA_STAGES;
      bool ok = true;
      if (lane == 0) ok = mbar_wait(&full[s], round & 1) && !*failed;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) {
        if (lane == 0 && !*failed) { *failed = 2; atomicExch(p.status, 12); }
        alive = false;
        break;
      }
      const unsigned char* kb = kv_s + s * 2 * KV_BYTES;
      const unsigned char* vb = kb + KV_BYTES;

      // mma.sync has a long latency on this part and a warp's MMAs into one accumulator run one
      // after the other: the k steps go to four accumulator sets in turn, added at the end
      float sc[2][4], sx[3][2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          sc[n][c] = 0.f;
#pragma unroll
          for (int a = 0; a < 3; ++a) sx[a][n][c] = 0.f;
        }
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        unsigned b[4];
        ldmatrix_x4(b, kb + swz<HD>(koff + (lane >> 4) * 8 + (lane & 7), ks * 2 + ((lane >> 3) & 1)));
        if ((ks & 3) == 0) {
          mma_bf16(sc[0], qf[ks], b[0], b[1]);
          mma_bf16(sc[1], qf[ks], b[2], b[3]);
        } else {
          mma_bf16(sx[(ks & 3) - 1][0], qf[ks], b[0], b[1]);
          mma_bf16(sx[(ks & 3) - 1][1], qf[ks], b[2], b[3]);
        }
      }
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) sc[n][c] += (sx[0][n][c] + sx[1][n][c]) + sx[2][n][c];
      const int kbase = tile0 + tile * TA_BN + koff;
      float mx[2] = {-INFINITY, -INFINITY};
      // Only a tile at an edge of some row's key range needs the mask; the warp decides once.
      const bool edge = kbase < lo_r[0] || kbase < lo_r[1] || kbase + 16 > hi_r[0] || kbase + 16 > hi_r[1];
      if (__any_sync(0xffffffffu, edge)) {
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int key = kbase + n * 8 + 2 * t4 + (c & 1);
            const int i = c >> 1;
            const float v = (key < hi_r[i] && key >= lo_r[i]) ? sc[n][c] * p.scale_log2 : -INFINITY;
            sc[n][c] = v;
            mx[i] = fmaxf(mx[i], v);
          }
      } else {
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            sc[n][c] *= p.scale_log2;
            mx[c >> 1] = fmaxf(mx[c >> 1], sc[n][c]);
          }
      }
      float corr[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        const float m_new = fmaxf(m_r[i], mx[i]);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        corr[i] = exp2f(m_r[i] - m_use);
        m_r[i] = m_new;
        mx[i] = m_use;
        l_r[i] *= corr[i];
      }
      // the running maximum seldom moves after the first tiles: rescale the output only when it did
      if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
        for (int d = 0; d < DT; ++d) {
          o[d][0] *= corr[0]; o[d][1] *= corr[0];
          o[d][2] *= corr[1]; o[d][3] *= corr[1];
        }
      }
      unsigned pf[4];
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const float p0 = exp2f(sc[n][0] - mx[0]), p1 = exp2f(sc[n][1] - mx[0]);
        const float p2 = exp2f(sc[n][2] - mx[1]), p3 = exp2f(sc[n][3] - mx[1]);
        l_r[0] += p0 + p1;
        l_r[1] += p2 + p3;
        pf[n * 2 + 0] = pack_bf16(p0, p1);
        pf[n * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int d = 0; d < DT; d += 2) {
        unsigned b[4];
        ldmatrix_x4_trans(b, vb + swz<HD>(koff + (lane & 7) + ((lane >> 3) & 1) * 8, d + (lane >> 4)));
        mma_bf16(o[d], pf, b[0], b[1]);
        mma_bf16(o[d + 1], pf, b[2], b[3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);             // this warp has read the stage
    }

#pragma unroll
    for (int i = 0; i < 2; ++i) {
      l_r[i] += __shfl_xor_sync(0xffffffffu, l_r[i], 1);
      l_r[i] += __shfl_xor_sync(0xffffffffu, l_r[i], 2);
    }
    // the four warps hold partial results for the same 16 rows over different keys: merge them.
    // The merge buffer lies over the stages, which nobody reads or fills any more once all four warps
    // are here (every copy that was issued has been waited for).
    asm volatile("bar.sync 1, 128;" ::: "memory");
    float* mo = reinterpret_cast<float*>(kv_s);                // [4][16][HD]
    float* mm = mo + 4 * 16 * HD;                              // [4][16] maxima, then [4][16] sums
    float* ml = mm + 64;
    static_assert(sizeof(float) * (4 * 16 * HD + 128) <= TA_STAGES * 2 * KV_BYTES, "merge buffer");
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = g + 8 * i;
#pragma unroll
      for (int d = 0; d < DT; ++d)
        *reinterpret_cast<float2*>(mo + (warp * 16 + r) * HD + d * 8 + 2 * t4) = make_float2(o[d][2 * i], o[d][2 * i + 1]);
      if (t4 == 0) {
        mm[warp * 16 + r] = m_r[i];
        ml[warp * 16 + r] = l_r[i];
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (!*failed) {
      for (int idx = tid; idx < 16 * (HD / 4); idx += 128) {
        const int r = idx / (HD / 4), d4 = (idx % (HD / 4)) * 4;
        const int row = row0 + r;
        if (row >= rows_total) continue;
        float mt = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mt = fmaxf(mt, mm[w * 16 + r]);
        float lt = 0.f, f[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          f[w] = ml[w * 16 + r] > 0.f ? exp2f(mm[w * 16 + r] - mt) : 0.f;
          lt += ml[w * 16 + r] * f[w];
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const float4 v = *reinterpret_cast<const float4*>(mo + (w * 16 + r) * HD + d4);
          acc.x += v.x * f[w]; acc.y += v.y * f[w]; acc.z += v.z * f[w]; acc.w += v.w * f[w];
        }
        const float inv = lt > 0.f ? 1.f / lt : 0.f;
        const size_t orow = (size_t)(q0 + row / G) * p.nq + kvh * G + row % G;
        if (p.num_splits > 1) {
          float* po = p.part_o + ((size_t)split * p.total_tokens * p.nq + orow) * HD + d4;
          *reinterpret_cast<float4*>(po) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
          if (d4 == 0) p.part_lse[(size_t)split * p.total_tokens * p.nq + orow] = lt > 0.f ? mt + log2f(lt) : -INFINITY;
        } else {
          *reinterpret_cast<uint2*>(p.out + orow * HD + d4) =
              make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
        }
      }
    }
  }
  // common exit: if something gave up, let the copies that were issued land before the shared
  // memory goes back (bounded), then leave
  __syncthreads();
  pdl_launch_dependents();
  if (*failed && tid == 0) {
    for (int s = 0; s < TA_STAGES; ++s) mbar_wait(&full[s], 0, TMA_DRAIN_NS);
  }
}

constexpr int TA_MAX_SPLITS = 128;     // the merge keeps one weight a range in shared memory
constexpr int TA_MERGE_WARPS = 8;      // at most

template <int HD>
__global__ void attention_tma_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                             __nv_bfloat16* __restrict__ out, int rows, int num_splits,
                                             const int* __restrict__ tile_seq, const int* __restrict__ q_start, int nq) {
  // One CTA per (tile, query head, token of the tile's request): the rows the decode form wrote and no others, so
  // that a step's other rows (a prompt portion's, the prefill form's) are neither read nor touched.  The step's
  // description is read before the wait for the kernel before.  The ranges' weights are found by the threads side
  // by side (a range a thread); then the warps share the ranges and the lanes the row's columns, so that a cut into
  // many ranges (one request at a long context) leaves no thread a long chain of dependent loads.
  constexpr int VEC = HD / 64;                                 // pairs of columns a lane holds
  __shared__ float w[TA_MAX_SPLITS];
  __shared__ float red[2][TA_MERGE_WARPS];
  __shared__ float2 sums[TA_MERGE_WARPS][HD / 2];
  const int seq = tile_seq[blockIdx.x];
  const int q0 = q_start[seq], q_len = q_start[seq + 1] - q0;
  pdl_launch_dependents();       // a short kernel: the successor may be set up behind it
  pdl_wait();
  if ((int)blockIdx.z >= q_len) return;
  const int row = (q0 + (int)blockIdx.z) * nq + (int)blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  float mt = -INFINITY;
  for (int s = tid; s < num_splits; s += blockDim.x) {
    const float l = part_lse[(size_t)s * rows + row];
    w[s] = l;
    mt = fmaxf(mt, l);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
  if (lane == 0) red[0][warp] = mt;
  __syncthreads();
  mt = red[0][0];
  for (int i = 1; i < warps; ++i) mt = fmaxf(mt, red[0][i]);
  float tot = 0.f;
  for (int s = tid; s < num_splits; s += blockDim.x) {
    const float l = w[s];
    const float e = l == -INFINITY ? 0.f : exp2f(l - mt);     // a range without a key of this row weighs nothing
    w[s] = e;
    tot += e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
  if (lane == 0) red[1][warp] = tot;
  __syncthreads();
  tot = red[1][0];
  for (int i = 1; i < warps; ++i) tot += red[1][i];
  const float inv = tot > 0.f ? 1.f / tot : 0.f;
  // a warp takes every warps-th range, its lanes the row's columns in pairs; then the warps' sums are added
  float2 acc[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) acc[k] = make_float2(0.f, 0.f);
#pragma unroll 4
  for (int s = warp; s < num_splits; s += warps) {
    const float e = w[s];
    if (e != 0.f) {                                           // what such a range left is not read
      const float2* src = reinterpret_cast<const float2*>(part_o + ((size_t)s * rows + row) * HD);
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        const float2 v = src[k * 32 + lane];
        acc[k].x = fmaf(v.x, e, acc[k].x);
        acc[k].y = fmaf(v.y, e, acc[k].y);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < VEC; ++k) sums[warp][k * 32 + lane] = acc[k];
  __syncthreads();
  for (int c = tid; c < HD / 2; c += blockDim.x) {
    float2 t = sums[0][c];
    for (int i = 1; i < warps; ++i) { t.x += sums[i][c].x; t.y += sums[i][c].y; }
    *reinterpret_cast<__nv_bfloat162*>(out + (size_t)row * HD + 2 * c) = __floats2bfloat162_rn(t.x * inv, t.y * inv);
  }
}

// tensor maps of the caches seen so far: (base, rows, page size, head size) -> map
struct MapKey {
  const void* base; long long rows; int ps, hd, nkv_run;      // nkv_run: 0 for the per-page map, else the kv heads of the run map
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && ps == o.ps && hd == o.hd && nkv_run == o.nkv_run;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (std::hash<long long>()(k.rows) * 31) ^ (size_t)(k.ps * 131 + k.hd + k.nkv_run * 7919);
  }
};
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
static std::mutex g_maps_mutex;

// nkv_run == 0: the map of one page a box; else the map whose box is the TA_BN / ps pages of a tile with consecutive ids
static bool cache_map(const void* base, long long rows, int ps, int hd, CUtensorMap* out, int nkv_run = 0) {
  std::lock_guard<std::mutex> lock(g_maps_mutex);
  MapKey key{base, rows, ps, hd, nkv_run};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return true;
  }
  if (rows > 0x7fffffffLL) return false;
  if (nkv_run == 0) {
    if (!make_map_rows(out, base, rows, hd / 64, ps)) return false;
  } else {
    if (!make_map_page_run(out, base, rows / ((long long)nkv_run * ps), nkv_run, ps, hd, TA_BN / ps, true)) return false;
  }
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps.emplace(key, *out);
  return true;
}

// dynamic shared memory of a CTA: the K/V stages, the queries, the barriers, the cached block table, alignment slack
constexpr size_t ta_smem(int hd) {
  return (size_t)TA_STAGES * 2 * TA_BN * hd * 2 + 16 * (hd + 8) * 2 + 2 * TA_STAGES * 8 + 16 + TA_BT_CACHE * 4 + 1024;
}

template <int HD>
static int launch_ta(const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& rk, const CUtensorMap& rv,
                     const AttnTmaParams& p, int tiles, cudaStream_t stream) {
  constexpr size_t smem = ta_smem(HD);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_tma_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      set_error("attention_tma: cannot raise the shared memory limit");
      return SLLM_ERR_LAUNCH;
    }
    configured = true;
  }
  dim3 grid((unsigned)tiles * p.nkv, 1, p.num_splits);
  launch_kernel(attention_tma_decode_kernel<HD>, grid, TA_THREADS, smem, stream, mk, mv, rk, rv, p);
  int rc = launch_status("attention_tma");
  if (rc != SLLM_OK) return rc;
  if (p.num_splits > 1) {
    const int G = p.nq / p.nkv;
    // a warp a range up to eight warps (batch 8, nine ranges: the step takes 3.18 ms so, 3.21 with three warps)
    const int merge_warps = p.num_splits < TA_MERGE_WARPS ? (p.num_splits > 2 ? p.num_splits : 2) : TA_MERGE_WARPS;
    launch_kernel(attention_tma_combine_kernel<HD>, dim3((unsigned)tiles, (unsigned)p.nq, (unsigned)(16 / G > 0 ? 16 / G : 1)),
                  32 * merge_warps, 0, stream, (const float*)p.part_o, (const float*)p.part_lse, p.out, p.total_tokens * p.nq,
                  p.num_splits, p.tile_seq, p.q_start, p.nq);
    rc = launch_status("attention_tma_combine");
  }
  return rc;
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_attention_tma_supports(int hd, int page_size) {
  // a page's box must start on a 1024-byte boundary of the swizzled tile: page sizes 8, 16, 32, 64
  return (hd == 64 || hd == 128) && page_size >= 8 && page_size <= 64 && 64 % page_size == 0 && encode_fn() != nullptr;
}

// CTAs of the decode form that share an SM (by shared memory: 228 KB an SM, 1 KB of it reserved per CTA): what the
// host sizes its cut of the context for
SLLM_EXPORT int sllm_attention_tma_ctas_per_sm(int hd) {
  const size_t per_cta = ta_smem(hd == 64 ? 64 : 128) + 1024;
  const int by_smem = (int)((size_t)228 * 1024 / per_cta), by_threads = 2048 / TA_THREADS;
  return by_smem < by_threads ? (by_smem < 1 ? 1 : by_smem) : by_threads;
}

// The decode form only: every tile holds at most 16 (token, head-in-group) rows.  num_pages: pages in the
// cache tensors [num_pages, nkv, page_size, hd].  status: one int of device memory, zero before the launch.
SLLM_EXPORT int sllm_attention_tma_decode(const void* q, const void* k_cache, const void* v_cache, long long num_pages,
                                          void* out, float* part_o, float* part_lse, const int* block_tables,
                                          int max_pages, const int* q_start, const int* ctx_len, const int* tile_seq,
                                          const int* tile_row0, int tiles, int num_splits, int total_tokens, int nq,
                                          int nkv, int hd, int page_size, float scale, int window, int* status,
                                          cudaStream_t stream) {
  SLLM_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_tma: bad head counts nq=%d nkv=%d", nq, nkv);
  SLLM_REQUIRE(sllm_attention_tma_supports(hd, page_size), "attention_tma: head_dim=%d page_size=%d not taken", hd, page_size);
  SLLM_REQUIRE(max_pages > 0 && tiles >= 0 && total_tokens >= 0 && num_pages > 0, "attention_tma: bad sizes");
  SLLM_REQUIRE(num_splits >= 1 && num_splits <= TA_MAX_SPLITS && nkv <= 65535, "attention_tma: bad grid nkv=%d splits=%d", nkv, num_splits);
  SLLM_REQUIRE(num_splits == 1 || (part_o && part_lse), "attention_tma: split-KV needs scratch");
  SLLM_REQUIRE(status != nullptr, "attention_tma: a status word is required");
  SLLM_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0, "attention_tma: the cache must be 16-byte aligned");
  if (tiles == 0) return SLLM_OK;
  CUtensorMap mk, mv;
  const long long rows = num_pages * nkv * page_size;
  if (!cache_map(k_cache, rows, page_size, hd, &mk) || !cache_map(v_cache, rows, page_size, hd, &mv)) {
    set_error("attention_tma: cuTensorMapEncodeTiled failed");
    return SLLM_ERR_LAUNCH;
  }
  // the maps whose box is a whole tile's pages, for tiles whose pages have consecutive ids (not needed
  // when a page is a tile already)
  CUtensorMap rk = mk, rv = mv;
  const bool runs = page_size < TA_BN && cache_map(k_cache, rows, page_size, hd, &rk, nkv) &&
                    cache_map(v_cache, rows, page_size, hd, &rv, nkv);
  AttnTmaParams p;
  p.page_runs = runs ? 1 : 0;
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.part_o = part_o; p.part_lse = part_lse;
  p.block_tables = block_tables; p.q_start = q_start; p.ctx_len = ctx_len; p.tile_seq = tile_seq; p.tile_row0 = tile_row0;
  p.status = status; p.max_pages = max_pages; p.page_size = page_size; p.nq = nq; p.nkv = nkv; p.window = window;
  p.num_splits = num_splits; p.total_tokens = total_tokens; p.scale_log2 = scale * 1.4426950408889634f;

  return hd == 128 ? launch_ta<128>(mk, mv, rk, rv, p, tiles, stream) : launch_ta<64>(mk, mv, rk, rv, p, tiles, stream);
}
