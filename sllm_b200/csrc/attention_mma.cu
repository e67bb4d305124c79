// Tensor-core attention over the paged cache for the bfloat16 path: causal GQA with an
// online softmax, for prompt portions and for decoding, in one kernel family.
//
// The query heads that share a kv head are stacked along the M dimension of the MMA:
// a tile's rows are (token, head-in-group) pairs of one request and one kv head, so a
// key/value tile fetched from the pages serves all of the group's heads.  Each row
// carries its own position, so a portion that starts anywhere in the context, and a
// single decoded token, are the same code.
//
//   PREFILL form: 128 rows per CTA, 8 warps x 16 rows, every warp walks all keys of a tile.
//   DECODE form:  16 rows per CTA (a request's one or two tokens x its group); the four
//                 warps take different 16-key slices of each 64-key tile and merge at the
//                 end; the grid's z dimension splits the context further (split-KV), the
//                 partial results go to scratch and a second kernel combines them.
//
// Scores, softmax and the output accumulation are float32 (mma.sync m16n8k16, bf16 in,
// f32 out); probabilities are rounded to bfloat16 for the P.V product.
// Formulas: ref/qwen3_5.py:373-390 (scores * scale, causal mask, softmax, P.V);
// ref/standard.py:65-68 (query head h reads kv head h / group).  The reference has no
// such kernel on the device: its decode attention is one CTA per head without tensor
// cores (kernels/cuda/kernels.cu:957-1025) and its prefill runs in numpy.
#include <math.h>
#include <stdio.h>

#include "mma.cuh"

namespace sllm {

struct AttnParams {
  const __nv_bfloat16* q;        // [T, nq, HD]
  const __nv_bfloat16* k_cache;  // [pages, nkv, page_size, HD]
  const __nv_bfloat16* v_cache;
  __nv_bfloat16* out;            // [T, nq, HD]
  float* part_o;                 // [splits, T, nq, HD]   (splits > 1)
  float* part_lse;               // [splits, T, nq]
  const int* block_tables;       // [S, max_pages]
  const int* q_start;            // [S+1]
  const int* ctx_len;            // [S]
  const int* tile_seq;           // [tiles]
  const int* tile_row0;          // [tiles]
  int max_pages, page_size, nq, nkv, window, num_splits, total_tokens;
  float scale_log2;              // scale * log2(e)
};

constexpr int ATT_BN = 64;     // keys per tile
// block-table entries a CTA keeps in shared memory (the decode form reads a split of the
// context only, and must leave room for two CTAs per SM)
template <bool DECODE> struct AttBtCache { static constexpr int value = DECODE ? 512 : 1024; };
template <bool DECODE> struct AttThreads { static constexpr int value = DECODE ? 128 : 256; };
template <bool DECODE> struct AttStages { static constexpr int value = DECODE ? 3 : 4; };

template <int HD, bool DECODE>
__global__ void __launch_bounds__(AttThreads<DECODE>::value) attention_mma_kernel(const AttnParams p) {
  constexpr int NTHREADS = AttThreads<DECODE>::value;
  constexpr int STRIDE = HD + 8;                 // 16 bytes of padding: ldmatrix rows fall in distinct banks
  constexpr int KSTEPS = HD / 16;
  constexpr int DT = HD / 8;                     // output n-tiles
  constexpr int BM = DECODE ? 16 : 128;
  constexpr int NT = DECODE ? 2 : 8;             // 8-key n-tiles a warp computes per key tile
  constexpr int CHUNKS = HD / 8;                 // 16-byte chunks per row
  // key/value tiles in flight.  Both forms are bound by the latency of a tile's loads, not by their
  // bandwidth: with 2 stages the prefill form took 234 us a layer at 7B sizes, with 4 stages 160 us.
  constexpr int STAGES = AttStages<DECODE>::value;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* k_s = q_s + BM * STRIDE;
  __nv_bfloat16* v_s = k_s + STAGES * ATT_BN * STRIDE;
  constexpr int BT_CACHE = AttBtCache<DECODE>::value;
  int* bt_s = reinterpret_cast<int*>(v_s + STAGES * ATT_BN * STRIDE);      // [BT_CACHE]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  pdl_wait();       // everything below reads what the step's earlier kernels or its batch upload wrote
  // the KV head is the grid's fastest index: tiles come longest first and CTAs start in grid order,
  // so every head's long tiles start in the first wave
  const int tile_i = blockIdx.x / p.nkv, kvh = blockIdx.x % p.nkv, split = blockIdx.z;
  const int seq = p.tile_seq[tile_i], row0 = p.tile_row0[tile_i];
  const int G = p.nq / p.nkv;
  const int q0 = p.q_start[seq], q_len = p.q_start[seq + 1] - q0, ctx = p.ctx_len[seq];
  const int rows_total = q_len * G;
  const int pos0 = ctx - q_len;                  // position of the request's first token of this step
  const int row_hi = min(row0 + BM, rows_total);
  const int* bt = p.block_tables + (size_t)seq * p.max_pages;

  int key_hi = pos0 + (row_hi - 1) / G + 1;      // exclusive: the last row's own position is its last key
  int key_lo = 0;
  if (p.window > 0) key_lo = max(0, pos0 + row0 / G - p.window + 1);
  if (p.num_splits > 1) {
    const int chunk = ((ctx + p.num_splits - 1) / p.num_splits + ATT_BN - 1) / ATT_BN * ATT_BN;
    key_lo = max(key_lo, split * chunk);
    key_hi = min(key_hi, (split + 1) * chunk);
  }
  const int tile0 = key_lo / ATT_BN * ATT_BN;    // tiles start at multiples of 64 keys, whatever the cut
  const int n_tiles = key_hi > tile0 ? (key_hi - tile0 + ATT_BN - 1) / ATT_BN : 0;

  // the pages of this CTA's key range, fetched once: a tile's loads then depend on shared
  // memory only, not on a global load of the table
  const int page_first = tile0 / p.page_size;
  const int page_count = n_tiles > 0 ? (key_hi - 1) / p.page_size - page_first + 1 : 0;
  const bool bt_cached = page_count <= BT_CACHE;
  if (bt_cached) {
    for (int i = tid; i < page_count; i += NTHREADS) bt_s[i] = bt[page_first + i];
    __syncthreads();
  }

  // ---- loads -----------------------------------------------------------------------
  auto load_q = [&]() {
    for (int c = tid; c < BM * CHUNKS; c += NTHREADS) {
      const int r = c / CHUNKS, ch = c % CHUNKS;
      const int row = row0 + r;
      const bool ok = row < rows_total;
      const int tok = ok ? row / G : 0, hg = ok ? row % G : 0;
      const __nv_bfloat16* src = p.q + ((size_t)(q0 + tok) * p.nq + kvh * G + hg) * HD + ch * 8;
      cp_async_16(q_s + r * STRIDE + ch * 8, src, ok);
    }
  };
  // each thread keeps one 16-byte column of the rows r_first, r_first + R_STEP, ...: the address
  // arithmetic of a tile is a handful of instructions per row
  constexpr int R_STEP = NTHREADS / CHUNKS;
  const int ch8 = (tid % CHUNKS) * 8, r_first = tid / CHUNKS;
  const int ps = p.page_size;
  const int ps_shift = (ps & (ps - 1)) == 0 ? __ffs(ps) - 1 : -1;
  const size_t head_off = (size_t)kvh * ps * HD + ch8;
  const size_t page_stride = (size_t)p.nkv * ps * HD;
  auto load_kv = [&](int tile, int buf) {
    const int kbase = tile0 + tile * ATT_BN;
#pragma unroll
    for (int r = r_first; r < ATT_BN; r += R_STEP) {
      const int key = kbase + r;
      bool ok = key < key_hi && key >= key_lo;
      int page = 0, off = 0;
      if (ok) {
        const int pi = ps_shift >= 0 ? key >> ps_shift : key / ps;
        off = key - pi * ps;
        page = bt_cached ? bt_s[pi - page_first] : bt[pi];
        ok = page >= 0;                           // a page given back is never read
        if (!ok) page = 0;
      }
      const size_t src = (size_t)page * page_stride + head_off + (size_t)off * HD;
      cp_async_16(k_s + (buf * ATT_BN + r) * STRIDE + ch8, p.k_cache + src, ok);
      cp_async_16(v_s + (buf * ATT_BN + r) * STRIDE + ch8, p.v_cache + src, ok);
    }
  };

  load_q();
  cp_async_commit();
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < n_tiles) load_kv(st, st);
    cp_async_commit();
  }

  // ---- per-thread rows: g and g+8 of the warp's 16-row block ---------------------------
  const int wrow = DECODE ? 0 : warp * 16;
  int hi_r[2], lo_r[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + wrow + g + 8 * i;
    if (row < rows_total) {
      const int pos = pos0 + row / G;
      hi_r[i] = min(pos + 1, key_hi);
      lo_r[i] = p.window > 0 ? max(key_lo, pos - p.window + 1) : key_lo;
    } else {
      hi_r[i] = 0;
      lo_r[i] = 1;                                // empty
    }
  }
  float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
  float o[DT][4];
#pragma unroll
  for (int d = 0; d < DT; ++d)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[d][c] = 0.f;

  cp_async_wait<STAGES - 1>();                    // the queries have landed
  __syncthreads();
  unsigned qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks)
    ldmatrix_x4(qf[ks], q_s + (wrow + (lane & 15)) * STRIDE + ks * 16 + (lane >> 4) * 8);

  const int koff = DECODE ? warp * 16 : 0;        // the warp's keys within a tile
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile % STAGES;
    if (tile + STAGES - 1 < n_tiles) load_kv(tile + STAGES - 1, (tile + STAGES - 1) % STAGES);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();                  // tile `tile` has landed
    __syncthreads();
    const __nv_bfloat16* kb = k_s + buf * ATT_BN * STRIDE;
    const __nv_bfloat16* vb = v_s + buf * ATT_BN * STRIDE;

    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[n][c] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int n = 0; n < NT; n += 2) {
        unsigned b[4];
        ldmatrix_x4(b, kb + (koff + n * 8 + (lane >> 4) * 8 + (lane & 7)) * STRIDE + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[n], qf[ks], b[0], b[1]);
        mma_bf16(s[n + 1], qf[ks], b[2], b[3]);
      }
    }
    // mask, scale (into the log2 domain), row maxima
    const int kbase = tile0 + tile * ATT_BN + koff;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = kbase + n * 8 + 2 * t4 + (c & 1);
        const int i = c >> 1;
        const float v = (key < hi_r[i] && key >= lo_r[i]) ? s[n][c] * p.scale_log2 : -INFINITY;
        s[n][c] = v;
        mx[i] = fmaxf(mx[i], v);
      }
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      const float m_new = fmaxf(m_r[i], mx[i]);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;    // a row with no key yet
      corr[i] = exp2f(m_r[i] - m_use);
      m_r[i] = m_new;
      mx[i] = m_use;
      l_r[i] *= corr[i];
    }
#pragma unroll
    for (int d = 0; d < DT; ++d) {
      o[d][0] *= corr[0]; o[d][1] *= corr[0];
      o[d][2] *= corr[1]; o[d][3] *= corr[1];
    }
    unsigned pf[NT / 2][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const float p0 = exp2f(s[n][0] - mx[0]), p1 = exp2f(s[n][1] - mx[0]);
      const float p2 = exp2f(s[n][2] - mx[1]), p3 = exp2f(s[n][3] - mx[1]);
      l_r[0] += p0 + p1;
      l_r[1] += p2 + p3;
      pf[n / 2][(n & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[n / 2][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
#pragma unroll
      for (int d = 0; d < DT; d += 2) {
        unsigned b[4];
        ldmatrix_x4_trans(b, vb + (koff + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + d * 8 + (lane >> 4) * 8);
        mma_bf16(o[d], pf[kk], b[0], b[1]);
        mma_bf16(o[d + 1], pf[kk], b[2], b[3]);
      }
    }
    __syncthreads();                              // the next iteration refills the buffer just read
  }
  cp_async_wait<0>();
  pdl_launch_dependents();             // all keys are read; the next kernel may begin during the epilogue

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_r[i] += __shfl_xor_sync(0xffffffffu, l_r[i], 1);
    l_r[i] += __shfl_xor_sync(0xffffffffu, l_r[i], 2);
  }

  if constexpr (!DECODE) {
    // each warp owns its rows
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = row0 + wrow + g + 8 * i;
      if (row >= rows_total) continue;
      const size_t orow = (size_t)(q0 + row / G) * p.nq + kvh * G + row % G;
      const float inv = l_r[i] > 0.f ? 1.f / l_r[i] : 0.f;
      if (p.num_splits > 1) {
        float* po = p.part_o + ((size_t)split * p.total_tokens * p.nq + orow) * HD;
#pragma unroll
        for (int d = 0; d < DT; ++d)
          *reinterpret_cast<float2*>(po + d * 8 + 2 * t4) = make_float2(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
        if (t4 == 0)
          p.part_lse[(size_t)split * p.total_tokens * p.nq + orow] = l_r[i] > 0.f ? m_r[i] + log2f(l_r[i]) : -INFINITY;
      } else {
        __nv_bfloat16* po = p.out + orow * HD;
#pragma unroll
        for (int d = 0; d < DT; ++d)
          *reinterpret_cast<unsigned*>(po + d * 8 + 2 * t4) = pack_bf16(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
      }
    }
  } else {
    // the four warps hold partial results for the same 16 rows over different keys: merge
    float* mo = reinterpret_cast<float*>(k_s);                 // [4][16][HD]
    float* mm = mo + 4 * 16 * HD;                              // [4][16] maxima, then [4][16] sums
    float* ml = mm + 64;
    static_assert(sizeof(float) * (4 * 16 * HD + 128) <= sizeof(__nv_bfloat16) * 2 * STAGES * ATT_BN * STRIDE, "merge buffer");
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
    __syncthreads();
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
        __nv_bfloat16* po = p.out + orow * HD + d4;
        *reinterpret_cast<uint2*>(po) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
      }
    }
  }
}

// out[row] = sum_s w_s part_o[s][row], w_s = 2^(lse_s - max) / sum: the splits of one row merged.
template <int HD>
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                             __nv_bfloat16* __restrict__ out, int rows, int num_splits,
                                             const int* __restrict__ tile_seq, const int* __restrict__ q_start, int nq) {
  // One CTA per (tile, query head, token of the tile's request): the rows the decode form wrote and no others, so
  // that a step's other rows (a prompt portion's, the prefill form's) are neither read nor touched.  The step's
  // description is read before the wait for the kernel before.
  const int seq = tile_seq[blockIdx.x];
  const int q0 = q_start[seq], q_len = q_start[seq + 1] - q0;
  pdl_launch_dependents();       // a short kernel: the successor may be set up behind it
  pdl_wait();
  if ((int)blockIdx.z >= q_len) return;
  const int row = (q0 + (int)blockIdx.z) * nq + (int)blockIdx.y;
  float mt = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mt = fmaxf(mt, part_lse[(size_t)s * rows + row]);
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

template <int HD, bool DECODE>
static int launch_attention(const AttnParams& p, int tiles, cudaStream_t stream) {
  constexpr int BM = DECODE ? 16 : 128;
  constexpr size_t smem = sizeof(__nv_bfloat16) * (size_t)(BM + 2 * AttStages<DECODE>::value * ATT_BN) * (HD + 8) +
                          sizeof(int) * AttBtCache<DECODE>::value;
  static bool configured = false;                 // per template instance
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<HD, DECODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      set_error("attention_mma: cannot raise the shared memory limit");
      return SLLM_ERR_LAUNCH;
    }
    configured = true;
  }
  dim3 grid((unsigned)tiles * p.nkv, 1, p.num_splits);
  launch_kernel(attention_mma_kernel<HD, DECODE>, grid, AttThreads<DECODE>::value, smem, stream, p);
  int rc = launch_status("attention_mma");
  if (rc != SLLM_OK) return rc;
  if (p.num_splits > 1) {
    const int G = p.nq / p.nkv;
    launch_kernel(attention_combine_kernel<HD>, dim3((unsigned)tiles, (unsigned)p.nq, (unsigned)(16 / G > 0 ? 16 / G : 1)), HD >= 128 ? 128 : 64, 0, stream,
                  (const float*)p.part_o, (const float*)p.part_lse, p.out, p.total_tokens * p.nq, p.num_splits, p.tile_seq,
                  p.q_start, p.nq);
    rc = launch_status("attention_combine");
  }
  return rc;
}

}  // namespace sllm

using namespace sllm;

// 1 if the tensor-core kernel takes this head size (others go to the CUDA-core kernel).
SLLM_EXPORT int sllm_attention_mma_supports(int hd) { return hd == 16 || hd == 32 || hd == 64 || hd == 128; }

// tiles: tile_seq/tile_row0 [tiles] describe 128-row (decode == 0) or 16-row (decode == 1) tiles of
// (token, head-in-group) rows.  part_o/part_lse are scratch for num_splits > 1:
// float32 [num_splits, T, nq, hd] and [num_splits, T, nq].
SLLM_EXPORT int sllm_attention_mma(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o,
                                   float* part_lse, const int* block_tables, int max_pages, const int* q_start,
                                   const int* ctx_len, const int* tile_seq, const int* tile_row0, int tiles,
                                   int decode, int num_splits, int total_tokens, int nq, int nkv, int hd,
                                   int page_size, float scale, int window, cudaStream_t stream) {
  SLLM_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_mma: bad head counts nq=%d nkv=%d", nq, nkv);
  SLLM_REQUIRE(sllm_attention_mma_supports(hd), "attention_mma: head_dim=%d is not one of 16, 32, 64, 128", hd);
  SLLM_REQUIRE(page_size > 0 && max_pages > 0 && tiles >= 0 && total_tokens >= 0, "attention_mma: bad sizes");
  SLLM_REQUIRE(num_splits >= 1 && num_splits <= 65535 && nkv <= 65535, "attention_mma: bad grid nkv=%d splits=%d", nkv, num_splits);
  SLLM_REQUIRE(num_splits == 1 || (part_o && part_lse), "attention_mma: split-KV needs scratch");
  if (tiles == 0) return SLLM_OK;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.out = (__nv_bfloat16*)out; p.part_o = part_o; p.part_lse = part_lse; p.block_tables = block_tables;
  p.q_start = q_start; p.ctx_len = ctx_len; p.tile_seq = tile_seq; p.tile_row0 = tile_row0;
  p.max_pages = max_pages; p.page_size = page_size; p.nq = nq; p.nkv = nkv; p.window = window;
  p.num_splits = num_splits; p.total_tokens = total_tokens;
  p.scale_log2 = scale * 1.4426950408889634f;
#define DISPATCH(HD_)                                                             \
  case HD_:                                                                       \
    return decode ? launch_attention<HD_, true>(p, tiles, stream) : launch_attention<HD_, false>(p, tiles, stream);
  switch (hd) {
    DISPATCH(16) DISPATCH(32) DISPATCH(64) DISPATCH(128)
  }
#undef DISPATCH
  return SLLM_ERR_UNSUPPORTED;
}
