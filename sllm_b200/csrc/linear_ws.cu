// Weight-streaming linear layer for at most 16 tokens and a modest number of output rows (the
// attention and down projections of a decode step): y[M, N] = x[M, K] W[N, K]^T.
//
// linear_stream.cu gives 128 weight rows to a CTA and, when N is small, splits K over the grid,
// leaving partial sums for the consumer.  Here a CTA owns 16 output rows over the whole of K and
// its 8 warps split K among themselves: warp w takes the 32-wide k blocks w, w+8, w+16, ...
// (so the CTA reads 512 contiguous bytes of each row at a time), four blocks in flight per warp,
// weights and activations both loaded straight into MMA fragments (same k permutation as in
// linear_stream.cu), no shared memory and no barrier inside the loop.  At the end the warps'
// partial tiles are added through shared memory in warp order (a fixed order), and since the CTA
// holds complete sums the epilogue can finish the layer's job:
//   store      out[M, N] (+ bias), float32 or bfloat16
//   residual   residual[M, N] += y (+ bias): the float32 stream is updated in place, so the next
//              norm has nothing to add
//   rotary     for the fused q|k|v matrix of an attention layer: bias, rotary encoding and the write
//              of the new keys and values into their cache pages, so that the decode step needs no
//              kernel between this product and the attention.  A CTA then takes the 8 rows j..j+7
//              of a head and the 8 rows hd/2 apart: the two rows of a rotation pair are the two
//              rows (g, g+8) of one MMA accumulator, and meet in one thread of the epilogue
//              (ref/qwen3_5.py:355-370; cache content ref/incremental.py:135-139).
// About N/16 CTAs keep every SM busy without splitting K over the grid; their number is rounded up
// to a multiple of the SM count and the rows dealt evenly (N = 3584: 296 CTAs of 12 or 13 rows
// instead of 224 of 16, of which 76 SMs would get two and 72 one).
//
// The reference calls cublasGemmEx for these products and adds the residual in its next
// add_rms kernel (kernels/cuda/kernels.cu:752-767, 791-839; kernels/device_decode.py:312-325).
#include <stdio.h>

#include "common.cuh"

namespace sllm {

#define WS_EPI_STORE 0
#define WS_EPI_RESID 1
#define WS_EPI_ROPE 2

// what the rotary epilogue needs beside the product: the rows of W are q heads, then k heads, then v
// heads of `hd` rows each; table [max_pos][2][hd/2] holds cos then sin (rotary_dim == hd), or is null
// (no rotation); a token's key and value go to slot_mapping[token] of the paged caches
// [page][kv head][slot in page][hd] (null: not written), its queries to q_out [M, nq * hd].
struct WsRope {
  const int* positions;
  const float* table;
  const int* slot_mapping;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  __nv_bfloat16* q_out;
  int max_pos, nq, nkv, hd, page_size, num_pages;
};

__device__ __forceinline__ uint4 ws_ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ws_ldg(const void* p) {       // activations: small, shared by all CTAs, keep in L1
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void ws_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                       unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int WS_WARPS = 8;
// k blocks a warp keeps in flight per group (two groups): with two token tiles half as many, so that the
// activation fragments fit the registers of two CTAs an SM (four: 174 registers a thread, one CTA an SM)
__host__ __device__ constexpr int ws_depth(int nt) { return nt == 1 ? 4 : (nt == 2 ? 2 : 1); }
constexpr int WS_SSQ_MAX = 608;     // partial sums of squares per token a consumer takes (the producer's CTAs: at most 592 for 8192 columns)
// with four token tiles (17..32 tokens: small matrices only, where a step is bound by its number of kernels) the table
// is kept to what fits static shared memory beside the warps' tiles: streams of up to 3,072 columns
__host__ __device__ constexpr int ws_ssq_max(int nt) { return nt <= 2 ? WS_SSQ_MAX : 192; }

// An RMSNorm taken apart, so that a decode step needs no kernel for it (y = x * rsqrt(mean(x^2) + eps) * gain,
// ref/standard.py:25-31).  The product that completes the residual stream (residual epilogue) also writes
// xg_out = bfloat16(stream * gain) and, per CTA, each token's sum of squares over the CTA's columns of the
// stream (ssq_out[token][cta]); the product that consumes the normed activations reads xg as its input and
// multiplies each token's row of its result by rsqrt(sum of the token's partial sums / width + eps):
// W (x g / rms) = (W (x g)) / rms.  The partial sums are added in a fixed order.  A table of partial sums is
// [tokens][stride] float32 with stride = parts rounded up to a multiple of 4 (rows start on 16 bytes); what
// lies between parts and stride is never written and never added.
struct WsNorm {
  const float* ssq_in = nullptr;     // consumer: [M][(parts_in + 3) & ~3]
  int parts_in = 0;
  float eps_in = 0.f, inv_width_in = 0.f;
  const float* gain = nullptr;       // producer (residual epilogue): the next norm's gain [N]
  __nv_bfloat16* xg_out = nullptr;   // [M, N]
  float* ssq_out = nullptr;          // [M][(gridDim.x + 3) & ~3]
};

// NT: 8-token tiles (M <= 8 * NT).  OUT: float or __nv_bfloat16 (store epilogue only).  SCALED: the input
// comes with a norm still owed (WsNorm::ssq_in).
template <int NT, int EPI, typename OUT, bool SCALED>
__global__ void __launch_bounds__(WS_WARPS * 32, 2)
linear_ws_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W,
                 const float* __restrict__ bias, OUT* __restrict__ out, float* __restrict__ residual,
                 int M, int N, int K, const WsRope rope, const WsNorm norm) {
  constexpr int WS_DEPTH = ws_depth(NT);
  __shared__ float red[WS_WARPS][16][8 * NT + 1];
  __shared__ float row_scale[8 * NT];
  __shared__ __align__(16) float ssq_s[SCALED ? 8 * NT : 1][SCALED ? ws_ssq_max(NT) : 4];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  // the CTA's rows [n0, n1): at most 16, the N rows dealt evenly over the grid (so that a grid of a
  // whole number of CTAs per SM gives every SM the same bytes to stream)
  int n0 = (int)(((long long)blockIdx.x * N) / gridDim.x), n1 = (int)(((long long)(blockIdx.x + 1) * N) / gridDim.x);
  const int k_blocks = K / 32;

  int r0 = min(n0 + g, n1 - 1), r1 = min(n0 + g + 8, n1 - 1);   // rows past the CTA's: clamped loads, skipped stores
  if constexpr (EPI == WS_EPI_ROPE) {
    // CTA b of a head's hd/16: rows [8c, 8c+8) of the head and the 8 rows hd/2 further
    const int per_head = rope.hd / 16;
    n0 = ((int)blockIdx.x / per_head) * rope.hd + ((int)blockIdx.x % per_head) * 8;
    n1 = n0 + 16;                                  // (not a range: local row r is n0 + (r & 7) + (r >> 3) * hd/2)
    r0 = n0 + g;
    r1 = n0 + rope.hd / 2 + g;
  }
  const __nv_bfloat16* w0 = W + (size_t)r0 * K + t4 * 8;
  const __nv_bfloat16* w1 = W + (size_t)r1 * K + t4 * 8;
  const __nv_bfloat16* xr[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) xr[j] = x + (size_t)min(8 * j + g, M - 1) * K + t4 * 8;   // tokens past M: clamped, skipped

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;

  // Two groups of WS_DEPTH k blocks are in flight per warp: while one is multiplied, the loads of
  // the next (weights and activations) are already under way.  The first weights do not depend
  // on the step's earlier kernels and are fetched before the wait; the activations after it.
  uint4 wa0[WS_DEPTH], wb0[WS_DEPTH], wa1[WS_DEPTH], wb1[WS_DEPTH];
  uint4 x0[WS_DEPTH][NT], x1[WS_DEPTH][NT];
  auto load_w = [&](uint4 (&wa)[WS_DEPTH], uint4 (&wb)[WS_DEPTH], int kb) {
#pragma unroll
    for (int d = 0; d < WS_DEPTH; ++d) {
      const int b = kb + d * WS_WARPS;
      if (b < k_blocks) {
        wa[d] = ws_ldg_stream(w0 + (size_t)b * 32);
        wb[d] = ws_ldg_stream(w1 + (size_t)b * 32);
      }
    }
  };
  auto load_x = [&](uint4 (&xv)[WS_DEPTH][NT], int kb) {
#pragma unroll
    for (int d = 0; d < WS_DEPTH; ++d) {
      const int b = kb + d * WS_WARPS;
      if (b < k_blocks) {
#pragma unroll
        for (int j = 0; j < NT; ++j) xv[d][j] = ws_ldg(xr[j] + (size_t)b * 32);
      }
    }
  };
  auto compute = [&](const uint4 (&wa)[WS_DEPTH], const uint4 (&wb)[WS_DEPTH], const uint4 (&xv)[WS_DEPTH][NT], int kb) {
#pragma unroll
    for (int d = 0; d < WS_DEPTH; ++d) {
      if (kb + d * WS_WARPS < k_blocks) {
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          ws_mma(acc[j], wa[d].x, wb[d].x, wa[d].y, wb[d].y, xv[d][j].x, xv[d][j].y);
          ws_mma(acc[j], wa[d].z, wb[d].z, wa[d].w, wb[d].w, xv[d][j].z, xv[d][j].w);
        }
      }
    }
  };
  constexpr int GROUP = WS_DEPTH * WS_WARPS;        // k blocks the CTA covers per group
  int kb = warp;
  load_w(wa0, wb0, kb);
  pdl_wait();
  load_x(x0, kb);
  // a norm still owed on the input: the tokens' partial sums of squares are copied to shared memory under
  // the stream and added after the loop
  if constexpr (SCALED) {
    const int stride = (norm.parts_in + 3) & ~3, chunks = stride >> 2;
    for (int c = tid; c < M * chunks; c += WS_WARPS * 32) {
      const int tok = c / chunks, piece = c % chunks;
      const unsigned dst = (unsigned)__cvta_generic_to_shared(&ssq_s[tok][piece * 4]);
      asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(norm.ssq_in + (size_t)tok * stride + piece * 4));
    }
    asm volatile("cp.async.commit_group;\n" ::);
  }
  for (; kb < k_blocks; kb += 2 * GROUP) {
    load_w(wa1, wb1, kb + GROUP);
    load_x(x1, kb + GROUP);
    compute(wa0, wb0, x0, kb);
    load_w(wa0, wb0, kb + 2 * GROUP);
    load_x(x0, kb + 2 * GROUP);
    compute(wa1, wb1, x1, kb + GROUP);
  }
  pdl_launch_dependents();

  if constexpr (SCALED) asm volatile("cp.async.wait_group 0;\n" ::);
  // ---- add the warps' tiles in warp order; acc[j][c]: c0,c1 = (row g, tokens 8j+2t, +1); c2,c3 = (row g+8, ...) ----
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) red[warp][g + ((c & 2) ? 8 : 0)][8 * j + 2 * t4 + (c & 1)] = acc[j][c];
  __syncthreads();
  if constexpr (SCALED) {
    // warp w adds the partial sums of tokens w, w + 8: lane l takes l, l + 32, ..., then the lanes are added
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int tok = warp + 8 * j;
      float sum = 0.f;
      if (tok < M)
        for (int p = lane; p < norm.parts_in; p += 32) sum += ssq_s[tok][p];
      sum = warp_sum(sum);
      if (lane == 0) row_scale[tok] = rsqrtf(sum * norm.inv_width_in + norm.eps_in);
    }
    __syncthreads();
  }
  if constexpr (EPI == WS_EPI_ROPE) {
    const int half = rope.hd / 2;
    const int head = n0 / rope.hd, j0 = n0 % rope.hd;            // j0 = 8c: the pair's lower dimension starts here
    for (int idx = tid; idx < 8 * 8 * NT; idx += WS_WARPS * 32) {
      const int i = idx % 8, tok = idx / 8;                        // consecutive threads -> consecutive dimensions of one token
      if (tok >= M) continue;
      float lo = 0.f, hi = 0.f;
#pragma unroll
      for (int w = 0; w < WS_WARPS; ++w) { lo += red[w][i][tok]; hi += red[w][i + 8][tok]; }
      if constexpr (SCALED) {
        lo *= row_scale[tok];
        hi *= row_scale[tok];
      }
      if (bias) { lo += bias[n0 + i]; hi += bias[n0 + half + i]; }
      __nv_bfloat16* dst;
      if (head < rope.nq) {
        dst = rope.q_out + ((size_t)tok * rope.nq + head) * rope.hd;
      } else {
        int slot = rope.slot_mapping ? rope.slot_mapping[tok] : -1;
        if (slot < 0 || slot / rope.page_size >= rope.num_pages) continue;     // not written (padding row, borrowed cache)
        const bool is_k = head < rope.nq + rope.nkv;
        const int kvh = is_k ? head - rope.nq : head - rope.nq - rope.nkv;
        dst = (is_k ? rope.k_cache : rope.v_cache) +
              (((size_t)(slot / rope.page_size) * rope.nkv + kvh) * rope.page_size + slot % rope.page_size) * rope.hd;
      }
      if (rope.table != nullptr && head < rope.nq + rope.nkv) {
        int pos = rope.positions[tok];
        pos = pos < 0 ? 0 : (pos >= rope.max_pos ? rope.max_pos - 1 : pos);
        const float* cs = rope.table + (size_t)pos * rope.hd;        // cos[half] then sin[half]
        const float c = cs[j0 + i], sn = cs[half + j0 + i];
        const float a = lo * c - hi * sn, b = hi * c + lo * sn;
        lo = a;
        hi = b;
      }
      dst[j0 + i] = __float2bfloat16_rn(lo);
      dst[j0 + half + i] = __float2bfloat16_rn(hi);
    }
    return;
  }
  for (int idx = tid; idx < 16 * 8 * NT; idx += WS_WARPS * 32) {
    const int row = idx % 16, tok = idx / 16;           // consecutive threads -> consecutive rows of one token
    const int n = n0 + row;
    const bool valid = tok < M && n < n1;               // (whole warps run the loop: 16 * 8 * NT is a multiple of 32)
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < WS_WARPS; ++w) v += red[w][row][tok];
    if constexpr (SCALED) v *= row_scale[tok];
    if (bias && valid) v += bias[n];
    if constexpr (EPI == WS_EPI_RESID) {
      float sq = 0.f;
      if (valid) {
        const float r = residual[(size_t)tok * N + n] + v;
        residual[(size_t)tok * N + n] = r;
        if (norm.xg_out != nullptr) {
          norm.xg_out[(size_t)tok * N + n] = __float2bfloat16_rn(r * norm.gain[n]);
          sq = r * r;
        }
      }
      if (norm.ssq_out != nullptr) {                    // the 16 rows of a token lie in 16 consecutive lanes
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (row == 0 && tok < M) norm.ssq_out[(size_t)tok * ((gridDim.x + 3) & ~3) + blockIdx.x] = sq;
      }
    } else if (valid) {
      out[(size_t)tok * N + n] = from_f32<OUT>(v);
    }
  }
}

// CTAs of 16 rows, or more of fewer rows where those would fill the SMs unevenly (two CTAs share an SM).  Between one
// and two CTAs an SM: the next multiple of the SM count (N = 3584: 296 CTAs of 12 or 13 rows for 224 of 16).  Beyond two
// an SM the fixed cost of more CTAs outweighs an uneven last wave unless the rows are long (measured at 8 tokens,
// N = 5120: K = 5120 13.5 us with 320 CTAs, 14.5 with 592; K = 27648 61.4 against 50.4).
static int ws_ctas(int N, int K, bool rope) {
  const int num_sms = sllm::num_sms();
  int ctas = (N + 15) / 16;
  if (rope || ctas <= num_sms) return ctas;
  int even = ctas;
  if (ctas < 2 * num_sms) even = (ctas + num_sms - 1) / num_sms * num_sms;
  else if (K > 8192) even = (ctas + 2 * num_sms - 1) / (2 * num_sms) * (2 * num_sms);
  return even <= N ? even : ctas;
}

template <int NT, int EPI, typename OUT>
static int launch_ws(const __nv_bfloat16* x, const __nv_bfloat16* W, const float* bias, void* out, float* residual,
                     int M, int N, int K, cudaStream_t stream, const WsRope& rope = WsRope{}, const WsNorm& norm = WsNorm{}) {
  const int ctas = ws_ctas(N, K, EPI == WS_EPI_ROPE);
  if (norm.ssq_in != nullptr)
    launch_kernel(linear_ws_kernel<NT, EPI, OUT, true>, ctas, WS_WARPS * 32, 0, stream, x, W, bias, (OUT*)out, residual, M, N, K, rope, norm);
  else
    launch_kernel(linear_ws_kernel<NT, EPI, OUT, false>, ctas, WS_WARPS * 32, 0, stream, x, W, bias, (OUT*)out, residual, M, N, K, rope, norm);
  return launch_status("linear_ws");
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_linear_ws_supports(int M, int N, int K) {
  return M >= 1 && M <= 32 && N >= 16 && K >= 32 && K % 32 == 0;
}

// CTAs a launch for N output columns over a reduction of K uses: the rows of the table of partial sums of squares
// that the residual epilogue writes when it is asked for the next norm's input (see WsNorm).
SLLM_EXPORT int sllm_linear_ws_parts(int N, int K) { return ws_ctas(N, K, false); }

static bool ws_norm_in(WsNorm& n, const float* ssq_in, int parts_in, float eps_in, int width_in, int M) {
  if (ssq_in == nullptr) return true;
  if (parts_in < 1 || parts_in > ws_ssq_max(M <= 16 ? 2 : 4) || width_in < 1 || ((uintptr_t)ssq_in & 15) != 0) return false;
  n.ssq_in = ssq_in; n.parts_in = parts_in; n.eps_in = eps_in; n.inv_width_in = 1.0f / (float)width_in;
  return true;
}

// residual != null: residual[M, N] (float32) += x W^T (+ bias) and `out` is ignored;
// else out[M, N] = x W^T (+ bias) in out_dtype.
// ssq_in != null: x is bfloat16(stream * gain) of a norm still owed and ssq_in [M][parts_in rounded up to 4] holds partial sums of
// squares of the stream's rows (width_in wide): each row of the product is multiplied by rsqrt(sum / width_in + eps_in).
// gain != null (residual epilogue only): also write xg_out [M, N] = bfloat16(residual * gain) and
// ssq_out [M][sllm_linear_ws_parts(N, K) rounded up to 4], the next norm's input in the same form.
SLLM_EXPORT int sllm_linear_ws(const void* x, const void* W, const float* bias, void* out, int out_dtype, float* residual,
                               int M, int N, int K, const float* ssq_in, int parts_in, float eps_in, int width_in,
                               const float* gain, void* xg_out, float* ssq_out, cudaStream_t stream) {
  SLLM_REQUIRE(sllm_linear_ws_supports(M, N, K), "linear_ws: sizes M=%d N=%d K=%d (needs M<=32, K%%32==0)", M, N, K);
  SLLM_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)W & 15) == 0, "linear_ws: operands must be 16-byte aligned");
  SLLM_REQUIRE(residual != nullptr || out != nullptr, "linear_ws: no destination");
  WsNorm nm;
  SLLM_REQUIRE(ws_norm_in(nm, ssq_in, parts_in, eps_in, width_in, M), "linear_ws: a table of %d partial sums (at most %d) over width %d",
               parts_in, ws_ssq_max(M <= 16 ? 2 : 4), width_in);
  if (gain != nullptr) {
    SLLM_REQUIRE(residual != nullptr && xg_out != nullptr && ssq_out != nullptr, "linear_ws: the next norm's input needs the residual epilogue and both destinations");
    nm.gain = gain; nm.xg_out = (__nv_bfloat16*)xg_out; nm.ssq_out = ssq_out;
  }
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  const __nv_bfloat16* wb = (const __nv_bfloat16*)W;
#define GO(NT_)                                                                                                        \
  if (residual) return launch_ws<NT_, WS_EPI_RESID, float>(xb, wb, bias, nullptr, residual, M, N, K, stream, WsRope{}, nm);          \
  if (out_dtype == SLLM_BF16) return launch_ws<NT_, WS_EPI_STORE, __nv_bfloat16>(xb, wb, bias, out, nullptr, M, N, K, stream, WsRope{}, nm); \
  return launch_ws<NT_, WS_EPI_STORE, float>(xb, wb, bias, out, nullptr, M, N, K, stream, WsRope{}, nm);
  if (M <= 8) { GO(1) }
  if (M <= 16) { GO(2) }
  GO(4)
#undef GO
}

SLLM_EXPORT int sllm_linear_ws_rope_supports(int M, int N, int K, int nq, int nkv, int hd, int rot) {
  return sllm_linear_ws_supports(M, N, K) && nq > 0 && nkv > 0 && hd >= 16 && hd % 16 == 0 && N == (nq + 2 * nkv) * hd &&
         (rot == 0 || rot == hd);
}

// The fused q|k|v product of an attention layer with its bias, rotary encoding and cache write:
// x [M, K] and W [(nq + 2 nkv) * hd, K] bfloat16; table null or rot == 0: no rotation, else rot == hd and
// table [max_pos][2][hd/2] float32; slot_mapping null: keys and values are not written.  ssq_in: as for sllm_linear_ws.
SLLM_EXPORT int sllm_linear_ws_rope(const void* x, const void* W, const float* bias, int M, int N, int K, const int* positions,
                                    const float* table, int rot, int max_pos, int nq, int nkv, int hd, const int* slot_mapping,
                                    int page_size, int num_pages, void* k_cache, void* v_cache, void* q_out,
                                    const float* ssq_in, int parts_in, float eps_in, int width_in, cudaStream_t stream) {
  SLLM_REQUIRE(sllm_linear_ws_rope_supports(M, N, K, nq, nkv, hd, rot),
               "linear_ws_rope: sizes M=%d N=%d K=%d nq=%d nkv=%d hd=%d rot=%d", M, N, K, nq, nkv, hd, rot);
  SLLM_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)W & 15) == 0, "linear_ws_rope: operands must be 16-byte aligned");
  SLLM_REQUIRE(q_out != nullptr && (rot == 0 || (table != nullptr && positions != nullptr && max_pos > 0)),
               "linear_ws_rope: destination or rotary table missing");
  SLLM_REQUIRE(slot_mapping == nullptr || (k_cache && v_cache && page_size > 0 && num_pages > 0), "linear_ws_rope: cache arguments missing");
  WsNorm nm;
  SLLM_REQUIRE(ws_norm_in(nm, ssq_in, parts_in, eps_in, width_in, M), "linear_ws_rope: a table of %d partial sums (at most %d) over width %d",
               parts_in, ws_ssq_max(M <= 16 ? 2 : 4), width_in);
  WsRope r;
  r.positions = positions; r.table = rot > 0 ? table : nullptr; r.slot_mapping = slot_mapping;
  r.k_cache = (__nv_bfloat16*)k_cache; r.v_cache = (__nv_bfloat16*)v_cache; r.q_out = (__nv_bfloat16*)q_out;
  r.max_pos = max_pos; r.nq = nq; r.nkv = nkv; r.hd = hd; r.page_size = page_size; r.num_pages = num_pages;
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  const __nv_bfloat16* wb = (const __nv_bfloat16*)W;
  if (M <= 8) return launch_ws<1, WS_EPI_ROPE, __nv_bfloat16>(xb, wb, bias, nullptr, nullptr, M, N, K, stream, r, nm);
  if (M <= 16) return launch_ws<2, WS_EPI_ROPE, __nv_bfloat16>(xb, wb, bias, nullptr, nullptr, M, N, K, stream, r, nm);
  return launch_ws<4, WS_EPI_ROPE, __nv_bfloat16>(xb, wb, bias, nullptr, nullptr, M, N, K, stream, r, nm);
}
