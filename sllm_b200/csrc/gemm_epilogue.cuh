// What the tcgen05 products do with a chunk of 32 accumulator columns of one row as it leaves tensor
// memory: bias and a float32 or bfloat16 store, or SiLU(gate) * up for a gate|up matrix whose rows alternate
// in blocks of 8.  Shared by the one-CTA and the CTA-pair form of the product.
#pragma once

#include "tcgen05.cuh"

namespace sllm {

#define TG_EPI_F32 0
#define TG_EPI_BF16 1
#define TG_EPI_SILU 2
#define TG_EPI_RESID 3     // residual[M, N] (float32) += the product (+ bias), in place; see TgExtra

// What an epilogue may do beyond its store, for the RMSNorm that a prompt portion's products take apart
// (y = x * rsqrt(mean(x^2) + eps) * gain, ref/standard.py:25-31; the same scheme as linear_ws.cu's WsNorm):
//   consumer side (any epilogue): the product's input was bfloat16(stream * gain) with the division still owed;
//     ssq_in [M][stride_in] holds parts_in partial sums of squares of each row of the stream, and each row of the
//     product is multiplied by rsqrt(sum / width + eps) before bias and activation;
//   producer side (TG_EPI_RESID): after residual += product, also write xg [M, N] = bfloat16(residual * gain) and,
//     per row and block of 128 columns, the sum of squares of the new residual: ssq_out [M][stride_out], entry
//     column / 128.  gain null: the residual update alone.
struct TgExtra {
  const float* ssq_in = nullptr;
  int parts_in = 0, stride_in = 0;
  float eps_in = 0.f, inv_width_in = 0.f;
  float* residual = nullptr;
  const float* gain = nullptr;
  __nv_bfloat16* xg = nullptr;
  float* ssq_out = nullptr;
  int stride_out = 0;
};

// the factor of row m (1 where nothing is owed); the partial sums are added in index order
__device__ __forceinline__ float tg_row_scale(const TgExtra& e, int m, int M) {
  if (e.ssq_in == nullptr || m >= M) return 1.f;
  const float* row = e.ssq_in + (size_t)m * e.stride_in;
  float sum = 0.f;
  for (int p = 0; p < e.parts_in; ++p) sum += row[p];
  return rsqrtf(sum * e.inv_width_in + e.eps_in);
}
__device__ __forceinline__ void tg_scale(uint32_t (&r)[32], float s) {
#pragma unroll
  for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * s);
}

// The epilogue warps run one to a scheduler with nothing to hide a dependent instruction behind, so what they
// do per value counts: the bias is fetched in 16-byte pieces and only where there is one, the bounds are
// tested per chunk, and SiLU uses the fast exponential and reciprocal (the result is rounded to bfloat16).
__device__ __forceinline__ void tg_values(const uint32_t (&r)[32], float (&v)[32], int n, int N, const float* __restrict__ bias) {
  if (bias == nullptr) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
  } else if (n + 32 <= N && (reinterpret_cast<uintptr_t>(bias) & 15) == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 b = __ldg(reinterpret_cast<const float4*>(bias + n) + j);
      v[4 * j] = __uint_as_float(r[4 * j]) + b.x;
      v[4 * j + 1] = __uint_as_float(r[4 * j + 1]) + b.y;
      v[4 * j + 2] = __uint_as_float(r[4 * j + 2]) + b.z;
      v[4 * j + 3] = __uint_as_float(r[4 * j + 3]) + b.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) + (n + i < N ? bias[n + i] : 0.f);
  }
}
__device__ __forceinline__ float tg_silu_mul(float g, float u) {
  // silu(g) * u = g * u / (1 + e^-g) (ref/qwen3_5.py:28-29)
  return __fdividef(g * u, 1.0f + __expf(-g));
}

// r: columns n .. n + 31 of row m of C = A W^T (float32 bits); out is [M, N] (or [M, N/2] for the SiLU form)
template <int EPI>
__device__ __forceinline__ void tg_store_chunk(const uint32_t (&r)[32], int m, int n, int N, const float* __restrict__ bias,
                                               void* __restrict__ out) {
  if constexpr (EPI == TG_EPI_SILU) {
    // columns alternate 8 gate, 8 up; out[m, (n/16)*8 + i] = silu(gate_i) * up_i
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)m * (N >> 1) + (n >> 1);
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      if (n + blk * 16 + 15 >= N) break;
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i] = tg_silu_mul(__uint_as_float(r[blk * 16 + i]), __uint_as_float(r[blk * 16 + 8 + i]));
      }
      if (((N >> 1) & 7) == 0) {               // rows of the result are 16-byte aligned
        *reinterpret_cast<uint4*>(o + blk * 8) = make_uint4(pack2(v[0], v[1]), pack2(v[2], v[3]), pack2(v[4], v[5]), pack2(v[6], v[7]));
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) o[blk * 8 + i] = __float2bfloat16_rn(v[i]);
      }
    }
  } else {
    float v[32];
    tg_values(r, v, n, N, bias);
    const bool whole = n + 32 <= N;
    if constexpr (EPI == TG_EPI_F32) {
      float* o = reinterpret_cast<float*>(out) + (size_t)m * N + n;
      if (whole && (N & 3) == 0) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) if (n + i < N) o[i] = v[i];
      }
    } else {
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)m * N + n;
      if (whole && (N & 7) == 0) {
#pragma unroll
        for (int i = 0; i < 32; i += 8)
          *reinterpret_cast<uint4*>(o + i) = make_uint4(pack2(v[i], v[i + 1]), pack2(v[i + 2], v[i + 3]),
                                                        pack2(v[i + 4], v[i + 5]), pack2(v[i + 6], v[i + 7]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) if (n + i < N) o[i] = __float2bfloat16_rn(v[i]);
      }
    }
  }
}

// ---- the same through shared memory and TMA stores ------------------------------------------------
// A lane of an epilogue warp holds one row of the accumulator, so direct stores put every lane on a line of
// its own: 32 requests of 16 bytes an instruction, and the step from tensor memory to global memory takes
// longer than the products it should hide behind.  Here the warp stages a box of 32 rows x 128 bytes of the
// result in shared memory (128-byte swizzle: the 16-byte piece j of row r lies at piece j ^ (r & 7)) and one
// lane hands it to the TMA unit, which writes whole lines and clips what lies outside the matrix.
// A box is 32 float32, 64 bfloat16 or (SiLU form) 128 accumulator columns wide.
template <int EPI> struct TgBox {
  static constexpr int ACC_COLS = (EPI == TG_EPI_F32 || EPI == TG_EPI_RESID) ? 32 : (EPI == TG_EPI_BF16 ? 64 : 128);   // accumulator columns a box covers
  static constexpr int ELEM = (EPI == TG_EPI_F32 || EPI == TG_EPI_RESID) ? 4 : 2;
};

__device__ __forceinline__ void tg_put_piece(unsigned char* row_base, int row, int piece, uint4 v) {
  *reinterpret_cast<uint4*>(row_base + ((piece ^ (row & 7)) << 4)) = v;
}

// the 32 accumulator columns `sub` (0 ..) of a box, of this lane's row, into the staged box; n is the result
// column (of C) of the chunk's first accumulator column, for the bias
template <int EPI>
__device__ __forceinline__ void tg_stage_chunk(const uint32_t (&r)[32], unsigned char* stage, int row, int sub, int n, int N,
                                               const float* __restrict__ bias) {
  unsigned char* row_base = stage + row * 128;
  if constexpr (EPI == TG_EPI_SILU) {
    // 32 columns: 8 gate, 8 up, 8 gate, 8 up -> 16 results = 2 pieces; a box holds 4 such chunks
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = tg_silu_mul(__uint_as_float(r[blk * 16 + i]), __uint_as_float(r[blk * 16 + 8 + i]));
      tg_put_piece(row_base, row, sub * 2 + blk, make_uint4(pack2(v[0], v[1]), pack2(v[2], v[3]), pack2(v[4], v[5]), pack2(v[6], v[7])));
    }
  } else {
    float v[32];
    tg_values(r, v, n, N, bias);
    if constexpr (EPI == TG_EPI_F32) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        tg_put_piece(row_base, row, j, make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]),
                                                  __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3])));
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        tg_put_piece(row_base, row, sub * 4 + j, make_uint4(pack2(v[8 * j], v[8 * j + 1]), pack2(v[8 * j + 2], v[8 * j + 3]),
                                                            pack2(v[8 * j + 4], v[8 * j + 5]), pack2(v[8 * j + 6], v[8 * j + 7])));
    }
  }
}

// ---- the residual epilogue through shared memory -----------------------------------------------------
// TG_EPI_RESID with a lane a row puts every lane's 16-byte pieces on a line of their own: per 128 x 512 tile of a
// CTA, 640 KB of the residual stream and of the next norm's input move as 40,000 single-line requests, about 20 us
// of the load/store unit where the products of the tile take 45.  Here a warp stages its 32 rows x 32 columns of the
// product in a box of shared memory (the layout of the boxes above) and walks it four rows at a time, eight lanes a
// row: the residual stream is read and written, and the next norm's input written, as whole lines.
// m0: the box's first row of C; n: its first column (N a multiple of 4: a 16-byte piece lies inside the matrix or
// outside).  sq[k] gathers, in the lanes 8 j of a warp, the sums of squares of the new residual values of the
// rows m0 + 4 k + j.
__device__ __forceinline__ void tg_resid_box(const uint32_t (&r)[32], unsigned char* box, int lane, int m0, int n, int M, int N,
                                             const float* __restrict__ bias, const TgExtra& e, float (&sq)[8]) {
  {
    float v[32];
    tg_values(r, v, n, N, bias);
    unsigned char* row_base = box + lane * 128;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      tg_put_piece(row_base, lane, j, make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]),
                                                 __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3])));
  }
  __syncwarp();
  const int piece = lane & 7, col = n + 4 * piece;
  const bool col_ok = col < N;
  float4 gain = make_float4(0.f, 0.f, 0.f, 0.f);
  if (e.xg != nullptr && col_ok) gain = *reinterpret_cast<const float4*>(e.gain + col);
  // all the loads first: eight lines of the residual stream in flight per lane group
  float4 old[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int m = m0 + 4 * k + (lane >> 3);
    old[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (m < M && col_ok) old[k] = *reinterpret_cast<const float4*>(e.residual + (size_t)m * N + col);
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int row = 4 * k + (lane >> 3), m = m0 + row;
    const float4 v = *reinterpret_cast<const float4*>(box + row * 128 + ((piece ^ (row & 7)) << 4));
    float s = 0.f;
    if (m < M && col_ok) {
      const float4 x = make_float4(old[k].x + v.x, old[k].y + v.y, old[k].z + v.z, old[k].w + v.w);
      *reinterpret_cast<float4*>(e.residual + (size_t)m * N + col) = x;
      if (e.xg != nullptr) {
        s = x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        *reinterpret_cast<uint2*>(e.xg + (size_t)m * N + col) = make_uint2(pack2(x.x * gain.x, x.y * gain.y), pack2(x.z * gain.z, x.w * gain.w));
      }
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    sq[k] += s;
  }
  __syncwarp();                                   // the box is free for the next chunk
}

// The float32 result the same way: rows m0 .. m0 + 31, columns n .. n + 31 of `out` [M, N] (N a multiple of 4),
// staged in the warp's box and written four rows an instruction.
__device__ __forceinline__ void tg_store_box_f32(const uint32_t (&r)[32], unsigned char* box, int lane, int m0, int n, int M, int N,
                                                 const float* __restrict__ bias, float* __restrict__ out) {
  {
    float v[32];
    tg_values(r, v, n, N, bias);
    unsigned char* row_base = box + lane * 128;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      tg_put_piece(row_base, lane, j, make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]),
                                                 __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3])));
  }
  __syncwarp();
  const int piece = lane & 7, col = n + 4 * piece;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int row = 4 * k + (lane >> 3), m = m0 + row;
    if (m < M && col < N)
      *reinterpret_cast<float4*>(out + (size_t)m * N + col) = *reinterpret_cast<const float4*>(box + row * 128 + ((piece ^ (row & 7)) << 4));
  }
  __syncwarp();                                   // the box is free for the next chunk
}

// the sums of squares gathered by tg_resid_box over a block of 128 columns, into ssq_out[row][block]
__device__ __forceinline__ void tg_resid_box_sums(float (&sq)[8], int lane, int m0, int M, int block, const TgExtra& e) {
  if (e.ssq_out != nullptr && (lane & 7) == 0) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int m = m0 + 4 * k + (lane >> 3);
      if (m < M) e.ssq_out[(size_t)m * e.stride_out + block] = sq[k];
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) sq[k] = 0.f;
}

}  // namespace sllm
