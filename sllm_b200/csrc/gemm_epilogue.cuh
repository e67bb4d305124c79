// What the tcgen05 products do with a chunk of 32 accumulator columns of one row as it leaves tensor
// memory: bias and a float32 or bfloat16 store, or SiLU(gate) * up for a gate|up matrix whose rows alternate
// in blocks of 8.  Shared by the one-CTA and the CTA-pair form of the product.
#pragma once

#include "tcgen05.cuh"

namespace sllm {

#define TG_EPI_F32 0
#define TG_EPI_BF16 1
#define TG_EPI_SILU 2

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
        const float g = __uint_as_float(r[blk * 16 + i]), u = __uint_as_float(r[blk * 16 + 8 + i]);
        v[i] = g * (1.0f / (1.0f + expf(-g))) * u;
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
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) + ((bias && n + i < N) ? bias[n + i] : 0.f);
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

}  // namespace sllm
