// Attention over the paged cache on the CUDA cores, all arithmetic in float32:
// the kernel of the float32 path, and the one that takes head sizes and dtypes the
// tensor-core kernel refuses.  One block per (token, query head): prompt portions and
// single decoded tokens are the same work, so a position's result cannot depend on
// how the batch was cut.
//
//   s_j = (q . k_j) * scale for keys j <= pos (and j > pos - window), softmax with the
//   maximum subtracted, o = sum p_j v_j   (ref/qwen3_5.py:373-390; one row:
//   ref/incremental.py:75-87; kernels/cuda/kernels.cu:957-1025 for one CTA per head).
//   Query head h reads kv head h / (nq / nkv) (ref/standard.py:65-68).
//
// Each of the block's warps takes keys w, w+W, w+2W, ... in ascending order with an
// online softmax; the warps' partial results are merged in warp order.  The order
// depends on the position alone.
#include <math.h>
#include <stdio.h>

#include "common.cuh"

namespace sllm {

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_HD = 256;

template <typename TQ, typename TC>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_simt_kernel(const TQ* __restrict__ q, const TC* __restrict__ k_cache, const TC* __restrict__ v_cache,
                      const int* __restrict__ block_tables, int max_pages, const int* __restrict__ positions,
                      const int* __restrict__ seq_of_token, int nq, int nkv, int hd, int page_size, float scale,
                      int window, TQ* __restrict__ out) {
  __shared__ float qs[ATT_MAX_HD];
  __shared__ float acc_s[ATT_WARPS][ATT_MAX_HD];
  __shared__ float m_s[ATT_WARPS], l_s[ATT_WARPS];
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int kvh = h / (nq / nkv);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = positions[t];
  const int* bt = block_tables + (size_t)seq_of_token[t] * max_pages;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  for (int d = threadIdx.x; d < hd; d += blockDim.x) qs[d] = to_f32(q[((size_t)t * nq + h) * hd + d]);
  __syncthreads();

  float acc[ATT_MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < ATT_MAX_HD / 32; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int j = lo + warp; j <= pos; j += ATT_WARPS) {
    const int page = bt[j / page_size];
    if (page < 0) continue;                          // never dereference a page that was given back
    const size_t row = (((size_t)page * nkv + kvh) * page_size + (j % page_size)) * hd;
    float dot = 0.f;
    for (int d = lane; d < hd; d += 32) dot = fmaf(qs[d], to_f32(k_cache[row + d]), dot);
    dot = warp_sum(dot);
    const float s = dot * scale;
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);              // exp(-inf) = 0 on the first key
    const float p = expf(s - m_new);
    l = l * corr + p;
#pragma unroll
    for (int i = 0; i < ATT_MAX_HD / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) acc[i] = acc[i] * corr + p * to_f32(v_cache[row + d]);
    }
    m = m_new;
  }
  if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
  for (int i = 0; i < ATT_MAX_HD / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) acc_s[warp][d] = acc[i];
  }
  __syncthreads();
  float mm = -INFINITY;
#pragma unroll
  for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, m_s[w]);
  float ll = 0.f;
  float f[ATT_WARPS];
#pragma unroll
  for (int w = 0; w < ATT_WARPS; ++w) {
    f[w] = l_s[w] > 0.f ? expf(m_s[w] - mm) : 0.f;
    ll += l_s[w] * f[w];
  }
  const float inv = ll > 0.f ? 1.0f / ll : 0.f;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) o += acc_s[w][d] * f[w];
    out[((size_t)t * nq + h) * hd + d] = from_f32<TQ>(o * inv);
  }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_attention_simt(const void* q, const void* k_cache, const void* v_cache, int dtype,
                                    const int* block_tables, int max_pages, const int* positions,
                                    const int* seq_of_token, int T, int nq, int nkv, int hd, int page_size,
                                    float scale, int window, void* out, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention: bad head counts nq=%d nkv=%d", nq, nkv);
  SLLM_REQUIRE(hd > 0 && hd <= ATT_MAX_HD, "attention: head_dim=%d is outside 1..%d", hd, ATT_MAX_HD);
  SLLM_REQUIRE(page_size > 0 && max_pages > 0, "attention: bad page_size=%d max_pages=%d", page_size, max_pages);
  SLLM_REQUIRE(nq <= 65535, "attention: %d query heads exceed one launch", nq);
  if (T == 0) return SLLM_OK;
  dim3 grid(T, nq);
  if (dtype == SLLM_F32)
    launch_kernel(attention_simt_kernel<float, float>, grid, ATT_WARPS * 32, 0, stream,
        (const float*)q, (const float*)k_cache, (const float*)v_cache, block_tables, max_pages, positions,
        seq_of_token, nq, nkv, hd, page_size, scale, window, (float*)out);
  else if (dtype == SLLM_BF16)
    launch_kernel(attention_simt_kernel<__nv_bfloat16, __nv_bfloat16>, grid, ATT_WARPS * 32, 0, stream,
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_tables,
        max_pages, positions, seq_of_token, nq, nkv, hd, page_size, scale, window, (__nv_bfloat16*)out);
  else
    SLLM_REQUIRE(false, "attention: unknown dtype %d", dtype);
  return launch_status("attention_simt");
}
