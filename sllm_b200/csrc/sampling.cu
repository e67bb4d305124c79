// Sampling on the device: greedy argmax and temperature sampling by inverse CDF over
// float32 logits [R, V], one block per row.
//
// greedy: the first maximum (runtime/sampler.py:8-9).
// temperature: p = softmax(logits / T) with the maximum subtracted; the token is the
// first index whose cumulative probability reaches the uniform u, clamped to V-1
// (runtime/sampler.py:54-58, 81-88); temperature <= 0 is greedy (runtime/sampler.py:50-53).
// The host draws u, one per sampled token, from the request's own generator.
// Sums are kept in float64 as the reference's sampler works in float64.
#include <math.h>
#include <stdio.h>

#include "common.cuh"

namespace sllm {

constexpr int SAMPLE_THREADS = 1024;

struct MaxIdx {
  float v;
  int i;
};
__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ MaxIdx block_argmax(const float* __restrict__ row, int V, MaxIdx* sh) {
  MaxIdx best{-INFINITY, 0x7fffffff};
  if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    // four values a load, four loads in flight; a thread's indices still ascend
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int n4 = V >> 2;
#pragma unroll 4
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 v = row4[i];
      if (v.x > best.v) best = MaxIdx{v.x, 4 * i};
      if (v.y > best.v) best = MaxIdx{v.y, 4 * i + 1};
      if (v.z > best.v) best = MaxIdx{v.z, 4 * i + 2};
      if (v.w > best.v) best = MaxIdx{v.w, 4 * i + 3};
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = row[i];
      if (v > best.v) best = MaxIdx{v, i};           // strict >: the first maximum wins
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = best;
  __syncthreads();
  if (warp == 0) {
    MaxIdx b = lane < (blockDim.x >> 5) ? sh[lane] : MaxIdx{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MaxIdx other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
      b = better(b, other);
    }
    if (lane == 0) sh[0] = b;
  }
  __syncthreads();
  MaxIdx r = sh[0];
  __syncthreads();
  if (r.i == 0x7fffffff) r.i = 0;
  return r;
}

__device__ double block_sum_f64(double v, double* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  if (warp == 0) {
    double t = lane < (blockDim.x >> 5) ? sh[lane] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) sh[32] = t;
  }
  __syncthreads();
  const double r = sh[32];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                   const double* __restrict__ uniform, int* __restrict__ out) {
  __shared__ MaxIdx sh_mi[32];
  __shared__ double sh_d[33];
  __shared__ double warp_tot[32];
  __shared__ int found;
  pdl_launch_dependents();       // a short kernel: the successor may be set up behind it
  pdl_wait();
  const float* row = logits + (size_t)blockIdx.x * V;
  const MaxIdx mx = block_argmax(row, V, sh_mi);
  const float temp = temperature ? temperature[blockIdx.x] : 0.f;
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) out[blockIdx.x] = mx.i;
    return;
  }
  const double inv_t = 1.0 / (double)temp;
  const double top = (double)mx.v * inv_t;
  double part = 0.0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) part += exp((double)row[i] * inv_t - top);
  const double total = block_sum_f64(part, sh_d);
  const double target = uniform[blockIdx.x] * total;
  // walk the row in index order, blockDim elements at a time, with a running prefix
  if (threadIdx.x == 0) found = 0x7fffffff;
  __syncthreads();
  double running = 0.0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int base = 0; base < V; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const double p = i < V ? exp((double)row[i] * inv_t - top) : 0.0;
    double incl = p;                                  // inclusive scan within the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    double before = running;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    const double cum = before + incl;
    if (i < V && cum >= target) atomicMin(&found, i);  // the lowest such index is the first
    double chunk = 0.0;
    for (int w = 0; w < nw; ++w) chunk += warp_tot[w];
    running += chunk;
    __syncthreads();
    if (found != 0x7fffffff) break;
  }
  if (threadIdx.x == 0) {
    int r = found;
    if (r < 0 || r >= V) r = V - 1;                    // u beyond the last cumulative value: clamp
    out[blockIdx.x] = r;
  }
}

}  // namespace sllm

using namespace sllm;

// temperature may be null (all rows greedy); uniform must hold R doubles when any temperature > 0.
SLLM_EXPORT int sllm_sample_rows(const float* logits, int R, int V, const float* temperature,
                                 const double* uniform, int* out, cudaStream_t stream) {
  SLLM_REQUIRE(R >= 0 && V > 0, "sample_rows: bad sizes R=%d V=%d", R, V);
  SLLM_REQUIRE(temperature == nullptr || uniform != nullptr, "sample_rows: temperatures without uniforms");
  if (R == 0) return SLLM_OK;
  launch_kernel(sample_rows_kernel, R, SAMPLE_THREADS, 0, stream, logits, V, temperature, uniform, out);
  return launch_status("sample_rows");
}
