// Shared helpers of the sm_100a kernels: dtype codes, conversions, launch checks.
// Every exported entry point is extern "C", takes raw device pointers and the
// stream to launch on, validates its arguments on the host and returns 0 or an
// error code (see sllm_error_string); nothing here traps on the device.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define SLLM_OK 0
#define SLLM_ERR_ARG 1        // a size, pointer or dtype the kernel refuses
#define SLLM_ERR_LAUNCH 2     // the launch itself failed (see cudaGetLastError text)
#define SLLM_ERR_UNSUPPORTED 3

#define SLLM_F32 0
#define SLLM_BF16 1

#define SLLM_EXPORT extern "C" __attribute__((visibility("default")))

namespace sllm {

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);   // round to nearest even, as the reference's to_bf16 does
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block in a fixed order (depends only on blockDim), result in all threads.
__device__ __forceinline__ float block_sum(float v, float* red /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

void set_error(const char* msg);   // remembers the text for sllm_last_error()

// ---- programmatic dependent launch ------------------------------------------------------------
// A decode step is a train of short kernels.  Every kernel of this library is launched with the
// programmatic-stream-serialization attribute: it may be scheduled while its predecessor in the
// stream is still running, does what does not depend on that predecessor (its own index
// arithmetic, the first loads of weights or tables), and then blocks in pdl_wait() until the
// predecessor has completed and its writes are visible.  Every kernel calls pdl_wait() before
// it reads or writes anything another kernel of the step touches, and before it exits, so
// completion stays transitive along the stream.  When a kernel releases its successor matters:
// the short kernels (norm, rotary, gather, embedding, combine, sampling) release it at their very
// top, which hides the successor's launch behind them; the long ones (the streaming linear layers,
// attention) only after their main loop, because a successor that is resident while a long kernel
// streams takes issue slots from it.  Measured on the 7B decode step (batch 8, context 4096, CUDA
// graph): 3.24 ms so; 3.29 ms with no early release in the short kernels; 6.05 ms with the release
// at the top of every kernel; 3.33 ms with SLLM_PDL=0 in the environment (the attribute off, plain
// stream order).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool pdl_enabled();
int num_sms();           // streaming multiprocessors of the current device (asked once per device)

template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // errors are read by launch_status()
}

inline int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    char buf[256];
    snprintf(buf, sizeof buf, "%s: launch failed: %s", what, cudaGetErrorString(e));
    set_error(buf);
    return SLLM_ERR_LAUNCH;
  }
  return SLLM_OK;
}

#define SLLM_REQUIRE(cond, ...)                         \
  do {                                                  \
    if (!(cond)) {                                      \
      char _b[256];                                     \
      snprintf(_b, sizeof _b, __VA_ARGS__);             \
      sllm::set_error(_b);                              \
      return SLLM_ERR_ARG;                              \
    }                                                   \
  } while (0)

}  // namespace sllm
