// Weight-streaming linear layer for few tokens (decoding): y[M, N] = x[M, K] W[N, K]^T with
// M <= 64, bfloat16 operands, float32 accumulation.  At these sizes the product is bound by
// reading W once from HBM, so the kernel is built around that stream:
//
//  * W is the M-side operand of mma.sync m16n8k16 (16 weight rows per warp), the tokens are
//    the N side (8 tokens per MMA), so no tensor-core work is wasted on padding tokens to 16+.
//  * Each thread reads its share of W straight from global memory into the MMA's A-fragment
//    registers with 16-byte loads, two chunks ahead of the math.  Within a 32-wide k block a
//    thread takes 8 consecutive k of two rows; the k order inside the block is permuted
//    identically for W and x (a dot product does not care), so no shuffle or shared-memory
//    staging of W is needed.
//  * The tokens' activations are staged per 128-wide k chunk in shared memory (double
//    buffered with cp.async) and shared by the CTA's 8 warps (128 weight rows).
//  * Small N (the attention and down projections) would leave most SMs idle, so the grid
//    also splits K; the partial sums go to scratch [splits, M, N] and the consumer (the
//    residual add + RMSNorm kernel, or the rotary kernel) adds them in a fixed order.
//  * Epilogues: bias; SiLU(gate)*up for a gate|up matrix whose rows alternate in blocks of 8
//    (rows g and g+8 of a warp's tile are a gate row and its up row, held by one thread).
//
// The reference's device path calls cublasGemmEx for these products
// (kernels/cuda/kernels.cu:752-767; kernels/device_decode.py:294-326) and applies SiLU*up
// in a kernel of its own (kernels.cu:898-919).
#include <stdio.h>

#include "common.cuh"

namespace sllm {

constexpr int LS_KC = 128;                 // k per chunk
constexpr int LS_ROWS = 128;               // weight rows per CTA (8 warps x 16)
constexpr int LS_XSTRIDE = LS_KC + 32;     // bf16 elements: 320 bytes, = 64 mod 128 -> conflict-free 16-byte reads

#define EPI_STORE 0
#define EPI_SILU 1

constexpr int LS_SSQ_MAX = 608;            // partial sums of squares per token a scaled launch takes (as in linear_ws.cu)

// A norm still owed on the input (see linear_ws.cu, WsNorm): x is bfloat16(stream * gain), ssq [M][stride]
// (stride = parts rounded up to 4) holds partial sums of squares of the stream's rows, and every row of the
// product is multiplied by rsqrt(sum / width + eps) before the epilogue's arithmetic.
struct LsScale {
  const float* ssq = nullptr;
  int parts = 0;
  float eps = 0.f, inv_width = 0.f;
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void ls_cp_async_16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void ls_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                       unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: 8-token tiles (M <= 8*NT).  OUT: float or __nv_bfloat16.  SCALED: the rows of the result are scaled
// (LsScale; unsplit launches only).
template <int NT, int EPI, typename OUT, bool SCALED>
__global__ void __launch_bounds__(256)
linear_stream_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W,
                     const float* __restrict__ bias, OUT* __restrict__ out, float* __restrict__ partial,
                     int M, int N, int K, int chunks_per_split, const LsScale scale) {
  extern __shared__ __align__(16) unsigned char ls_smem[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(ls_smem);          // [2][8*NT][LS_XSTRIDE]
  float* ssq_s = reinterpret_cast<float*>(ls_smem + sizeof(__nv_bfloat16) * 2 * 8 * NT * LS_XSTRIDE);   // SCALED: [8*NT][LS_SSQ_MAX]
  __shared__ float row_scale[8 * NT];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int n0 = blockIdx.x * LS_ROWS + warp * 16;
  const int split = blockIdx.y;
  const int total_chunks = K / LS_KC;
  const int c_begin = split * chunks_per_split;
  const int c_end = min(total_chunks, c_begin + chunks_per_split);
  const int n_chunks = max(c_end - c_begin, 0);

  // rows past N are clamped for the loads and skipped at the store
  const int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);
  const __nv_bfloat16* w0 = W + (size_t)r0 * K + (size_t)c_begin * LS_KC + t4 * 8;
  const __nv_bfloat16* w1 = W + (size_t)r1 * K + (size_t)c_begin * LS_KC + t4 * 8;

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;

  auto load_x = [&](int chunk, int buf) {
    // [8*NT tokens][128 k] -> 16 sixteen-byte pieces per token
    for (int c = tid; c < 8 * NT * (LS_KC / 8); c += 256) {
      const int tok = c / (LS_KC / 8), piece = c % (LS_KC / 8);
      const bool ok = tok < M;
      const __nv_bfloat16* src = x + (size_t)(ok ? tok : 0) * K + (size_t)(c_begin + chunk) * LS_KC + piece * 8;
      ls_cp_async_16(xs + ((size_t)buf * 8 * NT + tok) * LS_XSTRIDE + piece * 8, src, ok);
    }
  };
  auto load_w = [&](uint4 (&a)[8], int chunk) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      a[2 * b] = ldg_stream(w0 + (size_t)chunk * LS_KC + b * 32);
      a[2 * b + 1] = ldg_stream(w1 + (size_t)chunk * LS_KC + b * 32);
    }
  };
  auto compute = [&](const uint4 (&a)[8], int buf) {
    const __nv_bfloat16* xb = xs + (size_t)buf * 8 * NT * LS_XSTRIDE;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint4 ra = a[2 * b], rb = a[2 * b + 1];         // rows g and g+8: 8 consecutive k each
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xb + (size_t)(8 * j + g) * LS_XSTRIDE + b * 32 + t4 * 8);
        // first MMA: k slots (2t,2t+1) <- elements 0,1; slots (2t+8,2t+9) <- elements 2,3
        ls_mma(acc[j], ra.x, rb.x, ra.y, rb.y, xv.x, xv.y);
        // second MMA: elements 4,5 and 6,7
        ls_mma(acc[j], ra.z, rb.z, ra.w, rb.w, xv.z, xv.w);
      }
    }
  };

  uint4 wa[8], wb[8];
  // weights do not depend on the step's earlier kernels: start the stream (two chunks) now
  if (n_chunks > 0) load_w(wa, 0);
  if (n_chunks > 1) load_w(wb, 1);
  pdl_wait();                          // the activations do
  if (n_chunks > 0) load_x(0, 0);
  if constexpr (SCALED) {
    // the tokens' partial sums of squares come to shared memory with the first activations
    const int stride = (scale.parts + 3) & ~3, pieces = stride >> 2;
    for (int c = tid; c < M * pieces; c += 256) {
      const int tok = c / pieces, piece = c % pieces;
      ls_cp_async_16(ssq_s + (size_t)tok * LS_SSQ_MAX + piece * 4, scale.ssq + (size_t)tok * stride + piece * 4, true);
    }
  }
  asm volatile("cp.async.commit_group;\n" ::);
  for (int c = 0; c < n_chunks; c += 2) {
    // chunk c from wa, chunk c+1 from wb
    if (c + 1 < n_chunks) {
      load_x(c + 1, 1);
      if (c > 0) load_w(wb, c + 1);    // the first pair was fetched before the wait
    }
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 1;\n" ::);
    __syncthreads();
    compute(wa, 0);
    __syncthreads();
    if (c + 1 >= n_chunks) break;
    if (c + 2 < n_chunks) {
      load_x(c + 2, 0);
      load_w(wa, c + 2);
    }
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 1;\n" ::);
    __syncthreads();
    compute(wb, 1);
    __syncthreads();
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  pdl_launch_dependents();             // the stream is read; the next kernel may begin while the results are stored
  if constexpr (SCALED) {
    // warp w adds the partial sums of tokens w, w + 8, ...: lane l takes l, l + 32, ..., then the lanes are added
    // (the table has been visible to all since the loop's first barrier)
    for (int tok = warp; tok < 8 * NT; tok += 8) {
      float sum = 0.f;
      if (tok < M)
        for (int p = lane; p < scale.parts; p += 32) sum += ssq_s[(size_t)tok * LS_SSQ_MAX + p];
      sum = warp_sum(sum);
      if (lane == 0) row_scale[tok] = rsqrtf(sum * scale.inv_width + scale.eps);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[j][c] *= row_scale[8 * j + 2 * t4 + (c & 1)];
  }

  // ---- epilogue: acc[j][c]: c0,c1 = (row g, tokens 8j+2t, +1); c2,c3 = (row g+8, same tokens) ----
  const int row_a = n0 + g, row_b = n0 + g + 8;
  if (gridDim.y > 1) {
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int tok = 8 * j + 2 * t4 + (c & 1), row = (c & 2) ? row_b : row_a;
        if (tok < M && row < N)
          partial[((size_t)split * M + tok) * N + row] = acc[j][c] + ((bias && split == 0) ? bias[row] : 0.f);
      }
    return;
  }
  if constexpr (EPI == EPI_SILU) {
    // rows g (gate i) and g+8 (up i) of this 16-row tile; the output column is (n0/16)*8 + g
    const int col = (n0 >> 4) * 8 + g;
    const int I = N >> 1;
    if (row_b < N) {
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int tok = 8 * j + 2 * t4 + c;
          if (tok < M) {
            const float gate = acc[j][c], up = acc[j][c + 2];
            out[(size_t)tok * I + col] = from_f32<OUT>(gate * (1.0f / (1.0f + expf(-gate))) * up);
          }
        }
    }
  } else {
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int tok = 8 * j + 2 * t4 + (c & 1), row = (c & 2) ? row_b : row_a;
        if (tok < M && row < N) out[(size_t)tok * N + row] = from_f32<OUT>(acc[j][c] + (bias ? bias[row] : 0.f));
      }
  }
}

template <int NT, int EPI, typename OUT, bool SCALED = false>
static int launch_ls(const __nv_bfloat16* x, const __nv_bfloat16* W, const float* bias, void* out, float* partial,
                     int M, int N, int K, int splits, cudaStream_t stream, const LsScale& scale = LsScale{}) {
  constexpr size_t smem = sizeof(__nv_bfloat16) * 2 * 8 * NT * LS_XSTRIDE + (SCALED ? sizeof(float) * 8 * NT * LS_SSQ_MAX : 0);
  static bool configured = false;
  if (!configured && smem + 1024 > 48 * 1024) {      // (the kernel has a little static shared memory too)
    if (cudaFuncSetAttribute(linear_stream_kernel<NT, EPI, OUT, SCALED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      set_error("linear_stream: cannot raise the shared memory limit");
      return SLLM_ERR_LAUNCH;
    }
    configured = true;
  }
  const int total_chunks = K / LS_KC;
  const int per = (total_chunks + splits - 1) / splits;
  dim3 grid((N + LS_ROWS - 1) / LS_ROWS, (total_chunks + per - 1) / per);
  launch_kernel(linear_stream_kernel<NT, EPI, OUT, SCALED>, grid, 256, smem, stream, x, W, bias, (OUT*)out, partial, M, N, K, per, scale);
  return launch_status("linear_stream");
}

}  // namespace sllm

using namespace sllm;

// How many k-splits a launch with `splits_wanted` really uses (the scratch needs that many slices).
SLLM_EXPORT int sllm_linear_stream_splits(int K, int splits_wanted) {
  const int total_chunks = K / LS_KC;
  if (total_chunks <= 0) return 1;
  const int s = splits_wanted < 1 ? 1 : (splits_wanted > total_chunks ? total_chunks : splits_wanted);
  const int per = (total_chunks + s - 1) / s;
  return (total_chunks + per - 1) / per;
}

SLLM_EXPORT int sllm_linear_stream_supports(int M, int N, int K) {
  return M >= 1 && M <= 64 && N >= 16 && K >= LS_KC && K % LS_KC == 0;
}

// epilogue 0: out[M, N] (+bias) in out_dtype, or with splits > 1 float32 partial[splits, M, N];
// epilogue 1: out[M, N/2] = silu(gate) * up for rows interleaved in blocks of 8 (splits must be 1).
SLLM_EXPORT int sllm_linear_stream(const void* x, const void* W, const float* bias, void* out, int out_dtype,
                                   float* partial, int M, int N, int K, int splits, int epilogue,
                                   cudaStream_t stream) {
  SLLM_REQUIRE(sllm_linear_stream_supports(M, N, K), "linear_stream: sizes M=%d N=%d K=%d (needs M<=64, K%%128==0)", M, N, K);
  SLLM_REQUIRE(splits >= 1, "linear_stream: splits=%d", splits);
  SLLM_REQUIRE(splits == 1 || partial != nullptr, "linear_stream: k-splits need scratch");
  SLLM_REQUIRE(epilogue == EPI_STORE || (splits == 1 && N % 16 == 0 && out_dtype == SLLM_BF16),
               "linear_stream: the SiLU epilogue needs splits=1, N%%16==0 and a bfloat16 result");
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  const __nv_bfloat16* wb = (const __nv_bfloat16*)W;
  const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
#define GO(NT_)                                                                                              \
  if (epilogue == EPI_SILU) return launch_ls<NT_, EPI_SILU, __nv_bfloat16>(xb, wb, bias, out, partial, M, N, K, splits, stream); \
  if (out_dtype == SLLM_BF16) return launch_ls<NT_, EPI_STORE, __nv_bfloat16>(xb, wb, bias, out, partial, M, N, K, splits, stream); \
  return launch_ls<NT_, EPI_STORE, float>(xb, wb, bias, out, partial, M, N, K, splits, stream);
  switch (nt) {
    case 1: GO(1)
    case 2: GO(2)
    case 4: GO(4)
    default: GO(8)
  }
#undef GO
}

// The SiLU epilogue on an input whose norm is still owed: out[M, N/2] = silu(s gate) * (s up) with
// s[token] = rsqrt(sum of ssq[token][0..parts) / width + eps); x is bfloat16(stream * gain).  At most 32 tokens.
SLLM_EXPORT int sllm_linear_stream_silu_scaled(const void* x, const void* W, void* out, int M, int N, int K, const float* ssq,
                                               int parts, float eps, int width, cudaStream_t stream) {
  SLLM_REQUIRE(sllm_linear_stream_supports(M, N, K) && M <= 32 && N % 16 == 0,
               "linear_stream_silu_scaled: sizes M=%d N=%d K=%d (needs M<=32, N%%16==0, K%%128==0)", M, N, K);
  SLLM_REQUIRE(ssq != nullptr && ((uintptr_t)ssq & 15) == 0 && parts >= 1 && parts <= LS_SSQ_MAX && width >= 1,
               "linear_stream_silu_scaled: a table of %d partial sums (at most %d) over width %d", parts, LS_SSQ_MAX, width);
  LsScale sc;
  sc.ssq = ssq; sc.parts = parts; sc.eps = eps; sc.inv_width = 1.0f / (float)width;
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  const __nv_bfloat16* wb = (const __nv_bfloat16*)W;
  if (M <= 8) return launch_ls<1, EPI_SILU, __nv_bfloat16, true>(xb, wb, nullptr, out, nullptr, M, N, K, 1, stream, sc);
  if (M <= 16) return launch_ls<2, EPI_SILU, __nv_bfloat16, true>(xb, wb, nullptr, out, nullptr, M, N, K, 1, stream, sc);
  return launch_ls<4, EPI_SILU, __nv_bfloat16, true>(xb, wb, nullptr, out, nullptr, M, N, K, 1, stream, sc);
}

// ---------------------------------------------------------------------------------------------
// An entry point that allocates nothing (declared in sllm_noalloc.h; see the comment there).
// ---------------------------------------------------------------------------------------------
#include <mutex>

#include "sllm_noalloc.h"

namespace sllm {

// Scratch for the k-split partial sums, part of the library's image: every GPU that loads the
// library holds these 8 MiB until the process exits.
static __device__ __align__(256) float ls_noalloc_scratch[SLLM_NOALLOC_SCRATCH_FLOATS];

constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES];      // device address of the array, per device
static std::mutex g_noalloc_mutex;

// out[i] = sum over splits of partial[s][i]
__global__ void sum_partials_kernel(const float* __restrict__ partial, int splits, size_t n, float* __restrict__ out) {
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = 0.f;
  for (int s = 0; s < splits; ++s) v += partial[(size_t)s * n + i];
  out[i] = v;
}

}  // namespace sllm

SLLM_EXPORT int sllm_linear_stream_noalloc(const void* x, const void* W, const float* bias, float* out, int M, int N,
                                           int K, int splits, cudaStream_t stream) {
  SLLM_REQUIRE(sllm_linear_stream_supports(M, N, K), "linear_stream_noalloc: sizes M=%d N=%d K=%d (needs M<=64, K%%128==0)", M, N, K);
  SLLM_REQUIRE(splits >= 1, "linear_stream_noalloc: splits=%d", splits);
  const int real = sllm_linear_stream_splits(K, splits);
  if (real == 1)        // nothing to add up: the product goes straight to the caller's buffer
    return sllm_linear_stream(x, W, bias, out, SLLM_F32, nullptr, M, N, K, 1, EPI_STORE, stream);
  const size_t need = (size_t)real * M * N;
  SLLM_REQUIRE(need <= (size_t)SLLM_NOALLOC_SCRATCH_FLOATS,
               "linear_stream_noalloc: %d splits x %d x %d partial sums need %zu floats, the built-in scratch holds %d",
               real, M, N, need, SLLM_NOALLOC_SCRATCH_FLOATS);
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
    set_error("linear_stream_noalloc: cannot tell the current device");
    return SLLM_ERR_LAUNCH;
  }
  float* scratch;
  {
    // The array's name is a host-side handle, not a device address: its address on the
    // current device is asked for once per device and kept.
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, ls_noalloc_scratch);
      if (e != cudaSuccess || p == nullptr) {
        char buf[200];
        snprintf(buf, sizeof buf, "linear_stream_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        set_error(buf);
        return SLLM_ERR_LAUNCH;
      }
      g_noalloc_ptr[dev] = static_cast<float*>(p);
    }
    scratch = g_noalloc_ptr[dev];
  }
  int rc = sllm_linear_stream(x, W, bias, nullptr, SLLM_F32, scratch, M, N, K, real, EPI_STORE, stream);
  if (rc != SLLM_OK) return rc;
  const size_t n = (size_t)M * N;
  launch_kernel(sum_partials_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, (const float*)scratch, real, n, out);
  return launch_status("linear_stream_noalloc");
}
