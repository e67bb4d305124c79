// Memory-bound kernels of a step: embedding gather, residual add fused with
// RMSNorm, rotary encoding fused with the paged key/value write, SiLU-multiply,
// row gather.  All arithmetic in float32; operands float32 or bfloat16.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace sllm {

static thread_local char g_error[256] = "";
void set_error(const char* msg) {
  strncpy(g_error, msg, sizeof g_error - 1);
  g_error[sizeof g_error - 1] = 0;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("SLLM_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

int num_sms() {
  // per device: a process may hold models on several
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    cached[dev] = n;
  }
  return cached[dev];
}

// ---------------------------------------------------------------------------
// out[t, :] = float(table[ids[t], :])      (kernels/cuda/kernels.cu:770-787 does one row)
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int H, int V) {
  pdl_launch_dependents();       // a short kernel: the successor may be set up behind it
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);     // the host validates ids; never read outside the table
  const TW* row = table + (size_t)id * H;
  float* o = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

// ---------------------------------------------------------------------------
// residual += sum of `parts` delta slices (if any); out = residual * rsqrt(mean(residual^2)+eps) * w
// Formula ref/standard.py:25-31; fusion with the add as kernels/cuda/kernels.cu:791-839;
// 1/sqrtf, not rsqrtf (kernels.cu:818-820).  The sum over a row is taken in an order
// that depends on H and the block size only, never on the batch.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&a);
  raw.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// VEC: H and the part stride are multiples of 4 and every pointer is 16-byte aligned; four
// elements a thread, the partial sums read with independent loads.
template <typename TD, typename TO, bool VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int parts,
                                   size_t part_stride, const float* __restrict__ w, float eps,
                                   TO* __restrict__ out, int H) {
  __shared__ float red[33];
  pdl_launch_dependents();       // a short kernel: the successor may be set up behind it
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * H;
  float ss = 0.f;
  if constexpr (VEC) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 v = load4(residual + base + i);
      if (delta != nullptr) {
#pragma unroll 8
        for (int p = 0; p < parts; ++p) {
          const float4 d = load4(delta + p * part_stride + base + i);
          v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        }
        store4(residual + base + i, v);
      }
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = residual[base + i];
      if (delta != nullptr) {
        for (int p = 0; p < parts; ++p) v += to_f32(delta[p * part_stride + base + i]);
        residual[base + i] = v;
      }
      ss += v * v;
    }
  }
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  if constexpr (VEC) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      const float4 v = load4(residual + base + i), g = load4(w + i);
      store4(out + base + i, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[base + i] = from_f32<TO>(residual[base + i] * inv * w[i]);
  }
}

// Many rows (prompt portions): the kernel is bound by memory, so a thread keeps VPT vectors of its
// row in registers (one read of the stream, no second pass) and a row takes few threads, which
// leaves many rows resident per SM and many loads in flight.  One part only.
template <typename TD, typename TO, int VPT>
__global__ void add_rmsnorm_rows_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                        const float* __restrict__ w, float eps, TO* __restrict__ out, int H) {
  __shared__ float red[33];
  pdl_launch_dependents();       // a short kernel: the successor may be set up behind it
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * H;
  float4 v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 4;
    v[k] = i < H ? load4(residual + base + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (delta != nullptr) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = (threadIdx.x + k * blockDim.x) * 4;
      if (i < H) {
        const float4 d = load4(delta + base + i);
        v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w;
        store4(residual + base + i, v[k]);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < VPT; ++k) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 4;
    if (i < H) {
      const float4 g = load4(w + i);
      store4(out + base + i, make_float4(v[k].x * inv * g.x, v[k].y * inv * g.y, v[k].z * inv * g.z, v[k].w * inv * g.w));
    }
  }
}

// ---------------------------------------------------------------------------
// out[t, i] = silu(g) * u with g = gu[t, gi(i)], u = gu[t, gi(i) + blk], gi(i) = (i/blk)*2*blk + i%blk
// silu(z) = z / (1 + exp(-z))  (ref/qwen3_5.py:28-29; kernels/cuda/kernels.cu:898-907)
// ---------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void silu_mul_kernel(const TI* __restrict__ gu, TO* __restrict__ out, int I, int blk, size_t n) {
  pdl_launch_dependents();       // a short kernel: the successor may be set up behind it
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const size_t t = idx / I;
  const int i = (int)(idx % I);
  const size_t gi = t * 2 * (size_t)I + (size_t)(i / blk) * 2 * blk + (i % blk);
  const float g = to_f32(gu[gi]);
  const float u = to_f32(gu[gi + blk]);
  out[idx] = from_f32<TO>(g * (1.0f / (1.0f + expf(-g))) * u);
}

// out[r, :] = sum over parts of x[part][rows[r], :]
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, int parts, size_t part_stride,
                                   const int* __restrict__ rows, T* __restrict__ out, int H, int n_src) {
  pdl_launch_dependents();       // a short kernel: the successor may be set up behind it
  pdl_wait();
  int r = rows[blockIdx.x];
  r = r < 0 ? 0 : (r >= n_src ? n_src - 1 : r);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    if (parts == 1) {
      out[(size_t)blockIdx.x * H + i] = x[(size_t)r * H + i];
    } else {
      float v = 0.f;
      for (int p = 0; p < parts; ++p) v += to_f32(x[p * part_stride + (size_t)r * H + i]);
      out[(size_t)blockIdx.x * H + i] = from_f32<T>(v);
    }
  }
}

// ---------------------------------------------------------------------------
// Per (token, head) of the fused q|k|v row: add the bias; rotate the first `rot`
// dims of q and k heads by the token's position, pairs (j, j+rot/2):
//   o[j] = x[j] c_j - x[j+rot/2] s_j ; o[j+rot/2] = x[j+rot/2] c_j + x[j] s_j
// (ref/qwen3_5.py:337-370; kernels/cuda/kernels.cu:846-895), dims >= rot pass.
// q goes to q_out; k (after bias and rotation) and v (after bias) go to the token's
// slot of the paged cache [page][kv head][slot in page][hd]
// (cache content: ref/incremental.py:135-139; kernels.cu:923-953 for the contiguous form).
// table: [max_pos][2][rot/2] cos then sin, float32 made from float64 angles.
// ---------------------------------------------------------------------------
// The q|k|v rows may arrive as `parts` partial sums (a k-split product), `part_stride` apart;
// they are added here in order.  A block takes `hpb` consecutive heads of one token (one head when
// few tokens leave the GPU idle otherwise, all heads for prompt portions).
template <typename TI, typename TC>
__global__ void rope_kv_write_kernel(const TI* __restrict__ qkv, int parts, size_t part_stride,
                                     const float* __restrict__ bias,
                                     const int* __restrict__ positions, const float* __restrict__ table,
                                     int rot, int max_pos, int nq, int nkv, int hd, int hpb,
                                     const int* __restrict__ slot_mapping, int page_size, int num_pages,
                                     TC* __restrict__ k_cache, TC* __restrict__ v_cache, TC* __restrict__ q_out) {
  pdl_launch_dependents();       // a short kernel: the successor may be set up behind it
  pdl_wait();
  const int t = blockIdx.x;
  const int heads = nq + 2 * nkv;
  const int head0 = blockIdx.y * hpb;
  const int nheads = min(hpb, heads - head0);
  const int width = heads * hd;
  const TI* xt = qkv + (size_t)t * width;
  auto ld = [&](int col) {                           // col: column of the fused row
    float v = to_f32(xt[col]);
    for (int p = 1; p < parts; ++p) v += to_f32(xt[p * part_stride + col]);
    return v + (bias ? bias[col] : 0.f);
  };
  // where a head's row goes: q_out, or the token's slot of the key / value pages (null: skip)
  int slot = -1;
  if (slot_mapping != nullptr) {
    slot = slot_mapping[t];
    if (slot < 0 || slot / page_size >= num_pages) slot = -1;   // the host checks tables; never write outside the pool
  }
  auto dst_of = [&](int head) -> TC* {
    if (head < nq) return q_out + (size_t)t * nq * hd + (size_t)head * hd;
    if (slot < 0) return nullptr;                    // this run reads another run's cache
    const bool is_k = head < nq + nkv;
    const int kvh = is_k ? head - nq : head - nq - nkv;
    const int page = slot / page_size, off = slot % page_size;
    return (is_k ? k_cache : v_cache) + (((size_t)page * nkv + kvh) * page_size + off) * hd;
  };
  const bool rotary = rot > 0 && table != nullptr;
  const int half = rot / 2;
  if (rotary) {
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = table + (size_t)pos * rot;     // cos[half] then sin[half]
    for (int item = threadIdx.x; item < nheads * half; item += blockDim.x) {
      const int head = head0 + item / half, j = item % half;
      if (head >= nq + nkv) break;                   // value heads are not rotated (items ascend by head)
      TC* dst = dst_of(head);
      if (dst == nullptr) continue;
      const float x1 = ld(head * hd + j), x2 = ld(head * hd + j + half);
      const float c = cs[j], sn = cs[half + j];
      dst[j] = from_f32<TC>(x1 * c - x2 * sn);
      dst[j + half] = from_f32<TC>(x2 * c + x1 * sn);
    }
  }
  // what is not rotated: dims >= rot of q and k heads, every dim of v heads
  for (int item = threadIdx.x; item < nheads * hd; item += blockDim.x) {
    const int head = head0 + item / hd, d = item % hd;
    if (rotary && head < nq + nkv && d < rot) continue;
    TC* dst = dst_of(head);
    if (dst == nullptr) continue;
    dst[d] = from_f32<TC>(ld(head * hd + d));
  }
}

// The same for a bfloat16 cache, one part, eight elements a thread (16-byte loads and stores):
// the form for prompt portions, where the kernel is bound by memory.  Needs rot % 16 == 0 and
// hd % 8 == 0.  An item is (head, chunk of 8 dims); the chunk below rot/2 also takes its partner
// rot/2 further, the chunks between rot/2 and rot are done by their partners.
template <typename TI>
__global__ void rope_kv_write_vec_kernel(const TI* __restrict__ qkv, const float* __restrict__ bias,
                                         const int* __restrict__ positions, const float* __restrict__ table,
                                         int rot, int max_pos, int nq, int nkv, int hd, int hpb,
                                         const int* __restrict__ slot_mapping, int page_size, int num_pages,
                                         __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                         __nv_bfloat16* __restrict__ q_out) {
  pdl_launch_dependents();       // a short kernel: the successor may be set up behind it
  pdl_wait();
  const int t = blockIdx.x;
  const int heads = nq + 2 * nkv;
  const int head0 = blockIdx.y * hpb;
  const int nheads = min(hpb, heads - head0);
  const TI* xt = qkv + (size_t)t * heads * hd;
  int slot = -1;
  if (slot_mapping != nullptr) {
    slot = slot_mapping[t];
    if (slot < 0 || slot / page_size >= num_pages) slot = -1;
  }
  const bool rotary = rot > 0 && table != nullptr;
  const int half = rot / 2, cph = hd / 8;
  const float* cs = nullptr;
  if (rotary) {
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    cs = table + (size_t)pos * rot;
  }
  auto ld8 = [&](int col, float* f) {
    if constexpr (sizeof(TI) == 4) {
      const float4 x0 = load4(xt + col), x1 = load4(xt + col + 4);
      f[0] = x0.x; f[1] = x0.y; f[2] = x0.z; f[3] = x0.w;
      f[4] = x1.x; f[5] = x1.y; f[6] = x1.z; f[7] = x1.w;
    } else {
      const uint4 raw = *reinterpret_cast<const uint4*>(xt + col);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 p = __bfloat1622float2(h2[k]);
        f[2 * k] = p.x; f[2 * k + 1] = p.y;
      }
    }
    if (bias != nullptr) {
      const float4 b0 = load4(bias + col), b1 = load4(bias + col + 4);
      f[0] += b0.x; f[1] += b0.y; f[2] += b0.z; f[3] += b0.w;
      f[4] += b1.x; f[5] += b1.y; f[6] += b1.z; f[7] += b1.w;
    }
  };
  auto st8 = [&](__nv_bfloat16* dst, const float* f) {
    uint4 raw;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) h2[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
    *reinterpret_cast<uint4*>(dst) = raw;
  };
  for (int item = threadIdx.x; item < nheads * cph; item += blockDim.x) {
    const int head = head0 + item / cph, d = (item % cph) * 8;
    __nv_bfloat16* dst;
    if (head < nq) {
      dst = q_out + (size_t)t * nq * hd + (size_t)head * hd;
    } else {
      if (slot < 0) continue;
      const bool is_k = head < nq + nkv;
      const int kvh = is_k ? head - nq : head - nq - nkv;
      const int page = slot / page_size, off = slot % page_size;
      dst = (is_k ? k_cache : v_cache) + (((size_t)page * nkv + kvh) * page_size + off) * hd;
    }
    const bool rotated = rotary && head < nq + nkv && d < rot;
    float a[8];
    if (!rotated) {
      ld8(head * hd + d, a);
      st8(dst + d, a);
    } else if (d < half) {
      float b[8], o1[8], o2[8];
      ld8(head * hd + d, a);
      ld8(head * hd + d + half, b);
      const float4 c0 = load4(cs + d), c1 = load4(cs + d + 4), s0 = load4(cs + half + d), s1 = load4(cs + half + d + 4);
      const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        o1[k] = a[k] * c[k] - b[k] * sn[k];
        o2[k] = b[k] * c[k] + a[k] * sn[k];
      }
      st8(dst + d, o1);
      st8(dst + d + half, o2);
    }
  }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT const char* sllm_last_error() { return g_error; }

// streaming multiprocessors of the current device: the dispatch sizes its splits for them
SLLM_EXPORT int sllm_num_sms() { return sllm::num_sms(); }

SLLM_EXPORT int sllm_embed_gather(const void* table, int table_dtype, const int* ids, float* out, int T, int H,
                                  int V, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && H > 0 && V > 0, "embed_gather: bad sizes T=%d H=%d V=%d", T, H, V);
  if (T == 0) return SLLM_OK;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == SLLM_F32)
    launch_kernel(embed_gather_kernel<float>, T, threads, 0, stream, (const float*)table, ids, out, H, V);
  else if (table_dtype == SLLM_BF16)
    launch_kernel(embed_gather_kernel<__nv_bfloat16>, T, threads, 0, stream, (const __nv_bfloat16*)table, ids, out, H, V);
  else
    SLLM_REQUIRE(false, "embed_gather: unknown dtype %d", table_dtype);
  return launch_status("embed_gather");
}

SLLM_EXPORT int sllm_add_rmsnorm(float* residual, const void* delta, int delta_dtype, int parts,
                                 size_t part_stride, const float* w, float eps, void* out, int out_dtype,
                                 int rows, int H, cudaStream_t stream) {
  SLLM_REQUIRE(rows >= 0 && H > 0, "add_rmsnorm: bad sizes rows=%d H=%d", rows, H);
  SLLM_REQUIRE(delta == nullptr || parts >= 1, "add_rmsnorm: parts=%d", parts);
  if (rows == 0) return SLLM_OK;
  const bool vec = H % 4 == 0 && part_stride % 4 == 0 && ((uintptr_t)residual % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
                   ((uintptr_t)out % 16 == 0) && (delta == nullptr || (uintptr_t)delta % 16 == 0);
  const int per = vec ? 4 : 1;
  // one pass of the row per thread where it fits: the kernel is bound by load latency, not by work
  int threads = ((H / per + 31) / 32) * 32;
  threads = threads > 1024 ? 1024 : (threads < 64 ? 64 : threads);
  constexpr int VPT = 4;
  const int row_threads = ((H / 4 + VPT - 1) / VPT + 31) / 32 * 32;
  const bool many = vec && rows >= 64 && (delta == nullptr || parts == 1) && row_threads <= 1024;
#define LAUNCH(TD, TO)                                                                                         \
  do {                                                                                                         \
    if (many)                                                                                                  \
      launch_kernel(add_rmsnorm_rows_kernel<TD, TO, VPT>, rows, row_threads, 0, stream, residual,             \
                    (const TD*)delta, w, eps, (TO*)out, H);                                                    \
    else if (vec)                                                                                              \
      launch_kernel(add_rmsnorm_kernel<TD, TO, true>, rows, threads, 0, stream, residual, (const TD*)delta,   \
                    parts, part_stride, w, eps, (TO*)out, H);                                                  \
    else                                                                                                       \
      launch_kernel(add_rmsnorm_kernel<TD, TO, false>, rows, threads, 0, stream, residual, (const TD*)delta,  \
                    parts, part_stride, w, eps, (TO*)out, H);                                                  \
  } while (0)
  if (delta_dtype == SLLM_F32 && out_dtype == SLLM_F32) LAUNCH(float, float);
  else if (delta_dtype == SLLM_F32 && out_dtype == SLLM_BF16) LAUNCH(float, __nv_bfloat16);
  else if (delta_dtype == SLLM_BF16 && out_dtype == SLLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (delta_dtype == SLLM_BF16 && out_dtype == SLLM_F32) LAUNCH(__nv_bfloat16, float);
  else SLLM_REQUIRE(false, "add_rmsnorm: unknown dtypes %d %d", delta_dtype, out_dtype);
#undef LAUNCH
  return launch_status("add_rmsnorm");
}

SLLM_EXPORT int sllm_silu_mul(const void* gu, int in_dtype, void* out, int out_dtype, int T, int I, int blk,
                              cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && I > 0 && blk > 0 && I % blk == 0, "silu_mul: bad sizes T=%d I=%d blk=%d", T, I, blk);
  const size_t n = (size_t)T * I;
  if (n == 0) return SLLM_OK;
  const unsigned blocks = (unsigned)((n + 255) / 256);
#define LAUNCH(TI, TO) launch_kernel(silu_mul_kernel<TI, TO>, blocks, 256, 0, stream, (const TI*)gu, (TO*)out, I, blk, n)
  if (in_dtype == SLLM_F32 && out_dtype == SLLM_F32) LAUNCH(float, float);
  else if (in_dtype == SLLM_F32 && out_dtype == SLLM_BF16) LAUNCH(float, __nv_bfloat16);
  else if (in_dtype == SLLM_BF16 && out_dtype == SLLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else SLLM_REQUIRE(false, "silu_mul: unsupported dtypes %d -> %d", in_dtype, out_dtype);
#undef LAUNCH
  return launch_status("silu_mul");
}

SLLM_EXPORT int sllm_gather_rows(const void* x, int dtype, int parts, size_t part_stride, const int* rows, void* out,
                                 int R, int H, int n_src, cudaStream_t stream) {
  SLLM_REQUIRE(R >= 0 && H > 0 && n_src > 0 && parts >= 1, "gather_rows: bad sizes R=%d H=%d n=%d parts=%d", R, H, n_src, parts);
  if (R == 0) return SLLM_OK;
  if (dtype == SLLM_F32)
    launch_kernel(gather_rows_kernel<float>, R, 256, 0, stream, (const float*)x, parts, part_stride, rows, (float*)out, H, n_src);
  else if (dtype == SLLM_BF16)
    launch_kernel(gather_rows_kernel<__nv_bfloat16>, R, 256, 0, stream, (const __nv_bfloat16*)x, parts, part_stride, rows, (__nv_bfloat16*)out, H, n_src);
  else
    SLLM_REQUIRE(false, "gather_rows: unknown dtype %d", dtype);
  return launch_status("gather_rows");
}

SLLM_EXPORT int sllm_rope_kv_write(const void* qkv, int in_dtype, int parts, size_t part_stride, const float* bias,
                                   const int* positions,
                                   const float* table, int rot, int max_pos, int nq, int nkv, int hd,
                                   const int* slot_mapping, int page_size, int num_pages, void* k_cache,
                                   void* v_cache, void* q_out, int cache_dtype, int T, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && nq > 0 && nkv > 0 && hd > 0, "rope_kv_write: bad sizes T=%d nq=%d nkv=%d hd=%d", T, nq, nkv, hd);
  SLLM_REQUIRE(parts >= 1, "rope_kv_write: parts=%d", parts);
  SLLM_REQUIRE(rot >= 0 && rot <= hd && rot % 2 == 0, "rope_kv_write: rotary_dim=%d must be even and <= head_dim=%d", rot, hd);
  SLLM_REQUIRE(rot == 0 || (table != nullptr && max_pos > 0), "rope_kv_write: rotary table missing");
  SLLM_REQUIRE(slot_mapping == nullptr || (page_size > 0 && num_pages > 0 && k_cache && v_cache),
               "rope_kv_write: cache arguments missing");
  if (T == 0) return SLLM_OK;
  const int heads = nq + 2 * nkv;
  // few tokens: a block per head, so that the launch fills the GPU; many: a block per token
  const int hpb = T >= 128 ? heads : 1;
  dim3 grid(T, (heads + hpb - 1) / hpb);
  const int threads = hpb == 1 ? (hd / 2 >= 64 ? 64 : 32) : 256;
  auto al16 = [](const void* p) { return (uintptr_t)p % 16 == 0; };
  if (cache_dtype == SLLM_BF16 && parts == 1 && rot % 16 == 0 && hd % 8 == 0 && al16(qkv) &&
      al16(bias) && al16(table) && al16(q_out) && al16(k_cache) && al16(v_cache)) {
    const int vthreads = hpb == 1 ? 32 : 256;
#define LAUNCH_VEC(TI)                                                                                           \
  launch_kernel(rope_kv_write_vec_kernel<TI>, grid, vthreads, 0, stream, (const TI*)qkv, bias, positions, table, rot, \
                max_pos, nq, nkv, hd, hpb, slot_mapping, page_size, num_pages, (__nv_bfloat16*)k_cache,            \
                (__nv_bfloat16*)v_cache, (__nv_bfloat16*)q_out)
    if (in_dtype == SLLM_F32) LAUNCH_VEC(float);
    else if (in_dtype == SLLM_BF16) LAUNCH_VEC(__nv_bfloat16);
    else SLLM_REQUIRE(false, "rope_kv_write: unsupported input dtype %d", in_dtype);
#undef LAUNCH_VEC
    return launch_status("rope_kv_write");
  }
#define LAUNCH(TI, TC)                                                                                         \
  launch_kernel(rope_kv_write_kernel<TI, TC>, grid, threads, 0, stream, (const TI*)qkv, parts, part_stride, bias,  \
                positions, table, rot, max_pos, nq, nkv, hd, hpb, slot_mapping, page_size, num_pages,              \
                (TC*)k_cache, (TC*)v_cache, (TC*)q_out)
  if (in_dtype == SLLM_F32 && cache_dtype == SLLM_F32) LAUNCH(float, float);
  else if (in_dtype == SLLM_F32 && cache_dtype == SLLM_BF16) LAUNCH(float, __nv_bfloat16);
  else if (in_dtype == SLLM_BF16 && cache_dtype == SLLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else SLLM_REQUIRE(false, "rope_kv_write: unsupported dtypes %d -> %d", in_dtype, cache_dtype);
#undef LAUNCH
  return launch_status("rope_kv_write");
}
