// Sampling on the device over float32 logits [R, V], one block of 1024 threads per row, and the
// repetition penalty that goes before it.
//
// greedy: the first maximum (runtime/sampler.py:8-9).
// temperature: p = softmax(logits / T) with the maximum subtracted; the token is the first index
// whose cumulative probability reaches the uniform u (runtime/sampler.py:54-58, 81-88);
// temperature <= 0 is greedy (runtime/sampler.py:50-53).
// top-k, then top-p over what it kept, restrict the tokens that can be drawn
// (runtime/sampler.py:60-79); a token outside the kept set is never returned, also at u = 0 and
// beyond the last cumulative value, where the reference's searchsorted would name token 0 or V-1.
// Of logits that tie at a cut, those with the lowest indices stay.
// The host draws u, one per sampled token, from the request's own generator.
// Probabilities are expf((logit - max) / T), exact to float32 as the logits are; every sum is float64
// as the reference's sampler works in float64.
//
// In this file, in order:
//   block_argmax                     the greedy row;
//   select_key / choose_bin          the general top-k / top-p: a five-level select over the row for the
//                                    key of the cut (by count or by mass), then the kept set is
//                                    {key > tau} and the ties at tau up to an index;
//   collect_candidates, select_in_candidates, draw_from_list
//                                    the one-pass forms: every thread keeps its largest logits, and if
//                                    the cut provably lies among those candidates the rest runs on a
//                                    short list in shared memory (sample_top_k_fast for top_k <= 256,
//                                    sample_top_p_fast for top_p alone on a peaked row);
//   sample_rows_kernel               picks the form for its row; the general inverse CDF walks the row
//                                    in index order (32 parts, the chosen part in 32 pieces, one warp's scan);
//   repetition_penalty_kernel        the penalty from explicit (row, id) pairs;
//   mark_seen_kernel, penalty_seen_kernel
//                                    the penalty from a table of seen ids kept on the device.
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

// ---- the kept set of top-k / top-p: {key > tau} and, of {key == tau}, the indices up to i_eq --------
//
// Keys are the logits' bits mapped so that unsigned order is float order.  The k-th largest key, and
// the key at which the descending cumulative probability first reaches top_p, are found by a
// five-level select over the row.  Each level builds a histogram of counts and of probability mass
// (one histogram per warp, summed afterwards) of the eligible logits in the range chosen so far,
// walks it from the largest logits down and chooses the bin that holds the target.  The first level's
// 256 bins are linear in the distance from the row's maximum (logits share few exponents, so their
// top bits would put a whole row on a handful of counters); the other four take 8 bits of the key
// each, within the chosen linear bin, and end at one key.
//
// Probabilities are p = expf((logit - max) / T), exact to float32 as the logits are; sums are float64.

constexpr int SEL_BINS = 256, SEL_WARPS = SAMPLE_THREADS / 32;
constexpr int SAMPLE_SMEM = SEL_WARPS * SEL_BINS * (int)(sizeof(int) + sizeof(float));
constexpr float SEL_LINEAR_SPAN = 24.f;     // the linear bins cover (max - logit) / T up to this; the last takes the rest

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ int linear_bin(float l, float mx, float lscale) {
  const float d = (mx - l) * lscale;               // >= 0, monotone in the logit
  return d >= (float)(SEL_BINS - 1) ? SEL_BINS - 1 : (int)d;
}
__device__ __forceinline__ float prob(float l, float mx, float inv_t) { return expf((l - mx) * inv_t); }

struct Select {
  int lbin;                   // the linear bin chosen at the first level
  uint32_t prefix, mask;      // the key bits chosen so far
  int cnt_above;              // eligible logits greater than the chosen range
  double mass_above;          // their probability mass
  int group_cnt;              // logits in the chosen range (after the last level: equal to the key)
  double group_mass;
  double target;              // by mass: the cumulative mass to reach
  int chosen;                 // the last level's bin, -1: the target lies beyond every eligible logit
};

// f(logit, index) over the row, eight loads in flight a thread
template <class F>
__device__ __forceinline__ void for_row(const float* __restrict__ row, int V, F f) {
  for (int i0 = threadIdx.x; i0 < V; i0 += SAMPLE_THREADS * 8) {
    float l[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * SAMPLE_THREADS;
      l[u] = i < V ? row[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * SAMPLE_THREADS;
      if (i < V) f(l[u], i);
    }
  }
}
// the same over [base, base + len) cut at `end`, by one warp
template <class F>
__device__ __forceinline__ void for_part(const float* __restrict__ row, int base, int len, int end, F f) {
  const int lane = threadIdx.x & 31;
  for (int o = 0; o < len; o += 32 * 8) {
    float l[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + o + u * 32 + lane;
      l[u] = (o + u * 32 < len && i < end) ? row[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + o + u * 32 + lane;
      if (o + u * 32 < len && i < end) f(l[u], i);
    }
  }
}

// Warp 0 walks the 256 bins from the largest logits down (eight bins a lane, the lanes' sums
// scanned) and records in *st the first bin at which the count reaches k or the mass the target.
// `may_miss`: this is the select's first level, where no bin may reach the target (chosen = -1); at
// a later level the range chosen one level up held it.
__device__ void choose_bin(int level, bool by_mass, int k, bool target_is_fraction, double fraction,
                           const int* bin_c, const double* bin_m, Select* st, bool may_miss) {
  const int lane = threadIdx.x & 31;
  int c[8], lc = 0;
  double m[8], lm = 0.0;
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int j = 8 * lane + u, b = level == 0 ? j : SEL_BINS - 1 - j;
    c[u] = bin_c[b];
    m[u] = bin_m[b];
    lc += c[u];
    lm += m[u];
  }
  int ic = lc;
  double im = lm;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int nc = __shfl_up_sync(0xffffffffu, ic, d);
    const double nm = __shfl_up_sync(0xffffffffu, im, d);
    if (lane >= d) { ic += nc; im += nm; }
  }
  const double all_m = __shfl_sync(0xffffffffu, im, 31);
  const double target = (level == 0 && by_mass && target_is_fraction) ? fraction * all_m : st->target;
  int ca = st->cnt_above + ic - lc;                  // above this lane's bins
  double ma = st->mass_above + im - lm;
  __syncwarp();
  int hit = -1, last = -1;
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    if (c[u] == 0 || hit >= 0) continue;
    last = u;
    if (by_mass ? (ma + m[u] >= target) : (ca + c[u] >= k)) {
      hit = u;
    } else {
      ca += c[u];
      ma += m[u];
    }
  }
  const uint32_t hits = __ballot_sync(0xffffffffu, hit >= 0), nonempty = __ballot_sync(0xffffffffu, last >= 0);
  int who = -1, u_sel = -1;
  if (hits) {
    who = __ffs(hits) - 1;
    u_sel = hit;
  } else if (!may_miss && nonempty) {
    // the range chosen one level up held the target; its parts were summed in another order and
    // fall short by rounding: the target is in the last part
    who = 31 - __clz(nonempty);
    u_sel = last;
    if (lane == who) { ca -= c[last]; ma -= m[last]; }
  }
  if (lane == 0) { st->chosen = -1; st->target = target; }
  __syncwarp();
  if (lane == who) {
    int cu = 0;
    double mu = 0.0;
#pragma unroll
    for (int u = 0; u < 8; ++u) if (u == u_sel) { cu = c[u]; mu = m[u]; }
    const int j = 8 * lane + u_sel, b = level == 0 ? j : SEL_BINS - 1 - j;
    st->chosen = b;
    st->cnt_above = ca;
    st->mass_above = ma;
    st->group_cnt = cu;
    st->group_mass = mu;
    if (level == 0) {
      st->lbin = b;
    } else {
      const int shift = 32 - 8 * level;
      st->prefix |= (uint32_t)b << shift;
      st->mask |= 255u << shift;
    }
  }
}

constexpr int SEL_CANDIDATES = 4096;        // the chosen linear bin's keys are gathered if they are no more than this

// by_mass false: the key of the k-th largest eligible logit.  by_mass true: the first key, going
// down, at which the cumulative mass reaches `target` (`target_is_fraction`: of the eligible total).
// Eligible: key > floor_key where has_floor.  The result is in *st (shared), the same for all threads.
__device__ void select_key(const float* __restrict__ row, int V, float mx, float inv_t, bool by_mass, int k,
                           double target, bool target_is_fraction, bool has_floor, uint32_t floor_key,
                           int* hist_c, float* hist_m, int* bin_c, double* bin_m, uint32_t* cand, int* n_cand, Select* st) {
  const int warp = threadIdx.x >> 5;
  const float lscale = inv_t * ((float)(SEL_BINS - 1) / SEL_LINEAR_SPAN);
  if (threadIdx.x == 0) { *st = Select{0, 0u, 0u, 0, 0.0, 0, 0.0, target, 0}; *n_cand = 0; }
  bool gathered = false;
  for (int level = 0; level < 5; ++level) {
    const int shift = 32 - 8 * level;              // levels 1..4: bits 24, 16, 8, 0
    for (int i = threadIdx.x; i < SEL_WARPS * SEL_BINS; i += blockDim.x) { hist_c[i] = 0; hist_m[i] = 0.f; }
    __syncthreads();
    const uint32_t prefix = st->prefix, mask = st->mask;
    const int lbin = st->lbin;
    if (level == 1 && st->group_cnt <= SEL_CANDIDATES) {
      // the keys of the chosen linear bin, in any order: the levels below read these, not the row
      for_row(row, V, [&](float l, int) {
        const uint32_t key = order_key(l);
        if ((!has_floor || key > floor_key) && linear_bin(l, mx, lscale) == lbin) cand[atomicAdd(n_cand, 1)] = key;
      });
      gathered = true;
      __syncthreads();
    }
    if (gathered) {
      const int n = *n_cand;
      for (int j = threadIdx.x; j < n; j += blockDim.x) {
        const uint32_t key = cand[j];
        if ((key & mask) != prefix) continue;
        const int b = (int)((key >> shift) & 255u);
        atomicAdd(&hist_c[warp * SEL_BINS + b], 1);
        atomicAdd(&hist_m[warp * SEL_BINS + b], prob(key_value(key), mx, inv_t));
      }
    } else {
      // The last linear bin takes every logit far below the maximum, most of a peaked row: those are
      // counted in registers, not on one shared counter.
      int far_c = 0;
      float far_m = 0.f;
      for_row(row, V, [&](float l, int) {
        const uint32_t key = order_key(l);
        if (has_floor && key <= floor_key) return;
        int b = linear_bin(l, mx, lscale);
        if (level > 0) {
          if (b != lbin || (key & mask) != prefix) return;
          b = (int)((key >> shift) & 255u);
        } else if (b == SEL_BINS - 1) {
          ++far_c;
          far_m += prob(l, mx, inv_t);
          return;
        }
        atomicAdd(&hist_c[warp * SEL_BINS + b], 1);
        atomicAdd(&hist_m[warp * SEL_BINS + b], prob(l, mx, inv_t));
      });
      if (level == 0) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          far_c += __shfl_xor_sync(0xffffffffu, far_c, o);
          far_m += __shfl_xor_sync(0xffffffffu, far_m, o);
        }
        if ((threadIdx.x & 31) == 0 && far_c) {
          atomicAdd(&hist_c[warp * SEL_BINS + SEL_BINS - 1], far_c);
          atomicAdd(&hist_m[warp * SEL_BINS + SEL_BINS - 1], far_m);
        }
      }
    }
    __syncthreads();
    if (threadIdx.x < SEL_BINS) {
      int c = 0;
      double m = 0.0;
      for (int w = 0; w < SEL_WARPS; ++w) { c += hist_c[w * SEL_BINS + threadIdx.x]; m += (double)hist_m[w * SEL_BINS + threadIdx.x]; }
      bin_c[threadIdx.x] = c;
      bin_m[threadIdx.x] = m;
    }
    __syncthreads();
    if (warp == 0) choose_bin(level, by_mass, k, target_is_fraction, target, bin_c, bin_m, st, level == 0);
    __syncthreads();
    if (st->chosen < 0) break;
  }
}

// What a thread needs to know of the kept set.
struct Kept {
  bool filtered;
  uint32_t tau;
  int i_eq;                   // ties at tau stay up to this index
};
__device__ __forceinline__ bool is_kept(const Kept& kp, float l, int i) {
  if (!kp.filtered) return true;
  const uint32_t key = order_key(l);
  return key > kp.tau || (key == kp.tau && i <= kp.i_eq);
}

// ---- a small top-k in one pass over the row ------------------------------------------------------
//
// Each thread keeps the five largest logits of its share of the row; the four largest of every
// thread are the candidates (4096 of them), the fifth bounds what the thread let go.  If the k-th
// largest candidate lies above every such bound, the k largest logits of the row are all among the
// candidates and the rest of the work (top-k's cut, top-p over what it kept, the draw in index
// order) runs on at most k values in shared memory.  Otherwise (a thread held more than four of the
// row's k largest) the general path above takes the row.  The probabilities of top-k's set are
// renormalised, so the sum over the whole row is never needed here.

constexpr int FAST_K = 256;                 // rows with top_k up to this try the one-pass form
constexpr int FAST_PER_THREAD = 4;
constexpr int FAST_CANDIDATES = SAMPLE_THREADS * FAST_PER_THREAD;
constexpr int FAST_TIES = 1024;
static_assert(FAST_CANDIDATES * 8 + SEL_BINS * 4 <= SAMPLE_SMEM, "the candidates live in the histograms' shared memory");

struct FastShared {
  uint32_t kept_key[FAST_K], sorted_key[FAST_K];
  int kept_idx[FAST_K], sorted_idx[FAST_K];
  double q[FAST_K];
  int tie_idx[FAST_TIES];
  int n_kept, n_ties, max_let_go, answer, last;
  double red[33];
};

// One pass over the row: every thread's four largest logits become the candidates (keys and
// indices in `dyn_smem`), the largest fifth one is recorded in fs->max_let_go (31 bits), *mx_out is
// the row's maximum (first index among equals).  WITH_SUM: *sum_out is the sum over the whole row of
// expf((logit - max) / T), from a second pass.
template <bool WITH_SUM>
__device__ void collect_candidates(const float* __restrict__ row, int V, float inv_t, unsigned char* dyn_smem, MaxIdx* sh_mi,
                                   double* red, FastShared* fs, MaxIdx* mx_out, double* sum_out) {
  uint32_t* cand_key = reinterpret_cast<uint32_t*>(dyn_smem);
  int* cand_idx = reinterpret_cast<int*>(cand_key + FAST_CANDIDATES);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float v0 = -INFINITY, v1 = -INFINITY, v2 = -INFINITY, v3 = -INFINITY, v4 = -INFINITY;
  int i0 = -1, i1 = -1, i2 = -1, i3 = -1, i4 = -1;
  for_row(row, V, [&](float l, int i) {
    if (l != l) return;                             // not a number: never a candidate
    if (l > v4 || i4 < 0) {                         // an equal later logit does not displace an earlier one
      v4 = l; i4 = i;
      if (v4 > v3 || i3 < 0) {
        float tv = v3; v3 = v4; v4 = tv; int ti = i3; i3 = i4; i4 = ti;
        if (v3 > v2 || i2 < 0) {
          tv = v2; v2 = v3; v3 = tv; ti = i2; i2 = i3; i3 = ti;
          if (v2 > v1 || i1 < 0) {
            tv = v1; v1 = v2; v2 = tv; ti = i1; i1 = i2; i2 = ti;
            if (v1 > v0 || i0 < 0) { tv = v0; v0 = v1; v1 = tv; ti = i0; i0 = i1; i1 = ti; }
          }
        }
      }
    }
  });
  // the row's maximum (first index among equals) from the threads' own
  {
    MaxIdx best{i0 >= 0 ? v0 : -INFINITY, i0 >= 0 ? i0 : 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MaxIdx other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = better(best, other);
    }
    if (lane == 0) sh_mi[warp] = best;
    if (threadIdx.x == 0) { fs->n_kept = 0; fs->n_ties = 0; fs->max_let_go = 0; fs->answer = 0x7fffffff; fs->last = -1; }
    __syncthreads();
    if (warp == 0) {
      MaxIdx b = sh_mi[lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        MaxIdx other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
        b = better(b, other);
      }
      if (lane == 0) { if (b.i == 0x7fffffff) b.i = 0; sh_mi[0] = b; }
    }
  }
  // the candidates, and the largest logit any thread let go
  {
    const float vs[FAST_PER_THREAD] = {v0, v1, v2, v3};
    const int is[FAST_PER_THREAD] = {i0, i1, i2, i3};
#pragma unroll
    for (int j = 0; j < FAST_PER_THREAD; ++j) {
      cand_key[threadIdx.x * FAST_PER_THREAD + j] = is[j] >= 0 ? order_key(vs[j]) : 0u;
      cand_idx[threadIdx.x * FAST_PER_THREAD + j] = is[j];
    }
    if (i4 >= 0) atomicMax(&fs->max_let_go, (int)(order_key(v4) >> 1));     // (31 bits: compared as such below)
  }
  __syncthreads();
  const MaxIdx mx = sh_mi[0];
  *mx_out = mx;
  if constexpr (WITH_SUM) {
    double part = 0.0;                              // a second, plain pass: the sum needs the maximum
    for_row(row, V, [&](float l, int) {
      if (l == l) part += (double)prob(l, mx.v, inv_t);
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) red[warp] = part;
    __syncthreads();
    if (warp == 0) {
      double t = red[lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (lane == 0) red[32] = t;
    }
    __syncthreads();
    *sum_out = red[32];
  }
}

// The select of select_key over the candidates in shared memory (a linear level, then the key's four
// bytes): the k-th largest candidate, or the candidate at which the descending cumulative probability
// reaches `target`.  sel->chosen < 0 afterwards: the candidates' mass does not reach the target.
__device__ void select_in_candidates(const uint32_t* cand_key, const int* cand_idx, float mx, float inv_t, bool by_mass, int k,
                                     double target, int* bin_c, float* hist_m, double* bin_m, Select* sel) {
  const float lscale = inv_t * ((float)(SEL_BINS - 1) / SEL_LINEAR_SPAN);
  if (threadIdx.x == 0) *sel = Select{0, 0u, 0u, 0, 0.0, 0, 0.0, target, 0};
  for (int level = 0; level < 5; ++level) {
    const int shift = 32 - 8 * level;
    if (threadIdx.x < SEL_BINS) { bin_c[threadIdx.x] = 0; hist_m[threadIdx.x] = 0.f; }
    __syncthreads();
    const uint32_t prefix = sel->prefix, mask = sel->mask;
    const int lbin = sel->lbin;
    int far_c = 0;                                   // the last linear bin: most candidates of a peaked row
    float far_m = 0.f;
#pragma unroll
    for (int j = 0; j < FAST_PER_THREAD; ++j) {
      const int c = threadIdx.x * FAST_PER_THREAD + j;
      if (cand_idx[c] < 0) continue;
      const uint32_t key = cand_key[c];
      const float l = key_value(key);
      int b = linear_bin(l, mx, lscale);
      if (level > 0) {
        if (b != lbin || (key & mask) != prefix) continue;
        b = (int)((key >> shift) & 255u);
      } else if (b == SEL_BINS - 1) {
        ++far_c;
        if (by_mass) far_m += prob(l, mx, inv_t);
        continue;
      }
      atomicAdd(&bin_c[b], 1);
      if (by_mass) atomicAdd(&hist_m[b], prob(l, mx, inv_t));
    }
    if (level == 0) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        far_c += __shfl_xor_sync(0xffffffffu, far_c, o);
        far_m += __shfl_xor_sync(0xffffffffu, far_m, o);
      }
      if ((threadIdx.x & 31) == 0 && far_c) {
        atomicAdd(&bin_c[SEL_BINS - 1], far_c);
        atomicAdd(&hist_m[SEL_BINS - 1], far_m);
      }
    }
    __syncthreads();
    if (threadIdx.x < SEL_BINS) bin_m[threadIdx.x] = (double)hist_m[threadIdx.x];
    __syncthreads();
    if ((threadIdx.x >> 5) == 0) choose_bin(level, by_mass, k, false, 0.0, bin_c, bin_m, sel, level == 0);
    __syncthreads();
    // a target in the last linear bin lies among logits far below the maximum: the general form's business
    if (sel->chosen < 0 || (level == 0 && sel->lbin == SEL_BINS - 1)) {
      __syncthreads();
      if (threadIdx.x == 0) sel->chosen = -1;
      __syncthreads();
      return;
    }
  }
}

// The draw from a short list of kept tokens (keys, indices; n at most one a thread): the cumulative
// probability in index order reaches u times the total at the answer (runtime/sampler.py:81-88).
__device__ void draw_from_list(const uint32_t* key, const int* idx, int n, float mx, float inv_t, double u, double* red,
                               FastShared* fs, int* out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  double cum = 0.0;
  int mine = -1;
  if (threadIdx.x < n) {
    mine = idx[threadIdx.x];
    for (int j = 0; j < n; ++j)
      if (idx[j] <= mine) cum += (double)prob(key_value(key[j]), mx, inv_t);
  }
  double total = cum;                               // the token with the largest index holds the total
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) total = fmax(total, __shfl_xor_sync(0xffffffffu, total, o));
  if (lane == 0) red[warp] = total;
  __syncthreads();
  if (warp == 0) {
    double t = red[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = fmax(t, __shfl_xor_sync(0xffffffffu, t, o));
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  const double target = u * red[32];
  if (mine >= 0) {
    atomicMax(&fs->last, mine);
    if (cum >= target) atomicMin(&fs->answer, mine);
  }
  __syncthreads();
  // u beyond the last cumulative value: the last kept token
  if (threadIdx.x == 0) *out = fs->answer != 0x7fffffff ? fs->answer : fs->last;
}

// true: out[row] is written.  false: the general path must take the row.  `mx` is set either way.
__device__ bool sample_top_k_fast(const float* __restrict__ row, int V, float inv_t, int k, float pfrac, double u,
                                  unsigned char* dyn_smem, int* bin_c, double* bin_m, Select* sel, MaxIdx* sh_mi,
                                  FastShared* fs, MaxIdx* mx_out, int* out) {
  uint32_t* cand_key = reinterpret_cast<uint32_t*>(dyn_smem);
  int* cand_idx = reinterpret_cast<int*>(cand_key + FAST_CANDIDATES);
  const int warp = threadIdx.x >> 5;
  collect_candidates<false>(row, V, inv_t, dyn_smem, sh_mi, nullptr, fs, mx_out, nullptr);
  const MaxIdx mx = *mx_out;
  // the k-th largest candidate
  select_in_candidates(cand_key, cand_idx, mx.v, inv_t, false, k, 0.0, bin_c, reinterpret_cast<float*>(cand_idx + FAST_CANDIDATES),
                       bin_m, sel);
  if (sel->chosen < 0) return false;
  const uint32_t tau = sel->prefix;
  const int n_eq = k - sel->cnt_above, ties = sel->group_cnt;
  // every logit a thread let go must lie below tau (the bound was kept to 31 bits: compare those)
  if ((int)(tau >> 1) <= fs->max_let_go || ties > FAST_TIES) return false;
  // top-k's set: above tau, and the first n_eq of the ties by index
#pragma unroll
  for (int j = 0; j < FAST_PER_THREAD; ++j) {
    const int c = threadIdx.x * FAST_PER_THREAD + j;
    if (cand_idx[c] < 0) continue;
    if (cand_key[c] > tau) {
      const int at = atomicAdd(&fs->n_kept, 1);
      fs->kept_key[at] = cand_key[c];
      fs->kept_idx[at] = cand_idx[c];
    } else if (cand_key[c] == tau) {
      fs->tie_idx[atomicAdd(&fs->n_ties, 1)] = cand_idx[c];
    }
  }
  __syncthreads();
  if (threadIdx.x < ties) {
    const int mine = fs->tie_idx[threadIdx.x];
    int rank = 0;
    for (int j = 0; j < ties; ++j) rank += fs->tie_idx[j] < mine;
    if (rank < n_eq) {
      const int at = atomicAdd(&fs->n_kept, 1);
      fs->kept_key[at] = tau;
      fs->kept_idx[at] = mine;
    }
  }
  __syncthreads();
  int m = fs->n_kept;                               // == k
  // top-p over the kept values in descending order, ties by index (runtime/sampler.py:68-79)
  if (pfrac >= 0.f) {
    if (threadIdx.x < m) {
      const uint32_t key = fs->kept_key[threadIdx.x];
      const int idx = fs->kept_idx[threadIdx.x];
      int rank = 0;
      for (int j = 0; j < m; ++j) rank += fs->kept_key[j] > key || (fs->kept_key[j] == key && fs->kept_idx[j] < idx);
      fs->sorted_key[rank] = key;
      fs->sorted_idx[rank] = idx;
    }
    __syncthreads();
    // the cumulative probability at every place of the sorted list, one place a thread
    if (threadIdx.x < m) fs->q[threadIdx.x] = (double)prob(key_value(fs->sorted_key[threadIdx.x]), mx.v, inv_t);
    if (threadIdx.x == 0) fs->n_kept = m;
    __syncthreads();
    double cum = 0.0;
    if (threadIdx.x < m)
      for (int j = 0; j <= (int)threadIdx.x; ++j) cum += fs->q[j];
    if ((int)threadIdx.x == m - 1) fs->red[0] = cum;        // the total
    __syncthreads();
    if (threadIdx.x < m && cum >= (double)pfrac * fs->red[0]) atomicMin(&fs->n_kept, (int)threadIdx.x + 1);
    __syncthreads();
    m = fs->n_kept;
    if (threadIdx.x < m) {
      fs->kept_key[threadIdx.x] = fs->sorted_key[threadIdx.x];
      fs->kept_idx[threadIdx.x] = fs->sorted_idx[threadIdx.x];
    }
    __syncthreads();
  }
  draw_from_list(fs->kept_key, fs->kept_idx, m, mx.v, inv_t, u, fs->red, fs, out);
  return true;
}

// ---- top-p alone, in one pass over the row where the row is peaked ------------------------------
//
// The same candidates, and the sum over the whole row from the same pass.  The descending cumulative
// probability is followed over the candidates (a select by mass on their keys); if it reaches top_p
// times the row's sum at a key above everything a thread let go, the kept set is exact and (at most
// FAST_P_KEPT tokens) is drawn from in shared memory.  A flat row, whose top_p set runs into the
// thousands, goes to the general path.

constexpr int FAST_P_KEPT = SAMPLE_THREADS;

__device__ bool sample_top_p_fast(const float* __restrict__ row, int V, float inv_t, float pfrac, double u,
                                  unsigned char* dyn_smem, int* bin_c, double* bin_m, Select* sel, MaxIdx* sh_mi,
                                  FastShared* fs, MaxIdx* mx_out, int* out) {
  uint32_t* cand_key = reinterpret_cast<uint32_t*>(dyn_smem);
  int* cand_idx = reinterpret_cast<int*>(cand_key + FAST_CANDIDATES);
  float* hist_m = reinterpret_cast<float*>(cand_idx + FAST_CANDIDATES);             // [256]
  uint32_t* kept_key = reinterpret_cast<uint32_t*>(hist_m + SEL_BINS);              // [FAST_P_KEPT]
  int* kept_idx = reinterpret_cast<int*>(kept_key + FAST_P_KEPT);
  static_assert(FAST_CANDIDATES * 8 + SEL_BINS * 4 + FAST_P_KEPT * 8 <= SAMPLE_SMEM, "the lists live in the histograms' shared memory");
  const int warp = threadIdx.x >> 5;
  double row_sum;
  collect_candidates<true>(row, V, inv_t, dyn_smem, sh_mi, fs->red, fs, mx_out, &row_sum);
  const MaxIdx mx = *mx_out;
  // the key at which the descending cumulative probability first reaches top_p of the row's sum
  select_in_candidates(cand_key, cand_idx, mx.v, inv_t, true, 0, (double)pfrac * row_sum, bin_c, hist_m, bin_m, sel);
  if (sel->chosen < 0) return false;                 // the candidates' mass does not reach it
  const uint32_t tau = sel->prefix;
  const int ties = sel->group_cnt;
  const double q = (double)prob(key_value(tau), mx.v, inv_t);
  const int n_eq = (int)fmin(fmax(ceil((sel->target - sel->mass_above) / q), 1.0), (double)ties);
  // exact only if every logit a thread let go lies below tau; short enough to be drawn from here
  if ((int)(tau >> 1) <= fs->max_let_go || ties > FAST_TIES || sel->cnt_above + n_eq > FAST_P_KEPT) return false;
#pragma unroll
  for (int j = 0; j < FAST_PER_THREAD; ++j) {
    const int c = threadIdx.x * FAST_PER_THREAD + j;
    if (cand_idx[c] < 0) continue;
    if (cand_key[c] > tau) {
      const int at = atomicAdd(&fs->n_kept, 1);
      kept_key[at] = cand_key[c];
      kept_idx[at] = cand_idx[c];
    } else if (cand_key[c] == tau) {
      fs->tie_idx[atomicAdd(&fs->n_ties, 1)] = cand_idx[c];
    }
  }
  __syncthreads();
  if (threadIdx.x < ties) {                          // of the ties, the first n_eq by index
    const int mine = fs->tie_idx[threadIdx.x];
    int rank = 0;
    for (int j = 0; j < ties; ++j) rank += fs->tie_idx[j] < mine;
    if (rank < n_eq) {
      const int at = atomicAdd(&fs->n_kept, 1);
      kept_key[at] = tau;
      kept_idx[at] = mine;
    }
  }
  __syncthreads();
  draw_from_list(kept_key, kept_idx, fs->n_kept, mx.v, inv_t, u, fs->red, fs, out);
  return true;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                   const double* __restrict__ uniform, const int* __restrict__ top_k, const float* __restrict__ top_p,
                   int* __restrict__ out) {
  extern __shared__ unsigned char sample_smem[];
  __shared__ MaxIdx sh_mi[32];
  __shared__ double part_sum[SEL_WARPS];
  __shared__ int part_cnt[SEL_WARPS], part_last[SEL_WARPS];
  __shared__ int bin_c[SEL_BINS];
  __shared__ double bin_m[SEL_BINS];
  __shared__ Select sel;
  __shared__ uint32_t cand[SEL_CANDIDATES];
  __shared__ int n_cand;
  __shared__ int pick_part, pick_need, i_eq_s, result;
  __shared__ double pick_before;
  pdl_launch_dependents();       // a short kernel: the successor may be set up behind it
  pdl_wait();
  __shared__ FastShared fast;
  const float* row = logits + (size_t)blockIdx.x * V;
  const float temp = temperature ? temperature[blockIdx.x] : 0.f;
  const int k = (top_k && temp > 0.f) ? top_k[blockIdx.x] : 0;
  const float pfrac = (top_p && temp > 0.f) ? top_p[blockIdx.x] : -1.f;
  const bool has_k = k > 0 && k < V, has_p = pfrac >= 0.f;
  const float inv_t = temp > 0.f ? 1.0f / temp : 0.f;
  MaxIdx mx;
  if (has_k && k <= FAST_K) {
    if (sample_top_k_fast(row, V, inv_t, k, pfrac, uniform[blockIdx.x], sample_smem, bin_c, bin_m, &sel, sh_mi, &fast, &mx,
                          out + blockIdx.x))
      return;
    __syncthreads();                                 // the general path reuses what the attempt wrote
  } else if (has_p && !has_k) {
    if (sample_top_p_fast(row, V, inv_t, pfrac, uniform[blockIdx.x], sample_smem, bin_c, bin_m, &sel, sh_mi, &fast, &mx,
                          out + blockIdx.x))
      return;
    __syncthreads();
  } else {
    mx = block_argmax(row, V, sh_mi);
  }
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) out[blockIdx.x] = mx.i;
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // the row in 32 parts of whole 32-element groups, one per warp, in index order
  const int part_len = (((V + SEL_WARPS - 1) / SEL_WARPS) + 31) & ~31;

  // ---- the kept set (runtime/sampler.py:60-79): top-k first, then top-p over what it kept ----
  Kept kp{has_k || has_p, 0u, 0x7fffffff};
  if (kp.filtered) {
    int* hist_c = reinterpret_cast<int*>(sample_smem);
    float* hist_m = reinterpret_cast<float*>(hist_c + SEL_WARPS * SEL_BINS);
    uint32_t tau = 0u;                     // with no top-k every key is above the floor
    int n_eq = 0x7fffffff, ties = 0;       // ties at tau: how many stay, how many there are
    double kept_mass = 0.0, above_k = 0.0;
    if (has_k) {
      select_key(row, V, mx.v, inv_t, false, k, 0.0, false, false, 0u, hist_c, hist_m, bin_c, bin_m, cand, &n_cand, &sel);
      tau = sel.prefix;
      n_eq = k - sel.cnt_above;            // of the ties at the k-th value, the first ones by index
      ties = sel.group_cnt;
      above_k = sel.mass_above;
      kept_mass = above_k + (double)n_eq * (double)prob(key_value(tau), mx.v, inv_t);
      __syncthreads();
    }
    if (has_p) {
      // the cumulative probability in descending order first reaches top_p at the last token that
      // stays (runtime/sampler.py:70-75); the probabilities are those renormalised after top-k, so
      // the target is top_p times the mass top-k kept
      select_key(row, V, mx.v, inv_t, true, 0, has_k ? (double)pfrac * kept_mass : (double)pfrac, !has_k, has_k, tau,
                 hist_c, hist_m, bin_c, bin_m, cand, &n_cand, &sel);
      if (sel.chosen >= 0) {
        const double q = (double)prob(key_value(sel.prefix), mx.v, inv_t);
        const double m = fmin(fmax(ceil((sel.target - sel.mass_above) / q), 1.0), (double)sel.group_cnt);
        tau = sel.prefix;
        n_eq = (int)m;
        ties = sel.group_cnt;
      } else if (has_k) {
        // not reached above the k-th value: the cut falls among its ties, or top-k's set stays whole
        const double q = (double)prob(key_value(tau), mx.v, inv_t);
        const double m = ceil(((double)pfrac * kept_mass - above_k) / q);
        if (m < (double)n_eq) n_eq = (int)fmax(m, 1.0);
      }
      __syncthreads();
    }
    if (tau == 0u && n_eq == 0x7fffffff) {
      kp.filtered = false;                 // top_p lies beyond the whole row: everything stays
    } else {
      kp.tau = tau;
      if (n_eq < ties) {
        // some ties go: find the index of the n_eq-th one
        int c = 0;
        const int base = warp * part_len;
        for (int o = 0; o < part_len; o += 32) {
          const int i = base + o + lane;
          c += __popc(__ballot_sync(0xffffffffu, i < V && order_key(row[i]) == tau));
        }
        if (lane == 0) part_cnt[warp] = c;
        __syncthreads();
        if (threadIdx.x == 0) {
          int before = 0, w = 0;
          for (; w < SEL_WARPS - 1 && before + part_cnt[w] < n_eq; ++w) before += part_cnt[w];
          pick_part = w;
          pick_need = n_eq - before;       // the tie of this rank (from 1) within the part
          i_eq_s = 0x7fffffff;
        }
        __syncthreads();
        if (warp == pick_part) {
          int need = pick_need;
          for (int o = 0; o < part_len; o += 32) {
            const int i = base + o + lane;
            const uint32_t b = __ballot_sync(0xffffffffu, i < V && order_key(row[i]) == tau);
            const int c2 = __popc(b);
            if (need <= c2) {
              if (lane == 0) i_eq_s = base + o + (int)__fns(b, 0, need);
              break;
            }
            need -= c2;
          }
        }
        __syncthreads();
        kp.i_eq = i_eq_s;
      }
    }
  }

  // ---- inverse CDF over the kept tokens in index order (runtime/sampler.py:81-88) ----
  // 1: each warp sums its part of the row
  {
    double s = 0.0;
    int last = -1;
    for_part(row, warp * part_len, part_len, V, [&](float l, int i) {
      if (is_kept(kp, l, i)) { s += (double)prob(l, mx.v, inv_t); last = i; }
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
    }
    if (lane == 0) { part_sum[warp] = s; part_last[warp] = last; }
  }
  __syncthreads();
  // 2: the part in which the cumulative sum reaches u times the total
  if (threadIdx.x == 0) {
    double total = 0.0;
    for (int w = 0; w < SEL_WARPS; ++w) total += part_sum[w];
    const double target = uniform[blockIdx.x] * total;
    double before = 0.0;
    int pick = -1, last = -1;
    for (int w = 0; w < SEL_WARPS; ++w) {
      if (part_last[w] >= 0) last = max(last, part_last[w]);
      if (pick < 0 && part_last[w] >= 0 && before + part_sum[w] >= target) pick = w;
      if (pick < 0) before += part_sum[w];
    }
    pick_part = pick;
    pick_before = pick >= 0 ? target - before : 0.0;      // what remains to be reached inside the part
    // u beyond the last cumulative value: the last kept token (the reference's clamp to V-1,
    // runtime/sampler.py:88, could name a token that a filter removed)
    result = last >= 0 ? last : V - 1;
  }
  __syncthreads();
  if (pick_part < 0) {
    if (threadIdx.x == 0) out[blockIdx.x] = result;
    return;
  }
  // 3: the chosen part, again in 32 pieces of whole groups; 4: the chosen piece, group by group
  const int part_base = pick_part * part_len;
  const int piece_len = (((part_len + SEL_WARPS - 1) / SEL_WARPS) + 31) & ~31;
  const double remain = pick_before;
  __syncthreads();
  {
    double s = 0.0;
    int last = -1;
    for_part(row, part_base + warp * piece_len, piece_len, min(part_base + part_len, V), [&](float l, int i) {
      if (is_kept(kp, l, i)) { s += (double)prob(l, mx.v, inv_t); last = i; }
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
    }
    if (lane == 0) { part_sum[warp] = s; part_last[warp] = last; }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double before = 0.0;
    int pick = -1, last_piece = -1;
    for (int w = 0; w < SEL_WARPS; ++w) {
      if (part_last[w] < 0) continue;
      last_piece = w;
      if (before + part_sum[w] >= remain) { pick = w; break; }
      before += part_sum[w];
    }
    pick_need = pick >= 0 ? pick : last_piece;
    // short by rounding against the part's own sum: nothing inside reaches it, and the walk below
    // ends at the piece's last kept token
    pick_before = pick >= 0 ? remain - before : INFINITY;
  }
  __syncthreads();
  if (pick_need < 0) {
    if (threadIdx.x == 0) out[blockIdx.x] = result;
    return;
  }
  if (warp == pick_need) {
    const int base = part_base + warp * piece_len, end = min(part_base + part_len, V);
    double left = pick_before;             // still to be reached
    int answer = -1, last = -1;
    for (int o = 0; o < piece_len && answer < 0; o += 32) {
      const int i = base + o + lane;
      const float l = i < end ? row[i] : 0.f;
      const bool keep = i < end && is_kept(kp, l, i);
      const double p = keep ? (double)prob(l, mx.v, inv_t) : 0.0;
      double incl = p;                     // inclusive scan within the group
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const double n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
      }
      const uint32_t hit = __ballot_sync(0xffffffffu, keep && incl >= left);
      const uint32_t kept_lanes = __ballot_sync(0xffffffffu, keep);
      if (kept_lanes) last = base + o + (31 - __clz(kept_lanes));
      if (hit) answer = base + o + (__ffs(hit) - 1);
      left -= __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) out[blockIdx.x] = answer >= 0 ? answer : (last >= 0 ? last : result);
  }
}

// Repetition penalty in place (runtime/sampler.py:12-33): for each (row, id) pair, a positive logit is
// divided by the row's penalty and a negative one multiplied.  The pairs name each (row, id) once.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, int V, const int* __restrict__ pair_row,
                                          const int* __restrict__ pair_id, const float* __restrict__ pair_penalty, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = pair_id[i];
  if (id < 0 || id >= V) return;
  float* p = logits + (size_t)pair_row[i] * V + id;
  const double v = (double)*p, pen = (double)pair_penalty[i];
  *p = (float)(v < 0 ? v * pen : v / pen);
}

// The same penalty from a table of seen ids kept on the device: seen[slot, id] != 0 once request
// `slot` has consumed token `id`.  mark_seen_kernel records a step's tokens (prompt portions and
// decoded tokens alike) before the step runs; penalty_seen_kernel changes the wanted logits rows of
// requests whose penalty is neither 0 nor 1.  Both read the step's description on the device, so they
// can be part of a captured decode step.
__global__ void mark_seen_kernel(unsigned char* __restrict__ seen, int V, const int* __restrict__ token_ids,
                                 const int* __restrict__ seq_of_token, const int* __restrict__ state_slots, int T, int slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const int id = token_ids[t], slot = state_slots[seq_of_token[t]];
  if (id >= 0 && id < V && slot >= 0 && slot < slots) seen[(size_t)slot * V + id] = 1;
}

__global__ void penalty_seen_kernel(float* __restrict__ logits, int V, const unsigned char* __restrict__ seen,
                                    const int* __restrict__ logit_rows, const int* __restrict__ seq_of_token,
                                    const int* __restrict__ state_slots, const float* __restrict__ penalty, int slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.y;
  const float pf = penalty[row];
  if (!(pf > 0.f) || pf == 1.0f) return;
  const int slot = state_slots[seq_of_token[logit_rows[row]]];
  if (slot < 0 || slot >= slots) return;
  const unsigned char* mine = seen + (size_t)slot * V;
  float* lr = logits + (size_t)row * V;
  const double pen = (double)pf;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += gridDim.x * blockDim.x) {
    if (mine[i]) {
      const double v = (double)lr[i];
      lr[i] = (float)(v < 0 ? v * pen : v / pen);
    }
  }
}

}  // namespace sllm

using namespace sllm;

// temperature may be null (all rows greedy); uniform must hold R doubles when any temperature > 0.
// top_k (int per row, <= 0: none) and top_p (float per row, < 0: none) may be null.
SLLM_EXPORT int sllm_sample_rows(const float* logits, int R, int V, const float* temperature,
                                 const double* uniform, const int* top_k, const float* top_p, int* out, cudaStream_t stream) {
  SLLM_REQUIRE(R >= 0 && V > 0, "sample_rows: bad sizes R=%d V=%d", R, V);
  SLLM_REQUIRE(temperature == nullptr || uniform != nullptr, "sample_rows: temperatures without uniforms");
  SLLM_REQUIRE(temperature != nullptr || (top_k == nullptr && top_p == nullptr), "sample_rows: filters without temperatures");
  if (R == 0) return SLLM_OK;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SAMPLE_SMEM) != cudaSuccess) {
      set_error("sample_rows: cannot raise the shared memory limit");
      return SLLM_ERR_LAUNCH;
    }
    configured = true;
  }
  const int smem = (top_k || top_p) ? SAMPLE_SMEM : 0;
  launch_kernel(sample_rows_kernel, R, SAMPLE_THREADS, smem, stream, logits, V, temperature, uniform, top_k, top_p, out);
  return launch_status("sample_rows");
}

// n (row, id, penalty) triples, each (row, id) named once; logits [R, V] float32 are changed in place
SLLM_EXPORT int sllm_repetition_penalty(float* logits, int R, int V, const int* pair_row, const int* pair_id,
                                        const float* pair_penalty, int n, cudaStream_t stream) {
  SLLM_REQUIRE(R >= 0 && V > 0 && n >= 0, "repetition_penalty: bad sizes R=%d V=%d n=%d", R, V, n);
  if (n == 0 || R == 0) return SLLM_OK;
  launch_kernel(repetition_penalty_kernel, (n + 255) / 256, 256, 0, stream, logits, V, pair_row, pair_id, pair_penalty, n);
  return launch_status("repetition_penalty");
}

// seen [slots, V] bytes; the step's T tokens with the request (row of state_slots) each belongs to
SLLM_EXPORT int sllm_mark_seen(unsigned char* seen, int slots, int V, const int* token_ids, const int* seq_of_token,
                               const int* state_slots, int T, cudaStream_t stream) {
  SLLM_REQUIRE(slots > 0 && V > 0 && T >= 0, "mark_seen: bad sizes slots=%d V=%d T=%d", slots, V, T);
  if (T == 0) return SLLM_OK;
  launch_kernel(mark_seen_kernel, (T + 255) / 256, 256, 0, stream, seen, V, token_ids, seq_of_token, state_slots, T, slots);
  return launch_status("mark_seen");
}

// logits [R, V] float32, changed in place; logit_rows [R] names the token each row belongs to;
// penalty [R] (0 or 1: the row stays as it is)
SLLM_EXPORT int sllm_penalty_seen(float* logits, int R, int V, const unsigned char* seen, int slots, const int* logit_rows,
                                  const int* seq_of_token, const int* state_slots, const float* penalty, cudaStream_t stream) {
  SLLM_REQUIRE(R >= 0 && V > 0 && slots > 0, "penalty_seen: bad sizes R=%d V=%d slots=%d", R, V, slots);
  if (R == 0) return SLLM_OK;
  const int sms = num_sms(), bx = (V + 1023) / 1024 < sms ? (V + 1023) / 1024 : sms;
  launch_kernel(penalty_seen_kernel, dim3(bx, R), 256, 0, stream, logits, V, seen, logit_rows, seq_of_token, state_slots, penalty, slots);
  return launch_status("penalty_seen");
}
