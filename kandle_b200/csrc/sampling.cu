// Device-side next-token sampling: temperature, top-k, top-p (nucleus), multinomial draw, greedy.
//
// The reference downloads the logits of every step (600 KB for a 151 936-entry vocabulary), sorts
// all indices on the host with a comparator and walks the sorted list
// (packages/model-utils/src/sampling/index.ts:103-238, helpers :260-306).  Here one CTA per
// sequence does the same selection without a sort and without the download:
//
//   order      "sorted by logit, descending; equal logits by ascending index" (a stable JS sort)
//              is never materialised.  A prefix of that order is described by a threshold key plus
//              the number of elements equal to the threshold that belong to the prefix (those with
//              the lowest indices).
//   softmax    p_i = fl32(exp(s_i - max) / sum), s_i = fl32(logit_i / T): exp and the division in
//              double, stored as float, the sum in 2^-62 fixed point -- the reference's Float32Array
//              storage with double arithmetic (:260-283).
//   top-k      radix select (4 passes of 8 bits over a monotone 32-bit key) for the k-th element.
//   top-p      the same radix walk over WEIGHTS: per-digit sums of p_i in 2^-62 fixed point
//              (integer adds: exact, order-independent, bit-reproducible), looking for the shortest
//              prefix whose probability mass reaches top_p (:196-214).  Equal keys have equal
//              probabilities, so the count of ties to keep follows from one division.
//   prefix     the shorter of the two prefixes is kept (top-p is evaluated on the top-k survivors,
//              both are prefixes of one order), the rest is zeroed, the survivors renormalised
//              (:216-222) and one token drawn by the running sum in INDEX order against the uniform
//              number r (:291-306), with a block-wide scan in double.
//
// Differences from the reference: r comes from a tensor of uniforms supplied by the caller instead
// of Math.random() (reproducible, graph-replayable); sums that the reference accumulates
// sequentially in double are exact integers here (they agree to ~1e-13, which can only matter when
// a cumulative sum equals top_p or r to 13 digits); the top-10 list the reference returns for display
// is not produced.  Bound: L2/HBM, two streaming passes, four radix passes when a filter is active
// (warp-aggregated histogram updates), and two passes in which every warp walks its own chunk; a
// cluster of four CTAs shares one sequence so that four SMs' worth of loads are in flight per row.
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.cuh"

namespace kd {

constexpr int SMP_THREADS = 1024;
constexpr double SMP_FIX = 4611686018427387904.0;   // 2^62

struct SampleParams {
  const float* logits;   // [B, V], row stride ld
  int64_t ld;
  int V;
  double inv_temp;       // 1 / temperature in double, as the reference computes it
  double temperature;
  int do_sample;
  int top_k;
  double top_p;
  const float* uniforms; // [B]
  float* probs;          // scratch [B, V]
  int64_t* out_ids;      // [B]
  float* out_logprob;    // [B] or NULL
};

__device__ __forceinline__ uint32_t order_key(float x) {
  if (x == 0.f) x = 0.f;                        // -0 and +0 compare equal in the reference's comparator
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);   // larger float -> larger key
}

// Block-wide sums / scans over SMP_THREADS threads; `sh` holds 32 entries per type.
template <typename T>
__device__ __forceinline__ T block_sum(T v, T* sh) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  T t = sh[threadIdx.x & 31];
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* sh) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = sh[threadIdx.x & 31];
  for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
  return t;
}
// Inclusive scan across the block in thread order (fixed tree: deterministic); returns this thread's
// inclusive value, *total = block total.
template <typename T>
__device__ __forceinline__ T block_scan_inclusive(T v, T* sh, T* total) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (int o = 1; o < 32; o <<= 1) {
    const T n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  __syncthreads();
  if (lane == 31) sh[w] = v;
  __syncthreads();
  T ws = sh[lane];
  for (int o = 1; o < 32; o <<= 1) {
    const T n = __shfl_up_sync(0xffffffffu, ws, o);
    if (lane >= o) ws += n;
  }
  const T before = __shfl_sync(0xffffffffu, ws, w > 0 ? w - 1 : 0);
  *total = __shfl_sync(0xffffffffu, ws, 31);
  return v + (w > 0 ? before : (T)0);
}

// Adds `w` into hist[d] for every lane with d < 256, one atomic per distinct digit in the warp.
__device__ __forceinline__ void warp_hist_add_u64(unsigned long long* hist, unsigned int d, unsigned long long w) {
  const unsigned int m = __match_any_sync(0xffffffffu, d);
  // 64-bit sum over the lanes of a group as three 21/21/22-bit pieces (32 x 2^22 fits in 32 bits)
  const unsigned int a = __reduce_add_sync(m, (unsigned int)(w & 0x1fffffu));
  const unsigned int b = __reduce_add_sync(m, (unsigned int)((w >> 21) & 0x1fffffu));
  const unsigned int c = __reduce_add_sync(m, (unsigned int)(w >> 42));
  if (d < 256u && (threadIdx.x & 31) == (unsigned)(__ffs(m) - 1))
    atomicAdd(&hist[d], (unsigned long long)a + ((unsigned long long)b << 21) + ((unsigned long long)c << 42));
}
// Count and weight histograms of the same digit with one match.
__device__ __forceinline__ void warp_hist_add_both(unsigned int* hist_c, unsigned long long* hist_w, unsigned int d,
                                                   unsigned long long w) {
  const unsigned int m = __match_any_sync(0xffffffffu, d);
  const unsigned int a = __reduce_add_sync(m, (unsigned int)(w & 0x1fffffu));
  const unsigned int b = __reduce_add_sync(m, (unsigned int)((w >> 21) & 0x1fffffu));
  const unsigned int c = __reduce_add_sync(m, (unsigned int)(w >> 42));
  if (d < 256u && (threadIdx.x & 31) == (unsigned)(__ffs(m) - 1)) {
    atomicAdd(&hist_c[d], (unsigned int)__popc(m));
    atomicAdd(&hist_w[d], (unsigned long long)a + ((unsigned long long)b << 21) + ((unsigned long long)c << 42));
  }
}
__device__ __forceinline__ void warp_hist_add_u32(unsigned int* hist, unsigned int d) {
  const unsigned int m = __match_any_sync(0xffffffffu, d);
  if (d < 256u && (threadIdx.x & 31) == (unsigned)(__ffs(m) - 1)) atomicAdd(&hist[d], (unsigned int)__popc(m));
}

// One sequence = one thread-block cluster of NC CTAs (NC = 1: a single CTA).  CTA `rank` owns the
// contiguous quarter [v0, v1) of the row; block-wide results are published in the CTA's shared memory,
// one 16-byte slot per exchange site, and read by the other CTAs of the cluster through distributed
// shared memory after a cluster barrier.  A slot is written once per launch, so one barrier per
// exchange suffices; the histograms ping-pong between two sets for the same reason.
template <int NC>
__global__ void __launch_bounds__(SMP_THREADS) sample_kernel(SampleParams p) {
  namespace cg = cooperative_groups;
  __shared__ unsigned long long hist_w[2][256];   // top-p walk: per-digit probability mass (fixed point)
  __shared__ unsigned int hist_pc[2][256];        // top-p walk: per-digit element count
  __shared__ unsigned int hist_kc[2][256];        // top-k walk: per-digit element count
  __shared__ unsigned long long m_w[256];         // the histograms summed over the cluster
  __shared__ unsigned int m_pc[256], m_kc[256];
  __shared__ double sh_d[32];
  __shared__ float sh_f[32];
  __shared__ unsigned long long sh_u[32];
  __shared__ int sh_i[32];
  __shared__ unsigned int s_k[3];              // digit, remaining rank, elements above (this level)
  __shared__ unsigned long long s_pw[2];       // remaining mass, mass of the chosen digit
  __shared__ unsigned int s_p[4];              // digit, elements above, elements in the digit, reached flag
  __shared__ int s_found;
  __shared__ __align__(16) unsigned long long xs[12][2];   // exchange slots (two 8-byte words each)

  const int tid = threadIdx.x, V = p.V;
  int rank = 0;
  if constexpr (NC > 1) rank = (int)cg::this_cluster().block_rank();
  const int row = (int)blockIdx.x / NC;
  auto cluster_sync = [&]() {
    if constexpr (NC > 1) cg::this_cluster().sync();
    else __syncthreads();
  };
  // word `w` of slot `site` as published by CTA `r` of the cluster
  auto peer = [&](int site, int w, int r) -> unsigned long long {
    if constexpr (NC > 1) return cg::this_cluster().map_shared_rank(&xs[site][w], r)[0];
    else return xs[site][w];
  };
  const float* lg = p.logits + (int64_t)row * p.ld;
  float* pr = p.probs + (int64_t)row * V;
  const int Vq = (((V + NC - 1) / NC) + 3) & ~3;
  const int v0 = min(V, rank * Vq), v1 = min(V, v0 + Vq), nv = v1 - v0;
  const bool greedy = !p.do_sample;
  const bool scale = !greedy && p.temperature != 1.0;
  const bool vec = (V % 4 == 0) && ((reinterpret_cast<uintptr_t>(lg) | reinterpret_cast<uintptr_t>(pr)) & 15) == 0;
  // greedy: probabilities of softmax((x - max) / T) (:150); sampling: s = fl32(x * (1/T)), softmax(s - max)
  auto scaled = [&](float x) { return scale ? (float)((double)x * p.inv_temp) : x; };
  // ---- pass 1: maximum (of the raw logits for greedy, of the scaled ones for sampling)
  float mx = -INFINITY;
  if (vec) {
    for (int i = v0 / 4 + tid; i < v1 / 4; i += SMP_THREADS) {
      const float4 v = reinterpret_cast<const float4*>(lg)[i];
      mx = fmaxf(fmaxf(mx, fmaxf(scaled(v.x), scaled(v.y))), fmaxf(scaled(v.z), scaled(v.w)));
    }
  } else {
    for (int i = v0 + tid; i < v1; i += SMP_THREADS) mx = fmaxf(mx, scaled(lg[i]));
  }
  mx = block_max(mx, sh_f);
  if (tid == 0) xs[0][0] = __float_as_uint(mx);
  cluster_sync();
  for (int r = 0; r < NC; ++r) mx = fmaxf(mx, __uint_as_float((unsigned int)peer(0, 0, r)));
  // ---- pass 2: e_i = fl32(exp(.)) kept in `pr`; sum of the FLOAT values in double (the reference
  // sums the stored floats sequentially; the fixed tree order here differs by ~1e-16 relative)
  auto expo = [&](float x) {
    const double d = greedy ? ((double)x - (double)mx) * p.inv_temp : (double)scaled(x) - (double)mx;
    return (float)exp(d);
  };
  double sum_local = 0.0;
  if (vec) {
    for (int i = v0 / 4 + tid; i < v1 / 4; i += SMP_THREADS) {
      const float4 v = reinterpret_cast<const float4*>(lg)[i];
      float4 e;
      e.x = expo(v.x); e.y = expo(v.y); e.z = expo(v.z); e.w = expo(v.w);
      reinterpret_cast<float4*>(pr)[i] = e;
      sum_local += (double)e.x + (double)e.y + (double)e.z + (double)e.w;
    }
  } else {
    for (int i = v0 + tid; i < v1; i += SMP_THREADS) {
      const float e = expo(lg[i]);
      pr[i] = e;
      sum_local += (double)e;
    }
  }
  sum_local = block_sum(sum_local, sh_d);
  if (tid == 0) xs[1][0] = (unsigned long long)__double_as_longlong(sum_local);
  cluster_sync();
  double sum_exp = 0.0;
  for (int r = 0; r < NC; ++r) sum_exp += __longlong_as_double((long long)peer(1, 0, r));   // rank order: deterministic
  auto prob = [&](float e) { return (float)((double)e / sum_exp); };   // p_i = fl32(e_i / sum)

  if (greedy) {
    // argmax with the lowest index on ties = first element of the stable descending sort
    uint32_t bk = 0;
    int bi = 0x7fffffff;
    for (int i = v0 + tid; i < v1; i += SMP_THREADS) {
      const uint32_t k = order_key(lg[i]);
      if (k > bk || (k == bk && i < bi)) { bk = k; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const uint32_t ok2 = __shfl_xor_sync(0xffffffffu, bk, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ok2 > bk || (ok2 == bk && oi < bi)) { bk = ok2; bi = oi; }
    }
    __syncthreads();
    if ((tid & 31) == 0) { sh_u[tid >> 5] = bk; sh_i[tid >> 5] = bi; }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < 32; ++w) {
        const uint32_t k2 = (uint32_t)sh_u[w];
        const int i2 = sh_i[w];
        if (k2 > bk || (k2 == bk && i2 < bi)) { bk = k2; bi = i2; }
      }
      xs[2][0] = bk;
      xs[2][1] = (unsigned long long)(unsigned int)bi;
    }
    cluster_sync();
    if (tid == 0 && rank == 0) {
      for (int r = 0; r < NC; ++r) {
        const uint32_t k2 = (uint32_t)peer(2, 0, r);
        const int i2 = (int)(unsigned int)peer(2, 1, r);
        if (k2 > bk || (k2 == bk && i2 < bi)) { bk = k2; bi = i2; }
      }
      p.out_ids[row] = bi;
      if (p.out_logprob) p.out_logprob[row] = (float)log((double)prob(__ldcg(pr + bi)) + 1e-10);
    }
    cluster_sync();      // nobody leaves while its shared memory may still be read
    return;
  }

  // ---- pass 3: p_i = fl32(e_i / sum)
  if (vec) {
    for (int i = v0 / 4 + tid; i < v1 / 4; i += SMP_THREADS) {
      float4 e = reinterpret_cast<float4*>(pr)[i];
      e.x = prob(e.x); e.y = prob(e.y); e.z = prob(e.z); e.w = prob(e.w);
      reinterpret_cast<float4*>(pr)[i] = e;
    }
  } else {
    for (int i = v0 + tid; i < v1; i += SMP_THREADS) pr[i] = prob(pr[i]);
  }
  __syncthreads();

  // ---- radix select: both thresholds descend in the same four passes over the row.
  // A prefix of the sorted order = (threshold key, how many of the elements equal to it).
  const bool use_k = p.top_k > 0 && p.top_k < V;
  const bool use_p = p.top_p < 1.0;
  uint32_t prefix_k = 0, prefix_p = 0, mask = 0;
  unsigned int rem_c = use_k ? (unsigned)p.top_k : 0u;                                     // rank still to descend (1-based)
  unsigned long long rem_w = use_p ? (unsigned long long)ceil(p.top_p * SMP_FIX) : 0ull;   // mass still to cover
  unsigned int gt_k = 0, eq_k = 0, gt_p = 0, eq_p = 0;
  unsigned long long w_digit_p = 0ull;
  bool p_reached = use_p;     // false: the whole mass stays below top_p (rounding), top-p keeps everything
  int level = 0;
  for (int shift = 24; shift >= 0 && (use_k || use_p); shift -= 8, ++level) {
    const int hs = level & 1;
    if (tid < 256) { hist_w[hs][tid] = 0ull; hist_pc[hs][tid] = 0u; hist_kc[hs][tid] = 0u; }
    __syncthreads();
    const int n_iter = (nv + SMP_THREADS - 1) / SMP_THREADS;
    for (int it = 0; it < n_iter; ++it) {        // every lane of a warp takes part in the warp-wide adds
      const int i = v0 + it * SMP_THREADS + tid;
      unsigned int dk = 256u, dp = 256u;
      unsigned long long w = 0ull;
      if (i < v1) {
        const uint32_t k = order_key(lg[i]);
        if (use_k && (k & mask) == prefix_k) dk = (k >> shift) & 255u;
        if (use_p && p_reached && (k & mask) == prefix_p) {
          dp = (k >> shift) & 255u;
          w = (unsigned long long)((double)pr[i] * SMP_FIX);
        }
      }
      if (__all_sync(0xffffffffu, dk == 256u && dp == 256u)) continue;   // no candidate in this warp
      if (use_k) warp_hist_add_u32(hist_kc[hs], dk);
      if (use_p && p_reached) warp_hist_add_both(hist_pc[hs], hist_w[hs], dp, w);
    }
    cluster_sync();
    // every CTA sums the cluster's histograms (integers: order-independent) and walks them itself
    if (tid < 256) {
      unsigned long long w = 0ull;
      unsigned int pc = 0u, kc = 0u;
      for (int r = 0; r < NC; ++r) {
        if constexpr (NC > 1) {
          w += cg::this_cluster().map_shared_rank(&hist_w[hs][tid], r)[0];
          pc += cg::this_cluster().map_shared_rank(&hist_pc[hs][tid], r)[0];
          kc += cg::this_cluster().map_shared_rank(&hist_kc[hs][tid], r)[0];
        } else {
          w += hist_w[hs][tid]; pc += hist_pc[hs][tid]; kc += hist_kc[hs][tid];
        }
      }
      m_w[tid] = w; m_pc[tid] = pc; m_kc[tid] = kc;
    }
    __syncthreads();
    if (tid == 0 && use_k) {
      unsigned int above = 0;
      int d = 255;
      for (; d > 0; --d) {
        if (above + m_kc[d] >= rem_c) break;
        above += m_kc[d];
      }
      s_k[0] = (unsigned)d; s_k[1] = rem_c - above; s_k[2] = above;
    }
    if (tid == 32 && use_p && p_reached) {
      unsigned long long above = 0ull;
      unsigned int above_c = 0;
      int d = 255;
      bool hit = false;
      for (; d >= 0; --d) {
        if (above + m_w[d] >= rem_w) { hit = true; break; }
        above += m_w[d];
        above_c += m_pc[d];
      }
      s_p[3] = hit ? 1u : 0u;
      if (hit) { s_p[0] = (unsigned)d; s_p[1] = above_c; s_p[2] = m_pc[d]; s_pw[0] = rem_w - above; s_pw[1] = m_w[d]; }
    }
    __syncthreads();
    if (use_k) {
      prefix_k |= s_k[0] << shift;
      rem_c = s_k[1];
      gt_k += s_k[2];
      eq_k = m_kc[s_k[0]];
    }
    if (use_p && p_reached) {
      if (!s_p[3]) p_reached = false;
      else {
        prefix_p |= s_p[0] << shift;
        gt_p += s_p[1];
        eq_p = s_p[2];
        rem_w = s_pw[0];
        w_digit_p = s_pw[1];
      }
    }
    mask |= 255u << shift;
    __syncthreads();
  }
  // Prefix lengths.  top-k: of the eq_k elements equal to its threshold the first rem_c belong to the
  // prefix.  top-p: the ties all have the same probability w, so ceil(rem_w / w) of them are needed.
  uint32_t fkey = 0;
  unsigned int f_eq = 0xffffffffu, f_eq_total = 0;
  {
    unsigned long long len_k = 0xffffffffffffffffull, len_p = 0xffffffffffffffffull;
    unsigned int neq_k = 0, neq_p = 0;
    if (use_k) { neq_k = rem_c < eq_k ? rem_c : eq_k; len_k = (unsigned long long)gt_k + neq_k; }
    if (use_p && p_reached) {
      const unsigned long long w_eq = eq_p > 0 ? w_digit_p / eq_p : 0ull;
      unsigned long long need = w_eq > 0 ? (rem_w + w_eq - 1) / w_eq : eq_p;
      if (need < 1) need = 1;
      neq_p = need < eq_p ? (unsigned int)need : eq_p;
      len_p = (unsigned long long)gt_p + neq_p;
    }
    if (use_k && len_k <= len_p) { fkey = prefix_k; f_eq = neq_k; f_eq_total = eq_k; }
    else if (use_p && p_reached) { fkey = prefix_p; f_eq = neq_p; f_eq_total = eq_p; }
  }
  const bool filtered = f_eq != 0xffffffffu;
  const bool partial_tie = filtered && f_eq < f_eq_total;   // only some of the ties survive: rank them by index

  // From here on every WARP owns one contiguous chunk of this CTA's part of the row (a multiple of
  // 32 elements, read 32 at a time), so that ranks and running sums in INDEX order need one scan over
  // the warps of the CTA and one over the CTAs of the cluster.
  const int warp = tid >> 5, lane = tid & 31;
  const int C = ((nv + 31) / 32 + 31) / 32 * 32;
  const int c0 = min(v1, v0 + warp * C), c1 = min(v1, c0 + C);
  const unsigned int lt_mask = (1u << lane) - 1u;

  // ---- pass A: zero everything outside the prefix (pr <- p_i or 0), sum the survivors
  int eq_before = 0;
  if (partial_tie) {      // (uniform over the cluster: every CTA derived the same thresholds)
    int cnt = 0;
    for (int i = c0 + lane; i < c1; i += 32) cnt += order_key(lg[i]) == fkey;
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    __syncthreads();
    if (lane == 0) sh_i[warp] = cnt;
    __syncthreads();
    int cta_total = 0;
    for (int w = 0; w < 32; ++w) { if (w < warp) eq_before += sh_i[w]; cta_total += sh_i[w]; }
    if (tid == 0) xs[4][0] = (unsigned long long)(unsigned int)cta_total;
    cluster_sync();
    for (int r = 0; r < rank; ++r) eq_before += (int)(unsigned int)peer(4, 0, r);
  }
  unsigned long long kept_w = 0ull;
  for (int b0 = c0; b0 < c1; b0 += 32) {
    const int i = b0 + lane;
    bool keep = i < c1;
    float pi = 0.f;
    uint32_t k = 0;
    if (i < c1) { pi = pr[i]; if (filtered) k = order_key(lg[i]); }
    if (filtered && i < c1 && k < fkey) keep = false;
    if (partial_tie) {
      const unsigned int eqm = __ballot_sync(0xffffffffu, i < c1 && k == fkey);
      if (i < c1 && k == fkey) keep = (unsigned)(eq_before + __popc(eqm & lt_mask)) < f_eq;
      eq_before += __popc(eqm);
    }
    if (i < c1) {
      if (!keep) { pi = 0.f; pr[i] = 0.f; }
      kept_w += (unsigned long long)((double)pi * SMP_FIX);
    }
  }
  kept_w = block_sum(kept_w, sh_u);
  if (tid == 0) xs[5][0] = kept_w;
  cluster_sync();
  kept_w = 0ull;
  for (int r = 0; r < NC; ++r) kept_w += peer(5, 0, r);
  const double prob_sum = (double)kept_w / SMP_FIX;
  auto renorm = [&](float pi) { return prob_sum > 0.0 ? (float)((double)pi / prob_sum) : pi; };   // :217-222

  // ---- pass B: first index with r < running sum of the renormalised probabilities (:291-298)
  const double r = (double)p.uniforms[row];
  double local = 0.0;
  int last_nonzero = -1;
  for (int i = c0 + lane; i < c1; i += 32) {
    const float q = renorm(pr[i]);
    local += (double)q;
    if (q > 0.f) last_nonzero = i;
  }
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);   // this warp's chunk total
  for (int o = 16; o > 0; o >>= 1) last_nonzero = max(last_nonzero, __shfl_xor_sync(0xffffffffu, last_nonzero, o));
  __syncthreads();
  if (lane == 0) { sh_d[warp] = local; sh_i[warp] = last_nonzero; }
  if (tid == 0) s_found = 0x7fffffff;
  __syncthreads();
  double before = 0.0, cta_total = 0.0;
  int cta_last = -1;
  for (int w = 0; w < 32; ++w) {
    if (w < warp) before += sh_d[w];
    cta_total += sh_d[w];
    cta_last = max(cta_last, sh_i[w]);
  }
  if (tid == 0) {
    xs[6][0] = (unsigned long long)__double_as_longlong(cta_total);
    xs[6][1] = (unsigned long long)(unsigned int)cta_last;
  }
  cluster_sync();
  // the CTA whose cumulative end first passes r owns the token; every CTA evaluates the same sums
  double cta_before = 0.0, run = 0.0;
  int owner = -1, cluster_last = -1;
  for (int rr = 0; rr < NC; ++rr) {
    const double tot = __longlong_as_double((long long)peer(6, 0, rr));
    if (rr < rank) cta_before += tot;
    if (owner < 0 && r < run + tot) owner = rr;
    run += tot;
    cluster_last = max(cluster_last, (int)(unsigned int)peer(6, 1, rr));
  }
  if (owner == rank) {
    before += cta_before;
    if (lane == 0 && r < before + local) atomicMin(&s_found, warp);   // the first chunk whose end passes r holds the token
  }
  __syncthreads();
  if (owner == rank && s_found == 0x7fffffff && tid == 0) s_found = 31;   // summation noise at the CTA's end: its last chunk
  __syncthreads();
  if (owner == rank && s_found == warp) {
    int tok = -1;
    double base = before;
    for (int b0 = c0; b0 < c1 && tok < 0; b0 += 32) {
      const int i = b0 + lane;
      double v = i < c1 ? (double)renorm(pr[i]) : 0.0;
      for (int o = 1; o < 32; o <<= 1) {
        const double n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
      }
      const unsigned int hit = __ballot_sync(0xffffffffu, i < c1 && r < base + v);
      if (hit) tok = b0 + __ffs(hit) - 1;
      base += __shfl_sync(0xffffffffu, v, 31);
    }
    if (tok < 0) tok = cta_last >= 0 ? cta_last : v0;   // summation-order noise at the very end: the last non-zero element
    if (lane == 0) {
      p.out_ids[row] = tok;
      if (p.out_logprob) p.out_logprob[row] = (float)log((double)renorm(pr[tok]) + 1e-10);
    }
  }
  if (owner < 0 && rank == 0 && tid == 0) {
    // r beyond the total (rounding): the last token with a non-zero probability, else 0 (:300-306)
    const int tk = cluster_last < 0 ? 0 : cluster_last;
    p.out_ids[row] = tk;
    if (p.out_logprob) p.out_logprob[row] = (float)log((double)renorm(__ldcg(pr + tk)) + 1e-10);
  }
  cluster_sync();      // nobody leaves while its shared memory may still be read
}

}  // namespace kd

using namespace kd;

KD_API int kd_sample(const kd_tensor* logits, double temperature, int top_k, double top_p, int do_sample,
                     const kd_tensor* uniforms, const kd_tensor* out_ids, const kd_tensor* out_logprob) {
  KD_TRY(require_init());
  KD_REQUIRE(logits && out_ids, "null tensor");
  KD_REQUIRE(logits->dtype == KD_F32 && (logits->ndim == 1 || logits->ndim == 2) && logits->strides[logits->ndim - 1] == 1,
             "logits must be fp32 [V] or [B,V] with unit stride along V");
  const int64_t V = logits->shape[logits->ndim - 1];
  const int64_t B = logits->ndim == 2 ? logits->shape[0] : 1;
  KD_REQUIRE(V >= 1 && V <= 0x7fffffff && B >= 0 && B <= 65535, "bad logits shape");
  KD_REQUIRE(temperature > 0.0, "temperature must be positive");
  KD_REQUIRE(top_k >= 0 && top_p > 0.0, "top_k must be >= 0 and top_p > 0");
  KD_REQUIRE(out_ids->dtype == KD_I64 && is_contiguous(out_ids) && numel(out_ids) == B, "out_ids must be contiguous int64 [B]");
  if (out_logprob) KD_REQUIRE(out_logprob->dtype == KD_F32 && is_contiguous(out_logprob) && numel(out_logprob) == B, "out_logprob must be contiguous fp32 [B]");
  if (do_sample) KD_REQUIRE(uniforms && uniforms->dtype == KD_F32 && is_contiguous(uniforms) && numel(uniforms) == B, "uniforms must be contiguous fp32 [B]");
  if (B == 0) return KD_OK;
  SampleParams p{};
  void *pl, *po, *pu = nullptr, *plp = nullptr, *scratch = nullptr;
  KD_TRY(tensor_ptr(logits, &pl));
  KD_TRY(tensor_ptr(out_ids, &po));
  if (do_sample) KD_TRY(tensor_ptr(uniforms, &pu));
  if (out_logprob) KD_TRY(tensor_ptr(out_logprob, &plp));
  KD_TRY(get_workspace((uint64_t)B * V * sizeof(float), &scratch));
  p.logits = static_cast<const float*>(pl);
  p.ld = logits->ndim == 2 ? logits->strides[0] : V;
  p.V = (int)V;
  p.temperature = temperature;
  p.inv_temp = 1.0 / temperature;
  p.do_sample = do_sample;
  p.top_k = top_k;
  p.top_p = top_p;
  p.uniforms = static_cast<const float*>(pu);
  p.probs = static_cast<float*>(scratch);
  p.out_ids = static_cast<int64_t*>(po);
  p.out_logprob = static_cast<float*>(plp);
  // a cluster of four CTAs per sequence when that still fits the machine; a single CTA otherwise
  if (B * 4 <= 4 * (int64_t)ctx().sm_count && V >= 16384) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(B * 4));
    cfg.blockDim = dim3(SMP_THREADS);
    cfg.stream = ctx().stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 4;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    KD_CUDA_CHECK(cudaLaunchKernelEx(&cfg, sample_kernel<4>, p));
  } else {
    sample_kernel<1><<<(unsigned)B, SMP_THREADS, 0, ctx().stream>>>(p);
  }
  return after_launch("sample_kernel");
}
