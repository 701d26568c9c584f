// Fused bf16 kernels for the pieces of a decoder layer that sit between the GEMMs and attention.
// Each replaces a run of eager operator calls of the reference (cited per kernel).  All of them are
// HBM-bound map / row-reduction kernels: 16-byte accesses where the layout allows, warp-shuffle
// reductions, fp32 arithmetic, one rounding to bf16 at the output.
//
// Several take their input either as a bf16 matrix or as fp32 split-K partial sums
// [splits][rows][cols] written by the skinny decode GEMM, which they add up on the fly.
#include <algorithm>

#include "common.cuh"
#include "kernels.cuh"

namespace kd {

// ----------------------------------------------------------------------------- RoPE tables
// cos/sin [S, D/2] in fp32: angle = f32(pos) * inv_freq in fp32, as the reference computes it on the
// device (packages/model-utils/src/rope.ts:192-261: mul(int32 positions, f32 inv_freq) -> cos/sin;
// the duplicated halves of cat(freqs, freqs) are not stored).  cosf/sinf are the accurate versions:
// angles reach thousands of radians.
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, const int* __restrict__ pos_dev, int pos_host,
                                  int seq, int half, float* __restrict__ cos_out, float* __restrict__ sin_out) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= seq * half) return;
  const int s = i / half, e = i - s * half;
  const int pos0 = pos_dev ? *pos_dev : pos_host;
  const float ang = (float)(pos0 + s) * inv_freq[e];
  cos_out[i] = cosf(ang);
  sin_out[i] = sinf(ang);
}

// ----------------------------------------------------------------------------- q/k-norm + RoPE + cache write
// Replaces, per layer: view -> rms_norm(q), rms_norm(k) over head_dim -> permute+contiguous x3 ->
// applyRotaryPosEmbDirect (16 pointwise/copy calls) -> StaticKVCache.update (2 copy_ calls)
// (packages/model-utils/src/attention/gqa.ts:274-322, rope.ts:546-644, kv-cache.ts:180-188).
struct QkvRopeParams {
  int tokens, S, Hq, Hkv;
  int splits;            // 0: bf16 source; >0: fp32 partials [splits][tokens][Ntot]
  float eps;
  int64_t kc_b, kc_h, kc_s;   // cache strides (elements)
  int max_s;
  int pos_host;
  // paged cache: the "cache" tensors are pools [pages,Hkv,128,D] and the page of position `pos` of
  // sequence b is table[b * max_pages + pos / 128] (NULL: contiguous [B,Hkv,maxS,D])
  const int* table;
  int max_pages;
};

template <int V>
struct VecF { float v[V]; };

// Loads V consecutive elements starting at element index `e` of a bf16 row or of the sum of fp32
// partial rows (rows are `stride` elements apart in the partial case).
template <int V>
__device__ __forceinline__ VecF<V> load_src(const void* src, int splits, int64_t row_off, int64_t split_stride, int e) {
  VecF<V> r;
  if (splits == 0) {
    const __nv_bfloat16* s = static_cast<const __nv_bfloat16*>(src) + row_off + e;
    if (V == 4) {
      const uint2 u = *reinterpret_cast<const uint2*>(s);
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
      for (int i = 0; i < V; ++i) r.v[i] = __bfloat162float(h[i]);
    } else {
      const uint32_t u = *reinterpret_cast<const uint32_t*>(s);
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
      for (int i = 0; i < V; ++i) r.v[i] = __bfloat162float(h[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) r.v[i] = 0.f;
    for (int sp = 0; sp < splits; ++sp) {
      const float* s = static_cast<const float*>(src) + sp * split_stride + row_off + e;
      if (V == 4) {
        const float4 f = *reinterpret_cast<const float4*>(s);
        r.v[0] += f.x; r.v[1] += f.y; r.v[2] += f.z; r.v[3] += f.w;
      } else {
        const float2 f = *reinterpret_cast<const float2*>(s);
        r.v[0] += f.x; r.v[1] += f.y;
      }
    }
  }
  return r;
}

template <int V>
__device__ __forceinline__ void store_bf16(__nv_bfloat16* dst, const float* v) {
  if (V == 4) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(dst) = u;
  } else {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<uint32_t*>(&a);
  }
}

// Half a warp (16 lanes) per (token, head).  Lane l holds V = D/32 consecutive elements of the
// first half of the head, [V*l, V*l+V), and the V elements D/2 further on, i.e. both members of
// each rotation pair (i, i + D/2); every access is one 4- or 8-byte (bf16) / 8- or 16-byte (fp32) vector.
template <int D>
__global__ void qkv_norm_rope_kernel(const void* __restrict__ src, const void* __restrict__ qw, int dt_qw,
                                     const void* __restrict__ kw, int dt_kw, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ q_out,
                                     __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                     const int* __restrict__ pos_dev, QkvRopeParams p, int* __restrict__ err) {
  pdl_wait();
  pdl_trigger();
  constexpr int V = D / 32;
  constexpr int HALF = D / 2;
  const int l16 = threadIdx.x & 15;
  // grid: x = token, y = group of 16 heads; 16 lanes per (token, head)
  const int heads = p.Hq + 2 * p.Hkv;
  const int token = blockIdx.x;
  const int head_raw = blockIdx.y * 16 + (threadIdx.x >> 4);
  const bool live = head_raw < heads;
  const int head = live ? head_raw : 0;
  const int64_t ntot = (int64_t)heads * D;
  const int64_t row_off = (int64_t)token * ntot + (int64_t)head * D;
  const int64_t split_stride = (int64_t)p.tokens * ntot;
  const int e0 = V * l16;
  VecF<V> x1 = load_src<V>(src, p.splits, row_off, split_stride, e0);
  VecF<V> x2 = load_src<V>(src, p.splits, row_off, split_stride, HALF + e0);
  const int b = token / p.S, s_idx = token - b * p.S;
  const bool is_q = head < p.Hq, is_k = !is_q && head < p.Hq + p.Hkv;
  // RMSNorm over head_dim: y = (x * (1/sqrt(mean(x^2)+eps))) * w   (normalize/shaderBuilder.ts:343-415)
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < V; ++i) ss += x1.v[i] * x1.v[i] + x2.v[i] * x2.v[i];
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // stays inside the 16-lane half
  if (!live) return;
  if (is_q || is_k) {
    const float sc = 1.0f / sqrtf(ss / (float)D + p.eps);
    const void* w = is_q ? qw : kw;
    const int dtw = is_q ? dt_qw : dt_kw;
    const VecF<V> w1 = load_src<V>(w, dtw == KD_BF16 ? 0 : 1, 0, 0, e0);
    const VecF<V> w2 = load_src<V>(w, dtw == KD_BF16 ? 0 : 1, 0, 0, HALF + e0);
    const VecF<V> c = load_src<V>(cos_t, 1, (int64_t)s_idx * HALF, 0, e0);
    const VecF<V> sn = load_src<V>(sin_t, 1, (int64_t)s_idx * HALF, 0, e0);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float y1 = (x1.v[i] * sc) * w1.v[i];
      const float y2 = (x2.v[i] * sc) * w2.v[i];
      // rotate: out[i] = y[i] cos - y[i+D/2] sin ; out[i+D/2] = y[i+D/2] cos + y[i] sin
      x1.v[i] = y1 * c.v[i] - y2 * sn.v[i];
      x2.v[i] = y2 * c.v[i] + y1 * sn.v[i];
    }
  }
  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out + ((int64_t)token * p.Hq + head) * D;
  } else {
    const int pos0 = pos_dev ? *pos_dev : p.pos_host;
    const int pos = pos0 + s_idx;
    if (pos < 0 || pos >= p.max_s) {  // never write outside the cache; report instead
      if (l16 == 0 && atomicCAS(err, 0, 102) == 0) { err[1] = pos; err[2] = p.max_s; }
      return;
    }
    const int hk = is_k ? head - p.Hq : head - p.Hq - p.Hkv;
    int64_t outer = b, row = pos;
    if (p.table) {
      outer = p.table[(int64_t)b * p.max_pages + pos / 128];
      row = pos % 128;
    }
    dst = (is_k ? k_cache : v_cache) + outer * p.kc_b + (int64_t)hk * p.kc_h + row * p.kc_s;
  }
  store_bf16<V>(dst + e0, x1.v);
  store_bf16<V>(dst + HALF + e0, x2.v);
}

// ----------------------------------------------------------------------------- SiLU(gate) * up
// Replaces silu + mul after the gate/up projections (packages/model-utils/src/mlp/swiglu.ts:121-131;
// silu formula packages/backend-webgpu/src/kernels/pointwise/ops.ts:299).  Columns of the source
// interleave 16 gate values with the 16 matching up values (the fused weight's row order).
__global__ void swiglu_kernel(const void* __restrict__ src, int splits, int rows, int inter,
                              __nv_bfloat16* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)rows * inter) return;
  const int m = (int)(i / inter), j = (int)(i - (int64_t)m * inter);
  const int64_t gcol = (int64_t)(j >> 4) * 32 + (j & 15);
  const int64_t ncol = 2 * (int64_t)inter;
  float g = 0.f, u = 0.f;
  if (splits == 0) {
    const __nv_bfloat16* s = static_cast<const __nv_bfloat16*>(src) + (int64_t)m * ncol;
    g = __bfloat162float(s[gcol]);
    u = __bfloat162float(s[gcol + 16]);
  } else {
    for (int sp = 0; sp < splits; ++sp) {
      const float* s = static_cast<const float*>(src) + ((int64_t)sp * rows + m) * ncol;
      g += s[gcol];
      u += s[gcol + 16];
    }
  }
  const float a = g / (1.0f + expf(-fminf(fmaxf(g, -88.f), 88.f)));
  out[i] = __float2bfloat16_rn(a * u);
}

// ----------------------------------------------------------------------------- (residual +) x -> RMSNorm
// Replaces the residual `add` followed by the next `rms_norm`
// (packages/model-utils/src/qwen3/decoder_layer.ts:224-232).  One CTA per row, 16-byte accesses,
// the row stays in registers between the reduction and the write.  The sum is rounded to bf16 first
// and the norm is taken of the rounded value, which is what the unfused sequence sees.
constexpr int ARN_THREADS = 128;
constexpr int ARN_MAXV = 4;  // vectors of 8 elements per thread: rows up to 4096 wide stay in registers

__global__ void __launch_bounds__(ARN_THREADS) add_rmsnorm_kernel(const void* __restrict__ src, int splits,
                                                                   const void* __restrict__ resid, int resid_f32,
                                                                   const void* __restrict__ w, int dt_w, float eps,
                                                                   void* __restrict__ sum_out, int sum_f32,
                                                                   __nv_bfloat16* __restrict__ norm_out, int rows, int n) {
  __shared__ float red[ARN_THREADS / 32];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const int nvec = n / 8;
  float v[ARN_MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int t = 0; t < ARN_MAXV; ++t) {
    const int vi = threadIdx.x + t * ARN_THREADS;
    if (vi < nvec) {
      if (splits == 0) {
        const uint4 u = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(src) + (int64_t)row * n)[vi];
        const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[t][e] = __bfloat162float(h[e]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[t][e] = 0.f;
        for (int sp = 0; sp < splits; ++sp) {
          const float4* s = reinterpret_cast<const float4*>(static_cast<const float*>(src) + ((int64_t)sp * rows + row) * n) + vi * 2;
          const float4 a = s[0], b = s[1];
          v[t][0] += a.x; v[t][1] += a.y; v[t][2] += a.z; v[t][3] += a.w;
          v[t][4] += b.x; v[t][5] += b.y; v[t][6] += b.z; v[t][7] += b.w;
        }
      }
      if (resid) {
        if (resid_f32) {
          const float4* rp = reinterpret_cast<const float4*>(static_cast<const float*>(resid) + (int64_t)row * n) + vi * 2;
          const float4 a = rp[0], b = rp[1];
          v[t][0] += a.x; v[t][1] += a.y; v[t][2] += a.z; v[t][3] += a.w;
          v[t][4] += b.x; v[t][5] += b.y; v[t][6] += b.z; v[t][7] += b.w;
        } else {
          const uint4 u = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(resid) + (int64_t)row * n)[vi];
          const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[t][e] += __bfloat162float(h[e]);
        }
      }
      if (sum_out && sum_f32) {
        float4* sp = reinterpret_cast<float4*>(static_cast<float*>(sum_out) + (int64_t)row * n) + vi * 2;
        sp[0] = make_float4(v[t][0], v[t][1], v[t][2], v[t][3]);
        sp[1] = make_float4(v[t][4], v[t][5], v[t][6], v[t][7]);
      } else if ((splits != 0 || resid) && !(sum_out == nullptr && sum_f32)) {
        // bf16 stream: round the sum first and normalise the rounded value, as the unfused sequence does
        uint4 o;
        __nv_bfloat16* ho = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          ho[e] = __float2bfloat16_rn(v[t][e]);
          v[t][e] = __bfloat162float(ho[e]);
        }
        if (sum_out) reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(sum_out) + (int64_t)row * n)[vi] = o;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[t][e] * v[t][e];
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < ARN_THREADS / 32; ++i) tot += red[i];
  const float sc = 1.0f / sqrtf(tot / (float)n + eps);
#pragma unroll
  for (int t = 0; t < ARN_MAXV; ++t) {
    const int vi = threadIdx.x + t * ARN_THREADS;
    if (vi < nvec) {
      uint4 o;
      __nv_bfloat16* ho = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
      for (int e = 0; e < 8; ++e) ho[e] = __float2bfloat16_rn((v[t][e] * sc) * load_float(w, dt_w, vi * 8 + e));
      reinterpret_cast<uint4*>(norm_out + (int64_t)row * n)[vi] = o;
    }
  }
}

// Many-row variant (prefill): one warp per row, 8 rows per CTA, no shared memory.  Same arithmetic.
constexpr int RWN_MAXV = 16;  // vectors of 8 per lane: rows up to 4096 wide
template <int NV>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const void* __restrict__ src, int src_f32,
                                                            const void* __restrict__ resid, int resid_f32,
                                                            const void* __restrict__ w, int dt_w, float eps,
                                                            void* __restrict__ sum_out, int sum_f32, int round_sum,
                                                            __nv_bfloat16* __restrict__ norm_out, int64_t rows, int n) {
  const int lane = threadIdx.x & 31;
  const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  const int nvec = n / 8;
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int t = 0; t < NV; ++t) {
    const int vi = lane + t * 32;
    if (vi < nvec) {
      if (src_f32) {
        const float4* sp = reinterpret_cast<const float4*>(static_cast<const float*>(src) + row * n) + vi * 2;
        const float4 a = sp[0], b = sp[1];
        v[t][0] = a.x; v[t][1] = a.y; v[t][2] = a.z; v[t][3] = a.w; v[t][4] = b.x; v[t][5] = b.y; v[t][6] = b.z; v[t][7] = b.w;
      } else {
        const uint4 u = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(src) + row * n)[vi];
        const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[t][e] = __bfloat162float(h[e]);
      }
      if (resid) {
        if (resid_f32) {
          const float4* rp = reinterpret_cast<const float4*>(static_cast<const float*>(resid) + row * n) + vi * 2;
          const float4 a = rp[0], b = rp[1];
          v[t][0] += a.x; v[t][1] += a.y; v[t][2] += a.z; v[t][3] += a.w; v[t][4] += b.x; v[t][5] += b.y; v[t][6] += b.z; v[t][7] += b.w;
        } else {
          const uint4 u = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(resid) + row * n)[vi];
          const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[t][e] += __bfloat162float(h[e]);
        }
      }
      if (sum_out && sum_f32) {
        float4* sp = reinterpret_cast<float4*>(static_cast<float*>(sum_out) + row * n) + vi * 2;
        sp[0] = make_float4(v[t][0], v[t][1], v[t][2], v[t][3]);
        sp[1] = make_float4(v[t][4], v[t][5], v[t][6], v[t][7]);
      } else if (round_sum) {
        uint4 o;
        __nv_bfloat16* ho = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          ho[e] = __float2bfloat16_rn(v[t][e]);
          v[t][e] = __bfloat162float(ho[e]);
        }
        if (sum_out) reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(sum_out) + row * n)[vi] = o;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[t][e] * v[t][e];
    }
  }
  ss = warp_sum(ss);
  const float sc = 1.0f / sqrtf(ss / (float)n + eps);
#pragma unroll
  for (int t = 0; t < NV; ++t) {
    const int vi = lane + t * 32;
    if (vi < nvec) {
      uint4 o;
      __nv_bfloat16* ho = reinterpret_cast<__nv_bfloat16*>(&o);
      float wv[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) wv[e] = 1.f;
      if (dt_w == KD_BF16) {
        const uint4 u = reinterpret_cast<const uint4*>(w)[vi];
        const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
        for (int e = 0; e < 8; ++e) wv[e] = __bfloat162float(h[e]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) wv[e] = load_float(w, dt_w, vi * 8 + e);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ho[e] = __float2bfloat16_rn((v[t][e] * sc) * wv[e]);
      reinterpret_cast<uint4*>(norm_out + row * n)[vi] = o;
    }
  }
}

__global__ void increment_i32_kernel(int* p, int delta) {
  pdl_wait();
  pdl_trigger();
  *p += delta;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace kd

using namespace kd;

KD_API int kd_rope_table(const kd_tensor* inv_freq, const kd_tensor* pos, int start_pos, int seq_len,
                         const kd_tensor* cos_out, const kd_tensor* sin_out) {
  KD_TRY(require_init());
  KD_REQUIRE(inv_freq && cos_out && sin_out, "null tensor");
  KD_REQUIRE(inv_freq->dtype == KD_F32 && inv_freq->ndim == 1 && is_contiguous(inv_freq), "inv_freq must be fp32 [D/2]");
  const int half = (int)inv_freq->shape[0];
  KD_REQUIRE(seq_len >= 0, "negative sequence length");
  KD_REQUIRE(cos_out->dtype == KD_F32 && sin_out->dtype == KD_F32 && is_contiguous(cos_out) && is_contiguous(sin_out) &&
                 numel(cos_out) == (int64_t)seq_len * half && numel(sin_out) == (int64_t)seq_len * half,
             "cos/sin outputs must be contiguous fp32 [seq_len, D/2]");
  const int* pos_dev = nullptr;
  if (pos) {
    KD_REQUIRE(pos->dtype == KD_I32 && numel(pos) == 1, "pos must be a device int32 scalar");
    void* pp = nullptr;
    KD_TRY(tensor_ptr(pos, &pp));
    pos_dev = static_cast<const int*>(pp);
  }
  if (seq_len == 0) return KD_OK;
  void *pi = nullptr, *pc = nullptr, *ps = nullptr;
  KD_TRY(tensor_ptr(inv_freq, &pi));
  KD_TRY(tensor_ptr(cos_out, &pc));
  KD_TRY(tensor_ptr(sin_out, &ps));
  const int total = seq_len * half;
  KD_CUDA_CHECK(launch_ex(rope_table_kernel, dim3((total + 255) / 256), dim3(256), 0, (const float*)pi, pos_dev, start_pos, seq_len,
                          half, (float*)pc, (float*)ps));
  return after_launch("rope_table_kernel");
}

static int qkv_norm_rope_cachewrite(const kd_tensor* qkv, const kd_tensor* q_norm_weight, const kd_tensor* k_norm_weight,
                                    float eps, const kd_tensor* cos, const kd_tensor* sin, const kd_tensor* k_cache,
                                    const kd_tensor* v_cache, const kd_tensor* block_table, const kd_tensor* pos, int start_pos,
                                    const kd_tensor* q_out) {
  KD_TRY(require_init());
  KD_REQUIRE(qkv && q_norm_weight && k_norm_weight && cos && sin && k_cache && v_cache && q_out, "null tensor");
  KD_REQUIRE(q_out->ndim == 4 && q_out->dtype == KD_BF16 && is_contiguous(q_out), "q_out must be contiguous bf16 [B,S,Hq,D]");
  KD_REQUIRE(k_cache->ndim == 4 && v_cache->ndim == 4 && k_cache->dtype == KD_BF16 && v_cache->dtype == KD_BF16,
             "caches must be bf16 [B,Hkv,maxS,D]");
  const int B = (int)q_out->shape[0], S = (int)q_out->shape[1], Hq = (int)q_out->shape[2], D = (int)q_out->shape[3];
  const int Hkv = (int)k_cache->shape[1];
  KD_REQUIRE(D == 64 || D == 128, "head_dim must be 64 or 128");
  const int* table = nullptr;
  int max_pages = 0;
  if (block_table) {
    KD_REQUIRE(block_table->dtype == KD_I32 && block_table->ndim == 2 && is_contiguous(block_table) && block_table->shape[0] == B,
               "block_table must be a contiguous int32 [B, max_pages] tensor");
    KD_REQUIRE(k_cache->shape[2] == 128, "a paged cache needs pages of 128 rows");
    void* pt = nullptr;
    KD_TRY(tensor_ptr(block_table, &pt));
    table = static_cast<const int*>(pt);
    max_pages = (int)block_table->shape[1];
  }
  const int64_t cache_rows = table ? (int64_t)max_pages * 128 : k_cache->shape[2];
  KD_REQUIRE((table || k_cache->shape[0] == B) && k_cache->shape[3] == D && k_cache->strides[3] == 1, "k_cache shape/stride mismatch");
  for (int i = 0; i < 4; ++i)
    KD_REQUIRE(v_cache->shape[i] == k_cache->shape[i] && v_cache->strides[i] == k_cache->strides[i],
               "v_cache must have k_cache's shape and strides");
  const int64_t tokens = (int64_t)B * S, ntot = (int64_t)(Hq + 2 * Hkv) * D;
  int splits = 0;
  if (qkv->dtype == KD_BF16) {
    KD_REQUIRE(is_contiguous(qkv) && numel(qkv) == tokens * ntot, "qkv must be contiguous bf16 [B,S,(Hq+2Hkv)*D]");
  } else {
    KD_REQUIRE(qkv->dtype == KD_F32 && is_contiguous(qkv) && numel(qkv) % (tokens * ntot) == 0 && numel(qkv) > 0,
               "qkv partials must be contiguous fp32 [splits, B*S, (Hq+2Hkv)*D]");
    splits = (int)(numel(qkv) / (tokens * ntot));
  }
  KD_REQUIRE(numel(q_norm_weight) == D && numel(k_norm_weight) == D && is_contiguous(q_norm_weight) && is_contiguous(k_norm_weight),
             "q/k norm weights must be contiguous [D]");
  KD_REQUIRE(cos->dtype == KD_F32 && sin->dtype == KD_F32 && is_contiguous(cos) && is_contiguous(sin) &&
                 numel(cos) == (int64_t)S * (D / 2) && numel(sin) == (int64_t)S * (D / 2),
             "cos/sin must be contiguous fp32 [S, D/2]");
  const int* pos_dev = nullptr;
  if (pos) {
    KD_REQUIRE(pos->dtype == KD_I32 && numel(pos) == 1, "pos must be a device int32 scalar");
    void* pp = nullptr;
    KD_TRY(tensor_ptr(pos, &pp));
    pos_dev = static_cast<const int*>(pp);
  } else {
    KD_REQUIRE(start_pos >= 0 && start_pos + S <= cache_rows, "Cache overflow: trying to write to position %d-%d, but maxSeqLen is %lld",
               start_pos, start_pos + S, (long long)cache_rows);
  }
  if (tokens == 0) return KD_OK;
  void *psrc, *pqw, *pkw, *pcos, *psin, *pkc, *pvc, *pqo;
  KD_TRY(tensor_ptr(qkv, &psrc));
  KD_TRY(tensor_ptr(q_norm_weight, &pqw));
  KD_TRY(tensor_ptr(k_norm_weight, &pkw));
  KD_TRY(tensor_ptr(cos, &pcos));
  KD_TRY(tensor_ptr(sin, &psin));
  KD_TRY(tensor_ptr(k_cache, &pkc));
  KD_TRY(tensor_ptr(v_cache, &pvc));
  KD_TRY(tensor_ptr(q_out, &pqo));
  QkvRopeParams p{};
  p.tokens = (int)tokens; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.splits = splits; p.eps = eps;
  p.kc_b = k_cache->strides[0]; p.kc_h = k_cache->strides[1]; p.kc_s = k_cache->strides[2];
  p.max_s = (int)cache_rows;
  p.pos_host = start_pos;
  p.table = table;
  p.max_pages = max_pages;
  const int threads = 256;                          // 16 heads of one token per CTA
  const dim3 blocks((unsigned)tokens, (unsigned)((Hq + 2 * Hkv + 15) / 16));
  KD_REQUIRE((q_norm_weight->dtype == KD_BF16 || q_norm_weight->dtype == KD_F32) &&
                 (k_norm_weight->dtype == KD_BF16 || k_norm_weight->dtype == KD_F32),
             "q/k norm weights must be bf16 or fp32");
  KD_REQUIRE((reinterpret_cast<uintptr_t>(pqw) & 15) == 0 && (reinterpret_cast<uintptr_t>(pkw) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(pcos) & 15) == 0 && (reinterpret_cast<uintptr_t>(psin) & 15) == 0,
             "norm weights and cos/sin tables must be 16-byte aligned");
  KD_REQUIRE(k_cache->strides[0] % 4 == 0 && k_cache->strides[1] % 4 == 0 && k_cache->strides[2] % 4 == 0,
             "cache strides must be multiples of 4 elements");
  KD_REQUIRE((reinterpret_cast<uintptr_t>(psrc) & 15) == 0 && (reinterpret_cast<uintptr_t>(pkc) & 7) == 0 &&
                 (reinterpret_cast<uintptr_t>(pvc) & 7) == 0 && (reinterpret_cast<uintptr_t>(pqo) & 7) == 0,
             "qkv / cache / q_out must be 16- / 8-byte aligned");
  KD_REQUIRE(tokens <= 0x7fffffff, "too many tokens for one launch");
  const void* csrc = psrc;
  const void *cqw = pqw, *ckw = pkw;
  if (D == 128)
    KD_CUDA_CHECK(launch_ex(qkv_norm_rope_kernel<128>, blocks, dim3(threads), 0, csrc, cqw, (int)q_norm_weight->dtype, ckw,
                            (int)k_norm_weight->dtype, (const float*)pcos, (const float*)psin, (__nv_bfloat16*)pqo,
                            (__nv_bfloat16*)pkc, (__nv_bfloat16*)pvc, pos_dev, p, ctx().error_flag));
  else
    KD_CUDA_CHECK(launch_ex(qkv_norm_rope_kernel<64>, blocks, dim3(threads), 0, csrc, cqw, (int)q_norm_weight->dtype, ckw,
                            (int)k_norm_weight->dtype, (const float*)pcos, (const float*)psin, (__nv_bfloat16*)pqo,
                            (__nv_bfloat16*)pkc, (__nv_bfloat16*)pvc, pos_dev, p, ctx().error_flag));
  return after_launch("qkv_norm_rope_kernel");
}

KD_API int kd_qkv_norm_rope_cachewrite(const kd_tensor* qkv, const kd_tensor* q_norm_weight, const kd_tensor* k_norm_weight,
                                       float eps, const kd_tensor* cos, const kd_tensor* sin, const kd_tensor* k_cache,
                                       const kd_tensor* v_cache, const kd_tensor* pos, int start_pos,
                                       const kd_tensor* q_out) {
  return qkv_norm_rope_cachewrite(qkv, q_norm_weight, k_norm_weight, eps, cos, sin, k_cache, v_cache, nullptr, pos, start_pos, q_out);
}

KD_API int kd_qkv_norm_rope_cachewrite_paged(const kd_tensor* qkv, const kd_tensor* q_norm_weight, const kd_tensor* k_norm_weight,
                                             float eps, const kd_tensor* cos, const kd_tensor* sin, const kd_tensor* k_pool,
                                             const kd_tensor* v_pool, const kd_tensor* block_table, const kd_tensor* pos,
                                             int start_pos, const kd_tensor* q_out) {
  KD_REQUIRE(block_table != nullptr, "kd_qkv_norm_rope_cachewrite_paged needs a block table");
  return qkv_norm_rope_cachewrite(qkv, q_norm_weight, k_norm_weight, eps, cos, sin, k_pool, v_pool, block_table, pos, start_pos, q_out);
}

// ----------------------------------------------------------------------------- contiguous K/V rows -> pages
// Rows [0,S) of k_src / v_src [B,Hkv,S,D] go to positions [start_pos, start_pos+S) of a paged cache.
// One thread per 16 bytes.
__global__ void kv_pages_write_kernel(const __nv_bfloat16* __restrict__ ks, const __nv_bfloat16* __restrict__ vs,
                                      __nv_bfloat16* __restrict__ kp, __nv_bfloat16* __restrict__ vp, const int* __restrict__ table,
                                      int max_pages, int B, int Hkv, int S, int D, int start_pos, int64_t ss_b, int64_t ss_h,
                                      int64_t ss_s, int64_t ps_p, int64_t ps_h, int64_t ps_s, int* __restrict__ err) {
  pdl_wait();
  pdl_trigger();
  const int vec = D / 8;
  const int64_t n = (int64_t)B * Hkv * S * vec;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % vec);
    int64_t r = i / vec;
    const int s = (int)(r % S); r /= S;
    const int h = (int)(r % Hkv);
    const int b = (int)(r / Hkv);
    const int pos = start_pos + s;
    if (pos < 0 || pos >= max_pages * 128) {
      if (atomicCAS(err, 0, 102) == 0) { err[1] = pos; err[2] = max_pages * 128; }
      continue;
    }
    const int page = table[(int64_t)b * max_pages + pos / 128];
    const int64_t src = (int64_t)b * ss_b + (int64_t)h * ss_h + (int64_t)s * ss_s + c * 8;
    const int64_t dst = (int64_t)page * ps_p + (int64_t)h * ps_h + (int64_t)(pos % 128) * ps_s + c * 8;
    *reinterpret_cast<uint4*>(kp + dst) = *reinterpret_cast<const uint4*>(ks + src);
    *reinterpret_cast<uint4*>(vp + dst) = *reinterpret_cast<const uint4*>(vs + src);
  }
}

KD_API int kd_kv_pages_write(const kd_tensor* k_src, const kd_tensor* v_src, const kd_tensor* k_pool, const kd_tensor* v_pool,
                             const kd_tensor* block_table, int start_pos) {
  KD_TRY(require_init());
  KD_REQUIRE(k_src && v_src && k_pool && v_pool && block_table, "null tensor");
  KD_REQUIRE(k_src->ndim == 4 && k_pool->ndim == 4 && k_src->dtype == KD_BF16 && v_src->dtype == KD_BF16 && k_pool->dtype == KD_BF16 &&
                 v_pool->dtype == KD_BF16,
             "sources [B,Hkv,S,D] and pools [pages,Hkv,128,D] must be bf16");
  const int B = (int)k_src->shape[0], Hkv = (int)k_src->shape[1], S = (int)k_src->shape[2], D = (int)k_src->shape[3];
  KD_REQUIRE(k_pool->shape[1] == Hkv && k_pool->shape[2] == 128 && k_pool->shape[3] == D && D % 8 == 0, "pool shape does not match the source");
  for (int i = 0; i < 4; ++i) {
    KD_REQUIRE(v_src->shape[i] == k_src->shape[i] && v_src->strides[i] == k_src->strides[i], "v_src must have k_src's shape and strides");
    KD_REQUIRE(v_pool->shape[i] == k_pool->shape[i] && v_pool->strides[i] == k_pool->strides[i], "v_pool must have k_pool's shape and strides");
  }
  KD_REQUIRE(k_src->strides[3] == 1 && k_pool->strides[3] == 1, "unit stride along head_dim required");
  for (int i = 0; i < 3; ++i) KD_REQUIRE(k_src->strides[i] % 8 == 0 && k_pool->strides[i] % 8 == 0, "strides must be multiples of 8 elements");
  KD_REQUIRE(block_table->dtype == KD_I32 && block_table->ndim == 2 && is_contiguous(block_table) && block_table->shape[0] == B,
             "block_table must be a contiguous int32 [B, max_pages] tensor");
  const int max_pages = (int)block_table->shape[1];
  KD_REQUIRE(start_pos >= 0 && start_pos + S <= max_pages * 128, "Cache overflow: trying to write to position %d-%d, but the block table covers %d",
             start_pos, start_pos + S, max_pages * 128);
  if ((int64_t)B * Hkv * S == 0) return KD_OK;
  void *pks, *pvs, *pkp, *pvp, *pt;
  KD_TRY(tensor_ptr(k_src, &pks)); KD_TRY(tensor_ptr(v_src, &pvs)); KD_TRY(tensor_ptr(k_pool, &pkp)); KD_TRY(tensor_ptr(v_pool, &pvp));
  KD_TRY(tensor_ptr(block_table, &pt));
  KD_REQUIRE(((reinterpret_cast<uintptr_t>(pks) | reinterpret_cast<uintptr_t>(pvs) | reinterpret_cast<uintptr_t>(pkp) |
               reinterpret_cast<uintptr_t>(pvp)) & 15) == 0, "operands must be 16-byte aligned");
  const int64_t n = (int64_t)B * Hkv * S * (D / 8);
  const int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)ctx().sm_count * 16);
  KD_CUDA_CHECK(launch_ex(kv_pages_write_kernel, dim3(blocks), dim3(256), 0, (const __nv_bfloat16*)pks, (const __nv_bfloat16*)pvs,
                          (__nv_bfloat16*)pkp, (__nv_bfloat16*)pvp, (const int*)pt, max_pages, B, Hkv, S, D, start_pos, (int64_t)k_src->strides[0],
                          (int64_t)k_src->strides[1], (int64_t)k_src->strides[2], (int64_t)k_pool->strides[0], (int64_t)k_pool->strides[1],
                          (int64_t)k_pool->strides[2], ctx().error_flag));
  return after_launch("kv_pages_write_kernel");
}

KD_API int kd_swiglu(const kd_tensor* gate_up, const kd_tensor* out) {
  KD_TRY(require_init());
  KD_REQUIRE(gate_up && out, "null tensor");
  KD_REQUIRE(out->dtype == KD_BF16 && is_contiguous(out) && out->ndim >= 1, "out must be contiguous bf16 [rows, I]");
  const int64_t inter = out->shape[out->ndim - 1];
  KD_REQUIRE(inter > 0 && inter % 16 == 0, "intermediate size must be a positive multiple of 16");
  const int64_t rows = numel(out) / inter;
  int splits = 0;
  if (gate_up->dtype == KD_BF16) {
    KD_REQUIRE(is_contiguous(gate_up) && numel(gate_up) == rows * inter * 2, "gate_up must be contiguous bf16 [rows, 2I]");
  } else {
    KD_REQUIRE(gate_up->dtype == KD_F32 && is_contiguous(gate_up) && rows > 0 && numel(gate_up) % (rows * inter * 2) == 0,
               "gate_up partials must be contiguous fp32 [splits, rows, 2I]");
    splits = (int)(numel(gate_up) / (rows * inter * 2));
  }
  if (rows == 0) return KD_OK;
  void *ps, *po;
  KD_TRY(tensor_ptr(gate_up, &ps));
  KD_TRY(tensor_ptr(out, &po));
  const int64_t total = rows * inter;
  swiglu_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx().stream>>>(ps, splits, (int)rows, (int)inter, (__nv_bfloat16*)po);
  return after_launch("swiglu_kernel");
}

KD_API int kd_add_rmsnorm(const kd_tensor* x, const kd_tensor* residual, const kd_tensor* weight, float eps,
                          const kd_tensor* sum_out, const kd_tensor* norm_out) {
  KD_TRY(require_init());
  KD_REQUIRE(x && weight && norm_out, "null tensor");
  KD_REQUIRE(norm_out->dtype == KD_BF16 && is_contiguous(norm_out) && norm_out->ndim >= 1, "norm_out must be contiguous bf16");
  const int64_t n = norm_out->shape[norm_out->ndim - 1];
  KD_REQUIRE(n > 0 && n % 8 == 0 && n <= 8 * ARN_THREADS * ARN_MAXV, "row width %lld must be a multiple of 8 and at most %d",
             (long long)n, 8 * ARN_THREADS * ARN_MAXV);
  const int64_t rows = numel(norm_out) / n;
  int splits = 0;
  if (x->dtype == KD_BF16) {
    KD_REQUIRE(is_contiguous(x) && numel(x) == rows * n, "x must be contiguous bf16 [rows, n]");
  } else {
    KD_REQUIRE(x->dtype == KD_F32 && is_contiguous(x) && rows > 0 && numel(x) % (rows * n) == 0 && numel(x) > 0,
               "x partials must be contiguous fp32 [splits, rows, n]");
    splits = (int)(numel(x) / (rows * n));
  }
  KD_REQUIRE(numel(weight) == n && is_contiguous(weight) && is_float_dtype(weight->dtype), "weight must be contiguous [n]");
  if (residual) KD_REQUIRE((residual->dtype == KD_BF16 || residual->dtype == KD_F32) && is_contiguous(residual) && numel(residual) == rows * n, "residual must be contiguous bf16/fp32 [rows, n]");
  if (sum_out) KD_REQUIRE((sum_out->dtype == KD_BF16 || sum_out->dtype == KD_F32) && is_contiguous(sum_out) && numel(sum_out) == rows * n, "sum_out must be contiguous bf16/fp32 [rows, n]");
  // with an fp32 input and no bf16 sum requested the value is normalised unrounded
  const int sum_f32 = sum_out ? (sum_out->dtype == KD_F32) : (x->dtype == KD_F32 && (!residual || residual->dtype == KD_F32));
  if (rows == 0) return KD_OK;
  KD_REQUIRE(rows <= 0x7fffffff, "too many rows");
  void *px, *pw, *pr = nullptr, *ps = nullptr, *pn;
  KD_TRY(tensor_ptr(x, &px));
  KD_TRY(tensor_ptr(weight, &pw));
  KD_TRY(tensor_ptr(norm_out, &pn));
  if (residual) KD_TRY(tensor_ptr(residual, &pr));
  if (sum_out) KD_TRY(tensor_ptr(sum_out, &ps));
  KD_REQUIRE(aligned16(px) && aligned16(pn) && (!pr || aligned16(pr)) && (!ps || aligned16(ps)), "operands must be 16-byte aligned");
  if (rows >= 1024 && splits <= 1 && n <= 8 * 32 * RWN_MAXV) {
    const int round_sum = ((splits != 0 || residual) && !(sum_out == nullptr && sum_f32)) ? 1 : 0;
    KD_REQUIRE((reinterpret_cast<uintptr_t>(pw) & 15) == 0, "weight must be 16-byte aligned");
    if (n <= 8 * 32 * 4)
      rmsnorm_rows_kernel<4><<<(unsigned)((rows + 7) / 8), 256, 0, ctx().stream>>>(
          px, splits == 1, pr, residual ? residual->dtype == KD_F32 : 0, pw, weight->dtype, eps, ps, sum_f32, round_sum,
          (__nv_bfloat16*)pn, rows, (int)n);
    else
      rmsnorm_rows_kernel<RWN_MAXV><<<(unsigned)((rows + 7) / 8), 256, 0, ctx().stream>>>(
          px, splits == 1, pr, residual ? residual->dtype == KD_F32 : 0, pw, weight->dtype, eps, ps, sum_f32, round_sum,
          (__nv_bfloat16*)pn, rows, (int)n);
    return after_launch("rmsnorm_rows_kernel");
  }
  KD_CUDA_CHECK(launch_ex(add_rmsnorm_kernel, dim3((unsigned)rows), dim3(ARN_THREADS), 0, (const void*)px, splits, (const void*)pr,
                          (int)(residual ? residual->dtype == KD_F32 : 0), (const void*)pw, (int)weight->dtype, eps, ps, sum_f32,
                          (__nv_bfloat16*)pn, (int)rows, (int)n));
  return after_launch("add_rmsnorm_kernel");
}

KD_API int kd_increment_i32(const kd_tensor* scalar, int delta) {
  KD_TRY(require_init());
  KD_REQUIRE(scalar && scalar->dtype == KD_I32 && numel(scalar) == 1, "scalar must be a device int32 scalar");
  void* p = nullptr;
  KD_TRY(tensor_ptr(scalar, &p));
  KD_CUDA_CHECK(launch_ex(increment_i32_kernel, dim3(1), dim3(1), 0, (int*)p, delta));
  return after_launch("increment_i32_kernel");
}

KD_API int kd_linear_bf16_skinny(const kd_tensor* x, const kd_tensor* weight, int epilogue, const kd_tensor* out) {
  KD_TRY(require_init());
  KD_REQUIRE(x && weight && out, "null tensor");
  KD_REQUIRE(epilogue == KD_EPI_NONE || epilogue == KD_EPI_SWIGLU, "kd_linear_bf16_skinny supports KD_EPI_NONE and KD_EPI_SWIGLU");
  KD_REQUIRE(x->dtype == KD_BF16 && weight->dtype == KD_BF16, "kd_linear_bf16_skinny needs bf16 activations and weights");
  KD_REQUIRE(is_contiguous(x) && x->ndim >= 1 && weight->ndim == 2 && weight->strides[1] == 1 && is_contiguous(out),
             "activations / output must be contiguous, weight [N,K] with unit K stride");
  const int64_t K = x->shape[x->ndim - 1], N = weight->shape[0];
  KD_REQUIRE(weight->shape[1] == K && K > 0, "weight has K=%lld, activations have K=%lld", (long long)weight->shape[1], (long long)K);
  const int64_t M = numel(x) / K;
  KD_REQUIRE(M >= 1 && M <= 128, "kd_linear_bf16_skinny handles 1..128 rows, got %lld", (long long)M);
  const int total_kb = (int)((K + 63) / 64);
  void *px, *pw, *po;
  KD_TRY(tensor_ptr(x, &px));
  KD_TRY(tensor_ptr(weight, &pw));
  KD_TRY(tensor_ptr(out, &po));
  if (epilogue == KD_EPI_SWIGLU) {
    KD_REQUIRE(out->dtype == KD_BF16 && numel(out) == M * (N / 2), "SiLU*up output must be bf16 [rows, N/2]");
    return gemm_bf16_skinny(px, K, pw, weight->strides[0], (int)M, (int)N, (int)K, 1, nullptr, po, 1);
  }
  if (out->dtype == KD_BF16) {
    KD_REQUIRE(numel(out) == M * N, "bf16 output must be [rows, N]");
    return gemm_bf16_skinny(px, K, pw, weight->strides[0], (int)M, (int)N, (int)K, 1, nullptr, po, 0);
  }
  KD_REQUIRE(out->dtype == KD_F32 && numel(out) % (M * N) == 0 && numel(out) > 0, "fp32 output must be [splits, rows, N]");
  const int out_splits = (int)(numel(out) / (M * N));
  KD_REQUIRE(out_splits <= total_kb, "output has %d split slices but K only has %d blocks of 64", out_splits, total_kb);
  return gemm_bf16_skinny(px, K, pw, weight->strides[0], (int)M, (int)N, (int)K, out_splits, (float*)po, nullptr, 0);
}

KD_API int kd_linear_bf16_skinny_splits(int64_t N, int64_t K, int* splits_out) {
  KD_TRY(require_init());
  KD_REQUIRE(splits_out && N > 0 && K > 0, "bad argument");
  *splits_out = gemm_skinny_auto_splits((int)N, (int)K);
  return KD_OK;
}

// ----------------------------------------------------------------------------- CUDA graphs
// Kernel launches recorded while capturing are not executions; they are remembered per graph and
// added to the launch counter each time the graph is replayed.
#include <unordered_map>
static std::unordered_map<uint64_t, uint64_t> g_graph_nodes;
static uint64_t g_capture_base = 0;

KD_API int kd_graph_begin(void) {
  KD_TRY(require_init());
  KD_CUDA_CHECK(cudaStreamBeginCapture(ctx().stream, cudaStreamCaptureModeRelaxed));
  g_capture_base = ctx().launches;
  return KD_OK;
}

KD_API int kd_graph_end(uint64_t* graph_out) {
  KD_TRY(require_init());
  if (!graph_out) return fail(KD_ERR_INVALID, "null argument");
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(ctx().stream, &g);
  if (e != cudaSuccess || g == nullptr) {
    cudaGetLastError();
    return fail(KD_ERR_CUDA, "stream capture failed: %s (an operator allocated or synchronised while capturing?)",
                cudaGetErrorString(e));
  }
  cudaGraphExec_t ex = nullptr;
  e = cudaGraphInstantiate(&ex, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(KD_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
  }
  *graph_out = reinterpret_cast<uint64_t>(ex);
  g_graph_nodes[*graph_out] = ctx().launches - g_capture_base;
  ctx().launches = g_capture_base;
  return KD_OK;
}

KD_API int kd_graph_launch(uint64_t graph) {
  KD_TRY(require_init());
  KD_CUDA_CHECK(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(graph), ctx().stream));
  auto it = g_graph_nodes.find(graph);
  ctx().launches += it != g_graph_nodes.end() ? it->second : 1;
  return KD_OK;
}

KD_API int kd_graph_destroy(uint64_t graph) {
  KD_TRY(require_init());
  KD_CUDA_CHECK(cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(graph)));
  g_graph_nodes.erase(graph);
  return KD_OK;
}
