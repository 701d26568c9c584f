// Row reductions: rms_norm, layer_norm, softmax, argmax; and the embedding gather.
//
// The reference runs each of these with ONE THREAD PER ROW
// (packages/backend-webgpu/src/kernels/normalize/executor.ts:167-170).  Here a row is owned by a
// warp (short rows, e.g. the 128-wide q/k-norm) or by a CTA (hidden-size and vocabulary rows),
// loads are 16 bytes wide where alignment allows, and reductions use warp shuffles.  All of them
// are HBM-bound: algorithmic traffic is one read and one write of the row.
//
// Formulas restated from packages/backend-webgpu/src/kernels/normalize/shaderBuilder.ts:
//   rms_norm   (:343-415)  rms = sqrt(sum(x^2)/N + eps); y = (x * (1/rms)) * w
//   layer_norm (:236-325)  biased variance, rstd = 1/sqrt(var+eps); y = (x-mean)*rstd*w + b
//   softmax    (:143-217)  running max starts at -1e38; y = exp(x-max)/sum
#include "common.cuh"

namespace kd {

// Leading-dims index -> element offset of a row; last dim has stride `last`.
struct RowIndex {
  int ndim;  // number of leading dims
  int64_t shape[KD_MAX_DIMS];
  int64_t strides[KD_MAX_DIMS];
  int64_t last;
  __device__ __forceinline__ int64_t row_offset(int64_t row) const {
    int64_t off = 0;
#pragma unroll 1
    for (int d = ndim - 1; d >= 0; --d) {
      const int64_t s = shape[d];
      const int64_t q = row / s;
      off += (row - q * s) * strides[d];
      row = q;
    }
    return off;
  }
};

static RowIndex make_row_index(const kd_tensor* x) {
  RowIndex r{};
  r.ndim = x->ndim - 1;
  for (int d = 0; d < r.ndim; ++d) { r.shape[d] = x->shape[d]; r.strides[d] = x->strides[d]; }
  r.last = x->ndim > 0 ? x->strides[x->ndim - 1] : 1;
  return r;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* smem) {
  v = warp_sum(v);
  if (THREADS == 32) return v;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) smem[w] = v;
  __syncthreads();
  float t = (lane < THREADS / 32) ? smem[lane] : 0.f;
  return warp_sum(t);
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* smem) {
  v = warp_max(v);
  if (THREADS == 32) return v;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) smem[w] = v;
  __syncthreads();
  float t = (lane < THREADS / 32) ? smem[lane] : -3.402823466e38f;
  return warp_max(t);
}

enum { NORM_RMS = 0, NORM_LAYER = 1, NORM_SOFTMAX = 2 };

// One group of G threads (G = 32: a warp, several rows per CTA; G = THREADS: whole CTA) per row.
// Rows are re-read from L1/L2 for the second pass; for the sizes on this path (<= 10 KB per row
// except the vocabulary softmax) the second read never reaches HBM.
template <int MODE, int THREADS, bool WARP_ROWS>
__global__ void __launch_bounds__(THREADS) norm_kernel(const void* __restrict__ x, int dt_x, const void* __restrict__ w,
                                                      int dt_w, const void* __restrict__ b, int dt_b,
                                                      void* __restrict__ y, int dt_y, RowIndex ridx, int64_t rows,
                                                      int64_t n, float eps) {
  __shared__ float red[32];
  constexpr int G = WARP_ROWS ? 32 : THREADS;
  const int tid = WARP_ROWS ? (threadIdx.x & 31) : threadIdx.x;
  const int64_t rows_per_cta = WARP_ROWS ? THREADS / 32 : 1;
  for (int64_t row0 = (int64_t)blockIdx.x * rows_per_cta; row0 < rows; row0 += (int64_t)gridDim.x * rows_per_cta) {
    const int64_t row = row0 + (WARP_ROWS ? (threadIdx.x >> 5) : 0);
    const bool active = row < rows;
    const int64_t base = active ? ridx.row_offset(row) : 0;
    const int64_t last = ridx.last;
    const int64_t cnt = active ? n : 0;
    float a0 = 0.f, a1 = 0.f;
    if (MODE == NORM_SOFTMAX) a0 = -1e38f;
    // pass 1
    if (dt_x == KD_F32 && last == 1 && ((n & 3) == 0) &&
        ((reinterpret_cast<uintptr_t>(static_cast<const float*>(x) + base) & 15) == 0)) {
      const float4* xv = reinterpret_cast<const float4*>(static_cast<const float*>(x) + base);
      for (int64_t i = tid; i < cnt / 4; i += G) {
        const float4 v = xv[i];
        if (MODE == NORM_RMS) a0 += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        else if (MODE == NORM_LAYER) a0 += (v.x + v.y) + (v.z + v.w);
        else a0 = fmaxf(a0, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
      }
    } else {
      for (int64_t i = tid; i < cnt; i += G) {
        const float v = load_float(x, dt_x, base + i * last);
        if (MODE == NORM_RMS) a0 += v * v;
        else if (MODE == NORM_LAYER) a0 += v;
        else a0 = fmaxf(a0, v);
      }
    }
    float stat0, stat1 = 0.f;
    if (MODE == NORM_SOFTMAX) stat0 = WARP_ROWS ? warp_max(a0) : block_max<THREADS>(a0, red);
    else stat0 = WARP_ROWS ? warp_sum(a0) : block_sum<THREADS>(a0, red);

    if (MODE == NORM_LAYER) {
      // two-pass variance around the mean (numerically at least as good as Welford)
      const float mean = stat0 / (float)n;
      for (int64_t i = tid; i < cnt; i += G) {
        const float d = load_float(x, dt_x, base + i * last) - mean;
        a1 += d * d;
      }
      stat1 = WARP_ROWS ? warp_sum(a1) : block_sum<THREADS>(a1, red);
      stat0 = mean;
    } else if (MODE == NORM_SOFTMAX) {
      for (int64_t i = tid; i < cnt; i += G) a1 += expf(load_float(x, dt_x, base + i * last) - stat0);
      stat1 = WARP_ROWS ? warp_sum(a1) : block_sum<THREADS>(a1, red);
    }
    // pass 2: write
    const int64_t obase = row * n;
    if (MODE == NORM_RMS) {
      const float rms = sqrtf(stat0 / (float)n + eps);
      const float sc = 1.0f / rms;
      for (int64_t i = tid; i < cnt; i += G) {
        float v = load_float(x, dt_x, base + i * last) * sc;
        if (w) v = v * load_float(w, dt_w, i);
        store_float(y, dt_y, obase + i, v);
      }
    } else if (MODE == NORM_LAYER) {
      const float rstd = 1.0f / sqrtf(stat1 / (float)n + eps);
      for (int64_t i = tid; i < cnt; i += G) {
        float v = (load_float(x, dt_x, base + i * last) - stat0) * rstd;
        if (w) v = v * load_float(w, dt_w, i);
        if (b) v = v + load_float(b, dt_b, i);
        store_float(y, dt_y, obase + i, v);
      }
    } else {
      for (int64_t i = tid; i < cnt; i += G)
        store_float(y, dt_y, obase + i, expf(load_float(x, dt_x, base + i * last) - stat0) / stat1);
    }
  }
}

// bf16 rows of up to 2048 elements, dense: one warp per row, the row held in registers between the
// statistics and the write (one read of x, 16-byte accesses).  Same arithmetic as norm_kernel.
template <int MODE, int NV>
__global__ void __launch_bounds__(256) norm_rows_bf16_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                            const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                                            int64_t rows, int n, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int nvec = n >> 3;
  for (int64_t row = warp0; row < rows; row += nwarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * n);
    float v[NV][8];
    float s = 0.f;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      const int vi = lane + t * 32;
      if (vi < nvec) {
        const uint4 u = xr[vi];
        const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          v[t][e] = __bfloat162float(h[e]);
          s += MODE == NORM_RMS ? v[t][e] * v[t][e] : v[t][e];
        }
      }
    }
    s = warp_sum(s);
    float mean = 0.f, sc;
    if (MODE == NORM_RMS) {
      sc = 1.0f / sqrtf(s / (float)n + eps);
    } else {
      mean = s / (float)n;
      float q = 0.f;
#pragma unroll
      for (int t = 0; t < NV; ++t) {
        if (lane + t * 32 < nvec) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float d = v[t][e] - mean;
            q += d * d;
          }
        }
      }
      q = warp_sum(q);
      sc = 1.0f / sqrtf(q / (float)n + eps);
    }
    uint4* yr = reinterpret_cast<uint4*>(y + row * n);
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      const int vi = lane + t * 32;
      if (vi < nvec) {
        float wv[8], bv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) { wv[e] = 1.f; bv[e] = 0.f; }
        if (w) {
          const uint4 u = reinterpret_cast<const uint4*>(w)[vi];
          const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
          for (int e = 0; e < 8; ++e) wv[e] = __bfloat162float(h[e]);
        }
        if (MODE == NORM_LAYER && b) {
          const uint4 u = reinterpret_cast<const uint4*>(b)[vi];
          const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
          for (int e = 0; e < 8; ++e) bv[e] = __bfloat162float(h[e]);
        }
        uint4 o;
        __nv_bfloat16* ho = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float r = (v[t][e] - mean) * sc;
          if (w) r = r * wv[e];
          if (MODE == NORM_LAYER && b) r = r + bv[e];
          ho[e] = __float2bfloat16_rn(r);
        }
        yr[vi] = o;
      }
    }
  }
}

template <int MODE, int NV>
static void launch_norm_rows_bf16(const void* x, const void* w, const void* b, void* y, int64_t rows, int n, float eps) {
  int64_t blocks = (rows + 7) / 8;
  const int64_t cap = (int64_t)ctx().sm_count * 16;
  if (blocks > cap) blocks = cap;
  norm_rows_bf16_kernel<MODE, NV><<<(int)blocks, 256, 0, ctx().stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(b),
      static_cast<__nv_bfloat16*>(y), rows, n, eps);
}

template <int MODE>
static int launch_norm(const kd_tensor* x, const kd_tensor* w, const kd_tensor* b, float eps, const kd_tensor* out,
                       const char* name) {
  KD_TRY(require_init());
  KD_REQUIRE(x && out, "null tensor");
  KD_REQUIRE(x->ndim >= 1, "%s needs at least one dimension", name);
  KD_REQUIRE(is_float_dtype(x->dtype) && is_float_dtype(out->dtype), "%s needs floating-point tensors", name);
  const int64_t n = x->shape[x->ndim - 1];
  const int64_t total = numel(x);
  KD_REQUIRE(numel(out) == total && is_contiguous(out), "%s output must be contiguous with the input's element count", name);
  if (total == 0) return KD_OK;
  if (w) KD_REQUIRE(numel(w) == n && is_contiguous(w), "%s weight must be contiguous with %lld elements", name, (long long)n);
  if (b) KD_REQUIRE(numel(b) == n && is_contiguous(b), "%s bias must be contiguous with %lld elements", name, (long long)n);
  void *px = nullptr, *pw = nullptr, *pb = nullptr, *py = nullptr;
  KD_TRY(tensor_ptr(x, &px));
  if (w) KD_TRY(tensor_ptr(w, &pw));
  if (b) KD_TRY(tensor_ptr(b, &pb));
  KD_TRY(tensor_ptr(out, &py));
  const int64_t rows = total / n;
  const RowIndex ridx = make_row_index(x);
  const int sms = ctx().sm_count;
  cudaStream_t st = ctx().stream;
  const int dw = w ? w->dtype : KD_F32, db = b ? b->dtype : KD_F32;
  if (MODE != NORM_SOFTMAX && x->dtype == KD_BF16 && out->dtype == KD_BF16 && is_contiguous(x) && n % 8 == 0 && n <= 2048 &&
      (!w || w->dtype == KD_BF16) && (!b || b->dtype == KD_BF16) &&
      ((reinterpret_cast<uintptr_t>(px) | reinterpret_cast<uintptr_t>(py) | reinterpret_cast<uintptr_t>(pw) |
        reinterpret_cast<uintptr_t>(pb)) & 15) == 0) {
    constexpr int M2 = MODE == NORM_SOFTMAX ? NORM_RMS : MODE;   // the softmax instantiation is never launched
    if (n <= 256) launch_norm_rows_bf16<M2, 1>(px, pw, pb, py, rows, (int)n, eps);
    else if (n <= 512) launch_norm_rows_bf16<M2, 2>(px, pw, pb, py, rows, (int)n, eps);
    else if (n <= 1024) launch_norm_rows_bf16<M2, 4>(px, pw, pb, py, rows, (int)n, eps);
    else launch_norm_rows_bf16<M2, 8>(px, pw, pb, py, rows, (int)n, eps);
    return after_launch(name);
  }
  if (n <= 512) {
    constexpr int T = 256;
    int64_t blocks = (rows + (T / 32) - 1) / (T / 32);
    if (blocks > (int64_t)sms * 32) blocks = (int64_t)sms * 32;
    norm_kernel<MODE, T, true><<<(int)blocks, T, 0, st>>>(px, x->dtype, pw, dw, pb, db, py, out->dtype, ridx, rows, n, eps);
  } else if (n <= 8192) {
    constexpr int T = 256;
    int64_t blocks = rows < (int64_t)sms * 16 ? rows : (int64_t)sms * 16;
    norm_kernel<MODE, T, false><<<(int)blocks, T, 0, st>>>(px, x->dtype, pw, dw, pb, db, py, out->dtype, ridx, rows, n, eps);
  } else {
    constexpr int T = 1024;
    int64_t blocks = rows < (int64_t)sms * 4 ? rows : (int64_t)sms * 4;
    norm_kernel<MODE, T, false><<<(int)blocks, T, 0, st>>>(px, x->dtype, pw, dw, pb, db, py, out->dtype, ridx, rows, n, eps);
  }
  return after_launch(name);
}

// ----------------------------------------------------------------------------- argmax
// CTA per row; (value, index) pairs reduced with shuffles; strict '>' as in
// packages/backend-webgpu/src/kernels/reduction/argShaderBuilder.ts:31, lowest index wins ties
// (the reference's tree reduction leaves the tie order undefined).
__device__ __forceinline__ void arg_combine(float& v, int64_t& i, float ov, int64_t oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

template <int THREADS>
__global__ void __launch_bounds__(THREADS) argmax_kernel(const void* __restrict__ x, int dt_x, void* __restrict__ out,
                                                        int dt_o, RowIndex ridx, int64_t rows, int64_t n) {
  __shared__ float sv[THREADS / 32];
  __shared__ int64_t si[THREADS / 32];
  pdl_wait();
  pdl_trigger();
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int64_t base = ridx.row_offset(row);
    float best = -3.402823466e38f;
    int64_t bi = 0x7fffffffffffffffLL;
    if (dt_x == KD_BF16 && ridx.last == 1 &&
        ((reinterpret_cast<uintptr_t>(static_cast<const __nv_bfloat16*>(x) + base) & 15) == 0)) {
      const uint4* xv = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(x) + base);
      for (int64_t i = threadIdx.x; i < n / 8; i += THREADS) {
        const uint4 u = xv[i];
        const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float v = __bfloat162float(h[j]);
          if (v > best) { best = v; bi = i * 8 + j; }
        }
      }
      for (int64_t i = (n / 8) * 8 + threadIdx.x; i < n; i += THREADS) {
        const float v = load_float(x, dt_x, base + i);
        if (v > best) { best = v; bi = i; }
      }
    } else if (dt_x == KD_F32 && ridx.last == 1 &&
               ((reinterpret_cast<uintptr_t>(static_cast<const float*>(x) + base) & 15) == 0)) {
      const float4* xv = reinterpret_cast<const float4*>(static_cast<const float*>(x) + base);
      for (int64_t i = threadIdx.x; i < n / 4; i += THREADS) {
        const float4 u = xv[i];
        if (u.x > best) { best = u.x; bi = i * 4; }
        if (u.y > best) { best = u.y; bi = i * 4 + 1; }
        if (u.z > best) { best = u.z; bi = i * 4 + 2; }
        if (u.w > best) { best = u.w; bi = i * 4 + 3; }
      }
      for (int64_t i = (n / 4) * 4 + threadIdx.x; i < n; i += THREADS) {
        const float v = load_float(x, dt_x, base + i);
        if (v > best) { best = v; bi = i; }
      }
    } else {
      for (int64_t i = threadIdx.x; i < n; i += THREADS) {
        const float v = load_float(x, dt_x, base + i * ridx.last);
        if (v > best) { best = v; bi = i; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int64_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
      arg_combine(best, bi, ov, oi);
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { sv[wid] = best; si[wid] = bi; }
    __syncthreads();
    if (wid == 0) {
      best = lane < THREADS / 32 ? sv[lane] : -3.402823466e38f;
      bi = lane < THREADS / 32 ? si[lane] : 0x7fffffffffffffffLL;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int64_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        arg_combine(best, bi, ov, oi);
      }
      if (lane == 0) {
        if (bi == 0x7fffffffffffffffLL) bi = 0;  // row of -FLT_MAX / NaN: index 0 like a serial scan
        if (dt_o == KD_I64) static_cast<int64_t*>(out)[row] = bi;
        else static_cast<int32_t*>(out)[row] = (int32_t)bi;
      }
    }
  }
}

// ----------------------------------------------------------------------------- index_select (dim 0)
// One warp per gathered row, 16-byte copies when the row width allows.  An index outside
// [0, rows) sets the device error flag and writes zeros instead of reading out of bounds.
__global__ void gather_rows_kernel(const char* __restrict__ table, const void* __restrict__ idx, int idx_dt,
                                   int64_t idx_stride, char* __restrict__ out, int64_t n_idx, int64_t table_rows,
                                   int64_t row_bytes, int64_t table_row_stride_bytes, int* __restrict__ err) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = warp; r < n_idx; r += nwarps) {
    int64_t id = idx_dt == KD_I64 ? static_cast<const int64_t*>(idx)[r * idx_stride]
                                  : (int64_t) static_cast<const int32_t*>(idx)[r * idx_stride];
    const bool bad = id < 0 || id >= table_rows;
    if (bad) {
      if (lane == 0 && atomicCAS(err, 0, 101) == 0) { err[1] = (int)r; err[2] = (int)id; }
    }
    const char* src = table + id * table_row_stride_bytes;
    char* dst = out + r * row_bytes;
    if ((row_bytes & 15) == 0 && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) &&
        ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
      for (int64_t i = lane; i < row_bytes / 16; i += 32)
        reinterpret_cast<uint4*>(dst)[i] = bad ? make_uint4(0, 0, 0, 0) : reinterpret_cast<const uint4*>(src)[i];
    } else {
      for (int64_t i = lane; i < row_bytes; i += 32) dst[i] = bad ? 0 : src[i];
    }
  }
}

}  // namespace kd

using namespace kd;

KD_API int kd_rms_norm(const kd_tensor* x, const kd_tensor* weight, float eps, const kd_tensor* out) {
  return launch_norm<NORM_RMS>(x, weight, nullptr, eps, out, "rms_norm");
}
KD_API int kd_layer_norm(const kd_tensor* x, const kd_tensor* weight, const kd_tensor* bias, float eps,
                         const kd_tensor* out) {
  return launch_norm<NORM_LAYER>(x, weight, bias, eps, out, "layer_norm");
}
KD_API int kd_softmax(const kd_tensor* x, const kd_tensor* out) {
  return launch_norm<NORM_SOFTMAX>(x, nullptr, nullptr, 0.f, out, "softmax");
}

KD_API int kd_argmax(const kd_tensor* x, const kd_tensor* out) {
  KD_TRY(require_init());
  KD_REQUIRE(x && out, "null tensor");
  KD_REQUIRE(x->ndim >= 1 && is_float_dtype(x->dtype), "argmax needs a floating-point tensor of rank >= 1");
  KD_REQUIRE(out->dtype == KD_I32 || out->dtype == KD_I64, "argmax output must be int32 or int64");
  const int64_t n = x->shape[x->ndim - 1];
  KD_REQUIRE(n > 0, "argmax over an empty dimension");
  const int64_t rows = numel(x) / n;
  KD_REQUIRE(numel(out) == rows && is_contiguous(out), "argmax output must be contiguous with one element per row");
  if (rows == 0) return KD_OK;
  void *px = nullptr, *po = nullptr;
  KD_TRY(tensor_ptr(x, &px));
  KD_TRY(tensor_ptr(out, &po));
  const RowIndex ridx = make_row_index(x);
  constexpr int T = 1024;
  const int64_t cap = (int64_t)ctx().sm_count * 2;
  KD_CUDA_CHECK(launch_ex(argmax_kernel<T>, dim3((unsigned)(rows < cap ? rows : cap)), dim3(T), 0, (const void*)px, (int)x->dtype, po,
                          (int)out->dtype, ridx, rows, n));
  return after_launch("argmax_kernel");
}

KD_API int kd_index_select(const kd_tensor* self, const kd_tensor* index, int dim, const kd_tensor* out) {
  KD_TRY(require_init());
  KD_REQUIRE(self && index && out, "null tensor");
  KD_REQUIRE(dim == 0, "index_select is implemented for dim 0 (row gather) only");
  KD_REQUIRE(self->ndim == 2 && self->strides[1] == 1, "index_select source must be 2-D with unit inner stride");
  KD_REQUIRE(index->ndim <= 1 && (index->dtype == KD_I32 || index->dtype == KD_I64), "index must be 1-D int32/int64");
  KD_REQUIRE(out->dtype == self->dtype && is_contiguous(out), "output must be contiguous and of the source dtype");
  const int64_t n_idx = numel(index);
  KD_REQUIRE(numel(out) == n_idx * self->shape[1], "output has the wrong number of elements");
  if (n_idx == 0) return KD_OK;
  void *ps = nullptr, *pi = nullptr, *po = nullptr;
  KD_TRY(tensor_ptr(self, &ps));
  KD_TRY(tensor_ptr(index, &pi));
  KD_TRY(tensor_ptr(out, &po));
  const int esz = dtype_size(self->dtype);
  const int threads = 256;
  int64_t blocks = (n_idx + 7) / 8;
  const int64_t cap = (int64_t)ctx().sm_count * 16;
  if (blocks > cap) blocks = cap;
  KD_CUDA_CHECK(launch_ex(gather_rows_kernel, dim3((unsigned)blocks), dim3(threads), 0, (const char*)ps, (const void*)pi,
                          (int)index->dtype, (int64_t)(index->ndim == 1 ? index->strides[0] : 1), (char*)po, n_idx,
                          (int64_t)self->shape[0], (int64_t)(self->shape[1] * esz), (int64_t)(self->strides[0] * esz),
                          ctx().error_flag));
  return after_launch("gather_rows_kernel");
}
