// Map kernels: pointwise arithmetic, strided copy / cast, fill, arange.
//
// Replaces the reference's generated pointwise shaders (fast contiguous path + general strided
// path, rank <= 8; packages/backend-webgpu/src/kernels/pointwise/executor.ts:60-130) and the
// copy family (packages/backend-webgpu/src/kernels/copy/index.ts:15-30).  Arithmetic is fp32
// whatever the storage type and rounds once at the output, as the reference does for 16-bit
// storage (packages/backend-webgpu/src/base/dtype.ts:50-74).
//
// HBM-bound: the contiguous paths move 16 bytes per thread per access and size the grid as a
// multiple of the SM count.
#include "common.cuh"

namespace kd {

__device__ __forceinline__ float clampf(float v, float lo, float hi) { return fminf(fmaxf(v, lo), hi); }

// Expression table restated from packages/backend-webgpu/src/kernels/pointwise/ops.ts:
//   add a + alpha*b (:437-444), silu x/(1+exp(-clamp(x,+-88))) (:299),
//   gelu 0.5x(1+tanh(clamp(0.7978845608(x+0.044715x^3),+-20))) (:301), tanh clamp +-20 (:211),
//   sigmoid clamp +-88 (:297).  expf/tanhf/cosf/sinf are the accurate library versions.
__device__ __forceinline__ float apply_op(int op, float a, float b, float s) {
  switch (op) {
    case KD_OP_ADD: return a + s * b;
    case KD_OP_SUB: return a - s * b;
    case KD_OP_MUL: return a * b;
    case KD_OP_MUL_SCALAR: return a * s;
    case KD_OP_NEG: return -a;
    case KD_OP_COS: return cosf(a);
    case KD_OP_SIN: return sinf(a);
    case KD_OP_SILU: return a / (1.0f + expf(-clampf(a, -88.f, 88.f)));
    case KD_OP_GELU: {
      const float inner = 0.7978845608f * (a + 0.044715f * a * a * a);
      return 0.5f * a * (1.0f + tanhf(clampf(inner, -20.f, 20.f)));
    }
    case KD_OP_ABS: return fabsf(a);
    case KD_OP_DIV: return a / b;
    case KD_OP_MAXIMUM: return fmaxf(a, b);
    case KD_OP_TANH: return tanhf(clampf(a, -20.f, 20.f));
    case KD_OP_SIGMOID: return 1.0f / (1.0f + expf(-clampf(a, -88.f, 88.f)));
    default: return a;
  }
}

struct PwParams {
  int op;
  int ndim;
  int dt_a, dt_b, dt_o;
  int has_b;
  int int_mode;  // both operands integer: move values as int64 without a float round trip
  float scalar;
  int64_t n;
  int64_t shape[KD_MAX_DIMS];
  int64_t sa[KD_MAX_DIMS], sb[KD_MAX_DIMS], so[KD_MAX_DIMS];
};

__global__ void pointwise_strided_kernel(const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ o,
                                         PwParams p) {
  pdl_wait();
  pdl_trigger();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.n; i += stride) {
    int64_t lin = i, oa = 0, ob = 0, oo = 0;
#pragma unroll 1
    for (int d = p.ndim - 1; d >= 0; --d) {
      const int64_t s = p.shape[d];
      const int64_t q = lin / s;
      const int64_t r = lin - q * s;
      oa += r * p.sa[d];
      ob += r * p.sb[d];
      oo += r * p.so[d];
      lin = q;
    }
    if (p.int_mode) {
      int64_t v;
      switch (p.dt_a) {
        case KD_I64: v = static_cast<const int64_t*>(a)[oa]; break;
        case KD_I32: v = static_cast<const int32_t*>(a)[oa]; break;
        default: v = static_cast<const uint8_t*>(a)[oa]; break;
      }
      switch (p.dt_o) {
        case KD_I64: static_cast<int64_t*>(o)[oo] = v; break;
        case KD_I32: static_cast<int32_t*>(o)[oo] = (int32_t)v; break;
        default: static_cast<uint8_t*>(o)[oo] = (uint8_t)v; break;
      }
      continue;
    }
    const float va = load_float(a, p.dt_a, oa);
    const float vb = p.has_b ? load_float(b, p.dt_b, ob) : 0.f;
    store_float(o, p.dt_o, oo, apply_op(p.op, va, vb, p.scalar));
  }
}

// Contiguous, same dtype for all operands: 16 bytes per thread per access.
template <typename T, int VEC>
__global__ void pointwise_contig_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ o, int op,
                                        int has_b, float scalar, int64_t n_vec, int64_t n) {
  struct alignas(16) Pack { T v[VEC]; };
  pdl_wait();
  pdl_trigger();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    Pack pa = reinterpret_cast<const Pack*>(a)[i];
    Pack pb;
    if (has_b) pb = reinterpret_cast<const Pack*>(b)[i];
    Pack po;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float va = (float)pa.v[j];
      const float vb = has_b ? (float)pb.v[j] : 0.f;
      po.v[j] = (T)apply_op(op, va, vb, scalar);
    }
    reinterpret_cast<Pack*>(o)[i] = po;
  }
  // tail
  const int64_t tail0 = n_vec * VEC;
  for (int64_t i = tail0 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float va = (float)a[i];
    const float vb = has_b ? (float)b[i] : 0.f;
    o[i] = (T)apply_op(op, va, vb, scalar);
  }
}

static int grid_for(int64_t work_items, int threads) {
  const int sms = ctx().sm_count > 0 ? ctx().sm_count : 148;
  int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = (int64_t)sms * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static bool same_shape(const kd_tensor* a, const kd_tensor* b) {
  if (a->ndim != b->ndim) return false;
  for (int i = 0; i < a->ndim; ++i)
    if (a->shape[i] != b->shape[i]) return false;
  return true;
}

// Right-align `t` against `out` and produce broadcast strides (0 where t's extent is 1).
static int broadcast_strides(const kd_tensor* t, const kd_tensor* out, int64_t* st, const char* what) {
  const int shift = out->ndim - t->ndim;
  if (shift < 0) return fail(KD_ERR_INVALID, "%s has higher rank (%d) than the output (%d)", what, t->ndim, out->ndim);
  for (int d = 0; d < out->ndim; ++d) {
    if (d < shift) { st[d] = 0; continue; }
    const int64_t e = t->shape[d - shift];
    if (e == out->shape[d]) st[d] = t->strides[d - shift];
    else if (e == 1) st[d] = 0;
    else return fail(KD_ERR_INVALID, "%s extent %lld does not broadcast to %lld at dim %d", what, (long long)e,
                     (long long)out->shape[d], d);
  }
  return KD_OK;
}

static int launch_pointwise(int op, const kd_tensor* a, const kd_tensor* b, float scalar, const kd_tensor* out) {
  KD_TRY(require_init());
  KD_REQUIRE(a && out, "null tensor");
  void *pa = nullptr, *pb = nullptr, *po = nullptr;
  KD_TRY(tensor_ptr(a, &pa));
  if (b) KD_TRY(tensor_ptr(b, &pb));
  KD_TRY(tensor_ptr(out, &po));
  const int64_t n = numel(out);
  if (n == 0) return KD_OK;
  cudaStream_t st = ctx().stream;

  const bool fast = is_contiguous(out) && is_contiguous(a) && same_shape(a, out) && a->dtype == out->dtype &&
                    (!b || (is_contiguous(b) && same_shape(b, out) && b->dtype == out->dtype)) && aligned16(pa) &&
                    aligned16(po) && (!b || aligned16(pb)) && (out->dtype == KD_F32 || out->dtype == KD_BF16);
  if (fast) {
    const int threads = 256;
    if (out->dtype == KD_F32) {
      const int64_t nv = n / 4;
      pointwise_contig_kernel<float, 4><<<grid_for(nv > 0 ? nv : n, threads), threads, 0, st>>>(
          (const float*)pa, (const float*)pb, (float*)po, op, b != nullptr, scalar, nv, n);
    } else {
      const int64_t nv = n / 8;
      pointwise_contig_kernel<__nv_bfloat16, 8><<<grid_for(nv > 0 ? nv : n, threads), threads, 0, st>>>(
          (const __nv_bfloat16*)pa, (const __nv_bfloat16*)pb, (__nv_bfloat16*)po, op, b != nullptr, scalar, nv, n);
    }
    return after_launch("pointwise_contig_kernel");
  }

  PwParams p{};
  p.op = op;
  p.ndim = out->ndim;
  p.dt_a = a->dtype;
  p.dt_b = b ? b->dtype : KD_F32;
  p.dt_o = out->dtype;
  p.has_b = b != nullptr;
  p.int_mode = (op < 0 && !is_float_dtype(a->dtype) && !is_float_dtype(out->dtype)) ? 1 : 0;
  p.scalar = scalar;
  p.n = n;
  for (int d = 0; d < out->ndim; ++d) {
    p.shape[d] = out->shape[d];
    p.so[d] = out->strides[d];
  }
  KD_TRY(broadcast_strides(a, out, p.sa, "input a"));
  if (b) KD_TRY(broadcast_strides(b, out, p.sb, "input b"));
  const int threads = 256;
  KD_CUDA_CHECK(launch_ex(pointwise_strided_kernel, dim3(grid_for(n, threads)), dim3(threads), 0, (const void*)pa, (const void*)pb, po, p));
  return after_launch("pointwise_strided_kernel");
}

// ----------------------------------------------------------------------------- fill / arange
template <typename T>
__global__ void fill_kernel(T* __restrict__ p, T v, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = v;
}

__global__ void fill_strided_kernel(void* __restrict__ p, int dt, float v, StridedIndex idx, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    store_float(p, dt, idx.offset_of(i), v);
}

__global__ void arange_kernel(void* __restrict__ p, int dt, double start, double step, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const double v = start + (double)i * step;
    if (dt == KD_I32) static_cast<int32_t*>(p)[i] = (int32_t)v;
    else if (dt == KD_I64) static_cast<int64_t*>(p)[i] = (int64_t)v;
    else store_float(p, dt, i, (float)v);
  }
}

}  // namespace kd

using namespace kd;

KD_API int kd_pointwise(int op, const kd_tensor* a, const kd_tensor* b, float scalar, const kd_tensor* out) {
  KD_REQUIRE(op >= KD_OP_ADD && op <= KD_OP_SUB, "unknown pointwise op %d", op);
  const bool binary = (op == KD_OP_ADD || op == KD_OP_MUL || op == KD_OP_DIV || op == KD_OP_MAXIMUM || op == KD_OP_SUB);
  KD_REQUIRE(!binary || b != nullptr, "binary pointwise op %d needs two inputs", op);
  return launch_pointwise(op, a, binary ? b : nullptr, scalar, out);
}

KD_API int kd_copy(const kd_tensor* dst, const kd_tensor* src) {
  KD_TRY(require_init());
  KD_REQUIRE(dst && src, "null tensor");
  // Same dtype, both contiguous, same element count: a device memcpy.
  if (dst->dtype == src->dtype && is_contiguous(dst) && is_contiguous(src) && numel(dst) == numel(src) &&
      same_shape(dst, src)) {
    void *pd = nullptr, *ps = nullptr;
    KD_TRY(tensor_ptr(dst, &pd));
    KD_TRY(tensor_ptr(src, &ps));
    const int64_t n = numel(dst);
    if (n == 0) return KD_OK;
    KD_CUDA_CHECK(cudaMemcpyAsync(pd, ps, (size_t)n * dtype_size(dst->dtype), cudaMemcpyDeviceToDevice, ctx().stream));
    ctx().launches++;
    return KD_OK;
  }
  return launch_pointwise(-1 /* identity */, src, nullptr, 0.f, dst);
}

KD_API int kd_fill(const kd_tensor* dst, double value) {
  KD_TRY(require_init());
  KD_REQUIRE(dst, "null tensor");
  void* p = nullptr;
  KD_TRY(tensor_ptr(dst, &p));
  const int64_t n = numel(dst);
  if (n == 0) return KD_OK;
  cudaStream_t st = ctx().stream;
  const int threads = 256;
  if (is_contiguous(dst)) {
    if (value == 0.0) {
      KD_CUDA_CHECK(cudaMemsetAsync(p, 0, (size_t)n * dtype_size(dst->dtype), st));
      ctx().launches++;
      return KD_OK;
    }
    const int g = grid_for(n, threads);
    switch (dst->dtype) {
      case KD_F32: fill_kernel<float><<<g, threads, 0, st>>>((float*)p, (float)value, n); break;
      case KD_BF16: fill_kernel<__nv_bfloat16><<<g, threads, 0, st>>>((__nv_bfloat16*)p, __float2bfloat16_rn((float)value), n); break;
      case KD_F16: fill_kernel<__half><<<g, threads, 0, st>>>((__half*)p, __float2half_rn((float)value), n); break;
      case KD_I32: fill_kernel<int32_t><<<g, threads, 0, st>>>((int32_t*)p, (int32_t)value, n); break;
      case KD_I64: fill_kernel<int64_t><<<g, threads, 0, st>>>((int64_t*)p, (int64_t)value, n); break;
      default: fill_kernel<uint8_t><<<g, threads, 0, st>>>((uint8_t*)p, (uint8_t)value, n); break;
    }
    return after_launch("fill_kernel");
  }
  StridedIndex idx{};
  idx.ndim = dst->ndim;
  for (int d = 0; d < dst->ndim; ++d) { idx.shape[d] = dst->shape[d]; idx.strides[d] = dst->strides[d]; }
  fill_strided_kernel<<<grid_for(n, threads), threads, 0, st>>>(p, dst->dtype, (float)value, idx, n);
  return after_launch("fill_strided_kernel");
}

KD_API int kd_arange(const kd_tensor* dst, double start, double step) {
  KD_TRY(require_init());
  KD_REQUIRE(dst && dst->ndim == 1 && is_contiguous(dst), "arange needs a contiguous 1-D output");
  void* p = nullptr;
  KD_TRY(tensor_ptr(dst, &p));
  const int64_t n = numel(dst);
  if (n == 0) return KD_OK;
  arange_kernel<<<grid_for(n, 256), 256, 0, ctx().stream>>>(p, dst->dtype, start, step, n);
  return after_launch("arange_kernel");
}
