// Shared declarations for libkandle_cuda.so (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <utility>

#include "../../include/kandle_cuda.h"

#define KD_API extern "C" __attribute__((visibility("default")))

namespace kd {

// ----------------------------------------------------------------------------- errors
void set_error(const char* fmt, ...);
int fail(int status, const char* fmt, ...);

#define KD_CUDA_CHECK(expr)                                                                    \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess)                                                                     \
      return ::kd::fail(KD_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),   \
                        __FILE__, __LINE__);                                                   \
  } while (0)

#define KD_REQUIRE(cond, ...)                                   \
  do {                                                          \
    if (!(cond)) return ::kd::fail(KD_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define KD_TRY(expr)          \
  do {                        \
    int _s = (expr);          \
    if (_s != KD_OK) return _s; \
  } while (0)

// ----------------------------------------------------------------------------- context
struct Storage {
  void* ptr;
  uint64_t bytes;        // requested size
  uint64_t block_bytes;  // size of the allocator block backing it
  int64_t refcount;
};

struct Context {
  bool ready = false;
  int device = -1;
  int sm_count = 0;
  cudaStream_t stream = nullptr;
  uint64_t launches = 0;
  int* error_flag = nullptr;  // device int, set by kernels that detect a problem
  bool pdl = false;           // launch kernels with programmatic dependent launch (kd_set_pdl)
  bool pdl_early_kv = false;  // kd_set_pdl(2): decode attention may fetch K/V tiles of earlier positions before its grid-dependency wait
  void* workspace = nullptr;  // library-owned scratch, grown on demand
  uint64_t workspace_bytes = 0;
};

Context& ctx();
int require_init();
// Record one kernel launch and pick up launch-configuration errors.
int after_launch(const char* name);
// Library-owned scratch buffer of at least `bytes` (stream ordered; contents undefined).
int get_workspace(uint64_t bytes, void** out);

// Device pointer of a tensor's first element (storage base + offset), or error.
int tensor_ptr(const kd_tensor* t, void** out);
int storage_lookup(uint64_t handle, Storage** out);

__host__ __device__ inline int dtype_size(int dt) {
  switch (dt) {
    case KD_F32: return 4;
    case KD_F16: return 2;
    case KD_BF16: return 2;
    case KD_I32: return 4;
    case KD_I64: return 8;
    default: return 1;
  }
}

inline int64_t numel(const kd_tensor* t) {
  int64_t n = 1;
  for (int i = 0; i < t->ndim; ++i) n *= t->shape[i];
  return n;
}

inline bool is_contiguous(const kd_tensor* t) {
  int64_t expect = 1;
  for (int i = t->ndim - 1; i >= 0; --i) {
    if (t->shape[i] != 1 && t->strides[i] != expect) return false;
    expect *= t->shape[i];
  }
  return true;
}

inline bool is_float_dtype(int dt) { return dt == KD_F32 || dt == KD_F16 || dt == KD_BF16; }

// ----------------------------------------------------------------------------- programmatic dependent launch
// Every kernel of the decode step starts with pdl_wait() (all writes of the preceding kernels are
// visible after it; without the launch attribute it is a no-op) and calls pdl_trigger() once its
// CTAs hold their resources, so that the next kernel's launch latency and prologue overlap this
// kernel's execution.  pdl_trigger() must come after any TMEM allocation: a dependent CTA that
// grabbed tensor memory first would block this kernel's allocation while waiting for it to finish.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx().stream;
  cudaLaunchAttribute attr[1];
  if (ctx().pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// ----------------------------------------------------------------------------- device helpers
__device__ __forceinline__ float load_float(const void* base, int dt, int64_t idx) {
  switch (dt) {
    case KD_F32: return static_cast<const float*>(base)[idx];
    case KD_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
    case KD_F16: return __half2float(static_cast<const __half*>(base)[idx]);
    case KD_I32: return (float)static_cast<const int32_t*>(base)[idx];
    case KD_I64: return (float)static_cast<const int64_t*>(base)[idx];
    default: return (float)static_cast<const uint8_t*>(base)[idx];
  }
}

__device__ __forceinline__ void store_float(void* base, int dt, int64_t idx, float v) {
  switch (dt) {
    case KD_F32: static_cast<float*>(base)[idx] = v; break;
    case KD_BF16: static_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v); break;
    case KD_F16: static_cast<__half*>(base)[idx] = __float2half_rn(v); break;
    case KD_I32: static_cast<int32_t*>(base)[idx] = (int32_t)v; break;
    case KD_I64: static_cast<int64_t*>(base)[idx] = (int64_t)v; break;
    default: static_cast<uint8_t*>(base)[idx] = (uint8_t)v; break;
  }
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

// Row-major decomposition of a linear index over `ndim` dims into an element offset.
struct StridedIndex {
  int ndim;
  int64_t shape[KD_MAX_DIMS];
  int64_t strides[KD_MAX_DIMS];
  __device__ __forceinline__ int64_t offset_of(int64_t linear) const {
    int64_t off = 0;
#pragma unroll 1
    for (int d = ndim - 1; d >= 0; --d) {
      const int64_t s = shape[d];
      const int64_t q = linear / s;
      off += (linear - q * s) * strides[d];
      linear = q;
    }
    return off;
  }
};

}  // namespace kd
