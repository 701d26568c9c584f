// Key `randn`: normal random numbers from the counter-based Philox4x32-10 generator.
//
// Same stream of numbers as the reference's random kernel
// (packages/backend-webgpu/src/kernels/random/shaderBuilder.ts:140-185, philox.wgsl.ts:17-155,
// executor.ts:31-49): element i belongs to pair i/2; the pair's counter is
// [pair + base_offset (mod 2^32), 0, 0, 0], the key is the 64-bit seed split into two words;
// member 0 of the pair takes words (x, y) of the Philox output, member 1 takes (z, w); a word
// becomes a uniform number in [0,1) as (w >> 8) * 2^-24, and the pair of uniforms goes through the
// cosine branch of Box-Muller with u1 clamped to 1e-10.  The result is mean + std * z.
//
// B200 specifics: counter-based means every element is computed from its own index, so a tensor-
// parallel rank fills its slice of a weight matrix with the numbers the full matrix would hold there
// (row0 / col0 / full_cols give the position of the slice), and a 4-billion-parameter model is
// initialised in HBM in milliseconds without touching the host.  Bound: HBM writes (2 or 4 bytes
// per element); the arithmetic (ten rounds of two 32x32->64 multiplies, one log, one sqrt, one cos)
// is a small multiple of that at 148 SMs.
#include "common.cuh"
#include "kernels.cuh"

namespace kd {

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
  const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
  const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
  const uint32_t n1 = (uint32_t)p1;
  const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
  const uint32_t n3 = (uint32_t)p0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

__global__ void __launch_bounds__(256)
randn_kernel(void* __restrict__ out, int dt, int64_t rows, int64_t cols, int64_t ld_out, int64_t row0, int64_t col0,
             int64_t full_cols, uint32_t key0, uint32_t key1, uint32_t base_offset, float mean, float stddev) {
  const int64_t n = rows * cols;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = t / cols, c = t - r * cols;
    const uint64_t i = (uint64_t)((row0 + r) * full_cols + col0 + c);   // index in the full tensor
    uint32_t ctr[4] = {(uint32_t)(i >> 1) + base_offset, 0u, 0u, 0u};
    philox4x32_10(ctr, key0, key1);
    const uint32_t w1 = (i & 1) ? ctr[2] : ctr[0], w2 = (i & 1) ? ctr[3] : ctr[1];
    const float u1 = fmaxf((float)(w1 >> 8) * 5.9604644775390625e-8f, 1e-10f);
    const float u2 = (float)(w2 >> 8) * 5.9604644775390625e-8f;
    const float z = sqrtf(-2.0f * logf(u1)) * cosf(6.283185307179586f * u2);
    store_float(out, dt, r * ld_out + c, fmaf(stddev, z, mean));
  }
}

}  // namespace kd

using namespace kd;

KD_API int kd_randn(const kd_tensor* out, uint64_t seed, uint32_t base_offset, float mean, float stddev, int64_t row0,
                    int64_t col0, int64_t full_cols) {
  KD_TRY(require_init());
  KD_REQUIRE(out != nullptr, "null tensor");
  KD_REQUIRE(is_float_dtype(out->dtype), "randn needs a floating-point output");
  const int64_t n = numel(out);
  if (n == 0) return KD_OK;
  int64_t rows, cols, ld;
  if (full_cols <= 0) {
    // plain case: the tensor is the whole tensor, numbered in row-major order
    KD_REQUIRE(is_contiguous(out), "randn: a whole tensor must be contiguous");
    KD_REQUIRE(row0 == 0 && col0 == 0, "randn: row0 / col0 need full_cols");
    rows = 1; cols = n; ld = n; full_cols = n;
  } else {
    KD_REQUIRE(out->ndim == 2 && out->strides[1] == 1 && out->strides[0] >= out->shape[1],
               "randn: a slice must be a 2-D tensor with unit column stride");
    rows = out->shape[0]; cols = out->shape[1]; ld = out->strides[0];
    KD_REQUIRE(row0 >= 0 && col0 >= 0 && col0 + cols <= full_cols, "randn: slice [%lld.., %lld..%lld) outside rows of %lld columns",
               (long long)row0, (long long)col0, (long long)(col0 + cols), (long long)full_cols);
  }
  void* p = nullptr;
  KD_TRY(tensor_ptr(out, &p));
  const int64_t blocks = (n + 255) / 256;
  const int grid = (int)(blocks < (int64_t)ctx().sm_count * 16 ? blocks : (int64_t)ctx().sm_count * 16);
  randn_kernel<<<grid, 256, 0, ctx().stream>>>(p, out->dtype, rows, cols, ld, row0, col0, full_cols, (uint32_t)(seed & 0xFFFFFFFFu),
                                               (uint32_t)(seed >> 32), base_offset, mean, stddev);
  return after_launch("randn_kernel");
}
