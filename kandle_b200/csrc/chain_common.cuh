// Helpers shared by the persistent decode kernels (decode_chain.cu, decode_layer.cu): grid-wide
// counters in global memory with bounded waits, the reference's SiLU, the 128-thread barrier of the
// epilogue warps.
#pragma once
#include "common.cuh"
#include "sm100.cuh"

namespace kd {

__device__ __forceinline__ float chain_silu(float x) {
  const float c = fminf(fmaxf(x, -88.f), 88.f);   // the reference clamps before exp (pointwise/ops.ts:299)
  return __fdividef(x, 1.f + __expf(-c));
}

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_add(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait until counter >= target (about one second, then the error word and the CTA's abort flag).
__device__ __forceinline__ bool counter_wait(const unsigned* cnt, unsigned target, volatile int* abort_flag, int* err, int code) {
  if (ld_acquire_u32(cnt) >= target) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (ld_acquire_u32(cnt) < target) {
    if (((++spins) & 15) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > sm100::WAIT_CYCLE_LIMIT) {
        *abort_flag = 1;
        if (atomicCAS(err, 0, code) == 0) { err[1] = (int)blockIdx.x; err[2] = (int)threadIdx.x; err[3] = (int)target; }
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// The same barrier, returning to all 128 threads whether ANY of them passed a true flag: decisions
// that steer the threads past further barriers must be uniform.
__device__ __forceinline__ bool epi_bar_any(bool flag) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"((uint32_t)flag)
      : "memory");
  return out != 0;
}

}  // namespace kd
