// Self-test of the bounded-wait error path that every pipelined kernel of this library relies on.
//
// The tensor-core kernels wait on mbarriers (TMA arrivals, tcgen05.commit) and, in the decode chain
// kernel, on counters in global memory.  Each wait gives up after about a second, records an error
// code in the context's device error word, raises the CTA's abort flag so that the other roles
// drain, and the kernel returns normally; the next synchronising call reports KD_ERR_DEVICE and
// the context stays usable.  kd_selftest_wait_timeout exercises exactly that code
// (sm100::mbar_wait_limit) with a wait that nothing will ever satisfy and a short limit, so that
// the path can be tested on a GPU without faulting, trapping or hanging it.
#include "common.cuh"
#include "sm100.cuh"

namespace kd {

__global__ void selftest_wait_timeout_kernel(long long limit_cycles, int* err, int* reached_end) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&bar, 1);     // one arrival expected; nobody arrives
    abort_flag = 0;
    sm100::fence_mbar_init();
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) ok = sm100::mbar_wait_limit(&bar, 0, &abort_flag, err, 901, limit_cycles);
  __syncthreads();
  // the other warps see the abort flag, as the consumer roles of the real kernels do
  if (threadIdx.x == 32 && abort_flag) atomicAdd(reached_end, 1);
  if (threadIdx.x == 0 && !ok) atomicAdd(reached_end, 1);
}

}  // namespace kd

using namespace kd;

KD_API int kd_selftest_wait_timeout(uint32_t limit_us) {
  KD_TRY(require_init());
  KD_REQUIRE(limit_us >= 1 && limit_us <= 100000, "limit must be 1..100000 microseconds");
  int* reached = nullptr;
  KD_CUDA_CHECK(cudaMalloc(&reached, sizeof(int)));
  KD_CUDA_CHECK(cudaMemsetAsync(reached, 0, sizeof(int), ctx().stream));
  // clock64 counts SM cycles: at most ~2 per nanosecond
  selftest_wait_timeout_kernel<<<1, 64, 0, ctx().stream>>>((long long)limit_us * 2000, ctx().error_flag, reached);
  int s = after_launch("selftest_wait_timeout_kernel");
  int h = 0;
  cudaError_t e = cudaMemcpyAsync(&h, reached, sizeof(int), cudaMemcpyDeviceToHost, ctx().stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx().stream);
  cudaFree(reached);
  if (s != KD_OK) return s;
  if (e != cudaSuccess) return fail(KD_ERR_CUDA, "self-test kernel failed: %s", cudaGetErrorString(e));
  if (h != 2) return fail(KD_ERR_CUDA, "self-test kernel did not reach its end after the wait ran out");
  return KD_OK;   // the error word is now set: the next kd_synchronize reports KD_ERR_DEVICE (code 901)
}
