// One-shot all-reduce over peer memory, fused with the residual add and RMSNorm that follow it in
// a tensor-parallel decode step.
//
// Tensor parallelism (an addition: the reference is single-device) leaves every rank with a
// partial sum of o_proj / down_proj, [sequences, hidden] fp32: 80 KB for 8 sequences of the 4B
// model.  A library all-reduce costs its launch and protocol latency 72 times per decode step for
// these small messages, and is followed by a kernel that adds the residual and normalises.  Here
// one kernel does all of it over NVLink peer memory with plain loads and stores:
//
//   every rank owns a buffer that its peers have mapped (CUDA IPC): two data slots and a table of
//   flags.  CTA r of a call handles sequence row r:
//     1. sums its own split-K partials of row r (fixed order) into slot (seq & 1) of ITS buffer;
//     2. fence (system scope), then writes the call's tag into flag [slot][r][my rank] of EVERY
//        rank's buffer (a store into peer memory);
//     3. waits, polling its LOCAL flags only, until all ranks' tags for row r are there (bounded:
//        about five seconds, then error code 601, and the call's output is undefined);
//     4. reads row r from every rank's slot in rank order (peer loads, L1 bypassed), adds the
//        residual, writes the fp32 sum and the bf16 RMSNorm of it.
//   Rank order makes the sum bit-identical on every rank.  A slot is rewritten two calls later; by
//   then every peer has left the call that read it, because it had to publish its flag for the
//   next call first.  The call counter lives in device memory and is advanced by the last CTA, so
//   a captured graph can be replayed.
//
// No TMA, no multicast, no multimem: ordinary ld/st on mapped peer addresses.  With fewer GPUs
// than ranks the same kernel runs all ranks in one cooperative launch on one GPU (blockIdx.y = rank,
// buffers all local), which is how the single-GPU tests exercise the protocol, including a rank
// whose flag never arrives.
#include <vector>

#include "common.cuh"
#include "kernels.cuh"
#include "p2p_layout.cuh"

namespace kd {

constexpr int P2P_THREADS = 128;
constexpr int P2P_MAXV = 8;                                 // 8-element vectors per thread: rows up to 8192 wide

struct P2pState {
  bool ready = false;
  int nranks = 1, rank = 0;
  int emulate = 0;                        // > 0: that many ranks emulated on this GPU
  long long silent_wait = 0;              // > 0: the peers are local stand-ins that never answer (self-test); the wait bound to use
  void* local[P2P_MAX_RANKS] = {nullptr}; // buffers this process allocated (1, or `emulate`)
  void* peer[P2P_MAX_RANKS] = {nullptr};  // address of every rank's buffer as seen from here
  bool opened[P2P_MAX_RANKS] = {false};
  unsigned* seq = nullptr;                // [P2P_MAX_RANKS] call counters (one per emulated rank), [8] completion tickets,
                                          // [16] call counter of the layer kernel, [17] its completion ticket
};
static P2pState g_p2p;

int p2p_peers(P2pPeers* out) {
  if (!g_p2p.ready || g_p2p.emulate) return fail(KD_ERR_INVALID, "peer buffers are not connected (kd_p2p_prepare + kd_p2p_connect)");
  for (int r = 0; r < P2P_MAX_RANKS; ++r) out->buf[r] = static_cast<char*>(g_p2p.peer[r]);
  out->nranks = g_p2p.nranks;
  out->rank = g_p2p.rank;
  out->layer_seq = g_p2p.seq + 2 * P2P_MAX_RANKS;
  out->wait_cycles = g_p2p.silent_wait > 0 ? g_p2p.silent_wait : P2P_WAIT_CYCLES;
  return KD_OK;
}

struct P2pArgs {
  char* buf[P2P_MAX_RANKS];
  int nranks, rank, emulate;
  int drop_rank;                 // test support: this rank never publishes its flags (-1: none)
  long long wait_cycles;
  unsigned* seq;
  const float* x;                // [splits][rows][n] partial sums (per emulated rank: + rank * x_rank_stride)
  int64_t x_rank_stride;
  int splits, rows, n;
  const float* resid;            // [rows][n] fp32 or null
  const void* w; int dt_w;
  float eps;
  float* sum_out;                // [rows][n] fp32 (per emulated rank: + rank * out_rank_stride)
  __nv_bfloat16* norm_out;
  int64_t out_rank_stride;
  int* err;
};

__global__ void __launch_bounds__(P2P_THREADS) allreduce_add_rmsnorm_kernel(const P2pArgs a) {
  __shared__ float red[P2P_THREADS / 32];
  __shared__ int failed;
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const int me = a.emulate ? (int)blockIdx.y : a.rank;
  const unsigned seq = a.seq[me];
  const int slot = (int)(seq & 1u);
  const unsigned tag = seq + 1u;
  const int nvec = a.n / 8;
  if (threadIdx.x == 0) failed = 0;
  const float* x = a.x + (a.emulate ? (int64_t)me * a.x_rank_stride : 0);
  float* my_row = reinterpret_cast<float*>(a.buf[me] + (size_t)slot * P2P_SLOT_BYTES) + (int64_t)row * a.n;
  // 1. this rank's contribution to the row
  for (int vi = threadIdx.x; vi < nvec; vi += P2P_THREADS) {
    float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
    for (int sp = 0; sp < a.splits; ++sp) {
      const float4* s = reinterpret_cast<const float4*>(x + ((int64_t)sp * a.rows + row) * a.n) + vi * 2;
      const float4 p0 = s[0], p1 = s[1];
      lo.x += p0.x; lo.y += p0.y; lo.z += p0.z; lo.w += p0.w;
      hi.x += p1.x; hi.y += p1.y; hi.z += p1.z; hi.w += p1.w;
    }
    reinterpret_cast<float4*>(my_row)[vi * 2] = lo;
    reinterpret_cast<float4*>(my_row)[vi * 2 + 1] = hi;
  }
  __syncthreads();
  // 2. publish: the row is complete in this rank's slot
  if ((int)threadIdx.x < a.nranks && me != a.drop_rank) {
    __threadfence_system();
    unsigned* flags = reinterpret_cast<unsigned*>(a.buf[threadIdx.x] + P2P_FLAG_OFFSET);
    st_release_sys(flags + ((size_t)slot * P2P_MAX_ROWS + row) * P2P_MAX_RANKS + me, tag);
  }
  // 3. wait for every rank's row (local flags only)
  if ((int)threadIdx.x < a.nranks) {
    const unsigned* f = reinterpret_cast<const unsigned*>(a.buf[me] + P2P_FLAG_OFFSET) +
                        ((size_t)slot * P2P_MAX_ROWS + row) * P2P_MAX_RANKS + threadIdx.x;
    const long long t0 = clock64();
    int spins = 0;
    while (ld_acquire_sys(f) != tag) {
      if (((++spins) & 7) == 0 && clock64() - t0 > a.wait_cycles) {
        failed = 1;
        if (atomicCAS(a.err, 0, 601) == 0) { a.err[1] = row; a.err[2] = (int)threadIdx.x; a.err[3] = me; }
        break;
      }
    }
  }
  __syncthreads();
  // 4. sum over ranks in rank order, residual, RMSNorm (skipped after a wait that ran out)
  float v[P2P_MAXV][8];
  float ss = 0.f;
  const bool go = failed == 0;
#pragma unroll
  for (int t = 0; t < P2P_MAXV; ++t) {
    const int vi = threadIdx.x + t * P2P_THREADS;
    if (go && vi < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[t][e] = 0.f;
      for (int r = 0; r < a.nranks; ++r) {
        const float4* s = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.buf[r] + (size_t)slot * P2P_SLOT_BYTES) + (int64_t)row * a.n) + vi * 2;
        const float4 p0 = ld_peer_f4(s), p1 = ld_peer_f4(s + 1);
        v[t][0] += p0.x; v[t][1] += p0.y; v[t][2] += p0.z; v[t][3] += p0.w;
        v[t][4] += p1.x; v[t][5] += p1.y; v[t][6] += p1.z; v[t][7] += p1.w;
      }
      if (a.resid) {
        const float4* rp = reinterpret_cast<const float4*>(a.resid + (int64_t)row * a.n) + vi * 2;
        const float4 p0 = rp[0], p1 = rp[1];
        v[t][0] += p0.x; v[t][1] += p0.y; v[t][2] += p0.z; v[t][3] += p0.w;
        v[t][4] += p1.x; v[t][5] += p1.y; v[t][6] += p1.z; v[t][7] += p1.w;
      }
      if (a.sum_out) {
        float4* so = reinterpret_cast<float4*>(a.sum_out + (a.emulate ? (int64_t)me * a.out_rank_stride : 0) + (int64_t)row * a.n) + vi * 2;
        so[0] = make_float4(v[t][0], v[t][1], v[t][2], v[t][3]);
        so[1] = make_float4(v[t][4], v[t][5], v[t][6], v[t][7]);
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
  for (int i = 0; i < P2P_THREADS / 32; ++i) tot += red[i];
  const float sc = 1.0f / sqrtf(tot / (float)a.n + a.eps);
#pragma unroll
  for (int t = 0; t < P2P_MAXV; ++t) {
    const int vi = threadIdx.x + t * P2P_THREADS;
    if (go && vi < nvec) {
      uint4 o;
      __nv_bfloat16* ho = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
      for (int e = 0; e < 8; ++e) ho[e] = __float2bfloat16_rn((v[t][e] * sc) * load_float(a.w, a.dt_w, vi * 8 + e));
      reinterpret_cast<uint4*>(a.norm_out + (a.emulate ? (int64_t)me * a.out_rank_stride : 0) + (int64_t)row * a.n)[vi] = o;
    }
  }
  // 5. the last CTA of this rank advances the call counter
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned ticket = atomicAdd(a.seq + P2P_MAX_RANKS + me, 1u);
    if (ticket == (unsigned)a.rows - 1) {
      a.seq[P2P_MAX_RANKS + me] = 0u;
      a.seq[me] = seq + 1u;
      __threadfence();
    }
  }
}

static int p2p_alloc_local(int count) {
  for (int i = 0; i < count; ++i) {
    if (g_p2p.local[i]) continue;
    KD_CUDA_CHECK(cudaMalloc(&g_p2p.local[i], P2P_BUF_BYTES));
    KD_CUDA_CHECK(cudaMemsetAsync(g_p2p.local[i], 0, P2P_BUF_BYTES, ctx().stream));
  }
  if (!g_p2p.seq) {
    KD_CUDA_CHECK(cudaMalloc(&g_p2p.seq, (2 * P2P_MAX_RANKS + 2) * sizeof(unsigned)));
    KD_CUDA_CHECK(cudaMemsetAsync(g_p2p.seq, 0, (2 * P2P_MAX_RANKS + 2) * sizeof(unsigned), ctx().stream));
  }
  KD_CUDA_CHECK(cudaStreamSynchronize(ctx().stream));
  return KD_OK;
}

int p2p_shutdown() {
  if (g_p2p.seq || g_p2p.local[0]) cudaStreamSynchronize(ctx().stream);
  for (int r = 0; r < P2P_MAX_RANKS; ++r) {
    if (g_p2p.opened[r]) cudaIpcCloseMemHandle(g_p2p.peer[r]);
    if (g_p2p.local[r]) cudaFree(g_p2p.local[r]);
  }
  if (g_p2p.seq) cudaFree(g_p2p.seq);
  cudaGetLastError();
  g_p2p = P2pState();
  return KD_OK;
}

}  // namespace kd

using namespace kd;

KD_API int kd_p2p_prepare(char* handle_out, size_t handle_bytes) {
  KD_TRY(require_init());
  KD_REQUIRE(handle_out && handle_bytes >= sizeof(cudaIpcMemHandle_t), "handle buffer must hold %zu bytes", sizeof(cudaIpcMemHandle_t));
  KD_REQUIRE(!g_p2p.ready, "peer buffers are already connected");
  KD_TRY(p2p_alloc_local(1));
  cudaIpcMemHandle_t h;
  KD_CUDA_CHECK(cudaIpcGetMemHandle(&h, g_p2p.local[0]));
  memcpy(handle_out, &h, sizeof(h));
  return KD_OK;
}

KD_API int kd_p2p_connect(int nranks, int rank, const char* handles, size_t handle_bytes) {
  KD_TRY(require_init());
  KD_REQUIRE(nranks >= 1 && nranks <= P2P_MAX_RANKS && rank >= 0 && rank < nranks, "bad rank %d of %d (at most %d ranks)", rank, nranks, P2P_MAX_RANKS);
  KD_REQUIRE(handles && handle_bytes >= sizeof(cudaIpcMemHandle_t), "handles must be %d records of at least %zu bytes", nranks, sizeof(cudaIpcMemHandle_t));
  KD_REQUIRE(!g_p2p.ready && g_p2p.local[0], "call kd_p2p_prepare first (once)");
  for (int r = 0; r < nranks; ++r) {
    if (r == rank) { g_p2p.peer[r] = g_p2p.local[0]; continue; }
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + (size_t)r * handle_bytes, sizeof(h));
    cudaError_t e = cudaIpcOpenMemHandle(&g_p2p.peer[r], h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(KD_ERR_CUDA, "cudaIpcOpenMemHandle for rank %d failed: %s", r, cudaGetErrorString(e));
    }
    g_p2p.opened[r] = true;
  }
  g_p2p.nranks = nranks;
  g_p2p.rank = rank;
  g_p2p.emulate = 0;
  g_p2p.ready = true;
  return KD_OK;
}

KD_API int kd_p2p_emulate(int nranks) {
  KD_TRY(require_init());
  KD_REQUIRE(nranks >= 1 && nranks <= P2P_MAX_RANKS, "1..%d emulated ranks", P2P_MAX_RANKS);
  KD_REQUIRE(!g_p2p.ready, "peer buffers are already connected");
  KD_TRY(p2p_alloc_local(nranks));
  for (int r = 0; r < nranks; ++r) g_p2p.peer[r] = g_p2p.local[r];
  g_p2p.nranks = nranks;
  g_p2p.rank = 0;
  g_p2p.emulate = nranks;
  g_p2p.ready = true;
  return KD_OK;
}

KD_API int kd_p2p_selftest_silent_peers(int nranks, uint32_t wait_cycles, uint32_t answered_tag) {
  KD_TRY(require_init());
  KD_REQUIRE(nranks >= 2 && nranks <= P2P_MAX_RANKS, "2..%d ranks", P2P_MAX_RANKS);
  KD_REQUIRE(wait_cycles > 0, "wait_cycles must be positive");
  KD_REQUIRE(!g_p2p.ready, "peer buffers are already connected");
  KD_TRY(p2p_alloc_local(nranks));
  for (int r = 0; r < nranks; ++r) g_p2p.peer[r] = g_p2p.local[r];
  g_p2p.nranks = nranks;
  g_p2p.rank = 0;
  g_p2p.emulate = 0;
  g_p2p.silent_wait = (long long)wait_cycles;
  if (answered_tag) {
    // the stand-ins "answered" the launch with this tag: their flags in this rank's buffer carry it,
    // their partial sums are the zeros the buffers were cleared to
    std::vector<unsigned> flags(2 * P2P_MAX_ROWS * P2P_MAX_RANKS, 0u);
    for (size_t i = 0; i < flags.size(); ++i)
      if ((int)(i % P2P_MAX_RANKS) >= 1 && (int)(i % P2P_MAX_RANKS) < nranks) flags[i] = answered_tag;
    KD_CUDA_CHECK(cudaMemcpyAsync(static_cast<char*>(g_p2p.local[0]) + P2P_LAYER_FLAG_OFFSET, flags.data(), flags.size() * sizeof(unsigned),
                                  cudaMemcpyHostToDevice, ctx().stream));
    KD_CUDA_CHECK(cudaStreamSynchronize(ctx().stream));
  }
  g_p2p.ready = true;
  return KD_OK;
}

KD_API int kd_p2p_info(int* ready, int* nranks, int* rank) {
  if (ready) *ready = g_p2p.ready ? 1 : 0;
  if (nranks) *nranks = g_p2p.nranks;
  if (rank) *rank = g_p2p.rank;
  return KD_OK;
}

KD_API int kd_p2p_disconnect(void) { return p2p_shutdown(); }

static int allreduce_add_rmsnorm(const kd_tensor* x, const kd_tensor* residual, const kd_tensor* weight, float eps,
                                 const kd_tensor* sum_out, const kd_tensor* norm_out, int drop_rank, long long wait_cycles) {
  KD_TRY(require_init());
  KD_REQUIRE(g_p2p.ready, "peer buffers are not connected (kd_p2p_prepare + kd_p2p_connect, or kd_p2p_emulate)");
  KD_REQUIRE(x && weight && norm_out, "null tensor");
  const int emu = g_p2p.emulate;
  KD_REQUIRE(norm_out->dtype == KD_BF16 && is_contiguous(norm_out) && norm_out->ndim >= 2, "norm_out must be contiguous bf16 [rows, n]");
  const int64_t n = norm_out->shape[norm_out->ndim - 1];
  const int64_t rows = numel(norm_out) / n / (emu ? emu : 1);
  KD_REQUIRE(n > 0 && n % 8 == 0 && n <= 8 * P2P_THREADS * P2P_MAXV, "row width %lld must be a multiple of 8 and at most %d", (long long)n,
             8 * P2P_THREADS * P2P_MAXV);
  KD_REQUIRE(rows >= 1 && rows <= P2P_MAX_ROWS, "%lld rows; the one-shot all-reduce handles 1..%d", (long long)rows, P2P_MAX_ROWS);
  KD_REQUIRE((size_t)rows * n * sizeof(float) <= P2P_SLOT_BYTES, "%lld x %lld fp32 does not fit the %zu-byte peer slot", (long long)rows,
             (long long)n, P2P_SLOT_BYTES);
  const int64_t per_rank = numel(x) / (emu ? emu : 1);
  KD_REQUIRE(x->dtype == KD_F32 && is_contiguous(x) && per_rank > 0 && per_rank % (rows * n) == 0,
             "x must be contiguous fp32 [splits, rows, n] partial sums");
  const int splits = (int)(per_rank / (rows * n));
  KD_REQUIRE(numel(weight) == n && is_contiguous(weight) && is_float_dtype(weight->dtype), "weight must be contiguous [n]");
  if (residual) KD_REQUIRE(residual->dtype == KD_F32 && is_contiguous(residual) && numel(residual) == rows * n, "residual must be contiguous fp32 [rows, n]");
  if (sum_out) KD_REQUIRE(sum_out->dtype == KD_F32 && is_contiguous(sum_out) && numel(sum_out) == rows * n * (emu ? emu : 1), "sum_out must be contiguous fp32 [rows, n]");
  void *px, *pw, *pn, *pr = nullptr, *ps = nullptr;
  KD_TRY(tensor_ptr(x, &px));
  KD_TRY(tensor_ptr(weight, &pw));
  KD_TRY(tensor_ptr(norm_out, &pn));
  if (residual) KD_TRY(tensor_ptr(residual, &pr));
  if (sum_out) KD_TRY(tensor_ptr(sum_out, &ps));
  KD_REQUIRE(((reinterpret_cast<uintptr_t>(px) | reinterpret_cast<uintptr_t>(pn) | reinterpret_cast<uintptr_t>(pr) | reinterpret_cast<uintptr_t>(ps)) & 15) == 0,
             "operands must be 16-byte aligned");
  P2pArgs a{};
  for (int r = 0; r < g_p2p.nranks; ++r) a.buf[r] = static_cast<char*>(g_p2p.peer[r]);
  a.nranks = g_p2p.nranks; a.rank = g_p2p.rank; a.emulate = emu;
  a.drop_rank = drop_rank;
  a.wait_cycles = wait_cycles;
  a.seq = g_p2p.seq;
  a.x = static_cast<const float*>(px); a.x_rank_stride = per_rank;
  a.splits = splits; a.rows = (int)rows; a.n = (int)n;
  a.resid = static_cast<const float*>(pr);
  a.w = pw; a.dt_w = weight->dtype; a.eps = eps;
  a.sum_out = static_cast<float*>(ps);
  a.norm_out = static_cast<__nv_bfloat16*>(pn);
  a.out_rank_stride = rows * n;
  a.err = ctx().error_flag;
  if (emu) {
    // all emulated ranks in one cooperative launch: their CTAs wait on one another
    KD_REQUIRE(rows * emu <= ctx().sm_count, "%lld rows x %d emulated ranks exceed one wave of CTAs", (long long)rows, emu);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows, (unsigned)emu);
    cfg.blockDim = dim3(P2P_THREADS);
    cfg.stream = ctx().stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    KD_CUDA_CHECK(cudaLaunchKernelEx(&cfg, allreduce_add_rmsnorm_kernel, a));
  } else {
    KD_CUDA_CHECK(launch_ex(allreduce_add_rmsnorm_kernel, dim3((unsigned)rows), dim3(P2P_THREADS), 0, a));
  }
  return after_launch("allreduce_add_rmsnorm_kernel");
}

KD_API int kd_allreduce_add_rmsnorm(const kd_tensor* x, const kd_tensor* residual, const kd_tensor* weight, float eps,
                                    const kd_tensor* sum_out, const kd_tensor* norm_out) {
  return allreduce_add_rmsnorm(x, residual, weight, eps, sum_out, norm_out, -1, P2P_WAIT_CYCLES);
}

KD_API int kd_p2p_selftest_dropped_flag(const kd_tensor* x, const kd_tensor* weight, const kd_tensor* norm_out, int drop_rank,
                                        uint32_t wait_cycles) {
  KD_REQUIRE(g_p2p.ready && g_p2p.emulate > 0, "the dropped-flag self-test runs on emulated ranks (kd_p2p_emulate)");
  return allreduce_add_rmsnorm(x, nullptr, weight, 1e-6f, nullptr, norm_out, drop_rank, (long long)wait_cycles);
}
