// Key `matmul`: general strided batched GEMM with fp32 accumulation on the CUDA cores.
//
// This is the exact-fp32 path (tcgen05 has no fp32 input format; tf32 would break the fp32
// parity bound), and the fallback for operand layouts the tensor-core path does not take.  It
// accepts everything MatmulDispatchResult can describe
// (packages/core/src/dispatch/matmulOps.ts:32-125): transpose flags, 4-D element strides with
// broadcast batch dims, alpha/beta/C -- a superset of the reference shader, which only honours
// one batch stride (packages/backend-webgpu/src/kernels/matrix/builder.ts:948-978).
//
// 128x128x16 CTA tile, 256 threads, 8x8 outputs per thread held in registers.
#include "common.cuh"
#include "kernels.cuh"

namespace kd {

struct MmParams {
  int64_t M, N, K;
  int64_t b0, b1;
  // logical strides: A(m,k), B(k,n), C(m,n), O(m,n) plus two batch dims each
  int64_t a_b0, a_b1, a_m, a_k;
  int64_t b_b0, b_b1, b_k, b_n;
  int64_t c_b0, c_b1, c_m, c_n;
  int64_t o_b0, o_b1, o_m, o_n;
  int dt_a, dt_b, dt_c, dt_o;
  int has_c;
  float alpha, beta;
};

constexpr int BM = 128, BN = 128, BK = 16, LDS = 132;

__global__ void __launch_bounds__(256) matmul_f32_kernel(const void* __restrict__ A, const void* __restrict__ B,
                                                        const void* __restrict__ C, void* __restrict__ O, MmParams p) {
  __shared__ __align__(16) float As[BK][LDS];
  __shared__ __align__(16) float Bs[BK][LDS];
  const int t = threadIdx.x;
  const int tx = t & 15, ty = t >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
  const int64_t bz = blockIdx.z;
  const int64_t ib0 = bz / p.b1, ib1 = bz - ib0 * p.b1;
  const int64_t a_base = ib0 * p.a_b0 + ib1 * p.a_b1;
  const int64_t b_base = ib0 * p.b_b0 + ib1 * p.b_b1;
  const bool a_kfast = (p.a_k == 1), b_kfast = (p.b_k == 1);

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  for (int64_t k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = t + i * 256;
      int m, k;
      if (a_kfast) { k = e & 15; m = e >> 4; } else { m = e & 127; k = e >> 7; }
      const int64_t gm = m0 + m, gk = k0 + k;
      As[k][m] = (gm < p.M && gk < p.K) ? load_float(A, p.dt_a, a_base + gm * p.a_m + gk * p.a_k) : 0.f;
      int n, kb;
      if (b_kfast) { kb = e & 15; n = e >> 4; } else { n = e & 127; kb = e >> 7; }
      const int64_t gn = n0 + n, gkb = k0 + kb;
      Bs[kb][n] = (gn < p.N && gkb < p.K) ? load_float(B, p.dt_b, b_base + gkb * p.b_k + gn * p.b_n) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[k][64 + tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }

  const int64_t c_base = ib0 * p.c_b0 + ib1 * p.c_b1;
  const int64_t o_base = ib0 * p.o_b0 + ib1 * p.o_b1;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (gm >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (gn >= p.N) continue;
      float r = p.alpha * acc[i][j];
      if (p.has_c) r += p.beta * load_float(C, p.dt_c, c_base + gm * p.c_m + gn * p.c_n);
      store_float(O, p.dt_o, o_base + gm * p.o_m + gn * p.o_n, r);
    }
  }
}

// Splits a tensor of rank 2..4 into (batch0, batch1, row, col) strides / extents.
static void split4(const kd_tensor* t, int64_t* ext, int64_t* st) {
  for (int i = 0; i < 4; ++i) { ext[i] = 1; st[i] = 0; }
  const int shift = 4 - t->ndim;
  for (int d = 0; d < t->ndim; ++d) { ext[d + shift] = t->shape[d]; st[d + shift] = t->strides[d]; }
}

int matmul_f32_dispatch(const kd_matmul_cfg* cfg, const kd_tensor* a, const kd_tensor* b, const kd_tensor* c,
                        const kd_tensor* out) {
  int64_t ea[4], sa[4], eb[4], sb[4], eo[4], so[4], ec[4], sc[4];
  KD_REQUIRE(a->ndim >= 2 && a->ndim <= 4 && b->ndim >= 2 && b->ndim <= 4 && out->ndim >= 2 && out->ndim <= 4,
             "matmul operands must have rank 2..4");
  split4(a, ea, sa);
  split4(b, eb, sb);
  split4(out, eo, so);
  MmParams p{};
  p.M = cfg->M; p.N = cfg->N; p.K = cfg->K;
  const int64_t am = cfg->transpose_a ? ea[3] : ea[2], ak = cfg->transpose_a ? ea[2] : ea[3];
  const int64_t bk = cfg->transpose_b ? eb[3] : eb[2], bn = cfg->transpose_b ? eb[2] : eb[3];
  KD_REQUIRE(am == p.M && ak == p.K, "matmul: A is [%lld,%lld] but cfg says M=%lld K=%lld", (long long)am, (long long)ak,
             (long long)p.M, (long long)p.K);
  KD_REQUIRE(bk == p.K && bn == p.N, "matmul: B is [%lld,%lld] but cfg says K=%lld N=%lld", (long long)bk, (long long)bn,
             (long long)p.K, (long long)p.N);
  KD_REQUIRE(eo[2] == p.M && eo[3] == p.N, "matmul: output is [%lld,%lld], expected [%lld,%lld]", (long long)eo[2],
             (long long)eo[3], (long long)p.M, (long long)p.N);
  p.b0 = eo[0]; p.b1 = eo[1];
  for (int d = 0; d < 2; ++d) {
    KD_REQUIRE(ea[d] == eo[d] || ea[d] == 1, "matmul: A batch dim %d (%lld) does not broadcast to %lld", d, (long long)ea[d], (long long)eo[d]);
    KD_REQUIRE(eb[d] == eo[d] || eb[d] == 1, "matmul: B batch dim %d (%lld) does not broadcast to %lld", d, (long long)eb[d], (long long)eo[d]);
  }
  p.a_b0 = ea[0] == 1 ? 0 : sa[0]; p.a_b1 = ea[1] == 1 ? 0 : sa[1];
  p.b_b0 = eb[0] == 1 ? 0 : sb[0]; p.b_b1 = eb[1] == 1 ? 0 : sb[1];
  p.a_m = cfg->transpose_a ? sa[3] : sa[2]; p.a_k = cfg->transpose_a ? sa[2] : sa[3];
  p.b_k = cfg->transpose_b ? sb[3] : sb[2]; p.b_n = cfg->transpose_b ? sb[2] : sb[3];
  p.o_b0 = so[0]; p.o_b1 = so[1]; p.o_m = so[2]; p.o_n = so[3];
  p.dt_a = a->dtype; p.dt_b = b->dtype; p.dt_o = out->dtype; p.dt_c = KD_F32;
  p.alpha = cfg->alpha; p.beta = cfg->beta;
  p.has_c = (cfg->has_c && c != nullptr && cfg->beta != 0.f) ? 1 : 0;
  void *pa = nullptr, *pb = nullptr, *pc = nullptr, *po = nullptr;
  KD_TRY(tensor_ptr(a, &pa));
  KD_TRY(tensor_ptr(b, &pb));
  KD_TRY(tensor_ptr(out, &po));
  if (p.has_c) {
    KD_REQUIRE(c->ndim <= 4, "matmul: C rank must be <= 4");
    split4(c, ec, sc);
    for (int d = 0; d < 4; ++d)
      KD_REQUIRE(ec[d] == eo[d] || ec[d] == 1, "matmul: C dim %d (%lld) does not broadcast to %lld", d, (long long)ec[d], (long long)eo[d]);
    p.c_b0 = ec[0] == 1 ? 0 : sc[0]; p.c_b1 = ec[1] == 1 ? 0 : sc[1];
    p.c_m = ec[2] == 1 ? 0 : sc[2]; p.c_n = ec[3] == 1 ? 0 : sc[3];
    p.dt_c = c->dtype;
    KD_TRY(tensor_ptr(c, &pc));
  }
  if (p.M == 0 || p.N == 0 || p.b0 * p.b1 == 0) return KD_OK;
  const int64_t gx = (p.N + BN - 1) / BN, gy = (p.M + BM - 1) / BM, gz = p.b0 * p.b1;
  KD_REQUIRE(gy <= 65535 && gz <= 65535, "matmul: grid too large (M tiles %lld, batch %lld)", (long long)gy, (long long)gz);
  dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)gz);
  matmul_f32_kernel<<<grid, 256, 0, ctx().stream>>>(pa, pb, pc, po, p);
  return after_launch("matmul_f32_kernel");
}

}  // namespace kd
