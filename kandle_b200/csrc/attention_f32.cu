// Key `flash_attention`, exact-fp32 path on the CUDA cores (any storage dtype, fp32 math).
//
// Same mathematics as the reference shader
// (packages/backend-webgpu/src/kernels/attention/builder.ts:138-329): score = dot(q,k)*scale,
// causal / out-of-range columns get -1e20, running max starts at -1e20, online-softmax
// rescaling per KV tile, final O/l.  The tiling is different: one warp owns one query row (the
// reference uses 8x4 tiles sized for 16 KB of workgroup memory and a serial per-row softmax),
// 16 rows per CTA share each 32-row K/V tile staged in shared memory, the softmax statistics
// live in registers and are combined with warp shuffles.  Unlike the reference kernel, operand
// strides are honoured (the reference assumes contiguous [B,H,S,D]).
#include "common.cuh"
#include "kernels.cuh"

namespace kd {


constexpr int ATT_WARPS = 16;
constexpr int ATT_TKV = 32;

template <int DPL>  // head dims per lane: head_dim <= 32*DPL, padded with zeros
__global__ void __launch_bounds__(ATT_WARPS * 32) attention_f32_kernel(const void* __restrict__ Q,
                                                                      const void* __restrict__ K,
                                                                      const void* __restrict__ V, void* __restrict__ O,
                                                                      AttnParams p) {
  constexpr int D = 32 * DPL;   // padded head dim; p.D is the real one
  extern __shared__ float smem[];
  float* Ks = smem;                          // [TKV][D+1]
  float* Vs = Ks + ATT_TKV * (D + 1);        // [TKV][D]
  float* Qs = Vs + ATT_TKV * D;              // [WARPS][D]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int row0 = blockIdx.x * ATT_WARPS;
  const int row = row0 + warp;
  const bool row_ok = row < p.Sq;
  const float NEG = -1e20f;

  const int64_t q_off = (int64_t)b * p.sq[0] + (int64_t)h * p.sq[1] + (int64_t)row * p.sq[2];
  for (int d = lane; d < D; d += 32) Qs[warp * D + d] = (row_ok && d < p.D) ? load_float(Q, p.dt_q, q_off + d * p.sq[3]) : 0.f;

  float acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
  float m = NEG, l = 0.f;

  const int last_row = min(row0 + ATT_WARPS - 1, p.Sq - 1);
  const int kv_end = p.causal ? min(p.Skv, last_row + 1) : p.Skv;
  const int64_t k_base = (int64_t)b * p.sk[0] + (int64_t)hk * p.sk[1];
  const int64_t v_base = (int64_t)b * p.sv[0] + (int64_t)hk * p.sv[1];

  for (int j0 = 0; j0 < kv_end; j0 += ATT_TKV) {
    __syncthreads();
    for (int e = threadIdx.x; e < ATT_TKV * D; e += ATT_WARPS * 32) {
      const int r = e / D, d = e - r * D;
      const int j = j0 + r;
      float kv = 0.f, vv = 0.f;
      if (j < p.Skv && d < p.D) {
        kv = load_float(K, p.dt_k, k_base + (int64_t)j * p.sk[2] + d * p.sk[3]);
        vv = load_float(V, p.dt_v, v_base + (int64_t)j * p.sv[2] + d * p.sv[3]);
      }
      Ks[r * (D + 1) + d] = kv;
      Vs[r * D + d] = vv;
    }
    __syncthreads();
    if (!row_ok) continue;
    if (p.causal && j0 > row) continue;  // every column of this tile is masked for this row
    const int j = j0 + lane;
    float s;
    if (j >= p.Skv || (p.causal && j > row)) {
      s = NEG;
    } else {
      s = 0.f;
      const float* kr = Ks + lane * (D + 1);
      const float* qr = Qs + warp * D;
#pragma unroll 8
      for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
      s *= p.scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float sf = expf(m - m_new);
    const float pj = expf(s - m_new);
    l = l * sf + warp_sum(pj);
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] *= sf;
#pragma unroll 4
    for (int jj = 0; jj < ATT_TKV; ++jj) {
      const float pv = __shfl_sync(0xffffffffu, pj, jj);
      const float* vr = Vs + jj * D + lane;
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[i] = fmaf(pv, vr[32 * i], acc[i]);
    }
    m = m_new;
  }
  if (row_ok) {
    const int64_t o_off = (int64_t)b * p.so[0] + (int64_t)h * p.so[1] + (int64_t)row * p.so[2];
#pragma unroll
    for (int i = 0; i < DPL; ++i)
      if (lane + 32 * i < p.D) store_float(O, p.dt_o, o_off + (int64_t)(lane + 32 * i) * p.so[3], acc[i] / l);
  }
}

static void to4(const kd_tensor* t, int64_t* ext, int64_t* st) {
  for (int i = 0; i < 4; ++i) { ext[i] = 1; st[i] = 0; }
  const int shift = 4 - t->ndim;
  for (int d = 0; d < t->ndim; ++d) { ext[d + shift] = t->shape[d]; st[d + shift] = t->strides[d]; }
}

// Validates the operands of flash_attention and fills AttnParams (shared by all attention paths).
int attention_params(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v, const kd_tensor* out, float scale,
                     int is_causal, AttnParams* p) {
  KD_REQUIRE(q && k && v && out, "null tensor");
  KD_REQUIRE(q->ndim >= 2 && q->ndim <= 4 && k->ndim == q->ndim && v->ndim == q->ndim && out->ndim == q->ndim,
             "flash_attention operands must all have the same rank (2, 3 or 4)");
  int64_t eq[4], ek[4], ev[4], eo[4];
  to4(q, eq, p->sq); to4(k, ek, p->sk); to4(v, ev, p->sv); to4(out, eo, p->so);
  KD_REQUIRE(ek[0] == eq[0] && ev[0] == eq[0] && eo[0] == eq[0], "flash_attention: batch sizes differ");
  KD_REQUIRE(ek[3] == eq[3] && ev[3] == eq[3] && eo[3] == eq[3], "flash_attention: head dims differ");
  KD_REQUIRE(ev[1] == ek[1] && ev[2] == ek[2], "flash_attention: K and V shapes differ");
  KD_REQUIRE(eo[1] == eq[1] && eo[2] == eq[2], "flash_attention: output shape differs from Q");
  KD_REQUIRE(ek[1] > 0 && eq[1] % ek[1] == 0, "flash_attention: %lld query heads is not a multiple of %lld KV heads",
             (long long)eq[1], (long long)ek[1]);
  KD_REQUIRE(is_float_dtype(q->dtype) && is_float_dtype(k->dtype) && is_float_dtype(v->dtype) && is_float_dtype(out->dtype),
             "flash_attention needs floating-point tensors");
  p->B = (int)eq[0]; p->Hq = (int)eq[1]; p->Hkv = (int)ek[1]; p->Sq = (int)eq[2]; p->Skv = (int)ek[2]; p->D = (int)eq[3];
  p->dt_q = q->dtype; p->dt_k = k->dtype; p->dt_v = v->dtype; p->dt_o = out->dtype;
  p->scale = scale;
  p->causal = is_causal ? 1 : 0;
  return KD_OK;
}

template <int DPL>
static int launch_attention_f32(const void* pq, const void* pk, const void* pv, void* po, const AttnParams& p) {
  constexpr int D = 32 * DPL;
  const size_t smem = sizeof(float) * (ATT_TKV * (D + 1) + ATT_TKV * D + ATT_WARPS * D);
  if (smem > 48 * 1024)
    KD_CUDA_CHECK(cudaFuncSetAttribute(attention_f32_kernel<DPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((p.Sq + ATT_WARPS - 1) / ATT_WARPS, p.Hq, p.B);
  attention_f32_kernel<DPL><<<grid, ATT_WARPS * 32, smem, ctx().stream>>>(pq, pk, pv, po, p);
  return after_launch("attention_f32_kernel");
}

int attention_f32_dispatch(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v, const kd_tensor* out,
                           const AttnParams& p) {
  void *pq = nullptr, *pk = nullptr, *pv = nullptr, *po = nullptr;
  KD_TRY(tensor_ptr(q, &pq));
  KD_TRY(tensor_ptr(k, &pk));
  KD_TRY(tensor_ptr(v, &pv));
  KD_TRY(tensor_ptr(out, &po));
  if (p.B == 0 || p.Hq == 0 || p.Sq == 0) return KD_OK;
  KD_REQUIRE(p.Skv > 0, "flash_attention: empty key/value sequence");
  KD_REQUIRE(p.Hq <= 65535 && p.B <= 65535, "flash_attention: too many heads or batches for one launch");
  KD_REQUIRE(p.D >= 1, "flash_attention: empty head dimension");
  if (p.D <= 32) return launch_attention_f32<1>(pq, pk, pv, po, p);
  if (p.D <= 64) return launch_attention_f32<2>(pq, pk, pv, po, p);
  if (p.D <= 128) return launch_attention_f32<4>(pq, pk, pv, po, p);
  if (p.D <= 256) return launch_attention_f32<8>(pq, pk, pv, po, p);
  return fail(KD_ERR_UNSUPPORTED, "flash_attention: head_dim %d exceeds 256", p.D);
}

}  // namespace kd
