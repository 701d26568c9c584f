// Entry points that choose between the exact-fp32 CUDA-core kernels and the bf16 tensor-core
// kernels: `matmul`, `flash_attention`, `conv1d`.
#include "common.cuh"
#include "kernels.cuh"

using namespace kd;

KD_API int kd_matmul(const kd_matmul_cfg* cfg, const kd_tensor* a, const kd_tensor* b, const kd_tensor* c,
                     const kd_tensor* out) {
  KD_TRY(require_init());
  KD_REQUIRE(cfg && a && b && out, "null argument");
  KD_REQUIRE(cfg->M >= 0 && cfg->N >= 0 && cfg->K >= 0, "matmul: negative extent");
  KD_REQUIRE(is_float_dtype(a->dtype) && is_float_dtype(b->dtype) && is_float_dtype(out->dtype),
             "matmul needs floating-point tensors");
  int handled = 0;
  KD_TRY(matmul_tc_try(cfg, a, b, c, out, &handled));
  if (handled) return KD_OK;
  return matmul_f32_dispatch(cfg, a, b, c, out);
}

KD_API int kd_flash_attention(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v, const kd_tensor* out,
                              float scale, int is_causal) {
  KD_TRY(require_init());
  AttnParams p{};
  KD_TRY(attention_params(q, k, v, out, scale, is_causal, &p));
  int handled = 0;
  KD_TRY(attention_tc_try(q, k, v, out, p, &handled));
  if (handled) return KD_OK;
  return attention_f32_dispatch(q, k, v, out, p);
}
