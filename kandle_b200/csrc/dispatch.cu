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

KD_API int kd_linear_bf16(const kd_tensor* x, const kd_tensor* weight, const kd_tensor* residual, int epilogue,
                          const kd_tensor* out) {
  KD_TRY(require_init());
  KD_REQUIRE(x && weight && out, "null tensor");
  KD_REQUIRE(epilogue >= KD_EPI_NONE && epilogue <= KD_EPI_SWIGLU, "unknown epilogue %d", epilogue);
  KD_REQUIRE(x->dtype == KD_BF16 && weight->dtype == KD_BF16, "kd_linear_bf16 needs bf16 activations and weights");
  KD_REQUIRE(out->dtype == KD_BF16 || out->dtype == KD_F32, "kd_linear_bf16 output must be bf16 or fp32");
  KD_REQUIRE(x->ndim >= 1 && weight->ndim == 2 && weight->strides[1] == 1, "weight must be [N,K] with unit K stride");
  KD_REQUIRE(is_contiguous(x) && is_contiguous(out), "kd_linear_bf16 needs contiguous activations and output");
  const int64_t K = x->shape[x->ndim - 1], N = weight->shape[0];
  KD_REQUIRE(weight->shape[1] == K, "weight has K=%lld, activations have K=%lld", (long long)weight->shape[1], (long long)K);
  const int64_t M = K ? numel(x) / K : 0;
  const int64_t n_out = epilogue == KD_EPI_SWIGLU ? N / 2 : N;
  KD_REQUIRE(numel(out) == M * n_out, "output has %lld elements, expected %lld", (long long)numel(out), (long long)(M * n_out));
  if (M == 0) return KD_OK;
  void *px = nullptr, *pw = nullptr, *pr = nullptr, *po = nullptr;
  KD_TRY(tensor_ptr(x, &px));
  KD_TRY(tensor_ptr(weight, &pw));
  KD_TRY(tensor_ptr(out, &po));
  if (epilogue == KD_EPI_RESIDUAL) {
    KD_REQUIRE(residual && residual->dtype == KD_BF16 && is_contiguous(residual) && numel(residual) == M * N,
               "residual must be a contiguous bf16 tensor of the output's shape");
    KD_TRY(tensor_ptr(residual, &pr));
  }
  return gemm_bf16(px, K, pw, weight->strides[0], po, n_out, out->dtype == KD_F32, pr, N, (int)M, (int)N, (int)K, epilogue);
}
