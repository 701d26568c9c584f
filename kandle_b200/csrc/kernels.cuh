// Internal entry points shared between translation units.
#pragma once
#include "common.cuh"

namespace kd {

struct AttnParams {
  int B, Hq, Hkv, Sq, Skv, D;
  int64_t sq[4], sk[4], sv[4], so[4];
  int dt_q, dt_k, dt_v, dt_o;
  float scale;
  int causal;
};

int matmul_f32_dispatch(const kd_matmul_cfg* cfg, const kd_tensor* a, const kd_tensor* b, const kd_tensor* c,
                        const kd_tensor* out);
// Tensor-core GEMM; sets *handled = 1 when it took the call (bf16 operands in a supported layout).
int matmul_tc_try(const kd_matmul_cfg* cfg, const kd_tensor* a, const kd_tensor* b, const kd_tensor* c,
                  const kd_tensor* out, int* handled);

int attention_params(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v, const kd_tensor* out, float scale,
                     int is_causal, AttnParams* p);
int attention_f32_dispatch(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v, const kd_tensor* out,
                           const AttnParams& p);
// out[M, N or N/2] = epilogue(A[M,K] * W[N,K]^T) on tcgen05; device pointers, ld* in elements.
int gemm_bf16(const void* A, int64_t lda, const void* W, int64_t ldw, void* out, int64_t ldo, int out_f32,
              const void* resid, int64_t ldr, int M, int N, int K, int epi);
int gemm_bf16_bias_act(const void* A, int64_t lda, const void* W, int64_t ldw, void* out, int64_t ldo, int out_f32,
              const void* resid, int64_t ldr, int M, int N, int K, int epi, const void* bias, int act);
// Tensor-core attention; sets *handled = 1 when it took the call.
int attention_tc_try(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v, const kd_tensor* out,
                     const AttnParams& p, int* handled);

int gemm_bf16_qkv_rope(const void* A, int64_t lda, const void* W, int64_t ldw, int M, int K, int S, int Hq, int Hkv, int pos0,
                       float eps, const float* cos_t, const float* sin_t, const void* qw, const void* kw, void* q_out,
                       void* k_cache, void* v_cache, int64_t kc_b, int64_t kc_h, int64_t kc_s);
int gemm_skinny_auto_splits(int N, int K);
// x [Mb<=128,K] * W[N,K]^T -> fp32 partials [splits][Mb][N], or bf16 [Mb][N] when out_bf16 != NULL (splits == 1).
int gemm_bf16_skinny(const void* x, int64_t ldx, const void* W, int64_t ldw, int Mb, int N, int K, int splits,
                     float* out_f32, void* out_bf16, int swiglu);
size_t attention_decode_scratch_bytes(int B, int Hkv, int group, int splits, int D);
int attention_decode(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v, const kd_tensor* out, float scale,
                     const int* ctx_dev, int ctx_host, const int* block_table, int max_pages, int splits,
                     void* scratch, size_t scratch_bytes);

int attention_decode_static(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v, const kd_tensor* out, float scale,
                            const int* ctx_dev, int ctx_host, int splits);

int attention_decode_static_fill(int byte_value);

}  // namespace kd
