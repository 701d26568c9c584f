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
  // bf16 activations whose leading dimensions do not collapse into one row stride (the (L,N,E) view
  // of a batch-first tensor that nn.MultiheadAttention projects,
  // packages/core/src/nn/modules/attention/MultiheadAttention.ts:302-348): one strided copy into a
  // dense temporary costs a few bytes per element, the general fp32-accumulate kernel costs two
  // orders of magnitude more than the tensor-core GEMM that the copy makes possible.
  if (a->dtype == KD_BF16 && b->dtype == KD_BF16 && b->ndim == 2 && a->ndim >= 3 && !cfg->transpose_a && !is_contiguous(a) &&
      numel(a) >= (1 << 16)) {
    kd_tensor dense = *a;
    int64_t st = 1;
    for (int d = a->ndim - 1; d >= 0; --d) { dense.strides[d] = st; st *= a->shape[d]; }
    dense.offset = 0;
    KD_TRY(kd_storage_alloc((uint64_t)numel(a) * 2, 0, &dense.storage));
    int rc = kd_copy(&dense, a);
    if (rc == KD_OK) rc = matmul_tc_try(cfg, &dense, b, c, out, &handled);
    if (rc == KD_OK && !handled) rc = matmul_f32_dispatch(cfg, &dense, b, c, out);
    kd_storage_release(dense.storage);   // stream-ordered: later users of the block queue behind the GEMM
    return rc;
  }
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
    KD_REQUIRE(residual && residual->dtype == out->dtype && is_contiguous(residual) && numel(residual) == M * N,
               "residual must be contiguous, of the output's shape and dtype");
    KD_TRY(tensor_ptr(residual, &pr));
  }
  return gemm_bf16(px, K, pw, weight->strides[0], po, n_out, out->dtype == KD_F32, pr, N, (int)M, (int)N, (int)K, epilogue);
}

KD_API int kd_linear_bf16_bias(const kd_tensor* x, const kd_tensor* weight, const kd_tensor* bias, const kd_tensor* residual,
                               int activation, const kd_tensor* out) {
  KD_TRY(require_init());
  KD_REQUIRE(x && weight && out, "null tensor");
  KD_REQUIRE(activation == KD_ACT_NONE || activation == KD_ACT_GELU, "unknown activation %d", activation);
  KD_REQUIRE(x->dtype == KD_BF16 && weight->dtype == KD_BF16 && out->dtype == KD_BF16, "kd_linear_bf16_bias needs bf16 tensors");
  KD_REQUIRE(x->ndim >= 1 && weight->ndim == 2 && weight->strides[1] == 1, "weight must be [N,K] with unit K stride");
  KD_REQUIRE(is_contiguous(x) && is_contiguous(out), "kd_linear_bf16_bias needs contiguous activations and output");
  const int64_t K = x->shape[x->ndim - 1], N = weight->shape[0];
  KD_REQUIRE(weight->shape[1] == K, "weight has K=%lld, activations have K=%lld", (long long)weight->shape[1], (long long)K);
  const int64_t M = K ? numel(x) / K : 0;
  KD_REQUIRE(numel(out) == M * N, "output has %lld elements, expected %lld", (long long)numel(out), (long long)(M * N));
  if (M == 0) return KD_OK;
  void *px = nullptr, *pw = nullptr, *pb = nullptr, *pr = nullptr, *po = nullptr;
  KD_TRY(tensor_ptr(x, &px));
  KD_TRY(tensor_ptr(weight, &pw));
  KD_TRY(tensor_ptr(out, &po));
  if (bias) {
    KD_REQUIRE(bias->dtype == KD_BF16 && is_contiguous(bias) && numel(bias) == N, "bias must be contiguous bf16 [N]");
    KD_TRY(tensor_ptr(bias, &pb));
  }
  if (residual) {
    KD_REQUIRE(residual->dtype == KD_BF16 && is_contiguous(residual) && numel(residual) == M * N,
               "residual must be contiguous bf16 of the output's shape");
    KD_TRY(tensor_ptr(residual, &pr));
  }
  return gemm_bf16_bias_act(px, K, pw, weight->strides[0], po, N, 0, pr, N, (int)M, (int)N, (int)K, residual ? KD_EPI_RESIDUAL : KD_EPI_NONE,
                            pb, activation);
}

static int decode_common(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v, const kd_tensor* block_table,
                         const kd_tensor* ctx_len, int ctx_len_host, float scale, int splits, const kd_tensor* out) {
  KD_TRY(require_init());
  KD_REQUIRE(q && k && v && out, "null tensor");
  KD_REQUIRE(q->ndim == 4 && k->ndim == 4, "decode attention operands must be 4-D");
  const int* ctx_dev = nullptr;
  if (ctx_len) {
    KD_REQUIRE(ctx_len->dtype == KD_I32 && numel(ctx_len) == 1, "ctx_len must be a device int32 scalar");
    void* pc = nullptr;
    KD_TRY(tensor_ptr(ctx_len, &pc));
    ctx_dev = static_cast<const int*>(pc);
  }
  const int* table = nullptr;
  int max_pages = 0;
  if (block_table) {
    KD_REQUIRE(block_table->dtype == KD_I32 && block_table->ndim == 2 && is_contiguous(block_table) &&
                   block_table->shape[0] == q->shape[0],
               "block_table must be a contiguous int32 [B, max_pages] tensor");
    void* pt = nullptr;
    KD_TRY(tensor_ptr(block_table, &pt));
    table = static_cast<const int*>(pt);
    max_pages = (int)block_table->shape[1];
  }
  const int B = (int)q->shape[0], Hq = (int)q->shape[1], Hkv = (int)k->shape[1], D = (int)q->shape[3];
  KD_REQUIRE(Hkv > 0 && Hq % Hkv == 0, "bad head counts");
  const int max_keys = table ? max_pages * 128 : (int)k->shape[2];
  const int max_blocks = (max_keys + 63) / 64;     // 64-key tiles
  if (splits <= 0) {
    // one wave of CTAs (2 per SM), never more splits than key tiles
    const int pairs = B * Hkv > 0 ? B * Hkv : 1;
    splits = (2 * ctx().sm_count) / pairs;   // two CTAs fit per SM: stay within one wave
    if (splits > max_blocks) splits = max_blocks;
    if (splits < 1) splits = 1;
  }
  const size_t need = attention_decode_scratch_bytes(B, Hkv, Hq / Hkv, splits, D);
  void* scratch = nullptr;
  KD_TRY(get_workspace(need, &scratch));
  return attention_decode(q, k, v, out, scale, ctx_dev, ctx_len_host, table, max_pages, splits, scratch, need);
}

KD_API int kd_attention_decode(const kd_tensor* q, const kd_tensor* k_cache, const kd_tensor* v_cache,
                               const kd_tensor* ctx_len, int ctx_len_host, float scale, int splits,
                               const kd_tensor* out) {
  return decode_common(q, k_cache, v_cache, nullptr, ctx_len, ctx_len_host, scale, splits, out);
}

KD_API int kd_attention_decode_paged(const kd_tensor* q, const kd_tensor* k_pool, const kd_tensor* v_pool,
                                     const kd_tensor* block_table, const kd_tensor* ctx_len, int ctx_len_host,
                                     float scale, int splits, const kd_tensor* out) {
  KD_REQUIRE(block_table != nullptr, "kd_attention_decode_paged needs a block table");
  return decode_common(q, k_pool, v_pool, block_table, ctx_len, ctx_len_host, scale, splits, out);
}

KD_API int kd_attention_decode_noalloc(const kd_tensor* q, const kd_tensor* k_cache, const kd_tensor* v_cache,
                                       const kd_tensor* ctx_len, int ctx_len_host, float scale, int splits,
                                       const kd_tensor* out) {
  KD_TRY(require_init());
  KD_REQUIRE(q && k_cache && v_cache && out, "null tensor");
  const int* ctx_dev = nullptr;
  if (ctx_len) {
    KD_REQUIRE(ctx_len->dtype == KD_I32 && numel(ctx_len) == 1, "ctx_len must be a device int32 scalar");
    void* pc = nullptr;
    KD_TRY(tensor_ptr(ctx_len, &pc));
    ctx_dev = static_cast<const int*>(pc);
  }
  return attention_decode_static(q, k_cache, v_cache, out, scale, ctx_dev, ctx_len_host, splits);
}

KD_API int kd_qkv_linear_norm_rope_cachewrite(const kd_tensor* x, const kd_tensor* wqkv, const kd_tensor* q_norm_weight,
                                              const kd_tensor* k_norm_weight, float eps, const kd_tensor* cos,
                                              const kd_tensor* sin, const kd_tensor* k_cache, const kd_tensor* v_cache,
                                              int start_pos, const kd_tensor* q_out) {
  KD_TRY(require_init());
  KD_REQUIRE(x && wqkv && q_norm_weight && k_norm_weight && cos && sin && k_cache && v_cache && q_out, "null tensor");
  KD_REQUIRE(q_out->ndim == 4 && q_out->dtype == KD_BF16 && is_contiguous(q_out), "q_out must be contiguous bf16 [B,S,Hq,D]");
  const int B = (int)q_out->shape[0], S = (int)q_out->shape[1], Hq = (int)q_out->shape[2], D = (int)q_out->shape[3];
  KD_REQUIRE(D == 128, "the fused QKV projection handles head_dim 128 (use kd_linear_bf16 + kd_qkv_norm_rope_cachewrite otherwise)");
  KD_REQUIRE(k_cache->ndim == 4 && k_cache->dtype == KD_BF16 && v_cache->dtype == KD_BF16 && k_cache->shape[0] == B &&
                 k_cache->shape[3] == D && k_cache->strides[3] == 1,
             "caches must be bf16 [B,Hkv,maxS,128] with unit head_dim stride");
  const int Hkv = (int)k_cache->shape[1];
  for (int i = 0; i < 4; ++i)
    KD_REQUIRE(v_cache->shape[i] == k_cache->shape[i] && v_cache->strides[i] == k_cache->strides[i],
               "v_cache must have k_cache's shape and strides");
  for (int i = 0; i < 3; ++i) KD_REQUIRE(k_cache->strides[i] % 8 == 0, "cache strides must be multiples of 8 elements");
  KD_REQUIRE(start_pos >= 0 && start_pos + S <= k_cache->shape[2],
             "Cache overflow: trying to write to position %d-%d, but maxSeqLen is %lld", start_pos, start_pos + S,
             (long long)k_cache->shape[2]);
  const int64_t tokens = (int64_t)B * S, N = (int64_t)(Hq + 2 * Hkv) * D;
  KD_REQUIRE(x->dtype == KD_BF16 && is_contiguous(x) && x->ndim >= 1 && numel(x) % tokens == 0, "x must be contiguous bf16 [B*S, K]");
  const int64_t K = numel(x) / tokens;
  KD_REQUIRE(wqkv->dtype == KD_BF16 && wqkv->ndim == 2 && wqkv->shape[0] == N && wqkv->shape[1] == K && wqkv->strides[1] == 1,
             "wqkv must be bf16 [(Hq+2Hkv)*128, K]");
  KD_REQUIRE(q_norm_weight->dtype == KD_BF16 && k_norm_weight->dtype == KD_BF16 && numel(q_norm_weight) == D &&
                 numel(k_norm_weight) == D && is_contiguous(q_norm_weight) && is_contiguous(k_norm_weight),
             "q/k norm weights must be contiguous bf16 [128]");
  KD_REQUIRE(cos->dtype == KD_F32 && sin->dtype == KD_F32 && is_contiguous(cos) && is_contiguous(sin) &&
                 numel(cos) == (int64_t)S * 64 && numel(sin) == (int64_t)S * 64,
             "cos/sin must be contiguous fp32 [S, 64]");
  if (tokens == 0) return KD_OK;
  void *px, *pw, *pqw, *pkw, *pc, *ps, *pkc, *pvc, *pq;
  KD_TRY(tensor_ptr(x, &px));
  KD_TRY(tensor_ptr(wqkv, &pw));
  KD_TRY(tensor_ptr(q_norm_weight, &pqw));
  KD_TRY(tensor_ptr(k_norm_weight, &pkw));
  KD_TRY(tensor_ptr(cos, &pc));
  KD_TRY(tensor_ptr(sin, &ps));
  KD_TRY(tensor_ptr(k_cache, &pkc));
  KD_TRY(tensor_ptr(v_cache, &pvc));
  KD_TRY(tensor_ptr(q_out, &pq));
  const uintptr_t all = reinterpret_cast<uintptr_t>(pqw) | reinterpret_cast<uintptr_t>(pkw) | reinterpret_cast<uintptr_t>(pc) |
                        reinterpret_cast<uintptr_t>(ps) | reinterpret_cast<uintptr_t>(pkc) | reinterpret_cast<uintptr_t>(pvc) |
                        reinterpret_cast<uintptr_t>(pq);
  KD_REQUIRE((all & 15) == 0, "operands must be 16-byte aligned");
  return gemm_bf16_qkv_rope(px, K, pw, wqkv->strides[0], (int)tokens, (int)K, S, Hq, Hkv, start_pos, eps, (const float*)pc,
                            (const float*)ps, pqw, pkw, pq, pkc, pvc, k_cache->strides[0], k_cache->strides[1], k_cache->strides[2]);
}
