// CPU oracle for the transformer-forward hot path of final-kk/kandle.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, in plain C++ (fp32 storage,
// fp32 arithmetic, IEEE libm), the arithmetic that the reference performs in
// its WGSL compute shaders and composite dispatch handlers.  It is the checker
// for the CUDA kernels and the timed CPU baseline; nothing in the shipped
// library links, loads or calls it.
//
// PARITY UNPINNED: the reference ships no test files, golden vectors or
// known-answer fixtures for these operators (its browser test console imports
// files that are not in the tree) and cannot be executed here (WebGPU only, no
// JS runtime).  The oracle is therefore pinned only to (a) the shader text it
// restates, cited per function below, and (b) independent float64 evaluations
// in tests/test_oracle.py.
//
// All citations are paths inside the reference project.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

typedef float v8f __attribute__((vector_size(32)));

static inline v8f ld8(const float* p) {
  v8f v;
  __builtin_memcpy(&v, p, 32);
  return v;
}
static inline float hsum8(v8f v) {
  return ((v[0] + v[4]) + (v[1] + v[5])) + ((v[2] + v[6]) + (v[3] + v[7]));
}

ORC_API int orc_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}

// ---------------------------------------------------------------------------
// linear / matmul
// ---------------------------------------------------------------------------
// out[M,N] = alpha * A[M,K] * W[N,K]^T  (+ beta * C[M,N])
// Follows the `linear` composite (packages/core/src/dispatch/handlers/composite.ts:55-77):
// the weight is stored [N,K] row-major and passed with transposeB=true, and the
// tiled shader's epilogue is `alpha*acc + beta*C`
// (packages/backend-webgpu/src/kernels/matrix/builder.ts:290-355, 1019-1057).
// Accumulation is fp32; the K reduction is 8-lane blocked instead of strictly
// serial (the reference reduces serially in 32-wide tiles), which only changes
// rounding order.
ORC_API void orc_gemm_nt(const float* A, int64_t lda, const float* W, int64_t ldw,
                         float* out, int64_t ldo, int64_t M, int64_t N, int64_t K,
                         float alpha, float beta, const float* C, int64_t ldc) {
  const int64_t MB = 4, NB = 4;
  const int64_t mt = (M + MB - 1) / MB, nt = (N + NB - 1) / NB;
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t ti = 0; ti < mt; ++ti) {
    for (int64_t tj = 0; tj < nt; ++tj) {
      const int64_t i0 = ti * MB, j0 = tj * NB;
      const int64_t mi = std::min(MB, M - i0), nj = std::min(NB, N - j0);
      float acc[4][4] = {{0}};
      if (mi == 4 && nj == 4) {
        v8f c[4][4];
        for (int a = 0; a < 4; ++a)
          for (int b = 0; b < 4; ++b) c[a][b] = v8f{0, 0, 0, 0, 0, 0, 0, 0};
        const float* a0 = A + (i0 + 0) * lda;
        const float* a1 = A + (i0 + 1) * lda;
        const float* a2 = A + (i0 + 2) * lda;
        const float* a3 = A + (i0 + 3) * lda;
        const float* b0 = W + (j0 + 0) * ldw;
        const float* b1 = W + (j0 + 1) * ldw;
        const float* b2 = W + (j0 + 2) * ldw;
        const float* b3 = W + (j0 + 3) * ldw;
        int64_t k = 0;
        for (; k + 8 <= K; k += 8) {
          v8f x0 = ld8(a0 + k), x1 = ld8(a1 + k), x2 = ld8(a2 + k), x3 = ld8(a3 + k);
          v8f y0 = ld8(b0 + k), y1 = ld8(b1 + k), y2 = ld8(b2 + k), y3 = ld8(b3 + k);
          c[0][0] += x0 * y0; c[0][1] += x0 * y1; c[0][2] += x0 * y2; c[0][3] += x0 * y3;
          c[1][0] += x1 * y0; c[1][1] += x1 * y1; c[1][2] += x1 * y2; c[1][3] += x1 * y3;
          c[2][0] += x2 * y0; c[2][1] += x2 * y1; c[2][2] += x2 * y2; c[2][3] += x2 * y3;
          c[3][0] += x3 * y0; c[3][1] += x3 * y1; c[3][2] += x3 * y2; c[3][3] += x3 * y3;
        }
        for (int a = 0; a < 4; ++a)
          for (int b = 0; b < 4; ++b) acc[a][b] = hsum8(c[a][b]);
        for (; k < K; ++k) {
          for (int a = 0; a < 4; ++a)
            for (int b = 0; b < 4; ++b)
              acc[a][b] += A[(i0 + a) * lda + k] * W[(j0 + b) * ldw + k];
        }
      } else {
        for (int64_t a = 0; a < mi; ++a)
          for (int64_t b = 0; b < nj; ++b) {
            float s = 0.f;
            for (int64_t k = 0; k < K; ++k) s += A[(i0 + a) * lda + k] * W[(j0 + b) * ldw + k];
            acc[a][b] = s;
          }
      }
      for (int64_t a = 0; a < mi; ++a)
        for (int64_t b = 0; b < nj; ++b) {
          float r = alpha * acc[a][b];
          if (C != nullptr && beta != 0.f) r += beta * C[(i0 + a) * ldc + (j0 + b)];
          out[(i0 + a) * ldo + (j0 + b)] = r;
        }
    }
  }
}

// Fully general batched matmul with 4-D element strides, offsets, transpose
// flags and alpha/beta, as described by MatmulDispatchResult
// (packages/core/src/dispatch/matmulOps.ts:32-125, 701-814).  Logical operand
// A is [b0,b1,M,K] after applying transposeA (then its stored last two dims are
// [K,M]); same for B.  Strides are those of the STORED tensor right-aligned
// into 4 slots.  Output is contiguous [b0,b1,M,N].  K is reduced serially in
// fp32 exactly like the shader's inner loop
// (packages/backend-webgpu/src/kernels/matrix/builder.ts:1019-1057).
ORC_API void orc_matmul4d(const float* A, const int64_t* sa, int transA,
                          const float* B, const int64_t* sb, int transB,
                          const float* C, const int64_t* sc, float* out,
                          int64_t b0, int64_t b1, int64_t M, int64_t N, int64_t K,
                          float alpha, float beta) {
  const int64_t a_m = transA ? sa[3] : sa[2], a_k = transA ? sa[2] : sa[3];
  const int64_t b_k = transB ? sb[3] : sb[2], b_n = transB ? sb[2] : sb[3];
#pragma omp parallel for schedule(static) collapse(3)
  for (int64_t x = 0; x < b0; ++x)
    for (int64_t y = 0; y < b1; ++y)
      for (int64_t i = 0; i < M; ++i) {
        const float* ap = A + x * sa[0] + y * sa[1] + i * a_m;
        const float* bp = B + x * sb[0] + y * sb[1];
        float* op = out + ((x * b1 + y) * M + i) * N;
        for (int64_t j = 0; j < N; ++j) {
          float acc = 0.f;
          for (int64_t k = 0; k < K; ++k) acc += ap[k * a_k] * bp[k * b_k + j * b_n];
          float r = alpha * acc;
          if (C != nullptr && beta != 0.f)
            r += beta * C[x * sc[0] + y * sc[1] + i * sc[2] + j * sc[3]];
          op[j] = r;
        }
      }
}

// ---------------------------------------------------------------------------
// scaled_dot_product_attention (fused "flash_attention" kernel)
// ---------------------------------------------------------------------------
// Tile selection restated from
// packages/backend-webgpu/src/kernels/attention/types.ts:69-122
// (largest (Bq,Bkv) in {32,16,8,4}^2, Bq-major order, fitting 16 KB of fp32).
ORC_API void orc_sdpa_tile_config(int D, int Sq, int Skv, int* bq_out, int* bkv_out) {
  auto storage = [&](int br, int bc) { return (br * D + bc * D + bc * D + br * bc + br * D + br + br) * 4; };
  const int cands[4] = {32, 16, 8, 4};
  int bq = 32, bkv = 32;
  for (int i = 0; i < 4; ++i) {
    bool found = false;
    for (int j = 0; j < 4; ++j)
      if (storage(cands[i], cands[j]) <= 16384) { bq = cands[i]; bkv = cands[j]; found = true; break; }
    if (found) break;
  }
  bq = std::min(bq, Sq);
  bkv = std::min(bkv, Skv);
  if (storage(bq, bkv) > 16384) { bq = 4; bkv = 4; }
  *bq_out = bq; *bkv_out = bkv;
}

// Q [B,Hq,Sq,D], K/V [B,Hkv,Skv,D], O [B,Hq,Sq,D], contiguous row-major.
// Restates packages/backend-webgpu/src/kernels/attention/builder.ts:138-329:
//   head_kv = head_q / (Hq/Hkv)                               (:143)
//   score = dot(q,k) * scale, scale applied after the dot     (:253-256)
//   causal: k_col > q_row -> -1e20 (top-left aligned)         (:248-249)
//   out-of-range column -> -1e20                              (:258-260)
//   causal block skip when kv_start > last row of the Q block (:205-210)
//   online softmax per KV block: m_new, l_new, O rescale      (:270-311)
//   O / l                                                     (:319-329)
// m starts at -1e20 and l at 0 (:181-184).  block_kv <= 0 selects the tile
// size the reference would choose.
ORC_API void orc_sdpa(const float* Q, const float* K, const float* V, float* O,
                      int B, int Hq, int Hkv, int Sq, int Skv, int D, float scale,
                      int causal, int block_kv) {
  int bq = 0, bkv = 0;
  orc_sdpa_tile_config(D, Sq, Skv, &bq, &bkv);
  if (block_kv > 0) bkv = block_kv;
  const int ratio = Hq / Hkv;
  const float NEG = -1e20f;
#pragma omp parallel for schedule(dynamic, 4) collapse(3)
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < Hq; ++h)
      for (int i = 0; i < Sq; ++i) {
        const int hk = h / ratio;
        const float* q = Q + (((int64_t)b * Hq + h) * Sq + i) * D;
        const float* kb = K + ((int64_t)b * Hkv + hk) * (int64_t)Skv * D;
        const float* vb = V + ((int64_t)b * Hkv + hk) * (int64_t)Skv * D;
        float* o = O + (((int64_t)b * Hq + h) * Sq + i) * D;
        std::vector<float> acc(D, 0.f), s(bkv);
        float m = NEG, l = 0.f;
        const int q_block_last = (i / bq) * bq + bq - 1;
        for (int j0 = 0; j0 < Skv; j0 += bkv) {
          if (causal && j0 > q_block_last) continue;
          for (int jj = 0; jj < bkv; ++jj) {
            const int j = j0 + jj;
            float sc;
            if (j >= Skv) sc = NEG;
            else if (causal && j > i) sc = NEG;
            else {
              sc = 0.f;
              const float* kr = kb + (int64_t)j * D;
              for (int d = 0; d < D; ++d) sc += q[d] * kr[d];
              sc *= scale;
            }
            s[jj] = sc;
          }
          float m_new = m;
          for (int jj = 0; jj < bkv; ++jj) m_new = std::max(m_new, s[jj]);
          const float sf = std::exp(m - m_new);
          float l_new = l * sf;
          // p = exp(s - m_new) is evaluated once per column here; the shader
          // re-evaluates the same expression per output element.
          for (int jj = 0; jj < bkv; ++jj) { s[jj] = std::exp(s[jj] - m_new); l_new += s[jj]; }
          for (int d = 0; d < D; ++d) {
            float ov = acc[d] * sf;
            for (int jj = 0; jj < bkv; ++jj) {
              const int j = j0 + jj;
              const float vv = (j < Skv) ? vb[(int64_t)j * D + d] : 0.f;
              ov += s[jj] * vv;
            }
            acc[d] = ov;
          }
          m = m_new; l = l_new;
        }
        for (int d = 0; d < D; ++d) o[d] = acc[d] / l;
      }
}

// ---------------------------------------------------------------------------
// normalisation
// ---------------------------------------------------------------------------
// packages/backend-webgpu/src/kernels/normalize/shaderBuilder.ts:343-415:
// sum_sq serial in fp32, rms = sqrt(sum_sq/N + eps), y = (x * (1/rms)) * w.
ORC_API void orc_rms_norm(const float* x, const float* w, float* y, int64_t rows,
                          int64_t n, float eps) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * n;
    float* yr = y + r * n;
    float ss = 0.f;
    for (int64_t i = 0; i < n; ++i) ss += xr[i] * xr[i];
    const float rms = std::sqrt(ss / (float)n + eps);
    const float sc = 1.0f / rms;
    for (int64_t i = 0; i < n; ++i) {
      float v = xr[i] * sc;
      if (w) v = v * w[i];
      yr[i] = v;
    }
  }
}

// packages/backend-webgpu/src/kernels/normalize/shaderBuilder.ts:236-325:
// Welford mean/M2, biased variance, rstd = 1/sqrt(var+eps),
// y = (x-mean)*rstd [* w] [+ b].
ORC_API void orc_layer_norm(const float* x, const float* w, const float* b, float* y,
                            int64_t rows, int64_t n, float eps) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * n;
    float* yr = y + r * n;
    float mean = 0.f, m2 = 0.f, count = 0.f;
    for (int64_t i = 0; i < n; ++i) {
      const float v = xr[i];
      count += 1.f;
      const float d = v - mean;
      mean += d / count;
      const float d2 = v - mean;
      m2 += d * d2;
    }
    const float var = m2 / (float)n;
    const float rstd = 1.0f / std::sqrt(var + eps);
    for (int64_t i = 0; i < n; ++i) {
      float v = (xr[i] - mean) * rstd;
      if (w) v = v * w[i];
      if (b) v = v + b[i];
      yr[i] = v;
    }
  }
}

// packages/backend-webgpu/src/kernels/normalize/shaderBuilder.ts:143-217:
// max starts at -1e38; exp(x-max)/sum.
ORC_API void orc_softmax(const float* x, float* y, int64_t rows, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * n;
    float* yr = y + r * n;
    float mx = -1e38f;
    for (int64_t i = 0; i < n; ++i) mx = std::max(mx, xr[i]);
    float s = 0.f;
    for (int64_t i = 0; i < n; ++i) s += std::exp(xr[i] - mx);
    for (int64_t i = 0; i < n; ++i) yr[i] = std::exp(xr[i] - mx) / s;
  }
}

// ---------------------------------------------------------------------------
// pointwise  (packages/backend-webgpu/src/kernels/pointwise/ops.ts)
// ---------------------------------------------------------------------------
enum { ORC_NEG = 0, ORC_COS = 1, ORC_SIN = 2, ORC_SILU = 3, ORC_GELU = 4, ORC_ABS = 5, ORC_TANH = 6, ORC_SIGMOID = 7 };

static inline float clampf(float v, float lo, float hi) { return std::min(std::max(v, lo), hi); }

// silu  : x / (1 + exp(-clamp(x,-88,88)))                              (ops.ts:299)
// gelu  : 0.5 x (1 + tanh(clamp(0.7978845608 (x + 0.044715 x^3), +-20))) always
//         the tanh form, whatever `approximate` says                   (ops.ts:301)
// tanh  : tanh(clamp(x,-20,20))                                        (ops.ts:211)
// sigmoid: 1/(1+exp(-clamp(x,-88,88)))                                 (ops.ts:297)
ORC_API void orc_unary(int op, const float* x, float* y, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float v = x[i];
    float r;
    switch (op) {
      case ORC_NEG: r = -v; break;
      case ORC_COS: r = std::cos(v); break;
      case ORC_SIN: r = std::sin(v); break;
      case ORC_SILU: r = v / (1.0f + std::exp(-clampf(v, -88.f, 88.f))); break;
      case ORC_GELU: {
        const float inner = 0.7978845608f * (v + 0.044715f * v * v * v);
        r = 0.5f * v * (1.0f + std::tanh(clampf(inner, -20.f, 20.f)));
        break;
      }
      case ORC_ABS: r = std::fabs(v); break;
      case ORC_TANH: r = std::tanh(clampf(v, -20.f, 20.f)); break;
      case ORC_SIGMOID: r = 1.0f / (1.0f + std::exp(-clampf(v, -88.f, 88.f))); break;
      default: r = v;
    }
    y[i] = r;
  }
}

// ---------------------------------------------------------------------------
// gather / argmax
// ---------------------------------------------------------------------------
// embedding -> index_select(dim 0): out[i,:] = W[ids[i],:]
// (packages/core/src/dispatch/handlers/composite.ts:149-245,
//  packages/backend-webgpu/src/kernels/gather/shaderBuilder.ts:107-137)
ORC_API void orc_index_select_rows(const float* W, const int32_t* ids, float* out,
                                   int64_t n_ids, int64_t width) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n_ids; ++i)
    std::memcpy(out + i * width, W + (int64_t)ids[i] * width, sizeof(float) * width);
}

// Row argmax with strict '>' (packages/backend-webgpu/src/kernels/reduction/
// argShaderBuilder.ts:29-35).  The reference's tree reduction does not define
// which of several equal maxima wins; this oracle and the CUDA kernel both
// return the LOWEST index among equal maxima.
ORC_API void orc_argmax_rows(const float* x, int32_t* out, int64_t rows, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * n;
    float best = -3.402823466e38f;
    int32_t bi = 0;
    for (int64_t i = 0; i < n; ++i)
      if (xr[i] > best) { best = xr[i]; bi = (int32_t)i; }
    out[r] = bi;
  }
}

// ---------------------------------------------------------------------------
// conv1d through im2col + GEMM
// ---------------------------------------------------------------------------
// packages/backend-webgpu/src/kernels/window/algorithms/im2col.ts:124-268,514-607:
// col[b*Wout + t, c*k + j] = x[b, c, t*stride - pad + j] (0 outside), then
// GEMM with the flattened weight [Cout, Cin*k]^T, then + bias, then the
// [B*Wout, Cout] -> [B, Cout, Wout] transpose.
ORC_API void orc_conv1d(const float* x, const float* w, const float* bias, float* y,
                        int B, int Cin, int L, int Cout, int ksz, int stride, int pad) {
  const int Wout = (L + 2 * pad - ksz) / stride + 1;
  const int64_t Kc = (int64_t)Cin * ksz;
  std::vector<float> col((size_t)B * Wout * Kc);
#pragma omp parallel for schedule(static) collapse(2)
  for (int b = 0; b < B; ++b)
    for (int t = 0; t < Wout; ++t) {
      float* cr = col.data() + ((int64_t)b * Wout + t) * Kc;
      for (int c = 0; c < Cin; ++c)
        for (int j = 0; j < ksz; ++j) {
          const int p = t * stride - pad + j;
          cr[c * ksz + j] = (p >= 0 && p < L) ? x[((int64_t)b * Cin + c) * L + p] : 0.f;
        }
    }
  std::vector<float> tmp((size_t)B * Wout * Cout);
  orc_gemm_nt(col.data(), Kc, w, Kc, tmp.data(), Cout, (int64_t)B * Wout, Cout, Kc, 1.f, 0.f, nullptr, 0);
#pragma omp parallel for schedule(static) collapse(2)
  for (int b = 0; b < B; ++b)
    for (int co = 0; co < Cout; ++co)
      for (int t = 0; t < Wout; ++t) {
        float v = tmp[((int64_t)b * Wout + t) * Cout + co];
        if (bias) v += bias[co];
        y[((int64_t)b * Cout + co) * Wout + t] = v;
      }
}
