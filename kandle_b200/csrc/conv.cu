// Key `conv1d`: im2col + GEMM + bias + [B*Wout,Cout] -> [B,Cout,Wout] transpose, the same
// decomposition as the reference (packages/backend-webgpu/src/kernels/window/algorithms/
// im2col.ts:124-268,514-607), with the GEMM routed through kd_matmul (tensor cores for bf16).
#include "common.cuh"
#include "kernels.cuh"

namespace kd {

__global__ void im2col1d_kernel(const void* __restrict__ x, int dt_x, int64_t sxb, int64_t sxc, int64_t sxl,
                                void* __restrict__ col, int dt_c, int B, int Cin, int L, int Wout, int ksz, int stride,
                                int pad) {
  const int64_t Kc = (int64_t)Cin * ksz;
  const int64_t total = (int64_t)B * Wout * Kc;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int64_t row = i / Kc;
    const int kc = (int)(i - row * Kc);
    const int c = kc / ksz, j = kc - c * ksz;
    const int b = (int)(row / Wout), t = (int)(row - (int64_t)b * Wout);
    const int pos = t * stride - pad + j;
    const float v = (pos >= 0 && pos < L) ? load_float(x, dt_x, b * sxb + c * sxc + pos * sxl) : 0.f;
    store_float(col, dt_c, i, v);
  }
}

// tmp [B*Wout, Cout] -> out [B, Cout, Wout] with bias; 32x32 smem transpose tiles.
__global__ void bias_transpose_kernel(const void* __restrict__ tmp, int dt_t, const void* __restrict__ bias, int dt_b,
                                      void* __restrict__ out, int dt_o, int Wout, int Cout) {
  __shared__ float tile[32][33];
  const int b = blockIdx.z;
  const int t0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int t = t0 + i, c = c0 + threadIdx.x;
    tile[i][threadIdx.x] = (t < Wout && c < Cout) ? load_float(tmp, dt_t, ((int64_t)b * Wout + t) * Cout + c) : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, t = t0 + threadIdx.x;
    if (t < Wout && c < Cout) {
      float v = tile[threadIdx.x][i];
      if (bias) v += load_float(bias, dt_b, c);
      store_float(out, dt_o, ((int64_t)b * Cout + c) * Wout + t, v);
    }
  }
}

// Token-major im2col: x [B, L, C] bf16 (C % 8 == 0) -> col [B*Wout, ksz*C], row (b,t) = the ksz input
// rows t*stride - pad .. + ksz - 1 side by side (zeros outside the sequence).  16-byte copies,
// coalesced on both sides.
__global__ void im2col_tokens_bf16_kernel(const uint4* __restrict__ x, uint4* __restrict__ col, int B, int L, int cvec, int Wout,
                                          int ksz, int stride, int pad) {
  const int64_t rowvec = (int64_t)ksz * cvec;
  const int64_t total = (int64_t)B * Wout * rowvec;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int64_t row = i / rowvec;
    const int rem = (int)(i - row * rowvec);
    const int j = rem / cvec, cv = rem - j * cvec;
    const int b = (int)(row / Wout), t = (int)(row - (int64_t)b * Wout);
    const int pos = t * stride - pad + j;
    col[i] = (pos >= 0 && pos < L) ? x[((int64_t)b * L + pos) * cvec + cv] : make_uint4(0u, 0u, 0u, 0u);
  }
}

}  // namespace kd

using namespace kd;

KD_API int kd_conv1d_tokens_bf16(const kd_tensor* input, const kd_tensor* weight_kc, const kd_tensor* bias,
                                 const kd_tensor* residual, int activation, int ksz, int stride, int padding,
                                 const kd_tensor* out) {
  KD_TRY(require_init());
  KD_REQUIRE(input && weight_kc && out, "null tensor");
  KD_REQUIRE(input->ndim == 3 && weight_kc->ndim == 2 && out->ndim == 3, "conv1d_tokens: input/output must be 3-D, the weight 2-D");
  KD_REQUIRE(input->dtype == KD_BF16 && weight_kc->dtype == KD_BF16 && out->dtype == KD_BF16, "conv1d_tokens needs bf16 tensors");
  KD_REQUIRE(is_contiguous(input) && is_contiguous(weight_kc) && is_contiguous(out), "conv1d_tokens needs contiguous tensors");
  KD_REQUIRE(ksz >= 1 && stride >= 1 && padding >= 0, "conv1d_tokens: bad kernel size/stride/padding");
  KD_REQUIRE(activation == KD_ACT_NONE || activation == KD_ACT_GELU, "unknown activation %d", activation);
  const int B = (int)input->shape[0], L = (int)input->shape[1], C = (int)input->shape[2];
  const int Cout = (int)weight_kc->shape[0];
  KD_REQUIRE(C % 8 == 0 && Cout % 8 == 0, "conv1d_tokens: channel counts must be multiples of 8");
  KD_REQUIRE(weight_kc->shape[1] == (int64_t)ksz * C, "conv1d_tokens: weight must be [Cout, ksz*Cin] with the tap index major");
  const int Wout = (L + 2 * padding - ksz) / stride + 1;
  KD_REQUIRE(Wout > 0, "conv1d_tokens: empty output");
  KD_REQUIRE(out->shape[0] == B && out->shape[1] == Wout && out->shape[2] == Cout, "conv1d_tokens: output must be [%d,%d,%d]", B, Wout,
             Cout);
  void *px = nullptr, *pw = nullptr, *pb = nullptr, *pr = nullptr, *po = nullptr, *pcol = nullptr;
  KD_TRY(tensor_ptr(input, &px));
  KD_TRY(tensor_ptr(weight_kc, &pw));
  KD_TRY(tensor_ptr(out, &po));
  if (bias) {
    KD_REQUIRE(bias->dtype == KD_BF16 && numel(bias) == Cout && is_contiguous(bias), "conv1d_tokens: bias must be contiguous bf16 [%d]", Cout);
    KD_TRY(tensor_ptr(bias, &pb));
  }
  const int64_t rows = (int64_t)B * Wout, Kc = (int64_t)ksz * C;
  if (residual) {
    KD_REQUIRE(residual->dtype == KD_BF16 && is_contiguous(residual) && numel(residual) == rows * Cout,
               "conv1d_tokens: residual must be contiguous bf16 of the output's shape");
    KD_TRY(tensor_ptr(residual, &pr));
  }
  KD_REQUIRE((reinterpret_cast<uintptr_t>(px) & 15) == 0, "conv1d_tokens: input must be 16-byte aligned");
  uint64_t col_s = 0;
  KD_TRY(kd_storage_alloc((uint64_t)rows * Kc * 2, 0, &col_s));
  kd_tensor col{};
  col.storage = col_s; col.dtype = KD_BF16; col.ndim = 2; col.shape[0] = rows; col.shape[1] = Kc; col.strides[0] = Kc; col.strides[1] = 1;
  int st = tensor_ptr(&col, &pcol);
  if (st == KD_OK) {
    const int64_t total = rows * (Kc / 8);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)ctx().sm_count * 32;
    if (blocks > cap) blocks = cap;
    im2col_tokens_bf16_kernel<<<(int)blocks, 256, 0, ctx().stream>>>(static_cast<const uint4*>(px), static_cast<uint4*>(pcol), B, L, C / 8,
                                                                    Wout, ksz, stride, padding);
    st = after_launch("im2col_tokens_bf16_kernel");
  }
  if (st == KD_OK)
    st = gemm_bf16_bias_act(pcol, Kc, pw, Kc, po, Cout, 0, pr, Cout, (int)rows, Cout, (int)Kc, residual ? KD_EPI_RESIDUAL : KD_EPI_NONE, pb,
                            activation);
  kd_storage_release(col_s);
  return st;
}

KD_API int kd_conv1d(const kd_tensor* input, const kd_tensor* weight, const kd_tensor* bias, int stride, int padding,
                     const kd_tensor* out) {
  KD_TRY(require_init());
  KD_REQUIRE(input && weight && out, "null tensor");
  KD_REQUIRE(input->ndim == 3 && weight->ndim == 3 && out->ndim == 3, "conv1d: input, weight and output must be 3-D");
  KD_REQUIRE(stride >= 1 && padding >= 0, "conv1d: bad stride/padding");
  const int B = (int)input->shape[0], Cin = (int)input->shape[1], L = (int)input->shape[2];
  const int Cout = (int)weight->shape[0], ksz = (int)weight->shape[2];
  KD_REQUIRE(weight->shape[1] == Cin, "conv1d: weight has %lld input channels, input has %d", (long long)weight->shape[1], Cin);
  KD_REQUIRE(is_contiguous(weight), "conv1d: weight must be contiguous");
  const int Wout = (L + 2 * padding - ksz) / stride + 1;
  KD_REQUIRE(Wout > 0, "conv1d: empty output");
  KD_REQUIRE(out->shape[0] == B && out->shape[1] == Cout && out->shape[2] == Wout && is_contiguous(out),
             "conv1d: output must be contiguous [%d,%d,%d]", B, Cout, Wout);
  if (bias) KD_REQUIRE(numel(bias) == Cout && is_contiguous(bias), "conv1d: bias must be contiguous [%d]", Cout);
  void *px = nullptr, *pb = nullptr, *po = nullptr;
  KD_TRY(tensor_ptr(input, &px));
  if (bias) KD_TRY(tensor_ptr(bias, &pb));
  KD_TRY(tensor_ptr(out, &po));
  const int64_t rows = (int64_t)B * Wout, Kc = (int64_t)Cin * ksz;
  const int cdt = weight->dtype;  // column matrix in the weight's dtype so bf16 takes the tensor-core GEMM
  uint64_t col_s = 0, tmp_s = 0;
  KD_TRY(kd_storage_alloc((uint64_t)rows * Kc * dtype_size(cdt), 0, &col_s));
  int st = kd_storage_alloc((uint64_t)rows * Cout * dtype_size(out->dtype), 0, &tmp_s);
  if (st != KD_OK) { kd_storage_release(col_s); return st; }
  kd_tensor col{}, tmp{}, w2{};
  col.storage = col_s; col.dtype = cdt; col.ndim = 2; col.shape[0] = rows; col.shape[1] = Kc; col.strides[0] = Kc; col.strides[1] = 1;
  tmp.storage = tmp_s; tmp.dtype = out->dtype; tmp.ndim = 2; tmp.shape[0] = rows; tmp.shape[1] = Cout; tmp.strides[0] = Cout; tmp.strides[1] = 1;
  w2 = *weight; w2.ndim = 2; w2.shape[0] = Cout; w2.shape[1] = Kc; w2.strides[0] = Kc; w2.strides[1] = 1;
  void *pcol = nullptr, *ptmp = nullptr;
  st = tensor_ptr(&col, &pcol);
  if (st == KD_OK) st = tensor_ptr(&tmp, &ptmp);
  if (st == KD_OK) {
    const int64_t total = rows * Kc;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)ctx().sm_count * 16;
    if (blocks > cap) blocks = cap;
    im2col1d_kernel<<<(int)blocks, 256, 0, ctx().stream>>>(px, input->dtype, input->strides[0], input->strides[1],
                                                          input->strides[2], pcol, cdt, B, Cin, L, Wout, ksz, stride, padding);
    st = after_launch("im2col1d_kernel");
  }
  if (st == KD_OK) {
    kd_matmul_cfg cfg{};
    cfg.M = rows; cfg.N = Cout; cfg.K = Kc; cfg.transpose_a = 0; cfg.transpose_b = 1; cfg.alpha = 1.f; cfg.beta = 0.f;
    st = kd_matmul(&cfg, &col, &w2, nullptr, &tmp);
  }
  if (st == KD_OK) {
    dim3 grid((Wout + 31) / 32, (Cout + 31) / 32, B);
    bias_transpose_kernel<<<grid, dim3(32, 8), 0, ctx().stream>>>(ptmp, tmp.dtype, pb, bias ? bias->dtype : KD_F32, po,
                                                                  out->dtype, Wout, Cout);
    st = after_launch("bias_transpose_kernel");
  }
  kd_storage_release(col_s);
  kd_storage_release(tmp_s);
  return st;
}
