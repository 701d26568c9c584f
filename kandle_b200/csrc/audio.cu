// Whisper log-mel front end on the device: the step right before the audio encoder.
//
// The reference computes it as pad -> as_strided framing -> mul(window) -> rfft (Bluestein for the
// 400-point transform) -> abs -> square -> transpose -> matmul with the mel filterbank -> transpose,
// then downloads the result and runs log10 / clamp / scale in a JavaScript loop
// (packages/core/src/dispatch/handlers/composite.ts:527-681, audio/functional/spectrogram.ts:28-76,
// audio/transforms/MelScale.ts:95-108, playground-node/src/whisper/audio.ts:362-405).  Here:
//
//   kd_stft_frames          frames[b,t,n] = x[b, t*hop + n - pad] * w[n]  (zero outside the signal:
//                           the reference's centre padding is constant-mode whatever pad_mode says)
//   kd_matmul (fp32)        frames [T, n_fft] x basis [n_fft, 2F]  -> real parts | imaginary parts;
//                           a 400-point DFT as a small dense GEMM (0.5 GFLOP for 30 s of audio)
//                           instead of a chirp-z pipeline
//   kd_power_spectrum       |X|^2 the reference's way: fl32(sqrt(re^2+im^2)) squared
//   kd_matmul (fp32)        power [T, F] x filterbank [F, M]
//   kd_whisper_log_mel_norm transpose to [M, T'], log10(max(x, 1e-10)), max over the item,
//                           clamp to max - 8, (x + 4) / 4, dropping the frames beyond T'
// All fp32: this runs once per 30 s of audio and is bound by launch latency, not arithmetic.
#include "common.cuh"
#include "kernels.cuh"

namespace kd {

__global__ void stft_frames_kernel(const float* __restrict__ x, int64_t x_stride, int64_t L, const float* __restrict__ w,
                                   int n_fft, int hop, int pad, int64_t T, float* __restrict__ out, int64_t total) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int n = (int)(idx % n_fft);
  const int64_t bt = idx / n_fft;
  const int64_t t = bt % T, b = bt / T;
  const int64_t src = t * hop + n - pad;
  const float v = (src >= 0 && src < L) ? x[b * x_stride + src] : 0.f;
  out[idx] = v * w[n];
}

__global__ void power_spectrum_kernel(const float* __restrict__ spec, int F, float* __restrict__ out, int64_t total) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t row = idx / F;
  const int k = (int)(idx - row * F);
  const float re = spec[row * 2 * F + k], im = spec[row * 2 * F + F + k];
  const float mag = sqrtf(__fadd_rn(__fmul_rn(re, re), __fmul_rn(im, im)));   // abs of the complex value, then squared
  out[idx] = __fmul_rn(mag, mag);
}

// Monotone map float -> unsigned so that atomicMax orders floats (negative values included).
__device__ __forceinline__ unsigned int float_order(float f) {
  const unsigned int b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float float_unorder(unsigned int u) {
  return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

__device__ __forceinline__ float whisper_log10(float x) {
  // Math.log10 on the float value in double, stored into a Float32Array
  return (float)log10((double)fmaxf(x, 1e-10f));
}

// mel [B, T, M]; item maximum of log10(max(x,1e-10)) over the first `keep` frames
__global__ void log_mel_max_kernel(const float* __restrict__ mel, int64_t T, int M, int64_t keep, unsigned int* __restrict__ mx) {
  const int b = blockIdx.y;
  const int64_t total = keep * M;
  float m = -INFINITY;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    m = fmaxf(m, whisper_log10(mel[(int64_t)b * T * M + i]));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0 && m > -INFINITY) atomicMax(&mx[b], float_order(m));
}

// out [B, M, keep]
__global__ void log_mel_finish_kernel(const float* __restrict__ mel, int64_t T, int M, int64_t keep,
                                      const unsigned int* __restrict__ mx, float* __restrict__ out) {
  __shared__ float tile[32][33];
  const int b = blockIdx.z;
  const int64_t t0 = (int64_t)blockIdx.x * 32;
  const int m0 = blockIdx.y * 32;
  const float threshold = float_unorder(mx[b]) - 8.0f;   // Float32Array max, JS double subtraction: exact here
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int64_t t = t0 + r;
    const int m = m0 + threadIdx.x;
    float v = 0.f;
    if (t < keep && m < M) {
      v = whisper_log10(mel[((int64_t)b * T + t) * M + m]);
      if ((double)v < (double)threshold) v = threshold;
      v = (float)(((double)v + 4.0) / 4.0);
    }
    tile[r][threadIdx.x] = v;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int m = m0 + r;
    const int64_t t = t0 + threadIdx.x;
    if (t < keep && m < M) out[((int64_t)b * M + m) * keep + t] = tile[threadIdx.x][r];
  }
}

}  // namespace kd

using namespace kd;

KD_API int kd_stft_frames(const kd_tensor* waveform, const kd_tensor* window, int n_fft, int hop_length, int center,
                          const kd_tensor* frames_out) {
  KD_TRY(require_init());
  KD_REQUIRE(waveform && window && frames_out, "null tensor");
  KD_REQUIRE(waveform->dtype == KD_F32 && window->dtype == KD_F32 && frames_out->dtype == KD_F32, "stft_frames works in fp32");
  KD_REQUIRE(waveform->ndim == 2 && waveform->strides[1] == 1, "waveform must be [B, L] with unit stride along L");
  KD_REQUIRE(n_fft > 0 && hop_length > 0, "n_fft and hop_length must be positive");
  KD_REQUIRE(window->ndim == 1 && window->shape[0] == n_fft && is_contiguous(window), "window must be contiguous [n_fft]");
  const int64_t B = waveform->shape[0], L = waveform->shape[1];
  const int pad = center ? n_fft / 2 : 0;
  const int64_t padded = L + 2 * pad;
  KD_REQUIRE(padded >= n_fft, "signal shorter than one frame");
  const int64_t T = 1 + (padded - n_fft) / hop_length;
  KD_REQUIRE(frames_out->ndim == 3 && frames_out->shape[0] == B && frames_out->shape[1] == T && frames_out->shape[2] == n_fft &&
                 is_contiguous(frames_out),
             "frames_out must be contiguous [B, %lld, %d]", (long long)T, n_fft);
  void *px, *pw, *po;
  KD_TRY(tensor_ptr(waveform, &px));
  KD_TRY(tensor_ptr(window, &pw));
  KD_TRY(tensor_ptr(frames_out, &po));
  const int64_t total = B * T * n_fft;
  if (total == 0) return KD_OK;
  stft_frames_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx().stream>>>(
      (const float*)px, waveform->strides[0], L, (const float*)pw, n_fft, hop_length, pad, T, (float*)po, total);
  return after_launch("stft_frames_kernel");
}

KD_API int kd_power_spectrum(const kd_tensor* spec_re_im, const kd_tensor* power_out) {
  KD_TRY(require_init());
  KD_REQUIRE(spec_re_im && power_out, "null tensor");
  KD_REQUIRE(spec_re_im->dtype == KD_F32 && power_out->dtype == KD_F32 && is_contiguous(spec_re_im) && is_contiguous(power_out),
             "power_spectrum needs contiguous fp32 tensors");
  KD_REQUIRE(spec_re_im->ndim >= 1 && power_out->ndim == spec_re_im->ndim, "rank mismatch");
  const int64_t F2 = spec_re_im->shape[spec_re_im->ndim - 1], F = power_out->shape[power_out->ndim - 1];
  KD_REQUIRE(F2 == 2 * F && F > 0 && numel(spec_re_im) == 2 * numel(power_out), "spec must be [..., 2F] (real parts, then imaginary parts), out [..., F]");
  void *ps, *po;
  KD_TRY(tensor_ptr(spec_re_im, &ps));
  KD_TRY(tensor_ptr(power_out, &po));
  const int64_t total = numel(power_out);
  power_spectrum_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx().stream>>>((const float*)ps, (int)F, (float*)po, total);
  return after_launch("power_spectrum_kernel");
}

KD_API int kd_whisper_log_mel_norm(const kd_tensor* mel, const kd_tensor* out) {
  KD_TRY(require_init());
  KD_REQUIRE(mel && out, "null tensor");
  KD_REQUIRE(mel->dtype == KD_F32 && out->dtype == KD_F32 && is_contiguous(mel) && is_contiguous(out) && mel->ndim == 3 && out->ndim == 3,
             "mel [B, T, M] and out [B, M, T'] must be contiguous fp32");
  const int64_t B = mel->shape[0], T = mel->shape[1], M = mel->shape[2], keep = out->shape[2];
  KD_REQUIRE(out->shape[0] == B && out->shape[1] == M && keep >= 1 && keep <= T && B <= 65535 && M <= 0x7fffffff,
             "out must be [B, M, T'] with 1 <= T' <= T");
  void *pm, *po, *scratch;
  KD_TRY(tensor_ptr(mel, &pm));
  KD_TRY(tensor_ptr(out, &po));
  KD_TRY(get_workspace((uint64_t)B * sizeof(unsigned int), &scratch));
  KD_CUDA_CHECK(cudaMemsetAsync(scratch, 0, (size_t)B * sizeof(unsigned int), ctx().stream));   // below every ordered float
  ctx().launches++;
  const int64_t total = keep * M;
  int g = (int)((total + 255) / 256);
  if (g > 592) g = 592;
  log_mel_max_kernel<<<dim3(g, (unsigned)B), 256, 0, ctx().stream>>>((const float*)pm, T, (int)M, keep, (unsigned int*)scratch);
  KD_TRY(after_launch("log_mel_max_kernel"));
  dim3 grid((unsigned)((keep + 31) / 32), (unsigned)((M + 31) / 32), (unsigned)B);
  log_mel_finish_kernel<<<grid, dim3(32, 8), 0, ctx().stream>>>((const float*)pm, T, (int)M, keep, (const unsigned int*)scratch, (float*)po);
  return after_launch("log_mel_finish_kernel");
}
