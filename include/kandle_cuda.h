/*
 * kandle_cuda.h -- C ABI of libkandle_cuda.so, the sm_100a compute backend for Kandle.
 *
 * This is the boundary a Kandle backend package binds through N-API / FFI / ctypes.  Every entry
 * point replaces one kernel key (or one storage operation) of the reference's backend contract;
 * the comment above each declaration names the reference interface it stands in for, by path
 * inside the reference project.
 *
 * Conventions
 *   - Every function returns 0 on success and a non-zero kd_status otherwise; the message is
 *     retrieved with kd_last_error().  A binding turns non-zero into a thrown Error, which is how
 *     the reference reports misuse (synchronous exceptions from dispatch / kernels).
 *   - All operators only ENQUEUE work on the library's stream of the current device, in program
 *     order, exactly like the reference's queue.submit model.  kd_download and kd_synchronize are
 *     the only synchronisation points (the reference's dataAsync()).
 *   - Tensors are described by value with kd_tensor: storage handle + element offset + dtype +
 *     shape + strides (strides and offset in ELEMENTS, as in
 *     packages/backend-webgpu/src/base/tensor.ts:178-183).  Views are metadata only.
 *   - One process drives one GPU (one rank per GPU); kd_init selects it.
 *   - There is no CPU fallback: without a usable sm_100 device kd_init fails.
 */
#ifndef KANDLE_CUDA_H_
#define KANDLE_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KD_MAX_DIMS 8

typedef enum kd_status {
  KD_OK = 0,
  KD_ERR_INVALID = 1,     /* bad argument: shape/dtype/stride the operator does not accept */
  KD_ERR_CUDA = 2,        /* a CUDA runtime / driver call failed                           */
  KD_ERR_OOM = 3,         /* device allocation failed                                      */
  KD_ERR_NOT_INIT = 4,    /* kd_init has not been called                                   */
  KD_ERR_UNSUPPORTED = 5, /* valid request outside what this build implements              */
  KD_ERR_DEVICE = 6       /* a kernel reported an error flag (bounded wait ran out, ...)   */
} kd_status;

/* Logical dtypes = Kandle's DType (packages/types/src/base.ts:5-20) plus bfloat16. */
typedef enum kd_dtype {
  KD_F32 = 0,
  KD_F16 = 1,
  KD_BF16 = 2,
  KD_I32 = 3,
  KD_I64 = 4,
  KD_U8 = 5,
  KD_BOOL = 6
} kd_dtype;

/* Mirrors ITensorHandle's metadata (packages/types/src/tensor.ts:6-55). */
typedef struct kd_tensor {
  uint64_t storage; /* handle returned by kd_storage_alloc */
  int64_t offset;   /* in elements */
  int32_t dtype;    /* kd_dtype */
  int32_t ndim;
  int64_t shape[KD_MAX_DIMS];
  int64_t strides[KD_MAX_DIMS]; /* in elements */
} kd_tensor;

/* ---------------------------------------------------------------------------------------------
 * Device / context.  Replaces WebGPUBackend.create + WebGPUDeviceManager.init
 * (packages/backend-webgpu/src/index.ts:73-85, base/device.ts:95-176).
 * ------------------------------------------------------------------------------------------- */
/* One process drives one GPU from one host thread: kd_init binds the device to the calling thread
 * (the other entry points do not rebind it, so calls from another thread would reach that thread's
 * current device), launch configurations and scratch are kept per process, and a second kd_init
 * with another ordinal while the first context lives returns KD_ERR_UNSUPPORTED (kd_shutdown
 * first).  For N GPUs start N processes. */
int kd_init(int device_ordinal, unsigned flags);
int kd_shutdown(void);
int kd_synchronize(void);
int kd_device_count(int* count);
/* Thread-local message of the most recent failing call on this thread. */
int kd_last_error(char* buf, size_t buf_len);
/* Native stream handle (cudaStream_t) the library enqueues on, for event timing by the host. */
int kd_stream(void** stream_out);
/* Self-test of the bounded waits: runs a one-CTA kernel whose mbarrier wait can never be satisfied,
 * with a limit of `limit_us` microseconds (1..100000) instead of the ~1 s the real kernels use.
 * The kernel gives up, records error code 901, raises its abort flag and returns; the call
 * returns KD_OK and the NEXT kd_synchronize / kd_download reports KD_ERR_DEVICE, after which the
 * context works normally.  No reference counterpart (WebGPU has no device-side waits). */
int kd_selftest_wait_timeout(uint32_t limit_us);
/* Number of kernel launches the library has issued since kd_init (or the last reset). */
int kd_launch_count(uint64_t* count, int reset);

/* ---------------------------------------------------------------------------------------------
 * Storage.  Replaces WebGPUStorage: refcounted device buffers, new storage zero-initialised on
 * request, upload / stream-synchronising download
 * (packages/backend-webgpu/src/base/storage.ts:60-143,191-243; IStorage in
 * packages/types/src/storage.ts:5-25).
 * ------------------------------------------------------------------------------------------- */
int kd_storage_alloc(uint64_t bytes, int zero, uint64_t* storage_out);
int kd_storage_retain(uint64_t storage);
int kd_storage_release(uint64_t storage);
int kd_storage_bytes(uint64_t storage, uint64_t* bytes_out);
int kd_storage_device_ptr(uint64_t storage, void** ptr_out);
int kd_upload(uint64_t storage, uint64_t dst_offset_bytes, const void* host, uint64_t bytes);
int kd_download(uint64_t storage, uint64_t src_offset_bytes, void* host, uint64_t bytes);
/* Asynchronous variants for pinned host buffers (no implicit synchronisation). */
int kd_upload_async(uint64_t storage, uint64_t dst_offset_bytes, const void* host, uint64_t bytes);
int kd_download_async(uint64_t storage, uint64_t src_offset_bytes, void* host, uint64_t bytes);
int kd_host_alloc_pinned(uint64_t bytes, void** host_out);
int kd_host_free_pinned(void* host);
/* Allocator statistics: bytes handed out, bytes cached in free lists, bytes obtained from CUDA. */
int kd_memory_stats(uint64_t* in_use, uint64_t* cached, uint64_t* reserved);
/* Size of the library-owned scratch buffer (split-KV partials, split-K partials, sampling state).  It
 * is obtained straight from CUDA, outside the allocator above, and only ever grows.  No counterpart
 * in the reference (its kernels create their own temporaries,
 * packages/backend-webgpu/src/kernels/normalize/executor.ts:120-122). */
int kd_workspace_bytes(uint64_t* bytes_out);
/* Test support, no counterpart in the reference: overwrites that scratch buffer and the built-in
 * buffer of kd_attention_decode_noalloc with `byte_value` (stream-ordered), so that a test can tell
 * a kernel that read a slot it never wrote (0xFF gives NaN patterns) from one that did not. */
int kd_debug_fill_scratch(int byte_value);
int kd_empty_cache(void);

/* ---------------------------------------------------------------------------------------------
 * Operators, one per registry key.
 * ------------------------------------------------------------------------------------------- */

/* Key `flash_attention` (q,k,v,out,scale,isCausal):
 * packages/backend-webgpu/src/kernels/attention/executor.ts:41-235 and builder.ts:51-331.
 * q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D], out [B,Hq,Sq,D]; 3-D means B=1, 2-D means B=Hq=1.
 * Hq must be a multiple of Hkv (head_kv = head_q / (Hq/Hkv)).  Causal masking is top-left
 * aligned (column > row is masked).  Unlike the reference kernel, strides are honoured. */
int kd_flash_attention(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v,
                       const kd_tensor* out, float scale, int is_causal);

/* Key `matmul` (cfg, a, b): MatmulDispatchResult,
 * packages/core/src/dispatch/matmulOps.ts:32-125; executor
 * packages/backend-webgpu/src/kernels/matrix/executor.ts:47-76,438-598.
 * out = beta*c + alpha*op(a)*op(b); batch dims broadcast; full strides honoured. */
typedef struct kd_matmul_cfg {
  int64_t M, N, K;
  int32_t transpose_a, transpose_b; /* stored last two dims are [K,M] / [N,K] when set */
  float alpha, beta;
  int32_t has_c;
  int32_t reserved;
} kd_matmul_cfg;
int kd_matmul(const kd_matmul_cfg* cfg, const kd_tensor* a, const kd_tensor* b, const kd_tensor* c,
              const kd_tensor* out);

/* Keys `rms_norm`, `layer_norm`, `softmax` (inputs, params) -> result:
 * packages/backend-webgpu/src/kernels/normalize/executor.ts:26-183, shaderBuilder.ts:143-415.
 * Normalise over the last dimension; strided input, contiguous output; weight/bias may be NULL. */
int kd_rms_norm(const kd_tensor* x, const kd_tensor* weight, float eps, const kd_tensor* out);
int kd_layer_norm(const kd_tensor* x, const kd_tensor* weight, const kd_tensor* bias, float eps,
                  const kd_tensor* out);
int kd_softmax(const kd_tensor* x, const kd_tensor* out);

/* Key `index_select` (self, index, {dim}, output), dim 0 only (the embedding lookup):
 * packages/backend-webgpu/src/kernels/gather/executor.ts:34-155.  Indices int32 or int64;
 * an out-of-range index sets the device error flag instead of reading out of bounds. */
int kd_index_select(const kd_tensor* self, const kd_tensor* index, int dim, const kd_tensor* out);

/* Iterator keys (add, mul, mul_scalar, neg, cos, sin, silu, gelu, abs, div, maximum, tanh,
 * sigmoid): packages/backend-webgpu/src/kernels/pointwise/executor.ts:60-130 with the expression
 * table packages/backend-webgpu/src/kernels/pointwise/ops.ts.  Inputs broadcast to out's shape
 * (stride 0), rank <= 8.  `scalar` is alpha for add, the multiplier for mul_scalar. */
typedef enum kd_pointwise_op {
  KD_OP_ADD = 0,
  KD_OP_MUL = 1,
  KD_OP_MUL_SCALAR = 2,
  KD_OP_NEG = 3,
  KD_OP_COS = 4,
  KD_OP_SIN = 5,
  KD_OP_SILU = 6,
  KD_OP_GELU = 7,
  KD_OP_ABS = 8,
  KD_OP_DIV = 9,
  KD_OP_MAXIMUM = 10,
  KD_OP_TANH = 11,
  KD_OP_SIGMOID = 12,
  KD_OP_SUB = 13
} kd_pointwise_op;
int kd_pointwise(int op, const kd_tensor* a, const kd_tensor* b, float scalar, const kd_tensor* out);

/* Keys `copy`, `contiguous`, `copy_`, `cast`, `clone`: strided copy with dtype conversion,
 * packages/backend-webgpu/src/kernels/copy/index.ts:15-30.  src broadcasts to dst's shape. */
int kd_copy(const kd_tensor* dst, const kd_tensor* src);
/* Keys `zeros`, `ones`, `full`, `empty`. */
int kd_fill(const kd_tensor* dst, double value);
/* Key `arange` (packages/backend-webgpu/src/kernels/factory/index.ts:27): dst[i] = start+i*step. */
int kd_arange(const kd_tensor* dst, double start, double step);
/* Key `randn` (packages/backend-webgpu/src/kernels/random/shaderBuilder.ts:140-185 with the
 * Philox4x32-10 generator of random/philox.wgsl.ts:17-155 and the counter / key rule of
 * random/executor.ts:31-49): element i of the tensor takes member i % 2 of pair i / 2, whose counter
 * is [i / 2 + base_offset (mod 2^32), 0, 0, 0] under the key (seed & 0xffffffff, seed >> 32);
 * uniform = (word >> 8) * 2^-24; cosine branch of Box-Muller with u1 clamped to 1e-10;
 * out = mean + stddev * z.  `seed` and `base_offset` are what the reference's RandomState hands its
 * kernel (packages/types/src/random.ts:77-96); the binding keeps that state.
 * full_cols <= 0: `out` is a whole contiguous tensor numbered in row-major order (row0 = col0 = 0).
 * full_cols  > 0: `out` is the [rows, cols] slice at (row0, col0) of a row-major matrix with
 * full_cols columns and receives exactly the numbers that matrix would hold there, which is how a
 * tensor-parallel rank initialises its share of a weight (no counterpart in the reference). */
int kd_randn(const kd_tensor* out, uint64_t seed, uint32_t base_offset, float mean, float stddev, int64_t row0,
             int64_t col0, int64_t full_cols);
/* Key `argmax` over the last dimension, int32 or int64 output; lowest index wins ties:
 * packages/backend-webgpu/src/kernels/reduction/argShaderBuilder.ts:29-247. */
int kd_argmax(const kd_tensor* x, const kd_tensor* out);
/* Key `conv1d` (cfg, input, weight, bias?) -> [B,Cout,Wout]:
 * packages/backend-webgpu/src/kernels/window/algorithms/im2col.ts:124-268. */
int kd_conv1d(const kd_tensor* input, const kd_tensor* weight, const kd_tensor* bias, int stride,
              int padding, const kd_tensor* out);

/* ---------------------------------------------------------------------------------------------
 * Whisper log-mel front end (fp32), the step before the audio encoder.  Replaces the chain
 * stft -> abs -> square -> MelScale of packages/core/src/dispatch/handlers/composite.ts:527-681,
 * audio/functional/spectrogram.ts:28-76, audio/transforms/MelScale.ts:95-108, and the host loop of
 * playground-node/src/whisper/audio.ts:379-405.
 *   kd_stft_frames: frames_out[b,t,n] = waveform[b, t*hop + n - (center ? n_fft/2 : 0)] * window[n],
 *     zero outside the signal (the reference pads in constant mode whatever pad_mode says);
 *     frames_out is [B, 1 + (L + 2 pad - n_fft) / hop, n_fft].  The DFT itself is a kd_matmul of the
 *     frames with a [n_fft, 2F] basis (cosines, then minus sines), F = n_fft/2 + 1.
 *   kd_power_spectrum: spec [..., 2F] (real parts then imaginary parts) -> |X|^2 [..., F], computed
 *     as the reference does: the magnitude rounded to fp32, then squared.
 *   kd_whisper_log_mel_norm: mel [B, T, M] -> out [B, M, T'] (T' <= T: the reference drops the last
 *     frame), out = (max(log10(max(mel, 1e-10)), item_max - 8) + 4) / 4.
 * ------------------------------------------------------------------------------------------- */
int kd_stft_frames(const kd_tensor* waveform, const kd_tensor* window, int n_fft, int hop_length, int center,
                   const kd_tensor* frames_out);
int kd_power_spectrum(const kd_tensor* spec_re_im, const kd_tensor* power_out);
int kd_whisper_log_mel_norm(const kd_tensor* mel, const kd_tensor* out);

/* ---------------------------------------------------------------------------------------------
 * Next-token sampling on the device.  Replaces `sample` / `sampleGreedy`
 * (packages/model-utils/src/sampling/index.ts:103-238): temperature, top-k, top-p, renormalise,
 * draw by running sum in index order; do_sample == 0 is the greedy branch (argmax, lowest index on
 * ties).  logits fp32 [V] or [B,V]; uniforms fp32 [B] in [0,1) stand in for Math.random() (one per
 * sequence; ignored when greedy); out_ids int64 [B]; out_logprob fp32 [B] or NULL receives
 * log(p_token + 1e-10) of the filtered, renormalised distribution, as SampleResult.logProb.  The
 * reference's host path (download, stable sort of V indices, Float32Array storage with double
 * arithmetic) is reproduced without a sort: radix selection on a monotone key with the sort's tie
 * rule, probability mass in exact fixed point.  Its display list (top-10 ids/probs) is not produced.
 * ------------------------------------------------------------------------------------------- */
int kd_sample(const kd_tensor* logits, double temperature, int top_k, double top_p, int do_sample,
              const kd_tensor* uniforms, const kd_tensor* out_ids, const kd_tensor* out_logprob);

/* ---------------------------------------------------------------------------------------------
 * Timing.  CUDA events recorded on the library's stream (the reference only has host-side
 * performance.now() around dataAsync(), playground-node/src/qwen3/index.ts:161,253).
 * ------------------------------------------------------------------------------------------- */
int kd_event_create(uint64_t* event_out);
int kd_event_record(uint64_t event);
int kd_event_elapsed_ms(uint64_t start, uint64_t stop, float* ms_out); /* synchronises on `stop` */
int kd_event_destroy(uint64_t event);

/* ---------------------------------------------------------------------------------------------
 * Fused bf16 fast paths.  Each one computes what a run of the reference's eager operator calls
 * computes; the comment names that run.  They exist because one decoder layer is ~41 separate
 * kernel submissions on the eager path (packages/model-utils/src/attention/gqa.ts:246-430,
 * mlp/swiglu.ts:119-134, qwen3/decoder_layer.ts:191-241).
 * ------------------------------------------------------------------------------------------- */
typedef enum kd_epilogue {
  KD_EPI_NONE = 0,
  KD_EPI_RESIDUAL = 1, /* out = residual + x W^T : `linear` followed by the residual `add`;
                          residual has the output's dtype (bf16, or fp32 residual stream) */
  KD_EPI_SWIGLU = 2    /* out = silu(x Wg^T) * (x Wu^T) : gate/up `linear`, `silu`, `mul`;
                          weight rows interleave 16 gate rows / 16 up rows per 32-row block      */
} kd_epilogue;
/* `linear` on the tensor cores (tcgen05): x [tokens,K] bf16, weight [N,K] bf16 (K-major, as
 * composite.ts:62-70 passes it), out [tokens,N] (or [tokens,N/2] for SWIGLU) bf16 or fp32. */
int kd_linear_bf16(const kd_tensor* x, const kd_tensor* weight, const kd_tensor* residual, int epilogue,
                   const kd_tensor* out);
typedef enum kd_activation { KD_ACT_NONE = 0, KD_ACT_GELU = 1 } kd_activation;
/* out = residual + act(x W^T + bias): `linear` with its bias (composite.ts:55-77), the `gelu` that
 * follows fc1 in the Whisper block (packages/model-utils/src/whisper/block.ts:150-200; tanh form with
 * the +-20 clamp of packages/backend-webgpu/src/kernels/pointwise/ops.ts:301) and the residual `add`,
 * all in the GEMM epilogue on the fp32 accumulator.  bias [N] and residual [tokens,N] are optional
 * (NULL); everything is bf16 and contiguous, weight rows may be strided (a row slice of a packed
 * in_proj_weight, MultiheadAttention.ts:333-348). */
int kd_linear_bf16_bias(const kd_tensor* x, const kd_tensor* weight, const kd_tensor* bias,
                        const kd_tensor* residual, int activation, const kd_tensor* out);
/* conv1d on token-major activations for the Whisper stem (packages/model-utils/src/whisper/encoder.ts:
 * 202-215: conv1 -> gelu -> conv2 -> gelu -> permute(0,2,1) -> + embed_positions): input [B,L,Cin],
 * weight_kc [Cout, ksz*Cin] = the reference's [Cout,Cin,ksz] weight with the tap index moved in
 * front of the channel index, out [B,Wout,Cout] = the reference's conv1d output already permuted to
 * (0,2,1).  A vectorised im2col (three input rows side by side per output row) feeds the tensor-core
 * GEMM; bias, GELU and an optional residual [B,Wout,Cout] (the position table repeated per clip) are
 * applied in its epilogue.  All bf16, contiguous, channel counts multiples of 8. */
int kd_conv1d_tokens_bf16(const kd_tensor* input, const kd_tensor* weight_kc, const kd_tensor* bias,
                          const kd_tensor* residual, int activation, int ksz, int stride, int padding,
                          const kd_tensor* out);

/* `linear` for 1..128 activation rows (decode): weights are streamed once from HBM with the
 * operands swapped so that weight rows fill the MMA's M dimension.  The shape and dtype of `out`
 * select the form: bf16 [rows,N] (no split-K); bf16 [rows,N/2] with epilogue = KD_EPI_SWIGLU; or fp32
 * [splits,rows,N] split-K partial sums that the consumers below add up (kd_linear_bf16_skinny_splits
 * suggests `splits` for a given weight shape). */
int kd_linear_bf16_skinny(const kd_tensor* x, const kd_tensor* weight, int epilogue, const kd_tensor* out);
int kd_linear_bf16_skinny_splits(int64_t N, int64_t K, int* splits_out);

/* cos/sin tables [seq_len, D/2] fp32 for positions start..start+seq_len-1: arange -> mul(inv_freq)
 * -> cos / sin of packages/model-utils/src/rope.ts:192-261.  `pos` (device int32 scalar) overrides
 * start_pos when given. */
int kd_rope_table(const kd_tensor* inv_freq, const kd_tensor* pos, int start_pos, int seq_len,
                  const kd_tensor* cos_out, const kd_tensor* sin_out);
/* q/k RMSNorm over head_dim + RoPE + [B,S,H,D] layout + KV-cache write in one pass
 * (packages/model-utils/src/attention/gqa.ts:274-322, rope.ts:546-644, kv-cache.ts:180-188).
 * qkv: bf16 [B,S,(Hq+2Hkv)*D] (q heads, then k heads, then v heads) or fp32 split-K partials
 * [splits,B*S,(Hq+2Hkv)*D].  Writes q_out bf16 [B,S,Hq,D] and rows [pos, pos+S) of the caches
 * [B,Hkv,maxS,D].  A write position outside the cache sets the device error flag. */
int kd_qkv_norm_rope_cachewrite(const kd_tensor* qkv, const kd_tensor* q_norm_weight,
                                const kd_tensor* k_norm_weight, float eps, const kd_tensor* cos,
                                const kd_tensor* sin, const kd_tensor* k_cache, const kd_tensor* v_cache,
                                const kd_tensor* pos, int start_pos, const kd_tensor* q_out);
/* The same into a PAGED cache (no counterpart in the reference, whose only cache is the contiguous
 * StaticKVCache; the update semantics of packages/model-utils/src/kv-cache.ts:164-212 are kept:
 * positions [pos, pos+S) of every sequence are overwritten, nothing else moves): k_pool / v_pool
 * [pages,Hkv,128,D], block_table int32 [B,max_pages] names the page of each run of 128 positions. */
int kd_qkv_norm_rope_cachewrite_paged(const kd_tensor* qkv, const kd_tensor* q_norm_weight,
                                      const kd_tensor* k_norm_weight, float eps, const kd_tensor* cos,
                                      const kd_tensor* sin, const kd_tensor* k_pool, const kd_tensor* v_pool,
                                      const kd_tensor* block_table, const kd_tensor* pos, int start_pos,
                                      const kd_tensor* q_out);
/* Scatters rows [0,S) of contiguous K / V [B,Hkv,S,D] (what a prefill produced) into positions
 * [start_pos, start_pos+S) of a paged cache.  Same cache-update semantics as above. */
int kd_kv_pages_write(const kd_tensor* k_src, const kd_tensor* v_src, const kd_tensor* k_pool, const kd_tensor* v_pool,
                      const kd_tensor* block_table, int start_pos);
/* The QKV projection and kd_qkv_norm_rope_cachewrite in one tensor-core GEMM whose epilogue does the
 * q/k-norm, RoPE and KV-cache write (head_dim 128, prefill): x bf16 [B*S,K], wqkv bf16 [(Hq+2Hkv)*128,K]
 * (q rows, k rows, v rows). */
int kd_qkv_linear_norm_rope_cachewrite(const kd_tensor* x, const kd_tensor* wqkv, const kd_tensor* q_norm_weight,
                                       const kd_tensor* k_norm_weight, float eps, const kd_tensor* cos,
                                       const kd_tensor* sin, const kd_tensor* k_cache, const kd_tensor* v_cache,
                                       int start_pos, const kd_tensor* q_out);
/* silu(gate) * up (packages/model-utils/src/mlp/swiglu.ts:121-131) from a bf16 [rows,2I] matrix or
 * fp32 partials [splits,rows,2I] whose columns interleave 16 gate / 16 up values. */
int kd_swiglu(const kd_tensor* gate_up, const kd_tensor* out);
/* (residual + x) -> bf16 sum_out, then RMSNorm(sum) * weight -> norm_out
 * (packages/model-utils/src/qwen3/decoder_layer.ts:224-232).  x: bf16 [rows,n] or fp32 partials
 * [splits,rows,n] (a plain fp32 matrix is the splits = 1 case); residual and sum_out may be NULL
 * (plain RMSNorm) and are bf16 or fp32 (an fp32 residual stream is summed without rounding). */
int kd_add_rmsnorm(const kd_tensor* x, const kd_tensor* residual, const kd_tensor* weight, float eps,
                   const kd_tensor* sum_out, const kd_tensor* norm_out);
int kd_increment_i32(const kd_tensor* scalar, int delta);

/* CUDA-graph capture of everything enqueued between begin and end (no counterpart in the
 * reference, whose per-op host overhead is what this removes). */
/* Enables programmatic dependent launch for the kernels of the decode step (they all begin with a
 * grid-dependency wait), so that each kernel's launch latency overlaps its predecessor.
 * enabled = 2 additionally lets kd_attention_decode[_paged/_noalloc] read the context length and
 * fetch the K/V tiles that do not hold the LAST position (context length - 1) BEFORE its
 * grid-dependency wait, while the kernel before it is still draining.  The caller then promises
 * that, of everything the call reads, only the query and the cache rows of that last position
 * were written by the launch directly before it; the context length, the block table and all
 * earlier cache rows must date from launches that are separated from the call by at least one
 * kernel of this library other than the fused layer kernel and the decode attention itself
 * (every other kernel passes its grid-dependency wait before it lets its successor start).  A decode step that writes one new
 * row per layer, as Qwen3Engine's does, satisfies this. */
int kd_set_pdl(int enabled);
int kd_graph_begin(void);
int kd_graph_end(uint64_t* graph_out);
int kd_graph_launch(uint64_t graph);
int kd_graph_destroy(uint64_t graph);

/* Decode attention: one new query position per sequence against a KV cache.  Computes what the
 * reference computes with `_repeatKv` (materialised GQA expansion) + `flash_attention` with
 * isCausal=false on the cache prefix views (packages/model-utils/src/attention/gqa.ts:325-336,
 * 407-414; cache layout packages/model-utils/src/kv-cache.ts:123-130,197-211), without the copies.
 * q/out [B,Hq,1,D]; k_cache/v_cache [B,Hkv,maxS,D]; keys [0, ctx) are attended.  ctx comes from
 * `ctx_len` (device int32 scalar, so a captured graph can be replayed as the sequence grows) or,
 * when that is NULL, from ctx_len_host.  splits = 0 picks the split-KV factor automatically.
 * Scratch for the split partials is library-owned and grows on demand (the first call at a larger
 * size allocates, so make that call before capturing a graph).  Whole 64-row key tiles are loaded:
 * cache rows between ctx and the end of the last tile get probability 0 but are multiplied in, so
 * they must hold finite values (the reference's cache is created from zeros, kv-cache.ts:123-130). */
int kd_attention_decode(const kd_tensor* q, const kd_tensor* k_cache, const kd_tensor* v_cache,
                        const kd_tensor* ctx_len, int ctx_len_host, float scale, int splits,
                        const kd_tensor* out);
/* Same computation as kd_attention_decode for callers that are not allowed to allocate device
 * memory while they run: a serving loop that has handed the whole GPU to its own pool, code running
 * inside a memory-budgeted plugin host, or a latency path where a cudaMalloc (which can synchronise
 * the device) is unacceptable.  It has no counterpart in the reference.  The split-KV partials go to
 * an 8 MiB buffer built into the library image instead of the growing workspace, and the call makes
 * no cudaMalloc / cudaFree and uses no allocating library routine.  Limits and rules:
 *   - B * Hkv * splits * (Hq/Hkv) * (D + 2) * 4 bytes must fit in 8 MiB, otherwise the call fails
 *     with KD_ERR_INVALID and a message that names both sizes (pass a smaller `splits`);
 *   - the first call on a device looks up the buffer's device address; make that call before any
 *     stream capture begins;
 *   - all calls share the one buffer, which keeps whatever the previous call left in it (nothing in
 *     it needs clearing: every slot a call reads was written by that same call), so two calls that
 *     overlap on the GPU race with each other; keep them on one stream;
 *   - every GPU that loads the library holds the 8 MiB until the process exits. */
int kd_attention_decode_noalloc(const kd_tensor* q, const kd_tensor* k_cache, const kd_tensor* v_cache,
                                const kd_tensor* ctx_len, int ctx_len_host, float scale, int splits,
                                const kd_tensor* out);
/* Paged variant (no counterpart in the reference, which only has the contiguous static cache):
 * k_pool/v_pool [pages,Hkv,128,D]; block_table [B,max_pages] int32 names the page of each
 * 128-key tile of each sequence. */
int kd_attention_decode_paged(const kd_tensor* q, const kd_tensor* k_pool, const kd_tensor* v_pool,
                              const kd_tensor* block_table, const kd_tensor* ctx_len, int ctx_len_host,
                              float scale, int splits, const kd_tensor* out);

/* Everything a decoder layer does between two attention calls of a decode step, as ONE
 * persistent cooperative kernel (one CTA per SM; phases separated by grid-wide counters instead of
 * kernel boundaries, weight tiles of the next phase prefetched while the current one finishes):
 *   h1 = resid_in + attn W_o^T                      o_proj + residual add   (decoder_layer.ts:218-224)
 *   x  = rmsnorm(h1) * post_norm_w                  post_attention_layernorm (decoder_layer.ts:226)
 *   act = silu(x Wg^T) * (x Wu^T)                   mlp/swiglu.ts:119-134 (w_gate_up rows interleaved 16/16)
 *   resid_out = h1 + act W_down^T                   down_proj + residual add (decoder_layer.ts:232-238)
 *   x_out = rmsnorm(resid_out) * next_norm_w        the next layer's input_layernorm, or the final norm
 *   qkv_partials[s] = x_out W_qkv_next^T (split s)  the next layer's q/k/v projections (gqa.ts:246-290),
 *                                                   consumed by kd_qkv_norm_rope_cachewrite
 * (paths under packages/model-utils/src/qwen3/ and .../attention/).  attn [Mb,Hq*D] bf16 (row
 * stride a multiple of 8), resid_* fp32 [Mb,H] (resid_out may be resid_in; resid_mid is scratch that
 * receives h1), x_out [Mb,H] and act [Mb,I] bf16, qkv_partials fp32 [splits,Mb,Nqkv] with `splits`
 * as kd_decode_layer_chain_splits suggests (any value whose K split leaves no slice empty works).
 * w_qkv_next and qkv_partials are NULL after the last layer.  1 <= Mb <= 128, H <= 4096.  The
 * launch fails (no hang) if the device cannot hold one CTA per SM at once.  A wait that runs out
 * (about one second) reports KD_ERR_DEVICE at the next synchronisation, codes 501-507. */
int kd_decode_layer_chain(const kd_tensor* attn, const kd_tensor* w_o, const kd_tensor* resid_in,
                          const kd_tensor* post_norm_w, const kd_tensor* w_gate_up, const kd_tensor* w_down,
                          const kd_tensor* next_norm_w, float eps, const kd_tensor* w_qkv_next,
                          const kd_tensor* resid_mid, const kd_tensor* resid_out, const kd_tensor* x_out,
                          const kd_tensor* act, const kd_tensor* qkv_partials);
int kd_decode_layer_chain_splits(int64_t N, int64_t K, int* splits_out);
/* The same stretch of a decode step in FOUR dependent phases and without split-K phases, and further: up
 * to and including the next layer's q_norm / k_norm, rotary embedding and KV-cache write
 * (packages/model-utils/src/attention/gqa.ts:274-322, rope.ts:546-644, kv-cache.ts:164-212), so that
 * a decode step is two launches per layer (this one and kd_attention_decode).
 *   h1 = resid_in + attn W_o^T
 *   act = silu(rs1 (x1 Wg^T)) * (rs1 (x1 Wu^T))   x1 = bf16(h1 * post_norm_w), rs1 = 1/sqrt(mean(h1^2)+eps):
 *                                              RMSNorm's per-sequence scale is applied to the fp32
 *                                              accumulator instead of to the activations
 *   resid_out = h1 + act W_down^T               x2 = bf16(resid_out * next_norm_w)
 *   qkv = rs2 (x2 W_qkv_next^T)                 one head per unit of work, whose epilogue does that head's
 *                                              RMSNorm (q_norm_w / k_norm_w), the rotation by cos/sin
 *                                              [1,64] and stores q into q_out [Mb,1,Hq,128] or k / v into
 *                                              row *pos of the next layer's caches (contiguous
 *                                              [B,Hkv,maxS,128], or pools [pages,Hkv,128,128] addressed
 *                                              through block_table int32 [B,max_pages] when it is given)
 * The sequences are the rows of every accumulator and a unit of work is a narrow slice of weight
 * rows, so an epilogue thread owns one sequence; where o_proj or down_proj would leave most SMs
 * idle, the K of a slice is split over the 2 or 4 CTAs of a thread-block cluster, which hand their
 * partial sums to the first of them through distributed shared memory (no partial sum ever goes
 * through global memory).
 * With w_qkv_next == NULL (after the last layer) the launch ends with
 * x_final = bf16(resid_out * rs2 * next_norm_w), the lm_head's input, and the arguments from
 * q_norm_w to q_out are ignored.  head_dim 128 only; 1 <= Mb <= 128; hidden size a multiple of 16;
 * resid_out may be resid_in.  A cache row outside [0, maxS) is not written and reports KD_ERR_DEVICE
 * code 102, a wait that runs out codes 521-529.  Results are bit-identical from launch to launch;
 * the launch plan (unit widths, K splits: kd_debug_decode_layer_plan), and with it the order of the
 * sums, follows the shapes including the number of sequences. */
/* Test / profiling support, no counterpart in the reference: device-side timestamps of the last
 * kd_decode_layer_fused launch, [SMs][16] nanoseconds (0: start; per phase g: 1+3g dependency seen,
 * 2+3g accumulator ready, 3+3g outputs published); only in a process started with
 * KD_DECODE_LAYER_TRACE=1. */
int kd_debug_decode_layer_trace(uint64_t* out, int max_entries);
int kd_decode_layer_fused(const kd_tensor* attn, const kd_tensor* w_o, const kd_tensor* resid_in,
                          const kd_tensor* post_norm_w, const kd_tensor* w_gate_up, const kd_tensor* w_down,
                          const kd_tensor* next_norm_w, float eps, const kd_tensor* w_qkv_next,
                          const kd_tensor* q_norm_w, const kd_tensor* k_norm_w, const kd_tensor* cos,
                          const kd_tensor* sin, const kd_tensor* pos, const kd_tensor* k_cache_next,
                          const kd_tensor* v_cache_next, const kd_tensor* block_table, const kd_tensor* q_out,
                          const kd_tensor* resid_out, const kd_tensor* x_final);
/* The tensor-parallel form (no counterpart in the reference): every rank passes ITS slices (W_o and
 * W_down: input columns; W_gate_up and W_qkv_next: rows; attn, caches and q_out: its heads) and the
 * same residual; the partial sums of o_proj and down_proj are exchanged INSIDE the kernel, unit by
 * unit, through the peer-mapped buffers of kd_p2p_connect (plain stores and loads, one flag per unit
 * written into every peer's buffer, local polling, every wait bounded at about five seconds: error
 * code 531) and summed in rank order, so every rank holds the same residual bit for bit.  All ranks
 * must issue the same sequence of calls.  After an error 531 reconnect the peer buffers. */
/* Test support: the launch plan (cluster size; per phase rows per unit, units, K split, k-blocks per
 * CTA of a split group, k-blocks per bulk copy) that kd_decode_layer_fused[_tp] would use for these
 * shapes when `grid_plain` / `grid_cluster2` / `grid_cluster4` CTAs can be resident together with
 * clusters of 1 / 2 / 4 (0: not available).  Touches no device.  out: 29 ints, [0] = cluster size
 * (0: no configuration), then 7 per phase: N, K, rows per unit, units, split, k-blocks per CTA, k-blocks
 * per copy. */
int kd_debug_decode_layer_plan(int sequences, int hidden, int attn_width, int inter, int qkv_rows, int tensor_parallel,
                               int grid_plain, int grid_cluster2, int grid_cluster4, int* out, int out_len);
int kd_decode_layer_fused_tp(const kd_tensor* attn, const kd_tensor* w_o, const kd_tensor* resid_in,
                             const kd_tensor* post_norm_w, const kd_tensor* w_gate_up, const kd_tensor* w_down,
                             const kd_tensor* next_norm_w, float eps, const kd_tensor* w_qkv_next,
                             const kd_tensor* q_norm_w, const kd_tensor* k_norm_w, const kd_tensor* cos,
                             const kd_tensor* sin, const kd_tensor* pos, const kd_tensor* k_cache_next,
                             const kd_tensor* v_cache_next, const kd_tensor* block_table, const kd_tensor* q_out,
                             const kd_tensor* resid_out, const kd_tensor* x_final);

/* ---------------------------------------------------------------------------------------------
 * Tensor-parallel collectives (no counterpart in the reference, which is single-device).  One
 * process per GPU; NCCL is loaded at run time from `nccl_path` (NULL/"" = the system libnccl.so.2).
 * Rank 0 creates the 128-byte id with kd_comm_unique_id, the host program distributes it, every
 * rank calls kd_comm_init.  kd_allreduce_sum is enqueued on the library's stream (in place, bf16 or
 * fp32) and is a no-op without a communicator.  kd_comm_check polls for asynchronous NCCL errors
 * and aborts the communicator when one is found.  Destroy every graph that captured an all-reduce
 * (kd_graph_destroy) before kd_comm_destroy: NCCL waits for such references to go away.
 * ------------------------------------------------------------------------------------------- */
int kd_comm_unique_id(const char* nccl_path, char* id_out, size_t id_bytes);
int kd_comm_init(const char* nccl_path, int nranks, int rank, const char* id, size_t id_bytes);
int kd_comm_info(int* nranks, int* rank);
int kd_allreduce_sum(const kd_tensor* t);
int kd_comm_check(void);
int kd_comm_destroy(void);

/* One-shot all-reduce over NVLink peer memory for the small messages of a tensor-parallel decode
 * step, fused with the residual add and RMSNorm that follow (no counterpart in the reference; the
 * steps it replaces per rank are o_proj / down_proj partial sums -> residual add -> RMSNorm,
 * packages/model-utils/src/qwen3/decoder_layer.ts:218-238).  Every rank owns one buffer (two 2 MiB
 * data slots + flags) that its peers map through CUDA IPC; the kernel uses ordinary loads and
 * stores on those addresses (no TMA, no multicast), publishes one flag per row into every peer's
 * buffer and polls only local flags, each wait bounded (about five seconds, then KD_ERR_DEVICE code
 * 601 at the next synchronisation and an undefined result for that call).
 *   kd_p2p_prepare     allocates the buffer and returns its 64-byte IPC handle; the host program
 *                      gathers the handles of all ranks (rank order)
 *   kd_p2p_connect     maps the peers' buffers (at most 8 ranks, all on one node)
 *   kd_p2p_emulate     instead of the two calls above: `nranks` ranks emulated on this one GPU, all in
 *                      one cooperative launch (tests on a single GPU); tensors then carry a leading
 *                      [nranks] dimension for x, sum_out and norm_out
 *   kd_allreduce_add_rmsnorm
 *                      x fp32 [splits,rows,n] split-K partial sums of this rank;
 *                      sum_out = sum over ranks (rank order, so identical bits on every rank) of
 *                      sum over splits of x, + residual (fp32 [rows,n], may be NULL);
 *                      norm_out = bf16 RMSNorm(sum_out) * weight.  rows <= 128, rows*n*4 <= 2 MiB.
 *                      Every rank must make the same sequence of calls; capture into a graph is
 *                      possible (the call counter lives in device memory).
 *   kd_p2p_selftest_dropped_flag
 *                      emulated ranks only: rank `drop_rank` never publishes its flags, the others'
 *                      waits run out after `wait_cycles` clock cycles; used to test the error path.
 *   kd_p2p_selftest_silent_peers
 *                      connects this process as rank 0 of `nranks` whose other ranks are buffers on
 *                      this GPU that nobody writes: kd_decode_layer_fused_tp then publishes its
 *                      partial sums, waits `wait_cycles` clock cycles for peers that never answer
 *                      and reports error 531; used to test that error path without a second GPU
 *                      and without a hang.  With answered_tag = t the stand-ins' flags already
 *                      carry the tag of launch number t (launches count from 1) and their partial
 *                      sums are zero: that launch completes and must give the result of
 *                      kd_decode_layer_fused.  kd_p2p_disconnect ends it. */
int kd_p2p_prepare(char* handle_out, size_t handle_bytes);
int kd_p2p_connect(int nranks, int rank, const char* handles, size_t handle_bytes);
int kd_p2p_emulate(int nranks);
int kd_p2p_info(int* ready, int* nranks, int* rank);
int kd_p2p_disconnect(void);
int kd_allreduce_add_rmsnorm(const kd_tensor* x, const kd_tensor* residual, const kd_tensor* weight, float eps,
                             const kd_tensor* sum_out, const kd_tensor* norm_out);
int kd_p2p_selftest_silent_peers(int nranks, uint32_t wait_cycles, uint32_t answered_tag);
int kd_p2p_selftest_dropped_flag(const kd_tensor* x, const kd_tensor* weight, const kd_tensor* norm_out, int drop_rank,
                                 uint32_t wait_cycles);

#ifdef __cplusplus
}
#endif
#endif /* KANDLE_CUDA_H_ */
