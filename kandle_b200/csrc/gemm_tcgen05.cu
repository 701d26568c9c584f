// bf16 GEMM on the 5th-generation tensor cores: out[M,N] = A[M,K] * W[N,K]^T (+ epilogue).
//
// This is the `linear` hot op of the prefill (the reference computes it with a 32x32 scalar-FMA
// WGSL tile, packages/backend-webgpu/src/kernels/matrix/builder.ts:837-1066).  Both operands are
// K-major, which is exactly what `linear` passes: activations [tokens, K] and the weight stored
// [N, K] (packages/core/src/dispatch/handlers/composite.ts:62-70).
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: 128x64 A tile + BLOCK_Nx64 W tile per stage, 128-byte swizzle,
//               mbarrier complete_tx; loads are plain tiled loads (no cluster multicast).
//   warp 1      one elected thread issues tcgen05.mma (M=128, N=BLOCK_N, K=16 x4 per stage) into a
//               TMEM accumulator; tcgen05.commit releases the smem stage / publishes the tile.
//   warps 2-5   epilogue: tcgen05.ld the 128xBLOCK_N fp32 tile (one row per thread), apply the
//               fused epilogue, convert and store.  Two TMEM accumulators let the epilogue of tile
//               i overlap the mainloop of tile i+1.
// Fused epilogues: residual add (o_proj / down_proj) and SiLU(gate)*up for a weight whose rows
// interleave 16 gate rows with the 16 matching up rows per 32-row block.
//
// Roofline: tensor-core bound; 2*M*N*K flops per call.
#include "common.cuh"
#include "kernels.cuh"
#include "sm100.cuh"

namespace kd {

using namespace sm100;

// ----------------------------------------------------------------------------- tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                      uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(KD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  KD_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base address must be 16-byte aligned");
  KD_REQUIRE((row_stride * 2) % 16 == 0, "TMA row stride must be a multiple of 16 bytes (got %llu elements)",
             (unsigned long long)row_stride);
  KD_REQUIRE(box_cols * 2 <= 128 && box_rows <= 256, "TMA box [%u,%u] too large for 128-byte swizzle", box_rows, box_cols);
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {row_stride * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstr, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(KD_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return KD_OK;
}

int make_tmap_bf16_3d(CUtensorMap* out, const void* base, uint64_t d2, uint64_t rows, uint64_t cols, uint64_t stride2,
                      uint64_t row_stride, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(KD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  KD_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base address must be 16-byte aligned");
  KD_REQUIRE((row_stride * 2) % 16 == 0 && (stride2 * 2) % 16 == 0, "TMA strides must be multiples of 16 bytes");
  KD_REQUIRE(box_cols * 2 <= 128 && box_rows <= 256, "TMA box [%u,%u] too large for 128-byte swizzle", box_rows, box_cols);
  cuuint64_t gdim[3] = {cols, rows, d2};
  cuuint64_t gstr[2] = {row_stride * 2, stride2 * 2};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstr, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(KD_ERR_CUDA, "cuTensorMapEncodeTiled (3-D) failed with code %d", (int)r);
  return KD_OK;
}

// ----------------------------------------------------------------------------- kernel
struct GemmParams {
  int M, N, K;            // N = rows of W (for EPI_SWIGLU the output is N/2 wide)
  void* out;
  int64_t ldo;
  int out_f32;            // 0: bf16 output, 1: fp32 output
  const void* resid;      // bf16 when the output is bf16, fp32 when the output is fp32
  int64_t ldr;
  int epi;
  const __nv_bfloat16* bias;   // [N] added to the accumulator before the activation and the residual, or null
  int act;                     // 0 none, 1 GELU (tanh form) after the bias
  int wide_store;              // bf16 output rows start on 32-byte boundaries: 32-byte vector stores
  int wide_f32, wide_resid;    // the same for an fp32 output and for the residual operand
  int num_m_tiles, num_n_tiles;
  int* err;
  // epi == 3: the columns are (Hq + 2 Hkv) heads of 128; q/k heads get RMSNorm over the head + RoPE,
  // q goes to q_out [tokens, Hq, 128], k/v rows to the KV cache at position pos0 + (token % S)
  int S, Hq, Hkv, pos0;
  float eps;
  const float* cos_t;
  const float* sin_t;
  const __nv_bfloat16* qw;
  const __nv_bfloat16* kw;
  __nv_bfloat16* q_out;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  int64_t kc_b, kc_h, kc_s;
};

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
// GELU as the reference's shader writes it (packages/backend-webgpu/src/kernels/pointwise/ops.ts:301):
// 0.5 x (1 + tanh(clamp(u, +-20))), u = 0.7978845608 (x + 0.044715 x^3), evaluated as
// x / (1 + exp(-2u)) (the same function; tanh(+-20) is +-1 in fp32, so the clamp changes nothing).
// The epilogue is bound by the special-function unit (a quarter-rate pipe shared by the four
// epilogue warps of an SM), so this form spends exactly two such operations per element, ex2 and
// rcp, and four FMA-pipe instructions: a = -2 u log2(e) = x (c1 + c2 x^2).
__device__ __forceinline__ float gelu_f(float x) {
  const float a = x * fmaf(x * x, -0.1029432394f, -2.3022081983f);
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(a));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return x * r;
}
// x / (1 + exp(-clamp(x, +-88))) (packages/backend-webgpu/src/kernels/pointwise/ops.ts:299) as
// x * rcp(1 + ex2(-x log2 e)): beyond the clamp the quotient is x or (-)0 to fp32 precision either way.
__device__ __forceinline__ float silu_f(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return x * r;
}

template <int BLOCK_N, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmParams p) {
  constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  constexpr int B_BYTES = BLOCK_N * GEMM_BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BLOCK_N < 32 ? 32 : 2 * BLOCK_N;
  constexpr uint32_t IDESC = make_idesc_bf16(GEMM_BM, BLOCK_N, 0, 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 4); }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_k_blocks = (p.K + GEMM_BK - 1) / GEMM_BK;
  const int total_tiles = p.num_m_tiles * p.num_n_tiles;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int m_tile = tile / p.num_n_tiles, n_tile = tile - m_tile * p.num_n_tiles;
        for (int kb = 0; kb < num_k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.err, 201)) { ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &full[stage], kb * GEMM_BK, m_tile * GEMM_BM);
          tma_load_2d(sa + A_BYTES, &tmap_b, &full[stage], kb * GEMM_BK, n_tile * BLOCK_N);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.err, 202)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BLOCK_N);
        for (int kb = 0; kb < num_k_blocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.err, 203)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            const uint64_t adesc = make_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(b_addr + k * 32, 16, 1024);
            umma_ss(d_tmem, adesc, bdesc, IDESC, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int m_tile = tile / p.num_n_tiles, n_tile = tile - m_tile * p.num_n_tiles;
      bool ok = mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.err, 204);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m_tile * GEMM_BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      bool released = false;   // accumulator already handed back inside the branch
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BLOCK_N);
      if (BLOCK_N == 256 && p.epi == 3) {
        // q/k-norm + RoPE + cache write (see fused.cu for the stand-alone kernel and the reference
        // operators it replaces).  A thread owns one token row; a head is 128 consecutive columns,
        // so the norm and both members of every rotation pair (i, i+64) are thread-local.
        const int b_idx = row / p.S, s_idx = row - b_idx * p.S;
#pragma unroll 1
        for (int hd = 0; hd < BLOCK_N / 128; ++hd) {
          uint32_t x[128];
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_row + hd * 128 + c * 32, &x[c * 32]);
          tmem_wait_ld();
          const int head = n_tile * (BLOCK_N / 128) + hd;
          if (!row_ok || head >= p.Hq + 2 * p.Hkv) continue;
          const bool is_q = head < p.Hq, is_k = !is_q && head < p.Hq + p.Hkv;
          if (is_q || is_k) {
            float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
            for (int i = 0; i < 128; i += 2) {
              ss0 = fmaf(__uint_as_float(x[i]), __uint_as_float(x[i]), ss0);
              ss1 = fmaf(__uint_as_float(x[i + 1]), __uint_as_float(x[i + 1]), ss1);
            }
            const float sc = 1.0f / sqrtf((ss0 + ss1) * (1.0f / 128.0f) + p.eps);
            const __nv_bfloat16* w = is_q ? p.qw : p.kw;
            const float4* cr = reinterpret_cast<const float4*>(p.cos_t + (int64_t)s_idx * 64);
            const float4* sr = reinterpret_cast<const float4*>(p.sin_t + (int64_t)s_idx * 64);
#pragma unroll
            for (int g = 0; g < 8; ++g) {   // 8 rotation pairs per step
              const uint4 wa = reinterpret_cast<const uint4*>(w)[g], wb = reinterpret_cast<const uint4*>(w + 64)[g];
              const uint32_t* wau = reinterpret_cast<const uint32_t*>(&wa);
              const uint32_t* wbu = reinterpret_cast<const uint32_t*>(&wb);
              const float4 c0 = cr[2 * g], c1 = cr[2 * g + 1], s0 = sr[2 * g], s1 = sr[2 * g + 1];
              const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
              const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const int i = g * 8 + e;
                const float w1 = (e & 1) ? bf16_hi(wau[e >> 1]) : bf16_lo(wau[e >> 1]);
                const float w2 = (e & 1) ? bf16_hi(wbu[e >> 1]) : bf16_lo(wbu[e >> 1]);
                const float y1 = (__uint_as_float(x[i]) * sc) * w1;
                const float y2 = (__uint_as_float(x[i + 64]) * sc) * w2;
                x[i] = __float_as_uint(y1 * cc[e] - y2 * sn[e]);
                x[i + 64] = __float_as_uint(y2 * cc[e] + y1 * sn[e]);
              }
            }
          }
          __nv_bfloat16* dst;
          if (is_q) {
            dst = p.q_out + ((int64_t)row * p.Hq + head) * 128;
          } else {
            const int hk = is_k ? head - p.Hq : head - p.Hq - p.Hkv;
            dst = (is_k ? p.k_cache : p.v_cache) + (int64_t)b_idx * p.kc_b + (int64_t)hk * p.kc_h + (int64_t)(p.pos0 + s_idx) * p.kc_s;
          }
          if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              uint32_t v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) v[e] = pack_bf16(__uint_as_float(x[g * 16 + 2 * e]), __uint_as_float(x[g * 16 + 2 * e + 1]));
              st_global_v8(dst + g * 16, v);
            }
          } else {
#pragma unroll
            for (int g = 0; g < 16; ++g)
              reinterpret_cast<uint4*>(dst)[g] = make_uint4(pack_bf16(__uint_as_float(x[g * 8 + 0]), __uint_as_float(x[g * 8 + 1])),
                                                            pack_bf16(__uint_as_float(x[g * 8 + 2]), __uint_as_float(x[g * 8 + 3])),
                                                            pack_bf16(__uint_as_float(x[g * 8 + 4]), __uint_as_float(x[g * 8 + 5])),
                                                            pack_bf16(__uint_as_float(x[g * 8 + 6]), __uint_as_float(x[g * 8 + 7])));
          }
        }
      } else if (p.epi == 2) {
        // SiLU(gate) * up.  Weight rows interleave 16 gate rows with the 16 matching up rows, so each
        // 32-column chunk of the accumulator holds 16 (gate, up) pairs and yields 16 outputs.
        __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(p.out) + (int64_t)row * p.ldo + (int64_t)n_tile * (BLOCK_N / 2);
        auto process = [&](uint32_t (&r)[32], const int c0) {
          const int col = n_tile * (BLOCK_N / 2) + c0 / 2;
          if (row_ok && col + 16 <= p.N / 2) {
            uint32_t o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float a0 = silu_f(__uint_as_float(r[2 * e])) * __uint_as_float(r[16 + 2 * e]);
              const float a1 = silu_f(__uint_as_float(r[2 * e + 1])) * __uint_as_float(r[16 + 2 * e + 1]);
              o[e] = pack_bf16(a0, a1);
            }
            if (p.wide_store) {
              st_global_v8(orow + c0 / 2, o);
            } else {
              *reinterpret_cast<uint4*>(orow + c0 / 2) = make_uint4(o[0], o[1], o[2], o[3]);
              *reinterpret_cast<uint4*>(orow + c0 / 2 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
            }
          }
        };
        // same two-buffer schedule as the plain epilogue below
        uint32_t ra[32], rb[32];
        tmem_ld_32x32(t_row, ra);
#pragma unroll 1
        for (int c0 = 0; c0 < BLOCK_N; c0 += 64) {
          tmem_wait_ld();
          tmem_ld_32x32(t_row + c0 + 32, rb);
          process(ra, c0);
          tmem_wait_ld();
          if (c0 + 64 < BLOCK_N) {
            tmem_ld_32x32(t_row + c0 + 64, ra);
          } else {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[acc]);
            released = true;
          }
          process(rb, c0 + 32);
        }
      } else {
        // Two register buffers: the TMEM load of the next 32 columns is in flight while the current
        // 32 are biased, activated, added to the residual, converted and stored; the accumulator is
        // handed back to the MMA warp as soon as its last column has been read.
        auto process = [&](uint32_t (&r)[32], const int c0) {
          if (row_ok) {
            const int col0 = n_tile * BLOCK_N + c0;
            if (p.bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (col0 + j * 8 + 8 <= p.N) {
                  const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col0 + j * 8);
                  const uint32_t* bb = reinterpret_cast<const uint32_t*>(&bv);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    r[j * 8 + 2 * e] = __float_as_uint(__uint_as_float(r[j * 8 + 2 * e]) + bf16_lo(bb[e]));
                    r[j * 8 + 2 * e + 1] = __float_as_uint(__uint_as_float(r[j * 8 + 2 * e + 1]) + bf16_hi(bb[e]));
                  }
                }
              }
            }
            if (p.act == 1) {
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(gelu_f(__uint_as_float(r[i])));
            }
            if (p.epi == 1) {
              if (p.out_f32) {
                const float* rrow = static_cast<const float*>(p.resid) + (int64_t)row * p.ldr + col0;
                if (p.wide_resid && col0 + 32 <= p.N) {
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    uint32_t v[8];
                    ld_global_v8(rrow + j * 8, v);
#pragma unroll
                    for (int e = 0; e < 8; ++e) r[j * 8 + e] = __float_as_uint(__uint_as_float(r[j * 8 + e]) + __uint_as_float(v[e]));
                  }
                } else
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  if (col0 + j * 4 + 4 <= p.N) {
                    const float4 rv = *reinterpret_cast<const float4*>(rrow + j * 4);
                    r[j * 4 + 0] = __float_as_uint(__uint_as_float(r[j * 4 + 0]) + rv.x);
                    r[j * 4 + 1] = __float_as_uint(__uint_as_float(r[j * 4 + 1]) + rv.y);
                    r[j * 4 + 2] = __float_as_uint(__uint_as_float(r[j * 4 + 2]) + rv.z);
                    r[j * 4 + 3] = __float_as_uint(__uint_as_float(r[j * 4 + 3]) + rv.w);
                  }
                }
              } else {
                const __nv_bfloat16* rrow = static_cast<const __nv_bfloat16*>(p.resid) + (int64_t)row * p.ldr + col0;
                if (p.wide_resid && col0 + 32 <= p.N) {
#pragma unroll
                  for (int j = 0; j < 2; ++j) {
                    uint32_t v[8];
                    ld_global_v8(rrow + j * 16, v);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                      r[j * 16 + 2 * e] = __float_as_uint(__uint_as_float(r[j * 16 + 2 * e]) + bf16_lo(v[e]));
                      r[j * 16 + 2 * e + 1] = __float_as_uint(__uint_as_float(r[j * 16 + 2 * e + 1]) + bf16_hi(v[e]));
                    }
                  }
                } else
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (col0 + j * 8 + 8 <= p.N) {
                    const uint4 rv = *reinterpret_cast<const uint4*>(rrow + j * 8);
                    const uint32_t* rr = reinterpret_cast<const uint32_t*>(&rv);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      r[j * 8 + 2 * e] = __float_as_uint(__uint_as_float(r[j * 8 + 2 * e]) + bf16_lo(rr[e]));
                      r[j * 8 + 2 * e + 1] = __float_as_uint(__uint_as_float(r[j * 8 + 2 * e + 1]) + bf16_hi(rr[e]));
                    }
                  }
                }
              }
            }
            if (p.out_f32) {
              float* orow = static_cast<float*>(p.out) + (int64_t)row * p.ldo + col0;
              if (p.wide_f32 && col0 + 32 <= p.N) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint32_t v[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] = r[j * 8 + e];
                  st_global_v8(orow + j * 8, v);
                }
              } else
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (col0 + j * 4 + 4 <= p.N)
                  *reinterpret_cast<float4*>(orow + j * 4) =
                      make_float4(__uint_as_float(r[j * 4]), __uint_as_float(r[j * 4 + 1]), __uint_as_float(r[j * 4 + 2]),
                                  __uint_as_float(r[j * 4 + 3]));
              }
            } else {
              __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(p.out) + (int64_t)row * p.ldo + col0;
              if (p.wide_store && col0 + 32 <= p.N) {
                // 32-byte stores: every store instruction fills whole 32-byte sectors of its 32 rows
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                  uint32_t v[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] = pack_bf16(__uint_as_float(r[j * 16 + 2 * e]), __uint_as_float(r[j * 16 + 2 * e + 1]));
                  st_global_v8(orow + j * 16, v);
                }
              } else
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (col0 + j * 8 + 8 <= p.N) {
                  uint4 v;
                  v.x = pack_bf16(__uint_as_float(r[j * 8 + 0]), __uint_as_float(r[j * 8 + 1]));
                  v.y = pack_bf16(__uint_as_float(r[j * 8 + 2]), __uint_as_float(r[j * 8 + 3]));
                  v.z = pack_bf16(__uint_as_float(r[j * 8 + 4]), __uint_as_float(r[j * 8 + 5]));
                  v.w = pack_bf16(__uint_as_float(r[j * 8 + 6]), __uint_as_float(r[j * 8 + 7]));
                  *reinterpret_cast<uint4*>(orow + j * 8) = v;
                }
              }
            }
          }
        };
        uint32_t ra[32], rb[32];
        tmem_ld_32x32(t_row, ra);
#pragma unroll 1
        for (int c0 = 0; c0 < BLOCK_N; c0 += 64) {
          tmem_wait_ld();
          tmem_ld_32x32(t_row + c0 + 32, rb);
          process(ra, c0);
          tmem_wait_ld();
          if (c0 + 64 < BLOCK_N) {
            tmem_ld_32x32(t_row + c0 + 64, ra);
          } else {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[acc]);
            released = true;
          }
          process(rb, c0 + 32);
        }
      }
      if (!released) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // teardown: every role falls through to here, also after an aborted wait
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BLOCK_N, int STAGES>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p) {
  constexpr int STAGE_BYTES = GEMM_BM * GEMM_BK * 2 + BLOCK_N * GEMM_BK * 2;
  constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
  static bool configured[64] = {false};   // per device: kd_shutdown + kd_init may move the library to another GPU
  if (!configured[ctx().device & 63]) {
    KD_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BLOCK_N, STAGES>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured[ctx().device & 63] = true;
  }
  p.num_m_tiles = (p.M + GEMM_BM - 1) / GEMM_BM;
  p.num_n_tiles = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int total = p.num_m_tiles * p.num_n_tiles;
  const int grid = total < ctx().sm_count ? total : ctx().sm_count;
  gemm_bf16_tcgen05_kernel<BLOCK_N, STAGES><<<grid, GEMM_THREADS, SMEM, ctx().stream>>>(ta, tb, p);
  return after_launch("gemm_bf16_tcgen05_kernel");
}

// out[M, N or N/2] = epilogue(A[M,K] * W[N,K]^T).  Pointers are device pointers; ld* in elements.
int gemm_bf16(const void* A, int64_t lda, const void* W, int64_t ldw, void* out, int64_t ldo, int out_f32,
              const void* resid, int64_t ldr, int M, int N, int K, int epi) {
  return gemm_bf16_bias_act(A, lda, W, ldw, out, ldo, out_f32, resid, ldr, M, N, K, epi, nullptr, 0);
}

int gemm_bf16_bias_act(const void* A, int64_t lda, const void* W, int64_t ldw, void* out, int64_t ldo, int out_f32,
                       const void* resid, int64_t ldr, int M, int N, int K, int epi, const void* bias, int act) {
  KD_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty problem");
  KD_REQUIRE((bias == nullptr && act == 0) || epi == 0 || epi == 1, "gemm: bias / activation combine only with the plain and residual epilogues");
  KD_REQUIRE((reinterpret_cast<uintptr_t>(bias) & 15) == 0, "gemm: bias must be 16-byte aligned");
  KD_REQUIRE(K % 8 == 0, "gemm: K=%d must be a multiple of 8 for the tensor-core path", K);
  const int n_out = epi == 2 ? N / 2 : N;
  KD_REQUIRE(n_out % 8 == 0 && ldo % (out_f32 ? 4 : 8) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
             "gemm: output width / leading dimension / address not 16-byte aligned");
  if (epi == 1)
    KD_REQUIRE(resid != nullptr && ldr % (out_f32 ? 4 : 8) == 0 && (reinterpret_cast<uintptr_t>(resid) & 15) == 0,
               "gemm: residual operand must be 16-byte aligned");
  if (epi == 2) KD_REQUIRE(N % 32 == 0 && !out_f32, "gemm: SwiGLU epilogue needs N %% 32 == 0 and a bf16 output");
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.out_f32 = out_f32;
  p.resid = resid; p.ldr = ldr;
  p.epi = epi;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.act = act;
  p.wide_store = !out_f32 && ldo % 16 == 0 && (reinterpret_cast<uintptr_t>(out) & 31) == 0;
  p.wide_f32 = out_f32 && ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 31) == 0;
  p.wide_resid = resid != nullptr && ldr % (out_f32 ? 8 : 16) == 0 && (reinterpret_cast<uintptr_t>(resid) & 31) == 0;
  p.err = ctx().error_flag;
  CUtensorMap ta, tb;
  KD_TRY(make_tmap_bf16_2d(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, GEMM_BM, GEMM_BK));
  if (N >= 256 || epi == 2) {
    KD_TRY(make_tmap_bf16_2d(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 256, GEMM_BK));
    return launch_gemm<256, 4>(ta, tb, p);
  }
  if (N > 64) {
    KD_TRY(make_tmap_bf16_2d(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 128, GEMM_BK));
    return launch_gemm<128, 6>(ta, tb, p);
  }
  KD_TRY(make_tmap_bf16_2d(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 64, GEMM_BK));
  return launch_gemm<64, 8>(ta, tb, p);
}

// QKV projection with the q/k-norm + RoPE + KV-cache write done in the epilogue (head_dim 128).
int gemm_bf16_qkv_rope(const void* A, int64_t lda, const void* W, int64_t ldw, int M, int K, int S, int Hq, int Hkv, int pos0,
                       float eps, const float* cos_t, const float* sin_t, const void* qw, const void* kw, void* q_out,
                       void* k_cache, void* v_cache, int64_t kc_b, int64_t kc_h, int64_t kc_s) {
  KD_REQUIRE(M > 0 && K > 0 && K % 8 == 0, "qkv gemm: K=%d must be a positive multiple of 8", K);
  const int N = (Hq + 2 * Hkv) * 128;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.epi = 3;
  p.err = ctx().error_flag;
  p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.pos0 = pos0; p.eps = eps;
  p.cos_t = cos_t; p.sin_t = sin_t;
  p.qw = static_cast<const __nv_bfloat16*>(qw); p.kw = static_cast<const __nv_bfloat16*>(kw);
  p.q_out = static_cast<__nv_bfloat16*>(q_out);
  p.k_cache = static_cast<__nv_bfloat16*>(k_cache); p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  p.kc_b = kc_b; p.kc_h = kc_h; p.kc_s = kc_s;
  CUtensorMap ta, tb;
  KD_TRY(make_tmap_bf16_2d(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, GEMM_BM, GEMM_BK));
  KD_TRY(make_tmap_bf16_2d(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 256, GEMM_BK));
  return launch_gemm<256, 4>(ta, tb, p);
}

// ----------------------------------------------------------------------------- skinny (decode) GEMM
// y[m, n] = sum_k x[m, k] W[n, k] for a handful of rows m (one per sequence being decoded).  The
// reference runs this through its "skinny" tile of the generic shader
// (packages/backend-webgpu/src/kernels/matrix/tileSelector.ts:57-66,169-203); there is no GEMV path.
//
// The problem is HBM-bound (every weight byte is used once per step), so the kernel is organised
// around streaming W: the operands are swapped, W rows become the M dimension of the MMA (128 rows
// per CTA, all of them useful) and the few activation rows become the N dimension (16..128).  Each
// stage then carries 16 KB of weights and only a few KB of activations, and a deep TMA ring keeps
// ~100+ KB of weight traffic in flight per SM.  When N/128 gives too few CTAs the K range is split
// across CTAs; every split writes fp32 partial sums [split][m][n], which the consumer kernels
// (norm+RoPE, SwiGLU, residual+RMSNorm) add up while they do their own work.
// Roofline: HBM, N*K*2 bytes of weights per call.
struct SkinnyParams {
  int Mb, N, K;
  int mb_pad;             // MMA N extent: multiple of 16 covering Mb
  int x_box;              // rows of the activation TMA box (smem rows per stage)
  int splits, kblocks_per_split, stages;
  uint32_t tmem_cols;
  float* out_f32;         // [splits][Mb][N]
  __nv_bfloat16* out_bf16;  // [Mb][N] (or [Mb][N/2] with the SiLU*up epilogue), only with splits == 1
  int swiglu;             // rows of W interleave 16 gate / 16 up rows: write silu(gate)*up
  int* err;
};

__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_skinny_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                           SkinnyParams p) {
  constexpr int W_BYTES = 128 * GEMM_BK * 2;
  const int x_bytes = p.x_box * GEMM_BK * 2;
  const int stage_bytes = W_BYTES + x_bytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_full = empty + p.stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x, split = blockIdx.y;
  const int total_kb = (p.K + GEMM_BK - 1) / GEMM_BK;
  const int kb_begin = split * p.kblocks_per_split;
  const int kb_end = min(total_kb, kb_begin + p.kblocks_per_split);
  const int n_kb = max(0, kb_end - kb_begin);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_w);
    prefetch_tmap(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();      // nothing above touches global memory
  pdl_trigger();   // after the TMEM allocation (see common.cuh)

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < n_kb; ++i) {
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.err, 211)) break;
        uint8_t* sw = smem + stage * stage_bytes;
        mbar_arrive_expect_tx(&full[stage], (uint32_t)stage_bytes);
        tma_load_2d(sw, &tmap_w, &full[stage], (kb_begin + i) * GEMM_BK, n_tile * 128);
        tma_load_2d(sw + W_BYTES, &tmap_x, &full[stage], (kb_begin + i) * GEMM_BK, 0);
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(128, p.mb_pad, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < n_kb; ++i) {
        if (!mbar_wait(&full[stage], phase, abort_flag, p.err, 212)) { ok = false; break; }
        tc_fence_after();
        const uint32_t w_addr = smem_u32(smem + stage * stage_bytes);
        const uint32_t x_addr = w_addr + W_BYTES;
#pragma unroll
        for (int k = 0; k < GEMM_BK / 16; ++k)
          umma_ss(tmem_base, make_smem_desc_sw128(w_addr + k * 32, 16, 1024), make_smem_desc_sw128(x_addr + k * 32, 16, 1024),
                  idesc, (i | k) != 0 ? 1u : 0u);
        umma_commit(&empty[stage]);
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    const int q = warp & 3;
    bool ok = true;
    if (n_kb > 0) {
      ok = mbar_wait(acc_full, 0, abort_flag, p.err, 213);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const int n = n_tile * 128 + q * 32 + lane;
      const bool n_ok = n < p.N;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
      for (int c0 = 0; c0 < p.mb_pad; c0 += 16) {
        uint32_t r[16];
        if (n_kb > 0) {
          tmem_ld_32x16(t_row + c0, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = 0u;
        }
        if (p.swiglu) {
          // lanes 0-15 of a warp hold 16 gate rows, lanes 16-31 the matching up rows
          const int j = (n_tile * 128 + q * 32) / 2 + (lane & 15);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float mine = __uint_as_float(r[i]);
            const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
            const int m = c0 + i;
            if (lane < 16 && m < p.Mb && j < p.N / 2)
              p.out_bf16[(int64_t)m * (p.N / 2) + j] = __float2bfloat16_rn(silu_f(mine) * other);
          }
        } else if (n_ok) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int m = c0 + i;
            if (m < p.Mb) {
              if (p.out_bf16) p.out_bf16[(int64_t)m * p.N + n] = __float2bfloat16_rn(__uint_as_float(r[i]));
              else p.out_f32[((int64_t)split * p.Mb + m) * p.N + n] = __uint_as_float(r[i]);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

// Picks the split-K factor for a skinny GEMM.  One CTA streams its 128 weight rows at roughly
// 100 GB/s, so about 40 CTAs already saturate HBM; beyond that more splits only add partial-sum
// traffic.  Each split keeps at least 8 k-blocks (128 KB of weights).
int gemm_skinny_auto_splits(int N, int K) {
  const int tiles = (N + 127) / 128;
  const int total_kb = (K + GEMM_BK - 1) / GEMM_BK;
  int splits = (40 + tiles - 1) / tiles;
  if (splits > total_kb / 8) splits = total_kb / 8;
  if (splits < 1) splits = 1;
  return splits;
}

// x [Mb<=128, K] bf16, W [N, K] bf16 -> fp32 partials [splits][Mb][N] (or bf16 [Mb][N] when
// out_bf16 != NULL and splits == 1).
int gemm_bf16_skinny(const void* x, int64_t ldx, const void* W, int64_t ldw, int Mb, int N, int K, int splits,
                     float* out_f32, void* out_bf16, int swiglu) {
  KD_REQUIRE(Mb >= 1 && Mb <= 128, "skinny gemm: %d rows; this path handles 1..128", Mb);
  KD_REQUIRE(N > 0 && K > 0 && K % 8 == 0, "skinny gemm: K=%d must be a positive multiple of 8", K);
  KD_REQUIRE(splits >= 1, "skinny gemm: splits must be >= 1");
  KD_REQUIRE(out_bf16 == nullptr || splits == 1, "skinny gemm: bf16 output needs splits == 1");
  KD_REQUIRE(!swiglu || (out_bf16 != nullptr && N % 32 == 0), "skinny gemm: the SiLU*up epilogue needs a bf16 output and N %% 32 == 0");
  SkinnyParams p{};
  p.Mb = Mb; p.N = N; p.K = K;
  p.mb_pad = (Mb + 15) / 16 * 16;
  p.x_box = p.mb_pad <= 32 ? 32 : (p.mb_pad <= 64 ? 64 : 128);
  const int total_kb = (K + GEMM_BK - 1) / GEMM_BK;
  if (splits > total_kb) splits = total_kb;
  p.kblocks_per_split = (total_kb + splits - 1) / splits;
  p.splits = splits;
  const int stage_bytes = 128 * GEMM_BK * 2 + p.x_box * GEMM_BK * 2;
  int stages = (200 * 1024) / stage_bytes;
  if (stages > 10) stages = 10;
  if (stages > p.kblocks_per_split) stages = p.kblocks_per_split < 2 ? 2 : p.kblocks_per_split;
  // many tiles (lm_head): a shallower ring lets two CTAs share an SM, so that one CTA's prologue and
  // epilogue overlap the other's streaming
  if ((int64_t)((N + 127) / 128) * splits >= 2 * ctx().sm_count) {
    const int two_per_sm = (108 * 1024) / stage_bytes;
    if (stages > two_per_sm) stages = two_per_sm;
  }
  p.stages = stages;
  p.tmem_cols = p.mb_pad <= 32 ? 32 : (p.mb_pad <= 64 ? 64 : 128);
  p.out_f32 = out_f32;
  p.out_bf16 = static_cast<__nv_bfloat16*>(out_bf16);
  p.swiglu = swiglu;
  p.err = ctx().error_flag;
  CUtensorMap tw, tx;
  KD_TRY(make_tmap_bf16_2d(&tw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 128, GEMM_BK));
  KD_TRY(make_tmap_bf16_2d(&tx, x, (uint64_t)Mb, (uint64_t)K, (uint64_t)ldx, (uint32_t)p.x_box, GEMM_BK));
  const int smem = stages * stage_bytes + 1024 + 256;
  static bool skinny_configured[64] = {false};   // per device
  if (!skinny_configured[ctx().device & 63]) {
    KD_CUDA_CHECK(cudaFuncSetAttribute(gemm_skinny_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    skinny_configured[ctx().device & 63] = true;
  }
  dim3 grid((N + 127) / 128, splits);
  KD_CUDA_CHECK(launch_ex(gemm_skinny_tcgen05_kernel, grid, dim3(GEMM_THREADS), (size_t)smem, tw, tx, p));
  return after_launch("gemm_skinny_tcgen05_kernel");
}

// ----------------------------------------------------------------------------- dispatch from kd_matmul
int matmul_tc_try(const kd_matmul_cfg* cfg, const kd_tensor* a, const kd_tensor* b, const kd_tensor* c,
                  const kd_tensor* out, int* handled) {
  *handled = 0;
  if (a->dtype != KD_BF16 || b->dtype != KD_BF16) return KD_OK;
  if (out->dtype != KD_BF16 && out->dtype != KD_F32) return KD_OK;
  if (cfg->alpha != 1.0f) return KD_OK;
  if (a->ndim < 2 || b->ndim != 2 || !is_contiguous(out)) return KD_OK;
  // A must be logically [rows..., K] with unit K stride and collapsible leading dims.
  if (cfg->transpose_a) return KD_OK;
  if (a->strides[a->ndim - 1] != 1 && a->shape[a->ndim - 1] != 1) return KD_OK;
  int64_t lda = a->strides[a->ndim - 2];
  int64_t rows = a->shape[a->ndim - 2];
  for (int d = a->ndim - 3; d >= 0; --d) {
    if (a->shape[d] != 1 && a->strides[d] != lda * rows) return KD_OK;
    rows *= a->shape[d];
  }
  // W must be K-major: stored [N,K] with transposeB, or a [K,N] view with strides [1, ld].
  int64_t ldw;
  if (cfg->transpose_b) {
    if (b->strides[1] != 1) return KD_OK;
    ldw = b->strides[0];
  } else {
    if (b->strides[0] != 1) return KD_OK;
    ldw = b->strides[1];
  }
  const int64_t M = rows, N = cfg->N, K = cfg->K;
  if (M <= 0 || N <= 0 || K <= 0 || M > 0x7fffffff) return KD_OK;
  if (K % 8 || N % 8 || lda % 8 || ldw % 8) return KD_OK;
  int epi = 0;
  void* pc = nullptr;
  if (cfg->has_c && c != nullptr && cfg->beta != 0.f) {
    if (cfg->beta != 1.0f || c->dtype != out->dtype || !is_contiguous(c) || numel(c) != M * N) return KD_OK;
    KD_TRY(tensor_ptr(c, &pc));
    epi = 1;
  }
  void *pa = nullptr, *pb = nullptr, *po = nullptr;
  KD_TRY(tensor_ptr(a, &pa));
  KD_TRY(tensor_ptr(b, &pb));
  KD_TRY(tensor_ptr(out, &po));
  if ((reinterpret_cast<uintptr_t>(pa) | reinterpret_cast<uintptr_t>(pb) | reinterpret_cast<uintptr_t>(po)) & 15) return KD_OK;
  if (pc && (reinterpret_cast<uintptr_t>(pc) & 15)) return KD_OK;
  KD_TRY(gemm_bf16(pa, lda, pb, ldw, po, N, out->dtype == KD_F32, pc, N, (int)M, (int)N, (int)K, epi));
  *handled = 1;
  return KD_OK;
}

}  // namespace kd
