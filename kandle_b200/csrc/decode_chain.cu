// One persistent kernel for everything a decoder layer does between two attention calls of a
// decode step (one new token per sequence):
//
//   G0  o_proj         p0[s]   = attn  Wo^T          (split-K, fp32 partial sums)
//   N0  add + RMSNorm  h1 = h + sum_s p0[s];  x = rmsnorm(h1) * w_post
//   G1  gate/up        act     = silu(x Wg^T) * (x Wu^T)   (rows of Wgu interleaved 16/16)
//   G2  down           p2[s]   = act  Wd^T            (split-K)
//   N1  add + RMSNorm  h = h1 + sum_s p2[s];  x = rmsnorm(h) * w_next
//   G3  next layer's QKV   qkv[s] = x  Wqkv^T        (split-K partials; absent after the last layer)
//
// which is the reference's `o_proj`, residual add, `post_attention_layernorm`, SwiGLU MLP, residual
// add and the next layer's `input_layernorm` + q/k/v projections
// (packages/model-utils/src/qwen3/decoder_layer.ts:191-241, attention/gqa.ts:246-290,
// mlp/swiglu.ts:119-134).  Run as six kernels these steps cost ~6 us each although every one of them
// moves only 2-12 MB: launch latency, pipeline fill and the tail dominate.  Here they are phases of
// one cooperative launch (one CTA per SM, all co-resident) separated by grid-wide counters in
// global memory instead of kernel boundaries, and -- the point of the exercise -- the weight
// stream does not stop at a phase boundary: weights depend on nothing, so the TMA producer of a CTA
// runs ahead into its next unit's weight tiles while the activations that unit needs are still
// being produced elsewhere.
//
// Every GEMM is the swapped skinny form of gemm_tcgen05.cu: D[128 weight rows, tokens] =
// W_tile[128, K_chunk] * X[tokens, K_chunk]^T on tcgen05 with the accumulator in TMEM (two
// buffers).  A phase's work is cut into units (one 128-row weight tile x one K split); unit u of a
// phase runs on CTA (u + rot) mod gridDim, `rot` chosen per phase so that CTAs that idle in one
// phase own work (and prefetch its weights) in the next.
//
//   warp 0     TMA producer (weights early, activations once the phase they come from is complete)
//   warp 1     tcgen05.mma issuer
//   warps 2-5  epilogues (TMEM -> global), the add+RMSNorm phases, and the phase counters
//
// Grid-wide ordering: after its part of phase p a CTA does fence + red.release on counter p; a
// consumer spins (bounded, ~1 s, then error 5xx and the CTA drains) on ld.acquire until the counter
// reaches gridDim.  The last CTA to leave zeroes the counters for the next launch.
// Roofline: HBM, the bytes of the four weight matrices per launch.
#include "chain_common.cuh"
#include "common.cuh"
#include "kernels.cuh"
#include "sm100.cuh"

namespace kd {

using namespace sm100;

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                      uint32_t box_rows, uint32_t box_cols);

constexpr int CH_BK = 64;                       // K elements per stage (one 128-byte swizzle atom)
constexpr int CH_W_BYTES = 128 * CH_BK * 2;     // weight tile bytes per stage
constexpr int CH_THREADS = 192;
constexpr int CH_PHASES = 6;
constexpr int CH_MAXV = 4;                      // 8-element vectors per thread in the norm phases

struct ChainGemm {
  int N, K;                   // weight matrix [N, K]
  int splits, kb_per_split;
  int rot;                    // unit u runs on CTA (u + rot) % gridDim.x
  int swiglu;                 // bf16 [Mb, N/2] output with the SiLU*up epilogue (splits == 1)
  float* out_f32;             // [splits][Mb][N]
  __nv_bfloat16* out_bf16;
};

struct ChainNorm {
  const float* partials;      // [splits][Mb][H]
  int splits;
  int rot;                    // row r runs on CTA (r + rot) % gridDim.x
  const float* resid_in;      // [Mb][H]
  float* resid_out;           // [Mb][H]
  const __nv_bfloat16* w;     // [H]
  __nv_bfloat16* x_out;       // [Mb][H]
};

struct ChainParams {
  int Mb, mb_pad, x_box, stages, H;
  int n_phases;               // 5 (no QKV phase) or 6
  uint32_t acc_cols;          // TMEM columns per accumulator buffer
  float eps;
  ChainGemm g[4];
  ChainNorm n[2];
  unsigned* counters;         // [8]: one per phase, [7] = exit ticket
  int* err;
};

struct ChainMaps {
  CUtensorMap w[4];
  CUtensorMap x[4];
};

// phase p: 0 G0, 1 N0, 2 G1, 3 G2, 4 N1, 5 G3
__device__ __forceinline__ int phase_gemm_index(int p) { return p == 0 ? 0 : (p == 2 ? 1 : (p == 3 ? 2 : (p == 5 ? 3 : -1))); }

__global__ void __launch_bounds__(CH_THREADS, 1)
decode_chain_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainParams p) {
  const int x_bytes = p.x_box * CH_BK * 2;
  const int stage_bytes = CH_W_BYTES + x_bytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_full = empty + p.stages;     // 2
  uint64_t* acc_empty = acc_full + 2;        // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red = reinterpret_cast<float*>(tmem_slot + 2);   // 4 floats
  __nv_bfloat16* epi_stage = reinterpret_cast<__nv_bfloat16*>(tmem_slot + 8);   // 4 warps x [32 tokens][16] bf16

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  const unsigned target = (unsigned)G;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 4); }
    *abort_flag = 0;
    fence_mbar_init();
    for (int i = 0; i < 4; ++i) {
      if (i == 3 && p.n_phases < CH_PHASES) break;
      prefetch_tmap(&maps.w[i]);
      prefetch_tmap(&maps.x[i]);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * p.acc_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t ring_phase = 0;
      bool ok = true;
      for (int ph = 0; ok && ph < p.n_phases; ++ph) {
        const int gi = phase_gemm_index(ph);
        if (gi < 0) continue;
        const ChainGemm& g = p.g[gi];
        const int tiles = (g.N + 127) / 128;
        const int units = tiles * g.splits;
        const int total_kb = (g.K + CH_BK - 1) / CH_BK;
        bool dep_ready = (ph == 0);
        for (int u = (cta - g.rot % G + G) % G; ok && u < units; u += G) {
          const int tile = u % tiles, split = u / tiles;
          const int kb0 = split * g.kb_per_split;
          const int n_kb = max(0, min(total_kb, kb0 + g.kb_per_split) - kb0);
          int i = 0;
          if (!dep_ready) {
            // weights first, as far as the ring reaches; their activations follow once they exist
            const int pre = min(n_kb, p.stages);
            const int stage0 = stage;
            for (; i < pre; ++i) {
              if (!mbar_wait(&empty[stage], ring_phase ^ 1, abort_flag, p.err, 501)) { ok = false; break; }
              mbar_arrive_expect_tx(&full[stage], (uint32_t)stage_bytes);
              tma_load_2d(smem + stage * stage_bytes, &maps.w[gi], &full[stage], (kb0 + i) * CH_BK, tile * 128);
              if (++stage == p.stages) { stage = 0; ring_phase ^= 1; }
            }
            if (!ok) break;
            if (!counter_wait(p.counters + (ph - 1), target, abort_flag, p.err, 502)) { ok = false; break; }
            // the activations were written through the generic proxy by other SMs; TMA reads them
            // through the async proxy
            asm volatile("fence.proxy.async;" ::: "memory");
            dep_ready = true;
            for (int t = 0; t < pre; ++t) {
              const int st = (stage0 + t) % p.stages;
              tma_load_2d(smem + st * stage_bytes + CH_W_BYTES, &maps.x[gi], &full[st], (kb0 + t) * CH_BK, 0);
            }
          }
          for (; i < n_kb; ++i) {
            if (!mbar_wait(&empty[stage], ring_phase ^ 1, abort_flag, p.err, 503)) { ok = false; break; }
            mbar_arrive_expect_tx(&full[stage], (uint32_t)stage_bytes);
            tma_load_2d(smem + stage * stage_bytes, &maps.w[gi], &full[stage], (kb0 + i) * CH_BK, tile * 128);
            tma_load_2d(smem + stage * stage_bytes + CH_W_BYTES, &maps.x[gi], &full[stage], (kb0 + i) * CH_BK, 0);
            if (++stage == p.stages) { stage = 0; ring_phase ^= 1; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(128, p.mb_pad, 0, 0);
      int stage = 0;
      uint32_t ring_phase = 0;
      int acc_n = 0;
      bool ok = true;
      for (int ph = 0; ok && ph < p.n_phases; ++ph) {
        const int gi = phase_gemm_index(ph);
        if (gi < 0) continue;
        const ChainGemm& g = p.g[gi];
        const int tiles = (g.N + 127) / 128;
        const int units = tiles * g.splits;
        const int total_kb = (g.K + CH_BK - 1) / CH_BK;
        for (int u = (cta - g.rot % G + G) % G; ok && u < units; u += G) {
          const int split = u / tiles;
          const int kb0 = split * g.kb_per_split;
          const int n_kb = max(0, min(total_kb, kb0 + g.kb_per_split) - kb0);
          const int buf = acc_n & 1, use = acc_n >> 1;
          if (!mbar_wait(&acc_empty[buf], (uint32_t)((use & 1) ^ 1), abort_flag, p.err, 504)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)buf * p.acc_cols;
          for (int i = 0; i < n_kb; ++i) {
            if (!mbar_wait(&full[stage], ring_phase, abort_flag, p.err, 505)) { ok = false; break; }
            tc_fence_after();
            const uint32_t w_addr = smem_u32(smem + stage * stage_bytes);
            const uint32_t x_addr = w_addr + CH_W_BYTES;
#pragma unroll
            for (int k = 0; k < CH_BK / 16; ++k)
              umma_ss(d_tmem, make_smem_desc_sw128(w_addr + k * 32, 16, 1024), make_smem_desc_sw128(x_addr + k * 32, 16, 1024),
                      idesc, (i | k) != 0 ? 1u : 0u);
            umma_commit(&empty[stage]);
            if (++stage == p.stages) { stage = 0; ring_phase ^= 1; }
          }
          if (!ok) break;
          umma_commit(&acc_full[buf]);
          ++acc_n;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogues, norm phases, counters
    const int q = warp & 3;
    const int et = q * 32 + lane;           // 0..127 (TMEM lane of this thread)
    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
    int acc_n = 0;
    bool ok = true;
    // Control flow between the 128-thread barriers below must not depend on `ok`: a warp that gave
    // up still walks through every phase (skipping the GEMM epilogues) so that nobody waits at a
    // barrier for it.
    for (int ph = 0; ph < p.n_phases; ++ph) {
      const int gi = phase_gemm_index(ph);
      if (gi >= 0) {
        const ChainGemm& g = p.g[gi];
        const int tiles = (g.N + 127) / 128;
        const int units = tiles * g.splits;
        const int total_kb = (g.K + CH_BK - 1) / CH_BK;
        for (int u = (cta - g.rot % G + G) % G; ok && u < units; u += G) {
          const int tile = u % tiles, split = u / tiles;
          const int kb0 = split * g.kb_per_split;
          const int n_kb = max(0, min(total_kb, kb0 + g.kb_per_split) - kb0);
          const int buf = acc_n & 1, use = acc_n >> 1;
          ok = mbar_wait(&acc_full[buf], (uint32_t)(use & 1), abort_flag, p.err, 506);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          const int n = tile * 128 + et;
          const uint32_t t_acc = t_row + (uint32_t)buf * p.acc_cols;
          for (int c0 = 0; c0 < p.mb_pad; c0 += 16) {
            uint32_t r[16];
            if (n_kb > 0) {
              tmem_ld_32x16(t_acc + c0, r);
              tmem_wait_ld();
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) r[i] = 0u;
            }
            if (g.swiglu) {
              // lanes 0-15 of a warp hold 16 gate rows, lanes 16-31 the matching up rows: 16 outputs
              // j per token m.  They go through shared memory so that each lane stores one token's
              // 32 contiguous bytes instead of 16 two-byte stores.
              // Branch-free and in three passes (exchange, arithmetic, store): with one warp per
              // scheduler nothing else hides the latency of a shuffle -> exp -> divide chain.
              __nv_bfloat16* stg = epi_stage + q * (32 * 16);
              float other[16], val[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) other[i] = __shfl_xor_sync(0xffffffffu, __uint_as_float(r[i]), 16);
#pragma unroll
              for (int i = 0; i < 16; ++i) val[i] = chain_silu(__uint_as_float(r[i])) * other[i];   // meaningful in lanes 0-15
              if (lane < 16) {
#pragma unroll
                for (int i = 0; i < 16; ++i) stg[((c0 + i) & 31) * 16 + lane] = __float2bfloat16_rn(val[i]);
              }
              if (c0 + 16 >= p.mb_pad || ((c0 + 16) & 31) == 0) {
                // a group of up to 32 tokens is staged: flush it, one token per lane
                __syncwarp();
                const int m = (c0 & ~31) + lane;
                const int j0 = (tile * 128 + q * 32) / 2;
                if (m < p.Mb && j0 + 16 <= g.N / 2) {
                  const uint4* src = reinterpret_cast<const uint4*>(stg + (lane) * 16);
                  uint4* dst = reinterpret_cast<uint4*>(g.out_bf16 + (int64_t)m * (g.N / 2) + j0);
                  dst[0] = src[0];
                  dst[1] = src[1];
                }
                __syncwarp();
              }
            } else if (n < g.N) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int m = c0 + i;
                if (m < p.Mb) g.out_f32[((int64_t)split * p.Mb + m) * g.N + n] = __uint_as_float(r[i]);
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
          ++acc_n;
        }
      } else {
        const ChainNorm& nm = p.n[ph == 1 ? 0 : 1];
        const int nvec = p.H / 8;
        bool waited = false;
        for (int row = (cta - nm.rot % G + G) % G; row < p.Mb; row += G) {
          if (!waited) {
            // the partial sums of the preceding GEMM phase must be complete (after a failed wait the
            // row is still computed, from whatever is there: the launch has already reported an error)
            if (et == 0) counter_wait(p.counters + (ph - 1), target, abort_flag, p.err, 507);
            epi_bar_sync();
            waited = true;
          }
          float v[CH_MAXV][8];
          float ss = 0.f;
#pragma unroll
          for (int t = 0; t < CH_MAXV; ++t) {
            const int vi = et + t * 128;
            if (vi < nvec) {
#pragma unroll
              for (int e = 0; e < 8; ++e) v[t][e] = 0.f;
              // four splits per round: eight independent 16-byte loads in flight per thread
              const float4* s0 = reinterpret_cast<const float4*>(nm.partials + (int64_t)row * p.H) + vi * 2;
              const int64_t sstride = (int64_t)p.Mb * p.H / 4;   // float4 between consecutive splits
              for (int sp = 0; sp < nm.splits; sp += 4) {
                float4 a[4], b[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  if (sp + u < nm.splits) {
                    a[u] = __ldcg(s0 + (sp + u) * sstride);
                    b[u] = __ldcg(s0 + (sp + u) * sstride + 1);
                  } else {
                    a[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    b[u] = a[u];
                  }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  v[t][0] += a[u].x; v[t][1] += a[u].y; v[t][2] += a[u].z; v[t][3] += a[u].w;
                  v[t][4] += b[u].x; v[t][5] += b[u].y; v[t][6] += b[u].z; v[t][7] += b[u].w;
                }
              }
              const float4* rp = reinterpret_cast<const float4*>(nm.resid_in + (int64_t)row * p.H) + vi * 2;
              const float4 a = __ldcg(rp), b = __ldcg(rp + 1);
              v[t][0] += a.x; v[t][1] += a.y; v[t][2] += a.z; v[t][3] += a.w;
              v[t][4] += b.x; v[t][5] += b.y; v[t][6] += b.z; v[t][7] += b.w;
              float4* so = reinterpret_cast<float4*>(nm.resid_out + (int64_t)row * p.H) + vi * 2;
              so[0] = make_float4(v[t][0], v[t][1], v[t][2], v[t][3]);
              so[1] = make_float4(v[t][4], v[t][5], v[t][6], v[t][7]);
#pragma unroll
              for (int e = 0; e < 8; ++e) ss += v[t][e] * v[t][e];
            }
          }
          ss = warp_sum(ss);
          epi_bar_sync();                 // `red` of the previous row has been read by everyone
          if (lane == 0) red[q] = ss;
          epi_bar_sync();
          const float tot = red[0] + red[1] + red[2] + red[3];
          const float sc = 1.0f / sqrtf(tot / (float)p.H + p.eps);
#pragma unroll
          for (int t = 0; t < CH_MAXV; ++t) {
            const int vi = et + t * 128;
            if (vi < nvec) {
              const uint4 wu = reinterpret_cast<const uint4*>(nm.w)[vi];
              const __nv_bfloat16* wh = reinterpret_cast<const __nv_bfloat16*>(&wu);
              uint4 o;
              __nv_bfloat16* ho = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
              for (int e = 0; e < 8; ++e) ho[e] = __float2bfloat16_rn(v[t][e] * sc * __bfloat162float(wh[e]));
              reinterpret_cast<uint4*>(nm.x_out + (int64_t)row * p.H)[vi] = o;
            }
          }
        }
      }
      // this CTA's part of phase `ph` is in global memory: publish
      // (the barrier orders the other 127 threads' writes before thread 0's release, which is cumulative)
      epi_bar_sync();
      if (et == 0 && *abort_flag == 0) {
        __threadfence();
        red_release_add(p.counters + ph, 1u);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * p.acc_cols);
  }
  if (threadIdx.x == 0 && *abort_flag == 0) {
    // the last CTA out re-arms the counters for the next launch
    const unsigned ticket = atomicAdd(p.counters + 7, 1u);
    if (ticket == target - 1) {
      for (int i = 0; i < 8; ++i) p.counters[i] = 0u;
      __threadfence();
    }
  }
}

// ----------------------------------------------------------------------------- host side
static unsigned* g_chain_counters[64] = {nullptr};

// Called when a kernel reported an error: a chain kernel that gave up leaves its counters dirty.
int decode_chain_reset_counters() {
  const int dev = ctx().device;
  if (dev >= 0 && dev < 64 && g_chain_counters[dev])
    KD_CUDA_CHECK(cudaMemsetAsync(g_chain_counters[dev], 0, 8 * sizeof(unsigned), ctx().stream));
  return KD_OK;
}

struct ChainOperand { const void* w; int N, K; const void* x; int64_t ldx; };

int decode_chain_launch(int Mb, int H, float eps, const ChainOperand* ops, int n_gemms, const int* splits,
                        float* part0, float* part2, float* qkv_partials, __nv_bfloat16* act, const float* resid_in,
                        float* resid_mid, float* resid_out, const __nv_bfloat16* w_post, const __nv_bfloat16* w_next,
                        __nv_bfloat16* x_out) {
  Context& c = ctx();
  const int dev = c.device;
  KD_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
  if (!g_chain_counters[dev]) {
    KD_CUDA_CHECK(cudaMalloc(&g_chain_counters[dev], 8 * sizeof(unsigned)));
    KD_CUDA_CHECK(cudaMemsetAsync(g_chain_counters[dev], 0, 8 * sizeof(unsigned), c.stream));
  }
  static ChainMaps maps;   // large: keep it off the stack
  ChainParams p{};
  p.Mb = Mb; p.H = H; p.eps = eps;
  p.mb_pad = (Mb + 15) / 16 * 16;
  p.x_box = p.mb_pad <= 32 ? 32 : (p.mb_pad <= 64 ? 64 : 128);
  p.acc_cols = p.mb_pad <= 32 ? 32u : (p.mb_pad <= 64 ? 64u : 128u);
  p.n_phases = n_gemms == 4 ? 6 : 5;
  const int stage_bytes = CH_W_BYTES + p.x_box * CH_BK * 2;
  p.stages = (200 * 1024) / stage_bytes;
  if (p.stages > 10) p.stages = 10;
  p.counters = g_chain_counters[dev];
  p.err = c.error_flag;
  const int G = c.sm_count;
  for (int i = 0; i < n_gemms; ++i) {
    ChainGemm& g = p.g[i];
    g.N = ops[i].N; g.K = ops[i].K;
    const int total_kb = (g.K + CH_BK - 1) / CH_BK;
    int s = splits[i] < 1 ? 1 : splits[i];
    if (s > total_kb) s = total_kb;
    g.kb_per_split = (total_kb + s - 1) / s;
    g.splits = (total_kb + g.kb_per_split - 1) / g.kb_per_split;
    KD_REQUIRE(g.splits == splits[i], "split factor %d of GEMM %d leaves a split without work", splits[i], i);
    KD_TRY(make_tmap_bf16_2d(&maps.w[i], ops[i].w, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.K, 128, CH_BK));
    KD_TRY(make_tmap_bf16_2d(&maps.x[i], ops[i].x, (uint64_t)Mb, (uint64_t)g.K, (uint64_t)ops[i].ldx, (uint32_t)p.x_box, CH_BK));
  }
  if (n_gemms < 4) { maps.w[3] = maps.w[0]; maps.x[3] = maps.x[0]; }
  p.g[0].out_f32 = part0;
  p.g[1].swiglu = 1; p.g[1].out_bf16 = act;
  p.g[2].out_f32 = part2;
  if (n_gemms == 4) p.g[3].out_f32 = qkv_partials;
  // Rotations: the gate/up units (few, long) go to the highest CTAs, which have no o_proj unit when
  // there are fewer units than CTAs, so their weight prefetch starts at once.
  auto units = [&](int i) { return ((p.g[i].N + 127) / 128) * p.g[i].splits; };
  p.g[0].rot = 0;
  p.g[1].rot = (G - units(1) % G) % G;
  p.g[2].rot = 0;
  if (n_gemms == 4) p.g[3].rot = (G - units(3) % G) % G;
  p.n[0] = ChainNorm{part0, p.g[0].splits, 0, resid_in, resid_mid, w_post, x_out};
  p.n[1] = ChainNorm{part2, p.g[2].splits, 0, resid_mid, resid_out, w_next, x_out};
  const int smem = p.stages * stage_bytes + 1024 + 256 + 4096;
  static bool configured[64] = {false};   // per device: kd_shutdown + kd_init may move the library to another GPU
  if (!configured[ctx().device & 63]) {
    KD_CUDA_CHECK(cudaFuncSetAttribute(decode_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    configured[ctx().device & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G);
  cfg.blockDim = dim3(CH_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = c.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // all CTAs co-resident, or the launch fails
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;

  KD_CUDA_CHECK(cudaLaunchKernelEx(&cfg, decode_chain_kernel, maps, p));
  return after_launch("decode_chain_kernel");
}

}  // namespace kd

using namespace kd;

static bool chain_bf16_2d(const kd_tensor* t, int64_t rows, int64_t cols) {
  return t && t->dtype == KD_BF16 && t->ndim == 2 && t->shape[0] == rows && t->shape[1] == cols && t->strides[1] == 1 &&
         t->strides[0] % 8 == 0;
}
static bool chain_f32_rows(const kd_tensor* t, int64_t rows, int64_t cols) {
  return t && t->dtype == KD_F32 && is_contiguous(t) && numel(t) == rows * cols;
}

KD_API int kd_decode_layer_chain(const kd_tensor* attn, const kd_tensor* w_o, const kd_tensor* resid_in,
                                 const kd_tensor* post_norm_w, const kd_tensor* w_gate_up, const kd_tensor* w_down,
                                 const kd_tensor* next_norm_w, float eps, const kd_tensor* w_qkv_next,
                                 const kd_tensor* resid_mid, const kd_tensor* resid_out, const kd_tensor* x_out,
                                 const kd_tensor* act, const kd_tensor* qkv_partials) {
  KD_TRY(require_init());
  KD_REQUIRE(attn && w_o && resid_in && post_norm_w && w_gate_up && w_down && next_norm_w && resid_mid && resid_out && x_out && act,
             "null tensor");
  KD_REQUIRE(attn->ndim == 2 && w_o->ndim == 2 && w_gate_up->ndim == 2 && w_down->ndim == 2, "operands must be 2-D");
  const int64_t Mb = attn->shape[0], Ko = attn->shape[1], H = w_o->shape[0], I2 = w_gate_up->shape[0], I = I2 / 2;
  KD_REQUIRE(Mb >= 1 && Mb <= 128, "%lld sequences; this path handles 1..128", (long long)Mb);
  KD_REQUIRE(Mb <= ctx().sm_count, "more sequences than SMs");
  KD_REQUIRE(H % 8 == 0 && H <= 8 * 128 * CH_MAXV, "hidden size %lld must be a multiple of 8 and at most %d", (long long)H, 8 * 128 * CH_MAXV);
  KD_REQUIRE(I2 % 32 == 0, "gate/up rows must be a multiple of 32");
  KD_REQUIRE(chain_bf16_2d(attn, Mb, Ko) && chain_bf16_2d(w_o, H, Ko) && is_contiguous(w_o), "attn [Mb,Ko] / w_o [H,Ko] must be bf16");
  KD_REQUIRE(chain_bf16_2d(w_gate_up, I2, H) && is_contiguous(w_gate_up) && chain_bf16_2d(w_down, H, I) && is_contiguous(w_down),
             "w_gate_up [2I,H] / w_down [H,I] must be contiguous bf16");
  KD_REQUIRE(chain_bf16_2d(x_out, Mb, H) && is_contiguous(x_out) && chain_bf16_2d(act, Mb, I) && is_contiguous(act),
             "x_out [Mb,H] / act [Mb,I] must be contiguous bf16");
  KD_REQUIRE(chain_f32_rows(resid_in, Mb, H) && chain_f32_rows(resid_mid, Mb, H) && chain_f32_rows(resid_out, Mb, H),
             "residual tensors must be contiguous fp32 [Mb,H]");
  KD_REQUIRE(post_norm_w->dtype == KD_BF16 && next_norm_w->dtype == KD_BF16 && is_contiguous(post_norm_w) &&
                 is_contiguous(next_norm_w) && numel(post_norm_w) == H && numel(next_norm_w) == H,
             "norm weights must be contiguous bf16 [H]");
  KD_REQUIRE(Ko % 8 == 0 && I % 8 == 0, "inner dimensions must be multiples of 8");
  int64_t Nq = 0;
  int qkv_splits = 0;
  if (w_qkv_next) {
    KD_REQUIRE(qkv_partials, "qkv_partials is required with w_qkv_next");
    KD_REQUIRE(w_qkv_next->ndim == 2 && chain_bf16_2d(w_qkv_next, w_qkv_next->shape[0], H) && is_contiguous(w_qkv_next),
               "w_qkv_next must be contiguous bf16 [Nqkv,H]");
    Nq = w_qkv_next->shape[0];
    KD_REQUIRE(qkv_partials->dtype == KD_F32 && is_contiguous(qkv_partials) && qkv_partials->ndim == 3 &&
                   qkv_partials->shape[1] == Mb && qkv_partials->shape[2] == Nq && qkv_partials->shape[0] >= 1,
               "qkv_partials must be contiguous fp32 [splits,Mb,Nqkv]");
    qkv_splits = (int)qkv_partials->shape[0];
    const int total_kb = (int)((H + CH_BK - 1) / CH_BK);
    const int kbps = (total_kb + qkv_splits - 1) / qkv_splits;
    KD_REQUIRE((total_kb + kbps - 1) / kbps == qkv_splits, "%d splits do not divide %d k-blocks evenly enough: every split must own work",
               qkv_splits, total_kb);
  }
  void *p_attn, *p_wo, *p_ri, *p_pn, *p_wgu, *p_wd, *p_nn, *p_rm, *p_ro, *p_x, *p_act, *p_wq = nullptr, *p_qp = nullptr;
  KD_TRY(tensor_ptr(attn, &p_attn)); KD_TRY(tensor_ptr(w_o, &p_wo)); KD_TRY(tensor_ptr(resid_in, &p_ri));
  KD_TRY(tensor_ptr(post_norm_w, &p_pn)); KD_TRY(tensor_ptr(w_gate_up, &p_wgu)); KD_TRY(tensor_ptr(w_down, &p_wd));
  KD_TRY(tensor_ptr(next_norm_w, &p_nn)); KD_TRY(tensor_ptr(resid_mid, &p_rm)); KD_TRY(tensor_ptr(resid_out, &p_ro));
  KD_TRY(tensor_ptr(x_out, &p_x)); KD_TRY(tensor_ptr(act, &p_act));
  if (w_qkv_next) { KD_TRY(tensor_ptr(w_qkv_next, &p_wq)); KD_TRY(tensor_ptr(qkv_partials, &p_qp)); }
  const uintptr_t all = reinterpret_cast<uintptr_t>(p_ri) | reinterpret_cast<uintptr_t>(p_pn) | reinterpret_cast<uintptr_t>(p_nn) |
                        reinterpret_cast<uintptr_t>(p_rm) | reinterpret_cast<uintptr_t>(p_ro) | reinterpret_cast<uintptr_t>(p_x) |
                        reinterpret_cast<uintptr_t>(p_act) | reinterpret_cast<uintptr_t>(p_qp);
  KD_REQUIRE((all & 15) == 0, "operands must be 16-byte aligned");
  // Split factors of the two projections back into the hidden size: about one unit per two SMs.
  // More splits shorten the weight stream of a unit (which is prefetched anyway) but lengthen the
  // add+RMSNorm phase, which reads every partial sum.
  const int G = ctx().sm_count;
  auto pick = [&](int64_t n, int64_t k) {
    const int tiles = (int)((n + 127) / 128), total_kb = (int)((k + CH_BK - 1) / CH_BK);
    int s = G / (2 * tiles);
    if (s < 1) s = 1;
    if (s > total_kb) s = total_kb;
    const int kbps = (total_kb + s - 1) / s;
    return (total_kb + kbps - 1) / kbps;
  };
  const int s0 = pick(H, Ko), s2 = pick(H, I);
  void* ws = nullptr;
  KD_TRY(get_workspace((uint64_t)(s0 + s2) * Mb * H * sizeof(float), &ws));
  float* part0 = static_cast<float*>(ws);
  float* part2 = part0 + (size_t)s0 * Mb * H;
  ChainOperand ops[4] = {
      {p_wo, (int)H, (int)Ko, p_attn, attn->strides[0]},
      {p_wgu, (int)I2, (int)H, p_x, H},
      {p_wd, (int)H, (int)I, p_act, I},
      {p_wq, (int)Nq, (int)H, p_x, H},
  };
  const int splits[4] = {s0, 1, s2, qkv_splits};
  return decode_chain_launch((int)Mb, (int)H, eps, ops, w_qkv_next ? 4 : 3, splits, part0, part2, static_cast<float*>(p_qp),
                             static_cast<__nv_bfloat16*>(p_act), static_cast<const float*>(p_ri), static_cast<float*>(p_rm),
                             static_cast<float*>(p_ro), static_cast<const __nv_bfloat16*>(p_pn),
                             static_cast<const __nv_bfloat16*>(p_nn), static_cast<__nv_bfloat16*>(p_x));
}

KD_API int kd_decode_layer_chain_splits(int64_t N, int64_t K, int* splits_out) {
  KD_TRY(require_init());
  KD_REQUIRE(splits_out && N > 0 && K > 0, "bad argument");
  const int tiles = (int)((N + 127) / 128), total_kb = (int)((K + CH_BK - 1) / CH_BK);
  int s = ctx().sm_count / tiles;
  if (s < 1) s = 1;
  if (s > total_kb) s = total_kb;
  const int kbps = (total_kb + s - 1) / s;
  *splits_out = (total_kb + kbps - 1) / kbps;
  return KD_OK;
}
