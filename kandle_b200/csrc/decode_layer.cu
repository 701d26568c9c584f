// Everything a decoder layer does between two attention calls of a decode step, and the head of
// the next layer, as ONE persistent kernel with FOUR dependent phases:
//
//   P0  o_proj (split-K)   the last split to finish a 128-row tile sums the splits in a fixed order,
//                          adds the residual: h1; writes x1 = bf16(h1 * w_post) and the tile's share
//                          of sum(h1^2) per sequence
//   P1  gate/up            act = silu(rs1 * (x1 Wg^T)) * (rs1 * (x1 Wu^T)),  rs1 = 1/sqrt(mean(h1^2)+eps)
//   P2  down (split-K)     h2 = h1 + act Wd^T; x2 = bf16(h2 * w_next); sum(h2^2) shares
//   P3  next layer's QKV   (split-K) the last split of a head's tile sums the splits, scales by rs2,
//                          then does that head's q/k RMSNorm, RoPE and the KV-cache write / q store
//       (after the last layer instead: x_final = bf16(h2 * rs2 * w_next), the lm_head's input)
//
// i.e. o_proj, residual add, post_attention_layernorm, the SwiGLU MLP, residual add, the next
// input_layernorm, the q/k/v projections, q_norm/k_norm, rotary embedding and the cache update of
// packages/model-utils/src/qwen3/decoder_layer.ts:191-241, attention/gqa.ts:246-322,
// mlp/swiglu.ts:119-134, rope.ts:546-644 and kv-cache.ts:164-212.
//
// Compared with decode_chain.cu (six phases + a separate q/k-norm + RoPE kernel) the two add+RMSNorm
// phases are gone: RMSNorm is (h * w) * rs with rs a per-sequence scalar, so the producer of h
// hands on bf16(h * w) and per-tile sums of squares, and the consumer applies rs to its fp32
// accumulator.  The split-K reduction is done by whichever CTA finishes a tile last (a ticket per
// tile; the partial sums are always added in split order, so results do not depend on who that is
// and are bit-identical from launch to launch).  Every grid-wide dependency costs a few
// microseconds of memory round trips whatever its size, which is what a decode step of 32
// sequences is made of: 4 dependencies per layer instead of 7.
//
// Structure as in decode_chain.cu: warp 0 TMA producer (weight tiles of a CTA's next unit are
// fetched while the activations they meet are still being produced), warp 1 tcgen05.mma issuer
// (swapped skinny form: D[128 weight rows, sequences] in TMEM, two accumulators), warps 2-5
// epilogues, reductions and counters.  One CTA per SM, cooperative launch, every wait bounded
// (codes 521-529).  Roofline: HBM, the bytes of the four weight matrices; in practice latency.
#include "chain_common.cuh"
#include "common.cuh"
#include "kernels.cuh"
#include "sm100.cuh"

namespace kd {

using namespace sm100;

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                      uint32_t box_rows, uint32_t box_cols);
int decode_layer_reset_counters();

constexpr int DL_BK = 64;                       // K elements per stage (one 128-byte swizzle atom)
constexpr int DL_W_BYTES = 128 * DL_BK * 2;     // weight tile bytes per stage
constexpr int DL_THREADS = 192;
constexpr int DL_MAX_TILES = 64;                // 128-row tiles of the widest split-K output (QKV rows <= 8192)
constexpr int DL_COUNTERS = 8 + 3 * DL_MAX_TILES;
constexpr int DL_CHUNK = 32;                    // sequences handled per pass of the QKV head epilogue

struct DlGemm {
  int N, K;
  int splits, kb_per_split;
  int rot;                    // unit u runs on CTA (u + rot) % gridDim.x
  float* part;                // [splits][Mb][N] fp32 partial sums (split-K phases)
  unsigned* tile_cnt;         // [tiles] tickets (split-K phases)
};

struct DlParams {
  int Mb, mb_pad, x_box, stages, H;
  int has_qkv;                // 1: phase 3 is the next layer's QKV; 0: phase 3 writes x_final
  uint32_t acc_cols;
  float eps;
  DlGemm g[4];
  unsigned target[3];         // arrivals that complete phases 0..2
  // P0 / P2 reductions
  const float* resid_in;      // h   [Mb][H]
  float* resid_mid;           // h1
  float* resid_out;           // h2
  const __nv_bfloat16* w_post;
  const __nv_bfloat16* w_next;
  __nv_bfloat16* x1;          // [Mb][H] bf16(h1 * w_post)
  __nv_bfloat16* x2;          // [Mb][H] bf16(h2 * w_next)
  float* ssq1;                // [tilesH][Mb]
  float* ssq2;
  __nv_bfloat16* act;         // [Mb][I]
  // P3: head epilogue of the next layer
  int Hq, Hkv, max_s;
  const __nv_bfloat16* qw;    // [128]
  const __nv_bfloat16* kw;
  const float* cos_t;         // [64] for the position being decoded
  const float* sin_t;
  const int* pos;             // device scalar: cache row to write
  __nv_bfloat16* q_out;       // [Mb][Hq][128]
  __nv_bfloat16* k_cache;     // [Mb][Hkv][max_s][128] with strides kc_*
  __nv_bfloat16* v_cache;
  int64_t kc_b, kc_h, kc_s;
  __nv_bfloat16* x_final;     // [Mb][H] (last layer)
  unsigned* counters;         // [DL_COUNTERS]: phases 0..2, [7] exit ticket, then the tile tickets
  int* err;
};

struct DlMaps {
  CUtensorMap w[4];
  CUtensorMap x[4];
};

__global__ void __launch_bounds__(DL_THREADS, 1)
decode_layer_kernel(const __grid_constant__ DlMaps maps, const __grid_constant__ DlParams p) {
  const int x_bytes = p.x_box * DL_BK * 2;
  const int stage_bytes = DL_W_BYTES + x_bytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_full = empty + p.stages;     // 2
  uint64_t* acc_empty = acc_full + 2;        // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile unsigned* ticket_s = reinterpret_cast<volatile unsigned*>(tmem_slot + 2);
  float* rs1 = reinterpret_cast<float*>(tmem_slot + 4);      // [128] 1/rms of h1 per sequence
  float* rs2 = rs1 + 128;                                    // [128] 1/rms of h2
  float* red = rs2 + 128;                                    // [4 warps][128 sequences]
  __nv_bfloat16* epi_stage = reinterpret_cast<__nv_bfloat16*>(red + 4 * 128);   // 4 warps x [32][16] bf16
  float* ybuf = reinterpret_cast<float*>(epi_stage + 4 * 32 * 16);              // [DL_CHUNK][128] fp32

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  const int n_gemms = p.has_qkv ? 4 : 3;
  const int tilesH = (p.H + 127) / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 4); }
    *abort_flag = 0;
    fence_mbar_init();
    for (int i = 0; i < n_gemms; ++i) {
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
      for (int gi = 0; ok && gi < n_gemms; ++gi) {
        const DlGemm& g = p.g[gi];
        const int tiles = (g.N + 127) / 128;
        const int units = tiles * g.splits;
        const int total_kb = (g.K + DL_BK - 1) / DL_BK;
        bool dep_ready = (gi == 0);
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
              if (!mbar_wait(&empty[stage], ring_phase ^ 1, abort_flag, p.err, 521)) { ok = false; break; }
              mbar_arrive_expect_tx(&full[stage], (uint32_t)stage_bytes);
              tma_load_2d(smem + stage * stage_bytes, &maps.w[gi], &full[stage], (kb0 + i) * DL_BK, tile * 128);
              if (++stage == p.stages) { stage = 0; ring_phase ^= 1; }
            }
            if (!ok) break;
            if (!counter_wait(p.counters + (gi - 1), p.target[gi - 1], abort_flag, p.err, 522)) { ok = false; break; }
            // the activations were written through the generic proxy by other SMs; TMA reads them
            // through the async proxy
            asm volatile("fence.proxy.async;" ::: "memory");
            dep_ready = true;
            for (int t = 0; t < pre; ++t) {
              const int st = (stage0 + t) % p.stages;
              tma_load_2d(smem + st * stage_bytes + DL_W_BYTES, &maps.x[gi], &full[st], (kb0 + t) * DL_BK, 0);
            }
          }
          for (; i < n_kb; ++i) {
            if (!mbar_wait(&empty[stage], ring_phase ^ 1, abort_flag, p.err, 523)) { ok = false; break; }
            mbar_arrive_expect_tx(&full[stage], (uint32_t)stage_bytes);
            tma_load_2d(smem + stage * stage_bytes, &maps.w[gi], &full[stage], (kb0 + i) * DL_BK, tile * 128);
            tma_load_2d(smem + stage * stage_bytes + DL_W_BYTES, &maps.x[gi], &full[stage], (kb0 + i) * DL_BK, 0);
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
      for (int gi = 0; ok && gi < n_gemms; ++gi) {
        const DlGemm& g = p.g[gi];
        const int tiles = (g.N + 127) / 128;
        const int units = tiles * g.splits;
        const int total_kb = (g.K + DL_BK - 1) / DL_BK;
        for (int u = (cta - g.rot % G + G) % G; ok && u < units; u += G) {
          const int split = u / tiles;
          const int kb0 = split * g.kb_per_split;
          const int n_kb = max(0, min(total_kb, kb0 + g.kb_per_split) - kb0);
          const int buf = acc_n & 1, use = acc_n >> 1;
          if (!mbar_wait(&acc_empty[buf], (uint32_t)((use & 1) ^ 1), abort_flag, p.err, 524)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)buf * p.acc_cols;
          for (int i = 0; i < n_kb; ++i) {
            if (!mbar_wait(&full[stage], ring_phase, abort_flag, p.err, 525)) { ok = false; break; }
            tc_fence_after();
            const uint32_t w_addr = smem_u32(smem + stage * stage_bytes);
            const uint32_t x_addr = w_addr + DL_W_BYTES;
#pragma unroll
            for (int k = 0; k < DL_BK / 16; ++k)
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
    // ------------------------------------------------------------------ epilogues, reductions, counters
    const int q = warp & 3;
    const int et = q * 32 + lane;           // 0..127: TMEM lane of this thread = row of the weight tile
    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
    int acc_n = 0;
    bool ok = true;
    // Control flow between the 128-thread barriers below never depends on per-thread state: `ok`
    // is made uniform (a barrier that ORs the threads' flags) before it decides anything.
    for (int gi = 0; gi < n_gemms; ++gi) {
      const DlGemm& g = p.g[gi];
      const int tiles = (g.N + 127) / 128;
      const int units = tiles * g.splits;
      const int total_kb = (g.K + DL_BK - 1) / DL_BK;
      const bool has_unit = ((cta - g.rot % G + G) % G) < units;
      // 1/rms per sequence of the activations this phase consumes
      if (has_unit && (gi == 1 || gi == 3)) {
        if (et == 0) counter_wait(p.counters + (gi - 1), p.target[gi - 1], abort_flag, p.err, 526);
        epi_bar_sync();
        const float* ssq = gi == 1 ? p.ssq1 : p.ssq2;
        float* rs = gi == 1 ? rs1 : rs2;
        if (et < p.Mb) {
          float tot = 0.f;
          for (int t = 0; t < tilesH; ++t) tot += __ldcg(ssq + t * p.Mb + et);
          rs[et] = 1.0f / sqrtf(tot / (float)p.H + p.eps);
        }
        epi_bar_sync();
      }
      for (int u = (cta - g.rot % G + G) % G; u < units; u += G) {
        const int tile = u % tiles, split = u / tiles;
        const int kb0 = split * g.kb_per_split;
        const int n_kb = max(0, min(total_kb, kb0 + g.kb_per_split) - kb0);
        const int buf = acc_n & 1, use = acc_n >> 1;
        if (ok) ok = mbar_wait(&acc_full[buf], (uint32_t)(use & 1), abort_flag, p.err, 527);
        if (epi_bar_any(!ok || *abort_flag != 0)) ok = false;   // one answer for all 128 threads
        if (!ok) continue;
        tc_fence_after();
        const int n = tile * 128 + et;
        const uint32_t t_acc = t_row + (uint32_t)buf * p.acc_cols;
        if (gi == 1) {
          // ---- gate/up: scale by rs1, SiLU(gate) * up, bf16 through shared memory (one token's 32 bytes per lane)
          for (int c0 = 0; c0 < p.mb_pad; c0 += 16) {
            uint32_t r[16];
            tmem_ld_32x16(t_acc + c0, r);
            tmem_wait_ld();
            __nv_bfloat16* stg = epi_stage + q * (32 * 16);
            float mine[16], other[16], val[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) mine[i] = __uint_as_float(r[i]) * rs1[min(c0 + i, 127)];
#pragma unroll
            for (int i = 0; i < 16; ++i) other[i] = __shfl_xor_sync(0xffffffffu, mine[i], 16);
#pragma unroll
            for (int i = 0; i < 16; ++i) val[i] = chain_silu(mine[i]) * other[i];   // meaningful in lanes 0-15
            if (lane < 16) {
#pragma unroll
              for (int i = 0; i < 16; ++i) stg[((c0 + i) & 31) * 16 + lane] = __float2bfloat16_rn(val[i]);
            }
            if (c0 + 16 >= p.mb_pad || ((c0 + 16) & 31) == 0) {
              __syncwarp();
              const int m = (c0 & ~31) + lane;
              const int j0 = (tile * 128 + q * 32) / 2;
              if (m < p.Mb && j0 + 16 <= g.N / 2) {
                const uint4* src = reinterpret_cast<const uint4*>(stg + lane * 16);
                uint4* dst = reinterpret_cast<uint4*>(p.act + (int64_t)m * (g.N / 2) + j0);
                dst[0] = src[0];
                dst[1] = src[1];
              }
              __syncwarp();
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
          ++acc_n;
          epi_bar_sync();
          if (et == 0 && *abort_flag == 0) {
            __threadfence();
            red_release_add(p.counters + 1, 1u);
          }
          continue;
        }
        // ---- split-K phases: publish this split's partial sums, take a ticket
        for (int c0 = 0; c0 < p.mb_pad; c0 += 16) {
          uint32_t r[16];
          if (n_kb > 0) {
            tmem_ld_32x16(t_acc + c0, r);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = 0u;
          }
          if (n < g.N) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int m = c0 + i;
              if (m < p.Mb) g.part[((int64_t)split * p.Mb + m) * g.N + n] = __uint_as_float(r[i]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
        ++acc_n;
        epi_bar_sync();                      // every thread's partial sums are issued
        if (et == 0) {
          __threadfence();
          const unsigned t = atomicAdd(g.tile_cnt + tile, 1u);
          __threadfence();
          *ticket_s = t;
        }
        epi_bar_sync();
        if (*ticket_s != (unsigned)(g.splits - 1)) continue;
        // ---- this CTA completed the tile: reduce it (fixed split order), then the fused tail
        if (gi == 0 || gi == 2) {
          const float* resid = gi == 0 ? p.resid_in : p.resid_mid;
          float* h_out = gi == 0 ? p.resid_mid : p.resid_out;
          __nv_bfloat16* x_out = gi == 0 ? p.x1 : p.x2;
          float* ssq = gi == 0 ? p.ssq1 : p.ssq2;
          const bool live = n < p.H;
          const float wn = live ? __bfloat162float((gi == 0 ? p.w_post : p.w_next)[n]) : 0.f;
          for (int m0 = 0; m0 < p.Mb; m0 += 4) {
            float a[4] = {0.f, 0.f, 0.f, 0.f};
            if (live) {
              for (int s = 0; s < g.splits; ++s) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  if (m0 + j < p.Mb) a[j] += __ldcg(g.part + ((int64_t)s * p.Mb + m0 + j) * g.N + n);
              }
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (m0 + j < p.Mb) a[j] += __ldcg(resid + (int64_t)(m0 + j) * p.H + n);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int m = m0 + j;
              if (m < p.Mb) {       // uniform over the warp
                if (live) {
                  h_out[(int64_t)m * p.H + n] = a[j];
                  x_out[(int64_t)m * p.H + n] = __float2bfloat16_rn(a[j] * wn);
                }
                const float sq = warp_sum(a[j] * a[j]);
                if (lane == 0) red[q * 128 + m] = sq;
              }
            }
          }
          epi_bar_sync();
          if (et < p.Mb) ssq[tile * p.Mb + et] = red[et] + red[128 + et] + red[256 + et] + red[384 + et];
          epi_bar_sync();                    // stores issued; `red` free again
          if (et == 0 && *abort_flag == 0) {
            __threadfence();
            red_release_add(p.counters + gi, 1u);
          }
        } else {
          // QKV: this tile is one head (128 rows = head_dim); thread et owns element d = et
          const int head = tile;
          const bool is_q = head < p.Hq, is_k = !is_q && head < p.Hq + p.Hkv;
          const float wd = is_q ? __bfloat162float(p.qw[et]) : (is_k ? __bfloat162float(p.kw[et]) : 1.f);
          const float cs = p.cos_t[et & 63], sn = p.sin_t[et & 63];
          const int pos = *p.pos;
          const bool pos_ok = pos >= 0 && pos < p.max_s;
          if (!is_q && !pos_ok && et == 0 && atomicCAS(p.err, 0, 102) == 0) { p.err[1] = pos; p.err[2] = p.max_s; }
          for (int m0 = 0; m0 < p.Mb; m0 += DL_CHUNK) {
            const int mc = min(DL_CHUNK, p.Mb - m0);
            float v[DL_CHUNK];
#pragma unroll
            for (int j = 0; j < DL_CHUNK; ++j) v[j] = 0.f;
            for (int s = 0; s < g.splits; ++s) {
#pragma unroll
              for (int j = 0; j < DL_CHUNK; ++j)
                if (j < mc) v[j] += __ldcg(g.part + ((int64_t)s * p.Mb + m0 + j) * g.N + n);
            }
#pragma unroll
            for (int j = 0; j < DL_CHUNK; ++j) {
              if (j < mc) {
                v[j] *= rs2[m0 + j];
                if (is_q || is_k) {
                  const float sq = warp_sum(v[j] * v[j]);
                  if (lane == 0) red[q * 128 + j] = sq;
                }
              }
            }
            if (is_q || is_k) {
              epi_bar_sync();
#pragma unroll
              for (int j = 0; j < DL_CHUNK; ++j) {
                if (j < mc) {
                  const float tot = red[j] + red[128 + j] + red[256 + j] + red[384 + j];
                  const float sc = 1.0f / sqrtf(tot / 128.f + p.eps);
                  v[j] = (v[j] * sc) * wd;
                  ybuf[j * 128 + et] = v[j];
                }
              }
              epi_bar_sync();
#pragma unroll
              for (int j = 0; j < DL_CHUNK; ++j) {
                if (j < mc) {
                  const float other = ybuf[j * 128 + (et ^ 64)];
                  // out[i] = y[i] cos - y[i+64] sin ; out[i+64] = y[i+64] cos + y[i] sin
                  v[j] = et < 64 ? v[j] * cs - other * sn : v[j] * cs + other * sn;
                }
              }
              epi_bar_sync();                // ybuf and red are rewritten by the next chunk
            }
#pragma unroll
            for (int j = 0; j < DL_CHUNK; ++j) {
              if (j < mc) {
                const int m = m0 + j;
                if (is_q) {
                  p.q_out[((int64_t)m * p.Hq + head) * 128 + et] = __float2bfloat16_rn(v[j]);
                } else if (pos_ok) {
                  const int hk = is_k ? head - p.Hq : head - p.Hq - p.Hkv;
                  __nv_bfloat16* dst = (is_k ? p.k_cache : p.v_cache) + (int64_t)m * p.kc_b + (int64_t)hk * p.kc_h + (int64_t)pos * p.kc_s;
                  dst[et] = __float2bfloat16_rn(v[j]);
                }
              }
            }
          }
        }
      }
    }
    if (!p.has_qkv) {
      // ---- after the last layer: the normalised hidden state the lm_head reads
      if (cta < p.Mb) {
        if (et == 0) counter_wait(p.counters + 2, p.target[2], abort_flag, p.err, 528);
        epi_bar_sync();
        const int m = cta;
        float tot = 0.f;
        for (int t = 0; t < tilesH; ++t) tot += __ldcg(p.ssq2 + t * p.Mb + m);
        const float sc = 1.0f / sqrtf(tot / (float)p.H + p.eps);
        for (int j = et; j < p.H; j += 128)
          p.x_final[(int64_t)m * p.H + j] = __float2bfloat16_rn((__ldcg(p.resid_out + (int64_t)m * p.H + j) * sc) * __bfloat162float(p.w_next[j]));
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
    // the last CTA out re-arms the counters and tickets for the next launch
    const unsigned ticket = atomicAdd(p.counters + 7, 1u);
    if (ticket == (unsigned)G - 1) {
      for (int i = 0; i < DL_COUNTERS; ++i) p.counters[i] = 0u;
      __threadfence();
    }
  }
}

// ----------------------------------------------------------------------------- host side
static unsigned* g_dl_counters[64] = {nullptr};

// Called when a kernel reported an error: a launch that gave up leaves counters and tickets dirty.
int decode_layer_reset_counters() {
  const int dev = ctx().device;
  if (dev >= 0 && dev < 64 && g_dl_counters[dev])
    KD_CUDA_CHECK(cudaMemsetAsync(g_dl_counters[dev], 0, DL_COUNTERS * sizeof(unsigned), ctx().stream));
  return KD_OK;
}

static int dl_pick_splits(int total_kb, int tiles, int G, int target_kb) {
  int s = (total_kb + target_kb - 1) / target_kb;
  // no more units than about one per SM: every extra split is another partial sum to add up
  while (s > 1 && tiles * s > G) --s;
  if (s < 1) s = 1;
  const int kbps = (total_kb + s - 1) / s;
  return (total_kb + kbps - 1) / kbps;
}

}  // namespace kd

using namespace kd;

static bool dl_bf16_2d(const kd_tensor* t, int64_t rows, int64_t cols) {
  return t && t->dtype == KD_BF16 && t->ndim == 2 && t->shape[0] == rows && t->shape[1] == cols && t->strides[1] == 1 &&
         t->strides[0] % 8 == 0;
}
static bool dl_f32_rows(const kd_tensor* t, int64_t rows, int64_t cols) {
  return t && t->dtype == KD_F32 && is_contiguous(t) && numel(t) == rows * cols;
}

KD_API int kd_decode_layer_fused(const kd_tensor* attn, const kd_tensor* w_o, const kd_tensor* resid_in,
                                 const kd_tensor* post_norm_w, const kd_tensor* w_gate_up, const kd_tensor* w_down,
                                 const kd_tensor* next_norm_w, float eps, const kd_tensor* w_qkv_next,
                                 const kd_tensor* q_norm_w, const kd_tensor* k_norm_w, const kd_tensor* cos,
                                 const kd_tensor* sin, const kd_tensor* pos, const kd_tensor* k_cache_next,
                                 const kd_tensor* v_cache_next, const kd_tensor* q_out, const kd_tensor* resid_out,
                                 const kd_tensor* x_final) {
  KD_TRY(require_init());
  KD_REQUIRE(attn && w_o && resid_in && post_norm_w && w_gate_up && w_down && next_norm_w && resid_out, "null tensor");
  KD_REQUIRE(attn->ndim == 2 && w_o->ndim == 2 && w_gate_up->ndim == 2 && w_down->ndim == 2, "operands must be 2-D");
  const int64_t Mb = attn->shape[0], Ko = attn->shape[1], H = w_o->shape[0], I2 = w_gate_up->shape[0], I = I2 / 2;
  Context& c = ctx();
  const int G = c.sm_count;
  KD_REQUIRE(Mb >= 1 && Mb <= 128, "%lld sequences; this path handles 1..128", (long long)Mb);
  KD_REQUIRE(Mb <= G, "more sequences than SMs");
  KD_REQUIRE(H % 8 == 0 && H <= 128 * DL_MAX_TILES, "hidden size %lld must be a multiple of 8 and at most %d", (long long)H, 128 * DL_MAX_TILES);
  KD_REQUIRE(I2 % 32 == 0, "gate/up rows must be a multiple of 32");
  KD_REQUIRE(dl_bf16_2d(attn, Mb, Ko) && dl_bf16_2d(w_o, H, Ko) && is_contiguous(w_o), "attn [Mb,Ko] / w_o [H,Ko] must be bf16");
  KD_REQUIRE(dl_bf16_2d(w_gate_up, I2, H) && is_contiguous(w_gate_up) && dl_bf16_2d(w_down, H, I) && is_contiguous(w_down),
             "w_gate_up [2I,H] / w_down [H,I] must be contiguous bf16");
  KD_REQUIRE(dl_f32_rows(resid_in, Mb, H) && dl_f32_rows(resid_out, Mb, H), "residual tensors must be contiguous fp32 [Mb,H]");
  KD_REQUIRE(post_norm_w->dtype == KD_BF16 && next_norm_w->dtype == KD_BF16 && is_contiguous(post_norm_w) &&
                 is_contiguous(next_norm_w) && numel(post_norm_w) == H && numel(next_norm_w) == H,
             "norm weights must be contiguous bf16 [H]");
  KD_REQUIRE(Ko % 8 == 0 && I % 8 == 0, "inner dimensions must be multiples of 8");
  const bool has_qkv = w_qkv_next != nullptr;
  int64_t Nq = 0;
  int Hq = 0, Hkv = 0;
  if (has_qkv) {
    KD_REQUIRE(q_norm_w && k_norm_w && cos && sin && pos && k_cache_next && v_cache_next && q_out, "the QKV phase needs norm weights, cos/sin, pos, caches and q_out");
    Nq = w_qkv_next->shape[0];
    KD_REQUIRE(w_qkv_next->ndim == 2 && dl_bf16_2d(w_qkv_next, Nq, H) && is_contiguous(w_qkv_next), "w_qkv_next must be contiguous bf16 [Nqkv,H]");
    KD_REQUIRE(Nq % 128 == 0 && Nq <= 128 * DL_MAX_TILES, "QKV rows must be whole heads of 128 (at most %d rows)", 128 * DL_MAX_TILES);
    KD_REQUIRE(q_out->ndim == 4 && q_out->dtype == KD_BF16 && is_contiguous(q_out) && q_out->shape[0] == Mb && q_out->shape[1] == 1 &&
                   q_out->shape[3] == 128,
               "q_out must be contiguous bf16 [Mb,1,Hq,128]");
    Hq = (int)q_out->shape[2];
    KD_REQUIRE(k_cache_next->ndim == 4 && k_cache_next->dtype == KD_BF16 && v_cache_next->dtype == KD_BF16 &&
                   k_cache_next->shape[0] >= Mb && k_cache_next->shape[3] == 128 && k_cache_next->strides[3] == 1,
               "caches must be bf16 [B>=Mb,Hkv,maxS,128] with unit head_dim stride");
    Hkv = (int)k_cache_next->shape[1];
    for (int i = 0; i < 4; ++i)
      KD_REQUIRE(v_cache_next->shape[i] == k_cache_next->shape[i] && v_cache_next->strides[i] == k_cache_next->strides[i],
                 "v_cache must have k_cache's shape and strides");
    KD_REQUIRE((int64_t)(Hq + 2 * Hkv) * 128 == Nq, "w_qkv_next has %lld rows, q_out / caches imply %d heads", (long long)Nq, Hq + 2 * Hkv);
    KD_REQUIRE(q_norm_w->dtype == KD_BF16 && k_norm_w->dtype == KD_BF16 && numel(q_norm_w) == 128 && numel(k_norm_w) == 128 &&
                   is_contiguous(q_norm_w) && is_contiguous(k_norm_w),
               "q/k norm weights must be contiguous bf16 [128]");
    KD_REQUIRE(cos->dtype == KD_F32 && sin->dtype == KD_F32 && is_contiguous(cos) && is_contiguous(sin) && numel(cos) == 64 && numel(sin) == 64,
               "cos/sin must be contiguous fp32 [1,64] (the position being decoded)");
    KD_REQUIRE(pos->dtype == KD_I32 && numel(pos) == 1, "pos must be a device int32 scalar");
  } else {
    KD_REQUIRE(x_final && dl_bf16_2d(x_final, Mb, H) && is_contiguous(x_final), "x_final [Mb,H] bf16 is required after the last layer");
  }
  void *p_attn, *p_wo, *p_ri, *p_pn, *p_wgu, *p_wd, *p_nn, *p_ro;
  KD_TRY(tensor_ptr(attn, &p_attn)); KD_TRY(tensor_ptr(w_o, &p_wo)); KD_TRY(tensor_ptr(resid_in, &p_ri));
  KD_TRY(tensor_ptr(post_norm_w, &p_pn)); KD_TRY(tensor_ptr(w_gate_up, &p_wgu)); KD_TRY(tensor_ptr(w_down, &p_wd));
  KD_TRY(tensor_ptr(next_norm_w, &p_nn)); KD_TRY(tensor_ptr(resid_out, &p_ro));
  void *p_wq = nullptr, *p_qw = nullptr, *p_kw = nullptr, *p_cos = nullptr, *p_sin = nullptr, *p_pos = nullptr, *p_kc = nullptr,
       *p_vc = nullptr, *p_q = nullptr, *p_xf = nullptr;
  if (has_qkv) {
    KD_TRY(tensor_ptr(w_qkv_next, &p_wq)); KD_TRY(tensor_ptr(q_norm_w, &p_qw)); KD_TRY(tensor_ptr(k_norm_w, &p_kw));
    KD_TRY(tensor_ptr(cos, &p_cos)); KD_TRY(tensor_ptr(sin, &p_sin)); KD_TRY(tensor_ptr(pos, &p_pos));
    KD_TRY(tensor_ptr(k_cache_next, &p_kc)); KD_TRY(tensor_ptr(v_cache_next, &p_vc)); KD_TRY(tensor_ptr(q_out, &p_q));
  } else {
    KD_TRY(tensor_ptr(x_final, &p_xf));
  }
  KD_REQUIRE(((reinterpret_cast<uintptr_t>(p_attn) | reinterpret_cast<uintptr_t>(p_wo) | reinterpret_cast<uintptr_t>(p_wgu) |
               reinterpret_cast<uintptr_t>(p_wd) | reinterpret_cast<uintptr_t>(p_wq)) & 15) == 0,
             "matrix operands must be 16-byte aligned");

  DlParams p{};
  p.Mb = (int)Mb; p.H = (int)H; p.eps = eps;
  p.mb_pad = ((int)Mb + 15) / 16 * 16;
  p.x_box = p.mb_pad <= 32 ? 32 : (p.mb_pad <= 64 ? 64 : 128);
  p.acc_cols = p.mb_pad <= 32 ? 32u : (p.mb_pad <= 64 ? 64u : 128u);
  p.has_qkv = has_qkv ? 1 : 0;
  const int stage_bytes = DL_W_BYTES + p.x_box * DL_BK * 2;
  const int extra = 8192 + DL_CHUNK * 128 * 4;     // barriers, per-sequence scalars, epilogue staging + the head buffer
  p.stages = (226 * 1024 - 1024 - extra) / stage_bytes;
  if (p.stages > 10) p.stages = 10;
  const int dev = c.device;
  KD_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
  if (!g_dl_counters[dev]) {
    KD_CUDA_CHECK(cudaMalloc(&g_dl_counters[dev], DL_COUNTERS * sizeof(unsigned)));
    KD_CUDA_CHECK(cudaMemsetAsync(g_dl_counters[dev], 0, DL_COUNTERS * sizeof(unsigned), c.stream));
  }
  p.counters = g_dl_counters[dev];
  p.err = c.error_flag;

  const int tilesH = (int)((H + 127) / 128);
  struct Op { const void* w; int N, K; int splits; } ops[4] = {
      {p_wo, (int)H, (int)Ko, 0}, {p_wgu, (int)I2, (int)H, 1}, {p_wd, (int)H, (int)I, 0}, {p_wq, (int)Nq, (int)H, 0}};
  const int n_gemms = has_qkv ? 4 : 3;
  for (int i = 0; i < n_gemms; ++i) {
    const int total_kb = (ops[i].K + DL_BK - 1) / DL_BK;
    const int tiles = (ops[i].N + 127) / 128;
    if (i != 1) ops[i].splits = dl_pick_splits(total_kb, tiles, G, 8);
    DlGemm& g = p.g[i];
    g.N = ops[i].N; g.K = ops[i].K; g.splits = ops[i].splits;
    g.kb_per_split = (total_kb + g.splits - 1) / g.splits;
  }
  // scratch: partial sums of the three split-K phases, h1, x1, x2, act, sums of squares
  const size_t n_part0 = (size_t)p.g[0].splits * Mb * H, n_part2 = (size_t)p.g[2].splits * Mb * H,
               n_partq = has_qkv ? (size_t)p.g[3].splits * Mb * Nq : 0;
  size_t bytes = (n_part0 + n_part2 + n_partq + (size_t)Mb * H + 2 * (size_t)tilesH * Mb) * sizeof(float) +
                 ((size_t)2 * Mb * H + (size_t)Mb * I) * sizeof(__nv_bfloat16) + 256;
  void* ws = nullptr;
  KD_TRY(get_workspace(bytes, &ws));
  float* f = static_cast<float*>(ws);
  p.g[0].part = f; f += n_part0;
  p.g[2].part = f; f += n_part2;
  p.g[3].part = has_qkv ? f : nullptr; f += n_partq;
  p.resid_mid = f; f += (size_t)Mb * H;
  p.ssq1 = f; f += (size_t)tilesH * Mb;
  p.ssq2 = f; f += (size_t)tilesH * Mb;
  __nv_bfloat16* h16 = reinterpret_cast<__nv_bfloat16*>((reinterpret_cast<uintptr_t>(f) + 127) & ~uintptr_t(127));
  p.x1 = h16; h16 += (size_t)Mb * H;
  p.x2 = h16; h16 += (size_t)Mb * H;
  p.act = h16;
  p.g[0].tile_cnt = p.counters + 8;
  p.g[2].tile_cnt = p.counters + 8 + DL_MAX_TILES;
  p.g[3].tile_cnt = p.counters + 8 + 2 * DL_MAX_TILES;
  auto units = [&](int i) { return ((p.g[i].N + 127) / 128) * p.g[i].splits; };
  // Rotations: gate/up units (long weight streams) go to the highest CTAs and the down units to the
  // CTAs after the o_proj ones, so that both start fetching their weights at once.
  p.g[0].rot = 0;
  p.g[1].rot = (G - units(1) % G) % G;
  p.g[2].rot = units(0) % G;
  p.g[3].rot = 0;
  p.target[0] = (unsigned)tilesH;
  p.target[1] = (unsigned)units(1);
  p.target[2] = (unsigned)tilesH;
  p.resid_in = static_cast<const float*>(p_ri);
  p.resid_out = static_cast<float*>(p_ro);
  p.w_post = static_cast<const __nv_bfloat16*>(p_pn);
  p.w_next = static_cast<const __nv_bfloat16*>(p_nn);
  p.Hq = Hq; p.Hkv = Hkv;
  if (has_qkv) {
    p.max_s = (int)k_cache_next->shape[2];
    p.qw = static_cast<const __nv_bfloat16*>(p_qw); p.kw = static_cast<const __nv_bfloat16*>(p_kw);
    p.cos_t = static_cast<const float*>(p_cos); p.sin_t = static_cast<const float*>(p_sin);
    p.pos = static_cast<const int*>(p_pos);
    p.q_out = static_cast<__nv_bfloat16*>(p_q);
    p.k_cache = static_cast<__nv_bfloat16*>(p_kc); p.v_cache = static_cast<__nv_bfloat16*>(p_vc);
    p.kc_b = k_cache_next->strides[0]; p.kc_h = k_cache_next->strides[1]; p.kc_s = k_cache_next->strides[2];
  }
  p.x_final = static_cast<__nv_bfloat16*>(p_xf);

  static DlMaps maps;   // large: keep it off the stack
  const void* xs[4] = {p_attn, p.x1, p.act, p.x2};
  const int64_t ldx[4] = {attn->strides[0], H, I, H};
  for (int i = 0; i < n_gemms; ++i) {
    KD_TRY(make_tmap_bf16_2d(&maps.w[i], ops[i].w, (uint64_t)ops[i].N, (uint64_t)ops[i].K, (uint64_t)ops[i].K, 128, DL_BK));
    KD_TRY(make_tmap_bf16_2d(&maps.x[i], xs[i], (uint64_t)Mb, (uint64_t)ops[i].K, (uint64_t)ldx[i], (uint32_t)p.x_box, DL_BK));
  }
  if (n_gemms < 4) { maps.w[3] = maps.w[0]; maps.x[3] = maps.x[0]; }
  const int smem = p.stages * stage_bytes + 1024 + extra;
  static bool configured[64] = {false};
  if (!configured[dev]) {
    KD_CUDA_CHECK(cudaFuncSetAttribute(decode_layer_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G);
  cfg.blockDim = dim3(DL_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = c.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // all CTAs co-resident, or the launch fails
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  KD_CUDA_CHECK(cudaLaunchKernelEx(&cfg, decode_layer_kernel, maps, p));
  return after_launch("decode_layer_kernel");
}
