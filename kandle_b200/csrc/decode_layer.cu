// Everything a decoder layer does between two attention calls of a decode step, and the head of
// the next layer, as ONE persistent kernel with FOUR dependent phases and no split-K through global
// memory (where K is split, it is split inside a thread-block cluster and summed through
// distributed shared memory; in the tensor-parallel form the ranks' partial sums cross NVLink
// inside the epilogue, see DlParams):
//
//   P0  o_proj             h1 = h + attn Wo^T;  x1 = bf16(h1 * w_post);  per-unit sums of h1^2
//   P1  gate/up            act = silu(rs1 (x1 Wg^T)) * (rs1 (x1 Wu^T)),  rs1 = 1/sqrt(mean(h1^2)+eps)
//   P2  down               h2 = h1 + act Wd^T;  x2 = bf16(h2 * w_next);  per-unit sums of h2^2
//   P3  next layer's QKV   one head per unit: rs2 (x2 Wqkv^T), that head's q/k RMSNorm, RoPE, and
//                          the q store or the KV-cache write
//       (after the last layer instead: x_final = bf16(h2 * rs2 * w_next), the lm_head's input)
//
// i.e. o_proj, residual add, post_attention_layernorm, the SwiGLU MLP, residual add, the next
// input_layernorm, the q/k/v projections, q_norm/k_norm, rotary embedding and the cache update of
// packages/model-utils/src/qwen3/decoder_layer.ts:191-241, attention/gqa.ts:246-322,
// mlp/swiglu.ts:119-134, rope.ts:546-644 and kv-cache.ts:164-212.
//
// What a decode step of a few dozen sequences costs is not bytes but dependent memory round trips:
// every hand-over between SMs (publish, observe, fetch) is a few microseconds whatever its size.
// decode_chain.cu needs seven of them per layer (six phases and a separate q/k-norm + RoPE kernel),
// because its GEMMs put the weight rows on the MMA's M side in tiles of 128 and must split K to
// occupy the SMs, and every split-K sum is another hand-over.  Here the GEMMs are the other way
// round: the SEQUENCES are the rows of the accumulator (TMEM lane m = sequence m; the MMA's M is
// 128 whatever the batch, the unused rows read whatever follows the activation tile in shared
// memory and produce rows nobody looks at), and a unit of work is a NARROW slice of weight rows
// (16..128, the MMA's N) over the WHOLE of K.  So
//   - there is no split-K phase and no partial sum in global memory: four hand-overs per layer;
//   - a thread of the epilogue owns one sequence and sees a contiguous run of output features, so
//     the residual add, the sums of squares RMSNorm needs, SiLU(gate)*up (gate and up rows are
//     interleaved 16/16), a head's RMSNorm and its rotation are all plain per-thread loops with
//     16-byte loads and stores, no shuffles, no shared memory;
//   - RMSNorm is (h * w) * rs with rs one scalar per sequence, so the producer of h hands on
//     bf16(h * w) and the consumer applies rs to its fp32 accumulator.
// The price is that every unit reads all of the activations (L2 hits, 64-192 KB per unit at 32
// sequences), which is why units are not made narrower than they need to be to occupy the SMs.
//
// warp 0 TMA producer (the weight tiles of a CTA's next unit are fetched while the activations they
// meet are still being produced), warps 1 and 6 tcgen05.mma issuers (even / odd k-blocks into two
// halves of each of the two accumulators in TMEM), warps 2-5 epilogues and counters.  One CTA per SM, all CTAs resident together (a cooperative launch, or a plain
// one inside a decode step: see the launch code), every wait bounded (codes 521-531).
// Results are bit-identical from launch to launch; the launch plan (and with it the order of the
// sums) follows the shapes, the number of sequences included.
// Roofline: HBM, the bytes of the four weight matrices; in practice latency.
#include <algorithm>

#include "chain_common.cuh"
#include "common.cuh"
#include "kernels.cuh"
#include "p2p_layout.cuh"
#include "sm100.cuh"

namespace kd {

using namespace sm100;

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                      uint32_t box_rows, uint32_t box_cols);
int decode_layer_reset_counters();

constexpr int DL_BK = 64;                       // K elements per k-block (one 128-byte swizzle atom)
constexpr int DL_THREADS = 224;                 // warp 0 producer, warps 1 and 6 MMA issuers, warps 2-5 epilogues
// A slot of the shared-memory ring holds a GROUP of consecutive k-blocks: the activation tiles of
// the group (one bulk tensor copy, a 3-D box [k-blocks, rows, 64]) and the weight tiles of the group
// (another).  What a unit that walks 16-48 k-blocks pays for is neither bandwidth nor the tensor
// pipe but the instructions its two single-thread roles execute per k-block (wait, arm, issue,
// commit); with groups the producer and the barriers work per group, and the MMA thread's inner
// loop is four tcgen05.mma with descriptors advanced by additions.
constexpr int DL_X_AREA = 16 * 1024, DL_W_AREA = 32 * 1024, DL_SLOT = DL_X_AREA + DL_W_AREA, DL_STAGES = 4;
constexpr int DL_MAX_UNITS = 512;               // units of a phase that publish sums of squares
constexpr int DL_COUNTERS = 8;
// K split inside a thread-block cluster: the CTAs of a group (2 or 4 neighbours of one cluster) take
// consecutive ranges of k-blocks of the same weight slice; the others ship their partial sums into
// this much shared memory of the group's first CTA ([split - 1][n_unit / 4][sequences] float4).
constexpr int DL_RED_BYTES = 24 * 1024;

struct DlGemm {
  int N, K;                   // weight matrix [N, K]
  int n_unit;                 // weight rows per unit (multiple of 16, at most 128)
  int units;
  int rot;                    // unit u runs on CTA group (u + rot) % (gridDim.x / split)
  int kg;                     // k-blocks per slot (per activation copy and per weight copy)
  int split;                  // 1, or CTAs of a cluster that share a slice's K (phases 0 and 2 only)
  int kb_per;                 // k-blocks per CTA of the group (an even multiple of kg; all of them when split == 1)
  int grouped;                // 1: tensor maps are [k-block, row, 64] (K a multiple of 64); 0: [1, row, K], one k-block per copy
};

struct DlParams {
  int Mb, x_box, H;
  int has_qkv;                // 1: phase 3 is the next layer's QKV; 0: phase 3 writes x_final
  float eps;
  DlGemm g[4];
  const float* resid_in;      // h   [Mb][H]
  float* resid_mid;           // h1
  float* resid_out;           // h2
  const __nv_bfloat16* w_post;
  const __nv_bfloat16* w_next;
  __nv_bfloat16* x1;          // [Mb][H] bf16(h1 * w_post)
  __nv_bfloat16* x2;          // [Mb][H] bf16(h2 * w_next)
  float* ssq1;                // [units of P0][Mb]
  float* ssq2;                // [units of P2][Mb]
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
  const int* table;           // paged cache: page of position pos of sequence m = table[m * max_pages + pos / 128] (NULL: contiguous)
  int max_pages;
  __nv_bfloat16* x_final;     // [Mb][H] (last layer)
  unsigned* counters;         // [8]: phases 0..2, [7] exit ticket
  int* err;
  unsigned long long* trace;  // optional [gridDim][16] nanosecond timestamps (kd_debug_decode_layer_trace)
  // Tensor parallel (tp > 1): W_o and W_down hold this rank's input columns, so phases 0 and 2 give
  // PARTIAL sums; each unit's epilogue exchanges them with the same unit on the other ranks through
  // the peer-mapped buffers (plain stores / loads) before the residual add.
  int tp, tp_rank;
  char* peer[P2P_MAX_RANKS];
  unsigned* tp_seq;           // [0] call counter (tags), advanced by the last CTA of each launch
  long long tp_wait;
};

struct DlMaps {
  CUtensorMap w[4];
  CUtensorMap x[4];
};

__device__ __forceinline__ unsigned long long dl_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define DL_TRACE(slot) do { if (p.trace) p.trace[(size_t)blockIdx.x * 16 + (slot)] = dl_now(); } while (0)

// tcgen05.mma with both shared-memory descriptors given as (low word, shared high word).
__device__ __forceinline__ void umma_ss_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void ld_f32x16(const float* p, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 t = __ldcg(reinterpret_cast<const float4*>(p) + i);
    v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
  }
}
__device__ __forceinline__ void ld_bf16x16(const __nv_bfloat16* p, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint4 u = reinterpret_cast<const uint4*>(p)[i];
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[8 * i + e] = __bfloat162float(h[e]);
  }
}
__device__ __forceinline__ void st_bf16x16(__nv_bfloat16* p, const float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint4 u;
    __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(&u);
#pragma unroll
    for (int e = 0; e < 8; ++e) h[e] = __float2bfloat16_rn(v[8 * i + e]);
    reinterpret_cast<uint4*>(p)[i] = u;
  }
}

// 16 / 32 accumulator columns of this thread's row: the sum of the two issuers' halves (128 columns
// apart); a unit with a single k-block only has the first half.
__device__ __forceinline__ void dl_acc16(uint32_t t_acc, bool two, float (&v)[16]) {
  uint32_t a[16], b[16];
  tmem_ld_32x16(t_acc, a);
  if (two) tmem_ld_32x16(t_acc + 128u, b);
  tmem_wait_ld();
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(a[i]) + (two ? __uint_as_float(b[i]) : 0.f);
}
__device__ __forceinline__ void dl_acc32(uint32_t t_acc, bool two, float (&v)[32]) {
  uint32_t a[32];
  tmem_ld_32x32(t_acc, a);
  tmem_wait_ld();
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(a[i]);
  if (two) {
    tmem_ld_32x32(t_acc + 128u, a);
    tmem_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] += __uint_as_float(a[i]);
  }
}

// 1/rms of a sequence from the per-unit sums of squares its producer phase published.
__device__ __forceinline__ float dl_rs(const float* ssq, int units, int Mb, int m, int H, float eps) {
  float tot = 0.f;
  int u = 0;
  for (; u + 8 <= units; u += 8) {
    float t[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = __ldcg(ssq + (u + j) * Mb + m);
#pragma unroll
    for (int j = 0; j < 8; ++j) tot += t[j];
  }
  for (; u < units; ++u) tot += __ldcg(ssq + u * Mb + m);
  return 1.0f / sqrtf(tot / (float)H + eps);
}

// ---- thread-block cluster helpers (distributed shared memory)
__device__ __forceinline__ uint32_t dl_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t dl_cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctaid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void dl_cluster_sync() {
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t dl_mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void dl_st_cluster_f4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void dl_arrive_remote(uint32_t bar_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}
// Wait (bounded) for a phase of an mbarrier whose arrivals come from other CTAs of the cluster.
__device__ __forceinline__ bool dl_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
  const long long t0 = clock64();
  int spins = 0;
  for (;;) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    if (done) return true;
    if (((++spins) & 15) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > WAIT_CYCLE_LIMIT) {
        *abort_flag = 1;
        if (atomicCAS(err, 0, code) == 0) { err[1] = (int)blockIdx.x; err[2] = (int)threadIdx.x; err[3] = (int)parity; }
        return false;
      }
    }
  }
}

// Tensor-parallel exchange, pass B (see the call site): flat over the unit's [sequences x n_unit] block.
// Kept out of line: its eight vector loads in flight would otherwise raise the register count of
// the whole kernel.
__device__ __noinline__ void dl_tp_sum_ranks(const DlParams& p, int n_unit, int N, int gi, int u, int n0, int t, size_t slot_off,
                                   const float* resid, float* h_out, __nv_bfloat16* x_out, const __nv_bfloat16* wn) {
  const int vpr = n_unit >> 2;              // items per sequence: 4, 8, 16 or 32
  const int items = p.Mb * vpr;
  for (int i0 = 0; i0 < items; i0 += 128) {
    const int i = i0 + t;
    const int row = i / vpr, col = n0 + (i % vpr) * 4;
    const bool inb = i < items && col < N;
    float part = 0.f;
    if (inb) {
      const int64_t off = (int64_t)row * p.H + col;
      float4 v[P2P_MAX_RANKS];
#pragma unroll
      for (int rk = 0; rk < P2P_MAX_RANKS; ++rk)
        if (rk < p.tp) v[rk] = ld_peer_f4(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.peer[rk] + slot_off) + off));
      float4 a = __ldcg(reinterpret_cast<const float4*>(resid + off));
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int rk = 0; rk < P2P_MAX_RANKS; ++rk)
        if (rk < p.tp) { sum.x += v[rk].x; sum.y += v[rk].y; sum.z += v[rk].z; sum.w += v[rk].w; }
      a.x += sum.x; a.y += sum.y; a.z += sum.z; a.w += sum.w;
      part = a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
      *reinterpret_cast<float4*>(h_out + off) = a;
      const uint2 wraw = *reinterpret_cast<const uint2*>(wn + col);
      const __nv_bfloat16* wh = reinterpret_cast<const __nv_bfloat16*>(&wraw);
      uint2 xo;
      __nv_bfloat16* xh = reinterpret_cast<__nv_bfloat16*>(&xo);
      xh[0] = __float2bfloat16_rn(a.x * __bfloat162float(wh[0]));
      xh[1] = __float2bfloat16_rn(a.y * __bfloat162float(wh[1]));
      xh[2] = __float2bfloat16_rn(a.z * __bfloat162float(wh[2]));
      xh[3] = __float2bfloat16_rn(a.w * __bfloat162float(wh[3]));
      *reinterpret_cast<uint2*>(x_out + off) = xo;
    }
    for (int o = vpr >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (inb && (i % vpr) == 0) (gi == 0 ? p.ssq1 : p.ssq2)[u * p.Mb + row] = part;
  }
}

// The units of a phase that a CTA works on, and its range of k-blocks.
struct DlWork { int first, step, sub, kb0, kb1; };
__device__ __forceinline__ DlWork dl_work(const DlGemm& g, int cta, int G) {
  DlWork w;
  const int S = g.split, GS = G / S;
  w.sub = cta % S;
  w.first = (cta / S - g.rot % GS + GS) % GS;
  w.step = GS;
  const int n_kb = (g.K + DL_BK - 1) / DL_BK;
  w.kb0 = w.sub * g.kb_per;
  w.kb1 = min(n_kb, w.kb0 + g.kb_per);
  return w;
}

__global__ void __launch_bounds__(DL_THREADS, 1)
decode_layer_kernel(const __grid_constant__ DlMaps maps, const __grid_constant__ DlParams p) {
  const int x1 = p.x_box * DL_BK * 2;                 // bytes of one activation k-block tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + DL_STAGES * DL_SLOT);   // slot s: [activations DL_X_AREA][weights DL_W_AREA]
  uint64_t* empty = full + DL_STAGES;
  uint64_t* acc_full = empty + DL_STAGES;       // 2
  uint64_t* acc_empty = acc_full + 2;           // 2
  uint64_t* red_bar = acc_empty + 2;            // 2: partial sums of the group's other CTAs have landed (phase 0, phase 2)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(red_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
#define DL_RED (reinterpret_cast<float4*>(smem + DL_STAGES * DL_SLOT + 1024))
  // phase 3: q-norm weights [128], k-norm weights [128], cos [64], sin [64] as fp32, staged once per CTA
  float* head_c = reinterpret_cast<float*>(smem + DL_STAGES * DL_SLOT + 1024 + DL_RED_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  const int n_gemms = p.has_qkv ? 4 : 3;

  if (threadIdx.x == 0) {
    // both MMA issuers release a slot and complete an accumulator
    for (int s = 0; s < DL_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 2); }
    for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 2); mbar_init(&acc_empty[s], 4); }
    // every epilogue thread of every other CTA of the group arrives once
    for (int s = 0; s < 2; ++s) mbar_init(&red_bar[s], (uint32_t)(max(p.g[2 * s].split, 2) - 1) * 128u);
    *abort_flag = 0;
    fence_mbar_init();
    for (int i = 0; i < n_gemms; ++i) {
      prefetch_tmap(&maps.w[i]);
      prefetch_tmap(&maps.x[i]);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);              // two accumulator buffers x two halves (one per MMA issuer) of up to 128 columns
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (dl_cluster_size() > 1) dl_cluster_sync();      // the neighbours' barriers exist before anybody arrives on them
  if (threadIdx.x == 0) DL_TRACE(0);
  // Programmatic dependent launch, both ways.  The next kernel (the attention of the next layer) may
  // start filling SMs as this kernel's CTAs leave them: it waits for this whole grid before it reads
  // anything.  And this kernel may have been started while the attention before it was still
  // running: nothing that depends on earlier kernels is touched before pdl_wait() below (the weight
  // tiles of phase 0 are fetched ahead of it, they depend on nothing).
  pdl_trigger();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t ring_phase = 0;
      bool ok = true;
      for (int gi = 0; ok && gi < n_gemms; ++gi) {
        const DlGemm& g = p.g[gi];
        const DlWork wk = dl_work(g, cta, G);
        const int grp0 = wk.kb0 / g.kg;                                  // kb_per is a multiple of kg
        const int n_grp = (wk.kb1 - wk.kb0 + g.kg - 1) / g.kg;           // groups of THIS CTA's k range
        const uint32_t tx = (uint32_t)(g.kg * (x1 + g.n_unit * DL_BK * 2));
        const CUtensorMap* wm = &maps.w[gi];
        const CUtensorMap* xm = &maps.x[gi];
        // group `grp` of this unit: k-blocks [grp * kg, grp * kg + kg)
        auto load_w = [&](int st, int grp, int row0) {
          if (g.grouped) tma_load_3d(smem + st * DL_SLOT + DL_X_AREA, wm, &full[st], 0, row0, grp * g.kg);
          else tma_load_3d(smem + st * DL_SLOT + DL_X_AREA, wm, &full[st], grp * DL_BK, row0, 0);
        };
        auto load_x = [&](int st, int grp) {
          if (g.grouped) tma_load_3d(smem + st * DL_SLOT, xm, &full[st], 0, 0, grp * g.kg);
          else tma_load_3d(smem + st * DL_SLOT, xm, &full[st], grp * DL_BK, 0, 0);
        };
        bool dep_ready = false;
        for (int u = wk.first; ok && u < g.units && n_grp > 0; u += wk.step) {
          const int row0 = u * g.n_unit;
          int i = 0;
          if (!dep_ready) {
            // weights first, as far as the ring reaches; their activations follow once they exist
            const int pre = min(n_grp, DL_STAGES);
            const int stage0 = stage;
            for (; i < pre; ++i) {
              if (!mbar_wait(&empty[stage], ring_phase ^ 1, abort_flag, p.err, 521)) { ok = false; break; }
              mbar_arrive_expect_tx(&full[stage], tx);
              load_w(stage, grp0 + i, row0);
              if (++stage == DL_STAGES) { stage = 0; ring_phase ^= 1; }
            }
            if (!ok) break;
            if (gi == 0) pdl_wait();          // the attention output: complete when the preceding kernels are
            else if (!counter_wait(p.counters + (gi - 1), (unsigned)p.g[gi - 1].units, abort_flag, p.err, 522)) { ok = false; break; }
            // the activations were written through the generic proxy by other SMs; TMA reads them
            // through the async proxy
            asm volatile("fence.proxy.async;" ::: "memory");
            dep_ready = true;
            DL_TRACE(1 + 3 * gi);
            for (int t = 0; t < pre; ++t) {
              int st = stage0 + t;
              if (st >= DL_STAGES) st -= DL_STAGES;
              load_x(st, grp0 + t);
            }
          }
          for (; i < n_grp; ++i) {
            if (!mbar_wait(&empty[stage], ring_phase ^ 1, abort_flag, p.err, 523)) { ok = false; break; }
            mbar_arrive_expect_tx(&full[stage], tx);
            load_w(stage, grp0 + i, row0);
            load_x(stage, grp0 + i);
            if (++stage == DL_STAGES) { stage = 0; ring_phase ^= 1; }
          }
        }
      }
    }
  } else if (warp == 1 || warp == 6) {
    // ------------------------------------------------------------------ MMA issuers
    // One thread issues a tcgen05.mma of this size every ~55-95 cycles however narrow it is, while
    // the tensor pipe takes one every ~40-50: two issuing warps share a unit's k-blocks (even ones to
    // warp 1, odd ones to warp 6), each accumulating into its own half of the buffer; the epilogue
    // adds the halves.
    if (lane == 0) {
      const int me = warp == 1 ? 0 : 1;
      int stage = 0;
      uint32_t ring_phase = 0;
      int acc_n = 0;
      bool ok = true;
      // shared-memory descriptors (128-byte swizzle, K-major, 8-row groups 1024 bytes apart): the high
      // word is constant, the low word is the address in 16-byte units plus the (unused) leading offset
      constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t smem_lo = ((smem_u32(smem) >> 4) & 0x3FFFu) | (1u << 16);
      for (int gi = 0; ok && gi < n_gemms; ++gi) {
        const DlGemm& g = p.g[gi];
        const DlWork wk = dl_work(g, cta, G);
        const uint32_t x_step = (uint32_t)x1 >> 4, w_step = (uint32_t)(g.n_unit * DL_BK * 2) >> 4;
        // D[128 sequence rows, n_unit weight rows] += X[128, 16] * W[n_unit, 16]^T
        const uint32_t idesc = make_idesc_bf16(128, g.n_unit, 0, 0);
        for (int u = wk.first; ok && u < g.units && wk.kb0 < wk.kb1; u += wk.step) {
          const int buf = acc_n & 1, use = acc_n >> 1;
          if (!mbar_wait(&acc_empty[buf], (uint32_t)((use & 1) ^ 1), abort_flag, p.err, 524)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)buf * 256u + (uint32_t)me * 128u;
          uint32_t acc = 0u;
          for (int kb = wk.kb0; kb < wk.kb1; kb += g.kg) {
            if (!mbar_wait(&full[stage], ring_phase, abort_flag, p.err, 525)) { ok = false; break; }
            tc_fence_after();
            // an activation tile holds x_box rows; the MMA's other rows are read from whatever follows
            // it in the slot (later tiles, the weight area) and give accumulator rows of no sequence
            const int nk = min(g.kg, wk.kb1 - kb);
            const int j0 = (kb + me) & 1 ? 1 : 0;          // this issuer's first k-block of the group: global index parity == me
            uint32_t xl = smem_lo + (uint32_t)(stage * (DL_SLOT >> 4)) + (uint32_t)j0 * x_step;
            uint32_t wl = smem_lo + (uint32_t)(stage * (DL_SLOT >> 4)) + (uint32_t)(DL_X_AREA >> 4) + (uint32_t)j0 * w_step;
            for (int j = j0; j < nk; j += 2) {
              umma_ss_lohi(d_tmem, xl, wl, DESC_HI, idesc, acc);
              umma_ss_lohi(d_tmem, xl + 2, wl + 2, DESC_HI, idesc, 1u);
              umma_ss_lohi(d_tmem, xl + 4, wl + 4, DESC_HI, idesc, 1u);
              umma_ss_lohi(d_tmem, xl + 6, wl + 6, DESC_HI, idesc, 1u);
              acc = 1u;
              xl += 2 * x_step;
              wl += 2 * w_step;
            }
            umma_commit(&empty[stage]);
            if (++stage == DL_STAGES) { stage = 0; ring_phase ^= 1; }
          }
          if (!ok) break;
          umma_commit(&acc_full[buf]);
          ++acc_n;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogues and counters
    const int q = warp & 3;
    const int m = q * 32 + lane;            // TMEM lane of this thread = sequence
    const bool valid = m < p.Mb;
    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
    int acc_n = 0;
    bool ok = true;
    pdl_wait();      // residual, position, tables: produced by earlier kernels
    const unsigned tp_tag = p.tp > 1 ? p.tp_seq[0] + 1u : 0u;     // this launch's tag on the exchange flags
    // Control flow between the 128-thread barriers below never depends on per-thread state: `ok`
    // is made uniform (a barrier that ORs the threads' flags) before it decides anything.
    for (int gi = 0; gi < n_gemms; ++gi) {
      const DlGemm& g = p.g[gi];
      const DlWork wk = dl_work(g, cta, G);
      const bool has_unit = wk.first < g.units && wk.kb0 < wk.kb1;
      const bool leader = wk.sub == 0;          // of the group that shares a slice's K (always, when the phase is not split)
      float rs = 1.f;
      if (has_unit && gi == 3) {
        // (visible to the 128 threads after the barrier below)
        const int t = (int)(threadIdx.x & 127);
        head_c[t] = __bfloat162float(p.qw[t]);
        head_c[128 + t] = __bfloat162float(p.kw[t]);
        if (t < 64) head_c[256 + t] = p.cos_t[t];
        else head_c[320 + (t - 64)] = p.sin_t[t - 64];
      }
      if (has_unit && (gi == 1 || gi == 3)) {
        // 1/rms of this thread's sequence, from the sums of squares of the phase that produced x
        if ((threadIdx.x & 127) == 0) counter_wait(p.counters + (gi - 1), (unsigned)p.g[gi - 1].units, abort_flag, p.err, 526);
        epi_bar_sync();
        if (valid) rs = dl_rs(gi == 1 ? p.ssq1 : p.ssq2, p.g[gi - 1].units, p.Mb, m, p.H, p.eps);
      } else if (has_unit && gi == 2 && leader) {
        // h1 (the residual of this phase) is complete once phase 0 is: only then may it be fetched early
        if ((threadIdx.x & 127) == 0) counter_wait(p.counters + 0, (unsigned)p.g[0].units, abort_flag, p.err, 526);
        epi_bar_sync();
      }
      for (int u = wk.first; has_unit && u < g.units; u += wk.step) {
        const int buf = acc_n & 1, use = acc_n >> 1;
        const int n0 = u * g.n_unit;
        // the residual and the norm weights do not depend on the GEMM: fetch the first columns' worth
        // while the MMAs run (the first 16 columns; the later ones are loaded in the loop below, where
        // their latency hides behind the work on the columns before them)
        // (the first 16 columns of the residual into registers; the unit's norm weights, which are the
        // same for every sequence, into shared memory: the 128-thread barrier after the accumulator wait
        // makes them visible)
        float pre_r[16];
        float* w_s = head_c + 384;       // [n_unit]
        if ((gi == 0 || gi == 2) && n0 < g.N && p.tp == 1 && leader) {
          const int t = (int)(threadIdx.x & 127);
          if (t < g.n_unit && n0 + t < g.N) w_s[t] = __bfloat162float((gi == 0 ? p.w_post : p.w_next)[n0 + t]);
          if (valid) ld_f32x16((gi == 0 ? p.resid_in : p.resid_mid) + (int64_t)m * p.H + n0, pre_r);
        }
        if (ok) ok = mbar_wait(&acc_full[buf], (uint32_t)(use & 1), abort_flag, p.err, 527);
        // the group's other CTAs have shipped their partial sums (a split phase is one unit per CTA, so
        // each of the two barriers completes once per launch)
        if (ok && g.split > 1 && leader) ok = dl_wait_cluster(&red_bar[gi >> 1], 0u, abort_flag, p.err, 529);
        if (epi_bar_any(!ok || *abort_flag != 0)) ok = false;   // one answer for all 128 threads
        if (!ok) continue;
        tc_fence_after();
        if ((threadIdx.x & 127) == 0) DL_TRACE(2 + 3 * gi);
        const uint32_t t_acc = t_row + (uint32_t)buf * 256u;
        const bool two = wk.kb1 - wk.kb0 > 1;   // the second issuer had at least one k-block (kb0 is even)
        if (!leader) {
          // ---- partial sums of this CTA's k range: into the leader's shared memory, row m of column
          // group c4 at [(sub - 1)][c4][m]; every thread arrives on the leader's barrier (release at
          // cluster scope), valid row or not
          const uint32_t lead_rank = dl_cluster_rank() - (uint32_t)wk.sub;
          const uint32_t red_remote = dl_mapa(smem_u32(DL_RED), lead_rank);
          const int vpr = g.n_unit >> 2;
          for (int c0 = 0; c0 < g.n_unit; c0 += 16) {
            float r[16];
            dl_acc16(t_acc + c0, two, r);
            if (valid) {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                dl_st_cluster_f4(red_remote + (uint32_t)((((wk.sub - 1) * vpr + (c0 >> 2) + i) * p.Mb + m) << 4), r[4 * i], r[4 * i + 1],
                                 r[4 * i + 2], r[4 * i + 3]);
            }
          }
          dl_arrive_remote(dl_mapa(smem_u32(&red_bar[gi >> 1]), lead_rank));
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
          ++acc_n;
          if ((threadIdx.x & 127) == 0) DL_TRACE(3 + 3 * gi);
          continue;
        }
        if (gi == 0 || gi == 2) {
          // ---- residual add; hand on h, bf16(h * w) and this unit's share of sum(h^2)
          const float* resid = gi == 0 ? p.resid_in : p.resid_mid;
          float* h_out = gi == 0 ? p.resid_mid : p.resid_out;
          __nv_bfloat16* x_out = gi == 0 ? p.x1 : p.x2;
          const __nv_bfloat16* wn = gi == 0 ? p.w_post : p.w_next;
          float ss = 0.f;
          if (p.tp > 1) {
            // ---- exchange with the same unit on the other ranks.  Pass A: this rank's partial sums into
            // its own slot of the exchange buffer, then one flag per (phase, unit) into EVERY rank's
            // buffer; wait on the LOCAL flags (bounded).
            const size_t slot_off = P2P_LAYER_SLOT_OFFSET + (gi == 0 ? 0 : P2P_SLOT_BYTES);
            float* mine = reinterpret_cast<float*>(p.peer[p.tp_rank] + slot_off);
            for (int c0 = 0; c0 < g.n_unit; c0 += 16) {
              float r[16];
              dl_acc16(t_acc + c0, two, r);
              if (valid && n0 + c0 < g.N) {
                float4* o = reinterpret_cast<float4*>(mine + (int64_t)m * p.H + n0 + c0);
#pragma unroll
                for (int i = 0; i < 4; ++i) o[i] = make_float4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
              }
            }
            // the accumulator is read: the MMA warps may start this CTA's next unit during the exchange
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            ++acc_n;
            epi_bar_sync();
            const int t = (int)(threadIdx.x & 127);
            bool failed = false;
            if (t < p.tp) {
              const size_t fidx = ((size_t)(gi == 0 ? 0 : 1) * P2P_MAX_ROWS + u) * P2P_MAX_RANKS;
              __threadfence_system();
              st_release_sys(reinterpret_cast<unsigned*>(p.peer[t] + P2P_LAYER_FLAG_OFFSET) + fidx + p.tp_rank, tp_tag);
              const unsigned* f = reinterpret_cast<const unsigned*>(p.peer[p.tp_rank] + P2P_LAYER_FLAG_OFFSET) + fidx + t;
              const long long t0 = clock64();
              int spins = 0;
              while (ld_acquire_sys(f) != tp_tag) {
                if (((++spins) & 7) == 0 && (*abort_flag || clock64() - t0 > p.tp_wait)) {
                  failed = true;
                  *abort_flag = 1;
                  if (atomicCAS(p.err, 0, 531) == 0) { p.err[1] = u; p.err[2] = t; p.err[3] = gi; }
                  break;
                }
              }
            }
            if (epi_bar_any(failed)) {      // a peer's partial sums never came: stop working on units
              ok = false;
              continue;
            }
            // Pass B, flat over the unit's [sequences x n_unit] block so that every thread has work and all
            // peer loads of a thread are in flight together (a peer load is a round trip over NVLink):
            // item i = four columns of one sequence; sum over ranks in rank order (the same bits on every
            // rank), residual add, h and bf16(h * w) stores; the row's share of sum(h^2) is reduced over
            // the adjacent lanes that hold the row (n_unit is a power of two here).
            dl_tp_sum_ranks(p, g.n_unit, g.N, gi, u, n0, t, slot_off, resid, h_out, x_out, wn);
            epi_bar_sync();
            if (t == 0 && *abort_flag == 0) {
              red_release_add(p.counters + gi, 1u);
              DL_TRACE(3 + 3 * gi);
            }
            continue;
          }
          // one 16-column chunk: add the accumulator to the residual, store h and bf16(h * w)
          auto chunk = [&](int c0, float (&a)[16]) {
            float r[16];
            dl_acc16(t_acc + c0, two, r);
            if (g.split > 1 && valid) {
              // + the other CTAs' k ranges, in the order of the ranges
              const int vpr = g.n_unit >> 2;
              for (int sgrp = 0; sgrp < g.split - 1; ++sgrp) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float4 v = DL_RED[((sgrp * vpr + (c0 >> 2) + i) * p.Mb + m)];
                  r[4 * i] += v.x; r[4 * i + 1] += v.y; r[4 * i + 2] += v.z; r[4 * i + 3] += v.w;
                }
              }
            }
            if (valid && n0 + c0 < g.N) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                a[i] += r[i];
                ss += a[i] * a[i];
              }
              float4* ho = reinterpret_cast<float4*>(h_out + (int64_t)m * p.H + n0 + c0);
#pragma unroll
              for (int i = 0; i < 4; ++i) ho[i] = make_float4(a[4 * i], a[4 * i + 1], a[4 * i + 2], a[4 * i + 3]);
#pragma unroll
              for (int i = 0; i < 16; ++i) a[i] *= w_s[c0 + i];
              st_bf16x16(x_out + (int64_t)m * p.H + n0 + c0, a);
            }
          };
          // the residual of the next 16 columns is requested before the current ones are worked on
          for (int c0 = 0; c0 < g.n_unit; c0 += 16) {
            float nxt[16];
            if (c0 + 16 < g.n_unit && valid && n0 + c0 + 16 < g.N) ld_f32x16(resid + (int64_t)m * p.H + n0 + c0 + 16, nxt);
            chunk(c0, pre_r);
#pragma unroll
            for (int i = 0; i < 16; ++i) pre_r[i] = nxt[i];
          }
          if (valid) (gi == 0 ? p.ssq1 : p.ssq2)[u * p.Mb + m] = ss;
        } else if (gi == 1) {
          // ---- gate/up: columns come in groups of 16 gate rows followed by the 16 matching up rows
          for (int c0 = 0; c0 < g.n_unit; c0 += 32) {
            float r[32];
            dl_acc32(t_acc + c0, two, r);
            if (valid && n0 + c0 < g.N) {
              float o[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] = chain_silu(r[i] * rs) * (r[16 + i] * rs);
              st_bf16x16(p.act + (int64_t)m * (g.N / 2) + (n0 + c0) / 2, o);
            }
          }
        } else {
          // ---- QKV: this unit is one head (128 columns = head_dim); two passes over the accumulator
          const int head = u;
          const bool is_q = head < p.Hq, is_k = !is_q && head < p.Hq + p.Hkv;
          float sc = 1.f;
          if (is_q || is_k) {
            float ss = 0.f;
            for (int c0 = 0; c0 < 128; c0 += 32) {
              float r[32];
              dl_acc32(t_acc + c0, two, r);
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float v = r[i] * rs;
                ss += v * v;
              }
            }
            sc = 1.0f / sqrtf(ss / 128.f + p.eps);
          }
          const int pos = *p.pos;
          const bool pos_ok = pos >= 0 && pos < p.max_s;
          if (!is_q && !pos_ok && (threadIdx.x & 127) == 0 && atomicCAS(p.err, 0, 102) == 0) { p.err[1] = pos; p.err[2] = p.max_s; }
          __nv_bfloat16* dst = nullptr;
          if (valid) {
            if (is_q) dst = p.q_out + ((int64_t)m * p.Hq + head) * 128;
            else if (pos_ok) {
              const int hk = is_k ? head - p.Hq : head - p.Hq - p.Hkv;
              int64_t outer = m, row = pos;
              if (p.table) {
                outer = p.table[(int64_t)m * p.max_pages + pos / 128];
                row = pos % 128;
              }
              dst = (is_k ? p.k_cache : p.v_cache) + outer * p.kc_b + (int64_t)hk * p.kc_h + row * p.kc_s;
            }
          }
          const float* hw = is_q ? head_c : head_c + 128;
          for (int c0 = 0; c0 < 64; c0 += 16) {
            // elements d = c0..c0+15 and their rotation partners d + 64
            float y1[16], y2[16];
            dl_acc16(t_acc + c0, two, y1);
            dl_acc16(t_acc + 64 + c0, two, y2);
            if (dst) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                y1[i] *= rs;
                y2[i] *= rs;
              }
              if (is_q || is_k) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  const float a = (y1[i] * sc) * hw[c0 + i], b = (y2[i] * sc) * hw[64 + c0 + i];
                  const float cs = head_c[256 + c0 + i], sn = head_c[320 + c0 + i];
                  // out[i] = y[i] cos - y[i+64] sin ; out[i+64] = y[i+64] cos + y[i] sin
                  y1[i] = a * cs - b * sn;
                  y2[i] = b * cs + a * sn;
                }
              }
              st_bf16x16(dst + c0, y1);
              st_bf16x16(dst + 64 + c0, y2);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
        ++acc_n;
        if (gi < 3) {
          // this unit's outputs are in global memory: publish
          // (the barrier orders the other 127 threads' writes before thread 0's release, which is cumulative)
          epi_bar_sync();
          if ((threadIdx.x & 127) == 0 && *abort_flag == 0) {
            red_release_add(p.counters + gi, 1u);     // release at gpu scope: no separate fence needed
            DL_TRACE(3 + 3 * gi);
          }
        } else if ((threadIdx.x & 127) == 0) {
          DL_TRACE(3 + 3 * gi);
        }
      }
    }
    if (!p.has_qkv) {
      // ---- after the last layer: the normalised hidden state the lm_head reads, one CTA per sequence
      if (cta < p.Mb) {
        if ((threadIdx.x & 127) == 0) counter_wait(p.counters + 2, (unsigned)p.g[2].units, abort_flag, p.err, 528);
        epi_bar_sync();
        const int row = cta;
        const float sc = dl_rs(p.ssq2, p.g[2].units, p.Mb, row, p.H, p.eps);
        for (int j = q * 32 + lane; j < p.H; j += 128)
          p.x_final[(int64_t)row * p.H + j] =
              __float2bfloat16_rn((__ldcg(p.resid_out + (int64_t)row * p.H + j) * sc) * __bfloat162float(p.w_next[j]));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  // no CTA leaves while a neighbour may still write into its shared memory or arrive on its barriers
  if (dl_cluster_size() > 1) dl_cluster_sync();
  if (threadIdx.x == 0 && *abort_flag == 0) {
    // the last CTA out re-arms the counters for the next launch
    const unsigned ticket = atomicAdd(p.counters + 7, 1u);
    if (ticket == (unsigned)G - 1) {
      for (int i = 0; i < DL_COUNTERS; ++i) p.counters[i] = 0u;
      if (p.tp > 1) p.tp_seq[0] += 1u;       // every CTA has read this launch's tag long ago
      __threadfence();
    }
  }
}

// ----------------------------------------------------------------------------- host side
static unsigned* g_dl_counters[64] = {nullptr};
static bool g_dl_no_clusters[64] = {false};   // a clustered launch was refused on this device: plan without clusters
static unsigned long long* g_dl_trace = nullptr;     // [sm_count][16], only with KD_DECODE_LAYER_TRACE=1

// Called when a kernel reported an error: a launch that gave up leaves its counters dirty.
int decode_layer_reset_counters() {
  const int dev = ctx().device;
  if (dev >= 0 && dev < 64 && g_dl_counters[dev])
    KD_CUDA_CHECK(cudaMemsetAsync(g_dl_counters[dev], 0, DL_COUNTERS * sizeof(unsigned), ctx().stream));
  return KD_OK;
}

typedef CUresult (*DlEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                               CUtensorMapFloatOOBfill);

// bf16 tensor map with dims (innermost first) {d0, d1, d2}, byte strides {s1, s2} of d1 and d2, box {64, b1, b2},
// 128-byte swizzle, zero fill outside.
static int dl_tmap3(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2, uint32_t b1,
                    uint32_t b2) {
  static DlEncodeFn fn = nullptr;
  if (!fn) {
    void* q = nullptr;
    cudaDriverEntryPointQueryResult r;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &r) == cudaSuccess && r == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<DlEncodeFn>(q);
  }
  if (!fn) return fail(KD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  KD_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0 && s1 % 16 == 0 && s2 % 16 == 0, "TMA base and strides must be multiples of 16 bytes");
  KD_REQUIRE(b1 >= 1 && b1 <= 256 && b2 >= 1 && b2 <= 256, "TMA box [%u,%u] out of range", b1, b2);
  cuuint64_t gdim[3] = {d0, d1, d2};
  cuuint64_t gstr[2] = {s1, s2};
  cuuint32_t box[3] = {(cuuint32_t)DL_BK, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(KD_ERR_CUDA, "cuTensorMapEncodeTiled (decode layer) failed with code %d", (int)r);
  return KD_OK;
}

// CTAs of a cooperative launch with clusters of `cs` CTAs (one CTA of `smem` bytes per SM): the
// largest whole number of clusters that are resident together (132 of 148 SMs for clusters of 4 on
// B200: clusters do not straddle GPCs).  0: such a launch is not possible.
__global__ void decode_layer_kernel(const __grid_constant__ DlMaps maps, const __grid_constant__ DlParams p);
static int dl_cluster_grid(int cs, int smem) {
  static int cached[64][5] = {};
  const int dev = ctx().device & 63;
  if (cs == 1) return ctx().sm_count;
  if (cached[dev][cs] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cs);
    cfg.blockDim = dim3(DL_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cs; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, decode_layer_kernel, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
    cached[dev][cs] = n > 0 ? n * cs : -1;
  }
  return cached[dev][cs] > 0 ? cached[dev][cs] : 0;
}

// Cost model behind the choice of the cluster size and of each phase's unit width and K split, in
// microseconds, fitted to device-side timelines of the kernel (Qwen3-0.6B and 4B widths):
//   - a CTA issues the MMAs of one k-block in about 0.127 us whatever the width of the slice (up to
//     64 rows; wider: 0.17) and streams its weights at 80 GB/s at best; a phase as a whole cannot
//     stream faster than about 5.5 TB/s;
//   - an epilogue costs about 1 us plus 0.02 us per column of the slice (one thread owns a sequence
//     and walks the columns), half as much again per partial sum it adds in;
//   - a hand-over of partial sums inside a cluster about 0.6 us.
static float dl_phase_cost(int N, int K, int n_unit, int split, int kb_per, int G) {
  const int slices = (N + n_unit - 1) / n_unit;
  const int waves = split > 1 ? 1 : (slices + G - 1) / G;
  const float mma = kb_per * (n_unit > 64 ? 0.17f : 0.127f);
  const float stream = (float)n_unit * kb_per * DL_BK * 2 / 80e3f;
  const float floor_all = (float)N * K * 2 / 5.5e6f;
  const float epi = 1.0f + 0.02f * n_unit * (1.0f + 0.5f * (split - 1));
  return std::max(waves * std::max(mma, stream), floor_all) + waves * epi + (split > 1 ? 0.6f : 0.f);
}


// What the launch plan depends on, and nothing else (no device is touched: the plan can be checked on a CPU).
struct DlPlanIn {
  int Mb, x_box;              // sequences; rows of an activation tile (8 / 16 / 32 / 64 / 128)
  int n_gemms;                // 4, or 3 after the last layer
  int N[4], K[4];             // the weight matrices of the phases
  int tensor_parallel;
  int no_groups;              // experiment: one k-block per bulk copy
  int want_n[3];              // experiment: fixed unit width of phases 0..2 (0: free)
  int grid[5];                // [1], [2], [4]: CTAs that are resident together with clusters of that size (0: not available)
};

// The best unit width and K split of each phase by the cost model above, for every cluster size
// that can be launched; the cluster size with the lowest sum wins (the smaller one on a near tie).
// Returns the cluster size (0: no configuration) and fills plan[0 .. n_gemms).  Guarantees, for a
// phase with split S > 1: the K ranges of the S CTAs start at even k-blocks and at whole groups of
// k-blocks, none is empty, one wave of S-CTA groups covers all slices, and the partial sums of a
// group fit DL_RED_BYTES.
static int dl_make_plan(const DlPlanIn& in, DlGemm* plan) {
  const int x1 = in.x_box * DL_BK * 2;
  auto grouped_of = [&](int K) { return K % DL_BK == 0 && !in.no_groups; };
  auto kg_of = [&](int n_unit, int K) {
    const int n_kb = (K + DL_BK - 1) / DL_BK;
    return grouped_of(K) ? std::max(1, std::min(std::min(DL_X_AREA / x1, DL_W_AREA / (n_unit * DL_BK * 2)), std::min(n_kb, 16))) : 1;
  };
  int cluster = 0;
  float best_total = 1e30f;
  for (int cs = 1; cs <= 4; cs *= 2) {
    if (in.tensor_parallel && cs > 1) continue;       // K is already split over the ranks; the exchange replaces the cluster reduce
    const int Gc = in.grid[cs];
    if (Gc <= 0 || in.Mb > Gc) continue;
    DlGemm cand[4] = {};
    float total = 0.f;
    bool feasible = true;
    for (int i = 0; i < in.n_gemms && feasible; ++i) {
      DlGemm& g = cand[i];
      g.N = in.N[i]; g.K = in.K[i];
      const int n_kb = (g.K + DL_BK - 1) / DL_BK;
      if (i == 1 || i == 3) {
        g.split = 1;
        g.kb_per = n_kb;
        g.n_unit = 128;                 // phase 3: one head per unit
        if (i == 1) {
          float best1 = 1e30f;
          for (int n = 32; n <= 128; n += 32) {
            if (in.want_n[1] && n != in.want_n[1]) continue;
            if ((g.N + n - 1) / n > DL_MAX_UNITS) continue;
            const float cost = dl_phase_cost(g.N, g.K, n, 1, n_kb, Gc);
            if (cost < best1 - 0.05f) { best1 = cost; g.n_unit = n; }
          }
        }
        g.units = (g.N + g.n_unit - 1) / g.n_unit;
        if (g.units > DL_MAX_UNITS) { feasible = false; break; }
        total += dl_phase_cost(g.N, g.K, g.n_unit, 1, n_kb, Gc);
        continue;
      }
      float best = 1e30f;
      for (int n = 16; n <= 128; n += 16) {
        if (in.want_n[i] && n != in.want_n[i]) continue;
        if (in.tensor_parallel && (n & (n - 1))) continue;      // the exchange epilogue reduces over adjacent lanes: powers of two
        const int slices = (g.N + n - 1) / n;
        if (in.tensor_parallel && slices > P2P_MAX_ROWS) continue;   // one exchange flag per unit
        if (slices > DL_MAX_UNITS) continue;
        const int kg = kg_of(n, g.K);
        for (int S = 1; S <= cs; S *= 2) {
          int kb_per = n_kb;
          if (S > 1) {
            if (!grouped_of(g.K) || slices > Gc / S || (size_t)(S - 1) * in.Mb * n * sizeof(float) > (size_t)DL_RED_BYTES) continue;
            const int q = (kg % 2) ? 2 * kg : kg;                  // ranges start at even k-blocks and at whole groups
            kb_per = ((n_kb + S - 1) / S + q - 1) / q * q;
            if (kb_per * (S - 1) >= n_kb) continue;                // somebody's range would be empty
          }
          const float cost = dl_phase_cost(g.N, g.K, n, S, kb_per, Gc);
          if (cost < best - 0.05f) {
            best = cost;
            g.n_unit = n; g.units = slices; g.split = S; g.kb_per = kb_per;
          }
        }
      }
      if (best > 1e29f) feasible = false;
      total += best;
    }
    if (!feasible) continue;
    if (total < best_total - 0.3f) {
      best_total = total;
      cluster = cs;
      for (int i = 0; i < 4; ++i) plan[i] = cand[i];
    }
  }
  // what the tensor maps and the kernel derive from the plan
  for (int i = 0; cluster > 0 && i < in.n_gemms; ++i) {
    plan[i].grouped = grouped_of(plan[i].K) ? 1 : 0;
    plan[i].kg = kg_of(plan[i].n_unit, plan[i].K);
  }
  return cluster;
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

// Timestamps of the last kd_decode_layer_fused launch (nanoseconds, [sm_count][16]: 0 start; per phase
// g: 1+3g dependency seen by the producer, 2+3g accumulator seen by the epilogue, 3+3g outputs
// published).  Filled only when the process runs with KD_DECODE_LAYER_TRACE=1.
KD_API int kd_debug_decode_layer_trace(uint64_t* out, int max_entries) {
  KD_TRY(require_init());
  KD_REQUIRE(out && max_entries > 0, "bad argument");
  KD_REQUIRE(g_dl_trace != nullptr, "no trace: start the process with KD_DECODE_LAYER_TRACE=1");
  const int n = ctx().sm_count * 16 < max_entries ? ctx().sm_count * 16 : max_entries;
  KD_CUDA_CHECK(cudaStreamSynchronize(ctx().stream));
  KD_CUDA_CHECK(cudaMemcpy(out, g_dl_trace, (size_t)n * sizeof(uint64_t), cudaMemcpyDeviceToHost));
  return KD_OK;
}

static int decode_layer_fused(bool tensor_parallel, const kd_tensor* attn, const kd_tensor* w_o, const kd_tensor* resid_in,
                              const kd_tensor* post_norm_w, const kd_tensor* w_gate_up, const kd_tensor* w_down,
                              const kd_tensor* next_norm_w, float eps, const kd_tensor* w_qkv_next,
                              const kd_tensor* q_norm_w, const kd_tensor* k_norm_w, const kd_tensor* cos,
                              const kd_tensor* sin, const kd_tensor* pos, const kd_tensor* k_cache_next,
                              const kd_tensor* v_cache_next, const kd_tensor* block_table, const kd_tensor* q_out,
                              const kd_tensor* resid_out, const kd_tensor* x_final) {
  KD_TRY(require_init());
  KD_REQUIRE(attn && w_o && resid_in && post_norm_w && w_gate_up && w_down && next_norm_w && resid_out, "null tensor");
  KD_REQUIRE(attn->ndim == 2 && w_o->ndim == 2 && w_gate_up->ndim == 2 && w_down->ndim == 2, "operands must be 2-D");
  const int64_t Mb = attn->shape[0], Ko = attn->shape[1], H = w_o->shape[0], I2 = w_gate_up->shape[0], I = I2 / 2;
  Context& c = ctx();
  int G = c.sm_count;
  KD_REQUIRE(Mb >= 1 && Mb <= 128, "%lld sequences; this path handles 1..128", (long long)Mb);
  KD_REQUIRE(Mb <= G, "more sequences than SMs");
  KD_REQUIRE(H % 16 == 0, "hidden size %lld must be a multiple of 16", (long long)H);
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
    KD_REQUIRE(Nq % 128 == 0 && Nq / 128 <= DL_MAX_UNITS, "QKV rows must be whole heads of 128");
    KD_REQUIRE(q_out->ndim == 4 && q_out->dtype == KD_BF16 && is_contiguous(q_out) && q_out->shape[0] == Mb && q_out->shape[1] == 1 &&
                   q_out->shape[3] == 128,
               "q_out must be contiguous bf16 [Mb,1,Hq,128]");
    Hq = (int)q_out->shape[2];
    KD_REQUIRE(k_cache_next->ndim == 4 && k_cache_next->dtype == KD_BF16 && v_cache_next->dtype == KD_BF16 &&
                   (block_table || k_cache_next->shape[0] >= Mb) && k_cache_next->shape[3] == 128 && k_cache_next->strides[3] == 1,
               "caches must be bf16 [B>=Mb,Hkv,maxS,128] (or pools [pages,Hkv,128,128] with a block table) with unit head_dim stride");
    if (block_table)
      KD_REQUIRE(block_table->dtype == KD_I32 && block_table->ndim == 2 && is_contiguous(block_table) && block_table->shape[0] >= Mb &&
                     k_cache_next->shape[2] == 128,
                 "block_table must be a contiguous int32 [B>=Mb, max_pages] tensor and the pools must have pages of 128 rows");
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
       *p_vc = nullptr, *p_q = nullptr, *p_xf = nullptr, *p_bt = nullptr;
  if (has_qkv) {
    KD_TRY(tensor_ptr(w_qkv_next, &p_wq)); KD_TRY(tensor_ptr(q_norm_w, &p_qw)); KD_TRY(tensor_ptr(k_norm_w, &p_kw));
    KD_TRY(tensor_ptr(cos, &p_cos)); KD_TRY(tensor_ptr(sin, &p_sin)); KD_TRY(tensor_ptr(pos, &p_pos));
    KD_TRY(tensor_ptr(k_cache_next, &p_kc)); KD_TRY(tensor_ptr(v_cache_next, &p_vc)); KD_TRY(tensor_ptr(q_out, &p_q));
    if (block_table) KD_TRY(tensor_ptr(block_table, &p_bt));
  } else {
    KD_TRY(tensor_ptr(x_final, &p_xf));
  }
  KD_REQUIRE(((reinterpret_cast<uintptr_t>(p_attn) | reinterpret_cast<uintptr_t>(p_wo) | reinterpret_cast<uintptr_t>(p_wgu) |
               reinterpret_cast<uintptr_t>(p_wd) | reinterpret_cast<uintptr_t>(p_wq)) & 15) == 0,
             "matrix operands must be 16-byte aligned");
  KD_REQUIRE(((reinterpret_cast<uintptr_t>(p_ri) | reinterpret_cast<uintptr_t>(p_ro) | reinterpret_cast<uintptr_t>(p_pn) |
               reinterpret_cast<uintptr_t>(p_nn) | reinterpret_cast<uintptr_t>(p_qw) | reinterpret_cast<uintptr_t>(p_kw) |
               reinterpret_cast<uintptr_t>(p_cos) | reinterpret_cast<uintptr_t>(p_sin) | reinterpret_cast<uintptr_t>(p_kc) |
               reinterpret_cast<uintptr_t>(p_vc) | reinterpret_cast<uintptr_t>(p_q) | reinterpret_cast<uintptr_t>(p_xf)) & 15) == 0,
             "residuals, norm weights, cos/sin, caches and outputs must be 16-byte aligned");
  if (has_qkv)
    for (int i = 0; i < 3; ++i) KD_REQUIRE(k_cache_next->strides[i] % 8 == 0, "cache strides must be multiples of 8 elements");

  DlParams p{};
  p.Mb = (int)Mb; p.H = (int)H; p.eps = eps;
  p.x_box = Mb <= 8 ? 8 : (Mb <= 16 ? 16 : (Mb <= 32 ? 32 : (Mb <= 64 ? 64 : 128)));
  p.has_qkv = has_qkv ? 1 : 0;
  const int dev = c.device;
  KD_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
  if (!g_dl_counters[dev]) {
    KD_CUDA_CHECK(cudaMalloc(&g_dl_counters[dev], DL_COUNTERS * sizeof(unsigned)));
    KD_CUDA_CHECK(cudaMemsetAsync(g_dl_counters[dev], 0, DL_COUNTERS * sizeof(unsigned), c.stream));
  }
  p.counters = g_dl_counters[dev];
  p.err = c.error_flag;
  static const bool want_trace = [] { const char* e = getenv("KD_DECODE_LAYER_TRACE"); return e && e[0] == '1'; }();
  if (want_trace && !g_dl_trace) KD_CUDA_CHECK(cudaMalloc(&g_dl_trace, (size_t)G * 16 * sizeof(unsigned long long)));
  if (g_dl_trace) KD_CUDA_CHECK(cudaMemsetAsync(g_dl_trace, 0, (size_t)G * 16 * sizeof(unsigned long long), c.stream));
  p.trace = g_dl_trace;

  struct Op { const void* w; int N, K, step; } ops[4] = {
      {p_wo, (int)H, (int)Ko, 16}, {p_wgu, (int)I2, (int)H, 32}, {p_wd, (int)H, (int)I, 16}, {p_wq, (int)Nq, (int)H, 128}};
  const int n_gemms = has_qkv ? 4 : 3;
  const int smem = DL_STAGES * DL_SLOT + 1024 + DL_RED_BYTES + 2048 + 1024;
  static bool configured[64] = {false};
  if (!configured[dev]) {      // before the occupancy queries below, which need the shared memory to be allowed
    KD_CUDA_CHECK(cudaFuncSetAttribute(decode_layer_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    configured[dev] = true;
  }
  const int x1 = p.x_box * DL_BK * 2;
  static const bool no_groups = [] { const char* e = getenv("KD_DL_NO_GROUPS"); return e && e[0] == '1'; }();
  auto grouped_of = [&](int K) { return K % DL_BK == 0 && !no_groups; };
  auto kg_of = [&](int n_unit, int K) {
    const int n_kb = (K + DL_BK - 1) / DL_BK;
    return grouped_of(K) ? std::max(1, std::min(std::min(DL_X_AREA / x1, DL_W_AREA / (n_unit * DL_BK * 2)), std::min(n_kb, 16))) : 1;
  };
  // experiment hooks: KD_DL_CLUSTER = 1 | 2 | 4 fixes the cluster size, KD_DL_N0 / N1 / N2 the unit width of a phase
  auto env_int = [](const char* name) { const char* e = getenv(name); return e ? atoi(e) : 0; };
  const int want_cluster = env_int("KD_DL_CLUSTER");
  const int want_n[3] = {env_int("KD_DL_N0"), env_int("KD_DL_N1"), env_int("KD_DL_N2")};
  DlPlanIn pin{};
  pin.Mb = (int)Mb; pin.x_box = p.x_box; pin.n_gemms = n_gemms; pin.tensor_parallel = tensor_parallel ? 1 : 0;
  pin.no_groups = no_groups ? 1 : 0;
  for (int i = 0; i < 4; ++i) { pin.N[i] = ops[i].N; pin.K[i] = ops[i].K; }
  for (int i = 0; i < 3; ++i) pin.want_n[i] = want_n[i];
  for (int cs = 1; cs <= 4; cs *= 2) {
    const bool allowed = !(want_cluster && cs != want_cluster) && !(cs > 1 && g_dl_no_clusters[dev]);
    pin.grid[cs] = allowed ? dl_cluster_grid(cs, smem) : 0;
  }
  DlGemm plan[4] = {};
  const int cluster = dl_make_plan(pin, plan);
  KD_REQUIRE(cluster > 0, "no launch configuration for these shapes (hidden %lld, %lld sequences)", (long long)H, (long long)Mb);
  G = dl_cluster_grid(cluster, smem);
  for (int i = 0; i < n_gemms; ++i) p.g[i] = plan[i];
  if (tensor_parallel) {
    P2pPeers peers;
    KD_TRY(p2p_peers(&peers));
    KD_REQUIRE((size_t)Mb * H * sizeof(float) <= P2P_SLOT_BYTES, "%lld x %lld fp32 partial sums do not fit the %zu-byte exchange slot",
               (long long)Mb, (long long)H, P2P_SLOT_BYTES);
    p.tp = peers.nranks;
    p.tp_rank = peers.rank;
    for (int r = 0; r < P2P_MAX_RANKS; ++r) p.peer[r] = peers.buf[r];
    p.tp_seq = peers.layer_seq;
    p.tp_wait = peers.wait_cycles;
  } else {
    p.tp = 1;
  }
  // scratch: h1, x1, x2, act, per-unit sums of squares
  size_t bytes = ((size_t)Mb * H + (size_t)(p.g[0].units + p.g[2].units) * Mb) * sizeof(float) +
                 ((size_t)2 * Mb * H + (size_t)Mb * I) * sizeof(__nv_bfloat16) + 256;
  void* ws = nullptr;
  KD_TRY(get_workspace(bytes, &ws));
  float* f = static_cast<float*>(ws);
  p.resid_mid = f; f += (size_t)Mb * H;
  p.ssq1 = f; f += (size_t)p.g[0].units * Mb;
  p.ssq2 = f; f += (size_t)p.g[2].units * Mb;
  __nv_bfloat16* h16 = reinterpret_cast<__nv_bfloat16*>((reinterpret_cast<uintptr_t>(f) + 127) & ~uintptr_t(127));
  p.x1 = h16; h16 += (size_t)Mb * H;
  p.x2 = h16; h16 += (size_t)Mb * H;
  p.act = h16;
  // Rotations: a phase's units go to CTAs that are idle in the phase before it, so that their weight
  // tiles are already in shared memory when the activations arrive.
  p.g[0].rot = 0;
  p.g[1].rot = (G - p.g[1].units % G) % G;
  p.g[2].rot = 0;
  p.g[3].rot = (p.g[2].units * p.g[2].split) % G;
  p.resid_in = static_cast<const float*>(p_ri);
  p.resid_out = static_cast<float*>(p_ro);
  p.w_post = static_cast<const __nv_bfloat16*>(p_pn);
  p.w_next = static_cast<const __nv_bfloat16*>(p_nn);
  p.Hq = Hq; p.Hkv = Hkv;
  if (has_qkv) {
    p.table = static_cast<const int*>(p_bt);
    p.max_pages = block_table ? (int)block_table->shape[1] : 0;
    p.max_s = block_table ? p.max_pages * 128 : (int)k_cache_next->shape[2];
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
    DlGemm& g = p.g[i];
    const int n_kb = (g.K + DL_BK - 1) / DL_BK;
    g.grouped = grouped_of(g.K) ? 1 : 0;
    g.kg = kg_of(g.n_unit, g.K);
    if (g.grouped) {
      // [k-block, row, 64]: the k-blocks of a row are 128 bytes apart, rows a whole row apart
      int rc = dl_tmap3(&maps.w[i], ops[i].w, DL_BK, (uint64_t)g.N, (uint64_t)n_kb, (uint64_t)g.K * 2, 128, (uint32_t)g.n_unit, (uint32_t)g.kg);
      if (rc == KD_OK) rc = dl_tmap3(&maps.x[i], xs[i], DL_BK, (uint64_t)Mb, (uint64_t)n_kb, (uint64_t)ldx[i] * 2, 128, (uint32_t)p.x_box, (uint32_t)g.kg);
      if (rc != KD_OK) { g.grouped = 0; g.kg = 1; }   // the driver refused the view: one k-block per copy
    }
    if (!g.grouped) {
      KD_TRY(dl_tmap3(&maps.w[i], ops[i].w, (uint64_t)g.K, (uint64_t)g.N, 1, (uint64_t)g.K * 2, (uint64_t)g.K * 2 * (uint64_t)g.N, (uint32_t)g.n_unit, 1));
      KD_TRY(dl_tmap3(&maps.x[i], xs[i], (uint64_t)g.K, (uint64_t)Mb, 1, (uint64_t)ldx[i] * 2, (uint64_t)ldx[i] * 2 * (uint64_t)Mb, (uint32_t)p.x_box, 1));
    }
  }
  if (n_gemms < 4) { maps.w[3] = maps.w[0]; maps.x[3] = maps.x[0]; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G);
  cfg.blockDim = dim3(DL_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = c.stream;
  cudaLaunchAttribute attr[3];
  cfg.attrs = attr;
  cfg.numAttrs = 0;
  // The CTAs wait for one another, so all of them must become resident together.  A cooperative
  // launch guarantees that, but it holds the whole grid back until the kernel before it has left
  // every SM the grid needs.  Inside a decode step (programmatic dependent launch enabled) the grid
  // is launched plainly instead, so that its CTAs start as SMs become free and fetch their first
  // weight tiles while the attention kernel drains (measured: 2.31 -> 2.27 ms per decode step at 32
  // sequences, 1.35 -> 1.30 at 4).  That is safe there: the grid is never larger than what the
  // occupancy query says fits an otherwise empty GPU; the kernels before it finish on their own; the
  // kernels after it are not started before every CTA of this grid has (they start when all CTAs have
  // executed launch_dependents); and should something else hold SMs for longer than the bounded
  // waits (about a second), the launch ends with an error code, not a hang.  KD_DL_COOP=1 / 0 forces
  // either form.
  static const int coop_env = [] { const char* e = getenv("KD_DL_COOP"); return e ? (e[0] == '0' ? 0 : 1) : -1; }();
  const bool cooperative = coop_env >= 0 ? coop_env == 1 : !c.pdl;
  if (cooperative) {
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.numAttrs = 1;
  }
  if (cluster > 1) {
    attr[cfg.numAttrs].id = cudaLaunchAttributeClusterDimension;
    attr[cfg.numAttrs].val.clusterDim.x = cluster;
    attr[cfg.numAttrs].val.clusterDim.y = 1;
    attr[cfg.numAttrs].val.clusterDim.z = 1;
    ++cfg.numAttrs;
  }
  if (c.pdl) {
    attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
    ++cfg.numAttrs;
  }
  const cudaError_t launched = cudaLaunchKernelEx(&cfg, decode_layer_kernel, maps, p);
  if (launched != cudaSuccess && cluster > 1 && !want_cluster) {
    // The clustered grid was refused (fewer SMs are available than the occupancy query promised, e.g.
    // under a profiler that keeps some for itself): plan again without clusters, from now on.
    cudaGetLastError();
    g_dl_no_clusters[dev] = true;
    return decode_layer_fused(tensor_parallel, attn, w_o, resid_in, post_norm_w, w_gate_up, w_down, next_norm_w, eps, w_qkv_next, q_norm_w,
                              k_norm_w, cos, sin, pos, k_cache_next, v_cache_next, block_table, q_out, resid_out, x_final);
  }
  KD_CUDA_CHECK(launched);
  return after_launch("decode_layer_kernel");
}

// The launch plan of kd_decode_layer_fused[_tp] for given shapes and grid sizes, without touching a
// device.  out: [0] cluster size (0: no configuration), then per phase 7 numbers: N, K, rows per
// unit, units, K split, k-blocks per CTA of a split group, k-blocks per bulk copy.
KD_API int kd_debug_decode_layer_plan(int sequences, int hidden, int attn_width, int inter, int qkv_rows, int tensor_parallel,
                                      int grid_plain, int grid_cluster2, int grid_cluster4, int* out, int out_len) {
  KD_REQUIRE(out && out_len >= 29, "out must hold 29 ints");
  KD_REQUIRE(sequences >= 1 && sequences <= 128 && hidden > 0 && attn_width > 0 && inter > 0 && qkv_rows >= 0, "bad shape");
  DlPlanIn in{};
  in.Mb = sequences;
  in.x_box = sequences <= 8 ? 8 : (sequences <= 16 ? 16 : (sequences <= 32 ? 32 : (sequences <= 64 ? 64 : 128)));
  in.n_gemms = qkv_rows > 0 ? 4 : 3;
  in.N[0] = hidden; in.K[0] = attn_width;
  in.N[1] = 2 * inter; in.K[1] = hidden;
  in.N[2] = hidden; in.K[2] = inter;
  in.N[3] = qkv_rows; in.K[3] = hidden;
  in.tensor_parallel = tensor_parallel ? 1 : 0;
  in.grid[1] = grid_plain; in.grid[2] = grid_cluster2; in.grid[4] = grid_cluster4;
  DlGemm plan[4] = {};
  out[0] = dl_make_plan(in, plan);
  for (int i = 0; i < 4; ++i) {
    int* o = out + 1 + 7 * i;
    o[0] = plan[i].N; o[1] = plan[i].K; o[2] = plan[i].n_unit; o[3] = plan[i].units; o[4] = plan[i].split; o[5] = plan[i].kb_per;
    o[6] = plan[i].kg;
  }
  return KD_OK;
}

KD_API int kd_decode_layer_fused(const kd_tensor* attn, const kd_tensor* w_o, const kd_tensor* resid_in,
                                 const kd_tensor* post_norm_w, const kd_tensor* w_gate_up, const kd_tensor* w_down,
                                 const kd_tensor* next_norm_w, float eps, const kd_tensor* w_qkv_next,
                                 const kd_tensor* q_norm_w, const kd_tensor* k_norm_w, const kd_tensor* cos,
                                 const kd_tensor* sin, const kd_tensor* pos, const kd_tensor* k_cache_next,
                                 const kd_tensor* v_cache_next, const kd_tensor* block_table, const kd_tensor* q_out,
                                 const kd_tensor* resid_out, const kd_tensor* x_final) {
  return decode_layer_fused(false, attn, w_o, resid_in, post_norm_w, w_gate_up, w_down, next_norm_w, eps, w_qkv_next, q_norm_w, k_norm_w,
                            cos, sin, pos, k_cache_next, v_cache_next, block_table, q_out, resid_out, x_final);
}

KD_API int kd_decode_layer_fused_tp(const kd_tensor* attn, const kd_tensor* w_o, const kd_tensor* resid_in,
                                    const kd_tensor* post_norm_w, const kd_tensor* w_gate_up, const kd_tensor* w_down,
                                    const kd_tensor* next_norm_w, float eps, const kd_tensor* w_qkv_next,
                                    const kd_tensor* q_norm_w, const kd_tensor* k_norm_w, const kd_tensor* cos,
                                    const kd_tensor* sin, const kd_tensor* pos, const kd_tensor* k_cache_next,
                                    const kd_tensor* v_cache_next, const kd_tensor* block_table, const kd_tensor* q_out,
                                    const kd_tensor* resid_out, const kd_tensor* x_final) {
  return decode_layer_fused(true, attn, w_o, resid_in, post_norm_w, w_gate_up, w_down, next_norm_w, eps, w_qkv_next, q_norm_w, k_norm_w,
                            cos, sin, pos, k_cache_next, v_cache_next, block_table, q_out, resid_out, x_final);
}
