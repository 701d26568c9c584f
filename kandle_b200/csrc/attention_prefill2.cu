// Key `flash_attention`, bf16 prefill shapes: two query sub-tiles per CTA share every K/V tile.
//
// The one-tile kernel (attention_tcgen05.cu) re-reads all of K and V for every 128-row query tile
// of every query head; at 2048-token prompts that is several TB/s of L2 -> shared-memory traffic,
// which, not the tensor pipe or the softmax, bounds it.  Here a CTA owns TWO 128-row sub-tiles
// that use the same K/V stream:
//   - with grouped-query attention (an even number of query heads per KV head): the same query rows
//     of two heads of one KV group;
//   - otherwise: two consecutive query tiles of one head (the second may run one block longer under
//     the causal mask, or be absent at the end of the sequence).
// so every K/V tile fetched into shared memory feeds two S = QK^T and two O += PV products.
//
//   warps 0-3   softmax + epilogue of sub-tile A (one query row per thread)
//   warps 4-7   the same for sub-tile B
//   warp 8      TMA producer: both Q tiles once, then K/V tiles through a 4-slot ring
//   warp 9      tcgen05.mma issuer, order  QK_A(0) QK_B(0) | PV_A(j) QK_A(j+1) PV_B(j) QK_B(j+1) | ...
//               so the tensor pipe works on one sub-tile while the other's softmax runs
//   warps 10-11 idle: they complete the third warpgroup, which hands most of its registers to the
//               softmax warpgroups (setmaxnreg: 56 against 224 per thread)
// TMEM (512 columns): S_A, S_B (fp32, overwritten in place by P as packed bf16), O_A, O_B.
// The softmax reads its S row (128 scores) from tensor memory ONCE and keeps it in registers for the
// maximum and the exponentials; P is handed to the MMA warp in two halves of 64 keys, so that the
// first four k-steps of P V run while the second half is still being exponentiated.  The softmax
// warps are bound by the instructions they issue (the special-function unit, at 16 exponentials per
// clock and SM, would allow slightly more), so the arithmetic around the exponential is packed:
// three-input maxima, two-wide fused multiply-adds and adds (max.f32 with three operands,
// fma.rn.f32x2, add.rn.f32x2): 3 instructions per score instead of 4.5.  Computing a quarter of the
// exponentials on the FMA pipe instead (round-to-nearest split, cubic polynomial, exponent added
// with integer arithmetic) was measured and made the kernel 7 % slower: more instructions.  Mathematics as in attention_tcgen05.cu / the reference
// shader (packages/backend-webgpu/src/kernels/attention/builder.ts:138-329).
#include "common.cuh"
#include "kernels.cuh"
#include "sm100.cuh"

namespace kd {

using namespace sm100;

__device__ __forceinline__ float fa2_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float fa2_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// (x0, x1) = (a0, a1) * s + m
__device__ __forceinline__ void fa2_fma2(float& x0, float& x1, float a0, float a1, float s, float m) {
  asm("{\n\t.reg .b64 a, b, c, d;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %4};\n\tmov.b64 c, {%5, %5};\n\t"
      "fma.rn.f32x2 d, a, b, c;\n\tmov.b64 {%0, %1}, d;\n\t}"
      : "=f"(x0), "=f"(x1) : "f"(a0), "f"(a1), "f"(s), "f"(m));
}
// (s0, s1) += (a0, a1)
__device__ __forceinline__ void fa2_add2(float& s0, float& s1, float a0, float a1) {
  asm("{\n\t.reg .b64 a, b, d;\n\tmov.b64 a, {%0, %1};\n\tmov.b64 b, {%2, %3};\n\tadd.rn.f32x2 d, a, b;\n\tmov.b64 {%0, %1}, d;\n\t}"
      : "+f"(s0), "+f"(s1) : "f"(a0), "f"(a1));
}

struct Fa2Params {
  int B, Hq, Hkv, Sq, Skv;
  int causal;
  int pair_heads;      // 1: sub-tiles are two heads of one KV group; 0: two consecutive query tiles
  int num_q_tiles;     // 128-row tiles in Sq
  float scale_log2;
  __nv_bfloat16* o;
  int64_t so_b, so_h, so_s;
  int* err;
};

constexpr int FA2_BQ = 128, FA2_BKV = 128, FA2_THREADS = 384, FA2_NSLOT = 4;

template <int D>
__global__ void __launch_bounds__(FA2_THREADS, 1)
flash_attention_prefill2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                                const __grid_constant__ CUtensorMap tmap_v, Fa2Params p) {
  constexpr int SLABS = D / 64;
  constexpr int Q_BYTES = FA2_BQ * D * 2;
  constexpr int KV_BYTES = FA2_BKV * D * 2;
  constexpr int SLAB_BYTES = FA2_BKV * 128;
  constexpr uint32_t TMEM_COLS = 512;
  // TMEM columns: S of sub-tile t at 128 t, O at 256 + D t
  constexpr uint32_t IDESC_QK = make_idesc_bf16(FA2_BQ, FA2_BKV, 0, 0);
  constexpr uint32_t IDESC_PV = make_idesc_bf16(FA2_BQ, D, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;                                  // [2][Q_BYTES]
  uint8_t* ring = q_smem + 2 * Q_BYTES;                    // [NSLOT][KV_BYTES]: K0 V0 K1 V1 ...
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + FA2_NSLOT * KV_BYTES);
  uint64_t* q_full = bars;          // 1
  uint64_t* t_full = bars + 1;      // 4
  uint64_t* t_empty = bars + 5;     // 4
  uint64_t* s_full = bars + 9;      // 2 (per sub-tile)
  uint64_t* p_ready = bars + 11;    // 4: [sub-tile][half of the keys]
  uint64_t* o_done = bars + 15;     // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  // sub-tile coordinates
  int head[2], q0[2], nblk[2], kv_end[2];
  int hk;
  {
    const int x = (int)gridDim.x - 1 - (int)blockIdx.x;     // heavy causal tiles first
    if (p.pair_heads) {
      head[0] = 2 * blockIdx.y; head[1] = head[0] + 1;
      q0[0] = q0[1] = x * FA2_BQ;
    } else {
      head[0] = head[1] = blockIdx.y;
      q0[0] = 2 * x * FA2_BQ; q0[1] = q0[0] + FA2_BQ;
    }
    hk = head[0] / (p.Hq / p.Hkv);
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (q0[t] >= p.Sq) { nblk[t] = 0; kv_end[t] = 0; continue; }
      kv_end[t] = p.causal ? min(p.Skv, q0[t] + FA2_BQ) : p.Skv;
      nblk[t] = (kv_end[t] + FA2_BKV - 1) / FA2_BKV;
    }
  }
  const int n_blocks = max(nblk[0], nblk[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FA2_NSLOT; ++s) { mbar_init(&t_full[s], 1); mbar_init(&t_empty[s], 1); }
    for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&o_done[t], 1); }
    for (int t = 0; t < 4; ++t) mbar_init(&p_ready[t], 4);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  if (warp == 8) {
    if (lane == 0) {
      // an absent second sub-tile still gets a (zero-filled, out-of-range) load so that the byte count is fixed
      mbar_arrive_expect_tx(q_full, 2 * Q_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int s = 0; s < SLABS; ++s)
          tma_load_4d(q_smem + t * Q_BYTES + s * SLAB_BYTES, &tmap_q, q_full, s * 64, q0[t], head[t], b);
      for (int j = 0; j < n_blocks; ++j) {
        const int tk = 2 * j, tv = 2 * j + 1;
        const int sk = tk % FA2_NSLOT, sv = tv % FA2_NSLOT;
        if (!mbar_wait(&t_empty[sk], (uint32_t)(((tk / FA2_NSLOT) & 1) ^ 1), abort_flag, p.err, 401)) break;
        mbar_arrive_expect_tx(&t_full[sk], KV_BYTES);
#pragma unroll
        for (int s = 0; s < SLABS; ++s)
          tma_load_4d(ring + sk * KV_BYTES + s * SLAB_BYTES, &tmap_k, &t_full[sk], s * 64, j * FA2_BKV, hk, b);
        if (!mbar_wait(&t_empty[sv], (uint32_t)(((tv / FA2_NSLOT) & 1) ^ 1), abort_flag, p.err, 402)) break;
        mbar_arrive_expect_tx(&t_full[sv], KV_BYTES);
#pragma unroll
        for (int s = 0; s < SLABS; ++s)
          tma_load_4d(ring + sv * KV_BYTES + s * SLAB_BYTES, &tmap_v, &t_full[sv], s * 64, j * FA2_BKV, hk, b);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, 403);
      // S_t(j) = Q_t K(j)^T.  The K tile is waited for once per block (by whichever sub-tile comes first).
      auto issue_qk = [&](int t, int j, bool wait_k) -> bool {
        const int stage = (2 * j) % FA2_NSLOT;
        if (wait_k && !mbar_wait(&t_full[stage], (uint32_t)(((2 * j) / FA2_NSLOT) & 1), abort_flag, p.err, 404)) return false;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(q_smem + t * Q_BYTES);
        const uint32_t k_addr = smem_u32(ring + stage * KV_BYTES);
        const uint32_t d_tmem = tmem_base + (uint32_t)(t * 128);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (uint32_t)((k / 4) * SLAB_BYTES + (k % 4) * 32);
          umma_ss(d_tmem, make_smem_desc_sw128(q_addr + off, 16, 1024), make_smem_desc_sw128(k_addr + off, 16, 1024),
                  IDESC_QK, k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
        return true;
      };
      // the K slot of block j is released after the last QK^T that reads it
      auto release_k = [&](int j) { umma_commit(&t_empty[(2 * j) % FA2_NSLOT]); };
      auto issue_pv = [&](int t, int j, bool wait_v) -> bool {
        const int stage = (2 * j + 1) % FA2_NSLOT;
        if (wait_v && !mbar_wait(&t_full[stage], (uint32_t)(((2 * j + 1) / FA2_NSLOT) & 1), abort_flag, p.err, 406)) return false;
        const uint32_t v_addr = smem_u32(ring + stage * KV_BYTES);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (!mbar_wait(&p_ready[2 * t + half], (uint32_t)(j & 1), abort_flag, p.err, 405)) return false;
          tc_fence_after();
#pragma unroll
          for (int k = 4 * half; k < 4 * half + 4; ++k) {
            const uint64_t vdesc = make_smem_desc_sw128(v_addr + (uint32_t)(k * 2048), SLAB_BYTES, 1024);
            umma_ts(tmem_base + (uint32_t)(256 + t * D), tmem_base + (uint32_t)(t * 128 + k * 8), vdesc, IDESC_PV, (j | k) != 0 ? 1u : 0u);
          }
        }
        umma_commit(&o_done[t]);
        return true;
      };
      if (ok && n_blocks > 0) {
        const bool a0 = nblk[0] > 0, b0 = nblk[1] > 0;
        if (a0) ok = issue_qk(0, 0, true);
        if (ok && b0) ok = issue_qk(1, 0, !a0);
        if (ok) release_k(0);
      }
      for (int j = 0; ok && j < n_blocks; ++j) {
        const bool a_now = j < nblk[0], b_now = j < nblk[1];
        const bool a_next = j + 1 < nblk[0], b_next = j + 1 < nblk[1];
        if (a_now) ok = issue_pv(0, j, true);
        if (ok && a_next) ok = issue_qk(0, j + 1, true);
        if (ok && b_now) ok = issue_pv(1, j, !a_now);
        if (ok) umma_commit(&t_empty[(2 * j + 1) % FA2_NSLOT]);          // V slot of block j
        if (ok && b_next) ok = issue_qk(1, j + 1, !a_next);
        if (ok && (a_next || b_next)) release_k(j + 1);
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int t = warp >> 2;                // sub-tile of this warpgroup
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const int my_q0 = t ? q0[1] : q0[0], my_head = t ? head[1] : head[0];
    const int my_kv_end = t ? kv_end[1] : kv_end[0];
    const int row = my_q0 + row_in_tile;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t s_addr = lane_addr + (uint32_t)(t * 128);
    const uint32_t o_addr = lane_addr + (uint32_t)(256 + t * D);
    const int nb = t ? nblk[1] : nblk[0];
    float m_used = -1e30f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nb; ++j) {
      ok = mbar_wait(&s_full[t], (uint32_t)(j & 1), abort_flag, p.err, 407);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int kv0 = j * FA2_BKV;
      const bool masked = (kv0 + FA2_BKV > my_kv_end) || (p.causal && kv0 + FA2_BKV - 1 > my_q0);
      // the whole S row of this thread, once
      uint32_t r[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(s_addr + c * 32, r + c * 32);
      tmem_wait_ld();
      if (masked) {
        // key kv0 + i is visible to this row iff i <= lim
        const int lim = (p.causal ? min(p.Skv - 1, row) : p.Skv - 1) - kv0;
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i > lim) r[i] = __float_as_uint(-1e30f);
      }
      float mx0 = -1e30f, mx1 = -1e30f, mx2 = -1e30f, mx3 = -1e30f;
#pragma unroll
      for (int i = 0; i < 128; i += 8) {
        mx0 = fa2_max3(mx0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
        mx1 = fa2_max3(mx1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
        mx2 = fa2_max3(mx2, __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
        mx3 = fa2_max3(mx3, __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
      }
      const float m_blk = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
      float alpha = 1.f;
      bool rescale = false;
      if (j == 0) {
        m_used = m_blk;
      } else if (m_blk - m_used > 8.0f) {      // lazy rescale, see attention_tcgen05.cu
        alpha = fa2_exp2(m_used - m_blk);
        m_used = m_blk;
        rescale = true;
      }
      if (__any_sync(0xffffffffu, rescale)) {
        ok = mbar_wait(&o_done[t], (uint32_t)((j - 1) & 1), abort_flag, p.err, 408);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < D / 16; ++c) {      // narrow chunks: the 128 scores stay in registers meanwhile
          uint32_t orr[16];
          tmem_ld_32x16(o_addr + c * 16, orr);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
          tmem_st_32x16(o_addr + c * 16, orr);
        }
        l *= alpha;
      }
      // P = exp2(s*c - m) as packed bf16 over the first 64 columns of S (packed column k holds keys
      // 2k, 2k+1), written and handed over in two halves of 64 keys.  The packed values replace the
      // scores in r[] from the front (r[i] <- keys 2i, 2i+1: never ahead of what is still to be read).
      float sum0 = 0.f, sum1 = 0.f;
      const float neg_m = -m_used;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int i = 32 * half; i < 32 * half + 32; ++i) {
          float x0, x1;
          fa2_fma2(x0, x1, __uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]), p.scale_log2, neg_m);
          const float e0 = fa2_exp2(x0), e1 = fa2_exp2(x1);
          fa2_add2(sum0, sum1, e0, e1);
          __nv_bfloat162 v = __floats2bfloat162_rn(e0, e1);
          r[i] = *reinterpret_cast<uint32_t*>(&v);
        }
        tmem_st_32x32(s_addr + half * 32, r + half * 32);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[2 * t + half]);
      }
      l += sum0 + sum1;
    }
    if (ok && nb > 0) {
      ok = mbar_wait(&o_done[t], (uint32_t)((nb - 1) & 1), abort_flag, p.err, 409);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && nb > 0) {
      tc_fence_after();
      const float inv_l = 1.0f / l;
      __nv_bfloat16* orow = p.o + (int64_t)b * p.so_b + (int64_t)my_head * p.so_h + (int64_t)row * p.so_s;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t orr[32];
        tmem_ld_32x32(o_addr + c * 32, orr);
        tmem_wait_ld();
        if (row < p.Sq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            uint32_t* vv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 tt = __floats2bfloat162_rn(__uint_as_float(orr[g * 8 + 2 * e]) * inv_l,
                                                        __uint_as_float(orr[g * 8 + 2 * e + 1]) * inv_l);
              vv[e] = *reinterpret_cast<uint32_t*>(&tt);
            }
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = v;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D>
static int launch_fa2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const Fa2Params& p, dim3 grid) {
  constexpr int SMEM = 2 * FA2_BQ * D * 2 + FA2_NSLOT * FA2_BKV * D * 2 + 1024 + 256;
  static bool configured[64] = {false};   // per device: kd_shutdown + kd_init may move the library to another GPU
  if (!configured[ctx().device & 63]) {
    KD_CUDA_CHECK(cudaFuncSetAttribute(flash_attention_prefill2_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured[ctx().device & 63] = true;
  }
  flash_attention_prefill2_kernel<D><<<grid, FA2_THREADS, SMEM, ctx().stream>>>(tq, tk, tv, p);
  return after_launch("flash_attention_prefill2_kernel");
}

int attention_prefill2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& a, void* out) {
  Fa2Params p{};
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Sq = a.Sq; p.Skv = a.Skv;
  p.causal = a.causal;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.o = static_cast<__nv_bfloat16*>(out);
  p.so_b = a.so[0]; p.so_h = a.so[1]; p.so_s = a.so[2];
  p.num_q_tiles = (a.Sq + FA2_BQ - 1) / FA2_BQ;
  p.err = ctx().error_flag;
  const int group = a.Hq / a.Hkv;
  p.pair_heads = (group % 2 == 0) ? 1 : 0;
  dim3 grid;
  if (p.pair_heads) grid = dim3(p.num_q_tiles, a.Hq / 2, a.B);
  else grid = dim3((p.num_q_tiles + 1) / 2, a.Hq, a.B);
  if (a.D == 128) return launch_fa2<128>(tq, tk, tv, p, grid);
  return launch_fa2<64>(tq, tk, tv, p, grid);
}

}  // namespace kd
