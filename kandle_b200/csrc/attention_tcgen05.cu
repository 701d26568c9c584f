// Key `flash_attention` for bf16 tensors on the 5th-generation tensor cores (prefill shapes).
//
// Same mathematics as the reference's fused attention shader
// (packages/backend-webgpu/src/kernels/attention/builder.ts:138-329: GQA head map, score =
// dot*scale, causal mask top-left aligned, online softmax, O/l), re-tiled for sm_100a:
//
//   CTA = one 128-row query tile of one (batch, q-head); 192 threads.
//   warp 0     TMA producer: Q tile once, then 128-row K and V tiles through a 2-stage ring
//              (plain tiled loads with 128-byte swizzle, one 64-wide head-dim slab per load).
//   warp 1     one elected thread issues tcgen05.mma:
//                S = Q K^T   (A = Q in smem, K-major; B = K tile, K-major; fp32 S in TMEM, 2 buffers)
//                O += P V    (A = P read from TMEM as packed bf16; B = V tile, MN-major)
//   warps 2-5  softmax: each thread owns one query row; tcgen05.ld the S row, scale, mask,
//              running max / sum in registers (exp2 with the scale folded in), write P back into
//              the S buffer as packed bf16 (tcgen05.st), rescale O in TMEM only when the running
//              max grew by more than 2^8 (the accumulated sum uses the same stale max, so the
//              result is exact), and finally O/l -> bf16 -> global.
//   QK^T of block j+1 is issued before softmax(j) finishes, so the tensor pipe overlaps the softmax.
//
// Causal tiles stop at the diagonal block (only that block is masked element-wise); key columns
// beyond Skv in the last block are masked.  Heavy (late) query tiles are scheduled first.
//
// Roofline: tensor-core bound, 4*B*Hq*D*P flops (P = number of unmasked (q,k) pairs).
#include "common.cuh"
#include "kernels.cuh"
#include "sm100.cuh"

namespace kd {

using namespace sm100;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [b, h, s, d] bf16 tensor with element strides st[0..2] (d contiguous); box = [1,1,box_rows,64].
static int make_tmap_bhsd(CUtensorMap* out, const void* base, const int64_t* ext, const int64_t* st, uint32_t box_rows) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  if (!fn) return fail(KD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[4] = {(cuuint64_t)ext[3], (cuuint64_t)ext[2], (cuuint64_t)ext[1], (cuuint64_t)ext[0]};
  cuuint64_t gstr[3] = {(cuuint64_t)st[2] * 2, (cuuint64_t)st[1] * 2, (cuuint64_t)st[0] * 2};
  // a dimension of extent 1 may carry any stride; the encoder still wants a multiple of 16 bytes
  for (int i = 0; i < 3; ++i)
    if (gdim[i + 1] == 1) gstr[i] = (i == 0 ? (cuuint64_t)ext[3] * 2 : gstr[i - 1] * gdim[i]);
  cuuint32_t box[4] = {64, box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), gdim, gstr, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(KD_ERR_CUDA, "cuTensorMapEncodeTiled (attention) failed with code %d", (int)r);
  return KD_OK;
}

struct FaParams {
  int B, Hq, Hkv, Sq, Skv;
  int causal;
  float scale_log2;  // scale * log2(e)
  __nv_bfloat16* o;
  int64_t so_b, so_h, so_s;
  int num_q_tiles;
  int* err;
};

constexpr int FA_BQ = 128;
constexpr int FA_BKV = 128;
constexpr int FA_THREADS = 192;
constexpr int FA_STAGES = 2;

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                               const __grid_constant__ CUtensorMap tmap_v, FaParams p) {
  constexpr int SLABS = D / 64;                     // 64-wide head-dim slabs (one swizzle atom each)
  constexpr int Q_BYTES = FA_BQ * D * 2;
  constexpr int KV_BYTES = FA_BKV * D * 2;
  constexpr int SLAB_BYTES = FA_BKV * 128;          // 128 rows x 128 B
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL0 = 0, O_COL0 = 256;      // S buffers at columns 0 and 128, O at 256
  constexpr uint32_t IDESC_QK = make_idesc_bf16(FA_BQ, FA_BKV, 0, 0);
  constexpr uint32_t IDESC_PV = make_idesc_bf16(FA_BQ, D, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;
  uint8_t* k_smem = q_smem + Q_BYTES;                       // [STAGES][KV_BYTES]
  uint8_t* v_smem = k_smem + FA_STAGES * KV_BYTES;          // [STAGES][KV_BYTES]
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + FA_STAGES * KV_BYTES);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = bars + 1;             // 2
  uint64_t* k_empty = bars + 3;            // 2
  uint64_t* v_full = bars + 5;             // 2
  uint64_t* v_empty = bars + 7;            // 2
  uint64_t* s_full = bars + 9;             // 2
  uint64_t* p_ready = bars + 11;           // 2
  uint64_t* o_done = bars + 13;            // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = p.num_q_tiles - 1 - (int)blockIdx.x;   // heavy causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = q_tile * FA_BQ;
  int kv_end = p.Skv;
  if (p.causal) kv_end = min(p.Skv, q0 + FA_BQ);
  const int n_blocks = (kv_end + FA_BKV - 1) / FA_BKV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FA_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&p_ready[s], 4); }
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int s = 0; s < SLABS; ++s) tma_load_4d(q_smem + s * SLAB_BYTES, &tmap_q, q_full, s * 64, q0, h, b);
      int stage = 0;
      uint32_t phase = 0;
      for (int j = 0; j < n_blocks; ++j) {
        if (!mbar_wait(&k_empty[stage], phase ^ 1, abort_flag, p.err, 301)) break;
        mbar_arrive_expect_tx(&k_full[stage], KV_BYTES);
#pragma unroll
        for (int s = 0; s < SLABS; ++s)
          tma_load_4d(k_smem + stage * KV_BYTES + s * SLAB_BYTES, &tmap_k, &k_full[stage], s * 64, j * FA_BKV, hk, b);
        if (!mbar_wait(&v_empty[stage], phase ^ 1, abort_flag, p.err, 302)) break;
        mbar_arrive_expect_tx(&v_full[stage], KV_BYTES);
#pragma unroll
        for (int s = 0; s < SLABS; ++s)
          tma_load_4d(v_smem + stage * KV_BYTES + s * SLAB_BYTES, &tmap_v, &v_full[stage], s * 64, j * FA_BKV, hk, b);
        if (++stage == FA_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, 303);
      const uint32_t q_addr = smem_u32(q_smem);
      // S(j) = Q K(j)^T into S buffer j&1
      auto issue_qk = [&](int j) -> bool {
        const int stage = j % FA_STAGES;
        if (!mbar_wait(&k_full[stage], (uint32_t)((j / FA_STAGES) & 1), abort_flag, p.err, 304)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(k_smem + stage * KV_BYTES);
        const uint32_t d_tmem = tmem_base + S_COL0 + (uint32_t)((j & 1) * FA_BKV);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (uint32_t)((k / 4) * SLAB_BYTES + (k % 4) * 32);
          umma_ss(d_tmem, make_smem_desc_sw128(q_addr + off, 16, 1024), make_smem_desc_sw128(k_addr + off, 16, 1024),
                  IDESC_QK, k != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[stage]);
        umma_commit(&s_full[j & 1]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; ok && j < n_blocks; ++j) {
        if (j + 1 < n_blocks) {
          if (!issue_qk(j + 1)) break;
        }
        const int stage = j % FA_STAGES;
        if (!mbar_wait(&p_ready[j & 1], (uint32_t)((j >> 1) & 1), abort_flag, p.err, 305)) break;
        if (!mbar_wait(&v_full[stage], (uint32_t)((j / FA_STAGES) & 1), abort_flag, p.err, 306)) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(v_smem + stage * KV_BYTES);
        const uint32_t p_tmem = tmem_base + S_COL0 + (uint32_t)((j & 1) * FA_BKV);
        const uint32_t o_tmem = tmem_base + O_COL0;
#pragma unroll
        for (int k = 0; k < FA_BKV / 16; ++k) {
          // V tile is [kv rows][64-wide d slabs]: MN-major B; 16 kv rows = 2048 bytes per k step
          const uint64_t vdesc = make_smem_desc_sw128(v_addr + (uint32_t)(k * 2048), SLAB_BYTES, 1024);
          umma_ts(o_tmem, p_tmem + (uint32_t)(k * 8), vdesc, IDESC_PV, (j | k) != 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[stage]);
        umma_commit(o_done);
      }
    }
  } else {
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const int row = q0 + row_in_tile;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    float m_used = -1e30f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      ok = mbar_wait(&s_full[j & 1], (uint32_t)((j >> 1) & 1), abort_flag, p.err, 307);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_addr = lane_addr + S_COL0 + (uint32_t)((j & 1) * FA_BKV);
      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(s_addr + c * 32, sr[c]);
      tmem_wait_ld();
      const int kv0 = j * FA_BKV;
      // Only the diagonal block of a causal tile and the last (ragged) key block need masking;
      // the test is hoisted so that the common path carries no per-element predicates.
      if ((kv0 + FA_BKV > kv_end) || (p.causal && kv0 + FA_BKV - 1 > q0)) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = kv0 + c * 32 + i;
            if (col >= p.Skv || (p.causal && col > row)) sr[c][i] = __float_as_uint(-1e30f);
          }
      }
      float mx0 = -1e30f, mx1 = -1e30f;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mx0 = fmaxf(mx0, fmaxf(__uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1])));
          mx1 = fmaxf(mx1, fmaxf(__uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3])));
        }
      // scores are scaled inside the exponential: exp2(s*c - m*c) with c = scale*log2(e) > 0
      const float m_blk = fmaxf(mx0, mx1) * p.scale_log2;
      // Lazy rescale: keep the stale max unless it is more than 2^8 too small.
      float alpha = 1.f;
      bool rescale = false;
      if (j == 0) {
        m_used = m_blk;
      } else if (m_blk - m_used > 8.0f) {
        alpha = fast_exp2(m_used - m_blk);
        m_used = m_blk;
        rescale = true;
      }
      if (__any_sync(0xffffffffu, rescale)) {
        // O holds the sum over blocks < j; PV(j-1) must have completed before touching it.
        ok = mbar_wait(o_done, (uint32_t)((j - 1) & 1), abort_flag, p.err, 308);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t orr[32];
          tmem_ld_32x32(lane_addr + O_COL0 + c * 32, orr);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
          tmem_st_32x32(lane_addr + O_COL0 + c * 32, orr);
        }
        l *= alpha;
      }
      // P = exp2(s - m_used) as packed bf16 into the first 64 columns of this S buffer
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int e = c * 64 + 2 * i;
          const float p0 = fast_exp2(fmaf(__uint_as_float(sr[e >> 5][e & 31]), p.scale_log2, -m_used));
          const float p1 = fast_exp2(fmaf(__uint_as_float(sr[(e + 1) >> 5][(e + 1) & 31]), p.scale_log2, -m_used));
          sum0 += p0;
          sum1 += p1;
          __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
          pk[i] = *reinterpret_cast<uint32_t*>(&v);
        }
        tmem_st_32x32(s_addr + c * 32, pk);
      }
      l += sum0 + sum1;
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[j & 1]);
    }
    if (ok) {
      ok = mbar_wait(o_done, (uint32_t)((n_blocks - 1) & 1), abort_flag, p.err, 309);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.0f / l;
      __nv_bfloat16* orow = p.o + (int64_t)b * p.so_b + (int64_t)h * p.so_h + (int64_t)row * p.so_s;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t orr[32];
        tmem_ld_32x32(lane_addr + O_COL0 + c * 32, orr);
        tmem_wait_ld();
        if (row < p.Sq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            uint32_t* vv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(orr[g * 8 + 2 * e]) * inv_l,
                                                       __uint_as_float(orr[g * 8 + 2 * e + 1]) * inv_l);
              vv[e] = *reinterpret_cast<uint32_t*>(&t);
            }
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = v;
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
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D>
static int launch_fa(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& p) {
  constexpr int SMEM = FA_BQ * D * 2 + 2 * FA_STAGES * FA_BKV * D * 2 + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    KD_CUDA_CHECK(cudaFuncSetAttribute(flash_attention_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured = true;
  }
  dim3 grid(p.num_q_tiles, p.Hq, p.B);
  flash_attention_tcgen05_kernel<D><<<grid, FA_THREADS, SMEM, ctx().stream>>>(tq, tk, tv, p);
  return after_launch("flash_attention_tcgen05_kernel");
}

int attention_tc_try(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v, const kd_tensor* out,
                     const AttnParams& a, int* handled) {
  *handled = 0;
  if (a.dt_q != KD_BF16 || a.dt_k != KD_BF16 || a.dt_v != KD_BF16 || a.dt_o != KD_BF16) return KD_OK;
  if (a.D != 64 && a.D != 128) return KD_OK;
  if (!(a.scale > 0.f)) return KD_OK;  // the kernel takes the row max before scaling
  if (a.Sq < 16) return KD_OK;  // single-row (decode) shapes are bandwidth-bound: CUDA-core / split-KV kernels
  if (a.B == 0 || a.Hq == 0 || a.Skv == 0) return KD_OK;
  if (a.Hq > 65535 || a.B > 65535) return KD_OK;
  if (a.sq[3] != 1 || a.sk[3] != 1 || a.sv[3] != 1 || a.so[3] != 1) return KD_OK;
  for (int i = 0; i < 3; ++i) {
    if ((a.sq[i] % 8) || (a.sk[i] % 8) || (a.sv[i] % 8) || (a.so[i] % 8)) return KD_OK;
  }
  void *pq = nullptr, *pk = nullptr, *pv = nullptr, *po = nullptr;
  KD_TRY(tensor_ptr(q, &pq));
  KD_TRY(tensor_ptr(k, &pk));
  KD_TRY(tensor_ptr(v, &pv));
  KD_TRY(tensor_ptr(out, &po));
  if ((reinterpret_cast<uintptr_t>(pq) | reinterpret_cast<uintptr_t>(pk) | reinterpret_cast<uintptr_t>(pv) |
       reinterpret_cast<uintptr_t>(po)) & 15)
    return KD_OK;
  const int64_t eq[4] = {a.B, a.Hq, a.Sq, a.D}, ek[4] = {a.B, a.Hkv, a.Skv, a.D};
  CUtensorMap tq, tk, tv;
  KD_TRY(make_tmap_bhsd(&tq, pq, eq, a.sq, FA_BQ));
  KD_TRY(make_tmap_bhsd(&tk, pk, ek, a.sk, FA_BKV));
  KD_TRY(make_tmap_bhsd(&tv, pv, ek, a.sv, FA_BKV));
  FaParams p{};
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Sq = a.Sq; p.Skv = a.Skv;
  p.causal = a.causal;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.o = static_cast<__nv_bfloat16*>(po);
  p.so_b = a.so[0]; p.so_h = a.so[1]; p.so_s = a.so[2];
  p.num_q_tiles = (a.Sq + FA_BQ - 1) / FA_BQ;
  p.err = ctx().error_flag;
  if (a.D == 128) KD_TRY(launch_fa<128>(tq, tk, tv, p));
  else KD_TRY(launch_fa<64>(tq, tk, tv, p));
  *handled = 1;
  return KD_OK;
}

}  // namespace kd
