// Key `flash_attention` for bf16 tensors on the 5th-generation tensor cores (prefill shapes).
//
// Same mathematics as the reference's fused attention shader
// (packages/backend-webgpu/src/kernels/attention/builder.ts:138-329: GQA head map, score =
// dot*scale, causal mask top-left aligned, online softmax, O/l), re-tiled for sm_100a:
//
//   CTA = one 128-row query tile of one (batch, q-head); 320 threads (192 in decode mode).
//   warp 0     TMA producer: Q tile once, then 128-row K and V tiles through a 2-stage ring
//              (plain tiled loads with 128-byte swizzle, one 64-wide head-dim slab per load).
//   warp 1     one elected thread issues tcgen05.mma:
//                S = Q K^T   (A = Q in smem, K-major; B = K tile, K-major; fp32 S in TMEM, 2 buffers)
//                O += P V    (A = P read from TMEM as packed bf16; B = V tile, MN-major)
//   warps 2-9  softmax, two warpgroups that split the key columns of every row (decode: one
//              warpgroup); each thread: tcgen05.ld its part of the S row, scale, mask,
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
//
// DECODE mode (one new token per sequence against a KV cache) reuses the same pipeline with the
// query tile holding the Hq/Hkv query heads that share one KV head (the other rows of the 128-row
// MMA tile are zero padding, which costs nothing: the kernel is HBM-bound).  The key range of a
// (batch, kv-head) pair is split across CTAs (split-KV); each CTA writes an un-normalised partial
// output plus its (max, sum) statistics to scratch and a second kernel combines the splits.  The
// context length is read from device memory so that a captured CUDA graph can be replayed while
// the sequence grows.  The cache is either contiguous [B,Hkv,maxS,D] (the reference's
// StaticKVCache layout, packages/model-utils/src/kv-cache.ts:123-130) or paged: a pool
// [pages,Hkv,128,D] addressed through a per-sequence block table (one page = one key tile).
// Roofline for decode: HBM, 2*B*Hkv*ctx*D*2 bytes.
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
  // decode mode
  const int* ctx_ptr;          // device scalar: number of valid keys (NULL: use Skv)
  const int* block_table;      // paged cache: [B, max_pages] page indices (NULL: contiguous cache)
  int max_pages;
  int splits;
  int group;                   // query heads per KV head (valid rows of the tile)
  float* part_o;               // [B, Hkv, splits, group, D] un-normalised partial outputs
  float* part_ml;              // [B, Hkv, splits, group, 2] (running max in the log2 domain, sum)
  int direct;                  // splits == 1: write O/l as bf16 straight to `o` (no combine kernel)
  int colsplit;                // decode, group <= 8: each softmax warp handles a quarter of the key columns (see kernel)
  int early_kv;                // decode: K/V tiles that do not hold the last position may be fetched before the grid-dependency wait
};

constexpr int FA_BQ = 128;
constexpr int FA_BKV = 128;          // key tile of the prefill kernels
constexpr int FA_DEC_BKV = 64;       // key tile of the decode kernel: six 64-key ring slots instead of three 128-key ones
                                     // keep more loads in flight per CTA in the same shared memory
constexpr int FA_THREADS = 192;           // decode: TMA warp, MMA warp, one softmax warpgroup
constexpr int FA_THREADS_PREFILL = 320;   // prefill: two softmax warpgroups
constexpr int FA_STAGES = 2;

template <int D, bool DECODE>
__global__ void __launch_bounds__(DECODE ? FA_THREADS : FA_THREADS_PREFILL, DECODE ? 2 : 1)
flash_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                               const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ FaParams p) {
  constexpr int SLABS = D / 64;                     // 64-wide head-dim slabs (one swizzle atom each)
  // Decode: only the first Hq/Hkv (<= 16) rows of the query tile are real, so only 16 rows are
  // staged; the MMA still reads 128 rows, the other 112 come from whatever follows in shared
  // memory (the first K/V slot) and produce rows of S/O that are never looked at.
  constexpr int QROWS = DECODE ? 16 : FA_BQ;
  constexpr int Q_BYTES = QROWS * D * 2;
  constexpr int Q_SLAB = QROWS * 128;
  constexpr int BKV = DECODE ? FA_DEC_BKV : FA_BKV;  // keys per tile
  constexpr int KV_BYTES = BKV * D * 2;
  constexpr int SLAB_BYTES = BKV * 128;             // BKV rows x 128 B
  // Two S buffers of BKV columns each, then O: prefill S at columns 0 and 128, O at 256 (512 columns);
  // decode S at 0 and 64, O at 128 (256 columns, so that two CTAs fit on an SM).  The next Q K^T is
  // issued before the current block's softmax has finished.
  constexpr int NSBUF = 2;
  constexpr int NWG = DECODE ? 1 : 2;   // softmax warpgroups
  // K and V tiles travel through one ring in the order K0 V0 K1 V1 ...: tile t uses slot t % NSLOT
  constexpr int NSLOT = DECODE ? 6 : 2 * FA_STAGES;
  constexpr uint32_t TMEM_COLS = DECODE ? 256 : 512;
  constexpr uint32_t S_COL0 = 0, O_COL0 = DECODE ? 128 : 256;
  constexpr uint32_t IDESC_QK = make_idesc_bf16(FA_BQ, BKV, 0, 0);
  constexpr uint32_t IDESC_PV = make_idesc_bf16(FA_BQ, D, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;
  uint8_t* ring = q_smem + Q_BYTES;                         // [NSLOT][KV_BYTES]
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + NSLOT * KV_BYTES);
  uint64_t* q_full = bars;                 // 1
  uint64_t* t_full = bars + 1;             // NSLOT (<= 6)
  uint64_t* t_empty = bars + 7;            // NSLOT
  uint64_t* s_full = bars + 13;            // 2
  uint64_t* p_ready = bars + 15;           // 2
  uint64_t* o_done = bars + 17;            // 1
  uint64_t* x_bar = bars + 18;             // 2: row-maximum exchange between the softmax warpgroups
  // Completion of the LAST P V product.  It cannot be read off o_done: with two S buffers Q K^T of
  // block j+1 is issued before P V of block j, so when the softmax warps have finished the last
  // block the tensor pipe is only known to have completed P V of block n-3; o_done may then still be
  // two phases behind, and a parity wait cannot tell "phase n-1 complete" from "phase n-3 complete".
  uint64_t* o_final = bars + 20;           // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xchg = reinterpret_cast<float*>(tmem_slot + 4);   // [2 buffers][2 warpgroups][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  int h, hk, q0, kv_len, j_begin, j_end, kv_end;
  // (early_kv: the caller guarantees that the context length and all cache rows but the last
  // position's are older than the launch before this one; see kd_set_pdl)
  if (DECODE && !p.early_kv) pdl_wait();
  int n_early = 0;            // this CTA's leading key tiles that may be fetched before the wait
  if (DECODE) {
    hk = blockIdx.y;
    h = hk;                     // Q tensor map is indexed by (row-in-group, kv head, batch)
    q0 = 0;
    kv_len = p.ctx_ptr ? *p.ctx_ptr : p.Skv;
    kv_len = max(0, min(kv_len, p.Skv));
    kv_end = kv_len;
    const int n_total = (kv_len + BKV - 1) / BKV;
    const int per_split = (n_total + p.splits - 1) / p.splits;
    j_begin = (int)blockIdx.x * per_split;
    j_end = min(n_total, j_begin + per_split);
    // the ring takes three K/V tile pairs without anybody having to free a slot; the tile that holds
    // position kv_len - 1 is the last one of the last split
    if (p.early_kv) n_early = max(0, min(min(j_end, n_total - 1) - j_begin, NSLOT / 2));
    if (j_begin >= j_end) {     // nothing for this split: publish an empty partial and leave
      if (p.early_kv) pdl_wait();
      if (p.direct) {
        // a single split without any key (context length 0 read from device memory): attention over
        // no keys is defined here as a zero row, so that `out` never keeps stale contents
        for (int i = threadIdx.x; i < p.group * D; i += blockDim.x)
          p.o[(int64_t)b * p.so_b + (int64_t)(hk * p.group + i / D) * p.so_h + (i % D)] = __float2bfloat16_rn(0.f);
      } else if ((int)threadIdx.x < p.group) {
        const int64_t slot = (((int64_t)b * p.Hkv + hk) * p.splits + blockIdx.x) * p.group + threadIdx.x;
        p.part_ml[slot * 2] = -1e30f;
        p.part_ml[slot * 2 + 1] = 0.f;
      }
      return;
    }
  } else {
    const int q_tile = p.num_q_tiles - 1 - (int)blockIdx.x;   // heavy causal tiles first
    h = blockIdx.y;
    hk = h / (p.Hq / p.Hkv);
    q0 = q_tile * FA_BQ;
    kv_len = p.Skv;
    kv_end = p.Skv;
    if (p.causal) kv_end = min(p.Skv, q0 + FA_BQ);
    j_begin = 0;
    j_end = (kv_end + FA_BKV - 1) / FA_BKV;
  }
  const int n_blocks = j_end - j_begin;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < NSLOT; ++s) { mbar_init(&t_full[s], 1); mbar_init(&t_empty[s], 1); }
    for (int s = 0; s < NSBUF; ++s) { mbar_init(&s_full[s], 1); mbar_init(&p_ready[s], 4 * NWG); }
    for (int s = 0; s < 2; ++s) mbar_init(&x_bar[s], 4 * NWG);
    mbar_init(o_done, 1);
    mbar_init(o_final, 1);
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
  if (DECODE) pdl_trigger();   // after the TMEM allocation

  if (warp == 0) {
    if (lane == 0) {
      auto load_q = [&]() {
        mbar_arrive_expect_tx(q_full, Q_BYTES);
#pragma unroll
        for (int s = 0; s < SLABS; ++s) tma_load_4d(q_smem + s * Q_SLAB, &tmap_q, q_full, s * 64, q0, h, b);
      };
      if (!(DECODE && p.early_kv)) load_q();
      for (int jj = 0; jj < n_blocks; ++jj) {
        if (DECODE && p.early_kv && jj == n_early) {
          // everything else (the query, the newest cache row) was written by the launch before this one
          pdl_wait();
          load_q();
        }
        // key-tile coordinates: rows j*BKV.. of sequence b, or the matching rows of the 128-row page
        // the block table names
        int row = (j_begin + jj) * BKV, outer = b;
        if (DECODE && p.block_table) {
          outer = p.block_table[(int64_t)b * p.max_pages + row / 128];
          row = row % 128;
        }
        const int tk = 2 * jj, tv = 2 * jj + 1;
        const int sk = tk % NSLOT, sv = tv % NSLOT;
        if (!mbar_wait(&t_empty[sk], (uint32_t)(((tk / NSLOT) & 1) ^ 1), abort_flag, p.err, 301)) break;
        mbar_arrive_expect_tx(&t_full[sk], KV_BYTES);
#pragma unroll
        for (int s = 0; s < SLABS; ++s)
          tma_load_4d(ring + sk * KV_BYTES + s * SLAB_BYTES, &tmap_k, &t_full[sk], s * 64, row, hk, outer);
        if (!mbar_wait(&t_empty[sv], (uint32_t)(((tv / NSLOT) & 1) ^ 1), abort_flag, p.err, 302)) break;
        mbar_arrive_expect_tx(&t_full[sv], KV_BYTES);
#pragma unroll
        for (int s = 0; s < SLABS; ++s)
          tma_load_4d(ring + sv * KV_BYTES + s * SLAB_BYTES, &tmap_v, &t_full[sv], s * 64, row, hk, outer);
      }
      if (DECODE && p.early_kv && n_early >= n_blocks) {   // all of this CTA's tiles were early ones
        pdl_wait();
        load_q();
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, 303);
      const uint32_t q_addr = smem_u32(q_smem);
      // S(j) = Q K(j)^T into S buffer j % NSBUF   (j counts this CTA's key tiles from 0)
      auto issue_qk = [&](int j) -> bool {
        const int t = 2 * j, stage = t % NSLOT;
        if (!mbar_wait(&t_full[stage], (uint32_t)((t / NSLOT) & 1), abort_flag, p.err, 304)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(ring + stage * KV_BYTES);
        const uint32_t d_tmem = tmem_base + S_COL0 + (uint32_t)((j % NSBUF) * BKV);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t qoff = (uint32_t)((k / 4) * Q_SLAB + (k % 4) * 32);
          const uint32_t koff = (uint32_t)((k / 4) * SLAB_BYTES + (k % 4) * 32);
          // colsplit: a stride of 0 between the 8-row groups of the A tile makes every group read rows
          // 0-7 of the Q tile, i.e. query r appears in S rows r, 8 + r, ..., 120 + r
          umma_ss(d_tmem, make_smem_desc_sw128(q_addr + qoff, 16, (DECODE && p.colsplit) ? 0u : 1024u),
                  make_smem_desc_sw128(k_addr + koff, 16, 1024), IDESC_QK, k != 0 ? 1u : 0u);
        }
        umma_commit(&t_empty[stage]);
        umma_commit(&s_full[j % NSBUF]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; ok && j < n_blocks; ++j) {
        // with two S buffers the next QK^T is issued before this block's softmax has finished
        if (NSBUF == 2 && j + 1 < n_blocks) {
          if (!issue_qk(j + 1)) break;
        }
        const int t = 2 * j + 1, stage = t % NSLOT;
        if (!mbar_wait(&p_ready[j % NSBUF], (uint32_t)((j / NSBUF) & 1), abort_flag, p.err, 305)) break;
        if (!mbar_wait(&t_full[stage], (uint32_t)((t / NSLOT) & 1), abort_flag, p.err, 306)) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(ring + stage * KV_BYTES);
        const uint32_t p_tmem = tmem_base + S_COL0 + (uint32_t)((j % NSBUF) * BKV);
        const uint32_t o_tmem = tmem_base + O_COL0;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          // V tile is [kv rows][64-wide d slabs]: MN-major B; 16 kv rows = 2048 bytes per k step
          const uint64_t vdesc = make_smem_desc_sw128(v_addr + (uint32_t)(k * 2048), SLAB_BYTES, 1024);
          umma_ts(o_tmem, p_tmem + (uint32_t)(k * 8), vdesc, IDESC_PV, (j | k) != 0 ? 1u : 0u);
        }
        umma_commit(&t_empty[stage]);
        umma_commit(o_done);
        if (j + 1 == n_blocks) umma_commit(o_final);
        // one S buffer: the next QK^T overwrites P, so it is issued after PV (in-order pipe)
        if (NSBUF == 1 && j + 1 < n_blocks) {
          if (!issue_qk(j + 1)) break;
        }
      }
    }
  } else {
    // Softmax.  Prefill runs two warpgroups on the same query tile: warps 2-5 own key columns 0-63
    // of every row, warps 6-9 columns 64-127 (a warp may only touch the TMEM lanes of its own
    // quarter, so the two threads that share a row sit in warps w and w+4).  They exchange the row
    // maximum through shared memory every block and the row sum once at the end; everything else
    // (P, the O rescale, the output store) is split by columns.  Decode runs one warpgroup.
    constexpr int CW = BKV / NWG;        // S columns per thread
    constexpr int NCH = CW / 32;
    constexpr int DW = D / NWG;          // O columns per thread
    const int wg = (warp - 2) >> 2;
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const int row = q0 + row_in_tile;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    bool colsplit_done = false;
    if constexpr (DECODE) {
      if (p.colsplit) {
        // Decode with at most 8 query heads per KV head.  One thread per S row would leave 120 of the
        // 128 softmax threads on padding rows and the valid rows' threads with 128 exponentials each:
        // the per-tile latency of that serial row, not HBM, then limits a CTA to ~21 GB/s.  Here the Q
        // tile is replicated into every 8-row group (descriptor stride 0), so query r is S row 32 w + r
        // in the lanes of EVERY softmax warp w, and warp w handles key columns [32 w, 32 w + 32) of it:
        // 32 exponentials per thread.  The row maximum is exchanged through shared memory once per
        // tile; each warp writes its 32 probabilities into its own rows of P and zeros elsewhere, so
        // that the P V product leaves a partial O per warp in rows 32 w + r, summed in the epilogue.
        colsplit_done = true;
        constexpr int QC = BKV / 4;        // key columns per warp and block (16)
        float* xm = xchg;                 // [2 buffers][4 quarters][32 lanes] row maxima
        float* xl = xchg + 256;           // [4 quarters][32 lanes] row sums
        float* xmu = xchg + 384;          // [32 lanes] the running maximum each row ended with
        float m_used = -1e30f, l = 0.f;
        bool ok = true;
        // No thread leaves this loop between the 128-thread barriers except right after one, where
        // all of them see the same abort flag (every failed wait raises it).
        for (int j = 0; j < n_blocks; ++j) {
          const uint32_t s_addr = lane_addr + S_COL0 + (uint32_t)((j % NSBUF) * BKV);
          ok = mbar_wait(&s_full[j % NSBUF], (uint32_t)((j / NSBUF) & 1), abort_flag, p.err, 307);
          ok = __all_sync(0xffffffffu, ok);
          uint32_t sr[QC];
          float* slot = xm + (j & 1) * 128;
          if (ok) {
            tc_fence_after();
            tmem_ld_32x16(s_addr + q * QC, sr);
            tmem_wait_ld();
            const int kv0 = (j_begin + j) * BKV + q * QC;
            if (kv0 + QC > kv_end) {
#pragma unroll
              for (int i = 0; i < QC; ++i)
                if (kv0 + i >= kv_len) sr[i] = __float_as_uint(-1e30f);
            }
            float mx0 = -1e30f, mx1 = -1e30f;
#pragma unroll
            for (int i = 0; i < QC; i += 4) {
              mx0 = fmaxf(mx0, fmaxf(__uint_as_float(sr[i]), __uint_as_float(sr[i + 1])));
              mx1 = fmaxf(mx1, fmaxf(__uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3])));
            }
            slot[q * 32 + lane] = fmaxf(mx0, mx1);
          }
          asm volatile("bar.sync 2, 128;" ::: "memory");        // the four softmax warps
          if (*abort_flag) { ok = false; break; }
          const float m_blk = fmaxf(fmaxf(slot[lane], slot[32 + lane]), fmaxf(slot[64 + lane], slot[96 + lane])) * p.scale_log2;
          float alpha = 1.f;
          bool rescale = false;
          if (j == 0 || lane >= p.group) {
            m_used = m_blk;          // first block; or a padding row, whose values nobody reads
          } else if (m_blk - m_used > 8.0f) {
            alpha = fast_exp2(m_used - m_blk);
            m_used = m_blk;
            rescale = true;
          }
          // the four threads of a row see the same maxima, hence take the same decision; warps may
          // differ in whether ANY of their rows rescales, which only affects their own O rows
          if (__any_sync(0xffffffffu, rescale)) {
            ok = mbar_wait(o_done, (uint32_t)((j - 1) & 1), abort_flag, p.err, 308);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) continue;     // the abort flag is up: everybody leaves after the next barrier
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
          // P row: this warp's QC probabilities in packed columns [QC/2 q, QC/2 (q+1)), zeros in the rest
          float sum0 = 0.f, sum1 = 0.f;
          uint32_t pk[QC / 2];
#pragma unroll
          for (int i = 0; i < QC / 2; ++i) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(sr[2 * i]), p.scale_log2, -m_used));
            const float p1 = fast_exp2(fmaf(__uint_as_float(sr[2 * i + 1]), p.scale_log2, -m_used));
            sum0 += p0;
            sum1 += p1;
            __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
            pk[i] = *reinterpret_cast<uint32_t*>(&v);
          }
          l += sum0 + sum1;
          uint32_t zero[QC / 2];
#pragma unroll
          for (int i = 0; i < QC / 2; ++i) zero[i] = 0u;
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_st_32x8(s_addr + c * (QC / 2), c == q ? pk : zero);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_ready[j % NSBUF]);
        }
        if (ok) {
          ok = mbar_wait(o_final, 0, abort_flag, p.err, 309);
          ok = __all_sync(0xffffffffu, ok);
        }
        // Epilogue: sum the four partial O rows and row sums of every query through shared memory
        // (the K/V ring is idle now: every tile has landed and every MMA has completed).
        float* osum = reinterpret_cast<float*>(ring);        // [4 quarters][8 rows][D]
        if (ok) {
          tc_fence_after();
          xl[q * 32 + lane] = l;
          if (q == 0) xmu[lane] = m_used;   // identical in the four threads of a row
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t orr[32];
            tmem_ld_32x32(lane_addr + O_COL0 + c * 32, orr);
            tmem_wait_ld();
            if (lane < p.group) {
#pragma unroll
              for (int g = 0; g < 8; ++g)
                *reinterpret_cast<float4*>(osum + (q * 8 + lane) * D + c * 32 + g * 4) =
                    make_float4(__uint_as_float(orr[g * 4]), __uint_as_float(orr[g * 4 + 1]), __uint_as_float(orr[g * 4 + 2]),
                                __uint_as_float(orr[g * 4 + 3]));
            }
          }
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (ok && *abort_flag == 0) {
          // 128 threads: thread t handles query row t / 16 (8 rows) and D/16 consecutive columns
          const int t = (warp - 2) * 32 + lane;
          const int r = t >> 4, cw = D / 16, c0 = (t & 15) * cw;
          if (r < p.group) {
            const float lsum = xl[r] + xl[32 + r] + xl[64 + r] + xl[96 + r];
            float acc[D / 16];
#pragma unroll
            for (int i = 0; i < cw; ++i)
              acc[i] = osum[(0 * 8 + r) * D + c0 + i] + osum[(1 * 8 + r) * D + c0 + i] + osum[(2 * 8 + r) * D + c0 + i] +
                       osum[(3 * 8 + r) * D + c0 + i];
            if (p.direct) {
              const float inv_l = 1.0f / lsum;
              __nv_bfloat16* orow = p.o + (int64_t)b * p.so_b + (int64_t)(hk * p.group + r) * p.so_h + c0;
#pragma unroll
              for (int i = 0; i < cw; i += 2) {
                __nv_bfloat162 v = __floats2bfloat162_rn(acc[i] * inv_l, acc[i + 1] * inv_l);
                *reinterpret_cast<__nv_bfloat162*>(orow + i) = v;
              }
            } else {
              const int64_t slot_o = (((int64_t)b * p.Hkv + hk) * p.splits + blockIdx.x) * p.group + r;
              if ((t & 15) == 0) {
                p.part_ml[slot_o * 2] = xmu[r];
                p.part_ml[slot_o * 2 + 1] = lsum;
              }
              float* prow = p.part_o + slot_o * D + c0;
#pragma unroll
              for (int i = 0; i < cw; ++i) prow[i] = acc[i];
            }
          }
        }
      }
    }
    if (!colsplit_done) {
    float m_used = -1e30f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      ok = mbar_wait(&s_full[j % NSBUF], (uint32_t)((j / NSBUF) & 1), abort_flag, p.err, 307);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_addr = lane_addr + S_COL0 + (uint32_t)((j % NSBUF) * BKV);
      uint32_t sr[NCH][32];
#pragma unroll
      for (int c = 0; c < NCH; ++c) tmem_ld_32x32(s_addr + wg * CW + c * 32, sr[c]);
      tmem_wait_ld();
      const int kv0 = (j_begin + j) * BKV;
      // Only the diagonal block of a causal tile and the last (ragged) key block need masking;
      // the test is hoisted so that the common path carries no per-element predicates.
      if ((kv0 + BKV > kv_end) || (p.causal && kv0 + BKV - 1 > q0)) {
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = kv0 + wg * CW + c * 32 + i;
            if (col >= kv_len || (p.causal && col > row)) sr[c][i] = __float_as_uint(-1e30f);
          }
      }
      float mx0 = -1e30f, mx1 = -1e30f;
#pragma unroll
      for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mx0 = fmaxf(mx0, fmaxf(__uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1])));
          mx1 = fmaxf(mx1, fmaxf(__uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3])));
        }
      float mloc = fmaxf(mx0, mx1);
      if (NWG == 2) {
        // exchange with the thread that owns the other half of this row (double-buffered by j&1)
        float* slot = xchg + (j & 1) * 256;
        slot[wg * 128 + row_in_tile] = mloc;
        __syncwarp();
        if (lane == 0) mbar_arrive(&x_bar[j & 1]);
        ok = mbar_wait(&x_bar[j & 1], (uint32_t)((j >> 1) & 1), abort_flag, p.err, 310);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        mloc = fmaxf(mloc, slot[(wg ^ 1) * 128 + row_in_tile]);
      }
      // scores are scaled inside the exponential: exp2(s*c - m*c) with c = scale*log2(e) > 0
      const float m_blk = mloc * p.scale_log2;
      // Lazy rescale: keep the stale max unless it is more than 2^8 too small.  Both owners of a row
      // see the same m_blk and the same history, so they take the same decision.
      float alpha = 1.f;
      bool rescale = false;
      if (j == 0 || (DECODE && row_in_tile >= p.group)) {
        m_used = m_blk;   // first block; or a padding row of the decode tile, whose values nobody reads
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
        for (int c = 0; c < DW / 32; ++c) {
          uint32_t orr[32];
          tmem_ld_32x32(lane_addr + O_COL0 + wg * DW + c * 32, orr);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
          tmem_st_32x32(lane_addr + O_COL0 + wg * DW + c * 32, orr);
        }
        l *= alpha;
      }
      // P = exp2(s - m_used) as packed bf16 into the first 64 columns of this S buffer
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int c = 0; c < CW / 64; ++c) {
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
        tmem_st_32x32(s_addr + wg * (CW / 2) + c * 32, pk);
      }
      l += sum0 + sum1;
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[j % NSBUF]);
    }
    if (ok) {
      ok = mbar_wait(o_final, 0, abort_flag, p.err, 309);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && NWG == 2) {
      // total row sum = the two column halves; use the exchange buffer the last block did not use
      const int jb = n_blocks & 1;
      float* slot = xchg + jb * 256;
      slot[wg * 128 + row_in_tile] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(&x_bar[jb]);
      ok = mbar_wait(&x_bar[jb], (uint32_t)((n_blocks >> 1) & 1), abort_flag, p.err, 311);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) l += slot[(wg ^ 1) * 128 + row_in_tile];
    }
    if (ok) {
      tc_fence_after();
      if (DECODE && p.direct) {
        // a single split holds the whole key range: normalise and store the real rows directly
        const bool valid = row_in_tile < p.group;
        const float inv_l = 1.0f / l;
        __nv_bfloat16* orow = p.o + (int64_t)b * p.so_b + (int64_t)(hk * p.group + row_in_tile) * p.so_h;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t orr[32];
          tmem_ld_32x32(lane_addr + O_COL0 + c * 32, orr);
          tmem_wait_ld();
          if (valid) {
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
      } else if (DECODE) {
        // un-normalised partial output + statistics; only the first `group` rows are real queries
        const int64_t slot = (((int64_t)b * p.Hkv + hk) * p.splits + blockIdx.x) * p.group + row_in_tile;
        const bool valid = row_in_tile < p.group;
        if (valid) {
          p.part_ml[slot * 2] = m_used;
          p.part_ml[slot * 2 + 1] = l;
        }
        float* prow = p.part_o + slot * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t orr[32];
          tmem_ld_32x32(lane_addr + O_COL0 + c * 32, orr);
          tmem_wait_ld();
          if (valid) {
#pragma unroll
            for (int g = 0; g < 8; ++g)
              *reinterpret_cast<float4*>(prow + c * 32 + g * 4) =
                  make_float4(__uint_as_float(orr[g * 4]), __uint_as_float(orr[g * 4 + 1]), __uint_as_float(orr[g * 4 + 2]),
                              __uint_as_float(orr[g * 4 + 3]));
          }
        }
      } else {
        const float inv_l = 1.0f / l;
        __nv_bfloat16* orow = p.o + (int64_t)b * p.so_b + (int64_t)h * p.so_h + (int64_t)row * p.so_s + wg * DW;
#pragma unroll 1
        for (int c = 0; c < DW / 32; ++c) {
          uint32_t orr[32];
          tmem_ld_32x32(lane_addr + O_COL0 + wg * DW + c * 32, orr);
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
    }   // !colsplit_done
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D, bool DECODE>
static int launch_fa(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& p, dim3 grid) {
  constexpr int SMEM = (DECODE ? 16 : FA_BQ) * D * 2 + (DECODE ? 6 * FA_DEC_BKV : 2 * FA_STAGES * FA_BKV) * D * 2 + 1024 + 256 + 2048;
  static bool configured[64] = {false};   // per device: kd_shutdown + kd_init may move the library to another GPU
  if (!configured[ctx().device & 63]) {
    KD_CUDA_CHECK(cudaFuncSetAttribute(flash_attention_tcgen05_kernel<D, DECODE>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured[ctx().device & 63] = true;
  }
  if (DECODE) KD_CUDA_CHECK(launch_ex(flash_attention_tcgen05_kernel<D, DECODE>, grid, dim3(FA_THREADS), (size_t)SMEM, tq, tk, tv, p));
  else flash_attention_tcgen05_kernel<D, DECODE><<<grid, FA_THREADS_PREFILL, SMEM, ctx().stream>>>(tq, tk, tv, p);
  return after_launch(DECODE ? "flash_attention_tcgen05_kernel<decode>" : "flash_attention_tcgen05_kernel");
}

// attention_prefill2.cu: two query sub-tiles per CTA share each K/V tile.
int attention_prefill2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& a, void* out);

int attention_tc_try(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v, const kd_tensor* out,
                     const AttnParams& a, int* handled) {
  *handled = 0;
  if (a.dt_q != KD_BF16 || a.dt_k != KD_BF16 || a.dt_v != KD_BF16 || a.dt_o != KD_BF16) return KD_OK;
  if (a.D != 64 && a.D != 128) return KD_OK;
  if (!(a.scale > 0.f)) return KD_OK;  // the kernel takes the row max before scaling
  if (a.Sq < 16) return KD_OK;  // single-row (decode) shapes go through kd_attention_decode or the CUDA-core kernel
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
  // More than one query tile per KV head: the kernel that shares K/V tiles between two sub-tiles.
  // KD_ATTENTION_ONE_TILE=1 in the environment keeps the one-tile kernel (for comparisons).
  static const bool one_tile = [] { const char* e = getenv("KD_ATTENTION_ONE_TILE"); return e && e[0] == '1'; }();
  if (!one_tile && ((a.Hq / a.Hkv) % 2 == 0 || a.Sq > FA_BQ)) {
    KD_TRY(attention_prefill2(tq, tk, tv, a, po));
    *handled = 1;
    return KD_OK;
  }
  FaParams p{};
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Sq = a.Sq; p.Skv = a.Skv;
  p.causal = a.causal;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.o = static_cast<__nv_bfloat16*>(po);
  p.so_b = a.so[0]; p.so_h = a.so[1]; p.so_s = a.so[2];
  p.num_q_tiles = (a.Sq + FA_BQ - 1) / FA_BQ;
  p.err = ctx().error_flag;
  dim3 grid(p.num_q_tiles, p.Hq, p.B);
  if (a.D == 128) KD_TRY((launch_fa<128, false>(tq, tk, tv, p, grid)));
  else KD_TRY((launch_fa<64, false>(tq, tk, tv, p, grid)));
  *handled = 1;
  return KD_OK;
}

// ----------------------------------------------------------------------------- split-KV combine
// out[b, h, :] = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s,  M = max_s m_s.
// One warp per (batch, query head); lanes stride over the head dimension.
__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      __nv_bfloat16* __restrict__ out, int64_t so_b, int64_t so_h, int B, int Hkv,
                                      int group, int splits, int D) {
  pdl_wait();
  pdl_trigger();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int Hq = Hkv * group;
  if (warp >= B * Hq) return;
  const int b = warp / Hq, h = warp - b * Hq;
  const int hk = h / group, r = h - hk * group;
  const int64_t base = ((int64_t)b * Hkv + hk) * splits;
  float M = -1e30f;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[((base + s) * group + r) * 2]);
  float denom = 0.f;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int s = 0; s < splits; ++s) {
    const int64_t slot = (base + s) * group + r;
    const float l = part_ml[slot * 2 + 1];
    if (l == 0.f) continue;  // empty split: its output row was never written
    const float w = exp2f(part_ml[slot * 2] - M);
    denom += w * l;
    const float* po = part_o + slot * D;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = lane + 32 * i;
      if (d < D) acc[i] += w * po[d];
    }
  }
  const float inv = denom > 0.f ? 1.0f / denom : 0.f;   // no key at all (context length 0): a zero row
  __nv_bfloat16* orow = out + (int64_t)b * so_b + (int64_t)h * so_h;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int d = lane + 32 * i;
    if (d < D) orow[d] = __float2bfloat16_rn(acc[i] * inv);
  }
}

// Scratch needed by attention_decode for a given problem (bytes).
size_t attention_decode_scratch_bytes(int B, int Hkv, int group, int splits, int D) {
  return (size_t)B * Hkv * splits * group * (D + 2) * sizeof(float);
}

// q [B,Hq,1,D] (any strides, unit d stride), cache k/v [B,Hkv,maxS,D] or pool [pages,Hkv,128,D]
// with block_table [B,max_pages]; out [B,Hq,1,D].  `scratch` holds the split partials.
int attention_decode(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v, const kd_tensor* out, float scale,
                     const int* ctx_dev, int ctx_host, const int* block_table, int max_pages, int splits,
                     void* scratch, size_t scratch_bytes) {
  KD_REQUIRE(q->ndim == 4 && k->ndim == 4 && v->ndim == 4 && out->ndim == 4, "attention_decode: operands must be 4-D");
  KD_REQUIRE(q->dtype == KD_BF16 && k->dtype == KD_BF16 && v->dtype == KD_BF16 && out->dtype == KD_BF16,
             "attention_decode: bf16 tensors required");
  const int B = (int)q->shape[0], Hq = (int)q->shape[1], D = (int)q->shape[3];
  const int Hkv = (int)k->shape[1];
  KD_REQUIRE(q->shape[2] == 1 && out->shape[2] == 1, "attention_decode: exactly one query position per sequence");
  KD_REQUIRE(D == 64 || D == 128, "attention_decode: head_dim must be 64 or 128");
  KD_REQUIRE(Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= 16, "attention_decode: %d query heads per KV head; this kernel stages at most 16", Hkv > 0 ? Hq / Hkv : 0);
  KD_REQUIRE(v->shape[1] == Hkv && v->shape[2] == k->shape[2] && v->shape[3] == D && k->shape[3] == D,
             "attention_decode: K and V cache shapes differ");
  KD_REQUIRE(scale > 0.f, "attention_decode: scale must be positive");
  KD_REQUIRE(splits >= 1 && splits <= 1024, "attention_decode: splits out of range");
  const int group = Hq / Hkv;
  int Skv;
  if (block_table) {
    KD_REQUIRE(k->shape[2] == 128, "attention_decode: paged cache needs pages of 128 rows");
    Skv = max_pages * 128;
  } else {
    KD_REQUIRE(k->shape[0] == B, "attention_decode: cache batch differs from the query batch");
    Skv = (int)k->shape[2];
  }
  if (!ctx_dev) KD_REQUIRE(ctx_host >= 1 && ctx_host <= Skv, "attention_decode: context length %d outside [1,%d]", ctx_host, Skv);
  KD_REQUIRE(q->strides[3] == 1 && k->strides[3] == 1 && v->strides[3] == 1 && out->strides[3] == 1,
             "attention_decode: unit stride along head_dim required");
  for (int i = 0; i < 3; ++i)
    KD_REQUIRE(q->strides[i] % 8 == 0 && k->strides[i] % 8 == 0 && v->strides[i] % 8 == 0,
               "attention_decode: strides must be multiples of 8 elements");
  KD_REQUIRE(scratch_bytes >= attention_decode_scratch_bytes(B, Hkv, group, splits, D), "attention_decode: scratch too small");
  void *pq = nullptr, *pk = nullptr, *pv = nullptr, *po = nullptr;
  KD_TRY(tensor_ptr(q, &pq));
  KD_TRY(tensor_ptr(k, &pk));
  KD_TRY(tensor_ptr(v, &pv));
  KD_TRY(tensor_ptr(out, &po));
  KD_REQUIRE(((reinterpret_cast<uintptr_t>(pq) | reinterpret_cast<uintptr_t>(pk) | reinterpret_cast<uintptr_t>(pv)) & 15) == 0,
             "attention_decode: operands must be 16-byte aligned");
  if (B == 0) return KD_OK;
  // Q viewed as [B, Hkv, group, D]: the tile's rows are the query heads of one KV group.
  const int64_t eq[4] = {B, Hkv, group, D};
  const int64_t sq[3] = {q->strides[0], q->strides[1] * group, q->strides[1]};
  const int64_t ek[4] = {k->shape[0], Hkv, k->shape[2], D};
  CUtensorMap tq, tk, tv;
  KD_TRY(make_tmap_bhsd(&tq, pq, eq, sq, 16));
  KD_TRY(make_tmap_bhsd(&tk, pk, ek, k->strides, FA_DEC_BKV));
  KD_TRY(make_tmap_bhsd(&tv, pv, ek, v->strides, FA_DEC_BKV));
  FaParams p{};
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = group; p.Skv = ctx_dev ? Skv : ctx_host;
  p.causal = 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = ctx().error_flag;
  p.ctx_ptr = ctx_dev;
  p.block_table = block_table;
  p.max_pages = max_pages;
  p.splits = splits;
  p.group = group;
  p.part_o = static_cast<float*>(scratch);
  p.part_ml = p.part_o + (size_t)B * Hkv * splits * group * D;
  // one split and a 16-byte aligned output: the attention kernel writes the result itself
  // column-split softmax: the Q tile is replicated into every 8-row group, so at most 8 query heads per KV head
  static const bool no_colsplit = [] { const char* e = getenv("KD_DECODE_NO_COLSPLIT"); return e && e[0] == '1'; }();
  p.colsplit = (group <= 8 && !no_colsplit) ? 1 : 0;
  p.early_kv = ctx().pdl_early_kv ? 1 : 0;
  p.direct = (splits == 1 && (reinterpret_cast<uintptr_t>(po) & 15) == 0 && out->strides[0] % 8 == 0 && out->strides[1] % 8 == 0) ? 1 : 0;
  p.o = static_cast<__nv_bfloat16*>(po);
  p.so_b = out->strides[0]; p.so_h = out->strides[1]; p.so_s = out->strides[2];
  dim3 grid(splits, Hkv, B);
  if (D == 128) KD_TRY((launch_fa<128, true>(tq, tk, tv, p, grid)));
  else KD_TRY((launch_fa<64, true>(tq, tk, tv, p, grid)));
  if (p.direct) return KD_OK;
  const int warps = B * Hq;
  KD_CUDA_CHECK(launch_ex(decode_combine_kernel, dim3((warps * 32 + 255) / 256), dim3(256), 0, (const float*)p.part_o,
                          (const float*)p.part_ml, static_cast<__nv_bfloat16*>(po), (int64_t)out->strides[0],
                          (int64_t)out->strides[1], B, Hkv, group, splits, D));
  return after_launch("decode_combine_kernel");
}

// ----------------------------------------------------------------------------- decode attention without allocation
// Scratch for the entry point that must not allocate: it lives in the library image, so every
// GPU that loads the library carries these 8 MiB until the process exits.
constexpr size_t STATIC_SCRATCH_BYTES = 8u << 20;
static __device__ __align__(256) unsigned char g_decode_static_scratch[STATIC_SCRATCH_BYTES];

// In host code the array's name is only a handle for the symbol, not a device address: the
// address the kernels may use has to be asked for, once per device, with that device current.
static int static_scratch_address(void** out) {
  static void* scratch_ptr[64] = {nullptr};
  const int dev = ctx().device;
  KD_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
  if (scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return fail(KD_ERR_CUDA, "cudaGetSymbolAddress for the static decode scratch failed: %s", cudaGetErrorString(e));
    }
    scratch_ptr[dev] = p;
  }
  *out = scratch_ptr[dev];
  return KD_OK;
}

// Test support: overwrite the built-in scratch with a byte pattern (stream-ordered).
int attention_decode_static_fill(int byte_value) {
  void* p = nullptr;
  KD_TRY(static_scratch_address(&p));
  KD_CUDA_CHECK(cudaMemsetAsync(p, byte_value, STATIC_SCRATCH_BYTES, ctx().stream));
  return KD_OK;
}

int attention_decode_static(const kd_tensor* q, const kd_tensor* k, const kd_tensor* v, const kd_tensor* out, float scale,
                            const int* ctx_dev, int ctx_host, int splits) {
  void* scratch = nullptr;
  KD_TRY(static_scratch_address(&scratch));
  KD_REQUIRE(q && k && q->ndim == 4 && k->ndim == 4, "decode attention operands must be 4-D");
  const int B = (int)q->shape[0], Hq = (int)q->shape[1], Hkv = (int)k->shape[1], D = (int)q->shape[3];
  KD_REQUIRE(Hkv > 0 && Hq % Hkv == 0, "bad head counts");
  const int max_blocks = (int)((k->shape[2] + FA_DEC_BKV - 1) / FA_DEC_BKV);
  if (splits <= 0) {
    const int pairs = B * Hkv > 0 ? B * Hkv : 1;
    splits = (2 * ctx().sm_count) / pairs;   // two CTAs fit per SM: stay within one wave
    if (splits > max_blocks) splits = max_blocks;
    if (splits < 1) splits = 1;
  }
  const size_t need = attention_decode_scratch_bytes(B, Hkv, Hq / Hkv, splits, D);
  if (need > STATIC_SCRATCH_BYTES)
    return fail(KD_ERR_INVALID,
                "kd_attention_decode_noalloc: batch %d x %d kv heads x %d splits needs %zu bytes of scratch, the built-in "
                "buffer holds %zu; lower `splits` or use kd_attention_decode",
                B, Hkv, splits, need, STATIC_SCRATCH_BYTES);
  return attention_decode(q, k, v, out, scale, ctx_dev, ctx_host, nullptr, 0, splits, scratch, STATIC_SCRATCH_BYTES);
}

}  // namespace kd
