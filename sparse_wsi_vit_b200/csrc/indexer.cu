// DSA lightning indexer + per-query top-k for sm_100a.
//
// Replaces the reference's `_indexer_fwd` Triton kernel
// (src/sparse_wsi_vit/models/deepseek_sparse_attention_kernels/kernels.py:19-113).
//
// Pipeline (all on the caller's stream):
//   1. collapse_heads_kernel : wq[t,:] = sum_h W[h] q_idx[t,h,:]  (and wk), fp32, padded to 64.
//   2. indexer_tiles_kernel<HIST> : radix select of every row's K-th largest score.  Each CTA owns
//      128 query rows, streams all key tiles through TMA, recomputes the 128x128 score tile with
//      tcgen05 TF32 MMAs into TMEM; 16 epilogue warps keep per-row counters in shared memory.
//        speculative pass : top 16 bits (estimate from a sample of key tiles, exact check);
//        candidate pass   : low 16 bits and the tie count from a per-row candidate list;
//        classic passes   : 8 bits each, only for query tiles flagged by the two passes above.
//   3. indexer_tiles_kernel<EMIT> : recomputes the tiles once more (bit-identical: same
//      instruction sequence) and writes idx / scores in ascending key order plus the
//      tile-major membership bitmask.  Ties at the threshold go to the lower key index.
//   4. fill_valid_kernel : valid[.., s] = s < min(K, Tk); zero padding of idx/scores.
// The N x N score matrix never reaches global memory.
#include <cmath>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <type_traits>

#include "common.cuh"

namespace swv {

// ------------------------------------------------------------------ collapse
template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

// out[(b*T + t)*64 + d] = sum_h w[h] * x[b,t,h,d]  (d < ID), 0 for ID <= d < 64.
// Products are rounded before the sum (no FMA contraction), heads in ascending order.
template <typename T>
__global__ void collapse_heads_kernel(const T* __restrict__ x, int64_t sb, int64_t st, int64_t sh, int64_t sd,
                                      const float* __restrict__ w, float* __restrict__ out, int B, int Tn, int IH,
                                      int ID) {
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(B) * Tn * kIdxDim;
  if (gid >= total) return;
  const int d = static_cast<int>(gid % kIdxDim);
  const int64_t bt = gid / kIdxDim;
  const int t = static_cast<int>(bt % Tn);
  const int b = static_cast<int>(bt / Tn);
  float acc = 0.f;
  if (d < ID) {
    const T* p = x + b * sb + t * st + d * sd;
    for (int h = 0; h < IH; ++h) {
      acc = __fadd_rn(acc, __fmul_rn(to_f32<T>(p[h * sh]), w[h]));
    }
  }
  out[gid] = acc;
}

// ------------------------------------------------------------------ prologue
// Token-local prologue of a DSA layer in ONE launch (the reference runs these as separate ATen /
// Triton steps: deepseek_sparse_attention.py:54-59 and, for the rotary term, vit_5/models_vit5.py:84-90):
//   * 2-D rotary embedding of q and k, in place on the fused projection output (optional);
//   * head collapse of the indexer projections, wq[t,:] = sum_h W[h] q_idx[t,h,:] (and wk), written
//     straight into the indexer workspace, with exactly the arithmetic of collapse_heads_kernel.
// One warp per token.
template <typename TQ, typename TI>
__global__ void __launch_bounds__(128)
    dsa_prologue_kernel(TQ* __restrict__ q, int64_t qsb, int64_t qst, int64_t qsh, TQ* __restrict__ k, int64_t ksb,
                        int64_t kst, int64_t ksh, const TI* __restrict__ qi, int64_t qib, int64_t qit, int64_t qih,
                        int64_t qid, const TI* __restrict__ ki, int64_t kib, int64_t kit, int64_t kih, int64_t kid,
                        const float* __restrict__ w, const float* __restrict__ coords, float inv_high,
                        float log2_theta, int skip, float* __restrict__ wq, float* __restrict__ wk, int B, int T,
                        int H, int D, int IH, int ID) {
  const int lane = threadIdx.x & 31;
  const int64_t tok = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (tok >= static_cast<int64_t>(B) * T) return;
  const int t = static_cast<int>(tok % T);
  const int b = static_cast<int>(tok / T);
  if (coords != nullptr && t >= skip) {
    const int pairs = D / 2, half_pairs = pairs / 2, dim = D / 2;
    const float c0 = __fmul_rn(coords[tok * 2], inv_high), c1 = __fmul_rn(coords[tok * 2 + 1], inv_high);
    for (int i = lane; i < H * pairs; i += 32) {
      const int hh = i / pairs, pr = i - hh * pairs;
      const int axis = pr >= half_pairs ? 1 : 0;
      const int f = pr - axis * half_pairs;
      const float freq = exp2f(-log2_theta * (2.0f * f) / dim);
      const float ang = __fmul_rn(axis ? c1 : c0, freq);
      float sn, cs;
      sincosf(ang, &sn, &cs);
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        TQ* xp = which == 0 ? q + b * qsb + t * qst + hh * qsh + 2 * pr : k + b * ksb + t * kst + hh * ksh + 2 * pr;
        const float x0 = to_f32<TQ>(xp[0]), x1 = to_f32<TQ>(xp[1]);
        // (same expression and rounding order as rope2d_kernel in block_sparse.cu)
        const float o0 = __fmaf_rn(x0, cs, -__fmul_rn(x1, sn)), o1 = __fmaf_rn(x1, cs, __fmul_rn(x0, sn));
        if constexpr (sizeof(TQ) == 4) {
          xp[0] = o0;
          xp[1] = o1;
        } else {
          xp[0] = __float2bfloat16_rn(o0);
          xp[1] = __float2bfloat16_rn(o1);
        }
      }
    }
  }
  for (int d = lane; d < kIdxDim; d += 32) {
    float aq = 0.f, ak = 0.f;
    if (d < ID) {
      const TI* pq = qi + b * qib + t * qit + d * qid;
      const TI* pk = ki + b * kib + t * kit + d * kid;
      for (int h = 0; h < IH; ++h) {
        aq = __fadd_rn(aq, __fmul_rn(to_f32<TI>(pq[h * qih]), w[h]));
        ak = __fadd_rn(ak, __fmul_rn(to_f32<TI>(pk[h * kih]), w[h]));
      }
    }
    wq[tok * kIdxDim + d] = aq;
    wk[tok * kIdxDim + d] = ak;
  }
}

// --------------------------------------------------------------- tile kernel
constexpr int kModeHist = 0;
constexpr int kModeEmit = 1;
constexpr int kStages = 2;                         // wk ring depth
constexpr int kTileBytes = kTile * kIdxDim * 4;    // 32 KiB fp32 tile (two 16 KiB K-halves)
constexpr int kHistStride = 259;                   // words per histogram row (256 bins + 3: odd, bank spread)
constexpr int kListCap = 512;                      // candidate pass: low-16-bit values kept per row
constexpr int kListStride = 513;                   // uint16 per row (+1: bank spread)
constexpr int kListBytes = kTile * kListStride * 2;
constexpr int kHistBytes = (kTile * kHistStride * 4 > kListBytes + kTile * 4) ? kTile * kHistStride * 4
                                                                              : kListBytes + kTile * 4;
constexpr int kKindFirst = 0, kKindMid = 1, kKindCand = 2, kKindSpec = 3, kKindEstimate = 4;
constexpr int kSampleTiles = 8;                    // speculative pass: key tiles sampled for the top-byte guess
constexpr int kEstimateTiles = 32;                 // estimate pass: key tiles sampled (evenly spread over the key range)
constexpr int kTmemCols = 256;                     // two 128-column score buffers

struct IndexerParams {
  int B, Tq, Tk, top_k;
  int nQT, nKT;
  int pass;               // HIST: 0..3
  int kind;               // HIST: first byte / later byte / candidate collection of the low 16 bits
  int only_flagged;       // HIST: run only for the query tiles flagged in `flags_in`
  const uint32_t* flags_in;   // [B*nQT]
  uint32_t* flags_out;    // [B*nQT] written by the speculative and the candidate pass (1 = redo classically)
  uint32_t* st_prefix;    // [B*Tq] known high bits of the threshold
  uint32_t* st_kth;       // [B*Tq] rank still to find inside the prefix bucket
  uint32_t* st_neq;       // [B*Tq] after the last pass: number of keys whose score equals the threshold
  int32_t* st_excl;       // [B*Tq][kMaxExcl] EMIT: keys equal to the threshold that are NOT selected (ties cut by key
                          // index), ascending, the first kMaxExcl of them
  // Key-range split: with few query tiles (a rank of a sequence-sharded run) `split` = 2 CTAs share
  // a query tile, each sweeping half of the key tiles; the part that finishes last merges.
  int split, nKT0;               // CTAs per query tile; key tiles of part 0
  const uint32_t* flags_spec;    // [tiles] speculative pass failed: the candidate pass runs unsplit
  uint32_t* flags_unsplit;       // [tiles] written by the candidate pass: emit runs unsplit
  uint32_t* tickets;             // [tiles] arrival counter of a tile's parts (reset by the last one)
  uint32_t* ghist;               // [tiles][2][kTile * kHistStride] per-part window histograms
  uint16_t* glist;               // [tiles][2][kTile * kListStride] per-part candidate lists
  uint32_t* gcnt;                // [tiles][2][kTile] per-part candidate counts
  uint32_t* st_cnt0;             // [B*Tq] selected keys of the row strictly above the threshold in part 0's range
  uint32_t* st_eq0;              // [B*Tq] keys equal to the threshold in part 0's range
  int32_t* idx;           // EMIT outputs
  float* scores;
  uint32_t* maskbits;     // may be null
  int* status;
  // Estimate / collect / select (the short form of the selection for sparse top-k on long key ranges):
  // the estimate pass leaves a LOWER bound of every row's threshold in st_prefix (the value at rank
  // `est_rank` of a sample of the keys, a little below the rank of the threshold); the collect pass (EMIT with
  // `collect` set) lists every key at or above it -- a superset of the selection, in ascending key
  // order, per part -- and a per-row kernel selects the exact top-k from those lists.
  int collect;                   // EMIT: write candidates instead of the final lists
  int est_rank;                  // ESTIMATE: the rank (in the sample of kEstimateTiles key tiles) of the lower bound
  int cand_cap;                  // candidates per (row, part)
  int32_t* cand_idx;             // [B*Tq][split][cand_cap]
  float* cand_sc;                // [B*Tq][split][cand_cap]
  uint32_t* cand_cnt;            // [B*Tq][split] candidates found (may exceed cand_cap: the tile is flagged then)
};

struct TileSmemCtl {
  uint64_t q_full;
  uint64_t k_full[kStages];
  uint64_t k_empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t overflow;
  uint32_t ticket;
};

// EMIT: per epilogue warp a [32 columns][32 lanes] word tile, then the row exchange [2][128][4] x 8 B,
// then per row two rings (key index, score bits) of kRing entries that turn the 4-byte appends into
// 32-byte stores
constexpr int kRing = 32;
constexpr int kRingStride = kRing + 1;             // words per row (+1: bank spread)
constexpr int kStageBytes = 16 * 32 * 32 * 4 + 2 * kTile * 4 * 8 + 2 * kTile * kRingStride * 4;
constexpr size_t tile_smem_bytes(int mode) {
  return 1024 /*alignment slack*/ + kTileBytes * (1 + kStages) + (mode == kModeHist ? kHistBytes : kStageBytes) +
         sizeof(TileSmemCtl) + 64;
}

// Bit pattern of max(x, 0) for a float x given as bits: as SIGNED integers the negative
// floats (and -0) are negative, the non-negative floats keep their order.
__device__ __forceinline__ uint32_t relu_bits(uint32_t raw) {
  return static_cast<uint32_t>(max(static_cast<int>(raw), 0));
}
__device__ __forceinline__ void red_inc_shared(uint32_t saddr) {
  asm volatile("red.shared.add.u32 [%0], 1;" ::"r"(saddr) : "memory");
}
// if (t < span) ++*saddr, as one compare and one predicated reduction (no branch)
__device__ __forceinline__ void red_inc_shared_if_lt(uint32_t saddr, uint32_t t, uint32_t span) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %1, %2;\n\t@p red.shared.add.u32 [%0], 1;\n\t}" ::"r"(saddr), "r"(t),
               "r"(span)
               : "memory");
}
// w |= bit where v >= t / v == t   (one compare + one predicated OR)
__device__ __forceinline__ void or_bit_if_ge(uint32_t& w, uint32_t v, uint32_t t, uint32_t bit) {
  asm("{\n\t.reg .pred p;\n\tsetp.ge.u32 p, %1, %2;\n\t@p or.b32 %0, %0, %3;\n\t}" : "+r"(w) : "r"(v), "r"(t), "r"(bit));
}
// signed compare on raw float bits: negative floats are negative integers
__device__ __forceinline__ void or_bit_if_ge_s32(uint32_t& w, uint32_t v, int t, uint32_t bit) {
  asm("{\n\t.reg .pred p;\n\tsetp.ge.s32 p, %1, %2;\n\t@p or.b32 %0, %0, %3;\n\t}" : "+r"(w) : "r"(v), "r"(t), "r"(bit));
}
__device__ __forceinline__ void or_bit_if_eq(uint32_t& w, uint32_t v, uint32_t t, uint32_t bit) {
  asm("{\n\t.reg .pred p;\n\tsetp.eq.u32 p, %1, %2;\n\t@p or.b32 %0, %0, %3;\n\t}" : "+r"(w) : "r"(v), "r"(t), "r"(bit));
}

// Adds the 32 scores of one thread (one 32-column TMEM chunk) to its row histogram
// (`hrow` = shared-memory address of the row's 256 counters).  A score takes part iff it
// lies in the bucket [lo, lo + span) already known to hold the threshold (pass 0: all of
// them); its bin is the next 8 bits.  CHECK guards the ragged last key tile.
template <bool CHECK, bool FIRST>
__device__ __forceinline__ void hist_update(const uint32_t (&r0)[32], uint32_t hrow, int shift, uint32_t lo,
                                            uint32_t span, int nvalid, uint32_t& zeros) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const uint32_t u = relu_bits(r0[i]);
    if (FIRST) {
      // scores that are exactly zero (half of them after the ReLU) are counted in a register
      const uint32_t t = CHECK ? (i < nvalid ? u : 0xFFFFFFFFu) : u;
      zeros += (t == 0u) ? 1u : 0u;
      red_inc_shared_if_lt(hrow + ((u >> 24) << 2), t - 1u, 0xFFFFFFFEu);
    } else {
      const uint32_t t = u - lo;
      red_inc_shared_if_lt(hrow + ((t >> shift) << 2), CHECK ? (i < nvalid ? t : span) : t, span);
    }
  }
}

// Speculative pass, 32 scores of one thread.  Row layout of this pass: word 0 takes every score
// below the window, word 1 + b the scores of bucket b = (u - lo) >> 16 (b < 256), word 257 every
// score at or beyond lo + 2^24.  The reduction is unconditional (a predicated one compiles to a
// branch around it); padding columns of the ragged last key tile land in word 0.
template <bool CHECK>
__device__ __forceinline__ void window_update(const uint32_t (&r0)[32], uint32_t hrow, uint32_t lo, int nvalid) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    int t = static_cast<int>(relu_bits(r0[i]) - lo);          // both < 2^31: negative iff below the window
    if (CHECK && i >= nvalid) t = -1;
    const int bin = min(max(t >> 16, -1), 256);               // arithmetic shift keeps the sign
    red_inc_shared(hrow + 4u + static_cast<uint32_t>(bin << 2));
  }
}

template <int MODE>
__global__ void __launch_bounds__(576, 1)
    indexer_tiles_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                         const IndexerParams p) {
  constexpr int kEpiWarps = 16;
  constexpr uint32_t kIdesc = make_idesc(/*tf32*/ 2, kTile, kTile, 0, 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sm_q = smem;
  uint8_t* sm_k = smem + kTileBytes;
  uint32_t* sm_hist = reinterpret_cast<uint32_t*>(smem + kTileBytes * (1 + kStages));
  TileSmemCtl* ctl = reinterpret_cast<TileSmemCtl*>(smem + kTileBytes * (1 + kStages) +
                                                    (MODE == kModeHist ? kHistBytes : kStageBytes));

  const int tile = blockIdx.x / p.split;         // (batch, query tile)
  const int part = blockIdx.x - tile * p.split;  // which share of the key range
  if (p.only_flagged != 0 && p.flags_in[tile] == 0u) return;
  // Which launches split the key range: the speculative pass always; the candidate pass unless the
  // speculative pass failed for the tile; emit unless the candidate pass said otherwise; the
  // classic histogram passes never.  An unsplit tile is swept by part 0 alone.
  bool use_split = false;
  if (p.split > 1) {
    if (MODE == kModeEmit) use_split = p.collect != 0 || p.flags_unsplit[tile] == 0u;
    else if (p.kind == kKindSpec) use_split = true;
    else if (p.kind == kKindCand) use_split = p.flags_spec[tile] == 0u;
    if (!use_split && part != 0) return;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int b = tile / p.nQT;
  const int qt = tile % p.nQT;
  const int kt0 = (use_split && part == 1) ? p.nKT0 : 0;                 // first key tile of this CTA
  const int nKT = (use_split ? (part == 0 ? p.nKT0 : p.nKT - p.nKT0) : p.nKT);   // key tiles of this CTA
  // The speculative pass first streams a sample of nSample key tiles twice (top byte, then second
  // byte of every row's estimated threshold; the same tiles for every part), then its key range.
  const bool estimate = MODE == kModeHist && p.kind == kKindEstimate;
  const int nSample = (MODE == kModeHist && p.kind == kKindSpec) ? min(p.nKT, kSampleTiles)
                      : estimate                                 ? min(p.nKT, kEstimateTiles)
                                                                 : 0;
  const int nPre = 2 * nSample;
  const int nIt = estimate ? nPre : nKT + nPre;       // the estimate pass streams only its sample
  const int sample_step = estimate ? p.nKT / nSample : 1;   // ... spread evenly over the key range

  if (threadIdx.x == 0) {
    ctl->overflow = 0;
    mbar_init(&ctl->q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ctl->k_full[s], 1);
      mbar_init(&ctl->k_empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&ctl->acc_full[a], 1);
      mbar_init(&ctl->acc_empty[a], kEpiWarps);
    }
    ctl->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      mbar_expect_tx(&ctl->q_full, kTileBytes);
      tma_load_3d(sm_q, &tm_q, &ctl->q_full, 0, qt * kTile, b);
      tma_load_3d(sm_q + kTileBytes / 2, &tm_q, &ctl->q_full, 32, qt * kTile, b);
      for (int it = 0; it < nIt; ++it) {
        const int j = it < nPre ? (it < nSample ? it : it - nSample) * sample_step : kt0 + it - nPre;
        const int s = it % kStages;
        if (!mbar_wait_bounded(&ctl->k_empty[s], ((it / kStages) & 1) ^ 1, abort_flag)) {
          record_status(p.status, kDevWaitStageEmpty);
          break;
        }
        uint8_t* dst = sm_k + s * kTileBytes;
        mbar_expect_tx(&ctl->k_full[s], kTileBytes);
        tma_load_3d(dst, &tm_k, &ctl->k_full[s], 0, j * kTile, b);
        tma_load_3d(dst + kTileBytes / 2, &tm_k, &ctl->k_full[s], 32, j * kTile, b);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait_bounded(&ctl->q_full, 0, abort_flag);
      if (!ok) record_status(p.status, kDevWaitQ);
      const uint32_t q_addr = smem_u32(sm_q);
      for (int j = 0; ok && j < nIt; ++j) {
        const int s = j % kStages;
        const int a = j & 1;
        if (!mbar_wait_bounded(&ctl->k_full[s], (j / kStages) & 1, abort_flag)) {
          record_status(p.status, kDevWaitTmaFull);
          break;
        }
        if (!mbar_wait_bounded(&ctl->acc_empty[a], ((j >> 1) & 1) ^ 1, abort_flag)) {
          record_status(p.status, kDevWaitAccEmpty);
          break;
        }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sm_k + s * kTileBytes);
        const uint32_t d_tmem = tmem_base + a * kTile;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * (kTileBytes / 2) + (ks & 3) * 32;
          umma_tf32_ss(d_tmem, smem_desc_sw128(q_addr + off), smem_desc_sw128(k_addr + off), kIdesc, ks > 0);
        }
        umma_commit(&ctl->k_empty[s]);
        umma_commit(&ctl->acc_full[a]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int ew = warp - 2;                 // 0..kEpiWarps-1
    const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;     // row inside the query tile
    const int qrow = qt * kTile + row;       // query index
    const bool row_ok = qrow < p.Tq;
    const int64_t grow = static_cast<int64_t>(b) * p.Tq + qrow;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    bool ok = true;

    if (MODE == kModeHist && (p.kind == kKindSpec || p.kind == kKindEstimate)) {
      // Speculative fusion of the two first radix passes.  Phase 1 estimates, per row, the top 16
      // bits of the K-th largest score from a sample of key tiles (rank scaled to the sample; two
      // 8-bit histogram rounds).  Phase 2 streams all keys against a 2^24-wide window of bit
      // patterns centred on that estimate (aligned to 2^16): scores beyond the window are counted,
      // scores inside it are binned on 2^16-wide buckets.  The estimate is then CHECKED with the
      // exact counts (above < K <= above + inside); a tile with any row that fails is flagged and
      // redone by the two classic passes.
      const int ch = ew >> 2;
      const int et = threadIdx.x - 64;
      for (int i = et; i < kTile * kHistStride; i += 512) sm_hist[i] = 0u;
      asm volatile("bar.sync 1, 512;" ::: "memory");
      uint32_t* hrow = sm_hist + row * kHistStride;
      const uint32_t hrow_s = smem_u32(hrow);
      const uint32_t k_eff = static_cast<uint32_t>(min(p.top_k, p.Tk));
      uint32_t zeros = 0, lo = 0, rank = 1, est_hi = 0;
      // end of a sample round: take the digit that holds the scaled rank, clear the histogram
      auto end_round = [&](bool first_round) {
        if (first_round) {
          if (zeros != 0u) atomicAdd(hrow, zeros);
          const uint32_t n_s = static_cast<uint32_t>(min(p.Tk, nSample * kTile));
          const uint64_t want = static_cast<uint64_t>(k_eff) * n_s;
          rank = estimate ? static_cast<uint32_t>(p.est_rank) : static_cast<uint32_t>((want + p.Tk - 1) / p.Tk);
          rank = max(rank, 1u);
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");
        uint32_t cum = 0, digit = 0;
        for (int bin = 255; bin >= 0; --bin) {
          const uint32_t c = hrow[bin];
          if (cum + c >= rank) {
            digit = static_cast<uint32_t>(bin);
            break;
          }
          cum += c;
        }
        rank -= min(cum, rank - 1u);
        if (first_round) {
          est_hi = digit;
          lo = digit << 24;
        } else {
          const uint32_t est16 = (est_hi << 8) | digit;
          if (estimate) lo = est16 << 16;                 // the low edge of the bucket that holds the scaled rank
          else lo = (est16 > 128u ? est16 - 128u : 0u) << 16;
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");
        for (int i = et; i < kTile * kHistStride; i += 512) sm_hist[i] = 0u;
        asm volatile("bar.sync 1, 512;" ::: "memory");
      };
      for (int it = 0; it < nIt; ++it) {
        const int j = it < nPre ? (it < nSample ? it : it - nSample) * sample_step : kt0 + it - nPre;
        const int a = it & 1;
        if (it == nSample || it == nPre) end_round(it == nSample);
        // (a wait that gave up keeps looping without work: every thread passes the same barriers)
        if (ok && !mbar_wait_bounded(&ctl->acc_full[a], (it >> 1) & 1, abort_flag)) {
          record_status(p.status, kDevWaitAccFull);
          ok = false;
        }
        if (!ok) continue;
        tc_fence_after();
        uint32_t r0[32];
        tmem_ld32(lane_base + a * kTile + ch * 32, r0);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->acc_empty[a]);
        const int nvalid = p.Tk - (j * kTile + ch * 32);
        if (it < nSample) {
          if (nvalid >= 32) hist_update<false, true>(r0, hrow_s, 24, 0u, 0u, 32, zeros);
          else hist_update<true, true>(r0, hrow_s, 24, 0u, 0u, nvalid, zeros);
        } else if (it < nPre) {
          if (nvalid >= 32) hist_update<false, false>(r0, hrow_s, 16, lo, 1u << 24, 32, zeros);
          else hist_update<true, false>(r0, hrow_s, 16, lo, 1u << 24, nvalid, zeros);
        } else {
          if (nvalid >= 32) window_update<false>(r0, hrow_s, lo, 32);
          else window_update<true>(r0, hrow_s, lo, nvalid);
        }
      }
      if (estimate) {
        // a lower bound of the row's threshold (the collect pass lists every key at or above it)
        end_round(false);
        if (ch == 0 && row_ok) p.st_prefix[grow] = (ok && *abort_flag == 0u) ? lo : 0u;
      } else {
      asm volatile("bar.sync 1, 512;" ::: "memory");
      // Split key range: every part publishes its histogram; the part that arrives last adds the
      // other one's to its own and finishes the tile (the estimate, hence the window, is the same
      // in both parts: it comes from the same sample tiles).
      bool finisher = true;
      const uint32_t* h0_row = nullptr;          // part 0's histogram of this row (global), for the part-0 count
      if (use_split) {
        uint32_t* gh = p.ghist + (static_cast<size_t>(tile) * 2 + part) * (kTile * kHistStride);
        for (int i = et; i < kTile * kHistStride; i += 512) gh[i] = sm_hist[i];
        __threadfence();
        asm volatile("bar.sync 1, 512;" ::: "memory");
        if (et == 0) ctl->ticket = atomicAdd(p.tickets + tile, 1u);
        asm volatile("bar.sync 1, 512;" ::: "memory");
        finisher = ctl->ticket == static_cast<uint32_t>(p.split - 1);
        if (finisher) {
          __threadfence();
          if (et == 0) p.tickets[tile] = 0u;
          const uint32_t* go = p.ghist + (static_cast<size_t>(tile) * 2 + (1 - part)) * (kTile * kHistStride);
          for (int i = et; i < kTile * kHistStride; i += 512) sm_hist[i] += __ldcg(go + i);
          h0_row = p.ghist + static_cast<size_t>(tile) * 2 * (kTile * kHistStride) + row * kHistStride;
          asm volatile("bar.sync 1, 512;" ::: "memory");
        }
      }
      if (finisher) {
      bool row_valid = true;
      uint32_t digit = 0, cum = 0, kth = 0;
      if (ch == 0 && row_ok) {
        const uint32_t n_above = hrow[257];      // scores beyond the window
        row_valid = n_above < k_eff;
        if (row_valid) {
          kth = k_eff - n_above;
          row_valid = false;
          for (int bin = 255; bin >= 0; --bin) {
            const uint32_t c = hrow[1 + bin];
            if (cum + c >= kth) {
              digit = static_cast<uint32_t>(bin);
              row_valid = true;
              break;
            }
            cum += c;
          }
        }
        if (!row_valid) atomicOr(&ctl->overflow, 1u);
      }
      asm volatile("bar.sync 1, 512;" ::: "memory");
      const bool redo = ctl->overflow != 0u || !ok || *abort_flag != 0u;
      if (et == 0) p.flags_out[tile] = redo ? 1u : 0u;
      if (!redo && ch == 0 && row_ok) {
        p.st_prefix[grow] = (lo >> 16) + digit;
        p.st_kth[grow] = kth - cum;
        if (h0_row != nullptr) {
          // keys of part 0's range whose top 16 bits lie above the threshold's
          uint32_t above0 = __ldcg(h0_row + 257);
          for (int bin = 255; bin > static_cast<int>(digit); --bin) above0 += __ldcg(h0_row + 1 + bin);
          p.st_cnt0[grow] = above0;
        }
      }
      }
      }   // (not the estimate pass)
    } else if (MODE == kModeHist && p.kind == kKindCand) {
      // Candidate pass: the top 16 bits of every row's threshold are known.  The low 16 bits of
      // the scores inside that bucket are collected per row (a few dozen on continuous data) and
      // the exact threshold is selected from the list, replacing the two last histogram passes.
      // A row with more than kListCap candidates (massive ties) marks the whole query tile for
      // the histogram passes instead; nothing of the tile's state is written then.
      const int ch = ew >> 2;
      const int et = threadIdx.x - 64;
      uint16_t* list = reinterpret_cast<uint16_t*>(sm_hist);
      uint32_t* cnt = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(sm_hist) + kListBytes);
      if (et < kTile) cnt[et] = 0u;
      asm volatile("bar.sync 1, 512;" ::: "memory");
      const uint32_t prefix = row_ok ? p.st_prefix[grow] : 0xFFFFu;
      const uint32_t lo = prefix << 16;
      uint16_t* lrow = list + row * kListStride;
      for (int j = 0; j < nKT; ++j) {
        const int a = j & 1;
        if (!mbar_wait_bounded(&ctl->acc_full[a], (j >> 1) & 1, abort_flag)) {
          record_status(p.status, kDevWaitAccFull);
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t r0[32];
        tmem_ld32(lane_base + a * kTile + ch * 32, r0);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->acc_empty[a]);
        const int nvalid = p.Tk - ((kt0 + j) * kTile + ch * 32);
        // two instances of the scan: the bounds test only exists for the ragged last key tile
        auto scan = [&](auto check) {
          constexpr bool kCheck = decltype(check)::value;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            uint32_t t[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              t[q] = relu_bits(r0[i + q]) - lo;
              if (kCheck && i + q >= nvalid) t[q] = 0xFFFFFFFFu;
            }
            if (min(min(t[0], t[1]), min(t[2], t[3])) < 65536u) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                if (t[q] < 65536u) {
                  const uint32_t pos = atomicAdd(cnt + row, 1u);
                  if (pos < kListCap) lrow[pos] = static_cast<uint16_t>(t[q]);
                }
              }
            }
          }
        };
        if (nvalid >= 32) scan(std::false_type{});
        else scan(std::true_type{});
      }
      asm volatile("bar.sync 1, 512;" ::: "memory");
      uint32_t n = cnt[row];
      uint32_t n0 = 0;                           // entries [0, n0) of the row's list come from part 0's key range
      bool finisher = true;
      if (use_split) {
        // every part publishes its lists; the part that arrives last reloads both (part 0's first)
        uint16_t* gl = p.glist + (static_cast<size_t>(tile) * 2 + part) * (kTile * kListStride) + row * kListStride;
        const uint32_t n_own = min(n, static_cast<uint32_t>(kListCap));
        for (uint32_t i = ch; i < n_own; i += 4) gl[i] = lrow[i];
        if (ch == 0) p.gcnt[(static_cast<size_t>(tile) * 2 + part) * kTile + row] = n;
        __threadfence();
        asm volatile("bar.sync 1, 512;" ::: "memory");
        if (et == 0) ctl->ticket = atomicAdd(p.tickets + tile, 1u);
        asm volatile("bar.sync 1, 512;" ::: "memory");
        finisher = ctl->ticket == static_cast<uint32_t>(p.split - 1);
        if (finisher) {
          __threadfence();
          if (et == 0) p.tickets[tile] = 0u;
          const uint32_t c0 = __ldcg(p.gcnt + (static_cast<size_t>(tile) * 2 + 0) * kTile + row);
          const uint32_t c1 = __ldcg(p.gcnt + (static_cast<size_t>(tile) * 2 + 1) * kTile + row);
          n = c0 + c1;
          if (c0 > kListCap || c1 > kListCap) n = kListCap + 1;     // a part overflowed
          n0 = c0;
          if (n <= kListCap) {
            const uint16_t* g0 = p.glist + (static_cast<size_t>(tile) * 2 + 0) * (kTile * kListStride) + row * kListStride;
            const uint16_t* g1 = g0 + kTile * kListStride;
            for (uint32_t i = ch; i < c0; i += 4) lrow[i] = __ldcg(g0 + i);
            for (uint32_t i = ch; i < c1; i += 4) lrow[c0 + i] = __ldcg(g1 + i);
          }
          asm volatile("bar.sync 1, 512;" ::: "memory");
        }
      }
      if (finisher) {
      if (ch == 0 && row_ok && n > kListCap) atomicOr(&ctl->overflow, 1u);
      asm volatile("bar.sync 1, 512;" ::: "memory");
      const bool tile_overflow = ctl->overflow != 0u;
      if (et == 0) {
        p.flags_out[tile] = tile_overflow ? 1u : 0u;
        if (p.split > 1) p.flags_unsplit[tile] = (tile_overflow || !use_split) ? 1u : 0u;
      }
      if (ok && ch == 0 && row_ok && !tile_overflow && *abort_flag == 0u) {
        uint32_t kth = p.st_kth[grow];
        uint32_t val = 0;
        for (int bit = 15; bit >= 0; --bit) {
          const uint32_t want = (val >> bit) | 1u;
          uint32_t c = 0;
          for (uint32_t i = 0; i < n; ++i) c += ((static_cast<uint32_t>(lrow[i]) >> bit) == want) ? 1u : 0u;
          if (c >= kth) val |= 1u << bit;
          else kth -= c;
        }
        uint32_t n_eq = 0;
        for (uint32_t i = 0; i < n; ++i) n_eq += (lrow[i] == val) ? 1u : 0u;
        p.st_prefix[grow] = lo | val;
        p.st_kth[grow] = kth;
        p.st_neq[grow] = n_eq;
        if (use_split) {
          // part 0's share: candidates above the threshold (added to the keys above the bucket
          // that the speculative pass counted) and candidates equal to it
          uint32_t in0 = 0, eq0 = 0;
          for (uint32_t i = 0; i < n0; ++i) {
            in0 += (lrow[i] > val) ? 1u : 0u;
            eq0 += (lrow[i] == val) ? 1u : 0u;
          }
          p.st_cnt0[grow] += in0;
          p.st_eq0[grow] = eq0;
        }
      }
      }
    } else if constexpr (MODE == kModeHist) {
      const int ch = ew >> 2;                // column quarter 0..3 (32 columns each)
      const int et = threadIdx.x - 64;       // 0..511
      for (int i = et; i < kTile * kHistStride; i += 512) sm_hist[i] = 0u;
      asm volatile("bar.sync 1, 512;" ::: "memory");

      const int pass = p.pass;
      const int shift = 24 - 8 * pass;
      const uint32_t prefix = (pass > 0 && row_ok) ? p.st_prefix[grow] : 0u;
      uint32_t* hrow = sm_hist + row * kHistStride;
      const uint32_t hrow_s = smem_u32(hrow);
      const uint32_t lo = pass > 0 ? prefix << (shift + 8) : 0u;     // low edge of the known bucket
      const uint32_t span = pass > 0 ? 1u << (shift + 8) : 0u;
      uint32_t zeros = 0;

      for (int j = 0; j < nKT; ++j) {
        const int a = j & 1;
        if (!mbar_wait_bounded(&ctl->acc_full[a], (j >> 1) & 1, abort_flag)) {
          record_status(p.status, kDevWaitAccFull);
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t r0[32];
        tmem_ld32(lane_base + a * kTile + ch * 32, r0);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->acc_empty[a]);

        const int nvalid = p.Tk - (j * kTile + ch * 32);   // columns of this quarter that are real keys
        if (pass == 0) {
          if (nvalid >= 32) hist_update<false, true>(r0, hrow_s, shift, lo, span, 32, zeros);
          else hist_update<true, true>(r0, hrow_s, shift, lo, span, nvalid, zeros);
        } else {
          if (nvalid >= 32) hist_update<false, false>(r0, hrow_s, shift, lo, span, 32, zeros);
          else hist_update<true, false>(r0, hrow_s, shift, lo, span, nvalid, zeros);
        }
      }
      if (zeros != 0u) atomicAdd(hrow, zeros);
      asm volatile("bar.sync 1, 512;" ::: "memory");
      if (ok && ch == 0 && row_ok && *abort_flag == 0u) {
        uint32_t kth = pass == 0 ? static_cast<uint32_t>(min(p.top_k, p.Tk)) : p.st_kth[grow];
        uint32_t cum = 0, in_bin = 0;
        int digit = 0;
        for (int bin = 255; bin >= 0; --bin) {
          const uint32_t c = hrow[bin];
          if (cum + c >= kth) {
            digit = bin;
            in_bin = c;
            break;
          }
          cum += c;
        }
        p.st_prefix[grow] = (prefix << 8) | static_cast<uint32_t>(digit);
        p.st_kth[grow] = kth - cum;
        if (pass == 3) p.st_neq[grow] = in_bin;
      }
    } else {
      // EMIT: four threads per query row (one per 32-column quarter of the tile), ascending keys.
      // Per tile every thread stages its 32 relu'd scores in a per-warp shared tile, builds a
      // 32-bit member word (and a word of exact ties where a row's ties are cut), and the four
      // threads of a row exchange their words through shared memory (one named barrier per tile,
      // double-buffered) so each knows its output offset.  All four keep identical running counts.
      // Appends go to the row's ring in shared memory; after the NEXT tile's barrier one of the four
      // threads writes the completed groups of 8 entries as 32-byte stores (a 4-byte store per entry
      // costs the L2 a sector write each).  A tile that would overrun the ring writes directly.
      const int ch = ew >> 2;
      const uint32_t thr = row_ok ? p.st_prefix[grow] : 0xFFFFFFFFu;
      // (collect: `thr` is the estimate pass's lower bound, every key at or above it is listed)
      const bool collect = p.collect != 0;
      const uint32_t take_eq = row_ok && !collect ? p.st_kth[grow] : 0u;   // how many keys == thr to keep
      const uint32_t n_eq = row_ok && !collect ? p.st_neq[grow] : 0u;      // how many keys == thr exist
      const bool partial = row_ok && take_eq < n_eq;            // ties cut by key index (lowest first)
      const bool warp_partial = __any_sync(0xffffffffu, partial);
      const uint32_t thr_min = partial ? thr + 1u : thr;        // member iff bits >= thr_min (+ chosen ties)
      const int thr_signed = thr_min == 0u ? static_cast<int>(0x80000000u) : static_cast<int>(thr_min);
      // A second part starts behind part 0's share of the row: the keys above the threshold in part
      // 0's range plus the ties part 0 takes (ties are taken in ascending key order).
      uint32_t eq_seen = 0;
      uint32_t ex_seen = 0;                                     // ties of the row left out so far (cut rows only)
      int cnt = 0;
      if (use_split && part == 1 && row_ok && !collect) {
        const uint32_t eq0 = p.st_eq0[grow];
        eq_seen = min(eq0, partial ? take_eq : 0xFFFFFFFFu);
        cnt = static_cast<int>(p.st_cnt0[grow] + eq_seen);
        if (partial) ex_seen = eq0 - eq_seen;
        else eq_seen = 0;
      }
      int32_t* excl_row = p.st_excl + grow * kMaxExcl;
      // collect: every part has its own list of the row; capacity cand_cap instead of top_k
      const int cap_out = collect ? p.cand_cap : p.top_k;
      const int64_t cand_row = (grow * p.split + part) * p.cand_cap;
      int32_t* idx_row = collect ? p.cand_idx + cand_row : p.idx + grow * p.top_k;
      float* sc_row = collect ? p.cand_sc + cand_row : p.scores + grow * p.top_k;
      // 32-bit shared addresses: the staging tiles share the histogram's slot, then the exchange
      // words [2][128 rows][4 quarters] x 8 B, then the two rings
      const uint32_t stage = smem_u32(sm_hist) + static_cast<uint32_t>(ew * (32 * 32) + lane * 4) * 4u;
      const uint32_t xchg = smem_u32(sm_hist) + static_cast<uint32_t>(kEpiWarps * (32 * 32)) * 4u;
      const uint32_t ring_i = xchg + 2u * kTile * 4u * 8u + static_cast<uint32_t>(row * kRingStride) * 4u;
      const uint32_t ring_s = ring_i + static_cast<uint32_t>(kTile * kRingStride) * 4u;
      const bool vec_ok = collect ? (p.cand_cap & 3) == 0
                                  : ((reinterpret_cast<uintptr_t>(p.idx) | reinterpret_cast<uintptr_t>(p.scores)) & 15) == 0 &&
                                        (p.top_k & 3) == 0;
      int flushed = cnt;                                        // entries of the row below this index are not this CTA's to write
      // entries [from, to) of the row leave the ring
      auto flush = [&](int from, int to) {
        int e = from;
        while (e < to) {
          if (vec_ok && (e & 7) == 0 && e + 8 <= to) {
            uint32_t vi[8], vs[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              vi[t] = lds32(ring_i + (((e + t) & (kRing - 1)) << 2));
              vs[t] = lds32(ring_s + (((e + t) & (kRing - 1)) << 2));
            }
            *reinterpret_cast<uint4*>(idx_row + e) = make_uint4(vi[0], vi[1], vi[2], vi[3]);
            *reinterpret_cast<uint4*>(idx_row + e + 4) = make_uint4(vi[4], vi[5], vi[6], vi[7]);
            *reinterpret_cast<uint4*>(sc_row + e) = make_uint4(vs[0], vs[1], vs[2], vs[3]);
            *reinterpret_cast<uint4*>(sc_row + e + 4) = make_uint4(vs[4], vs[5], vs[6], vs[7]);
            e += 8;
          } else {
            idx_row[e] = static_cast<int32_t>(lds32(ring_i + ((e & (kRing - 1)) << 2)));
            sc_row[e] = __uint_as_float(lds32(ring_s + ((e & (kRing - 1)) << 2)));
            ++e;
          }
        }
      };
      uint4* mask_row = nullptr;
      if (p.maskbits != nullptr) {
        mask_row = reinterpret_cast<uint4*>(p.maskbits) +
                   ((static_cast<int64_t>(b) * p.nQT + qt) * p.nKT + kt0) * kTile + row;
      }
      for (int j = 0; j < nKT; ++j) {
        const int a = j & 1;
        // (a wait that gave up keeps looping without work: every thread passes the same barriers)
        if (ok && !mbar_wait_bounded(&ctl->acc_full[a], (j >> 1) & 1, abort_flag)) {
          record_status(p.status, kDevWaitAccFull);
          ok = false;
        }
        uint32_t w = 0, e = 0;
        const int key0 = (kt0 + j) * kTile + ch * 32;
        if (ok) {
          tc_fence_after();
          uint32_t r[32];
          tmem_ld32(lane_base + a * kTile + ch * 32, r);
          tc_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->acc_empty[a]);
          // Raw scores are staged four to a 16-byte store; membership compares the raw bits as
          // signed integers (a negative score is a negative integer, below every positive
          // threshold; a zero threshold admits everything: max(score, 0) >= 0).
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            sts128(stage + static_cast<uint32_t>((i >> 2) * 32 * 16), r[i], r[i + 1], r[i + 2], r[i + 3]);
#pragma unroll
          for (int i = 0; i < 32; ++i) or_bit_if_ge_s32(w, r[i], thr_signed, 1u << i);
          if (warp_partial) {
#pragma unroll
            for (int i = 0; i < 32; ++i) or_bit_if_eq(e, relu_bits(r[i]), thr, 1u << i);
          }
          const int nvalid = p.Tk - key0;
          if (nvalid < 32) {
            const uint32_t vm = nvalid <= 0 ? 0u : ((1u << nvalid) - 1u);
            w &= vm;
            e &= vm;
          }
        }
        const uint32_t x = xchg + static_cast<uint32_t>((a * kTile + row) * 4) * 8u;
        sts64(x + ch * 8, w, e);
        asm volatile("bar.sync %0, 128;" ::"r"(1 + quarter) : "memory");
        const uint4 x01 = lds128(x);
        const uint4 x23 = lds128(x + 16);
        uint32_t fw[4] = {x01.x, x01.z, x23.x, x23.z};
        if (partial) {
          const uint32_t ee[4] = {x01.y, x01.w, x23.y, x23.w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t eb = ee[c];
            while (eb != 0u && eq_seen < take_eq) {
              const uint32_t low = eb & (0u - eb);
              fw[c] |= low;
              eb ^= low;
              ++eq_seen;
            }
            // The ties that stay out are listed for the attention sweep, which otherwise selects
            // by `score >= threshold` (one writer per row; a second part continues part 0's list).
            if (ch == 0) {
              while (eb != 0u) {
                if (ex_seen < static_cast<uint32_t>(kMaxExcl))
                  excl_row[ex_seen] = (kt0 + j) * kTile + c * 32 + (__ffs(eb) - 1);
                eb &= eb - 1u;
                ++ex_seen;
              }
            }
          }
        }
        int off = cnt, cnt_new = cnt;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int n = __popc(fw[c]);
          if (c < ch) off += n;
          cnt_new += n;
        }
        // (identical for the row's four threads) entries of earlier tiles are visible since the barrier
        const bool ring_ok = cnt_new - flushed <= kRing;
        const int upto = min(ring_ok ? (cnt & ~7) : cnt, cap_out);
        if (row_ok && ch == (j & 3) && upto > flushed) flush(flushed, upto);
        uint32_t mine = fw[0];
#pragma unroll
        for (int c = 1; c < 4; ++c) mine = (ch == c) ? fw[c] : mine;
        while (mine != 0u) {
          const int i = __ffs(mine) - 1;
          mine &= mine - 1u;
          if (row_ok && off < cap_out) {
            (void)checked_index(key0 + i, p.Tk, p.status);
            const uint32_t v = relu_bits(lds32(stage + static_cast<uint32_t>((i >> 2) * 32 * 16 + (i & 3) * 4)));
            if (ring_ok) {
              sts32(ring_i + ((off & (kRing - 1)) << 2), static_cast<uint32_t>(key0 + i));
              sts32(ring_s + ((off & (kRing - 1)) << 2), v);
            } else {
              idx_row[off] = key0 + i;
              sc_row[off] = __uint_as_float(v);
            }
          }
          ++off;
        }
        flushed = ring_ok ? max(flushed, upto) : min(cnt_new, cap_out);
        cnt = cnt_new;
        if (mask_row != nullptr && ch == (j & 3)) {
          mask_row[static_cast<int64_t>(j) * kTile] = make_uint4(fw[0], fw[1], fw[2], fw[3]);
        }
        __syncwarp();   // the staging tile is rewritten by the next tile
      }
      asm volatile("bar.sync %0, 128;" ::"r"(1 + quarter) : "memory");
      if (row_ok && ch == 0) flush(flushed, min(cnt, cap_out));
      if (collect) {
        // how many candidates this part found for the row; a list over capacity flags the query tile
        if (row_ok && ch == 0) {
          p.cand_cnt[grow * p.split + part] = static_cast<uint32_t>(cnt);
          if (cnt > cap_out || !ok) p.flags_out[tile] = 1u;
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- exact top-k of every row among the candidates the collect pass listed (all keys at or above a
// lower bound of the row's threshold, ascending per part).  One CTA of four warps per row: the candidates' score
// bits go to shared memory, a 4 x 8-bit radix select finds the k-th largest (lanes with the same digit
// add to the histogram with one atomic), then the candidates are filtered in order: keys above the
// threshold and the first `take` keys equal to it, ascending.  The row's membership bits are collected
// in shared memory and written as the row's 16-byte pieces of the tile-major mask; unselected ties go
// to the row's exclusion list.  A row with fewer than k candidates (the lower bound was too high) flags
// its query tile for the exact passes.
struct SelectParams {
  int B, Tq, Tk, top_k, k_eff, nQT, nKT, split, cand_cap;
  const int32_t* cand_idx;
  const float* cand_sc;
  const uint32_t* cand_cnt;
  uint32_t* flags;             // [B*nQT]
  int32_t* idx;
  float* scores;
  uint32_t *st_prefix, *st_kth, *st_neq;
  int32_t* st_excl;
  uint32_t* maskbits;          // may be null
};
constexpr int kSelWarps = 4;                      // one row per CTA of four warps (~17 KB of shared memory at 4 k candidates;
                                                  // eight warps per row measured slower)

__global__ void __launch_bounds__(32 * kSelWarps) dsa_select_kernel(const SelectParams p) {
  extern __shared__ uint32_t sel_smem[];
  constexpr int kThreads = 32 * kSelWarps;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t row = blockIdx.x;
  const int cap_all = p.split * p.cand_cap;
  uint32_t* sc_s = sel_smem;                     // the candidates' score bits, later their output slots
  uint32_t* hist = sc_s + cap_all;               // 256 bins
  uint32_t* xch = hist + 256;                    // 32 words of exchange between the warps
  const int b = static_cast<int>(row / p.Tq), t = static_cast<int>(row % p.Tq);
  const int tile = b * p.nQT + t / kTile;
  // Another row of the same query tile may flag the tile while this CTA starts: ONE thread reads the
  // flag, so the whole CTA takes the same way (threads that left alone would leave the exchange words
  // and the histogram of the others unwritten).
  __shared__ uint32_t tile_flagged;
  // (the row's counts and lower bound are asked for before the flag is waited for: one memory
  // latency instead of three in a row)
  int n_part[2] = {0, 0};
  n_part[0] = static_cast<int>(__ldg(p.cand_cnt + row * p.split));
  if (p.split > 1) n_part[1] = static_cast<int>(__ldg(p.cand_cnt + row * p.split + 1));
  const uint32_t t0 = __ldcg(p.st_prefix + row);
  if (tid == 0) tile_flagged = *reinterpret_cast<volatile uint32_t*>(p.flags + tile);
  __syncthreads();
  if (tile_flagged != 0u) return;
  if (static_cast<uint32_t>(n_part[0]) > static_cast<uint32_t>(p.cand_cap) ||
      static_cast<uint32_t>(n_part[1]) > static_cast<uint32_t>(p.cand_cap))
    return;                                                          // (flagged by the collect pass)
  const int n = n_part[0] + n_part[1];
  if (n < p.k_eff) {
    if (tid == 0) p.flags[tile] = 1u;
    return;
  }
  hist[tid] = 0u;
  hist[tid + 128] = 0u;
  if (tid < 32) xch[tid] = 0u;
  __syncthreads();
  // ---- k-th largest bit pattern (scores are >= 0: bit patterns order like the values).  Every
  // candidate is >= the row's lower bound t0 and the threshold lies a little above it, so the select
  // runs on u = bits - t0 as three 8-bit digits of a 24-bit number (candidates with u >= 2^24, far
  // above the threshold, are only counted).  The candidates come in with 16-byte loads (the lists
  // start on 32-byte boundaries and their capacity is a multiple of 8, so the last load may bring up
  // to three unused entries); the same loop counts the far-above ones and bins the first digit.
  uint32_t kth = static_cast<uint32_t>(p.k_eff), n_eq = 0, prefix = 0;
  {
    uint32_t big = 0;
    for (int q = 0, off = 0; q < p.split; off += n_part[q], ++q) {
      const float4* src4 = reinterpret_cast<const float4*>(p.cand_sc + (row * p.split + q) * p.cand_cap);
      const int nq = n_part[q], n4 = (nq + 3) >> 2;
#pragma unroll 4
      for (int i4 = tid; i4 < n4; i4 += kThreads) {
        const float4 x = __ldg(src4 + i4);
        const uint32_t xb[4] = {__float_as_uint(x.x), __float_as_uint(x.y), __float_as_uint(x.z), __float_as_uint(x.w)};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = i4 * 4 + e;
          if (i < nq) {
            sc_s[off + i] = xb[e];
            const uint32_t u = xb[e] - t0;
            if (u >= (1u << 24)) ++big;
            else atomicAdd(&hist[u >> 16], 1u);
          }
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) big += __shfl_xor_sync(0xffffffffu, big, o);
    if (lane == 0 && big != 0u) atomicAdd(&xch[0], big);
    __syncthreads();
    big = xch[0];
    if (big >= kth) {                              // the threshold is far above the bound: leave it to the exact passes
      if (tid == 0) p.flags[tile] = 1u;
      return;
    }
    kth -= big;
  }
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = 16 - 8 * pass;
    if (pass > 0) {
      for (int i = tid; i < n; i += kThreads) {
        const uint32_t u = sc_s[i] - t0;
        if (u < (1u << 24) && (u >> (shift + 8)) == (prefix >> (shift + 8))) atomicAdd(&hist[(u >> shift) & 255u], 1u);
      }
      __syncthreads();
    }
    if (warp == 0) {
      // lane l owns bins 8 * (31 - l) .. + 7: lane 0 the highest digits
      uint32_t c = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) c += hist[(31 - lane) * 8 + i];
      uint32_t cum = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, cum, o);
        if (lane >= o) cum += up;
      }
      const uint32_t hit = __ballot_sync(0xffffffffu, cum >= kth);     // never empty: the counted candidates are >= kth
      const int L = __ffs(hit) - 1;
      if (lane == L) {
        uint32_t above = cum - c;
        for (int i = 7; i >= 0; --i) {
          const uint32_t h = hist[(31 - lane) * 8 + i];
          if (above + h >= kth) {
            xch[1] = static_cast<uint32_t>((31 - lane) * 8 + i);      // the digit
            xch[2] = above;
            xch[3] = h;
            break;
          }
          above += h;
        }
      }
    }
    __syncthreads();
    prefix |= xch[1] << shift;
    kth -= xch[2];
    n_eq = xch[3];
    __syncthreads();
    hist[tid] = 0u;
    hist[tid + 128] = 0u;
    __syncthreads();
  }
  const uint32_t thr = prefix + t0, take = kth;  // `take` of the n_eq keys equal to the threshold are selected
  // ---- filter, ascending.  First in shared memory only: every candidate's score is replaced by its
  // output slot (or a code for "unselected tie" / "rejected").  Every warp takes a contiguous quarter
  // of the candidates: the quarters are counted first (keys above the threshold, ties), then every warp
  // knows where its quarter starts and walks it on its own.
  constexpr uint32_t kRejected = 0xffffffffu, kCutTie = 0x80000000u;
  const uint32_t lt = (1u << lane) - 1u;
  {
    const int quarter = ((n + kThreads - 1) / kThreads) * 32;       // candidates per warp, a multiple of 32
    const int lo_i = warp * quarter, hi_i = min(n, lo_i + quarter);
    uint32_t gt = 0, eq = 0;
    for (int i = lo_i + lane; i < hi_i; i += 32) {
      const uint32_t v = sc_s[i];
      gt += v > thr ? 1u : 0u;
      eq += v == thr ? 1u : 0u;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      gt += __shfl_xor_sync(0xffffffffu, gt, o);
      eq += __shfl_xor_sync(0xffffffffu, eq, o);
    }
    if (lane == 0) {
      xch[4 + 2 * warp] = gt;
      xch[5 + 2 * warp] = eq;
    }
    __syncthreads();
    uint32_t out = 0, eq_seen = 0, ex_seen = 0;       // totals of the quarters before this one
    for (int w = 0; w < warp; ++w) {
      const uint32_t g = xch[4 + 2 * w], e = xch[5 + 2 * w];
      const uint32_t tk = min(e, take > eq_seen ? take - eq_seen : 0u);   // ties of that quarter that are selected
      out += g + tk;
      ex_seen += e - tk;
      eq_seen += e;
    }
    for (int base = lo_i; base < hi_i; base += 32) {
      const int i = base + lane;
      const bool in = i < hi_i;
      const uint32_t v = in ? sc_s[i] : 0u;
      const bool is_eq = in && v == thr;
      const uint32_t eq_mask = __ballot_sync(0xffffffffu, is_eq);
      const bool taken = is_eq && eq_seen + __popc(eq_mask & lt) < take;
      const uint32_t taken_mask = __ballot_sync(0xffffffffu, taken);
      const bool sel = (in && v > thr) || taken;
      const uint32_t sel_mask = __ballot_sync(0xffffffffu, sel);
      if (in) {
        uint32_t code = kRejected;
        if (sel) code = out + __popc(sel_mask & lt);
        else if (is_eq) code = kCutTie | (ex_seen + __popc((eq_mask & ~taken_mask) & lt));
        sc_s[i] = code;
      }
      out += __popc(sel_mask);
      eq_seen += __popc(eq_mask);
      ex_seen += __popc(eq_mask & ~taken_mask);
    }
  }
  __syncthreads();
  // ---- then the outputs: independent steps over the candidate lists in global memory
  int32_t* idx_row = p.idx + row * p.top_k;
  float* sc_row = p.scores + row * p.top_k;
  const int qt = t / kTile, r = t % kTile;
  for (int q = 0, off = 0; q < p.split; off += n_part[q], ++q) {
    const int4* ksrc4 = reinterpret_cast<const int4*>(p.cand_idx + (row * p.split + q) * p.cand_cap);
    const float4* vsrc4 = reinterpret_cast<const float4*>(p.cand_sc + (row * p.split + q) * p.cand_cap);
    const int nq = n_part[q], n4 = (nq + 3) >> 2;
#pragma unroll 2
    for (int i4 = tid; i4 < n4; i4 += kThreads) {
      const int4 kk = __ldg(ksrc4 + i4);
      const float4 vv = __ldg(vsrc4 + i4);
      const int keys[4] = {kk.x, kk.y, kk.z, kk.w};
      const float vals[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = i4 * 4 + e;
        if (i >= nq) break;
        const uint32_t code = sc_s[off + i];
        const int key = keys[e];
        if (code == kRejected || (code & kCutTie)) {
          // the collect pass set the bit of every candidate
          if (p.maskbits != nullptr) {
            const size_t word = (((static_cast<size_t>(b) * p.nQT + qt) * p.nKT + (key >> 7)) * kTile + r) * 4 + ((key & 127) >> 5);
            atomicAnd(p.maskbits + word, ~(1u << (key & 31)));
          }
          if (code != kRejected) {
            const uint32_t ex = code & ~kCutTie;
            if (ex < static_cast<uint32_t>(kMaxExcl)) p.st_excl[row * kMaxExcl + ex] = key;
          }
        } else if (code < static_cast<uint32_t>(p.k_eff)) {     // (always: gt + take == k_eff)
          idx_row[code] = key;
          sc_row[code] = vals[e];
        }
      }
    }
  }
  if (tid == 0) {
    p.st_prefix[row] = thr;
    p.st_kth[row] = take;
    p.st_neq[row] = n_eq;
  }
}

// valid[b,t,s] = s < k_eff ; slots >= k_eff of idx / scores are zeroed.  VEC consecutive slots per
// thread (VEC divides top_k, so a thread never crosses a row).
template <int VEC>
__global__ void fill_valid_kernel(float* __restrict__ valid, int32_t* __restrict__ idx, float* __restrict__ scores,
                                  int64_t total, int top_k, int k_eff) {
  const int64_t gid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
  if (gid >= total) return;
  const int s0 = static_cast<int>(gid % top_k);
  if constexpr (VEC == 4) {
    *reinterpret_cast<float4*>(valid + gid) = make_float4(s0 < k_eff ? 1.f : 0.f, s0 + 1 < k_eff ? 1.f : 0.f,
                                                          s0 + 2 < k_eff ? 1.f : 0.f, s0 + 3 < k_eff ? 1.f : 0.f);
  } else {
    valid[gid] = s0 < k_eff ? 1.f : 0.f;
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    if (s0 + i >= k_eff) {
      idx[gid + i] = 0;
      scores[gid + i] = 0.f;
    }
  }
}

// -------------------------------------------------------------------- host
static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct WorkspaceLayout {
  size_t wq_off, wk_off, prefix_off, kth_off, neq_off, excl_off, kmax_off, flags_off, flags2_off;
  size_t flags3_off, tickets_off, cnt0_off, eq0_off, ghist_off, glist_off, gcnt_off;   // key-range split only
  int split;
  size_t total;
};
// Two CTAs share a query tile (each sweeps half of the key tiles) when that fills the SMs better:
// with few query tiles (one rank of a sequence-sharded run: 64 tiles on 148 SMs) or when the last
// wave of whole-tile CTAs would be far from full (512 tiles = 3.46 waves), provided the key range
// is long enough to be worth merging.
constexpr int kSplitMinKeyTiles = 64;
static int split_factor(int B, int Tq, int Tk) {
  const int64_t tiles = static_cast<int64_t>(B) * ((Tq + kTile - 1) / kTile);
  if ((Tk + kTile - 1) / kTile < kSplitMinKeyTiles) return 1;
  const int n_sm = sm_count();
  const double whole = static_cast<double>((tiles + n_sm - 1) / n_sm);
  const double halves = static_cast<double>((2 * tiles + n_sm - 1) / n_sm) / 2 + 0.05;   // + merge
  return halves < whole ? 2 : 1;
}
static WorkspaceLayout workspace_layout(int B, int Tq, int Tk) {
  WorkspaceLayout L;
  size_t off = 0;
  L.wq_off = off;
  off += align_up(static_cast<size_t>(B) * Tq * kIdxDim * 4, 1024);
  L.wk_off = off;
  off += align_up(static_cast<size_t>(B) * Tk * kIdxDim * 4, 1024);
  L.prefix_off = off;
  off += align_up(static_cast<size_t>(B) * Tq * 4, 1024);
  L.kth_off = off;
  off += align_up(static_cast<size_t>(B) * Tq * 4, 1024);
  L.neq_off = off;
  off += align_up(static_cast<size_t>(B) * Tq * 4, 1024);
  L.excl_off = off;     // per query row: the unselected keys among the ties at its threshold
  off += align_up(static_cast<size_t>(B) * Tq * kMaxExcl * 4, 1024);
  L.kmax_off = off;     // per (batch, head) key-norm maxima of the attention kernel, up to 1024 entries
  off += 4096;
  const size_t tiles = static_cast<size_t>(B) * ((Tq + kTile - 1) / kTile);
  L.flags_off = off;    // per 128-query tile: redo the two first passes classically
  off += align_up(tiles * 4, 1024);
  L.flags2_off = off;   // per 128-query tile: redo the two last passes classically
  off += align_up(tiles * 4, 1024);
  L.split = split_factor(B, Tq, Tk);
  L.flags3_off = L.tickets_off = L.cnt0_off = L.eq0_off = L.ghist_off = L.glist_off = L.gcnt_off = off;
  if (L.split > 1) {
    L.flags3_off = off;   // per tile: emit runs unsplit
    off += align_up(tiles * 4, 1024);
    L.tickets_off = off;
    off += align_up(tiles * 4, 1024);
    L.cnt0_off = off;
    off += align_up(static_cast<size_t>(B) * Tq * 4, 1024);
    L.eq0_off = off;
    off += align_up(static_cast<size_t>(B) * Tq * 4, 1024);
    L.ghist_off = off;
    off += align_up(tiles * 2 * kTile * kHistStride * 4, 1024);
    L.glist_off = off;
    off += align_up(tiles * 2 * kTile * kListStride * 2, 1024);
    L.gcnt_off = off;
    off += align_up(tiles * 2 * kTile * 4, 1024);
  }
  L.total = off;
  return L;
}

// The short form of the selection (estimate, collect, select) needs candidate lists behind the base
// layout: 2.0-2.5 k candidates per row (1.3-1.7 k expected), divided over the parts of a split key range.
struct FastLayout {
  bool ok;                 // the shape qualifies
  int cand_cap;            // per (row, part)
  int est_rank;            // rank in the sample at which the estimate pass takes a row's lower bound
  size_t idx_off, sc_off, cnt_off, total;
};
static FastLayout fast_layout(int B, int Tq, int Tk, int top_k) {
  FastLayout F;
  const WorkspaceLayout L = workspace_layout(B, Tq, Tk);
  const int k_eff = top_k < Tk ? top_k : Tk;
  // Worth it where the sweeps dominate: the sample (2 x 32 key tiles) is a small part of a sweep and the
  // per-row select (rows x 1.5 k candidates) is small beside one (measured: 4.7 against 6.5 ms at 65536
  // tokens and one key in 32; slower than the three-sweep form at 16384 and 32768 tokens).
  F.ok = Tk >= 49152 && Tk <= 262144 && static_cast<int64_t>(k_eff) * 16 <= Tk;
  // The lower bound is the sample's value at rank r = m * mu, mu = k n_s / Tk the expected number of a
  // row's selected keys inside the sample of n_s keys.  Too high a bound (the row finds fewer than k
  // candidates) needs more than r of the row's selected keys inside the sample: (m - 1) sqrt(mu)
  // standard deviations, set to 4.75 (one row in a million; a query tile has 128).  Too low a bound
  // overflows the lists: the candidates number about m k (1 +- 1 / sqrt(r)), plus ~5 % for rounding
  // the bound down to a multiple of 2^16 bit patterns; the lists hold 4.5 standard deviations more
  // than that (2.0 k at one key in 32, 2.4 k at one in 64), and beyond 2.5 k -- selections sparser
  // than about one key in 70 -- the three sweeps are kept.
  F.est_rank = 0;
  int64_t cap_all = 16;
  if (F.ok) {
    const double n_s = static_cast<double>(kEstimateTiles) * kTile;
    const double mu = static_cast<double>(k_eff) * n_s / Tk;
    const double r = std::ceil(mu + 4.75 * std::sqrt(mu));
    const double cap = 1.05 * (r / mu) * k_eff * (1.0 + 4.5 / std::sqrt(r));
    cap_all = (static_cast<int64_t>(std::ceil(cap)) + 15) / 16 * 16;
    F.ok = cap <= 2.5 * k_eff && cap_all <= 12288;
    F.est_rank = static_cast<int>(r);
  }
  F.cand_cap = static_cast<int>(cap_all / L.split);
  const size_t rows = static_cast<size_t>(B) * Tq;
  size_t off = L.total;
  F.idx_off = off;
  off += align_up(rows * cap_all * 4, 1024);
  F.sc_off = off;
  off += align_up(rows * cap_all * 4, 1024);
  F.cnt_off = off;
  off += align_up(rows * L.split * 4, 1024);
  F.total = F.ok ? off : L.total;
  return F;
}

// Where the collapsed indexer queries / keys of the last indexer call live inside its workspace.
void dsa_workspace_views(void* workspace, int B, int Tq, int Tk, float** wq, float** wk, uint32_t** prefix,
                         uint32_t** kth, uint32_t** neq, uint32_t** kmax2, int32_t** excl) {
  const WorkspaceLayout L = workspace_layout(B, Tq, Tk);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  *wq = reinterpret_cast<float*>(ws + L.wq_off);
  *wk = reinterpret_cast<float*>(ws + L.wk_off);
  *prefix = reinterpret_cast<uint32_t*>(ws + L.prefix_off);
  *kth = reinterpret_cast<uint32_t*>(ws + L.kth_off);
  *neq = reinterpret_cast<uint32_t*>(ws + L.neq_off);
  *kmax2 = reinterpret_cast<uint32_t*>(ws + L.kmax_off);
  *excl = reinterpret_cast<int32_t*>(ws + L.excl_off);
}

template <typename T>
static void launch_collapse(const void* x, const int64_t* s, const float* w, float* out, int B, int Tn, int IH,
                            int ID, cudaStream_t st) {
  const int64_t total = static_cast<int64_t>(B) * Tn * kIdxDim;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
  collapse_heads_kernel<T><<<blocks, threads, 0, st>>>(static_cast<const T*>(x), s[0], s[1], s[2], s[3], w, out, B,
                                                         Tn, IH, ID);
}

int dsa_workspace_bytes_topk_impl(int B, int Tq, int Tk, int top_k, size_t* bytes) {
  if (bytes == nullptr) return SWV_ERR_NULL;
  if (B < 1 || Tq < 1 || Tk < 1 || top_k < 1) return SWV_ERR_SHAPE;
  *bytes = fast_layout(B, Tq, Tk, top_k).total;
  return SWV_OK;
}

int dsa_workspace_bytes_impl(int B, int Tq, int Tk, size_t* bytes) {
  if (bytes == nullptr) return SWV_ERR_NULL;
  if (B < 1 || Tq < 1 || Tk < 1) return SWV_ERR_SHAPE;
  *bytes = workspace_layout(B, Tq, Tk).total;
  return SWV_OK;
}

int dsa_mask_bytes_impl(int B, int Tq, int Tk, size_t* bytes) {
  if (bytes == nullptr) return SWV_ERR_NULL;
  if (B < 1 || Tq < 1 || Tk < 1) return SWV_ERR_SHAPE;
  const size_t nQT = (Tq + kTile - 1) / kTile, nKT = (Tk + kTile - 1) / kTile;
  *bytes = static_cast<size_t>(B) * nQT * nKT * kTile * 16;
  return SWV_OK;
}

int dsa_indexer_topk_impl(const void* q_idx, const int64_t* qs, const void* k_idx, const int64_t* ks, int dtype,
                          const float* w, int B, int Tq, int Tk, int IH, int ID, int top_k, int32_t* idx,
                          float* valid, float* scores, uint32_t* maskbits, void* workspace, size_t workspace_bytes,
                          int* status, cudaStream_t st, bool allow_split) {
  // q_idx == k_idx == NULL: the workspace already holds the collapsed indexer vectors of these
  // B x Tq queries and B x Tk keys (swv_dsa_prologue_fwd wrote them); the collapse step is skipped
  const bool precollapsed = q_idx == nullptr && k_idx == nullptr;
  if ((!precollapsed && (!q_idx || !k_idx || !w || !qs || !ks)) || !idx || !valid || !scores || !workspace || !status)
    return SWV_ERR_NULL;
  if (dtype != SWV_F32 && dtype != SWV_BF16 && dtype != SWV_F16) return SWV_ERR_DTYPE;
  if (B < 1 || Tq < 1 || Tk < 1 || IH < 1 || ID < 1 || top_k < 1) return SWV_ERR_SHAPE;
  if (ID > kIdxDim) return SWV_ERR_UNSUPPORTED;
  WorkspaceLayout L = workspace_layout(B, Tq, Tk);
  if (!allow_split && L.split > 1) {
    L.split = 1;
    L.total = L.flags3_off;      // the split regions are the tail of the layout
  }
  if (workspace_bytes < L.total) return SWV_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return SWV_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(idx) & 3) || (reinterpret_cast<uintptr_t>(scores) & 3) ||
      (reinterpret_cast<uintptr_t>(valid) & 3) || (maskbits && (reinterpret_cast<uintptr_t>(maskbits) & 15)))
    return SWV_ERR_ALIGN;

  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* wq = reinterpret_cast<float*>(ws + L.wq_off);
  float* wk = reinterpret_cast<float*>(ws + L.wk_off);

  CUtensorMap tm_q, tm_k;
  int rc = make_tmap_3d(&tm_q, wq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, kIdxDim, Tq, B, kIdxDim * 4,
                        static_cast<uint64_t>(Tq) * kIdxDim * 4, 32, kTile);
  if (rc != SWV_OK) return rc;
  rc = make_tmap_3d(&tm_k, wk, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, kIdxDim, Tk, B, kIdxDim * 4,
                    static_cast<uint64_t>(Tk) * kIdxDim * 4, 32, kTile);
  if (rc != SWV_OK) return rc;

  if (precollapsed) {
    // nothing to do
  } else if (dtype == SWV_F32) {
    launch_collapse<float>(q_idx, qs, w, wq, B, Tq, IH, ID, st);
    launch_collapse<float>(k_idx, ks, w, wk, B, Tk, IH, ID, st);
  } else if (dtype == SWV_BF16) {
    launch_collapse<__nv_bfloat16>(q_idx, qs, w, wq, B, Tq, IH, ID, st);
    launch_collapse<__nv_bfloat16>(k_idx, ks, w, wk, B, Tk, IH, ID, st);
  } else {
    launch_collapse<__half>(q_idx, qs, w, wq, B, Tq, IH, ID, st);
    launch_collapse<__half>(k_idx, ks, w, wk, B, Tk, IH, ID, st);
  }

  IndexerParams p;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.top_k = top_k;
  p.nQT = (Tq + kTile - 1) / kTile;
  p.nKT = (Tk + kTile - 1) / kTile;
  p.st_prefix = reinterpret_cast<uint32_t*>(ws + L.prefix_off);
  p.st_kth = reinterpret_cast<uint32_t*>(ws + L.kth_off);
  p.st_neq = reinterpret_cast<uint32_t*>(ws + L.neq_off);
  p.st_excl = reinterpret_cast<int32_t*>(ws + L.excl_off);
  p.idx = idx; p.scores = scores; p.maskbits = maskbits; p.status = status; p.pass = 0;
  p.kind = kKindFirst; p.only_flagged = 0;
  uint32_t* flags_a = reinterpret_cast<uint32_t*>(ws + L.flags_off);
  uint32_t* flags_b = reinterpret_cast<uint32_t*>(ws + L.flags2_off);
  p.flags_in = flags_a; p.flags_out = flags_a;
  p.split = L.split;
  p.nKT0 = (p.nKT + 1) / 2;
  p.flags_spec = flags_a;
  p.flags_unsplit = reinterpret_cast<uint32_t*>(ws + L.flags3_off);
  p.tickets = reinterpret_cast<uint32_t*>(ws + L.tickets_off);
  p.st_cnt0 = reinterpret_cast<uint32_t*>(ws + L.cnt0_off);
  p.st_eq0 = reinterpret_cast<uint32_t*>(ws + L.eq0_off);
  p.ghist = reinterpret_cast<uint32_t*>(ws + L.ghist_off);
  p.glist = reinterpret_cast<uint16_t*>(ws + L.glist_off);
  p.gcnt = reinterpret_cast<uint32_t*>(ws + L.gcnt_off);
  if (L.split > 1)
    SWV_CUDA_OK(cudaMemsetAsync(p.tickets, 0, static_cast<size_t>(B) * p.nQT * 4, st));

  SWV_CUDA_OK(cudaFuncSetAttribute(indexer_tiles_kernel<kModeHist>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(tile_smem_bytes(kModeHist))));
  SWV_CUDA_OK(cudaFuncSetAttribute(indexer_tiles_kernel<kModeEmit>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(tile_smem_bytes(kModeEmit))));
  const unsigned grid = static_cast<unsigned>(B) * p.nQT * L.split;
  // Radix select of every row's K-th largest score, 32 bits:
  //   bytes 0-1: one speculative fused pass (top 16 bits estimated from a sample, checked with exact
  //              counts); query tiles where the check fails redo the two classic histogram passes;
  //   bytes 2-3: one candidate-list pass; tiles whose list overflowed (massive ties) redo the two
  //              classic histogram passes.
  const size_t hs = tile_smem_bytes(kModeHist);
  p.collect = 0; p.est_rank = 0; p.cand_cap = 0;
  p.cand_idx = nullptr; p.cand_sc = nullptr; p.cand_cnt = nullptr;
  const FastLayout F = fast_layout(B, Tq, Tk, top_k);
  if (F.ok && allow_split && workspace_bytes >= F.total) {
    // Sparse top-k on a long key range, and the caller brought the larger workspace
    // (swv_dsa_workspace_bytes_topk): TWO sweeps instead of three.
    //   estimate: a lower bound of every row's threshold from a sample of 32 key tiles -- the value a
    //             little below the row's rank in the sample (4.75 standard deviations of safety);
    //   collect : one sweep lists every key at or above the bound (1.5 k per row at one key in 32), ascending, and
    //             writes their membership bits;
    //   select  : per row, the exact k-th largest among its candidates, the final lists, the bits of the
    //             rejected candidates cleared.
    // A query tile with a row that found fewer than k candidates, or more than the lists hold, is
    // flagged and redone by the four classic histogram passes and the emit pass (which return at once
    // for unflagged tiles).
    p.cand_cap = F.cand_cap;
    p.cand_idx = reinterpret_cast<int32_t*>(ws + F.idx_off);
    p.cand_sc = reinterpret_cast<float*>(ws + F.sc_off);
    p.cand_cnt = reinterpret_cast<uint32_t*>(ws + F.cnt_off);
    SWV_CUDA_OK(cudaMemsetAsync(flags_a, 0, static_cast<size_t>(B) * p.nQT * 4, st));
    p.pass = 0; p.kind = kKindEstimate; p.only_flagged = 0; p.est_rank = F.est_rank;
    indexer_tiles_kernel<kModeHist><<<grid, 576, hs, st>>>(tm_q, tm_k, p);
    p.collect = 1; p.flags_out = flags_a;
    indexer_tiles_kernel<kModeEmit><<<grid, 576, tile_smem_bytes(kModeEmit), st>>>(tm_q, tm_k, p);
    {
      SelectParams sp;
      sp.B = B; sp.Tq = Tq; sp.Tk = Tk; sp.top_k = top_k; sp.k_eff = top_k < Tk ? top_k : Tk;
      sp.nQT = p.nQT; sp.nKT = p.nKT; sp.split = L.split; sp.cand_cap = F.cand_cap;
      sp.cand_idx = p.cand_idx; sp.cand_sc = p.cand_sc; sp.cand_cnt = p.cand_cnt;
      sp.flags = flags_a; sp.idx = idx; sp.scores = scores;
      sp.st_prefix = p.st_prefix; sp.st_kth = p.st_kth; sp.st_neq = p.st_neq; sp.st_excl = p.st_excl;
      sp.maskbits = maskbits;
      const size_t sel_smem = (static_cast<size_t>(L.split) * F.cand_cap + 256 + 32) * 4;
      SWV_CUDA_OK(cudaFuncSetAttribute(dsa_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sel_smem)));
      const int64_t rows = static_cast<int64_t>(B) * Tq;
      dsa_select_kernel<<<static_cast<unsigned>(rows), 32 * kSelWarps, sel_smem, st>>>(sp);
    }
    p.collect = 0; p.only_flagged = 1; p.flags_in = flags_a; p.flags_unsplit = flags_a;
    for (int pass = 0; pass < 4; ++pass) {
      p.pass = pass; p.kind = pass == 0 ? kKindFirst : kKindMid;
      indexer_tiles_kernel<kModeHist><<<grid, 576, hs, st>>>(tm_q, tm_k, p);
    }
    indexer_tiles_kernel<kModeEmit><<<grid, 576, tile_smem_bytes(kModeEmit), st>>>(tm_q, tm_k, p);
  } else {
  p.pass = 1; p.kind = kKindSpec; p.only_flagged = 0; p.flags_out = flags_a;
  indexer_tiles_kernel<kModeHist><<<grid, 576, hs, st>>>(tm_q, tm_k, p);
  p.only_flagged = 1; p.flags_in = flags_a;
  p.pass = 0; p.kind = kKindFirst;
  indexer_tiles_kernel<kModeHist><<<grid, 576, hs, st>>>(tm_q, tm_k, p);
  p.pass = 1; p.kind = kKindMid;
  indexer_tiles_kernel<kModeHist><<<grid, 576, hs, st>>>(tm_q, tm_k, p);
  p.pass = 2; p.kind = kKindCand; p.only_flagged = 0; p.flags_out = flags_b;
  indexer_tiles_kernel<kModeHist><<<grid, 576, hs, st>>>(tm_q, tm_k, p);
  p.only_flagged = 1; p.flags_in = flags_b; p.kind = kKindMid;
  for (int pass = 2; pass < 4; ++pass) {
    p.pass = pass;
    indexer_tiles_kernel<kModeHist><<<grid, 576, hs, st>>>(tm_q, tm_k, p);
  }
  p.only_flagged = 0;
  indexer_tiles_kernel<kModeEmit><<<grid, 576, tile_smem_bytes(kModeEmit), st>>>(tm_q, tm_k, p);
  }

  const int64_t total = static_cast<int64_t>(B) * Tq * top_k;
  const int k_eff = top_k < Tk ? top_k : Tk;
  if ((top_k & 3) == 0 && (reinterpret_cast<uintptr_t>(valid) & 15) == 0)
    fill_valid_kernel<4><<<static_cast<unsigned>((total / 4 + 255) / 256), 256, 0, st>>>(valid, idx, scores, total,
                                                                                          top_k, k_eff);
  else
    fill_valid_kernel<1><<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(valid, idx, scores, total, top_k,
                                                                                      k_eff);
  SWV_CUDA_OK(cudaGetLastError());
  return SWV_OK;
}

int dsa_prologue_impl(void* q, const int64_t* qs, void* k, const int64_t* ks, int qk_dtype, const void* q_idx,
                      const int64_t* qis, const void* k_idx, const int64_t* kis, int idx_dtype, const float* w,
                      const float* coords, float coord_high, float theta, int skip, int B, int T, int H, int D, int IH,
                      int ID, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (!q_idx || !k_idx || !w || !workspace || !qis || !kis) return SWV_ERR_NULL;
  if (coords != nullptr && (!q || !k || !qs || !ks)) return SWV_ERR_NULL;
  if (B < 1 || T < 1 || IH < 1 || ID < 1) return SWV_ERR_SHAPE;
  if (ID > kIdxDim) return SWV_ERR_UNSUPPORTED;
  if (idx_dtype != SWV_F32 && idx_dtype != SWV_BF16 && idx_dtype != SWV_F16) return SWV_ERR_DTYPE;
  if (coords != nullptr) {
    if (qk_dtype != SWV_F32 && qk_dtype != SWV_BF16) return SWV_ERR_DTYPE;
    if (H < 1 || D < 4 || (D % 4) != 0 || coord_high == 0.f || theta <= 0.f || skip < 0) return SWV_ERR_SHAPE;
    if (qs[3] != 1 || ks[3] != 1) return SWV_ERR_ALIGN;
  }
  WorkspaceLayout L = workspace_layout(B, T, T);
  if (workspace_bytes < L.flags3_off) return SWV_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return SWV_ERR_ALIGN;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* wq = reinterpret_cast<float*>(ws + L.wq_off);
  float* wk = reinterpret_cast<float*>(ws + L.wk_off);
  const unsigned grid = static_cast<unsigned>((static_cast<int64_t>(B) * T + 3) / 4);
  const float inv_high = coords != nullptr ? 1.0f / coord_high : 0.f;
  const float l2t = coords != nullptr ? log2f(theta) : 0.f;
  const int64_t z[4] = {0, 0, 0, 1};
  const int64_t* qq = coords != nullptr ? qs : z;
  const int64_t* kk = coords != nullptr ? ks : z;
#define SWV_PROLOGUE(TQ_, TI_)                                                                                 \
  dsa_prologue_kernel<TQ_, TI_><<<grid, 128, 0, st>>>(                                                         \
      static_cast<TQ_*>(q), qq[0], qq[1], qq[2], static_cast<TQ_*>(k), kk[0], kk[1], kk[2],                    \
      static_cast<const TI_*>(q_idx), qis[0], qis[1], qis[2], qis[3], static_cast<const TI_*>(k_idx), kis[0],  \
      kis[1], kis[2], kis[3], w, coords, inv_high, l2t, skip, wq, wk, B, T, H, D, IH, ID)
  const bool q32 = coords != nullptr && qk_dtype == SWV_F32;
  if (idx_dtype == SWV_F32) {
    if (q32) SWV_PROLOGUE(float, float);
    else SWV_PROLOGUE(__nv_bfloat16, float);
  } else if (idx_dtype == SWV_BF16) {
    if (q32) SWV_PROLOGUE(float, __nv_bfloat16);
    else SWV_PROLOGUE(__nv_bfloat16, __nv_bfloat16);
  } else {
    if (q32) SWV_PROLOGUE(float, __half);
    else SWV_PROLOGUE(__nv_bfloat16, __half);
  }
#undef SWV_PROLOGUE
  SWV_CUDA_OK(cudaGetLastError());
  return SWV_OK;
}

// ------------------------------------------------- entry point without a workspace argument
// Scratch for swv_dsa_indexer_topk_static_fwd: the same layout workspace_layout() describes,
// sized for kStaticMaxTokens query tokens and as many key tokens (batch included).  Every GPU
// whose context loads this library holds these bytes until the process exits.
constexpr int kStaticMaxTokens = 8192;
constexpr size_t kStaticScratchBytes =
    2 * static_cast<size_t>(kStaticMaxTokens) * kIdxDim * 4 + (3 + kMaxExcl) * static_cast<size_t>(kStaticMaxTokens) * 4 +
    4096 +
    2 * 32 * 1024 /* tile flags: up to 8192 query tiles (a batch of one-token sequences) */ +
    8 * 1024 /* per-section rounding */;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

int dsa_indexer_topk_static_impl(const void* q_idx, const int64_t* qs, const void* k_idx, const int64_t* ks,
                                 int dtype, const float* w, int B, int Tq, int Tk, int IH, int ID, int top_k,
                                 int32_t* idx, float* valid, float* scores, uint32_t* maskbits, int* status,
                                 cudaStream_t st) {
  if (B < 1 || Tq < 1 || Tk < 1) return SWV_ERR_SHAPE;
  if (static_cast<int64_t>(B) * Tq > kStaticMaxTokens || static_cast<int64_t>(B) * Tk > kStaticMaxTokens)
    return SWV_ERR_TOO_LARGE;
  if (workspace_layout(B, Tq, Tk).flags3_off > kStaticScratchBytes) return SWV_ERR_TOO_LARGE;
  // In host code `g_static_scratch` names a host-side stand-in, not device memory: the device
  // address has to be asked for, once per device, with that device current.
  // The address is cached per device in an atomic slot: host threads that make their first calls
  // at the same time each look it up and store the same value.
  constexpr int kMaxDevices = 64;
  static std::atomic<void*> dev_ptr[kMaxDevices];
  int dev = 0;
  SWV_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return SWV_ERR_UNSUPPORTED;
  void* scratch = dev_ptr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    if (cudaGetSymbolAddress(&scratch, g_static_scratch) != cudaSuccess || scratch == nullptr) return SWV_ERR_CUDA;
    dev_ptr[dev].store(scratch, std::memory_order_release);
  }
  return dsa_indexer_topk_impl(q_idx, qs, k_idx, ks, dtype, w, B, Tq, Tk, IH, ID, top_k, idx, valid, scores, maskbits,
                               scratch, kStaticScratchBytes, status, st, /*allow_split=*/false);
}

}  // namespace swv
