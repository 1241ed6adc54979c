// DSA top-k attention forward for sm_100a, dense-tile form.
//
// Replaces the reference's `_dsa_attention_fwd` Triton kernel
// (src/sparse_wsi_vit/models/deepseek_sparse_attention_kernels/kernels.py:450-564)
// for key lists produced by the indexer of this library, fused with the
// `routing_weights = scores * valid` step of the module
// (src/sparse_wsi_vit/models/deepseek_sparse_attention.py:73).
//
// With per-query token-granular selection and one K/V per head, gathering the
// selected rows moves one byte per FLOP; at top_k/T >= ~1/64 it is faster to
// sweep ALL key tiles on the tensor cores and apply the selection inside the
// online softmax.  One CTA owns (batch, 128 queries, a PAIR of heads):
//   warp 0      : TMA producer: collapsed indexer queries + Q of both heads once;
//                 per key tile the collapsed indexer keys, K and V of both heads.
//   warp 1      : UMMA issuer (one thread) of
//                   R    = wq wk^T       TF32, the routing-weight tile, shared by both heads;
//                                        bit-identical to the scores the indexer emitted
//   warps 10,11 : UMMA issuer (one thread each) of head 0 / head 1:
//                   S_h  = Q_h K_h^T     bf16
//                   O_h += P_h V_h       P from TMEM, V MN-major from smem, O stays in TMEM
//   warps 2..9  : softmax.  One-pass path: warp (quarter, half) owns 32 query rows x 64 key
//                 columns of every tile for both heads; two-pass path: warps 2..5 head 0,
//                 warps 6..9 head 1, one thread per query row
// Two softmax paths, chosen per CTA from the row constants the indexer left behind:
//   one pass  : a key is selected iff its recomputed score >= the row threshold; the
//               stabiliser is a constant Cauchy-Schwarz bound of the row's logits, so there
//               is no running maximum and no rescaling:  p = 2^(s*c - bound) * score.  The
//               weights of a tile are first packed to bf16 in registers so that R is free
//               for the next tile while the probabilities are computed.
//   two pass  : membership from the tile-major bitmask (ties cut by key index, members of
//               weight zero), exact maximum over the selected logits beside a lazily raised
//               stabiliser, the reference's 1e-6 clamp on the denominator reproduced:
//               out = O*c / max(l*c, 1e-6), c = 2^(m_used - m_true).
// TMEM (512 columns): R [0,128) | S_h fp32 [128+128h, +128), P_h (bf16x2) overwrites columns
// [0,32) (keys 0..63) and [64,96) (keys 64..127) of S_h as they are consumed | O_h fp32 [384+64h, +64).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace swv {

constexpr int kHeadDim = 64;
constexpr int kQTileBytes = kTile * kHeadDim * 2;     // 16 KiB bf16 tile
constexpr int kWTileBytes = kTile * kIdxDim * 4;      // 32 KiB fp32 indexer tile (two K halves)
constexpr int kAttnTmemCols = 512;
constexpr uint32_t kColR = 0, kColS = 128, kColO = 384;
#ifndef SWV_ATTN_SLICES
#define SWV_ATTN_SLICES 2
#endif
constexpr int kSlices = SWV_ATTN_SLICES;              // one-pass path: column slices of a tile (warps per row quarter)
constexpr int kSoftWarps = 4 * kSlices;               // softmax warps
constexpr int kSliceCols = kTile / kSlices;
constexpr int kAttnThreads = 64 + 32 * kSoftWarps + 64;   // TMA, R issuer, softmax warps, two head issuers
// Packed probabilities of the 16 keys starting at key0 (a multiple of 16) live in 8 columns inside the
// score columns of the slice that owns those keys, so a thread only overwrites scores it has read.
__host__ __device__ constexpr uint32_t p_col_of_key(int key0) {
  return static_cast<uint32_t>((key0 / kSliceCols) * kSliceCols + (key0 % kSliceCols) / 2);
}
constexpr float kRescaleStep = 8.0f;                  // raise the stabiliser only in steps of 2^8
constexpr float kMaxBound = 40.0f;                    // one-pass path: largest admissible |logit| bound (log2 units)

// shared memory map (bytes from the 1024-aligned base)
constexpr int kOffWq = 0;
constexpr int kOffWk = kOffWq + kWTileBytes;              // 2 stages
constexpr int kOffQ = kOffWk + 2 * kWTileBytes;           // 2 heads
constexpr int kOffK = kOffQ + 2 * kQTileBytes;            // [head][2 stages]
constexpr int kOffV = kOffK + 4 * kQTileBytes;            // [head] single stage
constexpr int kOffCtl = kOffV + 2 * kQTileBytes;

struct AttnParams {
  int B, H, Tq, Tk, nQT, nKT, nHP;
  const uint32_t* maskbits;
  const uint32_t *st_prefix, *st_kth, *st_neq;   // per query row, written by the indexer's select passes
  const int32_t* st_excl;                        // [B*Tq][kMaxExcl] ties at the threshold that are not selected
  const uint32_t* kmax2;                         // [B*H] max squared key norm, float bits
  const __nv_bfloat16* q;
  int64_t qsb, qsh, qst;
  void* o;
  int64_t osb, osh, ost;
  int o_dtype;
  float scale_log2;
  int* status;
  // Key-range split: with few CTAs (a rank of a sequence-sharded run) `split` CTAs share one
  // (query tile, head pair), each sweeping a share of the key tiles; every part leaves its
  // unnormalised output rows and row statistics in `scratch`, the part that arrives last adds them up.
  int split;
  float* scratch;        // [CTAs][split][2 heads][128 rows][kPartRec floats]
  uint32_t* tickets;     // [CTAs]
  // Diagnostic instantiation only: [B*Tq] number of keys each query row treated as selected (summed
  // over the column slices; counted once, by head pair 0).
  int* member_count;
  // When set: [B*nQT*nHP] only the (query tile, head pair)s with a non-zero entry are computed (the
  // list-driven kernel leaves those with a too large logit bound to this one).
  const uint32_t* only_flagged;
};
constexpr int kPartRec = kHeadDim + 4;                // output row + (l, m_used, m_true, pad)

struct AttnCtl {
  uint64_t q_full;
  uint64_t wk_full[2], wk_empty[2];
  uint64_t k_full[2][2], k_empty[2][2];
  uint64_t v_full[2], v_empty[2];
  uint64_t r_full, r_free;
  uint64_t s_full[2], p_full[2], pv_done[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t cta_exact;          // some row of the CTA needs the two-pass path
  uint32_t ticket;
  int next_ex[32 * kSoftWarps];   // per softmax thread: next key tile with an unselected tie of its row to drop
};

constexpr size_t attn_smem_bytes() { return 1024 + kOffCtl + sizeof(AttnCtl) + 64; }

// Phase timers of the profiling build (-DSWV_PROFILE, `build.py --profile`, a library of its own):
// lane 0 of every role adds the cycles it spent per phase to a table in device memory that
// swv_debug_attn_profile() reads.  In the regular build every member is an empty inline function.
#ifdef SWV_PROFILE
__device__ unsigned long long g_attn_prof[64];
struct Prof {
  long long last;
  unsigned long long acc[8];
  __device__ __forceinline__ void start() {
    last = clock64();
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0;
  }
  __device__ __forceinline__ void tick(int k) {
    const long long t = clock64();
    acc[k] += static_cast<unsigned long long>(t - last);
    last = t;
  }
  __device__ __forceinline__ void flush(int base, bool on) {
    if (!on) return;
#pragma unroll
    for (int i = 0; i < 8; ++i) atomicAdd(&g_attn_prof[base + i], acc[i]);
  }
};
#else
struct Prof {
  __device__ __forceinline__ void start() {}
  __device__ __forceinline__ void tick(int) {}
  __device__ __forceinline__ void flush(int, bool) {}
};
#endif

// ------------------------------------------------------------ softmax helpers
// Membership and weight on the FMA pipe (compare and select run at half rate on the ALU pipe, which
// would bound the weight conversion).  With t = the float just below thr, r >= thr <=> r - t > 0, and
// the smallest positive r - t (one ulp of a threshold >= 4e-6) times 2^60 is far above 1:
//   step = saturate(r * 2^60 - t * 2^60)  is exactly 0 or 1;   weight = r * step.
// `neg_c` = -t * 2^60 (-inf for rows that select nothing).
// (s0, s1) * sc + neg_b as one packed fp32x2 instruction
__device__ __forceinline__ void scale_shift2(float s0, float s1, float sc, float neg_b, float& x0, float& x1) {
  asm("{\n\t.reg .b64 a, b, c, d;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %4};\n\tmov.b64 c, {%5, %5};\n\t"
      "fma.rn.f32x2 d, a, b, c;\n\tmov.b64 {%0, %1}, d;\n\t}"
      : "=f"(x0), "=f"(x1)
      : "f"(s0), "f"(s1), "f"(sc), "f"(neg_b));
}
// (a0 * b0, a1 * b1) as one packed fp32x2 instruction
__device__ __forceinline__ void mul2(float a0, float a1, float b0, float b1, float& x0, float& x1) {
  asm("{\n\t.reg .b64 a, b, d;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %5};\n\t"
      "mul.rn.f32x2 d, a, b;\n\tmov.b64 {%0, %1}, d;\n\t}"
      : "=f"(x0), "=f"(x1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

struct SoftmaxRow {
  float m_true, m_used, l;
  float thr_ge;            // one-pass path: a key is selected iff its raw score >= thr_ge
  float bound;             // one-pass path: log2-domain upper bound of every logit of the row
  float sc;
  uint32_t lane_base, s_col, o_col;
  const uint4* mask_tile;
  int members;             // two-pass path: bits set in the row's mask words so far
};

// One-pass per-tile loop, column-split: the warp owns 32 query rows x 64 key columns
// (`slice` = which 64) of every tile, for BOTH heads of the CTA.  Every logit of a row is bounded
// by the row's `bound` (Cauchy-Schwarz on q and the largest key norm of the head), so
// 2^(s*sc - bound) never overflows and the accumulator never needs rescaling.  Membership:
// recomputed score >= row threshold.  The routing weights (score >= thr ? score : 0) of a tile's 64
// columns are packed to bf16 pairs in registers ONCE for both heads and R is released; per head,
// p = 2^(s*c - bound) * weight goes to TMEM as bf16.  With eight warps on one head's tile at a
// time, a head's S -> P -> PV -> next S chain is short enough to hide behind the other head's pass.
//
// Measured with the phase timers of the profiling build (65536 tokens, cycles per tile and
// scheduler): a plain pass takes 1080-1220 cycles against the exp unit's 1024 (two warps share a
// scheduler's 4 exp lanes: 2 x 64 instructions x 8 cycles), whether 2 or 4 warps share the
// scheduler; a weight conversion on its own costs another 400 cycles during which the exp unit
// idles.  With the conversion of the NEXT tile's weights inside head 1's pass (FUSE) that pass
// takes 1430-1490 cycles: about 17 dispatch cycles per column pair (half-rate ALU / conversion
// instructions count twice) beside 16 exp cycles, i.e. the scheduler's dispatch port and the exp
// unit are both close to saturated and the tile period (3230 cycles, of which ~350 are waits for
// the tensor pipe) sits ~1.5x above either floor.  Splitting the conversion evenly over the two
// passes (head 0's pass converting half of its own tile just in time) measured 7 % slower: the
// routing-weight tile, issued when the previous one is released, then has only half a pass to
// complete behind the other head's PV and QK in the in-order tensor pipe.

// 16 raw scores -> 8 packed bf16 weight pairs; COUNT also adds the number of selected ones to `cnt`
template <bool COUNT>
__device__ __forceinline__ void convert_chunk(const uint32_t (&r)[16], float neg_c, uint32_t* w8, float& cnt) {
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const float r0 = __uint_as_float(r[i]), r1 = __uint_as_float(r[i + 1]);
    float st0, st1, w0, w1;
    asm("fma.rn.sat.f32 %0, %1, 0f5D800000, %2;" : "=f"(st0) : "f"(r0), "f"(neg_c));   // 0x5D800000 = 2^60
    asm("fma.rn.sat.f32 %0, %1, 0f5D800000, %2;" : "=f"(st1) : "f"(r1), "f"(neg_c));
    mul2(r0, r1, st0, st1, w0, w1);
    if (COUNT) cnt += st0 + st1;
    w8[i >> 1] = pack_bf16x2(w0, w1);
  }
}

// Routing weights of tile j for the warp's 64 columns on their own (the first tile, and CTAs with
// one head); R is released as soon as it has been read.
template <bool COUNT>
__device__ __forceinline__ bool convert_weights(AttnCtl* ctl, uint32_t r_col, int j, int lane, float neg_c,
                                                uint32_t (&w)[kSliceCols / 2], float& cnt, int* status,
                                                volatile uint32_t* abort_flag, Prof& prof) {
  prof.tick(7);
  if (!mbar_wait_bounded(&ctl->r_full, j & 1, abort_flag)) {
    record_status(status, kDevWaitAccFull);
    return false;
  }
  prof.tick(0);
  tc_fence_after();
  uint32_t ra[16], rb[16];
  tmem_ld16(r_col, ra);
#pragma unroll
  for (int u = 0; u < kSliceCols / 16; ++u) {
    tc_wait_ld();
    if (u + 1 < kSliceCols / 16) {
      if (u & 1) tmem_ld16(r_col + (u + 1) * 16, ra);
      else tmem_ld16(r_col + (u + 1) * 16, rb);
    }
    if (u & 1) convert_chunk<COUNT>(rb, neg_c, &w[u * 8], cnt);
    else convert_chunk<COUNT>(ra, neg_c, &w[u * 8], cnt);
  }
  tc_fence_before();
  __syncwarp();
  if (lane == 0) mbar_arrive(&ctl->r_free);
  prof.tick(1);
  return true;
}

// One head's pass over the warp's 64 columns of tile j: p = 2^(s*c - bound) * weight -> TMEM as bf16
// pairs over the first 32 of those columns, always behind this thread's own reads.  FUSE (the
// tile's last pass): the weights of tile j + 1 are converted from R(j + 1) in the same loop and
// replace those of tile j in `wpk`, 16 columns at a time, as soon as this pass has used them.
template <bool FUSE, bool COUNT>
__device__ __forceinline__ bool softmax_pass(AttnCtl* ctl, uint32_t s_col, uint32_t r_col, int x, int j, int lane,
                                             float sc, float neg_b, float neg_c, uint32_t (&wpk)[kSliceCols / 2],
                                             float& cnt, float& l0, float& l1, int* status,
                                             volatile uint32_t* abort_flag, Prof& prof) {
  prof.tick(7);
  if (!mbar_wait_bounded(&ctl->s_full[x], j & 1, abort_flag)) {
    record_status(status, kDevWaitAccFull);
    return false;
  }
  prof.tick(2 + 2 * x);
  if (FUSE) {
    if (!mbar_wait_bounded(&ctl->r_full, (j + 1) & 1, abort_flag)) {
      record_status(status, kDevWaitAccFull);
      return false;
    }
    prof.tick(0);
  }
  tc_fence_after();
  // One 16-column chunk of S per step.  Plain pass: the next chunk is requested before the
  // current one is used (two register buffers).  Fused pass: one buffer -- the next S chunk is
  // requested as soon as the current one has been consumed and arrives while the R chunk is
  // converted, which keeps the pass within the register budget.
  uint32_t sa[16], sb[FUSE ? 1 : 16], ra[FUSE ? 16 : 1];
  tmem_ld16(s_col, sa);
  if constexpr (FUSE) tmem_ld16(r_col, ra);
#pragma unroll
  for (int u = 0; u < kSliceCols / 16; ++u) {
    tc_wait_ld();
    if constexpr (!FUSE) {
      if (u + 1 < kSliceCols / 16) {
        if (u & 1) tmem_ld16(s_col + (u + 1) * 16, sa);
        else tmem_ld16(s_col + (u + 1) * 16, sb);
      }
    }
    uint32_t packed[8];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const bool odd = !FUSE && (u & 1);
      const float s0 = __uint_as_float(odd ? sb[FUSE ? 0 : i] : sa[i]);
      const float s1 = __uint_as_float(odd ? sb[FUSE ? 0 : i + 1] : sa[i + 1]);
      // both exponentials rounded to bf16, times the packed weights; the row sum adds exactly
      // the bf16 products the tensor core will see
      float x0, x1;
      scale_shift2(s0, s1, sc, neg_b, x0, x1);
      const uint32_t pp = mul_bf16x2(pack_bf16x2(ex2_approx(x0), ex2_approx(x1)), wpk[u * 8 + (i >> 1)]);
      add_bf16x2_to_f32(l0, l1, pp);
      packed[i >> 1] = pp;
      if constexpr (FUSE) {
        // The next tile's weight pair takes the register of the pair just used (written pair by
        // pair between the exponentials: a warp issues in order).
        const float r0 = __uint_as_float(ra[i]), r1 = __uint_as_float(ra[i + 1]);
        float st0, st1, w0, w1;
        asm("fma.rn.sat.f32 %0, %1, 0f5D800000, %2;" : "=f"(st0) : "f"(r0), "f"(neg_c));
        asm("fma.rn.sat.f32 %0, %1, 0f5D800000, %2;" : "=f"(st1) : "f"(r1), "f"(neg_c));
        mul2(r0, r1, st0, st1, w0, w1);
        if (COUNT) cnt += st0 + st1;
        wpk[u * 8 + (i >> 1)] = pack_bf16x2(w0, w1);
      }
    }
    if constexpr (FUSE) {
      if (u + 1 < kSliceCols / 16) {
        tmem_ld16(s_col + (u + 1) * 16, sa);
        tmem_ld16(r_col + (u + 1) * 16, ra);
      }
    }
    tmem_st8(s_col + u * 8, packed);
  }
  tc_wait_st();
  tc_fence_before();
  __syncwarp();
  if (lane == 0) {
    mbar_arrive(&ctl->p_full[x]);
    if (FUSE) mbar_arrive(&ctl->r_free);
  }
  prof.tick(3 + 2 * x);
  return true;
}

// Rows whose ties at the threshold are cut by key index (a few per 10^4 rows on continuous data: two
// keys with bit-identical scores around the K-th place) carry a list of the tied keys that are NOT
// selected.  `score >= threshold` admits them; when the sweep reaches the tile of such a key, the
// thread that owns its column clears that weight.  `tile_of(e)` = key tile relative to the CTA's
// first one.  Returns the next tile (> j) in which this thread has to do so again, or INT_MAX.
template <bool COUNT>
__device__ __forceinline__ int drop_excluded(uint32_t (&w)[kSliceCols / 2], float& cnt, const int32_t* list, int n,
                                             int kt0, int slice, int j) {
  int nxt = 0x7fffffff;
  for (int i = 0; i < n; ++i) {
    const int e = __ldg(list + i);
    if (((e & (kTile - 1)) / kSliceCols) != slice) continue;
    const int t = e / kTile - kt0;
    if (t == j) {
      const int pos = e & (kSliceCols - 1);
      const uint32_t keep = (pos & 1) ? 0x0000ffffu : 0xffff0000u;
      // (opaque to the compiler on purpose: written as plain C++ the unrolled compare-and-clear is
      // folded back into a dynamically indexed store, which moves the weights to local memory)
#pragma unroll
      for (int r = 0; r < kSliceCols / 2; ++r)
        asm("{\n\t.reg .pred p;\n\tsetp.eq.s32 p, %1, %2;\n\t@p and.b32 %0, %0, %3;\n\t}"
            : "+r"(w[r])
            : "r"(pos >> 1), "r"(r), "r"(keep));
      if (COUNT) cnt -= 1.f;
    } else if (t > j && t < nxt) {
      nxt = t;
    }
  }
  return nxt;
}

template <bool COUNT>
__device__ __forceinline__ bool softmax_tiles_split(AttnCtl* ctl, uint32_t lane_base, int slice, int nh, int nKT,
                                                    int lane, float thr, float sc, const float (&bound)[2],
                                                    float (&l_out)[2], float& cnt, const AttnParams& p, bool warp_cut,
                                                    int grow0, int kt0, int* status, volatile uint32_t* abort_flag) {
  Prof prof;
  prof.start();
  const uint32_t r_col = lane_base + kColR + slice * kSliceCols;
  const uint32_t s_col0 = lane_base + kColS + slice * kSliceCols;   // this slice's score columns of head 0
  // -(float just below the threshold) * 2^60; a +inf threshold (tail rows) gives -inf: nothing selected
  const float neg_c = -__uint_as_float(__float_as_uint(thr) - 1u) * 0x1p60f;
  float l[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  uint32_t w[kSliceCols / 2];
  cnt = 0.f;
  if (!convert_weights<COUNT>(ctl, r_col, 0, lane, neg_c, w, cnt, status, abort_flag, prof)) return false;
  int* next_ex = &ctl->next_ex[threadIdx.x - 64];   // written by this thread before the loop: -1 = look the list up
  for (int j = 0; j < nKT; ++j) {
    const bool more = j + 1 < nKT;
    if (warp_cut && *next_ex <= j) {                  // warp_cut: some row of this warp has cut ties (rare)
      const int64_t grow = grow0 + (threadIdx.x & 127);
      const int n_ex = static_cast<int>(p.st_neq[grow] - p.st_kth[grow]);
      *next_ex = drop_excluded<COUNT>(w, cnt, p.st_excl + grow * kMaxExcl, n_ex, kt0, slice, j);
    }
    if (!softmax_pass<false, COUNT>(ctl, s_col0, r_col, 0, j, lane, sc, -bound[0], neg_c, w, cnt, l[0][0], l[0][1],
                                    status, abort_flag, prof))
      return false;
    bool ok;
    if (nh == 2) {
      ok = more ? softmax_pass<true, COUNT>(ctl, s_col0 + kTile, r_col, 1, j, lane, sc, -bound[1], neg_c, w, cnt,
                                            l[1][0], l[1][1], status, abort_flag, prof)
                : softmax_pass<false, COUNT>(ctl, s_col0 + kTile, r_col, 1, j, lane, sc, -bound[1], neg_c, w, cnt,
                                             l[1][0], l[1][1], status, abort_flag, prof);
    } else {
      ok = !more || convert_weights<COUNT>(ctl, r_col, j + 1, lane, neg_c, w, cnt, status, abort_flag, prof);
    }
    if (!ok) return false;
  }
  l_out[0] = l[0][0] + l[0][1];
  l_out[1] = l[1][0] + l[1][1];
  prof.flush(slice & 1 ? 8 : 0, lane == 0);
  return true;
}

// One warp per (head, 32 rows), all 128 columns.  The barriers count one arrival per softmax warp
// of the column-split layout: a warp arrives `r_arrivals` times on r_free and kSlices times on p_full.
__device__ __forceinline__ bool softmax_tiles_exact(SoftmaxRow& st, AttnCtl* ctl, int x, int nKT, int lane,
                                                    int r_arrivals, int* status, volatile uint32_t* abort_flag) {
  const float ninf = -__int_as_float(0x7f800000);
  const float sc = st.sc;
  const uint32_t s_col = st.s_col;
  const uint32_t r_col = st.lane_base + kColR;
  uint4 mw = __ldg(st.mask_tile);

  for (int j = 0; j < nKT; ++j) {
    uint4 mw_next = make_uint4(0, 0, 0, 0);
    if (j + 1 < nKT) mw_next = __ldg(st.mask_tile + static_cast<int64_t>(j + 1) * kTile);
    const uint32_t words[4] = {mw.x, mw.y, mw.z, mw.w};

    if (!mbar_wait_bounded(&ctl->s_full[x], j & 1, abort_flag) ||
        !mbar_wait_bounded(&ctl->r_full, j & 1, abort_flag)) {
      record_status(status, kDevWaitAccFull);
      return false;
    }
    tc_fence_after();

    // pass 1: maximum over the selected logits of this tile
    float mt0 = ninf, mt1 = ninf;
#pragma unroll 1
    for (int u = 0; u < 8; ++u) {
      uint32_t s[16];
      tmem_ld16(s_col + u * 16, s);
      tc_wait_ld();
      const uint32_t w = words[u >> 1] >> ((u & 1) * 16);
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        mt0 = fmaxf(mt0, (w & (1u << i)) ? __uint_as_float(s[i]) : ninf);
        mt1 = fmaxf(mt1, (w & (2u << i)) ? __uint_as_float(s[i + 1]) : ninf);
      }
    }
    st.m_true = fmaxf(st.m_true, fmaxf(mt0, mt1) * sc);
    if (__any_sync(0xffffffffu, st.m_true > st.m_used + kRescaleStep)) {
      const float factor = (st.m_true == st.m_used) ? 1.f : ex2_approx(st.m_used - st.m_true);
      st.m_used = st.m_true;
      st.l *= factor;
      if (j > 0) {
        // O of the tiles before this one is complete once PV(j-1) retired
        if (!mbar_wait_bounded(&ctl->pv_done[x], (j - 1) & 1, abort_flag)) {
          record_status(status, kDevWaitPvDone);
          return false;
        }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[16];
          tmem_ld16(st.o_col + c * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
          tmem_st16(st.o_col + c * 16, o);
        }
        tc_wait_st();
      }
    }
    const float neg_m = -st.m_used;

    // pass 2: routing-weighted probabilities of the selected keys -> TMEM (bf16)
    float l0 = 0.f, l1 = 0.f;
#pragma unroll 1
    for (int u = 0; u < 8; ++u) {
      uint32_t s[16], r[16];
      tmem_ld16(s_col + u * 16, s);
      tmem_ld16(r_col + u * 16, r);
      tc_wait_ld();
      const uint32_t w = words[u >> 1] >> ((u & 1) * 16);
      uint32_t packed[8];
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        float p0 = ex2_approx(fmaf(__uint_as_float(s[i]), sc, neg_m)) * fmaxf(__uint_as_float(r[i]), 0.f);
        float p1 = ex2_approx(fmaf(__uint_as_float(s[i + 1]), sc, neg_m)) * fmaxf(__uint_as_float(r[i + 1]), 0.f);
        p0 = (w & (1u << i)) ? p0 : 0.f;
        p1 = (w & (2u << i)) ? p1 : 0.f;
        l0 += p0;
        l1 += p1;
        packed[i >> 1] = pack_bf16x2(p0, p1);
      }
      tmem_st8(s_col + p_col_of_key(u * 16), packed);
    }
    st.l += l0 + l1;
    tc_fence_before();
    __syncwarp();
    if (lane < r_arrivals) mbar_arrive(&ctl->r_free);
    tc_wait_st();
    tc_fence_before();
    __syncwarp();
    if (lane < kSlices) mbar_arrive(&ctl->p_full[x]);
    st.members += __popc(mw.x) + __popc(mw.y) + __popc(mw.z) + __popc(mw.w);
    mw = mw_next;
  }
  return true;
}

// max over keys of |K[b,h,k,:]|^2, as float bits (non-negative floats order like unsigned ints)
__global__ void key_norm_max_kernel(const __nv_bfloat16* __restrict__ k, int64_t sb, int64_t sh, int64_t st_,
                                    int B, int H, int Tk, uint32_t* __restrict__ out) {
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(B) * H * Tk;
  float n2 = 0.f;
  int bh = 0;
  if (gid < total) {
    const int t = static_cast<int>(gid % Tk);
    bh = static_cast<int>(gid / Tk);
    const int h = bh % H, b = bh / H;
    const uint4* row = reinterpret_cast<const uint4*>(k + b * sb + h * sh + t * st_);
#pragma unroll
    for (int i = 0; i < kHeadDim / 8; ++i) {
      const uint4 v = __ldg(row + i);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float lo = __uint_as_float(w[q] << 16), hi = __uint_as_float(w[q] & 0xffff0000u);
        n2 = fmaf(lo, lo, fmaf(hi, hi, n2));
      }
    }
  }
  // keys of one (b,h) are contiguous in gid: reduce inside the warp when it does not straddle
  const int bh0 = __shfl_sync(0xffffffffu, bh, 0);
  if (__all_sync(0xffffffffu, bh == bh0)) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) n2 = fmaxf(n2, __shfl_xor_sync(0xffffffffu, n2, off));
    if ((threadIdx.x & 31) == 0 && gid < total) atomicMax(out + bh, __float_as_uint(n2));
  } else if (gid < total) {
    atomicMax(out + bh, __float_as_uint(n2));
  }
}

template <bool kSplit,      // the key range of a (query tile, head pair) is shared by p.split CTAs
          bool kCount = false>   // diagnostic: also write how many keys every row treated as selected
__global__ void __launch_bounds__(kAttnThreads, 1)
    dsa_attn_masked_kernel(const __grid_constant__ CUtensorMap tm_wq, const __grid_constant__ CUtensorMap tm_wk,
                           const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                           const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  constexpr uint32_t kIdescR = make_idesc(/*tf32*/ 2, kTile, kTile, 0, 0);
  constexpr uint32_t kIdescQK = make_idesc(/*bf16*/ 1, kTile, kTile, 0, 0);
  constexpr uint32_t kIdescPV = make_idesc(/*bf16*/ 1, kTile, kHeadDim, 0, /*V is MN-major*/ 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  AttnCtl* ctl = reinterpret_cast<AttnCtl*>(smem + kOffCtl);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta = kSplit ? blockIdx.x / p.split : blockIdx.x;     // (batch, query tile, head pair)
  const int part = kSplit ? blockIdx.x - cta * p.split : 0;       // which share of the key tiles
  if (p.only_flagged != nullptr && p.only_flagged[cta] == 0u) return;
  const int hp = cta % p.nHP;
  const int qt = (cta / p.nHP) % p.nQT;
  const int b = cta / (p.nHP * p.nQT);
  const int kt0 = kSplit ? static_cast<int>(static_cast<int64_t>(part) * p.nKT / p.split) : 0;   // first key tile
  const int nKT = kSplit ? static_cast<int>(static_cast<int64_t>(part + 1) * p.nKT / p.split) - kt0 : p.nKT;
  const int h0 = hp * 2;
  const int nh = (h0 + 1 < p.H) ? 2 : 1;   // heads handled by this CTA

  if (threadIdx.x == 0) {
    mbar_init(&ctl->q_full, 1);
    mbar_init(&ctl->r_full, 1);
    mbar_init(&ctl->r_free, kSoftWarps);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl->wk_full[s], 1);
      mbar_init(&ctl->wk_empty[s], 1);
      mbar_init(&ctl->v_full[s], 1);
      mbar_init(&ctl->v_empty[s], 1);
      mbar_init(&ctl->s_full[s], 1);
      mbar_init(&ctl->p_full[s], kSoftWarps);
      mbar_init(&ctl->pv_done[s], 1);
      for (int t = 0; t < 2; ++t) {
        mbar_init(&ctl->k_full[s][t], 1);
        mbar_init(&ctl->k_empty[s][t], 1);
      }
    }
    ctl->abort_flag = 0;
    ctl->cta_exact = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, kAttnTmemCols);
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
      tma_prefetch_desc(&tm_wq);
      tma_prefetch_desc(&tm_wk);
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_expect_tx(&ctl->q_full, kWTileBytes + nh * kQTileBytes);
      tma_load_3d(smem + kOffWq, &tm_wq, &ctl->q_full, 0, qt * kTile, b);
      tma_load_3d(smem + kOffWq + kWTileBytes / 2, &tm_wq, &ctl->q_full, 32, qt * kTile, b);
      for (int x = 0; x < nh; ++x)
        tma_load_4d(smem + kOffQ + x * kQTileBytes, &tm_q, &ctl->q_full, 0, qt * kTile, h0 + x, b);

      // The slots are freed in a fixed order in time -- within tile i: K_x(i) (its QK retired), the
      // indexer keys, then V_0(i), V_1(i) (their PV retired) -- so one thread refills them in that
      // order with suspending waits instead of polling five barriers in a busy loop, which costs
      // the scheduler it shares with two softmax warps a quarter of its issue slots.
      bool ok = true;
      auto load_wk = [&](int j) {
        if (!ok) return;
        if (!mbar_wait_bounded(&ctl->wk_empty[j & 1], ((j >> 1) & 1) ^ 1, abort_flag)) { ok = false; return; }
        uint8_t* dst = smem + kOffWk + (j & 1) * kWTileBytes;
        mbar_expect_tx(&ctl->wk_full[j & 1], kWTileBytes);
        tma_load_3d(dst, &tm_wk, &ctl->wk_full[j & 1], 0, (kt0 + j) * kTile, b);
        tma_load_3d(dst + kWTileBytes / 2, &tm_wk, &ctl->wk_full[j & 1], 32, (kt0 + j) * kTile, b);
      };
      auto load_k = [&](int x, int j) {
        if (!ok || x >= nh) return;
        if (!mbar_wait_bounded(&ctl->k_empty[x][j & 1], ((j >> 1) & 1) ^ 1, abort_flag)) { ok = false; return; }
        mbar_expect_tx(&ctl->k_full[x][j & 1], kQTileBytes);
        tma_load_4d(smem + kOffK + (x * 2 + (j & 1)) * kQTileBytes, &tm_k, &ctl->k_full[x][j & 1], 0, (kt0 + j) * kTile,
                    h0 + x, b);
      };
      auto load_v = [&](int x, int j) {
        if (!ok || x >= nh) return;
        if (!mbar_wait_bounded(&ctl->v_empty[x], (j & 1) ^ 1, abort_flag)) { ok = false; return; }
        mbar_expect_tx(&ctl->v_full[x], kQTileBytes);
        tma_load_4d(smem + kOffV + x * kQTileBytes, &tm_v, &ctl->v_full[x], 0, (kt0 + j) * kTile, h0 + x, b);
      };
      for (int j = 0; j < 2 && j < nKT; ++j) {
        load_wk(j);
        load_k(0, j);
        load_k(1, j);
      }
      load_v(0, 0);
      load_v(1, 0);
      for (int i = 0; i < nKT && ok; ++i) {
        if (i + 2 < nKT) {
          load_k(0, i + 2);
          load_k(1, i + 2);
          load_wk(i + 2);
        }
        if (i + 1 < nKT) {
          load_v(0, i + 1);
          load_v(1, i + 1);
        }
      }
      if (!ok) record_status(p.status, kDevWaitStageEmpty);
    }
  } else if (warp == 1) {
    // ------------------------------------------- MMA issuer of the routing-weight tiles R(j)
    // (Three issuing threads, one per independent MMA stream: a single thread spends most of a
    // tile period inside the issue sequences and makes the streams wait for each other.)
    if (lane == 0) {
      const uint32_t wq_addr = smem_u32(smem + kOffWq);
      const uint32_t wk_addr = smem_u32(smem + kOffWk);
      bool ok = mbar_wait_bounded(&ctl->q_full, 0, abort_flag);
      if (!ok) record_status(p.status, kDevWaitQ);
      Prof prof;
      prof.start();
      for (int j = 0; ok && j < nKT; ++j) {
        const int s = j & 1;
        // needs the indexer key tile and every softmax warp done with R(j-1)
        bool got = mbar_wait_bounded(&ctl->wk_full[s], (j >> 1) & 1, abort_flag);
        prof.tick(0);
        got = got && (j == 0 || mbar_wait_bounded(&ctl->r_free, (j - 1) & 1, abort_flag));
        prof.tick(1);
        if (!got) {
          record_status(p.status, kDevWaitTmaFull);
          break;
        }
        tc_fence_after();
        // descriptors advance in 16-byte units: +2 per 32-byte K step, +1024 for the second K half
        const uint64_t da = smem_desc_sw128(wq_addr), db = smem_desc_sw128(wk_addr + s * kWTileBytes);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t off = (ks >> 2) * (kWTileBytes / 32) + (ks & 3) * 2;
          umma_tf32_ss(tmem_base + kColR, da + off, db + off, kIdescR, ks > 0);
        }
        umma_commit(&ctl->wk_empty[s]);
        umma_commit(&ctl->r_full);
        prof.tick(2);
      }
      prof.flush(16, true);
    }
  } else if (warp >= 2 + kSoftWarps) {
    // ------------------------------------- MMA issuer of one head: S_x(j) and O_x += P_x(j) V_x(j)
    const int x = warp - (2 + kSoftWarps);
    if (lane == 0 && x < nh) {
      const uint32_t q_addr = smem_u32(smem + kOffQ + x * kQTileBytes);
      const uint32_t k_addr = smem_u32(smem + kOffK + x * 2 * kQTileBytes);
      const uint32_t v_addr = smem_u32(smem + kOffV + x * kQTileBytes);
      const uint32_t s_col = tmem_base + kColS + x * kTile;
      const uint32_t o_col = tmem_base + kColO + x * kHeadDim;
      const uint64_t dq = smem_desc_sw128(q_addr), dv = smem_desc_sw128(v_addr);
      bool ok = mbar_wait_bounded(&ctl->q_full, 0, abort_flag);
      if (!ok) record_status(p.status, kDevWaitQ);
      Prof prof;
      prof.start();
      // S_x(j) overwrites P_x(j-1), so it is issued behind PV_x(j-1): the tensor pipe executes
      // one thread's MMAs in issue order.
      for (int j = 0; ok && j <= nKT; ++j) {
        if (j > 0) {
          // PV_x(j-1): needs P_x(j-1) in TMEM and V_x(j-1) in smem
          const int jp = j - 1;
          bool got = mbar_wait_bounded(&ctl->p_full[x], jp & 1, abort_flag);
          prof.tick(0);
          got = got && mbar_wait_bounded(&ctl->v_full[x], jp & 1, abort_flag);
          prof.tick(1);
          if (!got) {
            record_status(p.status, kDevWaitPReady);
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)   // 16 keys per step: 8 packed P columns, 2 KiB of V rows
            umma_f16_ts(o_col, s_col + p_col_of_key(ks * 16), dv + ks * 128, kIdescPV, (jp > 0 || ks > 0));
          umma_commit(&ctl->v_empty[x]);
          umma_commit(&ctl->pv_done[x]);
          prof.tick(2);
        }
        if (j < nKT) {
          const int s = j & 1;
          const bool got = mbar_wait_bounded(&ctl->k_full[x][s], (j >> 1) & 1, abort_flag);
          prof.tick(3);
          if (!got) {
            record_status(p.status, kDevWaitTmaFull);
            break;
          }
          tc_fence_after();
          const uint64_t dk = smem_desc_sw128(k_addr + s * kQTileBytes);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) umma_f16_ss(s_col, dq + ks * 2, dk + ks * 2, kIdescQK, ks > 0);
          umma_commit(&ctl->k_empty[x][s]);
          umma_commit(&ctl->s_full[x]);
          prof.tick(4);
        }
      }
      prof.flush(24 + 8 * x, true);
#ifdef SWV_PROFILE
      if (x == 0) atomicAdd(&g_attn_prof[63], static_cast<unsigned long long>(nKT));
#endif
    }
  } else {
    // ----------------------------------------------------------------- softmax
    const int slice = (warp - 2) >> 2;          // one-pass layout: column slice; two-pass layout: slices 0, 1 = head
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int qrow = qt * kTile + row;
    const bool row_ok = qrow < p.Tq;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);

    // Row constants from the indexer's select passes: threshold bits, how many keys equal
    // to the threshold are selected, how many exist.  The one-pass path is exact when
    //   - the threshold is positive and at most kMaxExcl ties at it are left out (membership =
    //     score >= thr, minus the row's listed keys),
    //   - every weight exceeds the 1e-6 clamp on the denominator (the clamp cannot bind),
    //   - the logits of the row are provably small (|s*sc| <= bound <= kMaxBound), both heads.
    // One row that fails sends the whole CTA to the two-pass bitmask path.
    bool flagged = false;
    bool cut_row = false;                        // some of this row's ties at the threshold are cut
    float thr_ge = __int_as_float(0x7f800000);   // tail rows: nothing selected
    float bound[2] = {0.f, 0.f};
    if (row_ok) {
      const int64_t grow = static_cast<int64_t>(b) * p.Tq + qrow;
      const uint32_t thr_bits = p.st_prefix[grow];
      thr_ge = __uint_as_float(thr_bits);
      bool small = true;
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        if (x >= nh) continue;
        const uint4* qv = reinterpret_cast<const uint4*>(p.q + b * p.qsb + (h0 + x) * p.qsh + qrow * p.qst);
        float q2 = 0.f;
#pragma unroll
        for (int i = 0; i < kHeadDim / 8; ++i) {
          const uint4 v = __ldg(qv + i);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float lo = __uint_as_float(w[q] << 16), hi = __uint_as_float(w[q] & 0xffff0000u);
            q2 = fmaf(lo, lo, fmaf(hi, hi, q2));
          }
        }
        const float k2 = __uint_as_float(p.kmax2[b * p.H + h0 + x]);
        bound[x] = sqrtf(q2 * k2) * p.scale_log2 * 1.001f + 1e-3f;
        small = small && bound[x] <= kMaxBound;
      }
      const uint32_t n_cut = p.st_neq[grow] - p.st_kth[grow];     // ties at the threshold that are not selected
      flagged = !(thr_bits != 0u && n_cut <= static_cast<uint32_t>(kMaxExcl) && thr_ge >= 4e-6f && small);
      cut_row = n_cut != 0u;
    }
    if (__any_sync(0xffffffffu, flagged) && lane == 0) atomicOr(&ctl->cta_exact, 1u);
    asm volatile("bar.sync 2, %0;" ::"r"(32 * kSoftWarps) : "memory");
    const bool exact = *reinterpret_cast<volatile uint32_t*>(&ctl->cta_exact) != 0u;
#ifdef SWV_PROFILE
    if (exact && warp == 2 && lane == 0) atomicAdd(&g_attn_prof[62], 1ull);
#endif

    // Output duty.  One-pass layout: slice s writes head s % 2, channels [d0, d0 + nd) with the 64
    // channels of a head divided among the slices that share it; two-pass layout: slices 0 and 1
    // write all channels of their head, the other slices idle.
    constexpr int kParts = kSlices / 2;
    const int x = slice & 1;                      // head whose output rows this thread writes
    const int h = h0 + x;
    const int d0 = exact ? 0 : (slice >> 1) * (kHeadDim / kParts);
    const int nd = exact ? (slice < 2 ? kHeadDim : 0) : kHeadDim / kParts;
    const uint32_t o_col = lane_base + kColO + x * kHeadDim + d0;
    bool ok = true;
    float inv = 0.f;
    float row_l = 0.f, row_mu = 0.f, row_mt = 0.f;   // row statistics of this CTA's key range (for the split merge)
    if (!exact) {
      float l_part[2], cnt = 0.f;
      ctl->next_ex[threadIdx.x - 64] = cut_row ? -1 : 0x7fffffff;
      ok = softmax_tiles_split<kCount>(ctl, lane_base, slice, nh, nKT, lane, thr_ge, p.scale_log2, bound, l_part, cnt,
                                       p, __any_sync(0xffffffffu, cut_row), b * p.Tq + qt * kTile, kt0, p.status,
                                       abort_flag);
      if (kCount && hp == 0 && row_ok) atomicAdd(p.member_count + static_cast<int64_t>(b) * p.Tq + qrow, static_cast<int>(cnt));
      // The column slices of a row add their partial sums through the indexer-query tile:
      // every routing-weight MMA that read it has retired once any warp has left its loop.
      float* lsum = reinterpret_cast<float*>(smem + kOffWq);      // [2 heads][128 rows][kSlices]
      lsum[(0 * kTile + row) * kSlices + slice] = l_part[0];
      lsum[(1 * kTile + row) * kSlices + slice] = l_part[1];
      asm volatile("bar.sync 2, %0;" ::"r"(32 * kSoftWarps) : "memory");
      float lt = 0.f;
#pragma unroll
      for (int i = 0; i < kSlices; ++i) lt += lsum[(x * kTile + row) * kSlices + i];
      inv = 1.f / lt;                             // the clamp cannot bind
      row_l = lt;
    } else if (slice < 2 && x < nh) {
      SoftmaxRow st;
      st.lane_base = lane_base;
      st.s_col = lane_base + kColS + x * kTile;
      st.o_col = lane_base + kColO + x * kHeadDim;
      st.mask_tile =
          reinterpret_cast<const uint4*>(p.maskbits) +
          ((static_cast<int64_t>(b) * p.nQT + qt) * p.nKT + kt0) * kTile + row;
      st.sc = p.scale_log2;
      st.m_true = st.m_used = -__int_as_float(0x7f800000);
      st.l = 0.f;
      st.members = 0;
      ok = softmax_tiles_exact(st, ctl, x, nKT, lane, kSoftWarps / (4 * nh), p.status, abort_flag);
      if (kCount && hp == 0 && x == 0 && row_ok) atomicAdd(p.member_count + static_cast<int64_t>(b) * p.Tq + qrow, st.members);
      // the reference's clamp: out = O c / max(l c, 1e-6), c = 2^(m_used - m_true)
      const float corr = (st.m_used == st.m_true) ? 1.f : ex2_approx(st.m_used - st.m_true);
      inv = corr / fmaxf(st.l * corr, 1e-6f);
      row_l = st.l;
      row_mu = st.m_used;
      row_mt = st.m_true;
    }
    const bool duty = x < nh && nd > 0;
    if (duty && ok && !mbar_wait_bounded(&ctl->pv_done[x], (nKT - 1) & 1, abort_flag)) {
      record_status(p.status, kDevWaitPvDone);
      ok = false;
    }
    if (duty && ok) tc_fence_after();

    // writes 16 channels [d0 + c*16, +16) of the output row, scaled
    auto store_chunk = [&](int c, const float (&acc)[16], float scale) {
      if (p.o_dtype == SWV_F32) {
        float* orow = static_cast<float*>(p.o) + b * p.osb + h * p.osh + qrow * p.ost + d0 + c * 16;
#pragma unroll
        for (int i = 0; i < 16; i += 4)
          *reinterpret_cast<float4*>(orow + i) =
              make_float4(acc[i] * scale, acc[i + 1] * scale, acc[i + 2] * scale, acc[i + 3] * scale);
      } else {
        uint16_t* orow = static_cast<uint16_t*>(p.o) + b * p.osb + h * p.osh + qrow * p.ost + d0 + c * 16;
#pragma unroll
        for (int i = 0; i < 16; i += 8) {
          uint32_t w4[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float a0 = acc[i + 2 * q] * scale, a1 = acc[i + 2 * q + 1] * scale;
            if (p.o_dtype == SWV_BF16) {
              w4[q] = pack_bf16x2(a0, a1);
            } else {
              const __half2 h2 = __floats2half2_rn(a0, a1);
              w4[q] = *reinterpret_cast<const uint32_t*>(&h2);
            }
          }
          *reinterpret_cast<uint4*>(orow + i) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
        }
      }
    };

    if constexpr (!kSplit) {
      if (duty && ok) {
        for (int c = 0; c < nd / 16; ++c) {
          uint32_t o[16];
          tmem_ld16(o_col + c * 16, o);
          tc_wait_ld();
          if (!row_ok) continue;
          float acc[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = __uint_as_float(o[i]);
          store_chunk(c, acc, inv);
        }
      }
    } else {
      // every part leaves its unnormalised rows and statistics; the last one to arrive merges
      const size_t rec_stride = static_cast<size_t>(2) * kTile * kPartRec;          // floats per part
      float* rec0 = p.scratch + static_cast<size_t>(cta) * p.split * rec_stride + (static_cast<size_t>(x) * kTile + row) * kPartRec;
      if (duty && ok) {
        float* mine = rec0 + part * rec_stride;
        for (int c = 0; c < nd / 16; ++c) {
          uint32_t o[16];
          tmem_ld16(o_col + c * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<float4*>(mine + d0 + c * 16 + i) =
                make_float4(__uint_as_float(o[i]), __uint_as_float(o[i + 1]), __uint_as_float(o[i + 2]),
                            __uint_as_float(o[i + 3]));
        }
        if (d0 == 0) *reinterpret_cast<float4*>(mine + kHeadDim) = make_float4(row_l, row_mu, row_mt, 0.f);
      }
      __threadfence();
      asm volatile("bar.sync 2, %0;" ::"r"(32 * kSoftWarps) : "memory");
      if (threadIdx.x == 64) ctl->ticket = atomicAdd(p.tickets + cta, 1u);
      asm volatile("bar.sync 2, %0;" ::"r"(32 * kSoftWarps) : "memory");
      if (*reinterpret_cast<volatile uint32_t*>(&ctl->ticket) == static_cast<uint32_t>(p.split - 1)) {
        __threadfence();
        if (threadIdx.x == 64) p.tickets[cta] = 0u;
        if (duty && row_ok && *abort_flag == 0u) {
          // one-pass parts share the constant stabiliser (statistics m = 0): plain sums.  Two-pass
          // parts are first brought to the largest stabiliser among them.
          float m_all = -__int_as_float(0x7f800000), mt_all = m_all;
          for (int q = 0; q < p.split; ++q) {
            const float4 stq = __ldcg(reinterpret_cast<const float4*>(rec0 + q * rec_stride + kHeadDim));
            m_all = fmaxf(m_all, stq.y);
            mt_all = fmaxf(mt_all, stq.z);
          }
          float l_all = 0.f;
          float f[4] = {0.f, 0.f, 0.f, 0.f};
          for (int q = 0; q < p.split; ++q) {
            const float4 stq = __ldcg(reinterpret_cast<const float4*>(rec0 + q * rec_stride + kHeadDim));
            f[q] = !exact ? 1.f : (stq.y == m_all ? 1.f : ex2_approx(stq.y - m_all));   // 2^(-inf) = 0 for empty parts
            l_all += stq.x * f[q];
          }
          float scale;
          if (!exact) {
            scale = 1.f / l_all;
          } else {
            const float corr = (m_all == mt_all) ? 1.f : ex2_approx(m_all - mt_all);
            scale = corr / fmaxf(l_all * corr, 1e-6f);
          }
          for (int c = 0; c < nd / 16; ++c) {
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = 0.f;
            for (int q = 0; q < p.split; ++q) {
              const float* src = rec0 + q * rec_stride + d0 + c * 16;
#pragma unroll
              for (int i = 0; i < 16; i += 4) {
                const float4 v4 = __ldcg(reinterpret_cast<const float4*>(src + i));
                acc[i] = fmaf(v4.x, f[q], acc[i]);
                acc[i + 1] = fmaf(v4.y, f[q], acc[i + 1]);
                acc[i + 2] = fmaf(v4.z, f[q], acc[i + 2]);
                acc[i + 3] = fmaf(v4.w, f[q], acc[i + 3]);
              }
            }
            store_chunk(c, acc, scale);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, kAttnTmemCols);
  }
}

// ---------------------------------------------------------------------- host
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// kmax2[b*H + h] = float bits of the largest squared key norm of head h (for the logit bounds)
int dsa_key_norm_max(const void* k, const int64_t* ks, int B, int H, int Tk, uint32_t* kmax2, cudaStream_t st) {
  SWV_CUDA_OK(cudaMemsetAsync(kmax2, 0, static_cast<size_t>(B) * H * 4, st));
  const int64_t total = static_cast<int64_t>(B) * H * Tk;
  key_norm_max_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(k), ks[0], ks[1], ks[2], B, H, Tk, kmax2);
  SWV_CUDA_OK(cudaGetLastError());
  return SWV_OK;
}

void dsa_workspace_views(void* workspace, int B, int Tq, int Tk, float** wq, float** wk, uint32_t** prefix,
                         uint32_t** kth, uint32_t** neq, uint32_t** kmax2, int32_t** excl);

// How many CTAs share one (query tile, head pair): with grids of only a few waves the last wave is
// far from full, so the key range is divided (1, 2 or 4 ways) to even the load out.
int dsa_attn_split_factor(int B, int H, int Tq, int Tk) {
  const int64_t ctas = static_cast<int64_t>(B) * ((Tq + kTile - 1) / kTile) * ((H + 1) / 2);
  const int n_kt = (Tk + kTile - 1) / kTile;
  const int n_sm = sm_count();
  if (ctas >= 4 * n_sm) return 1;
  int best = 1;
  double best_cost = static_cast<double>((ctas + n_sm - 1) / n_sm);
  for (int s = 2; s <= 4; s *= 2) {
    if (n_kt / s < 32) break;
    const double cost = static_cast<double>((ctas * s + n_sm - 1) / n_sm) / s + 0.02 * s;   // + merge overhead
    if (cost < best_cost - 1e-9) {
      best = s;
      best_cost = cost;
    }
  }
  return best;
}

int dsa_attn_scratch_bytes_impl(int B, int H, int Tq, int Tk, size_t* bytes) {
  if (!bytes) return SWV_ERR_NULL;
  if (B < 1 || H < 1 || Tq < 1 || Tk < 1) return SWV_ERR_SHAPE;
  const int s = dsa_attn_split_factor(B, H, Tq, Tk);
  const size_t ctas = static_cast<size_t>(B) * ((Tq + kTile - 1) / kTile) * ((H + 1) / 2);
  *bytes = s == 1 ? 0 : ((ctas * 4 + 255) / 256 * 256 + ctas * s * 2 * kTile * kPartRec * 4);
  return SWV_OK;
}

int dsa_attn_masked_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                         const int64_t* vs, const uint32_t* maskbits, void* workspace, void* o,
                         const int64_t* os, int o_dtype, int B, int H, int Tq, int Tk, int D, void* scratch,
                         size_t scratch_bytes, int* status, cudaStream_t st, int* member_count,
                         const uint32_t* only_flagged) {
  if (!q || !k || !v || !maskbits || !workspace || !o || !status || !qs || !ks || !vs || !os) return SWV_ERR_NULL;
  if (B < 1 || H < 1 || Tq < 1 || Tk < 1) return SWV_ERR_SHAPE;
  if (D != kHeadDim) return SWV_ERR_UNSUPPORTED;
  if (o_dtype != SWV_F32 && o_dtype != SWV_BF16 && o_dtype != SWV_F16) return SWV_ERR_DTYPE;
  const int64_t* ss[3] = {qs, ks, vs};
  const void* ps[3] = {q, k, v};
  for (int i = 0; i < 3; ++i) {
    if (ss[i][3] != 1) return SWV_ERR_ALIGN;
    if (!aligned16(ps[i])) return SWV_ERR_ALIGN;
    if ((ss[i][0] * 2) % 16 || (ss[i][1] * 2) % 16 || (ss[i][2] * 2) % 16) return SWV_ERR_ALIGN;
  }
  const int osz = o_dtype == SWV_F32 ? 4 : 2;
  if (os[3] != 1 || !aligned16(o) || (os[0] * osz) % 16 || (os[1] * osz) % 16 || (os[2] * osz) % 16)
    return SWV_ERR_ALIGN;
  if (!aligned16(maskbits) || (reinterpret_cast<uintptr_t>(workspace) & 255)) return SWV_ERR_ALIGN;

  float *wq = nullptr, *wk = nullptr;
  uint32_t *st_prefix = nullptr, *st_kth = nullptr, *st_neq = nullptr, *kmax2 = nullptr;
  int32_t* st_excl = nullptr;
  dsa_workspace_views(workspace, B, Tq, Tk, &wq, &wk, &st_prefix, &st_kth, &st_neq, &kmax2, &st_excl);
  if (static_cast<int64_t>(B) * H > 1024) return SWV_ERR_UNSUPPORTED;

  CUtensorMap tm_wq, tm_wk, tm_q, tm_k, tm_v;
  int rc = make_tmap_3d(&tm_wq, wq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, kIdxDim, Tq, B, kIdxDim * 4,
                        static_cast<uint64_t>(Tq) * kIdxDim * 4, 32, kTile);
  if (rc != SWV_OK) return rc;
  rc = make_tmap_3d(&tm_wk, wk, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, kIdxDim, Tk, B, kIdxDim * 4,
                    static_cast<uint64_t>(Tk) * kIdxDim * 4, 32, kTile);
  if (rc != SWV_OK) return rc;
  rc = make_tmap_4d(&tm_q, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, Tq, H, B, qs[2] * 2, qs[1] * 2, qs[0] * 2,
                    kHeadDim, kTile);
  if (rc != SWV_OK) return rc;
  rc = make_tmap_4d(&tm_k, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, Tk, H, B, ks[2] * 2, ks[1] * 2, ks[0] * 2,
                    kHeadDim, kTile);
  if (rc != SWV_OK) return rc;
  rc = make_tmap_4d(&tm_v, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, Tk, H, B, vs[2] * 2, vs[1] * 2, vs[0] * 2,
                    kHeadDim, kTile);
  if (rc != SWV_OK) return rc;

  AttnParams p;
  p.B = B; p.H = H; p.Tq = Tq; p.Tk = Tk;
  p.nQT = (Tq + kTile - 1) / kTile;
  p.nKT = (Tk + kTile - 1) / kTile;
  p.nHP = (H + 1) / 2;
  p.maskbits = maskbits;
  p.st_prefix = st_prefix; p.st_kth = st_kth; p.st_neq = st_neq; p.st_excl = st_excl;
  p.kmax2 = kmax2;
  p.q = static_cast<const __nv_bfloat16*>(q); p.qsb = qs[0]; p.qsh = qs[1]; p.qst = qs[2];
  p.o = o; p.osb = os[0]; p.osh = os[1]; p.ost = os[2]; p.o_dtype = o_dtype;
  p.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(D));
  p.status = status;

  // the key range is split only if the caller brought the scratch buffer for it
  p.split = 1;
  p.scratch = nullptr;
  p.tickets = nullptr;
  {
    size_t need = 0;
    dsa_attn_scratch_bytes_impl(B, H, Tq, Tk, &need);
    if (need > 0 && member_count == nullptr && scratch != nullptr && scratch_bytes >= need &&
        (reinterpret_cast<uintptr_t>(scratch) & 255) == 0) {
      const size_t ctas = static_cast<size_t>(B) * p.nQT * p.nHP;
      p.split = dsa_attn_split_factor(B, H, Tq, Tk);
      p.tickets = static_cast<uint32_t*>(scratch);
      p.scratch = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + (ctas * 4 + 255) / 256 * 256);
      SWV_CUDA_OK(cudaMemsetAsync(p.tickets, 0, ctas * 4, st));
    }
  }
  p.only_flagged = only_flagged;
  if (only_flagged == nullptr) {        // (the caller that passes flags has filled kmax2 already)
    const int rck = dsa_key_norm_max(k, ks, B, H, Tk, kmax2, st);
    if (rck != SWV_OK) return rck;
  }
  const unsigned grid = static_cast<unsigned>(B) * p.nQT * p.nHP * p.split;
  p.member_count = member_count;
  if (member_count != nullptr) {
    SWV_CUDA_OK(cudaMemsetAsync(member_count, 0, static_cast<size_t>(B) * Tq * sizeof(int), st));
    SWV_CUDA_OK(cudaFuncSetAttribute(dsa_attn_masked_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(attn_smem_bytes())));
    dsa_attn_masked_kernel<false, true><<<grid, kAttnThreads, attn_smem_bytes(), st>>>(tm_wq, tm_wk, tm_q, tm_k, tm_v, p);
  } else if (p.split == 1) {
    SWV_CUDA_OK(cudaFuncSetAttribute(dsa_attn_masked_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(attn_smem_bytes())));
    dsa_attn_masked_kernel<false><<<grid, kAttnThreads, attn_smem_bytes(), st>>>(tm_wq, tm_wk, tm_q, tm_k, tm_v, p);
  } else {
    SWV_CUDA_OK(cudaFuncSetAttribute(dsa_attn_masked_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(attn_smem_bytes())));
    dsa_attn_masked_kernel<true><<<grid, kAttnThreads, attn_smem_bytes(), st>>>(tm_wq, tm_wk, tm_q, tm_k, tm_v, p);
  }
  SWV_CUDA_OK(cudaGetLastError());
  return SWV_OK;
}

}  // namespace swv

#ifdef SWV_PROFILE
// Profiling build only: copies the 64 phase counters of dsa_attn_masked_kernel to `out_host`
// (synchronises the device) and clears them when `reset` is non-zero.
extern "C" int swv_debug_attn_profile(unsigned long long* out_host, int reset) {
  if (cudaDeviceSynchronize() != cudaSuccess) return SWV_ERR_CUDA;
  if (out_host != nullptr &&
      cudaMemcpyFromSymbol(out_host, swv::g_attn_prof, sizeof(unsigned long long) * 64) != cudaSuccess)
    return SWV_ERR_CUDA;
  if (reset) {
    static const unsigned long long zeros[64] = {0};
    if (cudaMemcpyToSymbol(swv::g_attn_prof, zeros, sizeof(zeros)) != cudaSuccess) return SWV_ERR_CUDA;
  }
  return SWV_OK;
}
#endif
