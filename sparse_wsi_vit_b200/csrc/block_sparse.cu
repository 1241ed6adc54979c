// Static block-sparse flash attention forward for sm_100a, driven by a CSR list of key
// blocks per query block, plus 2-D rotary embedding.
//
// The reference's static sparse attention
// (src/sparse_wsi_vit/models/static_sparse_attention.py:62-188) materialises a dense
// (N, N*ctx) mask and runs three SDPA calls; the 2-D block pattern the target asks for has
// no reference code at all.  Both are served by one kernel:
//   mode 0  : every listed key block is attended in full (block mask, shared by all heads);
//   mode 1  : inside the listed blocks the reference's token-level pattern applies:
//             query i sees key j iff  i < C  or  j < C  or
//             (|i - j| <= W*d and (i - j) % d == 0)      (C CLS tokens first, window W, dilation d)
//             -- exactly the mask static_sparse_attention.py:159-176 builds.
// One CTA owns (batch, head, one query block).  The score tile is M = 128 query rows by
// N = BS keys (BS = 64: the 64 rows behind the block are computed and dropped).
//   warp 0     : TMA producer (Q once; K, V blocks of the list through 2-stage rings)
//   warp 1     : UMMA issuer: S(j) = Q K(j)^T into one of TWO score buffers, O += P(j) V(j) with
//                P read from TMEM; S(j+2) is issued as soon as the softmax has read S(j), so the
//                tensor pipe works one tile ahead of the softmax
//   warps 2..9 : online softmax, two threads per query row (one per half of the key columns), ONE
//                pass per tile: exponentials are
//                taken against the current stabiliser while the tile's maximum is tracked; only
//                if some row's maximum exceeds its stabiliser by more than 2^8 is the stabiliser
//                raised, O (in TMEM) rescaled and the pass repeated (S stays intact: P has its
//                own columns)
// TMEM: S fp32 [0,BS) and [BS,2BS) | P (bf16x2) [2BS, 2.5BS) and [2.5BS, 3BS) | O fp32 [3BS, 3BS+D).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace swv {

struct BsaParams {
  int B, H, Tq, Tk, nQB;
  const int32_t* row_ptr;   // [nQB + 1]
  const int32_t* col_idx;   // [nnz] key block index
  int mode, num_cls, window, dilation;
  int kv_group;             // query heads per key/value head (grouped-query attention), >= 1
  float* lse;               // optional (B,H,Tq): natural-log sum of exponentials per row, -inf for empty rows
  // Optional gated epilogue (the NSA branches): the rows are scaled by sigmoid(gate[b,t,h,gate_idx])
  // (gate (B,Tq,H,3) fp32) and added to `acc_in` (fp32 contiguous (B,H,Tq,D), may be null) before
  // they are written to `o`.
  const float* gate;
  int gate_idx;
  const float* acc_in;
  void* o;
  int64_t osb, osh, ost;
  int o_dtype;
  float scale_log2;
  int* status;
};

struct BsaCtl {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2], p_full[2], pv_done[2];   // per score / probability buffer (tile parity)
  uint32_t tmem_base;
  uint32_t abort_flag;
  float xm[2][kTile][2];                       // per tile parity and row: the tile maximum seen by each column half
  float xl[kTile][2];                          // per row: the probability sum of each column half
};

template <int BS, int D>
struct BsaCfg {
  static constexpr int kQBytes = kTile * D * 2;     // 128 query rows
  static constexpr int kKVBytes = BS * D * 2;       // one key / value block
  static constexpr int kOffK = kQBytes;
  static constexpr int kOffV = kOffK + 2 * kKVBytes;
  static constexpr int kOffCtl = kOffV + 2 * kKVBytes;
  static constexpr uint32_t kColP = 2 * BS;          // two probability buffers of BS/2 columns
  static constexpr uint32_t kColO = 3 * BS;
  static constexpr uint32_t kTmemCols = (3 * BS + D <= 256) ? 256 : 512;
  // at least 80 KiB so that no more than two CTAs (2 x 256 TMEM columns) share an SM
  static constexpr size_t kSmemNeed = 1024 + kOffCtl + sizeof(BsaCtl) + 64;
  static constexpr size_t kSmem = kSmemNeed > 80 * 1024 ? kSmemNeed : 80 * 1024;
};

// One softmax pass of a thread over its row of the score tile: p = 2^(s*sc + neg_m) for the kept
// columns, written as bf16 pairs; returns the row's maximum raw score over the kept columns and
// the sum of the probabilities.  Loads run one 16-column unit ahead.
template <int BS, bool MASKED>
__device__ __forceinline__ void bsa_pass(uint32_t s_col, uint32_t p_col, const uint32_t (&keep)[(BS + 31) / 32], float sc,
                                         float neg_m, float& mt_out, float& l_out) {
  const float ninf = -__int_as_float(0x7f800000);
  float mt0 = ninf, mt1 = ninf, l0 = 0.f, l1 = 0.f;
  uint32_t sa[16], sb[16];
  tmem_ld16(s_col, sa);
#pragma unroll
  for (int u = 0; u < BS / 16; ++u) {
    tc_wait_ld();
    if (u + 1 < BS / 16) {
      if (u & 1) tmem_ld16(s_col + (u + 1) * 16, sa);
      else tmem_ld16(s_col + (u + 1) * 16, sb);
    }
    const uint32_t w = MASKED ? keep[u >> 1] >> ((u & 1) * 16) : 0xFFFFu;   // (BS = 32: one word)
    uint32_t packed[8];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const float s0 = __uint_as_float((u & 1) ? sb[i] : sa[i]);
      const float s1 = __uint_as_float((u & 1) ? sb[i + 1] : sa[i + 1]);
      float p0 = ex2_approx(fmaf(s0, sc, neg_m));
      float p1 = ex2_approx(fmaf(s1, sc, neg_m));
      if (MASKED) {
        const bool k0 = (w & (1u << i)) != 0u, k1 = (w & (2u << i)) != 0u;
        mt0 = fmaxf(mt0, k0 ? s0 : ninf);
        mt1 = fmaxf(mt1, k1 ? s1 : ninf);
        p0 = k0 ? p0 : 0.f;
        p1 = k1 ? p1 : 0.f;
      } else {
        mt0 = fmaxf(mt0, s0);
        mt1 = fmaxf(mt1, s1);
      }
      l0 += p0;
      l1 += p1;
      packed[i >> 1] = pack_bf16x2(p0, p1);
    }
    tmem_st8(p_col + u * 8, packed);
  }
  mt_out = fmaxf(mt0, mt1);
  l_out = l0 + l1;
}


// Token-level pattern of the reference's static attention (mode 1).
// With window 0 a patch sees the CLS keys only, not itself (static_sparse_attention.py:92-95).
__device__ __forceinline__ bool static_pattern(int qi, int kj, int C, int reach, int d) {
  if (qi < C || kj < C) return true;
  const int diff = qi - kj;
  const int ad = diff < 0 ? -diff : diff;
  return reach > 0 && ad <= reach && (ad % d) == 0;
}

template <int BS, int D>
__global__ void __launch_bounds__(320, 1)
    block_sparse_attn_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                             const __grid_constant__ CUtensorMap tm_v, const BsaParams p) {
  using Cfg = BsaCfg<BS, D>;
  constexpr uint32_t kIdescQK = make_idesc(/*bf16*/ 1, kTile, BS, 0, 0);
  constexpr uint32_t kIdescPV = make_idesc(/*bf16*/ 1, kTile, D, 0, /*V is MN-major*/ 1);
  constexpr float kStep = 8.0f;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  BsaCtl* ctl = reinterpret_cast<BsaCtl*>(smem + Cfg::kOffCtl);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // query blocks fastest, heads slowest: the CTAs in flight at any time work on one or two heads,
  // whose keys and values stay in L2 (all heads' K/V together can exceed it)
  const int qb = blockIdx.x % p.nQB;
  const int h = (blockIdx.x / p.nQB) % p.H;
  const int b = blockIdx.x / (p.H * p.nQB);
  const int list0 = p.row_ptr[qb];
  const int nblk = p.row_ptr[qb + 1] - list0;

  if (threadIdx.x == 0) {
    mbar_init(&ctl->q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl->k_full[s], 1);
      mbar_init(&ctl->k_empty[s], 1);
      mbar_init(&ctl->v_full[s], 1);
      mbar_init(&ctl->v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl->s_full[s], 1);
      mbar_init(&ctl->p_full[s], 8);
      mbar_init(&ctl->pv_done[s], 1);
    }
    ctl->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && nblk > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_expect_tx(&ctl->q_full, Cfg::kQBytes);
#pragma unroll
      for (int c = 0; c < D / 64; ++c)
        tma_load_4d(smem + c * (kTile * 128), &tm_q, &ctl->q_full, c * 64, qb * BS, h, b);
      const int hk = h / p.kv_group;
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        const int key0 = checked_index(p.col_idx[list0 + j], (p.Tk + BS - 1) / BS, p.status) * BS;
        if (!mbar_wait_bounded(&ctl->k_empty[s], par, abort_flag)) {
          record_status(p.status, kDevWaitStageEmpty);
          break;
        }
        mbar_expect_tx(&ctl->k_full[s], Cfg::kKVBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem + Cfg::kOffK + s * Cfg::kKVBytes + c * (BS * 128), &tm_k, &ctl->k_full[s], c * 64, key0, hk,
                      b);
        if (!mbar_wait_bounded(&ctl->v_empty[s], par, abort_flag)) {
          record_status(p.status, kDevWaitStageEmpty);
          break;
        }
        mbar_expect_tx(&ctl->v_full[s], Cfg::kKVBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem + Cfg::kOffV + s * Cfg::kKVBytes + c * (BS * 128), &tm_v, &ctl->v_full[s], c * 64, key0, hk,
                      b);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0 && nblk > 0) {
      const uint32_t q_addr = smem_u32(smem);
      const uint32_t k_addr = smem_u32(smem + Cfg::kOffK);
      const uint32_t v_addr = smem_u32(smem + Cfg::kOffV);
      bool ok = mbar_wait_bounded(&ctl->q_full, 0, abort_flag);
      if (!ok) record_status(p.status, kDevWaitQ);

      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait_bounded(&ctl->k_full[s], (j >> 1) & 1, abort_flag)) {
          record_status(p.status, kDevWaitTmaFull);
          return false;
        }
        tc_fence_after();
        const uint64_t da = smem_desc_sw128(q_addr);
        const uint64_t db = smem_desc_sw128(k_addr + s * Cfg::kKVBytes);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          // 64-element halves of the head dimension are separate swizzled tiles
          const uint64_t offa = (ks >> 2) * (kTile * 128 / 16) + (ks & 3) * 2;
          const uint64_t offb = (ks >> 2) * (BS * 128 / 16) + (ks & 3) * 2;
          umma_f16_ss(tmem_base + s * BS, da + offa, db + offb, kIdescQK, ks > 0);
        }
        umma_commit(&ctl->k_empty[s]);
        umma_commit(&ctl->s_full[s]);
        return true;
      };

      if (ok) ok = issue_qk(0);
      if (ok && nblk > 1) ok = issue_qk(1);
      for (int j = 0; ok && j < nblk; ++j) {
        const int s = j & 1;
        if (!mbar_wait_bounded(&ctl->v_full[s], (j >> 1) & 1, abort_flag)) {
          record_status(p.status, kDevWaitTmaFull);
          break;
        }
        if (!mbar_wait_bounded(&ctl->p_full[s], (j >> 1) & 1, abort_flag)) {
          record_status(p.status, kDevWaitPReady);
          break;
        }
        tc_fence_after();
        // V block: rows = keys (128 bytes per 64 head-dim elements), column halves BS*128 bytes apart
        const uint64_t dv = smem_desc_sw128(v_addr + s * Cfg::kKVBytes, BS * 128);
#pragma unroll
        for (int ks = 0; ks < BS / 16; ++ks)
          umma_f16_ts(tmem_base + Cfg::kColO, tmem_base + Cfg::kColP + s * (BS / 2) + ks * 8, dv + ks * 128, kIdescPV,
                      (j > 0 || ks > 0));
        umma_commit(&ctl->v_empty[s]);
        umma_commit(&ctl->pv_done[s]);
        // the softmax has read S(j) (it delivered P(j)): its buffer takes S(j+2)
        if (j + 2 < nblk) ok = issue_qk(j + 2);
      }
    }
  } else {
    // ----------------------------------------------------------------- softmax
    // Eight warps: warp (quarter, half) owns 32 query rows and half of the tile's key columns.  The
    // two warps of a row quarter exchange their tile maxima through shared memory (one named
    // barrier per tile), so both take the same decision on raising the stabiliser; each keeps the
    // probability sum of its columns and rescales / writes its half of the output channels.
    constexpr int HC = BS / 2;                 // key columns per warp
    constexpr int DH = D / 2;                  // output channels per warp
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int qrow = qb * BS + row;
    const bool row_ok = row < BS && qrow < p.Tq;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t o_col = lane_base + Cfg::kColO + half * DH;
    const float sc = p.scale_log2;
    const float ninf = -__int_as_float(0x7f800000);
    const int reach = p.window * p.dilation;
    const int dil = p.dilation > 0 ? p.dilation : 1;

    float m_used = ninf, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      const int key0 = checked_index(p.col_idx[list0 + j], (p.Tk + BS - 1) / BS, p.status) * BS;
      const int sb = j & 1;
      const uint32_t s_col = lane_base + sb * BS + half * HC;
      const uint32_t p_col = lane_base + Cfg::kColP + sb * (BS / 2) + half * (HC / 2);
      // S(j) computed; P's buffer no longer read by PV(j-2).  (A wait that gave up keeps looping
      // without work: both warps of a quarter pass the same barriers.)
      if (ok && (!mbar_wait_bounded(&ctl->s_full[sb], (j >> 1) & 1, abort_flag) ||
                 (j >= 2 && !mbar_wait_bounded(&ctl->pv_done[sb], ((j >> 1) & 1) ^ 1, abort_flag)))) {
        record_status(p.status, kDevWaitAccFull);
        ok = false;
      }
      tc_fence_after();
      // which of its columns the row attends (bit i of word c = column half*HC + 32c + i)
      // Token-pattern mode: a block whose every (query, key) pair lies inside the window (no CLS
      // row or column involved, dilation 1) needs no per-element pattern test.
      bool inside = false;
      if (p.mode != 0 && dil == 1 && qb * BS >= p.num_cls && key0 >= p.num_cls) {
        const int q0 = qb * BS, far = max(q0 + BS - 1 - key0, key0 + BS - 1 - q0);
        inside = far <= reach;
      }
      const bool masked = (p.mode != 0 && !inside) || key0 + BS > p.Tk;
      uint32_t keep[(HC + 31) / 32];
#pragma unroll
      for (int c = 0; c < (HC + 31) / 32; ++c) {
        uint32_t w = 0xFFFFFFFFu;
        const int base = key0 + half * HC + c * 32;
        if (p.mode != 0 && !inside) {
          w = 0;
#pragma unroll 4
          for (int i = 0; i < 32; ++i) {
            const int kj = base + i;
            if (kj < p.Tk && static_pattern(qrow, kj, p.num_cls, reach, dil)) w |= 1u << i;
          }
        } else if (masked) {
          const int nv = p.Tk - base;
          w = nv >= 32 ? 0xFFFFFFFFu : (nv <= 0 ? 0u : ((1u << nv) - 1u));
        }
        keep[c] = w;
      }

      // rows that have attended nothing yet have m_used = -inf; their stabiliser is 0 for now
      float mt = ninf, lt = 0.f;
      if (ok) {
        if (masked) bsa_pass<HC, true>(s_col, p_col, keep, sc, (m_used == ninf) ? 0.f : -m_used, mt, lt);
        else bsa_pass<HC, false>(s_col, p_col, keep, sc, (m_used == ninf) ? 0.f : -m_used, mt, lt);
      }
      ctl->xm[sb][row][half] = mt;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
      const float m_new = fmaxf(m_used, fmaxf(ctl->xm[sb][row][0], ctl->xm[sb][row][1]) * sc);
      if (__any_sync(0xffffffffu, m_new > m_used + kStep)) {
        // raise the stabiliser, rescale what has been accumulated, repeat the pass
        const float factor = (m_new == m_used) ? 1.f : ex2_approx(m_used - m_new);
        l *= factor;
        m_used = m_new;
        if (j > 0) {
          // O of the tiles before this one is complete once PV(j-1) retired
          if (ok && !mbar_wait_bounded(&ctl->pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag)) {
            record_status(p.status, kDevWaitPvDone);
            ok = false;
          }
          if (ok) {
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < DH / 16; ++c) {
              uint32_t o[16];
              tmem_ld16(o_col + c * 16, o);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
              tmem_st16(o_col + c * 16, o);
            }
            tc_wait_st();
          }
        }
        if (ok) {
          if (masked) bsa_pass<HC, true>(s_col, p_col, keep, sc, (m_used == ninf) ? 0.f : -m_used, mt, lt);
          else bsa_pass<HC, false>(s_col, p_col, keep, sc, (m_used == ninf) ? 0.f : -m_used, mt, lt);
        }
      }
      l += lt;
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(&ctl->p_full[sb]);
    }

    if (nblk > 0 && ok && !mbar_wait_bounded(&ctl->pv_done[(nblk - 1) & 1], ((nblk - 1) >> 1) & 1, abort_flag)) {
      record_status(p.status, kDevWaitPvDone);
      ok = false;
    }
    // the row's probability sum: both column halves
    ctl->xl[row][half] = l;
    asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
    l = ctl->xl[row][0] + ctl->xl[row][1];
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      if (p.lse != nullptr && row_ok && half == 0) {
        p.lse[(static_cast<int64_t>(b) * p.H + h) * p.Tq + qrow] =
            l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : ninf;
      }
#pragma unroll 1
      for (int c = 0; c < DH / 16; ++c) {
        uint32_t o[16];
        if (nblk > 0) {
          tmem_ld16(o_col + c * 16, o);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = 0u;
        }
        if (!row_ok) continue;
        if (p.gate != nullptr) {
          // gated accumulate: value = acc_in + sigmoid(g) * (o * inv), the order the stand-alone
          // gate kernel adds the branches in
          const float gl = p.gate[((static_cast<int64_t>(b) * p.Tq + qrow) * p.H + h) * 3 + p.gate_idx];
          const float gs = 1.f / (1.f + __expf(-gl));
          const float* arow = p.acc_in == nullptr ? nullptr
                                                  : p.acc_in + ((static_cast<int64_t>(b) * p.H + h) * p.Tq + qrow) * D +
                                                        half * DH + c * 16;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float a = __uint_as_float(o[i]) * inv;
            o[i] = __float_as_uint(arow == nullptr ? gs * a : fmaf(gs, a, arow[i]));
          }
        }
        const float inv_w = p.gate != nullptr ? 1.f : inv;      // (already applied above)
        if (p.o_dtype == SWV_F32) {
          float* orow = static_cast<float*>(p.o) + b * p.osb + h * p.osh + qrow * p.ost + half * DH + c * 16;
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            *reinterpret_cast<float4*>(orow + i) =
                make_float4(__uint_as_float(o[i]) * inv_w, __uint_as_float(o[i + 1]) * inv_w,
                            __uint_as_float(o[i + 2]) * inv_w, __uint_as_float(o[i + 3]) * inv_w);
          }
        } else {
          uint16_t* orow = static_cast<uint16_t*>(p.o) + b * p.osb + h * p.osh + qrow * p.ost + half * DH + c * 16;
#pragma unroll
          for (int i = 0; i < 16; i += 8) {
            uint32_t w4[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float a0 = __uint_as_float(o[i + 2 * q]) * inv_w, a1 = __uint_as_float(o[i + 2 * q + 1]) * inv_w;
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
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------ 2-D RoPE
// x (L, H, hd) rotated in place-compatible fashion into y: first half of the head uses
// coords[:,0], second half coords[:,1]; hd/4 frequencies theta^(-2i/(hd/2)), each for two
// adjacent channels; (x0, x1) -> (x0 cos - x1 sin, x1 cos + x0 sin)
// (src/sparse_wsi_vit/models/vit_5/rope.py:33-37, 56-59, 81-97).  Tokens < skip are copied.
template <typename T>
__global__ void rope2d_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ coords,
                              int64_t L, int H, int hd, int64_t xs_l, int64_t xs_h, int64_t ys_l, int64_t ys_h,
                              float inv_high, float log2_theta, int skip) {
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int pairs = hd / 2;
  const int64_t total = L * H * pairs;
  if (gid >= total) return;
  const int pr = static_cast<int>(gid % pairs);
  const int hh = static_cast<int>((gid / pairs) % H);
  const int64_t t = gid / (static_cast<int64_t>(pairs) * H);
  const T* xp = x + t * xs_l + hh * xs_h + 2 * pr;
  T* yp = y + t * ys_l + hh * ys_h + 2 * pr;
  float x0, x1;
  if constexpr (sizeof(T) == 4) {
    x0 = xp[0];
    x1 = xp[1];
  } else {
    x0 = __bfloat162float(xp[0]);
    x1 = __bfloat162float(xp[1]);
  }
  float o0 = x0, o1 = x1;
  if (t >= skip) {
    const int half_pairs = pairs / 2;                 // pairs per coordinate axis
    const int axis = pr >= half_pairs ? 1 : 0;
    const int f = pr - axis * half_pairs;             // frequency index
    const int dim = hd / 2;
    const float freq = exp2f(-log2_theta * (2.0f * f) / dim);
    const float ang = __fmul_rn(__fmul_rn(coords[t * 2 + axis], inv_high), freq);
    float sn, cs;
    sincosf(ang, &sn, &cs);
    // explicit rounding order (the fused prologue kernel in indexer.cu computes the same expression
    // and must give the same bits)
    o0 = __fmaf_rn(x0, cs, -__fmul_rn(x1, sn));
    o1 = __fmaf_rn(x1, cs, __fmul_rn(x0, sn));
  }
  if constexpr (sizeof(T) == 4) {
    yp[0] = o0;
    yp[1] = o1;
  } else {
    yp[0] = __float2bfloat16_rn(o0);
    yp[1] = __float2bfloat16_rn(o1);
  }
}

// Mean pooling of overlapping token windows: y[b,h,c,:] = mean_{i < win} x[b,h,c*stride + i,:]
// (the compressed keys / values of the NSA compressed branch).  One thread per output pair of channels.
__global__ void pool_tokens_kernel(const __nv_bfloat16* __restrict__ x, int64_t sb, int64_t sh, int64_t st_,
                                   __nv_bfloat16* __restrict__ y, int B, int H, int T, int D, int nC, int win,
                                   int stride) {
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int pairs = D / 2;
  const int64_t total = static_cast<int64_t>(B) * H * nC * pairs;
  if (gid >= total) return;
  const int pr = static_cast<int>(gid % pairs);
  const int c = static_cast<int>((gid / pairs) % nC);
  const int h = static_cast<int>((gid / (static_cast<int64_t>(pairs) * nC)) % H);
  const int b = static_cast<int>(gid / (static_cast<int64_t>(pairs) * nC * H));
  const __nv_bfloat16* xp = x + b * sb + h * sh + static_cast<int64_t>(c) * stride * st_ + 2 * pr;
  float a0 = 0.f, a1 = 0.f;
  for (int i = 0; i < win; ++i) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(xp + i * st_);
    a0 += __bfloat162float(v.x);
    a1 += __bfloat162float(v.y);
  }
  const float inv = 1.0f / win;
  __nv_bfloat162 o;
  o.x = __float2bfloat16_rn(a0 * inv);
  o.y = __float2bfloat16_rn(a1 * inv);
  *reinterpret_cast<__nv_bfloat162*>(y + ((static_cast<int64_t>(b) * H + h) * nC + c) * D + 2 * pr) = o;
}

// ---------------------------------------------------------------------- host
static bool bsa_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int BS, int D>
static int launch_bsa(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const BsaParams& p,
                      cudaStream_t st) {
  using Cfg = BsaCfg<BS, D>;
  SWV_CUDA_OK(cudaFuncSetAttribute(block_sparse_attn_kernel<BS, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(Cfg::kSmem)));
  const unsigned grid = static_cast<unsigned>(p.B) * p.nQB * p.H;
  block_sparse_attn_kernel<BS, D><<<grid, 320, Cfg::kSmem, st>>>(tq, tk, tv, p);
  SWV_CUDA_OK(cudaGetLastError());
  return SWV_OK;
}

int block_sparse_attn_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                           const int64_t* vs, const int32_t* row_ptr, const int32_t* col_idx, int block, int mode,
                           int num_cls, int window, int dilation, int kv_group, float* lse, void* o,
                           const int64_t* os, int o_dtype, int B, int H, int Tq, int Tk, int D, int* status,
                           cudaStream_t st, const float* gate, int gate_idx, const float* acc_in) {
  if (!q || !k || !v || !row_ptr || !col_idx || !o || !status || !qs || !ks || !vs || !os) return SWV_ERR_NULL;
  if (B < 1 || H < 1 || Tq < 1 || Tk < 1) return SWV_ERR_SHAPE;
  if (kv_group < 1 || H % kv_group != 0) return SWV_ERR_SHAPE;
  if ((block != 64 && block != 128) || (D != 64 && D != 128)) return SWV_ERR_UNSUPPORTED;
  if (mode != 0 && mode != 1) return SWV_ERR_UNSUPPORTED;
  if (mode == 1 && (num_cls < 0 || window < 0 || dilation < 1)) return SWV_ERR_SHAPE;
  if (o_dtype != SWV_F32 && o_dtype != SWV_BF16 && o_dtype != SWV_F16) return SWV_ERR_DTYPE;
  const int64_t* ss[3] = {qs, ks, vs};
  const void* ps[3] = {q, k, v};
  for (int i = 0; i < 3; ++i) {
    if (ss[i][3] != 1 || !bsa_aligned16(ps[i])) return SWV_ERR_ALIGN;
    if ((ss[i][0] * 2) % 16 || (ss[i][1] * 2) % 16 || (ss[i][2] * 2) % 16) return SWV_ERR_ALIGN;
  }
  const int osz = o_dtype == SWV_F32 ? 4 : 2;
  if (os[3] != 1 || !bsa_aligned16(o) || (os[0] * osz) % 16 || (os[1] * osz) % 16 || (os[2] * osz) % 16)
    return SWV_ERR_ALIGN;

  CUtensorMap tq, tk, tv;
  int rc = make_tmap_4d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, Tq, H, B, qs[2] * 2, qs[1] * 2, qs[0] * 2, 64,
                        kTile);
  if (rc != SWV_OK) return rc;
  const int Hkv = H / kv_group;
  rc = make_tmap_4d(&tk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, Tk, Hkv, B, ks[2] * 2, ks[1] * 2, ks[0] * 2, 64, block);
  if (rc != SWV_OK) return rc;
  rc = make_tmap_4d(&tv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, Tk, Hkv, B, vs[2] * 2, vs[1] * 2, vs[0] * 2, 64, block);
  if (rc != SWV_OK) return rc;

  BsaParams p;
  p.B = B; p.H = H; p.Tq = Tq; p.Tk = Tk;
  p.nQB = (Tq + block - 1) / block;
  p.row_ptr = row_ptr; p.col_idx = col_idx;
  p.mode = mode; p.num_cls = num_cls; p.window = window; p.dilation = dilation;
  p.kv_group = kv_group; p.lse = lse;
  p.gate = gate; p.gate_idx = gate_idx; p.acc_in = acc_in;
  p.o = o; p.osb = os[0]; p.osh = os[1]; p.ost = os[2]; p.o_dtype = o_dtype;
  p.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(D));
  p.status = status;
  if (block == 64 && D == 64) return launch_bsa<64, 64>(tq, tk, tv, p, st);
  if (block == 64 && D == 128) return launch_bsa<64, 128>(tq, tk, tv, p, st);
  if (block == 128 && D == 64) return launch_bsa<128, 64>(tq, tk, tv, p, st);
  return launch_bsa<128, 128>(tq, tk, tv, p, st);
}

int pool_tokens_impl(const void* x, const int64_t* xs, void* y, int B, int H, int T, int D, int win, int stride,
                     cudaStream_t st) {
  if (!x || !y || !xs) return SWV_ERR_NULL;
  if (B < 1 || H < 1 || T < win || win < 1 || stride < 1 || D < 2 || (D & 1)) return SWV_ERR_SHAPE;
  if (xs[3] != 1 || (xs[0] & 1) || (xs[1] & 1) || (xs[2] & 1) || (reinterpret_cast<uintptr_t>(x) & 3)) return SWV_ERR_ALIGN;
  const int nC = (T - win) / stride + 1;
  const int64_t total = static_cast<int64_t>(B) * H * nC * (D / 2);
  pool_tokens_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), xs[0], xs[1], xs[2], static_cast<__nv_bfloat16*>(y), B, H, T, D, nC, win,
      stride);
  SWV_CUDA_OK(cudaGetLastError());
  return SWV_OK;
}

int rope2d_impl(const void* x, const int64_t* xs, void* y, const int64_t* ys, int dtype, const float* coords,
                int64_t L, int H, int hd, float coord_high, float theta, int skip, cudaStream_t st) {
  if (!x || !y || !coords || !xs || !ys) return SWV_ERR_NULL;
  if (L < 1 || H < 1 || hd < 4 || (hd % 4) != 0 || coord_high == 0.f || theta <= 0.f || skip < 0) return SWV_ERR_SHAPE;
  if (xs[2] != 1 || ys[2] != 1) return SWV_ERR_ALIGN;
  if (dtype != SWV_F32 && dtype != SWV_BF16) return SWV_ERR_DTYPE;
  const int64_t total = L * H * (hd / 2);
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  if (dtype == SWV_F32) {
    rope2d_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(y), coords, L, H, hd,
                                               xs[0], xs[1], ys[0], ys[1], 1.0f / coord_high, log2f(theta), skip);
  } else {
    rope2d_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                       static_cast<__nv_bfloat16*>(y), coords, L, H, hd, xs[0], xs[1],
                                                       ys[0], ys[1], 1.0f / coord_high, log2f(theta), skip);
  }
  SWV_CUDA_OK(cudaGetLastError());
  return SWV_OK;
}

}  // namespace swv
