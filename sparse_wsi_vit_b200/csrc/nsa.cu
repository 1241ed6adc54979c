// NSA-style attention forward for sm_100a: block importance, per-query block selection, attention
// over the selected blocks for a whole grouped-query group, and the gated sum of the branches.
//
// The reference has no NSA code (it only names the idea, scripts/virchow_preprocess.py:44-53); the
// semantics are this library's own:
//   importance[b, g, t, s] = sum over the G query heads h of kv group g and over the compressed
//                            tokens c whose first key lies in selection block s of
//                            exp(q_h[t] . kc_g[c] / sqrt(D) - lse_h[t])
//   (lse = log-sum-exp of the compressed branch), the `n_sel` largest blocks per (b, g, t) are
//   selected, ties to the lower block index, reported in ascending order.
// Kernels:
//   nsa_importance_kernel : per CTA 128 queries of one kv group; for every tile of 128 compressed
//                           keys and every head of the group S = Q_h Kc^T on the tensor cores
//                           (TMA rings -> tcgen05 -> two TMEM accumulators), eight epilogue warps
//                           turn scores into probabilities and add them up per selection block.
//   nsa_select_kernel     : one warp per (b, g, t): iterative arg-max over the importance row.
//   nsa_selected_attn_mma_kernel : one warp per (b, g, t), the G heads as rows of mma.sync tiles: every
//                           selected key / value row is read once for the whole group
//                           (nsa_selected_attn_kernel: the same on CUDA cores, for unaligned layouts).
//   nsa_combine_kernel    : out = sum_b sigmoid(gate_b) * O_b.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace swv {

// ---------------------------------------------------------------- importance
struct NsaImpParams {
  int B, Hq, Hkv, G, Tq, nC, nQT, nCT, n_pad;
  const float* lse;     // (B, Hq, Tq) natural log
  float* imp;           // (B, Hkv, Tq, n_pad)
  float scale_log2;
  int* status;
};

struct NsaImpCtl {
  uint64_t q_full[2], q_empty[2], k_full[2], k_empty[2], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

constexpr int kNsaMaxGroup = 16;

template <int D>
struct NsaImpCfg {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kOffK = 2 * kTileBytes;
  static constexpr int kOffLse = 4 * kTileBytes;
  static constexpr int kOffCtl = kOffLse + kNsaMaxGroup * kTile * 4;
  static constexpr size_t kSmem = 1024 + kOffCtl + sizeof(NsaImpCtl) + 64;
};

// R = compressed tokens per selection block (selection block size / compression stride).
template <int D, int R>
__global__ void __launch_bounds__(320, 1)
    nsa_importance_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const NsaImpParams p) {
  using Cfg = NsaImpCfg<D>;
  constexpr uint32_t kIdesc = make_idesc(/*bf16*/ 1, kTile, kTile, 0, 0);
  constexpr int kAcc = 64 / R;                       // selection blocks per warp and key tile

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* lse_sm = reinterpret_cast<float*>(smem + Cfg::kOffLse);
  NsaImpCtl* ctl = reinterpret_cast<NsaImpCtl*>(smem + Cfg::kOffCtl);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qt = blockIdx.x % p.nQT;
  const int g = (blockIdx.x / p.nQT) % p.Hkv;
  const int b = blockIdx.x / (p.nQT * p.Hkv);
  const int G = p.G;
  const int nIt = p.nCT * G;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl->q_full[s], 1);
      mbar_init(&ctl->q_empty[s], 1);
      mbar_init(&ctl->k_full[s], 1);
      mbar_init(&ctl->k_empty[s], 1);
      mbar_init(&ctl->acc_full[s], 1);
      mbar_init(&ctl->acc_empty[s], 8);
    }
    ctl->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, 256);
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
      for (int it = 0; it < nIt; ++it) {
        const int jt = it / G, hh = it - jt * G, s = it & 1;
        if (!mbar_wait_bounded(&ctl->q_empty[s], ((it >> 1) & 1) ^ 1, abort_flag)) {
          record_status(p.status, kDevWaitStageEmpty);
          break;
        }
        mbar_expect_tx(&ctl->q_full[s], Cfg::kTileBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem + s * Cfg::kTileBytes + c * (kTile * 128), &tm_q, &ctl->q_full[s], c * 64, qt * kTile,
                      g * G + hh, b);
        if (hh == 0) {
          const int ks = jt & 1;
          if (!mbar_wait_bounded(&ctl->k_empty[ks], ((jt >> 1) & 1) ^ 1, abort_flag)) {
            record_status(p.status, kDevWaitStageEmpty);
            break;
          }
          mbar_expect_tx(&ctl->k_full[ks], Cfg::kTileBytes);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(smem + Cfg::kOffK + ks * Cfg::kTileBytes + c * (kTile * 128), &tm_k, &ctl->k_full[ks], c * 64,
                        jt * kTile, g, b);
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t q_addr = smem_u32(smem);
      const uint32_t k_addr = smem_u32(smem + Cfg::kOffK);
      for (int it = 0; it < nIt; ++it) {
        const int jt = it / G, hh = it - jt * G, s = it & 1, ks = jt & 1;
        if (!mbar_wait_bounded(&ctl->q_full[s], (it >> 1) & 1, abort_flag) ||
            (hh == 0 && !mbar_wait_bounded(&ctl->k_full[ks], (jt >> 1) & 1, abort_flag))) {
          record_status(p.status, kDevWaitTmaFull);
          break;
        }
        if (!mbar_wait_bounded(&ctl->acc_empty[s], ((it >> 1) & 1) ^ 1, abort_flag)) {
          record_status(p.status, kDevWaitAccEmpty);
          break;
        }
        tc_fence_after();
        const uint64_t da = smem_desc_sw128(q_addr + s * Cfg::kTileBytes);
        const uint64_t db = smem_desc_sw128(k_addr + ks * Cfg::kTileBytes);
#pragma unroll
        for (int k16 = 0; k16 < D / 16; ++k16) {
          // 64-element halves of the head dimension are separate swizzled tiles
          const uint64_t off = (k16 >> 2) * (kTile * 128 / 16) + (k16 & 3) * 2;
          umma_f16_ss(tmem_base + s * kTile, da + off, db + off, kIdesc, k16 > 0);
        }
        umma_commit(&ctl->q_empty[s]);
        if (hh == G - 1) umma_commit(&ctl->k_empty[ks]);
        umma_commit(&ctl->acc_full[s]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const int half = ew >> 2;
    const int row = quarter * 32 + lane;
    const int qrow = qt * kTile + row;
    const bool row_ok = qrow < p.Tq;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const int et = threadIdx.x - 64;
    for (int i = et; i < G * kTile; i += 256) {
      const int hh = i / kTile, r = i - hh * kTile, t = qt * kTile + r;
      // +inf for rows behind the end: their probabilities are 0
      lse_sm[i] = t < p.Tq ? p.lse[(static_cast<int64_t>(b) * p.Hq + g * G + hh) * p.Tq + t] * 1.4426950408889634f
                           : __int_as_float(0x7f800000);
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    float* out_row = p.imp + ((static_cast<int64_t>(b) * p.Hkv + g) * p.Tq + qrow) * p.n_pad + half * kAcc;
    bool ok = true;
    for (int jt = 0; ok && jt < p.nCT; ++jt) {
      float acc[kAcc];
#pragma unroll
      for (int i = 0; i < kAcc; ++i) acc[i] = 0.f;
      const int col0 = jt * kTile + half * 64;        // first compressed token of this warp's columns
      const int nvalid = p.nC - col0;
      for (int hh = 0; hh < G; ++hh) {
        const int it = jt * G + hh, s = it & 1;
        if (!mbar_wait_bounded(&ctl->acc_full[s], (it >> 1) & 1, abort_flag)) {
          record_status(p.status, kDevWaitAccFull);
          ok = false;
          break;
        }
        tc_fence_after();
        const float neg_l = -lse_sm[hh * kTile + row];
        const uint32_t s_col = lane_base + s * kTile + half * 64;
        uint32_t sa[16], sb[16];
        tmem_ld16(s_col, sa);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          tc_wait_ld();
          if (u + 1 < 4) {
            if (u & 1) tmem_ld16(s_col + (u + 1) * 16, sa);
            else tmem_ld16(s_col + (u + 1) * 16, sb);
          } else {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->acc_empty[s]);
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float pr = ex2_approx(fmaf(__uint_as_float((u & 1) ? sb[i] : sa[i]), p.scale_log2, neg_l));
            if (nvalid < 64 && u * 16 + i >= nvalid) pr = 0.f;
            acc[(u * 16 + i) / R] += pr;
          }
        }
      }
      if (ok && row_ok) {
        float* dst = out_row + jt * (kTile / R);
        if constexpr (kAcc % 4 == 0) {
#pragma unroll
          for (int i = 0; i < kAcc; i += 4)
            *reinterpret_cast<float4*>(dst + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < kAcc; ++i) dst[i] = acc[i];
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, 256);
  }
}

// ------------------------------------------------------------------- select
// One warp per (b, g, t).  Importance values are >= 0; taken entries are marked -1, entries
// behind the last selection block -2.  Ties go to the lower block index; output ascending.
__global__ void __launch_bounds__(128) nsa_select_kernel(const float* __restrict__ imp, int n_pad, int n_s, int k_eff,
                                                         int64_t rows, int32_t* __restrict__ blocks) {
  extern __shared__ float sel_sm[];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * 4 + wib;
  if (r >= rows) return;
  const int n = (n_s + 31) & ~31;                     // scanned range, a multiple of 32
  float* v = sel_sm + wib * n;
  const float* src = imp + r * n_pad;
  for (int i = lane; i < n; i += 32) v[i] = i < n_s ? (i < n_pad ? src[i] : 0.f) : -2.f;
  __syncwarp();
  for (int s = 0; s < k_eff; ++s) {
    float best = -3.f;
    int bi = 0x7fffffff;
    for (int i = lane; i < n; i += 32) {
      const float x = v[i];
      if (x > best) {                                 // ascending scan, strict: the lowest index of equals
        best = x;
        bi = i;
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
    if (lane == 0) v[bi] = -1.f;
    __syncwarp();
  }
  int32_t* dst = blocks + r * k_eff;
  int cnt = 0;
  for (int i0 = 0; i0 < n; i0 += 32) {
    const bool taken = v[i0 + lane] == -1.f;
    const uint32_t m = __ballot_sync(0xffffffffu, taken);
    if (taken) dst[cnt + __popc(m & ((1u << lane) - 1u))] = i0 + lane;
    cnt += __popc(m);
  }
}

// ------------------------------------------------------- selected attention
// One warp per (b, g, t): plain softmax attention of the G query heads of kv group g over the keys
// of the selected blocks.  Scores: every lane owns one key of a 32-key chunk and accumulates the G
// dot products (q broadcast from shared memory); values: every lane owns D/32 channels.
struct NsaSelParams {
  const __nv_bfloat16 *q, *k, *v;
  int64_t qs[4], ks[4], vs[4];
  const int32_t* blocks;    // (B, Hkv, Tq, n_sel)
  float* o;                 // (B, Hq, Tq, D) fp32 contiguous
  // Gated form (whole-pass call): o is the running gated sum of the branches and this branch adds
  // sigmoid(gate[b,t,h,1]) * (its rows) to it; gate (B,Tq,Hq,3) fp32, null = plain store.
  const float* gate;
  int B, Hq, Hkv, G, Tq, Tk, n_sel, sel_block;
  float scale_log2;
};

template <int D, int GMAX>
__global__ void __launch_bounds__(128) nsa_selected_attn_kernel(const NsaSelParams p) {
  constexpr int DPL = D / 32;
  __shared__ float qsm[4][GMAX][D];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t wid = static_cast<int64_t>(blockIdx.x) * 4 + wib;
  const int64_t total = static_cast<int64_t>(p.B) * p.Hkv * p.Tq;
  if (wid >= total) return;
  const int t = static_cast<int>(wid % p.Tq);
  const int g = static_cast<int>((wid / p.Tq) % p.Hkv);
  const int b = static_cast<int>(wid / (static_cast<int64_t>(p.Tq) * p.Hkv));
  const int G = p.G;

  for (int i = lane; i < G * D; i += 32) {
    const int hh = i / D, d = i - hh * D;
    qsm[wib][hh][d] = __bfloat162float(p.q[b * p.qs[0] + (g * G + hh) * p.qs[1] + t * p.qs[2] + d]) * p.scale_log2;
  }
  __syncwarp();
  const __nv_bfloat16* kbase = p.k + b * p.ks[0] + g * p.ks[1];
  const __nv_bfloat16* vbase = p.v + b * p.vs[0] + g * p.vs[1];
  const int32_t* blk = p.blocks + ((static_cast<int64_t>(b) * p.Hkv + g) * p.Tq + t) * p.n_sel;
  const float ninf = -__int_as_float(0x7f800000);

  float o[GMAX][DPL];
  float m[GMAX], l[GMAX];
#pragma unroll
  for (int hh = 0; hh < GMAX; ++hh) {
    m[hh] = ninf;
    l[hh] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[hh][i] = 0.f;
  }

  const int chunks_per_block = p.sel_block / 32;
  for (int s = 0; s < p.n_sel; ++s) {
    const int key_block0 = blk[s] * p.sel_block;
    for (int c = 0; c < chunks_per_block; ++c) {
      const int key = key_block0 + c * 32 + lane;
      const bool ok = key < p.Tk;
      // ---- scores of this lane's key against the G heads (log2 domain)
      float sc[GMAX];
#pragma unroll
      for (int hh = 0; hh < GMAX; ++hh) sc[hh] = 0.f;
      if (ok) {
        const uint4* kr = reinterpret_cast<const uint4*>(kbase + static_cast<int64_t>(key) * p.ks[2]);
#pragma unroll 2
        for (int d8 = 0; d8 < D / 8; ++d8) {
          const uint4 kv = __ldg(kr + d8);
          const uint32_t w[4] = {kv.x, kv.y, kv.z, kv.w};
          float kf[8];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            kf[2 * q] = __uint_as_float(w[q] << 16);
            kf[2 * q + 1] = __uint_as_float(w[q] & 0xffff0000u);
          }
#pragma unroll
          for (int hh = 0; hh < GMAX; ++hh) {
            if (hh < G) {
              const float4 qa = *reinterpret_cast<const float4*>(&qsm[wib][hh][d8 * 8]);
              const float4 qb = *reinterpret_cast<const float4*>(&qsm[wib][hh][d8 * 8 + 4]);
              sc[hh] = fmaf(qa.x, kf[0], fmaf(qa.y, kf[1], fmaf(qa.z, kf[2], fmaf(qa.w, kf[3], sc[hh]))));
              sc[hh] = fmaf(qb.x, kf[4], fmaf(qb.y, kf[5], fmaf(qb.z, kf[6], fmaf(qb.w, kf[7], sc[hh]))));
            }
          }
        }
      }
      // ---- online softmax per head; probabilities stay in the lane that owns the key
      float pr[GMAX];
#pragma unroll
      for (int hh = 0; hh < GMAX; ++hh) {
        pr[hh] = 0.f;
        if (hh < G) {
          float gm = ok ? sc[hh] : ninf;
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, off));
          const float m_new = fmaxf(m[hh], gm);
          if (m_new != ninf) {
            const float alpha = (m[hh] == m_new) ? 1.f : ex2_approx(m[hh] - m_new);
            pr[hh] = ok ? ex2_approx(sc[hh] - m_new) : 0.f;
            float ps = pr[hh];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
            l[hh] = l[hh] * alpha + ps;
#pragma unroll
            for (int i = 0; i < DPL; ++i) o[hh][i] *= alpha;
            m[hh] = m_new;
          }
        }
      }
      // ---- O += P V: the chunk's value rows are read once for all heads
      const int nk = min(32, p.Tk - (key_block0 + c * 32));
      for (int j = 0; j < nk; ++j) {
        const __nv_bfloat16* vr = vbase + static_cast<int64_t>(key_block0 + c * 32 + j) * p.vs[2] + lane * DPL;
        float vf[DPL];
        if constexpr (DPL == 4) {
          const uint2 vv = __ldg(reinterpret_cast<const uint2*>(vr));
          vf[0] = __uint_as_float(vv.x << 16);
          vf[1] = __uint_as_float(vv.x & 0xffff0000u);
          vf[2] = __uint_as_float(vv.y << 16);
          vf[3] = __uint_as_float(vv.y & 0xffff0000u);
        } else {
          const uint32_t vv = __ldg(reinterpret_cast<const uint32_t*>(vr));
          vf[0] = __uint_as_float(vv << 16);
          vf[1] = __uint_as_float(vv & 0xffff0000u);
        }
#pragma unroll
        for (int hh = 0; hh < GMAX; ++hh) {
          if (hh < G) {
            const float pj = __shfl_sync(0xffffffffu, pr[hh], j);
#pragma unroll
            for (int i = 0; i < DPL; ++i) o[hh][i] = fmaf(pj, vf[i], o[hh][i]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int hh = 0; hh < GMAX; ++hh) {
    if (hh < G) {
      const float inv = l[hh] > 0.f ? 1.f / l[hh] : 0.f;
      float* dst = p.o + ((static_cast<int64_t>(b) * p.Hq + g * G + hh) * p.Tq + t) * D + lane * DPL;
      if (p.gate != nullptr) {
        const float gl = p.gate[((static_cast<int64_t>(b) * p.Tq + t) * p.Hq + g * G + hh) * 3 + 1];
        const float gs = 1.f / (1.f + __expf(-gl));
#pragma unroll
        for (int i = 0; i < DPL; ++i) dst[i] = fmaf(gs, o[hh][i] * inv, dst[i]);
      } else {
#pragma unroll
        for (int i = 0; i < DPL; ++i) dst[i] = o[hh][i] * inv;
      }
    }
  }
}

// ---------------------------------------- selected attention on mma.sync tiles
// The same operator with the two products on warp-level tensor-core tiles (m16n8k16, bf16 in, fp32
// accumulate): the G <= 8 heads of the kv group are the rows of a 16-row tile (the other rows are
// zero), so one tile multiplies all heads of a query with 8 keys (scores) or 8 channels (output).
// tcgen05 tiles are 128 rows tall and would be 6 % used here; the limit of this kernel is the
// gather of the selected key / value rows from L2 anyway.  One warp per (b, g, t); keys in chunks
// of 16, copied with cp.async into a per-warp double buffer (rows padded to D*2 + 16 bytes so that
// ldmatrix reads are free of bank conflicts).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
// d += a (16x16, row) * b (16x8, col); the tile's rows 8..15 are zero: a1 = a3 = 0
__device__ __forceinline__ void mma_16816_top(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

template <int D>
__global__ void __launch_bounds__(128) nsa_selected_attn_mma_kernel(const NsaSelParams p) {
  constexpr int kRowBytes = D * 2 + 16;              // padded key / value row
  constexpr int kChunk = 16;                         // keys per step
  constexpr int kBufBytes = kChunk * kRowBytes;      // one K or V chunk
  extern __shared__ __align__(16) uint8_t sel_smem[];   // [4 warps][2 buffers][K chunk, V chunk]
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g4 = lane >> 2, t4 = lane & 3;           // fragment row / column-pair indices
  const int64_t wid = static_cast<int64_t>(blockIdx.x) * 4 + wib;
  const int64_t total = static_cast<int64_t>(p.B) * p.Hkv * p.Tq;
  if (wid >= total) return;
  const int t = static_cast<int>(wid % p.Tq);
  const int g = static_cast<int>((wid / p.Tq) % p.Hkv);
  const int b = static_cast<int>(wid / (static_cast<int64_t>(p.Tq) * p.Hkv));
  const int G = p.G;
  const uint32_t sbase = smem_u32(sel_smem) + wib * (4 * kBufBytes);
  const __nv_bfloat16* kbase = p.k + b * p.ks[0] + g * p.ks[1];
  const __nv_bfloat16* vbase = p.v + b * p.vs[0] + g * p.vs[1];
  const int32_t* blk = p.blocks + ((static_cast<int64_t>(b) * p.Hkv + g) * p.Tq + t) * p.n_sel;
  const float ninf = -__int_as_float(0x7f800000);

  // Q fragments: row g4 = head g4 of the group (zero for g4 >= G), 16 channels per k-step
  uint32_t qa0[D / 16], qa2[D / 16];
  {
    const __nv_bfloat16* qrow = p.q + b * p.qs[0] + (g * G + min(g4, G - 1)) * p.qs[1] + t * p.qs[2];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const uint32_t lo = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t4);
      const uint32_t hi = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t4);
      qa0[ks] = g4 < G ? lo : 0u;
      qa2[ks] = g4 < G ? hi : 0u;
    }
  }

  const int chunks_per_block = p.sel_block / kChunk;
  const int n_chunks = p.n_sel * chunks_per_block;
  // copies chunk c (16 key rows and 16 value rows) into buffer c & 1
  auto issue = [&](int c) {
    const int key0 = blk[c / chunks_per_block] * p.sel_block + (c % chunks_per_block) * kChunk;
    const uint32_t dst = sbase + (c & 1) * (2 * kBufBytes);
    constexpr int kPieces = kChunk * (D * 2 / 16);   // 16-byte pieces per chunk
#pragma unroll
    for (int i = 0; i < kPieces / 32; ++i) {
      const int piece = i * 32 + lane;
      const int r = piece / (D * 2 / 16), cpi = piece % (D * 2 / 16);
      const int key = min(key0 + r, p.Tk - 1);
      cp_async16(dst + r * kRowBytes + cpi * 16, kbase + static_cast<int64_t>(key) * p.ks[2] + cpi * 8);
      cp_async16(dst + kBufBytes + r * kRowBytes + cpi * 16, vbase + static_cast<int64_t>(key) * p.vs[2] + cpi * 8);
    }
    cp_async_commit();
  };

  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m = ninf, l = 0.f;

  issue(0);
  for (int c = 0; c < n_chunks; ++c) {
    if (c + 1 < n_chunks) {
      issue(c + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncwarp();
    const uint32_t kb = sbase + (c & 1) * (2 * kBufBytes);
    const uint32_t vb = kb + kBufBytes;
    const int key0 = blk[c / chunks_per_block] * p.sel_block + (c % chunks_per_block) * kChunk;

    // ---- scores: s[nt][0..1] = head g4 against keys key0 + 8*nt + 2*t4 (+1)
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      // four 8x8 matrices: (keys 0-7 | 8-15) x (channels 16ks..+7 | +8..+15)
      uint32_t kf[4];
      const int mat = lane >> 3, mr = lane & 7;
      ldmatrix_x4(kf, kb + ((mat >> 1) * 8 + mr) * kRowBytes + ks * 32 + (mat & 1) * 16);
      mma_16816_top(s[0], qa0[ks], qa2[ks], kf[0], kf[1]);
      mma_16816_top(s[1], qa0[ks], qa2[ks], kf[2], kf[3]);
    }
    // ---- online softmax of row g4 (log2 domain); the four lanes of a row hold 4 keys each
    float sv[4];
    float mx = ninf;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = key0 + nt * 8 + 2 * t4 + e;
        sv[nt * 2 + e] = key < p.Tk ? s[nt][e] * p.scale_log2 : ninf;
        mx = fmaxf(mx, sv[nt * 2 + e]);
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m, mx);
    const float alpha = (m == m_new) ? 1.f : ex2_approx(m - m_new);      // m_new = -inf only if m is too
    float pr[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) pr[e] = (m_new == ninf) ? 0.f : ex2_approx(sv[e] - m_new);
    l = l * alpha + (pr[0] + pr[1]) + (pr[2] + pr[3]);
    m = m_new;
    const uint32_t pa0 = pack_bf16x2(pr[0], pr[1]);   // keys 2*t4, +1 of the first eight
    const uint32_t pa2 = pack_bf16x2(pr[2], pr[3]);   // of the second eight
    // ---- O = O * alpha + P V
#pragma unroll
    for (int n2 = 0; n2 < D / 16; ++n2) {
      // four 8x8 matrices, transposed on load: (keys 0-7 | 8-15) x (channels 16*n2..+7 | +8..+15)
      uint32_t vf[4];
      const int mat = lane >> 3, mr = lane & 7;
      ldmatrix_x4_trans(vf, vb + ((mat & 1) * 8 + mr) * kRowBytes + n2 * 32 + (mat >> 1) * 16);
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        float (&acc)[4] = o[n2 * 2 + h2];
        acc[0] *= alpha;
        acc[1] *= alpha;
        mma_16816_top(acc, pa0, pa2, vf[h2 * 2], vf[h2 * 2 + 1]);
      }
    }
    __syncwarp();   // the buffer is refilled two chunks later
  }
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  if (g4 < G) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    float* dst = p.o + ((static_cast<int64_t>(b) * p.Hq + g * G + g4) * p.Tq + t) * D + 2 * t4;
    if (p.gate != nullptr) {
      const float gl = p.gate[((static_cast<int64_t>(b) * p.Tq + t) * p.Hq + g * G + g4) * 3 + 1];
      const float gs = 1.f / (1.f + __expf(-gl));
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        const float2 a = *reinterpret_cast<const float2*>(dst + n * 8);
        *reinterpret_cast<float2*>(dst + n * 8) = make_float2(fmaf(gs, o[n][0] * inv, a.x), fmaf(gs, o[n][1] * inv, a.y));
      }
    } else {
#pragma unroll
      for (int n = 0; n < D / 8; ++n) *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][0] * inv, o[n][1] * inv);
    }
  }
}

// ------------------------------------------------------------------ combine
// out[b,h,t,:] = sum_j sigmoid(gate[b,t,h,j]) * o_j[b,h,t,:], branches (B,Hq,T,D) fp32 contiguous.
__global__ void nsa_combine_kernel(const float* __restrict__ o_cmp, const float* __restrict__ o_sel,
                                   const float* __restrict__ o_win, const float* __restrict__ gate, void* out,
                                   int out_dtype, int B, int Hq, int T, int D) {
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(B) * Hq * T * D;
  if (gid >= total) return;
  const int64_t bht = gid / D;
  const int t = static_cast<int>(bht % T);
  const int h = static_cast<int>((bht / T) % Hq);
  const int b = static_cast<int>(bht / (static_cast<int64_t>(T) * Hq));
  const float* gp = gate + ((static_cast<int64_t>(b) * T + t) * Hq + h) * 3;
  const float g0 = 1.f / (1.f + __expf(-gp[0])), g1 = 1.f / (1.f + __expf(-gp[1])), g2 = 1.f / (1.f + __expf(-gp[2]));
  const float x = g0 * o_cmp[gid] + g1 * o_sel[gid] + g2 * o_win[gid];
  if (out_dtype == SWV_F32) static_cast<float*>(out)[gid] = x;
  else if (out_dtype == SWV_BF16) static_cast<__nv_bfloat16*>(out)[gid] = __float2bfloat16_rn(x);
  else static_cast<__half*>(out)[gid] = __float2half_rn(x);
}

// --------------------------------------------------------------------- host
static bool nsa_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int D, int R>
static int launch_importance(const CUtensorMap& tq, const CUtensorMap& tk, const NsaImpParams& p, cudaStream_t st) {
  using Cfg = NsaImpCfg<D>;
  SWV_CUDA_OK(cudaFuncSetAttribute(nsa_importance_kernel<D, R>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(Cfg::kSmem)));
  nsa_importance_kernel<D, R><<<static_cast<unsigned>(p.B) * p.Hkv * p.nQT, 320, Cfg::kSmem, st>>>(tq, tk, p);
  SWV_CUDA_OK(cudaGetLastError());
  return SWV_OK;
}

int nsa_importance_bytes_impl(int B, int Hkv, int Tq, int nC, int cmp_stride, int sel_block, size_t* bytes) {
  if (!bytes) return SWV_ERR_NULL;
  if (B < 1 || Hkv < 1 || Tq < 1 || nC < 1 || cmp_stride < 1 || sel_block < cmp_stride || sel_block % cmp_stride)
    return SWV_ERR_SHAPE;
  const int R = sel_block / cmp_stride;
  const size_t n_pad = static_cast<size_t>((nC + kTile - 1) / kTile) * (kTile / R);
  *bytes = static_cast<size_t>(B) * Hkv * Tq * n_pad * 4;
  return SWV_OK;
}

int nsa_select_blocks_impl(const void* q, const int64_t* qs, const void* kc, const int64_t* kcs, const float* lse,
                           int B, int Hq, int Hkv, int Tq, int Tk, int nC, int D, int cmp_stride, int sel_block,
                           int n_sel, float* importance, size_t importance_bytes, int32_t* blocks, int* status,
                           cudaStream_t st) {
  if (!q || !kc || !lse || !importance || !blocks || !status || !qs || !kcs) return SWV_ERR_NULL;
  if (B < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv || Tq < 1 || Tk < 1 || nC < 1 || n_sel < 1) return SWV_ERR_SHAPE;
  if (cmp_stride < 1 || sel_block < cmp_stride || sel_block % cmp_stride) return SWV_ERR_SHAPE;
  const int G = Hq / Hkv, R = sel_block / cmp_stride;
  if (G > kNsaMaxGroup || (D != 64 && D != 128) || (R != 1 && R != 2 && R != 4 && R != 8)) return SWV_ERR_UNSUPPORTED;
  size_t need = 0;
  nsa_importance_bytes_impl(B, Hkv, Tq, nC, cmp_stride, sel_block, &need);
  if (importance_bytes < need) return SWV_ERR_WORKSPACE;
  if (qs[3] != 1 || kcs[3] != 1 || !nsa_aligned16(q) || !nsa_aligned16(kc) || !nsa_aligned16(importance))
    return SWV_ERR_ALIGN;
  for (int i = 0; i < 3; ++i)
    if ((qs[i] * 2) % 16 || (kcs[i] * 2) % 16) return SWV_ERR_ALIGN;
  const int n_s = (Tk + sel_block - 1) / sel_block;
  const int k_eff = n_sel < n_s ? n_sel : n_s;

  CUtensorMap tq, tk;
  int rc = make_tmap_4d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, Tq, Hq, B, qs[2] * 2, qs[1] * 2, qs[0] * 2, 64,
                        kTile);
  if (rc != SWV_OK) return rc;
  rc = make_tmap_4d(&tk, kc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, nC, Hkv, B, kcs[2] * 2, kcs[1] * 2, kcs[0] * 2, 64,
                    kTile);
  if (rc != SWV_OK) return rc;

  NsaImpParams p;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.Tq = Tq; p.nC = nC;
  p.nQT = (Tq + kTile - 1) / kTile;
  p.nCT = (nC + kTile - 1) / kTile;
  p.n_pad = p.nCT * (kTile / R);
  p.lse = lse; p.imp = importance;
  p.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(D));
  p.status = status;
  if (D == 64) {
    if (R == 1) rc = launch_importance<64, 1>(tq, tk, p, st);
    else if (R == 2) rc = launch_importance<64, 2>(tq, tk, p, st);
    else if (R == 4) rc = launch_importance<64, 4>(tq, tk, p, st);
    else rc = launch_importance<64, 8>(tq, tk, p, st);
  } else {
    if (R == 1) rc = launch_importance<128, 1>(tq, tk, p, st);
    else if (R == 2) rc = launch_importance<128, 2>(tq, tk, p, st);
    else if (R == 4) rc = launch_importance<128, 4>(tq, tk, p, st);
    else rc = launch_importance<128, 8>(tq, tk, p, st);
  }
  if (rc != SWV_OK) return rc;

  const int64_t rows = static_cast<int64_t>(B) * Hkv * Tq;
  const int n = (n_s + 31) & ~31;
  const size_t sm = static_cast<size_t>(4) * n * 4;
  if (sm > 200 * 1024) return SWV_ERR_UNSUPPORTED;
  if (sm > 48 * 1024)
    SWV_CUDA_OK(cudaFuncSetAttribute(nsa_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(sm)));
  nsa_select_kernel<<<static_cast<unsigned>((rows + 3) / 4), 128, sm, st>>>(importance, p.n_pad, n_s, k_eff, rows,
                                                                            blocks);
  SWV_CUDA_OK(cudaGetLastError());
  return SWV_OK;
}

int nsa_selected_attn_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                           const int64_t* vs, const int32_t* blocks, int B, int Hq, int Hkv, int Tq, int Tk, int D,
                           int sel_block, int n_sel, float* o, cudaStream_t st, const float* gate) {
  if (!q || !k || !v || !blocks || !o || !qs || !ks || !vs) return SWV_ERR_NULL;
  if (B < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv || Tq < 1 || Tk < 1 || n_sel < 1) return SWV_ERR_SHAPE;
  if (sel_block < 32 || sel_block % 32) return SWV_ERR_UNSUPPORTED;
  const int G = Hq / Hkv;
  if (G > 8 || (D != 64 && D != 128)) return SWV_ERR_UNSUPPORTED;
  if (qs[3] != 1 || ks[3] != 1 || vs[3] != 1 || !nsa_aligned16(k) || !nsa_aligned16(v)) return SWV_ERR_ALIGN;
  for (int i = 0; i < 3; ++i)
    if ((ks[i] * 2) % 16 || (vs[i] * 2) % 16) return SWV_ERR_ALIGN;
  NsaSelParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  for (int i = 0; i < 4; ++i) { p.qs[i] = qs[i]; p.ks[i] = ks[i]; p.vs[i] = vs[i]; }
  p.blocks = blocks; p.o = o; p.gate = gate;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.Tq = Tq; p.Tk = Tk; p.n_sel = n_sel; p.sel_block = sel_block;
  p.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(D));
  const int64_t total = static_cast<int64_t>(B) * Hkv * Tq;
  const unsigned grid = static_cast<unsigned>((total + 3) / 4);
  // tensor-core tiles when the layout allows 16-byte row copies (the usual case), else CUDA cores
  const bool mma_ok = sel_block % 16 == 0 && nsa_aligned16(q) && (qs[0] * 2) % 4 == 0 && (qs[1] * 2) % 4 == 0 &&
                      (qs[2] * 2) % 4 == 0;
  if (mma_ok) {
    if (D == 64) {
      const size_t sm = 4 * 4 * 16 * (64 * 2 + 16);
      SWV_CUDA_OK(cudaFuncSetAttribute(nsa_selected_attn_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sm)));
      nsa_selected_attn_mma_kernel<64><<<grid, 128, sm, st>>>(p);
    } else {
      const size_t sm = 4 * 4 * 16 * (128 * 2 + 16);
      SWV_CUDA_OK(cudaFuncSetAttribute(nsa_selected_attn_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sm)));
      nsa_selected_attn_mma_kernel<128><<<grid, 128, sm, st>>>(p);
    }
  } else if (D == 64) {
    nsa_selected_attn_kernel<64, 8><<<grid, 128, 0, st>>>(p);
  } else {
    nsa_selected_attn_kernel<128, 8><<<grid, 128, 0, st>>>(p);
  }
  SWV_CUDA_OK(cudaGetLastError());
  return SWV_OK;
}

int nsa_combine_impl(const float* o_cmp, const float* o_sel, const float* o_win, const float* gate, void* out,
                     int out_dtype, int B, int Hq, int T, int D, cudaStream_t st) {
  if (!o_cmp || !o_sel || !o_win || !gate || !out) return SWV_ERR_NULL;
  if (B < 1 || Hq < 1 || T < 1 || D < 1) return SWV_ERR_SHAPE;
  if (out_dtype != SWV_F32 && out_dtype != SWV_BF16 && out_dtype != SWV_F16) return SWV_ERR_DTYPE;
  const int64_t total = static_cast<int64_t>(B) * Hq * T * D;
  nsa_combine_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(o_cmp, o_sel, o_win, gate, out,
                                                                                 out_dtype, B, Hq, T, D);
  SWV_CUDA_OK(cudaGetLastError());
  return SWV_OK;
}


// ------------------------------------------------------- whole forward pass
// Key-block lists of the two tensor-core branches, built on the device (one CTA):
//   compressed branch: every query block attends all `n_cb` blocks of compressed tokens;
//   window branch    : the 128-token blocks that intersect [q0 - reach, q1 + reach].
__global__ void nsa_build_lists_kernel(int n_qb, int n_cb, int T, int reach, int32_t* full_ptr, int32_t* full_col,
                                       int32_t* win_ptr, int32_t* win_col) {
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int i = 0; i < n_qb; ++i) {
      full_ptr[i] = i * n_cb;
      win_ptr[i] = acc;
      const int lo = max(0, i * kTile - reach) / kTile;
      const int hi = min(T - 1, min(T, (i + 1) * kTile) - 1 + reach) / kTile;
      acc += hi - lo + 1;
    }
    full_ptr[n_qb] = n_qb * n_cb;
    win_ptr[n_qb] = acc;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_qb * n_cb; i += blockDim.x) full_col[i] = i % n_cb;
  for (int i = threadIdx.x; i < n_qb; i += blockDim.x) {
    const int lo = max(0, i * kTile - reach) / kTile;
    const int n = win_ptr[i + 1] - win_ptr[i];
    for (int j = 0; j < n; ++j) win_col[win_ptr[i] + j] = lo + j;
  }
}

int pool_tokens_impl(const void* x, const int64_t* xs, void* y, int B, int H, int T, int D, int win, int stride,
                     cudaStream_t st);
int block_sparse_attn_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                           const int64_t* vs, const int32_t* row_ptr, const int32_t* col_idx, int block, int mode,
                           int num_cls, int window, int dilation, int kv_group, float* lse, void* o,
                           const int64_t* os, int o_dtype, int B, int H, int Tq, int Tk, int D, int* status,
                           cudaStream_t st, const float* gate, int gate_idx, const float* acc_in);

struct NsaLayout {
  size_t kc, vc, acc, lse, imp, blocks, full_ptr, full_col, win_ptr, win_col, total;
  int nC, n_qb, n_cb, k_eff, win_blocks;
};
static size_t nsa_up(size_t x) { return (x + 255) / 256 * 256; }
static int nsa_layout(int B, int Hq, int Hkv, int T, int D, int cmp_block, int cmp_stride, int sel_block, int n_sel,
                      int window, NsaLayout* L) {
  if (B < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv || T < cmp_block || cmp_block < 1 || cmp_stride < 1 || n_sel < 1 ||
      window < 0)
    return SWV_ERR_SHAPE;
  L->nC = (T - cmp_block) / cmp_stride + 1;
  L->n_qb = (T + kTile - 1) / kTile;
  L->n_cb = (L->nC + kTile - 1) / kTile;
  const int n_s = (T + sel_block - 1) / sel_block;
  L->k_eff = n_sel < n_s ? n_sel : n_s;
  L->win_blocks = 2 * ((window / 2 + kTile - 1) / kTile) + 2;
  size_t imp_bytes = 0;
  const int rc = nsa_importance_bytes_impl(B, Hkv, T, L->nC, cmp_stride, sel_block, &imp_bytes);
  if (rc != SWV_OK) return rc;
  size_t off = 0;
  const size_t branch = static_cast<size_t>(B) * Hq * T * D * 4;
  L->kc = off; off += nsa_up(static_cast<size_t>(B) * Hkv * L->nC * D * 2);
  L->vc = off; off += nsa_up(static_cast<size_t>(B) * Hkv * L->nC * D * 2);
  L->acc = off; off += nsa_up(branch);      // the running gated sum of the branches, fp32
  L->lse = off; off += nsa_up(static_cast<size_t>(B) * Hq * T * 4);
  L->imp = off; off += nsa_up(imp_bytes);
  L->blocks = off; off += nsa_up(static_cast<size_t>(B) * Hkv * T * L->k_eff * 4);
  L->full_ptr = off; off += nsa_up((L->n_qb + 1) * 4);
  L->full_col = off; off += nsa_up(static_cast<size_t>(L->n_qb) * L->n_cb * 4);
  L->win_ptr = off; off += nsa_up((L->n_qb + 1) * 4);
  L->win_col = off; off += nsa_up(static_cast<size_t>(L->n_qb) * L->win_blocks * 4);
  L->total = off;
  return SWV_OK;
}

int nsa_workspace_bytes_impl(int B, int Hq, int Hkv, int T, int D, int cmp_block, int cmp_stride, int sel_block,
                             int n_sel, int window, size_t* bytes) {
  if (!bytes) return SWV_ERR_NULL;
  NsaLayout L;
  const int rc = nsa_layout(B, Hq, Hkv, T, D, cmp_block, cmp_stride, sel_block, n_sel, window, &L);
  if (rc == SWV_OK) *bytes = L.total;
  return rc;
}

int nsa_attn_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                  const int64_t* vs, const float* gate, void* out, int out_dtype, int B, int Hq, int Hkv, int T,
                  int D, int cmp_block, int cmp_stride, int sel_block, int n_sel, int window, void* workspace,
                  size_t workspace_bytes, int32_t* blocks_out, int* status, cudaStream_t st) {
  if (!q || !k || !v || !gate || !out || !workspace || !status || !qs || !ks || !vs) return SWV_ERR_NULL;
  NsaLayout L;
  int rc = nsa_layout(B, Hq, Hkv, T, D, cmp_block, cmp_stride, sel_block, n_sel, window, &L);
  if (rc != SWV_OK) return rc;
  if (workspace_bytes < L.total) return SWV_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return SWV_ERR_ALIGN;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  void* kc = ws + L.kc;
  void* vc = ws + L.vc;
  float* acc = reinterpret_cast<float*>(ws + L.acc);
  float* lse = reinterpret_cast<float*>(ws + L.lse);
  float* imp = reinterpret_cast<float*>(ws + L.imp);
  int32_t* blocks = reinterpret_cast<int32_t*>(ws + L.blocks);
  int32_t* full_ptr = reinterpret_cast<int32_t*>(ws + L.full_ptr);
  int32_t* full_col = reinterpret_cast<int32_t*>(ws + L.full_col);
  int32_t* win_ptr = reinterpret_cast<int32_t*>(ws + L.win_ptr);
  int32_t* win_col = reinterpret_cast<int32_t*>(ws + L.win_col);
  const int G = Hq / Hkv;
  const int reach = window / 2;

  nsa_build_lists_kernel<<<1, 256, 0, st>>>(L.n_qb, L.n_cb, T, reach, full_ptr, full_col, win_ptr, win_col);
  SWV_CUDA_OK(cudaGetLastError());
  rc = pool_tokens_impl(k, ks, kc, B, Hkv, T, D, cmp_block, cmp_stride, st);
  if (rc != SWV_OK) return rc;
  rc = pool_tokens_impl(v, vs, vc, B, Hkv, T, D, cmp_block, cmp_stride, st);
  if (rc != SWV_OK) return rc;
  const int64_t cs[4] = {static_cast<int64_t>(Hkv) * L.nC * D, static_cast<int64_t>(L.nC) * D, D, 1};
  const int64_t os[4] = {static_cast<int64_t>(Hq) * T * D, static_cast<int64_t>(T) * D, D, 1};
  // The gate is applied in the branch epilogues: acc = s(g0) cmp; acc += s(g1) sel; out = acc + s(g2) win
  // (the order in which the stand-alone gate kernel adds them), so no branch output goes to HBM on
  // its own.
  // compressed branch (all compressed tokens, log-sum-exp kept for the selection)
  rc = block_sparse_attn_impl(q, qs, kc, cs, vc, cs, full_ptr, full_col, kTile, 0, 0, 0, 1, G, lse, acc, os,
                              SWV_F32, B, Hq, T, L.nC, D, status, st, gate, 0, nullptr);
  if (rc != SWV_OK) return rc;
  // selection + selected branch
  size_t imp_bytes = 0;
  nsa_importance_bytes_impl(B, Hkv, T, L.nC, cmp_stride, sel_block, &imp_bytes);
  rc = nsa_select_blocks_impl(q, qs, kc, cs, lse, B, Hq, Hkv, T, T, L.nC, D, cmp_stride, sel_block, n_sel, imp,
                              imp_bytes, blocks, status, st);
  if (rc != SWV_OK) return rc;
  rc = nsa_selected_attn_impl(q, qs, k, ks, v, vs, blocks, B, Hq, Hkv, T, T, D, sel_block, L.k_eff, acc, st, gate);
  if (rc != SWV_OK) return rc;
  // sliding-window branch: token pattern |i - j| <= window / 2 inside the listed blocks
  rc = block_sparse_attn_impl(q, qs, k, ks, v, vs, win_ptr, win_col, kTile, 1, 0, reach, 1, G, nullptr, out, os,
                              out_dtype, B, Hq, T, T, D, status, st, gate, 2, acc);
  if (rc != SWV_OK) return rc;
  if (blocks_out != nullptr)
    SWV_CUDA_OK(cudaMemcpyAsync(blocks_out, blocks, static_cast<size_t>(B) * Hkv * T * L.k_eff * 4,
                                cudaMemcpyDeviceToDevice, st));
  return SWV_OK;
}

}  // namespace swv
