// DSA top-k attention forward for sm_100a, dense-tile form.
//
// Replaces the reference's `_dsa_attention_fwd` Triton kernel
// (src/sparse_wsi_vit/models/deepseek_sparse_attention_kernels/kernels.py:450-564)
// for key lists produced by the indexer of this library.
//
// With per-query token-granular selection and one K/V per head, gathering the
// selected rows moves one byte per FLOP; at top_k/T >= ~1/64 it is faster to
// sweep ALL key tiles on the tensor cores and apply the selection inside the
// online softmax.  One CTA owns (batch, head, 128 queries):
//   warp 0      : TMA producer (Q once, K and V tiles through 2-deep rings)
//   warp 1      : UMMA issuer  S = Q K^T (bf16, fp32 accumulate in TMEM),
//                               O += P V  (P read from TMEM, V MN-major from smem)
//   warps 2..5  : softmax, one thread per query row.  Membership comes from the
//                 tile-major bitmask, the routing weight of the c-th selected key
//                 of a row is weights[row][c] (ascending key order).
//                   p = 2^(s*scale*log2e - m_used) * w      (members only)
//                 The exact maximum over the selected logits is tracked beside the
//                 (lazily raised) stabiliser m_used so that the reference's
//                 1e-6 clamp on the denominator is reproduced exactly.
// TMEM columns: S [0,128) fp32 | P [128,192) bf16x2 | O [192,256) fp32.
// Two CTAs share an SM (80 KiB smem, 256 TMEM columns each), so one CTA's MMAs
// overlap the other's softmax.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace swv {

constexpr int kHeadDim = 64;
constexpr int kQTileBytes = kTile * kHeadDim * 2;   // 16 KiB bf16 tile
constexpr int kAttnTmemCols = 256;
constexpr uint32_t kColS = 0, kColP = 128, kColO = 192;
constexpr float kRescaleStep = 8.0f;                // raise the stabiliser only in steps of 2^8

struct AttnParams {
  int B, H, Tq, Tk, top_k, nQT, nKT;
  const uint32_t* maskbits;
  const float* weights;
  void* o;
  int64_t osb, osh, ost;
  int o_dtype;
  float scale_log2;
  int* status;
};

struct AttnCtl {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full, s_free, p_full, pv_done;
  uint32_t tmem_base;
  uint32_t abort_flag;
};

constexpr size_t attn_smem_bytes() { return 1024 + kQTileBytes * 5 + sizeof(AttnCtl) + 64; }

__global__ void __launch_bounds__(192, 2)
    dsa_attn_masked_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                           const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  constexpr uint32_t kIdescQK = make_idesc(/*bf16*/ 1, kTile, kTile, 0, 0);
  constexpr uint32_t kIdescPV = make_idesc(/*bf16*/ 1, kTile, kHeadDim, 0, /*V is MN-major*/ 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sm_q = smem;
  uint8_t* sm_k = smem + kQTileBytes;
  uint8_t* sm_v = smem + kQTileBytes * 3;
  AttnCtl* ctl = reinterpret_cast<AttnCtl*>(smem + kQTileBytes * 5);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int h = blockIdx.x % p.H;
  const int qt = (blockIdx.x / p.H) % p.nQT;
  const int b = blockIdx.x / (p.H * p.nQT);
  const int nKT = p.nKT;

  if (threadIdx.x == 0) {
    mbar_init(&ctl->q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl->k_full[s], 1);
      mbar_init(&ctl->k_empty[s], 1);
      mbar_init(&ctl->v_full[s], 1);
      mbar_init(&ctl->v_empty[s], 1);
    }
    mbar_init(&ctl->s_full, 1);
    mbar_init(&ctl->s_free, 4);
    mbar_init(&ctl->p_full, 4);
    mbar_init(&ctl->pv_done, 1);
    ctl->abort_flag = 0;
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
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_expect_tx(&ctl->q_full, kQTileBytes);
      tma_load_4d(sm_q, &tm_q, &ctl->q_full, 0, qt * kTile, h, b);
      for (int j = 0; j < nKT; ++j) {
        const int s = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait_bounded(&ctl->k_empty[s], par, abort_flag)) {
          record_status(p.status, kDevWaitStageEmpty);
          break;
        }
        mbar_expect_tx(&ctl->k_full[s], kQTileBytes);
        tma_load_4d(sm_k + s * kQTileBytes, &tm_k, &ctl->k_full[s], 0, j * kTile, h, b);
        if (!mbar_wait_bounded(&ctl->v_empty[s], par, abort_flag)) {
          record_status(p.status, kDevWaitStageEmpty);
          break;
        }
        mbar_expect_tx(&ctl->v_full[s], kQTileBytes);
        tma_load_4d(sm_v + s * kQTileBytes, &tm_v, &ctl->v_full[s], 0, j * kTile, h, b);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t q_addr = smem_u32(sm_q);
      const uint32_t k_addr = smem_u32(sm_k);
      const uint32_t v_addr = smem_u32(sm_v);
      bool ok = mbar_wait_bounded(&ctl->q_full, 0, abort_flag);
      if (!ok) record_status(p.status, kDevWaitQ);

      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait_bounded(&ctl->k_full[s], (j >> 1) & 1, abort_flag)) {
          record_status(p.status, kDevWaitTmaFull);
          return false;
        }
        if (j > 0 && !mbar_wait_bounded(&ctl->s_free, (j - 1) & 1, abort_flag)) {
          record_status(p.status, kDevWaitAccEmpty);
          return false;
        }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          umma_f16_ss(tmem_base + kColS, smem_desc_sw128(q_addr + ks * 32),
                      smem_desc_sw128(k_addr + s * kQTileBytes + ks * 32), kIdescQK, ks > 0);
        }
        umma_commit(&ctl->k_empty[s]);
        umma_commit(&ctl->s_full);
        return true;
      };

      if (ok) ok = issue_qk(0);
      for (int j = 0; ok && j < nKT; ++j) {
        if (j + 1 < nKT) {
          ok = issue_qk(j + 1);
          if (!ok) break;
        }
        const int s = j & 1;
        if (!mbar_wait_bounded(&ctl->v_full[s], (j >> 1) & 1, abort_flag)) {
          record_status(p.status, kDevWaitTmaFull);
          break;
        }
        if (!mbar_wait_bounded(&ctl->p_full, j & 1, abort_flag)) {
          record_status(p.status, kDevWaitPReady);
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          // 16 keys per step: 8 packed TMEM columns of P, 16 rows (2 KiB) of the V tile
          umma_f16_ts(tmem_base + kColO, tmem_base + kColP + ks * 8,
                      smem_desc_sw128(v_addr + s * kQTileBytes + ks * 2048), kIdescPV, (j > 0 || ks > 0));
        }
        umma_commit(&ctl->v_empty[s]);
        umma_commit(&ctl->pv_done);
      }
    }
  } else {
    // ----------------------------------------------------------------- softmax
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int qrow = qt * kTile + row;
    const bool row_ok = qrow < p.Tq;
    const int64_t grow = static_cast<int64_t>(b) * p.Tq + (row_ok ? qrow : 0);
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const float* wrow = p.weights + grow * p.top_k;
    const uint4* mask_tile =
        reinterpret_cast<const uint4*>(p.maskbits) + (static_cast<int64_t>(b) * p.nQT + qt) * nKT * kTile + row;
    const float sc = p.scale_log2;
    const float ninf = -__int_as_float(0x7f800000);

    float m_true = ninf, m_used = ninf, l = 0.f;
    int cnt = 0;
    bool ok = true;
    uint4 mw = __ldg(mask_tile);

    for (int j = 0; j < nKT; ++j) {
      uint4 mw_next = make_uint4(0, 0, 0, 0);
      if (j + 1 < nKT) mw_next = __ldg(mask_tile + static_cast<int64_t>(j + 1) * kTile);
      if (!mbar_wait_bounded(&ctl->s_full, j & 1, abort_flag)) {
        record_status(p.status, kDevWaitAccFull);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t words[4] = {mw.x, mw.y, mw.z, mw.w};

      // pass 1: maximum over the selected logits of this tile
      float mt = ninf;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(lane_base + kColS + c * 32, r);
        tc_wait_ld();
        const uint32_t w = words[c];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (w & (1u << i)) mt = fmaxf(mt, __uint_as_float(r[i]));
        }
      }
      m_true = fmaxf(m_true, mt * sc);
      const bool need = m_true > m_used + kRescaleStep;
      const bool any = __any_sync(0xffffffffu, need);
      float factor = 1.f;
      if (any) {
        factor = (m_true == m_used) ? 1.f : ex2_approx(m_used - m_true);
        m_used = m_true;
        l *= factor;
      }
      if (j > 0) {
        if (!mbar_wait_bounded(&ctl->pv_done, (j - 1) & 1, abort_flag)) {
          record_status(p.status, kDevWaitPvDone);
          ok = false;
          break;
        }
        tc_fence_after();
        if (any) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t r[32];
            tmem_ld32(lane_base + kColO + c * 32, r);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
            tmem_st32(lane_base + kColO + c * 32, r);
          }
          tc_wait_st();
        }
      }

      // pass 2: probabilities of the selected keys, routing-weighted, to TMEM as bf16
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(lane_base + kColS + c * 32, r);
        tc_wait_ld();
        if (c == 3) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->s_free);
        }
        const uint32_t w = words[c];
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = 0.f, p1 = 0.f;
          if (w & (1u << i)) {
            const float wt = __ldg(wrow + cnt);
            ++cnt;
            p0 = ex2_approx(fmaf(__uint_as_float(r[i]), sc, -m_used)) * wt;
            l += p0;
          }
          if (w & (2u << i)) {
            const float wt = __ldg(wrow + cnt);
            ++cnt;
            p1 = ex2_approx(fmaf(__uint_as_float(r[i + 1]), sc, -m_used)) * wt;
            l += p1;
          }
          packed[i >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st16(lane_base + kColP + c * 16, packed);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->p_full);
      mw = mw_next;
    }

    if (ok) {
      if (!mbar_wait_bounded(&ctl->pv_done, (nKT - 1) & 1, abort_flag)) {
        record_status(p.status, kDevWaitPvDone);
        ok = false;
      }
    }
    if (ok) {
      tc_fence_after();
      const float corr = (m_used == m_true) ? 1.f : ex2_approx(m_used - m_true);
      const float inv = corr / fmaxf(l * corr, 1e-6f);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(lane_base + kColO + c * 32, r);
        tc_wait_ld();
        if (row_ok) {
          if (p.o_dtype == SWV_F32) {
            float* orow = static_cast<float*>(p.o) + b * p.osb + h * p.osh + qrow * p.ost + c * 32;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              float4 v4 = make_float4(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv,
                                      __uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
              *reinterpret_cast<float4*>(orow + i) = v4;
            }
          } else {
            uint16_t* orow = static_cast<uint16_t*>(p.o) + b * p.osb + h * p.osh + qrow * p.ost + c * 32;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint32_t w4[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float a0 = __uint_as_float(r[i + 2 * q]) * inv;
                const float a1 = __uint_as_float(r[i + 2 * q + 1]) * inv;
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
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, kAttnTmemCols);
  }
}

// ------------------------------------------------------------- gather kernel
// One warp per (batch, head, query).  Lanes split the key slots for q.k, then the
// head dimension for the weighted sum over V.  fp32 throughout; any index list.
struct GatherParams {
  const void *q, *k, *v;
  int64_t qs[4], ks[4], vs[4];
  const int32_t* idx;
  const float* valid;
  const float* rw;
  int64_t is[3], vls[3], rs[3];
  void* o;
  int64_t os[4];
  int o_dtype;
  int B, H, Tq, Tk, D, top_k;
  float scale;
};

template <typename T>
__device__ __forceinline__ float ld_f32(const T* p);
template <>
__device__ __forceinline__ float ld_f32<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <>
__device__ __forceinline__ float ld_f32<__half>(const __half* p) { return __half2float(*p); }

__device__ __forceinline__ void st_out(void* o, int dtype, int64_t off, float x) {
  if (dtype == SWV_F32) static_cast<float*>(o)[off] = x;
  else if (dtype == SWV_BF16) static_cast<__nv_bfloat16*>(o)[off] = __float2bfloat16_rn(x);
  else static_cast<__half*>(o)[off] = __float2half_rn(x);
}

// DPL = head-dim elements per lane in the PV phase; handles any D <= 32*DPL.
template <typename T, int DPL>
__global__ void __launch_bounds__(128) dsa_attn_gather_kernel(const GatherParams p) {
  constexpr int DMAX = 32 * DPL;
  __shared__ float qsm[4][DMAX];
  const int D = p.D;
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t wid = static_cast<int64_t>(blockIdx.x) * 4 + wib;
  const int64_t total = static_cast<int64_t>(p.B) * p.H * p.Tq;
  if (wid >= total) return;
  const int qi = static_cast<int>(wid % p.Tq);
  const int h = static_cast<int>((wid / p.Tq) % p.H);
  const int b = static_cast<int>(wid / (static_cast<int64_t>(p.Tq) * p.H));

  const T* qrow = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1] + qi * p.qs[2];
  for (int d = lane; d < D; d += 32) qsm[wib][d] = ld_f32<T>(qrow + d * p.qs[3]);
  __syncwarp();

  const T* kbase = static_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
  const T* vbase = static_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];
  const int32_t* idx_row = p.idx + b * p.is[0] + qi * p.is[1];
  const float* val_row = p.valid + b * p.vls[0] + qi * p.vls[1];
  const float* rw_row = p.rw + b * p.rs[0] + qi * p.rs[1];
  const float ninf = -__int_as_float(0x7f800000);

  float o[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) o[i] = 0.f;
  float m = ninf, l = 0.f;

  for (int s0 = 0; s0 < p.top_k; s0 += 32) {
    const int slot = s0 + lane;
    const bool in = slot < p.top_k;
    int id = 0;
    float w = 0.f;
    bool ok = false;
    if (in) {
      id = idx_row[slot * p.is[2]];
      ok = val_row[slot * p.vls[2]] > 0.f;
      w = rw_row[slot * p.rs[2]];
    }
    id = min(max(id, 0), p.Tk - 1);
    float logit = ninf;
    if (ok) {
      const T* kr = kbase + static_cast<int64_t>(id) * p.ks[2];
      float acc = 0.f;
#pragma unroll 4
      for (int d = 0; d < D; ++d) acc = fmaf(qsm[wib][d], ld_f32<T>(kr + d * p.ks[3]), acc);
      logit = acc * p.scale;
    }
    float gm = logit;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, off));
    const float m_new = fmaxf(m, gm);
    if (m_new == ninf) continue;   // no valid slot so far (uniform across the warp)
    const float alpha = (m == m_new) ? 1.f : expf(m - m_new);
    float pj = ok ? expf(logit - m_new) * w : 0.f;
    float ps = pj;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
    l = l * alpha + ps;
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] *= alpha;
    for (int j = 0; j < 32; ++j) {
      const float pp = __shfl_sync(0xffffffffu, pj, j);
      const int ii = __shfl_sync(0xffffffffu, id, j);
      if (pp != 0.f) {
        const T* vr = vbase + static_cast<int64_t>(ii) * p.vs[2];
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          const int d = lane * DPL + i;
          if (d < D) o[i] = fmaf(pp, ld_f32<T>(vr + d * p.vs[3]), o[i]);
        }
      }
    }
    m = m_new;
  }
  const float inv = 1.f / fmaxf(l, 1e-6f);
  const int64_t obase = b * p.os[0] + h * p.os[1] + qi * p.os[2];
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane * DPL + i;
    if (d < D) st_out(p.o, p.o_dtype, obase + d * p.os[3], o[i] * inv);
  }
}

// ---------------------------------------------------------------------- host
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int dsa_attn_masked_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                         const int64_t* vs, const uint32_t* maskbits, const float* weights, int top_k, void* o,
                         const int64_t* os, int o_dtype, int B, int H, int Tq, int Tk, int D, int* status,
                         cudaStream_t st) {
  if (!q || !k || !v || !maskbits || !weights || !o || !status || !qs || !ks || !vs || !os) return SWV_ERR_NULL;
  if (B < 1 || H < 1 || Tq < 1 || Tk < 1 || top_k < 1) return SWV_ERR_SHAPE;
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
  if (!aligned16(maskbits) || (reinterpret_cast<uintptr_t>(weights) & 3)) return SWV_ERR_ALIGN;

  CUtensorMap tm_q, tm_k, tm_v;
  int rc = make_tmap_4d(&tm_q, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, Tq, H, B, qs[2] * 2, qs[1] * 2, qs[0] * 2,
                        kHeadDim, kTile);
  if (rc != SWV_OK) return rc;
  rc = make_tmap_4d(&tm_k, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, Tk, H, B, ks[2] * 2, ks[1] * 2, ks[0] * 2,
                    kHeadDim, kTile);
  if (rc != SWV_OK) return rc;
  rc = make_tmap_4d(&tm_v, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, Tk, H, B, vs[2] * 2, vs[1] * 2, vs[0] * 2,
                    kHeadDim, kTile);
  if (rc != SWV_OK) return rc;

  AttnParams p;
  p.B = B; p.H = H; p.Tq = Tq; p.Tk = Tk; p.top_k = top_k;
  p.nQT = (Tq + kTile - 1) / kTile;
  p.nKT = (Tk + kTile - 1) / kTile;
  p.maskbits = maskbits; p.weights = weights;
  p.o = o; p.osb = os[0]; p.osh = os[1]; p.ost = os[2]; p.o_dtype = o_dtype;
  p.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(D));
  p.status = status;

  SWV_CUDA_OK(cudaFuncSetAttribute(dsa_attn_masked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(attn_smem_bytes())));
  const unsigned grid = static_cast<unsigned>(B) * p.nQT * H;
  dsa_attn_masked_kernel<<<grid, 192, attn_smem_bytes(), st>>>(tm_q, tm_k, tm_v, p);
  SWV_CUDA_OK(cudaGetLastError());
  return SWV_OK;
}

template <typename T>
static int launch_gather(const GatherParams& p, int D, cudaStream_t st) {
  const int64_t total = static_cast<int64_t>(p.B) * p.H * p.Tq;
  const unsigned grid = static_cast<unsigned>((total + 3) / 4);
  if (D <= 32) dsa_attn_gather_kernel<T, 1><<<grid, 128, 0, st>>>(p);
  else if (D <= 64) dsa_attn_gather_kernel<T, 2><<<grid, 128, 0, st>>>(p);
  else if (D <= 128) dsa_attn_gather_kernel<T, 4><<<grid, 128, 0, st>>>(p);
  else if (D <= 256) dsa_attn_gather_kernel<T, 8><<<grid, 128, 0, st>>>(p);
  else return SWV_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? SWV_OK : SWV_ERR_CUDA;
}

int dsa_attn_gather_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                         const int64_t* vs, int dtype, const int32_t* idx, const int64_t* is, const float* valid,
                         const int64_t* vls, const float* rw, const int64_t* rs, void* o, const int64_t* os,
                         int o_dtype, int B, int H, int Tq, int Tk, int D, int top_k, int* status,
                         cudaStream_t st) {
  if (!q || !k || !v || !idx || !valid || !rw || !o || !status || !qs || !ks || !vs || !is || !vls || !rs || !os)
    return SWV_ERR_NULL;
  if (B < 1 || H < 1 || Tq < 1 || Tk < 1 || top_k < 1) return SWV_ERR_SHAPE;
  if (dtype != SWV_F32 && dtype != SWV_BF16 && dtype != SWV_F16) return SWV_ERR_DTYPE;
  if (o_dtype != SWV_F32 && o_dtype != SWV_BF16 && o_dtype != SWV_F16) return SWV_ERR_DTYPE;
  if (D < 1 || D > 256) return SWV_ERR_UNSUPPORTED;
  GatherParams p;
  p.q = q; p.k = k; p.v = v; p.idx = idx; p.valid = valid; p.rw = rw; p.o = o; p.o_dtype = o_dtype;
  for (int i = 0; i < 4; ++i) { p.qs[i] = qs[i]; p.ks[i] = ks[i]; p.vs[i] = vs[i]; p.os[i] = os[i]; }
  for (int i = 0; i < 3; ++i) { p.is[i] = is[i]; p.vls[i] = vls[i]; p.rs[i] = rs[i]; }
  p.B = B; p.H = H; p.Tq = Tq; p.Tk = Tk; p.D = D; p.top_k = top_k;
  p.scale = 1.0f / sqrtf(static_cast<float>(D));
  if (dtype == SWV_F32) return launch_gather<float>(p, D, st);
  if (dtype == SWV_BF16) return launch_gather<__nv_bfloat16>(p, D, st);
  return launch_gather<__half>(p, D, st);
}

}  // namespace swv
