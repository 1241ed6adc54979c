// Backward of the DSA path for sm_100a: gradients of the routing-weighted top-k attention and of
// the lightning indexer, as the reference's backward kernels define them
// (src/sparse_wsi_vit/models/deepseek_sparse_attention_kernels/kernels.py:
//  `_dsa_attention_bwd` :569-762 launched by DSAAttentionFunction.backward :812-853;
//  `_indexer_bwd_dQ/dK/dW` :128-339 launched by LightningIndexerFunction.backward :388-445).
//
// Both are gather / scatter work over the per-query key lists (one byte moved per FLOP, nothing
// for the tensor cores): one warp owns a query row, reads the selected key / value rows through
// 16-byte loads, keeps the row's logits in shared memory between the statistics pass and the
// gradient pass, and scatters dK / dV with vector reductions (red.global.add.v2.f32) into fp32
// accumulators.  Where the reference accumulates dK / dV with atomics in the storage dtype of k
// and v, the accumulators here are fp32 and the caller rounds once at the end.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "common.cuh"

namespace swv {

template <typename T>
__device__ __forceinline__ float bw_f32(T x);
template <>
__device__ __forceinline__ float bw_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float bw_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float bw_f32<__half>(__half x) { return __half2float(x); }

__device__ __forceinline__ void red_add_v2(float* p, float a, float b) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(a), "f"(b) : "memory");
}

// dot(x[0..D), row[0..D)) with the row read by ONE lane, unit stride
template <typename T>
__device__ __forceinline__ float row_dot(const float* __restrict__ x, const T* __restrict__ row, int D) {
  float acc = 0.f;
  if constexpr (sizeof(T) == 2) {
    if ((D & 7) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
      const uint4* r4 = reinterpret_cast<const uint4*>(row);
      for (int i = 0; i < D / 8; ++i) {
        const uint4 v = __ldg(r4 + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float lo, hi;
          if constexpr (std::is_same<T, __nv_bfloat16>::value) {
            lo = __uint_as_float(w[c] << 16);
            hi = __uint_as_float(w[c] & 0xffff0000u);
          } else {
            const __half2 h2 = *reinterpret_cast<const __half2*>(&w[c]);
            lo = __low2float(h2);
            hi = __high2float(h2);
          }
          acc = fmaf(x[i * 8 + 2 * c], lo, acc);
          acc = fmaf(x[i * 8 + 2 * c + 1], hi, acc);
        }
      }
      return acc;
    }
  } else {
    if ((D & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
      const float4* r4 = reinterpret_cast<const float4*>(row);
      for (int i = 0; i < D / 4; ++i) {
        const float4 v = __ldg(r4 + i);
        acc = fmaf(x[i * 4], v.x, fmaf(x[i * 4 + 1], v.y, fmaf(x[i * 4 + 2], v.z, fmaf(x[i * 4 + 3], v.w, acc))));
      }
      return acc;
    }
  }
  for (int d = 0; d < D; ++d) acc = fmaf(x[d], bw_f32<T>(row[d]), acc);
  return acc;
}

// ------------------------------------------------------------------ attention backward
struct AttnBwdParams {
  const void *d_out, *q, *k, *v, *o;
  int64_t dos[4], qs[4], ks[4], vs[4], os[4];
  const int32_t* idx;
  const float *valid, *rw;
  int64_t is[3], vls[3], rs[3];
  float *dq, *dk, *dv, *drw;      // fp32 contiguous: (B,H,Tq,D), (B,H,Tk,D), (B,H,Tk,D), (B,Tq,K)
  int B, H, Tq, Tk, D, top_k;
  float scale;
  int* status;
};

constexpr int kBwdWarps = 4;

// One warp per (batch, head, query).  DPL = head-dim elements per lane (pairs of adjacent
// channels, so that the scatter uses 8-byte vector reductions); D <= 32 * DPL.
// Shared memory per warp: q row, dO row (fp32) and, when CACHE, the row's top_k logits.
template <typename T, typename TO, int DPL, bool CACHE>
__global__ void __launch_bounds__(32 * kBwdWarps) dsa_attn_bwd_kernel(const AttnBwdParams p) {
  constexpr int DMAX = 32 * DPL;
  extern __shared__ float bw_smem[];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qsm = bw_smem + wib * (2 * DMAX + (CACHE ? p.top_k : 0));
  float* dosm = qsm + DMAX;
  float* lsm = dosm + DMAX;
  const int64_t wid = static_cast<int64_t>(blockIdx.x) * kBwdWarps + wib;
  const int64_t total = static_cast<int64_t>(p.B) * p.H * p.Tq;
  if (wid >= total) return;
  const int D = p.D;
  const int qi = static_cast<int>(wid % p.Tq);
  const int h = static_cast<int>((wid / p.Tq) % p.H);
  const int b = static_cast<int>(wid / (static_cast<int64_t>(p.Tq) * p.H));

  const T* qrow = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1] + qi * p.qs[2];
  const TO* dorow = static_cast<const TO*>(p.d_out) + b * p.dos[0] + h * p.dos[1] + qi * p.dos[2];
  const TO* orow = static_cast<const TO*>(p.o) + b * p.os[0] + h * p.os[1] + qi * p.os[2];
  float di = 0.f;                                        // Di = sum_d dO * O   (K:641-656)
  for (int d = lane; d < DMAX; d += 32) {
    const bool in = d < D;
    const float dov = in ? bw_f32<TO>(dorow[d * p.dos[3]]) : 0.f;
    qsm[d] = in ? bw_f32<T>(qrow[d * p.qs[3]]) : 0.f;
    dosm[d] = dov;
    if (in) di = fmaf(dov, bw_f32<TO>(orow[d * p.os[3]]), di);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) di += __shfl_xor_sync(0xffffffffu, di, off);
  __syncwarp();

  const T* kbase = static_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
  const T* vbase = static_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];
  const int32_t* idx_row = p.idx + b * p.is[0] + qi * p.is[1];
  const float* val_row = p.valid + b * p.vls[0] + qi * p.vls[1];
  const float* rw_row = p.rw + b * p.rs[0] + qi * p.rs[1];
  const float ninf = -__int_as_float(0x7f800000);

  // slot -> (key index, valid, logit); an index outside [0, Tk) is reported and the slot dropped
  auto slot_logit = [&](int slot, int& id, bool& ok) -> float {
    id = 0;
    ok = false;
    if (slot < p.top_k) {
      id = idx_row[slot * p.is[2]];
      ok = val_row[slot * p.vls[2]] > 0.f;
      if (ok && (id < 0 || id >= p.Tk)) {
        record_status(p.status, kDevBadIndex);
        ok = false;
      }
    }
    if (!ok) return ninf;
    return row_dot<T>(qsm, kbase + static_cast<int64_t>(id) * p.ks[2], D) * p.scale;
  };

  // ---- pass 1: row maximum m and l = sum exp(logit - m) * rw   (K:596-637)
  float m = ninf;
  for (int s0 = 0; s0 < p.top_k; s0 += 32) {
    int id;
    bool ok;
    const float logit = slot_logit(s0 + lane, id, ok);
    if (CACHE && s0 + lane < p.top_k) lsm[s0 + lane] = logit;
    m = fmaxf(m, logit);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  __syncwarp();
  float* dq_row = p.dq + ((static_cast<int64_t>(b) * p.H + h) * p.Tq + qi) * D;
  if (m == ninf) {                                         // no valid slot: every gradient of the row is zero
    for (int d = lane; d < D; d += 32) dq_row[d] = 0.f;
    return;
  }
  float l = 0.f;
  for (int s0 = 0; s0 < p.top_k; s0 += 32) {
    const int slot = s0 + lane;
    float logit = ninf;
    if (CACHE) {
      if (slot < p.top_k) logit = lsm[slot];
    } else {
      int id;
      bool ok;
      logit = slot_logit(slot, id, ok);
    }
    if (logit != ninf) l = fmaf(__expf(logit - m), rw_row[slot * p.rs[2]], l);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
  const float inv_l = 1.f / fmaxf(l, 1e-6f);                // l_safe (K:637)

  // ---- pass 2: gradients   (K:659-748)
  float dq_acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) dq_acc[i] = 0.f;
  float* dk_base = p.dk + (static_cast<int64_t>(b) * p.H + h) * p.Tk * D;
  float* dv_base = p.dv + (static_cast<int64_t>(b) * p.H + h) * p.Tk * D;
  float* drw_row = p.drw + (static_cast<int64_t>(b) * p.Tq + qi) * p.top_k;
  for (int s0 = 0; s0 < p.top_k; s0 += 32) {
    const int slot = s0 + lane;
    int id = 0;
    bool ok = false;
    float logit = ninf;
    if (CACHE) {
      if (slot < p.top_k) {
        logit = lsm[slot];
        id = idx_row[slot * p.is[2]];
        ok = logit != ninf;
      }
    } else {
      logit = slot_logit(slot, id, ok);
    }
    float ds = 0.f, pv = 0.f;
    if (ok) {
      const float w = rw_row[slot * p.rs[2]];
      const float sm = __expf(logit - m) * inv_l;                                   // K:677
      const float dp = row_dot<T>(dosm, vbase + static_cast<int64_t>(id) * p.vs[2], D);   // K:693
      const float g = sm * (dp - di);
      atomicAdd(drw_row + slot, g);                                                 // summed over heads (K:702-708)
      ds = w * g * p.scale;                                                         // K:710
      pv = sm * w;                                                                  // K:678, :697
    }
    const unsigned any = __ballot_sync(0xffffffffu, ok && (ds != 0.f || pv != 0.f));
    for (unsigned rest = any; rest != 0u; rest &= rest - 1u) {
      const int j = __ffs(rest) - 1;
      const float dsj = __shfl_sync(0xffffffffu, ds, j);
      const float pvj = __shfl_sync(0xffffffffu, pv, j);
      const int idj = __shfl_sync(0xffffffffu, id, j);
      const T* kr = kbase + static_cast<int64_t>(idj) * p.ks[2];
      float* dkr = dk_base + static_cast<int64_t>(idj) * D;
      float* dvr = dv_base + static_cast<int64_t>(idj) * D;
#pragma unroll
      for (int i = 0; i < DPL; i += 2) {
        const int d = lane * 2 + i * 32;                  // channels (d, d+1) of this lane's i-th pair
        if (d + 1 < D) {
          const float k0 = bw_f32<T>(kr[d]), k1 = bw_f32<T>(kr[d + 1]);
          dq_acc[i] = fmaf(dsj, k0, dq_acc[i]);           // K:735-741
          dq_acc[i + 1] = fmaf(dsj, k1, dq_acc[i + 1]);
          red_add_v2(dkr + d, dsj * qsm[d], dsj * qsm[d + 1]);          // K:742-748
          red_add_v2(dvr + d, pvj * dosm[d], pvj * dosm[d + 1]);        // K:694-700
        } else if (d < D) {
          dq_acc[i] = fmaf(dsj, bw_f32<T>(kr[d]), dq_acc[i]);
          atomicAdd(dkr + d, dsj * qsm[d]);
          atomicAdd(dvr + d, pvj * dosm[d]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < DPL; i += 2) {
    const int d = lane * 2 + i * 32;
    if (d < D) dq_row[d] = dq_acc[i];
    if (d + 1 < D) dq_row[d + 1] = dq_acc[i + 1];
  }
}

template <typename T, typename TO>
static int launch_attn_bwd(const AttnBwdParams& p, cudaStream_t st) {
  const int64_t total = static_cast<int64_t>(p.B) * p.H * p.Tq;
  const unsigned grid = static_cast<unsigned>((total + kBwdWarps - 1) / kBwdWarps);
  const int dpl = p.D <= 64 ? 2 : (p.D <= 128 ? 4 : 8);
  const bool cache = p.top_k <= 4096;
  const size_t smem = static_cast<size_t>(kBwdWarps) * (2 * 32 * dpl + (cache ? p.top_k : 0)) * sizeof(float);
#define SWV_BWD_LAUNCH(DPL_, CACHE_)                                                                      \
  do {                                                                                                    \
    if (smem > 48 * 1024)                                                                                 \
      SWV_CUDA_OK(cudaFuncSetAttribute(dsa_attn_bwd_kernel<T, TO, DPL_, CACHE_>,                          \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))); \
    dsa_attn_bwd_kernel<T, TO, DPL_, CACHE_><<<grid, 32 * kBwdWarps, smem, st>>>(p);                      \
  } while (0)
  if (cache) {
    if (dpl == 2) SWV_BWD_LAUNCH(2, true);
    else if (dpl == 4) SWV_BWD_LAUNCH(4, true);
    else SWV_BWD_LAUNCH(8, true);
  } else {
    if (dpl == 2) SWV_BWD_LAUNCH(2, false);
    else if (dpl == 4) SWV_BWD_LAUNCH(4, false);
    else SWV_BWD_LAUNCH(8, false);
  }
#undef SWV_BWD_LAUNCH
  return cudaGetLastError() == cudaSuccess ? SWV_OK : SWV_ERR_CUDA;
}

int dsa_attn_bwd_impl(const void* d_out, const int64_t* dos, const void* q, const int64_t* qs, const void* k,
                      const int64_t* ks, const void* v, const int64_t* vs, int dtype, const void* o,
                      const int64_t* os, int o_dtype, const int32_t* idx, const int64_t* is, const float* valid,
                      const int64_t* vls, const float* rw, const int64_t* rs, float* dq, float* dk, float* dv,
                      float* drw, int B, int H, int Tq, int Tk, int D, int top_k, int* status, cudaStream_t st) {
  if (!d_out || !q || !k || !v || !o || !idx || !valid || !rw || !dq || !dk || !dv || !drw || !status || !dos || !qs ||
      !ks || !vs || !os || !is || !vls || !rs)
    return SWV_ERR_NULL;
  if (B < 1 || H < 1 || Tq < 1 || Tk < 1 || top_k < 1) return SWV_ERR_SHAPE;
  if (dtype != SWV_F32 && dtype != SWV_BF16 && dtype != SWV_F16) return SWV_ERR_DTYPE;
  if (o_dtype != SWV_F32 && o_dtype != SWV_BF16 && o_dtype != SWV_F16) return SWV_ERR_DTYPE;
  if (D < 1 || D > 256) return SWV_ERR_UNSUPPORTED;
  if (ks[3] != 1 || vs[3] != 1) return SWV_ERR_ALIGN;          // key / value rows are read as vectors
  if ((reinterpret_cast<uintptr_t>(dk) & 7) || (reinterpret_cast<uintptr_t>(dv) & 7) || (D & 1)) return SWV_ERR_ALIGN;
  AttnBwdParams p;
  p.d_out = d_out; p.q = q; p.k = k; p.v = v; p.o = o; p.idx = idx; p.valid = valid; p.rw = rw;
  for (int i = 0; i < 4; ++i) { p.dos[i] = dos[i]; p.qs[i] = qs[i]; p.ks[i] = ks[i]; p.vs[i] = vs[i]; p.os[i] = os[i]; }
  for (int i = 0; i < 3; ++i) { p.is[i] = is[i]; p.vls[i] = vls[i]; p.rs[i] = rs[i]; }
  p.dq = dq; p.dk = dk; p.dv = dv; p.drw = drw;
  p.B = B; p.H = H; p.Tq = Tq; p.Tk = Tk; p.D = D; p.top_k = top_k;
  p.scale = 1.0f / sqrtf(static_cast<float>(D));
  p.status = status;
  const size_t kv_bytes = static_cast<size_t>(B) * H * Tk * D * sizeof(float);
  SWV_CUDA_OK(cudaMemsetAsync(dk, 0, kv_bytes, st));
  SWV_CUDA_OK(cudaMemsetAsync(dv, 0, kv_bytes, st));
  SWV_CUDA_OK(cudaMemsetAsync(drw, 0, static_cast<size_t>(B) * Tq * top_k * sizeof(float), st));
#define SWV_BWD_O(T_)                                                                   \
  (o_dtype == SWV_F32 ? launch_attn_bwd<T_, float>(p, st)                               \
                      : (o_dtype == SWV_BF16 ? launch_attn_bwd<T_, __nv_bfloat16>(p, st) \
                                             : launch_attn_bwd<T_, __half>(p, st)))
  if (dtype == SWV_F32) return SWV_BWD_O(float);
  if (dtype == SWV_BF16) return SWV_BWD_O(__nv_bfloat16);
  return SWV_BWD_O(__half);
#undef SWV_BWD_O
}

// -------------------------------------------------------------------- indexer backward
struct IdxBwdParams {
  const float* d_scores;
  int64_t dss[3];
  const void *q_idx, *k_idx;
  int64_t qs[4], ks[4];
  const float* w;
  const int32_t* idx;
  const float* valid;
  int64_t is[3], vls[3];
  float *dq, *dk, *dw;            // fp32 contiguous (B,Tq,IH,ID), (B,Tk,IH,ID), (IH)
  int B, Tq, Tk, IH, ID, top_k;
  int* status;
};

// One warp per (batch, query).  The IH*ID elements of an indexer row are spread over the lanes,
// EPL consecutive PAIRS per lane (element e = 2*lane + 64*i, +1), so that the scatter into dK uses
// 8-byte vector reductions and every key row is read coalesced.  Needs ID even.
template <typename T, int EPL>
__global__ void __launch_bounds__(32 * kBwdWarps) dsa_indexer_bwd_kernel(const IdxBwdParams p) {
  __shared__ float dw_sm[64];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 64; i += blockDim.x) dw_sm[i] = 0.f;
  __syncthreads();
  const int64_t wid = static_cast<int64_t>(blockIdx.x) * kBwdWarps + wib;
  const int64_t total = static_cast<int64_t>(p.B) * p.Tq;
  const int E = p.IH * p.ID;
  if (wid < total) {
    const int qi = static_cast<int>(wid % p.Tq);
    const int b = static_cast<int>(wid / p.Tq);
    const T* qrow = static_cast<const T*>(p.q_idx) + b * p.qs[0] + qi * p.qs[1];
    const T* kbase = static_cast<const T*>(p.k_idx) + b * p.ks[0];
    float qv[2 * EPL], wv[EPL], dq_acc[2 * EPL], dw_acc[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int e = 2 * lane + 64 * i;
      const int hh = e / p.ID, d = e - hh * p.ID;
      const bool in = e < E;
      qv[2 * i] = in ? bw_f32<T>(qrow[hh * p.qs[2] + d * p.qs[3]]) : 0.f;
      qv[2 * i + 1] = in ? bw_f32<T>(qrow[hh * p.qs[2] + (d + 1) * p.qs[3]]) : 0.f;
      wv[i] = in ? p.w[hh] : 0.f;
      dq_acc[2 * i] = dq_acc[2 * i + 1] = 0.f;
      dw_acc[i] = 0.f;
    }
    const int32_t* idx_row = p.idx + b * p.is[0] + qi * p.is[1];
    const float* val_row = p.valid + b * p.vls[0] + qi * p.vls[1];
    const float* ds_row = p.d_scores + b * p.dss[0] + qi * p.dss[1];
    float* dk_b = p.dk + static_cast<int64_t>(b) * p.Tk * E;
    for (int s0 = 0; s0 < p.top_k; s0 += 32) {
      const int slot = s0 + lane;
      float g = 0.f;
      int id = 0;
      if (slot < p.top_k) {
        g = ds_row[slot * p.dss[2]] * val_row[slot * p.vls[2]];       // dS * valid (K:172, :256, :312)
        id = idx_row[slot * p.is[2]];
        if (g != 0.f && (id < 0 || id >= p.Tk)) {
          record_status(p.status, kDevBadIndex);
          g = 0.f;
        }
      }
      for (unsigned rest = __ballot_sync(0xffffffffu, g != 0.f); rest != 0u; rest &= rest - 1u) {
        const int j = __ffs(rest) - 1;
        const float gj = __shfl_sync(0xffffffffu, g, j);
        const int idj = __shfl_sync(0xffffffffu, id, j);
        const T* krow = kbase + static_cast<int64_t>(idj) * p.ks[1];
        float* dkr = dk_b + static_cast<int64_t>(idj) * E;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          const int e = 2 * lane + 64 * i;
          if (e < E) {
            const int hh = e / p.ID, d = e - hh * p.ID;
            const float k0 = bw_f32<T>(krow[hh * p.ks[2] + d * p.ks[3]]);
            const float k1 = bw_f32<T>(krow[hh * p.ks[2] + (d + 1) * p.ks[3]]);
            const float gw = gj * wv[i];
            dq_acc[2 * i] = fmaf(gw, k0, dq_acc[2 * i]);                       // K:175
            dq_acc[2 * i + 1] = fmaf(gw, k1, dq_acc[2 * i + 1]);
            red_add_v2(dkr + e, gw * qv[2 * i], gw * qv[2 * i + 1]);           // K:259-266
            dw_acc[i] = fmaf(gj, fmaf(qv[2 * i], k0, qv[2 * i + 1] * k1), dw_acc[i]);   // K:330-335
          }
        }
      }
    }
    float* dq_row = p.dq + (static_cast<int64_t>(b) * p.Tq + qi) * E;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int e = 2 * lane + 64 * i;
      if (e < E) {
        dq_row[e] = dq_acc[2 * i];
        dq_row[e + 1] = dq_acc[2 * i + 1];
        if (dw_acc[i] != 0.f) atomicAdd(&dw_sm[(e / p.ID) & 63], dw_acc[i]);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < p.IH && i < 64; i += blockDim.x)
    if (dw_sm[i] != 0.f) atomicAdd(p.dw + i, dw_sm[i]);
}

template <typename T>
static int launch_idx_bwd(const IdxBwdParams& p, cudaStream_t st) {
  const int64_t total = static_cast<int64_t>(p.B) * p.Tq;
  const unsigned grid = static_cast<unsigned>((total + kBwdWarps - 1) / kBwdWarps);
  const int E = p.IH * p.ID;
  if (E <= 64) dsa_indexer_bwd_kernel<T, 1><<<grid, 32 * kBwdWarps, 0, st>>>(p);
  else if (E <= 128) dsa_indexer_bwd_kernel<T, 2><<<grid, 32 * kBwdWarps, 0, st>>>(p);
  else if (E <= 256) dsa_indexer_bwd_kernel<T, 4><<<grid, 32 * kBwdWarps, 0, st>>>(p);
  else if (E <= 512) dsa_indexer_bwd_kernel<T, 8><<<grid, 32 * kBwdWarps, 0, st>>>(p);
  else return SWV_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? SWV_OK : SWV_ERR_CUDA;
}

int dsa_indexer_bwd_impl(const float* d_scores, const int64_t* dss, const void* q_idx, const int64_t* qs,
                         const void* k_idx, const int64_t* ks, int dtype, const float* w, const int32_t* idx,
                         const int64_t* is, const float* valid, const int64_t* vls, float* dq, float* dk, float* dw,
                         int B, int Tq, int Tk, int IH, int ID, int top_k, int* status, cudaStream_t st) {
  if (!d_scores || !q_idx || !k_idx || !w || !idx || !valid || !dq || !dk || !dw || !status || !dss || !qs || !ks ||
      !is || !vls)
    return SWV_ERR_NULL;
  if (B < 1 || Tq < 1 || Tk < 1 || IH < 1 || ID < 1 || top_k < 1) return SWV_ERR_SHAPE;
  if (dtype != SWV_F32 && dtype != SWV_BF16 && dtype != SWV_F16) return SWV_ERR_DTYPE;
  if ((ID & 1) || IH > 64 || IH * ID > 512) return SWV_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(dk) & 7) return SWV_ERR_ALIGN;
  IdxBwdParams p;
  p.d_scores = d_scores; p.q_idx = q_idx; p.k_idx = k_idx; p.w = w; p.idx = idx; p.valid = valid;
  for (int i = 0; i < 4; ++i) { p.qs[i] = qs[i]; p.ks[i] = ks[i]; }
  for (int i = 0; i < 3; ++i) { p.dss[i] = dss[i]; p.is[i] = is[i]; p.vls[i] = vls[i]; }
  p.dq = dq; p.dk = dk; p.dw = dw;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.IH = IH; p.ID = ID; p.top_k = top_k; p.status = status;
  SWV_CUDA_OK(cudaMemsetAsync(dk, 0, static_cast<size_t>(B) * Tk * IH * ID * sizeof(float), st));
  SWV_CUDA_OK(cudaMemsetAsync(dw, 0, static_cast<size_t>(IH) * sizeof(float), st));
  if (dtype == SWV_F32) return launch_idx_bwd<float>(p, st);
  if (dtype == SWV_BF16) return launch_idx_bwd<__nv_bfloat16>(p, st);
  return launch_idx_bwd<__half>(p, st);
}

}  // namespace swv
