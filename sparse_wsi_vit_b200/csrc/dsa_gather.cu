// Routing-weighted attention over explicit per-query key lists (any order,
// repeats allowed), CUDA-core fp32 arithmetic.
//
// Replaces the reference's `_dsa_attention_fwd` Triton kernel
// (src/sparse_wsi_vit/models/deepseek_sparse_attention_kernels/kernels.py:450-564)
// one to one: it is the operator behind DSAAttentionFunction.  The dense
// tensor-core kernel in dsa_attn.cu is the fast path for lists produced by this
// library's own indexer.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace swv {

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
  int kv_group;   // query heads per key/value head
  float scale;
  int* status;    // receives kDevBadIndex when a valid slot names a key outside [0, Tk)
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

  const int hk = h / p.kv_group;
  const T* kbase = static_cast<const T*>(p.k) + b * p.ks[0] + hk * p.ks[1];
  const T* vbase = static_cast<const T*>(p.v) + b * p.vs[0] + hk * p.vs[1];
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
    if (ok && (id < 0 || id >= p.Tk)) {
      // a valid slot that names no key: reported through the status word, the slot is dropped
      // (nothing is read through it)
      record_status(p.status, kDevBadIndex);
      ok = false;
      w = 0.f;
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
                         int o_dtype, int B, int H, int Tq, int Tk, int D, int top_k, int kv_group, int* status,
                         cudaStream_t st) {
  if (!q || !k || !v || !idx || !valid || !rw || !o || !status || !qs || !ks || !vs || !is || !vls || !rs || !os)
    return SWV_ERR_NULL;
  if (B < 1 || H < 1 || Tq < 1 || Tk < 1 || top_k < 1) return SWV_ERR_SHAPE;
  if (dtype != SWV_F32 && dtype != SWV_BF16 && dtype != SWV_F16) return SWV_ERR_DTYPE;
  if (o_dtype != SWV_F32 && o_dtype != SWV_BF16 && o_dtype != SWV_F16) return SWV_ERR_DTYPE;
  if (D < 1 || D > 256) return SWV_ERR_UNSUPPORTED;
  if (kv_group < 1 || H % kv_group != 0) return SWV_ERR_SHAPE;
  GatherParams p;
  p.q = q; p.k = k; p.v = v; p.idx = idx; p.valid = valid; p.rw = rw; p.o = o; p.o_dtype = o_dtype;
  for (int i = 0; i < 4; ++i) { p.qs[i] = qs[i]; p.ks[i] = ks[i]; p.vs[i] = vs[i]; p.os[i] = os[i]; }
  for (int i = 0; i < 3; ++i) { p.is[i] = is[i]; p.vls[i] = vls[i]; p.rs[i] = rs[i]; }
  p.B = B; p.H = H; p.Tq = Tq; p.Tk = Tk; p.D = D; p.top_k = top_k; p.kv_group = kv_group;
  p.scale = 1.0f / sqrtf(static_cast<float>(D));
  p.status = status;
  if (dtype == SWV_F32) return launch_gather<float>(p, D, st);
  if (dtype == SWV_BF16) return launch_gather<__nv_bfloat16>(p, D, st);
  return launch_gather<__half>(p, D, st);
}

}  // namespace swv
