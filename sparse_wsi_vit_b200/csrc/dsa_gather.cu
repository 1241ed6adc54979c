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

// ------------------------------------------------------- 16-bit fast path
// bf16 / fp16 q, k, v with unit inner stride and 16-byte aligned rows, D in {32, 64, 128}.
// One CTA per (batch, query) and up to eight heads, one warp per head: the row of idx / valid /
// rw is read ONCE for all heads (256 slots at a time through shared memory).  D / 8 lanes share a
// selected row, each reading one 16-byte chunk of the key row (mixed-precision FMAs: bf16 x bf16
// products are exact in fp32; the partial dot products are added across the row's lanes) and then of
// the value row (p split into two 16-bit halves so that the products stay exact to 2^-17, fp32
// accumulators per lane, folded once at the end).  The running maximum is exact (the accumulators
// are rescaled whenever it rises, a handful of times per row).  Every selected row crosses the
// L2 -> SM path once per head: 2 * top_k * D * 2 bytes per (query, head), one byte per FLOP -- the
// bound of this operator.
template <bool BF16>
__device__ __forceinline__ void fma_mixed2(float& acc0, float& acc1, uint32_t a, uint32_t b) {
  if (BF16) {
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\tmov.b32 {al, ah}, %2;\n\tmov.b32 {bl, bh}, %3;\n\t"
        "fma.rn.f32.bf16 %0, al, bl, %0;\n\tfma.rn.f32.bf16 %1, ah, bh, %1;\n\t}"
        : "+f"(acc0), "+f"(acc1)
        : "r"(a), "r"(b));
  } else {
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\tmov.b32 {al, ah}, %2;\n\tmov.b32 {bl, bh}, %3;\n\t"
        "fma.rn.f32.f16 %0, al, bl, %0;\n\tfma.rn.f32.f16 %1, ah, bh, %1;\n\t}"
        : "+f"(acc0), "+f"(acc1)
        : "r"(a), "r"(b));
  }
}
// x as (hi, lo) with hi = x rounded to 16 bits and lo = the rounded remainder, both halves of one
// word duplicated: {hi, hi} and {lo, lo}
template <bool BF16>
__device__ __forceinline__ void split16(float x, uint32_t& hi2, uint32_t& lo2) {
  if (BF16) {
    const __nv_bfloat16 h = __float2bfloat16_rn(x);
    const __nv_bfloat16 l = __float2bfloat16_rn(x - __bfloat162float(h));
    const uint32_t hb = __bfloat16_as_ushort(h), lb = __bfloat16_as_ushort(l);
    hi2 = hb | (hb << 16);
    lo2 = lb | (lb << 16);
  } else {
    const __half h = __float2half_rn(x);
    const __half l = __float2half_rn(x - __half2float(h));
    const uint32_t hb = __half_as_ushort(h), lb = __half_as_ushort(l);
    hi2 = hb | (hb << 16);
    lo2 = lb | (lb << 16);
  }
}

constexpr int kRowsSlots = 256;      // slots staged per round

// D / 8 lanes share one row (a lane reads ONE 16-byte chunk of it: 8 channels), so a warp-level load
// touches 32 * 16 / (2 D) rows = whole 128-byte lines instead of 32 different lines -- the per-lane
// form of this kernel ran at 99 % of the L1 pipe's tag rate.  G = 256 / D rows per step.
template <int D, bool BF16>
__global__ void __launch_bounds__(256) dsa_attn_gather_rows_kernel(const GatherParams p) {
  constexpr int LPR = D / 8;           // lanes per row
  constexpr int G = 32 / LPR;          // rows per warp step
  constexpr int STEPS = 32 / G;        // steps per 32 slots
  __shared__ int s_idx[kRowsSlots];
  __shared__ float s_w[kRowsSlots];    // routing weight (s_idx < 0 marks a slot that is not valid)
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int qi = blockIdx.x % p.Tq;
  const int b = blockIdx.x / p.Tq;
  const int h = blockIdx.y * nwarps + wib;
  const bool head_ok = h < p.H;
  const int grp = lane / LPR, chunk = lane % LPR;
  const uint16_t* q16 = static_cast<const uint16_t*>(p.q);
  const uint16_t* k16 = static_cast<const uint16_t*>(p.k);
  const uint16_t* v16 = static_cast<const uint16_t*>(p.v);
  uint4 qv = make_uint4(0, 0, 0, 0);   // this lane's 8 channels of q
  if (head_ok) qv = __ldg(reinterpret_cast<const uint4*>(q16 + b * p.qs[0] + h * p.qs[1] + qi * p.qs[2]) + chunk);
  const int hk = head_ok ? h / p.kv_group : 0;
  const uint16_t* kbase = k16 + b * p.ks[0] + hk * p.ks[1];
  const uint16_t* vbase = v16 + b * p.vs[0] + hk * p.vs[1];
  const int32_t* idx_row = p.idx + b * p.is[0] + qi * p.is[1];
  const float* val_row = p.valid + b * p.vls[0] + qi * p.vls[1];
  const float* rw_row = p.rw + b * p.rs[0] + qi * p.rs[1];
  const float ninf = -__int_as_float(0x7f800000);

  float o[8];                          // channels [8 * chunk, +8) summed over this lane's rows
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = 0.f;
  float m = ninf, l = 0.f;

  for (int base = 0; base < p.top_k; base += kRowsSlots) {
    __syncthreads();
    for (int i = threadIdx.x; i < kRowsSlots; i += blockDim.x) {
      const int slot = base + i;
      int id = -1;
      float w = 0.f;
      if (slot < p.top_k && val_row[slot * p.vls[2]] > 0.f) {
        id = idx_row[slot * p.is[2]];
        w = rw_row[slot * p.rs[2]];
        if (id < 0 || id >= p.Tk) {
          // a valid slot that names no key: reported through the status word, the slot is dropped
          record_status(p.status, kDevBadIndex);
          id = -1;
        }
      }
      s_idx[i] = id;
      s_w[i] = w;
    }
    __syncthreads();
    if (!head_ok) continue;
    const int n_here = min(kRowsSlots, p.top_k - base);
    for (int c0 = 0; c0 < n_here; c0 += 32) {
      // logits of the 32 slots: step s handles slots c0 + s * G + grp (one per lane group)
      float logit[STEPS];
      int ids[STEPS];
      float cmax = ninf;
#pragma unroll
      for (int s_ = 0; s_ < STEPS; ++s_) {
        const int id = s_idx[c0 + s_ * G + grp];
        ids[s_] = id;
        float a0 = 0.f, a1 = 0.f;
        if (id >= 0) {
          const uint4 kv = __ldg(reinterpret_cast<const uint4*>(kbase + static_cast<int64_t>(id) * p.ks[2]) + chunk);
          fma_mixed2<BF16>(a0, a1, qv.x, kv.x);
          fma_mixed2<BF16>(a0, a1, qv.y, kv.y);
          fma_mixed2<BF16>(a0, a1, qv.z, kv.z);
          fma_mixed2<BF16>(a0, a1, qv.w, kv.w);
        }
        float a = a0 + a1;
#pragma unroll
        for (int off = LPR / 2; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
        logit[s_] = id >= 0 ? a * p.scale : ninf;
        cmax = fmaxf(cmax, logit[s_]);
      }
#pragma unroll
      for (int off = 16; off >= LPR; off >>= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, off));
      if (cmax > m) {                                    // warp-uniform
        if (m != ninf) {
          const float f = __expf(m - cmax);
          l *= f;
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] *= f;
        }
        m = cmax;
      }
#pragma unroll
      for (int s_ = 0; s_ < STEPS; ++s_) {
        const int id = ids[s_];
        const float pj = id >= 0 ? __expf(logit[s_] - m) * s_w[c0 + s_ * G + grp] : 0.f;
        if (pj != 0.f) {                                  // uniform within the lane group
          if (chunk == 0) l += pj;
          uint32_t ph, pl;
          split16<BF16>(pj, ph, pl);
          const uint4 vv = __ldg(reinterpret_cast<const uint4*>(vbase + static_cast<int64_t>(id) * p.vs[2]) + chunk);
          const uint32_t vw[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            fma_mixed2<BF16>(o[2 * c], o[2 * c + 1], ph, vw[c]);
            fma_mixed2<BF16>(o[2 * c], o[2 * c + 1], pl, vw[c]);
          }
        }
      }
    }
  }
  if (!head_ok) return;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
  // add up the lane groups: afterwards every lane of a chunk column holds the full sums
#pragma unroll
  for (int off = 16; off >= LPR; off >>= 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] += __shfl_xor_sync(0xffffffffu, o[i], off);
  }
  if (grp == 0) {
    const float inv = 1.f / fmaxf(l, 1e-6f);
    const int64_t obase = b * p.os[0] + h * p.os[1] + qi * p.os[2];
#pragma unroll
    for (int i = 0; i < 8; ++i) st_out(p.o, p.o_dtype, obase + (chunk * 8 + i) * p.os[3], o[i] * inv);
  }
}

static bool rows_path_ok(const GatherParams& p, int dtype, int D) {
  if (dtype == SWV_F32 || (D != 32 && D != 64 && D != 128)) return false;
  auto a16 = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
  if (!a16(p.q) || !a16(p.k) || !a16(p.v)) return false;
  if (p.qs[3] != 1 || p.ks[3] != 1 || p.vs[3] != 1) return false;
  for (int i = 0; i < 3; ++i)
    if ((p.qs[i] * 2) % 16 || (p.ks[i] * 2) % 16 || (p.vs[i] * 2) % 16) return false;
  return true;
}

template <bool BF16>
static int launch_gather_rows(const GatherParams& p, int D, cudaStream_t st) {
  const int warps = p.H < 8 ? p.H : 8;
  const dim3 grid(static_cast<unsigned>(p.B) * p.Tq, static_cast<unsigned>((p.H + warps - 1) / warps));
  if (D == 32) dsa_attn_gather_rows_kernel<32, BF16><<<grid, 32 * warps, 0, st>>>(p);
  else if (D == 64) dsa_attn_gather_rows_kernel<64, BF16><<<grid, 32 * warps, 0, st>>>(p);
  else dsa_attn_gather_rows_kernel<128, BF16><<<grid, 32 * warps, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? SWV_OK : SWV_ERR_CUDA;
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
  if (rows_path_ok(p, dtype, D))
    return dtype == SWV_BF16 ? launch_gather_rows<true>(p, D, st) : launch_gather_rows<false>(p, D, st);
  if (dtype == SWV_F32) return launch_gather<float>(p, D, st);
  if (dtype == SWV_BF16) return launch_gather<__nv_bfloat16>(p, D, st);
  return launch_gather<__half>(p, D, st);
}

}  // namespace swv
