// DSA attention over the indexer's key lists as dense tensor-core tiles with a SPARSE softmax (the
// attention step of the reference's DSAAttentionFunction.forward, kernels.py:769-810, 450-564, for
// bf16 inputs with head dim 64).
//
// One CTA owns 128 query rows of one head pair and sweeps all key tiles, like dsa_attn_masked_kernel:
//   S_h = Q_h K_h^T        tcgen05.mma, Q resident in TMEM (A operand), K tiles by TMA, fp32 into TMEM
//   O_h += P_h [V_h | 1]   tcgen05.mma, P in shared memory, V tiles by TMA, O resident in TMEM; the
//                          accumulator is 80 wide, its column 64 collects the row sums of P
// but only the SELECTED (query, key) pairs are touched on the CUDA cores.  A row selects 1 key in 32
// or fewer, i.e. a 128 x 128 tile holds ~512 selected pairs.  dsa_tile_lists_kernel first turns the
// per-row lists (idx, routing weights) into one list per (query tile, key tile).  Per tile the 256
// softmax threads then
//   1. copy S_h out of TMEM into shared memory as fp16, every thread its own row of one head (the
//      only dense step: conversions, no exponentials);
//   2. clear the entries of P they wrote for the previous tile (once PV of that tile has retired);
//   3. share the tile's pairs evenly (2-3 each, loaded a tile ahead): per pair and head one logit
//      read, ONE exponential, times the routing weight, one bf16 store into the otherwise zero P tile.
// Per tile and head that is ~512 exponentials instead of 128 x 128, with no recomputation of the
// indexer scores: membership and weights come from the lists.
//
// Stabiliser: p' = 2^(s*c - bound) with `bound` a Cauchy-Schwarz bound of the row's logits (no running
// maximum, no rescaling of O).  out = O' / l'.  The reference's clamp max(l, 1e-6) acts on
// l = l' * 2^(bound - m) >= l', so it cannot bind when l' >= 1e-6; l' == 0 means every weight of the
// row is zero (output 0).  A (query tile, head pair) with a row in between, with a bound above
// kLMaxBound or with an over-full tile list raises its entry of `flags`; the host then runs
// dsa_attn_masked_kernel for the flagged ones only.
//
// TMEM (512 columns allocated): Q_h bf16x2 [32h, +32) | S_h fp32 [64 + 128h, +128) | O_h fp32 [320 + 80h, +80).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace swv {

// defined in dsa_attn.cu
int dsa_key_norm_max(const void* k, const int64_t* ks, int B, int H, int Tk, uint32_t* kmax2, cudaStream_t st);
int dsa_attn_split_factor(int B, int H, int Tq, int Tk);
int dsa_attn_scratch_bytes_impl(int B, int H, int Tq, int Tk, size_t* bytes);
int dsa_attn_masked_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                         const int64_t* vs, const uint32_t* maskbits, void* workspace, void* o, const int64_t* os,
                         int o_dtype, int B, int H, int Tq, int Tk, int D, void* scratch, size_t scratch_bytes,
                         int* status, cudaStream_t st, int* member_count, const uint32_t* only_flagged);
void dsa_workspace_views(void* workspace, int B, int Tq, int Tk, float** wq, float** wk, uint32_t** prefix,
                         uint32_t** kth, uint32_t** neq, uint32_t** kmax2, int32_t** excl);

namespace {

constexpr int kLD = 64;                                  // head dim
constexpr int kLNO = 80;                                 // PV accumulator width: 64 output channels + the row sum (x16)
constexpr int kLTileBytes = kTile * kLD * 2;             // 16 KiB: a K or V tile, and one 64-key half of a P tile
constexpr int kLTmemCols = 512;
constexpr uint32_t kLColQ = 0, kLColS = 64, kLColO = 320;
constexpr int kLSoftWarps = 8;                           // staging: warp = (head, 32 rows), thread = (head, row)
constexpr int kLSoft = 32 * kLSoftWarps;
constexpr int kLThreads = 64 + kLSoft + 64;              // TMA warp, TMEM warp, softmax warps, two head issuers
constexpr int kLStageBytes = 32 * kTile * 2;             // per softmax warp: 32 rows x 128 fp16 logits
constexpr float kLMaxBound = 40.0f;                      // largest admissible |logit| bound (log2 units)
constexpr int kLRec = kLD + 4;                           // split merge record: output row + (row sum, -, -, -)
constexpr int kLPre = 3;                                 // tile-list entries per thread held in registers (3 x 256 = 768)

// shared memory map (bytes from the 1024-aligned base)
constexpr int kLOffK = 0;                                // [head]
constexpr int kLOffV = kLOffK + 2 * kLTileBytes;         // [head]
constexpr int kLOffOnes = kLOffV + 2 * kLTileBytes;      // 16 key rows x 128 bytes of bf16 1.0 (the row-sum column of V)
constexpr int kLOffP = kLOffOnes + 2048;                 // [head][keys 0..63 | keys 64..127], K-major, 128-byte swizzle
constexpr int kLOffStage = kLOffP + 4 * kLTileBytes;     // [softmax warp = head * 4 + row quarter]
constexpr int kLOffBound = kLOffStage + kLSoftWarps * kLStageBytes;   // [head][row] fp32
constexpr int kLOffCtl = kLOffBound + 2 * kTile * 4;

struct ListParams {
  int B, H, Tq, Tk, nQT, nKT, nHP;
  const __nv_bfloat16* q;
  int64_t qsb, qsh, qst;
  const uint32_t* tl_cnt;  // [B*nQT*nKT] members of every (query tile, key tile)
  const uint2* tl_ent;     // [B*nQT*nKT][cap] {strip offset | P offset << 16, weight bits}
  const uint32_t* tl_over; // [B*nQT] some tile of the query tile overflowed its capacity
  int cap;
  const uint32_t* kmax2;   // [B*H] max squared key norm, float bits
  void* o;
  int64_t osb, osh, ost;
  int o_dtype;
  float scale_log2;
  int* status;
  uint32_t* flags;         // [CTAs] raised by a CTA that leaves its rows to dsa_attn_masked_kernel
  int split;               // CTAs per (query tile, head pair), each sweeping a share of the key tiles
  float* scratch;          // [CTAs][split][2 heads][128 rows][kLRec]
  uint32_t* tickets;       // [CTAs]
};

struct ListCtl {
  uint64_t k_full[2], k_empty[2];
  uint64_t v_full[2], v_empty[2];
  uint64_t s_full[2], s_free[2], p_full[2], pv_done[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t cta_flag;
  uint32_t ticket;
};

constexpr size_t lists_smem_bytes() { return 1024 + kLOffCtl + sizeof(ListCtl) + 64; }

// Phase timers of the profiling build (-DSWV_PROFILE): lane 0 of every role adds the cycles it spent
// per phase to a table that swv_debug_lists_profile() reads.  Empty inline functions otherwise.
#ifdef SWV_PROFILE
__device__ unsigned long long g_lists_prof[64];
struct LProf {
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
    for (int i = 0; i < 8; ++i) atomicAdd(&g_lists_prof[base + i], acc[i]);
  }
};
#else
struct LProf {
  __device__ __forceinline__ void start() {}
  __device__ __forceinline__ void tick(int) {}
  __device__ __forceinline__ void flush(int, bool) {}
};
#endif

// if (on) store
__device__ __forceinline__ void sts16_if(uint32_t saddr, uint16_t v, bool on) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p st.shared.b16 [%0], %1;\n\t}" ::"r"(saddr), "h"(v),
               "r"(static_cast<uint32_t>(on))
               : "memory");
}
__device__ __forceinline__ uint16_t lds16(uint32_t saddr) {
  uint16_t v;
  asm volatile("ld.shared.b16 %0, [%1];" : "=h"(v) : "r"(saddr) : "memory");
  return v;
}

// Offsets of element (row, col) of a 128 x 128 tile, as the tile-list entries carry them:
//   strip: inside the eight 8-KiB strips of one head's fp16 logits (strip = 32 rows; a row's 128
//          logits in sixteen 16-byte pieces, piece q of all 32 rows together);
//   P    : inside one head's P tile (two 64-key halves of 128 rows x 128 bytes, the 16-byte chunks
//          of a row XOR-swizzled with the row index as the 128-byte swizzle mode expects).
__host__ __device__ __forceinline__ uint32_t strip_offset(uint32_t row, uint32_t col) {
  return (row >> 5) * kLStageBytes + (row & 31u) * 16u + ((col & 0x78u) << 6) + ((col & 7u) << 1);
}
__host__ __device__ __forceinline__ uint32_t p_offset(uint32_t row, uint32_t col) {
  return ((col & 64u) << 8) + row * 128u + ((((col >> 3) & 7u) ^ (row & 7u)) << 4) + ((col & 7u) << 1);
}

// ---- the tile lists: every (query tile, key tile) gets the list of its selected (row, key) pairs
// with their routing weights, in any order, built from the per-row lists.  One CTA per
// query tile, `parts` threads per row (one with many query tiles, more when few CTAs would leave the
// GPU idle), each on a contiguous share of the row's list; the rows advance through their lists
// together, so the entries of a tile are written within a short time of each other.
__global__ void __launch_bounds__(1024)
    dsa_tile_lists_kernel(const int32_t* __restrict__ idx, const float* __restrict__ rw, int top_k, int n_valid, int Tq,
                          int nQT, int nKT, int cap, int parts, uint32_t* __restrict__ tl_cnt,
                          uint2* __restrict__ tl_ent, uint32_t* __restrict__ tl_over) {
  extern __shared__ uint32_t cnt_s[];          // [nKT]
  const int b = blockIdx.x / nQT, qt = blockIdx.x % nQT;
  const int row = threadIdx.x & (kTile - 1);
  const int part = threadIdx.x >> 7;
  const int qrow = qt * kTile + row;
  for (int i = threadIdx.x; i < nKT; i += blockDim.x) cnt_s[i] = 0u;
  __shared__ uint32_t over_s;
  if (threadIdx.x == 0) over_s = 0u;
  __syncthreads();
  const size_t tile0 = static_cast<size_t>(blockIdx.x) * nKT;
  if (qrow < Tq) {
    const size_t grow = static_cast<size_t>(b) * Tq + qrow;
    const int4* ip = reinterpret_cast<const int4*>(idx + grow * top_k);
    const float4* wp = reinterpret_cast<const float4*>(rw + grow * top_k);
    bool over = false;
    const int groups = (n_valid + 3) >> 2;
    const int s0 = 4 * static_cast<int>(static_cast<int64_t>(groups) * part / parts);
    const int s1 = min(n_valid, 4 * static_cast<int>(static_cast<int64_t>(groups) * (part + 1) / parts));
    // four groups of four slots are asked for at a time: the loop is bound by the latency of its loads
    // (measured at 512 query tiles: 0.77 ms one group at a time, 0.69 ms with four, 0.91 ms with eight,
    // which spread a query tile's writes over too many key tiles at a time)
    for (int s = s0; s < s1; s += 16) {
      int4 k4[4];
      float4 w4[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const bool in = s + 4 * g < s1;
        k4[g] = in ? __ldg(ip + (s >> 2) + g) : make_int4(0, 0, 0, 0);
        w4[g] = in ? __ldg(wp + (s >> 2) + g) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const int kk[4] = {k4[g].x, k4[g].y, k4[g].z, k4[g].w};
        const float ww[4] = {w4[g].x, w4[g].y, w4[g].z, w4[g].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (s + 4 * g + e < s1) {
            const uint32_t key = static_cast<uint32_t>(kk[e]);
            const uint32_t kt = key >> 7, col = key & 127u;
            if (kt < static_cast<uint32_t>(nKT)) {            // (a key index beyond the key range is dropped)
              const uint32_t pos = atomicAdd(&cnt_s[kt], 1u);
              if (pos < static_cast<uint32_t>(cap))
                tl_ent[(tile0 + kt) * cap + pos] =
                    make_uint2(strip_offset(row, col) | (p_offset(row, col) << 16), __float_as_uint(ww[e]));
              else
                over = true;
            }
          }
        }
      }
    }
    if (over) over_s = 1u;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nKT; i += blockDim.x) tl_cnt[tile0 + i] = min(cnt_s[i], static_cast<uint32_t>(cap));
  if (threadIdx.x == 0) tl_over[blockIdx.x] = over_s;
}

template <bool kSplit>
__global__ void __launch_bounds__(kLThreads, 1)
    dsa_attn_lists_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                          const ListParams p) {
  constexpr uint32_t kIdescQK = make_idesc(/*bf16*/ 1, kTile, kTile, 0, 0);
  constexpr uint32_t kIdescPV = make_idesc(/*bf16*/ 1, kTile, kLNO, 0, /*V is MN-major*/ 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  ListCtl* ctl = reinterpret_cast<ListCtl*>(smem + kLOffCtl);

#ifdef SWV_PROFILE
  const long long t_cta0 = clock64();
#endif
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta = kSplit ? blockIdx.x / p.split : blockIdx.x;     // (batch, query tile, head pair)
  const int part = kSplit ? blockIdx.x - cta * p.split : 0;       // which share of the key tiles
  const int hp = cta % p.nHP;
  const int qt = (cta / p.nHP) % p.nQT;
  const int b = cta / (p.nHP * p.nQT);
  const int kt0 = kSplit ? static_cast<int>(static_cast<int64_t>(part) * p.nKT / p.split) : 0;   // first key tile
  const int nKT = kSplit ? static_cast<int>(static_cast<int64_t>(part + 1) * p.nKT / p.split) - kt0 : p.nKT;
  const int h0 = hp * 2;
  const int nh = (h0 + 1 < p.H) ? 2 : 1;   // heads handled by this CTA

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl->v_full[s], 1);
      mbar_init(&ctl->v_empty[s], 1);
      mbar_init(&ctl->s_full[s], 1);
      mbar_init(&ctl->s_free[s], kLSoftWarps / 2);
      mbar_init(&ctl->p_full[s], 1);
      mbar_init(&ctl->pv_done[s], 1);
      mbar_init(&ctl->k_full[s], 1);
      mbar_init(&ctl->k_empty[s], 1);
    }
    ctl->abort_flag = 0;
    ctl->cta_flag = p.tl_over[b * p.nQT + qt];     // a tile list of this query tile is incomplete
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, kLTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  // ------------------------------------------------------------------ prologue (softmax warps)
  // Every softmax thread owns one query row of one head: it puts the row into TMEM (the A operand of
  // every S = Q K^T of the sweep), bounds the row's logits, and clears its share of the P tiles.
  const bool soft = warp >= 2 && warp < 2 + kLSoftWarps;
  const int ts = static_cast<int>(threadIdx.x) - 64;   // softmax thread index
  const int x = soft ? (warp - 2) >> 2 : 0;            // head of the pair
  const int quarter = warp & 3;                        // TMEM lane quarter this warp may touch
  const int row = quarter * 32 + lane;
  const int qrow = qt * kTile + row;
  const bool active = soft && x < nh;                  // warp-uniform
  const bool row_ok = active && qrow < p.Tq;
  const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
  if (soft) {
    uint32_t qw[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) qw[i] = 0u;
    bool flagged = false;
    float bound = 0.f;
    if (row_ok) {
      const uint4* qv = reinterpret_cast<const uint4*>(p.q + b * p.qsb + (h0 + x) * p.qsh + qrow * p.qst);
      float q2 = 0.f;
#pragma unroll
      for (int i = 0; i < kLD / 8; ++i) {
        const uint4 v = __ldg(qv + i);
        qw[4 * i] = v.x; qw[4 * i + 1] = v.y; qw[4 * i + 2] = v.z; qw[4 * i + 3] = v.w;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float lo = __uint_as_float(qw[4 * i + t] << 16), hi = __uint_as_float(qw[4 * i + t] & 0xffff0000u);
          q2 = fmaf(lo, lo, fmaf(hi, hi, q2));
        }
      }
      const float k2 = __uint_as_float(p.kmax2[b * p.H + h0 + x]);
      bound = sqrtf(q2 * k2) * p.scale_log2 * 1.001f + 1e-3f;
      flagged = !(bound <= kLMaxBound);                // also true for a NaN bound
    }
    reinterpret_cast<float*>(smem + kLOffBound)[x * kTile + row] = bound;
    if (active) {
      tmem_st32(lane_base + kLColQ + 32 * x, qw);
      tc_wait_st();
    }
    const uint32_t pz = smem_u32(smem + kLOffP) + ts * 256u;
#pragma unroll
    for (int i = 0; i < 16; ++i) sts128(pz + i * 16, 0u, 0u, 0u, 0u);
    if (ts < 128) sts128(smem_u32(smem + kLOffOnes) + ts * 16u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u);
    fence_proxy_async_smem();                          // the tensor core reads P and the ones through the async proxy
    if (__any_sync(0xffffffffu, flagged) && lane == 0) atomicOr(&ctl->cta_flag, 1u);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const bool skip = *reinterpret_cast<volatile uint32_t*>(&ctl->cta_flag) != 0u;
  if (skip && threadIdx.x == 0 && part == 0) p.flags[cta] = 1u;
#ifdef SWV_PROFILE
  const long long t_cta1 = clock64();
#endif

  if (skip) {
    // nothing: the masked kernel redoes this (query tile, head pair)
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      bool ok = true;
      // One K and one V buffer per head: a tile period is longer than the latency of a load, K(j+1)
      // is requested when S(j) is complete and V(j+1) when O += P(j) V(j) is.
      auto load_k = [&](int xx, int j) {
        if (!ok || xx >= nh) return;
        if (!mbar_wait_bounded(&ctl->k_empty[xx], (j & 1) ^ 1, abort_flag)) { ok = false; return; }
        mbar_expect_tx(&ctl->k_full[xx], kLTileBytes);
        tma_load_4d(smem + kLOffK + xx * kLTileBytes, &tm_k, &ctl->k_full[xx], 0, (kt0 + j) * kTile, h0 + xx, b);
      };
      auto load_v = [&](int xx, int j) {
        if (!ok || xx >= nh) return;
        if (!mbar_wait_bounded(&ctl->v_empty[xx], (j & 1) ^ 1, abort_flag)) { ok = false; return; }
        mbar_expect_tx(&ctl->v_full[xx], kLTileBytes);
        tma_load_4d(smem + kLOffV + xx * kLTileBytes, &tm_v, &ctl->v_full[xx], 0, (kt0 + j) * kTile, h0 + xx, b);
      };
      // in the order the buffers come free: K(j+1) when S(j) is complete (early in tile j-1's softmax),
      // V(j) when O += P(j-1) V(j-1) is (early in tile j's)
      load_k(0, 0);
      load_k(1, 0);
      load_v(0, 0);
      load_v(1, 0);
      if (nKT > 1) {
        load_k(0, 1);
        load_k(1, 1);
      }
      for (int i = 1; i < nKT && ok; ++i) {
        if (i + 1 < nKT) {
          load_k(0, i + 1);
          load_k(1, i + 1);
        }
        load_v(0, i);
        load_v(1, i);
      }
      if (!ok) record_status(p.status, kDevWaitStageEmpty);
    }
  } else if (warp >= 2 + kLSoftWarps) {
    // ------------------------------------- MMA issuer of one head: S_x(j) and O_x += P_x(j) V_x(j)
    const int xx = warp - (2 + kLSoftWarps);
    if (lane == 0 && xx < nh) {
      const uint64_t dk = smem_desc_sw128(smem_u32(smem + kLOffK + xx * kLTileBytes));
      const uint32_t v_addr = smem_u32(smem + kLOffV + xx * kLTileBytes);
      const uint32_t ones_addr = smem_u32(smem + kLOffOnes);
      const uint64_t dp = smem_desc_sw128(smem_u32(smem + kLOffP + xx * 2 * kLTileBytes));
      const uint32_t s_col = tmem_base + kLColS + xx * kTile;
      const uint32_t o_col = tmem_base + kLColO + xx * kLNO;
      const uint32_t q_col = tmem_base + kLColQ + xx * 32;
      bool ok = true;
      LProf prof;
      prof.start();
      auto issue_qk = [&](int j) {
        prof.tick(7);
        if (!mbar_wait_bounded(&ctl->k_full[xx], j & 1, abort_flag)) {
          record_status(p.status, kDevWaitTmaFull);
          ok = false;
          return;
        }
        prof.tick(0);
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) umma_f16_ts(s_col, q_col + ks * 8, dk + ks * 2, kIdescQK, ks > 0);
        umma_commit(&ctl->k_empty[xx]);
        umma_commit(&ctl->s_full[xx]);
        prof.tick(1);
      };
      issue_qk(0);
      for (int j = 0; ok && j < nKT; ++j) {
        if (j + 1 < nKT) {
          // S_x(j+1) may overwrite S_x(j) once the softmax warps have copied it out
          if (!mbar_wait_bounded(&ctl->s_free[xx], j & 1, abort_flag)) {
            record_status(p.status, kDevWaitAccEmpty);
            break;
          }
          prof.tick(2);
          issue_qk(j + 1);
          if (!ok) break;
        }
        prof.tick(7);
        bool got = mbar_wait_bounded(&ctl->p_full[xx], j & 1, abort_flag);
        prof.tick(3);
        got = got && mbar_wait_bounded(&ctl->v_full[xx], j & 1, abort_flag);
        prof.tick(4);
        if (!got) {
          record_status(p.status, kDevWaitPReady);
          break;
        }
        tc_fence_after();
        // 16 keys per step: 32 bytes along a P row, 2 KiB of V rows.  The accumulator is 80 wide: the
        // second 64-column block of the B operand is the block of ones (its distance from the V
        // rows of the step goes into the descriptor), so column 64 receives the row sums of P.
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t vb = v_addr + ks * 2048;
          umma_f16_ss(o_col, dp + (ks >> 2) * (kLTileBytes / 16) + (ks & 3) * 2, smem_desc_sw128(vb, ones_addr - vb),
                      kIdescPV, (j > 0 || ks > 0));
        }
        umma_commit(&ctl->v_empty[xx]);
        umma_commit(&ctl->pv_done[xx]);
        prof.tick(5);
      }
      prof.flush(16 + 8 * xx, true);
#ifdef SWV_PROFILE
      if (xx == 0) atomicAdd(&g_lists_prof[63], static_cast<unsigned long long>(nKT));
#endif
    }
  } else if (soft) {
    // ----------------------------------------------------------------- softmax
    bool ok = true;
    {
      const uint32_t s_col = lane_base + kLColS + x * kTile;
      const uint32_t strips = smem_u32(smem + kLOffStage);
      const uint32_t stage = strips + (x * 4 + quarter) * kLStageBytes + lane * 16;   // strip = (head, row quarter)
      const uint32_t p_tiles = smem_u32(smem + kLOffP);
      const uint32_t bound_s = smem_u32(smem + kLOffBound);
      const float sc = p.scale_log2;
      const size_t tile_base = (static_cast<size_t>(b) * p.nQT + qt) * p.nKT + kt0;
      // this thread's share of a tile's list: entries ts, ts + 256, ...; the first kLPre of the NEXT
      // tile are requested while the current tile is processed
      uint2 ent[kLPre], nent[kLPre];
      uint32_t cnt = 0, ncnt = 0;
      auto request = [&](int j) {
        ncnt = __ldg(p.tl_cnt + tile_base + j);
        const uint2* src = p.tl_ent + (tile_base + j) * p.cap;
#pragma unroll
        for (int k = 0; k < kLPre; ++k) {
          const int i = ts + k * kLSoft;
          nent[k] = i < p.cap ? __ldg(src + i) : make_uint2(0u, 0u);
        }
      };
      request(0);
      uint32_t prev_off[kLPre] = {0u, 0u, 0u};   // P offsets this thread wrote for the previous tile
      uint32_t prev_n = 0;               // how many of them; kLPre + 1: more than the registers hold
      LProf prof;
      prof.start();

      for (int j = 0; j < nKT; ++j) {
        prof.tick(7);
        cnt = ncnt;
#pragma unroll
        for (int k = 0; k < kLPre; ++k) ent[k] = nent[k];
        if (j + 1 < nKT) request(j + 1);
        // ---- this thread's row of S(j): TMEM -> fp16 -> its strip of shared memory
        if (active) {
          if (!mbar_wait_bounded(&ctl->s_full[x], j & 1, abort_flag)) {
            record_status(p.status, kDevWaitAccFull);
            ok = false;
          }
          prof.tick(0);
          if (ok) {
            tc_fence_after();
            uint32_t ra[32], rb[32];
            tmem_ld32(s_col, ra);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              tc_wait_ld();
              if (c + 1 < 4) {
                if (c & 1) tmem_ld32(s_col + (c + 1) * 32, ra);
                else tmem_ld32(s_col + (c + 1) * 32, rb);
              }
#pragma unroll
              for (int g = 0; g < 4; ++g) {            // 8 logits -> four fp16 pairs -> one 16-byte store
                uint32_t h[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                  const uint32_t u0 = (c & 1) ? rb[g * 8 + 2 * t] : ra[g * 8 + 2 * t];
                  const uint32_t u1 = (c & 1) ? rb[g * 8 + 2 * t + 1] : ra[g * 8 + 2 * t + 1];
                  const __half2 hh = __floats2half2_rn(__uint_as_float(u0), __uint_as_float(u1));
                  h[t] = *reinterpret_cast<const uint32_t*>(&hh);
                }
                sts128(stage + static_cast<uint32_t>((c * 4 + g) * 32 * 16), h[0], h[1], h[2], h[3]);
              }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->s_free[x]);
          }
        }
        prof.tick(1);

        // ---- P(j) of both heads: the tile's selected (row, key) pairs, evenly over the threads.
        // PV(j-1) must have read the P tiles first; then every thread clears the entries it wrote
        // for the previous tile.
        if (ok && j > 0) {
          for (int h = 0; h < nh; ++h) {
            if (!mbar_wait_bounded(&ctl->pv_done[h], (j - 1) & 1, abort_flag)) {
              record_status(p.status, kDevWaitPvDone);
              ok = false;
            }
          }
        }
        prof.tick(3);
        if (prev_n <= kLPre) {
#pragma unroll
          for (int k = 0; k < kLPre; ++k) {
            sts16_if(p_tiles + prev_off[k], 0, k < static_cast<int>(prev_n));
            sts16_if(p_tiles + 2 * kLTileBytes + prev_off[k], 0, k < static_cast<int>(prev_n) && nh == 2);
          }
        } else {
          // a dense tile: every thread clears 256 bytes of the P tiles (chunks rotated: no bank conflicts)
#pragma unroll
          for (int i = 0; i < 16; ++i) sts128(p_tiles + ts * 256u + (((i + lane) & 15) << 4), 0u, 0u, 0u, 0u);
        }
        prev_n = 0;
        // every strip of both heads is complete and the P tiles are clear (a wait that gave up keeps
        // passing the barriers)
        asm volatile("bar.sync 3, %0;" ::"r"(kLSoft) : "memory");
        prof.tick(2);
        // entries in registers
        uint32_t so[kLPre], po[kLPre];
        float wv[kLPre];
        bool on[kLPre];
        uint16_t hs[2][kLPre], pb[2][kLPre];
        float bd[2][kLPre];
#pragma unroll
        for (int k = 0; k < kLPre; ++k) {
          on[k] = static_cast<uint32_t>(ts + k * kLSoft) < cnt;
          so[k] = on[k] ? (ent[k].x & 0xffffu) : 0u;
          po[k] = on[k] ? (ent[k].x >> 16) : 0u;
          wv[k] = __uint_as_float(ent[k].y);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int k = 0; k < kLPre; ++k) {
            hs[h][k] = lds16(strips + h * 4 * kLStageBytes + so[k]);
            bd[h][k] = __uint_as_float(lds32(bound_s + (h * kTile + ((po[k] >> 7) & 127u)) * 4));
          }
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int k = 0; k < kLPre; ++k) {
            const float t = fmaf(__half2float(__ushort_as_half(hs[h][k])), sc, -bd[h][k]);
            pb[h][k] = __bfloat16_as_ushort(__float2bfloat16_rn(ex2_approx(t) * wv[k]));
          }
#pragma unroll
        for (int k = 0; k < kLPre; ++k) {
          sts16_if(p_tiles + po[k], pb[0][k], on[k]);
          sts16_if(p_tiles + 2 * kLTileBytes + po[k], pb[1][k], on[k] && nh == 2);
          prev_off[k] = po[k];
          prev_n += on[k] ? 1u : 0u;
        }
        // the rest of a dense tile's list, straight from global memory
        if (cnt > static_cast<uint32_t>(kLPre * kLSoft)) {
          const uint2* src = p.tl_ent + (tile_base + j) * p.cap;
          for (uint32_t i = ts + kLPre * kLSoft; i < cnt; i += kLSoft) {
            const uint2 e = __ldg(src + i);
            const uint32_t eso = e.x & 0xffffu, epo = e.x >> 16;
            for (int h = 0; h < nh; ++h) {
              const float t = fmaf(__half2float(__ushort_as_half(lds16(strips + h * 4 * kLStageBytes + eso))), sc,
                                   -__uint_as_float(lds32(bound_s + (h * kTile + ((epo >> 7) & 127u)) * 4)));
              sts16_if(p_tiles + h * 2 * kLTileBytes + epo,
                       __bfloat16_as_ushort(__float2bfloat16_rn(ex2_approx(t) * __uint_as_float(e.y))), true);
            }
          }
          prev_n = kLPre + 1;
        }
        prof.tick(4);
        fence_proxy_async_smem();
        // all of P(j) is written and nobody reads the strips of this tile any more
        asm volatile("bar.sync 3, %0;" ::"r"(kLSoft) : "memory");
        if (ts == 0) {
          mbar_arrive(&ctl->p_full[0]);
          if (nh == 2) mbar_arrive(&ctl->p_full[1]);
        }
        prof.tick(5);
      }
      if (active && ok && !mbar_wait_bounded(&ctl->pv_done[x], (nKT - 1) & 1, abort_flag)) {
        record_status(p.status, kDevWaitPvDone);
        ok = false;
      }
      if (ok) tc_fence_after();
      prof.flush(x * 8, lane == 0 && quarter == 0);
    }

    // ---- output.  Column 64 of the accumulator holds l' = sum of the row of P'.  With l' >= 1e-6 the
    // reference's clamp max(l, 1e-6) cannot bind (l = l' 2^(bound - m) >= l'), l' == 0 means every
    // weight of the row is zero (output 0); a row in between is left to the masked kernel.
    const int h = h0 + x;
    const uint32_t o_col = lane_base + kLColO + x * kLNO;
    auto store_chunk = [&](int c, const float (&acc)[16], float scale) {
      if (p.o_dtype == SWV_F32) {
        float* orow = static_cast<float*>(p.o) + b * p.osb + h * p.osh + qrow * p.ost + c * 16;
#pragma unroll
        for (int i = 0; i < 16; i += 4)
          *reinterpret_cast<float4*>(orow + i) =
              make_float4(acc[i] * scale, acc[i + 1] * scale, acc[i + 2] * scale, acc[i + 3] * scale);
      } else {
        uint16_t* orow = static_cast<uint16_t*>(p.o) + b * p.osb + h * p.osh + qrow * p.ost + c * 16;
#pragma unroll
        for (int i = 0; i < 16; i += 8) {
          uint32_t w4[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float a0 = acc[i + 2 * t] * scale, a1 = acc[i + 2 * t + 1] * scale;
            if (p.o_dtype == SWV_BF16) {
              w4[t] = pack_bf16x2(a0, a1);
            } else {
              const __half2 h2 = __floats2half2_rn(a0, a1);
              w4[t] = *reinterpret_cast<const uint32_t*>(&h2);
            }
          }
          *reinterpret_cast<uint4*>(orow + i) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
        }
      }
    };

    if constexpr (!kSplit) {
      bool bad = false;
      if (active && ok) {
        uint32_t lc[16];
        tmem_ld16(o_col + kLD, lc);
        tc_wait_ld();
        const float l = __uint_as_float(lc[0]);
        bad = row_ok && l > 0.f && l < 1e-6f;
        const float scale = l > 0.f ? 1.f / l : 0.f;
        for (int c = 0; c < kLD / 16; ++c) {
          uint32_t o[16];
          tmem_ld16(o_col + c * 16, o);
          tc_wait_ld();
          if (!row_ok) continue;
          float acc[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = __uint_as_float(o[i]);
          store_chunk(c, acc, scale);
        }
      }
      if (__any_sync(0xffffffffu, bad) && lane == 0) p.flags[cta] = 1u;
    } else {
      // every part leaves its unnormalised rows (row sum in column 64); the last one to arrive merges
      const size_t rec_stride = static_cast<size_t>(2) * kTile * kLRec;          // floats per part
      float* rec0 = p.scratch + static_cast<size_t>(cta) * p.split * rec_stride +
                    (static_cast<size_t>(x) * kTile + row) * kLRec;
      if (active && ok) {
        float* mine = rec0 + part * rec_stride;
        for (int c = 0; c < kLNO / 16; ++c) {
          uint32_t o[16];
          tmem_ld16(o_col + c * 16, o);
          tc_wait_ld();
          if (c == kLD / 16) {
            mine[kLD] = __uint_as_float(o[0]);
          } else {
#pragma unroll
            for (int i = 0; i < 16; i += 4)
              *reinterpret_cast<float4*>(mine + c * 16 + i) =
                  make_float4(__uint_as_float(o[i]), __uint_as_float(o[i + 1]), __uint_as_float(o[i + 2]),
                              __uint_as_float(o[i + 3]));
          }
        }
      }
      __threadfence();
      asm volatile("bar.sync 2, %0;" ::"r"(kLSoft) : "memory");
      if (threadIdx.x == 64) ctl->ticket = atomicAdd(p.tickets + cta, 1u);
      asm volatile("bar.sync 2, %0;" ::"r"(kLSoft) : "memory");
      if (*reinterpret_cast<volatile uint32_t*>(&ctl->ticket) == static_cast<uint32_t>(p.split - 1)) {
        __threadfence();
        if (threadIdx.x == 64) p.tickets[cta] = 0u;
        bool bad = false;
        if (row_ok && *abort_flag == 0u) {
          // all parts of a row share its constant stabiliser: plain sums
          float l_all = 0.f;
          for (int q = 0; q < p.split; ++q) l_all += __ldcg(rec0 + q * rec_stride + kLD);
          bad = l_all > 0.f && l_all < 1e-6f;
          const float scale = l_all > 0.f ? 1.f / l_all : 0.f;
          for (int c = 0; c < kLD / 16; ++c) {
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = 0.f;
            for (int q = 0; q < p.split; ++q) {
              const float* src = rec0 + q * rec_stride + c * 16;
#pragma unroll
              for (int i = 0; i < 16; i += 4) {
                const float4 v4 = __ldcg(reinterpret_cast<const float4*>(src + i));
                acc[i] += v4.x;
                acc[i + 1] += v4.y;
                acc[i + 2] += v4.z;
                acc[i + 3] += v4.w;
              }
            }
            store_chunk(c, acc, scale);
          }
        }
        if (__any_sync(0xffffffffu, bad) && lane == 0) p.flags[cta] = 1u;
      }
    }
  }

  // ---------------------------------------------------------------- teardown
#ifdef SWV_PROFILE
  const long long t_cta2 = clock64();
#endif
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, kLTmemCols);
  }
#ifdef SWV_PROFILE
  if (threadIdx.x == 64) {      // a softmax thread: [prologue, main + epilogue of this thread, teardown wait], CTA count
    atomicAdd(&g_lists_prof[56], static_cast<unsigned long long>(t_cta1 - t_cta0));
    atomicAdd(&g_lists_prof[57], static_cast<unsigned long long>(t_cta2 - t_cta1));
    atomicAdd(&g_lists_prof[58], static_cast<unsigned long long>(clock64() - t_cta2));
    atomicAdd(&g_lists_prof[59], 1ull);
  }
#endif
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
size_t align256(size_t x) { return (x + 255) / 256 * 256; }

// Capacity of one (query tile, key tile) list: the expected number of selected pairs plus a margin;
// a tile that holds more sends its query tile to the masked kernel.
int tile_list_capacity(int Tk, int top_k) {
  const double n_valid = top_k < Tk ? top_k : Tk;
  const double mean = static_cast<double>(kTile) * kTile * n_valid / Tk;
  int cap = static_cast<int>(mean * 1.25) + 128;
  cap = (cap + 63) / 64 * 64;
  return cap > kTile * kTile ? kTile * kTile : cap;
}

struct ListScratch {
  size_t flags_off, over_off, cnt_off, ent_off, inner_off, inner_bytes, total;
  int cap;
};
ListScratch list_scratch_layout(int B, int H, int Tq, int Tk, int top_k) {
  ListScratch L;
  const size_t nQT = (Tq + kTile - 1) / kTile, nKT = (Tk + kTile - 1) / kTile;
  const size_t ctas = static_cast<size_t>(B) * nQT * ((H + 1) / 2);
  L.cap = tile_list_capacity(Tk, top_k);
  size_t off = 0;
  L.flags_off = off;  off += align256(ctas * 4);
  L.over_off = off;   off += align256(static_cast<size_t>(B) * nQT * 4);
  L.cnt_off = off;    off += align256(static_cast<size_t>(B) * nQT * nKT * 4);
  L.ent_off = off;    off += align256(static_cast<size_t>(B) * nQT * nKT * L.cap * 8);
  L.inner_off = off;
  L.inner_bytes = 0;
  dsa_attn_scratch_bytes_impl(B, H, Tq, Tk, &L.inner_bytes);
  L.total = off + L.inner_bytes;
  return L;
}

}  // namespace

// scratch = [flags: one word per (batch, query tile, head pair)] [overflow word per query tile]
// [tile-list counts] [tile-list entries] [the scratch of the masked kernel: tickets + per-part records,
// shared by both kernels, which never run at the same time]
int dsa_attn_lists_scratch_bytes_impl(int B, int H, int Tq, int Tk, int top_k, size_t* bytes) {
  if (!bytes) return SWV_ERR_NULL;
  if (B < 1 || H < 1 || Tq < 1 || Tk < 1 || top_k < 1) return SWV_ERR_SHAPE;
  *bytes = list_scratch_layout(B, H, Tq, Tk, top_k).total;
  return SWV_OK;
}

int dsa_attn_lists_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                        const int64_t* vs, const int32_t* idx, const float* rw, int top_k, const uint32_t* maskbits,
                        void* workspace, void* o, const int64_t* os, int o_dtype, int B, int H, int Tq, int Tk, int D,
                        void* scratch, size_t scratch_bytes, int* status, cudaStream_t st) {
  if (!q || !k || !v || !idx || !rw || !maskbits || !workspace || !o || !status || !scratch || !qs || !ks || !vs || !os)
    return SWV_ERR_NULL;
  if (B < 1 || H < 1 || Tq < 1 || Tk < 1 || top_k < 1) return SWV_ERR_SHAPE;
  if (D != kLD || (top_k & 3) != 0) return SWV_ERR_UNSUPPORTED;
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
  if (!aligned16(idx) || !aligned16(rw) || !aligned16(maskbits)) return SWV_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(scratch) & 255)) return SWV_ERR_ALIGN;
  if (static_cast<int64_t>(B) * H > 1024) return SWV_ERR_UNSUPPORTED;
  const ListScratch L = list_scratch_layout(B, H, Tq, Tk, top_k);
  if (scratch_bytes < L.total) return SWV_ERR_WORKSPACE;

  float *wq = nullptr, *wk = nullptr;
  uint32_t *st_prefix = nullptr, *st_kth = nullptr, *st_neq = nullptr, *kmax2 = nullptr;
  int32_t* st_excl = nullptr;
  dsa_workspace_views(workspace, B, Tq, Tk, &wq, &wk, &st_prefix, &st_kth, &st_neq, &kmax2, &st_excl);

  CUtensorMap tm_k, tm_v;
  int rc = make_tmap_4d(&tm_k, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, Tk, H, B, ks[2] * 2, ks[1] * 2, ks[0] * 2, kLD,
                        kTile);
  if (rc != SWV_OK) return rc;
  rc = make_tmap_4d(&tm_v, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, D, Tk, H, B, vs[2] * 2, vs[1] * 2, vs[0] * 2, kLD, kTile);
  if (rc != SWV_OK) return rc;

  uint8_t* sb = static_cast<uint8_t*>(scratch);
  ListParams p;
  p.B = B; p.H = H; p.Tq = Tq; p.Tk = Tk;
  p.nQT = (Tq + kTile - 1) / kTile;
  p.nKT = (Tk + kTile - 1) / kTile;
  p.nHP = (H + 1) / 2;
  p.q = static_cast<const __nv_bfloat16*>(q); p.qsb = qs[0]; p.qsh = qs[1]; p.qst = qs[2];
  p.cap = L.cap;
  uint32_t* tl_cnt = reinterpret_cast<uint32_t*>(sb + L.cnt_off);
  uint2* tl_ent = reinterpret_cast<uint2*>(sb + L.ent_off);
  uint32_t* tl_over = reinterpret_cast<uint32_t*>(sb + L.over_off);
  p.tl_cnt = tl_cnt; p.tl_ent = tl_ent; p.tl_over = tl_over;
  p.kmax2 = kmax2;
  p.o = o; p.osb = os[0]; p.osh = os[1]; p.ost = os[2]; p.o_dtype = o_dtype;
  p.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(D));
  p.status = status;
  const size_t ctas = static_cast<size_t>(B) * p.nQT * p.nHP;
  p.flags = reinterpret_cast<uint32_t*>(sb + L.flags_off);
  uint8_t* inner = sb + L.inner_off;
  p.split = L.inner_bytes > 0 ? dsa_attn_split_factor(B, H, Tq, Tk) : 1;
  p.tickets = reinterpret_cast<uint32_t*>(inner);
  p.scratch = reinterpret_cast<float*>(inner + align256(ctas * 4));
  SWV_CUDA_OK(cudaMemsetAsync(p.flags, 0, ctas * 4, st));
  if (p.split > 1) SWV_CUDA_OK(cudaMemsetAsync(p.tickets, 0, ctas * 4, st));

  // the per-tile lists from the per-row lists
  const int n_valid = top_k < Tk ? top_k : Tk;
  if (static_cast<size_t>(p.nKT) * 4 > 48 * 1024) return SWV_ERR_TOO_LARGE;
  // one thread per row once there are two query tiles per SM (more threads per row spread the writes of
  // a query tile over more key tiles at a time: measured slower at 512 query tiles), more with fewer
  int parts = (2 * sm_count() + B * p.nQT - 1) / (B * p.nQT);
  parts = parts < 1 ? 1 : (parts > 8 ? 8 : parts);
  dsa_tile_lists_kernel<<<static_cast<unsigned>(B) * p.nQT, kTile * parts, static_cast<size_t>(p.nKT) * 4, st>>>(
      idx, rw, top_k, n_valid, Tq, p.nQT, p.nKT, L.cap, parts, tl_cnt, tl_ent, tl_over);
  SWV_CUDA_OK(cudaGetLastError());
  rc = dsa_key_norm_max(k, ks, B, H, Tk, kmax2, st);
  if (rc != SWV_OK) return rc;

  const unsigned grid = static_cast<unsigned>(ctas) * p.split;
  if (p.split == 1) {
    SWV_CUDA_OK(cudaFuncSetAttribute(dsa_attn_lists_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(lists_smem_bytes())));
    dsa_attn_lists_kernel<false><<<grid, kLThreads, lists_smem_bytes(), st>>>(tm_k, tm_v, p);
  } else {
    SWV_CUDA_OK(cudaFuncSetAttribute(dsa_attn_lists_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(lists_smem_bytes())));
    dsa_attn_lists_kernel<true><<<grid, kLThreads, lists_smem_bytes(), st>>>(tm_k, tm_v, p);
  }
  SWV_CUDA_OK(cudaGetLastError());
  // (query tile, head pair)s the list kernel left out: a logit bound too large for the constant
  // stabiliser, a tile list over capacity, or a row whose weights are small enough for the clamp
  return dsa_attn_masked_impl(q, qs, k, ks, v, vs, maskbits, workspace, o, os, o_dtype, B, H, Tq, Tk, D,
                              L.inner_bytes > 0 ? inner : nullptr, L.inner_bytes, status, st, nullptr, p.flags);
}

}  // namespace swv

#ifdef SWV_PROFILE
// Profiling build only: copies the 64 phase counters of dsa_attn_lists_kernel to `out_host`
// (synchronises the device) and clears them when `reset` is non-zero.
extern "C" int swv_debug_lists_profile(unsigned long long* out_host, int reset) {
  if (cudaDeviceSynchronize() != cudaSuccess) return SWV_ERR_CUDA;
  if (out_host != nullptr &&
      cudaMemcpyFromSymbol(out_host, swv::g_lists_prof, sizeof(unsigned long long) * 64) != cudaSuccess)
    return SWV_ERR_CUDA;
  if (reset) {
    static const unsigned long long zeros[64] = {0};
    if (cudaMemcpyToSymbol(swv::g_lists_prof, zeros, sizeof(zeros)) != cudaSuccess) return SWV_ERR_CUDA;
  }
  return SWV_OK;
}
#endif
