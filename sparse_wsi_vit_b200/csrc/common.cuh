// Shared host/device helpers: error codes, the device status word protocol,
// bounded waits with a CTA-wide abort flag, TMA descriptor encoding.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/swv_b200.h"
#include "ptx.cuh"

namespace swv {

constexpr int kTile = 128;        // query rows and key columns per score tile
constexpr int kIdxDim = 64;       // padded reduction depth of the indexer
constexpr int kMaxExcl = 4;       // ties at a row's threshold that are cut by key index: the unselected ones are
                                  // listed per row (up to this many) for the attention sweep
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // 1 s per wait, then give up

// Device status codes (written once, first error wins).
enum DeviceStatus : int {
  kDevOk = 0,
  kDevWaitTmaFull = 101,
  kDevWaitStageEmpty = 102,
  kDevWaitAccFull = 103,
  kDevWaitAccEmpty = 104,
  kDevWaitPReady = 105,
  kDevWaitPvDone = 106,
  kDevWaitQ = 107,
  kDevBadIndex = 120,
};

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void record_status(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// Bounds check of an index taken from a caller-supplied list.  In the checked build (-DSWV_CHECKS,
// `build.py --checks`, which writes libswv_b200_checked.so) an index outside [0, n) is reported
// through the status word as kDevBadIndex and replaced by 0, so nothing is accessed through it;
// the release build trusts the list.  This build is the stand-in for a memory checker on machines
// where none may be run.
__device__ __forceinline__ int checked_index(int i, int n, int* status) {
#ifdef SWV_CHECKS
  if (i < 0 || i >= n) {
    record_status(status, kDevBadIndex);
    return 0;
  }
#endif
  return i;
}

// Bounded mbarrier wait.  Gives up after kWaitLimitNs or as soon as another
// thread of the CTA raised `abort_flag`; on its own timeout raises the flag.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag != 0u) return false;
    if (globaltimer_ns() - t0 > kWaitLimitNs) {
      *abort_flag = 1u;
      return false;
    }
  }
}

// ---------------------------------------------------------------- host side
#define SWV_CUDA_OK(expr)                                   \
  do {                                                      \
    cudaError_t _e = (expr);                                \
    if (_e != cudaSuccess) return SWV_ERR_CUDA;             \
  } while (0)

// Number of SMs of the current device (cached), used to decide when a small grid should divide
// the key range; 148 (B200) when no device can be asked, e.g. a size query on a machine without one.
inline int sm_count() {
  static int cached = 0;
  if (cached > 0) return cached;
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) == cudaSuccess &&
      cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) {
    cached = n;
    return n;
  }
  (void)cudaGetLastError();
  return 148;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Resolves cuTensorMapEncodeTiled through the runtime so the library has no
// link-time dependency on libcuda (it must load on a machine without a driver).
inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// rank-3 tiled map with 128-byte swizzle.  dims/strides innermost first; the
// innermost stride is implicit (dense), strides[0..1] are BYTES for dims 1..2.
inline int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint64_t d0, uint64_t d1,
                        uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return SWV_ERR_CUDA;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SWV_OK : SWV_ERR_TENSORMAP;
}

// rank-4 tiled map (d, t, h, b) with 128-byte swizzle; strides in BYTES for dims 1..3.
inline int make_tmap_4d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint64_t d0, uint64_t d1,
                        uint64_t d2, uint64_t d3, uint64_t s1, uint64_t s2, uint64_t s3, uint32_t box0,
                        uint32_t box1) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return SWV_ERR_CUDA;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {s1, s2, s3};
  cuuint32_t box[4] = {box0, box1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SWV_OK : SWV_ERR_TENSORMAP;
}

}  // namespace swv
