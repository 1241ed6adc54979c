// extern "C" surface of libswv_b200.so (declared in include/swv_b200.h).
// Plain pointers and sizes only; every function validates its arguments before
// enqueuing work and never allocates or synchronises.
#include "common.cuh"

namespace swv {
int dsa_workspace_bytes_impl(int B, int Tq, int Tk, size_t* bytes);
int dsa_workspace_bytes_topk_impl(int B, int Tq, int Tk, int top_k, size_t* bytes);
int dsa_mask_bytes_impl(int B, int Tq, int Tk, size_t* bytes);
int dsa_indexer_topk_impl(const void* q_idx, const int64_t* qs, const void* k_idx, const int64_t* ks, int dtype,
                          const float* w, int B, int Tq, int Tk, int IH, int ID, int top_k, int32_t* idx,
                          float* valid, float* scores, uint32_t* maskbits, void* workspace, size_t workspace_bytes,
                          int* status, cudaStream_t st, bool allow_split);
int dsa_indexer_topk_static_impl(const void* q_idx, const int64_t* qs, const void* k_idx, const int64_t* ks,
                                 int dtype, const float* w, int B, int Tq, int Tk, int IH, int ID, int top_k,
                                 int32_t* idx, float* valid, float* scores, uint32_t* maskbits, int* status,
                                 cudaStream_t st);
int dsa_attn_masked_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                         const int64_t* vs, const uint32_t* maskbits, void* workspace, void* o,
                         const int64_t* os, int o_dtype, int B, int H, int Tq, int Tk, int D, void* scratch,
                         size_t scratch_bytes, int* status, cudaStream_t st, int* member_count,
                         const uint32_t* only_flagged);
int dsa_attn_scratch_bytes_impl(int B, int H, int Tq, int Tk, size_t* bytes);
int dsa_attn_lists_scratch_bytes_impl(int B, int H, int Tq, int Tk, int top_k, size_t* bytes);
int dsa_attn_lists_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                        const int64_t* vs, const int32_t* idx, const float* rw, int top_k, const uint32_t* maskbits,
                        void* workspace, void* o, const int64_t* os, int o_dtype, int B, int H, int Tq, int Tk, int D,
                        void* scratch, size_t scratch_bytes, int* status, cudaStream_t st);
int dsa_attn_gather_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                         const int64_t* vs, int dtype, const int32_t* idx, const int64_t* is, const float* valid,
                         const int64_t* vls, const float* rw, const int64_t* rs, void* o, const int64_t* os,
                         int o_dtype, int B, int H, int Tq, int Tk, int D, int top_k, int kv_group, int* status,
                         cudaStream_t st);
int block_sparse_attn_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                           const int64_t* vs, const int32_t* row_ptr, const int32_t* col_idx, int block, int mode,
                           int num_cls, int window, int dilation, int kv_group, float* lse, void* o,
                           const int64_t* os, int o_dtype, int B, int H, int Tq, int Tk, int D, int* status,
                           cudaStream_t st, const float* gate, int gate_idx, const float* acc_in);
int pool_tokens_impl(const void* x, const int64_t* xs, void* y, int B, int H, int T, int D, int win, int stride,
                     cudaStream_t st);
int rope2d_impl(const void* x, const int64_t* xs, void* y, const int64_t* ys, int dtype, const float* coords,
                int64_t L, int H, int hd, float coord_high, float theta, int skip, cudaStream_t st);
int nsa_importance_bytes_impl(int B, int Hkv, int Tq, int nC, int cmp_stride, int sel_block, size_t* bytes);
int nsa_select_blocks_impl(const void* q, const int64_t* qs, const void* kc, const int64_t* kcs, const float* lse,
                           int B, int Hq, int Hkv, int Tq, int Tk, int nC, int D, int cmp_stride, int sel_block,
                           int n_sel, float* importance, size_t importance_bytes, int32_t* blocks, int* status,
                           cudaStream_t st);
int nsa_selected_attn_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                           const int64_t* vs, const int32_t* blocks, int B, int Hq, int Hkv, int Tq, int Tk, int D,
                           int sel_block, int n_sel, float* o, cudaStream_t st, const float* gate);
int nsa_combine_impl(const float* o_cmp, const float* o_sel, const float* o_win, const float* gate, void* out,
                     int out_dtype, int B, int Hq, int T, int D, cudaStream_t st);
int dsa_attn_bwd_impl(const void* d_out, const int64_t* dos, const void* q, const int64_t* qs, const void* k,
                      const int64_t* ks, const void* v, const int64_t* vs, int dtype, const void* o,
                      const int64_t* os, int o_dtype, const int32_t* idx, const int64_t* is, const float* valid,
                      const int64_t* vls, const float* rw, const int64_t* rs, float* dq, float* dk, float* dv,
                      float* drw, int B, int H, int Tq, int Tk, int D, int top_k, int* status, cudaStream_t st);
int dsa_indexer_bwd_impl(const float* d_scores, const int64_t* dss, const void* q_idx, const int64_t* qs,
                         const void* k_idx, const int64_t* ks, int dtype, const float* w, const int32_t* idx,
                         const int64_t* is, const float* valid, const int64_t* vls, float* dq, float* dk, float* dw,
                         int B, int Tq, int Tk, int IH, int ID, int top_k, int* status, cudaStream_t st);
int dsa_prologue_impl(void* q, const int64_t* qs, void* k, const int64_t* ks, int qk_dtype, const void* q_idx,
                      const int64_t* qis, const void* k_idx, const int64_t* kis, int idx_dtype, const float* w,
                      const float* coords, float coord_high, float theta, int skip, int B, int T, int H, int D, int IH,
                      int ID, void* workspace, size_t workspace_bytes, cudaStream_t st);
int nsa_workspace_bytes_impl(int B, int Hq, int Hkv, int T, int D, int cmp_block, int cmp_stride, int sel_block,
                             int n_sel, int window, size_t* bytes);
int nsa_attn_impl(const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
                  const int64_t* vs, const float* gate, void* out, int out_dtype, int B, int Hq, int Hkv, int T,
                  int D, int cmp_block, int cmp_stride, int sel_block, int n_sel, int window, void* workspace,
                  size_t workspace_bytes, int32_t* blocks_out, int* status, cudaStream_t st);
}  // namespace swv

extern "C" {

int swv_version(void) { return 102; }

const char* swv_strerror(int code) {
  switch (code) {
    case SWV_OK: return "ok";
    case SWV_ERR_NULL: return "a required pointer is NULL";
    case SWV_ERR_ALIGN: return "pointer or stride alignment not supported (need 16-byte aligned rows, unit inner stride)";
    case SWV_ERR_DTYPE: return "unsupported element type";
    case SWV_ERR_SHAPE: return "non-positive or unsupported size";
    case SWV_ERR_WORKSPACE: return "workspace or mask buffer too small";
    case SWV_ERR_CUDA: return "a CUDA runtime call failed";
    case SWV_ERR_TENSORMAP: return "the driver rejected a TMA descriptor";
    case SWV_ERR_UNSUPPORTED: return "no kernel in this build for the requested shape";
    case SWV_ERR_TOO_LARGE: return "size beyond the fixed capacity of this entry point (8192 tokens)";
    case swv::kDevWaitTmaFull: return "device: timed out waiting for a TMA tile";
    case swv::kDevWaitStageEmpty: return "device: timed out waiting for a free shared-memory stage";
    case swv::kDevWaitAccFull: return "device: timed out waiting for an accumulator tile";
    case swv::kDevWaitAccEmpty: return "device: timed out waiting for a free accumulator";
    case swv::kDevWaitPReady: return "device: timed out waiting for the probability tile";
    case swv::kDevWaitPvDone: return "device: timed out waiting for the PV product";
    case swv::kDevWaitQ: return "device: timed out waiting for the query tile";
    case swv::kDevBadIndex: return "device: key index out of range";
    default: return "unknown code";
  }
}

int swv_dsa_workspace_bytes(int B, int Tq, int Tk, size_t* bytes) {
  return swv::dsa_workspace_bytes_impl(B, Tq, Tk, bytes);
}

int swv_dsa_workspace_bytes_topk(int B, int Tq, int Tk, int top_k, size_t* bytes) {
  return swv::dsa_workspace_bytes_topk_impl(B, Tq, Tk, top_k, bytes);
}

int swv_dsa_mask_bytes(int B, int Tq, int Tk, size_t* bytes) { return swv::dsa_mask_bytes_impl(B, Tq, Tk, bytes); }

int swv_dsa_indexer_topk_fwd(const void* q_idx, const int64_t q_strides[4], const void* k_idx,
                             const int64_t k_strides[4], int idx_dtype, const float* w, int B, int Tq, int Tk,
                             int IH, int ID, int top_k, int32_t* idx, float* valid, float* scores,
                             uint32_t* maskbits, void* workspace, size_t workspace_bytes, int* status,
                             void* stream) {
  return swv::dsa_indexer_topk_impl(q_idx, q_strides, k_idx, k_strides, idx_dtype, w, B, Tq, Tk, IH, ID, top_k, idx,
                                    valid, scores, maskbits, workspace, workspace_bytes, status,
                                    static_cast<cudaStream_t>(stream), /*allow_split=*/true);
}

// The variant for callers that cannot allocate: the scratch is a fixed device array inside the
// library (see the header for who needs this and for its limits).
int swv_dsa_indexer_topk_static_fwd(const void* q_idx, const int64_t q_strides[4], const void* k_idx,
                                    const int64_t k_strides[4], int idx_dtype, const float* w, int B, int Tq,
                                    int Tk, int IH, int ID, int top_k, int32_t* idx, float* valid, float* scores,
                                    uint32_t* maskbits, int* status, void* stream) {
  return swv::dsa_indexer_topk_static_impl(q_idx, q_strides, k_idx, k_strides, idx_dtype, w, B, Tq, Tk, IH, ID, top_k,
                                           idx, valid, scores, maskbits, status, static_cast<cudaStream_t>(stream));
}

int swv_dsa_attn_gather_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                            const void* v, const int64_t v_strides[4], int qkv_dtype, const int32_t* idx,
                            const int64_t idx_strides[3], const float* valid, const int64_t valid_strides[3],
                            const float* rw, const int64_t rw_strides[3], void* o, const int64_t o_strides[4],
                            int o_dtype, int B, int H, int Tq, int Tk, int D, int top_k, int kv_group,
                            int* status, void* stream) {
  return swv::dsa_attn_gather_impl(q, q_strides, k, k_strides, v, v_strides, qkv_dtype, idx, idx_strides, valid,
                                   valid_strides, rw, rw_strides, o, o_strides, o_dtype, B, H, Tq, Tk, D, top_k,
                                   kv_group, status, static_cast<cudaStream_t>(stream));
}

int swv_dsa_attn_bwd(const void* d_out, const int64_t d_out_strides[4], const void* q, const int64_t q_strides[4],
                     const void* k, const int64_t k_strides[4], const void* v, const int64_t v_strides[4], int qkv_dtype,
                     const void* o, const int64_t o_strides[4], int o_dtype, const int32_t* idx,
                     const int64_t idx_strides[3], const float* valid, const int64_t valid_strides[3], const float* rw,
                     const int64_t rw_strides[3], float* dq, float* dk, float* dv, float* drw, int B, int H, int Tq,
                     int Tk, int D, int top_k, int* status, void* stream) {
  return swv::dsa_attn_bwd_impl(d_out, d_out_strides, q, q_strides, k, k_strides, v, v_strides, qkv_dtype, o, o_strides,
                                o_dtype, idx, idx_strides, valid, valid_strides, rw, rw_strides, dq, dk, dv, drw, B, H,
                                Tq, Tk, D, top_k, status, static_cast<cudaStream_t>(stream));
}

int swv_dsa_indexer_bwd(const float* d_scores, const int64_t d_scores_strides[3], const void* q_idx,
                        const int64_t q_strides[4], const void* k_idx, const int64_t k_strides[4], int idx_dtype,
                        const float* w, const int32_t* idx, const int64_t idx_strides[3], const float* valid,
                        const int64_t valid_strides[3], float* dq_idx, float* dk_idx, float* dw, int B, int Tq, int Tk,
                        int IH, int ID, int top_k, int* status, void* stream) {
  return swv::dsa_indexer_bwd_impl(d_scores, d_scores_strides, q_idx, q_strides, k_idx, k_strides, idx_dtype, w, idx,
                                   idx_strides, valid, valid_strides, dq_idx, dk_idx, dw, B, Tq, Tk, IH, ID, top_k,
                                   status, static_cast<cudaStream_t>(stream));
}

int swv_dsa_prologue_fwd(void* q, const int64_t q_strides[4], void* k, const int64_t k_strides[4], int qk_dtype,
                         const void* q_idx, const int64_t qi_strides[4], const void* k_idx, const int64_t ki_strides[4],
                         int idx_dtype, const float* w, const float* coords, float coord_high, float theta,
                         int skip_tokens, int B, int T, int H, int D, int IH, int ID, void* workspace,
                         size_t workspace_bytes, void* stream) {
  return swv::dsa_prologue_impl(q, q_strides, k, k_strides, qk_dtype, q_idx, qi_strides, k_idx, ki_strides, idx_dtype, w,
                                coords, coord_high, theta, skip_tokens, B, T, H, D, IH, ID, workspace, workspace_bytes,
                                static_cast<cudaStream_t>(stream));
}

int swv_dsa_attn_scratch_bytes(int B, int H, int Tq, int Tk, size_t* bytes) {
  return swv::dsa_attn_scratch_bytes_impl(B, H, Tq, Tk, bytes);
}

int swv_dsa_attn_masked_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                            const void* v, const int64_t v_strides[4], const uint32_t* maskbits,
                            void* workspace, void* o, const int64_t o_strides[4], int o_dtype, int B, int H,
                            int Tq, int Tk, int D, void* scratch, size_t scratch_bytes, int* status, void* stream) {
  return swv::dsa_attn_masked_impl(q, q_strides, k, k_strides, v, v_strides, maskbits, workspace, o, o_strides,
                                   o_dtype, B, H, Tq, Tk, D, scratch, scratch_bytes, status,
                                   static_cast<cudaStream_t>(stream), nullptr, nullptr);
}

int swv_dsa_attn_lists_scratch_bytes(int B, int H, int Tq, int Tk, int top_k, size_t* bytes) {
  return swv::dsa_attn_lists_scratch_bytes_impl(B, H, Tq, Tk, top_k, bytes);
}

int swv_dsa_attn_lists_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                           const void* v, const int64_t v_strides[4], const int32_t* idx, const float* rw, int top_k,
                           const uint32_t* maskbits, void* workspace, void* o, const int64_t o_strides[4], int o_dtype,
                           int B, int H, int Tq, int Tk, int D, void* scratch, size_t scratch_bytes, int* status,
                           void* stream) {
  return swv::dsa_attn_lists_impl(q, q_strides, k, k_strides, v, v_strides, idx, rw, top_k, maskbits, workspace, o,
                                  o_strides, o_dtype, B, H, Tq, Tk, D, scratch, scratch_bytes, status,
                                  static_cast<cudaStream_t>(stream));
}

int swv_dsa_attn_masked_count_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                                  const void* v, const int64_t v_strides[4], const uint32_t* maskbits, void* workspace,
                                  void* o, const int64_t o_strides[4], int o_dtype, int B, int H, int Tq, int Tk, int D,
                                  int32_t* member_count, int* status, void* stream) {
  if (member_count == nullptr) return SWV_ERR_NULL;
  return swv::dsa_attn_masked_impl(q, q_strides, k, k_strides, v, v_strides, maskbits, workspace, o, o_strides,
                                   o_dtype, B, H, Tq, Tk, D, nullptr, 0, status, static_cast<cudaStream_t>(stream),
                                   member_count, nullptr);
}

int swv_block_sparse_attn_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                              const void* v, const int64_t v_strides[4], const int32_t* row_ptr,
                              const int32_t* col_idx, int block, int mode, int num_cls, int window, int dilation,
                              int kv_group, float* lse, void* o, const int64_t o_strides[4], int o_dtype, int B,
                              int H, int Tq, int Tk, int D, int* status, void* stream) {
  return swv::block_sparse_attn_impl(q, q_strides, k, k_strides, v, v_strides, row_ptr, col_idx, block, mode, num_cls,
                                     window, dilation, kv_group, lse, o, o_strides, o_dtype, B, H, Tq, Tk, D, status,
                                     static_cast<cudaStream_t>(stream), nullptr, 0, nullptr);
}

int swv_pool_tokens(const void* x, const int64_t x_strides[4], void* y, int B, int H, int T, int D, int window,
                    int stride, void* stream) {
  return swv::pool_tokens_impl(x, x_strides, y, B, H, T, D, window, stride, static_cast<cudaStream_t>(stream));
}

int swv_rope2d_apply(const void* x, const int64_t x_strides[3], void* y, const int64_t y_strides[3], int dtype,
                     const float* coords, int64_t L, int H, int head_dim, float coord_high, float theta,
                     int skip_tokens, void* stream) {
  return swv::rope2d_impl(x, x_strides, y, y_strides, dtype, coords, L, H, head_dim, coord_high, theta, skip_tokens,
                          static_cast<cudaStream_t>(stream));
}

int swv_nsa_importance_bytes(int B, int Hkv, int Tq, int nC, int cmp_stride, int sel_block, size_t* bytes) {
  return swv::nsa_importance_bytes_impl(B, Hkv, Tq, nC, cmp_stride, sel_block, bytes);
}

int swv_nsa_select_blocks_fwd(const void* q, const int64_t q_strides[4], const void* kc, const int64_t kc_strides[4],
                              const float* lse, int B, int Hq, int Hkv, int Tq, int Tk, int nC, int D,
                              int cmp_stride, int sel_block, int n_sel, float* importance, size_t importance_bytes,
                              int32_t* blocks, int* status, void* stream) {
  return swv::nsa_select_blocks_impl(q, q_strides, kc, kc_strides, lse, B, Hq, Hkv, Tq, Tk, nC, D, cmp_stride,
                                     sel_block, n_sel, importance, importance_bytes, blocks, status,
                                     static_cast<cudaStream_t>(stream));
}

int swv_nsa_selected_attn_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                              const void* v, const int64_t v_strides[4], const int32_t* blocks, int B, int Hq,
                              int Hkv, int Tq, int Tk, int D, int sel_block, int n_sel, float* o, void* stream) {
  return swv::nsa_selected_attn_impl(q, q_strides, k, k_strides, v, v_strides, blocks, B, Hq, Hkv, Tq, Tk, D,
                                     sel_block, n_sel, o, static_cast<cudaStream_t>(stream), nullptr);
}

int swv_nsa_combine_fwd(const float* o_cmp, const float* o_sel, const float* o_win, const float* gate, void* out,
                        int out_dtype, int B, int Hq, int T, int D, void* stream) {
  return swv::nsa_combine_impl(o_cmp, o_sel, o_win, gate, out, out_dtype, B, Hq, T, D,
                               static_cast<cudaStream_t>(stream));
}

int swv_nsa_workspace_bytes(int B, int Hq, int Hkv, int T, int D, int cmp_block, int cmp_stride, int sel_block,
                            int n_sel, int window, size_t* bytes) {
  return swv::nsa_workspace_bytes_impl(B, Hq, Hkv, T, D, cmp_block, cmp_stride, sel_block, n_sel, window, bytes);
}

int swv_nsa_attn_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                     const void* v, const int64_t v_strides[4], const float* gate, void* out, int out_dtype, int B,
                     int Hq, int Hkv, int T, int D, int cmp_block, int cmp_stride, int sel_block, int n_sel,
                     int window, void* workspace, size_t workspace_bytes, int32_t* blocks_out, int* status,
                     void* stream) {
  return swv::nsa_attn_impl(q, q_strides, k, k_strides, v, v_strides, gate, out, out_dtype, B, Hq, Hkv, T, D,
                            cmp_block, cmp_stride, sel_block, n_sel, window, workspace, workspace_bytes, blocks_out,
                            status, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
