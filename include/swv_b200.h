/* C ABI of the B200 sparse-attention forward path (libswv_b200.so).
 *
 * The reference project (p-adema/sparse-wsi-vit) has no FFI layer: its operator
 * boundary is two torch.autograd.Function classes that launch Triton kernels.
 * Each entry point below replaces the device work of one of those launches and
 * cites it as  <file>:<lines>  with
 *   K = src/sparse_wsi_vit/models/deepseek_sparse_attention_kernels/kernels.py
 *   M = src/sparse_wsi_vit/models/deepseek_sparse_attention.py
 *
 * Conventions
 *   - All pointers are DEVICE pointers unless the name ends in `_host`.
 *   - Strides are in ELEMENTS (not bytes), int64, order given per argument.
 *   - The caller owns every buffer (inputs, outputs, workspace, status word);
 *     no entry point allocates, frees or synchronises.  Work is enqueued on
 *     `stream` (a cudaStream_t passed as void*).
 *   - Return value: 0 on success, a negative SWV_ERR_* when an argument is
 *     rejected before anything is launched.
 *   - `status` points to one int32 in device memory, zeroed by the caller.
 *     Kernels write a positive code there when a bounded device-side wait gave
 *     up (see swv_strerror); the results of that call are then undefined.
 *   - Re-entrant; no global mutable state -- with ONE exception,
 *     swv_dsa_indexer_topk_static_fwd, whose scratch is a device array inside the
 *     library (see its comment).  Calls sharing a workspace, a mask buffer or a
 *     status word must be ordered on the GPU by the caller.
 *     swv_dsa_attn_masked_fwd writes the per-(batch, head) key-norm maxima into the
 *     indexer workspace it is given: two attention calls on one workspace must be ordered too.
 */
#ifndef SWV_B200_H_
#define SWV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SWV_OK 0
#define SWV_ERR_NULL (-1)        /* a required pointer is NULL                      */
#define SWV_ERR_ALIGN (-2)       /* pointer/stride alignment the kernels cannot take */
#define SWV_ERR_DTYPE (-3)       /* unsupported element type                        */
#define SWV_ERR_SHAPE (-4)       /* non-positive or unsupported size                */
#define SWV_ERR_WORKSPACE (-5)   /* workspace / mask buffer too small               */
#define SWV_ERR_CUDA (-6)        /* a CUDA runtime call failed                      */
#define SWV_ERR_TENSORMAP (-7)   /* the driver rejected a TMA descriptor            */
#define SWV_ERR_UNSUPPORTED (-8) /* valid request this build has no kernel for      */
#define SWV_ERR_TOO_LARGE (-9)   /* size beyond the fixed capacity of an entry point */

#define SWV_F32 0
#define SWV_BF16 1
#define SWV_F16 2

/* Library ABI version (major*100 + minor). */
int swv_version(void);

/* Text for a negative return code or a positive device status code. */
const char* swv_strerror(int code);

/* Bytes of scratch swv_dsa_indexer_topk_fwd needs for B batches of Tq queries
 * against Tk keys (256-byte aligned).  After the call it holds the collapsed
 * indexer vectors swv_dsa_attn_masked_fwd reads. */
int swv_dsa_workspace_bytes(int B, int Tq, int Tk, size_t* bytes);

/* The same for a call with `top_k` keys per query.  For a sparse selection on a long key range
 * (49152 to 262144 keys, between about one key in 70 and one in 16 selected, candidate lists of at
 * most 12288 entries per row, i.e. top_k up to about 5000) it is larger than
 * swv_dsa_workspace_bytes: swv_dsa_indexer_topk_fwd then has room for per-row candidate lists and
 * selects in two sweeps over the score tiles instead of three (same results).  With the smaller
 * workspace the entry takes the three-sweep form. */
int swv_dsa_workspace_bytes_topk(int B, int Tq, int Tk, int top_k, size_t* bytes);

/* Bytes of the tile-major membership bitmask for B x Tq x Tk:
 * [B][ceil(Tq/128)][ceil(Tk/128)][128 rows][4 x uint32]; bit c of word w of
 * row r says whether key 128*kt + 32*w + c is selected for query 128*qt + r. */
int swv_dsa_mask_bytes(int B, int Tq, int Tk, size_t* bytes);

/* DSA lightning indexer + per-query top-k.
 * Replaces LightningIndexerFunction.forward and its kernel (K:346-386, K:19-113):
 *   score[q,k] = relu( (sum_h W[h] q_idx[q,h,:]) . (sum_h W[h] k_idx[k,h,:]) )
 * (heads collapsed before the dot product, no scaling; TF32 tensor-core dot
 * with fp32 accumulation, as the reference's tl.dot on fp32 operands), then
 * for every query the top_k largest scores, ties broken towards the LOWER key
 * index.  Outputs, each contiguous (B, Tq, top_k):
 *   idx    int32  selected key indices in ASCENDING key order,
 *   valid  f32    1.0 for the first min(top_k, Tk) slots, else 0.0,
 *   scores f32    the score of each selected key (0 for unfilled slots).
 * N x N scores never reach memory: the radix select recomputes score tiles on the
 * tensor cores in three sweeps (a sampled two-byte pass with an exact check, a
 * candidate-list pass for the low 16 bits, the emit pass) and keeps per-row
 * histograms / candidate lists on chip; query tiles whose check fails or whose list
 * overflows redo the corresponding bytes with plain 8-bit histogram sweeps.
 *   q_idx (B,Tq,IH,ID), k_idx (B,Tk,IH,ID): strides (b,t,h,d); dtype SWV_F32/BF16/F16.
 *   q_idx = k_idx = NULL: the workspace already holds the collapsed vectors (swv_dsa_prologue_fwd).
 *   w: (IH,) f32.   ID <= 64.   maskbits: optional (may be NULL) bitmask output
 *   (see swv_dsa_mask_bytes) consumed by swv_dsa_attn_masked_fwd.
 */
int swv_dsa_indexer_topk_fwd(const void* q_idx, const int64_t q_strides[4], const void* k_idx,
                             const int64_t k_strides[4], int idx_dtype, const float* w, int B, int Tq, int Tk,
                             int IH, int ID, int top_k, int32_t* idx, float* valid, float* scores,
                             uint32_t* maskbits, void* workspace, size_t workspace_bytes, int* status,
                             void* stream);

/* Token-local prologue of a DSA layer in one launch: (optionally) the 2-D rotary embedding of q and
 * k, IN PLACE on the fused projection output, and the head collapse of the indexer projections
 * written into the indexer workspace.  Replaces the separate steps between the projections and the
 * indexer (M:54-59, the rotary placement of src/sparse_wsi_vit/models/vit_5/models_vit5.py:84-90) and
 * the collapse step of swv_dsa_indexer_topk_fwd: call that entry afterwards with q_idx = k_idx = NULL
 * and the same workspace, B, Tq = Tk = T.
 *   q, k (B,T,H,D) TOKEN-major strides (b,t,h,d), unit inner stride, dtype F32 or BF16; ignored when
 *   coords is NULL.  coords (B,T,2) f32 contiguous in the units of coord_high, one row per token
 *   (rows of the first skip_tokens tokens of every sequence are not read: CLS tokens stay unrotated).
 *   q_idx, k_idx (B,T,IH,ID) with strides, dtype F32/BF16/F16; w (IH,) f32; ID <= 64.
 *   workspace: swv_dsa_workspace_bytes(B, T, T) bytes.
 */
int swv_dsa_prologue_fwd(void* q, const int64_t q_strides[4], void* k, const int64_t k_strides[4], int qk_dtype,
                         const void* q_idx, const int64_t qi_strides[4], const void* k_idx, const int64_t ki_strides[4],
                         int idx_dtype, const float* w, const float* coords, float coord_high, float theta,
                         int skip_tokens, int B, int T, int H, int D, int IH, int ID, void* workspace,
                         size_t workspace_bytes, void* stream);

/* swv_dsa_indexer_topk_fwd without the workspace argument, for hosts that may not obtain
 * device memory for it.  It has no counterpart in the reference.
 * Who needs it: a caller that runs inside someone else's memory plan -- a serving runtime or
 * plug-in host that sizes every device buffer up front and hands the operator only its
 * input and output tensors, or a latency-critical loop that cannot afford the device-wide
 * synchronisation an allocation may imply.  Such a caller cannot produce the scratch buffer
 * the regular entry point asks for, so this one brings its own: a fixed array in the
 * library's device data segment.
 * Same arguments, outputs and arithmetic as swv_dsa_indexer_topk_fwd (the same kernels run).
 * Limits and rules:
 *   - B*Tq <= 8192 and B*Tk <= 8192 (any batch / length split of them); anything larger
 *     returns SWV_ERR_TOO_LARGE and launches nothing.  The array (about 4.5 MB) is held by every GPU
 *     that loads the library, until
 *     the process exits.
 *   - The first call on a device looks up the array's device address (with that device
 *     current); make that first call before any stream capture begins.
 *   - It calls no allocating or freeing routine.
 *   - All calls on a device share the one array and it keeps the previous call's contents.
 *     Nothing in it needs clearing: every word a call reads it has written first.  Two calls
 *     that overlap on the GPU (different streams, no ordering) race on it -- order them.
 *   - swv_dsa_attn_masked_fwd needs a workspace pointer and therefore cannot follow this call;
 *     use swv_dsa_attn_gather_fwd with the idx / valid / scores written here.
 */
int swv_dsa_indexer_topk_static_fwd(const void* q_idx, const int64_t q_strides[4], const void* k_idx,
                                    const int64_t k_strides[4], int idx_dtype, const float* w, int B, int Tq,
                                    int Tk, int IH, int ID, int top_k, int32_t* idx, float* valid, float* scores,
                                    uint32_t* maskbits, int* status, void* stream);

/* Routing-weighted attention over an explicit per-query key list.
 * Replaces DSAAttentionFunction.forward and its kernel (K:769-810, K:450-564):
 *   logit_j = q . k[idx_j] / sqrt(D)  for valid_j > 0,   m = max_j logit_j,
 *   p_j = exp(logit_j - m) * rw_j,    o = sum_j p_j v[idx_j] / max(sum_j p_j, 1e-6).
 * Accepts any index list (unsorted, repeated entries count twice, as in the
 * reference).  fp32 accumulation.
 *   q (B,H,Tq,D), k, v (B,H,Tk,D): strides (b,h,t,d), last stride 1; dtype F32/BF16/F16.
 *   idx int32, valid f32, rw f32: (B,Tq,top_k), strides (b,t,k).
 *   o (B,H,Tq,D): strides (b,h,t,d); o_dtype F32/BF16/F16.  1 <= D <= 256.
 *   kv_group: query heads per key/value head (1 for the reference's multi-head attention;
 *   k, v then have H/kv_group heads -- grouped-query attention, used by the NSA branches).
 */
int swv_dsa_attn_gather_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                            const void* v, const int64_t v_strides[4], int qkv_dtype, const int32_t* idx,
                            const int64_t idx_strides[3], const float* valid, const int64_t valid_strides[3],
                            const float* rw, const int64_t rw_strides[3], void* o, const int64_t o_strides[4],
                            int o_dtype, int B, int H, int Tq, int Tk, int D, int top_k, int kv_group,
                            int* status, void* stream);

/* Same arithmetic as swv_dsa_attn_gather_fwd for the key lists of the
 * swv_dsa_indexer_topk_fwd call that last wrote `maskbits` and `workspace`
 * (same B, Tq, Tk), fused with `routing_weights = scores * valid` (M:73-85):
 * a dense tensor-core flash-attention sweep (tcgen05 QK^T and PV, TMA-fed) with
 * the membership bitmask applied inside the online softmax and the routing
 * weights recomputed on the tensor cores from the collapsed indexer vectors
 * kept in the workspace (bit-identical to the emitted scores).
 * bf16 q/k/v only, D == 64; q,k,v,o rows 16-byte aligned, unit inner stride; B*H <= 1024.
 * `workspace` is read AND written (the key-norm maxima of this call live in it).
 * `scratch` (optional, may be NULL): swv_dsa_attn_scratch_bytes() bytes, 256-byte aligned.  With few
 * query tiles (one rank of a sequence-sharded run) the grid is only a few waves of CTAs; given the
 * scratch, 2 or 4 CTAs share a (query tile, head pair), each sweeping a share of the key tiles, and
 * the last one adds the partial rows up.  swv_dsa_attn_scratch_bytes returns 0 when no split helps.
 */
int swv_dsa_attn_scratch_bytes(int B, int H, int Tq, int Tk, size_t* bytes);
int swv_dsa_attn_masked_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                            const void* v, const int64_t v_strides[4], const uint32_t* maskbits,
                            void* workspace, void* o, const int64_t o_strides[4], int o_dtype, int B, int H,
                            int Tq, int Tk, int D, void* scratch, size_t scratch_bytes, int* status, void* stream);

/* Backward of the routing-weighted attention over explicit key lists.
 * Replaces DSAAttentionFunction.backward and its kernel (K:812-853, K:569-762), same arithmetic:
 *   sm_j = exp(logit_j - m) / max(l, 1e-6),  Di = sum_d dO O,  dP_j = dO . v[idx_j],
 *   dV[idx_j] += sm_j rw_j dO,   dRW_j = sum_heads sm_j (dP_j - Di),
 *   dS_j = rw_j sm_j (dP_j - Di) / sqrt(D),   dQ = sum_j dS_j k[idx_j],   dK[idx_j] += dS_j q.
 *   d_out, o (B,H,Tq,D) in o_dtype, q (B,H,Tq,D), k, v (B,H,Tk,D) in qkv_dtype, strides (b,h,t,d),
 *   k and v with unit inner stride; idx / valid / rw (B,Tq,top_k) as in swv_dsa_attn_gather_fwd.
 * Outputs are fp32 and contiguous (the reference accumulates in the storage dtype of q, k, v; the
 * caller rounds once): dq (B,H,Tq,D), dk, dv (B,H,Tk,D), drw (B,Tq,top_k).  dk, dv and drw are
 * zeroed by the call and accumulated with reductions, so their low bits depend on the order of
 * arrival.  D even, <= 256.
 */
int swv_dsa_attn_bwd(const void* d_out, const int64_t d_out_strides[4], const void* q, const int64_t q_strides[4],
                     const void* k, const int64_t k_strides[4], const void* v, const int64_t v_strides[4], int qkv_dtype,
                     const void* o, const int64_t o_strides[4], int o_dtype, const int32_t* idx,
                     const int64_t idx_strides[3], const float* valid, const int64_t valid_strides[3], const float* rw,
                     const int64_t rw_strides[3], float* dq, float* dk, float* dv, float* drw, int B, int H, int Tq,
                     int Tk, int D, int top_k, int* status, void* stream);

/* Backward of the lightning indexer.
 * Replaces LightningIndexerFunction.backward and its three kernels (K:388-445, K:128-339), same
 * arithmetic, with g = d_scores * valid:
 *   dQ[t,h,:] = sum_j g[t,j] W[h] K[idx[t,j],h,:],   dK[idx[t,j],h,:] += g[t,j] W[h] Q[t,h,:],
 *   dW[h] = sum_{t,j} g[t,j] (Q[t,h,:] . K[idx[t,j],h,:]).
 * (This is the gradient of sum_h W[h] q_h.k_h, the form the reference's backward assumes, K:116;
 * its forward computes relu((sum_h W_h q_h).(sum_h W_h k_h)), K:66-70.  A drop-in follows what the
 * reference's training loop runs.)
 *   d_scores (B,Tq,top_k) f32 with strides; q_idx (B,Tq,IH,ID), k_idx (B,Tk,IH,ID) as in the forward.
 * Outputs fp32 contiguous: dq_idx (B,Tq,IH,ID), dk_idx (B,Tk,IH,ID), dw (IH); dk_idx and dw are
 * zeroed by the call.  ID even, IH <= 64, IH*ID <= 512.
 */
int swv_dsa_indexer_bwd(const float* d_scores, const int64_t d_scores_strides[3], const void* q_idx,
                        const int64_t q_strides[4], const void* k_idx, const int64_t k_strides[4], int idx_dtype,
                        const float* w, const int32_t* idx, const int64_t idx_strides[3], const float* valid,
                        const int64_t valid_strides[3], float* dq_idx, float* dk_idx, float* dw, int B, int Tq, int Tk,
                        int IH, int ID, int top_k, int* status, void* stream);

/* Diagnostic twin of swv_dsa_attn_masked_fwd (no counterpart in the reference): the same kernel,
 * never split over the key range, that also writes `member_count` (B, Tq) int32 = the number of
 * keys every query row treated as selected while it swept the key tiles (rows on the one-pass
 * path: keys whose recomputed score >= the row threshold; rows on the two-pass path: bits set in
 * the membership mask).  It must equal min(top_k, Tk) on every row: that is the bit-level check
 * that the score tile recomputed inside the attention kernel equals the scores the indexer
 * selected on.  Output `o` as swv_dsa_attn_masked_fwd.
 */
int swv_dsa_attn_masked_count_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                                  const void* v, const int64_t v_strides[4], const uint32_t* maskbits, void* workspace,
                                  void* o, const int64_t o_strides[4], int o_dtype, int B, int H, int Tq, int Tk, int D,
                                  int32_t* member_count, int* status, void* stream);

/* Routing-weighted attention over the indexer's key lists as dense tensor-core tiles with a sparse
 * softmax (the attention step of DSAAttentionFunction.forward, K:769-810 and K:450-564, for the lists
 * swv_dsa_indexer_topk_fwd writes: bf16 q, k, v, head dim 64).  Same result as
 * swv_dsa_attn_masked_fwd; membership and routing weights are READ from the lists instead of being
 * recomputed from the indexer vectors:
 *   idx  (B, Tq, top_k) int32 contiguous: the keys of every row in its first min(top_k, Tk) slots (the
 *        rest is ignored), in any order, each key at most once; top_k a multiple of 4, 16-byte aligned;
 *   rw   (B, Tq, top_k) fp32 contiguous routing weights of those slots (scores * valid).
 * A key listed twice in a row counts once (the reference would add it twice); a key index outside
 * [0, Tk) is dropped.
 * `maskbits` and `workspace` are the ones the indexer call filled: a (query tile, head pair) whose
 * logits cannot be bounded below 2^40 is left to the kernel of swv_dsa_attn_masked_fwd, which this
 * entry launches behind its own for those tiles only.  `scratch` (256-byte aligned, at least
 * swv_dsa_attn_lists_scratch_bytes) is required.
 */
int swv_dsa_attn_lists_scratch_bytes(int B, int H, int Tq, int Tk, int top_k, size_t* bytes);
int swv_dsa_attn_lists_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                           const void* v, const int64_t v_strides[4], const int32_t* idx, const float* rw, int top_k,
                           const uint32_t* maskbits, void* workspace, void* o, const int64_t o_strides[4], int o_dtype,
                           int B, int H, int Tq, int Tk, int D, void* scratch, size_t scratch_bytes, int* status,
                           void* stream);

/* Static block-sparse flash attention forward driven by a CSR list of key blocks per
 * query block (shared by all batches and heads):
 *   o[q] = softmax_j( q.k_j / sqrt(D) ) v_j   over the keys j the pattern lets q see;
 * query rows that see no key return zeros.
 * mode 0: every key of a listed block is seen -- the 2-D block pattern (no counterpart in
 *         the reference; defined as dense attention under the expanded block mask).
 * mode 1: inside the listed blocks the token pattern of the reference's
 *         StaticSparseAttention applies (src/sparse_wsi_vit/models/static_sparse_attention.py:62-188):
 *         query i sees key j iff i < num_cls or j < num_cls or
 *         (|i-j| <= window*dilation and (i-j) % dilation == 0); the list must contain every
 *         block that holds such a pair.  Replaces the three SDPA calls at :87, :93/:97, :180.
 *   q (B,H,Tq,D), k, v (B,H,Tk,D) bf16, strides (b,h,t,d), unit inner stride, 16-byte rows.
 *   row_ptr int32[ceil(Tq/block)+1], col_idx int32[nnz]; block in {64,128}; D in {64,128}.
 *   kv_group: query heads per key/value head (k, v have H/kv_group heads); 1 = multi-head.
 *   lse: optional (may be NULL) f32 (B,H,Tq) contiguous, natural-log sum of exponentials of
 *   every row (-inf for rows that see no key).
 *   Tensor-core (tcgen05) QK^T and PV, fp32 softmax statistics.
 */
int swv_block_sparse_attn_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                              const void* v, const int64_t v_strides[4], const int32_t* row_ptr,
                              const int32_t* col_idx, int block, int mode, int num_cls, int window, int dilation,
                              int kv_group, float* lse, void* o, const int64_t o_strides[4], int o_dtype, int B,
                              int H, int Tq, int Tk, int D, int* status, void* stream);

/* Mean pooling of overlapping token windows, y[b,h,c,:] = mean_{i<window} x[b,h,c*stride+i,:],
 * c < (T-window)/stride + 1: the compressed keys and values of the NSA compressed branch
 * (no counterpart in the reference, which only names NSA as an intent,
 * scripts/virchow_preprocess.py:44-53).  x (B,H,T,D) bf16, strides (b,h,t,d) even, unit inner
 * stride; y contiguous (B,H,nC,D) bf16.
 */
int swv_pool_tokens(const void* x, const int64_t x_strides[4], void* y, int B, int H, int T, int D, int window,
                    int stride, void* stream);

/* NSA-style attention, selection step (no counterpart in the reference, which only names NSA as an
 * intent, scripts/virchow_preprocess.py:44-53).  For every (batch, kv head g, query t) the
 * importance of selection block s is the sum, over the Hq/Hkv query heads of group g and over the
 * compressed tokens c with (c * cmp_stride) / sel_block == s, of
 *   exp(q_h[t] . kc_g[c] / sqrt(D) - lse[b,h,t])
 * where lse is the log-sum-exp row statistic of the compressed branch
 * (swv_block_sparse_attn_fwd's `lse` output).  The n_sel most important of the
 * ceil(Tk / sel_block) blocks are written to `blocks` (B,Hkv,Tq,min(n_sel, n_blocks)) int32 in
 * ascending order; ties go to the lower block index.
 *   q (B,Hq,Tq,D), kc (B,Hkv,nC,D) bf16, unit inner stride, 16-byte aligned rows; D = 64 or 128;
 *   sel_block / cmp_stride in {1,2,4,8}; Hq / Hkv <= 16.
 *   importance: caller-owned scratch of swv_nsa_importance_bytes() bytes (the block scores, fp32).
 */
int swv_nsa_importance_bytes(int B, int Hkv, int Tq, int nC, int cmp_stride, int sel_block, size_t* bytes);
int swv_nsa_select_blocks_fwd(const void* q, const int64_t q_strides[4], const void* kc, const int64_t kc_strides[4],
                              const float* lse, int B, int Hq, int Hkv, int Tq, int Tk, int nC, int D,
                              int cmp_stride, int sel_block, int n_sel, float* importance, size_t importance_bytes,
                              int32_t* blocks, int* status, void* stream);

/* NSA-style attention, selected branch: plain softmax attention of every query head over the keys
 * of the blocks selected for its kv group, o (B,Hq,Tq,D) fp32 contiguous.  One pass reads every
 * selected key / value row once for the whole group (warp-level tensor-core tiles whose rows are the
 * heads of the group).  q, k, v bf16 as above; sel_block a multiple
 * of 32; Hq / Hkv <= 8; `blocks` (B,Hkv,Tq,n_sel) int32, block ids < ceil(Tk / sel_block).
 */
int swv_nsa_selected_attn_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                              const void* v, const int64_t v_strides[4], const int32_t* blocks, int B, int Hq,
                              int Hkv, int Tq, int Tk, int D, int sel_block, int n_sel, float* o, void* stream);

/* NSA-style attention, gate: out[b,h,t,:] = sum_j sigmoid(gate[b,t,h,j]) * o_j[b,h,t,:] for the three
 * branches j = compressed, selected, window; branches fp32 contiguous (B,Hq,T,D), gate fp32
 * contiguous (B,T,Hq,3), out contiguous in `out_dtype`.
 */
int swv_nsa_combine_fwd(const float* o_cmp, const float* o_sel, const float* o_win, const float* gate, void* out,
                        int out_dtype, int B, int Hq, int T, int D, void* stream);

/* NSA-style attention, whole forward pass in one call: mean-pooled compression (window cmp_block,
 * stride cmp_stride), compressed branch, block selection (n_sel blocks of sel_block keys per query
 * and kv group), selected branch, sliding-window branch (keys with |i - j| <= window / 2,
 * non-causal) and the gated sum.  Non-causal, batch-major tensors:
 *   q (B,Hq,T,D), k, v (B,Hkv,T,D) bf16, unit inner stride, 16-byte aligned rows; D = 64 or 128;
 *   gate (B,T,Hq,3) fp32 contiguous, logits in the order [compressed, selected, window];
 *   out (B,Hq,T,D) contiguous in out_dtype;
 *   workspace: swv_nsa_workspace_bytes() bytes, 256-byte aligned (pooled keys / values, ONE fp32
 *   accumulator of the gated branch sum -- every branch kernel applies its gate in its epilogue and
 *   adds its rows to it, the last one writes `out` -- row statistics, block scores, key-block lists);
 *   blocks_out: optional (B,Hkv,T,min(n_sel, ceil(T/sel_block))) int32, the selected block ids.
 * Limits as for the entry points it is built from (Hq / Hkv <= 8, sel_block a multiple of 32 and of
 * cmp_stride with sel_block / cmp_stride in {1,2,4,8}).
 */
int swv_nsa_workspace_bytes(int B, int Hq, int Hkv, int T, int D, int cmp_block, int cmp_stride, int sel_block,
                            int n_sel, int window, size_t* bytes);
int swv_nsa_attn_fwd(const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
                     const void* v, const int64_t v_strides[4], const float* gate, void* out, int out_dtype, int B,
                     int Hq, int Hkv, int T, int D, int cmp_block, int cmp_stride, int sel_block, int n_sel,
                     int window, void* workspace, size_t workspace_bytes, int32_t* blocks_out, int* status,
                     void* stream);

/* 2-D rotary embedding on per-token (y, x) coordinates.
 * Replaces VisionRotaryEmbedding.forward, dynamic branch
 * (src/sparse_wsi_vit/models/vit_5/rope.py:72-97, rotate_half :33-37), as applied to q and k in
 * src/sparse_wsi_vit/models/vit_5/models_vit5.py:84-90: head_dim/4 frequencies
 * theta^(-2i/(head_dim/2)), each used for two adjacent channels; the first half of the head
 * turns with coords[:,0]/coord_high, the second half with coords[:,1]/coord_high;
 * (x0,x1) -> (x0 cos - x1 sin, x1 cos + x0 sin).  The first `skip_tokens` tokens (CLS) are copied.
 *   x, y (L,H,head_dim): strides (l,h,d) with unit inner stride; dtype SWV_F32 or SWV_BF16; y may be x.
 *   coords (L,2) f32 contiguous.
 */
int swv_rope2d_apply(const void* x, const int64_t x_strides[3], void* y, const int64_t y_strides[3], int dtype,
                     const float* coords, int64_t L, int H, int head_dim, float coord_high, float theta,
                     int skip_tokens, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SWV_B200_H_ */
