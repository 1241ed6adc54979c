"""NSA-style attention forward (compressed, selected and sliding-window branches with a sigmoid
gate) assembled from this library's CUDA kernels.  The reference has no NSA code; the semantics
are the library-defined ones frozen in ``oracle/nsa.py`` (parity unpinned).

  compressed : `swv_pool_tokens` (mean pooling) + the block-sparse tensor-core kernel over ALL
               compressed tokens, grouped-query (kv_group), returning the log-sum-exp per row;
  selection  : `swv_nsa_select_blocks_fwd`: block importance recomputed on the tensor cores from
               q, the compressed keys and the log-sum-exp, then an arg-max kernel per query;
  selected   : `swv_nsa_selected_attn_fwd`: one warp per (kv group, query) reads each selected
               key / value row once for all heads of the group (the heads are the rows of
               warp-level tensor-core tiles);
  window     : the block-sparse kernel in token-pattern mode (|i-j| <= window/2);
  gate       : in the one-call form (`swv_nsa_attn_fwd`) every branch kernel applies its sigmoid gate
               in its epilogue and adds its rows to one fp32 accumulator, the last branch writes
               the output; the step-by-step form (`return_parts=True`) keeps the three branch
               outputs and sums them with `swv_nsa_combine_fwd`.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from ._lib import check, dtype_code, lib, strides
from .ops import _buffer, _require_cuda, _stream, block_sparse_attention, status_word
from .patterns import _to_csr, static_window_blocks


def pool_tokens(x, win, stride):
    """x (B,H,T,D) bf16 -> (B,H,nC,D) bf16, mean over windows of `win` tokens every `stride`."""
    _require_cuda(x)
    B, H, T, D = x.shape
    x = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    if x.stride(3) != 1 or any(s % 2 for s in x.stride()[:3]):
        x = x.contiguous()
    nC = (T - win) // stride + 1
    y = torch.empty((B, H, nC, D), dtype=torch.bfloat16, device=x.device)
    check(lib.swv_pool_tokens(x.data_ptr(), strides(x), y.data_ptr(), B, H, T, D, win, stride, _stream(x.device)),
          "swv_pool_tokens")
    return y


def _full_list(n_q_blocks, n_k_blocks, device):
    rp = torch.arange(0, (n_q_blocks + 1) * n_k_blocks, n_k_blocks, dtype=torch.int32, device=device)
    ci = torch.arange(n_k_blocks, dtype=torch.int32, device=device).repeat(n_q_blocks)
    return rp, ci


def select_blocks(q, kc, lse, T, cmp_stride, sel_block, sel_topk, kv_group):
    """Top `sel_topk` selection blocks per (batch, kv head, query), ascending block ids, int32
    (B, Hkv, Tq, k_eff).  Importance = compressed-branch probabilities summed over the group's query
    heads and over the compressed tokens whose first key lies in the block; ties -> lower block id."""
    _require_cuda(q, kc, lse)
    B, Hq, Tq, D = q.shape
    Hkv, nC = kc.shape[1], kc.shape[2]
    n_s = -(-T // sel_block)
    k_eff = min(sel_topk, n_s)
    nbytes = ctypes.c_size_t()
    check(lib.swv_nsa_importance_bytes(B, Hkv, Tq, nC, cmp_stride, sel_block, ctypes.byref(nbytes)),
          "swv_nsa_importance_bytes")
    imp = torch.empty(nbytes.value // 4, dtype=torch.float32, device=q.device)
    blocks = torch.empty((B, Hkv, Tq, k_eff), dtype=torch.int32, device=q.device)
    lse = lse.contiguous()
    check(lib.swv_nsa_select_blocks_fwd(q.data_ptr(), strides(q), kc.data_ptr(), strides(kc), lse.data_ptr(), B, Hq, Hkv,
                                        Tq, T, nC, D, cmp_stride, sel_block, sel_topk, imp.data_ptr(), nbytes.value,
                                        blocks.data_ptr(), status_word(q.device).data_ptr(), _stream(q.device)),
          "swv_nsa_select_blocks_fwd")
    return blocks


def selected_attention(q, k, v, blocks, sel_block):
    """Softmax attention of every query head over the keys of its kv group's selected blocks -> fp32."""
    _require_cuda(q, k, v, blocks)
    B, Hq, Tq, D = q.shape
    Hkv, Tk = k.shape[1], k.shape[2]
    o = torch.empty((B, Hq, Tq, D), dtype=torch.float32, device=q.device)
    blocks = blocks.contiguous()
    check(lib.swv_nsa_selected_attn_fwd(q.data_ptr(), strides(q), k.data_ptr(), strides(k), v.data_ptr(), strides(v),
                                        blocks.data_ptr(), B, Hq, Hkv, Tq, Tk, D, sel_block, blocks.shape[-1],
                                        o.data_ptr(), _stream(q.device)), "swv_nsa_selected_attn_fwd")
    return o


def nsa_attention(q, k, v, gate, cmp_block=32, cmp_stride=16, sel_block=64, sel_topk=16, window=512,
                  out_dtype=None, return_parts=False):
    """q (B,Hq,T,D), k, v (B,Hkv,T,D) bf16; gate (B,T,Hq,3) logits [compressed, selected, window].
    Returns (B,Hq,T,D).  One library call (`swv_nsa_attn_fwd`); with `return_parts` the same kernels
    are run one by one and the branch outputs and selected blocks are returned as well."""
    _require_cuda(q, k, v, gate)
    B, Hq, T, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    dev = q.device
    out_dtype = out_dtype or q.dtype
    q, k, v = (t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16) for t in (q, k, v))
    gate = gate.float().contiguous()
    out = torch.empty((B, Hq, T, D), dtype=out_dtype, device=dev)

    if not return_parts:
        nbytes = ctypes.c_size_t()
        check(lib.swv_nsa_workspace_bytes(B, Hq, Hkv, T, D, cmp_block, cmp_stride, sel_block, sel_topk, window,
                                          ctypes.byref(nbytes)), "swv_nsa_workspace_bytes")
        ws = _buffer("nsa_ws", dev, nbytes.value)         # kept between calls (the pass is stream-ordered)
        check(lib.swv_nsa_attn_fwd(q.data_ptr(), strides(q), k.data_ptr(), strides(k), v.data_ptr(), strides(v),
                                   gate.data_ptr(), out.data_ptr(), dtype_code(out_dtype), B, Hq, Hkv, T, D, cmp_block,
                                   cmp_stride, sel_block, sel_topk, window, ws.data_ptr(), nbytes.value, None,
                                   status_word(dev).data_ptr(), _stream(dev)), "swv_nsa_attn_fwd")
        return out

    # compressed branch
    kc, vc = pool_tokens(k, cmp_block, cmp_stride), pool_tokens(v, cmp_block, cmp_stride)
    nC = kc.shape[2]
    rp, ci = _full_list(-(-T // 128), -(-nC // 128), dev)
    o_cmp, lse = block_sparse_attention(q, kc, vc, rp, ci, 128, out_dtype=torch.float32, kv_group=G, return_lse=True)

    # selected branch
    blocks = select_blocks(q, kc, lse, T, cmp_stride, sel_block, sel_topk, G)       # (B,Hkv,T,k_eff)
    o_sel = selected_attention(q, k, v, blocks, sel_block)

    # sliding-window branch
    wrp, wci = static_window_blocks(T, 0, window // 2, 1, 128)
    o_win = block_sparse_attention(q, k, v, torch.from_numpy(wrp).to(dev), torch.from_numpy(wci).to(dev), 128, mode=1,
                                   num_cls=0, window=window // 2, dilation=1, out_dtype=torch.float32, kv_group=G)

    check(lib.swv_nsa_combine_fwd(o_cmp.data_ptr(), o_sel.data_ptr(), o_win.data_ptr(), gate.data_ptr(), out.data_ptr(),
                                  dtype_code(out_dtype), B, Hq, T, D, _stream(dev)), "swv_nsa_combine_fwd")
    return out, o_cmp, o_sel, o_win, blocks
