"""NSA-style attention forward (compressed, selected and sliding-window branches with a sigmoid
gate) assembled from this library's CUDA kernels.  The reference has no NSA code; the semantics
are the builder-defined ones frozen in ``oracle/nsa.py`` (parity unpinned).

  compressed : `swv_pool_tokens` (mean pooling) + the block-sparse tensor-core kernel over ALL
               compressed tokens, grouped-query (kv_group), returning the log-sum-exp per row;
  selection  : block importance from the compressed-branch probabilities.  This step is NOT a
               hand-written kernel yet: it recomputes q.Kc^T with cuBLAS (torch.matmul) in query
               chunks and uses torch.topk -- library code, stated as such in DESIGN.md;
  selected   : the gather kernel (`swv_dsa_attn_gather_fwd`, weights 1) over the keys of the
               selected blocks, one call per kv group (the lists are shared by the group's heads);
  window     : the block-sparse kernel in token-pattern mode (|i-j| <= window/2);
  gate       : sigmoid-weighted sum (elementwise, PyTorch).
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from ._lib import check, lib, strides
from .ops import _require_cuda, _stream, block_sparse_attention, dsa_attention_gather
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


def select_blocks(q, kc, lse, T, cmp_stride, sel_block, sel_topk, kv_group, chunk=2048):
    """Top `sel_topk` selection blocks per (batch, kv head, query), ascending block ids, int32
    (B, Hkv, T, k_eff).  Importance = compressed-branch probabilities summed over the group's query
    heads and over the compressed tokens whose first key lies in the block."""
    B, Hq, Tq, D = q.shape
    Hkv = Hq // kv_group
    nC = kc.shape[2]
    n_s = -(-T // sel_block)
    k_eff = min(sel_topk, n_s)
    owner = (torch.arange(nC, device=q.device) * cmp_stride) // sel_block
    scale = 1.0 / D ** 0.5
    out = torch.empty((B, Hkv, Tq, k_eff), dtype=torch.int32, device=q.device)
    qg = q.view(B, Hkv, kv_group, Tq, D)
    lg = lse.view(B, Hkv, kv_group, Tq)
    kcf = kc.float()
    for t0 in range(0, Tq, chunk):
        t1 = min(Tq, t0 + chunk)
        s = torch.einsum("bkgtd,bkcd->bkgtc", qg[:, :, :, t0:t1].float(), kcf) * scale
        p = torch.exp(s - lg[:, :, :, t0:t1, None]).sum(dim=2)                 # (B, Hkv, t, nC)
        imp = torch.zeros((B, Hkv, t1 - t0, n_s), dtype=torch.float32, device=q.device)
        imp.index_add_(3, owner, p)
        # ties -> lower block index: stable descending sort
        top = torch.sort(imp, dim=3, descending=True, stable=True).indices[..., :k_eff]
        out[:, :, t0:t1] = torch.sort(top, dim=3).values.to(torch.int32)
    return out


def nsa_attention(q, k, v, gate, cmp_block=32, cmp_stride=16, sel_block=64, sel_topk=16, window=512,
                  out_dtype=None, return_parts=False):
    """q (B,Hq,T,D), k, v (B,Hkv,T,D) bf16; gate (B,T,Hq,3) logits [compressed, selected, window].
    Returns (B,Hq,T,D)."""
    _require_cuda(q, k, v, gate)
    B, Hq, T, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    dev = q.device
    out_dtype = out_dtype or q.dtype
    q, k, v = (t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16) for t in (q, k, v))

    # compressed branch
    kc, vc = pool_tokens(k, cmp_block, cmp_stride), pool_tokens(v, cmp_block, cmp_stride)
    nC = kc.shape[2]
    rp, ci = _full_list(-(-T // 128), -(-nC // 128), dev)
    o_cmp, lse = block_sparse_attention(q, kc, vc, rp, ci, 128, out_dtype=torch.float32, kv_group=G, return_lse=True)

    # selected branch
    blocks = select_blocks(q, kc, lse, T, cmp_stride, sel_block, sel_topk, G)       # (B,Hkv,T,k_eff)
    k_eff = blocks.shape[-1]
    tok = (blocks[..., None].long() * sel_block + torch.arange(sel_block, device=dev)).reshape(B, Hkv, T, -1)
    valid = (tok < T).to(torch.float32)
    idx = tok.clamp_(max=T - 1).to(torch.int32)
    ones = torch.ones_like(valid)
    o_sel = torch.empty((B, Hq, T, D), dtype=torch.float32, device=dev)
    for g in range(Hkv):
        dsa_attention_gather(q[:, g * G:(g + 1) * G], k[:, g:g + 1], v[:, g:g + 1], idx[:, g].contiguous(),
                             valid[:, g].contiguous(), ones[:, g].contiguous(), o_sel[:, g * G:(g + 1) * G],
                             kv_group=G)

    # sliding-window branch
    wrp, wci = static_window_blocks(T, 0, window // 2, 1, 128)
    o_win = block_sparse_attention(q, k, v, torch.from_numpy(wrp).to(dev), torch.from_numpy(wci).to(dev), 128, mode=1,
                                   num_cls=0, window=window // 2, dilation=1, out_dtype=torch.float32, kv_group=G)

    gs = torch.sigmoid(gate.float()).permute(0, 2, 1, 3)                            # (B,Hq,T,3)
    out = (gs[..., 0:1] * o_cmp + gs[..., 1:2] * o_sel + gs[..., 2:3] * o_win).to(out_dtype)
    if return_parts:
        return out, o_cmp, o_sel, o_win, blocks
    return out
