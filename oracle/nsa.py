"""Library-defined CPU oracle of NSA-style attention (compressed + selected + sliding-window
branches, sigmoid gate).

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  PARITY UNPINNED: the reference contains
no NSA code (only a docstring intent, scripts/virchow_preprocess.py:44-53); every choice below is
frozen here (and restated in the design notes of the repository).

  q (Hq, T, D), k, v (Hkv, T, D), gate logits g (T, Hq, 3) ordered [compressed, selected, window];
  G = Hq / Hkv query heads share one key/value head (head h uses kv head h // G).
  compressed : keys/values mean-pooled over windows of `cmp_block` tokens with stride `cmp_stride`;
               plain softmax attention over all compressed tokens (non-causal).
  selected   : per (kv head, query) the importance of a selection block of `sel_block` keys is the
               sum, over the G query heads and over the compressed tokens whose FIRST key lies in
               the block, of the compressed-branch probabilities; the `sel_topk` most important
               blocks (ties -> lower block index) are attended with a plain softmax over their keys.
  window     : keys j with |i - j| <= window // 2 (non-causal).
  out = sum_b sigmoid(g_b) * O_b.
"""
from __future__ import annotations

import math

import torch


def pool_tokens(x, win, stride):
    T = x.shape[-2]
    n = (T - win) // stride + 1
    idx = torch.arange(n)[:, None] * stride + torch.arange(win)[None, :]
    return x[..., idx, :].mean(dim=-2)


def block_importance(p_cmp_group, T, cmp_stride, sel_block):
    """p_cmp_group (G, R, nC) probabilities of one kv group -> (R, n_blocks) importance."""
    nC = p_cmp_group.shape[-1]
    n_s = -(-T // sel_block)
    owner = (torch.arange(nC) * cmp_stride) // sel_block
    imp = torch.zeros((p_cmp_group.shape[1], n_s), dtype=p_cmp_group.dtype)
    imp.index_add_(1, owner, p_cmp_group.sum(dim=0))
    return imp


def select_blocks(p_cmp_group, T, cmp_stride, sel_block, sel_topk):
    """p_cmp_group (G, R, nC) probabilities of one kv group -> (R, k_eff) block ids, ascending."""
    imp = block_importance(p_cmp_group, T, cmp_stride, sel_block)
    k_eff = min(sel_topk, imp.shape[1])
    top = torch.sort(imp, dim=1, descending=True, stable=True).indices[:, :k_eff]
    return torch.sort(top, dim=1).values


def selection_margin(imp, sel_topk):
    """(R,) relative gap between the last selected and the first rejected block importance; rows
    with a tiny gap may legitimately select differently under another summation order."""
    if imp.shape[1] <= sel_topk:
        return torch.full((imp.shape[0],), float("inf"))
    srt = torch.sort(imp, dim=1, descending=True).values
    return (srt[:, sel_topk - 1] - srt[:, sel_topk]) / srt[:, sel_topk - 1].clamp_min(1e-30)


def nsa_attention(q, k, v, gate, cmp_block=32, cmp_stride=16, sel_block=64, sel_topk=16, window=512,
                  dtype=torch.float32, return_parts=False, rows=None, pooled_dtype=None):
    """q (Hq, T, D), k, v (Hkv, T, D), gate (T, Hq, 3).  With `rows` (1-D tensor of query indices)
    only those query rows are computed (outputs (Hq, len(rows), D)): long sequences are checked on
    a sample of rows against all keys.  `pooled_dtype` rounds the pooled keys / values to that
    dtype first (the library stores them in bf16).  With `return_parts` also the three branch
    outputs, the selected blocks (Hkv, R, k_eff) and the selection margins (Hkv, R)."""
    Hq, T, D = q.shape
    Hkv = k.shape[0]
    G = Hq // Hkv
    scale = 1.0 / math.sqrt(D)
    kf, vf = k.to(dtype), v.to(dtype)
    ridx = torch.arange(T) if rows is None else rows.long()
    qf = q.to(dtype)[:, ridx]
    R = len(ridx)
    kc, vc = pool_tokens(kf, cmp_block, cmp_stride), pool_tokens(vf, cmp_block, cmp_stride)
    if pooled_dtype is not None:
        kc, vc = kc.to(pooled_dtype).to(dtype), vc.to(pooled_dtype).to(dtype)
    o_cmp = torch.empty_like(qf)
    o_sel = torch.empty_like(qf)
    o_win = torch.empty_like(qf)
    win_mask = (ridx[:, None] - torch.arange(T)[None, :]).abs() <= window // 2
    blocks_all, margins = [], []
    for g in range(Hkv):
        hs = slice(g * G, (g + 1) * G)
        s = (qf[hs] @ kc[g].T) * scale                       # (G, R, nC)
        p = torch.softmax(s, dim=-1)
        o_cmp[hs] = p @ vc[g]
        blocks = select_blocks(p, T, cmp_stride, sel_block, sel_topk)   # (R, k_eff)
        margins.append(selection_margin(block_importance(p, T, cmp_stride, sel_block), sel_topk))
        blocks_all.append(blocks)
        sel_mask = torch.zeros((R, -(-T // sel_block)), dtype=torch.bool)
        sel_mask.scatter_(1, blocks, True)
        tok_mask = sel_mask.repeat_interleave(sel_block, dim=1)[:, :T]
        logits = (qf[hs] @ kf[g].T) * scale                  # (G, R, T)
        o_sel[hs] = torch.softmax(logits.masked_fill(~tok_mask, float("-inf")), dim=-1) @ vf[g]
        o_win[hs] = torch.softmax(logits.masked_fill(~win_mask, float("-inf")), dim=-1) @ vf[g]
    gs = torch.sigmoid(gate.to(dtype))[ridx].permute(1, 0, 2)      # (Hq, R, 3)
    out = gs[..., 0:1] * o_cmp + gs[..., 1:2] * o_sel + gs[..., 2:3] * o_win
    if return_parts:
        return out, o_cmp, o_sel, o_win, torch.stack(blocks_all), torch.stack(margins)
    return out
