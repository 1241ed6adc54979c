"""Builder-defined CPU oracle of NSA-style attention (compressed + selected + sliding-window
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


def select_blocks(p_cmp_group, T, cmp_stride, sel_block, sel_topk):
    """p_cmp_group (G, Tq, nC) probabilities of one kv group -> (Tq, k_eff) block ids, ascending."""
    nC = p_cmp_group.shape[-1]
    n_s = -(-T // sel_block)
    owner = (torch.arange(nC) * cmp_stride) // sel_block
    imp = torch.zeros((p_cmp_group.shape[1], n_s), dtype=p_cmp_group.dtype)
    imp.index_add_(1, owner, p_cmp_group.sum(dim=0))
    k_eff = min(sel_topk, n_s)
    top = torch.sort(imp, dim=1, descending=True, stable=True).indices[:, :k_eff]
    return torch.sort(top, dim=1).values


def nsa_attention(q, k, v, gate, cmp_block=32, cmp_stride=16, sel_block=64, sel_topk=16, window=512,
                  dtype=torch.float32, return_parts=False):
    Hq, T, D = q.shape
    Hkv = k.shape[0]
    G = Hq // Hkv
    scale = 1.0 / math.sqrt(D)
    qf, kf, vf = q.to(dtype), k.to(dtype), v.to(dtype)
    kc, vc = pool_tokens(kf, cmp_block, cmp_stride), pool_tokens(vf, cmp_block, cmp_stride)
    o_cmp = torch.empty_like(qf)
    o_sel = torch.empty_like(qf)
    o_win = torch.empty_like(qf)
    i = torch.arange(T)
    win_mask = (i[:, None] - i[None, :]).abs() <= window // 2
    blocks_all = []
    for g in range(Hkv):
        hs = slice(g * G, (g + 1) * G)
        s = (qf[hs] @ kc[g].T) * scale                       # (G, T, nC)
        p = torch.softmax(s, dim=-1)
        o_cmp[hs] = p @ vc[g]
        blocks = select_blocks(p, T, cmp_stride, sel_block, sel_topk)   # (T, k_eff)
        blocks_all.append(blocks)
        sel_mask = torch.zeros((T, -(-T // sel_block)), dtype=torch.bool)
        sel_mask.scatter_(1, blocks, True)
        tok_mask = sel_mask.repeat_interleave(sel_block, dim=1)[:, :T]
        logits = (qf[hs] @ kf[g].T) * scale                  # (G, T, T)
        o_sel[hs] = torch.softmax(logits.masked_fill(~tok_mask, float("-inf")), dim=-1) @ vf[g]
        o_win[hs] = torch.softmax(logits.masked_fill(~win_mask, float("-inf")), dim=-1) @ vf[g]
    gs = torch.sigmoid(gate.to(dtype)).permute(1, 0, 2)      # (Hq, T, 3)
    out = gs[..., 0:1] * o_cmp + gs[..., 1:2] * o_sel + gs[..., 2:3] * o_win
    if return_parts:
        return out, o_cmp, o_sel, o_win, torch.stack(blocks_all)
    return out
