"""CPU restatement of the reference's DeepSeek-style sparse attention forward.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Reference files (paths inside the reference project):
  K = src/sparse_wsi_vit/models/deepseek_sparse_attention_kernels/kernels.py
  M = src/sparse_wsi_vit/models/deepseek_sparse_attention.py

All functions work on one batch element at a time unless stated and compute in
float32 (float64 optional for tolerance studies), never in bf16.
"""
from __future__ import annotations

import math

import numpy as np
import torch


# --------------------------------------------------------------------------- #
# indexer scores  (K:40, K:66-71)
# --------------------------------------------------------------------------- #
def collapse_heads(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``wx[t, :] = sum_h W[h] * x[t, h, :]`` in float32 (K:66-67).

    The reference collapses the indexer heads with the head weights BEFORE the
    dot product.  x: (T, IH, ID) any float dtype, w: (IH,).  Returns (T, ID) f32.
    The sum runs over heads in ascending order, as ``tl.sum(axis=1)`` does for
    four heads in the interpreter (pairwise == sequential up to fp32 rounding;
    the fixtures pin the exact values).
    """
    xf = x.to(torch.float32)
    wf = w.to(torch.float32)
    return (xf * wf[None, :, None]).sum(dim=1)


def indexer_scores(q_idx: torch.Tensor, k_idx: torch.Tensor, w: torch.Tensor,
                   dtype=torch.float32) -> torch.Tensor:
    """Dense (T, T) ReLU scores ``relu(wq @ wk^T)`` (K:66-70).

    No 1/sqrt(ID) scale, ReLU applied once to the head-collapsed dot product.
    """
    wq = collapse_heads(q_idx, w).to(dtype)
    wk = collapse_heads(k_idx, w).to(dtype)
    return torch.relu(wq @ wk.T)


# --------------------------------------------------------------------------- #
# top-k  (K:42-43, K:74-113)
# --------------------------------------------------------------------------- #
def topk_lower_index(scores: torch.Tensor, top_k: int):
    """Per-row top-k with ties broken towards the LOWER key index.

    This is the rule the build implements.  It equals the reference's selected
    set on every row where no tie straddles the K-th largest value (K:84-97).
    Returns (idx int32, valid f32, sel_scores f32), each (T, top_k), with the
    selected keys listed in ASCENDING key order (the reference's slot order is
    insertion order and carries no meaning downstream; compare as sets).
    Unfilled slots (T < top_k) have idx = 0, valid = 0, score = 0 (K:99-113).
    """
    T = scores.shape[0]
    n = scores.shape[1]
    k_eff = min(top_k, n)
    # stable descending sort == ties to lower index
    order = torch.sort(scores, dim=1, descending=True, stable=True).indices[:, :k_eff]
    order = torch.sort(order, dim=1).values
    idx = torch.zeros((T, top_k), dtype=torch.int32)
    valid = torch.zeros((T, top_k), dtype=torch.float32)
    sel = torch.zeros((T, top_k), dtype=torch.float32)
    idx[:, :k_eff] = order.to(torch.int32)
    valid[:, :k_eff] = 1.0
    sel[:, :k_eff] = torch.gather(scores, 1, order).to(torch.float32)
    return idx, valid, sel


def topk_replace_min(scores: torch.Tensor, top_k: int):
    """Sequential simulation of the reference's streaming insertion (K:74-97).

    Keys are visited in ascending order; a key replaces the FIRST slot holding
    the running minimum iff its score is strictly larger.  Reproduces the
    reference's ``idx`` including slot order.  O(T*T*K): small cases only.
    """
    s = scores.to(torch.float32).numpy()
    T, n = s.shape
    idx = np.zeros((T, top_k), dtype=np.int32)
    valid = np.zeros((T, top_k), dtype=np.float32)
    sel = np.zeros((T, top_k), dtype=np.float32)
    for r in range(T):
        buf = np.full(top_k, -np.inf, dtype=np.float32)
        bidx = np.zeros(top_k, dtype=np.int32)
        for c in range(n):
            mn = buf.min()
            if s[r, c] > mn:
                slot = int(np.argmax(buf == mn))
                buf[slot] = s[r, c]
                bidx[slot] = c
        filled = buf > -np.inf
        idx[r] = bidx
        valid[r] = filled.astype(np.float32)
        sel[r] = np.where(filled, buf, 0.0)
    return torch.from_numpy(idx), torch.from_numpy(valid), torch.from_numpy(sel)


def rows_with_straddling_tie(scores: torch.Tensor, top_k: int) -> torch.Tensor:
    """Bool (T,) — rows where the K-th and (K+1)-th largest scores are equal.

    On those rows the reference's replace-min loop keeps an emergent subset of
    the tied keys that is NOT the lowest indices; index sets are compared with
    the reference only on the other rows.
    """
    n = scores.shape[1]
    if n <= top_k:
        return torch.zeros(scores.shape[0], dtype=torch.bool)
    srt = torch.sort(scores, dim=1, descending=True).values
    return srt[:, top_k - 1] == srt[:, top_k]


# --------------------------------------------------------------------------- #
# routing-weighted attention over the selected keys  (K:472, K:519-527, K:550-562)
# --------------------------------------------------------------------------- #
def dsa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                  idx: torch.Tensor, valid: torch.Tensor, rw: torch.Tensor,
                  dtype=torch.float32, chunk: int = 1024) -> torch.Tensor:
    """o[h, t] = sum_j p_j v[h, idx_j] / max(sum_j p_j, 1e-6),
    p_j = exp(logit_j - m) * rw_j, logit_j = q.k[idx_j]/sqrt(D), m = max over
    the valid slots (weight-0 slots included), invalid slots contribute nothing.

    q, k, v: (H, T, D); idx/valid/rw: (T, K).  Returns (H, T, D) in ``dtype``.
    """
    H, T, D = q.shape
    scale = 1.0 / math.sqrt(D)
    qf, kf, vf = q.to(dtype), k.to(dtype), v.to(dtype)
    out = torch.zeros((H, T, D), dtype=dtype)
    idl = idx.long()
    for t0 in range(0, T, chunk):
        t1 = min(T, t0 + chunk)
        ii = idl[t0:t1]                                  # (c, K)
        vm = valid[t0:t1] > 0
        w = rw[t0:t1].to(dtype)
        for h in range(H):
            kg = kf[h][ii]                               # (c, K, D)
            vg = vf[h][ii]
            logit = torch.einsum("cd,ckd->ck", qf[h, t0:t1], kg) * scale
            logit = torch.where(vm, logit, torch.full_like(logit, -float("inf")))
            m = logit.max(dim=1, keepdim=True).values
            p = torch.where(vm, torch.exp(logit - m) * w, torch.zeros_like(logit))
            l = p.sum(dim=1, keepdim=True)
            o = torch.einsum("ck,ckd->cd", p, vg)
            out[h, t0:t1] = o / torch.clamp(l, min=1e-6)
    return out


def dsa_attention_dense(q, k, v, scores, top_k, dtype=torch.float32):
    """Same result as ``dsa_attention(topk_lower_index(...))`` computed with a
    dense (T, T) membership mask; used to time a CPU baseline at sizes where
    the gathered form is too slow.  q, k, v: (H, T, D); scores (T, T) f32.
    """
    H, T, D = q.shape
    idx, valid, sel = topk_lower_index(scores, top_k)
    member = torch.zeros((T, T), dtype=torch.bool)
    k_eff = min(top_k, T)
    member.scatter_(1, idx[:, :k_eff].long(), True)
    scale = 1.0 / math.sqrt(D)
    out = torch.empty((H, T, D), dtype=dtype)
    wts = torch.where(member, scores, torch.zeros_like(scores)).to(dtype)
    for h in range(H):
        logit = (q[h].to(dtype) @ k[h].to(dtype).T) * scale
        logit = torch.where(member, logit, torch.full_like(logit, -float("inf")))
        m = logit.max(dim=1, keepdim=True).values
        p = torch.exp(logit - m) * wts
        l = p.sum(dim=1, keepdim=True)
        out[h] = (p @ v[h].to(dtype)) / torch.clamp(l, min=1e-6)
    return out


# --------------------------------------------------------------------------- #
# module-level forward core  (M:59-85)
# --------------------------------------------------------------------------- #
def dsa_forward(q, k, v, q_idx, k_idx, w, top_k, dtype=torch.float32):
    """Indexer + top-k (lower-index ties) + routing-weighted attention for one
    batch element.  Returns (o (H,T,D), idx, valid, sel_scores)."""
    s = indexer_scores(q_idx, k_idx, w)
    idx, valid, sel = topk_lower_index(s, top_k)
    rw = sel * valid                                      # M:73
    o = dsa_attention(q, k, v, idx, valid, rw, dtype=dtype)
    return o, idx, valid, sel


# --------------------------------------------------------------------------- #
# backward  (K:128-339 indexer, K:569-762 attention; K:388-445, K:812-853 the Functions)
# --------------------------------------------------------------------------- #
def dsa_attention_bwd(d_out, q, k, v, o, idx, valid, rw, dtype=torch.float32):
    """Gradients of the routing-weighted attention as the reference's `_dsa_attention_bwd`
    computes them (K:569-762), one batch element: q, k, v, o, d_out (H, T, D); idx/valid/rw (T, K).

      logit_j = q.k[idx_j]/sqrt(D); m = max over valid j; l = sum_j exp(logit_j - m) rw_j;
      l_safe = max(l, 1e-6); sm_j = exp(logit_j - m)/l_safe; P_j = sm_j rw_j      (K:596-637, K:676-678)
      Di = sum_d dO O (K:641-656);  dP_j = dO.v[idx_j]                              (K:693)
      dV[idx_j] += P_j valid_j dO (K:694-700);  dRW_j = sum_h sm_j (dP_j - Di)     (K:702-708)
      dS_j = rw_j sm_j (dP_j - Di)/sqrt(D) (K:710); dQ += sum_j dS_j k[idx_j]; dK[idx_j] += dS_j q (K:735-748)

    Returns dq, dk, dv (H, T, D) and drw (T, K).  Equal to autograd through ``dsa_attention``
    wherever the 1e-6 clamp is not active.
    """
    H, T, D = q.shape
    scale = 1.0 / math.sqrt(D)
    qf, kf, vf, of, dof = (t.to(dtype) for t in (q, k, v, o, d_out))
    dq, dk, dv = torch.zeros_like(qf), torch.zeros_like(kf), torch.zeros_like(vf)
    drw = torch.zeros(idx.shape, dtype=dtype)
    ii = idx.long()
    vm = valid > 0
    w = rw.to(dtype)
    for h in range(H):
        kg, vg = kf[h][ii], vf[h][ii]                                     # (T, K, D)
        logit = torch.einsum("td,tkd->tk", qf[h], kg) * scale
        logit = torch.where(vm, logit, torch.full_like(logit, -float("inf")))
        m = logit.max(dim=1, keepdim=True).values
        e = torch.where(vm, torch.exp(logit - m), torch.zeros_like(logit))
        l_safe = torch.clamp((e * w).sum(dim=1, keepdim=True), min=1e-6)
        sm = e / l_safe
        di = (dof[h] * of[h]).sum(dim=1, keepdim=True)
        dp = torch.einsum("td,tkd->tk", dof[h], vg)
        g = torch.where(vm, sm * (dp - di), torch.zeros_like(sm))
        drw += g
        ds = w * g * scale
        dq[h] = torch.einsum("tk,tkd->td", ds, kg)
        dk[h].index_add_(0, ii.reshape(-1), (ds[:, :, None] * qf[h][:, None, :]).reshape(-1, D))
        pv = torch.where(vm, sm * w, torch.zeros_like(sm))
        dv[h].index_add_(0, ii.reshape(-1), (pv[:, :, None] * dof[h][:, None, :]).reshape(-1, D))
    return dq, dk, dv, drw


def indexer_bwd(d_scores, q_idx, k_idx, w, idx, valid, dtype=torch.float32):
    """Gradients of the indexer as the reference's three backward kernels compute them
    (K:128-339), one batch element: q_idx, k_idx (T, IH, ID); d_scores, idx, valid (T, K).

      g = d_scores * valid
      dQ[t,h,:] = sum_j g[t,j] W[h] K[idx[t,j],h,:]          (K:128-203)
      dK[idx[t,j],h,:] += g[t,j] W[h] Q[t,h,:]                (K:206-270)
      dW[h] = sum_{t,j} g[t,j] (Q[t,h,:] . K[idx[t,j],h,:])   (K:273-339)

    This is the gradient of  sum_h W[h] q_h.k_h  (the form the reference's backward assumes,
    K:116), NOT of the forward's relu((sum_h W_h q_h).(sum_h W_h k_h)) (K:66-70): the reference
    is inconsistent with itself here, and a drop-in follows what its training loop runs.
    """
    qf, kf, wf = q_idx.to(dtype), k_idx.to(dtype), w.to(dtype)
    g = (d_scores.to(dtype) * valid.to(dtype))
    ii = idx.long()
    T, IH, ID = qf.shape
    kg = kf[ii]                                                            # (T, K, IH, ID)
    dq = torch.einsum("tj,h,tjhd->thd", g, wf, kg)
    dk = torch.zeros_like(kf)
    dk.index_add_(0, ii.reshape(-1), (g[:, :, None, None] * wf[None, None, :, None] * qf[:, None, :, :]).reshape(-1, IH, ID))
    dw = torch.einsum("tj,thd,tjhd->h", g, qf, kg)
    return dq, dk, dw
