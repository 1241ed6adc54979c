"""CPU restatements of the reference's static sparse attention and 2-D RoPE,
and the library-defined oracle for 2-D block-sparse attention.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Reference files:
  S = src/sparse_wsi_vit/models/static_sparse_attention.py
  R = src/sparse_wsi_vit/models/vit_5/rope.py
  V = src/sparse_wsi_vit/models/vit_5/models_vit5.py
"""
from __future__ import annotations

import math

import torch


def masked_attention(q, k, v, mask, dtype=torch.float32):
    """softmax(q k^T / sqrt(D) + mask) v with a boolean keep-mask.

    q (..., Tq, D), k, v (..., Tk, D), mask (Tq, Tk) bool (True = attend).
    This is the math both ``F.scaled_dot_product_attention`` call sites of the
    static path reduce to (S:87-89, S:93-95, S:180-186).  Rows with no kept key
    return zeros.
    """
    D = q.shape[-1]
    s = (q.to(dtype) @ k.to(dtype).transpose(-1, -2)) / math.sqrt(D)
    s = s.masked_fill(~mask, float("-inf"))
    m = s.max(dim=-1, keepdim=True).values
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = torch.exp(s - m)
    l = p.sum(dim=-1, keepdim=True)
    return (p @ v.to(dtype)) / torch.where(l == 0, torch.ones_like(l), l)


def static_window_mask(seq_len: int, num_cls: int, window: int, dilation: int) -> torch.Tensor:
    """Token-level keep-mask equivalent to the reference's static pattern.

    CLS rows attend everything (S:87-89); patch rows attend all CLS keys plus the
    patches ``i + j*dilation, j in [-window, window]`` inside the sequence, not
    wrapped (S:132-168).  With window == 0 patches see only the CLS keys (S:92-95).
    """
    i = torch.arange(seq_len)
    pi = i - num_cls
    diff = pi[:, None] - pi[None, :]
    near = (diff.abs() <= window * dilation) & (diff % max(dilation, 1) == 0)
    if window == 0:
        near = torch.zeros_like(near)
    is_cls_q = (i < num_cls)[:, None]
    is_cls_k = (i < num_cls)[None, :]
    return is_cls_q | is_cls_k | (near & ~is_cls_q & ~is_cls_k)


def static_sparse_attention(x, sd, num_heads, num_cls, window, dilation, dtype=torch.float32):
    """Forward of the reference module ``StaticSparseAttention`` (S:62-103) from its state_dict."""
    B, L, E = x.shape
    hd = E // num_heads
    qkv = torch.nn.functional.linear(x.to(dtype), sd["qkv.weight"].to(dtype), sd["qkv.bias"].to(dtype))
    qkv = qkv.reshape(B, L, 3, num_heads, hd).permute(2, 0, 3, 1, 4)
    q, k, v = qkv.unbind(0)
    mask = static_window_mask(L, num_cls, window, dilation)
    o = masked_attention(q, k, v, mask, dtype)
    o = o.transpose(1, 2).reshape(B, L, E)
    return torch.nn.functional.linear(o, sd["out_proj.weight"].to(dtype), sd["out_proj.bias"].to(dtype))


def expand_block_mask(row_ptr, col_idx, block: int, Tq: int, Tk: int, rows=None) -> torch.Tensor:
    """CSR list of key blocks per query block -> (Tq, Tk) boolean keep-mask; with `rows` (1-D
    tensor of query indices) only those rows, (len(rows), Tk), so that long sequences can be
    checked on a sample of rows."""
    if rows is not None:
        mask = torch.zeros((len(rows), Tk), dtype=torch.bool)
        for i, r in enumerate(rows.tolist()):
            qb = r // block
            for j in range(int(row_ptr[qb]), int(row_ptr[qb + 1])):
                kb = int(col_idx[j])
                mask[i, kb * block:min(Tk, (kb + 1) * block)] = True
        return mask
    mask = torch.zeros((Tq, Tk), dtype=torch.bool)
    nqb = len(row_ptr) - 1
    for qb in range(nqb):
        q0, q1 = qb * block, min(Tq, (qb + 1) * block)
        for j in range(int(row_ptr[qb]), int(row_ptr[qb + 1])):
            kb = int(col_idx[j])
            mask[q0:q1, kb * block:min(Tk, (kb + 1) * block)] = True
    return mask


def block_sparse_attention(q, k, v, row_ptr, col_idx, block, dtype=torch.float32):
    """Library-defined oracle ("parity unpinned": no such code in the reference).

    Plain softmax attention restricted to the listed key blocks; q (H,Tq,D),
    k, v (H,Tk,D).  Equivalent to dense SDPA under the expanded block mask, the
    same dense-mask equivalence the reference's static path satisfies.
    """
    mask = expand_block_mask(row_ptr, col_idx, block, q.shape[-2], k.shape[-2])
    return masked_attention(q, k, v, mask, dtype)


# ------------------------------------------------------------------- 2-D RoPE
def rope2d_angles(coords, head_dim: int, coord_high: float, theta: float = 10000.0):
    """Per-token rotation angles, (L, head_dim) (R:56-59, R:81-93).

    The module is built with ``dim = head_dim // 2`` (V:51-57) so there are
    head_dim/4 frequencies ``theta^(-2i/dim)``; each is repeated for two
    adjacent channels; the first half of the head uses coords[..., 0], the
    second half coords[..., 1], both divided by ``coord_high``.
    """
    dim = head_dim // 2
    freqs = 1.0 / (theta ** (torch.arange(0, dim, 2)[: dim // 2].float() / dim))
    t0 = coords[..., 0].float() / coord_high
    t1 = coords[..., 1].float() / coord_high
    f0 = (t0[..., None] * freqs).repeat_interleave(2, dim=-1)
    f1 = (t1[..., None] * freqs).repeat_interleave(2, dim=-1)
    return torch.cat([f0, f1], dim=-1)


def rope2d_apply(x, coords, coord_high: float, theta: float = 10000.0):
    """x (L, H, hd), coords (L, 2) -> rotated x (R:33-37, R:95-97):
    ``x*cos + rotate_half(x)*sin`` with rotate_half (x0, x1) -> (-x1, x0) on
    adjacent channel pairs."""
    L, H, hd = x.shape
    ang = rope2d_angles(coords, hd, coord_high, theta)   # (L, hd)
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xr = x.reshape(L, H, hd // 2, 2)
    rot = torch.stack((-xr[..., 1], xr[..., 0]), dim=-1).reshape(L, H, hd)
    return x * cos + rot * sin
