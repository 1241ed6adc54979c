"""Drop-in nn.Modules for the static sparse attention encoder.

Constructor arguments, forward signatures and parameter names follow
src/sparse_wsi_vit/models/static_sparse_attention.py (StaticSparseAttention :11-103,
StaticSparseViTBlock :191-236, StaticSparseViTSlideEncoder :239-345).  The attention runs on the
block-sparse tensor-core kernel (bf16 / fp16 activations, e.g. under autocast) with the reference's
token pattern applied inside the blocks the pattern touches, or -- for fp32 activations -- on the
exact list kernel over the pattern's explicit key lists, instead of the reference's dense
(N, N*ctx) masked SDPA.  Forward only; attention
dropout is not applied (the reference applies it in training mode only).

``BlockSparseAttention2D`` is the 2-D block pattern with optional 2-D RoPE the target asks for; the
reference has no such module.
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from .ops import block_sparse_attention, dsa_attention_gather, rope2d
from .patterns import static_window_blocks, static_window_lists

_BLOCK = 128


class StaticSparseAttention(nn.Module):
    def __init__(self, embed_dim: int, num_heads: int, num_cls: int = 1, window_size: int = 0, dilation: int = 1,
                 attn_dropout: float = 0.0) -> None:
        super().__init__()
        if embed_dim % num_heads != 0:
            raise ValueError(f"embed_dim ({embed_dim}) must be divisible by num_heads ({num_heads}) "
                             f"(preferably embed_dim/num_heads = 64)")
        self.embed_dim, self.num_heads = embed_dim, num_heads
        self.num_cls, self.window_size, self.dilation = num_cls, window_size, dilation
        self.head_dim = embed_dim // num_heads
        self.attn_dropout = attn_dropout
        self.qkv = nn.Linear(embed_dim, 3 * embed_dim, bias=True)
        self.out_proj = nn.Linear(embed_dim, embed_dim, bias=True)
        self._lists = {}

    def _block_list(self, seq_len, device):
        key = (seq_len, device)
        if key not in self._lists:
            rp, ci = static_window_blocks(seq_len, self.num_cls, self.window_size, self.dilation, _BLOCK)
            self._lists[key] = (torch.from_numpy(rp).to(device), torch.from_numpy(ci).to(device))
        return self._lists[key]

    def _key_lists(self, seq_len, device):
        key = ("lists", seq_len, device)
        if key not in self._lists:
            idx_p, val_p = static_window_lists(seq_len, self.num_cls, self.window_size, self.dilation)
            self._lists[key] = (torch.from_numpy(idx_p).to(device), torch.from_numpy(val_p).to(device))
        return self._lists[key]

    def _forward_fp32(self, q, k, v):
        """fp32 inputs keep fp32 arithmetic: the pattern is small explicit key lists (the CLS keys and
        the 2W+1 window keys of every patch row; all keys for the CLS rows), so the exact CUDA-core
        list kernel serves it (softmax weights 1).  Within 1e-4 of the reference's fp32 module."""
        B, H, L, D = q.shape
        C = self.num_cls
        o = torch.empty((B, H, L, D), dtype=q.dtype, device=q.device)
        if C > 0:
            idx_c = torch.arange(L, dtype=torch.int32, device=q.device).expand(B, C, L)
            ones = torch.ones((1, 1, 1), device=q.device).expand(B, C, L)
            dsa_attention_gather(q[:, :, :C], k, v, idx_c, ones, ones, o[:, :, :C])
        if L > C:
            idx_p, val_p = self._key_lists(L, q.device)
            idx_p, val_p = idx_p.expand(B, -1, -1), val_p.expand(B, -1, -1)
            dsa_attention_gather(q[:, :, C:], k, v, idx_p, val_p, val_p, o[:, :, C:])
        return o

    def forward(self, x: Tensor) -> Tensor:
        B, L, E = x.shape
        H, D = self.num_heads, self.head_dim
        qkv = self.qkv(x).view(B, L, 3, H, D)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        if qkv.dtype == torch.float32:
            o = self._forward_fp32(q, k, v)
            return self.out_proj(o.transpose(1, 2).reshape(B, L, E))
        rp, ci = self._block_list(L, x.device)
        o = block_sparse_attention(q, k, v, rp, ci, _BLOCK, mode=1, num_cls=self.num_cls, window=self.window_size,
                                   dilation=self.dilation, out_dtype=x.dtype)
        return self.out_proj(o.transpose(1, 2).reshape(B, L, E))


class StaticSparseViTBlock(nn.Module):
    def __init__(self, embed_dim: int, num_heads: int, num_cls: int = 1, window_size: int = 0, dilation: int = 1,
                 expansion_factor: float = 4.0, attn_dropout: float = 0.0, proj_dropout: float = 0.0) -> None:
        super().__init__()
        hidden = int(embed_dim * expansion_factor)
        self.norm1 = nn.LayerNorm(embed_dim)
        self.attn = StaticSparseAttention(embed_dim, num_heads, num_cls, window_size, dilation, attn_dropout)
        self.drop1 = nn.Dropout(proj_dropout)
        self.norm2 = nn.LayerNorm(embed_dim)
        self.mlp = nn.Sequential(nn.Linear(embed_dim, hidden), nn.GELU(), nn.Dropout(proj_dropout),
                                 nn.Linear(hidden, embed_dim), nn.Dropout(proj_dropout))

    def forward(self, x: Tensor) -> Tensor:
        x = x + self.drop1(self.attn(self.norm1(x)))
        return x + self.mlp(self.norm2(x))


class StaticSparseViTSlideEncoder(nn.Module):
    def __init__(self, in_features: int = 1280, out_features: int = 1, embed_dim: int = 384, num_heads: int = 6,
                 num_layers: int = 6, num_cls: int = 2, window_size: int = 0, dilation: int = 1,
                 expansion_factor: float = 4.0, attn_dropout: float = 0.0, proj_dropout: float = 0.0) -> None:
        super().__init__()
        self.num_cls, self.embed_dim, self.out_features = num_cls, embed_dim, out_features
        self.input_proj = nn.Linear(in_features, embed_dim)
        self.cls_tokens = nn.Parameter(torch.zeros(1, num_cls, embed_dim))
        nn.init.trunc_normal_(self.cls_tokens, std=0.02)
        self.blocks = nn.ModuleList(
            StaticSparseViTBlock(embed_dim, num_heads, num_cls, window_size, dilation, expansion_factor, attn_dropout,
                                 proj_dropout) for _ in range(num_layers))
        self.norm = nn.LayerNorm(embed_dim)
        self.cls_pool = nn.Linear(embed_dim, 1, bias=False)
        self.head = nn.Linear(embed_dim, out_features)
        nn.init.xavier_uniform_(self.input_proj.weight)
        nn.init.zeros_(self.input_proj.bias)
        nn.init.zeros_(self.head.bias)

    def forward(self, x: Tensor, coords=None) -> dict[str, Tensor]:
        """``coords`` is accepted and ignored: the reference's wrapper calls ``network(inputs, coords)``
        (experiments/lightning_wrappers/wsi_attn_wrapper.py:96) although this encoder, like the
        reference's, has no positional term."""
        if x.dim() == 2:
            x = x.unsqueeze(0)
        x = self.input_proj(x)
        x = torch.cat([self.cls_tokens.expand(x.shape[0], -1, -1).to(x.dtype), x], dim=1)
        for blk in self.blocks:
            x = blk(x)
        x = self.norm(x)
        cls = x[:, :self.num_cls]
        pooled = (torch.softmax(self.cls_pool(cls), dim=1) * cls).sum(dim=1)
        return {"logits": self.head(pooled)}


class BlockSparseAttention2D(nn.Module):
    """Multi-head attention under a 2-D block pattern given as a CSR key-block list, with 2-D RoPE on
    the patch tokens' grid coordinates when `coords` is passed (the last `num_global` tokens -- CLS --
    are not rotated, mirroring how the dense ViT-5 skips its CLS/register tokens,
    vit_5/models_vit5.py:84-90).  Same parameters as StaticSparseAttention (`qkv`, `out_proj`)."""

    def __init__(self, embed_dim: int, num_heads: int, block: int = 64, coord_high: float = 1.0,
                 theta: float = 10000.0) -> None:
        super().__init__()
        if embed_dim % num_heads != 0:
            raise ValueError(f"embed_dim ({embed_dim}) must be divisible by num_heads ({num_heads})")
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, embed_dim // num_heads
        self.block, self.coord_high, self.theta = block, coord_high, theta
        self.qkv = nn.Linear(embed_dim, 3 * embed_dim, bias=True)
        self.out_proj = nn.Linear(embed_dim, embed_dim, bias=True)

    def forward(self, x: Tensor, row_ptr: Tensor, col_idx: Tensor, coords: Tensor | None = None,
                num_global: int = 0) -> Tensor:
        B, L, E = x.shape
        H, D = self.num_heads, self.head_dim
        qkv = self.qkv(x).view(B, L, 3, H, D)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]          # (B, L, H, D) token-major views
        if coords is not None:
            if B != 1:
                raise ValueError("2-D RoPE handles one slide at a time (batch 1), like the reference")
            n_rot = L - num_global
            cpad = torch.zeros((L, 2), dtype=torch.float32, device=x.device)
            cpad[:n_rot] = coords.reshape(-1, 2)[:n_rot].float()
            # rotate the first n_rot tokens; the trailing global tokens keep angle 0 (identity)
            q = rope2d(q.to(torch.bfloat16), cpad, self.coord_high, self.theta)
            k = rope2d(k.to(torch.bfloat16), cpad, self.coord_high, self.theta)
        o = block_sparse_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), row_ptr, col_idx,
                                   self.block, mode=0, out_dtype=x.dtype)
        return self.out_proj(o.transpose(1, 2).reshape(B, L, E))


class BlockSparse2DViTBlock(nn.Module):
    """The reference's pre-norm block (static_sparse_attention.py:191-236) around ``BlockSparseAttention2D``."""

    def __init__(self, embed_dim: int, num_heads: int, block: int = 64, coord_high: float = 1.0, theta: float = 10000.0,
                 expansion_factor: float = 4.0, proj_dropout: float = 0.0) -> None:
        super().__init__()
        hidden = int(embed_dim * expansion_factor)
        self.norm1 = nn.LayerNorm(embed_dim)
        self.attn = BlockSparseAttention2D(embed_dim, num_heads, block, coord_high, theta)
        self.drop1 = nn.Dropout(proj_dropout)
        self.norm2 = nn.LayerNorm(embed_dim)
        self.mlp = nn.Sequential(nn.Linear(embed_dim, hidden), nn.GELU(), nn.Dropout(proj_dropout),
                                 nn.Linear(hidden, embed_dim), nn.Dropout(proj_dropout))

    def forward(self, x: Tensor, row_ptr: Tensor, col_idx: Tensor, coords: Tensor | None, num_global: int) -> Tensor:
        x = x + self.drop1(self.attn(self.norm1(x), row_ptr, col_idx, coords, num_global))
        return x + self.mlp(self.norm2(x))


class BlockSparse2DViTSlideEncoder(nn.Module):
    """Slide encoder over a 2-D block pattern: the skeleton of ``StaticSparseViTSlideEncoder`` (same
    parameter names: cls_tokens, input_proj, blocks.i.{norm1, attn.qkv, attn.out_proj, norm2, mlp},
    norm, cls_pool, head) with block-sparse attention and 2-D RoPE on the patch tokens.  The
    reference has no such model; it is the composite the 4096-patch / 64x64-grid configuration asks
    for.  Token order: patches first (block-major, one spatial tile per block), the CLS tokens in a
    trailing global block.  ``pool``: "cls" = the reference's softmax-weighted CLS pooling, "mean" =
    mean over the patch tokens."""

    def __init__(self, in_features: int = 1280, out_features: int = 1, embed_dim: int = 384, num_heads: int = 6,
                 num_layers: int = 2, num_cls: int = 1, block: int = 64, coord_high: float = 1.0,
                 rope_theta: float = 10000.0, expansion_factor: float = 4.0, proj_dropout: float = 0.0,
                 pool: str = "cls") -> None:
        super().__init__()
        if pool not in ("cls", "mean"):
            raise ValueError(f"pool must be 'cls' or 'mean', got {pool!r}")
        self.num_cls, self.embed_dim, self.out_features, self.block, self.pool = num_cls, embed_dim, out_features, block, pool
        self.input_proj = nn.Linear(in_features, embed_dim)
        self.cls_tokens = nn.Parameter(torch.zeros(1, num_cls, embed_dim))
        nn.init.trunc_normal_(self.cls_tokens, std=0.02)
        self.blocks = nn.ModuleList(
            BlockSparse2DViTBlock(embed_dim, num_heads, block, coord_high, rope_theta, expansion_factor, proj_dropout)
            for _ in range(num_layers))
        self.norm = nn.LayerNorm(embed_dim)
        self.cls_pool = nn.Linear(embed_dim, 1, bias=False)
        self.head = nn.Linear(embed_dim, out_features)
        nn.init.xavier_uniform_(self.input_proj.weight)
        nn.init.zeros_(self.input_proj.bias)
        nn.init.zeros_(self.head.bias)

    def forward(self, x: Tensor, coords: Tensor, row_ptr: Tensor, col_idx: Tensor) -> dict[str, Tensor]:
        """x (N, in_features) or (1, N, in_features); coords (N, 2); row_ptr / col_idx: the CSR key-block
        list over the N + num_cls tokens (int32, on x's device)."""
        if x.dim() == 2:
            x = x.unsqueeze(0)
        n = x.shape[1]
        x = torch.cat([self.input_proj(x), self.cls_tokens.expand(x.shape[0], -1, -1).to(x.dtype)], dim=1)
        for blk in self.blocks:
            x = blk(x, row_ptr, col_idx, coords, self.num_cls)
        x = self.norm(x)
        if self.pool == "mean":
            return {"logits": self.head(x[:, :n].mean(dim=1))}
        cls = x[:, n:]
        pooled = (torch.softmax(self.cls_pool(cls), dim=1) * cls).sum(dim=1)
        return {"logits": self.head(pooled)}
