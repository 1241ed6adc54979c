"""Drop-in nn.Modules for the DSA slide encoder.

Constructor arguments, forward signatures, parameter names and shapes follow
src/sparse_wsi_vit/models/deepseek_sparse_attention.py of the reference
(DeepSeekSparseAttention :19-88, IndexerProjection :93-105, DSAViTBlock :108-166,
DSAViTSlideEncoder :169-305) so that a reference ``state_dict`` loads unchanged
and configs that name these classes keep working.  The attention itself runs on
the sm_100a kernels (``ops.dsa_sparse_attention``); projections, LayerNorm and
the MLP stay PyTorch/cuBLAS.  With gradients enabled the attention is one
differentiable op backed by the backward kernels (``ops.DSAModuleFunction``).
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from .ops import DSAModuleFunction, Rope2dFunction, dsa_sparse_attention, rope2d


def rope_qk_(qkv: Tensor, coords: Tensor, coord_high: float, num_cls: int = 0, theta: float = 10000.0) -> None:
    """2-D rotary embedding, in place, on the q and k slices of a fused projection output
    ``qkv (B, T, 3, H, D)``: patch tokens turn with their (y, x) coordinates, the ``num_cls``
    leading CLS tokens are left as they are -- the placement of the reference's ViT-5 attention
    (src/sparse_wsi_vit/models/vit_5/models_vit5.py:84-90, rope.py:72-97).
    ``coords`` is (B, T - num_cls, 2) or (T - num_cls, 2), in the units of ``coord_high``."""
    B, T = qkv.shape[:2]
    c = coords.reshape(B, -1, 2) if coords.dim() == 3 else coords.reshape(1, -1, 2).expand(B, -1, -1)
    if c.shape[1] != T - num_cls:
        raise ValueError(f"coords cover {c.shape[1]} tokens, the sequence has {T - num_cls} patch tokens")
    if T == 0:
        return
    for b in range(B):
        cb = c[b].to(torch.float32)
        if num_cls:
            cb = torch.cat([cb.new_zeros((num_cls, 2)), cb], dim=0)
        for i in (0, 1):
            x = qkv[b, :, i]
            rope2d(x, cb, coord_high, theta=theta, skip_tokens=num_cls, out=x)


class IndexerProjection(nn.Module):
    """Two Linears producing the indexer queries/keys, (B, T, IH, ID) each."""

    def __init__(self, d_model, indexer_heads, indexer_dim):
        super().__init__()
        self.indexer_heads = indexer_heads
        self.indexer_dim = indexer_dim
        self.q_proj = nn.Linear(d_model, indexer_heads * indexer_dim)
        self.k_proj = nn.Linear(d_model, indexer_heads * indexer_dim)

    def forward(self, x):
        shape = (*x.shape[:2], self.indexer_heads, self.indexer_dim)
        return self.q_proj(x).view(shape), self.k_proj(x).view(shape)


class DeepSeekSparseAttention(nn.Module):
    """Token-level top-k sparse attention with a lightning indexer.

    ``BLOCK_Q/BLOCK_K/BLOCK_D`` are the reference's Triton tile sizes; they are
    accepted for signature compatibility and ignored.
    """

    def __init__(self, d_model, attention_heads, indexer_heads, indexer_dim, top_k, BLOCK_Q=None, BLOCK_K=None,
                 BLOCK_D=None):
        super().__init__()
        if d_model % attention_heads != 0:
            raise ValueError(f"d_model ({d_model}) must be divisible by attention_heads ({attention_heads})")
        self.d_model = d_model
        self.attention_heads = attention_heads
        self.head_dim = d_model // attention_heads
        self.indexer_heads = indexer_heads
        self.indexer_dim = indexer_dim
        self.top_k = top_k
        self.BLOCK_Q, self.BLOCK_K, self.BLOCK_D = BLOCK_Q, BLOCK_K, BLOCK_D

        self.indexer_head_weights = nn.Parameter(torch.randn(indexer_heads))
        self.indexer_proj = IndexerProjection(d_model, indexer_heads, indexer_dim)
        self.qkv_proj = nn.Linear(d_model, 3 * d_model)
        self.out_proj = nn.Linear(d_model, d_model)
        self._cat = None                     # (key, weight, bias) of the fused projection, inference only

    def _project(self, x):
        """qkv (B,T,3,H,D) and the indexer projections (B,T,IH,ID).  Without gradients the three Linears
        (qkv_proj, indexer q_proj, k_proj; deepseek_sparse_attention.py:54, :59) run as ONE GEMM over
        the concatenated weights (cached until a parameter changes); the results are views of its
        output."""
        B, T, _ = x.shape
        H, D, IH, ID = self.attention_heads, self.head_dim, self.indexer_heads, self.indexer_dim
        lins = (self.qkv_proj, self.indexer_proj.q_proj, self.indexer_proj.k_proj)
        if torch.is_grad_enabled() and any(p.requires_grad for l in lins for p in l.parameters()):
            q_idx, k_idx = self.indexer_proj(x)
            return self.qkv_proj(x).view(B, T, 3, H, D), q_idx, k_idx
        key = tuple((p.data_ptr(), p._version, p.dtype) for l in lins for p in l.parameters())
        if self._cat is None or self._cat[0] != key:
            with torch.no_grad():
                self._cat = (key, torch.cat([l.weight for l in lins], dim=0), torch.cat([l.bias for l in lins], dim=0))
        y = torch.nn.functional.linear(x, self._cat[1], self._cat[2])
        E3, n = 3 * self.d_model, IH * ID
        return (y[..., :E3].unflatten(-1, (3, H, D)), y[..., E3:E3 + n].unflatten(-1, (IH, ID)),
                y[..., E3 + n:].unflatten(-1, (IH, ID)))

    def forward(self, x, coords=None, coord_high=None, num_cls=0, rope_theta=10000.0):
        """``x (B, T, d_model)``.  The reference's layer has no positional term; with ``coords``
        (and ``coord_high``) q and k of the patch tokens are first turned by the 2-D rotary
        embedding (``rope_qk_``), the ``num_cls`` leading tokens excepted."""
        B, T, _ = x.shape
        H, D = self.attention_heads, self.head_dim
        # [q | k | v] outermost, then head, then head-dim; the kernels take the
        # (B, H, T, D) views as they are (strided), no contiguous copies.
        if coords is not None and coord_high is None:
            raise ValueError("coords need coord_high (the coordinate that maps to one radian per unit frequency)")
        qkv, q_idx, k_idx = self._project(x)
        if torch.is_grad_enabled() and (qkv.requires_grad or q_idx.requires_grad or
                                        self.indexer_head_weights.requires_grad):
            # training: one differentiable op (fused forward, the two backward kernels chained)
            qt, kt, vt = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]            # (B, T, H, D)
            if coords is not None:
                if B != 1:
                    raise ValueError("2-D RoPE handles one slide at a time (batch 1), like the reference")
                c = coords.reshape(-1, 2).to(torch.float32)
                c = torch.cat([c.new_zeros((num_cls, 2)), c], dim=0) if num_cls else c
                qt = Rope2dFunction.apply(qt, c, coord_high, rope_theta, num_cls)
                kt = Rope2dFunction.apply(kt, c, coord_high, rope_theta, num_cls)
            o = DSAModuleFunction.apply(qt.transpose(1, 2), kt.transpose(1, 2), vt.transpose(1, 2), q_idx, k_idx,
                                        self.indexer_head_weights, self.top_k, x.dtype)
            return self.out_proj(o.transpose(1, 2).reshape(B, T, H * D).to(x.dtype))
        rope = None
        if coords is not None:
            # rotated in place inside the prologue launch (one row of coordinates per token, zeros for CLS)
            c = coords.reshape(B if coords.dim() == 3 else 1, -1, 2).to(torch.float32)
            if c.shape[1] != T - num_cls:
                raise ValueError(f"coords cover {c.shape[1]} tokens, the sequence has {T - num_cls} patch tokens")
            c = torch.cat([c.new_zeros((c.shape[0], num_cls, 2)), c], dim=1) if num_cls else c
            rope = (c, coord_high, rope_theta, num_cls)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        o = dsa_sparse_attention(q, k, v, q_idx, k_idx, self.indexer_head_weights, self.top_k, out_dtype=x.dtype,
                                 rope=rope)
        return self.out_proj(o.transpose(1, 2).reshape(B, T, H * D).to(x.dtype))


class DSAViTBlock(nn.Module):
    """Pre-norm transformer block: x + attn(LN(x)); x + MLP(LN(x))."""

    def __init__(self, embed_dim: int, num_heads: int, indexer_heads: int = 4, indexer_dim: int = 32,
                 top_k: int = 512, block_q: int = 16, block_k: int = 32, block_d: int = 32,
                 expansion_factor: float = 4.0, attn_dropout: float = 0.0, proj_dropout: float = 0.0) -> None:
        super().__init__()
        hidden = int(embed_dim * expansion_factor)
        self.norm1 = nn.LayerNorm(embed_dim)
        self.attn = DeepSeekSparseAttention(embed_dim, num_heads, indexer_heads, indexer_dim, top_k, block_q,
                                            block_k, block_d)
        self.drop1 = nn.Dropout(proj_dropout)
        self.norm2 = nn.LayerNorm(embed_dim)
        self.mlp = nn.Sequential(nn.Linear(embed_dim, hidden), nn.GELU(), nn.Dropout(proj_dropout),
                                 nn.Linear(hidden, embed_dim), nn.Dropout(proj_dropout))

    def forward(self, x: Tensor, coords=None, coord_high=None, num_cls: int = 0, rope_theta: float = 10000.0) -> Tensor:
        x = x + self.drop1(self.attn(self.norm1(x), coords, coord_high, num_cls, rope_theta))
        return x + self.mlp(self.norm2(x))


class DSAViTSlideEncoder(nn.Module):
    """Bag of patch embeddings -> slide logits: input projection, learned CLS
    tokens in front, DSA blocks, LayerNorm, softmax-weighted pooling over the
    CLS tokens, linear head.  Returns ``{"logits": (B, out_features)}``."""

    def __init__(self, in_features: int = 1280, out_features: int = 1, embed_dim: int = 384, num_heads: int = 6,
                 num_layers: int = 6, num_cls: int = 2, indexer_heads: int = 4, indexer_dim: int = 32,
                 top_k: int = 512, block_q: int = 16, block_k: int = 32, block_d: int = 32,
                 expansion_factor: float = 4.0, attn_dropout: float = 0.0, proj_dropout: float = 0.0,
                 gradient_checkpointing: bool = False, rope_coord_high=None, rope_theta: float = 10000.0) -> None:
        super().__init__()
        if embed_dim % num_heads != 0:
            raise ValueError(f"embed_dim ({embed_dim}) must be divisible by num_heads ({num_heads}). "
                             f"Recommended: embed_dim // num_heads == 64 or 128.")
        self.gradient_checkpointing = gradient_checkpointing
        # Not in the reference's encoder: with a coordinate scale set, forward(x, coords) applies the
        # 2-D rotary embedding to q and k of the patch tokens in every layer.
        self.rope_coord_high = rope_coord_high
        self.rope_theta = rope_theta
        self.num_cls = num_cls
        self.embed_dim = embed_dim
        self.out_features = out_features

        self.input_proj = nn.Linear(in_features, embed_dim)
        self.cls_tokens = nn.Parameter(torch.zeros(1, num_cls, embed_dim))
        nn.init.trunc_normal_(self.cls_tokens, std=0.02)
        self.blocks = nn.ModuleList(
            DSAViTBlock(embed_dim, num_heads, indexer_heads, indexer_dim, top_k, block_q, block_k, block_d,
                        expansion_factor, attn_dropout, proj_dropout) for _ in range(num_layers))
        self.norm = nn.LayerNorm(embed_dim)
        self.cls_pool = nn.Linear(embed_dim, 1, bias=False)
        self.head = nn.Linear(embed_dim, out_features)
        nn.init.xavier_uniform_(self.input_proj.weight)
        nn.init.zeros_(self.input_proj.bias)
        nn.init.zeros_(self.head.bias)

    def forward(self, x: Tensor, coords=None) -> dict[str, Tensor]:
        """``x (B, N, in_features)`` or ``(N, in_features)``; ``coords`` (optional, (B, N, 2) or (N, 2))
        are used only when the encoder was built with ``rope_coord_high`` (the reference's wrapper
        calls ``network(inputs, coords)``, experiments/lightning_wrappers/wsi_attn_wrapper.py:96)."""
        if x.dim() == 2:
            x = x.unsqueeze(0)
        x = self.input_proj(x)
        x = torch.cat([self.cls_tokens.expand(x.shape[0], -1, -1).to(x.dtype), x], dim=1)
        rope = coords is not None and self.rope_coord_high is not None
        for blk in self.blocks:
            x = blk(x, coords, self.rope_coord_high, self.num_cls, self.rope_theta) if rope else blk(x)
        x = self.norm(x)
        cls = x[:, :self.num_cls]
        pooled = (torch.softmax(self.cls_pool(cls), dim=1) * cls).sum(dim=1)
        return {"logits": self.head(pooled)}
