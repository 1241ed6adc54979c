"""CPU restatement of the slide encoders around the attention layers, fp32.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

  M = src/sparse_wsi_vit/models/deepseek_sparse_attention.py   (DSAViTBlock :108-166, DSAViTSlideEncoder :169-305)
  S = src/sparse_wsi_vit/models/static_sparse_attention.py     (StaticSparseViTBlock :191-236, encoder :239-345)
  V = src/sparse_wsi_vit/models/vit_5/models_vit5.py            (RoPE placement :84-90)

The blocks are the reference's pre-norm blocks (x + attn(LN(x)); x + MLP(LN(x)), M:163-166), the head
is its softmax-weighted pooling over the CLS tokens (M:299-301).  Two composites that the reference
never builds are assembled here from those parts and are therefore PARITY UNPINNED as wholes:
  * the DSA encoder with 2-D RoPE on q / k of the patch tokens (CLS tokens unrotated, V:84-90);
  * the 2-D block-pattern encoder (block-sparse attention + 2-D RoPE), patches first and the CLS
    tokens in a trailing global block.
All functions take a ``state_dict`` with the reference's parameter names.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import dsa as O
from . import static_attn as SA


def _ln(x, sd, name):
    return F.layer_norm(x, (x.shape[-1],), sd[name + ".weight"], sd[name + ".bias"])


def _lin(x, sd, name):
    return F.linear(x, sd[name + ".weight"], sd.get(name + ".bias"))


def _mlp(x, sd, prefix):
    return _lin(F.gelu(_lin(x, sd, prefix + ".0")), sd, prefix + ".3")          # Linear, GELU, (Dropout), Linear (M:155-161)


def _cls_head(x_cls, sd):
    cls = _ln(x_cls, sd, "norm")                                                # M:297-301
    pooled = (torch.softmax(F.linear(cls, sd["cls_pool.weight"]), dim=0) * cls).sum(dim=0)
    return _lin(pooled, sd, "head")


def dsa_attention_layer(y, sd, prefix, H, IH, ID, top_k, coords=None, coord_high=None, num_cls=0, theta=10000.0):
    """y (T, E) -> (T, E): qkv / indexer projections, optional RoPE, indexer + top-k + routing-weighted
    attention (M:50-88), out_proj."""
    T, E = y.shape
    D = E // H
    qkv = _lin(y, sd, prefix + ".qkv_proj").view(T, 3, H, D)
    q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]                                   # (T, H, D)
    if coords is not None:
        c = torch.cat([torch.zeros(num_cls, 2), coords.float()], dim=0)
        q = torch.cat([q[:num_cls], SA.rope2d_apply(q, c, coord_high, theta)[num_cls:]], dim=0)
        k = torch.cat([k[:num_cls], SA.rope2d_apply(k, c, coord_high, theta)[num_cls:]], dim=0)
    qi = _lin(y, sd, prefix + ".indexer_proj.q_proj").view(T, IH, ID)
    ki = _lin(y, sd, prefix + ".indexer_proj.k_proj").view(T, IH, ID)
    o, _, _, _ = O.dsa_forward(q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1), qi, ki,
                               sd[prefix + ".indexer_head_weights"], top_k)
    return _lin(o.transpose(0, 1).reshape(T, E), sd, prefix + ".out_proj")


def dsa_encoder_forward(sd, x, num_layers, H, IH, ID, top_k, num_cls, coords=None, coord_high=None, theta=10000.0):
    """x (N, in_features) -> logits (out_features,).  Token order [CLS..., patches...] (M:287-288)."""
    sd = {k: v.float() for k, v in sd.items()}
    t = _lin(x.float(), sd, "input_proj")
    t = torch.cat([sd["cls_tokens"][0], t], dim=0)
    for i in range(num_layers):
        p = f"blocks.{i}"
        t = t + dsa_attention_layer(_ln(t, sd, p + ".norm1"), sd, p + ".attn", H, IH, ID, top_k, coords, coord_high,
                                    num_cls, theta)
        t = t + _mlp(_ln(t, sd, p + ".norm2"), sd, p + ".mlp")
    return _cls_head(t[:num_cls], sd)


def block2d_encoder_forward(sd, x, coords, row_ptr, col_idx, block, num_layers, H, num_cls, coord_high, theta=10000.0,
                            pool="cls"):
    """2-D block-pattern encoder: token order [patches..., CLS...] (the CLS tokens sit in trailing
    global blocks of the pattern), 2-D RoPE on q / k of the patch tokens, block-sparse attention
    (dense attention under the expanded block mask), the reference's blocks and head.  pool="mean"
    replaces the CLS pooling by the mean over the patch tokens."""
    sd = {k: v.float() for k, v in sd.items()}
    n = x.shape[0]
    t = torch.cat([_lin(x.float(), sd, "input_proj"), sd["cls_tokens"][0]], dim=0)
    T, E = t.shape
    D = E // H
    c = torch.cat([coords.float(), torch.zeros(num_cls, 2)], dim=0)
    mask = SA.expand_block_mask(row_ptr, col_idx, block, T, T)
    for i in range(num_layers):
        p = f"blocks.{i}"
        y = _ln(t, sd, p + ".norm1")
        qkv = _lin(y, sd, p + ".attn.qkv").view(T, 3, H, D)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        q = torch.cat([SA.rope2d_apply(q, c, coord_high, theta)[:n], q[n:]], dim=0)
        k = torch.cat([SA.rope2d_apply(k, c, coord_high, theta)[:n], k[n:]], dim=0)
        o = SA.masked_attention(q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1), mask)
        t = t + _lin(o.transpose(0, 1).reshape(T, E), sd, p + ".attn.out_proj")
        t = t + _mlp(_ln(t, sd, p + ".norm2"), sd, p + ".mlp")
    if pool == "mean":
        return _lin(_ln(t[:n], sd, "norm").mean(dim=0), sd, "head")
    return _cls_head(t[n:], sd)
