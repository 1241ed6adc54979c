"""Sequence sharding of the DSA forward across the GPUs of one box.

Every query row is independent given all keys, so each rank keeps a contiguous
slice of the slide's tokens (its queries) and the only exchange per attention
layer is an all-gather of the keys: the indexer keys first (small; the top-k
passes start as soon as they land), then K and V on a side stream, overlapped
with the indexer/top-k kernels.  Nothing is reduced: each rank writes its own
query rows.  The reference has no counterpart (it runs one slide per rank under
DDP, src/sparse_wsi_vit/experiments/trainer.py:100-106).

Layout: sharded K/V/indexer-K are TOKEN-major, (B, T_local, H, D), so that the
gathered tensor (B, T, H, D) is contiguous; the kernels read it through the
strided (B, H, T, D) view.  The last shard may be short; gathered rows past the
true length are padding the kernels never see (they take Tk explicitly).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ShardPlan:
    total: int       # tokens of the slide
    world: int
    rank: int
    per_rank: int    # padded shard length (equal on every rank)
    start: int       # first token owned by this rank
    stop: int        # one past the last token owned (start == stop: empty shard)

    @property
    def local(self) -> int:
        return self.stop - self.start


def plan_shards(total: int, world: int, rank: int, align: int = 8) -> ShardPlan:
    """Contiguous, equal-length (padded to `align`) token shards; only the tail may be short or empty."""
    if total < 1 or world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad shard request total={total} world={world} rank={rank}")
    per = -(-total // world)
    per = -(-per // align) * align
    start = min(rank * per, total)
    stop = min(start + per, total)
    return ShardPlan(total, world, rank, per, start, stop)


def plan_ragged(lengths, world: int, rank: int, align: int = 8):
    """One plan per slide of a ragged batch: every slide is split over all ranks, so the
    all-gathers stay regular and the load stays balanced whatever the slide lengths."""
    return [plan_shards(int(n), world, rank, align) for n in lengths]


def _pad_tokens(x: torch.Tensor, per_rank: int) -> torch.Tensor:
    if x.shape[1] == per_rank:
        return x.contiguous()
    out = x.new_zeros((x.shape[0], per_rank, *x.shape[2:]))
    out[:, :x.shape[1]] = x
    return out


def all_gather_tokens(x_local: torch.Tensor, plan: ShardPlan, group=None, out=None) -> torch.Tensor:
    """(B, T_local, ...) on every rank -> (B, world*per_rank, ...), rows >= plan.total are padding."""
    B = x_local.shape[0]
    xl = _pad_tokens(x_local, plan.per_rank)
    if plan.world == 1:
        return xl
    if B == 1:
        if out is None:
            out = xl.new_empty((1, plan.world * plan.per_rank, *xl.shape[2:]))
        dist.all_gather_into_tensor(out.view(plan.world * plan.per_rank, *xl.shape[2:]), xl[0], group=group)
        return out
    stage = xl.new_empty((plan.world, B, plan.per_rank, *xl.shape[2:]))
    dist.all_gather_into_tensor(stage, xl, group=group)
    return stage.transpose(0, 1).reshape(B, plan.world * plan.per_rank, *xl.shape[2:])


def sharded_dsa_attention(q_loc, k_loc, v_loc, qi_loc, ki_loc, w, top_k, plan: ShardPlan, group=None,
                          out_dtype=None, return_topk=False, compute=None, comm_stream=None):
    """DSA forward for this rank's queries against the whole slide.

    q_loc, k_loc, v_loc: (B, T_local, H, D) token-major; qi_loc, ki_loc: (B, T_local, IH, ID).
    Returns o (B, H, T_local, D) [and idx/valid/scores for the local queries].
    `compute` defaults to the CUDA path; tests on CPU ranks inject a checker.
    """
    if compute is None:
        from .ops import dsa_sparse_attention as compute
    use_side = comm_stream is not None and k_loc.is_cuda and plan.world > 1
    ki_all = all_gather_tokens(ki_loc, plan, group)
    if use_side:
        # Ordering contract: the gathers run on `comm_stream` behind everything already queued on
        # the current stream; the attention waits for `kv_ready` on the current stream.  With batch 1
        # the gathered buffers are allocated HERE, on the current stream: every later reader is
        # ordered on the current stream, the only foreign writer (the gather) finishes before
        # `kv_ready`, so the caching allocator may reuse them like any other block of this stream.
        # (Allocating them under `comm_stream` and marking them as used by the current stream keeps
        # each block out of the pool until the GPU catches up with the host: one device allocation
        # per gather while the host runs ahead, which at 8 ranks costs more than the step.)
        cur = torch.cuda.current_stream(k_loc.device)
        pre = k_loc.shape[0] == 1
        outs = [x.new_empty((1, plan.world * plan.per_rank, *x.shape[2:])) if pre else None for x in (k_loc, v_loc)]
        comm_stream.wait_stream(cur)
        with torch.cuda.stream(comm_stream):
            k_all = all_gather_tokens(k_loc, plan, group, out=outs[0])
            v_all = all_gather_tokens(v_loc, plan, group, out=outs[1])
        kv_ready = comm_stream.record_event()
        if not pre:
            k_all.record_stream(cur)
            v_all.record_stream(cur)
    else:
        k_all = all_gather_tokens(k_loc, plan, group)
        v_all = all_gather_tokens(v_loc, plan, group)
        kv_ready = None
    T = plan.total
    if plan.local == 0:
        # An empty tail shard (a short slide on many ranks) has taken part in every collective
        # above and has no query rows of its own: nothing to launch.
        B, _, H, D = q_loc.shape
        o = q_loc.new_zeros((B, H, 0, D), dtype=out_dtype or q_loc.dtype)
        if kv_ready is not None:
            torch.cuda.current_stream(k_loc.device).wait_event(kv_ready)
        if not return_topk:
            return o
        return (o, torch.zeros((B, 0, top_k), dtype=torch.int32, device=q_loc.device),
                torch.zeros((B, 0, top_k), dtype=torch.float32, device=q_loc.device),
                torch.zeros((B, 0, top_k), dtype=torch.float32, device=q_loc.device))
    q = q_loc.transpose(1, 2)                    # (B, H, T_local, D) view
    k = k_all[:, :T].transpose(1, 2)             # (B, H, T, D) view of the gathered buffer
    v = v_all[:, :T].transpose(1, 2)
    return compute(q, k, v, qi_loc, ki_all[:, :T], w, top_k, out_dtype=out_dtype, return_topk=return_topk,
                   **({"kv_ready": kv_ready} if kv_ready is not None else {}))


def sharded_encoder_forward(encoder, patches_local, plan: ShardPlan, group=None, comm_stream=None, compute=None,
                            coords_local=None):
    """Forward of a ``DSAViTSlideEncoder`` with the token sequence [CLS..., patches...] sharded over
    the ranks of `group` (weights replicated).

    `plan` shards the FULL sequence of ``encoder.num_cls + n_patches`` tokens; `patches_local` holds
    the patch embeddings of this rank's slice, (B, n_local_patches, in_features): rank 0's slice
    starts with the CLS tokens, so it gets ``plan.local - num_cls`` patches, every other rank
    ``plan.local`` (possibly none: a short slide on many ranks leaves empty tail shards, which
    still take part in every collective).  Token-local work (projections, LayerNorm, 2-D RoPE, MLP)
    runs on the shard with no communication; each attention layer all-gathers the indexer keys, K
    and V (``sharded_dsa_attention``).  With `coords_local` ((B, n_local_patches, 2), the (y, x)
    coordinates of this rank's patches) and an encoder built with ``rope_coord_high``, q and k of
    the local patch tokens are rotated before the gather, CLS tokens excepted
    (models/vit_5/models_vit5.py:84-90).  The CLS rows live on rank 0, which computes the logits and
    broadcasts them.  Returns {"logits": (B, out_features)} on every rank, the same dictionary
    ``DSAViTSlideEncoder.forward`` returns (deepseek_sparse_attention.py:267-305).
    """
    from .modules import rope_qk_
    C = encoder.num_cls
    if plan.world > 1 and plan.per_rank < C:
        raise ValueError("the CLS tokens must fit into rank 0's shard")
    if patches_local.dim() == 2:
        patches_local = patches_local.unsqueeze(0)
    B = patches_local.shape[0]
    x = encoder.input_proj(patches_local)
    n_cls_local = C if plan.rank == 0 else 0
    if plan.rank == 0:
        x = torch.cat([encoder.cls_tokens.expand(B, -1, -1).to(x.dtype), x], dim=1)
    Tl = x.shape[1]
    if Tl != plan.local:
        raise ValueError(f"rank {plan.rank} holds {Tl} tokens, the plan says {plan.local}")
    rope = coords_local is not None and getattr(encoder, "rope_coord_high", None) is not None
    for blk in encoder.blocks:
        attn = blk.attn
        H, D = attn.attention_heads, attn.head_dim
        y = blk.norm1(x)
        qkv = attn.qkv_proj(y).view(B, Tl, 3, H, D)
        if rope and Tl > 0:
            rope_qk_(qkv, coords_local, encoder.rope_coord_high, n_cls_local, encoder.rope_theta)
        q_idx, k_idx = attn.indexer_proj(y)
        o = sharded_dsa_attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], q_idx, k_idx, attn.indexer_head_weights,
                                  attn.top_k, plan, group=group, out_dtype=y.dtype, compute=compute,
                                  comm_stream=comm_stream)
        x = x + blk.drop1(attn.out_proj(o.transpose(1, 2).reshape(B, Tl, H * D).to(y.dtype)))
        x = x + blk.mlp(blk.norm2(x))
    logits = torch.empty((B, encoder.out_features), dtype=x.dtype, device=x.device)
    if plan.rank == 0:
        cls = encoder.norm(x[:, :C])
        pooled = (torch.softmax(encoder.cls_pool(cls), dim=1) * cls).sum(dim=1)
        logits = encoder.head(pooled).contiguous()
    if plan.world > 1:
        dist.broadcast(logits, src=0, group=group)
    return {"logits": logits}


def local_patch_range(plan: ShardPlan, num_cls: int):
    """Half-open range of PATCH indices (CLS tokens not counted) held by the rank of `plan`, which
    shards the full sequence [CLS..., patches...]."""
    return max(plan.start - num_cls, 0), max(plan.stop - num_cls, 0)


def sharded_ragged_forward(encoder, slides, world: int, rank: int, coords=None, group=None, comm_stream=None,
                           compute=None, align: int = 128):
    """A ragged batch of slides through a sharded ``DSAViTSlideEncoder``: the slides run back to
    back, each one split over ALL ranks (``plan_ragged``), so every all-gather is regular and the
    load is balanced whatever the slide lengths.  The reference asserts batch size 1
    (experiments/datamodules/h5_datamodule.py:22-24); this lifts it.

    `slides`: list of (n_i, in_features) arrays -- tensors, or anything with ``.shape`` that can be
    sliced by rows and converted with ``torch.as_tensor`` (a lazily read feature bag): a rank
    touches only rows [lo, hi) of each slide, its own shard.  `coords`: matching list of (n_i, 2)
    arrays or None.  Returns {"logits": (n_slides, out_features)} on every rank.
    """
    par = next(encoder.parameters())
    plans = plan_ragged([int(s.shape[0]) + encoder.num_cls for s in slides], world, rank, align)
    rows = []
    for i, plan in enumerate(plans):
        lo, hi = local_patch_range(plan, encoder.num_cls)
        x = torch.as_tensor(slides[i][lo:hi]).to(par.device, non_blocking=True)
        if not torch.is_autocast_enabled():
            x = x.to(par.dtype)
        c = None
        if coords is not None:
            c = torch.as_tensor(coords[i][lo:hi]).to(par.device, non_blocking=True)[None]
        out = sharded_encoder_forward(encoder, x[None], plan, group=group, comm_stream=comm_stream, compute=compute,
                                      coords_local=c)
        rows.append(out["logits"][0])
    return {"logits": torch.stack(rows, dim=0)}
