"""Sequence-sharding bookkeeping on CPU ranks (gloo, world_size 2 and 3): the shard planner, the
token all-gather with a short last shard, and the sharded forward assembled from per-rank
results equals the single-process result.  The compute step is injected (the CPU oracle), the
communication and layout code under test is the product's."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sparse_wsi_vit_b200.dist import all_gather_tokens, plan_ragged, plan_shards, sharded_dsa_attention


def test_plan_shards_cover_everything_once():
    for total in (1, 7, 128, 1000, 65536, 24001):
        for world in (1, 2, 3, 8):
            plans = [plan_shards(total, world, r) for r in range(world)]
            assert all(p.per_rank == plans[0].per_rank and p.per_rank % 8 == 0 for p in plans)
            covered = []
            for p in plans:
                covered += list(range(p.start, p.stop))
            assert covered == list(range(total))
            assert plans[0].per_rank * world >= total
    with pytest.raises(ValueError):
        plan_shards(0, 2, 0)
    with pytest.raises(ValueError):
        plan_shards(10, 2, 2)
    pl = plan_ragged([24000, 56000, 96000, 131000], 8, 3, align=128)
    assert [p.total for p in pl] == [24000, 56000, 96000, 131000] and all(p.local > 0 for p in pl)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _oracle_compute(q, k, v, qi, ki, w, top_k, out_dtype=None, return_topk=False, **_):
    from oracle import dsa as O
    o, idx, valid, sc = O.dsa_forward(q[0], k[0], v[0], qi[0], ki[0], w, top_k)
    return (o[None], idx[None], valid[None], sc[None]) if return_topk else o[None]


def _worker(rank, world, port, T, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        H, D, IH, ID, K = 2, 16, 2, 16, 8
        q = torch.randn(1, T, H, D, generator=g)
        k = torch.randn(1, T, H, D, generator=g)
        v = torch.randn(1, T, H, D, generator=g)
        qi = torch.randn(1, T, IH, ID, generator=g)
        ki = torch.randn(1, T, IH, ID, generator=g)
        w = torch.randn(IH, generator=g)
        plan = plan_shards(T, world, rank)
        sl = slice(plan.start, plan.stop)
        # gather alone: rows >= T of the gathered tensor are padding, the rest is the original
        full = all_gather_tokens(k[:, sl], plan)
        assert full.shape[1] == world * plan.per_rank
        assert torch.equal(full[:, :T], k)
        o, idx, valid, sc = sharded_dsa_attention(q[:, sl], k[:, sl], v[:, sl], qi[:, sl], ki[:, sl], w, K, plan,
                                                  return_topk=True, compute=_oracle_compute)
        ref_o, ref_idx, _, _ = _oracle_compute(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), qi, ki, w, K,
                                               return_topk=True)
        assert o.shape[2] == plan.local
        assert torch.allclose(o, ref_o[:, :, sl], atol=1e-6)
        assert torch.equal(idx, ref_idx[:, sl])
        out[rank] = True
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,T", [(2, 100), (3, 50), (2, 17)])
def test_sharded_forward_equals_single_process(world, T):
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, T, out), nprocs=world, join=True)
    assert all(out.get(r, False) for r in range(world))


def _encoder_worker(rank, world, port, n_patches, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sparse_wsi_vit_b200 as swv
        from sparse_wsi_vit_b200.dist import sharded_encoder_forward
        torch.manual_seed(0)
        enc = swv.DSAViTSlideEncoder(in_features=24, out_features=3, embed_dim=32, num_heads=2, num_layers=2,
                                     num_cls=2, indexer_heads=2, indexer_dim=16, top_k=8).eval()
        x = torch.randn(1, n_patches, 24, generator=torch.Generator().manual_seed(1))
        T = n_patches + enc.num_cls
        plan = plan_shards(T, world, rank)
        lo, hi = max(plan.start - enc.num_cls, 0), plan.stop - enc.num_cls
        with torch.no_grad():
            got = sharded_encoder_forward(enc, x[:, lo:hi], plan, compute=_oracle_compute)["logits"]
            whole = sharded_encoder_forward(enc, x, plan_shards(T, 1, 0), compute=_oracle_compute)["logits"]
        assert torch.allclose(got, whole, atol=1e-5), (got, whole)
        out[rank] = True
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n_patches", [(2, 61), (3, 40)])
def test_sharded_encoder_equals_unsharded(world, n_patches):
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_encoder_worker, args=(world, port, n_patches, out), nprocs=world, join=True)
    assert all(out.get(r, False) for r in range(world))


def test_batched_gather_layout():
    """B > 1 goes through the staged gather; with world == 1 it must be the identity + padding."""
    x = torch.arange(2 * 5 * 3, dtype=torch.float32).view(2, 5, 3)
    plan = plan_shards(5, 1, 0)
    y = all_gather_tokens(x, plan)
    assert y.shape == (2, 8, 3) and torch.equal(y[:, :5], x) and float(y[:, 5:].abs().sum()) == 0.0


def _empty_shard_worker(rank, world, port, out):
    """A short slide on many ranks: with T = 10 and shards padded to 8 tokens, ranks 2 and 3 own
    nothing.  They must still take part in every collective and return empty results."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sparse_wsi_vit_b200 as swv
        from sparse_wsi_vit_b200.dist import sharded_encoder_forward
        g = torch.Generator().manual_seed(0)
        T, H, D, IH, ID, K = 10, 2, 16, 2, 16, 4
        q, k, v = (torch.randn(1, T, H, D, generator=g) for _ in range(3))
        qi, ki = (torch.randn(1, T, IH, ID, generator=g) for _ in range(2))
        w = torch.randn(IH, generator=g)
        plan = plan_shards(T, world, rank, align=8)
        assert plan.local == (8, 2, 0, 0)[rank]
        sl = slice(plan.start, plan.stop)
        o, idx, valid, sc = sharded_dsa_attention(q[:, sl], k[:, sl], v[:, sl], qi[:, sl], ki[:, sl], w, K, plan,
                                                  return_topk=True, compute=_oracle_compute)
        ref_o, ref_idx, _, _ = _oracle_compute(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), qi, ki, w, K,
                                               return_topk=True)
        assert o.shape == (1, H, plan.local, D) and idx.shape == (1, plan.local, K)
        assert torch.allclose(o, ref_o[:, :, sl], atol=1e-6) and torch.equal(idx, ref_idx[:, sl])

        torch.manual_seed(0)
        enc = swv.DSAViTSlideEncoder(in_features=24, out_features=3, embed_dim=32, num_heads=2, num_layers=2,
                                     num_cls=2, indexer_heads=2, indexer_dim=16, top_k=4).eval()
        x = torch.randn(1, 8, 24, generator=torch.Generator().manual_seed(1))       # 8 patches + 2 CLS = 10 tokens
        eplan = plan_shards(10, world, rank, align=8)
        lo, hi = max(eplan.start - 2, 0), max(eplan.stop - 2, 0)
        with torch.no_grad():
            got = sharded_encoder_forward(enc, x[:, lo:hi], eplan, compute=_oracle_compute)["logits"]
            whole = sharded_encoder_forward(enc, x, plan_shards(10, 1, 0), compute=_oracle_compute)["logits"]
        assert torch.allclose(got, whole, atol=1e-5), (got, whole)
        out[rank] = True
    finally:
        dist.destroy_process_group()


def test_empty_tail_shards_join_every_collective():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_empty_shard_worker, args=(4, _free_port(), out), nprocs=4, join=True)
    assert all(out.get(r, False) for r in range(4))


def _ragged_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sparse_wsi_vit_b200 as swv
        from sparse_wsi_vit_b200.dist import sharded_ragged_forward
        torch.manual_seed(0)
        enc = swv.DSAViTSlideEncoder(in_features=24, out_features=2, embed_dim=32, num_heads=2, num_layers=1,
                                     num_cls=1, indexer_heads=2, indexer_dim=16, top_k=8).eval()
        g = torch.Generator().manual_seed(5)
        slides = [torch.randn(n, 24, generator=g) for n in (37, 5, 64)]       # 5 patches: an empty shard on rank 1
        with torch.no_grad():
            got = sharded_ragged_forward(enc, slides, world, rank, compute=_oracle_compute, align=8)["logits"]
            one = sharded_ragged_forward(enc, slides, 1, 0, compute=_oracle_compute, align=8)["logits"]
        assert got.shape == (3, 2) and torch.allclose(got, one, atol=1e-5), (got, one)
        out[rank] = True
    finally:
        dist.destroy_process_group()


def test_ragged_batch_equals_slide_by_slide():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_ragged_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert all(out.get(r, False) for r in range(2))
