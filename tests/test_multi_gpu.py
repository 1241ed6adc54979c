"""Sequence-sharded forward on real GPUs (NCCL, one process per GPU).  Needs >= 2 GPUs; skipped
otherwise.  Each rank checks its slice of the sharded result against the unsharded result
computed on its own GPU: attention outputs bit for bit (query rows are independent given the
gathered keys), the index sets exactly, the encoder logits to bf16/fp32 round-off."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import sparse_wsi_vit_b200 as swv
        from sparse_wsi_vit_b200.dist import plan_shards, sharded_dsa_attention, sharded_encoder_forward
        g = torch.Generator().manual_seed(0)
        T, H, D, IH, ID, K = 3000, 4, 64, 4, 64, 256
        mk = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).to(torch.bfloat16).to(dev)
        q, k, v = mk(1, T, H, D, sc=0.125), mk(1, T, H, D), mk(1, T, H, D)
        qi, ki = mk(1, T, IH, ID, sc=0.125), mk(1, T, IH, ID, sc=0.125)
        w = torch.randn(IH, generator=g).to(dev)
        plan = plan_shards(T, world, rank, align=128)
        sl = slice(plan.start, plan.stop)
        comm = torch.cuda.Stream(dev)
        o, idx, valid, sc = sharded_dsa_attention(q[:, sl], k[:, sl], v[:, sl], qi[:, sl], ki[:, sl], w, K, plan,
                                                  out_dtype=torch.float32, return_topk=True, comm_stream=comm)
        ref_o, ref_idx, _, ref_sc = swv.dsa_sparse_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                             qi, ki, w, K, out_dtype=torch.float32, return_topk=True)
        swv.check_status(dev)
        assert torch.equal(idx, ref_idx[:, sl]) and torch.equal(sc, ref_sc[:, sl])
        assert torch.equal(o, ref_o[:, :, sl])

        torch.manual_seed(1)
        enc = swv.DSAViTSlideEncoder(in_features=96, out_features=2, embed_dim=128, num_heads=2, num_layers=2,
                                     num_cls=2, indexer_heads=4, indexer_dim=32, top_k=64).to(dev).eval()
        x = torch.randn(1, 1500, 96, generator=torch.Generator().manual_seed(2)).to(dev)
        Tt = 1500 + enc.num_cls
        eplan = plan_shards(Tt, world, rank, align=8)
        lo, hi = max(eplan.start - enc.num_cls, 0), eplan.stop - enc.num_cls
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            got = sharded_encoder_forward(enc, x[:, lo:hi], eplan, comm_stream=comm)["logits"]
            whole = enc(x)["logits"]
        swv.check_status(dev)
        assert torch.allclose(got.float(), whole.float(), atol=2e-2), (got, whole)

        # ragged batch with 2-D RoPE: every slide split over both ranks == the same slides on one GPU;
        # the 5-patch slide leaves rank 1 an empty shard, which still joins every collective
        from sparse_wsi_vit_b200.dist import sharded_ragged_forward
        torch.manual_seed(2)
        renc = swv.DSAViTSlideEncoder(in_features=96, out_features=2, embed_dim=128, num_heads=2, num_layers=2,
                                      num_cls=2, indexer_heads=4, indexer_dim=32, top_k=64,
                                      rope_coord_high=224.0 * 64).to(dev).eval()
        gg = torch.Generator().manual_seed(3)
        slides = [torch.randn(n, 96, generator=gg).to(dev) for n in (900, 5, 1300)]
        coords = [(torch.randint(0, 64, (s_.shape[0], 2), generator=gg) * 224).float().to(dev) for s_ in slides]
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            sharded = sharded_ragged_forward(renc, slides, world, rank, coords=coords, comm_stream=comm)["logits"]
            single = sharded_ragged_forward(renc, slides, 1, 0, coords=coords)["logits"]
        swv.check_status(dev)
        assert sharded.shape == (3, 2)
        assert torch.allclose(sharded.float(), single.float(), atol=2e-2), (sharded, single)
        out[rank] = True
    finally:
        dist.destroy_process_group()


def test_sharded_matches_single_gpu():
    world = torch.cuda.device_count()
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert all(out.get(r, False) for r in range(world))
