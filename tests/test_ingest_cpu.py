"""Feature-bag ingestion (no GPU): row-range reads of both on-disk layouts equal the reference's
whole-slide load (restated here from h5_dataset.py:118-136), only the touched tiles are read, and
a ragged batch streamed shard by shard equals the same slides passed whole."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sparse_wsi_vit_b200.ingest import FeatureBag, ragged_collate, stream_ragged_batch


def _reference_load(features, coords, flatten_block=True, downscale_block=1):
    """What H5FeatureBagDataset.__getitem__ does to the arrays it read (h5_dataset.py:123-139)."""
    width = features.shape[-1]
    if downscale_block > 1:
        n_blocks = features.shape[0]
        bcount, bsize = 8 // downscale_block, downscale_block
        features = features.reshape(n_blocks, bcount, bsize, bcount, bsize, width).mean((2, 4))
        features = features.reshape(n_blocks, bcount * bcount, width)
        coords = coords.reshape(n_blocks, bcount, bsize, bcount, bsize, 2)[:, :, 0, :, 0, :]
    if flatten_block and features.ndim == 3:
        features, coords = features.reshape(-1, width), coords.reshape(-1, 2)
    return features.astype(np.float32), coords.astype(np.float32)


class _Counting:
    """ndarray wrapper that records which leading-index ranges were read (stands in for an h5py dataset)."""

    def __init__(self, a):
        self.a, self.shape, self.reads = a, a.shape, []

    def __getitem__(self, sl):
        self.reads.append((sl.start, sl.stop))
        return self.a[sl]


@pytest.mark.parametrize("downscale", [1, 2, 4, 8])
def test_block_major_row_ranges_equal_whole_load(downscale):
    r = np.random.RandomState(downscale)
    feats = r.randn(7, 64, 12).astype(np.float16)
    coords = (r.randint(0, 50, (7, 64, 2)) * 224).astype(np.int32)
    ref_f, ref_c = _reference_load(feats, coords, downscale_block=downscale)
    counted = _Counting(feats)
    bag = FeatureBag(counted, coords, downscale_block=downscale)
    assert len(bag) == ref_f.shape[0]
    per = (8 // downscale) ** 2
    for lo, hi in [(0, len(bag)), (3, 5), (per - 1, per + 2), (len(bag) - 3, len(bag)), (10, 10)]:
        counted.reads.clear()
        got = bag.features[lo:hi]
        np.testing.assert_allclose(got.astype(np.float32), ref_f[lo:hi], rtol=1e-3, atol=1e-3)
        np.testing.assert_array_equal(bag.coords[lo:hi].astype(np.float32), ref_c[lo:hi])
        if hi > lo:
            assert counted.reads == [(lo // per, -(-hi // per))]          # only the touched tiles


def test_flat_layout_and_collate():
    feats = np.arange(40, dtype=np.float32).reshape(10, 4)
    coords = np.arange(20, dtype=np.int32).reshape(10, 2)
    bag = FeatureBag(feats, coords)
    np.testing.assert_array_equal(bag.features[2:7], feats[2:7])
    with pytest.raises(TypeError):
        bag.features[::2]
    items = [{"input": torch.zeros(5, 4), "coords": torch.zeros(5, 2), "label": torch.tensor(1), "slide_name": "a"},
             {"input": torch.zeros(9, 4), "coords": torch.zeros(9, 2), "label": torch.tensor(0), "slide_name": "b"}]
    one = ragged_collate(items[:1])
    assert one["input"].shape == (1, 5, 4) and one["label"].shape == (1,)
    two = ragged_collate(items)
    assert [t.shape[0] for t in two["input"]] == [5, 9] and two["label"].tolist() == [1, 0]


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


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sparse_wsi_vit_b200 as swv
        from sparse_wsi_vit_b200.dist import sharded_ragged_forward
        torch.manual_seed(0)
        enc = swv.DSAViTSlideEncoder(in_features=12, out_features=2, embed_dim=32, num_heads=2, num_layers=1,
                                     num_cls=1, indexer_heads=2, indexer_dim=16, top_k=8).eval()
        r = np.random.RandomState(7)
        raw = [(r.randn(3, 64, 12).astype(np.float32), r.rand(3, 64, 2).astype(np.float32)),
               (r.randn(70, 12).astype(np.float32), r.rand(70, 2).astype(np.float32))]
        bags = [FeatureBag(f, c) for f, c in raw]
        whole = [torch.from_numpy(_reference_load(f, c)[0]) for f, c in raw]
        with torch.no_grad():
            got = stream_ragged_batch(enc, bags, world, rank, compute=_oracle_compute, align=8)["logits"]
            ref = sharded_ragged_forward(enc, whole, 1, 0, compute=_oracle_compute, align=8)["logits"]
        assert torch.allclose(got, ref, atol=1e-5), (got, ref)
        out[rank] = True
    finally:
        dist.destroy_process_group()


def test_streamed_ragged_batch_equals_whole_slides():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert all(out.get(r, False) for r in range(2))
