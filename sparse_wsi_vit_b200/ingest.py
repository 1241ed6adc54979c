"""Feature-bag ingestion into the sequence-sharded layout.

The reference reads one whole slide per step into host memory and asserts batch size 1
(src/sparse_wsi_vit/datasets/h5_slidedataset/h5_dataset.py:102-155,
src/sparse_wsi_vit/experiments/datamodules/h5_datamodule.py:9-30).  Here a rank reads only the
rows of ITS shard of every slide, through pinned host memory, while the previous slide computes,
and a batch may hold slides of any lengths (each is split over all ranks).

On-disk layouts handled (the two the reference's extractors write, h5_dataset.py:118-136):
  flat        features (N, F), coords (N, 2)
  block-major features (n_blocks, 64, F), coords (n_blocks, 64, 2)  -- 8 x 8 spatial tiles
              (scripts/virchow_preprocess.py:183-224), flattened to N = 64 * n_blocks rows, optionally
              mean-pooled inside each tile by `downscale_block` in {2, 4, 8} (h5_dataset.py:123-131).
A bag wraps any array-like with ``.shape`` and row slicing: an ``h5py.Dataset`` (read lazily, only
the touched blocks), a ``numpy.memmap`` / ``ndarray``, or a tensor.  ``h5py`` is imported only by
``FeatureBag.from_h5``.
"""
from __future__ import annotations

import numpy as np
import torch

from .dist import local_patch_range, plan_ragged, sharded_encoder_forward


class _Rows:
    """Row-sliceable view (N, width) over a flat (N, width) or block-major (n_blocks, 64, width) array."""

    def __init__(self, arr, downscale_block: int = 1, is_coords: bool = False):
        if downscale_block not in (1, 2, 4, 8):
            raise ValueError("downscale_block must be 1, 2, 4 or 8")
        if downscale_block > 1 and len(arr.shape) != 3:
            raise ValueError("downscaling needs the block-major layout (n_blocks, 64, width)")
        if len(arr.shape) == 3 and arr.shape[1] != 64:
            raise ValueError("block-major arrays hold 64 tokens (an 8 x 8 tile) per block")
        self.arr, self.ds, self.is_coords = arr, downscale_block, is_coords
        self.per_block = (8 // downscale_block) ** 2 if len(arr.shape) == 3 else 1
        n = arr.shape[0] * self.per_block if len(arr.shape) == 3 else arr.shape[0]
        self.shape = (n, arr.shape[-1])

    def __len__(self):
        return self.shape[0]

    def __getitem__(self, sl):
        if not isinstance(sl, slice) or sl.step not in (None, 1):
            raise TypeError("feature bags are read by contiguous row ranges")
        lo, hi, _ = sl.indices(self.shape[0])
        hi = max(hi, lo)
        if len(self.arr.shape) == 2:
            return np.asarray(self.arr[lo:hi])
        b0, b1 = lo // self.per_block, -(-hi // self.per_block)
        blk = np.asarray(self.arr[b0:b1])                                  # only the touched tiles are read
        if self.ds > 1:
            nb, width = blk.shape[0], blk.shape[-1]
            c, s = 8 // self.ds, self.ds
            blk = blk.reshape(nb, c, s, c, s, width)
            # features: mean over each s x s sub-tile; coordinates: its top-left patch (h5_dataset.py:126-131)
            blk = blk[:, :, 0, :, 0, :] if self.is_coords else blk.mean((2, 4))
            blk = blk.reshape(nb, c * c, width)
        flat = blk.reshape(-1, blk.shape[-1])
        return flat[lo - b0 * self.per_block: hi - b0 * self.per_block]


class FeatureBag:
    """One slide: ``features`` (N, F) and ``coords`` (N, 2), both read by row ranges."""

    def __init__(self, features, coords, downscale_block: int = 1, name: str = ""):
        self.features = _Rows(features, downscale_block, is_coords=False)
        self.coords = _Rows(coords, downscale_block, is_coords=True)
        if self.features.shape[0] != self.coords.shape[0]:
            raise ValueError("features and coords disagree on the number of patches")
        self.name = name
        self._file = None

    @classmethod
    def from_h5(cls, path, features_name: str = "features", coords_name: str = "coords", downscale_block: int = 1):
        """Opens ``path`` with h5py and keeps it open; rows are read on demand."""
        try:
            import h5py
        except ImportError as e:                                            # pragma: no cover
            raise ImportError("FeatureBag.from_h5 needs h5py; use FeatureBag(...) on arrays otherwise") from e
        f = h5py.File(path, "r")
        bag = cls(f[features_name], f[coords_name], downscale_block, name=str(path))
        bag._file = f
        return bag

    def close(self):
        if self._file is not None:
            self._file.close()
            self._file = None

    def __len__(self):
        return self.features.shape[0]


class ShardStreamer:
    """Double-buffered pinned staging of one rank's shards: ``fetch(i)`` starts reading slide i's local
    rows into pinned memory and copying them to the device on a side stream; ``get(i)`` returns the
    device tensors once the copy is ordered before the current stream.  While slide i computes, slide
    i + 1 is on its way."""

    def __init__(self, bags, plans, num_cls, device, dtype=torch.float32):
        self.bags, self.plans, self.num_cls = bags, plans, num_cls
        self.device, self.dtype = torch.device(device), dtype
        self.cuda = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.pending = {}

    def fetch(self, i):
        if i >= len(self.bags) or i in self.pending:
            return
        lo, hi = local_patch_range(self.plans[i], self.num_cls)
        x = torch.from_numpy(np.ascontiguousarray(self.bags[i].features[lo:hi])).to(self.dtype)
        c = torch.from_numpy(np.ascontiguousarray(self.bags[i].coords[lo:hi])).float()
        if not self.cuda:
            self.pending[i] = (x, c, None)
            return
        x, c = x.pin_memory(), c.pin_memory()
        with torch.cuda.stream(self.stream):
            xd = x.to(self.device, non_blocking=True)
            cd = c.to(self.device, non_blocking=True)
            ev = self.stream.record_event()
        self.pending[i] = (xd, cd, (ev, x, c))                              # the pinned sources live until get()

    def get(self, i):
        self.fetch(i)
        xd, cd, aux = self.pending.pop(i)
        if aux is not None:
            cur = torch.cuda.current_stream(self.device)
            cur.wait_event(aux[0])
            xd.record_stream(cur)
            cd.record_stream(cur)
        return xd, cd


def stream_ragged_batch(encoder, bags, world: int, rank: int, group=None, comm_stream=None, compute=None,
                        align: int = 128, use_coords=None, dtype=torch.float32):
    """Forward of a ragged batch of ``FeatureBag``s through a sharded ``DSAViTSlideEncoder``: each rank
    reads, pins and uploads only its own rows of every slide, one slide ahead of the compute.
    Returns {"logits": (n_slides, out_features)} on every rank."""
    par = next(encoder.parameters())
    plans = plan_ragged([len(b) + encoder.num_cls for b in bags], world, rank, align)
    if use_coords is None:
        use_coords = getattr(encoder, "rope_coord_high", None) is not None
    streamer = ShardStreamer(bags, plans, encoder.num_cls, par.device, dtype)
    streamer.fetch(0)
    rows = []
    for i, plan in enumerate(plans):
        x, c = streamer.get(i)
        streamer.fetch(i + 1)
        out = sharded_encoder_forward(encoder, x[None], plan, group=group, comm_stream=comm_stream, compute=compute,
                                      coords_local=c[None] if use_coords else None)
        rows.append(out["logits"][0])
    return {"logits": torch.stack(rows, dim=0)}


def ragged_collate(batch):
    """Collate function for ``torch.utils.data.DataLoader`` that lifts the reference's batch-size-1
    assertion (experiments/datamodules/h5_datamodule.py:22-24): variable-length bags stay a list.
    Keeps the reference's keys; a single-slide batch is stacked exactly as the reference does."""
    if len(batch) == 1:
        b = batch[0]
        return b | {"input": b["input"][None], "label": b["label"][None], "coords": b["coords"][None]}
    out = {"input": [b["input"] for b in batch], "coords": [b["coords"] for b in batch],
           "label": torch.stack([torch.as_tensor(b["label"]) for b in batch]),
           "slide_name": [b.get("slide_name", "") for b in batch]}
    if "class_weight" in batch[0]:
        out["class_weight"] = torch.as_tensor([b["class_weight"] for b in batch])
    return out
