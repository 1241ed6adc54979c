"""Host-side builders of CSR key-block lists for ``ops.block_sparse_attention``.

Each returns (row_ptr, col_idx) as int32 numpy arrays: the key blocks of query block i are
``col_idx[row_ptr[i]:row_ptr[i+1]]``, ascending and without repeats.
"""
from __future__ import annotations

import numpy as np


def _to_csr(rows):
    row_ptr = np.zeros(len(rows) + 1, dtype=np.int32)
    cols = []
    for i, r in enumerate(rows):
        r = sorted(set(int(c) for c in r))
        cols.extend(r)
        row_ptr[i + 1] = len(cols)
    return row_ptr, np.asarray(cols, dtype=np.int32)


def static_window_blocks(seq_len: int, num_cls: int, window: int, dilation: int, block: int):
    """Blocks touched by the reference's static pattern (static_sparse_attention.py:62-188):
    CLS rows see everything, every row sees the CLS block(s), patch rows see the blocks that
    intersect [i - window*dilation, i + window*dilation]."""
    nb = -(-seq_len // block)
    reach = window * dilation
    cls_blocks = list(range(-(-num_cls // block))) if num_cls > 0 else []
    rows = []
    for qb in range(nb):
        q0, q1 = qb * block, min(seq_len, (qb + 1) * block) - 1
        if q0 < num_cls:
            rows.append(range(nb))
            continue
        lo = max(num_cls, q0 - reach) if window > 0 else None
        r = list(cls_blocks)
        if window > 0:
            hi = min(seq_len - 1, q1 + reach)
            r += list(range(lo // block, hi // block + 1))
        rows.append(r)
    return _to_csr(rows)


def static_window_lists(seq_len: int, num_cls: int, window: int, dilation: int):
    """Explicit key lists of the PATCH rows of the reference's static pattern
    (static_sparse_attention.py:105-188): for patch row i (token num_cls + i) the CLS keys followed
    by the window keys i - W*d ... i + W*d step d, out-of-range neighbours marked invalid (they are
    masked, not wrapped, :159-168).  Returns (idx int32, valid float32), each (1, n_patches, C + 2W + 1)
    with token indices (patch position + num_cls).  With window 0 a patch sees the CLS keys only."""
    n = seq_len - num_cls
    width = num_cls + (2 * window + 1 if window > 0 else 0)
    idx = np.zeros((1, max(n, 0), max(width, 1)), dtype=np.int32)
    valid = np.zeros((1, max(n, 0), max(width, 1)), dtype=np.float32)
    if n <= 0:
        return idx, valid
    if num_cls > 0:
        idx[0, :, :num_cls] = np.arange(num_cls, dtype=np.int32)[None, :]
        valid[0, :, :num_cls] = 1.0
    if window > 0:
        pos = np.arange(n)[:, None] + (np.arange(-window, window + 1) * dilation)[None, :]
        ok = (pos >= 0) & (pos < n)
        idx[0, :, num_cls:] = np.where(ok, pos + num_cls, 0).astype(np.int32)
        valid[0, :, num_cls:] = ok.astype(np.float32)
    return idx, valid


def chebyshev_grid_blocks(grid_h: int, grid_w: int, radius: int = 1, global_blocks=()):
    """2-D pattern: the tokens of one block are one spatial tile; block (r, c) has index r*grid_w + c.
    Every block attends the blocks within Chebyshev distance `radius` plus the `global_blocks`
    (e.g. a trailing block holding the CLS tokens); global blocks attend everything."""
    n = grid_h * grid_w
    extra = [int(g) for g in global_blocks]
    total = max([n] + [g + 1 for g in extra])
    rows = []
    for b in range(total):
        if b in extra:
            rows.append(range(total))
            continue
        r, c = divmod(b, grid_w)
        nbrs = [rr * grid_w + cc for rr in range(max(0, r - radius), min(grid_h, r + radius + 1))
                for cc in range(max(0, c - radius), min(grid_w, c + radius + 1))] if b < n else []
        rows.append(nbrs + extra)
    return _to_csr(rows)


def band_random_blocks(n_blocks: int, band: int = 2, n_global: int = 1, p: float = 0.05, seed: int = 0):
    """Sweep pattern: local band of +-`band` blocks, the first `n_global` blocks, and extra key blocks
    drawn Bernoulli(p) per (query block, key block), seeded."""
    rng = np.random.default_rng(seed)
    rows = []
    for qb in range(n_blocks):
        r = set(range(max(0, qb - band), min(n_blocks, qb + band + 1))) | set(range(min(n_global, n_blocks)))
        if p > 0:
            r |= set(np.nonzero(rng.random(n_blocks) < p)[0].tolist())
        rows.append(r)
    return _to_csr(rows)
