"""Host-side block-list builders against the oracle's token masks (no GPU)."""
import numpy as np
import torch

from oracle import static_attn as S
from sparse_wsi_vit_b200 import patterns


def test_static_window_blocks_cover_the_token_pattern():
    for L, C, W, d, block in [(300, 2, 3, 2, 128), (1000, 1, 40, 3, 128), (260, 3, 0, 1, 64), (64, 1, 5, 1, 64),
                              (500, 0, 2, 1, 128)]:
        rp, ci = patterns.static_window_blocks(L, C, W, d, block)
        token = S.static_window_mask(L, C, W, d)
        blocks = S.expand_block_mask(rp, ci, block, L, L)
        assert not bool((token & ~blocks).any()), (L, C, W, d)
        assert rp[0] == 0 and rp[-1] == len(ci) and np.all(np.diff(rp) >= 0)
        for i in range(len(rp) - 1):
            row = ci[rp[i]:rp[i + 1]]
            assert np.all(np.diff(row) > 0)


def test_chebyshev_grid_blocks():
    rp, ci = patterns.chebyshev_grid_blocks(8, 8, 1, global_blocks=[64])
    assert len(rp) == 66
    corner = ci[rp[0]:rp[1]].tolist()
    assert corner == [0, 1, 8, 9, 64]
    centre = ci[rp[27]:rp[28]].tolist()
    assert centre == [18, 19, 20, 26, 27, 28, 34, 35, 36, 64]
    assert ci[rp[64]:rp[65]].tolist() == list(range(65))


def test_band_random_blocks_are_seeded_and_contain_band_and_global():
    a = patterns.band_random_blocks(64, 2, 1, 0.05, seed=3)
    b = patterns.band_random_blocks(64, 2, 1, 0.05, seed=3)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    rp, ci = a
    for qb in range(64):
        row = set(ci[rp[qb]:rp[qb + 1]].tolist())
        assert 0 in row and all(x in row for x in range(max(0, qb - 2), min(64, qb + 3)))
    dense = S.expand_block_mask(rp, ci, 4, 256, 256)
    assert 0.08 < float(dense.float().mean()) < 0.2


def test_static_window_lists_equal_the_reference_mask():
    """The explicit per-row key lists (used for fp32 activations) name exactly the keys the
    reference's static pattern lets every patch row see."""
    from sparse_wsi_vit_b200.patterns import static_window_lists
    for (L, C, W, d) in [(37, 2, 3, 2), (20, 1, 0, 1), (50, 3, 5, 1), (9, 0, 2, 1), (12, 2, 4, 3)]:
        idx, val = static_window_lists(L, C, W, d)
        mask = S.static_window_mask(L, C, W, d)
        got = torch.zeros(L - C, L, dtype=torch.bool)
        for i in range(L - C):
            keys = idx[0, i][val[0, i] > 0]
            assert len(set(keys.tolist())) == len(keys)          # no key listed twice
            got[i, torch.from_numpy(keys).long()] = True
        assert torch.equal(got, mask[C:]), (L, C, W, d)
