"""Helpers shared by the GPU parity tests."""
import torch

from oracle import dsa as O


def make_dsa_inputs(T, H, D, IH, ID, seed, dtype=torch.float32, B=1, device="cpu", w_mode="randn"):
    """Seeded inputs with the value distributions of the DSA benchmark configuration:
    q, k, v ~ N(0,1) with q pre-scaled by 1/sqrt(D); indexer q/k ~ N(0, 1/ID); W ~ N(0,1)."""
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, T, D, generator=g) / D ** 0.5).to(dtype)
    k = torch.randn(B, H, T, D, generator=g).to(dtype)
    v = torch.randn(B, H, T, D, generator=g).to(dtype)
    qi = (torch.randn(B, T, IH, ID, generator=g) / ID ** 0.5).to(dtype)
    ki = (torch.randn(B, T, IH, ID, generator=g) / ID ** 0.5).to(dtype)
    w = torch.randn(IH, generator=g)
    if w_mode == "abs":
        w = w.abs()
    return tuple(t.to(device) for t in (q, k, v, qi, ki, w))


def own_scores(qi, ki, w):
    """The library's own score matrix: asking for top_k == Tk returns every key, ascending."""
    import sparse_wsi_vit_b200 as swv
    Tk = ki.shape[1]
    idx, valid, scores = swv.dsa_indexer_topk(qi, ki, w, Tk)
    assert bool((valid == 1).all())
    ar = torch.arange(Tk, device=idx.device, dtype=torch.int32)
    assert bool((idx == ar).all())
    return scores


def sets_equal(idx_a, idx_b):
    return torch.equal(torch.sort(idx_a.long(), dim=-1).values, torch.sort(idx_b.long(), dim=-1).values)


def overlap_fraction(idx_a, idx_b, n_keys):
    """Mean |A & B| / |A| over rows, idx (R, K) with distinct entries per row."""
    R, K = idx_a.shape
    ma = torch.zeros(R, n_keys, dtype=torch.bool)
    mb = torch.zeros(R, n_keys, dtype=torch.bool)
    ma.scatter_(1, idx_a.long().cpu(), True)
    mb.scatter_(1, idx_b.long().cpu(), True)
    return float((ma & mb).sum()) / float(ma.sum())
