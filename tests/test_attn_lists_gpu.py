"""GPU parity tests of the list-driven attention kernel (dense tensor-core tiles, sparse softmax over
per-tile member lists): against the exact fp32 list kernel on the same key lists, and the cases in
which it hands tiles over to the dense sweep."""
import pytest
import torch

from oracle import dsa as O
from tests.util import make_dsa_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def swv():
    import sparse_wsi_vit_b200 as m
    return m


def _dev():
    return torch.device("cuda:0")


def _lists_vs_gather(swv, q, k, v, qi, ki, w, K, out_dtype=torch.float32):
    """Both kernels on the key lists of the library's own indexer; returns (lists output, exact output)."""
    from sparse_wsi_vit_b200.ops import dsa_attention_lists
    idx, valid, scores, sel = swv.dsa_indexer_topk(qi, ki, w, K, want_mask=True)
    B, H, Tq, D = q.shape
    o = torch.empty((B, H, Tq, D), dtype=out_dtype, device=q.device)
    dsa_attention_lists(q, k, v, idx, scores, sel, o)
    ref = torch.empty((B, H, Tq, D), dtype=torch.float32, device=q.device)
    swv.dsa_attention_gather(q, k, v, idx, valid, scores * valid, ref)
    swv.check_status(q.device)
    return o.float(), ref


def _close(o, ref):
    # the tolerance of the bf16 tensor-core paths: 2e-2 max-abs, 1e-3 mean-abs
    d = (o - ref).abs()
    assert torch.isfinite(o).all()
    assert float(d.max()) < 2e-2, float(d.max())
    assert float(d.mean()) < 1e-3, float(d.mean())


@pytest.mark.parametrize("B,T,H,K", [(1, 256, 2, 64), (1, 1000, 3, 128), (2, 512, 2, 64), (1, 96, 1, 128),
                                     (1, 4096, 2, 256), (1, 2500, 5, 64), (1, 130, 2, 4)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_lists_kernel_vs_exact_list_kernel(swv, B, T, H, K, out_dtype):
    """Ragged token counts, odd head counts, batches, T < top_k (every key selected), sparse and dense tiles."""
    q, k, v, qi, ki, w = make_dsa_inputs(T, H, 64, 4, 64, seed=T + 7 * K + H, dtype=torch.bfloat16, B=B, device=_dev())
    o, ref = _lists_vs_gather(swv, q, k, v, qi, ki, w, K, out_dtype)
    _close(o, ref)


def test_lists_kernel_vs_oracle(swv):
    T, H, K = 600, 2, 64
    q, k, v, qi, ki, w = make_dsa_inputs(T, H, 64, 4, 64, seed=5, dtype=torch.bfloat16, device=_dev())
    from sparse_wsi_vit_b200.ops import dsa_attention_lists
    idx, valid, scores, sel = swv.dsa_indexer_topk(qi, ki, w, K, want_mask=True)
    o = torch.empty((1, H, T, 64), dtype=torch.float32, device=_dev())
    dsa_attention_lists(q, k, v, idx, scores, sel, o)
    swv.check_status(_dev())
    ref = O.dsa_attention(q[0].float().cpu(), k[0].float().cpu(), v[0].float().cpu(), idx[0].cpu().long(),
                          valid[0].cpu(), (scores * valid)[0].cpu())
    _close(o[0].cpu(), ref)


def test_lists_kernel_short_query_range_splits_the_keys(swv):
    """One rank's share of a sharded slide: few query tiles against a long key range, several CTAs per
    (query tile, head pair) with a merge of their partial rows."""
    Tq, Tk, H, K = 384, 16384, 3, 512
    q, k, v, qi, ki, w = make_dsa_inputs(Tk, H, 64, 4, 64, seed=31, dtype=torch.bfloat16, device=_dev())
    o, ref = _lists_vs_gather(swv, q[:, :, :Tq].contiguous(), k, v, qi[:, :Tq].contiguous(), ki, w, K)
    _close(o, ref)


def test_lists_kernel_cut_ties(swv):
    """Keys that exist three times with K chosen so that every row's threshold falls inside a group: the
    lists say which of the tied keys are in."""
    T, H, K = 3072, 2, 304
    q, k, v, qi, ki, w = make_dsa_inputs(T, H, 64, 4, 64, seed=77, dtype=torch.bfloat16, device=_dev())
    ki[:, 1::3] = ki[:, 0::3]
    ki[:, 2::3] = ki[:, 0::3]
    o, ref = _lists_vs_gather(swv, q, k, v, qi, ki, w, K)
    _close(o, ref)


def test_large_logits_go_to_the_dense_sweep(swv):
    """Rows whose logits cannot be bounded below 2^40 are left to the masked kernel (flagged tiles)."""
    T, H, K = 1024, 2, 64
    q, k, v, qi, ki, w = make_dsa_inputs(T, H, 64, 4, 64, seed=3, dtype=torch.bfloat16, device=_dev())
    q = (q.float() * 40).to(torch.bfloat16)
    q[:, :, 300:] = (q[:, :, 300:].float() / 40).to(torch.bfloat16)       # only the first query tiles are hot
    o, ref = _lists_vs_gather(swv, q, k, v, qi, ki, w, K)
    d = (o - ref).abs()
    assert torch.isfinite(o).all() and float(d.max()) < 5e-2 and float(d.mean()) < 2e-3


def test_tiny_weights_reproduce_the_clamp(swv):
    """Routing weights so small that the reference's max(l, 1e-6) binds: those rows are recomputed by
    the masked kernel's exact path."""
    T, H, K = 512, 2, 32
    q, k, v, qi, ki, w = make_dsa_inputs(T, H, 64, 4, 64, seed=4, dtype=torch.bfloat16, device=_dev())
    o, ref = _lists_vs_gather(swv, q, k, v, qi, ki, w * 1e-5, K)
    assert float(ref.abs().max()) > 0           # damped, not zero
    d = (o - ref).abs()
    assert float(d.max()) <= 2e-2 * max(1.0, float(ref.abs().max())) and float(d.max()) < 2e-2
    rel = d.sum() / ref.abs().sum()
    assert float(rel) < 2e-2, float(rel)


def test_overfull_tiles_go_to_the_dense_sweep(swv):
    """Every query selects the same block of keys: the (query tile, key tile) lists of that block exceed
    their capacity and the query tiles are left to the masked kernel."""
    T, H, K = 4096, 2, 256
    q, k, v, qi, ki, w = make_dsa_inputs(T, H, 64, 4, 64, seed=6, dtype=torch.bfloat16, device=_dev(), w_mode="abs")
    qi = qi.abs()
    ki = -ki.abs()
    ki[:, 1024:1024 + K] = ki[:, 1024:1024 + K].abs() * 4      # the only keys with positive scores
    o, ref = _lists_vs_gather(swv, q, k, v, qi, ki, w, K)
    _close(o, ref)


def test_fused_path_picks_the_kernel_by_density(swv, monkeypatch):
    """dsa_sparse_attention gives the same result through the list kernel and through the dense sweep."""
    T, H, K = 4096, 2, 128                       # one key in 32: the list kernel
    q, k, v, qi, ki, w = make_dsa_inputs(T, H, 64, 4, 64, seed=8, dtype=torch.bfloat16, device=_dev())
    o_lists = swv.dsa_sparse_attention(q, k, v, qi, ki, w, K, out_dtype=torch.float32)
    monkeypatch.setenv("SWV_DSA_ATTN", "sweep")
    o_sweep = swv.dsa_sparse_attention(q, k, v, qi, ki, w, K, out_dtype=torch.float32)
    swv.check_status(_dev())
    assert float((o_lists - o_sweep).abs().max()) < 2e-3


def test_slot_order_of_a_row_does_not_matter(swv):
    """The per-tile lists are built from the rows' slots in whatever order they come."""
    from sparse_wsi_vit_b200.ops import dsa_attention_lists
    T, H, K = 2048, 2, 64
    q, k, v, qi, ki, w = make_dsa_inputs(T, H, 64, 4, 64, seed=12, dtype=torch.bfloat16, device=_dev())
    idx, valid, scores, sel = swv.dsa_indexer_topk(qi, ki, w, K, want_mask=True)
    o1 = torch.empty((1, H, T, 64), dtype=torch.float32, device=_dev())
    dsa_attention_lists(q, k, v, idx, scores, sel, o1)
    g = torch.Generator(device="cpu").manual_seed(1)
    perm = torch.stack([torch.randperm(K, generator=g) for _ in range(T)]).to(_dev())[None]
    o2 = torch.empty_like(o1)
    dsa_attention_lists(q, k, v, torch.gather(idx, 2, perm).contiguous(), torch.gather(scores, 2, perm).contiguous(), sel,
                        o2)
    swv.check_status(_dev())
    # the same products, added by the tensor cores in the same (key) order: identical up to the order in
    # which a tile's bf16 entries were rounded -- they are rounded one by one, so bit for bit
    assert torch.equal(o1, o2)
