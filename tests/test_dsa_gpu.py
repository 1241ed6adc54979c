"""GPU parity tests of the DSA forward path: the CUDA kernels, called through the
C ABI, against the CPU oracle and the reference-generated fixtures."""
import os

import numpy as np
import pytest
import torch

from oracle import dsa as O
from tests.golden.make_golden import dsa_cases
from tests.util import make_dsa_inputs, overlap_fraction, own_scores, sets_equal

pytestmark = pytest.mark.gpu

# TF32 operands keep 10 mantissa bits: each product is off by at most ~2^-9 relative.
SCORE_ATOL = 1e-2          # for the benchmark-distributed inputs, whose scores are O(1)


def score_error_bound(qi, ki, w):
    """Elementwise bound 2^-9 * sum_d |wq_d| |wk_d| on |tf32 score - fp32 score|."""
    wq = O.collapse_heads(qi, w).abs()
    wk = O.collapse_heads(ki, w).abs()
    return 2.0 ** -9 * (wq @ wk.T) + 1e-6


@pytest.fixture(scope="module")
def swv():
    import sparse_wsi_vit_b200 as m
    return m


def _dev():
    return torch.device("cuda:0")


def _check(swv):
    swv.check_status(_dev())


@pytest.mark.parametrize("T,K", [(1, 8), (5, 8), (63, 8), (64, 64), (65, 16), (127, 64), (200, 256), (1000, 64),
                                 (1000, 2048), (384, 128), (500, 33), (700, 100), (3000, 7)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_indexer_topk_small(swv, T, K, dtype):
    q, k, v, qi, ki, w = make_dsa_inputs(T, 1, 64, 4, 64, seed=T * 7 + K, dtype=dtype, device=_dev())
    idx, valid, scores = swv.dsa_indexer_topk(qi, ki, w, K)
    full = own_scores(qi, ki, w)[0]                      # (T, T) the library's own scores
    _check(swv)
    k_eff = min(K, T)
    # (1) bit-exact: the selected set is the lower-index top-k of the same score values
    ridx, rvalid, rsel = O.topk_lower_index(full.cpu(), K)
    assert torch.equal(idx[0].cpu(), ridx), "index sets differ from stable top-k of own scores"
    assert torch.equal(valid[0].cpu(), rvalid)
    assert torch.equal(scores[0].cpu(), rsel)
    # (2) the scores themselves against the fp32 oracle
    s_ref = O.indexer_scores(qi[0].cpu(), ki[0].cpu(), w.cpu())
    assert bool(((full.cpu() - s_ref).abs() <= score_error_bound(qi[0].cpu(), ki[0].cpu(), w.cpu())).all())
    # (3) set overlap with the fp32 oracle's selection
    oidx, _, _ = O.topk_lower_index(s_ref, K)
    tie = O.rows_with_straddling_tie(s_ref, K)
    if (~tie).any() and T > K:
        ov = overlap_fraction(idx[0, ~tie.to(idx.device), :k_eff], oidx[~tie, :k_eff], T)
        assert ov > 0.97, ov


def test_indexer_batch_and_strided_inputs(swv):
    B, T, IH, ID, K = 3, 150, 4, 32, 16
    g = torch.Generator().manual_seed(3)
    big_q = torch.randn(B, T, IH, 2 * ID, generator=g).to(_dev())
    big_k = torch.randn(T, B, IH, ID, generator=g).to(_dev())
    qi = big_q[..., ::2]                 # inner stride 2
    ki = big_k.transpose(0, 1)           # batch/time swapped strides
    w = torch.tensor([0.5, -1.0, 0.0, 2.0], device=_dev())
    idx, valid, scores = swv.dsa_indexer_topk(qi, ki, w, K)
    for b in range(B):
        full = own_scores(qi[b:b + 1].contiguous(), ki[b:b + 1].contiguous(), w)[0]
        ridx, _, rsel = O.topk_lower_index(full.cpu(), K)
        assert torch.equal(idx[b].cpu(), ridx)
        assert torch.equal(scores[b].cpu(), rsel)
        s_ref = O.indexer_scores(qi[b].cpu(), ki[b].cpu(), w.cpu())
        assert bool(((full.cpu() - s_ref).abs() <= score_error_bound(qi[b].cpu(), ki[b].cpu(), w.cpu())).all())
    _check(swv)


def test_indexer_ties_go_to_lower_index(swv):
    """Few distinct key rows -> many exact ties straddling the K-th value; rows with
    fewer than K positive scores -> ties at zero."""
    T, IH, ID, K = 300, 2, 16, 32
    g = torch.Generator().manual_seed(11)
    base = torch.randn(1, 7, IH, ID, generator=g)
    ki = base[:, torch.arange(T) % 7].contiguous().to(_dev())
    qi = torch.randn(1, T, IH, ID, generator=g).to(_dev())
    w = torch.tensor([1.0, 0.5], device=_dev())
    idx, valid, scores = swv.dsa_indexer_topk(qi, ki, w, K)
    full = own_scores(qi, ki, w)[0].cpu()
    assert O.rows_with_straddling_tie(full, K).sum() > T // 2
    ridx, _, rsel = O.topk_lower_index(full, K)
    assert torch.equal(idx[0].cpu(), ridx)
    assert torch.equal(scores[0].cpu(), rsel)
    # all-negative products: every score is 0, the first K keys win
    idx2, _, sc2 = swv.dsa_indexer_topk(qi.abs(), -ki.abs(), w, K)
    assert torch.equal(idx2[0].cpu(), torch.arange(K, dtype=torch.int32).expand(T, K))
    assert float(sc2.abs().max()) == 0.0
    _check(swv)


@pytest.mark.parametrize("case", [c[0] for c in dsa_cases()])
def test_against_reference_fixtures(swv, golden_dir, case):
    g = np.load(os.path.join(golden_dir, "dsa_reference.npz"))
    B, T, H, D, IH, ID, K = [int(x) for x in g[f"{case}.dims"]]
    t = lambda n: torch.from_numpy(g[f"{case}.{n}"]).to(_dev())
    # attention kernel on the REFERENCE's own idx/valid/scores: same inputs -> same output
    o = torch.zeros(B, H, T, D, device=_dev())
    rw = t("scores") * t("valid")
    out = swv.DSAAttentionFunction.apply(t("q"), t("k"), t("v"), t("idx"), t("valid"), rw, o, B, H, T, D, K,
                                         16, 16, H, 16)
    assert out.data_ptr() == o.data_ptr()
    assert (o - t("o")).abs().max() < 1e-4
    # indexer: scores per selected key agree with the reference's, sets agree off ties
    idx, valid, scores = swv.LightningIndexerFunction.apply(t("qi"), t("ki"), t("w"), B, T, IH, ID, K, 16, 16, 16,
                                                            IH)
    assert torch.equal(valid.sum(-1), t("valid").sum(-1))
    k_eff = min(K, T)
    for b in range(B):
        s_ref = O.indexer_scores(t("qi")[b].cpu(), t("ki")[b].cpu(), t("w").cpu())
        mine = torch.gather(s_ref, 1, idx[b, :, :k_eff].long().cpu())
        assert (mine - scores[b, :, :k_eff].cpu()).abs().max() < SCORE_ATOL
        tie = O.rows_with_straddling_tie(s_ref, K)
        rows = ~tie
        if rows.any() and T > K:
            ref_idx = t("idx")[b].cpu()
            ov = overlap_fraction(idx[b].cpu()[rows], ref_idx[rows], T)
            assert ov > 0.95, (case, ov)
    if T < K:
        assert bool((idx[..., T:] == 0).all()) and bool((scores[..., T:] == 0).all())
        assert bool((valid[..., T:] == 0).all())
    _check(swv)


@pytest.mark.parametrize("T,H,D,K", [(200, 2, 64, 32), (77, 1, 32, 8), (130, 2, 128, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gather_attention_vs_oracle(swv, T, H, D, K, dtype):
    q, k, v, qi, ki, w = make_dsa_inputs(T, H, D, 4, 64, seed=5 + T, dtype=dtype, device=_dev())
    idx, valid, scores = swv.dsa_indexer_topk(qi, ki, w, K)
    # unsorted list with a repeated entry and an invalid slot: the kernel must honour all of it
    perm = torch.randperm(K, generator=torch.Generator().manual_seed(1)).to(_dev())
    idx, valid, scores = idx[..., perm].contiguous(), valid[..., perm].contiguous(), scores[..., perm].contiguous()
    idx[:, :, 1] = idx[:, :, 0]
    valid[:, :, 2] = 0.0
    rw = scores * valid
    o = torch.zeros(1, H, T, D, device=_dev(), dtype=torch.float32)
    swv.dsa_attention_gather(q, k, v, idx, valid, rw, o)
    ref = O.dsa_attention(q[0].float().cpu(), k[0].float().cpu(), v[0].float().cpu(), idx[0].cpu(), valid[0].cpu(),
                          rw[0].cpu())
    assert (o[0].cpu() - ref).abs().max() < 1e-4          # fp32 accumulation on identical inputs
    _check(swv)


def _masked_vs_oracle(swv, T, H, K, seed, rows=None, out_dtype=torch.float32, w_mode="randn"):
    q, k, v, qi, ki, w = make_dsa_inputs(T, H, 64, 4, 64, seed=seed, dtype=torch.bfloat16, device=_dev(),
                                         w_mode=w_mode)
    o, idx, valid, scores = swv.dsa_sparse_attention(q, k, v, qi, ki, w, K, out_dtype=out_dtype, return_topk=True)
    _check(swv)
    assert torch.isfinite(o.float()).all()
    r = slice(None) if rows is None else rows
    ref = O.dsa_attention(q[0, :, r].float().cpu(), k[0].float().cpu(), v[0].float().cpu(), idx[0, r].cpu(),
                          valid[0, r].cpu(), (scores * valid)[0, r].cpu())
    diff = (o[0, :, r].float().cpu() - ref).abs()
    return diff, o, idx, valid, scores, (q, k, v, qi, ki, w)


@pytest.mark.parametrize("T,H,K", [(128, 1, 16), (200, 2, 32), (1000, 2, 64), (333, 1, 512), (1536, 2, 256)])
def test_masked_attention_vs_oracle(swv, T, H, K):
    """bf16 tensor-core path vs the fp32 oracle on the same (bf16-rounded) inputs and the same key lists.
    Tolerance from the specification of the path: 2e-2 max-abs, 1e-3 mean-abs."""
    diff, *_ = _masked_vs_oracle(swv, T, H, K, seed=T + K)
    assert diff.max() < 2e-2, float(diff.max())
    assert diff.mean() < 1e-3, float(diff.mean())


def test_masked_matches_gather_and_bf16_out(swv):
    diff, o, idx, valid, scores, (q, k, v, qi, ki, w) = _masked_vs_oracle(swv, 700, 2, 128, seed=9,
                                                                         out_dtype=torch.bfloat16)
    assert diff.max() < 2e-2
    og = torch.zeros(1, 2, 700, 64, device=_dev())
    swv.dsa_attention_gather(q, k, v, idx, valid, scores * valid, og)
    assert (og - o.float()).abs().max() < 2e-2
    _check(swv)


def test_all_zero_weights_give_exact_zero(swv):
    """Rows whose selected scores are all 0 produce exactly 0 (the 1e-6 clamp on the denominator)."""
    T, H, K = 256, 1, 32
    q, k, v, qi, ki, w = make_dsa_inputs(T, H, 64, 4, 64, seed=2, dtype=torch.bfloat16, device=_dev(), w_mode="abs")
    o = swv.dsa_sparse_attention(q, k, v, qi.abs(), -ki.abs(), w, K, out_dtype=torch.float32)
    assert float(o.abs().max()) == 0.0
    _check(swv)


def test_module_matches_reference_fixture(swv, golden_dir):
    g = np.load(os.path.join(golden_dir, "dsa_module_reference.npz"))
    m = swv.DeepSeekSparseAttention(d_model=64, attention_heads=2, indexer_heads=4, indexer_dim=16, top_k=16,
                                    BLOCK_Q=16, BLOCK_K=16, BLOCK_D=16)
    sd = {k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("sd.")}
    m.load_state_dict(sd, strict=True)
    m = m.to(_dev())
    with torch.no_grad():
        y = m(torch.from_numpy(g["x"]).to(_dev()))
    ref = torch.from_numpy(g["y"])
    # fp32 inputs: exact attention arithmetic; the TF32 indexer may swap two keys whose scores
    # differ by < 1e-3 at the K-th place, which moves one of 16 weights by that much.
    assert (y.cpu() - ref).abs().max() < 5e-3
    assert (y.cpu() - ref).abs().mean() < 2e-4
    _check(swv)


@pytest.mark.parametrize("T", [16384, 65536])
def test_benchmark_config_sampled_rows(swv, T):
    """8 heads x 64, 4x64 indexer, top-2048, bf16 at 16384 tokens (the single-layer DSA
    configuration) and at 65536 tokens (the workload the benchmark times): full GPU run, oracle on
    192 sampled query rows; own-score bit-exactness on the same rows."""
    H, K = 8, 2048
    rows = torch.randperm(T, generator=torch.Generator().manual_seed(0))[:192].sort().values
    diff, o, idx, valid, scores, (q, k, v, qi, ki, w) = _masked_vs_oracle(swv, T, H, K, seed=1234, rows=rows)
    assert diff.max() < 2e-2 and diff.mean() < 1e-3, (float(diff.max()), float(diff.mean()))
    # structural properties on every row
    assert bool((valid == 1).all())
    assert bool((idx[..., 1:] > idx[..., :-1]).all()) and int(idx.min()) >= 0 and int(idx.max()) < T
    # bit-exact top-k on the sampled rows: recompute those rows' full score vectors as a
    # (Tq=192, Tk=T, top_k=T) call and take the stable top-k on the CPU
    full = own_scores(qi[:, rows.to(_dev())].contiguous(), ki, w)[0].cpu()
    ridx, _, rsel = O.topk_lower_index(full, K)
    assert torch.equal(idx[0, rows.to(_dev())].cpu(), ridx)
    assert torch.equal(scores[0, rows.to(_dev())].cpu(), rsel)
    # against the fp32 oracle's selection
    s_ref = O.indexer_scores(qi[0, rows.to(_dev())].cpu(), ki[0].cpu(), w.cpu())
    assert bool(((full - s_ref).abs() <= score_error_bound(qi[0, rows.to(_dev())].cpu(), ki[0].cpu(), w.cpu())).all())
    oidx, _, _ = O.topk_lower_index(s_ref, K)
    assert overlap_fraction(ridx, oidx, T) > 0.99
    _check(swv)


def test_indexer_split_key_range(swv):
    """Few query tiles against a long key range (one rank of a sequence-sharded run): two CTAs per
    query tile sweep half of the keys each and merge.  Same bit-exact contract, including ties
    that straddle the two halves and rows selected entirely from one half."""
    Tq, Tk, IH, ID, K = 300, 8192 + 100, 4, 64, 512
    g = torch.Generator().manual_seed(21)
    qi = (torch.randn(1, Tq, IH, ID, generator=g) / 8).to(_dev())
    ki = (torch.randn(1, Tk, IH, ID, generator=g) / 8).to(_dev())
    w = torch.randn(IH, generator=g).to(_dev())
    idx, valid, scores = swv.dsa_indexer_topk(qi, ki, w, K)
    full = own_scores(qi, ki, w)[0].cpu()                # (Tq, Tk), itself through the split path (top_k = Tk)
    ridx, rvalid, rsel = O.topk_lower_index(full, K)
    assert torch.equal(idx[0].cpu(), ridx)
    assert torch.equal(scores[0].cpu(), rsel)
    assert torch.equal(valid[0].cpu(), rvalid)
    s_ref = O.indexer_scores(qi[0].cpu(), ki[0].cpu(), w.cpu())
    assert bool(((full - s_ref).abs() <= score_error_bound(qi[0].cpu(), ki[0].cpu(), w.cpu())).all())
    # ties: 9 distinct key rows repeated over the whole range, so every threshold value occurs in both halves
    base = torch.randn(1, 9, IH, ID, generator=g) / 8
    kt = base[:, torch.arange(Tk) % 9].contiguous().to(_dev())
    idx2, _, sc2 = swv.dsa_indexer_topk(qi, kt, w, K)
    full2 = own_scores(qi, kt, w)[0].cpu()
    assert O.rows_with_straddling_tie(full2, K).sum() > Tq // 2
    r2, _, s2 = O.topk_lower_index(full2, K)
    assert torch.equal(idx2[0].cpu(), r2)
    assert torch.equal(sc2[0].cpu(), s2)
    # every score zero: the first K keys win, all of them in the first half
    idx3, _, sc3 = swv.dsa_indexer_topk(qi.abs(), -ki.abs(), w.abs(), K)
    assert torch.equal(idx3[0].cpu(), torch.arange(K, dtype=torch.int32).expand(Tq, K))
    assert float(sc3.abs().max()) == 0.0
    _check(swv)


@pytest.mark.parametrize("K", [256, 6000])
def test_masked_attention_short_query_range(swv, K):
    """Queries are a slice of a longer key sequence (the sharded layout): fused path == gather path.
    With so few query tiles both the indexer and the attention split the key range over several
    CTAs; K = 6000 exceeds the number of positive scores of a row (threshold 0), which takes the
    two-pass softmax path through the same merge."""
    Tq, Tk, H, D = 256, 8192 + 64, 2, 64
    g = torch.Generator().manual_seed(22)
    q = (torch.randn(1, H, Tq, D, generator=g) / 8).to(torch.bfloat16).to(_dev())
    k = torch.randn(1, H, Tk, D, generator=g).to(torch.bfloat16).to(_dev())
    v = torch.randn(1, H, Tk, D, generator=g).to(torch.bfloat16).to(_dev())
    qi = (torch.randn(1, Tq, 4, 64, generator=g) / 8).to(torch.bfloat16).to(_dev())
    ki = (torch.randn(1, Tk, 4, 64, generator=g) / 8).to(torch.bfloat16).to(_dev())
    w = torch.randn(4, generator=g).to(_dev())
    idx, valid, scores, sel = swv.dsa_indexer_topk(qi, ki, w, K, want_mask=True)
    o = torch.zeros((1, H, Tq, D), dtype=torch.float32, device=_dev())
    swv.dsa_attention_masked(q, k, v, sel, o)
    o2 = torch.zeros_like(o)
    swv.dsa_attention_gather(q, k, v, idx, valid, scores * valid, o2)
    _check(swv)
    assert float((o - o2).abs().max()) < 2e-2
    assert float((o - o2).abs().mean()) < 1e-3


def test_split_paths_batch_odd_heads_ragged(swv):
    """The key-range splits with a batch of 2, an odd number of heads (a CTA with one head), query and
    key counts that are not multiples of the tile: fused path == gather path, indices == stable top-k."""
    B, Tq, Tk, H, D, K = 2, 200, 8192 + 37, 3, 64, 300
    g = torch.Generator().manual_seed(23)
    q = (torch.randn(B, H, Tq, D, generator=g) / 8).to(torch.bfloat16).to(_dev())
    k = torch.randn(B, H, Tk, D, generator=g).to(torch.bfloat16).to(_dev())
    v = torch.randn(B, H, Tk, D, generator=g).to(torch.bfloat16).to(_dev())
    qi = (torch.randn(B, Tq, 4, 64, generator=g) / 8).to(torch.bfloat16).to(_dev())
    ki = (torch.randn(B, Tk, 4, 64, generator=g) / 8).to(torch.bfloat16).to(_dev())
    w = torch.randn(4, generator=g).to(_dev())
    idx, valid, scores, sel = swv.dsa_indexer_topk(qi, ki, w, K, want_mask=True)
    o = torch.zeros((B, H, Tq, D), dtype=torch.float32, device=_dev())
    swv.dsa_attention_masked(q, k, v, sel, o)
    o2 = torch.zeros_like(o)
    swv.dsa_attention_gather(q, k, v, idx, valid, scores * valid, o2)
    _check(swv)
    for b in range(B):
        full = own_scores(qi[b:b + 1].contiguous(), ki[b:b + 1].contiguous(), w)[0].cpu()
        ridx, _, rsel = O.topk_lower_index(full, K)
        assert torch.equal(idx[b].cpu(), ridx)
        assert torch.equal(scores[b].cpu(), rsel)
    assert float((o - o2).abs().max()) < 2e-2
    assert float((o - o2).abs().mean()) < 1e-3


def _random_case(seed):
    r = np.random.RandomState(seed)
    B = int(r.choice([1, 1, 2]))
    Tq = int(r.randint(1, 600))
    Tk = Tq if r.rand() < 0.4 else int(r.randint(Tq, 9000))
    H = int(r.randint(1, 5))
    K = int(r.randint(1, min(Tk, 2500) + 1))
    quantised = bool(r.rand() < 0.3)                     # few distinct score values: many ties at the threshold
    return B, Tq, Tk, H, K, quantised


@pytest.mark.parametrize("seed", list(range(100, 112)))
def test_random_shapes(swv, seed):
    """Seeded random shapes (batch, ragged query / key counts, 1-4 heads, any top_k, some with heavily
    tied scores): indices == stable top-k of the library's own scores, fused path == gather path."""
    B, Tq, Tk, H, K, quantised = _random_case(seed)
    D = 64
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, Tq, D, generator=g) / 8).to(torch.bfloat16).to(_dev())
    k = torch.randn(B, H, Tk, D, generator=g).to(torch.bfloat16).to(_dev())
    v = torch.randn(B, H, Tk, D, generator=g).to(torch.bfloat16).to(_dev())
    qi = torch.randn(B, Tq, 4, 64, generator=g) / 8
    ki = torch.randn(B, Tk, 4, 64, generator=g) / 8
    if quantised:
        qi, ki = (qi * 4).round() / 4, (ki * 4).round() / 4
    qi, ki = qi.to(torch.bfloat16).to(_dev()), ki.to(torch.bfloat16).to(_dev())
    w = torch.randn(4, generator=g).to(_dev())
    idx, valid, scores, sel = swv.dsa_indexer_topk(qi, ki, w, K, want_mask=True)
    o = torch.zeros((B, H, Tq, D), dtype=torch.float32, device=_dev())
    swv.dsa_attention_masked(q, k, v, sel, o)
    o2 = torch.zeros_like(o)
    swv.dsa_attention_gather(q, k, v, idx, valid, scores * valid, o2)
    _check(swv)
    tag = f"B={B} Tq={Tq} Tk={Tk} H={H} K={K} quantised={quantised}"
    for b in range(B):
        full = own_scores(qi[b:b + 1].contiguous(), ki[b:b + 1].contiguous(), w)[0].cpu()
        ridx, rvalid, rsel = O.topk_lower_index(full, K)
        assert torch.equal(idx[b].cpu(), ridx), tag
        assert torch.equal(valid[b].cpu(), rvalid), tag
        assert torch.equal(scores[b].cpu(), rsel), tag
    assert torch.isfinite(o).all(), tag
    assert float((o - o2).abs().max()) < 2e-2, tag
    assert float((o - o2).abs().mean()) < 1e-3, tag


@pytest.mark.parametrize("T,H,K,mode", [(16384, 8, 2048, "bench"), (65536, 2, 2048, "bench"), (1500, 2, 300, "ties"),
                                        (900, 3, 800, "fewpos"), (4096, 2, 301, "twins"), (3072, 3, 301, "triplets"),
                                        (3072, 2, 302, "triplets"), (16384, 2, 2047, "twins")])
def test_attention_kernel_selects_exactly_the_indexer_members(swv, T, H, K, mode):
    """The dense attention sweep recomputes every score tile on the tensor cores and, on its one-pass
    path, treats a key as selected iff that score >= the row threshold the indexer found.  The
    diagnostic entry point counts those keys per row: exactly min(K, T) everywhere <=> the
    recomputed tiles are bit-identical to the scores the selection was made on (one flipped key
    would be invisible in the output tolerance).  Benchmark-distributed inputs at 16384 and 65536
    tokens (one-pass path), heavily tied scores and rows with fewer than K positive scores (the
    two-pass bitmask path), and keys that exist twice or three times with K chosen so that EVERY
    row's threshold falls inside such a group (ties cut by key index, one or two keys per row left
    out: the one-pass path with the row's list of unselected ties)."""
    q, k, v, qi, ki, w = make_dsa_inputs(T, H, 64, 4, 64, seed=77 + T, dtype=torch.bfloat16, device=_dev())
    if mode == "ties":
        qi, ki = (qi.float() * 32).round() / 32, (ki.float() * 32).round() / 32
        qi, ki = qi.to(torch.bfloat16), ki.to(torch.bfloat16)
    if mode == "fewpos":
        qi, ki = qi.abs(), -ki.abs()
        ki[:, ::5] = ki[:, ::5].abs()
    if mode == "twins":                       # key t + T/2 is key t: the twin sits in another key tile
        ki[:, T // 2:] = ki[:, :T // 2]
    if mode == "triplets":                    # keys 3m, 3m + 1, 3m + 2 are one key
        ki[:, 1::3] = ki[:, 0::3]
        ki[:, 2::3] = ki[:, 0::3]
    idx, valid, scores, sel = swv.dsa_indexer_topk(qi, ki, w, K, want_mask=True)
    if mode in ("twins", "triplets"):
        # the rows really are cut: the (K+1)-th score equals the K-th on (nearly) every row
        full = own_scores(qi[:, :256].contiguous(), ki, w)[0]
        srt = full.sort(dim=-1, descending=True).values
        assert float((srt[:, K - 1] == srt[:, K]).float().mean()) > 0.9
        o_list = torch.empty((1, H, T, 64), dtype=torch.float32, device=_dev())
        swv.dsa_attention_gather(q, k, v, idx, valid, scores * valid, o_list)
    o = torch.empty((1, H, T, 64), dtype=torch.float32, device=_dev())
    from sparse_wsi_vit_b200.ops import dsa_attention_masked_count
    cnt = dsa_attention_masked_count(q, k, v, sel, o)
    _check(swv)
    assert int(cnt.min()) == min(K, T) and int(cnt.max()) == min(K, T), (int(cnt.min()), int(cnt.max()))
    # and the output of the counting instantiation is the regular kernel's (which may split the key
    # range over several CTAs and add the parts up in another order)
    o2 = torch.empty_like(o)
    swv.dsa_attention_masked(q, k, v, sel, o2)
    _check(swv)
    assert float((o - o2).abs().max()) < 1e-3
    if mode in ("twins", "triplets"):
        assert float((o2 - o_list).abs().max()) < 2e-2 and float((o2 - o_list).abs().mean()) < 1e-3


@pytest.mark.parametrize("mode", ["sample_too_high", "sample_too_low", "plain"])
def test_two_sweep_selection_and_its_fallback(swv, mode):
    """Sparse top-k on a long key range takes the short form of the selection: a lower bound of every
    row's threshold from a sample of key tiles (every 12th tile at this size), one sweep that lists the
    keys above it, a per-row exact select.  When the sample misleads -- its keys score much higher or
    much lower than the rest -- rows find too few candidates or the lists overflow, and the query tiles
    are redone by the exact passes.  All three cases must give the exact top-k of the library's own scores."""
    T, K = 49152, 1024
    q, k, v, qi, ki, w = make_dsa_inputs(T, 1, 64, 4, 64, seed=123, dtype=torch.bfloat16, device=_dev())
    if mode != "plain":
        tiles = ki.view(1, T // 128, 128, 4, 64)
        scale = 3.0 if mode == "sample_too_high" else 0.05
        tiles[:, ::12] = (tiles[:, ::12].float() * scale).to(torch.bfloat16)    # the sampled key tiles
    idx, valid, scores, sel = swv.dsa_indexer_topk(qi, ki, w, K, want_mask=True)
    _check(swv)
    rows = torch.arange(0, T, 397, device=_dev())
    full = own_scores(qi[:, rows].contiguous(), ki, w)[0].cpu()
    ridx, rvalid, rsel = O.topk_lower_index(full, K)
    assert torch.equal(idx[0, rows].cpu(), ridx)
    assert torch.equal(scores[0, rows].cpu(), rsel)
    assert bool((valid == 1).all())
    # the membership mask agrees with the lists (the attention's dense sweep reads it)
    o1 = torch.empty((1, 1, T, 64), dtype=torch.float32, device=_dev())
    o2 = torch.empty_like(o1)
    swv.dsa_attention_masked(q, k, v, sel, o1)
    swv.dsa_attention_gather(q, k, v, idx, valid, scores * valid, o2)
    _check(swv)
    assert float((o1 - o2).abs().max()) < 2e-2


@pytest.mark.parametrize("scale", [1.0, 1.1, 1.15, 1.25])
def test_two_sweep_selection_on_a_rank_share(swv, scale):
    """One rank's share of a sharded slide: a ragged query range (49 tiles and 2 rows) against a long
    ragged key range (448 tiles and 2 keys), the key range split over two CTAs per query tile.  The
    sampled key tiles are scaled a little, so that the lower bound is marginal: in the same query tile
    some rows find enough candidates and others do not (they flag the tile while their neighbours are
    being selected)."""
    Tq, Tk, K = 6274, 57346, 2048
    q, k, v, qi, ki, w = make_dsa_inputs(Tk, 2, 64, 4, 64, seed=31, dtype=torch.bfloat16, device=_dev())
    step = ((Tk + 127) // 128) // 32
    for t in range(0, 32 * step, step):                                        # the sampled key tiles
        ki[:, t * 128:(t + 1) * 128] = (ki[:, t * 128:(t + 1) * 128].float() * scale).to(torch.bfloat16)
    qi_loc = qi[:, Tk - Tq:].contiguous()
    idx, valid, scores, sel = swv.dsa_indexer_topk(qi_loc, ki, w, K, want_mask=True)
    _check(swv)
    assert int(idx.min()) >= 0 and int(idx.max()) < Tk
    rows = torch.arange(0, Tq, 97, device=_dev())
    full = own_scores(qi_loc[:, rows].contiguous(), ki, w)[0].cpu()
    ridx, rvalid, rsel = O.topk_lower_index(full, K)
    assert torch.equal(idx[0, rows].cpu(), ridx)
    assert torch.equal(scores[0, rows].cpu(), rsel)
    # every row: K distinct keys in ascending order
    assert bool((idx[0, :, 1:] > idx[0, :, :-1]).all())
    q_loc = q[:, :, Tk - Tq:].contiguous()
    o1 = torch.empty((1, 2, Tq, 64), dtype=torch.float32, device=_dev())
    o2 = torch.empty_like(o1)
    swv.dsa_attention_masked(q_loc, k, v, sel, o1)
    swv.dsa_attention_gather(q_loc, k, v, idx, valid, scores * valid, o2)
    _check(swv)
    assert float((o1 - o2).abs().max()) < 2e-2
