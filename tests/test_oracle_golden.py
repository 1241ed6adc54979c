"""The CPU oracle against fixtures produced by the reference's own code
(tests/golden/make_golden.py).  No GPU, no reference checkout needed."""
import os

import numpy as np
import pytest
import torch

from oracle import dsa as O
from oracle import static_attn as S

from tests.golden.make_golden import dsa_cases


@pytest.fixture(scope="module")
def dsa_gold(golden_dir):
    return np.load(os.path.join(golden_dir, "dsa_reference.npz"))


def _t(a):
    return torch.from_numpy(np.asarray(a))


@pytest.mark.parametrize("case", [c[0] for c in dsa_cases()])
def test_indexer_scores_and_topk_match_reference(dsa_gold, case):
    g = dsa_gold
    B, T, H, D, IH, ID, K = [int(x) for x in g[f"{case}.dims"]]
    for b in range(B):
        s = O.indexer_scores(_t(g[f"{case}.qi"][b]), _t(g[f"{case}.ki"][b]), _t(g[f"{case}.w"]))
        ref_idx, ref_valid, ref_sc = (_t(g[f"{case}.{n}"][b]) for n in ("idx", "valid", "scores"))
        # 1) the sequential replace-min simulation reproduces the reference exactly, slot order included
        sim_idx, sim_valid, sim_sc = O.topk_replace_min(s, K)
        assert torch.equal(sim_valid, ref_valid)
        assert torch.equal(sim_idx, ref_idx)
        assert torch.allclose(sim_sc, ref_sc, rtol=0, atol=1e-6)
        # 2) the lower-index rule gives the same SET on every row without a straddling tie
        idx, valid, sc = O.topk_lower_index(s, K)
        assert torch.equal(valid.sum(1), ref_valid.sum(1))
        tie = O.rows_with_straddling_tie(s, K)
        k_eff = min(K, T)
        for r in range(T):
            if tie[r]:
                continue
            mine = sorted(idx[r, :k_eff].tolist())
            ref = sorted(ref_idx[r][ref_valid[r] > 0].tolist())
            assert mine == ref, (case, b, r)
        # unfilled slots
        if T < K:
            assert torch.all(idx[:, T:] == 0) and torch.all(sc[:, T:] == 0)
            assert torch.all(ref_idx[:, T:] == 0)


def test_tie_fixture_really_has_straddling_ties(dsa_gold):
    g = dsa_gold
    s = O.indexer_scores(_t(g["dsa_ties.qi"][0]), _t(g["dsa_ties.ki"][0]), _t(g["dsa_ties.w"]))
    assert O.rows_with_straddling_tie(s, 8).sum() >= 3
    s = O.indexer_scores(_t(g["dsa_fewpos.qi"][0]), _t(g["dsa_fewpos.ki"][0]), _t(g["dsa_fewpos.w"]))
    assert ((s > 0).sum(1) < 32).any()


@pytest.mark.parametrize("case", [c[0] for c in dsa_cases()])
def test_attention_matches_reference(dsa_gold, case):
    """Routing-weighted attention restatement, fed the REFERENCE's idx/valid/scores."""
    g = dsa_gold
    B = int(g[f"{case}.dims"][0])
    for b in range(B):
        idx, valid, sc = (_t(g[f"{case}.{n}"][b]) for n in ("idx", "valid", "scores"))
        o = O.dsa_attention(_t(g[f"{case}.q"][b]), _t(g[f"{case}.k"][b]), _t(g[f"{case}.v"][b]),
                            idx, valid, sc * valid)
        assert torch.allclose(o, _t(g[f"{case}.o"][b]), rtol=0, atol=2e-6), case


@pytest.mark.parametrize("case", [c[0] for c in dsa_cases()])
def test_lower_index_rule_leaves_attention_unchanged(dsa_gold, case):
    """Keys that differ between the two tie rules carry equal scores; the output
    moves only through which V rows sit behind equal weights -> equal when the
    tied weight is 0 (the common case), otherwise bounded."""
    g = dsa_gold
    B, T, H, D, IH, ID, K = [int(x) for x in g[f"{case}.dims"]]
    for b in range(B):
        o, idx, valid, sc = O.dsa_forward(_t(g[f"{case}.q"][b]), _t(g[f"{case}.k"][b]), _t(g[f"{case}.v"][b]),
                                          _t(g[f"{case}.qi"][b]), _t(g[f"{case}.ki"][b]), _t(g[f"{case}.w"]), K)
        s = O.indexer_scores(_t(g[f"{case}.qi"][b]), _t(g[f"{case}.ki"][b]), _t(g[f"{case}.w"]))
        tie = O.rows_with_straddling_tie(s, K)
        ref = _t(g[f"{case}.o"][b])
        ok_rows = ~tie
        assert torch.allclose(o[:, ok_rows], ref[:, ok_rows], rtol=0, atol=2e-6)
        # rows whose straddling tie is at score 0: weights are 0 -> same numerator; only the
        # max over selected logits can move, and it matters only through the 1e-6 clamp
        srt = torch.sort(s, dim=1, descending=True).values
        if T > K:
            zero_tie = tie & (srt[:, K - 1] == 0)
            l_big = (sc * valid).sum(1) > 1e-3
            rows = zero_tie & l_big
            if rows.any():
                assert torch.allclose(o[:, rows], ref[:, rows], rtol=0, atol=1e-5)


def test_dense_mask_form_equals_gathered_form(dsa_gold):
    g, case = dsa_gold, "dsa_rand"
    K = int(g[f"{case}.dims"][-1])
    q, k, v = (_t(g[f"{case}.{n}"][0]) for n in "qkv")
    s = O.indexer_scores(_t(g[f"{case}.qi"][0]), _t(g[f"{case}.ki"][0]), _t(g[f"{case}.w"]))
    o1 = O.dsa_attention_dense(q, k, v, s, K)
    o2 = O.dsa_forward(q, k, v, _t(g[f"{case}.qi"][0]), _t(g[f"{case}.ki"][0]), _t(g[f"{case}.w"]), K)[0]
    assert torch.allclose(o1, o2, atol=2e-6, rtol=0)


def test_static_attention_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "static_reference.npz"))
    for name in ("w3d2", "w0", "w2d1"):
        E, H, C, W, dil, N = [int(x) for x in g[f"{name}.cfg"]]
        sd = {k.split(".sd.")[1]: _t(g[k]) for k in g.files if k.startswith(f"{name}.sd.")}
        y = S.static_sparse_attention(_t(g[f"{name}.x"]), sd, H, C, W, dil)
        assert torch.allclose(y, _t(g[f"{name}.y"]), atol=2e-6, rtol=0), name


def test_rope_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "rope_reference.npz"))
    hd, high = [int(x) for x in g["cfg"]]
    y = S.rope2d_apply(_t(g["x"])[0], _t(g["coords"])[0], float(high))
    assert torch.allclose(y, _t(g["y"])[0], atol=1e-6, rtol=0)


def test_block_sparse_oracle_is_dense_under_full_list():
    torch.manual_seed(0)
    q, k, v = (torch.randn(2, 70, 16) for _ in range(3))
    nb = 3
    row_ptr = [0, 3, 6, 9]
    col = [0, 1, 2] * 3
    o = S.block_sparse_attention(q, k, v, row_ptr, col, 32)
    ref = torch.nn.functional.scaled_dot_product_attention(q[None], k[None], v[None])[0]
    assert torch.allclose(o, ref, atol=1e-5)


@pytest.mark.parametrize("case", ["bwd_rand", "bwd_batch2", "bwd_short"])
def test_backward_restatements_match_reference_gradients(golden_dir, case):
    """The oracle's backward formulas against gradients produced by the reference's own backward
    kernels (Triton interpreter, fixtures from make_golden.py): attention dq/dk/dv/d(routing
    weights) and the indexer's dq/dk/dW, fed with the routing-weight gradient the reference itself
    propagated."""
    import numpy as np
    g = np.load(os.path.join(golden_dir, "dsa_bwd_reference.npz"))
    B, T, H, D, IH, ID, K = [int(x) for x in g[f"{case}.dims"]]
    t = lambda n: torch.from_numpy(g[f"{case}.{n}"])
    dw_sum = torch.zeros(IH)
    for b in range(B):
        rw = (t("scores") * t("valid"))[b]
        dq, dk, dv, drw = O.dsa_attention_bwd(t("d_out")[b], t("q")[b], t("k")[b], t("v")[b], t("o")[b], t("idx")[b],
                                              t("valid")[b], rw)
        for mine, name in ((dq, "dq"), (dk, "dk"), (dv, "dv"), (drw, "drw")):
            ref = t(name)[b]
            assert (mine - ref).abs().max() <= 2e-5 * max(1.0, float(ref.abs().max())), (case, name)
        dqi, dki, dw = O.indexer_bwd(t("drw")[b] * t("valid")[b], t("qi")[b], t("ki")[b], t("w"), t("idx")[b],
                                     t("valid")[b])
        assert (dqi - t("dqi")[b]).abs().max() <= 1e-5 * max(1.0, float(t("dqi").abs().max()))
        assert (dki - t("dki")[b]).abs().max() <= 1e-5 * max(1.0, float(t("dki").abs().max()))
        dw_sum += dw
    assert (dw_sum - t("dw")).abs().max() <= 1e-4 * max(1.0, float(t("dw").abs().max()))


def test_attention_backward_is_the_gradient_of_the_forward():
    """Off the 1e-6 clamp the reference's hand-written attention backward equals autograd through
    the forward restatement."""
    g = torch.Generator().manual_seed(3)
    H, T, D, K = 2, 20, 8, 6
    q = torch.randn(H, T, D, generator=g, dtype=torch.float64).requires_grad_()
    k = torch.randn(H, T, D, generator=g, dtype=torch.float64).requires_grad_()
    v = torch.randn(H, T, D, generator=g, dtype=torch.float64).requires_grad_()
    idx = torch.stack([torch.randperm(T, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    valid = torch.ones(T, K)
    valid[:, -1] = 0
    rw = torch.rand(T, K, generator=g, dtype=torch.float64).requires_grad_()
    d_out = torch.randn(H, T, D, generator=g, dtype=torch.float64)
    o = O.dsa_attention(q, k, v, idx, valid, rw * valid, dtype=torch.float64)
    (o * d_out).sum().backward()
    dq, dk, dv, drw = O.dsa_attention_bwd(d_out, q.detach(), k.detach(), v.detach(), o.detach(), idx, valid,
                                          (rw * valid).detach(), dtype=torch.float64)
    assert torch.allclose(dq, q.grad, atol=1e-10) and torch.allclose(dk, k.grad, atol=1e-10)
    assert torch.allclose(dv, v.grad, atol=1e-10) and torch.allclose(drw * valid, rw.grad, atol=1e-10)
