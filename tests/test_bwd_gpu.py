"""GPU parity tests of the backward kernels (attention and indexer), called through the C ABI,
against the oracle's restatement of the reference's backward kernels and against gradients the
reference itself produced (fixtures)."""
import os

import numpy as np
import pytest
import torch

from oracle import dsa as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.fixture(scope="module")
def swv():
    import sparse_wsi_vit_b200 as m
    return m


def _close(a, b, rel=2e-4):
    ref = float(b.abs().max())
    return float((a.cpu().float() - b).abs().max()) <= rel * max(1.0, ref)


@pytest.mark.parametrize("case", ["bwd_rand", "bwd_batch2", "bwd_short"])
def test_backward_kernels_match_reference_gradients(swv, golden_dir, case):
    g = np.load(os.path.join(golden_dir, "dsa_bwd_reference.npz"))
    B, T, H, D, IH, ID, K = [int(x) for x in g[f"{case}.dims"]]
    t = lambda n: torch.from_numpy(g[f"{case}.{n}"])
    d = lambda n: t(n).to(DEV)
    rw = d("scores") * d("valid")
    dq, dk, dv, drw = swv.ops.dsa_attention_bwd(d("d_out"), d("q"), d("k"), d("v"), d("o"), d("idx"), d("valid"), rw)
    swv.check_status(DEV)
    for mine, name in ((dq, "dq"), (dk, "dk"), (dv, "dv"), (drw, "drw")):
        assert _close(mine, t(name)), (case, name)
    dqi, dki, dw = swv.ops.dsa_indexer_bwd(d("drw") * d("valid"), d("qi"), d("ki"), d("w"), d("idx"), d("valid"))
    swv.check_status(DEV)
    assert _close(dqi, t("dqi")) and _close(dki, t("dki")) and _close(dw, t("dw"), rel=1e-3), case


@pytest.mark.parametrize("T,Tk,H,D,K,dtype", [(200, 200, 2, 64, 32, torch.float32), (77, 300, 1, 32, 8, torch.float32),
                                              (130, 130, 2, 128, 64, torch.bfloat16), (50, 50, 3, 64, 5000, torch.float32),
                                              (64, 64, 1, 160, 16, torch.bfloat16)])
def test_attention_backward_vs_oracle(swv, T, Tk, H, D, K, dtype):
    """Unsorted lists with a repeated key and an invalid slot; cross lengths (queries are a slice of
    the keys); top_k beyond the logit cache (recompute path); head dims 32..160; bf16 inputs."""
    g = torch.Generator().manual_seed(T + K)
    q = (torch.randn(1, H, T, D, generator=g) / D ** 0.5).to(dtype)
    k = torch.randn(1, H, Tk, D, generator=g).to(dtype)
    v = torch.randn(1, H, Tk, D, generator=g).to(dtype)
    keff = min(K, Tk)
    idx = torch.zeros(1, T, K, dtype=torch.int32)
    valid = torch.zeros(1, T, K)
    for r in range(T):
        idx[0, r, :keff] = torch.randperm(Tk, generator=g)[:keff].to(torch.int32)
    valid[..., :keff] = 1.0
    idx[:, :, 1] = idx[:, :, 0]
    valid[:, :, 2] = 0.0
    rw = torch.rand(1, T, K, generator=g) * valid
    d_out = torch.randn(1, H, T, D, generator=g)
    o = O.dsa_attention(q[0].float(), k[0].float(), v[0].float(), idx[0], valid[0], rw[0])[None]
    dq, dk, dv, drw = swv.ops.dsa_attention_bwd(d_out.to(DEV), q.to(DEV), k.to(DEV), v.to(DEV), o.to(DEV), idx.to(DEV),
                                                valid.to(DEV), rw.to(DEV))
    swv.check_status(DEV)
    rq, rk, rv, rrw = O.dsa_attention_bwd(d_out[0], q[0].float(), k[0].float(), v[0].float(), o[0], idx[0], valid[0],
                                          rw[0])
    assert _close(dq[0], rq) and _close(dk[0], rk) and _close(dv[0], rv) and _close(drw[0], rrw)


@pytest.mark.parametrize("B,T,Tk,IH,ID,K,dtype", [(1, 150, 150, 4, 64, 16, torch.float32), (2, 60, 200, 2, 16, 8, torch.bfloat16),
                                                  (1, 40, 40, 4, 32, 64, torch.float32), (1, 33, 90, 8, 64, 12, torch.bfloat16)])
def test_indexer_backward_vs_oracle(swv, B, T, Tk, IH, ID, K, dtype):
    g = torch.Generator().manual_seed(B * 100 + T)
    qi = (torch.randn(B, T, IH, ID, generator=g) / ID ** 0.5).to(dtype)
    ki = (torch.randn(B, Tk, IH, ID, generator=g) / ID ** 0.5).to(dtype)
    w = torch.randn(IH, generator=g)
    keff = min(K, Tk)
    idx = torch.zeros(B, T, K, dtype=torch.int32)
    valid = torch.zeros(B, T, K)
    for b in range(B):
        for r in range(T):
            idx[b, r, :keff] = torch.randperm(Tk, generator=g)[:keff].to(torch.int32)
    valid[..., :keff] = 1.0
    ds = torch.randn(B, T, K, generator=g)
    dq, dk, dw = swv.ops.dsa_indexer_bwd(ds.to(DEV), qi.to(DEV), ki.to(DEV), w.to(DEV), idx.to(DEV), valid.to(DEV))
    swv.check_status(DEV)
    dw_ref = torch.zeros(IH)
    for b in range(B):
        rq, rk, rw_ = O.indexer_bwd(ds[b], qi[b].float(), ki[b].float(), w, idx[b], valid[b])
        assert _close(dq[b], rq) and _close(dk[b], rk)
        dw_ref += rw_
    assert _close(dw, dw_ref, rel=1e-3)


def test_autograd_functions_and_module_train_step(swv):
    """The two reference-shaped autograd Functions chained the way the reference module chains them,
    and the module's own differentiable path (fused forward): gradients reach q/k/v, the indexer
    projections and the head weights, and agree with the oracle's backward on the same lists."""
    B, T, H, D, IH, ID, K = 1, 300, 2, 64, 4, 32, 48
    g = torch.Generator().manual_seed(9)
    mk = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).to(DEV).requires_grad_()
    q, k, v = mk(B, H, T, D, sc=0.125), mk(B, H, T, D), mk(B, H, T, D)
    qi, ki = mk(B, T, IH, ID, sc=0.18), mk(B, T, IH, ID, sc=0.18)
    w = mk(IH)
    d_out = torch.randn(B, H, T, D, generator=g).to(DEV)
    idx, valid, scores = swv.LightningIndexerFunction.apply(qi, ki, w, B, T, IH, ID, K, 16, 16, 16, IH)
    rw = scores * valid
    o = torch.zeros(B, H, T, D, device=DEV)
    out = swv.DSAAttentionFunction.apply(q, k, v, idx.detach(), valid.detach(), rw, o, B, H, T, D, K, 16, 16, H, 16)
    (out * d_out).sum().backward()
    swv.check_status(DEV)
    c = lambda x: x.detach().cpu()
    rq, rk, rv, rrw = O.dsa_attention_bwd(c(d_out)[0], c(q)[0], c(k)[0], c(v)[0], c(out)[0], c(idx)[0], c(valid)[0],
                                          c(rw)[0])
    assert _close(q.grad[0], rq) and _close(k.grad[0], rk) and _close(v.grad[0], rv)
    rqi, rki, rdw = O.indexer_bwd(rrw * c(valid)[0], c(qi)[0], c(ki)[0], c(w), c(idx)[0], c(valid)[0])
    assert _close(qi.grad[0], rqi) and _close(ki.grad[0], rki) and _close(w.grad, rdw, rel=1e-3)

    # the module: bf16 fused forward, one differentiable op; every parameter gets a finite gradient
    torch.manual_seed(0)
    m = swv.DeepSeekSparseAttention(d_model=128, attention_heads=2, indexer_heads=4, indexer_dim=32, top_k=64).to(DEV)
    x = torch.randn(1, 400, 128, generator=torch.Generator().manual_seed(1)).to(DEV).requires_grad_()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = m(x)
    y.float().square().mean().backward()
    swv.check_status(DEV)
    assert torch.isfinite(x.grad).all() and float(x.grad.abs().max()) > 0
    for n, p_ in m.named_parameters():
        assert p_.grad is not None and torch.isfinite(p_.grad).all(), n
    assert float(m.indexer_head_weights.grad.abs().max()) > 0
    # against the fp32 gather-path Functions on the same weights and lists
    m32 = m.float()
    x2 = x.detach().clone().requires_grad_()
    y2 = m32(x2)
    assert (y2 - y.float()).abs().max() < 5e-2


def test_encoder_train_steps_reduce_the_loss(swv):
    """Three optimisation steps of a small DSA encoder through ``training.train_step`` (bf16 autocast,
    the backward kernels under autograd) on a fixed ragged batch: finite gradients everywhere and a
    falling loss."""
    from sparse_wsi_vit_b200.training import train_step
    torch.manual_seed(0)
    net = swv.DSAViTSlideEncoder(in_features=64, out_features=2, embed_dim=128, num_heads=2, num_layers=2, num_cls=2,
                                 indexer_heads=4, indexer_dim=32, top_k=64, rope_coord_high=224.0 * 16).to(DEV).train()
    g = torch.Generator().manual_seed(1)
    batch = {"input": [torch.randn(n, 64, generator=g).to(DEV) for n in (300, 450)],
             "coords": [(torch.randint(0, 16, (n, 2), generator=g) * 224).float().to(DEV) for n in (300, 450)],
             "label": torch.tensor([0, 1], device=DEV)}
    opt = torch.optim.AdamW(net.parameters(), lr=2e-3)
    losses = [train_step(net, opt, batch) for _ in range(4)]
    swv.check_status(DEV)
    assert all(np.isfinite(l) for l in losses), losses
    assert losses[-1] < losses[0], losses
    for n, p_ in net.named_parameters():
        assert p_.grad is not None and torch.isfinite(p_.grad).all(), n
