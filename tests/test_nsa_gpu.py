"""NSA-style attention (compressed / selected / sliding-window + gate) against the builder-defined
CPU oracle (parity unpinned: the reference has no NSA code)."""
import pytest
import torch

from oracle import nsa as N

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.mark.parametrize("T,Hq,Hkv,D,topk,window", [(700, 4, 2, 128, 4, 128), (1500, 8, 2, 64, 16, 512),
                                                    (300, 2, 1, 128, 16, 64), (1111, 8, 1, 128, 8, 256),
                                                    (900, 16, 2, 64, 4, 128)])
def test_nsa_vs_oracle(T, Hq, Hkv, D, topk, window):
    import sparse_wsi_vit_b200 as swv
    from sparse_wsi_vit_b200.nsa import nsa_attention
    g = torch.Generator().manual_seed(T)
    q = (torch.randn(1, Hq, T, D, generator=g)).to(torch.bfloat16)
    k = torch.randn(1, Hkv, T, D, generator=g).to(torch.bfloat16)
    v = torch.randn(1, Hkv, T, D, generator=g).to(torch.bfloat16)
    gate = torch.randn(1, T, Hq, 3, generator=g)
    out, o_cmp, o_sel, o_win, blocks = nsa_attention(q.to(DEV), k.to(DEV), v.to(DEV), gate.to(DEV), sel_topk=topk,
                                                     window=window, out_dtype=torch.float32, return_parts=True)
    swv.check_status(DEV)
    ref, r_cmp, r_sel, r_win, r_blocks = N.nsa_attention(q[0], k[0], v[0], gate[0], sel_topk=topk, window=window,
                                                        return_parts=True)
    tol = dict(atol=3e-2, rtol=0)
    assert torch.allclose(o_cmp[0].cpu(), r_cmp, **tol)
    assert torch.allclose(o_win[0].cpu(), r_win, **tol)
    # the selection is a top-k on sums of probabilities: allow a few near-tie swaps (bf16 pooled keys)
    same = (blocks[0].cpu().long() == r_blocks).all(dim=-1)            # (Hkv, T)
    assert same.float().mean() > 0.9
    rows = same.repeat_interleave(Hq // Hkv, dim=0)                    # (Hq, T)
    assert (o_sel[0].cpu() - r_sel)[rows].abs().max() < 3e-2
    assert (out[0].cpu() - ref)[rows].abs().max() < 3e-2
    assert (out[0].cpu() - ref).abs().mean() < 2e-3


def test_nsa_single_call_equals_stepwise():
    """`swv_nsa_attn_fwd` (one call, device-built block lists, caller workspace) runs the same kernels
    as the step-by-step composition: identical output bits."""
    import sparse_wsi_vit_b200 as swv
    from sparse_wsi_vit_b200.nsa import nsa_attention
    T, Hq, Hkv, D = 1100, 8, 2, 128
    g = torch.Generator().manual_seed(5)
    q = torch.randn(1, Hq, T, D, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(1, Hkv, T, D, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(1, Hkv, T, D, generator=g).to(torch.bfloat16).to(DEV)
    gate = torch.randn(1, T, Hq, 3, generator=g).to(DEV)
    one = nsa_attention(q, k, v, gate, sel_topk=8, window=256, out_dtype=torch.float32)
    parts = nsa_attention(q, k, v, gate, sel_topk=8, window=256, out_dtype=torch.float32, return_parts=True)
    swv.check_status(DEV)
    assert torch.equal(one, parts[0])
