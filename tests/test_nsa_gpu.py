"""NSA-style attention (compressed / selected / sliding-window + gate) against the library-defined
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
    ref, r_cmp, r_sel, r_win, r_blocks, margin = N.nsa_attention(q[0], k[0], v[0], gate[0], sel_topk=topk,
                                                                window=window, return_parts=True,
                                                                pooled_dtype=torch.bfloat16)
    _compare(Hq, Hkv, out[0].cpu(), o_cmp[0].cpu(), o_sel[0].cpu(), o_win[0].cpu(), blocks[0].cpu(), ref, r_cmp, r_sel,
             r_win, r_blocks, margin)


def _compare(Hq, Hkv, out, o_cmp, o_sel, o_win, blocks, ref, r_cmp, r_sel, r_win, r_blocks, margin):
    """The oracle pools from the same bf16-rounded values as the library, so the block importances
    agree to fp32 round-off: the selected blocks must be IDENTICAL on every row whose last selected
    and first rejected importance differ by more than 1e-5 relative (ten times the fp32 round-off of the sums) (a smaller gap is a near-tie
    that another summation order may legitimately break the other way), and such near-tie rows
    must be rare."""
    tol = dict(atol=3e-2, rtol=0)
    assert torch.allclose(o_cmp, r_cmp, **tol)
    assert torch.allclose(o_win, r_win, **tol)
    same = (blocks.long() == r_blocks).all(dim=-1)                     # (Hkv, R)
    clear = margin > 1e-5
    assert bool(same[clear].all()), f"{int((~same & clear).sum())} rows with a clear margin selected other blocks"
    assert clear.float().mean() > 0.9
    rows = same.repeat_interleave(Hq // Hkv, dim=0)                    # (Hq, R)
    assert (o_sel - r_sel)[rows].abs().max() < 3e-2
    assert (out - ref)[rows].abs().max() < 3e-2
    assert (out - ref)[rows].abs().mean() < 2e-3


def test_nsa_benchmark_size_sampled_rows():
    """65536 tokens, 16 query / 2 kv heads, head_dim 128, 32/16 compression, 16 blocks of 64, window
    512 (the NSA configuration that is timed): full GPU run, oracle on 96 sampled query rows
    against all keys."""
    import sparse_wsi_vit_b200 as swv
    from sparse_wsi_vit_b200.nsa import nsa_attention
    T, Hq, Hkv, D = 65536, 16, 2, 128
    g = torch.Generator().manual_seed(65)
    q = torch.randn(1, Hq, T, D, generator=g).to(torch.bfloat16)
    k = torch.randn(1, Hkv, T, D, generator=g).to(torch.bfloat16)
    v = torch.randn(1, Hkv, T, D, generator=g).to(torch.bfloat16)
    gate = torch.randn(1, T, Hq, 3, generator=g)
    rows = torch.cat([torch.arange(0, 16), torch.randperm(T, generator=g)[:64].sort().values, torch.arange(T - 16, T)])
    out, o_cmp, o_sel, o_win, blocks = nsa_attention(q.to(DEV), k.to(DEV), v.to(DEV), gate.to(DEV),
                                                     out_dtype=torch.float32, return_parts=True)
    one = nsa_attention(q.to(DEV), k.to(DEV), v.to(DEV), gate.to(DEV), out_dtype=torch.float32)
    swv.check_status(DEV)
    assert (one - out).abs().max() < 1e-5
    ref, r_cmp, r_sel, r_win, r_blocks, margin = N.nsa_attention(q[0], k[0], v[0], gate[0], return_parts=True,
                                                                rows=rows, pooled_dtype=torch.bfloat16)
    _compare(Hq, Hkv, out[0, :, rows].cpu(), o_cmp[0, :, rows].cpu(), o_sel[0, :, rows].cpu(), o_win[0, :, rows].cpu(),
             blocks[0][:, rows].cpu(), ref, r_cmp, r_sel, r_win, r_blocks, margin)


def test_nsa_single_call_equals_stepwise():
    """`swv_nsa_attn_fwd` (one call, device-built block lists, caller workspace, gates applied in the
    branch epilogues) against the step-by-step composition (branch outputs + gate kernel)."""
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
    # same kernels and the same order of additions; the fused epilogues contract g * o + acc into one
    # FMA where the stand-alone gate kernel may round the product first
    assert (one - parts[0]).abs().max() < 1e-5
