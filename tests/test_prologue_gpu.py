"""The fused token-local prologue (one launch: in-place 2-D RoPE of q / k + indexer head collapse)
and the single-GEMM projection of the inference path, against the separate steps they replace."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_prologue_equals_separate_rope_and_collapse(dtype):
    import sparse_wsi_vit_b200 as swv
    from sparse_wsi_vit_b200 import ops
    B, T, H, D, IH, ID, K, C = 1, 700, 2, 64, 4, 32, 48, 2
    g = torch.Generator().manual_seed(1)
    qkv = torch.randn(B, T, 3, H, D, generator=g).to(dtype).to(DEV)
    qi = (torch.randn(B, T, IH, ID, generator=g) / 6).to(dtype).to(DEV)
    ki = (torch.randn(B, T, IH, ID, generator=g) / 6).to(dtype).to(DEV)
    w = torch.randn(IH, generator=g).to(DEV)
    coords = torch.cat([torch.zeros(C, 2), (torch.randint(0, 40, (T - C, 2), generator=g) * 224).float()]).to(DEV)
    # separate steps
    ref = qkv.clone()
    for i in (0, 1):
        x = ref[0, :, i]
        swv.rope2d(x, coords, 224.0 * 40, skip_tokens=C, out=x)
    idx_r, valid_r, sc_r = swv.dsa_indexer_topk(qi, ki, w, K)
    # one launch
    got = qkv.clone()
    ws = ops.dsa_prologue(got[:, :, 0], got[:, :, 1], qi, ki, w, coords, 224.0 * 40, 10000.0, C)
    idx, valid, sc = swv.dsa_indexer_topk(qi, ki, w, K, workspace=ws, precollapsed=True)
    swv.check_status(DEV)
    assert torch.equal(got, ref), "in-place rotary embedding differs from the stand-alone kernel"
    assert torch.equal(idx, idx_r) and torch.equal(sc, sc_r) and torch.equal(valid, valid_r)
    # without coordinates only the collapse runs and q / k are left alone
    untouched = qkv.clone()
    ws2 = ops.dsa_prologue(untouched[:, :, 0], untouched[:, :, 1], qi, ki, w)
    idx2, _, sc2 = swv.dsa_indexer_topk(qi, ki, w, K, workspace=ws2, precollapsed=True)
    assert torch.equal(untouched, qkv) and torch.equal(idx2, idx_r) and torch.equal(sc2, sc_r)


def test_inference_module_uses_one_projection_gemm_and_matches_training_path():
    """Without gradients the three Linears run as one GEMM over concatenated weights and the prologue
    launch replaces the separate RoPE / collapse steps; with gradients the module takes the separate,
    differentiable route.  Same result (bf16 autocast) and the cache follows parameter updates."""
    import sparse_wsi_vit_b200 as swv
    torch.manual_seed(0)
    m = swv.DeepSeekSparseAttention(d_model=128, attention_heads=2, indexer_heads=4, indexer_dim=32, top_k=64).to(DEV)
    x = torch.randn(1, 500, 128, generator=torch.Generator().manual_seed(2)).to(DEV)
    coords = (torch.randint(0, 30, (498, 2), generator=torch.Generator().manual_seed(3)) * 224).float().to(DEV)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        with torch.no_grad():
            y_inf = m(x, coords, 224.0 * 30, 2)
        assert m._cat is not None
        y_trn = m(x.clone().requires_grad_(), coords, 224.0 * 30, 2)
    swv.check_status(DEV)
    assert (y_inf.float() - y_trn.float()).abs().max() < 3e-2
    key = m._cat[0]
    with torch.no_grad():
        m.qkv_proj.weight.mul_(1.5)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y2 = m(x, coords, 224.0 * 30, 2)
    assert m._cat[0] != key and (y2.float() - y_inf.float()).abs().max() > 1e-3
