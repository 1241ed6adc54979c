"""Assembled encoders on the GPU against the CPU restatement built from the reference's parts
(oracle/encoder.py): the 2-layer 2-D block-pattern model at 4096 patches on a 64x64 grid, and the
DSA encoder with 2-D RoPE (single GPU, whole and through the sharded ragged driver at world 1)."""
import pytest
import torch

from oracle import encoder as E

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _grid_coords(n_side=64, tile=8):
    """Block-major tokens: block b = tile (b // 8, b % 8) of an 8x8 tile grid, token t inside = (t // 8, t % 8)."""
    n = n_side * n_side
    t = torch.arange(n)
    per = tile * tile
    blk, tin = t // per, t % per
    tiles_per_row = n_side // tile
    return torch.stack([(blk // tiles_per_row) * tile + tin // tile, (blk % tiles_per_row) * tile + tin % tile], dim=1).float()


@pytest.mark.parametrize("pool", ["cls", "mean"])
def test_block2d_model_4096_patches(pool):
    """4096 patch embeddings (1280-d, N(0,1)) on a 64x64 grid, 1 CLS token, d_model 384, 6 heads x 64,
    2 layers, block 64 = one 8x8 tile, Chebyshev-1 neighbourhood + the global block, 2-D RoPE."""
    import sparse_wsi_vit_b200 as swv
    torch.manual_seed(0)
    net = swv.BlockSparse2DViTSlideEncoder(in_features=1280, out_features=2, embed_dim=384, num_heads=6, num_layers=2,
                                           num_cls=1, block=64, coord_high=64.0, pool=pool).eval()
    with torch.no_grad():
        net.cls_pool.weight.normal_(0, 0.2)
    x = torch.randn(4096, 1280, generator=torch.Generator().manual_seed(1))
    coords = _grid_coords()
    rp, ci = swv.patterns.chebyshev_grid_blocks(8, 8, 1, global_blocks=[64])
    ref = E.block2d_encoder_forward(net.state_dict(), x, coords, rp, ci, 64, 2, 6, 1, 64.0, pool=pool)
    net = net.to(DEV)
    with torch.no_grad():
        got = net(x.to(DEV), coords.to(DEV), torch.from_numpy(rp).to(DEV), torch.from_numpy(ci).to(DEV))["logits"][0]
    swv.check_status(DEV)
    # fp32 weights and projections, bf16 tensor-core attention inside
    assert (got.cpu() - ref).abs().max() < 3e-2, (got.cpu(), ref)


def test_dsa_encoder_with_rope_matches_assembled_oracle():
    import sparse_wsi_vit_b200 as swv
    from sparse_wsi_vit_b200.dist import sharded_ragged_forward
    torch.manual_seed(3)
    cfg = dict(in_features=96, out_features=3, embed_dim=128, num_heads=2, num_layers=2, num_cls=2, indexer_heads=4,
               indexer_dim=32, top_k=64)
    net = swv.DSAViTSlideEncoder(**cfg, rope_coord_high=224.0 * 32).eval()
    n = 700
    x = torch.randn(n, 96, generator=torch.Generator().manual_seed(4))
    coords = (torch.randint(0, 32, (n, 2), generator=torch.Generator().manual_seed(5)) * 224).float()
    ref = E.dsa_encoder_forward(net.state_dict(), x, 2, 2, 4, 32, 64, 2, coords=coords, coord_high=224.0 * 32)
    ref_plain = E.dsa_encoder_forward(net.state_dict(), x, 2, 2, 4, 32, 64, 2)
    net = net.to(DEV)
    with torch.no_grad():
        got = net(x.to(DEV), coords.to(DEV))["logits"][0]          # fp32: exact list kernel + TF32 indexer
        plain = net(x.to(DEV))["logits"][0]
        ragged = sharded_ragged_forward(net, [x, x[:300]], 1, 0, coords=[coords, coords[:300]], align=8)["logits"]
    swv.check_status(DEV)
    assert (ref - ref_plain).abs().max() > 1e-3                     # the rotary term matters in this setup
    # the TF32 indexer may swap keys whose scores tie to ~1e-3 at the K-th place (see the module test)
    assert (got.cpu() - ref).abs().max() < 1e-2, (got.cpu(), ref)
    assert (plain.cpu() - ref_plain).abs().max() < 1e-2
    assert torch.allclose(ragged[0].cpu(), got.cpu(), atol=1e-5)
    ref300 = E.dsa_encoder_forward(net.cpu().state_dict(), x[:300], 2, 2, 4, 32, 64, 2, coords=coords[:300],
                                   coord_high=224.0 * 32)
    assert (ragged[1].cpu() - ref300).abs().max() < 1e-2
