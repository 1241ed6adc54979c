"""GPU parity tests of the static / block-sparse attention kernel and the 2-D RoPE kernel against
the CPU oracle and the reference-generated fixtures."""
import os

import numpy as np
import pytest
import torch

from oracle import static_attn as S

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.fixture(scope="module")
def swv():
    import sparse_wsi_vit_b200 as m
    return m


def _qkv(T, H, D, seed, Tk=None):
    g = torch.Generator().manual_seed(seed)
    Tk = Tk or T
    q = torch.randn(1, H, T, D, generator=g).to(torch.bfloat16)
    k = torch.randn(1, H, Tk, D, generator=g).to(torch.bfloat16)
    v = torch.randn(1, H, Tk, D, generator=g).to(torch.bfloat16)
    return q, k, v


def _dev(*ts):
    return tuple(t.to(DEV) for t in ts)


def _check_vs_oracle(swv, q, k, v, rp, ci, block, rows=None, **kw):
    o = swv.block_sparse_attention(*_dev(q, k, v), torch.from_numpy(rp).to(DEV), torch.from_numpy(ci).to(DEV), block,
                                   out_dtype=torch.float32, **kw)
    swv.check_status(DEV)
    if kw.get("mode", 0) == 1:
        mask = S.static_window_mask(q.shape[2], kw["num_cls"], kw["window"], kw["dilation"])
        mask = mask if rows is None else mask[rows]
    else:
        mask = S.expand_block_mask(rp, ci, block, q.shape[2], k.shape[2], rows=rows)
    r = slice(None) if rows is None else rows
    ref = S.masked_attention(q[0, :, r].float(), k[0].float(), v[0].float(), mask)
    diff = (o[0, :, r].cpu() - ref).abs()
    assert torch.isfinite(o).all()
    assert diff.max() < 2e-2 and diff.mean() < 1e-3, (float(diff.max()), float(diff.mean()))
    return o


@pytest.mark.parametrize("T,H,D,block", [(300, 2, 64, 64), (1000, 2, 64, 128), (520, 2, 128, 128), (300, 1, 128, 64),
                                         (64, 1, 64, 64), (129, 1, 64, 128)])
def test_block_mask_vs_oracle(swv, T, H, D, block):
    nb = -(-T // block)
    rp, ci = swv.patterns.band_random_blocks(nb, band=1, n_global=1, p=0.3, seed=T)
    q, k, v = _qkv(T, H, D, seed=T + D)
    _check_vs_oracle(swv, q, k, v, rp, ci, block)


def test_empty_rows_and_full_list(swv):
    T, H, D, block = 512, 2, 64, 128
    q, k, v = _qkv(T, H, D, seed=3)
    rows = [[0, 1, 2, 3], [], [2], [0, 3]]
    rp = np.array([0, 4, 4, 5, 7], dtype=np.int32)
    ci = np.array([0, 1, 2, 3, 2, 0, 3], dtype=np.int32)
    o = _check_vs_oracle(swv, q, k, v, rp, ci, block)
    assert float(o[0, :, 128:256].abs().max()) == 0.0          # a query block with no key block -> zeros
    full_rp = np.arange(0, 17, 4, dtype=np.int32)
    full_ci = np.tile(np.arange(4, dtype=np.int32), 4)
    o = swv.block_sparse_attention(*_dev(q, k, v), torch.from_numpy(full_rp).to(DEV), torch.from_numpy(full_ci).to(DEV),
                                   block, out_dtype=torch.float32)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float())
    assert (o.cpu() - ref).abs().max() < 2e-2


def test_cross_lengths_and_small_head_dim(swv):
    """Tq != Tk, and a head dimension the kernel does not have natively (zero-padded to 64)."""
    q, k, v = _qkv(200, 2, 64, seed=5, Tk=450)
    rp, ci = swv.patterns._to_csr([[0, 1, 2, 3], [1, 3]])
    _check_vs_oracle(swv, q, k, v, rp, ci, 128)
    q, k, v = _qkv(300, 2, 16, seed=6)
    rp, ci = swv.patterns.band_random_blocks(3, 1, 1, 0.0, 0)
    _check_vs_oracle(swv, q, k, v, rp, ci, 128)


@pytest.mark.parametrize("T,C,W,d", [(300, 2, 3, 2), (700, 1, 5, 1), (260, 3, 0, 1), (1000, 2, 40, 3)])
def test_static_token_pattern_vs_oracle(swv, T, C, W, d):
    q, k, v = _qkv(T, 2, 64, seed=T + W)
    rp, ci = swv.patterns.static_window_blocks(T, C, W, d, 128)
    _check_vs_oracle(swv, q, k, v, rp, ci, 128, mode=1, num_cls=C, window=W, dilation=d)


def test_static_module_matches_reference_fixtures(swv, golden_dir):
    g = np.load(os.path.join(golden_dir, "static_reference.npz"))
    for name in ("w3d2", "w0", "w2d1"):
        E, H, C, W, dil, N = [int(x) for x in g[f"{name}.cfg"]]
        m = swv.StaticSparseAttention(E, H, num_cls=C, window_size=W, dilation=dil)
        sd = {k.split(".sd.")[1]: torch.from_numpy(g[k]) for k in g.files if k.startswith(f"{name}.sd.")}
        m.load_state_dict(sd, strict=True)
        m = m.to(DEV).eval()
        x = torch.from_numpy(g[f"{name}.x"]).to(DEV)
        with torch.no_grad():
            y = m(x)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                yb = m(x)
        ref = torch.from_numpy(g[f"{name}.y"])
        # fp32 activations: exact list kernel, the fp32 tolerance of the path (1e-4)
        assert (y.cpu() - ref).abs().max() < 1e-4, (name, float((y.cpu() - ref).abs().max()))
        # bf16 activations (autocast): tensor-core kernel, the bf16 tolerance
        assert (yb.float().cpu() - ref).abs().max() < 2e-2, name
        assert (yb.float().cpu() - ref).abs().mean() < 2e-3, name
    swv.check_status(DEV)


def test_rope2d_matches_reference_fixture(swv, golden_dir):
    g = np.load(os.path.join(golden_dir, "rope_reference.npz"))
    hd, high = [int(x) for x in g["cfg"]]
    x = torch.from_numpy(g["x"]).to(DEV)
    coords = torch.from_numpy(g["coords"]).to(DEV)
    y = swv.rope2d(x, coords, float(high))
    assert (y.cpu() - torch.from_numpy(g["y"])).abs().max() < 2e-6
    # bf16 and a skipped CLS prefix
    yb = swv.rope2d(x.to(torch.bfloat16), coords, float(high), skip_tokens=2)
    ref = S.rope2d_apply(x[0].to(torch.bfloat16).float().cpu(), coords[0].cpu(), float(high))
    assert torch.equal(yb[0, :2].cpu(), x[0, :2].to(torch.bfloat16).cpu())
    assert (yb[0, 2:].float().cpu() - ref[2:]).abs().max() < 2e-2


def test_grid_pattern_configuration(swv):
    """4096 patches on a 64x64 grid in 8x8 tiles (64 blocks of 64 tokens) + CLS tokens in a trailing
    global block, Chebyshev-1 neighbourhood, 6 heads x 64, 2-D RoPE on the grid coordinates."""
    H, D, block = 6, 64, 64
    n_cls = 1
    T = 4096 + n_cls
    rp, ci = swv.patterns.chebyshev_grid_blocks(8, 8, 1, global_blocks=[64])
    q, k, v = _qkv(T, H, D, seed=11)
    # block-major grid coordinates: block b = tile (b // 8, b % 8), token t inside = (t // 8, t % 8)
    t = torch.arange(4096)
    blk, tin = t // 64, t % 64
    coords = torch.stack([(blk // 8) * 8 + tin // 8, (blk % 8) * 8 + tin % 8], dim=1).float()
    cpad = torch.cat([coords, torch.zeros(n_cls, 2)])
    qr = swv.rope2d(q[0].transpose(0, 1).contiguous().to(DEV), cpad.to(DEV), 64.0)     # (T, H, D)
    kr = swv.rope2d(k[0].transpose(0, 1).contiguous().to(DEV), cpad.to(DEV), 64.0)
    q_ref = S.rope2d_apply(q[0].transpose(0, 1).float(), cpad, 64.0)
    assert (qr.float().cpu() - q_ref).abs().max() < 3e-2
    rows = torch.cat([torch.arange(0, 200), torch.arange(2000, 2100), torch.arange(T - 70, T)])
    _check_vs_oracle(swv, qr.transpose(0, 1)[None].cpu(), kr.transpose(0, 1)[None].cpu(), v, rp, ci, block, rows=rows)


def test_sweep_configuration_sampled_blocks(swv):
    """Band +-2, one global block, Bernoulli(0.05) extras, head_dim 128, block 128 at 8192 tokens."""
    T, H, D, block = 8192, 4, 128, 128
    rp, ci = swv.patterns.band_random_blocks(T // block, band=2, n_global=1, p=0.05, seed=7)
    q, k, v = _qkv(T, H, D, seed=21)
    rows = torch.cat([torch.arange(0, 256), torch.arange(4000, 4200), torch.arange(T - 128, T)])
    _check_vs_oracle(swv, q, k, v, rp, ci, block, rows=rows)


@pytest.mark.parametrize("T,p", [(32768, 0.25), (131072, 0.05)])
def test_sweep_sizes_sampled_rows(swv, T, p):
    """The block-sparse sweep at the sizes that are timed (band +-2, one global block, Bernoulli(p)
    extras, head_dim 128, block 128): full GPU run, oracle on sampled query rows (the first and
    last blocks and random rows) against exactly the key blocks their row lists name."""
    H, D, block = 2, 128, 128
    rp, ci = swv.patterns.band_random_blocks(T // block, band=2, n_global=1, p=p, seed=9)
    q, k, v = _qkv(T, H, D, seed=31)
    g = torch.Generator().manual_seed(T)
    rows = torch.cat([torch.arange(0, 64), torch.randperm(T, generator=g)[:128].sort().values, torch.arange(T - 64, T)])
    _check_vs_oracle(swv, q, k, v, rp, ci, block, rows=rows)
