"""Generate golden fixtures by running the REFERENCE's own code on the CPU.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference [group ...]

(groups: rope static dsa dsa_bwd dsa_module; default all)

The DSA Triton kernels are executed on CPU tensors by Triton's interpreter
(``TRITON_INTERPRET=1``); the static attention and the 2-D RoPE are plain
PyTorch.  The resulting ``*.npz`` files are committed; the tests never need
the reference checkout.
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t):
    return t.detach().cpu().numpy()


def dsa_cases():
    """(name, B, T, H, D, IH, ID, K, tile, mode)"""
    return [
        ("dsa_rand", 1, 96, 2, 32, 4, 32, 16, 32, "rand"),
        ("dsa_ragged", 1, 77, 2, 16, 4, 16, 8, 16, "rand"),
        ("dsa_short", 1, 5, 1, 16, 2, 16, 8, 16, "rand"),
        ("dsa_batch2_negw", 2, 48, 2, 16, 4, 16, 8, 16, "negw"),
        ("dsa_ties", 1, 40, 1, 16, 2, 16, 8, 16, "ties"),
        ("dsa_fewpos", 1, 64, 1, 16, 2, 16, 32, 16, "fewpos"),
    ]


def make_dsa(ref_kernels):
    out = {}
    for name, B, T, H, D, IH, ID, K, tile, mode in dsa_cases():
        g = torch.Generator().manual_seed(abs(hash(name)) % (2 ** 31) if False else sum(map(ord, name)))
        q = torch.randn(B, H, T, D, generator=g) / D ** 0.5
        k = torch.randn(B, H, T, D, generator=g)
        v = torch.randn(B, H, T, D, generator=g)
        qi = torch.randn(B, T, IH, ID, generator=g) / ID ** 0.5
        ki = torch.randn(B, T, IH, ID, generator=g) / ID ** 0.5
        w = torch.randn(IH, generator=g)
        if mode == "negw":
            w = -w.abs()
            w[0] = 0.7
        if mode == "ties":
            # only 5 distinct key rows -> many exact score ties straddling the K-th value
            base = torch.randn(B, 5, IH, ID, generator=g) / ID ** 0.5
            ki = base[:, torch.arange(T) % 5]
        if mode == "fewpos":
            # most scores negative before the ReLU -> rows with fewer than K positives
            ki = -ki.abs()
            qi = qi.abs()
            ki[:, ::7] = ki[:, ::7].abs()
        idx, valid, scores = ref_kernels.LightningIndexerFunction.apply(
            qi, ki, w, B, T, IH, ID, K, tile, tile, tile, IH)
        rw = scores * valid
        o = torch.zeros(B, H, T, D)
        o = ref_kernels.DSAAttentionFunction.apply(
            q, k, v, idx, valid, rw, o, B, H, T, D, K, tile, tile, H, tile)
        for key, val in dict(q=q, k=k, v=v, qi=qi, ki=ki, w=w, idx=idx, valid=valid,
                             scores=scores, o=o).items():
            out[f"{name}.{key}"] = _np(val)
        out[f"{name}.dims"] = np.array([B, T, H, D, IH, ID, K], dtype=np.int64)
        print(name, "done", flush=True)
    np.savez_compressed(os.path.join(HERE, "dsa_reference.npz"), **out)


def dsa_bwd_cases():
    """(name, B, T, H, D, IH, ID, K, tile)"""
    return [
        ("bwd_rand", 1, 48, 2, 16, 2, 16, 8, 16),
        ("bwd_batch2", 2, 40, 2, 32, 4, 16, 16, 16),
        ("bwd_short", 1, 6, 1, 16, 2, 16, 8, 16),
    ]


def make_dsa_bwd(ref_kernels):
    """Forward + backward of the reference's two autograd Functions (the op sequence of
    DeepSeekSparseAttention.forward) with a seeded upstream gradient; stores every gradient the
    reference produces: dq, dk, dv, the routing-weight gradient, and the indexer's dq_idx, dk_idx, dW."""
    out = {}
    for name, B, T, H, D, IH, ID, K, tile in dsa_bwd_cases():
        g = torch.Generator().manual_seed(sum(map(ord, name)))
        q = (torch.randn(B, H, T, D, generator=g) / D ** 0.5).requires_grad_()
        k = torch.randn(B, H, T, D, generator=g).requires_grad_()
        v = torch.randn(B, H, T, D, generator=g).requires_grad_()
        qi = (torch.randn(B, T, IH, ID, generator=g) / ID ** 0.5).requires_grad_()
        ki = (torch.randn(B, T, IH, ID, generator=g) / ID ** 0.5).requires_grad_()
        w = torch.randn(IH, generator=g).requires_grad_()
        d_out = torch.randn(B, H, T, D, generator=g)
        idx, valid, scores = ref_kernels.LightningIndexerFunction.apply(qi, ki, w, B, T, IH, ID, K, tile, tile, tile, IH)
        rw = scores * valid
        rw.retain_grad()
        o = torch.zeros(B, H, T, D)
        res = ref_kernels.DSAAttentionFunction.apply(q, k, v, idx.detach(), valid.detach(), rw, o, B, H, T, D, K,
                                                     tile, tile, H, tile)
        (res * d_out).sum().backward()
        for key, val in dict(q=q, k=k, v=v, qi=qi, ki=ki, w=w, d_out=d_out, idx=idx, valid=valid, scores=scores,
                             o=res, dq=q.grad, dk=k.grad, dv=v.grad, drw=rw.grad, dqi=qi.grad, dki=ki.grad,
                             dw=w.grad).items():
            out[f"{name}.{key}"] = _np(val)
        out[f"{name}.dims"] = np.array([B, T, H, D, IH, ID, K], dtype=np.int64)
        print(name, "done", flush=True)
    np.savez_compressed(os.path.join(HERE, "dsa_bwd_reference.npz"), **out)


def make_dsa_module(ref_mod):
    """Whole attention module (projections included) with its state_dict."""
    torch.manual_seed(1234)
    m = ref_mod.DeepSeekSparseAttention(d_model=64, attention_heads=2, indexer_heads=4,
                                        indexer_dim=16, top_k=16, BLOCK_Q=16, BLOCK_K=16, BLOCK_D=16)
    x = torch.randn(1, 50, 64)
    with torch.no_grad():
        y = m(x)
    out = {"x": _np(x), "y": _np(y)}
    for k, val in m.state_dict().items():
        out["sd." + k] = _np(val)
    np.savez_compressed(os.path.join(HERE, "dsa_module_reference.npz"), **out)
    print("dsa module done", flush=True)


def make_static(ref_static):
    out = {}
    for name, E, Hh, C, W, dil, N in [("w3d2", 32, 2, 2, 3, 2, 37), ("w0", 32, 2, 1, 0, 1, 20),
                                      ("w2d1", 64, 1, 1, 2, 1, 33)]:
        torch.manual_seed(sum(map(ord, name)))
        m = ref_static.StaticSparseAttention(E, Hh, num_cls=C, window_size=W, dilation=dil).eval()
        x = torch.randn(2, C + N, E)
        with torch.no_grad():
            y = m(x)
        out[f"{name}.x"] = _np(x)
        out[f"{name}.y"] = _np(y)
        out[f"{name}.cfg"] = np.array([E, Hh, C, W, dil, N], dtype=np.int64)
        for k, val in m.state_dict().items():
            out[f"{name}.sd.{k}"] = _np(val)
    np.savez_compressed(os.path.join(HERE, "static_reference.npz"), **out)
    print("static done", flush=True)


def make_rope(ref_rope):
    out = {}
    torch.manual_seed(7)
    hd = 64
    rope = ref_rope.VisionRotaryEmbedding(dim=hd // 2, pt_seq_len=16, coord_high=224.0 * 64, dynamic=True)
    L, H = 29, 3
    x = torch.randn(1, L, H, hd)
    coords = (torch.randint(0, 64, (1, L, 2)) * 224).float()
    with torch.no_grad():
        y = rope(x, coords)
    out.update(x=_np(x), coords=_np(coords), y=_np(y), cfg=np.array([hd, 224 * 64], dtype=np.int64))
    np.savez_compressed(os.path.join(HERE, "rope_reference.npz"), **out)
    print("rope done", flush=True)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: TRITON_INTERPRET=1 python tests/golden/make_golden.py <path to a sparse-wsi-vit checkout>")
    ref = sys.argv[1]
    sys.path.insert(0, os.path.join(ref, "src"))
    from sparse_wsi_vit.models.deepseek_sparse_attention_kernels import kernels as ref_kernels
    from sparse_wsi_vit.models import deepseek_sparse_attention as ref_mod
    from sparse_wsi_vit.models import static_sparse_attention as ref_static
    from sparse_wsi_vit.models.vit_5 import rope as ref_rope
    only = sys.argv[2:]                      # optional: names of the fixture groups to regenerate
    if not only or "rope" in only:
        make_rope(ref_rope)
    if not only or "static" in only:
        make_static(ref_static)
    if not only or "dsa" in only:
        make_dsa(ref_kernels)
    if not only or "dsa_bwd" in only:
        make_dsa_bwd(ref_kernels)
    if not only or "dsa_module" in only:
        make_dsa_module(ref_mod)


if __name__ == "__main__":
    main()
