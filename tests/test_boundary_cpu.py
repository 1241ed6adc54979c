"""Host-side tests that need no GPU: the C-ABI library loads and exports every symbol the
header declares, argument validation rejects bad calls before anything is launched, the
drop-in modules keep the reference's parameter names, and the package has no CPU path."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def swv():
    import __graft_entry__
    __graft_entry__.build()
    import sparse_wsi_vit_b200 as m
    return m


def test_library_exports_every_declared_symbol(swv):
    hdr = open(os.path.join(ROOT, "include", "swv_b200.h")).read()
    declared = set(re.findall(r"\b(swv_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations found in the header"
    lib = ctypes.CDLL(swv._lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/swv_b200.h but not exported"
    assert declared == set(swv._lib.EXPORTS), "python binding list and header disagree"
    assert swv._lib.lib.swv_version() >= 100


def test_error_strings(swv):
    for code in range(-8, 1):
        assert swv._lib.strerror(code) != "unknown code"
    assert "timed out" in swv._lib.strerror(103)
    assert swv._lib.strerror(12345) == "unknown code"


def test_size_queries(swv):
    L = swv._lib.lib
    n = ctypes.c_size_t()
    assert L.swv_dsa_workspace_bytes(1, 65536, 65536, ctypes.byref(n)) == 0
    assert n.value >= 2 * 65536 * 64 * 4 and n.value % 256 == 0
    assert L.swv_dsa_mask_bytes(2, 129, 300, ctypes.byref(n)) == 0
    assert n.value == 2 * 2 * 3 * 128 * 16
    assert L.swv_dsa_workspace_bytes(0, 1, 1, ctypes.byref(n)) == -4
    assert L.swv_dsa_workspace_bytes(1, 1, 1, None) == -1
    # key-range splits: only where they fill the SMs better
    small, big = ctypes.c_size_t(), ctypes.c_size_t()
    assert L.swv_dsa_workspace_bytes(1, 16384, 16384, ctypes.byref(small)) == 0     # 128 tiles: no split
    assert L.swv_dsa_workspace_bytes(1, 8192, 65536, ctypes.byref(big)) == 0        # 64 tiles, 512 key tiles: split
    assert big.value > 2 * 64 * 128 * 259 * 4
    assert L.swv_dsa_attn_scratch_bytes(1, 8, 65536, 65536, ctypes.byref(n)) == 0 and n.value == 0
    assert L.swv_dsa_attn_scratch_bytes(1, 8, 8192, 65536, ctypes.byref(n)) == 0 and n.value > 0
    assert L.swv_dsa_attn_scratch_bytes(1, 8, 256, 1024, ctypes.byref(n)) == 0 and n.value == 0
    assert L.swv_dsa_attn_scratch_bytes(0, 8, 1, 1, ctypes.byref(n)) == -4
    # the workspace with room for per-row candidate lists (two-sweep selection): larger than the base
    # workspace exactly on long key ranges with a selection between about one key in 70 and one in 16
    def topk_extra(T, K, Tq=None):
        a, c = ctypes.c_size_t(), ctypes.c_size_t()
        assert L.swv_dsa_workspace_bytes(1, Tq or T, T, ctypes.byref(a)) == 0
        assert L.swv_dsa_workspace_bytes_topk(1, Tq or T, T, K, ctypes.byref(c)) == 0
        assert c.value >= a.value and c.value % 256 == 0
        return c.value - a.value
    rows = 65536
    extra = topk_extra(65536, 2048)
    assert 2 * rows * 1.6 * 2048 * 4 < extra < 2 * rows * 2.5 * 2048 * 4 + (1 << 20)   # (key, score) lists
    assert topk_extra(65536, 2048, Tq=8192) * 7 < extra                # sized by the query rows of the call
    assert topk_extra(131072, 2048) > 0                                # one key in 64
    assert topk_extra(49152, 1024) > 0                                 # one key in 48
    assert topk_extra(16384, 512) == 0 and topk_extra(32768, 1024) == 0    # short key ranges
    assert topk_extra(65536, 8192) == 0                                # one key in 8: too dense
    assert topk_extra(262144, 2048) == 0                               # one key in 128: the sample is too small
    assert topk_extra(300000, 8192) == 0                               # beyond 262144 keys
    assert L.swv_dsa_workspace_bytes_topk(1, 1, 1, 0, ctypes.byref(n)) == -4
    assert L.swv_dsa_workspace_bytes_topk(1, 1, 1, 1, None) == -1
    # NSA sizes
    assert L.swv_nsa_importance_bytes(1, 2, 65536, 4095, 16, 64, ctypes.byref(n)) == 0
    assert n.value == 2 * 65536 * 1024 * 4
    assert L.swv_nsa_importance_bytes(1, 2, 65536, 4095, 16, 40, ctypes.byref(n)) == -4
    assert L.swv_nsa_workspace_bytes(1, 16, 2, 65536, 128, 32, 16, 64, 16, 512, ctypes.byref(n)) == 0
    assert n.value > 16 * 65536 * 128 * 4          # one fp32 accumulator of the gated branch sum
    assert L.swv_nsa_workspace_bytes(1, 16, 3, 65536, 128, 32, 16, 64, 16, 512, ctypes.byref(n)) == -4


def test_argument_validation_happens_before_any_launch(swv):
    """No CUDA device is needed: every rejected call returns its code from host-side checks."""
    L = swv._lib.lib
    i64x4 = (ctypes.c_int64 * 4)(1, 1, 1, 1)
    i64x3 = (ctypes.c_int64 * 3)(1, 1, 1)
    fake = ctypes.c_void_p(0x1000)           # never dereferenced: validation fails first
    null = ctypes.c_void_p(0)
    # NULL pointers
    rc = L.swv_dsa_indexer_topk_fwd(null, i64x4, fake, i64x4, 0, fake, 1, 8, 8, 4, 64, 4, fake, fake, fake, null,
                                    fake, 1 << 20, fake, null)
    assert rc == -1
    # bad dtype / sizes / indexer dim
    args = lambda dtype, T, ID, K, ws: (fake, i64x4, fake, i64x4, dtype, fake, 1, T, T, 4, ID, K, fake, fake, fake,
                                        null, fake, ws, fake, null)
    assert L.swv_dsa_indexer_topk_fwd(*args(7, 8, 64, 4, 1 << 20)) == -3
    assert L.swv_dsa_indexer_topk_fwd(*args(0, 0, 64, 4, 1 << 20)) == -4
    assert L.swv_dsa_indexer_topk_fwd(*args(0, 8, 64, 0, 1 << 20)) == -4
    assert L.swv_dsa_indexer_topk_fwd(*args(0, 8, 128, 4, 1 << 20)) == -8
    assert L.swv_dsa_indexer_topk_fwd(*args(0, 8, 64, 4, 16)) == -5
    # misaligned workspace
    rc = L.swv_dsa_indexer_topk_fwd(fake, i64x4, fake, i64x4, 0, fake, 1, 8, 8, 4, 64, 4, fake, fake, fake, null,
                                    ctypes.c_void_p(0x1004), 1 << 20, fake, null)
    assert rc == -2
    # gather attention
    g = lambda q, D, dt: (q, i64x4, fake, i64x4, fake, i64x4, dt, fake, i64x3, fake, i64x3, fake, i64x3, fake, i64x4,
                          0, 1, 1, 8, 8, D, 4, 1, fake, null)
    assert L.swv_dsa_attn_gather_fwd(*g(null, 64, 0)) == -1
    assert L.swv_dsa_attn_gather_fwd(*g(fake, 0, 0)) == -8
    assert L.swv_dsa_attn_gather_fwd(*g(fake, 64, 9)) == -3
    # block-sparse attention: block size, head dim, mode, GQA divisibility
    bs = lambda block, D, mode, grp: (fake, ok_strides, fake, ok_strides, fake, ok_strides, fake, fake, block, mode, 0,
                                      0, 1, grp, null, fake, ok_strides, 0, 1, 4, 8, 8, D, fake, null)
    ok_strides = (ctypes.c_int64 * 4)(4096, 512, 64, 1)
    assert L.swv_block_sparse_attn_fwd(*bs(32, 64, 0, 1)) == -8
    assert L.swv_block_sparse_attn_fwd(*bs(64, 96, 0, 1)) == -8
    assert L.swv_block_sparse_attn_fwd(*bs(64, 64, 2, 1)) == -8
    assert L.swv_block_sparse_attn_fwd(*bs(64, 64, 0, 3)) == -4
    # dense path: only head_dim 64, unit inner stride, 16-byte aligned rows
    m = lambda D, qs: (fake, qs, fake, i64x4, fake, i64x4, fake, fake, fake, i64x4, 0, 1, 1, 8, 8, D, null, 0, fake,
                       null)
    ok_strides = (ctypes.c_int64 * 4)(4096, 512, 64, 1)
    assert L.swv_dsa_attn_masked_fwd(*m(128, ok_strides)) == -8
    assert L.swv_dsa_attn_masked_fwd(*m(64, (ctypes.c_int64 * 4)(4096, 512, 64, 2))) == -2
    assert L.swv_dsa_attn_masked_fwd(*m(64, (ctypes.c_int64 * 4)(4096, 512, 63, 1))) == -2
    # list-driven attention: required pointers, top_k a multiple of 4, head dim 64, scratch large enough
    ls = lambda q_, D, K, scr, nscr: (q_, ok_strides, fake, ok_strides, fake, ok_strides, fake, fake, K, fake, fake, fake,
                                      ok_strides, 0, 1, 2, 256, 256, D, scr, nscr, fake, null)
    n = ctypes.c_size_t()
    assert L.swv_dsa_attn_lists_scratch_bytes(1, 2, 256, 256, 64, ctypes.byref(n)) == 0 and n.value > 0
    assert L.swv_dsa_attn_lists_scratch_bytes(1, 2, 0, 256, 64, ctypes.byref(n)) == -4
    assert L.swv_dsa_attn_lists_fwd(*ls(null, 64, 64, fake, 1 << 30)) == -1
    assert L.swv_dsa_attn_lists_fwd(*ls(fake, 64, 64, null, 1 << 30)) == -1
    assert L.swv_dsa_attn_lists_fwd(*ls(fake, 64, 66, fake, 1 << 30)) == -8
    assert L.swv_dsa_attn_lists_fwd(*ls(fake, 128, 64, fake, 1 << 30)) == -8
    assert L.swv_dsa_attn_lists_fwd(*ls(fake, 64, 64, ctypes.c_void_p(0x1000), 16)) == -5


def test_ops_refuse_cpu_tensors(swv):
    q = torch.zeros(1, 4, 2, 8)
    with pytest.raises(swv._lib.SwvError):
        swv.dsa_indexer_topk(q, q, torch.ones(2), 2)
    with pytest.raises(swv._lib.SwvError):
        swv.dsa_sparse_attention(torch.zeros(1, 1, 4, 64), torch.zeros(1, 1, 4, 64), torch.zeros(1, 1, 4, 64), q, q,
                                 torch.ones(2), 2)


def test_product_code_never_touches_the_oracle():
    pkg = os.path.join(ROOT, "sparse_wsi_vit_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "from oracle" not in text and "import oracle" not in text, f


def test_modules_keep_reference_parameter_names(swv, golden_dir):
    g = np.load(os.path.join(golden_dir, "dsa_module_reference.npz"))
    ref_keys = sorted(k[3:] for k in g.files if k.startswith("sd."))
    m = swv.DeepSeekSparseAttention(d_model=64, attention_heads=2, indexer_heads=4, indexer_dim=16, top_k=16,
                                    BLOCK_Q=16, BLOCK_K=16, BLOCK_D=16)
    assert sorted(m.state_dict().keys()) == ref_keys
    for k in ref_keys:
        assert tuple(m.state_dict()[k].shape) == tuple(g["sd." + k].shape)
    enc = swv.DSAViTSlideEncoder(in_features=32, out_features=2, embed_dim=64, num_heads=1, num_layers=2, num_cls=2,
                                 indexer_heads=2, indexer_dim=16, top_k=8)
    keys = set(enc.state_dict().keys())
    for k in ["cls_tokens", "input_proj.weight", "blocks.0.norm1.weight", "blocks.1.attn.indexer_head_weights",
              "blocks.0.attn.indexer_proj.q_proj.bias", "blocks.0.attn.qkv_proj.weight", "blocks.0.attn.out_proj.bias",
              "blocks.0.mlp.0.weight", "blocks.0.mlp.3.bias", "norm.weight", "cls_pool.weight", "head.bias"]:
        assert k in keys, k
    with pytest.raises(ValueError):
        swv.DSAViTSlideEncoder(embed_dim=100, num_heads=3)


def test_backward_has_no_cpu_path(swv):
    """The backward operators are CUDA kernels like the forward ones: CPU tensors are refused."""
    z = torch.zeros(1, 4, 2, 8)
    i = torch.zeros(1, 4, 2, dtype=torch.int32)
    f = torch.zeros(1, 4, 2)
    with pytest.raises(swv._lib.SwvError):
        swv.ops.dsa_indexer_bwd(f, z, z, torch.ones(2), i, f)
    with pytest.raises(swv._lib.SwvError):
        swv.ops.dsa_attention_bwd(z.transpose(1, 2), z.transpose(1, 2), z.transpose(1, 2), z.transpose(1, 2),
                                  z.transpose(1, 2), i, f, f)
