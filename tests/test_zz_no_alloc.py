"""The workspace-free indexer entry point, called through the C ABI.

Some hosts of this operator cannot give it scratch memory: a serving runtime or plug-in host that
plans every device buffer itself and passes the operator only its inputs and outputs, or a
latency-critical loop that must not trigger an allocation.  For them the library carries a fixed
scratch array in its own device data segment (8192 tokens at most).  This test drives that entry
point directly with ctypes and requires the same idx / valid / scores as the regular entry point,
bit for bit, on two consecutive calls with different inputs (the array keeps the first call's
contents, which must not leak into the second).  Collected last on purpose.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, qi, ki, w, top_k, dev):
    B, Tq, IH, ID = qi.shape
    Tk = ki.shape[1]
    idx = torch.full((B, Tq, top_k), -7, dtype=torch.int32, device=dev)
    valid = torch.full((B, Tq, top_k), -7.0, device=dev)
    scores = torch.full((B, Tq, top_k), -7.0, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    i64 = lambda t: (ctypes.c_int64 * 4)(*t.stride())
    rc = lib.swv_dsa_indexer_topk_static_fwd(
        qi.data_ptr(), i64(qi), ki.data_ptr(), i64(ki), 0, w.data_ptr(), B, Tq, Tk, IH, ID, top_k,
        idx.data_ptr(), valid.data_ptr(), scores.data_ptr(), None, status.data_ptr(),
        ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    return rc, idx, valid, scores, status


def test_static_scratch_entry_matches_regular_entry_twice():
    import sparse_wsi_vit_b200 as swv
    lib = swv._lib.lib
    dev = torch.device("cuda:0")
    for call, (T, K, seed) in enumerate([(700, 64, 1), (1333, 256, 2)]):
        g = torch.Generator().manual_seed(seed)
        qi = (torch.randn(1, T, 4, 64, generator=g) / 8).to(dev)
        ki = (torch.randn(1, T, 4, 64, generator=g) / 8).to(dev)
        w = torch.randn(4, generator=g).to(dev)
        rc, idx, valid, scores, status = _call_static(lib, qi, ki, w, K, dev)
        assert rc == 0, swv._lib.strerror(rc)
        torch.cuda.synchronize(dev)
        assert int(status.item()) == 0
        ridx, rvalid, rscores = swv.dsa_indexer_topk(qi, ki, w, K)
        swv.check_status(dev)
        assert torch.equal(idx, ridx), f"call {call}: indices differ"
        assert torch.equal(valid, rvalid), f"call {call}: valid differs"
        assert torch.equal(scores, rscores), f"call {call}: scores differ"


def test_static_scratch_entry_rejects_sizes_beyond_its_capacity():
    import sparse_wsi_vit_b200 as swv
    lib = swv._lib.lib
    dev = torch.device("cuda:0")
    T = 8193
    qi = torch.zeros(1, T, 1, 64, device=dev)
    w = torch.ones(1, device=dev)
    rc, idx, *_ = _call_static(lib, qi, qi, w, 8, dev)
    assert rc == -9 and "capacity" in swv._lib.strerror(rc)
    torch.cuda.synchronize(dev)
    assert bool((idx == -7).all()), "a rejected call must not launch anything"
