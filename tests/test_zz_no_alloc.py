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


def _call_static(lib, qi, ki, w, top_k, dev, want_mask=False):
    import sparse_wsi_vit_b200 as swv
    B, Tq, IH, ID = qi.shape
    Tk = ki.shape[1]
    idx = torch.full((B, Tq, top_k), -7, dtype=torch.int32, device=dev)
    valid = torch.full((B, Tq, top_k), -7.0, device=dev)
    scores = torch.full((B, Tq, top_k), -7.0, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    mask = torch.zeros(swv.ops.mask_bytes(B, Tq, Tk) // 4, dtype=torch.int32, device=dev) if want_mask else None
    i64 = lambda t: (ctypes.c_int64 * 4)(*t.stride())
    # everything the call may touch exists now: device memory must not move during the call
    torch.cuda.synchronize(dev)
    free_before = torch.cuda.mem_get_info(dev)[0]
    rc = lib.swv_dsa_indexer_topk_static_fwd(
        qi.data_ptr(), i64(qi), ki.data_ptr(), i64(ki), swv._lib.dtype_code(qi.dtype), w.data_ptr(), B, Tq, Tk, IH, ID,
        top_k, idx.data_ptr(), valid.data_ptr(), scores.data_ptr(), mask.data_ptr() if want_mask else None,
        status.data_ptr(), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    torch.cuda.synchronize(dev)
    free_after = torch.cuda.mem_get_info(dev)[0]
    return rc, idx, valid, scores, status, mask, free_before - free_after


def _inputs(B, Tq, Tk, seed, dtype, dev):
    g = torch.Generator().manual_seed(seed)
    qi = (torch.randn(B, Tq, 4, 64, generator=g) / 8).to(dtype).to(dev)
    ki = (torch.randn(B, Tk, 4, 64, generator=g) / 8).to(dtype).to(dev)
    w = torch.randn(4, generator=g).to(dev)
    return qi, ki, w


def test_static_scratch_entry_matches_regular_entry_twice():
    """Consecutive calls of different sizes (the third smaller than the second: stale words of a
    larger earlier call must not be read), a batch of 3 with more keys than queries in bf16, the
    membership bitmask, and a call at the capacity edge."""
    import sparse_wsi_vit_b200 as swv
    lib = swv._lib.lib
    dev = torch.device("cuda:0")
    cases = [(1, 700, 700, 64, torch.float32, False), (1, 1333, 1333, 256, torch.float32, False),
             (1, 300, 300, 32, torch.float32, True), (3, 500, 2100, 128, torch.bfloat16, True),
             (1, 8192, 8192, 64, torch.bfloat16, False), (1, 40, 40, 64, torch.float32, False),
             (64, 3, 50, 8, torch.float32, False)]
    for call, (B, Tq, Tk, K, dtype, want_mask) in enumerate(cases):
        qi, ki, w = _inputs(B, Tq, Tk, call + 1, dtype, dev)
        rc, idx, valid, scores, status, mask, grew = _call_static(lib, qi, ki, w, K, dev, want_mask)
        assert rc == 0, swv._lib.strerror(rc)
        assert int(status.item()) == 0
        assert grew == 0, f"call {call}: {grew} bytes of device memory were taken during the call"
        if want_mask:
            ridx, rvalid, rscores, (rmask, _) = swv.dsa_indexer_topk(qi, ki, w, K, want_mask=True,
                                                                      mask=torch.zeros_like(mask))
            assert torch.equal(mask, rmask), f"call {call}: membership bitmask differs"
        else:
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
    # the limit is on tokens, however they are split into batches: 4096 sequences of 2 tokens fit
    qs = torch.zeros(4096, 2, 1, 64, device=dev)
    rc, idx, valid, *_ = _call_static(lib, qs, qs, w, 2, dev)
    assert rc == 0 and bool((valid == 1).all())
