"""Operator layer: the reference's two autograd.Function signatures backed by
the sm_100a kernels, plus the fused module-level forward.

Mirrors  src/sparse_wsi_vit/models/deepseek_sparse_attention_kernels/kernels.py
  LightningIndexerFunction (kernels.py:344-386)   -> swv_dsa_indexer_topk_fwd
  DSAAttentionFunction     (kernels.py:767-810)   -> swv_dsa_attn_gather_fwd
and the op sequence of DeepSeekSparseAttention.forward
  (src/sparse_wsi_vit/models/deepseek_sparse_attention.py:59-85) -> dsa_sparse_attention.

Forward and backward.  All work runs on the current CUDA stream of the inputs' device.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib
from ._lib import SwvError, check, dtype_code, lib, strides

_scratch: dict = {}
_status: dict = {}
_CHECK = os.environ.get("SWV_CHECK_STATUS", "0") == "1"


def _require_cuda(*ts):
    for t in ts:
        if not t.is_cuda:
            raise SwvError("sparse_wsi_vit_b200 ops run on CUDA tensors only (no CPU path)")


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def status_word(dev) -> torch.Tensor:
    """Per-device int32 the kernels report bounded-wait failures into."""
    key = dev.index
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _status[key]


def check_status(dev, what="kernel"):
    """Synchronising read of the device status word; raises on a device-side error."""
    st = status_word(dev)
    code = int(st.item())
    if code != 0:
        st.zero_()
        raise SwvError(f"{what}: {_lib.strerror(code)} (device status {code})")


def _buffer(kind, dev, nbytes):
    key = (kind, dev.index)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(int(nbytes), dtype=torch.uint8, device=dev)
        _scratch[key] = buf
    return buf


def workspace_bytes(B, Tq, Tk, top_k=None):
    """Bytes of indexer workspace; with ``top_k`` the size that also lets a sparse selection on a long
    key range take the two-sweep form (room for per-row candidate lists)."""
    n = ctypes.c_size_t()
    if top_k is None:
        check(lib.swv_dsa_workspace_bytes(B, Tq, Tk, ctypes.byref(n)), "swv_dsa_workspace_bytes")
    else:
        check(lib.swv_dsa_workspace_bytes_topk(B, Tq, Tk, top_k, ctypes.byref(n)), "swv_dsa_workspace_bytes_topk")
    return n.value


def mask_bytes(B, Tq, Tk):
    n = ctypes.c_size_t()
    check(lib.swv_dsa_mask_bytes(B, Tq, Tk, ctypes.byref(n)), "swv_dsa_mask_bytes")
    return n.value


def dsa_prologue(qkv_q, qkv_k, q_idx, k_idx, w, coords=None, coord_high=1.0, theta=10000.0, skip_tokens=0,
                 top_k=None):
    """Token-local prologue in one launch: optional in-place 2-D RoPE of q and k (TOKEN-major
    (B,T,H,D) views of the projection output; ``coords`` (B,T,2) or (T,2), one row per token) and the
    indexer head collapse.  Returns the indexer workspace holding the collapsed vectors; pass it to
    ``dsa_indexer_topk(..., workspace=ws, precollapsed=True)``.  ``top_k``: size the workspace for an
    indexer call with that many keys per query (see ``workspace_bytes``)."""
    _require_cuda(q_idx, k_idx, w)
    B, T, IH, ID = q_idx.shape
    if k_idx.shape != q_idx.shape:
        raise SwvError("the prologue needs as many keys as queries (self-attention layer)")
    if k_idx.dtype != q_idx.dtype:
        k_idx = k_idx.to(q_idx.dtype)
    dev = q_idx.device
    ws = torch.empty(workspace_bytes(B, T, T, top_k), dtype=torch.uint8, device=dev)
    w32 = w.detach().to(torch.float32).contiguous()
    cptr, qp, kp, qs, ks, qdt, H, D = None, None, None, None, None, 0, 1, 4
    if coords is not None:
        _require_cuda(qkv_q, qkv_k, coords)
        if qkv_q.dtype != qkv_k.dtype or qkv_q.stride(-1) != 1 or qkv_k.stride(-1) != 1:
            raise SwvError("q and k must share a dtype and have unit inner stride")
        H, D = qkv_q.shape[2], qkv_q.shape[3]
        c = coords.reshape(-1, T, 2).to(torch.float32)
        c = (c.expand(B, T, 2) if c.shape[0] == 1 else c).contiguous()
        cptr, qp, kp, qs, ks, qdt = c.data_ptr(), qkv_q.data_ptr(), qkv_k.data_ptr(), strides(qkv_q), strides(qkv_k), \
            dtype_code(qkv_q.dtype)
    rc = lib.swv_dsa_prologue_fwd(qp, qs, kp, ks, qdt, q_idx.data_ptr(), strides(q_idx), k_idx.data_ptr(),
                                  strides(k_idx), dtype_code(q_idx.dtype), w32.data_ptr(), cptr, float(coord_high),
                                  float(theta), int(skip_tokens), B, T, H, D, IH, ID, ws.data_ptr(), ws.numel(),
                                  _stream(dev))
    check(rc, "swv_dsa_prologue_fwd")
    return ws


def dsa_indexer_topk(q_idx, k_idx, w, top_k, want_mask=False, out=None, mask=None, workspace=None,
                     precollapsed=False):
    """q_idx (B,Tq,IH,ID), k_idx (B,Tk,IH,ID), w (IH,) -> idx int32, valid f32, scores f32,
    each (B,Tq,top_k), keys in ascending order.  With `want_mask` also the selection handle
    ``(bitmask, workspace)`` that ``dsa_attention_masked`` consumes; it owns both buffers, so it
    stays valid across later indexer calls.  ``workspace`` + ``precollapsed``: the workspace
    ``dsa_prologue`` returned (the collapse step is then skipped; q_idx / k_idx give the shapes)."""
    _require_cuda(q_idx, k_idx, w)
    if q_idx.dim() != 4 or k_idx.dim() != 4:
        raise SwvError("indexer projections must be (B, T, IH, ID)")
    B, Tq, IH, ID = q_idx.shape
    Tk = k_idx.shape[1]
    if k_idx.shape[0] != B or k_idx.shape[2] != IH or k_idx.shape[3] != ID or w.numel() != IH:
        raise SwvError("indexer shape mismatch")
    if k_idx.dtype != q_idx.dtype:
        k_idx = k_idx.to(q_idx.dtype)
    dev = q_idx.device
    w32 = w.detach().to(torch.float32).contiguous()
    if out is None:
        idx = torch.empty((B, Tq, top_k), dtype=torch.int32, device=dev)
        valid = torch.empty((B, Tq, top_k), dtype=torch.float32, device=dev)
        scores = torch.empty((B, Tq, top_k), dtype=torch.float32, device=dev)
    else:
        idx, valid, scores = out
    nws = workspace_bytes(B, Tq, Tk, top_k)
    # a selection handle keeps its own workspace (the attention reads it); plain calls share one
    if workspace is not None:
        ws = workspace
    else:
        ws = torch.empty(nws, dtype=torch.uint8, device=dev) if want_mask else _buffer("ws", dev, nws)
    mptr = None
    if want_mask:
        if mask is None:
            mask = torch.empty(mask_bytes(B, Tq, Tk) // 4, dtype=torch.int32, device=dev)
        mptr = mask.data_ptr()
    st = status_word(dev)
    rc = lib.swv_dsa_indexer_topk_fwd(
        None if precollapsed else q_idx.data_ptr(), strides(q_idx), None if precollapsed else k_idx.data_ptr(),
        strides(k_idx), dtype_code(q_idx.dtype),
        w32.data_ptr(), B, Tq, Tk, IH, ID, top_k, idx.data_ptr(), valid.data_ptr(), scores.data_ptr(), mptr,
        ws.data_ptr(), ws.numel(), st.data_ptr(), _stream(dev))
    check(rc, "swv_dsa_indexer_topk_fwd")
    if _CHECK:
        check_status(dev, "swv_dsa_indexer_topk_fwd")
    return (idx, valid, scores, (mask, ws)) if want_mask else (idx, valid, scores)


def dsa_attention_gather(q, k, v, idx, valid, rw, o, kv_group=1):
    """Routing-weighted attention over explicit key lists; writes ``o`` in place.
    kv_group > 1: k, v have H/kv_group heads (grouped-query attention)."""
    _require_cuda(q, k, v, idx, valid, rw, o)
    B, H, Tq, D = q.shape
    Tk = k.shape[2]
    top_k = idx.shape[-1]
    if k.dtype != q.dtype or v.dtype != q.dtype:
        k, v = k.to(q.dtype), v.to(q.dtype)
    if idx.dtype != torch.int32:
        idx = idx.to(torch.int32)
    valid = valid.to(torch.float32)
    rw = rw.detach().to(torch.float32)
    dev = q.device
    st = status_word(dev)
    rc = lib.swv_dsa_attn_gather_fwd(
        q.data_ptr(), strides(q), k.data_ptr(), strides(k), v.data_ptr(), strides(v), dtype_code(q.dtype),
        idx.data_ptr(), strides(idx), valid.data_ptr(), strides(valid), rw.data_ptr(), strides(rw),
        o.data_ptr(), strides(o), dtype_code(o.dtype), B, H, Tq, Tk, D, top_k, kv_group, st.data_ptr(),
        _stream(dev))
    check(rc, "swv_dsa_attn_gather_fwd")
    return o


def _tma_ok(t):
    es = t.element_size()
    return (t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and
            all((s * es) % 16 == 0 for s in t.stride()[:-1]))


def dsa_attention_masked(q, k, v, selection, o):
    """Dense tensor-core sweep over all key tiles; `selection` is the (bitmask, workspace)
    pair returned by ``dsa_indexer_topk(..., want_mask=True)`` for the same queries and keys."""
    mask, ws = selection
    _require_cuda(q, k, v, mask, ws, o)
    B, H, Tq, D = q.shape
    Tk = k.shape[2]
    if q.dtype != torch.bfloat16 or D != 64:
        raise SwvError("dsa_attention_masked needs bf16 q/k/v with head_dim 64")
    q, k, v = (t if _tma_ok(t) else t.contiguous() for t in (q, k, v))
    dev = q.device
    st = status_word(dev)
    nscr = ctypes.c_size_t()
    check(lib.swv_dsa_attn_scratch_bytes(B, H, Tq, Tk, ctypes.byref(nscr)), "swv_dsa_attn_scratch_bytes")
    scr = _buffer("attn_scratch", dev, nscr.value) if nscr.value else None
    rc = lib.swv_dsa_attn_masked_fwd(
        q.data_ptr(), strides(q), k.data_ptr(), strides(k), v.data_ptr(), strides(v), mask.data_ptr(),
        ws.data_ptr(), o.data_ptr(), strides(o), dtype_code(o.dtype), B, H, Tq, Tk, D,
        scr.data_ptr() if scr is not None else None, nscr.value, st.data_ptr(), _stream(dev))
    check(rc, "swv_dsa_attn_masked_fwd")
    if _CHECK:
        check_status(dev, "swv_dsa_attn_masked_fwd")
    return o


def dsa_attention_lists(q, k, v, idx, rw, selection, o):
    """The same attention as ``dsa_attention_masked`` driven by the indexer's key lists:
    dense tensor-core tiles, one exponential per SELECTED key (``idx``, ``rw`` (B,Tq,top_k) as
    ``dsa_indexer_topk`` returns them, ``rw = scores * valid``); `selection` as for
    ``dsa_attention_masked`` (used for the few tiles whose logits cannot be bounded)."""
    mask, ws = selection
    _require_cuda(q, k, v, idx, rw, mask, ws, o)
    B, H, Tq, D = q.shape
    Tk = k.shape[2]
    top_k = idx.shape[-1]
    if q.dtype != torch.bfloat16 or D != 64 or top_k % 4:
        raise SwvError("dsa_attention_lists needs bf16 q/k/v with head_dim 64 and top_k a multiple of 4")
    if idx.dtype != torch.int32 or rw.dtype != torch.float32 or not idx.is_contiguous() or not rw.is_contiguous():
        raise SwvError("dsa_attention_lists needs contiguous int32 idx and fp32 rw")
    q, k, v = (t if _tma_ok(t) else t.contiguous() for t in (q, k, v))
    dev = q.device
    st = status_word(dev)
    nscr = ctypes.c_size_t()
    check(lib.swv_dsa_attn_lists_scratch_bytes(B, H, Tq, Tk, top_k, ctypes.byref(nscr)),
          "swv_dsa_attn_lists_scratch_bytes")
    scr = _buffer("attn_lists_scratch", dev, nscr.value)
    rc = lib.swv_dsa_attn_lists_fwd(
        q.data_ptr(), strides(q), k.data_ptr(), strides(k), v.data_ptr(), strides(v), idx.data_ptr(), rw.data_ptr(),
        top_k, mask.data_ptr(), ws.data_ptr(), o.data_ptr(), strides(o), dtype_code(o.dtype), B, H, Tq, Tk, D,
        scr.data_ptr(), nscr.value, st.data_ptr(), _stream(dev))
    check(rc, "swv_dsa_attn_lists_fwd")
    if _CHECK:
        check_status(dev, "swv_dsa_attn_lists_fwd")
    return o


# The list-driven kernel does a constant amount of work per (query tile, key tile) plus a little per
# selected key (three list entries per thread and tile are held in registers), the dense sweep one
# exponential per (query, key, head).  Measured on B200 (8 heads, top-2048): the lists win at 65536
# tokens (one key in 32: 9.5 + 0.8 ms against 13.1-14.5 ms) and lose at 32768 (one in 16).
LISTS_MAX_DENSITY = 1.0 / 24.0
# The tile lists take (Tq / 128) * (Tk / 128) * capacity * 8 bytes (1.6 GB at 65536 tokens, 9.7 GB at
# 262144); beyond this the fused path stays with the dense sweep.
LISTS_MAX_SCRATCH_BYTES = 16 << 30


def dsa_attention_dense(q, k, v, idx, scores, selection, o):
    """The attention step of the fused path on the tensor cores: the list-driven kernel
    (``dsa_attention_lists``) for sparse selections, the dense sweep (``dsa_attention_masked``)
    otherwise.  ``idx`` / ``scores`` / ``selection`` as ``dsa_indexer_topk(..., want_mask=True)``
    returns them (slots beyond min(top_k, Tk) are ignored, so ``scores`` serve as routing weights)."""
    B, H, Tq, _ = q.shape
    Tk = k.shape[2]
    top_k = idx.shape[-1]
    if top_k % 4 == 0 and min(top_k, Tk) <= LISTS_MAX_DENSITY * Tk and os.environ.get("SWV_DSA_ATTN", "") != "sweep":
        nscr = ctypes.c_size_t()
        check(lib.swv_dsa_attn_lists_scratch_bytes(B, H, Tq, Tk, top_k, ctypes.byref(nscr)),
              "swv_dsa_attn_lists_scratch_bytes")
        if nscr.value <= LISTS_MAX_SCRATCH_BYTES:
            return dsa_attention_lists(q, k, v, idx, scores, selection, o)
    return dsa_attention_masked(q, k, v, selection, o)


def dsa_attention_masked_count(q, k, v, selection, o):
    """Diagnostic: ``dsa_attention_masked`` (unsplit) that also returns, per query row, how many keys
    the kernel treated as selected, int32 (B, Tq); must equal min(top_k, Tk) everywhere."""
    mask, ws = selection
    _require_cuda(q, k, v, mask, ws, o)
    B, H, Tq, D = q.shape
    Tk = k.shape[2]
    if q.dtype != torch.bfloat16 or D != 64:
        raise SwvError("dsa_attention_masked needs bf16 q/k/v with head_dim 64")
    q, k, v = (t if _tma_ok(t) else t.contiguous() for t in (q, k, v))
    dev = q.device
    cnt = torch.empty((B, Tq), dtype=torch.int32, device=dev)
    rc = lib.swv_dsa_attn_masked_count_fwd(
        q.data_ptr(), strides(q), k.data_ptr(), strides(k), v.data_ptr(), strides(v), mask.data_ptr(),
        ws.data_ptr(), o.data_ptr(), strides(o), dtype_code(o.dtype), B, H, Tq, Tk, D, cnt.data_ptr(),
        status_word(dev).data_ptr(), _stream(dev))
    check(rc, "swv_dsa_attn_masked_count_fwd")
    return cnt


def dsa_sparse_attention(q, k, v, q_idx, k_idx, w, top_k, out_dtype=None, return_topk=False, kv_ready=None,
                         rope=None):
    """Indexer + top-k + routing-weighted attention (deepseek_sparse_attention.py:59-85).

    ``rope`` = (coords (T,2) or (B,T,2) with one row per token, coord_high, theta, skip_tokens): q and k
    (views of the projection output, rotated IN PLACE) get the 2-D rotary embedding first, in the same
    launch that collapses the indexer heads (``dsa_prologue``).

    q (B,H,Tq,D), k, v (B,H,Tk,D); q_idx (B,Tq,IH,ID), k_idx (B,Tk,IH,ID); w (IH,).
    bf16 with D == 64 takes the dense tensor-core path; anything else the gather
    kernel.  Both are CUDA kernels of this library.  `kv_ready` is an optional CUDA
    event after which k and v are complete (they may still be in flight on another
    stream while the indexer runs, which needs only q_idx / k_idx).
    """
    B, H, Tq, D = q.shape
    dev = q.device
    out_dtype = out_dtype or q.dtype
    o = torch.empty((B, H, Tq, D), dtype=out_dtype, device=dev)
    dense = q.dtype == torch.bfloat16 and D == 64
    ws, pre = None, False
    if rope is not None or (dense and q_idx.shape == k_idx.shape and kv_ready is None):
        # one launch for the token-local steps between the projections and the indexer
        coords, coord_high, theta, skip = rope if rope is not None else (None, 1.0, 10000.0, 0)
        ws = dsa_prologue(q.transpose(1, 2), k.transpose(1, 2), q_idx, k_idx, w, coords, coord_high, theta, skip,
                          top_k=top_k)
        pre = True
    if dense:
        idx, valid, scores, sel = dsa_indexer_topk(q_idx, k_idx, w, top_k, want_mask=True, workspace=ws,
                                                   precollapsed=pre)
        if kv_ready is not None:
            torch.cuda.current_stream(dev).wait_event(kv_ready)
        dsa_attention_dense(q, k, v, idx, scores, sel, o)
    else:
        idx, valid, scores = dsa_indexer_topk(q_idx, k_idx, w, top_k, workspace=ws, precollapsed=pre)
        if kv_ready is not None:
            torch.cuda.current_stream(dev).wait_event(kv_ready)
        dsa_attention_gather(q, k, v, idx, valid, scores * valid, o)
    return (o, idx, valid, scores) if return_topk else o


def dsa_attention_bwd(d_out, q, k, v, o, idx, valid, rw):
    """Gradients of the routing-weighted attention (kernels.py:569-762): returns fp32
    ``dq (B,H,Tq,D), dk, dv (B,H,Tk,D), drw (B,Tq,top_k)``."""
    _require_cuda(d_out, q, k, v, o, idx, valid, rw)
    B, H, Tq, D = q.shape
    Tk = k.shape[2]
    top_k = idx.shape[-1]
    if k.dtype != q.dtype or v.dtype != q.dtype:
        k, v = k.to(q.dtype), v.to(q.dtype)
    k = k if k.stride(-1) == 1 else k.contiguous()
    v = v if v.stride(-1) == 1 else v.contiguous()
    d_out = d_out if d_out.dtype == o.dtype else d_out.to(o.dtype)
    idx = idx if idx.dtype == torch.int32 else idx.to(torch.int32)
    valid, rw = valid.to(torch.float32), rw.detach().to(torch.float32)
    dev = q.device
    dq = torch.empty((B, H, Tq, D), dtype=torch.float32, device=dev)
    dk = torch.empty((B, H, Tk, D), dtype=torch.float32, device=dev)
    dv = torch.empty((B, H, Tk, D), dtype=torch.float32, device=dev)
    drw = torch.empty((B, Tq, top_k), dtype=torch.float32, device=dev)
    rc = lib.swv_dsa_attn_bwd(
        d_out.data_ptr(), strides(d_out), q.data_ptr(), strides(q), k.data_ptr(), strides(k), v.data_ptr(), strides(v),
        dtype_code(q.dtype), o.data_ptr(), strides(o), dtype_code(o.dtype), idx.data_ptr(), strides(idx),
        valid.data_ptr(), strides(valid), rw.data_ptr(), strides(rw), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
        drw.data_ptr(), B, H, Tq, Tk, D, top_k, status_word(dev).data_ptr(), _stream(dev))
    check(rc, "swv_dsa_attn_bwd")
    if _CHECK:
        check_status(dev, "swv_dsa_attn_bwd")
    return dq, dk, dv, drw


def dsa_indexer_bwd(d_scores, q_idx, k_idx, w, idx, valid):
    """Gradients of the indexer as the reference's backward defines them (kernels.py:128-339): returns
    fp32 ``dq_idx (B,Tq,IH,ID), dk_idx (B,Tk,IH,ID), dw (IH,)``."""
    _require_cuda(d_scores, q_idx, k_idx, w, idx, valid)
    B, Tq, IH, ID = q_idx.shape
    Tk = k_idx.shape[1]
    top_k = idx.shape[-1]
    if k_idx.dtype != q_idx.dtype:
        k_idx = k_idx.to(q_idx.dtype)
    d_scores = d_scores.to(torch.float32)
    idx = idx if idx.dtype == torch.int32 else idx.to(torch.int32)
    valid = valid.to(torch.float32)
    w32 = w.detach().to(torch.float32).contiguous()
    dev = q_idx.device
    dq = torch.empty((B, Tq, IH, ID), dtype=torch.float32, device=dev)
    dk = torch.empty((B, Tk, IH, ID), dtype=torch.float32, device=dev)
    dw = torch.empty((IH,), dtype=torch.float32, device=dev)
    rc = lib.swv_dsa_indexer_bwd(
        d_scores.data_ptr(), strides(d_scores), q_idx.data_ptr(), strides(q_idx), k_idx.data_ptr(), strides(k_idx),
        dtype_code(q_idx.dtype), w32.data_ptr(), idx.data_ptr(), strides(idx), valid.data_ptr(), strides(valid),
        dq.data_ptr(), dk.data_ptr(), dw.data_ptr(), B, Tq, Tk, IH, ID, top_k, status_word(dev).data_ptr(),
        _stream(dev))
    check(rc, "swv_dsa_indexer_bwd")
    if _CHECK:
        check_status(dev, "swv_dsa_indexer_bwd")
    return dq, dk, dw


class LightningIndexerFunction(torch.autograd.Function):
    """Same positional signature as the reference (kernels.py:346-352).  The tile
    sizes are accepted and ignored; outputs are allocated here (kernels.py:355-357)."""

    @staticmethod
    def forward(ctx, q_proj, k_proj, W, B, T, H, D, TOP_K, BLOCK_Q=None, BLOCK_K=None, BLOCK_D=None,
                BLOCK_INDEXER_H=None):
        if tuple(q_proj.shape) != (B, T, H, D):
            raise SwvError(f"q_proj has shape {tuple(q_proj.shape)}, expected {(B, T, H, D)}")
        idx, valid, scores = dsa_indexer_topk(q_proj.detach(), k_proj.detach(), W.detach(), TOP_K)
        ctx.mark_non_differentiable(idx, valid)
        ctx.save_for_backward(q_proj, k_proj, W, idx, valid)
        return idx, valid, scores

    @staticmethod
    def backward(ctx, d_idx, d_valid, d_scores):
        """kernels.py:388-445: gradients for q_proj, k_proj, W; none for the sizes and tile arguments."""
        q_proj, k_proj, W, idx, valid = ctx.saved_tensors
        if d_scores is None:
            d_scores = torch.zeros_like(valid)
        dq, dk, dw = dsa_indexer_bwd(d_scores, q_proj, k_proj, W, idx, valid)
        return (dq.to(q_proj.dtype), dk.to(k_proj.dtype), dw.to(W.dtype)) + (None,) * 9


class DSAAttentionFunction(torch.autograd.Function):
    """Same positional signature as the reference (kernels.py:769-775): the caller
    owns ``o``; it is written in place and returned (kernels.py:810)."""

    @staticmethod
    def forward(ctx, q, k, v, idx, valid, routing_weights, o, B, H, T, D, TOP_K, BLOCK_Q=None, BLOCK_K=None,
                BLOCK_ATTENTION_H=None, BLOCK_D=None):
        if tuple(q.shape) != (B, H, T, D):
            raise SwvError(f"q has shape {tuple(q.shape)}, expected {(B, H, T, D)}")
        dsa_attention_gather(q.detach(), k.detach(), v.detach(), idx, valid, routing_weights.detach(), o)
        ctx.mark_dirty(o)
        ctx.save_for_backward(q, k, v, idx, valid, routing_weights, o)
        return o

    @staticmethod
    def backward(ctx, d_out):
        """kernels.py:812-853: gradients for q, k, v and the routing weights."""
        q, k, v, idx, valid, rw, o = ctx.saved_tensors
        dq, dk, dv, drw = dsa_attention_bwd(d_out, q, k, v, o, idx, valid, rw)
        return (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None, drw.to(rw.dtype), None) + (None,) * 9


class DSAModuleFunction(torch.autograd.Function):
    """The module's whole attention step as ONE differentiable op: the forward is the fused path
    (indexer + top-k + dense tensor-core attention, ``dsa_sparse_attention``), the backward chains
    the two backward kernels the way autograd chains the reference's two Functions through
    ``routing_weights = scores * valid`` (deepseek_sparse_attention.py:63-85)."""

    @staticmethod
    def forward(ctx, q, k, v, q_idx, k_idx, w, top_k, out_dtype):
        o, idx, valid, scores = dsa_sparse_attention(q.detach(), k.detach(), v.detach(), q_idx.detach(),
                                                     k_idx.detach(), w.detach(), top_k, out_dtype=out_dtype,
                                                     return_topk=True)
        ctx.save_for_backward(q, k, v, q_idx, k_idx, w, idx, valid, scores, o)
        return o

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, q_idx, k_idx, w, idx, valid, scores, o = ctx.saved_tensors
        dq, dk, dv, drw = dsa_attention_bwd(d_out.contiguous(), q, k, v, o, idx, valid, scores * valid)
        # d scores = d rw * valid; the indexer backward multiplies by valid itself (valid is 0 or 1)
        dqi, dki, dw = dsa_indexer_bwd(drw, q_idx, k_idx, w, idx, valid)
        return (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dqi.to(q_idx.dtype), dki.to(k_idx.dtype),
                dw.to(w.dtype), None, None)


class Rope2dFunction(torch.autograd.Function):
    """``rope2d`` with its gradient: the rotation is orthogonal, so the gradient of the input is the
    upstream gradient turned by the opposite angles (the same kernel on negated coordinates)."""

    @staticmethod
    def forward(ctx, x, coords, coord_high, theta, skip_tokens):
        ctx.save_for_backward(coords)
        ctx.cfg = (coord_high, theta, skip_tokens)
        return rope2d(x.detach(), coords, coord_high, theta, skip_tokens)

    @staticmethod
    def backward(ctx, g):
        (coords,) = ctx.saved_tensors
        coord_high, theta, skip_tokens = ctx.cfg
        return rope2d(g.contiguous(), -coords, coord_high, theta, skip_tokens), None, None, None, None


# --------------------------------------------------------------------------- #
# static block-sparse attention and 2-D RoPE
# --------------------------------------------------------------------------- #
def block_sparse_attention(q, k, v, row_ptr, col_idx, block, mode=0, num_cls=0, window=0, dilation=1,
                           out_dtype=None, kv_group=1, return_lse=False):
    """Flash attention restricted to a CSR list of key blocks per query block.

    q (B,H,Tq,D), k, v (B,H,Tk,D) bf16 (other float dtypes are converted); row_ptr / col_idx int32
    CUDA tensors; block in {64, 128}; D in {64, 128}.  mode 0: whole listed blocks; mode 1: the
    reference's CLS + dilated-window token pattern inside the listed blocks
    (static_sparse_attention.py:62-188).  Rows that see no key return zeros.
    """
    _require_cuda(q, k, v, row_ptr, col_idx)
    B, H, Tq, D0 = q.shape
    Tk = k.shape[2]
    out_dtype = out_dtype or q.dtype
    if D0 > 128:
        raise SwvError("block_sparse_attention supports head_dim <= 128")
    D = 64 if D0 <= 64 else 128
    if D != D0:
        # zero-pad the head dimension to a supported width; q is rescaled so that the kernel's
        # 1/sqrt(D) equals the caller's 1/sqrt(D0); the padded output channels are zero
        pad = (0, D - D0)
        q = torch.nn.functional.pad(q.float() * (D / D0) ** 0.5, pad)
        k = torch.nn.functional.pad(k, pad)
        v = torch.nn.functional.pad(v, pad)
    q, k, v = (t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16) for t in (q, k, v))
    q, k, v = (t if _tma_ok(t) else t.contiguous() for t in (q, k, v))
    if row_ptr.dtype != torch.int32 or col_idx.dtype != torch.int32:
        raise SwvError("row_ptr and col_idx must be int32")
    nqb = -(-Tq // block)
    if row_ptr.numel() != nqb + 1:
        raise SwvError(f"row_ptr has {row_ptr.numel()} entries, expected {nqb + 1}")
    dev = q.device
    o = torch.empty((B, H, Tq, D), dtype=out_dtype, device=dev)
    lse = torch.empty((B, H, Tq), dtype=torch.float32, device=dev) if return_lse else None
    st = status_word(dev)
    rc = lib.swv_block_sparse_attn_fwd(
        q.data_ptr(), strides(q), k.data_ptr(), strides(k), v.data_ptr(), strides(v), row_ptr.data_ptr(),
        col_idx.data_ptr(), block, mode, num_cls, window, dilation, kv_group,
        lse.data_ptr() if return_lse else None, o.data_ptr(), strides(o), dtype_code(o.dtype),
        B, H, Tq, Tk, D, st.data_ptr(), _stream(dev))
    check(rc, "swv_block_sparse_attn_fwd")
    if _CHECK:
        check_status(dev, "swv_block_sparse_attn_fwd")
    o = o if D == D0 else o[..., :D0]
    return (o, lse) if return_lse else o


def rope2d(x, coords, coord_high, theta=10000.0, skip_tokens=0, out=None):
    """2-D rotary embedding (vit_5/rope.py:72-97).  x (L,H,hd) or (1,L,H,hd), fp32 or bf16, unit inner
    stride; coords (L,2) or (1,L,2) in the units of coord_high; the first skip_tokens tokens are copied."""
    _require_cuda(x, coords)
    squeeze = x.dim() == 4
    if squeeze:
        if x.shape[0] != 1:
            raise SwvError("rope2d handles one slide at a time (batch 1), like the reference")
        x = x[0]
    c = coords.reshape(-1, 2).to(torch.float32).contiguous()
    L, H, hd = x.shape
    if c.shape[0] != L:
        raise SwvError("coords must have one (y, x) pair per token")
    if x.stride(2) != 1:
        x = x.contiguous()
    y = torch.empty_like(x) if out is None else out
    s3 = lambda t: (ctypes.c_int64 * 3)(*t.stride())
    rc = lib.swv_rope2d_apply(x.data_ptr(), s3(x), y.data_ptr(), s3(y), dtype_code(x.dtype), c.data_ptr(), L, H, hd,
                              float(coord_high), float(theta), int(skip_tokens), _stream(x.device))
    check(rc, "swv_rope2d_apply")
    return y[None] if squeeze else y
